"""BiLoCoLinear backed by the fused kernel: y = (x/s) V diag(alpha) U^T + FP4(x/s) FP4(R)^T + b.

Same constructor, ``quantize`` and ``forward`` signatures as the reference module (``biloco/layer.py:16-64``), but
``quantize`` keeps what the fused kernel streams — packed NVFP4 codes and block scales of the residual, bit-packed
signs, bf16 coefficients — instead of dequantised bf16 copies, and ``forward`` is three enqueued device calls (the
NVFP4 activation quantiser with the SmoothQuant division folded in, then the fused linear), with no host
synchronisation. ``forward_fake_quant`` restates the reference's unfused bf16 forward on the same operands with
plain torch ops; the tests use it as the device-side comparator.
"""
import torch
import torch.nn as nn

from . import fp4
from .peel import decompose

METHODS = ("biloco", "fp4")
MAX_ROWS = 32     # activation rows per fused launch


class BiLoCoLinear(nn.Module):
    def __init__(self, linear: nn.Linear, rank: int, method: str = "biloco", smooth_factor: float = 0.5):
        super().__init__()
        assert method in METHODS, method
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.method = method
        self.rank = rank if method != "fp4" else 0
        self.smooth_factor = smooth_factor
        dev = linear.weight.device
        K, N, r = self.in_features, self.out_features, self.rank
        # The original weight is consumed by quantize() and then freed.
        self.weight = nn.Parameter(linear.weight.data.to(torch.bfloat16), requires_grad=False)
        self.bias = None if linear.bias is None else nn.Parameter(linear.bias.data.to(torch.bfloat16), requires_grad=False)
        self.register_buffer("smooth_scale", torch.ones(K, device=dev, dtype=torch.bfloat16))
        self.register_buffer("V_packed", torch.zeros(r, K // 8, device=dev, dtype=torch.uint8))
        self.register_buffer("U_packed", torch.zeros(r, N // 8, device=dev, dtype=torch.uint8))
        self.register_buffer("S", torch.zeros(r, device=dev, dtype=torch.bfloat16))
        self.register_buffer("W_codes", torch.zeros(N, K // 2, device=dev, dtype=torch.uint8))
        self.register_buffer("W_sf", torch.zeros(fp4.nvfp4_sf_bytes(N, K), device=dev, dtype=torch.uint8))
        self.register_buffer("w_gscale", torch.ones(1, device=dev, dtype=torch.float32))
        self._smoothed = None        # (decided from smooth_scale on first use, see `smoothed`)
        self._gemms = {}      # decode batch M -> BiLoCoGemm
        self._acts = {}       # (decode batch M, SwiGLU input?) -> reusable activation-quantiser outputs

    @classmethod
    def synthetic(cls, in_features: int, out_features: int, rank: int, device, seed: int = 0):
        """A quantised layer with random operands (random codes, block scales in [0.25, 2], random signs, coefficients
        ~ N(0, 0.01^2)), in the construction of the reference's timing scripts (scripts/problem.py:7-27): the same
        bytes and arithmetic as a decomposed layer without the decomposition. For throughput measurements."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        K, N, r = in_features, out_features, rank
        self.in_features, self.out_features, self.method, self.rank, self.smooth_factor = K, N, "biloco", r, 0.5
        g = torch.Generator(device=device).manual_seed(seed)
        self.weight, self.bias = None, None
        self.register_buffer("smooth_scale", torch.ones(K, device=device, dtype=torch.bfloat16))
        self.register_buffer("V_packed", torch.randint(0, 256, (r, K // 8), device=device, dtype=torch.uint8, generator=g))
        self.register_buffer("U_packed", torch.randint(0, 256, (r, N // 8), device=device, dtype=torch.uint8, generator=g))
        self.register_buffer("S", (torch.randn(r, device=device, generator=g) * 0.01).to(torch.bfloat16))
        self.register_buffer("W_codes", torch.randint(0, 256, (N, K // 2), device=device, dtype=torch.uint8, generator=g))
        sf = (torch.rand(fp4.nvfp4_sf_bytes(N, K), device=device, generator=g) * 1.75 + 0.25).to(torch.float8_e4m3fn)
        self.register_buffer("W_sf", sf.view(torch.uint8))
        self.register_buffer("w_gscale", torch.full((1,), 1e-3, device=device, dtype=torch.float32))
        self._smoothed = False
        self._gemms, self._acts = {}, {}
        return self

    @classmethod
    def from_operands(cls, ops: dict):
        """A quantised layer around given packed operands (the dict of export_operands, e.g. one rank's shard of a layer
        made by biloco_b200.parallel.shard_column_parallel / shard_row_parallel)."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        N, K = ops["W_codes"].shape[0], ops["W_codes"].shape[1] * 2
        self.in_features, self.out_features, self.method, self.smooth_factor = K, N, "biloco", 0.5
        self.rank = ops["V_packed"].shape[0]
        self.weight = None
        self.bias = None if ops.get("bias") is None else nn.Parameter(ops["bias"].to(torch.bfloat16), requires_grad=False)
        for name in ("smooth_scale", "V_packed", "U_packed", "S", "W_codes", "w_gscale"):
            self.register_buffer(name, ops[name].contiguous())
        self.register_buffer("W_sf", ops["W_sf"].view(torch.uint8).contiguous())
        self._smoothed = None
        self._gemms, self._acts = {}, {}
        return self

    # ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def quantize(self, act_col_max: torch.Tensor = None, T: int = 5, device=None):
        """Smooth, split off the binary low-rank component, and pack the residual as NVFP4 (biloco/layer.py:34-52)."""
        from .kernel import pack_signs
        device = device or self.weight.device
        W = self.weight.data.to(device=device, dtype=torch.float32)          # (out, in)
        if act_col_max is not None:
            a = act_col_max.to(device=device, dtype=torch.float32).clamp(min=1e-6)
            w_col_max = W.abs().max(dim=0).values.clamp(min=1e-6)
            s = (a ** self.smooth_factor) / (w_col_max ** (1 - self.smooth_factor))
            self.smooth_scale.copy_(s.to(torch.bfloat16))
            self._smoothed = True
            W = W * s
        if self.rank > 0:
            U, V, alpha, R = decompose(W, r=self.rank, T=T)
            self.V_packed.copy_(pack_signs(V.T.contiguous()))
            self.U_packed.copy_(pack_signs(U.T.contiguous()))
            self.S.copy_(alpha.to(torch.bfloat16))
        else:
            R = W
        codes, sf, gs = fp4.quantize_nvfp4(R.to(torch.bfloat16).float(), fp4.CONFIG_W)
        self.W_codes.copy_(codes)
        self.W_sf.copy_(sf.view(torch.uint8))
        self.w_gscale.copy_(gs)
        self.weight = None
        self._gemms.clear()

    @property
    def smoothed(self) -> bool:
        """Whether the activation has to be divided by smooth_scale (any entry different from 1). Derived from the buffer
        itself, once, so that a layer restored with load_state_dict or filled by copying buffers behaves like the one
        that was saved."""
        if self._smoothed is None:
            self._smoothed = bool((self.smooth_scale.float() != 1).any())
        return self._smoothed

    @smoothed.setter
    def smoothed(self, value):
        self._smoothed = None if value is None else bool(value)

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._smoothed = None

    def export_operands(self):
        """What the fused kernel consumes, as a dict of tensors (the packed counterpart of the reference's state dict)."""
        return dict(W_codes=self.W_codes, W_sf=self.W_sf.view(torch.float8_e4m3fn), w_gscale=self.w_gscale,
                    V_packed=self.V_packed, U_packed=self.U_packed, S=self.S, smooth_scale=self.smooth_scale,
                    bias=self.bias)

    # ------------------------------------------------------------------------------------------------------
    def _gemm_for(self, M, alpha):
        from .kernel import BiLoCoGemm, _FP4Only
        g = self._gemms.get(M)
        if g is None:
            if self.rank > 0:
                g = BiLoCoGemm(self.W_codes, self.W_sf.view(torch.float8_e4m3fn), alpha, self.V_packed, self.U_packed, self.S, M=M,
                               back_to_back=False)      # (a quantiser launch sits between the linears)
            else:
                g = _FP4Only(self.W_codes, self.W_sf.view(torch.float8_e4m3fn), alpha, M=M)
            if self.bias is not None:     # added inside the kernel, before its single bf16 rounding
                g.residual = self.bias.detach().to(torch.bfloat16).unsqueeze(0).expand(M, self.out_features).contiguous()
            self._gemms[M] = g
        return g

    def _rows(self, x2, residual=None, swiglu=False, gscale=None):
        M = x2.shape[0]
        q = fp4.quantize_activation(x2, fp4.CONFIG_X, smooth=self.smooth_scale if self.smoothed else None,
                                    w_gscale=self.w_gscale, rows=M, out=self._acts.get((M, swiglu)), swiglu=swiglu, gscale=gscale)
        self._acts[(M, swiglu)] = q
        g = self._gemm_for(M, q["alpha"])
        if self.bias is None:          # (with a bias, residual holds the broadcast bias)
            g.residual = residual
        return g(q["A"], q["A_sf"], q["X"], A_rec=q.get("A_rec")).view(-1, self.out_features)[:M]

    def forward_fused(self, x, residual=None, swiglu=False):
        """The kernel forward for at most 32 rows with the steps either side of the linear folded into its launches
        (not in the reference's interface): ``swiglu`` — x is [M, 2 * in_features] = [gate | up] and the layer's input is
        silu(gate) * up, formed inside the quantiser launch; ``residual`` (bf16 [M, out_features], layers without bias) is
        added inside the fused kernel before its single rounding to bf16."""
        assert self.weight is None and x.dim() == 2 and x.shape[0] <= MAX_ROWS and x.dtype == torch.bfloat16
        assert x.shape[1] == self.in_features * (2 if swiglu else 1)
        assert residual is None or (self.bias is None and residual.dtype == torch.bfloat16 and residual.is_contiguous()
                                    and residual.shape == (x.shape[0], self.out_features))
        return self._rows(x.contiguous(), residual=residual, swiglu=swiglu)

    def forward_quantized(self, q: dict, alpha: torch.Tensor):
        """The fused linear on an activation that has been quantised already (fp4.quantize_activation with this layer's
        rules and smoothing): q["A"], q["A_sf"], q["X"] for M <= 32 rows; alpha fp32 [1] = w_gscale * q["gscale"] on the
        device. Lets several layers that read the same activation (q/k/v, gate/up) share one quantiser launch."""
        M = q["X"].shape[0]
        g = self._gemm_for(M, alpha)
        if g.alpha.data_ptr() != alpha.data_ptr():       # (the launcher keeps the pointer it was built with)
            g.alpha = alpha
        return g(q["A"], q["A_sf"], q["X"], A_rec=q.get("A_rec")).view(-1, self.out_features)[:M]

    def forward(self, x):
        assert self.weight is None, "call quantize() first"
        shape = x.shape
        x2 = x.to(torch.bfloat16).reshape(-1, self.in_features).contiguous()
        if x2.shape[0] <= MAX_ROWS:
            y = self._rows(x2)
        else:
            # longer inputs (prefill, evaluation) go through in blocks of 32 rows that all use ONE tensor scale, taken over
            # the whole smoothed activation as the reference quantises it (biloco/fp4.py:3-4, biloco/layer.py:60)
            xs = (x2 / self.smooth_scale) if self.smoothed else x2
            gscale = fp4.activation_scale_from_amax(xs.float().abs().max().reshape(1), fp4.CONFIG_X)
            y = torch.cat([self._rows(x2[i:i + MAX_ROWS].contiguous(), gscale=gscale).clone()
                           for i in range(0, x2.shape[0], MAX_ROWS)], dim=0)
        return y.reshape(*shape[:-1], self.out_features).to(torch.bfloat16)

    # ------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_fake_quant(self, x):
        """The reference's unfused forward (biloco/layer.py:54-64) on this module's operands, plain torch ops."""
        from .kernel import unpack_signs
        x_s = x.to(torch.bfloat16) / self.smooth_scale
        y = torch.zeros((*x_s.shape[:-1], self.out_features), dtype=torch.bfloat16, device=x_s.device)
        if self.rank > 0:
            V_scaled = (unpack_signs(self.V_packed) * self.S.float().unsqueeze(1)).to(torch.bfloat16)    # [r, K]
            U_T = unpack_signs(self.U_packed).to(torch.bfloat16)                                          # [r, N]
            y = y + (x_s @ V_scaled.T) @ U_T
        x_fq = fp4.fake_quantize_fp4(x_s.reshape(-1, self.in_features), fp4.CONFIG_X).reshape(x_s.shape)
        weight_fp4 = fp4.dequantize_nvfp4(self.W_codes, self.W_sf.view(torch.float8_e4m3fn), self.w_gscale).to(torch.bfloat16)
        y = y + x_fq @ weight_fp4.T
        if self.bias is not None:
            y = y + self.bias
        return y.to(torch.bfloat16)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, method={self.method}, rank={self.rank}"
