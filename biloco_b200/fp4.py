"""NVFP4 (E2M1 codes, 16-element blocks, E4M3 block scales, fp32 tensor scale) operand preparation.

Stands in for the reference's ``biloco/fp4.py`` (a wrapper around the third-party ``fouroversix`` package,
which only offers quantise->dequantise) and adds what the fused kernel needs: the *packed* operands.

  * ``quantize_nvfp4``       offline weight path, plain torch ops in IEEE fp32 (any device); returns packed
                             codes, block scales in the 128x4 atom layout and the tensor scale.
  * ``quantize_activation``  per-call activation path: the CUDA quantiser of libbiloco_b200.so (codes, swizzled
                             scales, tensor scale and alpha = w_scale * a_scale stay on the device).
  * ``fake_quantize_fp4`` / ``set_scale_rules`` keep the reference's names (biloco/fp4.py:24-35).

Both paths perform the same sequence of single fp32 operations (documented in csrc/act_quant.cu), so they
agree bit for bit with each other and with the CPU oracle used by the tests.
"""
import torch

from . import _lib

SCALE_RULES = ("static_6", "static_4", "mse")
CONFIG_W = "mse"
CONFIG_X = "mse"

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def set_scale_rules(weight_rule: str = "mse", act_rule: str = "mse"):
    global CONFIG_W, CONFIG_X
    assert weight_rule in SCALE_RULES and act_rule in SCALE_RULES
    CONFIG_W, CONFIG_X = weight_rule, act_rule


def nvfp4_sf_bytes(rows: int, k: int) -> int:
    return (rows + 127) // 128 * 128 * ((k // 16 + 3) // 4 * 4)


def swizzle_scales(sf_linear: torch.Tensor) -> torch.Tensor:
    """uint8 [rows, K/16] -> float8_e4m3fn [nvfp4_sf_bytes]: 512-byte atoms of 128 rows x 4 blocks at
    (row%32)*16 + (row/32%4)*4 + block%4, atoms k-major inside each 128-row block (csrc/biloco_gemm.cu:3144-3145)."""
    rows, kb = sf_linear.shape
    rp, kp = (rows + 127) // 128 * 128, (kb + 3) // 4 * 4
    full = torch.zeros((rp, kp), dtype=torch.uint8, device=sf_linear.device)
    full[:rows, :kb] = sf_linear
    out = full.view(rp // 128, 4, 32, kp // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return out.reshape(-1).view(torch.float8_e4m3fn)


def unswizzle_scales(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """Inverse of swizzle_scales: -> uint8 [rows, k/16]."""
    kb = k // 16
    rp, kp = (rows + 127) // 128 * 128, (kb + 3) // 4 * 4
    v = sf.view(torch.uint8).reshape(-1)[: rp * kp].view(rp // 128, kp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return v.reshape(rp, kp)[:rows, :kb].contiguous()


def _e2m1_codes(q: torch.Tensor) -> torch.Tensor:
    a = q.abs()
    c = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8) + (a >= 1.75).to(torch.uint8)
         + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8) + (a > 5.0).to(torch.uint8))
    return c | (torch.signbit(q).to(torch.uint8) << 3)


def _e2m1_values(codes: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=codes.device)
    return lut[codes.long()]


def _div(a: torch.Tensor, scalar: float) -> torch.Tensor:
    """a / scalar, correctly rounded on every device: a CUDA tensor divided by a Python number is multiplied by the
    number's reciprocal instead (one ulp off for divisors such as 6 and 1536, enough to move a block scale that sits on an
    E4M3 rounding boundary to its neighbour); tensor / tensor on the same device is a true division."""
    return a / torch.full_like(a, scalar)


def _quant_with_div(xb, t, div, gs):
    sf = _div(t, div).clamp(0.0, 448.0).to(torch.float8_e4m3fn)
    d = sf.to(torch.float32) * gs
    live = d > 0
    q = xb / torch.where(live, d, torch.ones_like(d)).unsqueeze(-1)
    codes = torch.where(live.unsqueeze(-1), _e2m1_codes(q), torch.zeros_like(q, dtype=torch.uint8))
    deq = _e2m1_values(codes) * d.unsqueeze(-1)
    return codes, sf.view(torch.uint8), deq


@torch.no_grad()
def quantize_nvfp4(x: torch.Tensor, rule: str = None, global_scale=None):
    """x [rows, K] -> (codes uint8 [rows, K/2], block scales float8_e4m3fn (atom layout), tensor scale fp32 [1])."""
    rule = CONFIG_W if rule is None else rule
    assert rule in SCALE_RULES and x.dim() == 2 and x.shape[1] % 16 == 0
    x = x.to(torch.float32)
    rows, K = x.shape
    target = 448.0 if rule == "static_6" else 256.0
    if global_scale is None:
        amax = x.abs().max() if x.numel() else torch.zeros((), device=x.device)
        gs = torch.where(amax > 0, _div(amax, 6.0 * target), torch.ones_like(amax)).to(torch.float32)
    else:
        gs = torch.as_tensor(global_scale, dtype=torch.float32, device=x.device).reshape(())
    xb = x.view(rows, K // 16, 16)
    t = xb.abs().amax(dim=-1) / gs
    if rule == "static_6":
        codes, sf, _ = _quant_with_div(xb, t, 6.0, gs)
    elif rule == "static_4":
        codes, sf, _ = _quant_with_div(xb, t, 4.0, gs)
    else:
        c6, s6, q6 = _quant_with_div(xb, t, 6.0, gs)
        c4, s4, q4 = _quant_with_div(xb, t, 4.0, gs)
        e6 = torch.zeros_like(t)
        e4 = torch.zeros_like(t)
        for j in range(16):      # index order, separate multiply and add (matches the device quantiser)
            d6 = xb[..., j] - q6[..., j]
            d4 = xb[..., j] - q4[..., j]
            e6 = e6 + d6 * d6
            e4 = e4 + d4 * d4
        pick4 = e4 < e6
        codes = torch.where(pick4.unsqueeze(-1), c4, c6)
        sf = torch.where(pick4, s4, s6)
    codes = codes.view(rows, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, swizzle_scales(sf), gs.reshape(1)


@torch.no_grad()
def dequantize_nvfp4(packed: torch.Tensor, sf: torch.Tensor, gs, rows: int = None) -> torch.Tensor:
    """Inverse of quantize_nvfp4 -> fp32 [rows, K]."""
    rows = packed.shape[0] if rows is None else rows
    K = packed.shape[1] * 2
    codes = torch.stack([packed & 15, packed >> 4], dim=-1).view(packed.shape[0], K)[:rows]
    s = unswizzle_scales(sf, rows, K).view(torch.float8_e4m3fn).to(torch.float32)
    g = torch.as_tensor(gs, dtype=torch.float32, device=packed.device).reshape(())
    return (_e2m1_values(codes).view(rows, K // 16, 16) * (s * g).unsqueeze(-1)).view(rows, K)


def fake_quantize_fp4(x: torch.Tensor, config=None) -> torch.Tensor:
    """Quantize to NVFP4 and dequantize back (same dtype and shape); one tensor scale per call."""
    rule = CONFIG_W if config is None else config
    shape = x.shape
    p, sf, gs = quantize_nvfp4(x.reshape(-1, shape[-1]), rule)
    return dequantize_nvfp4(p, sf, gs).reshape(shape).to(x.dtype)


@torch.no_grad()
def activation_scale_from_amax(amax: torch.Tensor, rule: str = None) -> torch.Tensor:
    """Tensor scale the quantiser derives from max |x| (fp32 [1]); for callers that reduce amax across ranks."""
    rule = CONFIG_X if rule is None else rule
    target = 448.0 if rule == "static_6" else 256.0
    amax = amax.to(torch.float32).reshape(1)
    return torch.where(amax > 0, _div(amax, 6.0 * target), torch.ones_like(amax))


def _rec_buffer(M: int, K: int, dev):
    """Buffer for the per-k-tile activation record the fused kernel fetches with one copy per work unit (None when the
    shape has none: more than 32 rows or K not a multiple of 256)."""
    n = _lib.load().biloco_b200_act_rec_bytes(M, K) if (M <= 32 and K % 256 == 0) else 0
    return torch.empty(n, device=dev, dtype=torch.uint8) if n else None


def quantize_activation(x: torch.Tensor, rule: str = None, smooth: torch.Tensor = None, w_gscale: torch.Tensor = None,
                        rows: int = None, out: dict = None, gscale: torch.Tensor = None, norm_weight: torch.Tensor = None,
                        eps: float = 1e-6, swiglu: bool = False):
    """bf16 CUDA activation [M, K] -> dict(A [1, rows, K/2] uint8, A_sf float8 (atom layout), A_rec (the same codes and
    scales as the fused kernel stages them, or None), gscale fp32 [1],
    alpha fp32 [1] (= w_gscale * gscale, when w_gscale is given), X bf16 [M, K] (x / smooth when smoothing)).
    ``gscale`` (fp32 [1]) supplies the tensor scale instead of deriving it from this tensor's own maximum.
    Runs the library's quantiser on the current stream; nothing returns to the host. Pass ``out`` (a dict from
    an earlier call with the same shapes) to reuse its buffers, e.g. under CUDA-graph capture.
    ``norm_weight`` (bf16 [K]): RMS-normalise every row first (x * rsqrt(mean(x^2) + eps) -> bf16, * weight -> bf16) inside
    the same launch; X is then the normalised activation. ``w_gscale`` may hold n scales (fp32 [n]): alpha gets one entry
    per linear that consumes this activation.
    ``swiglu``: x is [M, 2K] = [gate | up] and the activation quantised is silu(gate) * up (each rounded to bf16, as the
    separate torch kernels would), computed inside the same launch; X is that activation."""
    rule = CONFIG_X if rule is None else rule
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    M, K = x.shape
    if swiglu:
        assert norm_weight is None and gscale is None and K % 2 == 0
        K //= 2
    rows = M if rows is None else rows
    dev = x.device
    if out is None:
        out = dict(A=torch.empty((1, rows, K // 2), device=dev, dtype=torch.uint8),
                   A_sf=torch.empty(nvfp4_sf_bytes(rows, K), device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn),
                   gscale=torch.empty(1, device=dev, dtype=torch.float32),
                   alpha=torch.empty(w_gscale.numel(), device=dev, dtype=torch.float32) if w_gscale is not None else None,
                   X=(torch.empty((M, K), device=dev, dtype=torch.bfloat16)
                      if (smooth is not None or norm_weight is not None or swiglu) else x),
                   A_rec=_rec_buffer(M, K, dev))
    elif smooth is None and norm_weight is None and not swiglu:
        out["X"] = x
    rule_id = _lib.RULES[rule]
    if gscale is not None:          # tensor scale agreed elsewhere (tensor-parallel K-slices): do not recompute it
        out["gscale"].copy_(gscale.reshape(1))
        rule_id |= 0x100
    n_alpha = w_gscale.numel() if w_gscale is not None else 1
    rec = out.get("A_rec")
    with torch.cuda.device(dev):
        if swiglu:
            rc = _lib.load().biloco_b200_swiglu_act_quant(
                x.data_ptr(), smooth.data_ptr() if smooth is not None else None, out["X"].data_ptr(), out["A"].data_ptr(),
                out["A_sf"].data_ptr(), rec.data_ptr() if rec is not None else None, out["gscale"].data_ptr(),
                out["alpha"].data_ptr() if w_gscale is not None else None,
                w_gscale.data_ptr() if w_gscale is not None else None, n_alpha, M, rows, K, rule_id,
                torch.cuda.current_stream().cuda_stream)
        elif norm_weight is None and n_alpha == 1 and rec is None:
            rc = _lib.load().biloco_b200_act_quant(
                x.data_ptr(), smooth.data_ptr() if smooth is not None else None,
                out["X"].data_ptr() if smooth is not None else None, out["A"].data_ptr(), out["A_sf"].data_ptr(),
                out["gscale"].data_ptr(), out["alpha"].data_ptr() if w_gscale is not None else None,
                w_gscale.data_ptr() if w_gscale is not None else None, M, rows, K, rule_id,
                torch.cuda.current_stream().cuda_stream)
        else:
            if norm_weight is not None:
                assert norm_weight.dtype == torch.bfloat16 and norm_weight.numel() == K and norm_weight.is_contiguous()
            rc = _lib.load().biloco_b200_norm_act_quant(
                x.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                smooth.data_ptr() if smooth is not None else None,
                out["X"].data_ptr() if (smooth is not None or norm_weight is not None) else None,
                out["A"].data_ptr(), out["A_sf"].data_ptr(), rec.data_ptr() if rec is not None else None, out["gscale"].data_ptr(),
                out["alpha"].data_ptr() if w_gscale is not None else None,
                w_gscale.data_ptr() if w_gscale is not None else None, n_alpha, M, rows, K, rule_id,
                torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, f"act_quant (M={M}, K={K}, rule={rule})")
    return out
