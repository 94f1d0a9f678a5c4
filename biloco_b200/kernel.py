"""Python side of the fused B200 kernel: sign packing, operand layouts, mode table and a launcher.

Mirrors the public interface of the reference's ``biloco/kernel.py`` (``BiLoCoGemm``, ``pack_signs``,
``pack_u_col32``, ``modes_for``, ``DEFAULT_MODE``, ``RANKS``, ``nvfp4_sf_bytes``, ``reference``,
``time_graph``) and registers the same ``torch.ops.biloco.*`` operators (``csrc/bindings.cpp:17-48``), so a
caller written against the reference runs unchanged. Underneath, every operator is one call into
``libbiloco_b200.so`` through the C ABI of ``include/biloco_b200.h``; there is no PyTorch or CPU fallback.

One launch computes  y = alpha * FP4(x) FP4(R)^T + sum_i S_i (x . v_i) u_i  for a decode batch of M <= 32 rows.
"""
import torch

from . import _lib
from . import ops as _ops  # noqa: F401  (registers torch.ops.biloco)

ops = torch.ops.biloco

# Ranks the mode table is measured for (the reference's RANKS, biloco/kernel.py:16, plus 1024).
RANKS = (16, 32, 64, 128, 256, 512, 1024)

# Schedules implemented by the fused kernel (see include/biloco_b200.h, BILOCO_MODE_*).
IMPLEMENTED_MODES = (2, 4, 5, 7)

# Time per call of every implemented mode per (M, rank) on B200 at K = N = 5120, HBM-cold, from `bench.py --table` (us;
# mode 2 / mode 5 / mode 7 where the mode takes the point; M = 16, 32: mode 2 only, z stage and expansion on the tensor cores):
#   r = 128 : M=1 11.3/9.6/8.5    M=2 12.0/9.7/8.5    M=4 12.9/12.7/10.5  M=8 14.7/14.7  M=16 20.4  M=32 25.0
#   r = 256 : M=1 11.9/9.8/8.2    M=2 12.7/10.1/8.6   M=4 14.6/14.4/10.4  M=8 17.1/16.5  M=16 21.8  M=32 26.3
#   r = 512 : M=1 12.7/10.2/8.9   M=2 14.7/12.6/9.4   M=4 16.9/16.0/10.7  M=8 21.6/20.4  M=16 24.4  M=32 29.9
#   r = 1024: M=1 14.9/14.1/10.2  M=2 17.6/18.5/12.4  M=4 21.6/21.5       M=8 29.9/31.3  M=16 31.5  M=32 39.6
# Mode 5 does not take M > 8, mode 7 not M > 4 (nor r = 1024 at M = 4); mode 4 loses everywhere. Ranks below 128 were not
# measured and follow r = 128. DEFAULT_MODE is the table WITHOUT mode 7 (what a stream with other kernels between the linears
# uses); default_mode() puts mode 7 in front of it for launches that follow one another directly.
_MODE2_WINS = {(2, 1024), (8, 1024)}
DEFAULT_MODE = {M: {r: (2 if (M > 8 or (M, r) in _MODE2_WINS) else 5) for r in RANKS} for M in (1, 2, 4, 8, 16, 32)}


def default_mode(M: int, rank: int, ok, back_to_back: bool = True):
    """The schedule BiLoCoGemm picks among the modes `ok` that the shape takes. Row slabs (mode 7) for one to four rows when
    the launches of a stream follow one another directly (the reference's measurement protocol, a chain of linears): a
    row-slab CTA takes the SM's whole tensor memory and relies on meeting exactly one CTA of the next launch on its SM.
    With other kernels in between (an activation quantiser per linear, the decode step) two CTAs of one launch can land
    on one SM and take turns (measured: 20.6 us per layer against 16.4 with the cluster schedule), so
    back_to_back=False keeps to the measured table of the other schedules; then the first that is available."""
    if M <= 4 and 7 in ok and back_to_back:
        return 7
    mode = DEFAULT_MODE.get(M, {}).get(rank)
    return mode if mode in ok else ([m for m in ok if m != 7] or [None])[0]


_TUNED = {}          # (device index, M, N, K, R, back_to_back) -> mode, filled by tuned_mode()
AUTOTUNE = False     # BiLoCoGemm(mode=None): measure the schedules once per shape instead of reading the 5120 x 5120 table


@torch.no_grad()
def tuned_mode(M: int, N: int, K: int, R: int, back_to_back: bool = True, device=None, verbose: bool = False):
    """The fastest schedule for this shape ON THIS GPU, measured once per process and cached: every schedule the shape
    takes runs a captured graph over enough distinct random weight copies to exceed L2 (HBM-cold, at most 16 copies), the
    median of 12 replays decides. With back_to_back=False a quantiser launch sits in front of every linear, as in a layer's
    forward, and the row-slab schedule is left out (see default_mode). The table DEFAULT_MODE holds what this returns at
    K = N = 5120; other shapes (8192 x 8192, 28672-wide MLPs, shards) do not always agree with it."""
    from . import fp4
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.index, M, N, K, R, back_to_back)
    if key in _TUNED:
        return _TUNED[key]
    with torch.cuda.device(dev):
        ok = [m for m in supported_modes(M, N, K, R) if back_to_back or m != 7]
        if len(ok) <= 1:
            _TUNED[key] = ok[0] if ok else None
            return _TUNED[key]
        wbytes = N * K // 2
        copies = max(2, min(16, -(-140_000_000 // wbytes)))
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        wgs = torch.full((1,), 1e-3, device=dev)
        q = fp4.quantize_activation(x, "mse", w_gscale=wgs, rows=M)
        V = torch.randint(0, 256, (R, K // 8), device=dev, dtype=torch.uint8, generator=g)
        U = torch.randint(0, 256, (R, N // 8), device=dev, dtype=torch.uint8, generator=g)
        S = (torch.randn(R, device=dev, generator=g) * 0.01).to(torch.bfloat16)
        Ws = [torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8, generator=g) for _ in range(copies)]
        sf = torch.full((nvfp4_sf_bytes(N, K),), 0x38, device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
        best, best_us, seen = None, None, {}
        for m in ok:
            gemms = [BiLoCoGemm(W, sf, q["alpha"], V, U, S, M=M, mode=m) for W in Ws]

            def run():
                for gm in gemms:
                    if not back_to_back:
                        fp4.quantize_activation(x, "mse", w_gscale=wgs, rows=M, out=q)
                    gm(q["A"], q["A_sf"], q["X"], A_rec=q.get("A_rec") if m != 7 else None)
            us = time_graph(run, None, iters=12, batch=1) / copies
            seen[m] = us
            if all(gm.status()[0] == 0 for gm in gemms) and (best_us is None or us < best_us):
                best, best_us = m, us
            del gemms
        if verbose:
            print(f"tuned_mode M={M} N={N} K={K} R={R} back_to_back={back_to_back}: " + ", ".join(f"mode {m}: {u:.1f} us" for m, u in seen.items()) + f" -> {best}")
    _TUNED[key] = best
    return best


def pack_signs(signs: torch.Tensor) -> torch.Tensor:
    """[..., n] +-1 -> uint8 [..., n/8]; bit i of byte j is set iff signs[..., 8j + i] >= 0
    (same bit order and zero-is-plus rule as biloco/kernel.py:29-34)."""
    assert signs.shape[-1] % 8 == 0
    b = (signs >= 0).reshape(*signs.shape[:-1], signs.shape[-1] // 8, 8).to(torch.int32)
    shifts = torch.arange(8, device=signs.device, dtype=torch.int32)
    return (b << shifts).sum(dim=-1).to(torch.uint8)


def unpack_signs(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., n/8] -> float32 [..., n] of +-1 (inverse of pack_signs)."""
    shifts = torch.arange(8, device=packed.device, dtype=torch.int32)
    bits = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & 1
    return bits.reshape(*packed.shape[:-1], packed.shape[-1] * 8).to(torch.float32) * 2.0 - 1.0


def pack_u_col32(U_packed: torch.Tensor, n_cols: int, rank: int) -> torch.Tensor:
    """U_packed [R, N/8] -> int32 [N, ceil(R/32)]: bit b of word w of column n is the sign bit of rank 32w + b
    (layout of biloco/kernel.py:37-47). CUDA tensors go through the library's re-layout kernel."""
    assert U_packed.dtype == torch.uint8 and U_packed.shape == (rank, n_cols // 8)
    words = (rank + 31) // 32
    if U_packed.is_cuda:
        out = torch.empty((n_cols, words), device=U_packed.device, dtype=torch.int32)
        with torch.cuda.device(U_packed.device):
            _lib.check(_lib.load().biloco_b200_pack_u_col32(U_packed.contiguous().data_ptr(), out.data_ptr(), n_cols, rank,
                                                            torch.cuda.current_stream().cuda_stream), "pack_u_col32")
        return out
    shifts = torch.arange(8, dtype=torch.int64)
    bits = ((U_packed.to(torch.int64).unsqueeze(-1) >> shifts) & 1).reshape(rank, n_cols)       # [R, N]
    pad = words * 32 - rank
    if pad:
        bits = torch.cat([bits, torch.zeros(pad, n_cols, dtype=torch.int64)], dim=0)
    w = (bits.reshape(words, 32, n_cols) << torch.arange(32, dtype=torch.int64).view(1, 32, 1)).sum(dim=1)  # [words, N]
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w)
    return w.t().contiguous().to(torch.int32)


def modes_for(M: int, rank: int, K: int = 5120):
    """Modes the fused kernel accepts for this (M, rank, K). The launch can still reject a shape in its
    host-side checks (K must be a multiple of 256, N of 8)."""
    if not (1 <= M <= 32) or rank < 1 or K % 256 != 0:
        return []
    return [m for m in IMPLEMENTED_MODES if (m != 5 or M <= 8) and (m != 7 or (M <= 4 and K % 512 == 0))]


def supported_modes(M: int, N: int, K: int, rank: int, num_sms: int = 0):
    """Modes the launch accepts for this full problem shape (modes_for knows only M, rank and K; mode 5 also
    depends on N and on the number of SMs). num_sms = 0 asks the current device."""
    lib = _lib.load()
    return [m for m in modes_for(M, rank, K) if lib.biloco_b200_mode_supported(M, N, K, rank, m, num_sms)]


def nvfp4_sf_bytes(rows: int, k: int) -> int:
    """Bytes of the NVFP4 block-scale tensor for a [rows, k] operand (rows padded to 128, k/16 padded to 4)."""
    return (rows + 127) // 128 * 128 * ((k // 16 + 3) // 4 * 4)


def scratch_bytes(M: int, N: int, K: int, R: int, num_sms: int = 0) -> int:
    """Scratch the fused kernel needs for this problem (0 SMs = ask the current device)."""
    n = _lib.load().biloco_b200_scratch_bytes(M, N, K, R, num_sms)
    if n == 0:
        raise RuntimeError(f"fused linear does not support M={M} N={N} K={K} R={R}")
    return n


class BiLoCoGemm:
    """Fused FP4 GEMM + binary low-rank term for one layer at a fixed decode batch M.

    W_fp4 [N, K/2] uint8 and W_sf: NVFP4 weight codes and block scales; alpha: fp32 [1];
    V_packed [R, K/8], U_packed [R, N/8]: packed signs; S: bf16 [R] coefficients.
    Call with the NVFP4 activation A [1, rows, K/2] uint8 (rows >= M; the reference pads to 128 rows, any
    row count from M to 128 is accepted), its block scales A_sf, and the BF16 activation X [M, K] (the
    low-rank term uses the unquantized activation).
    tile_weights=False skips the unit-contiguous copy of the weight (saves its memory, streams slower).
    Consecutive calls need no clearing of the scratch buffer: the kernel returns its counters to zero before it
    exits, so a CUDA graph containing calls can be replayed as is (calling reset() inside the captured region,
    as the reference requires, stays valid).
    """

    def __init__(self, W_fp4, W_sf, alpha, V_packed, U_packed, S, M: int, mode: int = None, tile_weights: bool = True,
                 back_to_back: bool = True):
        self.N, self.K = W_fp4.shape[0], W_fp4.shape[1] * 2
        self.R, self.M = V_packed.shape[0], M
        dev = W_fp4.device
        with torch.cuda.device(dev):
            ok = supported_modes(M, self.N, self.K, self.R)
        if mode is None and AUTOTUNE and len(ok) > 1:      # measured once per shape on this GPU
            mode = tuned_mode(M, self.N, self.K, self.R, back_to_back, device=dev)
        if mode is None:      # the table's choice if this shape takes it, else the first mode that does
            mode = default_mode(M, self.R, ok, back_to_back)
        self.mode = mode
        assert self.mode in ok, f"mode {self.mode} not available for M={M} N={self.N} K={self.K} R={self.R}"
        self.W_fp4, self.W_sf, self.alpha, self.V, self.S = W_fp4, W_sf, alpha, V_packed, S
        self.U_col32 = pack_u_col32(U_packed, n_cols=self.N, rank=self.R)
        self.none = torch.zeros(0, device=dev, dtype=torch.int64)
        # unit-contiguous copy of the weight (the counterpart of the reference's V_perm / U_rw re-layouts): the
        # kernel then reads sequential 18 KB records instead of 128 strided 128-byte rows per tile
        if self.mode == 7:    # the row-slab schedule streams its own re-laid copy (required)
            self.W_tiled = _ops.tile_weights_slab(W_fp4, W_sf)
        else:
            self.W_tiled = _ops.tile_weights(W_fp4, W_sf) if tile_weights else self.none
        with torch.cuda.device(dev):
            nbytes = scratch_bytes(M, self.N, self.K, self.R)
            self._head = _lib.load().biloco_b200_scratch_head_bytes(M, self.N, self.K, self.R, 0) // 4
        # one buffer holds status words, counters, the z hand-off area and the split-K partial sums
        self.z = torch.zeros(nbytes // 4, device=dev, dtype=torch.float32)
        self.epoch = 0
        self.residual = None      # optional bf16 [M, N] added before the single final rounding (e.g. a broadcast bias)
        self.fp32_out = False     # True: return the unrounded fp32 sum (partial outputs reduced across devices)
        self.peer_push = None     # row-parallel shards: PeerAllReduce.push_args(); the epilogue then also stores its outputs to the peers

    def reset(self):
        """Clear the status words and counters (needed only after a launch whose status reported a failed wait;
        harmless otherwise) and restart the epoch count."""
        self.z[: self._head].zero_()
        self.epoch = 0

    def status(self):
        """The 16 device status words (synchronises): word 0 is non-zero after a device-side wait ran out."""
        import ctypes
        out = (ctypes.c_int32 * 16)()
        with torch.cuda.device(self.z.device):
            _lib.check(_lib.load().biloco_b200_read_status(self.z.data_ptr(), out, torch.cuda.current_stream().cuda_stream),
                       "read_status")
        return list(out)

    def raw_supported(self) -> bool:
        """True when raw() can run this problem (row-slab schedule with room for the staged activation)."""
        if self.mode != 7:
            return False
        with torch.cuda.device(self.z.device):
            return bool(_lib.load().biloco_b200_fused_linear_act_supported(self.M, self.N, self.K, self.R, 0))

    def raw(self, x, w_gscale, rule="mse", norm_weight=None, eps=1e-6, smooth=None, swiglu=False, out=None, act_out=None):
        """One launch from the RAW bf16 activation (row-slab schedule only): RMS norm or silu(gate) * up, smoothing, NVFP4
        quantisation with `rule` and the linear; x [M, K] ([M, 2K] with swiglu), w_gscale fp32 [1] = the weights' tensor
        scale. Same bits as fp4.quantize_activation followed by __call__. Returns [M, N]. No counterpart in the reference
        (biloco/layer.py:55-63 runs smoothing, fake quantisation and the matmuls as separate kernels)."""
        assert self.mode == 7, "the raw-activation form exists for the row-slab schedule (mode 7)"
        self.epoch += 1
        return _ops.fused_linear_act(x, self.W_tiled, self.N, w_gscale, self.V, self.S, self.U_col32, self.z, self.epoch, rule,
                                     norm_weight=norm_weight, eps=eps, smooth=smooth, swiglu=swiglu, C=self.residual, out=out,
                                     fp32_out=self.fp32_out, act_out=act_out)

    def __call__(self, A_pad, A_sf, X_bf16, out=None, A_rec=None):
        """Returns bf16 [1, rows, N]; rows >= M are padding (left unwritten). Not in the reference's signature: ``out``,
        a [rows, N] tensor to write into instead of a fresh one (e.g. a slice of a buffer that is read back in one copy),
        and ``A_rec``, the activation quantiser's per-k-tile record (fp4.quantize_activation(...)["A_rec"]) with which the
        kernel fetches the activation side of a work unit in one copy."""
        self.epoch += 1
        if self.mode == 7:        # no operator of the reference's schema set stands for this schedule
            return _ops._fused(A_pad, self.W_fp4, A_sf, self.W_sf, self.alpha, X_bf16, self.V, self.S, self.U_col32, self.z,
                               self.M, self.epoch, self.mode, C=self.residual, out=out, B_tiled=self.W_tiled,
                               fp32_out=self.fp32_out)
        if self.residual is not None or self.fp32_out or out is not None or A_rec is not None:   # not expressible in the operator schemas
            return _ops._fused(A_pad, self.W_fp4, A_sf, self.W_sf, self.alpha, X_bf16, self.V, self.S, self.U_col32, self.z,
                               self.M, self.epoch, self.mode, C=self.residual, out=out, A_rec=A_rec,
                               B_tiled=self.W_tiled if self.W_tiled.numel() else None, fp32_out=self.fp32_out,
                               push=self.peer_push if self.fp32_out else None)
        a = (A_pad, self.W_fp4, A_sf, self.W_sf, self.alpha, X_bf16, self.V, self.S, self.U_col32)
        if self.mode == 2:
            return ops.biloco_gemm_mode2(*a, self.z, self.none, self.none, self.W_tiled, self.none, self.M, self.epoch)
        if self.mode == 4:
            return ops.biloco_gemm_mode4(*a, self.z, self.W_tiled, self.M, self.epoch)
        return ops.biloco_gemm_mode5(*a, self.z, self.W_tiled, self.none, self.M, self.epoch)


class GroupedBiLoCoGemm:
    """Several BiLoCoGemm problems that read the same activation (q/k/v, gate/up) as ONE launch: the weights stacked
    along N, the low-rank factors side by side (every linear keeps its own R ranks and its own decode scale). Built from
    the separate launchers, all for the same M, K and R and with N a multiple of 128; ``alpha`` at call time is the fp32
    [n] vector of decode scales in the same order (fp4.quantize_activation with w_gscale of n entries writes it).
    Returns the list of per-linear outputs, views [M, N_g] of one [M, sum N_g] result.
    No counterpart in the reference (one launch per linear)."""

    def __init__(self, gemms, mode: int = None):
        g0 = gemms[0]
        assert 2 <= len(gemms) <= 4 and all(isinstance(g, BiLoCoGemm) for g in gemms)
        assert all(g.K == g0.K and g.R == g0.R and g.M == g0.M and g.N % 128 == 0 for g in gemms) and g0.R % 32 == 0
        assert all(g.residual is None and not g.fp32_out for g in gemms)
        self.rows = [g.N for g in gemms]
        self.N, self.K, self.R, self.M = sum(self.rows), g0.K, g0.R, g0.M
        dev = g0.W_fp4.device
        cat = torch.cat
        self.W_fp4 = cat([g.W_fp4 for g in gemms], 0).contiguous()
        # (block scales are stored per 128-row block and the re-laid weight per 128-row tile: stacking is concatenation)
        self.W_sf = cat([g.W_sf.view(torch.uint8).reshape(-1) for g in gemms]).view(torch.float8_e4m3fn)
        # (the re-laid weight is stored per 128-row tile, so the stacked copy is the concatenation of the separate ones;
        # launchers on the row-slab schedule hold another layout, so the stack is re-laid here)
        self.W_tiled = _ops.tile_weights(self.W_fp4, self.W_sf)
        self.V = cat([g.V for g in gemms], 0).contiguous()
        self.S = cat([g.S for g in gemms]).contiguous()
        self.U_col32 = cat([g.U_col32 for g in gemms], 0).contiguous()
        with torch.cuda.device(dev):
            ok = [m for m in supported_modes(self.M, self.N, self.K, self.R * len(gemms)) if m != 7]   # (row slabs: one group)
            if mode is None:
                mode = default_mode(self.M, self.R, ok, back_to_back=False)
            assert mode in ok, f"mode {mode} not available for the stacked problem"
            self.mode = mode
            nbytes = scratch_bytes(self.M, self.N, self.K, self.R * len(gemms))
        self.z = torch.zeros(nbytes // 4, device=dev, dtype=torch.float32)
        self.epoch = 0

    status = BiLoCoGemm.status

    def __call__(self, alpha, A_pad, A_sf, X_bf16, out=None, A_rec=None, stacked=False):
        """The per-linear outputs, or (stacked=True) the [M, sum N_g] tensor they are views of."""
        self.epoch += 1
        D = _ops._fused(A_pad, self.W_fp4, A_sf, self.W_sf, alpha, X_bf16, self.V, self.S, self.U_col32, self.z, self.M,
                        self.epoch, self.mode, out=out, A_rec=A_rec, B_tiled=self.W_tiled, group_rows=self.rows)
        D = D.view(-1, self.N)[: self.M]
        return D if stacked else list(D.split(self.rows, dim=1))


class _FP4Only:
    """The NVFP4 GEMM alone (no low-rank term) with the launcher interface of BiLoCoGemm; used by BiLoCoLinear with
    method "fp4" (the NVFP4-only baseline of the reference, biloco/layer.py:4-5)."""

    def __init__(self, W_fp4, W_sf, alpha, M: int, tile_weights: bool = True):
        self.N, self.K, self.M = W_fp4.shape[0], W_fp4.shape[1] * 2, M
        self.W_fp4, self.W_sf, self.alpha = W_fp4, W_sf, alpha
        dev = W_fp4.device
        self.W_tiled = _ops.tile_weights(W_fp4, W_sf) if tile_weights else None
        with torch.cuda.device(dev):
            nbytes = scratch_bytes(M, self.N, self.K, 0)
        self.z = torch.zeros(nbytes // 4, device=dev, dtype=torch.float32)
        self.epoch = 0
        self.residual = None

    def __call__(self, A, A_sf, X_bf16=None, out=None, A_rec=None):
        self.epoch += 1
        return _ops._fused(A, self.W_fp4, A_sf, self.W_sf, self.alpha, None, None, None, None, self.z, self.M, self.epoch,
                           _lib.MODE_COUNTER, C=self.residual, B_tiled=self.W_tiled, out=out, A_rec=A_rec)


def reference(A_fp4, A_sf, W_fp4, W_sf, alpha, X_bf16, V_packed, U_packed, S):
    """Unfused reference: z = S * (X sign(V)^T), y_lr = z sign(U) (bf16), then the FP4 GEMM with y_lr added."""
    z = ops.binary_z_reference(X_bf16, V_packed, S).contiguous()
    y_lr = torch.empty(X_bf16.shape[0], U_packed.shape[1] * 8, device=X_bf16.device, dtype=torch.bfloat16)
    ops.binary_expand_reference(z, U_packed, y_lr)
    return ops.fp4_gemm_residual(A_fp4, W_fp4, A_sf, W_sf, alpha, y_lr)


def time_graph(fn, pre=None, iters: int = 30, batch: int = 64):
    """Median time per launch (us) of fn, replaying a CUDA graph of pre() followed by `batch` launches
    (the reference's timing protocol, biloco/kernel.py:145-168: same operands every launch, so L2-warm).
    This function follows the reference's step by step on purpose (warm-up, capture, 5 untimed replays, `iters` timed
    replays, median): numbers are only comparable with the reference's tables if the protocol is the same."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        if pre:
            pre()
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        if pre:
            pre()
        for _ in range(batch):
            fn()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) / batch * 1e3 for a, b in ev)
    return ts[len(ts) // 2]
