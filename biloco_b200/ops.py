"""torch.ops.biloco.* — the operator names and schemas of the reference's extension (csrc/bindings.cpp:17-48),
implemented as calls into libbiloco_b200.so through ctypes.

Arguments that only exist because of the reference's internal layouts (``Flags``, ``Diag``, ``V_perm``, ``U_rw``,
``Corr``, ``Cnt``) are accepted and ignored. The scratch argument (``Z_scratch`` / ``Ztag`` / ``Zbuf``) must be a
zero-initialised CUDA tensor of at least ``biloco_b200_scratch_bytes`` bytes, reused across calls with an epoch
that increases by one per call (``BiLoCoGemm`` owns it).
"""
import torch

from . import _lib

_SCHEMAS = [
    "fp4_gemm(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha) -> Tensor",
    "fp4_gemm_n64(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha) -> Tensor",
    "fp4_gemm_n128(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha) -> Tensor",
    "fp4_gemm_residual(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha, Tensor C_residual) -> Tensor",
    "biloco_gemm_mode2(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha, Tensor X_bf16, "
    "Tensor V_packed, Tensor S, Tensor U_col32, Tensor Z_scratch, Tensor Flags, Tensor Diag, "
    "Tensor V_perm, Tensor U_rw, int m_rows, int epoch) -> Tensor",
    "biloco_gemm_mode4(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha, Tensor X_bf16, "
    "Tensor V_packed, Tensor S, Tensor U_col32, Tensor Ztag, Tensor Diag, int m_rows, int epoch) -> Tensor",
    "biloco_gemm_mode5(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha, Tensor X_bf16, "
    "Tensor V_packed, Tensor S, Tensor U_col32, Tensor Zbuf, Tensor Corr, Tensor Cnt, int m_rows, int epoch) -> Tensor",
    "binary_z_reference(Tensor X, Tensor V_packed, Tensor S) -> Tensor",
    "binary_expand_reference(Tensor z, Tensor U_packed, Tensor(a!) Y) -> ()",
]

_library = torch.library.Library("biloco", "DEF")
for _s in _SCHEMAS:
    _library.define(_s)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _req(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _check_fp4_operands(A, B, A_sf, B_sf, alpha, n_alpha=1):
    # operand contract of csrc/element_traits.hpp:122-170 and csrc/biloco_gemm.cu:3092
    _req(A.dtype == torch.uint8 and B.dtype == torch.uint8, "A and B must be uint8")
    _req(A.dim() == 3 and A.size(0) == 1, "A must be [1, M, K/2]")
    _req(B.dim() == 2, "B must be [N, K/2]")
    _req(A.size(2) == B.size(1), f"inner dims mismatch: {A.size(2) * 2} vs {B.size(1) * 2}")
    _req(A_sf.dtype == torch.float8_e4m3fn and B_sf.dtype == torch.float8_e4m3fn, "block scales must be float8_e4m3fn")
    _req(alpha.dtype == torch.float32 and alpha.numel() == n_alpha and alpha.is_contiguous(),
         "alpha must be fp32 with one element" if n_alpha == 1 else f"alpha must be contiguous fp32 with {n_alpha} elements")
    _req(A.is_cuda and B.is_cuda and A_sf.is_cuda and B_sf.is_cuda and alpha.is_cuda, "all tensors must be CUDA")
    _req(A.is_contiguous() and B.is_contiguous() and A_sf.is_contiguous() and B_sf.is_contiguous(), "operands must be contiguous")
    rows, K, N = A.size(1), A.size(2) * 2, B.size(0)
    _req(A_sf.numel() >= (rows + 127) // 128 * 128 * (K // 16), "A_sf too small")
    _req(B_sf.numel() >= (N + 127) // 128 * 128 * (K // 16), "B_sf too small")
    return rows, N, K


def _fused(A, B, A_sf, B_sf, alpha, X, V, S, U_col32, scratch, m_rows, epoch, mode, C=None, out=None, B_tiled=None, fp32_out=False,
           A_rec=None, group_rows=None, push=None):
    """One launch of the fused linear. group_rows (list of ints) makes it a stacked launch of several linears that read
    the same activation: V and S hold the groups' ranks one after another, U_col32 each column's own group's words, alpha
    one scale per group (see biloco_b200_fused_linear_grouped)."""
    ng = len(group_rows) if group_rows is not None else 1
    rows, N, K = _check_fp4_operands(A, B, A_sf, B_sf, alpha, ng)
    _req(1 <= m_rows <= rows, "m_rows must be in [1, A.size(1)]")
    R = 0
    if group_rows is not None:
        _req(V is not None and V.size(0) % ng == 0, "grouped launch needs the stacked low-rank factors")
    if V is not None:
        R = V.size(0)
        _req(X.dtype == torch.bfloat16 and X.is_contiguous() and X.dim() == 2 and X.size(0) == m_rows and X.size(1) == K,
             "X_bf16 must be contiguous bf16 [m_rows, K]")
        _req(V.dtype == torch.uint8 and V.is_contiguous() and V.dim() == 2 and V.size(1) == K // 8,
             "V_packed must be contiguous uint8 [R, K/8]")
        _req(S.dtype == torch.bfloat16 and S.is_contiguous() and S.dim() == 1 and S.size(0) == R, "S must be contiguous bf16 [R]")
        _req(U_col32.dtype == torch.int32 and U_col32.is_contiguous() and U_col32.dim() == 2 and U_col32.size(0) == N
             and U_col32.size(1) == (R // ng + 31) // 32, "U_col32 must be contiguous int32 [N, ceil(R/32)]")
    _req(scratch.is_cuda and scratch.is_contiguous(), "scratch must be a contiguous CUDA tensor")
    if B_tiled is not None:
        with torch.cuda.device(A.device):
            want = (_lib.load().biloco_b200_slab_bytes(N, K, 0) if (mode & 0xff) == _lib.MODE_SLAB
                    else _lib.load().biloco_b200_tiled_bytes(N, K))
        _req(B_tiled.is_cuda and B_tiled.is_contiguous() and B_tiled.dtype == torch.uint8 and B_tiled.numel() == want,
             f"tiled weight copy must be a contiguous uint8 CUDA tensor of {want} bytes")
    D = out if out is not None else torch.empty((1, rows, N), device=A.device, dtype=torch.float32 if fp32_out else torch.bfloat16)
    if fp32_out:
        _req(D.dtype == torch.float32, "fp32 output buffer expected")
        mode |= 0x400
    if A_rec is not None:
        want = _lib.load().biloco_b200_act_rec_bytes(m_rows, K)
        _req(A_rec.is_cuda and A_rec.is_contiguous() and A_rec.dtype == torch.uint8 and A_rec.numel() == want and want > 0,
             f"activation record must be a contiguous uint8 CUDA tensor of {want} bytes")
    ptrs = (B.data_ptr(), B_sf.data_ptr(), B_tiled.data_ptr() if B_tiled is not None else None, alpha.data_ptr(), A.data_ptr(), A_sf.data_ptr(),
            A_rec.data_ptr() if A_rec is not None else None, X.data_ptr() if R else None, V.data_ptr() if R else None, U_col32.data_ptr() if R else None,
            S.data_ptr() if R else None, C.data_ptr() if C is not None else None, D.data_ptr(),
            scratch.data_ptr(), scratch.numel() * scratch.element_size())
    with torch.cuda.device(A.device):
        if push is not None:      # (table of the peers' receive buffers, status words, world, rank, slot elements): see parallel.PeerAllReduce
            _req(group_rows is None and fp32_out, "the epilogue push exists for single fp32-output launches")
            rc = _lib.load().biloco_b200_fused_linear_push(*ptrs, m_rows, rows, N, K, R, mode, epoch, push[0], push[1], push[2], push[3],
                                                           push[4], _stream())
        elif group_rows is None:
            rc = _lib.load().biloco_b200_fused_linear_rec(*ptrs, m_rows, rows, N, K, R, mode, epoch, _stream())
        else:
            import ctypes
            gr = (ctypes.c_int * ng)(*[int(g) for g in group_rows])
            rc = _lib.load().biloco_b200_fused_linear_grouped(*ptrs, m_rows, rows, N, K, R // ng, ng, gr, mode, epoch, _stream())
    _lib.check(rc, f"biloco fused linear (mode {mode}, M={m_rows}, N={N}, K={K}, R={R})")
    return D


def fused_linear_act(x, B_slab, N, w_gscale, V, S, U_col32, scratch, epoch, rule, norm_weight=None, eps=1e-6, smooth=None,
                     swiglu=False, C=None, out=None, fp32_out=False, act_out=None):
    """One launch of the fused linear on a RAW bf16 activation (biloco_b200_fused_linear_act): RMS norm or silu(gate) * up,
    smoothing, NVFP4 quantisation and the linear itself. x bf16 [M, K] ([M, 2K] with swiglu), M <= 2; B_slab the row-slab
    copy of the weight; w_gscale fp32 [1]. Returns bf16 (or fp32) [M, N]."""
    _req(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(), "x must be contiguous bf16 [M, K] on a CUDA device")
    M = x.size(0)
    K = x.size(1) // 2 if swiglu else x.size(1)
    _req(1 <= M <= 2, "the raw-activation form takes one or two rows")
    _req(w_gscale.dtype == torch.float32 and w_gscale.numel() == 1, "w_gscale must be fp32 [1]")
    for t, what in ((norm_weight, "norm_weight"), (smooth, "smooth")):
        _req(t is None or (t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() == K), f"{what} must be contiguous bf16 [K]")
    R = 0
    if V is not None:
        R = V.size(0)
        _req(V.dtype == torch.uint8 and V.is_contiguous() and V.dim() == 2 and V.size(1) == K // 8, "V_packed must be contiguous uint8 [R, K/8]")
        _req(S.dtype == torch.bfloat16 and S.is_contiguous() and S.numel() == R, "S must be contiguous bf16 [R]")
        _req(U_col32.dtype == torch.int32 and U_col32.is_contiguous() and tuple(U_col32.shape) == (N, (R + 31) // 32),
             "U_col32 must be contiguous int32 [N, ceil(R/32)]")
    lib = _lib.load()
    with torch.cuda.device(x.device):
        want = lib.biloco_b200_slab_bytes(N, K, 0)
    _req(want > 0 and B_slab.is_cuda and B_slab.dtype == torch.uint8 and B_slab.is_contiguous() and B_slab.numel() == want,
         f"row-slab weight copy must be a contiguous uint8 CUDA tensor of {want} bytes")
    _req(C is None or (C.dtype == torch.bfloat16 and C.is_contiguous() and tuple(C.shape) == (M, N)), "C must be contiguous bf16 [M, N]")
    D = out if out is not None else torch.empty((M, N), device=x.device, dtype=torch.float32 if fp32_out else torch.bfloat16)
    _req(D.is_contiguous() and D.dtype == (torch.float32 if fp32_out else torch.bfloat16) and D.numel() >= M * N, "output buffer")
    with torch.cuda.device(x.device):
        rc = lib.biloco_b200_fused_linear_act(
            B_slab.data_ptr(), w_gscale.data_ptr(), x.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None,
            float(eps), smooth.data_ptr() if smooth is not None else None, 1 if swiglu else 0, _lib.RULES[rule],
            V.data_ptr() if R else None, U_col32.data_ptr() if R else None, S.data_ptr() if R else None,
            C.data_ptr() if C is not None else None, D.data_ptr(), act_out.data_ptr() if act_out is not None else None,
            scratch.data_ptr(), scratch.numel() * scratch.element_size(), M, N, K, R, 0x400 if fp32_out else 0, epoch, _stream())
    _lib.check(rc, f"biloco fused linear on a raw activation (M={M}, N={N}, K={K}, R={R})")
    return D


def tile_weights(B, B_sf):
    """Unit-contiguous copy of the NVFP4 weight (codes [N, K/2] + block scales) that the fused kernel streams fastest."""
    N, K = B.size(0), B.size(1) * 2
    lib = _lib.load()
    nbytes = lib.biloco_b200_tiled_bytes(N, K)
    _req(nbytes > 0, f"cannot tile a weight with N={N} K={K}")
    out = torch.empty(nbytes, device=B.device, dtype=torch.uint8)
    with torch.cuda.device(B.device):
        _lib.check(lib.biloco_b200_tile_weights(B.data_ptr(), B_sf.data_ptr(), out.data_ptr(), N, K, _stream()), "tile_weights")
    return out


def tile_weights_slab(B, B_sf):
    """Row-slab copy of the NVFP4 weight for the row-slab schedule (mode 7, one to four activation rows)."""
    N, K = B.size(0), B.size(1) * 2
    lib = _lib.load()
    with torch.cuda.device(B.device):
        nbytes = lib.biloco_b200_slab_bytes(N, K, 0)
        _req(nbytes > 0, f"the row-slab schedule does not take a weight with N={N} K={K}")
        out = torch.empty(nbytes, device=B.device, dtype=torch.uint8)
        _lib.check(lib.biloco_b200_tile_weights_slab(B.data_ptr(), B_sf.data_ptr(), out.data_ptr(), N, K, 0, _stream()),
                   "tile_weights_slab")
    return out


def _tiled_or_none(t, N, K):
    # The schemas have no argument for the re-laid-out weight. BiLoCoGemm passes it in the slot of one of the
    # reference's own internal-layout tensors (V_perm / Diag / Corr). Whatever else a caller written against the
    # reference puts there (its pack_v_perm bytes, a Diag buffer) is accepted and ignored: only a uint8 tensor of exactly
    # biloco_b200_tiled_bytes(N, K) bytes is taken for the tiled weight.
    if t is None or t.numel() == 0 or t.dtype != torch.uint8 or not t.is_cuda:
        return None
    return t if t.numel() == _lib.load().biloco_b200_tiled_bytes(N, K) else None


def biloco_gemm_mode2(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Z_scratch, Flags, Diag, V_perm, U_rw,
                      m_rows, epoch):
    return _fused(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Z_scratch, m_rows, epoch, _lib.MODE_COUNTER,
                  B_tiled=_tiled_or_none(V_perm, B.size(0), B.size(1) * 2))


def biloco_gemm_mode4(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Ztag, Diag, m_rows, epoch):
    return _fused(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Ztag, m_rows, epoch, _lib.MODE_OWNER,
                  B_tiled=_tiled_or_none(Diag, B.size(0), B.size(1) * 2))


def biloco_gemm_mode5(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Zbuf, Corr, Cnt, m_rows, epoch):
    return _fused(A, B, A_sf, B_sf, alpha, X_bf16, V_packed, S, U_col32, Zbuf, m_rows, epoch, _lib.MODE_CLUSTER,
                  B_tiled=_tiled_or_none(Corr, B.size(0), B.size(1) * 2))


# ---- FP4-only GEMMs (the reference's unfused path and its baselines) ---------------------------------------
# They carry no scratch argument, so a scratch buffer per (device, M, N, K) is kept here with its own epoch.
_gemm_scratch = {}


def _scratch_for(dev, M, N, K):
    key = (dev.index, M, N, K)
    ent = _gemm_scratch.get(key)
    if ent is None or ent[1] > (1 << 20):
        with torch.cuda.device(dev):
            nbytes = _lib.load().biloco_b200_scratch_bytes(M, N, K, 0, 0)
        _req(nbytes > 0, f"fp4 gemm does not support M={M} N={N} K={K}")
        ent = [torch.zeros(nbytes // 4, device=dev, dtype=torch.float32), 0]
        _gemm_scratch[key] = ent
    ent[1] += 1
    return ent[0], ent[1]


def _sf_rows_chunk(A_sf, K, c):
    """Scale bytes of rows 32c..32c+31 moved to rows 0..31 of a fresh 128-row scale tensor."""
    atoms = A_sf.view(torch.uint8).reshape(-1)[: 128 * (K // 16)].view(K // 64, 32, 4, 4)
    out = torch.zeros_like(atoms)
    out[:, :, 0, :] = atoms[:, :, c, :]
    return out.reshape(-1).view(torch.float8_e4m3fn)


def _fp4_gemm(A, B, A_sf, B_sf, alpha, C=None):
    rows, N, K = _check_fp4_operands(A, B, A_sf, B_sf, alpha)
    if C is not None:
        _req(C.dtype == torch.bfloat16 and C.is_contiguous() and C.numel() == rows * N, "C_residual must be contiguous bf16 [M, N]")
    D = torch.empty((1, rows, N), device=A.device, dtype=torch.bfloat16)
    for c in range((rows + 31) // 32):   # the kernel takes up to 32 activation rows per launch
        r0, r1 = 32 * c, min(rows, 32 * c + 32)
        if rows <= 32:
            a, a_sf = A, A_sf
        else:
            a, a_sf = A[:, r0:r1].contiguous(), _sf_rows_chunk(A_sf, K, c)
        scratch, epoch = _scratch_for(A.device, r1 - r0, N, K)
        Cc = None if C is None else C.view(rows, N)[r0:r1]
        _fused(a, B, a_sf, B_sf, alpha, None, None, None, None, scratch, r1 - r0, epoch, _lib.MODE_COUNTER,
               C=Cc, out=D[0, r0:r1])
    return D


def fp4_gemm(A, B, A_sf, B_sf, alpha):
    return _fp4_gemm(A, B, A_sf, B_sf, alpha)


def fp4_gemm_residual(A, B, A_sf, B_sf, alpha, C_residual):
    return _fp4_gemm(A, B, A_sf, B_sf, alpha, C_residual)


def binary_z_reference(X, V_packed, S):
    _req(X.dim() == 2 and X.is_contiguous() and X.dtype == torch.bfloat16, "X must be 2D contiguous bf16")
    _req(V_packed.dim() == 2 and V_packed.is_contiguous() and V_packed.dtype == torch.uint8, "V_packed must be 2D contiguous uint8")
    _req(S.dim() == 1 and S.is_contiguous() and S.dtype == torch.bfloat16, "S must be 1D contiguous bf16")
    _req(X.is_cuda and V_packed.is_cuda and S.is_cuda, "all tensors must be CUDA")
    M, K = X.shape
    R = V_packed.size(0)
    _req(K % 8 == 0 and V_packed.size(1) == K // 8 and S.size(0) == R, "shape mismatch between X, V_packed and S")
    z = torch.empty((M, R), device=X.device, dtype=torch.float32)
    with torch.cuda.device(X.device):
        _lib.check(_lib.load().biloco_b200_binary_z(X.data_ptr(), V_packed.data_ptr(), S.data_ptr(), z.data_ptr(), M, K, R,
                                                    _stream()), "binary_z_reference")
    return z


def binary_expand_reference(z, U_packed, Y):
    _req(z.dim() == 2 and z.is_contiguous() and z.dtype == torch.float32, "z must be 2D contiguous fp32")
    _req(U_packed.dim() == 2 and U_packed.is_contiguous() and U_packed.dtype == torch.uint8, "U_packed must be 2D contiguous uint8")
    _req(Y.dim() == 2 and Y.is_contiguous() and Y.dtype == torch.bfloat16, "Y must be 2D contiguous bf16")
    M, R = z.shape
    N = Y.size(1)
    _req(N % 8 == 0 and U_packed.size(0) == R and U_packed.size(1) == N // 8 and Y.size(0) == M, "shape mismatch between z, U_packed and Y")
    with torch.cuda.device(z.device):
        _lib.check(_lib.load().biloco_b200_binary_expand(z.data_ptr(), U_packed.data_ptr(), Y.data_ptr(), M, N, R, _stream()),
                   "binary_expand_reference")


for _name, _fn in [("fp4_gemm", fp4_gemm), ("fp4_gemm_n64", fp4_gemm), ("fp4_gemm_n128", fp4_gemm),
                   ("fp4_gemm_residual", fp4_gemm_residual), ("biloco_gemm_mode2", biloco_gemm_mode2),
                   ("biloco_gemm_mode4", biloco_gemm_mode4), ("biloco_gemm_mode5", biloco_gemm_mode5),
                   ("binary_z_reference", binary_z_reference), ("binary_expand_reference", binary_expand_reference)]:
    _library.impl(_name, _fn, "CUDA")
