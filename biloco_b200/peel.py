"""Binary low-rank decomposition  W ~ U diag(alpha) V^T + R  with U, V in {+-1}.

Operand generator for the fused kernel: greedy rank-one sign peeling followed by a joint least-squares refit of the
coefficients. Same algorithm and seeding as the reference's ``biloco/peel.py`` (binary_peel :14-42, refit_alphas
:45-58, decompose :61-66). On a CUDA device the peeling runs in the library's own kernels (one pass over the residual
per alternation, the previous atom's rank-one update folded into the next atom's first pass: csrc/peel.cu); on the
CPU it is the plain torch restatement, which tests/golden pins to the reference's output.
"""
import torch

from . import _lib

_seed = 42


def set_peel_seed(seed: int):
    """Seed of the random sign initialisation (every binary_peel call restarts the stream from it)."""
    global _seed
    _seed = int(seed)


def _sgn(t: torch.Tensor) -> torch.Tensor:
    s = torch.sign(t)
    s[s == 0] = 1.0
    return s


def use_kernel(m: int, n: int) -> bool:
    """True when the library's peeling kernels take an m x n matrix (n a multiple of 4, at most 14336; wider matrices take the torch path)."""
    return bool(_lib.load().biloco_b200_peel_scratch_bytes(m, n, 148))


def _peel_on_device(W, r, T, gen):
    """binary_peel through biloco_b200_binary_peel. The start vectors are drawn one atom at a time from the generator, as
    the reference draws them (biloco/peel.py:31), before the kernels run."""
    m, n = W.shape
    dev = W.device
    lib = _lib.load()
    v0 = torch.empty((r, n), device=dev, dtype=torch.float32)
    for i in range(r):
        v0[i] = torch.randn(n, generator=gen, device=dev, dtype=torch.float32)
    R = W.contiguous().clone()
    U = torch.empty((m, r), device=dev, dtype=torch.float32)
    V = torch.empty((n, r), device=dev, dtype=torch.float32)
    S = torch.empty(r, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        nbytes = lib.biloco_b200_peel_scratch_bytes(m, n, 0)
        scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        _lib.check(lib.biloco_b200_binary_peel(R.data_ptr(), v0.data_ptr(), U.data_ptr(), V.data_ptr(), S.data_ptr(), scratch.data_ptr(),
                                               nbytes, m, n, r, T, torch.cuda.current_stream().cuda_stream), f"binary_peel (m={m}, n={n}, r={r})")
    return U, V, S, R


@torch.no_grad()
def binary_peel(W: torch.Tensor, r: int, T: int = 5, generator: torch.Generator = None):
    """Peel r sign atoms off W. Atom i: random signs v; T rounds of u = sgn(R v), v = sgn(R^T u);
    alpha = u^T R v / (m n); R <- R - alpha u v^T. Returns U (m, r), V (n, r), alpha (r,), R."""
    m, n = W.shape
    dev, dt = W.device, W.dtype
    gen = generator if generator is not None else torch.Generator(device=dev).manual_seed(_seed)
    if W.is_cuda and dt == torch.float32 and use_kernel(m, n):
        return _peel_on_device(W, r, T, gen)
    U = torch.empty((m, r), device=dev, dtype=dt)
    V = torch.empty((n, r), device=dev, dtype=dt)
    alphas = torch.empty(r, device=dev, dtype=dt)
    R = W.clone()
    scale = m * n
    for i in range(r):
        v = _sgn(torch.randn(n, generator=gen, device=dev, dtype=dt))
        u = None
        for _ in range(T):
            u = _sgn(R @ v)
            v = _sgn(R.T @ u)
        a = (u @ R @ v) / scale
        U[:, i], V[:, i], alphas[i] = u, v, a
        R = R - a * torch.outer(u, v)
    return U, V, alphas, R


@torch.no_grad()
def refit_alphas(W, U, V, S):
    """Coefficients that minimise ||W - U diag(a) V^T||_F for fixed signs: (U^T U * V^T V) a = diag(U^T W V),
    with a ridge of 1e-6 times the largest diagonal entry. Returns (a, W - U diag(a) V^T)."""
    Uf, Vf, Wf = U.float(), V.float(), W.float()
    G = (Uf.T @ Uf) * (Vf.T @ Vf)
    rhs = torch.diag(Uf.T @ Wf @ Vf)
    G = G + (1e-6 * G.diagonal().abs().max()) * torch.eye(G.shape[0], device=G.device, dtype=G.dtype)
    a = torch.linalg.solve(G, rhs)
    resid = W - Uf @ torch.diag(a) @ Vf.T
    return a.to(S.dtype), resid.to(W.dtype)


def decompose(W: torch.Tensor, r: int, T: int = 5):
    """binary_peel then refit_alphas. W fp32 (already smoothed if SmoothQuant is used). Returns U, V, alpha, R."""
    U, V, S, _ = binary_peel(W, r=r, T=T)
    S, R = refit_alphas(W, U, V, S)
    return U, V, S, R


def main():
    """python -m biloco_b200.peel [--m 5120 --n 5120 --r 64 --T 5]: decompose a random matrix on the GPU and report the
    time per atom of the peeling kernels, the residual norm, and the same for the torch-operations path (--torch)."""
    global use_kernel
    import argparse
    import json
    import time
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=5120)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--r", type=int, default=64)
    ap.add_argument("--T", type=int, default=5)
    ap.add_argument("--torch", action="store_true", help="also time the torch-operations path on the same GPU")
    a = ap.parse_args()
    assert torch.cuda.is_available(), "needs a CUDA device"
    torch.manual_seed(0)
    W = torch.randn(a.m, a.n, device="cuda") * 0.02
    out = {"m": a.m, "n": a.n, "r": a.r, "T": a.T, "kernel_path": use_kernel(a.m, a.n)}
    binary_peel(W, min(a.r, 2), a.T)
    torch.cuda.synchronize()
    t = time.perf_counter()
    U, V, S, R = binary_peel(W, a.r, a.T)
    torch.cuda.synchronize()
    out["ms_per_atom"] = (time.perf_counter() - t) * 1e3 / a.r
    out["residual_over_W"] = float(R.norm() / W.norm())
    if a.torch:
        keep, use_kernel = use_kernel, (lambda m, n: False)
        binary_peel(W, 2, a.T)
        torch.cuda.synchronize()
        t = time.perf_counter()
        _, _, _, R2 = binary_peel(W, a.r, a.T)
        torch.cuda.synchronize()
        out["torch_ms_per_atom"] = (time.perf_counter() - t) * 1e3 / a.r
        out["torch_residual_over_W"] = float(R2.norm() / W.norm())
        use_kernel = keep
    print(json.dumps(out))


if __name__ == "__main__":
    main()
