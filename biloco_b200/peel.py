"""Binary low-rank decomposition  W ~ U diag(alpha) V^T + R  with U, V in {+-1}.

Host-side (PyTorch) operand generator for the fused kernel: greedy rank-one sign peeling followed by a joint
least-squares refit of the coefficients. Same algorithm, seeding and operation order as the reference's
``biloco/peel.py`` (binary_peel :14-42, refit_alphas :45-58, decompose :61-66), so that with the same seed and
device the factors coincide; tests/golden pins this on CPU.
"""
import torch

_seed = 42


def set_peel_seed(seed: int):
    """Seed of the random sign initialisation (every binary_peel call restarts the stream from it)."""
    global _seed
    _seed = int(seed)


def _sgn(t: torch.Tensor) -> torch.Tensor:
    s = torch.sign(t)
    s[s == 0] = 1.0
    return s


@torch.no_grad()
def binary_peel(W: torch.Tensor, r: int, T: int = 5, generator: torch.Generator = None):
    """Peel r sign atoms off W. Atom i: random signs v; T rounds of u = sgn(R v), v = sgn(R^T u);
    alpha = u^T R v / (m n); R <- R - alpha u v^T. Returns U (m, r), V (n, r), alpha (r,), R."""
    m, n = W.shape
    dev, dt = W.device, W.dtype
    gen = generator if generator is not None else torch.Generator(device=dev).manual_seed(_seed)
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
