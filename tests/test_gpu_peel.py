"""The GPU peeling kernels (biloco_b200_binary_peel) against the algorithm of biloco/peel.py:14-42 restated with torch on
the CPU, on the same start vectors: bit for bit where every sum is exact in fp32, and through the algorithm's own
invariants at sizes where the order of the additions matters."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _peel_cpu(W, v0, T):
    """binary_peel with given start vectors (float32, CPU; true divisions)."""
    m, n = W.shape
    r = v0.shape[0]
    R = W.clone()
    U, V, S = torch.empty(m, r), torch.empty(n, r), torch.empty(r)
    sgn = lambda t: torch.where(t < 0, -torch.ones_like(t), torch.ones_like(t))
    for i in range(r):
        v = sgn(v0[i])
        for _ in range(T):
            u = sgn(R @ v)
            v = sgn(R.T @ u)
        a = (u @ R @ v) / torch.tensor(float(m * n))
        U[:, i], V[:, i], S[i] = u, v, a
        R = R - a * torch.outer(u, v)
    return U, V, S, R


def _peel_gpu(lib, W, v0, T):
    m, n = W.shape
    r = v0.shape[0]
    R = W.cuda().contiguous().clone()
    v0 = v0.cuda().contiguous()
    U = torch.empty(m, r, device="cuda")
    V = torch.empty(n, r, device="cuda")
    S = torch.empty(r, device="cuda")
    nb = lib.biloco_b200_peel_scratch_bytes(m, n, 0)
    assert nb > 0
    scratch = torch.empty(nb, device="cuda", dtype=torch.uint8)
    rc = lib.biloco_b200_binary_peel(R.data_ptr(), v0.data_ptr(), U.data_ptr(), V.data_ptr(), S.data_ptr(), scratch.data_ptr(), nb,
                                     m, n, r, T, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return U.cpu(), V.cpu(), S.cpu(), R.cpu()


@pytest.mark.parametrize("m,n", [(64, 64), (256, 128), (37, 512)])
def test_peel_exact_sums_bit_for_bit(lib, m, n):
    """Small-integer W: every dot product and the coefficient's numerator are exact in fp32 whatever the order of the additions, so kernel and CPU restatement must agree in every bit, ties
    (sums that are exactly zero take the sign +1) included. Two atoms: the second one works on the updated residual."""
    g = torch.Generator().manual_seed(m * 1000 + n)
    W = torch.randint(-4, 5, (m, n), generator=g).float()
    v0 = torch.randn(2, n, generator=g)
    v0[0, :3] = 0.0
    # (two atoms only for 64 x 64: alpha is then k / 4096 and the updated residual's sums still fit 24 bits)
    r = 2 if m * n == 4096 else 1
    want = _peel_cpu(W, v0[:r], T=3)
    got = _peel_gpu(lib, W, v0[:r], T=3)
    for a, b, name in zip(got, want, "UVSR"):
        assert torch.equal(a, b), name


@pytest.mark.parametrize("m,n,r,T", [(384, 512, 16, 5), (1000, 260, 8, 2), (130, 5120, 6, 5)])
def test_peel_invariants_and_quality(lib, m, n, r, T):
    """Random W: signs are +-1, S[i] is the Frobenius-optimal coefficient of atom i on the residual it was peeled from
    (recomputed in float64), the returned residual is W minus the atoms, the residual norm falls with every atom, and the
    final residual is as small as the CPU restatement's on the same start vectors (the greedy paths may part ways where a
    sum is within rounding of zero, so the norms are compared, not the signs)."""
    g = torch.Generator().manual_seed(7 * m + n + r)
    W = (torch.randn(m, n, generator=g) * 0.02)
    W[:, :4] *= 10
    v0 = torch.randn(r, n, generator=g)
    U, V, S, R = _peel_gpu(lib, W, v0, T)
    assert torch.equal(U.abs(), torch.ones_like(U)) and torch.equal(V.abs(), torch.ones_like(V))
    Rd = W.double()
    norms = [float(Rd.norm())]
    for i in range(r):
        u, v = U[:, i].double(), V[:, i].double()
        a = float(u @ Rd @ v) / (m * n)
        assert abs(a - float(S[i])) <= 1e-5 * abs(a) + 1e-9, (i, a, float(S[i]))
        assert a >= 0                      # v = sgn(R^T u) makes u^T R v = sum |R^T u| >= 0
        Rd = Rd - float(S[i]) * torch.outer(u, v)
        norms.append(float(Rd.norm()))
    assert all(b <= a + 1e-9 for a, b in zip(norms, norms[1:]))
    assert float((R.double() - Rd).abs().max()) <= 1e-6 * float(W.abs().max()) * r
    _, _, _, R_cpu = _peel_cpu(W, v0, T)
    assert abs(float(R.norm()) - float(R_cpu.norm())) <= 1e-2 * float(R_cpu.norm())


def test_decompose_on_device_runs_the_kernels_and_reconstructs():
    from biloco_b200 import peel
    torch.manual_seed(0)
    W = (torch.randn(512, 768, device="cuda") * 0.02)
    peel.set_peel_seed(42)
    U, V, S, R = peel.decompose(W, r=32, T=5)
    assert U.shape == (512, 32) and V.shape == (768, 32) and U.is_cuda
    assert torch.allclose(W, (U * S) @ V.T + R, atol=1e-5)
    assert float(R.norm()) < float(W.norm())
    # same seed, same result (the kernels add in a fixed order)
    peel.set_peel_seed(42)
    U2, V2, S2, R2 = peel.decompose(W, r=32, T=5)
    assert torch.equal(U, U2) and torch.equal(V, V2) and torch.equal(S, S2) and torch.equal(R, R2)
