"""GPU parity: every operator, called through the C ABI (via torch.ops.biloco / biloco_b200.kernel), against the CPU
oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import biloco_oracle as orc
from tests.gpu_util import check_against_exact, check_against_unfused, dev_problem, oracle_outputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kernel():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from biloco_b200 import kernel as k
    return k


@pytest.mark.parametrize("M,K,R", [(1, 64, 8), (3, 256, 20), (2, 5120, 512), (32, 1024, 64), (1, 72, 5)])
def test_binary_z(kernel, M, K, R):
    p = orc.random_problem(M, K, 128, R, seed=100 + M + R)
    t = dev_problem(p)
    z = kernel.ops.binary_z_reference(t["X"], t["V_packed"], t["S"]).cpu().numpy()
    want = orc.binary_z(p["X"], p["V_packed"], p["S"])
    assert z.shape == (M, R)
    tol = 1e-5 * np.abs(p["S"])[None, :] * np.sum(np.abs(p["X"]), axis=1, keepdims=True) + 1e-12
    assert np.all(np.abs(z - want) <= tol)


@pytest.mark.parametrize("M,N,R", [(1, 128, 8), (3, 264, 40), (2, 5120, 512), (32, 1024, 64)])
def test_binary_expand_and_u_col32(kernel, M, N, R):
    p = orc.random_problem(M, 64, N, R, seed=200 + M + R)
    t = dev_problem(p)
    z = orc.binary_z(p["X"], p["V_packed"], p["S"])
    Y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    kernel.ops.binary_expand_reference(torch.from_numpy(z).cuda(), t["U_packed"], Y)
    want = orc.binary_expand(z, p["U_packed"], True)
    exact = orc.binary_expand(z, p["U_packed"], False)
    y = Y.float().cpu().numpy()
    # one bf16 ulp of slack for fp32 summation order at rounding boundaries
    assert np.all(np.abs(y - want) <= 2.0 ** -7 * np.abs(exact) + 1e-6 * np.sum(np.abs(z), axis=1, keepdims=True))
    col = kernel.pack_u_col32(t["U_packed"], N, R).cpu().numpy()
    assert np.array_equal(col, orc.pack_u_col32(p["U_packed"], N, R))


@pytest.mark.parametrize("rule", ["mse", "static_6", "static_4"])
@pytest.mark.parametrize("M,K,rows,smooth", [(1, 5120, 128, False), (5, 256, 5, True), (32, 2560, 32, True), (8, 1024, 8, False)])
def test_act_quant_bit_exact(kernel, rule, M, K, rows, smooth):
    from biloco_b200 import fp4
    rng = np.random.default_rng(1000 * M + K)
    x = orc.bf16_round(rng.standard_normal((M, K)))
    idx = rng.permutation(K)[: max(1, K // 100)]
    x[:, idx] *= 20                                   # 1 % outlier channels x20
    x = orc.bf16_round(x)
    if M > 2:
        x[1, :32] = 0.0                               # two all-zero blocks
    s = orc.bf16_round(rng.random(K) * 3 + 0.25) if smooth else None
    xs = orc.bf16_round(x / s) if smooth else x
    codes, sf, gs = orc.nvfp4_quantize(xs, rule)
    wg = torch.tensor([0.0123], device="cuda")
    out = fp4.quantize_activation(torch.from_numpy(x).cuda().to(torch.bfloat16), rule,
                                  smooth=torch.from_numpy(s).cuda().to(torch.bfloat16) if smooth else None,
                                  w_gscale=wg, rows=rows)
    assert np.float32(out["gscale"].item()) == gs
    assert np.float32(out["alpha"].item()) == np.float32(np.float32(0.0123) * gs)
    A = out["A"].cpu().numpy()[0]
    assert np.array_equal(A[:M], codes) and not A[M:].any()
    sf_dev = out["A_sf"].view(torch.uint8).cpu().numpy()
    want_sf = np.zeros(orc.nvfp4_sf_bytes(rows, K), np.uint8)
    want_sf[: orc.nvfp4_sf_bytes(M, K)] = orc.sf_swizzle(sf, K) if M <= 128 else 0
    assert np.array_equal(sf_dev, want_sf)
    if smooth:
        assert np.array_equal(out["X"].float().cpu().numpy(), xs)
    # the per-k-tile record holds the same codes (128-byte swizzle: 16-byte chunk c of row r at chunk c ^ (r & 7)) and the
    # same scale atoms, zero beyond row M
    rec = out["A_rec"].cpu().numpy()
    mma_n = 8 if M <= 8 else (16 if M <= 16 else 32)
    rb = mma_n * 128 + 2048
    assert rec.size == (K // 256) * rb
    sw = orc.sf_swizzle(sf, K)
    for kt in range(K // 256):
        tile = rec[kt * rb: kt * rb + mma_n * 128].reshape(mma_n, 8, 16)
        for m in range(mma_n):
            row = codes[m, kt * 128:(kt + 1) * 128].reshape(8, 16) if m < M else np.zeros((8, 16), np.uint8)
            assert np.array_equal(tile[m][np.arange(8) ^ (m & 7)], row), (kt, m)
        atoms = np.zeros(2048, np.uint8)
        src = sw[kt * 2048:(kt + 1) * 2048] if M <= 128 else None
        atoms[: src.size] = src
        assert np.array_equal(rec[kt * rb + mma_n * 128: (kt + 1) * rb], atoms), kt


@pytest.mark.parametrize("rule", ["static_6", "static_4", "mse"])
def test_torch_quantiser_on_device_bit_exact_with_oracle(kernel, rule):
    """The torch quantiser (weights, and the fake-quant forward the layer tests compare with) run ON THE GPU gives the
    oracle's codes and scales bit for bit, also on inputs whose block scales sit on E4M3 rounding boundaries: a CUDA tensor
    divided by a Python number is multiplied by the reciprocal, one ulp off for 6 and 1536, which moved such a scale to its
    neighbour. Built from few distinct bf16 magnitudes so that max|block| / (6 gs) is a short binary fraction often."""
    from biloco_b200 import fp4
    rng = np.random.default_rng(5)
    K = 512
    vals = np.array([0.25, 0.375, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 7.0], np.float32)
    for trial in range(40):
        x = vals[rng.integers(0, 16, (6, K))] * np.where(rng.random((6, K)) < 0.5, -1.0, 1.0).astype(np.float32)
        x *= np.float32(2.0) ** rng.integers(-3, 3, (6, K // 16)).repeat(16, axis=1)
        x[0, 0] = np.float32([3.5, 7.0, 5.0, 3.0][trial % 4]) * 4          # the tensor maximum (6 x 256 does not divide it)
        x = orc.bf16_round(x)
        p, sf, gs = orc.nvfp4_quantize(x, rule)
        tp, tsf, tgs = fp4.quantize_nvfp4(torch.from_numpy(x).cuda(), rule)
        assert np.float32(tgs.item()) == gs
        assert np.array_equal(fp4.unswizzle_scales(tsf, 6, K).view(torch.uint8).cpu().numpy(), np.asarray(sf).view(np.uint8)), trial
        assert np.array_equal(tp.cpu().numpy(), p), trial
        q = fp4.quantize_activation(torch.from_numpy(x).cuda().to(torch.bfloat16), rule)
        assert np.array_equal(q["A"].cpu().numpy()[0], p) and np.float32(q["gscale"].item()) == gs, trial


@pytest.mark.parametrize("M,K,smooth", [(1, 2560, False), (8, 5120, False), (32, 1024, True), (3, 256, False)])
def test_norm_act_quant(kernel, M, K, smooth):
    """RMSNorm folded into the quantiser launch: the normalised activation agrees with the torch composition to one bf16
    unit in the last place (different summation order of the mean square), and codes, block scales, tensor scale and
    the per-consumer decode scales are bit-exact for the activation the kernel itself produced."""
    from biloco_b200 import fp4
    g = torch.Generator(device="cuda").manual_seed(10 * M + K)
    x = (torch.randn(M, K, device="cuda", generator=g) * 3).to(torch.bfloat16)
    w = (torch.rand(K, device="cuda", generator=g) + 0.5).to(torch.bfloat16)
    s = (torch.rand(K, device="cuda", generator=g) * 3 + 0.25).to(torch.bfloat16) if smooth else None
    wg = torch.tensor([0.0123, 0.5, 2.0], device="cuda")
    eps = 1e-6
    out = fp4.quantize_activation(x, "mse", smooth=s, w_gscale=wg, rows=M, norm_weight=w, eps=eps)
    xf = x.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * w
    if smooth:
        ref = ref / s
    xn = out["X"].float()
    ulp = torch.maximum(ref.float().abs(), torch.tensor(1e-30, device="cuda")) * 2.0 ** -7      # one bf16 ulp, at most
    assert bool(((xn - ref.float()).abs() <= ulp * (2.0 if smooth else 1.0)).all())
    assert float((xn != ref.float()).float().mean()) < 0.02                                      # and rarely different at all
    codes, sf, gs = orc.nvfp4_quantize(xn.cpu().numpy(), "mse")
    assert np.float32(out["gscale"].item()) == gs
    assert np.array_equal(out["alpha"].cpu().numpy(), (wg.cpu().numpy() * gs).astype(np.float32))
    assert np.array_equal(out["A"].cpu().numpy()[0][:M], codes)
    want_sf = np.zeros(orc.nvfp4_sf_bytes(M, K), np.uint8)
    want_sf[: orc.nvfp4_sf_bytes(M, K)] = orc.sf_swizzle(sf, K)
    assert np.array_equal(out["A_sf"].view(torch.uint8).cpu().numpy(), want_sf)


@pytest.mark.parametrize("M,K,N,R", [(1, 5120, 5120, 512), (8, 2560, 1024, 128), (32, 1024, 640, 64)])
def test_fused_with_activation_record(kernel, M, K, N, R):
    """The fused linear fed from the quantiser's per-k-tile record (one copy per work unit) gives bit-identical results to
    the tiled-TMA path on the same quantised activation."""
    from biloco_b200 import fp4
    p = orc.random_problem(M, K, N, R, scales="random", seed=5 * M + R)
    t = dev_problem(p)
    q = fp4.quantize_activation(t["X"], "mse", w_gscale=torch.tensor([1e-3], device="cuda"), rows=M)
    g = kernel.BiLoCoGemm(t["W"], t["W_sf"], q["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M)
    y_tma = g(q["A"], q["A_sf"], q["X"]).view(-1, N)[:M].clone()
    y_rec = g(q["A"], q["A_sf"], q["X"], A_rec=q["A_rec"]).view(-1, N)[:M].clone()
    torch.cuda.synchronize()
    assert g.status()[0] == 0
    assert torch.isfinite(y_rec.float()).all() and torch.equal(y_tma.view(torch.int16), y_rec.view(torch.int16))


@pytest.mark.parametrize("M,K,R,rows", [(1, 2560, 128, (1024, 256, 256)), (8, 1024, 64, (384, 128)),
                                        (32, 512, 32, (256, 256, 128, 128)), (16, 1024, 256, (512, 512)),
                                        (2, 5120, 512, (5120, 1024, 1024))])
def test_fused_grouped_launch(kernel, M, K, R, rows):
    """Several linears on one activation as ONE launch (weights stacked along N, every linear with its own ranks and
    decode scale): each linear's columns against the oracle's unfused and exact values for that linear, and against the
    linear's own separate launch; consecutive launches bit-identical."""
    probs = [orc.random_problem(M, K, n, R, scales="random", seed=31 * M + R + i) for i, n in enumerate(rows)]
    for q in probs[1:]:                         # all linears read the first problem's activation
        for k in ("X", "A", "A_pad", "A_sf"):
            q[k] = probs[0][k]
    ts = [dev_problem(q) for q in probs]
    t0 = ts[0]
    singles = [kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M) for t in ts]
    alpha = torch.cat([t["alpha"] for t in ts]).contiguous()
    refs = [oracle_outputs(q, M) for q in probs]
    N = sum(rows)
    for mode in [m for m in kernel.supported_modes(M, N, K, R * len(rows)) if m != 7]:      # (the row-slab schedule takes one group)
        g = kernel.GroupedBiLoCoGemm(singles, mode=mode)
        first = None
        for it in range(3):
            ys = [y.float().cpu().numpy() for y in g(alpha, t0["A_pad"], t0["A_sf"], t0["X"])]
            for i, (y, (y_ref, y_exact)) in enumerate(zip(ys, refs)):
                check_against_unfused(y, y_ref, f"grouped mode {mode} linear {i} launch {it}")
                check_against_exact(y, y_exact, f"grouped mode {mode} linear {i} launch {it}")
            if first is None:
                first = ys
            assert all(np.array_equal(a, b) for a, b in zip(ys, first)), f"grouped mode {mode}: launch {it} differs from launch 0"
        assert g.status()[0] == 0, f"device-side wait ran out: {g.status()[:4]}"
        for i, (sg, t) in enumerate(zip(singles, ts)):
            y1 = sg(t0["A_pad"], t0["A_sf"], t0["X"]).view(-1, rows[i])[:M].float().cpu().numpy()
            check_against_unfused(first[i], y1, f"grouped mode {mode} linear {i} vs its own launch")


def test_grouped_launch_rejects_bad_groups(kernel):
    from biloco_b200 import ops
    p = orc.random_problem(1, 256, 256, 64, scales="random", seed=3)
    t = dev_problem(p)
    g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=1)
    two = torch.cat([t["alpha"], t["alpha"]])
    with pytest.raises(RuntimeError):          # groups must be whole 128-column tiles
        ops._fused(t["A_pad"], t["W"], t["A_sf"], t["W_sf"], two, t["X"], t["V_packed"], t["S"],
                   g.U_col32[:, :1].contiguous(), g.z, 1, 1, 2, group_rows=[192, 64])
    with pytest.raises(RuntimeError):          # and add up to N
        ops._fused(t["A_pad"], t["W"], t["A_sf"], t["W_sf"], two, t["X"], t["V_packed"], t["S"],
                   g.U_col32[:, :1].contiguous(), g.z, 1, 1, 2, group_rows=[128, 256])


@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (4, 256, 1024), (3, 136, 512)])
def test_fp4_gemm_simt(kernel, lib, M, N, K):
    p = orc.random_problem(M, K, N, 8, scales="random", seed=7)
    t = dev_problem(p)
    D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    rc = lib.biloco_b200_fp4_gemm_simt(t["A_pad"].data_ptr(), t["A_sf"].data_ptr(), t["W"].data_ptr(), t["W_sf"].data_ptr(),
                                       t["alpha"].data_ptr(), None, D.data_ptr(), M, N, K, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    want = orc.fp4_gemm(p["A_pad"], p["A_sf"], p["W"], p["W_sf"], 1.0, M=M)
    check_against_unfused(D.float().cpu().numpy(), want, "simt gemm")


# --- tensor-core GEMM alone (R = 0): single unit, several k-tiles split over CTAs, several tiles, ragged N ---
@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (1, 128, 512), (1, 256, 256), (4, 256, 1024), (8, 136, 768),
                                   (16, 384, 2048), (32, 1024, 1024), (2, 2560, 9728)])
def test_fp4_gemm_tensor_core(kernel, M, N, K):
    p = orc.random_problem(M, K, N, 8, scales="random", seed=31 * M + N)
    t = dev_problem(p)
    alpha = torch.tensor([0.25], device="cuda")
    for it in range(2):
        D = kernel.ops.fp4_gemm(t["A"], t["W"], t["A_sf"], t["W_sf"], alpha)
        assert D.shape == (1, M, N)
        y = D.view(-1, N)[:M].float().cpu().numpy()
        want = orc.fp4_gemm(p["A"], p["A_sf"], p["W"], p["W_sf"], 0.25, M=M)
        exact = 0.25 * orc.fp4_gemm_acc(p["A"], p["A_sf"], p["W"], p["W_sf"], M=M)
        check_against_unfused(y, want, f"fp4_gemm call {it}")
        check_against_exact(y, exact, f"fp4_gemm call {it}")


def test_fp4_gemm_residual_and_padded_rows(kernel):
    M, N, K = 5, 256, 512
    p = orc.random_problem(M, K, N, 8, scales="random", seed=77)
    t = dev_problem(p)
    C = orc.bf16_round(np.random.default_rng(0).standard_normal((M, N)) * 10)
    D = kernel.ops.fp4_gemm_residual(t["A"], t["W"], t["A_sf"], t["W_sf"], t["alpha"], torch.from_numpy(C).cuda().to(torch.bfloat16))
    want = orc.fp4_gemm(p["A"], p["A_sf"], p["W"], p["W_sf"], 1.0, C=C, M=M)
    check_against_unfused(D.view(-1, N).float().cpu().numpy(), want, "residual")
    # the reference's FP4-only baseline passes the activation zero-padded to 128 rows
    D = kernel.ops.fp4_gemm_n64(t["A_pad"], t["W"], t["A_sf"], t["W_sf"], t["alpha"])
    assert D.shape == (1, 128, N)
    y = D.view(-1, N).float().cpu().numpy()
    check_against_unfused(y[:M], orc.fp4_gemm(p["A"], p["A_sf"], p["W"], p["W_sf"], 1.0, M=M), "padded")
    assert not y[M:].any()


def _run_fused(kernel, p, M, N, launches=5):
    t = dev_problem(p)
    y_ref, y_exact = oracle_outputs(p, M)
    # the unfused device path agrees with the oracle's unfused composition
    y_unf = kernel.reference(t["A"], t["A_sf"], t["W"], t["W_sf"], t["alpha"], t["X"], t["V_packed"], t["U_packed"], t["S"])
    check_against_unfused(y_unf.view(-1, N)[:M].float().cpu().numpy(), y_ref, "unfused device path")
    R = p["V_packed"].shape[0]
    for mode, tiled in [(m, tl) for m in kernel.supported_modes(M, N, p["X"].shape[1], R) for tl in (True, False)]:
        g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=mode,
                              tile_weights=tiled)
        mode = f"{mode}{'/tiled' if tiled else '/row-major'}"
        y_first = None
        for it in range(launches):                 # consecutive launches reuse the scratch without clearing
            y = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].float()
            torch.cuda.synchronize()
            y = y.cpu().numpy()
            check_against_unfused(y, y_ref, f"mode {mode} launch {it}")
            check_against_exact(y, y_exact, f"mode {mode} launch {it}")
            if y_first is None:
                y_first = y
            assert np.array_equal(y, y_first), f"mode {mode}: launch {it} is not bit-identical to launch 0"
        assert g.status()[0] == 0, f"device-side wait ran out: {g.status()[:4]}"
        g.reset()
        y = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].float().cpu().numpy()
        check_against_unfused(y, y_ref, f"mode {mode} after reset")


@pytest.mark.parametrize("M,N,K,R", [(1, 128, 256, 32), (1, 256, 512, 16), (2, 384, 1024, 40), (8, 1024, 2560, 128),
                                     (32, 640, 768, 64), (16, 136, 256, 256), (4, 384, 1024, 40), (3, 1024, 2560, 200),
                                     (4, 2560, 1536, 128), (3, 136, 512, 8),
                                     # rows of 7168 and 8192 elements: a z-stage thread's span is 28 / 32 activations (the fourth
                                     # round of the row's staging, a sign word per span), 32 k-tiles of activation codes at four rows
                                     (4, 1024, 8192, 64), (1, 1024, 8192, 64), (2, 2048, 8192, 96), (3, 512, 7168, 48)])
def test_fused_small_shapes_random_scales(kernel, M, N, K, R):
    _run_fused(kernel, orc.random_problem(M, K, N, R, scales="random", seed=M * 7 + R), M, N)


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("r", [16, 32, 64, 128, 256, 512, 1024])
def test_fused_reference_protocol(kernel, M, r):
    """tests/run_tests.py:33-45 of the reference: K = N = 5120, zero block scales (isolates the low-rank term),
    five consecutive launches per mode."""
    _run_fused(kernel, orc.random_problem(M, 5120, 5120, r), M, 5120)


@pytest.mark.parametrize("M,r", [(1, 512), (8, 128), (32, 512), (4, 512), (3, 512)])
def test_fused_full_size_random_scales(kernel, M, r):
    _run_fused(kernel, orc.random_problem(M, 5120, 5120, r, scales="random", seed=1000 * M + r), M, 5120, launches=2)


@pytest.mark.parametrize("K,N", [(5120, 1024), (2560, 9728), (9728, 2560)])
def test_fused_other_layer_shapes(kernel, K, N):
    _run_fused(kernel, orc.random_problem(2, K, N, 256, scales="random", seed=K + N), 2, N, launches=2)


def _slab_layout_numpy(W, W_sf, N, K, Rt, kg):
    """The row-slab weight copy stated in numpy: per CTA slab c and super-unit j (kg consecutive k-tiles) the codes of
    MMA row g * Rt + r with the 128-byte swizzle (16-byte chunk ch at chunk ch ^ (r & 7)), then 16 scale bytes per row."""
    nkt = K // 256
    G = (N + Rt - 1) // Rt
    out = np.zeros(G * nkt * Rt * 144, np.uint8)
    sf_rows = orc.sf_unswizzle(W_sf, N, K)                               # [N, K/16]
    for c in range(G):
        for j in range((nkt + kg - 1) // kg):
            nu = min(kg, nkt - j * kg)
            base = (c * nkt + j * kg) * Rt * 144
            for g in range(nu):
                kt = j * kg + g
                for r in range(Rt):
                    n = c * Rt + r
                    if n >= N:
                        continue
                    row = W[n, kt * 128:(kt + 1) * 128].reshape(8, 16)
                    dst = out[base + (g * Rt + r) * 128: base + (g * Rt + r + 1) * 128].reshape(8, 16)
                    dst[np.arange(8) ^ (r & 7)] = row
                    o = base + nu * Rt * 128 + (g * Rt + r) * 16
                    out[o:o + 16] = sf_rows[n, kt * 16:(kt + 1) * 16]
    return out


@pytest.mark.parametrize("N,K", [(128, 512), (384, 1024), (5120, 5120), (2560, 1536), (136, 512)])
def test_slab_weight_layout(kernel, lib, N, K):
    """biloco_b200_tile_weights_slab against the layout stated in numpy, byte for byte."""
    import ctypes
    from biloco_b200 import ops
    p = orc.random_problem(1, K, N, 8, scales="random", seed=N + K)
    t = dev_problem(p)
    info = (ctypes.c_int * 8)()
    assert lib.biloco_b200_slab_info(1, N, K, 8, 0, info) == 0
    got = ops.tile_weights_slab(t["W"], t["W_sf"]).cpu().numpy()
    want = _slab_layout_numpy(p["W"], p["W_sf"], N, K, info[0], info[1])
    assert got.size == want.size and np.array_equal(got, want)


@pytest.mark.parametrize("r", [128, 256, 1024])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_fused_config1_grid_random_scales(kernel, M, r):
    """The batch / rank sweep of the mode table (K = N = 5120) with NON-zero block scales, so that the tensor-core product
    and the low-rank term are both live at every point; every supported schedule, two launches each. (r = 512 is
    covered by test_fused_full_size_random_scales and the other tests.)"""
    _run_fused(kernel, orc.random_problem(M, 5120, 5120, r, scales="random", seed=77 * M + r), M, 5120, launches=2)


def _column_subset(p, cols):
    """The same problem restricted to the output columns `cols` (a multiple of 8 of them): y[:, n] depends on row n of W and
    column n of U only, so the oracle can check a slice of a layer that is too large to dequantise whole."""
    N = p["W"].shape[0]
    K = p["W"].shape[1] * 2
    q = dict(p)
    q["W"] = p["W"][cols]
    sf = orc.sf_unswizzle(p["W_sf"], N, K)[cols]
    q["W_sf"] = orc.sf_swizzle(sf, K)
    q["U"] = p["U"][:, cols]
    q["U_packed"] = orc.pack_signs(q["U"])
    return q


@pytest.mark.parametrize("r", [512, 1024])
@pytest.mark.parametrize("K,N", [(8192, 8192), (8192, 28672), (28672, 8192)])
def test_fused_config3_large_shapes(kernel, K, N, r):
    """Large-shape, large-batch linears (M = 32, r in {512, 1024}, non-zero scales), every supported schedule: the whole
    output against the device's unfused composition (itself checked against the oracle at the smaller sizes), and three
    256-column slices (first tile, a slice that straddles tiles in the middle, the last columns) against the CPU oracle's
    unfused and exact values."""
    M = 32
    p = orc.random_problem(M, K, N, r, scales="random", seed=K // 64 + N // 128 + r)
    t = dev_problem(p)
    y_unf = kernel.reference(t["A"], t["A_sf"], t["W"], t["W_sf"], t["alpha"], t["X"], t["V_packed"], t["U_packed"], t["S"])
    y_unf = y_unf.view(-1, N)[:M].float().cpu().numpy()
    slices = [np.arange(0, 256), np.arange(N // 2 - 64, N // 2 + 192), np.arange(N - 256, N)]
    refs = [oracle_outputs(_column_subset(p, c), M) for c in slices]
    for c, (y_ref, _) in zip(slices, refs):
        check_against_unfused(y_unf[:, c], y_ref, f"unfused device path, columns {c[0]}..")
    for mode in kernel.supported_modes(M, N, K, r):
        g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=mode)
        y0 = None
        for it in range(2):
            y = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].float().cpu().numpy()
            check_against_unfused(y, y_unf, f"config 3 K={K} N={N} r={r} mode {mode} launch {it}")
            for c, (y_ref, y_exact) in zip(slices, refs):
                check_against_unfused(y[:, c], y_ref, f"config 3 K={K} N={N} r={r} mode {mode} columns {c[0]}..")
                check_against_exact(y[:, c], y_exact, f"config 3 K={K} N={N} r={r} mode {mode} columns {c[0]}..")
            y0 = y if y0 is None else y0
            assert np.array_equal(y, y0)
        assert g.status()[0] == 0, f"device-side wait ran out: {g.status()[:4]}"
        del g


@pytest.mark.parametrize("mode", [2, 5, 7])
def test_fused_directly_after_relayout(kernel, lib, mode):
    """Re-layout kernels (tile_weights / tile_weights_slab / pack_u_col32) followed by the fused launch with NOTHING in
    between on the stream: the fused kernels read static operands ahead of their dependency wait when launched with
    programmatic stream serialization, so the library issues the first launch after a re-layout as a plain one. Called
    through the C ABI, repeatedly, on fresh buffers each time."""
    from biloco_b200 import _lib
    M, K, N, R = 1, 5120, 5120, 512
    p = orc.random_problem(M, K, N, R, scales="random", seed=41)
    t = dev_problem(p)
    y_ref, _ = oracle_outputs(p, M)
    stream = torch.cuda.current_stream().cuda_stream
    slab = mode == 7
    nbytes = lib.biloco_b200_slab_bytes(N, K, 0) if slab else lib.biloco_b200_tiled_bytes(N, K)
    scratch = torch.zeros(lib.biloco_b200_scratch_bytes(M, N, K, R, 0) // 4, device="cuda", dtype=torch.float32)
    for it in range(4):
        tiled = torch.full((nbytes,), 0x77, device="cuda", dtype=torch.uint8)          # stale bytes a too-early read would see
        ucol = torch.full((N, R // 32), -1, device="cuda", dtype=torch.int32)
        y = torch.zeros(128, N, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        if slab:
            rc = lib.biloco_b200_tile_weights_slab(t["W"].data_ptr(), t["W_sf"].data_ptr(), tiled.data_ptr(), N, K, 0, stream)
        else:
            rc = lib.biloco_b200_tile_weights(t["W"].data_ptr(), t["W_sf"].data_ptr(), tiled.data_ptr(), N, K, stream)
        assert rc == 0
        assert lib.biloco_b200_pack_u_col32(t["U_packed"].data_ptr(), ucol.data_ptr(), N, R, stream) == 0
        rc = lib.biloco_b200_fused_linear(t["W"].data_ptr(), t["W_sf"].data_ptr(), tiled.data_ptr(), t["alpha"].data_ptr(),
                                          t["A_pad"].data_ptr(), t["A_sf"].data_ptr(), t["X"].data_ptr(), t["V_packed"].data_ptr(),
                                          ucol.data_ptr(), t["S"].data_ptr(), None, y.data_ptr(), scratch.data_ptr(),
                                          scratch.numel() * 4, M, 128, N, K, R, mode, it + 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        check_against_unfused(y[:M].float().cpu().numpy(), y_ref, f"mode {mode}, call {it} directly after the re-layout")


def test_reference_layout_arguments_are_ignored(kernel):
    """A caller written against the reference passes ITS internal-layout tensors (pack_v_perm bytes as V_perm, a Diag
    buffer, Corr / Cnt scratch) to the mode operators; they are accepted and ignored, and the result is the same as
    with empty tensors in those slots."""
    M, K, N, R = 2, 5120, 1024, 64
    p = orc.random_problem(M, K, N, R, scales="random", seed=9)
    t = dev_problem(p)
    y_ref, _ = oracle_outputs(p, M)
    ucol = kernel.pack_u_col32(t["U_packed"], N, R)
    a = (t["A_pad"], t["W"], t["A_sf"], t["W_sf"], t["alpha"], t["X"], t["V_packed"], t["S"], ucol)
    z = torch.zeros(kernel.scratch_bytes(M, N, K, R) // 4, device="cuda")
    v_perm = torch.randint(0, 256, (R * 2 * 128 * 4,), device="cuda", dtype=torch.uint8)       # the reference's pack_v_perm size
    flags = torch.zeros(4096, device="cuda", dtype=torch.int32)
    diag = torch.zeros(4096, device="cuda", dtype=torch.int32)
    u_rw = ucol.t().contiguous()
    y2 = kernel.ops.biloco_gemm_mode2(*a, z, flags, diag, v_perm, u_rw, M, 1).view(-1, N)[:M].float().cpu().numpy()
    check_against_unfused(y2, y_ref, "mode 2 with the reference's V_perm / U_rw / Flags / Diag")
    y4 = kernel.ops.biloco_gemm_mode4(*a, z, diag.view(torch.uint8), M, 2).view(-1, N)[:M].float().cpu().numpy()
    check_against_unfused(y4, y_ref, "mode 4 with a Diag buffer")


@pytest.mark.parametrize("M,K,N,R", [(1, 5120, 5120, 512), (2, 5120, 5120, 512), (1, 1024, 2560, 128), (2, 2560, 1024, 40),
                                      (1, 9728, 2560, 256), (1, 512, 640, 0), (1, 8192, 1024, 512)])
@pytest.mark.parametrize("pre", ["plain", "smooth", "norm", "norm+smooth", "swiglu", "swiglu+smooth"])
def test_fused_raw_activation_matches_two_launches(kernel, M, K, N, R, pre):
    """biloco_b200_fused_linear_act (RMS norm / SwiGLU, smoothing, NVFP4 quantisation and the linear in ONE launch, the
    activation quantised by every CTA for itself) against the quantiser launch followed by the fused launch on the same
    schedule: the same bits, call after call, for every scale rule; and the two-launch result is the one the other tests
    pin to the oracle. Activations with outlier channels and an all-zero block."""
    from biloco_b200 import fp4
    if not kernel.supported_modes(M, N, K, R).count(7):
        pytest.skip("shape not on the row-slab schedule")
    g = torch.Generator(device="cuda").manual_seed(1000 * M + K + R)
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.02)
    codes, sf, wgs = fp4.quantize_nvfp4(W, "mse")
    if R > 0:
        V = torch.where(torch.randn(R, K, device="cuda", generator=g) >= 0, 1.0, -1.0)
        U = torch.where(torch.randn(R, N, device="cuda", generator=g) >= 0, 1.0, -1.0)
        Vp, Up = kernel.pack_signs(V), kernel.pack_signs(U)
        S = (torch.randn(R, device="cuda", generator=g) * 0.01).to(torch.bfloat16)
    swiglu = pre.startswith("swiglu")
    x = torch.randn(M, 2 * K if swiglu else K, device="cuda", generator=g)
    x[:, torch.randperm(x.shape[1], device="cuda", generator=g)[: max(1, K // 100)]] *= 20
    x[0, 32:48] = 0.0
    x = x.to(torch.bfloat16).contiguous()
    smooth = (torch.rand(K, device="cuda", generator=g) * 3 + 0.25).to(torch.bfloat16) if "smooth" in pre else None
    norm_w = (torch.rand(K, device="cuda", generator=g) + 0.5).to(torch.bfloat16) if pre.startswith("norm") else None
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    for rule in ("mse", "static_6", "static_4"):
        q = fp4.quantize_activation(x, rule, smooth=smooth, w_gscale=wgs, rows=M, norm_weight=norm_w, eps=1e-5, swiglu=swiglu)
        if R > 0:
            two = kernel.BiLoCoGemm(codes, sf, q["alpha"], Vp, Up, S, M=M, mode=7)
            one = kernel.BiLoCoGemm(codes, sf, q["alpha"], Vp, Up, S, M=M, mode=7)
        else:
            pytest.skip("FP4-only launcher has no row-slab form")
        two.residual = one.residual = res
        act = torch.zeros(2, device="cuda")
        for call in range(3):
            y2 = two(q["A"], q["A_sf"], q["X"]).view(-1, N)[:M].clone()
            y1 = one.raw(x, wgs, rule, norm_weight=norm_w, eps=1e-5, smooth=smooth, swiglu=swiglu, act_out=act).clone()
            torch.cuda.synchronize()
            assert one.status()[0] == 0 and two.status()[0] == 0
            assert torch.equal(act[:1], q["gscale"]) and torch.equal(act[1:], q["alpha"]), (rule, call)
            assert torch.equal(y1.view(torch.int16), y2.view(torch.int16)), (rule, call, float((y1.float() - y2.float()).abs().max()))


def test_tuned_mode_measures_and_caches(kernel):
    """kernel.tuned_mode picks a schedule the shape takes by timing them on this GPU, once per shape; with a quantiser launch
    between the linears (back_to_back=False) the row-slab schedule is not a candidate."""
    M, N, K, R = 1, 1024, 2048, 64
    ok = kernel.supported_modes(M, N, K, R)
    m1 = kernel.tuned_mode(M, N, K, R, back_to_back=True)
    assert m1 in ok
    assert kernel.tuned_mode(M, N, K, R, back_to_back=True) == m1 and (0, M, N, K, R, True) in kernel._TUNED
    m2 = kernel.tuned_mode(M, N, K, R, back_to_back=False)
    assert m2 in ok and m2 != 7


@pytest.mark.parametrize("M,K,N,R,mode", [(32, 5120, 5120, 512, 2), (16, 5120, 5120, 512, 2), (32, 1024, 1024, 128, 2), (32, 2560, 1024, 200, 2),
                                          (24, 256, 640, 72, 2), (32, 5120, 2560, 1024, 2), (8, 5120, 5120, 512, 5), (4, 2048, 1024, 64, 2),
                                          (17, 8192, 1024, 512, 2)])
def test_fused_with_tensor_core_z_launch(kernel, lib, M, K, N, R, mode):
    """The z stage as a tensor-core launch of its own in front of the fused launch (default from 16 rows; forced here for
    the smaller batches): against the oracle's unfused value with non-zero block scales, bit-identical call after call and
    within an ulp-level distance of the in-kernel CUDA-core z stage (same sums, other order of additions). Ranks that are
    not a multiple of 128, a K of four chunks, eight rank blocks."""
    from biloco_b200 import _lib
    if mode not in kernel.supported_modes(M, N, K, R):
        pytest.skip("schedule not available for this shape")
    p = orc.random_problem(M, K, N, R, scales="random", seed=300 + M + R)
    t = dev_problem(p)
    y_ref, _ = oracle_outputs(p, M)
    outs = {}
    try:
        for ztc in (1, 0):
            assert lib.biloco_b200_set_option(_lib.OPT_ZTC, ztc) == 0
            g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=mode)
            ys = []
            for _ in range(4):
                ys.append(g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].clone())
            torch.cuda.synchronize()
            assert g.status()[0] == 0, g.status()[:4]
            assert all(torch.equal(ys[0].view(torch.int16), y.view(torch.int16)) for y in ys[1:])
            check_against_unfused(ys[0].float().cpu().numpy(), y_ref, f"ztc={ztc}")
            outs[ztc] = ys[0].float()
    finally:
        lib.biloco_b200_set_option(_lib.OPT_ZTC, -1)
    assert float((outs[1] - outs[0]).abs().max()) <= 2.0 ** -7 * float(outs[0].abs().max())      # (bf16 outputs: at most an ulp apart)


@pytest.mark.parametrize("M,mode", [(1, 5), (1, 2), (8, 5), (32, 2)])
def test_fused_epilogue_pushes_outputs_to_peer_buffers(kernel, lib, M, mode):
    """Row-parallel use on one GPU: a 'group' of two whose second receive buffer is a local allocation. The fused launch's
    epilogue (biloco_b200_fused_linear_push) must leave {fp32 output bits, call number 1} for every output element in this
    rank's slot of the peer's buffer (set 1 of the two), and the output itself unchanged."""
    import ctypes
    K, N, R = (5120, 5120, 128) if mode == 5 else (2048, 1024, 128)      # (the cluster schedule needs enough tiles)
    if mode not in kernel.supported_modes(M, N, K, R):
        pytest.skip("schedule not available for this shape")
    p = orc.random_problem(M, K, N, R, scales="random", seed=77 + M)
    t = dev_problem(p)
    world, slot = 2, M * N
    nbytes = lib.biloco_b200_peer_buffer_bytes(world, slot)
    bufs = []
    for _ in range(2):
        ptr, h = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        assert lib.biloco_b200_peer_buffer_create(nbytes, ctypes.byref(ptr), h) == 0
        bufs.append(ptr.value)
    table = torch.tensor(bufs, dtype=torch.int64, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=mode)
    g.fp32_out = True
    y_plain = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].clone()
    g.peer_push = (table.data_ptr(), status.data_ptr(), world, 0, slot)
    y_push = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].clone()
    torch.cuda.synchronize()
    assert g.status()[0] == 0
    assert torch.equal(y_plain, y_push)
    # peer buffer: [2 sets][world][slot] words of (value bits, call number); call 1 uses set 1, this rank is sender 0
    words = torch.empty(2 * world * slot, 2, dtype=torch.int32, device="cuda")
    assert lib.biloco_b200_peer_buffer_bytes(world, slot) == words.numel() * 4
    # (the buffer is a raw allocation of the library: copy it into a tensor with the CUDA runtime that torch has loaded)
    rt = ctypes.CDLL("libcudart.so.12")
    assert rt.cudaMemcpy(ctypes.c_void_p(words.data_ptr()), ctypes.c_void_p(bufs[1]), ctypes.c_size_t(words.numel() * 4), 3) == 0    # device to device
    torch.cuda.synchronize()
    mine = words.view(2, world, slot, 2)[1, 0]
    assert torch.equal(mine[:, 0].contiguous().view(torch.float32), y_push.reshape(-1)), "pushed values differ from the outputs"
    assert bool((mine[:, 1] == 1).all()), "call number missing"
    assert not words.view(2, world, slot, 2)[0].any() and not words.view(2, world, slot, 2)[1, 1].any()
    for b in bufs:
        assert lib.biloco_b200_peer_buffer_destroy(b) == 0
