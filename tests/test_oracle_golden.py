"""The CPU oracle against vectors produced by running the reference's own Python (tests/golden/make_golden.py)."""
import numpy as np

from oracle import biloco_oracle as orc


def test_pack_signs_matches_reference(golden):
    assert np.array_equal(orc.pack_signs(golden["signs_in"]), golden["signs_packed"])
    assert np.array_equal(orc.pack_signs(golden["u_signs"]), golden["u_packed"])
    # zero counts as +1, and unpack inverts pack for +-1 inputs
    assert golden["signs_packed"][0, 0] & 0x1F == 0x1F
    assert np.array_equal(orc.unpack_signs(golden["u_packed"]), golden["u_signs"])


def test_pack_u_col32_matches_reference(golden):
    out = orc.pack_u_col32(golden["u_packed"], n_cols=24, rank=40)
    assert out.dtype == np.int32 and np.array_equal(out, golden["u_col32"])


def test_sf_bytes_matches_reference(golden):
    for rows, k, want in golden["sf_bytes_cases"]:
        assert orc.nvfp4_sf_bytes(int(rows), int(k)) == int(want)


def test_sf_swizzle_roundtrip_and_atom_layout():
    rng = np.random.default_rng(0)
    rows, K = 200, 320
    sf = rng.integers(0, 255, (rows, K // 16), dtype=np.uint8)
    sw = orc.sf_swizzle(sf, K)
    assert sw.size == orc.nvfp4_sf_bytes(rows, K)
    assert np.array_equal(orc.sf_unswizzle(sw, rows, K), sf)
    # spot-check the documented formula: row 37, block 6 of the first row-block
    r, c = 37, 6
    off = ((r // 128) * ((K // 16 + 3) // 4) + c // 4) * 512 + (r % 32) * 16 + (r // 32 % 4) * 4 + c % 4
    assert sw[off] == sf[r, c]
    # and of the second row-block
    r = 150
    off = ((r // 128) * ((K // 16 + 3) // 4) + c // 4) * 512 + (r % 32) * 16 + (r // 32 % 4) * 4 + c % 4
    assert sw[off] == sf[r, c]


def test_e2m1_codec_exhaustive():
    # decode table and nearest-even rounding checked against a brute-force search over the grid
    grid = orc.E2M1_VALUES.astype(np.float64)
    xs = np.concatenate([np.linspace(-7, 7, 2801), grid, -grid, (grid[1:] + grid[:-1]) / 2, -(grid[1:] + grid[:-1]) / 2])
    codes = orc.e2m1_encode(xs.astype(np.float32))
    for x, c in zip(xs, codes):
        a = min(abs(float(np.float32(x))), 6.0)
        d = np.abs(grid - a)
        best = np.flatnonzero(d == d.min())
        want = best[0] if len(best) == 1 else [b for b in best if b % 2 == 0][0]   # ties -> even code
        assert (c & 7) == want, (x, c, want)
        assert (c >> 3) == int(np.signbit(np.float32(x)))
    assert np.array_equal(orc.e2m1_decode(np.arange(16)), np.concatenate([orc.E2M1_VALUES, -orc.E2M1_VALUES]))


def test_e4m3_codec():
    b = np.arange(256, dtype=np.uint8)
    v = orc.e4m3_decode(b)
    finite = np.isfinite(v) & (v >= 0)
    assert np.array_equal(orc.e4m3_encode(v[finite]), b[finite] & 0x7F | (b[finite] & 0x80) * 0)  # non-negative round-trip
    assert orc.e4m3_decode(orc.e4m3_encode(np.array([1e9], np.float32)))[0] == 448.0            # saturates
    assert orc.e4m3_decode(orc.e4m3_encode(np.array([0.0019531251], np.float32)))[0] == 2.0 ** -9  # smallest subnormal


def test_quantiser_properties():
    rng = np.random.default_rng(1)
    x = orc.bf16_round(rng.standard_normal((5, 256)))
    x[:, 7] *= 20
    for rule in orc.RULES:
        p, sf, gs = orc.nvfp4_quantize(x, rule)
        assert p.shape == (5, 128) and sf.shape == (5, 16)
        dq = orc.nvfp4_dequantize(p, sf, gs)
        # block error bounded by half the largest grid step (2 -> step between 4 and 6) times the block scale
        d = (orc.e4m3_decode(sf).astype(np.float64) * float(gs))[..., None]
        err = np.abs(dq.reshape(5, 16, 16) - x.reshape(5, 16, 16))
        assert np.all(err <= 1.0 * d + 1e-12) or rule != "static_6"
        assert float(np.max(np.abs(dq))) <= float(np.max(np.abs(x))) * 1.13
    # mse never has a larger per-block squared error than static_6 or static_4 with the same tensor scale
    gs = orc.nvfp4_global_scale(x, "mse")
    e = {}
    for rule in orc.RULES:
        p, sf, _ = orc.nvfp4_quantize(x, rule, global_scale=gs)
        e[rule] = ((orc.nvfp4_dequantize(p, sf, gs) - x) ** 2).reshape(5, 16, 16).sum(-1)
    assert np.all(e["mse"] <= np.minimum(e["static_6"], e["static_4"]) * (1 + 1e-5) + 1e-12)
    # all-zero input
    p, sf, gs = orc.nvfp4_quantize(np.zeros((2, 64), np.float32), "mse")
    assert gs == 1.0 and not p.any() and not sf.any()


def test_layer_forward_matches_reference_layer(golden):
    """oracle.layer_forward against BiLoCoLinear.forward of the reference (run with the oracle quantiser plugged
    in for the missing fouroversix package)."""
    y = orc.layer_forward(golden["layer_x"], golden["layer_smooth"], golden["layer_V_scaled"], golden["layer_U_T"],
                          golden["layer_weight_fp4"], golden["layer_bias"], act_rule="mse")
    ref = golden["layer_y"]
    # torch accumulates its bf16 matmuls in fp32 in an unspecified order: allow one bf16 ulp of the largest value
    assert np.max(np.abs(y - ref)) <= 2.0 ** -7 * np.max(np.abs(ref))
    assert np.linalg.norm(y - ref) <= 2e-3 * np.linalg.norm(ref)


def test_torch_layer_matches_reference_layer(golden):
    """The timed CPU baseline (torch bf16 matmuls) is the same computation."""
    layer = orc.TorchLayer(golden["layer_smooth"], golden["layer_V_scaled"], golden["layer_U_T"], golden["layer_weight_fp4"],
                           golden["layer_bias"], "mse")
    y, ref = layer(golden["layer_x"]), golden["layer_y"]
    assert np.max(np.abs(y - ref)) <= 2.0 ** -7 * np.max(np.abs(ref))


def test_unfused_vs_exact_composition():
    p = orc.random_problem(3, 512, 256, 64, scales="random", seed=5)
    a = (p["A_pad"], p["A_sf"], p["W"], p["W_sf"], 0.37, p["X"], p["V_packed"], p["U_packed"], p["S"])
    y_ref = orc.reference_unfused(*a, M=3)
    y_ex = orc.fused_exact(*a, M=3)
    assert y_ref.shape == (3, 256)
    assert np.max(np.abs(y_ref - y_ex)) <= 2 * 2.0 ** -8 * np.max(np.abs(y_ex))
    # zero block scales isolate the low-rank term (scripts/problem.py:9-10)
    p0 = orc.random_problem(2, 256, 128, 32)
    y0 = orc.reference_unfused(p0["A_pad"], p0["A_sf"], p0["W"], p0["W_sf"], 1.0, p0["X"], p0["V_packed"], p0["U_packed"], p0["S"], M=2)
    z = orc.binary_z(p0["X"], p0["V_packed"], p0["S"])
    assert np.array_equal(y0, orc.binary_expand(z, p0["U_packed"]))
    # brute-force z on a tiny case
    zz = np.zeros((2, 32))
    for m in range(2):
        for i in range(32):
            zz[m, i] = float(p0["S"][i]) * float(np.sum(p0["V"][i].astype(np.float64) * p0["X"][m].astype(np.float64)))
    assert np.allclose(z, zz, rtol=1e-6, atol=1e-7)
