"""Host-side logic on CPU: packing, operand layouts, decomposition, the torch quantiser against the oracle,
the C-ABI surface, and the stream-K work split (simulated)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from biloco_b200 import _lib, fp4, kernel, peel
from oracle import biloco_oracle as orc

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def test_pack_signs_and_u_col32_against_reference_vectors(golden):
    assert np.array_equal(kernel.pack_signs(torch.from_numpy(golden["signs_in"])).numpy(), golden["signs_packed"])
    up = kernel.pack_signs(torch.from_numpy(golden["u_signs"]))
    assert np.array_equal(up.numpy(), golden["u_packed"])
    assert np.array_equal(kernel.pack_u_col32(up, n_cols=24, rank=40).numpy(), golden["u_col32"])
    # a rank that is a multiple of 32 and has the top bit set somewhere
    rng = np.random.default_rng(3)
    s = np.where(rng.standard_normal((64, 16)) >= 0, 1.0, -1.0).astype(np.float32)
    up = kernel.pack_signs(torch.from_numpy(s))
    assert np.array_equal(kernel.pack_u_col32(up, 16, 64).numpy(), orc.pack_u_col32(up.numpy(), 16, 64))


def test_sf_bytes_and_mode_table(golden):
    for rows, k, want in golden["sf_bytes_cases"]:
        assert kernel.nvfp4_sf_bytes(int(rows), int(k)) == int(want) == fp4.nvfp4_sf_bytes(int(rows), int(k))
    # every (M, rank) of the reference's table has a default mode here, and it is an available one
    for M in (1, 2, 4, 8, 16, 32):
        for r in golden["ranks"]:
            assert kernel.DEFAULT_MODE[M][int(r)] in kernel.supported_modes(M, 5120, 5120, int(r), num_sms=148)
    assert kernel.modes_for(64, 512) == [] and kernel.modes_for(1, 512, K=5000) == []
    # mode 5 (cluster per tile) needs few enough tiles for >= 2 CTAs each and at most 8 rows
    # mode 7 (row slabs) takes one to four rows, K a multiple of 512 and at most 128 weight rows per SM
    assert kernel.supported_modes(1, 5120, 5120, 512, num_sms=148) == [2, 4, 5, 7]
    assert kernel.supported_modes(2, 5120, 5120, 1024, num_sms=148) == [2, 4, 5, 7]
    assert kernel.supported_modes(4, 5120, 5120, 512, num_sms=148) == [2, 4, 5, 7]
    assert kernel.supported_modes(3, 5120, 5120, 256, num_sms=148) == [2, 4, 5, 7]
    assert kernel.supported_modes(4, 5120, 5120, 1024, num_sms=148) == [2, 4, 5]
    assert kernel.supported_modes(8, 5120, 5120, 512, num_sms=148) == [2, 4, 5]
    # three and four rows: rows of at most 8192 elements, at most 16 ranks per z slice (148 // M slices per row), a ring of two stages
    assert 7 in kernel.supported_modes(4, 5120, 5120, 576, num_sms=148) and 7 not in kernel.supported_modes(4, 5120, 5120, 600, num_sms=148)
    assert 7 in kernel.supported_modes(3, 5120, 2560, 512, num_sms=148) and 7 not in kernel.supported_modes(3, 2560, 16384, 512, num_sms=148)
    assert 7 not in kernel.supported_modes(4, 4096, 4096, 512, num_sms=148) and 7 in kernel.supported_modes(2, 4096, 4096, 512, num_sms=148)
    assert kernel.default_mode(4, 512, [2, 4, 5, 7]) == 7 and kernel.default_mode(4, 512, [2, 4, 5, 7], back_to_back=False) == 5
    assert kernel.supported_modes(16, 5120, 5120, 512, num_sms=148) == [2, 4]
    assert kernel.supported_modes(1, 28672, 8192, 512, num_sms=148) == [2, 4]
    assert kernel.supported_modes(1, 5120, 768, 64, num_sms=148) == [2, 4, 5]
    assert kernel.default_mode(1, 512, [2, 4, 5, 7]) == 7 and kernel.default_mode(4, 512, [2, 4, 5]) == 5


def test_peel_matches_reference(golden):
    torch.manual_seed(0)
    W = torch.randn(256, 384)
    peel.set_peel_seed(42)
    U, V, S, R = peel.binary_peel(W, r=32, T=5)
    assert set(U.unique().tolist()) <= {-1.0, 1.0} and set(V.unique().tolist()) <= {-1.0, 1.0}
    assert np.array_equal(kernel.pack_signs(U.T.contiguous()).numpy(), golden["peel_U_packed"])
    assert np.array_equal(kernel.pack_signs(V.T.contiguous()).numpy(), golden["peel_V_packed"])
    assert np.allclose(S.numpy(), golden["peel_S"], rtol=1e-5, atol=1e-7)
    # identities the reference's own test checks (tests/run_tests.py:18-30)
    assert torch.allclose(W, (U * S) @ V.T + R, atol=1e-4)
    assert R.norm() < W.norm()
    S2, R2 = peel.refit_alphas(W, U, V, S)
    assert torch.allclose(W, (U * S2) @ V.T + R2, atol=1e-3)
    assert R2.norm() <= R.norm() + 1e-4
    assert np.allclose(S2.numpy(), golden["peel_S_refit"], rtol=1e-4, atol=1e-6)
    U3, V3, S3, R3 = peel.decompose(W, r=32, T=5)
    assert torch.equal(U3, U) and torch.allclose(S3, S2) and torch.allclose(R3, R2)
    assert np.allclose([float(W.norm()), float(R.norm()), float(R2.norm())], golden["peel_R_norm"], rtol=1e-5)


@pytest.mark.parametrize("rule", ["static_6", "static_4", "mse"])
def test_torch_quantiser_bit_exact_with_oracle(rule):
    rng = np.random.default_rng(11)
    x = orc.bf16_round(rng.standard_normal((9, 320)) * 0.02)
    x[:, 5] *= 20
    x[3] = 0.0                       # an all-zero row -> zero scales and codes
    x[4, :16] = 0.0
    p, sf, gs = orc.nvfp4_quantize(x, rule)
    tp, tsf, tgs = fp4.quantize_nvfp4(torch.from_numpy(x), rule)
    assert np.float32(tgs.item()) == gs
    assert np.array_equal(tp.numpy(), p)
    assert np.array_equal(tsf.view(torch.uint8).numpy(), orc.sf_swizzle(sf, 320))
    assert np.array_equal(fp4.unswizzle_scales(tsf, 9, 320).numpy(), sf)
    dq = fp4.dequantize_nvfp4(tp, tsf, tgs).numpy()
    assert np.allclose(dq, orc.nvfp4_dequantize(p, sf, gs), rtol=1e-6, atol=0)
    fq = fp4.fake_quantize_fp4(torch.from_numpy(x), rule).numpy()
    assert np.allclose(fq, orc.fake_quantize_fp4(x, rule), rtol=1e-6, atol=0)


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "biloco_b200.h")).read()
    declared = set(re.findall(r"\b(biloco_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/biloco_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    assert lib.biloco_b200_abi_version() >= 1
    assert lib.biloco_b200_error_string(0) == b"ok" and b"scratch" in lib.biloco_b200_error_string(-4)
    assert lib.biloco_b200_sf_bytes(128, 5120) == 40960 and lib.biloco_b200_sf_bytes(5120, 5120) == 1638400


def test_host_side_argument_checks(lib):
    # rejected before anything touches a device
    assert lib.biloco_b200_binary_z(None, None, None, None, 1, 64, 8, None) == -1
    assert lib.biloco_b200_act_quant(None, None, None, None, None, None, None, None, 1, 1, 64, 2, None) == -1
    assert lib.biloco_b200_fused_linear(*([None] * 13), 0, 1, 1, 128, 256, 0, 2, 1, None) == -1
    assert lib.biloco_b200_scratch_bytes(33, 5120, 5120, 512, 148) == 0        # M > 32
    assert lib.biloco_b200_scratch_bytes(1, 5120, 5000, 512, 148) == 0         # K % 256 != 0
    assert lib.biloco_b200_scratch_bytes(1, 5128, 5120, 512, 148) > 0          # N % 8 == 0 is enough


def _simulate(ntile, nkt, G):
    """Python restatement of the device-side work split (csrc/schedule.h + the segment loop of the kernel)."""
    T = ntile * nkt
    first = lambda c: c * T // G
    cta_of = lambda u: ((u + 1) * G - 1) // T
    cover = np.zeros((ntile, nkt), dtype=np.int32)
    slots_used = {}
    owners = {}
    for c in range(G):
        u, u1 = first(c), first(c + 1)
        assert u1 > u or T < G
        while u < u1:
            t, k0 = divmod(u, nkt)
            cnt = min(nkt - k0, u1 - u)
            cover[t, k0:k0 + cnt] += 1
            c_first, c_last = cta_of(t * nkt), cta_of(t * nkt + nkt - 1)
            assert c_first <= c <= c_last
            slot = c - c_first
            if cnt == nkt:
                assert c_first == c_last == c
            elif c != c_last:
                assert slot not in slots_used.setdefault(t, set())
                slots_used[t].add(slot)
            else:
                owners[t] = (c, c_last - c_first)           # finisher waits for nc-1 partials
                assert k0 + cnt == nkt
            u += cnt
    assert np.all(cover == 1)
    for t, (c, need) in owners.items():
        assert slots_used.get(t, set()) == set(range(need))
    return max([len(s) for s in slots_used.values()] + [1])


@pytest.mark.parametrize("M,N,K", [(1, 5120, 5120), (32, 5120, 5120), (8, 1024, 5120), (1, 151936, 2560), (16, 28672, 8192),
                                   (4, 8192, 28672), (1, 128, 256), (2, 136, 512), (32, 9728, 2560), (1, 2560, 9728)])
def test_stream_k_split(lib, M, N, K):
    out = (ctypes.c_int * 6)()
    assert lib.biloco_b200_schedule_info(M, N, K, 512, 148, out) == 0
    ntile, nkt, G, max_slots, mma_n, stages = list(out)
    assert ntile == -(-N // 128) and nkt == K // 256 and G == min(148, ntile * nkt)
    assert mma_n == (8 if M <= 8 else 16 if M <= 16 else 32) and stages >= 4
    assert _simulate(ntile, nkt, G) <= max_slots
    need = lib.biloco_b200_scratch_bytes(M, N, K, 512, 148)
    assert need >= 64 + 64 + 4 * ntile + 2 * 32 * 512 * 4 + ntile * max_slots * mma_n * 128 * 4
