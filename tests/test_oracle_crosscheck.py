"""Cross-check of the oracle's NVFP4 quantiser against an independent implementation that is installed here: vLLM's
``nvfp4_emulation_utils`` (imported, not copied). It covers the format itself (E2M1 rounding with its tie rule, E4M3
block scales, the fp32 tensor scale aimed at 448) for the plain "static_6" rule. What stays unpinned is what only the
absent ``fouroversix`` package defines: the "mse" choice between the 4- and the 6-scaled candidate, its tie-break, and
the tensor-scale target of 256 for the 4/6 rules."""
import numpy as np
import pytest
import torch

from oracle import biloco_oracle as orc

vllm_ref = pytest.importorskip("vllm.model_executor.layers.quantization.utils.nvfp4_emulation_utils")


def _activation(rows, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    x[:, rng.permutation(K)[: max(1, K // 100)]] *= 20          # 1 % outlier channels
    return orc.bf16_round(x)


@pytest.mark.parametrize("rows,K,seed", [(1, 5120, 0), (8, 2560, 1), (32, 1024, 2)])
def test_static_6_agrees_with_vllm_emulation(rows, K, seed):
    x = _activation(rows, K, seed)
    codes, sf, gs = orc.nvfp4_quantize(x, "static_6")
    # vLLM's convention: the ENCODE scale 448 * 6 / amax, i.e. the reciprocal of the oracle's decode scale
    amax = np.float32(np.abs(x).max())
    enc = torch.tensor(np.float32(448.0 * 6.0) / amax, dtype=torch.float32)
    assert abs(float(gs) * float(enc) - 1.0) < 1e-6
    q_ref, sf_ref = vllm_ref.ref_nvfp4_quant(torch.from_numpy(x), enc, 16)
    # block scales: vLLM multiplies by reciprocals where the oracle divides, so a value on an E4M3 rounding boundary may
    # fall to the neighbouring code; everywhere else the bytes are the same
    sf_mine = orc.e4m3_decode(sf).reshape(rows, K // 16)
    sf_theirs = sf_ref.numpy().reshape(rows, K // 16)
    same_sf = sf_mine == sf_theirs
    assert same_sf.mean() > 0.995
    assert np.all(np.abs(sf_mine - sf_theirs) <= 0.125 * np.maximum(sf_mine, sf_theirs) + 1e-12)    # at most one E4M3 step
    # codes, on the blocks whose scale agrees: the same E2M1 value except at rounding ties of x / d (reciprocal vs division)
    unpacked = np.empty((rows, K), np.uint8)
    unpacked[:, 0::2], unpacked[:, 1::2] = codes & 15, codes >> 4
    mine = orc.e2m1_decode(unpacked)
    theirs = q_ref.numpy()
    blk = np.repeat(same_sf, 16, axis=1)
    assert (mine[blk] == theirs[blk]).mean() > 0.999
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
    step = np.abs(np.searchsorted(grid, np.abs(mine[blk])) - np.searchsorted(grid, np.abs(theirs[blk])))
    assert step.max() <= 1                                        # never further than the neighbouring E2M1 value


def test_e2m1_tie_rule_agrees_with_vllm_emulation():
    """Exactly on the midpoints between representable values both round to the even mantissa."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -1.25, -2.5, -5.0, 0.0, 6.0, 7.5], np.float32)
    mine = orc.e2m1_decode(orc.e2m1_encode(ties))
    theirs = vllm_ref.cast_to_fp4(torch.from_numpy(np.clip(ties, -6, 6).copy())).numpy()
    assert np.array_equal(mine, theirs)


def test_dequantise_agrees_with_vllm_emulation():
    """Codes + block scales (atom layout) + tensor scale -> values: the oracle's decode against vLLM's."""
    x = _activation(4, 512, 5)
    codes, sf, gs = orc.nvfp4_quantize(x, "mse")
    mine = orc.nvfp4_dequantize(codes, sf, gs)
    sw = orc.sf_swizzle(sf, 512)
    theirs = vllm_ref.dequantize_to_dtype(torch.from_numpy(codes), torch.from_numpy(sw).view(torch.float8_e4m3fn).reshape(128, -1),
                                          torch.tensor(1.0 / float(gs), dtype=torch.float32).reciprocal().reshape(()), torch.float32,
                                          16, True)
    assert np.allclose(mine, theirs.numpy()[:4], rtol=1e-6, atol=0)
