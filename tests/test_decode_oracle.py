"""The oracle's restatements of the decode-step pieces against the torch operations they stand for (CPU), and the
library's kernels against the oracle (GPU)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import biloco_oracle as orc


def _bf(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def test_swiglu_and_rms_norm_restate_the_torch_composition():
    rng = np.random.default_rng(0)
    g, u = rng.standard_normal((3, 512)).astype(np.float32) * 3, rng.standard_normal((3, 512)).astype(np.float32)
    want = (F.silu(_bf(g)) * _bf(u)).float().numpy()
    got = orc.swiglu_bf16(g, u)
    # exp may differ in the last place between the two libraries: at most a handful of values one bf16 ulp apart
    assert np.mean(got != want) < 0.01 and np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-30)
    x, w = rng.standard_normal((4, 256)).astype(np.float32), 1 + 0.1 * rng.standard_normal(256).astype(np.float32)
    xb = _bf(x)
    xf = xb.float()
    want = ((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * _bf(w)).float().numpy()
    got = orc.rms_norm_bf16(x, w, 1e-6)
    assert np.mean(got != want) < 0.01 and np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-30)


def test_attention_step_restates_the_torch_composition():
    rng = np.random.default_rng(1)
    M, H, KVH, D, L = 2, 4, 2, 64, 12
    inv = 1.0 / (1e6 ** (np.arange(0, D, 2, dtype=np.float32) / D))
    ang = np.arange(L, dtype=np.float32)[:, None] * inv[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    kc, vc = np.zeros((M, KVH, L, D), np.float32), np.zeros((M, KVH, L, D), np.float32)
    tk, tv = torch.zeros(M, KVH, L, D), torch.zeros(M, KVH, L, D)
    for pos in range(5):
        qkv = orc.bf16_round(rng.standard_normal((M, (H + 2 * KVH) * D)).astype(np.float32))
        got = orc.decode_attention_step(qkv, None, None, 1e-6, cos, sin, pos, kc, vc, H, KVH, D)
        t = torch.from_numpy(qkv)
        q, k, v = t.split([H * D, KVH * D, KVH * D], dim=-1)
        q, k, v = q.reshape(M, H, D), k.reshape(M, KVH, D), v.reshape(M, KVH, D)

        def rope(x):
            x1, x2 = x[..., : D // 2], x[..., D // 2:]
            c, s = torch.from_numpy(cos[pos]), torch.from_numpy(sin[pos])
            return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(torch.bfloat16).float()
        q, k = rope(q), rope(k)
        tk[:, :, pos], tv[:, :, pos] = k, v
        assert np.array_equal(kc[:, :, pos], k.numpy())
        ref = F.scaled_dot_product_attention(q.unsqueeze(2).double(), tk[:, :, : pos + 1].double(), tv[:, :, : pos + 1].double(),
                                             enable_gqa=True).reshape(M, H * D)
        assert np.allclose(got, ref.float().numpy(), rtol=2.0 ** -7, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("M,H,KVH,D,qk_norm", [(1, 8, 2, 128, True), (3, 4, 4, 64, False)])
def test_attention_kernel_against_oracle(M, H, KVH, D, qk_norm):
    from biloco_b200 import decode
    rng = np.random.default_rng(M + H)
    c = decode.DecoderConfig(1, H * D, 256, H, KVH, D, 512, qk_norm=qk_norm)
    model = decode.Decoder(c, device="cuda", meta=True)
    b = model.blocks[0]
    qn = kn = None
    if qk_norm:
        qn, kn = (orc.bf16_round(1 + 0.1 * rng.standard_normal(D).astype(np.float32)) for _ in range(2))
        b.q_norm.data, b.k_norm.data = _bf(qn).cuda(), _bf(kn).cuda()
    L = 24
    cache = model.new_cache(M, L)
    cos, sin = cache["cos"].cpu().numpy(), cache["sin"].cpu().numpy()
    kc, vc = np.zeros((M, KVH, L, D), np.float32), np.zeros((M, KVH, L, D), np.float32)
    for pos in range(0, 10):
        qkv = orc.bf16_round(rng.standard_normal((M, (H + 2 * KVH) * D)).astype(np.float32))
        want = orc.decode_attention_step(qkv, qn, kn, c.eps, cos, sin, pos, kc, vc, H, KVH, D)
        out = model._attention_step(_bf(qkv).cuda(), b, cache, cache["kv"][0][0], cache["kv"][0][1],
                                    torch.tensor([pos], device="cuda"), H, KVH).float().cpu().numpy()
        k_dev = cache["kv"][0][0][:, :, pos].float().cpu().numpy()
        assert np.all(np.abs(k_dev - kc[:, :, pos]) <= 2.0 ** -7 * np.abs(kc[:, :, pos]) + 1e-30)      # (norm: sum order)
        assert np.array_equal(cache["kv"][0][1][:, :, pos].float().cpu().numpy(), vc[:, :, pos])
        kc[:, :, pos] = k_dev                     # keep the two caches identical
        assert np.all(np.abs(out - want) <= 1e-2 * np.abs(want).max(axis=-1, keepdims=True))


@pytest.mark.gpu
def test_swiglu_quantiser_against_oracle():
    """The quantiser's SwiGLU prologue writes the oracle's activation (up to exp's last place) and quantises what it wrote
    exactly as the oracle quantises it."""
    from biloco_b200 import fp4
    rng = np.random.default_rng(5)
    M, K = 4, 1024
    gu = orc.bf16_round(2 * rng.standard_normal((M, 2 * K)).astype(np.float32))
    q = fp4.quantize_activation(_bf(gu).cuda(), "mse", w_gscale=torch.tensor([1e-3], device="cuda"), rows=M, swiglu=True)
    xa = q["X"].float().cpu().numpy()
    want = orc.swiglu_bf16(gu[:, :K], gu[:, K:])
    assert np.mean(xa != want) < 0.01 and np.all(np.abs(xa - want) <= 2.0 ** -7 * np.abs(want) + 1e-30)
    codes, sf, gs = orc.nvfp4_quantize(xa, "mse")
    assert np.array_equal(q["A"].view(-1, K // 2)[:M].cpu().numpy(), codes)
    assert np.float32(q["gscale"].item()) == np.float32(gs)
