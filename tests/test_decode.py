"""Decoder harness around the kernel-backed layers: host logic on CPU, decode steps on GPU."""
import numpy as np
import pytest
import torch

from biloco_b200 import decode
from biloco_b200.layer import BiLoCoLinear
from biloco_b200.model import replace_linears


def test_synthetic_quantize_replaces_every_linear_and_counts_bytes():
    c = decode.PRESETS["tiny"]
    model = decode.Decoder(c, device="cpu", meta=True)
    n = decode.synthetic_quantize(model, rank=32, seed=1)
    assert n == 7 * c.layers + 1
    layers = [m for m in model.modules() if isinstance(m, BiLoCoLinear)]
    assert len(layers) == n and all(m.weight is None for m in layers)
    want = 0
    for m in layers:
        K, N = m.in_features, m.out_features
        want += N * K // 2 + N * K // 16 + (N + K) * 32 // 8
        assert m.W_codes.shape == (N, K // 2) and m.V_packed.shape == (32, K // 8) and m.U_packed.shape == (32, N // 8)
    assert decode.linear_bytes(model) == want
    # the presets carry the shapes named for the whole-model configurations
    q = decode.PRESETS["qwen3-4b"]
    assert (q.layers, q.hidden, q.intermediate, q.heads, q.kv_heads, q.head_dim, q.vocab) == (36, 2560, 9728, 32, 8, 128, 151936)
    l = decode.PRESETS["llama3-70b"]
    assert (l.layers, l.hidden, l.intermediate, l.heads, l.kv_heads, l.head_dim, l.vocab) == (80, 8192, 28672, 64, 8, 128, 128256)


@pytest.mark.gpu
def test_decode_step_matches_fake_quant_layers_and_graph_replay():
    torch.manual_seed(0)
    c = decode.PRESETS["tiny"]
    model = decode.Decoder(c, device="cuda", std=0.05)
    layers = replace_linears(model, rank=32)
    for m in layers.values():
        m.quantize(T=2, device="cuda")
    M, P, steps = 3, 5, 6
    g = torch.Generator(device="cuda").manual_seed(1)
    prompt = torch.randint(0, c.vocab, (M, P), device="cuda", generator=g)

    # Reference pass with every linear on the reference's unfused bf16 forward, recording what each linear saw and
    # produced; then every linear's fused forward on exactly those inputs. (End-to-end logits are not compared: a one-ulp
    # difference upstream flips FP4 codes of the next layer's activation, so two correct decoders drift apart.)
    seen = []
    hooks = [m.register_forward_hook(lambda mod, inp, out, n=n: seen.append((n, inp[0].detach().clone(), out.detach().clone())))
             for n, m in layers.items()]
    fwd = BiLoCoLinear.forward
    with torch.no_grad():
        try:
            BiLoCoLinear.forward = BiLoCoLinear.forward_fake_quant
            model.fuse_norm_quant = False          # separate norm kernels, every linear through its own forward
            model.fuse_step = False                # (and the attention step, SwiGLU and residual adds in torch)
            cache = model.new_cache(M, P)
            for t in range(P):
                ref_logits = model.step(prompt[:, t], torch.tensor([t], device="cuda"), cache)
        finally:
            BiLoCoLinear.forward = fwd
            model.fuse_norm_quant = True
            model.fuse_step = True
            for h in hooks:
                h.remove()
        assert torch.isfinite(ref_logits.float()).all() and len(seen) == P * len(layers)
        # the unfused bf16 forward rounds z, alpha * v and both partial products to bf16 (about 3e-3 relative of its own on
        # layers this small, see test_layer_model.py), hence looser bounds than against the fp32-z unfused path
        for n, x, y_ref in seen:
            y = layers[n](x).float().cpu().numpy()
            y_ref = y_ref.float().cpu().numpy()
            assert np.max(np.abs(y - y_ref)) <= 0.02 * np.max(np.abs(y_ref)) + 1e-6, n     # (two bf16 ulps at the maximum)
            assert np.linalg.norm(y - y_ref) <= 1e-2 * np.linalg.norm(y_ref) + 1e-6, n
        cache = model.new_cache(M, P)
        for t in range(P):
            logits = model.step(prompt[:, t], torch.tensor([t], device="cuda"), cache)
        assert torch.isfinite(logits.float()).all()
    # greedy decode: the captured step replays to the same tokens as eager launches (the kernels are bit-reproducible)
    t_graph, _ = decode.greedy_decode(model, prompt, steps, use_graph=True)
    t_eager, _ = decode.greedy_decode(model, prompt, steps, use_graph=False)
    assert torch.equal(t_graph, t_eager)
    assert all(g_.status()[0] == 0 for m in layers.values() for g_ in m._gemms.values())
    # q/k/v and gate/up ran as one stacked launch each
    grouped = [st["grouped"] for st in model._shared.values() if st.get("grouped") is not None]
    assert len(grouped) == 2 * c.layers and all(g_.status()[0] == 0 for g_ in grouped)


@pytest.mark.gpu
@pytest.mark.parametrize("M,H,KVH,D,qk_norm", [(1, 32, 8, 128, True), (3, 4, 2, 64, True), (8, 8, 8, 128, False), (2, 6, 2, 64, False)])
def test_attention_step_kernel_matches_torch_composition(M, H, KVH, D, qk_norm):
    """biloco_b200_decode_attention against the decoder's own torch composition (q/k RMS norm, rotary embedding, cache
    update, masked attention) over several consecutive positions. Tolerances: the rotated key without a norm is
    bit-exact (same fp32 operations); with the norm one bf16 ulp (the sum of squares is taken in another order); the
    attention output 1e-2 of the row maximum (bf16 output, fp32 softmax on both sides)."""
    torch.manual_seed(M * 100 + H)
    c = decode.DecoderConfig(1, H * D, 256, H, KVH, D, 512, qk_norm=qk_norm)
    model = decode.Decoder(c, device="cuda", meta=True)
    b = model.blocks[0]
    if qk_norm:
        b.q_norm.data = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
        b.k_norm.data = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    L = 40
    ca, cb = model.new_cache(M, L), model.new_cache(M, L)
    for t in range(0, L, 3):          # (positions in between stay zero in both caches and take part in the softmax alike)
        pos = torch.tensor([t], device="cuda")
        qkv = torch.randn(M, (H + 2 * KVH) * D, device="cuda").to(torch.bfloat16)
        out = model._attention_step(qkv, b, ca, ca["kv"][0][0], ca["kv"][0][1], pos, H, KVH)
        q, k, v = qkv.split([H * D, KVH * D, KVH * D], dim=-1)
        q, k, v = q.reshape(M, H, D), k.reshape(M, KVH, D), v.reshape(M, KVH, D)
        if qk_norm:
            q, k = decode._rms(q, b.q_norm, c.eps), decode._rms(k, b.k_norm, c.eps)
        cos, sin = cb["cos"].index_select(0, pos), cb["sin"].index_select(0, pos)
        q, k = model._rope(q, cos, sin), model._rope(k, cos, sin)
        kc, vc = cb["kv"][0]
        kc.index_copy_(2, pos, k.unsqueeze(2))
        vc.index_copy_(2, pos, v.unsqueeze(2))
        mask = (cb["positions"] <= pos)[None, None, None, :]
        ref = torch.nn.functional.scaled_dot_product_attention(q.unsqueeze(2).float(), kc.float(), vc.float(), attn_mask=mask,
                                                               enable_gqa=True).reshape(M, H * D)
        ka, kb = ca["kv"][0][0][:, :, t].float(), kc[:, :, t].float()
        if qk_norm:
            assert torch.all((ka - kb).abs() <= 2.0 ** -7 * kb.abs() + 1e-30)
        else:
            assert torch.equal(ka, kb)
        assert torch.equal(ca["kv"][0][1][:, :, t], vc[:, :, t])
        err = (out.float() - ref).abs().max(dim=-1).values
        assert torch.all(err <= 1e-2 * ref.abs().max(dim=-1).values), (t, err)
        cb["kv"][0][0][:, :, t] = ca["kv"][0][0][:, :, t]     # keep the two caches identical for the next position


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,smooth", [(1, 9728, False), (8, 512, True), (32, 1024, False)])
def test_swiglu_quantiser_and_fused_residual(M, K, smooth):
    """The SwiGLU form of the quantiser writes exactly bf16(silu(gate)) * up as torch computes it and quantises it exactly as
    the plain quantiser does; forward_fused(residual=...) adds the residual inside the launch."""
    from biloco_b200 import fp4
    torch.manual_seed(K + M)
    gu = (2 * torch.randn(M, 2 * K, device="cuda")).to(torch.bfloat16)
    sm = (0.5 + torch.rand(K, device="cuda")).to(torch.bfloat16) if smooth else None
    wg = torch.tensor([1e-3], device="cuda")
    a = fp4.quantize_activation(gu, "mse", smooth=sm, w_gscale=wg, rows=M, swiglu=True)
    x = torch.nn.functional.silu(gu[:, :K]) * gu[:, K:]
    bq = fp4.quantize_activation(x.contiguous(), "mse", smooth=sm, w_gscale=wg, rows=M)
    assert torch.equal(a["X"].view(torch.int16), bq["X"].view(torch.int16))
    for k in ("A", "A_sf", "gscale", "alpha", "A_rec"):
        if a[k] is not None:
            assert torch.equal(a[k].view(torch.uint8), bq[k].view(torch.uint8)), k
    N = 256
    layer = BiLoCoLinear.synthetic(K, N, 64, "cuda", seed=7)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    y0 = layer(x).float()
    y1 = layer.forward_fused(gu, residual=res, swiglu=True).float()
    want = y0 + res.float()
    assert torch.all((y1 - want).abs() <= 2.0 ** -7 * want.abs().max())
    assert torch.equal(layer(x).float(), y0)          # the residual does not stick to the launcher


@pytest.mark.gpu
@pytest.mark.parametrize("M", [8, 32])
def test_captured_step_chain_at_full_layer_shapes(M):
    """A few Qwen3-4B-shaped layers (random packed operands) decoded through the captured step: every launch of the chain
    quantiser -> stacked q/k/v -> attention -> quantiser -> o -> quantiser -> stacked gate/up -> quantiser -> down runs
    back to back, each started early behind its predecessor where the launcher allows it. No device-side wait may run
    out (launches whose CTAs must all be resident together, placed beside a predecessor of another cluster shape, once
    did), and the captured step replays to the same tokens as eager launches."""
    c = decode.DecoderConfig(**{**decode.PRESETS["qwen3-4b"].__dict__, "layers": 3, "vocab": 8192})
    torch.manual_seed(0)
    model = decode.Decoder(c, device="cuda", meta=True)
    decode.synthetic_quantize(model, 512, seed=0)
    prompt = torch.randint(0, c.vocab, (M, 3), device="cuda")
    t_graph, sec = decode.greedy_decode(model, prompt, 4, use_graph=True)
    t_eager, _ = decode.greedy_decode(model, prompt, 4, use_graph=False)
    launchers = [g for m in model.modules() if isinstance(m, BiLoCoLinear) for g in m._gemms.values()]
    launchers += [st["grouped"] for st in model._shared.values() if st.get("grouped") is not None]
    assert len(launchers) >= 4 * c.layers + 1
    bad = [(g.N, g.K, g.mode, g.status()[:4]) for g in launchers if g.status()[0] != 0]
    assert not bad, f"device-side waits ran out: {bad}"
    assert torch.equal(t_graph, t_eager)
    assert sec / 4 < 0.05, f"{sec / 4 * 1e3:.1f} ms per step: a wait budget was spent somewhere"
