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
            cache = model.new_cache(M, P)
            for t in range(P):
                ref_logits = model.step(prompt[:, t], torch.tensor([t], device="cuda"), cache)
        finally:
            BiLoCoLinear.forward = fwd
            model.fuse_norm_quant = True
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
