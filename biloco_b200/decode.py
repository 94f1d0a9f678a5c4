"""Greedy decode of a Llama/Qwen-shaped decoder whose linears are kernel-backed BiLoCoLinear layers.

The decoder is an ordinary ``nn.Module`` built from ``nn.Linear`` layers (q/k/v/o, gate/up/down, lm_head), so the
model-level entry points apply to it unchanged (``biloco_b200.model.quantize_model`` / ``replace_linears``); for
throughput measurements ``synthetic_quantize`` swaps in layers with random packed operands instead of decomposing
random weights. Between the linears the step uses the library's fused launches where the layers allow it (RMSNorm or
SwiGLU inside the quantiser launch, q/k/v and gate/up as one stacked launch each, the attention step as one launch,
residual adds inside the o / down launches); embedding, final argmax and the fall-back paths are plain torch. One decode
step is captured in a CUDA graph and replayed for the prompt and the generated tokens with no host interaction in between.

    python -m biloco_b200.decode --model qwen3-4b --M 1 --prompt 128 --steps 256
    torchrun --nproc-per-node 8 -m biloco_b200.decode --model llama3-70b --M 1 --prompt 512 --steps 128     # tensor parallel

prints one JSON line: tokens/s, ms per step, the linears' algorithmic bytes per step and the fraction of the measured
HBM peak they correspond to (the decode regime streams every weight once per step).
"""
import argparse
import json
import math
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .layer import BiLoCoLinear


@dataclass
class DecoderConfig:
    layers: int
    hidden: int
    intermediate: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    qk_norm: bool = False
    rope_theta: float = 1e6
    eps: float = 1e-6


PRESETS = {
    # shapes of the configurations named in the baseline; random initialisation, no checkpoint involved
    "qwen3-4b": DecoderConfig(36, 2560, 9728, 32, 8, 128, 151936, qk_norm=True),
    "llama3-70b": DecoderConfig(80, 8192, 28672, 64, 8, 128, 128256, rope_theta=5e5, eps=1e-5),
    "tiny": DecoderConfig(2, 256, 512, 4, 2, 64, 512, qk_norm=True),
    # splits over 2 or 4 ranks: column shards of at least 128 rows (whole block-scale atoms), K shards of at least 256
    "tiny-tp": DecoderConfig(2, 256, 1024, 8, 8, 128, 512, qk_norm=True),
}


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class RowParallel(nn.Module):
    """A K-shard of a quantised linear: the local launch returns an fp32 partial sum over all N, one NCCL all-reduce adds
    the ranks' partials, and the sum is rounded to bf16 once (biloco_b200.parallel.ShardedBiLoCoLinear)."""

    def __init__(self, shard: BiLoCoLinear, group=None):
        super().__init__()
        self.shard, self.group, self._impl = shard, group, {}

    def _impl_for(self, M, local_scale):
        from .parallel import ShardedBiLoCoLinear
        key = (M, local_scale)
        if key not in self._impl:
            self._impl[key] = ShardedBiLoCoLinear(self.shard.export_operands(), "row", M, group=self.group, presharded=True,
                                                  local_scale=local_scale)
        return self._impl[key]

    def forward(self, x):
        x2 = x.reshape(-1, self.shard.in_features)
        return self._impl_for(x2.shape[0], False)(x2).reshape(*x.shape[:-1], self.shard.out_features)

    def forward_fused(self, x, residual=None, swiglu=False):
        """The decode-step form: every rank scales its own K-slice (no scale agreement), the residual travels inside rank
        0's partial sum, silu(gate) * up is formed in the quantiser launch. x [M, K_local] (or [M, 2 K_local])."""
        return self._impl_for(x.shape[0], True)(x, residual=residual, swiglu=swiglu)


class Block(nn.Module):
    def __init__(self, c: DecoderConfig, device, dtype, tp: int = 1):
        super().__init__()
        kw = dict(bias=False, device=device, dtype=dtype)
        # tensor parallel over `tp` ranks: q/k/v/gate/up keep N/tp output columns, o/down keep K/tp input columns
        self.q_proj = nn.Linear(c.hidden, c.heads * c.head_dim // tp, **kw)
        self.k_proj = nn.Linear(c.hidden, c.kv_heads * c.head_dim // tp, **kw)
        self.v_proj = nn.Linear(c.hidden, c.kv_heads * c.head_dim // tp, **kw)
        self.o_proj = nn.Linear(c.heads * c.head_dim // tp, c.hidden, **kw)
        self.gate_proj = nn.Linear(c.hidden, c.intermediate // tp, **kw)
        self.up_proj = nn.Linear(c.hidden, c.intermediate // tp, **kw)
        self.down_proj = nn.Linear(c.intermediate // tp, c.hidden, **kw)
        self.input_norm = nn.Parameter(torch.ones(c.hidden, device=device, dtype=dtype))
        self.post_norm = nn.Parameter(torch.ones(c.hidden, device=device, dtype=dtype))
        if c.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(c.head_dim, device=device, dtype=dtype))
            self.k_norm = nn.Parameter(torch.ones(c.head_dim, device=device, dtype=dtype))


class Decoder(nn.Module):
    """Decoder-only transformer for single-token steps over a static KV cache. ``meta=True`` builds the linears without
    storage (their weights are about to be replaced by synthetic quantised layers)."""

    def __init__(self, c: DecoderConfig, device="cuda", dtype=torch.bfloat16, meta=False, std=0.02, tp: int = 1, group=None):
        super().__init__()
        assert c.heads % tp == 0 and c.kv_heads % tp == 0 and c.intermediate % (256 * tp) == 0 and c.vocab % (8 * tp) == 0
        self.c, self.tp, self.group = c, tp, group
        self.fuse_norm_quant, self._shared = True, {}     # (see _normed_linears)
        self.fuse_groups = True                           # q/k/v and gate/up as one stacked launch each
        self.fuse_step = True                             # attention step as one launch; SwiGLU inside the down projection's
                                                          # quantiser launch; residual adds inside the o / down launches
        lin_dev = "meta" if meta else device
        self.embed = nn.Embedding(c.vocab, c.hidden, device=device, dtype=dtype)
        self.blocks = nn.ModuleList(Block(c, lin_dev, dtype, tp) for _ in range(c.layers))
        if meta:      # norm weights are real even when the linears are placeholders
            for b in self.blocks:
                for n in ("input_norm", "post_norm", "q_norm", "k_norm"):
                    if hasattr(b, n):
                        setattr(b, n, nn.Parameter(torch.ones(getattr(b, n).shape, device=device, dtype=dtype)))
        self.norm = nn.Parameter(torch.ones(c.hidden, device=device, dtype=dtype))
        self.lm_head = nn.Linear(c.hidden, c.vocab // tp, bias=False, device=lin_dev, dtype=dtype)     # vocabulary-parallel
        if not meta:
            for m in self.modules():
                if isinstance(m, (nn.Linear, nn.Embedding)):
                    nn.init.normal_(m.weight, std=std)
        else:
            nn.init.normal_(self.embed.weight, std=std)

    def new_cache(self, M, max_len, device=None, dtype=torch.bfloat16):
        c = self.c
        device = device or self.embed.weight.device
        kvh = c.kv_heads // self.tp
        kv = [(torch.zeros(M, kvh, max_len, c.head_dim, device=device, dtype=dtype),
               torch.zeros(M, kvh, max_len, c.head_dim, device=device, dtype=dtype)) for _ in range(c.layers)]
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=device, dtype=torch.float32) / c.head_dim))
        ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        return dict(kv=kv, cos=ang.cos(), sin=ang.sin(), positions=torch.arange(max_len, device=device))

    def _normed_linears(self, h, norm_w, layers, key, stacked=False):
        """[layer(rmsnorm(h) * norm_w) for layer in layers]. When the layers are unsmoothed kernel-backed BiLoCo layers
        the norm, the NVFP4 quantisation and one decode scale per layer come from ONE launch (the activation is the
        same for all of them), followed by ONE stacked fused-linear launch for all of them (fuse_groups; needs equal
        ranks and whole 128-column tiles) or one fused linear per layer; otherwise the plain composition.
        stacked=True returns the outputs side by side as one [M, sum N] tensor instead of a list."""
        from . import fp4
        M = h.shape[0]
        fusable = self.fuse_norm_quant and M <= 32 and all(isinstance(l, BiLoCoLinear) and l.weight is None and not l.smoothed
                                                           and l.rank > 0 for l in layers)
        if not fusable:
            x = _rms(h, norm_w, self.c.eps)
            ys = [l(x) for l in layers]
            return torch.cat(ys, dim=-1) if stacked else ys
        st = self._shared.get((key, M))
        if st is None:
            st = dict(w_gs=torch.cat([l.w_gscale.reshape(1) for l in layers]).contiguous(), q=None)
            self._shared[(key, M)] = st
        q = fp4.quantize_activation(h.contiguous(), fp4.CONFIG_X, w_gscale=st["w_gs"], rows=M, out=st["q"],
                                    norm_weight=norm_w, eps=self.c.eps)
        st["q"] = q
        if self.fuse_groups and 2 <= len(layers) <= 4 and "grouped" not in st:
            from .kernel import GroupedBiLoCoGemm
            ok = all(l.rank == layers[0].rank and l.rank % 32 == 0 and l.out_features % 128 == 0 and l.bias is None for l in layers)
            st["grouped"] = GroupedBiLoCoGemm([l._gemm_for(M, q["alpha"][i:i + 1]) for i, l in enumerate(layers)]) if ok else None
            if ok:                      # the stacked launcher holds its own copies of the operands
                for l in layers:
                    l._gemms.pop(M, None)
        if self.fuse_groups and st.get("grouped") is not None:
            return st["grouped"](q["alpha"], q["A"], q["A_sf"], q["X"], A_rec=q.get("A_rec"), stacked=stacked)
        ys = [l.forward_quantized(q, q["alpha"][i:i + 1]) for i, l in enumerate(layers)]
        return torch.cat(ys, dim=-1) if stacked else ys

    def _attention_step(self, qkv, b, cache, kc, vc, pos, heads, kv_heads):
        """q/k norms, rotary embedding, cache update and attention over the cache for the current position in ONE launch of
        the library (biloco_b200_decode_attention). qkv [M, (heads + 2 kv_heads) * head_dim] -> [M, heads * head_dim]."""
        from . import _lib
        c = self.c
        M = qkv.shape[0]
        out = torch.empty(M, heads * c.head_dim, device=qkv.device, dtype=torch.bfloat16)
        qn = b.q_norm if c.qk_norm else None
        kn = b.k_norm if c.qk_norm else None
        with torch.cuda.device(qkv.device):
            rc = _lib.load().biloco_b200_decode_attention(
                qkv.data_ptr(), qn.data_ptr() if qn is not None else None, kn.data_ptr() if kn is not None else None, float(c.eps),
                cache["cos"].data_ptr(), cache["sin"].data_ptr(), pos.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                M, heads, kv_heads, c.head_dim, kc.shape[2], torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "decode_attention")
        return out

    @staticmethod
    def _rope(x, cos, sin):                  # x [M, H, D]; cos/sin [1, D/2]
        x1, x2 = x[..., : x.shape[-1] // 2].float(), x[..., x.shape[-1] // 2:].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)

    def step(self, tokens, pos, cache):
        """tokens int64 [M], pos int64 device tensor [1] (the position being written), cache from new_cache().
        Returns the logits [M, vocab] of the next token."""
        c = self.c
        M = tokens.shape[0]
        heads, kv_heads = c.heads // self.tp, c.kv_heads // self.tp
        h = self.embed(tokens)
        cos = cache["cos"].index_select(0, pos)
        sin = cache["sin"].index_select(0, pos)
        mask = (cache["positions"] <= pos)[None, None, None, :]
        kc0 = cache["kv"][0][0]
        fuse = (self.fuse_step and h.is_cuda and M <= 32 and c.head_dim in (64, 128) and kc0.dtype == torch.bfloat16
                and kc0.is_contiguous())

        def kernel_layer(l):     # a quantised layer whose launches can take the residual / the gated activation
            if isinstance(l, RowParallel):
                l = l.shard
            return fuse and isinstance(l, BiLoCoLinear) and l.weight is None and l.bias is None and l.rank > 0
        for li, (b, (kc, vc)) in enumerate(zip(self.blocks, cache["kv"])):
            if fuse:
                qkv = self._normed_linears(h, b.input_norm, [b.q_proj, b.k_proj, b.v_proj], (li, "qkv"), stacked=True)
                a = self._attention_step(qkv.contiguous(), b, cache, kc, vc, pos, heads, kv_heads)
            else:
                q, k, v = self._normed_linears(h, b.input_norm, [b.q_proj, b.k_proj, b.v_proj], (li, "qkv"))
                q, k, v = q.view(M, heads, c.head_dim), k.view(M, kv_heads, c.head_dim), v.view(M, kv_heads, c.head_dim)
                if c.qk_norm:
                    q, k = _rms(q, b.q_norm, c.eps), _rms(k, b.k_norm, c.eps)
                q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
                kc.index_copy_(2, pos, k.unsqueeze(2).to(kc.dtype))
                vc.index_copy_(2, pos, v.unsqueeze(2).to(vc.dtype))
                a = F.scaled_dot_product_attention(q.unsqueeze(2), kc, vc, attn_mask=mask, enable_gqa=True)
                a = a.reshape(M, heads * c.head_dim)
            h = b.o_proj.forward_fused(a, residual=h) if kernel_layer(b.o_proj) else h + b.o_proj(a)
            if kernel_layer(b.down_proj):
                gu = self._normed_linears(h, b.post_norm, [b.gate_proj, b.up_proj], (li, "mlp"), stacked=True)
                h = b.down_proj.forward_fused(gu.contiguous(), residual=h, swiglu=True)
            else:
                gate, up = self._normed_linears(h, b.post_norm, [b.gate_proj, b.up_proj], (li, "mlp"))
                h = h + b.down_proj(F.silu(gate) * up)
        logits, = self._normed_linears(h, self.norm, [self.lm_head], (-1, "head"))
        if self.tp > 1:         # every rank gets the whole vocabulary (and takes the same argmax)
            parts = [torch.empty_like(logits) for _ in range(self.tp)]
            dist.all_gather(parts, logits.contiguous(), group=self.group)
            logits = torch.cat(parts, dim=-1)
        return logits


def synthetic_quantize(model: Decoder, rank: int, seed: int = 0):
    """Replace every nn.Linear of the decoder (lm_head included) by a BiLoCoLinear with random packed operands."""
    dev = model.embed.weight.device
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear):
                layer = BiLoCoLinear.synthetic(child.in_features, child.out_features, rank, dev, seed=seed + n)
                if model.tp > 1 and name in ("o_proj", "down_proj"):
                    layer = RowParallel(layer, model.group)
                setattr(parent, name, layer)
                n += 1
    return n


def shard_decoder(full: Decoder, world: int, rank: int, group=None) -> Decoder:
    """The tensor-parallel decoder of `rank` cut out of a single-GPU decoder whose linears are quantised layers: q/k/v,
    gate/up and lm_head keep their rank's output columns (whole heads), o and down their rank's input columns; embedding
    and norm weights are shared. For checking the tensor-parallel step against the single-GPU one on the same operands."""
    from .parallel import shard_column_parallel, shard_row_parallel
    dev = full.embed.weight.device
    tp = Decoder(full.c, device=dev, meta=True, tp=world, group=group)
    tp.fuse_norm_quant, tp.fuse_groups, tp.fuse_step = full.fuse_norm_quant, full.fuse_groups, full.fuse_step
    tp.embed, tp.norm = full.embed, full.norm
    for bt, bf in zip(tp.blocks, full.blocks):
        for n in ("input_norm", "post_norm", "q_norm", "k_norm"):
            if hasattr(bf, n):
                setattr(bt, n, getattr(bf, n))
        for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"):
            setattr(bt, n, BiLoCoLinear.from_operands(shard_column_parallel(getattr(bf, n).export_operands(), world, rank)))
        for n in ("o_proj", "down_proj"):
            setattr(bt, n, RowParallel(BiLoCoLinear.from_operands(shard_row_parallel(getattr(bf, n).export_operands(), world, rank)), group))
    tp.lm_head = BiLoCoLinear.from_operands(shard_column_parallel(full.lm_head.export_operands(), world, rank))
    return tp


def linear_bytes(model: nn.Module):
    """Algorithmic bytes one decode step streams through the linears: codes + block scales + packed U and V signs."""
    total = 0
    for m in model.modules():
        if isinstance(m, BiLoCoLinear):
            K, N, r = m.in_features, m.out_features, m.rank
            total += N * K // 2 + N * K // 16 + N * r // 8 + K * r // 8
    return total


@torch.no_grad()
def greedy_decode(model: Decoder, prompt: torch.Tensor, steps: int, use_graph: bool = True):
    """prompt int64 [M, P] on the model's device. Feeds the prompt one position at a time (filling the cache), then
    generates `steps` tokens greedily. Returns (tokens [M, steps], seconds spent on the generated steps)."""
    dev = prompt.device
    M, P = prompt.shape
    cache = model.new_cache(M, P + steps)
    pos = torch.zeros(1, device=dev, dtype=torch.long)
    nxt = torch.zeros(M, device=dev, dtype=torch.long)
    out = torch.zeros(M, P + steps, device=dev, dtype=torch.long)

    def one_step():
        # the token at position pos: from the prompt while inside it, else the previous step's argmax
        tok = torch.where(pos < P, prompt.index_select(1, pos.clamp(max=P - 1)).squeeze(1), nxt)
        logits = model.step(tok, pos, cache)
        nxt.copy_(logits.float().argmax(dim=-1))
        out.index_copy_(1, pos, nxt.unsqueeze(1))
        pos.add_(1)

    run = one_step
    if use_graph:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            one_step()                       # warm-up outside capture (lazy allocations, kernel launch set-up)
            torch.cuda.synchronize()
            pos.zero_()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                one_step()
        torch.cuda.current_stream().wait_stream(s)
        pos.zero_()
        run = g.replay
    for _ in range(P - 1):                   # positions 0 .. P-2: prompt tokens in, predictions discarded
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):                   # position P-1 predicts the first generated token, and so on
        run()
    e1.record()
    torch.cuda.synchronize()
    return out[:, P - 1:P - 1 + steps].clone(), e0.elapsed_time(e1) * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-4b", choices=sorted(PRESETS))
    ap.add_argument("--M", type=int, default=1, help="sequences decoded together (<= 32)")
    ap.add_argument("--rank", type=int, default=512)
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the preset's)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true", help="eager launches instead of a captured step")
    ap.add_argument("--autotune", action="store_true", help="pick every linear's schedule by measuring it once per shape on this GPU")
    ap.add_argument("--no-fuse", action="store_true", help="separate RMSNorm kernels and one quantiser launch per linear")
    ap.add_argument("--no-step-fusion", action="store_true", help="attention step, SwiGLU and residual adds as separate torch kernels")
    ap.add_argument("--no-groups", action="store_true", help="one fused-linear launch per linear (q, k, v, gate, up separately)")
    args = ap.parse_args()
    assert torch.cuda.is_available(), "decode needs a CUDA device (there is no CPU path)"
    c = PRESETS[args.model]
    if args.layers:
        c = DecoderConfig(**{**c.__dict__, "layers": args.layers})
    # tensor parallel when launched by torchrun: one rank per GPU, q/k/v/gate/up/lm_head column-parallel, o/down
    # row-parallel with an NCCL all-reduce of the fp32 partial sums
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(args.seed)
    model = Decoder(c, device=dev, meta=True, tp=world)
    if args.autotune:
        from . import kernel
        kernel.AUTOTUNE = True
    model.fuse_norm_quant = not args.no_fuse
    model.fuse_groups = not args.no_groups
    model.fuse_step = not args.no_step_fusion
    nlin = synthetic_quantize(model, args.rank, seed=args.seed + 1000 * rank)
    g = torch.Generator(device=dev).manual_seed(args.seed)           # (same prompt on every rank)
    prompt = torch.randint(0, c.vocab, (args.M, args.prompt), device=dev, generator=g)
    toks, sec = greedy_decode(model, prompt, args.steps, use_graph=not args.no_graph)
    nbytes = linear_bytes(model) * world
    if world > 1:
        t = torch.tensor([sec], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
        same = toks.clone()
        dist.broadcast(same, src=0)
        assert torch.equal(same, toks), "ranks disagree on the generated tokens"
        if rank != 0:
            dist.destroy_process_group()
            return
    peak = None
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peak = json.load(open(path)).get("hbm_gbs")
    gbs = nbytes * args.steps / sec / 1e9
    print(json.dumps({
        "metric": "decode tokens/s", "value": args.M * args.steps / sec, "unit": "tokens/s", "M": args.M, "n_gpus": world,
        "ms_per_step": sec / args.steps * 1e3, "model": args.model, "layers": c.layers, "linears": nlin, "rank": args.rank,
        "prompt": args.prompt, "steps": args.steps, "fused_norm_quant": model.fuse_norm_quant, "stacked_qkv_gateup": model.fuse_groups and model.fuse_norm_quant, "fused_step": model.fuse_step, "data": "synthetic (random packed operands, random prompt)",
        "linear_bytes_per_step": nbytes, "linear_GBps": gbs, "hbm_peak_GBps": peak,
        "roofline_frac": (gbs / (peak * world)) if peak else None, "finite": bool(torch.isfinite(toks.float()).all())}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
