"""Tensor-parallel check on real GPUs (one process per GPU, NCCL; 2 or 4 ranks). Launched by tests/test_gpu_tp.py or by hand:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 tests/tp_gpu_check.py

Every rank builds the same layer, runs its column-parallel and row-parallel shard through the fused kernel, and compares
with the whole layer run on its own GPU: column shards must equal the matching columns bit for bit (same arithmetic per
column), the all-reduced row-parallel output must match within the suite's tolerances."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
sys.path.insert(0, ROOT)


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    from biloco_b200 import fp4, kernel, parallel
    from tests.gpu_util import check_against_unfused

    M, K, N, R = 4, 2048, 2048, 128
    g = torch.Generator(device=dev).manual_seed(7)        # same operands on every rank
    W = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16).float()
    codes, sf, gs = fp4.quantize_nvfp4(W, "mse")
    V = torch.where(torch.randn(R, K, device=dev, generator=g) >= 0, 1.0, -1.0)
    U = torch.where(torch.randn(R, N, device=dev, generator=g) >= 0, 1.0, -1.0)
    ops = dict(W_codes=codes, W_sf=sf.view(torch.uint8), w_gscale=gs, V_packed=kernel.pack_signs(V), U_packed=kernel.pack_signs(U),
               S=(torch.randn(R, device=dev, generator=g) * 0.01).to(torch.bfloat16),
               smooth_scale=(torch.rand(K, device=dev, generator=g) * 2 + 0.5).to(torch.bfloat16), bias=None)
    x = torch.randn(M, K, device=dev, generator=g)
    x[:, torch.randperm(K, device=dev, generator=g)[: K // 100]] *= 20
    x = x.to(torch.bfloat16)

    # whole layer on this GPU
    q = fp4.quantize_activation(x, smooth=ops["smooth_scale"], w_gscale=gs, rows=M)
    full = kernel.BiLoCoGemm(codes, sf, q["alpha"], ops["V_packed"], ops["U_packed"], ops["S"], M=M)
    y_full = full(q["A"], q["A_sf"], q["X"]).view(-1, N)[:M].clone()

    col = parallel.ShardedBiLoCoLinear(ops, "column", M)
    lo, hi = parallel.shard_bounds(N, world, rank, 128)
    y_col = col(x)
    torch.cuda.synchronize()
    # a column's arithmetic is the same in the shard and in the whole layer except for the order in which the K-split
    # partial sums are added (the split follows the number of column tiles): equal bits at two ranks, where both split alike,
    # and within a bf16 ulp of the largest output otherwise
    ref_col = y_full[:, lo:hi].contiguous()
    if world == 2:
        assert torch.equal(y_col.view(torch.int16), ref_col.view(torch.int16)), "column shard differs"
    else:
        assert float((y_col.float() - ref_col.float()).abs().max()) <= 2.0 ** -7 * float(ref_col.float().abs().max()), "column shard differs"

    row = parallel.ShardedBiLoCoLinear(ops, "row", M)
    klo, khi = parallel.shard_bounds(K, world, rank, 256)
    for _ in range(2):
        y_row = row(x[:, klo:khi].contiguous())
    torch.cuda.synchronize()
    # the ranks' fp32 partial sums are added by the all-reduce and rounded to bf16 once: within the suite's tolerance
    check_against_unfused(y_row.float().cpu().numpy(), y_full.float().cpu().numpy(), f"row-parallel, rank {rank}")
    assert row.gemm.status()[0] == 0 and col.gemm.status()[0] == 0

    # decode-step form of the row shard: every rank scales its own K-slice (different FP4 codes than the single-GPU
    # quantisation, so the yardstick is the unquantised-activation value: no further from it than the single-GPU
    # kernel is), silu(gate) * up formed in the quantiser launch, the residual carried by rank 0's partial sum
    gu = torch.randn(M, 2 * K, device=dev, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    xa = torch.nn.functional.silu(gu[:, :K]) * gu[:, K:]
    xs = (xa / ops["smooth_scale"]).float()
    w = fp4.dequantize_nvfp4(codes, sf, gs).float()
    y_hp = xs @ w.T + ((xs @ V.T) * ops["S"].float()) @ U
    qa = fp4.quantize_activation(xa.contiguous(), smooth=ops["smooth_scale"], w_gscale=gs, rows=M)
    y_one = full(qa["A"], qa["A_sf"], qa["X"]).view(-1, N)[:M].float()
    loc = parallel.ShardedBiLoCoLinear(ops, "row", M, local_scale=True)
    for _ in range(2):
        y_loc = loc(torch.cat([gu[:, klo:khi], gu[:, K + klo:K + khi]], dim=1).contiguous(), residual=res, swiglu=True)
    torch.cuda.synchronize()
    assert loc.gemm.status()[0] == 0
    e_one = torch.linalg.norm(y_one - y_hp)
    e_loc = torch.linalg.norm(y_loc.float() - res.float() - y_hp)
    # (the residual is added before the single bf16 rounding of the sum: allow that rounding on top)
    slack = 2.0 ** -8 * torch.linalg.norm(y_loc.float())
    assert e_loc <= 1.25 * e_one + slack, (float(e_loc), float(e_one))

    # tensor-parallel decoder against the single-GPU decoder ON THE SAME OPERANDS: every rank builds the whole tiny model
    # from one seed, cuts its own shards out of it (q/k/v/gate/up/lm_head columns, o/down input columns) and steps both
    # on the same tokens; the gathered logits must agree with the single-GPU logits (the row shards quantise their K-slice
    # with their own scale, so not bit for bit: relative Frobenius error within 5e-2, and far closer than two unrelated
    # models would be), step after step through the KV cache
    from biloco_b200 import decode
    cfg = decode.PRESETS["tiny-tp"]
    torch.manual_seed(11)
    full_model = decode.Decoder(cfg, device=dev, meta=True, tp=1)
    decode.synthetic_quantize(full_model, rank=32, seed=100)          # same seed on every rank
    tp_model = decode.shard_decoder(full_model, world, rank)
    g = torch.Generator(device=dev).manual_seed(3)
    Mtok, steps = 2, 6
    toks = torch.randint(0, cfg.vocab, (Mtok, steps), device=dev, generator=g)
    c1, c2 = full_model.new_cache(Mtok, 16), tp_model.new_cache(Mtok, 16)
    worst = 0.0
    for t in range(steps):
        pos = torch.tensor([t], device=dev)
        l1 = full_model.step(toks[:, t], pos, c1).float()
        l2 = tp_model.step(toks[:, t], pos, c2).float()
        assert l1.shape == l2.shape == (Mtok, cfg.vocab) and torch.isfinite(l2).all()
        err = float(torch.linalg.norm(l2 - l1) / torch.linalg.norm(l1))
        worst = max(worst, err)
        assert err <= 5e-2, f"step {t}: tensor-parallel logits differ from the single-GPU logits by {err:.3g} (relative Frobenius)"
    same = torch.tensor([worst], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MAX)
    # the captured greedy decode of the sharded model runs and the ranks agree on its tokens
    prompt = toks[:, :4].contiguous()
    out, _ = decode.greedy_decode(tp_model, prompt, 5, use_graph=True)
    ref = out.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, out), "ranks disagree on the generated tokens"
    # the library's one-launch all-reduce over peer memory: the same bits on every rank, equal to the sum of the gathered
    # partials in rank order; call after call (both sets of slots, the device-side call counter), eagerly and as replays of
    # a captured graph; and the row-parallel layer gives the same output through it as through NCCL (two ranks: a + b)
    red = parallel.PeerAllReduce.for_group(None, dev, 32 * 8192)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for count, fp32_out in ((8192, False), (5, False), (32 * 8192, True), (8 * 2048, False)):
        for call in range(3):
            part = torch.randn(count, device=dev, generator=g)
            resid = torch.randn(count, device=dev, generator=g).to(torch.bfloat16) if call == 1 else None
            if resid is not None:
                dist.broadcast(resid, src=0)
            got = red(part, residual=resid, fp32_out=fp32_out)
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            want = torch.zeros_like(part)
            for q in parts:
                want = want + q
            if resid is not None:
                want = want + resid.float()
            want = want if fp32_out else want.to(torch.bfloat16)
            torch.cuda.synchronize()
            assert torch.equal(got, want), (count, call, float((got.float() - want.float()).abs().max()))
    part = torch.randn(4096, device=dev, generator=g)
    outg = torch.empty(4096, device=dev, dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        red(part, out=outg)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            red(part, out=outg)
            red(outg.float(), out=outg)
    torch.cuda.current_stream().wait_stream(side)
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    s1 = torch.zeros_like(part)
    for q in parts:
        s1 = s1 + q
    s1 = s1.to(torch.bfloat16).float()
    want = torch.zeros_like(part)
    for _ in range(world):
        want = want + s1
    want = want.to(torch.bfloat16)
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(outg, want), "captured peer all-reduce differs on replay"
    assert not red.failed()
    if world == 2:
        parallel.ShardedBiLoCoLinear.peer_allreduce = False
        y_nccl = row(x[:, klo:khi].contiguous()).clone()
        parallel.ShardedBiLoCoLinear.peer_allreduce = True
        y_peer = row(x[:, klo:khi].contiguous()).clone()
        torch.cuda.synchronize()
        assert torch.equal(y_nccl.view(torch.int16), y_peer.view(torch.int16)), "peer all-reduce and NCCL disagree"
    parallel.PeerAllReduce.close_all()
    dist.barrier()
    if rank == 0:
        print(f"tensor-parallel check ok on {world} GPUs (decoder logits vs single GPU: worst relative error {float(same):.3g})", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
