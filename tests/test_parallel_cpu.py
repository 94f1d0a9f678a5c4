"""Tensor-parallel sharding logic on CPU: two gloo ranks, the oracle in place of the kernel.

Column-parallel shards must reproduce the matching output columns exactly; row-parallel partial outputs, summed by an
all-reduce, must reproduce the full output (fp32 sums, then one bf16 rounding); the agreed activation scale must equal the
single-device one, so that the activation codes of a K-slice equal the slice of the single-device codes."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import biloco_oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make_ops(M, K, N, R, seed):
    from biloco_b200 import fp4
    rng = np.random.default_rng(seed)
    W = torch.from_numpy(orc.bf16_round(rng.standard_normal((N, K)) * 0.02))
    codes, sf, gs = fp4.quantize_nvfp4(W, "mse")
    V = np.where(rng.standard_normal((R, K)) >= 0, 1.0, -1.0).astype(np.float32)
    U = np.where(rng.standard_normal((R, N)) >= 0, 1.0, -1.0).astype(np.float32)
    ops = dict(W_codes=codes, W_sf=sf.view(torch.uint8), w_gscale=gs,
               V_packed=torch.from_numpy(orc.pack_signs(V)), U_packed=torch.from_numpy(orc.pack_signs(U)),
               S=torch.from_numpy(orc.bf16_round(rng.standard_normal(R) * 0.01)).to(torch.bfloat16),
               smooth_scale=torch.from_numpy(orc.bf16_round(rng.random(K) * 2 + 0.5)).to(torch.bfloat16), bias=None)
    x = orc.bf16_round(rng.standard_normal((M, K)))
    x[:, rng.permutation(K)[: K // 100]] *= 20
    return ops, orc.bf16_round(x)


def _oracle_forward(ops, x, gscale=None):
    """Unrounded float64 output of one (shard of a) layer through the oracle, plus the activation codes."""
    xs = orc.bf16_round(x / ops["smooth_scale"].float().numpy())
    codes, sf, gs = orc.nvfp4_quantize(xs, "mse", global_scale=gscale)
    a = orc.nvfp4_dequantize(codes, sf, gs)
    K = x.shape[1]
    N = ops["W_codes"].shape[0]
    from biloco_b200 import fp4
    w_sf = fp4.unswizzle_scales(ops["W_sf"], N, K).numpy()
    w = orc.nvfp4_dequantize(ops["W_codes"].numpy(), w_sf, float(ops["w_gscale"]))
    z = orc.binary_z(xs, ops["V_packed"].numpy(), ops["S"].float().numpy()).astype(np.float64)
    y = a @ w.T + orc.binary_expand(z, ops["U_packed"].numpy(), round_bf16=False)
    return y, codes, gs


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from biloco_b200 import parallel
    M, K, N, R = 3, 1024, 512, 64
    ops, x = _make_ops(M, K, N, R, seed=5)
    y_full, codes_full, gs_full = _oracle_forward(ops, x)

    # column-parallel
    col = parallel.shard_column_parallel(ops, world, rank)
    lo, hi = parallel.shard_bounds(N, world, rank, 128)
    y_col, _, _ = _oracle_forward(col, x)
    ok_col = np.allclose(y_col, y_full[:, lo:hi], rtol=1e-12, atol=1e-12)

    # row-parallel: agreed scale, codes of the slice, summed partial outputs
    row = parallel.shard_row_parallel(ops, world, rank)
    klo, khi = parallel.shard_bounds(K, world, rank, 256)
    x_loc = x[:, klo:khi]
    gs = parallel.agree_on_activation_scale(torch.from_numpy(x_loc), row["smooth_scale"], rule="mse")
    ok_gs = np.float32(gs.item()) == gs_full
    y_part, codes_loc, _ = _oracle_forward(row, x_loc, gscale=np.float32(gs.item()))
    ok_codes = np.array_equal(codes_loc, codes_full[:, klo // 2: khi // 2])
    t = torch.from_numpy(y_part.copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    # z is rounded to fp32 per shard (as the kernel does), so the sum matches to fp32 accuracy, not exactly
    ok_row = np.allclose(t.numpy(), y_full, rtol=1e-5, atol=1e-6 * float(np.max(np.abs(y_full))))
    q.put((rank, bool(ok_col), bool(ok_gs), bool(ok_codes), bool(ok_row)))
    dist.destroy_process_group()


def test_sharding_with_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in res:
        assert r[1:] == (True, True, True, True), f"rank {r[0]}: column={r[1]} scale={r[2]} codes={r[3]} row={r[4]}"


def test_shard_bounds_and_scale_layout():
    from biloco_b200 import fp4, parallel
    assert parallel.shard_bounds(8192, 8, 3, 128) == (3072, 4096)
    try:
        parallel.shard_bounds(5120, 8, 0, 256)       # 640 is not a multiple of 256
        assert False
    except AssertionError:
        pass
    # slicing the atom layout by rows / by k equals swizzling the sliced linear scales
    rng = np.random.default_rng(0)
    N, K = 256, 512
    lin = torch.from_numpy(rng.integers(0, 255, (N, K // 16), dtype=np.uint8))
    sw = fp4.swizzle_scales(lin).view(torch.uint8)
    ops = dict(W_codes=torch.zeros(N, K // 2, dtype=torch.uint8), W_sf=sw, w_gscale=torch.ones(1), V_packed=torch.zeros(8, K // 8, dtype=torch.uint8),
               U_packed=torch.zeros(8, N // 8, dtype=torch.uint8), S=torch.zeros(8), smooth_scale=torch.ones(K), bias=None)
    c = parallel.shard_column_parallel(ops, 2, 1)
    assert torch.equal(c["W_sf"], fp4.swizzle_scales(lin[128:]).view(torch.uint8))
    r = parallel.shard_row_parallel(ops, 2, 1)
    assert torch.equal(r["W_sf"], fp4.swizzle_scales(lin[:, 16:]).view(torch.uint8))
