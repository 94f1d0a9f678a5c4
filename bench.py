"""Benchmark of the fused BiLoCo decode linear on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--M 1] [--r 512]

A *step* is one pass of the fused linear over ``--layers`` distinct synthetic layers (K = N = 5120 by default),
i.e. ``--layers`` kernel launches that stream ``layers * bytes(K, N, r)`` algorithmic weight bytes; with the
default 64 layers that is 986 MB per step, far larger than L2, so every launch streams its weights from HBM
("inputs larger than L2"). One JSON line is printed by rank 0:

  value         algorithmic GB/s of the whole job, operands resident in HBM, CUDA-graph replay of the step,
                timed with CUDA events on the launching stream (max over ranks)
  e2e           the same metric through the public Python API with HOST activations: per step one pinned
                host->device copy of the step's bf16 activations, per layer the device NVFP4 quantiser and the
                fused linear, one device->host copy of the outputs; the step is captured in a CUDA graph once and a
                replay plus a synchronisation is timed (wall clock)
  roofline      achieved GB/s of the fused kernel vs the measured HBM copy peak (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle's fake-quant forward (biloco/layer.py:54-64 semantics) on the host cores,
                bounded sample

  tp_decode     (unless --no-decode) the sharded path: a Llama-3-70B-shaped decoder, every linear a rank-512 layer, q/k/v/
                gate/up/lm_head column-parallel and o/down row-parallel over the N ranks with an NCCL all-reduce of the
                fp32 partial sums inside the captured step (biloco_b200.decode); tokens/s, ms per step, all-reduces and
                bytes per step. At N = 1 the same model on one GPU, so that the per-N lines give the parallel efficiency
  comparator    (N = 1, default point, if oracle/_ref holds the reference's extension built for sm_100a) the reference's own
                fused kernel on this GPU, in a process of its own: L2-warm as the reference measures and HBM-cold

``--impl reference`` times that CPU forward alone and prints the same line shape with "impl": "reference".
``--table`` prints the per-(M, rank) report of scripts/kernel_table.py instead (every schedule, L2-warm and HBM-cold, error
over consecutive launches), as markdown.
Multi-GPU (torchrun, one rank per GPU): `value` is measured on replicas (every rank its own layers: the single linear
shards by layer / by output columns with no exchange, weak scaling); the tensor-parallel path is the tp_decode leg.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch at M=1, K=N=5120, r=512 from one ncu capture per kernel
# (summaries under profiles/; other shapes and kernels: null)
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"slab_kernel": 15_511_000, "fused_linear_kernel": 15_543_000}


def algorithmic_bytes(K, N, r):
    """E2M1 codes + E4M3 block scales of the residual + packed U and V sign bits."""
    return N * K // 2 + N * K // 16 + N * r // 8 + K * r // 8


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.t0, self.t1 = index, None, None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu=timestamp,{self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
            time.sleep(0.15)
        except Exception:
            self.proc = None

    def mark(self, which):
        setattr(self, which, time.time())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                ts = time.mktime(time.strptime(f[0].split(".")[0], "%Y/%m/%d %H:%M:%S")) + float("0." + f[0].split(".")[1])
                rows.append((ts, float(f[1]), float(f[2]), f[4:8]))
            except Exception:
                continue
        inside = [r for r in rows if self.t0 is not None and self.t0 - 0.05 <= r[0] <= (self.t1 or 1e18) + 0.05] or rows
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in inside for n, v in zip(names, r[3]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[0][2], "reasons": reasons,
                "samples": len(inside)}


def make_layers(torch, kernel, fp4, dev, L, M, K, N, r, seed, mode=None, share_act=False):
    """Synthetic layers in the construction of the reference's timing scripts (scripts/problem.py:7-27, random
    block scales in [0.25, 2]), activations ~N(0,1) with 1 % outlier channels x20 quantised by the device quantiser."""
    g = torch.Generator(device=dev).manual_seed(seed)
    layers = []
    for _ in range(L):
        W = torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8, generator=g)
        W_sf = (torch.rand(kernel.nvfp4_sf_bytes(N, K), device=dev, generator=g) * 1.75 + 0.25).to(torch.float8_e4m3fn)
        Vp = torch.randint(0, 256, (r, K // 8), device=dev, dtype=torch.uint8, generator=g)
        Up = torch.randint(0, 256, (r, N // 8), device=dev, dtype=torch.uint8, generator=g)
        S = (torch.randn(r, device=dev, generator=g) * 0.01).to(torch.bfloat16)
        w_gs = torch.full((1,), 1e-3, device=dev)
        x = torch.randn(M, K, device=dev, generator=g)
        idx = torch.randperm(K, device=dev, generator=g)[: K // 100]
        x[:, idx] *= 20
        x = x.to(torch.bfloat16).contiguous()
        if share_act and layers:      # one activation buffer for every layer, as the hidden state of a decoder is
            x, w_gs, q = layers[0]["x"], layers[0]["w_gs"], layers[0]["q"]
        else:
            q = fp4.quantize_activation(x, "mse", w_gscale=w_gs, rows=M)
        gemm = kernel.BiLoCoGemm(W, W_sf, q["alpha"], Vp, Up, S, M=M, mode=mode)
        layers.append(dict(gemm=gemm, q=q, x=x, w_gs=w_gs, ops=(W, W_sf, Vp, Up, S)))
    return layers


def cpu_forward_setup(M, K, N, r, seed=0):
    """Operands of the reference's fake-quant forward for one synthetic layer (numpy, bf16-exact float32)."""
    import numpy as np
    from oracle import biloco_oracle as orc
    rng = np.random.default_rng(seed)
    V = np.where(rng.standard_normal((r, K)) >= 0, 1.0, -1.0).astype(np.float32)
    U = np.where(rng.standard_normal((r, N)) >= 0, 1.0, -1.0).astype(np.float32)
    S = orc.bf16_round(rng.standard_normal(r) * 0.01)
    weight_fp4 = orc.bf16_round(orc.fake_quantize_fp4(orc.bf16_round(rng.standard_normal((N, K)) * 0.02), "static_6"))
    x = orc.bf16_round(rng.standard_normal((M, K)))
    x[:, rng.permutation(K)[: K // 100]] *= 20
    return dict(x=x, smooth=np.ones(K, np.float32), V_scaled=orc.bf16_round(V * S[:, None]), U_T=U, weight_fp4=weight_fp4)


def time_cpu_forward(M, K, N, r, calls, warm, budget_s):
    """Median seconds per call of the oracle's torch-CPU forward (bf16 matmuls on all host threads, as the
    reference module runs on a CPU); stops early when the time budget is used up."""
    from oracle import biloco_oracle as orc
    a = cpu_forward_setup(M, K, N, r)
    layer = orc.TorchLayer(a["smooth"], a["V_scaled"], a["U_T"], a["weight_fp4"], None, "mse")
    ts = []
    t_start = time.time()
    for i in range(warm + calls):
        t0 = time.perf_counter()
        layer(a["x"])
        dt = time.perf_counter() - t0
        if i >= warm:
            ts.append(dt)
        if time.time() - t_start > budget_s and len(ts) >= 3:
            break
    return statistics.median(ts), len(ts)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    # every host core, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)
    torch.set_num_threads(os.cpu_count() or 1)
    K, N, r, M = args.K, args.N, args.r, args.M
    sec, n = time_cpu_forward(M, K, N, r, calls=max(min(args.steps, 200), 3), warm=max(args.warmup, 3), budget_s=120)
    gbs = algorithmic_bytes(K, N, r) / sec / 1e9
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": "fused BiLoCo linear algorithmic HBM GB/s", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": n, "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 (+ f32 sign accumulate)", "data": "synthetic",
        "config": workload_config(args, layers=args.layers),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{n} calls of the fake-quant forward of ONE of the step's {args.layers} layers (M={M}, K={K}, "
                                   f"N={N}, r={r}), median; a step is {args.layers} such calls; torch threads = "
                                   f"{torch.get_num_threads()} of {cores} host cores"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_call": sec * 1e6,
    }
    line["ms_per_step"] = sec * 1e3 * args.layers
    print(json.dumps(line), flush=True)


def workload_config(args, layers):
    return {"workload": f"configs[1] point M={args.M}, r={args.r}: fused BiLoCo linear K={args.K} N={args.N}, "
                        f"{layers} distinct layers per step",
            "M": args.M, "K": args.K, "N": args.N, "r": args.r, "layers_per_step": layers,
            "l2_policy": "inputs larger than L2 (each step streams layers x weights from HBM; the device arm's launches read one "
                         "shared activation row, like a decoder's hidden state)",
            "algorithmic_bytes_per_call": algorithmic_bytes(args.K, args.N, args.r)}


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from biloco_b200 import _lib, fp4, kernel
    if args.no_pdl:
        _lib.load().biloco_b200_set_option(1, 0)
    if args.ring:
        _lib.load().biloco_b200_set_option(2, args.ring)
    if args.trigger >= 0:
        _lib.load().biloco_b200_set_option(3, args.trigger)
    if args.lr_tc >= 0:
        _lib.load().biloco_b200_set_option(4, args.lr_tc)

    K, N, r, M, L = args.K, args.N, args.r, args.M, args.layers
    # One activation buffer for all layers of the device arm, as the hidden state of a decoder is (written by the previous
    # kernel, so L2-resident when the linear reads it); the weights and factors are distinct per layer and come from HBM.
    layers = make_layers(torch, kernel, fp4, dev, L, M, K, N, r, seed=1234 + rank, mode=args.mode, share_act=not args.own_activations)
    bytes_call = algorithmic_bytes(K, N, r)

    def step_device():
        for ly in layers:
            g = ly["gemm"]
            ly["out"] = g(ly["q"]["A"], ly["q"]["A_sf"], ly["x"], A_rec=ly["q"].get("A_rec") if g.mode != 7 else None)

    # ---- device-resident arm: one CUDA graph per step -------------------------------------------------
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_device()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step_device()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    for ly in layers:
        st = ly["gemm"].status()
        assert st[0] == 0, f"device-side wait ran out during warm-up: {st[:4]}"

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark("t0")
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    sampler.mark("t1")
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    for ly in layers:
        st = ly["gemm"].status()
        assert st[0] == 0, f"device-side wait ran out in the timed region: {st[:4]}"
    ms_per_step = ms / args.steps
    us_per_call = ms_per_step * 1e3 / L
    value = world * L * bytes_call / (ms_per_step * 1e-3) / 1e9

    # ---- end-to-end arm: host activations in, host outputs back, through the Python API ----------------
    # One step = what a decode step of a host program does: the step's bf16 activations (all layers, one pinned host
    # buffer) are copied to the device, every layer runs the public calls (activation quantiser, fused linear), and the
    # outputs (one device buffer) are copied back to pinned host memory. The step is captured once in a CUDA graph, as
    # a serving loop would do; a replay plus a synchronisation is timed.
    x_host = torch.empty(L, M, K, dtype=torch.bfloat16).pin_memory()
    for i, ly in enumerate(layers):
        x_host[i].copy_(ly["x"].cpu())
    x_dev = torch.empty(L, M, K, device=dev, dtype=torch.bfloat16)
    y_dev = torch.empty(L, M, N, device=dev, dtype=torch.bfloat16)
    y_host = torch.empty(L, M, N, dtype=torch.bfloat16).pin_memory()

    # (the launchers of this arm are built for a stream in which a quantiser launch precedes every linear, as
    # BiLoCoLinear.forward builds them; when that is the same schedule as the device arm's the launcher is shared)
    for ly in layers:
        g0 = ly["gemm"]
        want = kernel.default_mode(M, r, kernel.supported_modes(M, N, K, r), back_to_back=False) if args.mode is None else args.mode
        ly["gemm_e2e"] = g0 if g0.mode == want else kernel.BiLoCoGemm(ly["ops"][0], ly["ops"][1], ly["q"]["alpha"], *ly["ops"][2:],
                                                                       M=M, mode=want)

    # Where the row-slab launcher takes the raw activation (M <= 2), the step is ONE launch per layer: the kernel
    # quantises the activation itself (--e2e-two-launches keeps the quantiser launch in front of every linear).
    one_launch = (not args.e2e_two_launches) and all(ly["gemm"].mode == 7 and ly["gemm"].raw_supported() for ly in layers)
    if one_launch:
        for ly in layers:
            ly["gemm_e2e"] = ly["gemm"]

    def step_e2e_body():
        x_dev.copy_(x_host, non_blocking=True)
        for i, ly in enumerate(layers):
            g = ly["gemm_e2e"]
            if one_launch:
                g.raw(x_dev[i], ly["w_gs"], "mse", out=y_dev[i])
                continue
            fp4.quantize_activation(x_dev[i], "mse", w_gscale=ly["w_gs"], rows=M, out=ly["q"])
            g(ly["q"]["A"], ly["q"]["A_sf"], x_dev[i], out=y_dev[i], A_rec=ly["q"].get("A_rec") if g.mode != 7 else None)
        y_host.copy_(y_dev, non_blocking=True)

    with torch.cuda.stream(side):
        step_e2e_body()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    y_check = y_host.clone()
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_e2e, stream=side):
        step_e2e_body()

    def step_e2e():
        graph_e2e.replay()
        torch.cuda.synchronize()

    e2e_steps = max(3, min(args.steps, 50))
    for _ in range(3):
        step_e2e()
    assert torch.equal(y_host, y_check), "graph replay of the end-to-end step changed the outputs"
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * L * bytes_call * e2e_steps / e2e_s / 1e9

    # ---- tensor-parallel decode leg (every rank takes part) ---------------------------------------------
    tp = None
    default_point = (M, K, N, r) == (1, 5120, 5120, 512)
    if not args.no_decode and default_point:
        mode0, mode_e2e = layers[0]["gemm"].mode, layers[0]["gemm_e2e"].mode
        del graph, graph_e2e
        layers.clear()
        torch.cuda.empty_cache()
        try:
            tp = tp_decode_leg(torch, dist, world, rank, dev, args)
        except Exception as e:      # the linear's line stands on its own
            tp = {"error": f"{type(e).__name__}: {e}"[:300]}
    else:
        mode0, mode_e2e = layers[0]["gemm"].mode, layers[0]["gemm_e2e"].mode

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_hbm_peak()
    kname = "slab_kernel" if mode0 == 7 else "fused_linear_kernel"
    achieved = bytes_call / (us_per_call * 1e-6) / 1e9
    line = {
        "metric": "fused BiLoCo linear algorithmic HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 (+ f32 sign accumulate)", "data": "synthetic",
        "config": workload_config(args, L),
        "us_per_call": us_per_call,
        "gpu_launches": args.steps * L,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": L * M * K * 2, "d2h_bytes_per_step": L * M * N * 2,
                "steps": e2e_steps, "us_per_call": e2e_s / e2e_steps / L * 1e6},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(kname) if (M, K, N, r) == (1, 5120, 5120, 512) else None,
                     "peak_source": f"{peak_kind} (STREAM-style copy)",
                     "kernel": kname, "schedule": mode0, "algorithmic_bytes_per_launch": bytes_call},
        "e2e_schedule": mode_e2e,
        "e2e_launches_per_layer": 1 if one_launch else 2,
    }
    if world == 1 and not args.no_cpu:
        sec, n = time_cpu_forward(M, K, N, r, calls=200, warm=3, budget_s=args.cpu_budget)
        line["cpu_baseline"] = {"value": bytes_call / sec / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                "us_per_call": sec * 1e6,
                                "sample": f"{n} calls of the CPU oracle's fake-quant forward of one layer "
                                          f"(M={M}, K={K}, N={N}, r={r}), median; BLAS threads = {torch.get_num_threads()}"}
    if tp is not None:
        line["tp_decode"] = tp
    if world == 1 and not args.no_decode and default_point:
        try:
            line["decode"] = decode_leg(torch)
        except Exception as e:      # the linear's line stands on its own
            line["decode"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if world == 1 and not args.no_comparator and default_point:
        line["comparator"] = comparator_leg()
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def comparator_leg():
    """The reference's own extension (built for sm_100a into oracle/_ref by oracle/build_ref_kernel.py) at the headline
    point, in a process of its own; absent library: says so."""
    so = os.path.join(ROOT, "oracle", "_ref", "biloco_ref_C.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/biloco_ref_C.so is not built (python -m oracle.build_ref_kernel)"}
    try:
        out = subprocess.run([sys.executable, "-m", "oracle.ref_kernel", "--Ms", "1"], cwd=ROOT, capture_output=True, text=True,
                             timeout=300)
        row = json.loads(out.stdout.strip().splitlines()[-1])["rows"]["1"]
        return {"what": "reference extension csrc/biloco_gemm.cu on this GPU, K=N=5120, r=512, M=1; us per launch",
                "fp4_only_pad_us_l2_warm": row["pad_us"], "fp4_only_pad_us_hbm_cold": row.get("pad_cold_us"),
                "fused_mode4_us_l2_warm": row["mode4_us"], "fused_mode4_us_hbm_cold": row.get("mode4_cold_us"),
                "fused_mode4_err_over_max": row["mode4_err_over_max"],
                "fused_mode2": "wrong result at M=1 on this device (max error = max |y_ref|), not timed"
                               if row["mode2_err_over_max"] > 0.01 else row["mode2_us"],
                "not_run": "fp4_gemm / fp4_gemm_residual (cluster multicast loads) and mode 5 (unbounded waits): closed on this pool"}
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def tp_decode_leg(torch, dist, world, rank, dev, args):
    """The N/K-sharded path: greedy decode of a Llama-3-70B-shaped decoder (80 layers, hidden 8192, intermediate 28672, 64
    query / 8 KV heads, vocabulary 128256; every linear a rank-512 layer with random packed operands) through the captured
    step of biloco_b200.decode: q/k/v, gate/up and lm_head column-parallel, o and down row-parallel with one all-reduce of
    the fp32 partial sums each inside the step (the library's one-launch all-reduce over peer memory; --tp-nccl: NCCL). One rank per GPU; at world size 1 the whole model on one."""
    from biloco_b200 import decode
    c = decode.PRESETS["llama3-70b"]
    if args.tp_layers:
        c = decode.DecoderConfig(**{**c.__dict__, "layers": args.tp_layers})
    torch.manual_seed(0)
    model = decode.Decoder(c, device=dev, meta=True, tp=world)
    nlin = decode.synthetic_quantize(model, 512, seed=1000 * rank)
    g = torch.Generator(device=dev).manual_seed(0)
    prompt = torch.randint(0, c.vocab, (args.tp_M, args.tp_prompt), device=dev, generator=g)
    from biloco_b200 import parallel
    ar = "none"
    if world > 1:
        # two eager steps first: if a poll of the library's peer-memory all-reduce ran out of its budget on any rank, the
        # timed run uses NCCL instead (and says so)
        parallel.ShardedBiLoCoLinear.peer_allreduce = not args.tp_nccl
        decode.greedy_decode(model, prompt[:, :2], 1, use_graph=False)
        bad = torch.tensor([1.0 if any(o.failed() for o in parallel.PeerAllReduce._by_group.values()) else 0.0], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if bad.item() > 0:
            parallel.ShardedBiLoCoLinear.peer_allreduce = False
        ar = ("one launch over peer memory (biloco_b200_peer_allreduce)" if parallel.ShardedBiLoCoLinear.peer_allreduce
              else ("ncclAllReduce + cast" + ("" if args.tp_nccl else " (the peer-memory all-reduce reported a failed wait)")))
    toks, sec = decode.greedy_decode(model, prompt, args.tp_steps, use_graph=True)
    if world > 1:
        parallel.PeerAllReduce.close_all()
    nbytes = decode.linear_bytes(model) * world
    if dist is not None:
        t = torch.tensor([sec], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    peak, _ = measured_hbm_peak()
    n_ar = 2 * c.layers if world > 1 else 0
    return {"model": f"Llama-3-70B-shaped ({c.layers} layers, hidden 8192, intermediate 28672, vocab 128256), random packed operands",
            "parallelism": f"tp{world}: q/k/v/gate/up/lm_head column shards, o/down row shards", "M": args.tp_M, "rank": 512,
            "linears_per_rank": nlin, "prompt": args.tp_prompt, "steps": args.tp_steps,
            "tokens_per_s": args.tp_M * args.tp_steps / sec, "ms_per_step": sec / args.tp_steps * 1e3,
            "all_reduce": ar, "all_reduces_per_step": n_ar, "all_reduce_bytes_each": args.tp_M * c.hidden * 4 if world > 1 else 0,
            "linear_bytes_per_step": nbytes, "hbm_frac_of_n_gpus": nbytes * args.tp_steps / sec / 1e9 / (peak * world),
            "finite": bool(torch.isfinite(toks.float()).all())}


def decode_leg(torch, prompt_len=16, steps=48):
    """The other half of the metric, reported beside the linear's number: greedy decode of a Qwen3-4B-shaped decoder (36
    layers, every linear a rank-512 layer with random packed operands, M = 1) through the captured step of
    biloco_b200.decode; tokens/s and the fraction of the HBM peak the linears' bytes reach. Short prompt and run, so
    that the default bench stays within minutes (a longer context adds attention time per step)."""
    from biloco_b200 import decode
    dev = torch.device("cuda", torch.cuda.current_device())
    c = decode.PRESETS["qwen3-4b"]
    torch.manual_seed(0)
    model = decode.Decoder(c, device=dev, meta=True)
    nlin = decode.synthetic_quantize(model, 512, seed=0)
    g = torch.Generator(device=dev).manual_seed(0)
    prompt = torch.randint(0, c.vocab, (1, prompt_len), device=dev, generator=g)
    toks, sec = decode.greedy_decode(model, prompt, steps, use_graph=True)
    nbytes = decode.linear_bytes(model)
    peak, _ = measured_hbm_peak()
    return {"model": "Qwen3-4B-shaped (36 layers, hidden 2560, vocab 151936), random packed operands", "M": 1, "rank": 512,
            "linears": nlin, "prompt": prompt_len, "steps": steps, "tokens_per_s": steps / sec, "ms_per_step": sec / steps * 1e3,
            "linear_bytes_per_step": nbytes, "hbm_frac": nbytes * steps / sec / 1e9 / peak,
            "finite": bool(torch.isfinite(toks.float()).all())}


def run_table(args):
    """The report of scripts/kernel_table.py:44-77 for this library on this GPU, as markdown: per (M, rank) at K = N = 5120
    every schedule the shape takes, timed L2-warm (the reference's protocol: a graph of 64 launches on the same operands,
    median of 30 replays) and HBM-cold (a graph over `--table-layers` distinct layers, > L2), with the largest error
    over `--stress` consecutive launches against the unfused device path (non-zero block scales: both terms live)."""
    import torch
    from biloco_b200 import fp4, kernel
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K, N, L = args.K, args.N, args.table_layers
    Ms = [int(x) for x in args.table_Ms.split(",")]
    ranks = [int(x) for x in args.table_ranks.split(",")]
    modes = (2, 4, 5, 7)
    print(f"# Kernel table, {torch.cuda.get_device_name()}, K={K} N={N}: us per launch, L2-warm / HBM-cold ({L} distinct layers); "
          f"error = max|y - y_unfused| / max|y_unfused| over {args.stress} launches\n")
    print("| M | r | " + " | ".join(f"mode {m}" for m in modes) + " | best cold | GB/s | of peak | max err |")
    print("|---|---|" + "---|" * (len(modes) + 4))
    peak, _ = measured_hbm_peak()
    for M in Ms:
        for r in ranks:
            layers = make_layers(torch, kernel, fp4, dev, L, M, K, N, r, seed=17 * M + r, mode=2)
            ly0 = layers[0]
            W, W_sf, Vp, Up, S = ly0["ops"]
            y_ref = kernel.reference(ly0["q"]["A"], ly0["q"]["A_sf"], W, W_sf, ly0["q"]["alpha"], ly0["x"], Vp, Up, S)
            y_ref = y_ref.view(-1, N)[:M].float()
            cells, best, worst = [], None, 0.0
            for mode in modes:
                if mode not in kernel.supported_modes(M, N, K, r):
                    cells.append("-")
                    continue
                gs = [kernel.BiLoCoGemm(*ly["ops"][:2], ly["q"]["alpha"], *ly["ops"][2:], M=M, mode=mode) for ly in layers]
                err = 0.0
                for _ in range(args.stress):
                    y = gs[0](ly0["q"]["A"], ly0["q"]["A_sf"], ly0["x"]).view(-1, N)[:M].float()
                    err = max(err, float((y - y_ref).abs().max() / y_ref.abs().max()))
                assert gs[0].status()[0] == 0
                warm = kernel.time_graph(lambda: gs[0](ly0["q"]["A"], ly0["q"]["A_sf"], ly0["x"]))
                cold = kernel.time_graph(lambda: [g(ly["q"]["A"], ly["q"]["A_sf"], ly["x"]) for g, ly in zip(gs, layers)], batch=1) / L
                cells.append(f"{warm:.2f} / {cold:.2f}")
                worst = max(worst, err)
                if best is None or cold < best[1]:
                    best = (mode, cold)
                del gs
            gbs = algorithmic_bytes(K, N, r) / (best[1] * 1e-6) / 1e9
            print(f"| {M} | {r} | " + " | ".join(cells) + f" | {best[1]:.2f} (mode {best[0]}) | {gbs:.0f} | {gbs / peak:.3f} | {worst:.1e} |",
                  flush=True)
            del layers
            torch.cuda.empty_cache()
    so = os.path.join(ROOT, "oracle", "_ref", "biloco_ref_C.so")
    if os.path.exists(so) and (K, N) == (5120, 5120):
        out = subprocess.run([sys.executable, "-m", "oracle.ref_kernel", "--Ms", "1,2,4,8", "--cold-layers", str(L)], cwd=ROOT,
                             capture_output=True, text=True, timeout=900)
        try:
            rows = json.loads(out.stdout.strip().splitlines()[-1])["rows"]
            print("\n# The reference's own extension (csrc/biloco_gemm.cu built for sm_100a) on the same GPU, r = 512: us per launch, "
                  "L2-warm / HBM-cold; fp4_gemm, fp4_gemm_residual and mode 5 are not run (closed on this pool)\n")
            print("| M | pad (FP4 only) | s128 (FP4 only) | mode 2 | mode 4 | mode 4 max err |")
            print("|---|---|---|---|---|---|")
            for M, row in rows.items():
                f = lambda k: f"{row[k]:.2f}" if k in row else "-"
                m2 = "wrong result" if row["mode2_err_over_max"] > 0.01 else f"{f('mode2_us')} / {f('mode2_cold_us')}"
                print(f"| {M} | {f('pad_us')} / {f('pad_cold_us')} | {f('s128_us')} / - | {m2} | {f('mode4_us')} / {f('mode4_cold_us')} | "
                      f"{row['mode4_err_over_max']:.1e} |")
        except Exception as e:
            print(f"\n(reference extension: no result: {type(e).__name__}: {e}; stderr tail: {out.stderr[-300:]})")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--K", type=int, default=5120)
    ap.add_argument("--N", type=int, default=5120)
    ap.add_argument("--r", type=int, default=512)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-pdl", action="store_true", help="plain launches instead of programmatic dependent launches")
    ap.add_argument("--ring", type=int, default=0, help="pipeline stages in flight (0 = library default)")
    ap.add_argument("--trigger", type=int, default=-1, help="where a CTA lets the next launch start (-1 = library default)")
    ap.add_argument("--lr-tc", type=int, default=-1, help="1/0: expansion on the tensor cores on/off (-1 = library default)")
    ap.add_argument("--mode", type=int, default=None, help="schedule of the fused kernel (default: the measured table)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode leg (default workload, one GPU only)")
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of CPU work for the baseline sample")
    ap.add_argument("--tp-nccl", action="store_true", help="tensor-parallel decode leg: NCCL all-reduce instead of the library's own")
    ap.add_argument("--e2e-two-launches", action="store_true",
                    help="end-to-end arm: quantiser launch + fused launch per layer instead of the one-launch raw-activation form")
    ap.add_argument("--own-activations", action="store_true",
                    help="device arm: every layer reads its own activation buffers (they then come from HBM too)")
    ap.add_argument("--no-comparator", action="store_true", help="skip the reference extension's leg (one GPU, default workload)")
    ap.add_argument("--tp-layers", type=int, default=0, help="tp_decode leg: decoder layers (0 = all 80)")
    ap.add_argument("--tp-M", type=int, default=1, help="tp_decode leg: sequences decoded together")
    ap.add_argument("--tp-prompt", type=int, default=512)
    ap.add_argument("--tp-steps", type=int, default=128)
    ap.add_argument("--table", action="store_true", help="print the per-(M, rank) kernel table as markdown instead")
    ap.add_argument("--table-Ms", default="1,2,4,8,16,32")
    ap.add_argument("--table-ranks", default="128,256,512,1024")
    ap.add_argument("--table-layers", type=int, default=24, help="distinct layers of the HBM-cold graph (24 x 15 MB > L2)")
    ap.add_argument("--stress", type=int, default=50, help="--table: launches checked against the unfused path per schedule")
    args = ap.parse_args()
    if args.table:
        run_table(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
