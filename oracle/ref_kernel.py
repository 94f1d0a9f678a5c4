"""GPU comparator (test infrastructure): the reference's OWN compiled extension, built for sm_100a by
``oracle/build_ref_kernel.py`` into ``oracle/_ref/biloco_ref_C.so``, timed with the reference's protocol.

    python -m oracle.ref_kernel [--Ms 1,2,8] [--r 512]

Runs in a process of its own: the extension registers the ``torch.ops.biloco`` namespace, which this repository's
package registers too. Prints one JSON line: per M the microseconds per launch of

    pad    torch.ops.biloco.fp4_gemm_n64 on the activation zero-padded to 128 rows  (the paper's FP4-only baseline)
    s128   torch.ops.biloco.fp4_gemm_n128 on the unpadded activation
    mode2  torch.ops.biloco.biloco_gemm_mode2   (fused; z by side CTAs and tiles, flag hand-off)
    mode4  torch.ops.biloco.biloco_gemm_mode4   (fused; z by side CTAs, epoch tags)

each the median over 30 replays of a CUDA graph holding the scratch reset and 64 launches on the same operands (so
L2-warm), as scripts/kernel_table.py:44-77 and biloco/kernel.py:145-168 measure, at K = N = 5120, and the largest error
of five consecutive fused launches against the CPU oracle's unfused value (tests/run_tests.py:33-45: zero block scales).

Not run, on purpose: ``fp4_gemm`` / ``fp4_gemm_residual`` (their 256x256 two-SM tile loads through a 4x1x1 cluster
with multicast) and mode 5 (it waits on counters without a bound, csrc/biloco_gemm.cu:2104); the fused modes that are
run bound their polls (csrc/biloco_gemm.cu:1067, 1149, 1180, 1288).

The host-side operand layouts the extension expects are restated here from biloco/kernel.py (file:line in each function);
nothing of the reference is imported at run time.
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
SO = os.path.join(HERE, "_ref", "biloco_ref_C.so")


def pack_v_perm(V_packed: np.ndarray) -> np.ndarray:
    """Mode-2 layout of V for K = 5120 (biloco/kernel.py:50-63): per rank two 32-bit words for each of 128 threads; thread t
    owns the 4-bit groups 128 j + t of the row (j < 10), word 0 carries j < 7 at bits 4 j, word 1 carries j >= 7."""
    R, kb = V_packed.shape
    assert kb * 8 == 5120
    v = V_packed.astype(np.int64)
    nib = np.stack([v & 15, v >> 4], axis=-1).reshape(R, 10, 128)          # [rank][j][t] = group 128 j + t
    w0 = np.zeros((R, 128), np.int64)
    w1 = np.zeros((R, 128), np.int64)
    for j in range(7):
        w0 |= nib[:, j, :] << (4 * j)
    for j in range(7, 10):
        w1 |= nib[:, j, :] << (4 * (j - 7))
    words = np.stack([w0, w1], axis=1).astype(np.uint32)                   # [R][2][128]
    return words.view(np.uint8).reshape(-1)


def time_graph(torch, fn, pre, iters=30, batch=64):
    """Median microseconds per launch over `iters` replays of a graph of pre() + `batch` launches (biloco/kernel.py:145-168)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        if pre:
            pre()
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        if pre:
            pre()
        for _ in range(batch):
            fn()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) / batch * 1e3 for a, b in ev)
    return ts[len(ts) // 2]


class RefGemm:
    """The scratch tensors and the call of the reference's BiLoCoGemm for modes 2 and 4 (biloco/kernel.py:96-130)."""

    def __init__(self, torch, ops, t, p, M, mode, N, K, R):
        from oracle import biloco_oracle as orc
        dev = t["W"].device
        self.ops, self.t, self.M, self.mode = ops, t, M, mode
        self.U_col32 = torch.from_numpy(orc.pack_u_col32(p["U_packed"], N, R)).to(dev)
        self.none = torch.zeros(0, device=dev, dtype=torch.int64)
        self.flags = None
        if mode == 2:
            self.V_perm = torch.from_numpy(pack_v_perm(p["V_packed"])).to(dev)
            self.U_rw = self.U_col32.t().contiguous()
            self.z = torch.zeros(8, M, R, 2, device=dev)
            self.flags = torch.zeros(4096, device=dev, dtype=torch.int32)
        else:
            rows = 8 * M if M <= 8 else max(8 * M, -(-(80 * (R // 32) * 1024) // (2 * R * M)) * M)
            self.z = torch.zeros(rows, 2 * R, device=dev)
        self.epoch = 0

    def reset(self):
        self.z.zero_()
        if self.flags is not None:
            self.flags.zero_()
        self.epoch = 0

    def __call__(self):
        t = self.t
        self.epoch += 1
        a = (t["A_pad"], t["W"], t["A_sf"], t["W_sf"], t["alpha"], t["X"], t["V_packed"], t["S"], self.U_col32)
        if self.mode == 2:
            return self.ops.biloco_gemm_mode2(*a, self.z, self.flags, self.none, self.V_perm, self.U_rw, self.M, self.epoch)
        return self.ops.biloco_gemm_mode4(*a, self.z, self.none, self.M, self.epoch)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--Ms", default="1,2,8")
    ap.add_argument("--r", type=int, default=512)
    ap.add_argument("--cold-layers", type=int, default=64,
                    help="distinct layers in the HBM-cold graph (64 x 15 MB > L2); 0 skips the cold arm")
    a = ap.parse_args()
    if not os.path.exists(SO):
        print(json.dumps({"comparator": "unavailable", "why": "oracle/_ref/biloco_ref_C.so has not been built"}))
        return
    import torch
    from oracle import biloco_oracle as orc
    torch.ops.load_library(SO)
    ops = torch.ops.biloco
    K = N = 5120
    R = a.r
    out = {"comparator": "reference extension (csrc/biloco_gemm.cu) built for sm_100a", "K": K, "N": N, "r": R,
           "device": torch.cuda.get_device_name(), "protocol": "graph of reset + 64 launches, same operands, median of 30 replays",
           "rows": {}}
    for M in map(int, a.Ms.split(",")):
        p = orc.random_problem(M, K, N, R)                     # zero block scales: the check isolates the low-rank term
        dev = "cuda"
        t = {k: torch.from_numpy(p[k]).to(dev) for k in ("V_packed", "A", "A_pad", "W")}
        t["X"] = torch.from_numpy(p["X"]).to(dev).to(torch.bfloat16)
        t["S"] = torch.from_numpy(p["S"]).to(dev).to(torch.bfloat16)
        t["A_sf"] = torch.from_numpy(p["A_sf"]).to(dev).view(torch.float8_e4m3fn)
        t["W_sf"] = torch.from_numpy(p["W_sf"]).to(dev).view(torch.float8_e4m3fn)
        t["alpha"] = torch.tensor([1.0], device=dev, dtype=torch.float32)
        y_ref = orc.binary_expand(orc.binary_z(p["X"], p["V_packed"], p["S"]), p["U_packed"], True)
        row = {}
        row["pad_us"] = time_graph(torch, lambda: ops.fp4_gemm_n64(t["A_pad"], t["W"], t["A_sf"], t["W_sf"], t["alpha"]), None)
        row["s128_us"] = time_graph(torch, lambda: ops.fp4_gemm_n128(t["A"], t["W"], t["A_sf"], t["W_sf"], t["alpha"]), None)
        for mode in (2, 4):
            g = RefGemm(torch, ops, t, p, M, mode, N, K, R)
            g.reset()
            worst = 0.0
            finite = True
            for _ in range(5):
                y = g().view(-1, N)[:M].float()
                torch.cuda.synchronize()
                finite = finite and bool(torch.isfinite(y).all())
                worst = max(worst, float(np.abs(y.cpu().numpy() - y_ref).max()))
            row[f"mode{mode}_err_over_max"] = worst / float(np.abs(y_ref).max())
            row[f"mode{mode}_finite"] = finite
            row[f"mode{mode}_us"] = time_graph(torch, g, g.reset)
        # HBM-cold arm: the same graph over `cold-layers` DISTINCT weights and factors (every launch streams its operands
        # from HBM), one launch per layer; the reference's own tables do not have this column
        if a.cold_layers > 0:
            rng = torch.Generator(device=dev).manual_seed(M)
            layers = []
            for _ in range(a.cold_layers):
                q = dict(t)
                q["W"] = torch.randint(0, 256, (N, K // 2), device=dev, dtype=torch.uint8, generator=rng)
                q["W_sf"] = torch.zeros_like(t["W_sf"])
                layers.append(q)
            row["pad_cold_us"] = time_graph(torch, lambda: [ops.fp4_gemm_n64(q["A_pad"], q["W"], q["A_sf"], q["W_sf"], q["alpha"])
                                                            for q in layers], None, batch=1) / len(layers)
            for mode in (2, 4):
                if row[f"mode{mode}_err_over_max"] > 0.01:
                    continue
                gs = []
                for q in layers:
                    pq = dict(p)
                    pq["V_packed"] = np.random.default_rng(len(gs)).integers(0, 256, p["V_packed"].shape, dtype=np.uint8)
                    pq["U_packed"] = np.random.default_rng(1000 + len(gs)).integers(0, 256, p["U_packed"].shape, dtype=np.uint8)
                    q = dict(q)
                    q["V_packed"] = torch.from_numpy(pq["V_packed"]).to(dev)
                    gs.append(RefGemm(torch, ops, q, pq, M, mode, N, K, R))

                def reset_all():
                    for g in gs:
                        g.reset()

                row[f"mode{mode}_cold_us"] = time_graph(torch, lambda: [g() for g in gs], reset_all, batch=1) / len(gs)
                del gs
            del layers
        out["rows"][str(M)] = row
        print(f"# M={M}: {row}", file=sys.stderr, flush=True)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
