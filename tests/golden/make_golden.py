"""Generate tests/golden/*.npz by RUNNING the reference's own Python on CPU.

    python tests/golden/make_golden.py [/path/to/reference]

The reference tree is only needed when regenerating; the committed .npz files are what the tests read.

What is taken from the reference (imported / executed, never copied):
  * biloco/peel.py            -> set_peel_seed, binary_peel, refit_alphas, decompose   (imported by path)
  * biloco/kernel.py          -> pack_signs, pack_u_col32, nvfp4_sf_bytes, modes_for, DEFAULT_MODE, RANKS
                                 (the module imports a compiled extension, so the function definitions are
                                 extracted with `ast` from the file and executed unchanged)
  * biloco/layer.py           -> BiLoCoLinear.quantize / forward, executed with a stand-in `fouroversix`
                                 module whose quantise/dequantise is the oracle's NVFP4 restatement
                                 (fouroversix itself is not installed; see oracle/biloco_oracle.py header)
"""
import ast
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)
from oracle import biloco_oracle as orc  # noqa: E402


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def extract_defs(path, names):
    """Execute only the named top-level functions / assignments of a Python file."""
    src = open(path).read()
    tree = ast.parse(src)
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in names for t in node.targets):
            keep.append(node)
    ns = {"torch": torch}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
    return ns


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BILOCO_REFERENCE", "")
    if not os.path.isdir(os.path.join(ref, "biloco")):
        sys.exit("usage: make_golden.py <path of a checkout of the reference>   (or set BILOCO_REFERENCE)")
    peel = load_by_path("ref_peel", os.path.join(ref, "biloco", "peel.py"))
    kern = extract_defs(os.path.join(ref, "biloco", "kernel.py"),
                        {"pack_signs", "pack_u_col32", "nvfp4_sf_bytes", "modes_for", "DEFAULT_MODE", "RANKS"})

    out = {}

    # ---- 1. sign packing -------------------------------------------------------------------
    g = torch.Generator().manual_seed(7)
    s = torch.sign(torch.randn(6, 64, generator=g))
    s[0, :5] = 0.0                                   # zero counts as +1
    out["signs_in"] = s.numpy()
    out["signs_packed"] = kern["pack_signs"](s).numpy()
    Ut = torch.sign(torch.randn(40, 24, generator=g)); Ut[Ut == 0] = 1   # [R=40, N=24]
    up = kern["pack_signs"](Ut)
    out["u_signs"] = Ut.numpy()
    out["u_packed"] = up.numpy()
    out["u_col32"] = kern["pack_u_col32"](up, n_cols=24, rank=40).numpy()
    out["sf_bytes_cases"] = np.array([[r, k, kern["nvfp4_sf_bytes"](r, k)]
                                      for r, k in [(1, 5120), (128, 5120), (5120, 5120), (129, 64), (1024, 2560), (9728, 80)]],
                                     dtype=np.int64)
    # mode table of the reference (availability + default), flattened
    Ms, Rs = (1, 2, 4, 8, 16, 32), kern["RANKS"]
    out["ranks"] = np.array(Rs, dtype=np.int64)
    out["default_mode"] = np.array([[kern["DEFAULT_MODE"][m][r] for r in Rs] for m in Ms], dtype=np.int64)
    avail = np.zeros((len(Ms), len(Rs), 3), dtype=np.int64)
    for i, m in enumerate(Ms):
        for j, r in enumerate(Rs):
            for mode in kern["modes_for"](m, r, 5120):
                avail[i, j, {2: 0, 4: 1, 5: 2}[mode]] = 1
    out["modes_avail_k5120"] = avail

    # ---- 2. decomposition (tests/run_tests.py:18-30 case, and a small layer) ----------------
    torch.manual_seed(0)
    W = torch.randn(256, 384)
    peel.set_peel_seed(42)
    U, V, S, R = peel.binary_peel(W, r=32, T=5)
    S2, R2 = peel.refit_alphas(W, U, V, S)
    out["peel_U_packed"] = kern["pack_signs"](U.T.contiguous()).numpy()     # [32, 256/8]
    out["peel_V_packed"] = kern["pack_signs"](V.T.contiguous()).numpy()     # [32, 384/8]
    out["peel_S"] = S.numpy()
    out["peel_S_refit"] = S2.numpy()
    out["peel_R_norm"] = np.array([float(W.norm()), float(R.norm()), float(R2.norm())], dtype=np.float64)

    # ---- 3. a small quantised layer through the reference's BiLoCoLinear ---------------------
    # stand-in for the missing third-party quantiser: the oracle's NVFP4 restatement (rule "mse")
    fo = types.ModuleType("fouroversix")

    class _QT:
        def __init__(self, deq, dtype):
            self.deq, self.dtype = deq, dtype

    def quantize_to_fp4(x, config=None):
        rule = getattr(config, "scale_rule", "mse")
        xn = x.detach().to(torch.float32).numpy()
        return _QT(torch.from_numpy(orc.fake_quantize_fp4(xn, rule)), x.dtype)

    fo.quantize_to_fp4 = quantize_to_fp4
    fq = types.ModuleType("fouroversix.quantize")
    fq.dequantize = lambda qt: qt.deq.to(qt.dtype)
    fqc = types.ModuleType("fouroversix.quantize.config")

    class QuantizationConfig:
        def __init__(self, scale_rule="mse"):
            self.scale_rule = scale_rule

    fqc.QuantizationConfig = QuantizationConfig
    fu = types.ModuleType("fouroversix.utils")

    class ScaleRule:
        static_4, static_6, abs_max, mse, mae = "static_4", "static_6", "abs_max", "mse", "mae"

    fu.ScaleRule = ScaleRule
    sys.modules.update({"fouroversix": fo, "fouroversix.quantize": fq,
                        "fouroversix.quantize.config": fqc, "fouroversix.utils": fu})
    pkg = types.ModuleType("biloco"); pkg.__path__ = [os.path.join(ref, "biloco")]
    sys.modules["biloco"] = pkg
    sys.modules["biloco.peel"] = load_by_path("biloco.peel", os.path.join(ref, "biloco", "peel.py"))
    sys.modules["biloco.fp4"] = load_by_path("biloco.fp4", os.path.join(ref, "biloco", "fp4.py"))
    layer = load_by_path("biloco.layer", os.path.join(ref, "biloco", "layer.py"))

    K, N, r, M = 256, 128, 32, 3
    torch.manual_seed(0)
    lin = torch.nn.Linear(K, N, bias=True)
    with torch.no_grad():
        lin.weight.copy_(0.02 * torch.randn(N, K))
        lin.bias.copy_(0.01 * torch.randn(N))
    sys.modules["biloco.peel"].set_peel_seed(42)
    bl = layer.BiLoCoLinear(lin, rank=r)
    act_max = torch.rand(K) * 4 + 0.5
    bl.quantize(act_col_max=act_max, T=5)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g)
    idx = torch.randperm(K, generator=g)[: max(1, K // 100)]
    x[:, idx] *= 20
    x = x.to(torch.bfloat16)
    y = bl(x)
    out["layer_W"] = lin.weight.detach().float().numpy()
    out["layer_act_max"] = act_max.numpy()
    out["layer_x"] = x.float().numpy()
    out["layer_y"] = y.float().numpy()
    out["layer_smooth"] = bl.smooth_scale.float().numpy()
    out["layer_V_scaled"] = bl.V_scaled.float().numpy()
    out["layer_U_T"] = bl.U_T.float().numpy()
    out["layer_weight_fp4"] = bl.weight_fp4.float().numpy()
    out["layer_bias"] = bl.bias.float().numpy()

    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"),
          {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
