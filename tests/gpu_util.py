"""Helpers shared by the GPU parity tests: move an oracle problem to the device and compare outputs."""
import numpy as np
import torch

from oracle import biloco_oracle as orc


def dev_problem(p, dev="cuda"):
    """numpy operands of oracle.random_problem -> CUDA tensors in the dtypes the operators take."""
    t = {}
    t["X"] = torch.from_numpy(p["X"]).to(dev).to(torch.bfloat16)
    t["S"] = torch.from_numpy(p["S"]).to(dev).to(torch.bfloat16)
    for k in ("V_packed", "U_packed", "A", "A_pad", "W"):
        t[k] = torch.from_numpy(p[k]).to(dev)
    t["A_sf"] = torch.from_numpy(p["A_sf"]).to(dev).view(torch.float8_e4m3fn)
    t["W_sf"] = torch.from_numpy(p["W_sf"]).to(dev).view(torch.float8_e4m3fn)
    t["alpha"] = torch.tensor([float(p["alpha"])], device=dev, dtype=torch.float32)
    return t


def check_against_unfused(y, y_ref, what=""):
    """The reference's own criterion (tests/run_tests.py:45): max |y - y_ref| <= 0.01 * max |y_ref|, plus the
    relative Frobenius bound 2e-3."""
    assert np.isfinite(y).all(), f"{what}: non-finite output"
    scale = float(np.max(np.abs(y_ref)))
    err = float(np.max(np.abs(y - y_ref)))
    assert err <= 0.01 * scale, f"{what}: max |err| {err:.5g} > 1% of max |y_ref| {scale:.5g}"
    fro = float(np.linalg.norm(y - y_ref)) / max(float(np.linalg.norm(y_ref)), 1e-30)
    assert fro <= 2e-3, f"{what}: relative Frobenius error {fro:.3g} > 2e-3"


def check_against_exact(y, y_exact, what=""):
    """Per-element relative error <= 1e-2 against the unrounded float64 result, with the denominator floored at
    1e-3 * max |y| (elements that cancel to nearly zero carry the fp32 accumulation noise of much larger terms)."""
    scale = float(np.max(np.abs(y_exact)))
    den = np.maximum(np.abs(y_exact), 1e-3 * scale)
    rel = np.abs(y - y_exact) / den
    assert float(rel.max()) <= 1e-2, f"{what}: per-element relative error {float(rel.max()):.3g} > 1e-2"


def oracle_outputs(p, M):
    a = (p["A_pad"], p["A_sf"], p["W"], p["W_sf"], float(p["alpha"]), p["X"], p["V_packed"], p["U_packed"], p["S"])
    zero_scales = not p["W_sf"].any() or not p["A_sf"].any()
    if zero_scales:      # the FP4 product is exactly 0: skip dequantising the weight
        z = orc.binary_z(p["X"], p["V_packed"], p["S"])
        return orc.binary_expand(z, p["U_packed"], True), orc.binary_expand(z, p["U_packed"], False)
    return orc.reference_unfused(*a, M=M), orc.fused_exact(*a, M=M)
