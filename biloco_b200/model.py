"""Whole-model post-training quantisation with kernel-backed layers.

Same entry points as the reference's ``biloco/model.py`` (replace_linears :11-18, collect_act_col_max :21-42,
quantize_model :45-60, save_quantized :63-67, load_quantized :70-84). The saved file holds the packed kernel operands
of every layer (NVFP4 codes, block scales, tensor scale, packed signs, coefficients, smoothing vector, bias), i.e.
exactly what the fused kernel streams, so loading needs no re-decomposition and no re-quantisation.
"""
import gc

import torch
import torch.nn as nn

from .layer import BiLoCoLinear

_SAVED = ("smooth_scale", "V_packed", "U_packed", "S", "W_codes", "W_sf", "w_gscale")


def replace_linears(model: nn.Module, rank: int, method: str = "biloco", smooth_factor: float = 0.5):
    """Swap every nn.Linear (lm_head included) for a BiLoCoLinear in place. Returns {qualified name: module}."""
    stack = [model]
    while stack:
        parent = stack.pop()
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear):
                setattr(parent, name, BiLoCoLinear(child, rank=rank, method=method, smooth_factor=smooth_factor))
            else:
                stack.append(child)
    return {n: m for n, m in model.named_modules() if isinstance(m, BiLoCoLinear)}


@torch.no_grad()
def collect_act_col_max(ref_model, names, batches, forward=None, calib_batches: int = 4):
    """Per-input-channel max |x| seen by every named nn.Linear of ref_model over the first calib_batches batches.
    `batches` yields model inputs; `forward(model, batch)` runs one of them (default: model(batch), or model(**batch)
    for a dict). The reference tokenises text batches itself (biloco/model.py:36-40); tokenisation is the caller's here."""
    col_max, hooks = {}, []

    def make_hook(name):
        def hook(_m, inp, _out):
            x = inp[0] if isinstance(inp, tuple) else inp
            mx = x.reshape(-1, x.shape[-1]).float().abs().max(dim=0).values.cpu()
            col_max[name] = mx if name not in col_max else torch.max(col_max[name], mx)
        return hook

    for name, mod in ref_model.named_modules():
        if isinstance(mod, nn.Linear) and name in names:
            hooks.append(mod.register_forward_hook(make_hook(name)))
    try:
        for i, batch in enumerate(batches):
            if i >= calib_batches:
                break
            if forward is not None:
                forward(ref_model, batch)
            elif isinstance(batch, dict):
                ref_model(**batch)
            else:
                ref_model(batch)
    finally:
        for h in hooks:
            h.remove()
    return col_max


@torch.no_grad()
def quantize_model(model, ref_model=None, batches=None, rank: int = 512, method: str = "biloco", T: int = 5,
                   smooth_factor: float = 0.5, calib_batches: int = 4, device=None, forward=None):
    """Quantise `model` in place. SmoothQuant statistics come from ref_model (an unmodified copy) run on `batches`;
    ref_model=None skips smoothing."""
    device = device or torch.device("cuda")
    layers = replace_linears(model, rank=rank, method=method, smooth_factor=smooth_factor)
    col_max = {}
    if ref_model is not None and batches is not None:
        col_max = collect_act_col_max(ref_model, set(layers), batches, forward=forward, calib_batches=calib_batches)
    for i, (name, m) in enumerate(layers.items()):
        m.quantize(act_col_max=col_max.get(name), T=T, device=device)
        if (i + 1) % 50 == 0:
            gc.collect()
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
    return model


def save_quantized(model, path: str, manifest: dict = None):
    """Save the packed kernel operands of every BiLoCoLinear (the rest of the model is the original checkpoint)."""
    layers = {}
    for n, m in model.named_modules():
        if isinstance(m, BiLoCoLinear):
            st = {k: getattr(m, k).detach().cpu() for k in _SAVED}
            st["smoothed"] = bool(m.smoothed)
            if m.bias is not None:
                st["bias"] = m.bias.detach().cpu()
            layers[n] = st
    torch.save({"layers": layers, "manifest": manifest or {}, "format": "biloco_b200.packed.v1"}, path)


@torch.no_grad()
def load_quantized(model, path: str, rank: int, method: str = "biloco"):
    """Replace the linears of a freshly built model and restore the saved packed operands. Returns the manifest."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    layers = replace_linears(model, rank=rank, method=method)
    for name, m in layers.items():
        st = blob["layers"][name]
        for k in _SAVED:
            getattr(m, k).copy_(st[k])
        m.smoothed = bool(st.get("smoothed", False))
        if m.bias is not None:
            m.bias.copy_(st["bias"])
        m.weight = None
    return blob["manifest"]
