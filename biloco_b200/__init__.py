"""biloco_b200: B200 (sm_100a) implementation of BiLoCo's fused decode linear
y = FP4(x) FP4(R)^T + sum_i alpha_i (x . v_i) u_i, behind the reference's ``biloco.kernel`` interface.

``biloco_b200.kernel`` needs libbiloco_b200.so (``python -m biloco_b200.csrc.build``) and raises if it is missing.
"""
from .fp4 import fake_quantize_fp4, quantize_activation, quantize_nvfp4, set_scale_rules  # noqa: F401
from .layer import BiLoCoLinear  # noqa: F401
from .model import load_quantized, quantize_model, replace_linears, save_quantized  # noqa: F401
from .peel import binary_peel, decompose, refit_alphas, set_peel_seed  # noqa: F401
