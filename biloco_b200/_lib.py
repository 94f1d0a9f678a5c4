"""ctypes binding of libbiloco_b200.so (the C ABI declared in include/biloco_b200.h).

There is no fallback: if the library is missing, loading raises with the build command.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbiloco_b200.so")

OK = 0
RULES = {"static_6": 0, "static_4": 1, "mse": 2}
MODE_COUNTER, MODE_OWNER, MODE_CLUSTER, MODE_SLAB = 2, 4, 5, 7
OPT_PDL, OPT_RING, OPT_TRIGGER, OPT_LR_TC, OPT_WAIT_BUDGET_US, OPT_SKIP_PUBLISH = 1, 2, 3, 4, 5, 6
OPT_ZTC = 8

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

# name -> (restype, argtypes); one entry per symbol declared in include/biloco_b200.h
SIGNATURES = {
    "biloco_b200_error_string": (ctypes.c_char_p, [_i]),
    "biloco_b200_abi_version": (_i, []),
    "biloco_b200_sf_bytes": (_sz, [_i, _i]),
    "biloco_b200_binary_z": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "biloco_b200_binary_expand": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "biloco_b200_pack_u_col32": (_i, [_vp, _vp, _i, _i, _vp]),
    "biloco_b200_act_quant": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "biloco_b200_norm_act_quant": (_i, [_vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "biloco_b200_swiglu_act_quant": (_i, [_vp] * 9 + [_i] * 5 + [_vp]),
    "biloco_b200_decode_attention": (_i, [_vp, _vp, _vp, ctypes.c_float] + [_vp] * 6 + [_i] * 5 + [_vp]),
    "biloco_b200_max_active_clusters": (_i, [_i, _i]),
    "biloco_b200_act_rec_bytes": (_sz, [_i, _i]),
    "biloco_b200_peer_buffer_bytes": (_sz, [_i, _i]),
    "biloco_b200_peer_buffer_create": (_i, [_sz, ctypes.POINTER(ctypes.c_void_p), _vp]),
    "biloco_b200_peer_buffer_open": (_i, [_vp, ctypes.POINTER(ctypes.c_void_p)]),
    "biloco_b200_peer_buffer_close": (_i, [_vp]),
    "biloco_b200_peer_buffer_destroy": (_i, [_vp]),
    "biloco_b200_peer_allreduce": (_i, [_vp] * 5 + [_i] * 5 + [_vp]),
    "biloco_b200_peel_scratch_bytes": (_sz, [_i, _i, _i]),
    "biloco_b200_binary_peel": (_i, [_vp] * 6 + [_sz] + [_i] * 4 + [_vp]),
    "biloco_b200_fused_linear_act_supported": (_i, [_i] * 5),
    "biloco_b200_fused_linear_act": (_i, [_vp, _vp, _vp, _vp, ctypes.c_float, _vp, _i, _i] + [_vp] * 7 + [_sz] + [_i] * 6 + [_vp]),
    "biloco_b200_fused_linear_rec": (_i, [_vp] * 14 + [_sz] + [_i] * 7 + [_vp]),
    "biloco_b200_fused_linear_push": (_i, [_vp] * 14 + [_sz] + [_i] * 7 + [_vp, _vp, _i, _i, _i, _vp]),
    "biloco_b200_fused_linear_grouped": (_i, [_vp] * 14 + [_sz] + [_i] * 6 + [ctypes.POINTER(ctypes.c_int)] + [_i] * 2 + [_vp]),
    "biloco_b200_scratch_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "biloco_b200_scratch_head_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "biloco_b200_mode_supported": (_i, [_i, _i, _i, _i, _i, _i]),
    "biloco_b200_schedule_info": (_i, [_i, _i, _i, _i, _i, ctypes.POINTER(ctypes.c_int)]),
    "biloco_b200_tiled_bytes": (_sz, [_i, _i]),
    "biloco_b200_tile_weights": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "biloco_b200_slab_bytes": (_sz, [_i, _i, _i]),
    "biloco_b200_slab_info": (_i, [_i, _i, _i, _i, _i, ctypes.POINTER(ctypes.c_int)]),
    "biloco_b200_tile_weights_slab": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "biloco_b200_fused_linear": (_i, [_vp] * 13 + [_sz] + [_i] * 7 + [_vp]),
    "biloco_b200_set_option": (_i, [_i, _i]),
    "biloco_b200_debug_stamps": (_i, [_vp, _sz]),
    "biloco_b200_fused_linear_noalloc": (_i, [_vp] * 12 + [_i] * 6 + [_vp]),
    "biloco_b200_noalloc_status": (_i, [ctypes.POINTER(ctypes.c_int32), _vp]),
    "biloco_b200_read_status": (_i, [_vp, ctypes.POINTER(ctypes.c_int32), _vp]),
    "biloco_b200_fp4_gemm_simt": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
}

_lib = None


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m biloco_b200.csrc.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header and library out of sync
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(code: int, what: str):
    if code != OK:
        msg = load().biloco_b200_error_string(code).decode()
        raise RuntimeError(f"{what}: {msg} (code {code})")
