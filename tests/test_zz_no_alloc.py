"""The allocation-free entry point (biloco_b200_fused_linear_noalloc), called through the C ABI.

It exists for hosts that cannot hand the library a scratch buffer (a plugin inside a server whose memory plan is
frozen, a callback that must not re-enter the framework's allocator): its scratch is an array built into the library.
The test checks that it gives the same output as the allocating entry point, bit for bit, on two calls in a row (the
second call meets whatever the first one left in the shared array), after a call with a different shape, and that it
turns down a problem larger than the built-in array. Collected last on purpose: a failure here must not hide the rest.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import biloco_oracle as orc
from tests.gpu_util import check_against_unfused, dev_problem, oracle_outputs

pytestmark = pytest.mark.gpu


def _run_both(kernel, lib, M, N, K, R, mode, seed):
    p = orc.random_problem(M, K, N, R, scales="random", seed=seed)
    t = dev_problem(p)
    stream = torch.cuda.current_stream().cuda_stream
    g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=mode)
    want = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].clone()
    torch.cuda.synchronize()
    check_against_unfused(want.float().cpu().numpy(), oracle_outputs(p, M)[0], "allocating entry point")
    outs = []
    for call in range(2):
        y = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        rc = lib.biloco_b200_fused_linear_noalloc(
            t["W"].data_ptr(), t["W_sf"].data_ptr(), g.W_tiled.data_ptr(), t["alpha"].data_ptr(), t["A_pad"].data_ptr(),
            t["A_sf"].data_ptr(), t["X"].data_ptr(), t["V_packed"].data_ptr(), g.U_col32.data_ptr(), t["S"].data_ptr(),
            None, y.data_ptr(), M, 128, N, K, R, mode, stream)
        assert rc == 0, lib.biloco_b200_error_string(rc)
        torch.cuda.synchronize()
        st = (ctypes.c_int32 * 16)()
        assert lib.biloco_b200_noalloc_status(st, stream) == 0 and st[0] == 0, list(st)[:4]
        outs.append(y)
    for call, y in enumerate(outs):
        # same kernel, same operands, deterministic reduction order: identical bits (tolerance of the suite: 0 here)
        assert torch.equal(y.view(torch.int16), want.view(torch.int16)), f"call {call} differs from the allocating entry point"


def test_noalloc_matches_allocating_entry_point(lib):
    from biloco_b200 import kernel
    assert torch.cuda.is_available()
    _run_both(kernel, lib, 4, 1024, 2560, 128, 2, seed=11)
    _run_both(kernel, lib, 1, 640, 768, 64, 4, seed=12)       # other shape and mode: the shared array is re-armed
    _run_both(kernel, lib, 4, 1024, 2560, 128, 2, seed=13)     # back to the first shape, fewer ranks left stale data


def test_noalloc_rejects_what_does_not_fit(lib):
    from biloco_b200 import kernel
    M, N, K, R = 32, 151936, 2560, 512
    assert kernel.scratch_bytes(M, N, K, R) > 4 * 1024 * 1024
    d = torch.zeros(64, device="cuda", dtype=torch.uint8)      # never dereferenced: the call must refuse first
    ptr = d.data_ptr()
    rc = lib.biloco_b200_fused_linear_noalloc(ptr, ptr, None, ptr, ptr, ptr, ptr, ptr, ptr, ptr, None, ptr, M, 32, N, K, R, 2,
                                              torch.cuda.current_stream().cuda_stream)
    assert rc == -8 and b"maximum" in lib.biloco_b200_error_string(rc)
