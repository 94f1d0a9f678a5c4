"""The failure path of the device-side waits, exercised without hanging or faulting anything: one CTA of a row-slab launch
is told (by a host option) to keep its z values to itself, so every consumer's bounded poll runs out of its (shortened)
budget, records its code in the scratch's status words and leaves through the common exit. The call returns, the status
says which wait gave up, reset() re-arms the scratch and the next call is bit-identical to a clean one.
Counterpart in the reference: the bounded polls that record a code in Diag[4095] (csrc/biloco_gemm.cu:1149-1151, 1288).
Collected late on purpose: it leaves the library's process-wide options at their defaults, but a failure here should not
hide the results of the other tests."""
import time

import numpy as np
import pytest
import torch

from oracle import biloco_oracle as orc
from tests.gpu_util import dev_problem

pytestmark = pytest.mark.gpu

ST_Z = 105          # status code of the z poll (csrc/fused_cfg.cuh)


@pytest.mark.parametrize("M", [1, 4])        # (the four-row kernel has a z poll of its own: two vectors per round trip)
def test_z_poll_runs_out_and_scratch_recovers(M):
    from biloco_b200 import _lib, kernel
    lib = _lib.load()
    K, N, R = 1024, 1024, 512              # (every CTA owns at least three ranks)
    assert 7 in kernel.supported_modes(M, N, K, R)
    p = orc.random_problem(M, K, N, R, scales="random", seed=11)
    t = dev_problem(p)
    g = kernel.BiLoCoGemm(t["W"], t["W_sf"], t["alpha"], t["V_packed"], t["U_packed"], t["S"], M=M, mode=7)

    def run():
        y = g(t["A_pad"], t["A_sf"], t["X"]).view(-1, N)[:M].clone()
        torch.cuda.synchronize()
        return y

    clean = run()
    assert g.status()[0] == 0
    try:
        lib.biloco_b200_set_option(_lib.OPT_WAIT_BUDGET_US, 2000)
        lib.biloco_b200_set_option(_lib.OPT_SKIP_PUBLISH, 0)          # CTA 0 computes its z slice and does not publish it
        t0 = time.perf_counter()
        run()
        dt = time.perf_counter() - t0
    finally:
        lib.biloco_b200_set_option(_lib.OPT_SKIP_PUBLISH, -1)
        lib.biloco_b200_set_option(_lib.OPT_WAIT_BUDGET_US, 0)         # back to the default budget
    st = g.status()
    assert st[0] == ST_Z, f"expected the z poll's code in the status word, got {st[:4]}"
    assert 0 <= st[1] < 148 * 2 and st[2] == g.epoch                   # the block that gave up first, the call's epoch
    assert dt < 1.0, f"the call took {dt:.3f} s: a wait did not honour its budget"
    # the status word is sticky until the scratch's head is cleared
    g.reset()
    assert g.status()[0] == 0
    again = run()
    assert g.status()[0] == 0
    assert torch.equal(again.view(torch.int16), clean.view(torch.int16)), "the call after reset() differs from a clean one"
    again = run()
    assert torch.equal(again.view(torch.int16), clean.view(torch.int16))


def test_peer_allreduce_wait_runs_out_and_reports(lib):
    """The peer all-reduce polls its own receive buffer for the peers' words with a time budget. Here a 'group' of two
    with nobody behind rank 1 (its buffer is a second local allocation that nothing reads or writes back): the poll runs
    out, the kernel records it and returns, the context stays usable, and a later launch on the same GPU is unaffected."""
    import ctypes
    world, slot = 2, 1024
    nbytes = lib.biloco_b200_peer_buffer_bytes(world, slot)
    bufs = []
    for _ in range(2):
        p, h = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        assert lib.biloco_b200_peer_buffer_create(nbytes, ctypes.byref(p), h) == 0
        bufs.append(p.value)
    table = torch.tensor(bufs, dtype=torch.int64, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    part = torch.ones(512, device="cuda")
    out = torch.zeros(512, device="cuda", dtype=torch.bfloat16)
    assert lib.biloco_b200_set_option(5, 2000) == 0              # BILOCO_OPT_WAIT_BUDGET_US
    try:
        rc = lib.biloco_b200_peer_allreduce(part.data_ptr(), None, out.data_ptr(), table.data_ptr(), status.data_ptr(), world, 0, 512, slot, 0,
                                            torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
    finally:
        lib.biloco_b200_set_option(5, 0)
    st = status.cpu().tolist()
    assert st[0] == 1 and st[2] == 1 and st[3] == 0, st            # gave up, in call 1, on rank 0
    assert (st[8] >> 20) == 1                                       # the call counter advanced all the same
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0   # the context still works
    for b in bufs:
        assert lib.biloco_b200_peer_buffer_destroy(b) == 0
