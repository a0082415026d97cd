"""The allocation-free decode matvec (bhd_matvec_noalloc) against the ordinary entry point.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else. The entry point exists for hosts that must not allocate device memory
while serving (real-time decode loops, processes that handed all of HBM to their own arena):
its scratch is a fixed array inside the library instead of the context workspace. bhd_matvec may
pick a different kernel for the same shape (the integer one for one or two vectors), so the two
agree within the path's stated tolerance, not to the bit; both are also held against the CPU
oracle. Two calls in a row with different inputs show that nothing of the first call's scratch
contents survives into the second. The first call runs on a context that has done nothing else,
and the free device memory the driver reports must be the same before and after it: the entry
point may not allocate.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3


def max_rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = np.maximum(np.abs(want), np.sqrt((want ** 2).mean()))
    return float((np.abs(got - want) / den).max())


@pytest.mark.parametrize("kind,rows,cols,batch", [(12, 1536, 4096, 1), (8, 768, 2048, 2), (14, 512, 4096, 4), (8, 64, 1024, 3)])
def test_noalloc_matvec_matches_the_allocating_entry_point_twice_in_a_row(oracle, kind, rows, cols, batch):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice, Weight, synth

    dev = CudaDevice(0)
    packed = synth.matrix(kind, 61, rows, cols)
    w = dev.upload_weight(Weight(packed, kind, rows, cols))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # Load the library's device code first (the driver loads a module lazily, on its first launch, and that
    # takes device memory) with a call that needs no workspace, so that the measurement below sees only
    # what the entry point itself does.
    probe = torch.zeros(8, device="cuda")
    assert dev.lib.bhd_debug_expf(dev.ctx, C.c_void_p(probe.data_ptr()), C.c_void_p(probe.data_ptr()), 8, stream) == 0
    for call in range(2):
        x_np = synth.activations(70 + call, (batch, cols))
        x = torch.from_numpy(x_np).cuda()
        got = torch.full((batch, rows), float("nan"), device="cuda")
        want = torch.empty((batch, rows), device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        # first thing this context ever runs (call 0): its workspace does not exist yet
        st = dev.lib.bhd_matvec_noalloc(dev.ctx, w.handle, 0, C.c_void_p(x.data_ptr()), C.c_void_p(got.data_ptr()), batch,
                                        1.0, 0, stream)
        assert st == 0, dev._message()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the free device memory"
        dev.check_status()
        dev.matvec_resident(w, x, want)
        dev.check_status()
        assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL, f"call {call}"
        assert max_rel_err(got.cpu().numpy(), oracle.matvec_batch(packed, kind, rows, cols, x_np)) <= TOL, f"call {call} vs oracle"
        # scaled accumulate form
        acc = torch.ones((batch, rows), device="cuda")
        st = dev.lib.bhd_matvec_noalloc(dev.ctx, w.handle, 0, C.c_void_p(x.data_ptr()), C.c_void_p(acc.data_ptr()), batch,
                                        0.5, 1, stream)
        assert st == 0, dev._message()
        assert max_rel_err(acc.cpu().numpy(), (1.0 + 0.5 * want).cpu().numpy()) <= TOL
    w.free()
    dev.close()


def test_noalloc_matvec_refuses_what_the_fixed_array_cannot_hold():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice, Weight, synth

    dev = CudaDevice(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows, cols = 16, 32768          # four vectors of 32768 columns need more than the fixed array holds
    w = dev.upload_weight(Weight(synth.matrix(12, 5, rows, cols), 12, rows, cols))
    x = torch.zeros((4, cols), device="cuda")
    y = torch.full((4, rows), 7.0, device="cuda")
    st = dev.lib.bhd_matvec_noalloc(dev.ctx, w.handle, 0, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 4, 1.0, 0, stream)
    assert st == -2 and "fixed" in dev._message()
    assert torch.all(y == 7.0)      # a refused call leaves the output alone
    w2 = dev.upload_weight(Weight(synth.matrix(12, 5, 16, 256), 12, 16, 256))
    x5 = torch.zeros((5, 256), device="cuda")
    y5 = torch.zeros((5, 16), device="cuda")
    st = dev.lib.bhd_matvec_noalloc(dev.ctx, w2.handle, 0, C.c_void_p(x5.data_ptr()), C.c_void_p(y5.data_ptr()), 5, 1.0, 0, stream)
    assert st == -2 and "at most 4" in dev._message()
    w.free(); w2.free(); dev.close()
