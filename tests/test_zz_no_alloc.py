"""The allocation-free decode matvec (bhd_matvec_noalloc) against the ordinary entry point.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else. The entry point exists for hosts that must not allocate device memory
while serving (real-time decode loops, processes that handed all of HBM to their own arena):
its scratch is a fixed array inside the library instead of the context workspace. Same kernels,
so the results must agree with bhd_matvec to the bit; the check allows the path's stated
tolerance. Two calls in a row with different inputs show that nothing of the first call's
scratch contents survives into the second.
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
def test_noalloc_matvec_matches_the_allocating_entry_point_twice_in_a_row(kind, rows, cols, batch):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice, Weight, synth

    dev = CudaDevice(0)
    w = dev.upload_weight(Weight(synth.matrix(kind, 61, rows, cols), kind, rows, cols))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        x = torch.from_numpy(synth.activations(70 + call, (batch, cols))).cuda()
        want = torch.empty((batch, rows), device="cuda")
        dev.matvec_resident(w, x, want)
        got = torch.full((batch, rows), float("nan"), device="cuda")
        st = dev.lib.bhd_matvec_noalloc(dev.ctx, w.handle, 0, C.c_void_p(x.data_ptr()), C.c_void_p(got.data_ptr()), batch,
                                        1.0, 0, stream)
        assert st == 0, dev._message()
        dev.check_status()
        assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL, f"call {call}"
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
