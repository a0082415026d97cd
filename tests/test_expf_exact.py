"""The device's expf against the host libm's, bit for bit.

The reference's softmax calls the host libm (Rust f32::exp, crates/beholdd-kernel/src/vecops.rs:
70-87) and stable_top_k ranks the resulting probabilities (crates/beholdd-model/src/qwen3moe/
forward.rs:1886-1924), so expert selection on the device is the CPU's selection only if both
expf give the same floats. The library restates the algorithm glibc uses; this sweeps it
against the libm of the host the test runs on: every 256th float of the argument range softmax
can produce (x <= 0 after the max is subtracted, down to underflow) and of the positive range
SiLU uses, 2^24 arguments in all.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_expf_equals_host_libm_on_a_strided_sweep(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from exec_beholdd_b200 import CudaDevice

    dev = CudaDevice(0)
    # Bit patterns of the finite floats with |x| <= 128, both signs, every 256th one: expf is 0 or inf outside.
    hi = np.float32(128.0).view(np.uint32)
    n = 1 << 23
    stride = max(1, int(hi) // n)
    mag = (np.arange(n, dtype=np.uint64) * stride).astype(np.uint32)
    args = np.concatenate([mag, mag | np.uint32(0x80000000)]).view(np.float32)
    assert args.size == 1 << 24
    want = oracle.expf(args)
    a = torch.from_numpy(args).cuda()
    out = torch.empty_like(a)
    st = dev.lib.bhd_debug_expf(dev.ctx, C.c_void_p(a.data_ptr()), C.c_void_p(out.data_ptr()), args.size,
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, dev._message()
    got = out.cpu().numpy()
    differ = np.flatnonzero(got.view(np.uint32) != want.view(np.uint32))
    print(f"expf sweep: {args.size} arguments, {differ.size} differ from the host libm")
    # Known: the published algorithm and this host's libm disagree on isolated arguments near underflow
    # (results below 2^-80, never reached by a probability that competes for the top-k).
    for i in differ[:10]:
        print(f"  x = {args[i]!r}: device {got[i]!r}, host {want[i]!r}")
    relevant = [i for i in differ if want[i] > 1e-20]
    assert not relevant, f"{len(relevant)} arguments with exp(x) > 1e-20 differ"
    assert differ.size <= 16
    dev.close()
