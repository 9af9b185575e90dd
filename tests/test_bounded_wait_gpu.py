"""The expiry path of the kernels' bounded waits, exercised without faulting anything: one
thread waits (1 ms limit) on a barrier phase that nothing completes.  The wait must give up,
record its code in the device status word and let the kernel return; the context must stay
usable, and the next ordinary launch must be correct."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_status_and_context_survives(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    from oracle import mgx_oracle as O
    lib = capi.load()
    assert capi.device_status() == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.mgx_cuda_selftest_bounded_wait(1_000_000, gave_up.data_ptr(), stream)
    assert rc == 0, capi.status_string(rc)
    torch.cuda.synchronize()          # the kernel returned by itself
    assert int(gave_up.item()) == 99  # the wait gave up and raised the CTA's abort flag
    assert capi.device_status() == 99  # ... and the host can see it (reading clears the word)
    assert capi.device_status() == 0
    # the context is intact: an ordinary launch right after it is bit-exact
    rng = np.random.default_rng(5)
    a = rng.integers(-128, 128, size=(128, 256), dtype=np.int8)
    b = rng.integers(-128, 128, size=(256, 128), dtype=np.int8)
    acc = capi.qgemm(torch.from_numpy(a).to(cuda_device), torch.from_numpy(b).to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(acc.cpu().numpy(), O.quant_dot_int8(a, b))
    assert capi.device_status() == 0
    # the probe refuses to park a GPU for long
    assert lib.mgx_cuda_selftest_bounded_wait(10**10, None, stream) == capi.E_INVALID_ARG
