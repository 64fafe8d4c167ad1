"""Device-side waits are bounded and report instead of hanging.

The pipelined kernels wait on shared-memory barriers with a time limit; a wait
that gives up bumps a per-device counter (fb_device_faults) and the kernel
returns.  The self-test entry runs that very wait on a barrier nothing will
complete, with a short limit, so the reporting path is exercised without
faulting, trapping or hanging anything.
"""
import time

import numpy as np
import pytest

from ferro_b200 import kinds as K

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    import ferro_b200.backend as b
    be = b.CudaBackend(0)
    be.synchronize()
    assert be.lib.fb_device_faults(1) >= 0  # clear whatever an earlier test left
    assert be.lib.fb_device_faults(0) == 0
    t0 = time.time()
    be._check(be.lib.fb_selftest_bounded_wait(be._s(), 50))
    be.stream.synchronize()
    assert time.time() - t0 < 5.0
    assert be.lib.fb_device_faults(0) == 1
    # the host mirror reports it at the next synchronisation (and clears the word)
    with pytest.raises(b.DeviceFault):
        be.synchronize()
    assert be.lib.fb_device_faults(0) == 0
    be.synchronize()
    # ... and at the next read-back
    be._check(be.lib.fb_selftest_bounded_wait(be._s(), 20))
    with pytest.raises(b.DeviceFault):
        be.copy_to_host(be.alloc_from_host(np.float32([1])))
    assert be.lib.fb_device_faults(0) == 0
    # the context is still usable
    x = be.alloc_from_host(np.float32([1, -2, 3]))
    assert be.copy_to_host(be.unary_dev(b.UnaryKind(K.UN_RELU, 0.0, 0.0), x)).tolist() == [1, 0, 3]
    # limits outside 1 .. 1000 ms are refused before anything is launched
    assert be.lib.fb_selftest_bounded_wait(be._s(), 0) != 0
    assert be.lib.fb_selftest_bounded_wait(be._s(), 5000) != 0
