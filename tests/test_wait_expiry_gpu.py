"""GPU: what happens when a bounded device-side wait runs out.

Every mbarrier wait in the tensor-core kernels has a probe limit; on expiry the kernel sets a
device status word, lets its copies land, frees its tensor memory and returns, and the host
reads the word through vaicu_device_status (VAICU_ERR_TIMEOUT, cleared on read) — the place
of the reference's lost-device report in NeuralNet::sync() (vAi vai/engine/neural-net.cpp:206-217).
Nothing in a healthy run ever sets the word, so the path is exercised with the library's own
self-test launch: a single warp that waits 1024 probes on a barrier nobody arrives on.  No
fault, no trap, no endless loop: the kernel returns normally and the context stays usable,
which the last step checks by running a Linear."""
import ctypes

import numpy as np
import pytest

from vai_b200 import _lib

pytestmark = pytest.mark.gpu

ERR_TIMEOUT = 8


def test_expired_wait_is_reported_once_and_the_context_survives(device):
    lib = device.lib
    word = ctypes.c_int(-1)
    assert lib.vaicu_device_status(device.handle, ctypes.byref(word)) == 0 and word.value == 0     # clean to begin with
    stream = device.create_stream()
    _lib.check(lib.vaicu_device_selftest_wait_expiry(device.handle, stream), "selftest")
    _lib.check(lib.vaicu_stream_sync(stream), "sync")                                                # the kernel came back
    assert lib.vaicu_device_status(device.handle, ctypes.byref(word)) == ERR_TIMEOUT and word.value != 0
    assert lib.vaicu_status_string(ERR_TIMEOUT) == b"a bounded device-side wait expired"
    assert lib.vaicu_device_status(device.handle, ctypes.byref(word)) == 0 and word.value == 0     # cleared by the read
    # the host API raises on it
    _lib.check(lib.vaicu_device_selftest_wait_expiry(device.handle, stream), "selftest")
    with pytest.raises(_lib.VaicuError) as err:
        device.check_status()
    assert err.value.status == ERR_TIMEOUT
    device.check_status()                                                                            # and only once
    # a tensor-core Linear right after: same context, right answer, no status
    from gpu_util import run_linear
    from linear_check import assert_close
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    w = (rng.standard_normal((128, 256)) / 16).astype(np.float32)
    got, want, node = run_linear(x, w, i_dtype="bf16", w_dtype="bf16")
    assert node.info.kernel == 4
    assert_close(got, want, (2e-4, 5e-5), "Linear after the self-test")
    device.check_status()
    lib.vaicu_stream_destroy(stream)
