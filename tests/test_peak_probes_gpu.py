"""The two measured ceilings bench.py quotes the convolution kernel against (include/mcb200_runtime.h):
the issue rate of tcgen05.mma on shared-memory operands and the rate of TMA pulls from L2 into
shared memory.  Checked here for plausibility only: they run, no bounded wait runs out, and the
figures are of the order the hardware's nominal numbers allow."""
import ctypes

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _mma(lib, bf16, n, pair, steps=2048):
    lib.mcb200_probe_mma_peak.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                          ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                          ctypes.c_void_p]
    ms, rate = ctypes.c_double(0.0), ctypes.c_double(0.0)
    rc = lib.mcb200_probe_mma_peak(bf16, n, pair, steps, 2, ctypes.byref(ms), ctypes.byref(rate), None)
    assert rc == 0, rc
    return ms.value, rate.value


def test_tf32_issue_rate(kernels):
    torch.zeros(1, device="cuda")
    rates = {}
    for n in (64, 128, 256):
        ms, rates[n] = _mma(kernels, 0, n, 0)
        assert ms > 0
    # nominal dense TF32 is 1.1 PFLOP/s; the wide tile must get within a factor of three of it and
    # cannot exceed it by much
    assert 350.0 < rates[256] < 1600.0, rates
    assert rates[64] <= rates[256] * 1.05, rates
    _, pair = _mma(kernels, 0, 256, 1)
    assert 350.0 < pair < 1600.0, pair


def test_bf16_issue_rate_is_about_twice_tf32(kernels):
    torch.zeros(1, device="cuda")
    _, tf32 = _mma(kernels, 0, 256, 0)
    _, bf16 = _mma(kernels, 1, 256, 0)
    assert 1.5 < bf16 / tf32 < 2.5, (tf32, bf16)


def test_mma_probe_rejects_bad_arguments(kernels):
    ms, rate = ctypes.c_double(0.0), ctypes.c_double(0.0)
    assert kernels.mcb200_probe_mma_peak(0, 96, 0, 16, 1, ctypes.byref(ms), ctypes.byref(rate), None) == -4
    assert kernels.mcb200_probe_mma_peak(0, 256, 0, 0, 1, ctypes.byref(ms), ctypes.byref(rate), None) == -1


def test_l2_to_shared_memory_rate(kernels):
    kernels.mcb200_probe_tma_l2_pull.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                                 ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]
    buf = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    ms, rate = ctypes.c_double(0.0), ctypes.c_double(0.0)
    rc = kernels.mcb200_probe_tma_l2_pull(ctypes.c_void_p(buf.data_ptr()), buf.numel(), 1024, 8, 2, ctypes.byref(ms),
                                          ctypes.byref(rate), None)
    assert rc == 0, rc
    # more than HBM delivers, less than anything an L2 could
    assert 5000.0 < rate.value < 80000.0, rate.value
    one_stage = ctypes.c_double(0.0)
    rc = kernels.mcb200_probe_tma_l2_pull(ctypes.c_void_p(buf.data_ptr()), buf.numel(), 1024, 1, 2, ctypes.byref(ms),
                                          ctypes.byref(one_stage), None)
    assert rc == 0 and one_stage.value < rate.value      # a deeper ring hides the round trip
