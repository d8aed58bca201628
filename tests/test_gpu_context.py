"""Context, Tensor, timing and failure-handling slices of AudioDevice / ComputeContext / Tensor.
Failures are injected on the host only (a test hook makes the next call reaching a site return a
chosen error); no GPU work is disturbed and nothing is faulted or hung."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_name_and_tensor_round_trip(device):
    from metalaudio_b200 import Tensor
    assert "NVIDIA" in device.name or len(device.name) > 0
    t = Tensor(device, (3, 1000))
    x = np.random.default_rng(0).standard_normal((3, 1000)).astype(np.float32)
    t.copy(x)
    assert np.array_equal(t.toArray(), x)
    t.zero()
    device.synchronize()
    assert not t.toArray().any()
    v = t.rows(1, 2)
    v.copy(x[1:3])
    assert np.array_equal(t.toArray()[1:], x[1:])
    with pytest.raises(Exception):
        t.copy(np.zeros(7, np.float32))
    t.free()


def test_timing_brackets_queued_work(device):
    from metalaudio_b200 import FFT, WindowType
    fft = FFT(device, FFT.Config(size=1024, windowType=WindowType.none))
    x = np.random.default_rng(1).standard_normal((64, 1024)).astype(np.float32)
    device.timingBegin()
    fft.forwardBatch(x)
    ms = device.timingEnd()
    assert 0.0 <= ms < 5000.0
    fft.close()


def test_injected_faults_surface_as_reference_errors(lib):
    """ma_test_inject_fault: allocation, launch and synchronisation failures map onto
    bufferAllocationFailed / gpuExecutionError; the context stays usable afterwards."""
    from metalaudio_b200 import AudioDevice, FFT, MetalAudioError, Tensor, WindowType
    from metalaudio_b200 import _lib as L
    dev = AudioDevice()
    lib.ma_test_inject_fault(dev.handle, L.FAULT_ALLOC, 2)  # cudaErrorMemoryAllocation
    with pytest.raises(MetalAudioError) as e:
        Tensor(dev, (10,))
    assert e.value.case == "bufferAllocationFailed"
    t = Tensor(dev, (10,))  # next call works again
    fft = FFT(dev, FFT.Config(size=256, windowType=WindowType.none))
    lib.ma_test_inject_fault(dev.handle, L.FAULT_LAUNCH, 719)  # cudaErrorLaunchFailure, injected on the host
    with pytest.raises(MetalAudioError) as e:
        fft.forwardBatch(np.ones((2, 256), np.float32))
    assert e.value.case == "gpuExecutionError" and lib.ma_last_cuda_error() == 719
    re, im = fft.forwardBatch(np.ones((2, 256), np.float32))
    assert abs(re[0, 0] - 256) < 1e-3
    lib.ma_test_inject_fault(dev.handle, L.FAULT_SYNC, 719)
    with pytest.raises(MetalAudioError):
        dev.synchronize()
    dev.synchronize()
    # non-throwing pointer API zeroes its outputs on failure (FFT.swift:826-835)
    lib.ma_test_inject_fault(dev.handle, L.FAULT_LAUNCH, 719)
    r = np.ones(256, np.float32); i = np.ones(256, np.float32)
    fft.forward(np.ones(256, np.float32), r, i)
    assert not r.any() and not i.any()
    fft.close(); t.free(); dev.close()


def test_device_loss_is_an_error_not_a_reroute(lib):
    """DeviceLossTests: markDeviceLost flips availability and every later call reports
    deviceLost; there is no CPU fallback to reroute to."""
    from metalaudio_b200 import AudioDevice, FFT, MetalAudioError, WindowType
    dev = AudioDevice()
    fft = FFT(dev, FFT.Config(size=256, windowType=WindowType.none))
    assert dev.isDeviceAvailable
    dev.markDeviceLost()
    assert not dev.isDeviceAvailable
    with pytest.raises(MetalAudioError) as e:
        dev.ensureAvailable()
    assert e.value.case == "deviceLost"
    with pytest.raises(MetalAudioError) as e:
        fft.forwardBatch(np.ones((1, 256), np.float32))
    assert e.value.case == "deviceLost"
    with pytest.raises(MetalAudioError):
        FFT(dev, FFT.Config(size=512))
    dev._lib.ma_context_destroy(dev.handle)
    dev._h = None


def test_two_contexts_are_independent_streams(lib):
    """RealtimeThreadSafetyTests shape: separate objects per thread/stream do not mix results."""
    import threading
    from metalaudio_b200 import AudioDevice, FFT, WindowType
    from oracle import float64 as o64
    results = {}

    def work(seed):
        dev = AudioDevice(pinnedBytes=1 << 20)
        fft = FFT(dev, FFT.Config(size=2048, windowType=WindowType.none))
        x = np.random.default_rng(seed).standard_normal((50, 2048)).astype(np.float32)
        for _ in range(5):
            re, im = fft.forwardBatch(x)
        results[seed] = o64.rel_rms(re + 1j * im, o64.fft_forward(x))
        fft.close(); dev.close()

    th = [threading.Thread(target=work, args=(s,)) for s in (1, 2, 3, 4)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert all(v <= 1e-5 for v in results.values()) and len(results) == 4


def test_host_deadline_runs_out_behind_queued_work_and_the_context_recovers(device, lib):
    """ComputeContext.executeSync's timeout (ComputeContext.swift:137, :176-208): a deadline far
    shorter than the queued work gives gpuTimeout and leaves the stream draining; a normal wait
    afterwards succeeds and the results are the ones a run without the timeout gives."""
    from metalaudio_b200 import FFT, MetalAudioError, Tensor, WindowType
    from metalaudio_b200 import _lib as L
    from oracle import float64 as o64
    n, hop, S, length = 4096, 1024, 32, 1 << 19
    w = np.hanning(n + 1)[:n].astype(np.float32)
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop), window=w)
    frames = (length - n) // hop + 1
    x = np.random.default_rng(3).uniform(-1, 1, (S, length)).astype(np.float32)
    sig = Tensor(device, (S, length)); sig.copy(x)
    spec = Tensor(device, (S, frames, n // 2 + 1, 2))
    device.synchronize()
    for _ in range(60):                                  # tens of milliseconds of queued kernels
        fft.stftTensor(sig, spec, None)
    st = lib.ma_context_sync(device.handle, 1e-4)
    assert st == L.MA_ERR_TIMEOUT
    with pytest.raises(MetalAudioError) as e:
        from metalaudio_b200.dsp import _raise_status
        _raise_status(st, "synchronize")
    assert e.value.case == "gpuTimeout"
    device.synchronize(30)                               # the work itself was never disturbed
    got = spec.toArray()[:2]
    assert o64.rel_rms(got[..., 0] + 1j * got[..., 1], o64.stft(x[:2], n, hop, w)) <= 1e-5
    fft.close(); sig.free(); spec.free()


def test_device_side_bounded_wait_gives_up_and_reports_timeout(lib):
    """A kernel-side wait that nothing satisfies runs into its poll limit, raises the context's
    error flag and returns; the next synchronisation reports gpuTimeout once, the one after is
    clean and the context still computes.  The wait is bounded by construction (a few thousand
    polls of a barrier in one thread): nothing hangs."""
    from metalaudio_b200 import AudioDevice, FFT, WindowType
    from metalaudio_b200 import _lib as L
    dev = AudioDevice(pinnedBytes=1 << 20)
    assert lib.ma_test_bounded_wait(dev.handle, 0) == L.MA_ERR_INVALID_ARGUMENT
    assert lib.ma_test_bounded_wait(dev.handle, 2000) == 0
    assert lib.ma_context_sync(dev.handle, 10.0) == L.MA_ERR_TIMEOUT
    assert lib.ma_context_sync(dev.handle, 10.0) == 0
    fft = FFT(dev, FFT.Config(size=256, windowType=WindowType.none))
    re, im = fft.forwardBatch(np.ones((2, 256), np.float32))
    assert abs(re[0, 0] - 256) < 1e-3
    fft.close(); dev.close()
