"""GPU parity of the one-shot FFT convolution (`.fft` mode) against the float32 port of the
reference's path and the float64 linear convolution; known-answer and error cases of
Tests/MetalDSPTests/ConvolutionTests.swift:94-140 and :336-385."""
import ctypes

import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp

pytestmark = pytest.mark.gpu
TOL = 1e-5


def fft_conv(device, channels=1):
    from metalaudio_b200 import Convolution
    return Convolution(device, Convolution.Mode.fft(), channels=channels)


def test_default_mode_is_fft(device):
    from metalaudio_b200 import Convolution
    assert Convolution(device).mode.kind == "fft"


def test_identity(device):
    """testFFTConvolutionIdentity: kernel [1,0,0,0] returns the input."""
    c = fft_conv(device)
    c.setKernel(np.array([1.0, 0.0, 0.0, 0.0], np.float32))
    y = c.process(np.array([1.0, 2.0, 3.0, 4.0], np.float32))
    assert y.size == c.fftSize == 8
    assert np.allclose(y[:4], [1, 2, 3, 4], atol=1e-5)


def test_impulse_response(device):
    """testFFTConvolutionImpulseResponse: an impulse returns the kernel."""
    k = np.array([1.0, 0.5, 0.25, 0.125], np.float32)
    c = fft_conv(device)
    c.setKernel(k)
    y = c.process(np.array([1.0, 0.0, 0.0, 0.0], np.float32))
    assert np.allclose(y[:4], k, atol=1e-5)


def test_input_size_mismatch_and_valid_size(device):
    """testFFTConvolutionInputSizeMismatchThrows / ValidInputSucceeds."""
    from metalaudio_b200 import ConvolutionError
    k = np.array([1.0, 0.5, 0.25, 0.125], np.float32)
    c = fft_conv(device)
    c.setKernel(k, expectedInputSize=64)
    assert c.maxInputSize == 64 and c.kernelTailLength == 3 and c.expectedOutputSize(64) == 67
    with pytest.raises(ConvolutionError) as e:
        c.process(np.ones(128, np.float32))
    assert e.value.case == "inputSizeMismatch" and e.value.inputSize == 128 and e.value.expectedMaxSize == 64
    assert "circular convolution" in e.value.errorDescription
    c.setKernel(k, expectedInputSize=128)
    assert c.process(np.ones(128, np.float32)).size == 256
    with pytest.raises(ConvolutionError) as e:
        fft_conv(device).setKernel(np.zeros(0, np.float32))
    assert e.value.case == "emptyKernel"
    with pytest.raises(ConvolutionError):
        fft_conv(device).process(np.ones(4, np.float32))      # kernel never set
    assert fft_conv(device).process(np.zeros(0, np.float32)).size == 0


@pytest.mark.parametrize("taps,expected,length", [(1, 1, 1), (4, 4, 3), (33, 100, 77), (200, 1000, 1000),
                                                  (1000, 3000, 2500), (4096, 4096, 4096), (5000, 12000, 11000),
                                                  (131072, 131072, 100000), (3, 600000, 600000)])
def test_matches_port_and_oracle(device, taps, expected, length):
    rng = np.random.default_rng(taps + length)
    h = (rng.standard_normal(taps) * np.exp(-np.arange(taps) / max(1.0, taps / 4))).astype(np.float32)
    x = rng.standard_normal(length).astype(np.float32)
    c = fft_conv(device)
    c.setKernel(h, expectedInputSize=expected)
    port = rp.FFTConvolution(h, expected)
    assert c.fftSize == max(2, port.fft_size)
    y = c.process(x)
    assert y.shape == (c.fftSize,)
    full = o64.convolve_full(x, h)
    assert o64.rel_rms(y[:full.size], full) < TOL
    yp = port.process(x)
    m = min(yp.size, y.size)
    assert o64.rel_rms(y[:m], yp[:m]) < TOL
    assert np.max(np.abs(y[full.size:]), initial=0.0) < 1e-4 * np.sqrt(np.mean(full ** 2))


def test_many_signals_device_pointers(device, lib):
    """The C ABI on device memory: strided input rows, one shared kernel, no allocation per call."""
    import torch
    from metalaudio_b200 import _lib as L
    rng = np.random.default_rng(5)
    taps, length, stride, sig = 700, 3000, 3200, 37
    h = rng.standard_normal(taps).astype(np.float32)
    x = rng.standard_normal((sig, stride)).astype(np.float32)
    fc = ctypes.c_void_p()
    assert lib.ma_fftconv_create(device.handle, h.ctypes.data_as(ctypes.c_void_p), taps, length, sig, ctypes.byref(fc)) == 0
    n = ctypes.c_int64(0)
    assert lib.ma_fftconv_fft_size(fc, ctypes.byref(n)) == 0 and n.value == 4096
    dx = torch.from_numpy(x).cuda()
    dy = torch.empty((sig, n.value), device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):   # the second call reuses every work buffer
        st = lib.ma_fftconv_process_dev(fc, ctypes.c_void_p(dx.data_ptr()), length, stride, sig, ctypes.c_void_p(dy.data_ptr()))
        assert st == 0
    device.synchronize(10)
    y = dy.cpu().numpy()
    for s in (0, 17, sig - 1):
        full = o64.convolve_full(x[s, :length], h)
        assert o64.rel_rms(y[s, :full.size], full) < TOL
    assert lib.ma_fftconv_process_dev(fc, ctypes.c_void_p(dx.data_ptr()), length + 1, stride, sig,
                                      ctypes.c_void_p(dy.data_ptr())) == L.MA_ERR_INPUT_SIZE_MISMATCH
    assert lib.ma_fftconv_process_dev(fc, ctypes.c_void_p(dx.data_ptr()), length, stride, sig + 1,
                                      ctypes.c_void_p(dy.data_ptr())) == L.MA_ERR_BATCH_OVERFLOW
    assert lib.ma_fftconv_destroy(fc) == 0
    bad = ctypes.c_void_p()
    assert lib.ma_fftconv_create(device.handle, h.ctypes.data_as(ctypes.c_void_p), 0, 10, 1, ctypes.byref(bad)) == L.MA_ERR_EMPTY_KERNEL
    assert lib.ma_fftconv_create(device.handle, h.ctypes.data_as(ctypes.c_void_p), taps, 1 << 24, 1, ctypes.byref(bad)) == L.MA_ERR_SIZE_TOO_LARGE


@pytest.mark.parametrize("length,stride", [(40000, 40192), (40192, 40192), (40000, 40000), (39999, 40004)])
def test_large_transform_loader_variants(device, lib, length, stride):
    """131072-point transforms (kernel of 30000 taps): the forward column pass stages its tile through a
    tensor map when the rows are 16-byte aligned and long enough for the row that holds the last sample
    - with a partly filled last row (40000 = 156 * 256 + 64), with none (40192 = 157 * 256) - and falls
    back to plain loads otherwise (dense rows shorter than the padded row count; a length that is not a
    multiple of four samples).  Every variant must give the same convolution."""
    import torch
    rng = np.random.default_rng(length + stride)
    taps, sig = 30000, 5
    h = (rng.standard_normal(taps) * np.exp(-np.arange(taps) / 6000.0)).astype(np.float32)
    x = rng.standard_normal((sig, stride)).astype(np.float32)
    fc = ctypes.c_void_p()
    assert lib.ma_fftconv_create(device.handle, h.ctypes.data_as(ctypes.c_void_p), taps, length, sig, ctypes.byref(fc)) == 0
    n = ctypes.c_int64(0)
    assert lib.ma_fftconv_fft_size(fc, ctypes.byref(n)) == 0 and n.value == 131072
    dx = torch.from_numpy(x).cuda()
    dy = torch.empty((sig, n.value), device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_fftconv_process_dev(fc, ctypes.c_void_p(dx.data_ptr()), length, stride, sig, ctypes.c_void_p(dy.data_ptr())) == 0
    device.synchronize(10)
    y = dy.cpu().numpy()
    for s in (0, sig - 1):
        full = o64.convolve_full(x[s, :length], h)
        assert o64.rel_rms(y[s, :full.size], full) < TOL
        assert np.max(np.abs(y[s, full.size:])) < 1e-3 * np.max(np.abs(full))  # the zero padding stayed zero
    assert lib.ma_fftconv_destroy(fc) == 0
