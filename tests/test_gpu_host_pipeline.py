"""The pipelined host forms (ma_stft_host, ma_istft_host, ma_pconv_process_host) on PINNED host arrays:
chunks travel on three streams through two workspace lanes.  A small workspace forces several chunks,
so every lane is reused; results must equal the pageable path's bit for bit (same kernels, same
chunk-independent arithmetic) and agree with the float64 oracle."""
import ctypes

import numpy as np
import pytest

from oracle import float64 as o64

pytestmark = pytest.mark.gpu
TOL = 1e-5


class Pinned:
    """float32 numpy views of page-locked host memory from ma_host_alloc."""

    def __init__(self, lib, dev):
        self.lib, self.dev, self.ptrs = lib, dev, []

    def array(self, shape):
        n = int(np.prod(shape))
        p = ctypes.c_void_p()
        assert self.lib.ma_host_alloc(self.dev.handle, 4 * max(n, 1), ctypes.byref(p)) == 0
        self.ptrs.append(p)
        a = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_float)), shape=(max(n, 1),))[:n]
        return a.reshape(shape)

    def close(self):
        for p in self.ptrs:
            assert self.lib.ma_host_free(self.dev.handle, p) == 0
        self.ptrs = []


def ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.fixture()
def small_device(lib):
    """A context of its own whose workspace lanes hold only a few rows."""
    from metalaudio_b200 import AudioDevice
    dev = AudioDevice()
    yield dev
    dev.close()


def test_convolution_host_pinned_groups(lib, small_device):
    """12 channels with per-pair impulse responses (groups of two stay together), strided host rows,
    workspace of 2 x 200 KB: three chunks of two groups.  Two consecutive calls."""
    from metalaudio_b200 import Convolution
    dev = small_device
    assert lib.ma_context_reserve_workspace(dev.handle, 400 << 10) == 0
    block, taps, length, channels = 64, 300, 5000, 12
    full = length + taps - 1
    rng = np.random.default_rng(12)
    irs = (rng.standard_normal((channels // 2, taps)) * np.exp(-np.arange(taps) / 80.0)).astype(np.float32)
    cmap = [c // 2 for c in range(channels)]
    pin = Pinned(lib, dev)
    try:
        in_stride, out_stride = length + 24, full + 40
        x = pin.array((channels, in_stride))
        y = pin.array((channels, out_stride))
        for call in range(2):
            x[:] = rng.standard_normal(x.shape).astype(np.float32)
            y[:] = -7.0
            c_pin = Convolution(dev, Convolution.Mode.partitioned(blockSize=block), channels=channels)
            c_pin.setKernel(irs, channelToKernel=cmap)
            c_page = Convolution(dev, Convolution.Mode.partitioned(blockSize=block), channels=channels)
            c_page.setKernel(irs, channelToKernel=cmap)
            for _ in range(call + 1):  # the second round checks a call that follows another on the same object
                assert lib.ma_pconv_process_host(c_pin._h, ptr(x), length, in_stride, ptr(y), out_stride) == 0
                ref_page = c_page.process(np.ascontiguousarray(x[:, :length]))
            assert np.array_equal(y[:, :full], ref_page)
            assert np.all(y[:, full:] == -7.0)  # nothing written beyond a row's L+K-1 samples
            for c in (0, 5, 11):
                assert o64.rel_rms(y[c, :full], o64.convolve_full(x[c, :length], irs[cmap[c]])) <= TOL
    finally:
        pin.close()


def test_stft_istft_host_pinned_chunks(lib, small_device):
    """9 signals of 30000 samples, N = 1024, hop 256, workspace of 2 x 1.5 MB: the signals go through in
    chunks of two.  Spectra, magnitudes and the reconstruction equal the pageable path's."""
    from metalaudio_b200 import FFT, WindowType
    from metalaudio_b200 import _lib as L
    dev = small_device
    assert lib.ma_context_reserve_workspace(dev.handle, 3 << 20) == 0
    n, hop, signals, length = 1024, 256, 9, 30000
    f = FFT(dev, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop))
    frames = f.frameCount(length)
    kh = n // 2 + 1
    out_len = (frames - 1) * hop + n
    rng = np.random.default_rng(9)
    pin = Pinned(lib, dev)
    try:
        x = pin.array((signals, length))
        spec = pin.array((signals, frames, kh, 2))
        mag = pin.array((signals, frames, kh))
        y = pin.array((signals, out_len))
        x[:] = rng.standard_normal(x.shape).astype(np.float32)
        assert lib.ma_stft_host(f._h, ptr(x), length, length, signals, ptr(spec), None, ptr(mag), L.MAG_MAGNITUDE, 1.0,
                                L.LAYOUT_HALF_INTERLEAVED) == 0
        spec_page, mag_page = f.stftBatch(np.array(x), magnitude=True)
        assert np.array_equal(spec.view(np.complex64).reshape(signals, frames, kh), spec_page)
        assert np.array_equal(mag, mag_page)
        from metalaudio_b200.dsp import validatedWindowFloor
        assert lib.ma_istft_host(f._h, ptr(spec), None, frames, signals, ptr(y), out_len, validatedWindowFloor(),
                                 L.LAYOUT_HALF_INTERLEAVED) == 0
        assert np.array_equal(y, f.istftBatch(spec_page))
        inner = slice(n, length - n)
        assert o64.rel_rms(y[:, inner], x[:, inner]) <= TOL
    finally:
        pin.close()


@pytest.mark.parametrize("n,batch", [(4096, 700), (65536, 40)])
def test_plain_transforms_host_pinned_chunks(lib, small_device, n, batch):
    """Batches above the pipeline threshold between pinned arrays, workspace of 2 x 4 MB: forward (with
    magnitudes) and inverse run in several chunks and equal the pageable path's results."""
    from metalaudio_b200 import FFT, WindowType
    from metalaudio_b200 import _lib as L
    dev = small_device
    assert lib.ma_context_reserve_workspace(dev.handle, 8 << 20) == 0
    f = FFT(dev, FFT.Config(size=n, windowType=WindowType.none))
    kh = n // 2 + 1
    rng = np.random.default_rng(n + batch)
    pin = Pinned(lib, dev)
    try:
        x = pin.array((batch, n))
        spec = pin.array((batch, kh, 2))
        mag = pin.array((batch, kh))
        y = pin.array((batch, n))
        x[:] = rng.standard_normal(x.shape).astype(np.float32)
        assert lib.ma_fft_forward_host(f._h, ptr(x), ptr(spec), None, ptr(mag), L.MAG_MAGNITUDE, 1.0, batch,
                                       L.LAYOUT_HALF_INTERLEAVED) == 0
        xs = np.array(x)
        spec_page = np.zeros((batch, kh, 2), np.float32)
        mag_page = np.zeros((batch, kh), np.float32)
        assert lib.ma_fft_forward_host(f._h, ptr(xs), ptr(spec_page), None, ptr(mag_page), L.MAG_MAGNITUDE, 1.0, batch,
                                       L.LAYOUT_HALF_INTERLEAVED) == 0
        assert np.array_equal(spec, spec_page) and np.array_equal(mag, mag_page)
        pick = [0, batch // 2, batch - 1]
        assert o64.rel_rms(spec[pick, :, 0] + 1j * spec[pick, :, 1], o64.rfft(xs[pick])) <= TOL
        assert lib.ma_fft_inverse_host(f._h, ptr(spec), None, ptr(y), batch, L.LAYOUT_HALF_INTERLEAVED) == 0
        y_page = np.zeros((batch, n), np.float32)
        assert lib.ma_fft_inverse_host(f._h, ptr(spec_page), None, ptr(y_page), batch, L.LAYOUT_HALF_INTERLEAVED) == 0
        assert np.array_equal(y, y_page)
        assert o64.rel_rms(y, xs) <= TOL
    finally:
        pin.close()
