"""GPU parity of the magnitude / phase glue around the STFT (the split and rebuild the reference's
HTDemucs caller does on the host, Sources/MetalNN/HTDemucs.swift:726-741 and :795-812; shader forms
Sources/MetalDSP/Shaders/DSP.metal:784-881) against the float32 port and the float64 definition."""
import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp

pytestmark = pytest.mark.gpu
TOL = 1e-5


def make_fft(device, n, hop):
    from metalaudio_b200 import FFT, WindowType
    return FFT(device, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop))


@pytest.mark.parametrize("n,hop,length,signals", [(256, 64, 2048, 3), (1024, 256, 9000, 2), (4096, 1024, 40000, 2),
                                                  (64, 16, 333, 1), (8192, 2048, 30000, 1), (512, 200, 4001, 2)])
def test_stft_polar_matches_oracle(device, n, hop, length, signals):
    rng = np.random.default_rng(n + hop)
    x = (rng.random((signals, length)) * 2 - 1).astype(np.float32)
    fft = make_fft(device, n, hop)
    mag, phase = fft.stftPolar(x)
    win = rp.window("hann", n)
    ref = o64.stft(x, n, hop, win)                       # complex128 (S, F, N/2+1)
    assert mag.shape == ref.shape and phase.shape == ref.shape
    assert o64.rel_rms(mag, np.abs(ref)) < TOL
    # phases compare as unit vectors weighted by the magnitude: immune to the +-pi branch cut
    assert o64.rel_rms(mag * np.exp(1j * phase.astype(np.float64)), ref) < TOL
    # against the float32 port of the reference path + host split
    re, im = zip(*(rp.stft(x[s], n, hop, win) for s in range(signals)))
    pm, pp = rp.to_polar(np.stack(re)[..., :n // 2 + 1], np.stack(im)[..., :n // 2 + 1])
    assert o64.rel_rms(mag, pm) < TOL
    assert o64.rel_rms(mag * np.exp(1j * phase.astype(np.float64)), pm * np.exp(1j * pp.astype(np.float64))) < TOL
    # the fused result equals the complex STFT followed by the standalone split
    spec = fft.stftBatch(x)
    assert o64.rel_rms(mag, np.abs(spec)) < 1e-6


@pytest.mark.parametrize("n,hop,length,signals", [(256, 64, 2048, 3), (1024, 256, 9000, 2), (4096, 1024, 40000, 2),
                                                  (64, 16, 333, 1), (512, 200, 4001, 2)])
def test_istft_polar_round_trip_and_parity(device, n, hop, length, signals):
    rng = np.random.default_rng(7 * n + hop)
    x = (rng.random((signals, length)) * 2 - 1).astype(np.float32)
    fft = make_fft(device, n, hop)
    mag, phase = fft.stftPolar(x)
    y = fft.istftPolar(mag, phase)
    frames = mag.shape[1]
    out_len = (frames - 1) * hop + n
    assert y.shape == (signals, out_len)
    win = rp.window("hann", n)
    ws = rp.window_sum(frames, n, hop, win, 0.0)
    keep = ws > 1e-3 * ws.max()        # where the window sum is tiny, rounding noise is divided by it
    # parity with the complex route on the same device
    y_complex = fft.istftBatch(fft.stftBatch(x))
    assert o64.rel_rms(y[:, keep], y_complex[:, keep]) < TOL
    # parity with the float64 definition fed the same polar data
    spec = mag.astype(np.float64) * np.exp(1j * phase.astype(np.float64))
    spec[..., 0] = spec[..., 0].real
    spec[..., -1] = spec[..., -1].real
    ref = o64.istft(spec, n, hop, win, float(rp.window_floor()))
    assert o64.rel_rms(y[:, keep], ref[:, keep]) < TOL
    assert o64.rel_rms(y[:, keep], x[:, :out_len][:, keep]) < TOL


def test_modified_magnitude_keeps_phase(device):
    """The consumer's use: scale magnitudes (a mask), rebuild with the original phase."""
    rng = np.random.default_rng(11)
    n, hop = 1024, 256
    x = (rng.random((2, 16384)) * 2 - 1).astype(np.float32)
    fft = make_fft(device, n, hop)
    mag, phase = fft.stftPolar(x)
    y = fft.istftPolar(0.5 * mag, phase)
    y_full = fft.istftPolar(mag, phase)
    assert o64.rel_rms(y, 0.5 * y_full) < 1e-6


def test_batched_forward_inverse_polar(device, lib):
    """The plain batched transforms accept the polar layout too (C ABI, host form)."""
    from metalaudio_b200 import _lib as L
    from metalaudio_b200 import FFT, WindowType
    rng = np.random.default_rng(3)
    n, batch = 2048, 5
    x = rng.standard_normal((batch, n)).astype(np.float32)
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.none))
    mag = np.empty((batch, n // 2 + 1), np.float32)
    ph = np.empty_like(mag)
    p = lambda a: a.ctypes.data
    assert lib.ma_fft_forward_host(fft._h, p(x), p(mag), p(ph), None, 0, 1.0, batch, L.LAYOUT_HALF_POLAR) == 0
    ref = np.fft.rfft(x.astype(np.float64), axis=-1)
    assert o64.rel_rms(mag * np.exp(1j * ph.astype(np.float64)), ref) < TOL
    y = np.empty_like(x)
    assert lib.ma_fft_inverse_host(fft._h, p(mag), p(ph), p(y), batch, L.LAYOUT_HALF_POLAR) == 0
    assert o64.rel_rms(y, x) < TOL
    assert lib.ma_fft_forward_host(fft._h, p(x), p(mag), None, None, 0, 1.0, batch, L.LAYOUT_HALF_POLAR) == L.MA_ERR_INVALID_ARGUMENT
    big = FFT(device, FFT.Config(size=16384, windowType=WindowType.none))
    xb = np.zeros((1, 16384), np.float32)
    mb = np.zeros((1, 8193), np.float32)
    assert lib.ma_fft_forward_host(big._h, p(xb), p(mb), p(mb.copy()), None, 0, 1.0, 1, L.LAYOUT_HALF_POLAR) == L.MA_ERR_UNSUPPORTED


def test_standalone_glue_kernels(device):
    """compute_magnitude/compute_phase, polar_to_complex and to_decibels on device arrays."""
    from metalaudio_b200 import Tensor, polarToSpectrum, spectrumToPolar, toDecibels
    rng = np.random.default_rng(5)
    count = 100003
    z = (rng.standard_normal(count) + 1j * rng.standard_normal(count)).astype(np.complex64)
    z[:4] = [0, 1, -1, 1j]
    spec = Tensor(device, (count, 2)); spec.copy(z.view(np.float32))
    mag = Tensor(device, (count,)); ph = Tensor(device, (count,)); back = Tensor(device, (count, 2))
    spectrumToPolar(device, spec, mag, ph)
    polarToSpectrum(device, mag, ph, back)
    m, p_ = mag.toArray(), ph.toArray()
    pm, pp = rp.to_polar(z.real, z.imag)
    assert np.max(np.abs(m - pm)) <= 1e-6 * np.max(pm)
    assert m[0] == 0 and p_[0] == 0 and abs(p_[2] - np.pi) < 1e-6 and abs(p_[3] - np.pi / 2) < 1e-6
    d = np.abs(np.angle(np.exp(1j * (p_.astype(np.float64) - pp))))
    assert np.max(d) < 1e-6
    zb = back.toArray().reshape(count, 2)
    re, im = rp.from_polar(pm, pp)
    assert o64.rel_rms(zb[:, 0] + 1j * zb[:, 1], re + 1j * im) < 1e-6
    assert o64.rel_rms(zb[:, 0] + 1j * zb[:, 1], z) < 1e-6
    # decibels: clamp, floor and the reference <= 0 fallback
    vals = np.concatenate([np.array([0.0, 1e-12, 1.0, 10.0, 2.0], np.float32), rng.random(1000).astype(np.float32)])
    t = Tensor(device, (vals.size,)); t.copy(vals)
    toDecibels(device, t, reference=2.0, minDB=-80.0)
    got = t.toArray()
    want = rp.to_decibels(vals, 2.0, -80.0)
    assert np.max(np.abs(got - want)) < 1e-4
    assert got[0] == -80.0 and abs(got[4]) < 1e-6
    t.copy(vals)
    toDecibels(device, t, reference=0.0, minDB=-60.0)
    assert np.all(t.toArray() == -60.0)


def test_istft_polar_unaligned_arrays_take_the_plain_path(device, lib):
    """Magnitude / phase arrays that do not start on a 16-byte boundary cannot be staged with bulk
    copies; the result must not depend on which kernel served the call."""
    import ctypes
    import torch
    from metalaudio_b200 import _lib as L
    rng = np.random.default_rng(21)
    n, hop, sig = 4096, 1024, 3
    x = (rng.random((sig, 40000)) * 2 - 1).astype(np.float32)
    fft = make_fft(device, n, hop)
    mag, phase = fft.stftPolar(x)
    frames, kh = mag.shape[1], mag.shape[2]
    out_len = (frames - 1) * hop + n
    count = sig * frames * kh
    outs = []
    for off in (0, 1, 2, 3):        # element offsets: 0 is aligned, the others are not
        dm = torch.zeros(count + 4, device="cuda"); dp = torch.zeros(count + 4, device="cuda")
        dm[off:off + count] = torch.from_numpy(mag.ravel()).cuda()
        dp[off:off + count] = torch.from_numpy(phase.ravel()).cuda()
        dy = torch.empty((sig, out_len), device="cuda")
        torch.cuda.synchronize()
        st = lib.ma_istft_dev(fft._h, ctypes.c_void_p(dm.data_ptr() + 4 * off), ctypes.c_void_p(dp.data_ptr() + 4 * off),
                              frames, sig, ctypes.c_void_p(dy.data_ptr()), out_len, 1e-8, L.LAYOUT_HALF_POLAR)
        assert st == 0
        device.synchronize(10)
        outs.append(dy.cpu().numpy())
    win = rp.window("hann", n)
    ws = rp.window_sum(frames, n, hop, win, 0.0)
    keep = ws > 1e-3 * ws.max()
    for y in outs[1:]:
        assert o64.rel_rms(y[:, keep], outs[0][:, keep]) < 1e-6
    assert o64.rel_rms(outs[0][:, keep], x[:, :out_len][:, keep]) < TOL
