"""GPU parity of STFT / iSTFT against the float64 oracle and the float32 port."""
import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp
from oracle import configs

pytestmark = pytest.mark.gpu
TOL = 1e-5


def interior(frames, n, hop, win, frac=1e-2):
    """Samples whose window sum is not vanishing: near the ends a symmetric window leaves
    sum(w^2) ~ 1e-8, where float32 rounding is amplified by 1/sum(w^2) in any implementation."""
    ws = rp.window_sum(frames, n, hop, win, 0.0)
    return ws >= frac * ws.max()


CASES = [(256, 64, 4000, "hann"), (512, 100, 5000, "hamming"), (64, 7, 700, "blackman"),
         (1024, 1024, 8192, "none"), (2048, 512, 40000, "hann"), (4096, 1024, 70000, "hann"),
         (8192, 2048, 70000, "hann"), (8, 2, 50, "hann"), (4, 1, 21, "hann"), (2, 1, 9, "none"),
         (256, 255, 3001, "hann"),
         # above 8192 points: the two-pass transforms with the window in the loader and a separate overlap-add
         (16384, 4096, 100000, "hann"), (32768, 8192, 140000, "hamming"), (65536, 65536, 200000, "none"),
         (16384, 1000, 60001, "blackman")]


@pytest.mark.parametrize("n,hop,length,kind", CASES)
def test_stft_istft_parity(device, n, hop, length, kind):
    from metalaudio_b200 import FFT, WindowType
    rng = np.random.default_rng(n * 7 + hop)
    x = rng.uniform(-1, 1, length).astype(np.float32)
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType(kind), hopSize=hop))
    res = fft.stft(x)
    w = rp.window(kind, n)
    frames = (length - n) // hop + 1
    assert res.frameCount == frames and res.binCount == n
    ref = o64.stft(x, n, hop, w)
    full_ref = o64.fft_forward(x[np.arange(frames)[:, None] * hop + np.arange(n)[None, :]].astype(np.float64) * w)
    assert o64.rel_rms(res.real + 1j * res.imag, full_ref) <= TOL
    pre, pim = rp.stft(x, n, hop, w)
    assert o64.rel_rms(res.real + 1j * res.imag, pre + 1j * pim) <= TOL
    y = fft.istft(res)
    assert y.shape == ((frames - 1) * hop + n,)
    floor = float(rp.window_floor())
    yref = o64.istft(ref, n, hop, w, floor)
    m = interior(frames, n, hop, w)
    assert o64.rel_rms(y[m], yref[m]) <= TOL
    yport = rp.istft(pre, pim, n, hop, w)
    assert o64.rel_rms(y[m], yport[m]) <= TOL
    # the ends are bounded by the amplification 1/sum(w^2) of float32 rounding
    assert np.isfinite(y).all()
    ws = np.maximum(rp.window_sum(frames, n, hop, w, floor), floor)
    assert np.all(np.abs(y - yref) <= 1e-5 * np.sqrt(n) / np.sqrt(ws) + 1e-5)


def test_stft_input_too_short(device):
    from metalaudio_b200 import FFT, FFTError
    fft = FFT(device, FFT.Config(size=256))
    with pytest.raises(FFTError) as e:
        fft.stft(np.zeros(100, np.float32))
    assert e.value.case == "inputTooShort" and e.value.inputSize == 100 and e.value.requiredSize == 256


def test_istft_empty(device):
    from metalaudio_b200 import FFT, STFTResult
    fft = FFT(device, FFT.Config(size=256))
    assert fft.istft(STFTResult(np.zeros((0, 256), np.float32), np.zeros((0, 256), np.float32))).size == 0


def test_config2_scaled_periodic_and_symmetric(device):
    """Benchmark configuration 2 at reduced signal count/length, with both window readings
    (periodic Hann as the configuration words it, symmetric as the reference computes it):
    half-spectrum complex + magnitude out, overlap-add reconstruction."""
    from metalaudio_b200 import FFT, WindowType
    n, hop = 4096, 1024
    x = configs.c2_signals(n_signals=6, length=1 << 16)
    for w in (rp.periodic_hann(n), rp.window("hann", n)):
        fft = FFT(device, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop), window=w)
        spec, mag = fft.stftBatch(x, magnitude=True)
        ref = o64.stft(x, n, hop, w)
        assert o64.rel_rms(spec, ref) <= TOL
        assert o64.rel_rms(mag, np.abs(ref)) <= TOL
        y = fft.istftBatch(spec)
        frames = spec.shape[1]
        m = interior(frames, n, hop, w)
        yref = o64.istft(ref, n, hop, w, float(rp.window_floor()))
        assert o64.rel_rms(y[:, m], yref[:, m]) <= TOL
        # COLA reconstruction of the input itself on the interior
        assert o64.rel_rms(y[:, m], x[:, :y.shape[1]][:, m]) <= TOL


def test_stft_bit_stable(device):
    from metalaudio_b200 import FFT
    fft = FFT(device, FFT.Config(size=512, hopSize=128))
    x = np.random.default_rng(1).uniform(-1, 1, 9000).astype(np.float32)
    a = fft.istft(fft.stft(x))
    b = fft.istft(fft.stft(x))
    assert np.array_equal(a, b)


def test_large_frames_many_signals_half_layout(device):
    """More frames than one scratch chunk holds (16384-point frames: 3027 per chunk) over two signals,
    half-spectrum layout with magnitudes, through the batched API."""
    from metalaudio_b200 import FFT, WindowType
    n, hop, length = 16384, 2048, 2048 * 3100 + 16384
    rng = np.random.default_rng(12)
    x = rng.uniform(-1, 1, (2, length)).astype(np.float32)
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop))
    spec, mag = fft.stftBatch(x, magnitude=True)
    frames = (length - n) // hop + 1
    assert spec.shape == (2, frames, n // 2 + 1) and frames > 3027
    w = rp.window("hann", n)
    pick = [0, 1, 3026, 3027, 3028, frames - 1]
    for s_ in range(2):
        fr = x[s_][np.array(pick)[:, None] * hop + np.arange(n)[None, :]].astype(np.float64) * w
        ref = np.fft.rfft(fr, axis=-1)
        assert o64.rel_rms(spec[s_, pick], ref) <= TOL
        assert o64.rel_rms(mag[s_, pick], np.abs(ref)) <= TOL
    y = fft.istftBatch(spec)
    m = interior(frames, n, hop, w)
    assert o64.rel_rms(y[:, m], x[:, :y.shape[1]][:, m]) <= TOL
