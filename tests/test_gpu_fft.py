"""GPU parity of the FFT entry points against the float64 oracle and the float32 port,
through the C ABI (via the host mirror).  Tolerance: relative RMS <= 1e-5 (the benchmark's
stated bound); the reference's own per-size bounds are asserted where it has them."""
import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp
from oracle import configs

pytestmark = pytest.mark.gpu
TOL = 1e-5
SIZES = [2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]


def make_fft(device, n, **kw):
    from metalaudio_b200 import FFT, WindowType
    kw.setdefault("windowType", WindowType.none)
    return FFT(device, FFT.Config(size=n, **kw))


@pytest.mark.parametrize("n", SIZES)
def test_forward_matches_oracle(device, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    fft = make_fft(device, n)
    re = np.zeros(n, np.float32)
    im = np.zeros(n, np.float32)
    fft.forward(x, re, im)
    ref = o64.fft_forward(x)
    assert o64.rel_rms(re + 1j * im, ref) <= TOL
    pre, pim = rp.fft_forward(x)
    assert o64.rel_rms(re + 1j * im, pre + 1j * pim) <= TOL
    # reference cross-implementation bound: 2.5e-5*sqrt(N/256) max abs error on unit-scale input
    assert np.max(np.abs((re + 1j * im) - ref)) < 2.5e-5 * max(1.0, np.sqrt(n / 256)) * np.sqrt(n)


@pytest.mark.parametrize("n", SIZES)
def test_round_trip_two_objects(device, n):
    """FFTTests round trip: forward object + inverse object reproduce the input."""
    rng = np.random.default_rng(100 + n)
    x = rng.standard_normal(n).astype(np.float32)
    f = make_fft(device, n)
    i = make_fft(device, n, inverse=True)
    re = np.zeros(n, np.float32)
    im = np.zeros(n, np.float32)
    y = np.zeros(n, np.float32)
    f.forward(x, re, im)
    i.inverse(re, im, y)
    assert o64.rel_rms(y, x) <= TOL
    assert np.max(np.abs(y - x)) < 1e-5  # reference regression ceiling


def test_config1_single_2048(device):
    """Benchmark configuration 1: one 2048-point frame of N(0,1), window off."""
    x = configs.c1_frame()
    n = 2048
    f = make_fft(device, n)
    i = make_fft(device, n, inverse=True)
    re = np.zeros(n, np.float32)
    im = np.zeros(n, np.float32)
    mag = np.zeros(n // 2 + 1, np.float32)
    y = np.zeros(n, np.float32)
    f.forward(x, re, im)
    f.magnitude(re, im, mag)
    i.inverse(re, im, y)
    ref = o64.fft_forward(x)
    assert o64.rel_rms(re + 1j * im, ref) <= TOL
    assert o64.rel_rms(mag, np.abs(ref[: n // 2 + 1])) <= TOL
    assert o64.rel_rms(y, x) <= TOL


def test_known_answers(device):
    """Impulse -> flat spectrum, DC -> N at bin 0, silence -> zeros, bin-k sine peaks at k,
    conjugate symmetry with Im X[0] = Im X[N/2] = 0 (FFTTests known-answer rows)."""
    n = 1024
    f = make_fft(device, n)
    re = np.zeros(n, np.float32)
    im = np.zeros(n, np.float32)
    x = np.zeros(n, np.float32); x[0] = 1
    f.forward(x, re, im)
    assert np.allclose(re, 1, atol=1e-6) and np.allclose(im, 0, atol=1e-6)
    f.forward(np.ones(n, np.float32), re, im)
    assert abs(re[0] - n) < 1e-3 and np.max(np.abs(re[1:])) < 1e-3 and np.max(np.abs(im)) < 1e-3
    f.forward(np.zeros(n, np.float32), re, im)
    assert not re.any() and not im.any()
    k = 37
    x = np.sin(2 * np.pi * k * np.arange(n) / n).astype(np.float32)
    f.forward(x, re, im)
    mag = np.zeros(n // 2 + 1, np.float32)
    f.magnitude(re, im, mag)
    assert int(np.argmax(mag)) == k and abs(mag[k] - n / 2) < 1e-2
    rng = np.random.default_rng(5)
    f.forward(rng.standard_normal(n).astype(np.float32), re, im)
    assert abs(im[0]) < 1e-5 and abs(im[n // 2]) < 1e-5
    assert np.allclose(re[1:n // 2], re[n - 1:n // 2:-1], atol=1e-5)
    assert np.allclose(im[1:n // 2], -im[n - 1:n // 2:-1], atol=1e-5)
    # Parseval within 1 %
    x = rng.standard_normal(n).astype(np.float32)
    f.forward(x, re, im)
    assert abs(np.sum(re.astype(np.float64) ** 2 + im.astype(np.float64) ** 2) / n - np.sum(x.astype(np.float64) ** 2)) \
        < 0.01 * np.sum(x.astype(np.float64) ** 2)


def test_magnitude_power_db(device):
    n = 512
    f = make_fft(device, n)
    rng = np.random.default_rng(9)
    re = rng.standard_normal(n).astype(np.float32)
    im = rng.standard_normal(n).astype(np.float32)
    kh = n // 2 + 1
    mag = np.zeros(kh, np.float32); pw = np.zeros(kh, np.float32); db = np.zeros(kh, np.float32)
    f.magnitude(re, im, mag); f.power(re, im, pw); f.magnitudeDB(re, im, db, reference=2.0)
    assert o64.rel_rms(mag, rp.magnitude(re, im)) <= TOL
    assert o64.rel_rms(pw, rp.power(re, im)) <= TOL
    assert np.max(np.abs(db - rp.magnitude_db(re, im, 2.0))) < 1e-3
    assert np.allclose(pw, mag * mag, rtol=1e-5)


@pytest.mark.parametrize("n,batch", [(64, 37), (256, 200), (1024, 33), (4096, 19), (8192, 5)])
def test_forward_inverse_batch(device, n, batch):
    rng = np.random.default_rng(n + batch)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    f = make_fft(device, n)
    re, im = f.forwardBatch(x)
    assert o64.rel_rms(re + 1j * im, o64.fft_forward(x)) <= TOL
    y = f.inverseBatch(re, im)
    assert o64.rel_rms(y, x) <= TOL
    r0, i0 = f.forwardBatch(np.zeros((0, n), np.float32))
    assert r0.shape == (0, n)


def test_reference_golden_vectors(device):
    """The 256-point vectors emitted by the reference's scripts/generate_references.py."""
    import json, os
    g = os.path.join(os.path.dirname(__file__), "golden")
    fwd = json.load(open(os.path.join(g, "fft_forward_256.json")))
    x = np.array(fwd["input"], np.float32)
    exp = np.array(fwd["expectedOutput"], np.float64)
    f = make_fft(device, 256)
    re = np.zeros(256, np.float32); im = np.zeros(256, np.float32)
    f.forward(x, re, im)
    assert np.max(np.abs(np.concatenate([re, im]) - exp)) < fwd["tolerance"] * 256 ** 0.5 * 4
    assert o64.rel_rms(np.concatenate([re, im]), exp) <= TOL
    rt = json.load(open(os.path.join(g, "fft_roundtrip_256.json")))
    i = make_fft(device, 256, inverse=True)
    y = np.zeros(256, np.float32)
    i.inverse(re, im, y)
    assert np.max(np.abs(y - np.array(rt["expectedOutput"]))) < rt["tolerance"]


def test_inverse_of_forward_object_is_time_reversed(device):
    """Reference semantics: direction comes from Config.inverse, not from the method."""
    n = 128
    f = make_fft(device, n)
    rng = np.random.default_rng(3)
    x = rng.standard_normal(n).astype(np.float32)
    re = np.zeros(n, np.float32); im = np.zeros(n, np.float32); y = np.zeros(n, np.float32)
    f.forward(x, re, im)
    f.inverse(re, im, y)
    assert o64.rel_rms(y, np.concatenate([x[:1], x[1:][::-1]])) <= TOL


def test_nan_inf_propagate_and_extremes_finite(device):
    n = 256
    f = make_fft(device, n)
    re = np.zeros(n, np.float32); im = np.zeros(n, np.float32)
    x = np.ones(n, np.float32); x[3] = np.nan
    f.forward(x, re, im)
    assert np.isnan(re).any()
    f.forward(np.full(n, 1e-30, np.float32), re, im)
    assert np.isfinite(re).all() and np.isfinite(im).all()
    f.forward(np.full(n, 1e6, np.float32), re, im)
    assert np.isfinite(re).all() and np.isfinite(im).all()


@pytest.mark.parametrize("n,batch", [(16384, 5), (32768, 3), (65536, 7), (131072, 2), (1 << 18, 1), (1 << 19, 1),
                                     (1 << 20, 2), (1 << 21, 1), (1 << 22, 1), (1 << 23, 1), (1 << 24, 1)])
def test_large_transforms(device, lib, n, batch):
    """Multi-pass path above 8192 points (the reference's MPSGraph size class), all layouts."""
    import ctypes
    from metalaudio_b200 import _lib as L
    rng = np.random.default_rng(n % 1000 + batch)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    f = make_fft(device, n)
    ref = o64.rfft(x)
    half = n // 2

    def p(a):
        return a.ctypes.data_as(ctypes.c_void_p)
    # half-interleaved + magnitude
    spec = np.zeros((batch, half + 1, 2), np.float32)
    mag = np.zeros((batch, half + 1), np.float32)
    assert lib.ma_fft_forward_host(f._h, p(x), p(spec), None, p(mag), L.MAG_MAGNITUDE, 1.0, batch,
                                   L.LAYOUT_HALF_INTERLEAVED) == 0
    assert o64.rel_rms(spec[..., 0] + 1j * spec[..., 1], ref) <= TOL
    assert o64.rel_rms(mag, np.abs(ref)) <= TOL
    y = np.zeros((batch, n), np.float32)
    assert lib.ma_fft_inverse_host(f._h, p(spec), None, p(y), batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    assert o64.rel_rms(y, x) <= TOL
    if n <= (1 << 20):
        # the reference's full-N split layout, through the mirrored API
        re, im = f.forwardBatch(x)
        assert o64.rel_rms(re + 1j * im, o64.fft_forward(x)) <= TOL
        assert o64.rel_rms(f.inverseBatch(re, im), x) <= TOL
        # packed layout
        pk = np.zeros((batch, half, 2), np.float32)
        assert lib.ma_fft_forward_host(f._h, p(x), p(pk), None, None, 0, 1.0, batch, L.LAYOUT_HALF_PACKED) == 0
        assert np.allclose(pk[:, 0, 0], ref[:, 0].real, rtol=1e-4, atol=1e-2)
        assert np.allclose(pk[:, 0, 1], ref[:, half].real, rtol=1e-4, atol=1e-2)
        assert o64.rel_rms(pk[:, 1:, 0] + 1j * pk[:, 1:, 1], ref[:, 1:half]) <= TOL
        y2 = np.zeros((batch, n), np.float32)
        assert lib.ma_fft_inverse_host(f._h, p(pk), None, p(y2), batch, L.LAYOUT_HALF_PACKED) == 0
        assert o64.rel_rms(y2, x) <= TOL


def test_config5_scaled(device, lib):
    """Configuration 5 at reduced batch: 65536-point forward + inverse on N(0,1) data, more
    transforms than one scratch chunk holds."""
    import ctypes
    from metalaudio_b200 import _lib as L
    n, batch = 65536, 400
    x = configs.c5_batch(batch=batch, n=n)
    f = make_fft(device, n)
    spec = np.zeros((batch, n // 2 + 1, 2), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert lib.ma_fft_forward_host(f._h, p(x), p(spec), None, None, 0, 1.0, batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    ref = o64.rfft(x[[0, 199, 399]])
    assert o64.rel_rms(spec[[0, 199, 399], :, 0] + 1j * spec[[0, 199, 399], :, 1], ref) <= TOL
    y = np.zeros_like(x)
    assert lib.ma_fft_inverse_host(f._h, p(spec), None, p(y), batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    assert o64.rel_rms(y, x) <= TOL


@pytest.mark.parametrize("offset", [0, 1, 2])
def test_large_forward_inverse_on_unaligned_device_rows(device, lib, offset):
    """65536-point transforms whose input (forward) or output (inverse) starts `offset` floats past a
    16-byte boundary: the column passes stage their tiles through tensor maps only for aligned arrays
    and must fall back to plain loads / stores otherwise, with identical results."""
    import ctypes
    import torch
    from metalaudio_b200 import _lib as L
    n, batch = 65536, 3
    rng = np.random.default_rng(offset)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    f = make_fft(device, n)
    buf = torch.zeros(batch * n + 4, device="cuda")
    buf[offset:offset + batch * n] = torch.from_numpy(x.ravel()).cuda()
    spec = torch.empty((batch, n // 2 + 1, 2), device="cuda")
    out = torch.zeros(batch * n + 4, device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_fft_forward_dev(f._h, ctypes.c_void_p(buf.data_ptr() + 4 * offset), ctypes.c_void_p(spec.data_ptr()), None,
                                  None, 0, 1.0, batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    assert lib.ma_fft_inverse_dev(f._h, ctypes.c_void_p(spec.data_ptr()), None, ctypes.c_void_p(out.data_ptr() + 4 * offset),
                                  batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    device.synchronize(10)
    z = spec.cpu().numpy()
    assert o64.rel_rms(z[..., 0] + 1j * z[..., 1], o64.rfft(x)) <= TOL
    y = out.cpu().numpy()
    assert o64.rel_rms(y[offset:offset + batch * n].reshape(batch, n), x) <= TOL
    assert np.all(y[:offset] == 0) and np.all(y[offset + batch * n:] == 0)  # nothing written outside the rows


def test_large_batch_over_several_chunks(device, lib):
    """A batch that needs three scratch chunks (23 + 23 + 4 transforms of 2^20 points): chunks alternate
    between the two lanes, the third reuses the first lane's scratch behind the first chunk, and the
    last one is ragged.  Transforms on both sides of every chunk boundary are checked against the
    float64 definition, the whole batch by its round trip."""
    import ctypes
    from metalaudio_b200 import _lib as L
    n, batch = 1 << 20, 50
    rng = np.random.default_rng(50)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    f = make_fft(device, n)
    spec = np.zeros((batch, n // 2 + 1, 2), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert lib.ma_fft_forward_host(f._h, p(x), p(spec), None, None, 0, 1.0, batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    pick = [0, 22, 23, 45, 46, 49]
    ref = o64.rfft(x[pick])
    assert o64.rel_rms(spec[pick, :, 0] + 1j * spec[pick, :, 1], ref) <= TOL
    y = np.zeros_like(x)
    assert lib.ma_fft_inverse_host(f._h, p(spec), None, p(y), batch, L.LAYOUT_HALF_INTERLEAVED) == 0
    for b in range(batch):
        assert o64.rel_rms(y[b], x[b]) <= TOL, b


@pytest.mark.parametrize("n", [2, 4, 16, 256, 2048, 4096, 8192, 16384, 65536, 1 << 18])
def test_complex_transform_matches_oracle(device, lib, n):
    """forwardGPU / inverseGPU (FFT.swift:945-1107, :1176-1315): complex DFT of interleaved
    (re, im) data, forward unscaled and inverse with 1/N, against numpy's float64 transforms;
    forward then inverse reproduces the input."""
    import ctypes
    rng = np.random.default_rng(7000 + n)
    batch = 3 if n <= 65536 else 1
    z = (rng.standard_normal((batch, n)) + 1j * rng.standard_normal((batch, n))).astype(np.complex64)
    fft = make_fft(device, n)
    out = np.empty((batch, 2 * n), np.float32)
    zin = np.ascontiguousarray(z).view(np.float32).reshape(batch, 2 * n)
    st = lib.ma_fft_complex_host(fft._h, zin.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                 batch, 0)
    assert st == 0
    got = out.view(np.complex64).reshape(batch, n)
    assert o64.rel_rms(got, np.fft.fft(z.astype(np.complex128), axis=-1)) <= TOL
    back = np.empty_like(out)
    st = lib.ma_fft_complex_host(fft._h, out.ctypes.data_as(ctypes.c_void_p), back.ctypes.data_as(ctypes.c_void_p),
                                 batch, 1)
    assert st == 0
    assert o64.rel_rms(back.view(np.complex64).reshape(batch, n), z) <= TOL
    inv = np.empty_like(out)
    st = lib.ma_fft_complex_host(fft._h, zin.ctypes.data_as(ctypes.c_void_p), inv.ctypes.data_as(ctypes.c_void_p),
                                 batch, 1)
    assert st == 0
    assert o64.rel_rms(inv.view(np.complex64).reshape(batch, n), np.fft.ifft(z.astype(np.complex128), axis=-1)) <= TOL
    fft.close()


def test_explicit_backend_api(device):
    """forwardGPU / inverseGPU / forwardMPSGraph / inverseMPSGraph / shouldUse* on the mirror:
    data formats, resizing of list outputs, truncation of oversized inputs, bufferSizeMismatch."""
    from metalaudio_b200 import Backend, FFTError, MetalAudioError
    n = 4096
    fft = make_fft(device, n)
    assert fft.shouldUseMetal and not fft.shouldUseMPSGraph and fft.shouldUseGPU
    rng = np.random.default_rng(11)
    x = rng.standard_normal(n).astype(np.float32)
    inter = np.zeros(2 * n + 10, np.float32)       # real signal as interleaved complex, oversized
    inter[0:2 * n:2] = x
    out = []
    assert fft.forwardGPU(inter, out) is Backend.cuda
    assert len(out) == 2 * n
    Z = np.asarray(out, np.float32).view(np.complex64)
    assert o64.rel_rms(Z, o64.fft_forward(x)) <= TOL
    back = np.zeros(2 * n, np.float32)
    fft.inverseGPU(out, back)
    assert o64.rel_rms(back[0::2], x) <= TOL and np.max(np.abs(back[1::2])) < 1e-5
    with pytest.raises(MetalAudioError) as e:
        fft.forwardGPU(np.zeros(100, np.float32), out)
    assert e.value.case == "bufferSizeMismatch" and (e.value.expected, e.value.actual) == (2 * n, 100)
    with pytest.raises(MetalAudioError):
        fft.inverseGPU(np.zeros(2 * n - 1, np.float32), out)
    re, im, y = [], [], []
    fft.forwardMPSGraph(x, re, im)
    assert len(re) == n and o64.rel_rms(np.asarray(re) + 1j * np.asarray(im), o64.fft_forward(x)) <= TOL
    fft.inverseMPSGraph(re, im, y)
    assert o64.rel_rms(np.asarray(y), x) <= TOL
    with pytest.raises(FFTError):
        fft.forwardMPSGraph(x[:10], re, im)
    big = make_fft(device, 16384)
    assert big.shouldUseMPSGraph and not big.shouldUseMetal
    small = make_fft(device, 1024)
    assert not small.shouldUseMetal and not small.shouldUseMPSGraph
    for f in (fft, big, small):
        f.close()


def test_output_validation_flags_non_finite_results(device):
    """fftValidationEnabled (FFT.swift:63): a NaN in the input reaches every output bin, and the
    sampled check notices; the call itself neither raises nor alters the result."""
    from metalaudio_b200 import dsp
    n = 1024
    fft = make_fft(device, n)
    x = np.ones(n, np.float32)
    x[5] = np.nan
    re, im = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dsp.fftValidationEnabled = True
    try:
        dsp.fftValidationLog.clear()
        fft.forward(x, re, im)
        assert np.isnan(re).all()
        assert any("NaN detected in outputReal" in m for m in dsp.fftValidationLog)
    finally:
        dsp.fftValidationEnabled = False
    fft.close()
