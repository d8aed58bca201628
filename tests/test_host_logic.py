"""CPU tests of the host-side mirror: configuration, windows, COLA, error vocabulary and the
C-ABI surface.  No GPU compute is called."""
import os
import re

import numpy as np
import pytest

from metalaudio_b200 import (COLACompliance, Convolution, ConvolutionError, FFT, FFTError, MetalAudioError,
                             WindowType, validatedWindowFloor)
from metalaudio_b200 import _lib as L
from metalaudio_b200.sharding import all_shards, shard_range
from oracle import reference_path as rp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_config_defaults_and_overlap():
    c = FFT.Config(size=2048)
    assert c.hopSize == 512 and c.windowType is WindowType.hann and not c.inverse
    assert FFT.Config(size=2).hopSize == 1
    assert FFT.Config(size=1024, hopSize=256).overlapPercent == 75
    assert FFT.Config(size=1024, hopSize=512).overlapPercent == 50


def test_cola_compliance_table():
    """FFTTests COLA rows: divisors [1] / [2,4] / [] / [3,4]."""
    assert WindowType.none.colaHopDivisors == [1]
    assert WindowType.hann.colaHopDivisors == [2, 4]
    assert WindowType.hamming.colaHopDivisors == []
    assert WindowType.blackman.colaHopDivisors == [3, 4]
    assert FFT.Config(size=2048, windowType=WindowType.hann, hopSize=512).colaCompliance is COLACompliance.perfect
    assert FFT.Config(size=2048, windowType=WindowType.hann, hopSize=1024).colaCompliance is COLACompliance.perfect
    assert FFT.Config(size=2048, windowType=WindowType.hann, hopSize=300).colaCompliance is COLACompliance.nonCompliant
    assert FFT.Config(size=2048, windowType=WindowType.hamming, hopSize=512).colaCompliance is COLACompliance.nearPerfect
    assert FFT.Config(size=2048, windowType=WindowType.hamming, hopSize=100).colaCompliance is COLACompliance.nonCompliant
    assert FFT.Config(size=2048, windowType=WindowType.none, hopSize=2048).colaCompliance is COLACompliance.perfect
    assert FFT.Config(size=1024, windowType=WindowType.blackman, hopSize=256).colaCompliance is COLACompliance.perfect
    ok, comp, msg = FFT.Config(size=2048, windowType=WindowType.hann, hopSize=512).validateCOLA()
    assert ok and "Hann" in msg and "512" in msg and "75%" in msg
    ok, comp, msg = FFT.Config(size=2048, windowType=WindowType.hann, hopSize=300).validateCOLA()
    assert not ok and "1024 (50% overlap)" in msg and "512 (75% overlap)" in msg
    ok, comp, msg = FFT.Config(size=2048, windowType=WindowType.hamming, hopSize=300).validateCOLA()
    assert not ok and "Consider using Hann" in msg
    assert "perfect" in COLACompliance.perfect.description.lower()


def test_window_tables_match_the_port():
    for kind in ("none", "hann", "hamming", "blackman"):
        for n in (1, 2, 8, 256, 4096):
            assert np.array_equal(WindowType(kind).table(n), rp.window(kind, n))
    w = WindowType.hann
    assert w.coefficient(0, 256) == 0 and abs(w.coefficient(128, 256) - 1) < 1e-3
    assert w.coefficient(3, 1) == 1.0
    t = WindowType.hann.table(256)
    assert all(abs(float(w.coefficient(i, 256)) - float(t[i])) < 1e-7 for i in (0, 1, 77, 255))


def test_fft_error_vocabulary():
    """FFTTests error rows: every description mentions its payload."""
    cases = [FFTError.inputTooShort(100, 256), FFTError.sizeTooLarge(1 << 25, 1 << 24), FFTError.sizeNotPowerOf2(300),
             FFTError.invalidHopSize(0, 256), FFTError.batchSizeOverflow(7, 4096),
             FFTError.istftOutputOverflow(5, 128, 512), FFTError.istftFrameOverflow(3, 128, 512, 1000)]
    for e, nums in zip(cases, [(100, 256), (1 << 25, 1 << 24), (300,), (0, 256), (7, 4096), (5, 128, 512),
                               (3, 128, 512, 1000)]):
        for v in nums:
            assert str(v) in e.errorDescription
    for e in (ConvolutionError.inputSizeMismatch(9, 8, 16), ConvolutionError.outputSizeOverflow(5, 6)):
        assert "5" in e.errorDescription or "9" in e.errorDescription
    assert "state" in ConvolutionError.invalidPartitionState("x=1").errorDescription
    assert ConvolutionError.emptyKernel().case == "emptyKernel"


def test_fft_init_validation_needs_no_device():
    """Validation order of FFT.init: power of two, maximum size, hop (FFT.swift:443-455)."""
    class NoDevice:  # construction must fail before the device is touched
        _lib = None
        handle = None
    with pytest.raises(FFTError) as e:
        FFT(NoDevice(), FFT.Config(size=300))
    assert e.value.case == "sizeNotPowerOf2" and e.value.size == 300
    with pytest.raises(FFTError) as e:
        FFT(NoDevice(), FFT.Config(size=1 << 25))
    assert e.value.case == "sizeTooLarge"
    with pytest.raises(FFTError) as e:
        FFT(NoDevice(), FFT.Config(size=256, hopSize=257))
    assert e.value.case == "invalidHopSize" and e.value.hopSize == 257
    with pytest.raises(FFTError):
        FFT(NoDevice(), FFT.Config(size=256, hopSize=0))


def test_window_floor_validation():
    assert validatedWindowFloor() == pytest.approx(1e-8)
    assert validatedWindowFloor(1e-12) == 1e-6 and validatedWindowFloor(0.7) == 0.1


def test_shard_ranges():
    assert all_shards(256, 8) == [(32 * i, 32 * i + 32) for i in range(8)]
    assert all_shards(10, 4) == [(0, 2), (2, 5), (5, 7), (7, 10)]
    # IR pairs stay together
    for lo, hi in all_shards(1024, 8, group=2):
        assert lo % 2 == 0 and hi % 2 == 0 and hi - lo == 128
    cover = all_shards(6, 4, group=2)
    assert cover[0][0] == 0 and cover[-1][1] == 6 and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))
    with pytest.raises(ValueError):
        shard_range(5, 0, 2, group=2)


def test_cabi_library_exports_every_declared_symbol(lib):
    """The shared library loads and exports exactly what include/metalaudio_cuda.h declares; the
    ctypes table binds the same set."""
    hdr = open(os.path.join(ROOT, "include", "metalaudio_cuda.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(ma_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 40
    assert declared == set(L.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.ma_status_string(L.MA_ERR_SIZE_NOT_POW2).decode().startswith("FFT size")
    assert lib.ma_status_string(0) == b"ok"


def test_no_cpu_fallback(lib):
    """Without a CUDA device the product fails loudly (and never computes on the CPU)."""
    if lib.ma_device_count() > 0:
        pytest.skip("a CUDA device is present")
    from metalaudio_b200 import AudioDevice
    with pytest.raises(MetalAudioError) as e:
        AudioDevice()
    assert e.value.case == "deviceNotFound"
    import ctypes
    h = ctypes.c_void_p()
    assert lib.ma_context_create(0, 0, ctypes.byref(h)) == L.MA_ERR_DEVICE_LOST
    # plan-level validation answers without a device, in the reference's order
    assert lib.ma_fft_plan_create(None, 300, None, 64, ctypes.byref(h)) == L.MA_ERR_SIZE_NOT_POW2
    assert lib.ma_fft_plan_create(None, 1 << 25, None, 64, ctypes.byref(h)) == L.MA_ERR_SIZE_TOO_LARGE
    assert lib.ma_fft_plan_create(None, 256, None, 0, ctypes.byref(h)) == L.MA_ERR_INVALID_HOP
    assert lib.ma_fft_plan_create(None, 256, None, 64, ctypes.byref(h)) == L.MA_ERR_INVALID_ARGUMENT


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "metalaudio_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f


def test_biquad_design_matches_port_and_validation():
    """Coefficient design and its validation order (Filters.swift:346-490) need no device."""
    from metalaudio_b200.dsp import BiquadFilter, FilterError
    from oracle import reference_path as rp
    T = BiquadFilter.FilterType
    cases = [(T.lowpass, "lowpass", 0.0), (T.highpass, "highpass", 0.0), (T.bandpass, "bandpass", 0.0),
             (T.notch, "notch", 0.0), (T.allpass, "allpass", 0.0), (T.peaking(6.0), "peaking", 6.0),
             (T.lowshelf(-12.0), "lowshelf", -12.0), (T.highshelf(3.0), "highshelf", 3.0)]
    for t, kind, g in cases:
        for fr, sr, q in [(1000.0, 44100.0, 0.707), (50.0, 48000.0, 12.0), (15000.0, 44100.0, 0.5)]:
            c = BiquadFilter.design(t, fr, sr, q).asArray()
            assert np.array_equal(c, rp.biquad_coefficients(kind, fr, sr, q, g))
            assert abs(c[4]) < 1 and abs(c[3]) < 1 + c[4]
    lp = BiquadFilter.design(T.lowpass, 1000.0, 44100.0).asArray().astype(np.float64)
    assert abs((lp[0] + lp[1] + lp[2]) / (1 + lp[3] + lp[4]) - 1.0) < 1e-4        # unity gain at DC
    hp = BiquadFilter.design(T.highpass, 1000.0, 44100.0).asArray().astype(np.float64)
    assert abs(hp[0] + hp[1] + hp[2]) < 1e-6                                      # zero at DC
    pk = BiquadFilter.design(T.peaking(0.0), 1000.0, 44100.0).asArray()
    assert np.allclose(pk[:3], [1.0, pk[3], pk[4]], atol=1e-7)                    # 0 dB peaking = identity
    for args, name in [((T.lowpass, 1000.0, 0.0), "sampleRate"), ((T.lowpass, 0.0, 44100.0), "frequency"),
                       ((T.lowpass, 30000.0, 44100.0), "frequency"), ((T.lowpass, 1000.0, 44100.0, 0.0), "q"),
                       ((T.lowpass, 1000.0, 44100.0, -1.0), "q")]:
        with pytest.raises(FilterError) as e:
            BiquadFilter.design(*args)
        assert e.value.case == "invalidParameter" and e.value.name == name
    assert "Invalid parameter 'q'" in FilterError.invalidParameter("q", 0.0, "must be > 0").errorDescription
    assert FilterError.unstable("x").errorDescription == "Filter is unstable: x"
    d = BiquadFilter.Coefficients()
    assert (d.b0, d.b1, d.b2, d.a1, d.a2) == (1, 0, 0, 0, 0)


def test_output_validation_samples_like_the_reference():
    """validateFFTOutput (FFT.swift:80-134): off by default; when enabled it samples about 50 evenly
    spaced values plus the last one, so a NaN between samples goes unseen, one on a sample or at the
    end is reported with its index, and nothing ever raises."""
    from metalaudio_b200 import dsp
    x = np.zeros(1000, np.float32)
    x[20] = np.nan
    assert dsp.validateFFTOutput(x, 1000, "outputReal") is False          # disabled
    dsp.fftValidationEnabled = True
    try:
        dsp.fftValidationLog.clear()
        assert dsp.validateFFTOutput(x, 1000, "outputReal") is True        # stride 20 lands on index 20
        assert dsp.fftValidationLog[-1] == "[FFT] Warning: NaN detected in outputReal near index 20"
        y = np.zeros(1000, np.float32)
        y[21] = np.inf                                                      # between two samples
        assert dsp.validateFFTOutput(y, 1000, "outputImag") is False
        y[999] = np.inf                                                     # the last element is always checked
        assert dsp.validateFFTOutput(y, 1000, "outputImag") is True
        assert dsp.fftValidationLog[-1] == "[FFT] Warning: Inf detected in outputImag near index 999"
        assert dsp.validateFFTOutput(np.zeros(0, np.float32), 0, "empty") is False
        z = np.array([np.nan, np.inf, 0.0], np.float32)                     # count < 50: every element
        assert dsp.validateFFTOutput(z, 3, "tiny") is True
        assert any("NaN" in m and "index 0" in m for m in dsp.fftValidationLog[-2:])
        assert any("Inf" in m and "index 1" in m for m in dsp.fftValidationLog[-2:])
        assert dsp.validateFFTOutput(np.ones(4096, np.float32), 4096, "clean") is False
    finally:
        dsp.fftValidationEnabled = False


def test_buffer_size_mismatch_error_text():
    e = MetalAudioError.bufferSizeMismatch(8192, 100)
    assert e.case == "bufferSizeMismatch" and (e.expected, e.actual) == (8192, 100)
    assert str(e) == "Buffer size mismatch: expected 8192 bytes, got 100"


def test_swift_package_calls_only_declared_entry_points():
    """The Swift sources (written against the header, never compiled here) may only call functions
    and use constants the C header declares."""
    header = open(os.path.join(ROOT, "include", "metalaudio_cuda.h")).read()
    declared = set(re.findall(r"\b(ma_[a-z0-9_]+)\s*\(", header))
    constants = set(re.findall(r"\b(MA_[A-Z0-9_]+)\b", header))
    swift_dir = os.path.join(ROOT, "swift", "Sources")
    seen = set()
    for dirpath, _, files in os.walk(swift_dir):
        for f in files:
            if not f.endswith(".swift"):
                continue
            text = open(os.path.join(dirpath, f)).read()
            assert "NOT COMPILED" in text.splitlines()[0], f
            for name in re.findall(r"\b(ma_[a-z0-9_]+)\s*\(", text):
                if name == "ma_status":      # the status type used as a converting initialiser
                    continue
                assert name in declared, (f, name)
                seen.add(name)
            for name in re.findall(r"\b(MA_[A-Z0-9_]+)\b", text):
                assert name in constants, (f, name)
    assert {"ma_context_create", "ma_fft_plan_create", "ma_stft_host", "ma_istft_host", "ma_pconv_process_host",
            "ma_fft_complex_host", "ma_fftconv_process_host"} <= seen
    assert os.path.exists(os.path.join(ROOT, "swift", "Package.swift"))
    assert os.path.exists(os.path.join(ROOT, "swift", "Sources", "CMetalAudioCUDA", "module.modulemap"))
