"""float32 restatement ("port") of the reference's CPU path for FFT, STFT/iSTFT and
uniformly partitioned convolution.  TEST INFRASTRUCTURE: see ``oracle/__init__.py``.

The reference executes these steps with Apple vDSP calls; every vDSP routine used on
the path is a textbook operation (DFT, element-wise multiply / add / scale / clip /
divide), restated here with numpy.  The FFT itself is ``scipy.fft`` on float32 input,
which computes in float32 (pocketfft), i.e. the same arithmetic type as vDSP.

Each function cites the reference lines it follows (paths within the reference tree).
"""
from __future__ import annotations

import numpy as np
import scipy.fft as sfft

F32 = np.float32

# Threads scipy.fft may use (None: one).  The CPU-baseline legs of the benchmark set this to
# the host core count; parity tests leave it alone.
WORKERS = None

# --------------------------------------------------------------------------- windows


def window(kind: str, length: int) -> np.ndarray:
    """Window table exactly as Sources/MetalDSP/FFT.swift:268-294 builds it:
    SYMMETRIC (denominator N-1), evaluated in float64, rounded once to float32;
    length 1 gives 1.0.  ``kind`` is one of none / hann / hamming / blackman."""
    if length <= 1 or kind == "none":
        return np.ones(max(length, 0), dtype=F32)
    n = np.arange(length, dtype=np.float64)
    denom = float(length) - 1.0
    if kind == "hann":
        w = 0.5 * (1.0 - np.cos(2.0 * np.pi * n / denom))
    elif kind == "hamming":
        w = 0.54 - 0.46 * np.cos(2.0 * np.pi * n / denom)
    elif kind == "blackman":
        w = 0.42 - 0.5 * np.cos(2.0 * np.pi * n / denom) + 0.08 * np.cos(4.0 * np.pi * n / denom)
    else:
        raise ValueError(f"unknown window {kind!r}")
    return w.astype(F32)


def periodic_hann(length: int) -> np.ndarray:
    """Periodic Hann (denominator N), the window the benchmark configuration names.
    Not what the reference computes; offered because the window table is an input of
    the kernels, so both can be served."""
    n = np.arange(length, dtype=np.float64)
    return (0.5 * (1.0 - np.cos(2.0 * np.pi * n / float(length)))).astype(F32)


# --------------------------------------------------------------------------- FFT


def fft_forward(x: np.ndarray):
    """Unnormalised DFT of real frames, full-N split output (real[N], imag[N]).
    Sources/MetalDSP/FFT.swift:818-855 (imaginary input zero, forward sign
    exp(-2*pi*i*k*n/N), no scaling).  ``x``: (..., N) float32."""
    x = np.ascontiguousarray(x, dtype=F32)
    X = sfft.fft(x.astype(np.complex64), axis=-1, workers=WORKERS)
    return np.ascontiguousarray(X.real, dtype=F32), np.ascontiguousarray(X.imag, dtype=F32)


def fft_inverse(re: np.ndarray, im: np.ndarray) -> np.ndarray:
    """Inverse DFT of a full-N split spectrum, real part scaled by 1/N.
    Sources/MetalDSP/FFT.swift:889-919 (an ``inverse: true`` object)."""
    Z = np.asarray(re, dtype=F32) + 1j * np.asarray(im, dtype=F32)
    n = Z.shape[-1]
    z = sfft.ifft(Z.astype(np.complex64), axis=-1, norm="forward", workers=WORKERS)  # unscaled
    return (z.real.astype(F32) * F32(1.0 / F32(n))).astype(F32)


def magnitude(re: np.ndarray, im: np.ndarray) -> np.ndarray:
    """sqrt(re^2 + im^2) over bins 0..N/2 inclusive.  FFT.swift:1780-1791."""
    n = re.shape[-1]
    k = n // 2 + 1
    r = np.asarray(re[..., :k], dtype=F32)
    i = np.asarray(im[..., :k], dtype=F32)
    return np.sqrt(r * r + i * i, dtype=F32)


def power(re: np.ndarray, im: np.ndarray) -> np.ndarray:
    """re^2 + im^2 over bins 0..N/2.  FFT.swift:1804-1815."""
    n = re.shape[-1]
    k = n // 2 + 1
    r = np.asarray(re[..., :k], dtype=F32)
    i = np.asarray(im[..., :k], dtype=F32)
    return (r * r + i * i).astype(F32)


def magnitude_db(re: np.ndarray, im: np.ndarray, reference: float = 1.0) -> np.ndarray:
    """20*log10(magnitude/reference), no clamping (silence -> -inf).
    FFT.swift:1833-1847 (vDSP_vdbcon with the amplitude flag)."""
    m = magnitude(re, im)
    with np.errstate(divide="ignore"):
        return (F32(20.0) * np.log10(m / F32(reference))).astype(F32)


# --------------------------------------------------------------------------- STFT


def stft_frame_count(length: int, n: int, hop: int) -> int:
    """(L - N)/hop + 1, integer division; L < N is an error.  STFT.swift:45-49."""
    if length < n:
        raise ValueError(f"inputTooShort(inputSize: {length}, requiredSize: {n})")
    return (length - n) // hop + 1


def stft(x: np.ndarray, n: int, hop: int, win: np.ndarray):
    """Frames at i*hop (no centring, no padding), times the analysis window, forward
    DFT; returns (real, imag) each (F, N).  STFT.swift:40-81."""
    x = np.asarray(x, dtype=F32)
    f = stft_frame_count(x.shape[-1], n, hop)
    idx = np.arange(f)[:, None] * hop + np.arange(n)[None, :]
    frames = x[..., idx] * np.asarray(win, dtype=F32)
    return fft_forward(frames)


def window_floor(configured: float = 1e-8) -> np.float32:
    """Floor rule of STFT.swift:491-501: below 1e-10 -> 1e-6, above 0.1 -> 0.1.
    The default 1e-8 is ToleranceConfiguration.conservative()'s windowFloorEpsilon
    (Sources/MetalAudioKit/Config/ToleranceConfiguration.swift:166-181), the profile an
    unknown GPU maps to."""
    c = F32(configured)
    if c < F32(1e-10):
        return F32(1e-6)
    if c > F32(0.1):
        return F32(0.1)
    return c


def window_sum(frames: int, n: int, hop: int, win: np.ndarray, floor: float) -> np.ndarray:
    """Sum of squared window over covering frames, denormals zeroed, clamped to the
    floor.  STFT.swift:448-479, :513-520.  Accumulated frame by frame in float32 in
    the same order as the reference's sequential loop."""
    out_len = (frames - 1) * hop + n
    wsq = (np.asarray(win, dtype=F32) ** 2).astype(F32)
    ws = np.zeros(out_len, dtype=F32)
    for f in range(frames):
        ws[f * hop:f * hop + n] += wsq
    ws[ws < np.finfo(F32).tiny] = 0
    return np.maximum(ws, F32(floor)).astype(F32)


def istft(re: np.ndarray, im: np.ndarray, n: int, hop: int, win: np.ndarray,
          floor: float | None = None) -> np.ndarray:
    """Inverse DFT per frame (x 1/N), times the synthesis window, overlap-add,
    divided by max(sum w^2, floor).  STFT.swift:384-527.

    Deliberate deviation, shared with the CUDA path: the reference runs the frames
    through the object's own (forward-direction) DFT setup (STFT.swift:356-362), which
    returns each frame time-reversed; this restatement, like the float64 definition the
    benchmark demands, uses the true inverse."""
    re = np.asarray(re, dtype=F32)
    im = np.asarray(im, dtype=F32)
    frames = re.shape[0]
    if frames == 0:
        return np.zeros(0, dtype=F32)
    fl = window_floor() if floor is None else F32(floor)
    out_len = (frames - 1) * hop + n
    y = fft_inverse(re, im) * np.asarray(win, dtype=F32)
    out = np.zeros(out_len, dtype=F32)
    for f in range(frames):
        out[f * hop:f * hop + n] += y[f]
    return (out / window_sum(frames, n, hop, win, fl)).astype(F32)


# ----------------------------------------------------------- partitioned convolution


class PartitionedConvolution:
    """Block-sequential uniformly partitioned overlap-add convolution with a
    frequency-domain delay line, following Convolution.swift:250-322 (set-up),
    :529-758 (process) and :764-775 (reset).

    ``fftSize = 2B``; ``P = ceil(K/B)``; partition spectra keep all 2B bins; the ring
    holds the last P input-block spectra; every block multiplies ring slot
    ``(w + (P - p) % P) % P`` (the spectrum of block t-p) with partition p, sums over
    p in a running float32 sum, inverse-transforms (x 1/(2B)) and adds all 2B samples at
    ``t*B`` truncated at L+K-1.  State survives across ``process`` calls until ``reset``.
    """

    def __init__(self, block_size: int):
        if block_size <= 0:
            raise ValueError(f"Block size must be positive, got {block_size}")
        self.block = int(block_size)
        self.fft_size = 2 * self.block
        self.kernel = None

    def set_kernel(self, kernel: np.ndarray) -> None:
        kernel = np.asarray(kernel, dtype=F32)
        if kernel.size == 0:
            raise ValueError("Kernel must not be empty for partitioned convolution")
        b, n = self.block, self.fft_size
        self.kernel = kernel
        self.partitions = (kernel.size + b - 1) // b
        padded = np.zeros(self.partitions * b, dtype=F32)
        padded[:kernel.size] = kernel
        blocks = np.zeros((self.partitions, n), dtype=F32)
        blocks[:, :b] = padded.reshape(self.partitions, b)
        self.h = sfft.fft(blocks.astype(np.complex64), axis=-1)        # (P, 2B) complex64
        self.reset()

    def reset(self) -> None:
        self.ring = np.zeros((self.partitions, self.fft_size), dtype=np.complex64)
        self.write_index = 0

    def process(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, dtype=F32)
        if x.size == 0:
            return np.zeros(0, dtype=F32)
        b, n, p_count = self.block, self.fft_size, self.partitions
        full = x.size + self.kernel.size - 1
        total_blocks = (full + b - 1) // b
        out = np.zeros(full + n, dtype=F32)
        p_idx = np.arange(p_count)
        offsets = (p_count - p_idx) % p_count
        block = np.zeros(n, dtype=F32)
        for t in range(total_blocks):
            lo = t * b
            block[:] = 0
            if lo < x.size:
                seg = x[lo:lo + b]
                block[:seg.size] = seg
            self.ring[self.write_index] = sfft.fft(block.astype(np.complex64))
            slots = (self.write_index + offsets) % p_count
            prod = self.ring[slots] * self.h                       # (P, 2B) complex64
            # running float32 sum over p in increasing p, as the two vDSP_vadd calls do
            acc = np.add.reduce(prod, axis=0, dtype=np.complex64)
            y = sfft.ifft(acc, norm="forward").real.astype(F32) * F32(1.0 / F32(n))
            out[lo:lo + n] += y
            self.write_index = (self.write_index + 1) % p_count
        return out[:full].copy()


# ----------------------------------------------------------- one-shot FFT convolution


class FFTConvolution:
    """The `.fft` mode, following Convolution.swift:210-248 (set-up) and :437-493 (process):
    ``fftSize = 1 << ceil(log2(expected + K - 1))``, full-size float32 complex transforms of the
    zero-padded kernel (once) and input, bin-by-bin complex product, inverse scaled by 1/fftSize;
    the result has ``fftSize`` samples.  Inputs longer than ``expected`` are refused
    (ConvolutionError.inputSizeMismatch, :461-467)."""

    def __init__(self, kernel: np.ndarray, expected_input_size=None):
        kernel = np.asarray(kernel, dtype=F32)
        if kernel.size == 0:
            raise ValueError("Convolution kernel cannot be empty")
        self.kernel = kernel
        self.expected = int(kernel.size if expected_input_size is None else expected_input_size)
        min_size = self.expected + kernel.size - 1
        self.fft_size = 1 << int(np.ceil(np.log2(float(min_size))))
        padded = np.zeros(self.fft_size, dtype=F32)
        padded[:kernel.size] = kernel
        self.h = sfft.fft(padded.astype(np.complex64))

    def process(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, dtype=F32)
        if x.size == 0:
            return np.zeros(0, dtype=F32)
        if x.size > self.expected:
            raise ValueError(f"input size {x.size} exceeds expected maximum {self.expected} (FFT size: {self.fft_size})")
        padded = np.zeros(self.fft_size, dtype=F32)
        padded[:x.size] = x
        spec = sfft.fft(padded.astype(np.complex64))
        re = spec.real * self.h.real - spec.imag * self.h.imag       # the reference's scalar loop (:476-480)
        im = spec.real * self.h.imag + spec.imag * self.h.real
        y = sfft.ifft((re + 1j * im).astype(np.complex64), norm="forward").real.astype(F32)
        return (y * F32(1.0 / F32(self.fft_size))).astype(F32)


# ----------------------------------------------------------- magnitude / phase glue


def to_polar(re: np.ndarray, im: np.ndarray):
    """Magnitude and phase per bin as the STFT's consumer computes them in float32
    (HTDemucs.swift:735-738; shader forms DSP.metal:784-813): sqrt(re^2 + im^2), atan2(im, re)."""
    re = np.asarray(re, dtype=F32)
    im = np.asarray(im, dtype=F32)
    return np.sqrt(re * re + im * im).astype(F32), np.arctan2(im, re).astype(F32)


def from_polar(mag: np.ndarray, phase: np.ndarray):
    """mag*cos(phase), mag*sin(phase) in float32 (HTDemucs.swift:803-804; DSP.metal:821-834)."""
    mag = np.asarray(mag, dtype=F32)
    phase = np.asarray(phase, dtype=F32)
    return (mag * np.cos(phase)).astype(F32), (mag * np.sin(phase)).astype(F32)


def to_decibels(data: np.ndarray, reference: float, min_db: float) -> np.ndarray:
    """DSP.metal:861-881: 20*log10(max(x/reference, 1e-10)) floored at min_db; a reference <= 0
    yields min_db everywhere."""
    data = np.asarray(data, dtype=F32)
    if reference <= 0:
        return np.full(data.shape, F32(min_db), dtype=F32)
    ratio = np.maximum(data / F32(reference), F32(1e-10))
    return np.maximum(F32(20.0) * np.log10(ratio), F32(min_db)).astype(F32)


# ----------------------------------------------------------- biquad filters


def biquad_coefficients(kind: str, frequency: float, sample_rate: float, q: float = 0.7071067811865476,
                        gain_db: float = 0.0) -> np.ndarray:
    """(b0, b1, b2, a1, a2) in float32 as BiquadFilter.configure derives them
    (Filters.swift:226-345, :386-437): float32 parameters widened to float64, the cookbook forms,
    division by a0, rounding to float32.  Validation is not restated here."""
    f, sr, qq = (float(F32(v)) for v in (frequency, sample_rate, q))
    w = 2.0 * np.pi * f / sr
    sn, cs = np.sin(w), np.cos(w)
    al = sn / (2.0 * qq)
    amp = 10.0 ** (float(F32(gain_db)) / 40.0)
    if kind == "lowpass":
        b, a = [(1 - cs) / 2, 1 - cs, (1 - cs) / 2], [1 + al, -2 * cs, 1 - al]
    elif kind == "highpass":
        b, a = [(1 + cs) / 2, -(1 + cs), (1 + cs) / 2], [1 + al, -2 * cs, 1 - al]
    elif kind == "bandpass":
        b, a = [al, 0.0, -al], [1 + al, -2 * cs, 1 - al]
    elif kind == "notch":
        b, a = [1.0, -2 * cs, 1.0], [1 + al, -2 * cs, 1 - al]
    elif kind == "allpass":
        b, a = [1 - al, -2 * cs, 1 + al], [1 + al, -2 * cs, 1 - al]
    elif kind == "peaking":
        b, a = [1 + al * amp, -2 * cs, 1 - al * amp], [1 + al / amp, -2 * cs, 1 - al / amp]
    elif kind == "lowshelf":
        r = 2 * np.sqrt(amp) * al
        b = [amp * ((amp + 1) - (amp - 1) * cs + r), 2 * amp * ((amp - 1) - (amp + 1) * cs),
             amp * ((amp + 1) - (amp - 1) * cs - r)]
        a = [(amp + 1) + (amp - 1) * cs + r, -2 * ((amp - 1) + (amp + 1) * cs), (amp + 1) + (amp - 1) * cs - r]
    elif kind == "highshelf":
        r = 2 * np.sqrt(amp) * al
        b = [amp * ((amp + 1) + (amp - 1) * cs + r), -2 * amp * ((amp - 1) + (amp + 1) * cs),
             amp * ((amp + 1) + (amp - 1) * cs - r)]
        a = [(amp + 1) - (amp - 1) * cs + r, 2 * ((amp - 1) - (amp + 1) * cs), (amp + 1) - (amp - 1) * cs - r]
    else:
        raise ValueError(kind)
    return np.array([b[0] / a[0], b[1] / a[0], b[2] / a[0], a[1] / a[0], a[2] / a[0]]).astype(F32)


def biquad_process(x: np.ndarray, coeffs: np.ndarray, state=None, dtype=F32):
    """Direct Form II Transposed recurrence of BiquadFilter.process(sample:) (Filters.swift:515-537)
    and the biquad_filter_multichannel shader (DSP.metal:727-735) over the last axis of x, in
    `dtype` arithmetic; returns (y, final (z1, z2)).  scipy.signal.lfilter implements exactly this
    structure, with `zi` holding (z1, z2)."""
    import scipy.signal as ssig
    x = np.asarray(x, dtype=dtype)
    c = np.asarray(coeffs, dtype=dtype)
    b = c[:3]
    a = np.concatenate([np.ones(1, dtype=dtype), c[3:5]])
    zi = np.zeros(x.shape[:-1] + (2,), dtype=dtype) if state is None else np.asarray(state, dtype=dtype)
    y, zf = ssig.lfilter(b, a, x, axis=-1, zi=zi)
    return y.astype(dtype), zf.astype(dtype)
