"""float64 definition of the hot-path operations: the tolerance oracle.
TEST INFRASTRUCTURE: see ``oracle/__init__.py``.

Acceptance everywhere: ``rms(y - y_ref) / rms(y_ref) <= 1e-5`` with float32 kernels
compared against these float64 results computed on the same float32 inputs.
"""
from __future__ import annotations

import numpy as np
import scipy.signal as ssig


def _wide(a):
    a = np.asarray(a)
    return a.astype(np.complex128 if np.iscomplexobj(a) else np.float64)


def rel_rms(y, ref) -> float:
    """rms(y - ref) / rms(ref) in float64 (0 when both are all-zero)."""
    y = _wide(y)
    ref = _wide(ref)
    den = np.sqrt(np.mean(np.abs(ref) ** 2))
    num = np.sqrt(np.mean(np.abs(y - ref) ** 2))
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return float(num / den)


def max_over_rms(y, ref) -> float:
    """max|y - ref| / rms(ref)."""
    y = _wide(y)
    ref = _wide(ref)
    den = np.sqrt(np.mean(np.abs(ref) ** 2))
    return float(np.max(np.abs(y - ref)) / den) if den > 0 else 0.0


def fft_forward(x):
    """Full-N complex DFT of real frames (forward sign, unscaled), complex128."""
    return np.fft.fft(np.asarray(x, dtype=np.float64), axis=-1)


def rfft(x):
    """Half spectrum, bins 0..N/2."""
    return np.fft.rfft(np.asarray(x, dtype=np.float64), axis=-1)


def irfft(X, n):
    """Real inverse with 1/N scaling from bins 0..N/2."""
    return np.fft.irfft(np.asarray(X, dtype=np.complex128), n=n, axis=-1)


def fft_inverse(re, im):
    """Real part of the 1/N-scaled inverse DFT of a full-N spectrum."""
    Z = np.asarray(re, dtype=np.float64) + 1j * np.asarray(im, dtype=np.float64)
    return np.fft.ifft(Z, axis=-1).real


def stft(x, n, hop, win):
    """(F, N/2+1) complex128 half spectra of windowed frames at i*hop."""
    x = np.asarray(x, dtype=np.float64)
    f = (x.shape[-1] - n) // hop + 1
    idx = np.arange(f)[:, None] * hop + np.arange(n)[None, :]
    return np.fft.rfft(x[..., idx] * np.asarray(win, dtype=np.float64), axis=-1)


def istft(X, n, hop, win, floor):
    """Overlap-add inverse of half spectra (..., F, N/2+1) with the reference's
    normaliser: out / max(sum w^2, floor)."""
    X = np.asarray(X, dtype=np.complex128)
    frames = X.shape[-2]
    w = np.asarray(win, dtype=np.float64)
    y = np.fft.irfft(X, n=n, axis=-1) * w
    out_len = (frames - 1) * hop + n
    out = np.zeros(X.shape[:-2] + (out_len,), dtype=np.float64)
    ws = np.zeros(out_len, dtype=np.float64)
    for f in range(frames):
        out[..., f * hop:f * hop + n] += y[..., f, :]
        ws[f * hop:f * hop + n] += w * w
    return out / np.maximum(ws, float(floor))


def convolve_full(x, h):
    """Full linear convolution (length L+K-1) in float64 via FFT."""
    return ssig.fftconvolve(np.asarray(x, dtype=np.float64), np.asarray(h, dtype=np.float64), mode="full")


def convolve_spot(x, h, indices):
    """Exact float64 dot-product values of the full convolution at chosen output
    indices (each costs K multiply-adds); the spot check for sizes where a full
    direct convolution is too slow."""
    x = np.asarray(x, dtype=np.float64)
    h = np.asarray(h, dtype=np.float64)
    L, K = x.size, h.size
    out = np.empty(len(indices), dtype=np.float64)
    for j, n in enumerate(indices):
        lo = max(0, n - (K - 1))
        hi = min(L - 1, n)
        if hi < lo:
            out[j] = 0.0
            continue
        xs = x[lo:hi + 1]
        hs = h[n - hi:n - lo + 1][::-1]
        out[j] = float(np.dot(xs, hs))
    return out
