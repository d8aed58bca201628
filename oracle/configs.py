"""Seeded synthetic inputs for the five benchmark configurations.
TEST INFRASTRUCTURE: see ``oracle/__init__.py``.

The reference's own benchmarks use synthetic sines and name no public dataset; these
generators are synthetic by construction.  Generator: ``numpy.random.Generator(PCG64(seed))``,
drawn in float64 and rounded to float32.  Every function takes size overrides so the
same distributions serve the small parity cases.
"""
from __future__ import annotations

import numpy as np

SEEDS = {"c1": 1001, "c2": 1002, "c3_ir": 1003, "c3_x": 1013, "c4_ir": 1004, "c4_x": 1014, "c5": 1005}


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def c1_frame(n: int = 2048) -> np.ndarray:
    """One frame of i.i.d. N(0,1)."""
    return _rng(SEEDS["c1"]).standard_normal(n).astype(np.float32)


def c2_signals(n_signals: int = 256, length: int = 1 << 20, first_signal: int = 0) -> np.ndarray:
    """Uniform[-1,1) white noise, one independent stream per signal index so that a
    shard [first_signal, first_signal+n_signals) equals the same rows of the full set."""
    out = np.empty((n_signals, length), dtype=np.float32)
    for i in range(n_signals):
        g = np.random.Generator(np.random.PCG64([SEEDS["c2"], first_signal + i]))
        out[i] = g.uniform(-1.0, 1.0, length).astype(np.float32)
    return out


def decaying_ir(taps: int, seed, rt60_s: float = 1.5, rate: float = 48000.0) -> np.ndarray:
    """Gaussian noise times exp decay reaching -60 dB at rt60 (factor 1e-3 in
    amplitude: exp(-6.9078 n / (rt60*rate))), scaled to unit energy."""
    g = np.random.Generator(np.random.PCG64(seed))
    n = np.arange(taps, dtype=np.float64)
    h = g.standard_normal(taps) * np.exp(-6.907755278982137 * n / (rt60_s * rate))
    h /= np.sqrt(np.sum(h * h))
    return h.astype(np.float32)


def c3_ir(taps: int = 131072) -> np.ndarray:
    return decaying_ir(taps, SEEDS["c3_ir"])


def c3_input(channels: int = 512, length: int = 1 << 20, first_channel: int = 0) -> np.ndarray:
    """N(0, sigma=0.1) white noise, one independent stream per channel."""
    out = np.empty((channels, length), dtype=np.float32)
    for c in range(channels):
        g = np.random.Generator(np.random.PCG64([SEEDS["c3_x"], first_channel + c]))
        out[c] = (0.1 * g.standard_normal(length)).astype(np.float32)
    return out


def c4_irs(n_irs: int = 512, taps: int = 262144, first_ir: int = 0) -> np.ndarray:
    out = np.empty((n_irs, taps), dtype=np.float32)
    for i in range(n_irs):
        out[i] = decaying_ir(taps, [SEEDS["c4_ir"], first_ir + i])
    return out


def c4_input(channels: int = 1024, length: int = 524288, first_channel: int = 0) -> np.ndarray:
    out = np.empty((channels, length), dtype=np.float32)
    for c in range(channels):
        g = np.random.Generator(np.random.PCG64([SEEDS["c4_x"], first_channel + c]))
        out[c] = (0.1 * g.standard_normal(length)).astype(np.float32)
    return out


def c5_batch(batch: int = 4096, n: int = 65536, first: int = 0) -> np.ndarray:
    out = np.empty((batch, n), dtype=np.float32)
    for i in range(batch):
        g = np.random.Generator(np.random.PCG64([SEEDS["c5"], first + i]))
        out[i] = g.standard_normal(n).astype(np.float32)
    return out
