"""CPU execution of the CUDA kernel bodies (FFT stages, Hermitian pre/post-process, window,
overlap-add) through a thread-per-lane emulator: the same templated code the kernels
instantiate, compiled for the host.  Checks the index arithmetic where no GPU exists."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kernel_emulation", "emulate_fft.cu")
OUT = os.path.join(HERE, "kernel_emulation", "libemulate_fft.so")
LL = ctypes.c_longlong
FP = ctypes.POINTER(ctypes.c_float)


def fp(a):
    return None if a is None else a.ctypes.data_as(FP)


@pytest.fixture(scope="module")
def emul():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    deps = [SRC, os.path.join(HERE, "kernel_emulation", "host_cta.h"),
            os.path.join(HERE, "..", "metalaudio_b200", "csrc", "fft_core.cuh"),
            os.path.join(HERE, "..", "metalaudio_b200", "csrc", "fft_kernels.cuh"),
            os.path.join(HERE, "..", "metalaudio_b200", "csrc", "pconv_tiling.h")]
    if not os.path.exists(OUT) or any(os.path.getmtime(d) > os.path.getmtime(OUT) for d in deps):
        subprocess.run([nvcc, "-std=c++17", "-O1", "-shared", "-Xcompiler", "-fPIC", "-diag-suppress", "20011,20014",
                        "-Wno-deprecated-gpu-targets", "-o", OUT, SRC, "-lpthread"], check=True)
    lib = ctypes.CDLL(OUT)
    lib.emul_r2c.argtypes = [ctypes.c_int, ctypes.c_int, FP, LL, LL, LL, LL, ctypes.c_int, ctypes.c_int, FP, FP, FP,
                             FP, LL, LL, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int]
    lib.emul_c2r.argtypes = [ctypes.c_int, FP, FP, LL, LL, LL, LL, ctypes.c_int, FP, ctypes.c_int]
    lib.emul_istft.argtypes = [ctypes.c_int, ctypes.c_int, FP, FP, LL, LL, LL, LL, ctypes.c_int, FP, ctypes.c_float,
                               FP, LL, LL, ctypes.c_int, ctypes.c_int]
    lib.emul_tiled_rows.argtypes = [ctypes.c_int, LL, ctypes.POINTER(LL)]
    lib.emul_tiled_rows.restype = LL
    return lib


@pytest.mark.parametrize("n", [2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192])
def test_forward_and_inverse_all_layouts(emul, n):
    m = n // 2
    batch = 3
    rng = np.random.default_rng(n)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    out = np.zeros((batch, m + 1, 2), np.float32)
    mag = np.zeros((batch, m + 1), np.float32)
    assert emul.emul_r2c(n, 1, fp(x), n, batch, batch, batch * n, n, n, None, fp(out), None, fp(mag),
                         batch * (m + 1), m + 1, 0, 0, 1.0, 2) == 0
    ref = o64.rfft(x)
    assert o64.rel_rms(out[..., 0] + 1j * out[..., 1], ref) <= 1e-6
    assert o64.rel_rms(mag, np.abs(ref)) <= 1e-6
    re = np.zeros((batch, n), np.float32)
    im = np.zeros((batch, n), np.float32)
    assert emul.emul_r2c(n, 0, fp(x), n, batch, batch, batch * n, n, n, None, fp(re), fp(im), None, 0, 0, 1, -1,
                         1.0, 1) == 0
    assert o64.rel_rms(re + 1j * im, o64.fft_forward(x)) <= 1e-6
    pk = np.zeros((batch, m, 2), np.float32)
    assert emul.emul_r2c(n, 1, fp(x), n, batch, batch, batch * n, n, n, None, fp(pk), None, None, batch * m, m, 2,
                         -1, 1.0, 2) == 0
    assert np.allclose(pk[:, 0, 0], ref[:, 0].real, atol=1e-3) and np.allclose(pk[:, 0, 1], ref[:, m].real, atol=1e-3)
    for layout, a, b, ss, fs in ((0, out, None, batch * (m + 1), m + 1), (1, re, im, 0, 0), (2, pk, None, batch * m, m)):
        y = np.zeros((batch, n), np.float32)
        assert emul.emul_c2r(n, fp(a), fp(b), ss, fs, batch, 1, layout, fp(y), 2) == 0
        assert o64.rel_rms(y, x) <= 1e-6


def test_zero_padded_frames(emul):
    """Loader guards: samples past frame_valid / signal_len read as zero (the convolution's
    zero-padded input blocks and partition blocks)."""
    n, b = 128, 64
    rng = np.random.default_rng(0)
    taps = rng.standard_normal(150).astype(np.float32)   # 3 partitions, the last one ragged
    out = np.zeros((3, n // 2, 2), np.float32)
    assert emul.emul_r2c(n, 0, fp(taps), 0, 3, 3, 150, b, b, None, fp(out), None, None, 0, n // 2, 2, -1, 1.0, 1) == 0
    blocks = np.zeros((3, n)); padded = np.zeros(192); padded[:150] = taps
    blocks[:, :b] = padded.reshape(3, b)
    ref = np.fft.rfft(blocks, axis=-1)
    assert o64.rel_rms(out[:, 1:, 0] + 1j * out[:, 1:, 1], ref[:, 1:n // 2]) <= 1e-6


@pytest.mark.parametrize("n,hop,length,chunks,kind", [(256, 64, 3000, 1, "hann"), (256, 64, 3000, 3, "hann"),
                                                      (512, 100, 4000, 2, "hamming"), (64, 7, 500, 4, "blackman"),
                                                      (1024, 1024, 8192, 2, "none"), (8, 2, 50, 2, "hann"),
                                                      (4, 1, 20, 1, "hann"), (2, 1, 9, 2, "none"),
                                                      (4096, 1024, 30000, 2, "hann"), (4096, 256, 12000, 1, "hann"),
                                                      (2048, 1024, 9000, 3, "hamming"), (64, 8, 300, 1, "hann")])
def test_stft_istft(emul, n, hop, length, chunks, kind):
    m = n // 2
    w = rp.window(kind, n)
    x = np.random.default_rng(n + hop).uniform(-1, 1, (2, length)).astype(np.float32)
    f = (length - n) // hop + 1
    spec = np.zeros((2, f, m + 1, 2), np.float32)
    aligned = int(hop % 2 == 0 and length % 2 == 0)
    assert emul.emul_r2c(n, aligned, fp(x), length, f, 2 * f, length, hop, n, fp(w), fp(spec), None, None,
                         f * (m + 1), m + 1, 0, -1, 1.0, 3) == 0
    ref = o64.stft(x, n, hop, w)
    assert o64.rel_rms(spec[..., 0] + 1j * spec[..., 1], ref) <= 1e-6
    out_len = (f - 1) * hop + n
    y = np.zeros((2, out_len), np.float32)
    floor = float(rp.window_floor())
    rc = emul.emul_istft(n, hop, fp(spec), None, f * (m + 1), m + 1, f, 2, 0, fp(w), floor, fp(y), out_len,
                         out_len, chunks, 3)
    assert rc in (0, 1)  # 1: the prefetching thread-private overlap-add variant served it
    yref = o64.istft(ref, n, hop, w, floor)
    ws = rp.window_sum(f, n, hop, w, 0.0)
    msk = ws >= 1e-2 * ws.max()
    assert o64.rel_rms(y[:, msk], yref[:, msk]) <= 1e-5


@pytest.mark.parametrize("partitions", [1, 4, 5, 8, 15, 16, 17, 20, 24, 31, 32, 33, 64, 100, 512])
@pytest.mark.parametrize("blocks", [1, 3, 63, 64, 65, 200])
def test_tiled_multiply_accumulate_row_schedule(emul, partitions, blocks):
    """The whole-signal multiply-accumulate stages timeline rows a chunk of 16 partitions ahead.
    For partition counts that are not multiples of 16 (and below 16) the staged range reaches
    before the first timeline row: every fetch must stay inside the channel's timeline, and every
    row that feeds a stored output must be the genuine one."""
    counts = (LL * 2)()
    assert emul.emul_tiled_rows(partitions, blocks, counts) == 0, (counts[0], counts[1])
