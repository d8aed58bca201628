"""GPU parity of uniformly partitioned convolution against the float32 port of the
reference's block loop and the float64 linear-convolution oracle."""
import ctypes

import numpy as np
import pytest

from oracle import float64 as o64
from oracle import reference_path as rp
from oracle import configs

pytestmark = pytest.mark.gpu
TOL = 1e-5


def conv(device, block, channels=1):
    from metalaudio_b200 import Convolution
    return Convolution(device, Convolution.Mode.partitioned(blockSize=block), channels=channels)


def test_identity_kernel(device):
    """ConvolutionTests: delta kernel, block 64, 256-sample ramp reproduces the input."""
    c = conv(device, 64)
    c.setKernel(np.array([1.0], np.float32))
    x = np.arange(256, dtype=np.float32) / 256
    y = c.process(x)
    assert y.shape == (256,)
    assert np.max(np.abs(y - x)) < 100 * 1e-6


@pytest.mark.parametrize("block,taps,length", [(64, 1, 256), (64, 64, 640), (64, 200, 1000), (128, 1000, 5000),
                                               (256, 4096, 10000), (512, 3000, 7777), (1, 5, 17), (2, 7, 33),
                                               (4, 9, 40), (16, 100, 333), (1024, 5000, 9000), (4096, 9000, 20000)])
def test_process_matches_port_and_oracle(device, block, taps, length):
    rng = np.random.default_rng(block + taps)
    h = (rng.standard_normal(taps) * np.exp(-np.arange(taps) / max(1, taps / 4))).astype(np.float32)
    x = rng.standard_normal(length).astype(np.float32)
    c = conv(device, block)
    c.setKernel(h)
    assert c.partitionCount == (taps + block - 1) // block
    y = c.process(x)
    assert y.shape == (length + taps - 1,)
    ref = o64.convolve_full(x, h)
    assert o64.rel_rms(y, ref) <= TOL
    port = rp.PartitionedConvolution(block)
    port.set_kernel(h)
    assert o64.rel_rms(y, port.process(x)) <= TOL
    assert c.expectedOutputSize(length) == length + taps - 1 and c.kernelTailLength == taps - 1
    assert c.maxInputSize == 0


def test_consecutive_calls_and_reset(device):
    """The delay line survives across process() calls (Convolution.swift ring semantics), but
    every call pushes ceil((L+K-1)/B) >= ceil(L/B) + P - 1 blocks, so the input-bearing
    spectra have aged out of reach (p <= P-1) by the next call: consecutive calls agree with
    the port and with a fresh convolution.  reset() then same input -> same output, bit-stable."""
    block, taps = 64, 257
    rng = np.random.default_rng(4)
    h = rng.standard_normal(taps).astype(np.float32)
    x1 = rng.standard_normal(128).astype(np.float32)
    x2 = rng.standard_normal(500).astype(np.float32)
    c = conv(device, block)
    c.setKernel(h)
    port = rp.PartitionedConvolution(block)
    port.set_kernel(h)
    a1, p1 = c.process(x1), port.process(x1)
    a2, p2 = c.process(x2), port.process(x2)
    assert o64.rel_rms(a1, p1) <= TOL and o64.rel_rms(a2, p2) <= TOL
    assert o64.rel_rms(a2, o64.convolve_full(x2, h)) <= TOL
    c.reset()
    a3 = c.process(x2)
    assert np.array_equal(a3, a2)
    c.reset()
    assert np.array_equal(c.process(x2), a3)


def test_multichannel_shared_and_per_pair_irs(device):
    block, taps, length, ch = 64, 1000, 3000, 8
    rng = np.random.default_rng(8)
    x = (0.1 * rng.standard_normal((ch, length))).astype(np.float32)
    # shared IR (configuration 3 shape)
    h = configs.decaying_ir(taps, 77, rt60_s=0.01)
    c = conv(device, block, channels=ch)
    c.setKernel(h)
    y = c.process(x)
    for i in range(ch):
        assert o64.rel_rms(y[i], o64.convolve_full(x[i], h)) <= TOL
    # one IR per channel pair (configuration 4 shape)
    hs = np.stack([configs.decaying_ir(taps, [78, i], rt60_s=0.01) for i in range(ch // 2)])
    c2 = conv(device, block, channels=ch)
    c2.setKernel(hs, channelToKernel=[i // 2 for i in range(ch)])
    y2 = c2.process(x)
    for i in range(ch):
        assert o64.rel_rms(y2[i], o64.convolve_full(x[i], hs[i // 2])) <= TOL
    # arbitrary mapping, odd channel count
    c3 = conv(device, block, channels=3)
    c3.setKernel(hs, channelToKernel=[2, 0, 2])
    y3 = c3.process(x[:3])
    for i, ir in enumerate([2, 0, 2]):
        assert o64.rel_rms(y3[i], o64.convolve_full(x[i], hs[ir])) <= TOL


@pytest.mark.parametrize("block,taps,channels", [(64, 1000, 4), (256, 5000, 3), (1, 3, 2), (2, 9, 5), (32, 700, 8), (64, 30, 2),
                                                 (128, 128, 3), (128, 129, 4)])
def test_streaming_step_equals_whole_signal(device, lib, block, taps, channels):
    """The causal one-block step (the HBM-streaming kernel) produces the same samples as
    the whole-signal call."""
    rng = np.random.default_rng(block * 3 + taps)
    h = (rng.standard_normal(taps) / np.sqrt(taps)).astype(np.float32)
    n_blocks = 40
    length = n_blocks * block
    x = rng.standard_normal((channels, length)).astype(np.float32)
    c = conv(device, block, channels=channels)
    c.setKernel(h)
    from metalaudio_b200 import Tensor
    tin = Tensor(device, (channels, length)); tin.copy(x)
    tout = Tensor(device, (channels, length))
    for t in range(n_blocks):
        st = lib.ma_pconv_step_dev(c._h, ctypes.c_void_p(tin.pointer + 4 * t * block), length,
                                   ctypes.c_void_p(tout.pointer + 4 * t * block), length)
        assert st == 0
    device.synchronize()
    y = tout.toArray()
    for i in range(channels):
        ref = o64.convolve_full(x[i], h)[:length]
        assert o64.rel_rms(y[i], ref) <= TOL
    # whole-signal call after reset agrees on the same samples
    c.reset()
    z = c.process(x)
    assert o64.rel_rms(y, z[:, :length]) <= TOL


@pytest.mark.parametrize("splits", [1, 3, 16, 18, 20, 37, 40])
def test_streaming_step_with_forced_partition_splits(device, lib, splits):
    """ma_pconv_step_splits: the step's multiply-accumulate split into 1, 3, 16, 18, 20, 37 or 40 ranges of
    the 100 partitions gives the same samples.  From 16 splits up, consecutive splits form thread-block
    clusters of 8, 4 or 2 CTAs (16 and 40: eight; 20: four; 18: two; 37: none, and then the partial spectra
    go through their own summing kernel) that add their sums up on chip.  Changing the count between steps
    of a running stream is allowed."""
    from metalaudio_b200 import Tensor
    block, taps, channels, n_blocks = 64, 6400, 8, 30
    rng = np.random.default_rng(splits)
    h = (rng.standard_normal(taps) / np.sqrt(taps)).astype(np.float32)
    length = n_blocks * block
    x = rng.standard_normal((channels, length)).astype(np.float32)
    c = conv(device, block, channels=channels)
    c.setKernel(h)
    got = ctypes.c_int32(0)
    assert lib.ma_pconv_step_splits(c._h, 0, ctypes.byref(got)) == 0 and got.value >= 1
    chosen = got.value
    assert lib.ma_pconv_step_splits(c._h, 101, None) != 0 and lib.ma_pconv_step_splits(c._h, 65, None) != 0
    tin = Tensor(device, (channels, length)); tin.copy(x)
    tout = Tensor(device, (channels, length))
    for t in range(n_blocks):
        if t == 10:   # switch in mid-stream
            assert lib.ma_pconv_step_splits(c._h, splits, ctypes.byref(got)) == 0 and got.value == splits
        if t == 20:
            assert lib.ma_pconv_step_splits(c._h, chosen, None) == 0
        assert lib.ma_pconv_step_dev(c._h, ctypes.c_void_p(tin.pointer + 4 * t * block), length,
                                     ctypes.c_void_p(tout.pointer + 4 * t * block), length) == 0
    device.synchronize()
    y = tout.toArray()
    for i in range(channels):
        assert o64.rel_rms(y[i], o64.convolve_full(x[i], h)[:length]) <= TOL


def test_config3_scaled(device):
    """Configuration 3 at reduced channel count / length: one shared exponentially decaying
    noise IR, block 256, float64 oracle plus exact dot-product spot checks."""
    h = configs.c3_ir(16384)
    x = configs.c3_input(channels=8, length=1 << 15)
    c = conv(device, 256, channels=8)
    c.setKernel(h)
    assert c.partitionCount == 64
    y = c.process(x)
    ref = np.stack([o64.convolve_full(x[i], h) for i in range(8)])
    assert o64.rel_rms(y, ref) <= TOL
    idx = np.random.default_rng(0).integers(0, y.shape[1], 200)
    spot = o64.convolve_spot(x[3], h, idx)
    assert np.sqrt(np.mean((y[3, idx] - spot) ** 2)) / np.sqrt(np.mean(ref[3] ** 2)) <= TOL


def test_config4_scaled(device):
    """Configuration 4 at reduced size: block 64, one IR per channel pair, long partition
    count (accumulation over 512 partitions)."""
    irs = configs.c4_irs(n_irs=4, taps=32768)
    x = configs.c4_input(channels=8, length=1 << 14)
    c = conv(device, 64, channels=8)
    c.setKernel(irs, channelToKernel=[i // 2 for i in range(8)])
    assert c.partitionCount == 512
    y = c.process(x)
    ref = np.stack([o64.convolve_full(x[i], irs[i // 2]) for i in range(8)])
    assert o64.rel_rms(y, ref) <= TOL
    assert o64.max_over_rms(y, ref) <= 1e-4


C4_BLOCK, C4_TAPS = 64, 262144          # configuration 4's own block size and tap count: P = 4096


def _c4_case(channels=4, extra_blocks=256):
    """Input long enough that every one of the 4096 partitions meets a non-zero block spectrum:
    4096 + extra_blocks input blocks per channel, two impulse responses for four channels."""
    irs = configs.c4_irs(n_irs=channels // 2, taps=C4_TAPS)
    x = configs.c4_input(channels=channels, length=(C4_TAPS // C4_BLOCK + extra_blocks) * C4_BLOCK)
    ref = np.stack([o64.convolve_full(x[i], irs[i // 2]) for i in range(channels)])
    return irs, x, ref


def test_config4_true_partition_count_whole_signal(device):
    """Configuration 4 at its real partition count (block 64, 262144 taps, 4096 partitions, one
    impulse response per channel pair): the whole-signal call sums 4096 products per output bin in
    float32; against the float64 linear convolution and the float32 port of the reference loop."""
    irs, x, ref = _c4_case()
    c = conv(device, C4_BLOCK, channels=4)
    c.setKernel(irs, channelToKernel=[0, 0, 1, 1])
    assert c.partitionCount == 4096
    y = c.process(x)
    assert y.shape == ref.shape
    assert o64.rel_rms(y, ref) <= TOL
    assert o64.max_over_rms(y, ref) <= 5e-5
    # the steady-state part alone (all 4096 partitions active), where the sums are longest
    lo = C4_TAPS
    assert o64.rel_rms(y[:, lo:lo + 16384], ref[:, lo:lo + 16384]) <= TOL
    # the reference's own float32 block loop on one channel's first 32 blocks past the ramp-up
    port = rp.PartitionedConvolution(C4_BLOCK)
    port.set_kernel(irs[0])
    short = x[0, :(4096 + 32) * C4_BLOCK]
    yp = port.process(short)
    ys = c.process(np.stack([short] * 4))[0]
    assert o64.rel_rms(ys, yp) <= TOL


def test_config4_true_partition_count_streaming(device, lib):
    """The same case through the causal streaming step (every step reads all 4096 delay-line
    spectra of every channel): 4352 steps, compared with the float64 linear convolution."""
    from metalaudio_b200 import Tensor
    irs, x, ref = _c4_case()
    channels, length = x.shape
    c = conv(device, C4_BLOCK, channels=channels)
    c.setKernel(irs, channelToKernel=[0, 0, 1, 1])
    tin = Tensor(device, (channels, length)); tin.copy(x)
    tout = Tensor(device, (channels, length))
    for t in range(length // C4_BLOCK):
        st = lib.ma_pconv_step_dev(c._h, ctypes.c_void_p(tin.pointer + 4 * t * C4_BLOCK), length,
                                   ctypes.c_void_p(tout.pointer + 4 * t * C4_BLOCK), length)
        assert st == 0
    device.synchronize(60)
    y = tout.toArray()
    assert o64.rel_rms(y, ref[:, :length]) <= TOL
    assert o64.max_over_rms(y, ref[:, :length]) <= 5e-5
    assert o64.rel_rms(y[:, C4_TAPS:], ref[:, C4_TAPS:length]) <= TOL


def test_step_after_other_library_work_reads_fresh_input(device, lib):
    """A streaming step whose input block was produced by another kernel of the library queued
    just before it (here a biquad) must see that kernel's output: the step's first kernel is only
    allowed to start early when it directly follows the previous step."""
    from metalaudio_b200 import Tensor
    block, taps, channels, steps = 64, 300, 4, 24
    rng = np.random.default_rng(77)
    h = (rng.standard_normal(taps) / np.sqrt(taps)).astype(np.float32)
    x = rng.standard_normal((channels, steps * block)).astype(np.float32)
    c = conv(device, block, channels=channels)
    c.setKernel(h)
    bq = ctypes.c_void_p()
    assert lib.ma_biquad_create(device.handle, channels, 1, ctypes.byref(bq)) == 0
    gain = np.array([[0.5, 0.0, 0.0, 0.0, 0.0]], np.float32)    # y = 0.5 x, no memory
    assert lib.ma_biquad_set_coefficients(bq, gain.ctypes.data_as(ctypes.c_void_p), 1, None) == 0
    tin = Tensor(device, x.shape); tin.copy(x)
    mid = Tensor(device, (channels, block))
    tout = Tensor(device, x.shape)
    n = steps * block
    for t in range(steps):
        assert lib.ma_biquad_process_dev(bq, ctypes.c_void_p(tin.pointer + 4 * t * block), n,
                                         ctypes.c_void_p(mid.pointer), block, block) == 0
        assert lib.ma_pconv_step_dev(c._h, ctypes.c_void_p(mid.pointer), block,
                                     ctypes.c_void_p(tout.pointer + 4 * t * block), n) == 0
    device.synchronize()
    y = tout.toArray()
    lib.ma_biquad_destroy(bq)
    for i in range(channels):
        assert o64.rel_rms(y[i], 0.5 * o64.convolve_full(x[i], h)[:n]) <= TOL


def test_errors(device):
    from metalaudio_b200 import Convolution, ConvolutionError, MetalAudioError
    c = conv(device, 64)
    with pytest.raises(ConvolutionError) as e:
        c.setKernel(np.zeros(0, np.float32))
    assert e.value.case == "emptyKernel"
    with pytest.raises(ConvolutionError):
        c.process(np.ones(10, np.float32))
    assert c.process(np.zeros(0, np.float32)).size == 0
    with pytest.raises(MetalAudioError):
        Convolution(device, Convolution.Mode.partitioned(blockSize=0)).setKernel(np.ones(4, np.float32))
