"""The benchmark configurations at their full sizes, checked through properties that need no CPU
oracle pass over gigabytes: reconstruction, linearity, Parseval, impulse responses.  Checking
arithmetic runs in torch on the device; the transforms under test go through the C ABI."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def rel(a, b):
    return float((a - b).double().pow(2).mean().sqrt() / b.double().pow(2).mean().sqrt())


def test_config2_full_size_round_trip_and_linearity(device, lib):
    """256 signals x 2^20 samples, n_fft 4096, hop 1024, periodic Hann: iSTFT(STFT(x)) = x away from
    the ends, the transform is linear, and magnitudes match the spectrum."""
    import torch
    from metalaudio_b200 import FFT, WindowType
    S, L, n, hop = 256, 1 << 20, 4096, 1024
    frames, kh = (L - n) // hop + 1, n // 2 + 1
    k = np.arange(n, dtype=np.float64)
    window = (0.5 * (1.0 - np.cos(2.0 * np.pi * k / n))).astype(np.float32)
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop), window=window)
    g = torch.Generator(device="cuda"); g.manual_seed(1002)
    x = torch.rand((S, L), device="cuda", generator=g) * 2 - 1
    spec = torch.empty((S, frames, kh, 2), device="cuda")
    mag = torch.empty((S, frames, kh), device="cuda")
    y = torch.empty((S, L), device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_stft_dev(fft._h, ptr(x), L, L, S, ptr(spec), None, ptr(mag), 0, 1.0, 0) == 0
    assert lib.ma_istft_dev(fft._h, ptr(spec), None, frames, S, ptr(y), L, 1e-8, 0) == 0
    device.synchronize(30)
    torch.cuda.synchronize()
    assert rel(y[:, n:L - n], x[:, n:L - n]) < 1e-5
    assert rel(mag[::17], spec[::17].pow(2).sum(-1).sqrt()) < 1e-6
    # Parseval per frame on a subset: sum |X_k|^2 over the full spectrum = N * sum (w x)^2
    sub = spec[:4].double()
    e_spec = 2 * sub.pow(2).sum(-1).sum(-1) - sub[..., 0, :].pow(2).sum(-1) - sub[..., -1, :].pow(2).sum(-1)
    fr = x[:4].unfold(1, n, hop).double() * torch.from_numpy(window).cuda().double()
    assert rel(e_spec, n * fr.pow(2).sum(-1)) < 1e-5
    # linearity on 8 signals: STFT(2.5 a - b) = 2.5 STFT(a) - STFT(b)
    a, b = x[:8], x[8:16]
    z = (2.5 * a - b).contiguous()
    sz = torch.empty((8, frames, kh, 2), device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_stft_dev(fft._h, ptr(z), L, L, 8, ptr(sz), None, None, 0, 1.0, 0) == 0
    device.synchronize(30)
    torch.cuda.synchronize()
    assert rel(sz, 2.5 * spec[:8] - spec[8:16]) < 1e-5


def test_config5_full_size_round_trip_and_parseval(device, lib):
    """4096 transforms of 65536 points: inverse(forward(x)) = x, Parseval, and agreement of a subset
    with torch's float64 FFT."""
    import torch
    from metalaudio_b200 import FFT, WindowType
    n, batch = 65536, 4096
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.none))
    g = torch.Generator(device="cuda"); g.manual_seed(1005)
    x = torch.randn((batch, n), device="cuda", generator=g)
    spec = torch.empty((batch, n // 2 + 1, 2), device="cuda")
    y = torch.empty_like(x)
    torch.cuda.synchronize()
    assert lib.ma_fft_forward_dev(fft._h, ptr(x), ptr(spec), None, None, 0, 1.0, batch, 0) == 0
    assert lib.ma_fft_inverse_dev(fft._h, ptr(spec), None, ptr(y), batch, 0) == 0
    device.synchronize(30)
    torch.cuda.synchronize()
    assert rel(y, x) < 1e-5
    s = spec.double()
    energy = 2 * s.pow(2).sum(-1).sum(-1) - s[:, 0].pow(2).sum(-1) - s[:, -1].pow(2).sum(-1)
    assert rel(energy, n * x.double().pow(2).sum(-1)) < 1e-5
    pick = [0, 1, 189, 190, 759, 760, 761, batch - 1]          # both sides of chunk boundaries
    ref = torch.view_as_real(torch.fft.rfft(x[pick].double(), dim=-1))
    assert rel(spec[pick], ref) < 1e-5


def test_config3_full_size_impulses(device, lib):
    """512 channels sharing a 131072-tap response, block 256, 2^20 samples each: a unit impulse at a
    different position in every channel returns the response at that offset and nothing else; the
    call is linear."""
    import torch
    from metalaudio_b200 import Convolution
    C, B, taps, L = 512, 256, 131072, 1 << 20
    rng = np.random.default_rng(1003)
    h = rng.standard_normal(taps) * np.exp(-6.907755278982137 * np.arange(taps) / 72000.0)
    h = (h / np.sqrt(np.sum(h * h))).astype(np.float32)
    conv = Convolution(device, Convolution.Mode.partitioned(blockSize=B), channels=C)
    conv.setKernel(h)
    assert lib.ma_pconv_reserve(conv._h, L) == 0
    full = L + taps - 1
    pos = torch.from_numpy(rng.integers(0, L, C)).cuda()
    amp = torch.from_numpy(rng.uniform(0.5, 2.0, C).astype(np.float32)).cuda()
    x = torch.zeros((C, L), device="cuda")
    x[torch.arange(C, device="cuda"), pos] = amp
    y = torch.empty((C, full), device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_pconv_process_dev(conv._h, ptr(x), L, L, ptr(y), full) == 0
    device.synchronize(60)
    torch.cuda.synchronize()
    hd = torch.from_numpy(h).cuda()
    idx = pos[:, None] + torch.arange(taps, device="cuda")[None, :]
    got = torch.gather(y, 1, idx)
    want = amp[:, None] * hd[None, :]
    assert rel(got, want) < 1e-5
    # everything outside [pos, pos + taps) is numerically nothing
    outside = y.clone()
    outside.scatter_(1, idx, 0.0)
    assert float(outside.abs().max()) < 1e-6 * float(want.abs().max()) * 50
    conv.close()


def test_config4_full_size_impulses_and_dense_subset(device, lib):
    """Configuration 4 at full size: 1024 channels, block 64, 512 impulse responses of 262144 taps
    (one per channel pair, 4096 partitions), 2^19 samples per channel.  A unit impulse at a
    different position in most channels returns that pair's response at that offset; eight
    channels carry dense noise and are compared with torch's float64 FFT convolution."""
    import torch
    from metalaudio_b200 import Convolution
    C, B, taps, L = 1024, 64, 262144, 1 << 19
    n_irs = C // 2
    g = torch.Generator(device="cuda"); g.manual_seed(1004)
    decay = torch.exp(-6.907755278982137 * torch.arange(taps, device="cuda", dtype=torch.float64) / 72000.0)
    irs = torch.randn((n_irs, taps), device="cuda", generator=g, dtype=torch.float64) * decay
    irs = (irs / irs.pow(2).sum(-1, keepdim=True).sqrt()).float()
    conv = Convolution(device, Convolution.Mode.partitioned(blockSize=B), channels=C)
    conv.setKernel(irs.cpu().numpy(), channelToKernel=[c // 2 for c in range(C)])
    assert conv.partitionCount == 4096
    assert lib.ma_pconv_reserve(conv._h, L) == 0
    full = L + taps - 1
    rng = np.random.default_rng(1014)
    pos = torch.from_numpy(rng.integers(0, L, C)).cuda()
    amp = torch.from_numpy(rng.uniform(0.5, 2.0, C).astype(np.float32)).cuda()
    x = torch.zeros((C, L), device="cuda")
    x[torch.arange(C, device="cuda"), pos] = amp
    dense = [0, 1, 510, 511, 512, 513, 1022, 1023]
    x[dense] = 0.1 * torch.randn((len(dense), L), device="cuda", generator=g)
    y = torch.empty((C, full), device="cuda")
    torch.cuda.synchronize()
    assert lib.ma_pconv_process_dev(conv._h, ptr(x), L, L, ptr(y), full) == 0
    device.synchronize(120)
    torch.cuda.synchronize()
    sparse = torch.tensor([c for c in range(C) if c not in dense], device="cuda")
    for lo in range(0, sparse.numel(), 128):          # gather in slices: bounded temporary memory
        ch = sparse[lo:lo + 128]
        idx = pos[ch][:, None] + torch.arange(taps, device="cuda")[None, :]
        got = torch.gather(y[ch], 1, idx)
        want = amp[ch][:, None] * irs[ch // 2]
        assert rel(got, want) < 1e-5
        outside = y[ch].clone()
        outside.scatter_(1, idx, 0.0)
        assert float(outside.abs().max()) < 1e-6 * float(want.abs().max()) * 50
    nfft = 1 << 20
    for c in dense:
        X = torch.fft.rfft(x[c].double(), n=nfft)
        H = torch.fft.rfft(irs[c // 2].double(), n=nfft)
        ref = torch.fft.irfft(X * H, n=nfft)[:full]
        assert rel(y[c], ref) < 1e-5
    conv.close()
