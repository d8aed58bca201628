"""The allocation-free forward transform (ma_fft_forward_static_dev).

Some callers may not allocate device memory at the moment they need a transform: an audio
render callback on a deadline (an allocation can stall for milliseconds), or a process whose
device-memory budget was fixed at start-up.  For them the library carries a fixed 8 MiB scratch buffer compiled into it,
and this entry point runs the above-8192-point forward transform through that buffer instead of
through memory allocated for the plan.  Here it is called through the C ABI and compared with
the regular entry point on the same inputs, twice in a row (the buffer is shared and keeps the
previous call's contents, so a second call with other data must still be right), with a batch
that needs several passes through the buffer, and the size limit is checked.

This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest

from oracle import float64 as o64

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _run(lib, fn, plan, x, spec, mag, batch, n):
    from metalaudio_b200 import _lib as L
    st = fn(plan, ctypes.c_void_p(x.pointer), ctypes.c_void_p(spec.pointer), None, ctypes.c_void_p(mag.pointer),
            L.MAG_MAGNITUDE, 1.0, batch, L.LAYOUT_HALF_INTERLEAVED)
    assert st == 0, lib.ma_status_string(st)


def test_static_scratch_forward_matches_regular_entry_point(device, lib):
    from metalaudio_b200 import FFT, Tensor, WindowType
    from metalaudio_b200 import _lib as L
    n, batch = 65536, 70          # 8 MiB / 264192 B = 31 transforms per pass -> three passes
    fft = FFT(device, FFT.Config(size=n, windowType=WindowType.none))
    x = Tensor(device, (batch, n))
    ref_spec = Tensor(device, (batch, n // 2 + 1, 2))
    ref_mag = Tensor(device, (batch, n // 2 + 1))
    new_spec = Tensor(device, (batch, n // 2 + 1, 2))
    new_mag = Tensor(device, (batch, n // 2 + 1))
    rng = np.random.default_rng(2024)
    for call in range(2):         # two calls in a row, different data each time
        host = rng.standard_normal((batch, n)).astype(np.float32) * (1.0 + call)
        x.copy(host)
        new_spec.zero()
        new_mag.zero()
        _run(lib, lib.ma_fft_forward_dev, fft._h, x, ref_spec, ref_mag, batch, n)
        _run(lib, lib.ma_fft_forward_static_dev, fft._h, x, new_spec, new_mag, batch, n)
        device.synchronize(30)
        a, b = ref_spec.toArray(), new_spec.toArray()
        assert o64.rel_rms(b, a) <= TOL
        assert o64.rel_rms(new_mag.toArray(), ref_mag.toArray()) <= TOL
        # and both agree with the float64 oracle on a few rows
        rows = [0, 30, 31, 69]
        want = o64.rfft(host[rows])
        assert o64.rel_rms(b[rows, :, 0] + 1j * b[rows, :, 1], want) <= TOL
    fft.close()


def test_static_scratch_limit_and_small_sizes(device, lib):
    from metalaudio_b200 import FFT, Tensor, WindowType
    from metalaudio_b200 import _lib as L
    # above the limit: one 2^21-point transform needs about 8.4 MB of intermediate data
    big = FFT(device, FFT.Config(size=1 << 21, windowType=WindowType.none))
    x = Tensor(device, (1, 1 << 21))
    out = Tensor(device, (1, (1 << 20) + 1, 2))
    st = lib.ma_fft_forward_static_dev(big._h, ctypes.c_void_p(x.pointer), ctypes.c_void_p(out.pointer), None, None,
                                       0, 1.0, 1, L.LAYOUT_HALF_INTERLEAVED)
    assert st == L.MA_ERR_SCRATCH_LIMIT
    assert b"static buffer" in lib.ma_status_string(st)
    big.close()
    # 2^20 points is the largest size served
    edge = FFT(device, FFT.Config(size=1 << 20, windowType=WindowType.none))
    host = np.random.default_rng(5).standard_normal((2, 1 << 20)).astype(np.float32)
    x2 = Tensor(device, (2, 1 << 20)); x2.copy(host)
    o2 = Tensor(device, (2, (1 << 19) + 1, 2))
    st = lib.ma_fft_forward_static_dev(edge._h, ctypes.c_void_p(x2.pointer), ctypes.c_void_p(o2.pointer), None, None,
                                       0, 1.0, 2, L.LAYOUT_HALF_INTERLEAVED)
    assert st == 0
    device.synchronize(30)
    got = o2.toArray()
    assert o64.rel_rms(got[..., 0] + 1j * got[..., 1], o64.rfft(host)) <= TOL
    edge.close()
    # plans that need no scratch are forwarded to the regular entry point
    small = FFT(device, FFT.Config(size=1024, windowType=WindowType.none))
    h3 = np.random.default_rng(6).standard_normal((3, 1024)).astype(np.float32)
    x3 = Tensor(device, (3, 1024)); x3.copy(h3)
    o3 = Tensor(device, (3, 513, 2))
    st = lib.ma_fft_forward_static_dev(small._h, ctypes.c_void_p(x3.pointer), ctypes.c_void_p(o3.pointer), None, None,
                                       0, 1.0, 3, L.LAYOUT_HALF_INTERLEAVED)
    assert st == 0
    device.synchronize(30)
    g3 = o3.toArray()
    assert o64.rel_rms(g3[..., 0] + 1j * g3[..., 1], o64.rfft(h3)) <= TOL
    small.close()
