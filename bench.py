#!/usr/bin/env python
"""Benchmark of the MetalDSP hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the hot path over one batch of synthetic input: the batched
STFT + iSTFT configuration (256 mono signals of 2^20 uniform[-1,1) samples per GPU,
n_fft 4096, hop 1024, periodic Hann; half-spectrum complex + magnitude out, COLA
overlap-add reconstruction back).  Metric: STFT frames/s, whole job over all GPUs, with the
signals already resident in HBM.  Under torchrun every rank runs its own 256 independent signals
(no collective on the data path; weak scaling), the timed region is bracketed by barrier + device
synchronisation and the maximum over ranks is reported.

The JSON line also carries
  roofline      the dominant kernel's achieved HBM GB/s (algorithmic bytes / CUDA-event time)
                against the measured copy bandwidth of this pool's B200s,
  kernels       the same for every kernel of the step,
  e2e           the same metric through the public Tensor API with pinned host buffers,
                host->device and device->host copies inside the timed region; beside it the
                copy-only time of the same transfers (what the box's host links allow) and the
                figure through the host-buffer entry points ma_stft_host / ma_istft_host, which
                bring the spectra back to the host as the reference's stft() does,
  strong        the FIXED workloads split over the ranks (256 signals; 512 convolution channels;
                1024 low-latency channels by impulse-response pair): time = maximum over ranks,
  cpu_baseline  the float32 CPU port of the reference path timed on the host cores (N=1 only),
  conv, conv_low_latency, large_fft (N=1)
                the partitioned-convolution configurations as streaming steps and as whole-signal
                calls, and the 65536-point batch, each with its own roofline fraction, CPU
                baseline (one thread and all cores) and end-to-end figure from host buffers,
  next_rows     polar STFT / iSTFT, one-shot FFT convolution, biquad cascades.

`--impl reference` times the CPU port of the reference path (the reference itself is Swift +
Apple Accelerate and cannot run here) on all host cores over the same 256 signals per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_FFT, HOP = 4096, 1024
SIGNALS_PER_GPU, SIGNAL_LEN = 256, 1 << 20
FRAMES = (SIGNAL_LEN - N_FFT) // HOP + 1
KH = N_FFT // 2 + 1
STFT_BYTES_PER_SIGNAL = SIGNAL_LEN * 4 + FRAMES * (KH * 8 + KH * 4)   # read signal once, write complex + magnitude
ISTFT_BYTES_PER_SIGNAL = FRAMES * KH * 8 + SIGNAL_LEN * 4             # read complex, write signal
CONV3 = dict(name="conv", channels=512, block=256, taps=131072, length=1 << 20, group=1, steps=200, warm=16)
CONV4 = dict(name="conv_low_latency", channels=1024, block=64, taps=262144, length=1 << 19, group=2, steps=40, warm=8)
LARGE = dict(n=65536, batch=4096)
DECAY = 6.907755278982137 / (1.5 * 48000.0)     # -60 dB after 1.5 s at 48 kHz


def periodic_hann(n: int) -> np.ndarray:
    """0.5(1 - cos(2 pi k/n)), computed in float64: the window the benchmark configuration names."""
    k = np.arange(n, dtype=np.float64)
    return (0.5 * (1.0 - np.cos(2.0 * np.pi * k / float(n)))).astype(np.float32)


def decaying_irs(n_irs: int, taps: int, seed: int, first: int = 0) -> np.ndarray:
    """Synthetic room responses: Gaussian noise with an exponential decay reaching -60 dB after
    1.5 s at 48 kHz, each scaled to unit energy; response i is seeded by (seed, first + i) so a
    rank's shard equals the same rows of the whole set."""
    decay = np.exp(-DECAY * np.arange(taps, dtype=np.float64)).astype(np.float32)
    out = np.empty((n_irs, taps), dtype=np.float32)
    for i in range(n_irs):
        g = np.random.Generator(np.random.PCG64([seed, first + i]))
        h = g.standard_normal(taps, dtype=np.float32) * decay
        out[i] = h / np.float32(np.sqrt(np.sum(h.astype(np.float64) ** 2)))
    return out


def conv_bytes_per_channel_block(block: int, partitions: int, sharing: int) -> float:
    """Algorithmic HBM bytes of one streaming step per channel: block in, block out, the new
    spectrum, the whole delay line, and the impulse-response spectra divided by the channels that
    share them on this GPU."""
    return 4 * block + 4 * block + 8 * (block + 1) * (1 + partitions + partitions / sharing)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_traffic_per_signal():
    """DRAM bytes per signal of the two headline kernels from their profiler capture: lines
    `kernel_name read_bytes write_bytes signals` in a text file kept beside the capture's summary.
    Missing file or kernel: no traffic figure."""
    out = {}
    try:
        with open(os.path.join(ROOT, "profiles", "stft_istft_n4096_hop1024.traffic.txt")) as f:
            for ln in f:
                if ln.startswith("#") or not ln.strip():
                    continue
                name, rd, wr, sig = ln.split()
                out[name] = (float(rd) + float(wr)) / float(sig)
    except Exception:
        pass
    return out


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        # The thread is started ahead of the timed region (NVML's first queries take tens of
        # milliseconds) and keeps only what it reads while `recording` is set.
        self.recording = False
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                if self.recording:
                    self.samples.append(mhz)
                    for bit, name in names.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def bind_to_gpu_cpus(index: int):
    """Runs this process on the CPUs NVML lists as local to the GPU (read-only query), so that the
    pinned host buffers allocated afterwards are first touched on the GPU's own NUMA node.  Returns
    (previous affinity, number of CPUs now allowed); changes nothing when the query fails or the
    local set does not intersect the CPUs this process may use."""
    before = os.sched_getaffinity(0)
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (max(before) // 64) + 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        local = {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        want = local & before
        if want:
            os.sched_setaffinity(0, want)
            return before, len(want)
    except Exception:
        pass
    return before, len(before)


# ----------------------------------------------------------------------------- CPU arm

def cpu_port_stft_istft(signals: np.ndarray, window: np.ndarray, cores: int) -> float:
    """Runs the float32 port of the reference path (STFT.swift:40-81 then :384-527) over
    `signals` with a pool of `cores` threads, one signal per task; returns seconds."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import reference_path as rp

    def one(x):
        re, im = rp.stft(x, N_FFT, HOP, window)
        kh = N_FFT // 2 + 1
        mag = np.sqrt(re[:, :kh] ** 2 + im[:, :kh] ** 2)
        y = rp.istft(re, im, N_FFT, HOP, window)
        return float(y[0]) + float(mag[0, 0])

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=cores) as ex:
        list(ex.map(one, list(signals)))
    return time.perf_counter() - t0


def run_reference(args, rank: int, world: int):
    """`--impl reference`: the CPU port on all host cores over the configuration's own 256 signals
    per step; rank 0 only."""
    if rank != 0:
        return
    from oracle import configs
    cores = len(os.sched_getaffinity(0)) or 1
    x = configs.c2_signals(n_signals=SIGNALS_PER_GPU, length=SIGNAL_LEN)
    w = periodic_hann(N_FFT)
    for _ in range(min(args.warmup, 1)):            # one pass over a core's worth of signals warms pocketfft's plans
        cpu_port_stft_istft(x[:cores], w, cores)
    times = [cpu_port_stft_istft(x, w, cores) for _ in range(args.steps)]
    total = float(np.sum(times))
    frames = SIGNALS_PER_GPU * FRAMES * args.steps
    value = frames / total
    line = {
        "impl": "reference", "metric": "stft_istft_frames_per_s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": f"all {SIGNALS_PER_GPU} signals x 2^20 samples per step ({SIGNALS_PER_GPU * FRAMES} "
                                   f"frames) on one host, float32 scipy.fft + numpy port of the reference's "
                                   f"stft/istft, {cores} threads; the host does not grow with --gpus, so the rate "
                                   "is the same at every N"},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, signals: int = SIGNALS_PER_GPU):
    return {"workload": f"batched STFT+iSTFT: {signals} mono fp32 signals x 2^20 samples per GPU, uniform[-1,1), "
                        "n_fft=4096, hop=1024, periodic Hann, half-spectrum complex + magnitude out, "
                        "COLA overlap-add reconstruction",
            "signals_per_gpu": signals, "signal_len": SIGNAL_LEN, "n_fft": N_FFT, "hop": HOP,
            "frames_per_gpu": signals * FRAMES, "window": "periodic_hann",
            "sharding": f"independent signals per rank, no collective ({n_gpus} ranks)",
            "cache": "inputs (1.07 GB) and outputs (6.4 GB) per step exceed the 126 MB L2; no flush needed"}


def _port_seconds_per_block(block: int, taps: int, blocks: int, seed: int) -> float:
    """Seconds per block of the float32 port of the reference's block loop over `blocks` blocks of
    one channel (also run as `bench.py --port-worker ...` in child processes)."""
    from oracle import reference_path as rp
    h = decaying_irs(1, taps, 1003)[0]
    x = (0.1 * np.random.default_rng(seed).standard_normal(blocks * block)).astype(np.float32)
    port = rp.PartitionedConvolution(block)
    port.set_kernel(h)
    port.kernel = h[:1]                      # process() then pushes exactly the sampled blocks
    t0 = time.perf_counter()
    port.process(x)
    return (time.perf_counter() - t0) / blocks


def cpu_conv_baseline(cfg, cores: int):
    """CPU arm of a partitioned-convolution configuration: (1) the float32 port of the reference's
    block loop (Convolution.swift:529-758) timed over a run of blocks of ONE channel - every block
    costs the same P multiply-accumulates, so the whole call is blocks x that, an extrapolation;
    then the same with one channel per core at once, in separate processes as the reference's
    one-object-per-thread use would run; (2) scipy.signal.oaconvolve (float32) as the best library
    routine available here, one thread and all cores."""
    import subprocess
    from concurrent.futures import ThreadPoolExecutor
    import scipy.signal as ssig
    B, taps, L = cfg["block"], cfg["taps"], cfg["length"]
    P = taps // B
    h = decaying_irs(1, taps, 1003)[0]
    total_blocks = (L + taps - 1 + B - 1) // B
    sample_blocks = 2048 if P <= 1024 else 1024
    one = _port_seconds_per_block(B, taps, sample_blocks, 1)
    # one channel per core at once: plain child processes of this script (no CUDA in them), started
    # together; each prints its own seconds per block
    env = dict(os.environ, OMP_NUM_THREADS="1", OPENBLAS_NUM_THREADS="1", MKL_NUM_THREADS="1")
    kids = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--port-worker", str(B), str(taps),
                              str(sample_blocks), str(10 + i)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                             env=env, text=True) for i in range(cores)]
    per = []
    for k in kids:
        try:
            txt, _ = k.communicate(timeout=180)
            per.append(float(txt.strip().splitlines()[-1]))
        except Exception:
            k.kill()
    if not per:
        per = [one * cores]                                  # children unavailable: no better than one thread
    per_block_all = max(per) / len(per)                      # seconds per channel-block with every core busy
    xs = (0.1 * np.random.default_rng(2).standard_normal((cores, L))).astype(np.float32)
    t0 = time.perf_counter()
    ssig.oaconvolve(xs[0], h)
    oa_one = time.perf_counter() - t0
    with ThreadPoolExecutor(max_workers=cores) as ex:
        t0 = time.perf_counter()
        list(ex.map(lambda r: ssig.oaconvolve(r, h)[0], list(xs)))
        oa_all = (time.perf_counter() - t0) / cores
    return {"unit": "channel-samples/s", "kind": "port", "cores": cores,
            "value": L / (total_blocks * per_block_all),
            "port_one_thread": L / (total_blocks * one), "port_all_cores": L / (total_blocks * per_block_all),
            "oaconvolve_one_thread": L / oa_one, "oaconvolve_all_cores": L / oa_all,
            "sample": f"port: {sample_blocks} blocks of one channel per core, scaled to the call's {total_blocks} "
                      f"blocks per channel (an extrapolation: every block costs the same {P} partition products); "
                      f"scipy.signal.oaconvolve: whole 2^{int(np.log2(L))}-sample channels, one per thread; "
                      "rates are input channel-samples/s of the whole-signal call"}


def cpu_large_baseline(cores: int):
    """65536-point forward + inverse pairs in float32 with scipy.fft (pocketfft), one thread and
    all cores, on 256 of the 4096 transforms."""
    import scipy.fft as sfft
    n, sub = LARGE["n"], 256
    x = np.random.default_rng(1005).standard_normal((sub, n)).astype(np.float32)
    res = {}
    for label, workers in (("one_thread", 1), ("all_cores", cores)):
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            z = sfft.rfft(x, axis=-1, workers=workers)
            sfft.irfft(z, n=n, axis=-1, workers=workers)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        res[label] = sub / best
    return {"unit": "pairs/s", "kind": "port", "cores": cores, "value": res["all_cores"],
            "scipy_fft_one_thread": res["one_thread"], "scipy_fft_all_cores": res["all_cores"],
            "sample": f"{sub} of the {LARGE['batch']} transforms, scipy.fft.rfft + irfft in float32, best of 3"}


# ----------------------------------------------------------------------------- GPU arm

class Rig:
    """What every measurement needs: the device context, its stream as a torch stream, the
    process group (if any) and helpers for event timing with the maximum over ranks."""

    def __init__(self, local_rank: int, rank: int, world: int):
        import torch
        from metalaudio_b200 import AudioDevice
        self.torch = torch
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.dist = None
        if world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            self.dist = dist
        self.dev = AudioDevice(local_rank)
        self.lib = self.dev._lib
        self.device = torch.device("cuda", local_rank)
        self.stream = torch.cuda.ExternalStream(self.lib.ma_context_stream(self.dev.handle), device=self.device)
        self.peak, self.peak_kind = measured_peak_gbs()

    def barrier(self):
        self.dev.synchronize(600)
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()

    def max_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = self.torch.tensor(list(values), device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def timed(self, fn, reps: int, warm: int = 1):
        """Milliseconds per call of fn (which queues work on the context's stream), CUDA events on
        that stream, after `warm` untimed calls; barrier on both sides, maximum over ranks."""
        torch = self.torch
        for _ in range(warm):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(reps):
            fn()
        e1.record(self.stream)
        self.dev.synchronize(600)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if self.dist is not None:
            self.dist.barrier()
        return self.max_ranks([ms])[0]

    def pinned(self, shape):
        """float32 torch tensor over pinned host memory from the library's own allocator."""
        torch = self.torch
        n = int(np.prod(shape))
        p = ctypes.c_void_p()
        st = self.lib.ma_host_alloc(self.dev.handle, 4 * n, ctypes.byref(p))
        if st != 0:
            raise RuntimeError(f"ma_host_alloc failed: {st}")
        arr = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_float)), shape=(n,)).reshape(shape)
        t = torch.from_numpy(arr)
        t._ma_ptr = p
        return t

    def unpin(self, t):
        self.lib.ma_host_free(self.dev.handle, t._ma_ptr)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch
    from metalaudio_b200 import AudioDevice, FFT, Tensor, WindowType
    from metalaudio_b200.sharding import shard_range

    affinity_before, cpus_bound = bind_to_gpu_cpus(local_rank)
    rig = Rig(local_rank, rank, world)
    dev, lib, stream, peak = rig.dev, rig.lib, rig.stream, rig.peak

    window = periodic_hann(N_FFT)
    fft = FFT(dev, FFT.Config(size=N_FFT, windowType=WindowType.hann, hopSize=HOP), window=window)
    S = args.signals
    sig = Tensor(dev, (S, SIGNAL_LEN))
    spec = Tensor(dev, (S, FRAMES, KH, 2))
    mag = Tensor(dev, (S, FRAMES, KH))
    rec = Tensor(dev, (S, SIGNAL_LEN))

    # Synthetic input: uniform[-1,1), seeded per rank, generated into pinned host memory (the e2e
    # legs copy it from there every step).
    host_in = rig.pinned((S, SIGNAL_LEN))
    host_out = rig.pinned((S, SIGNAL_LEN))
    host_in.uniform_(-1.0, 1.0, generator=torch.Generator().manual_seed(1002 + rank))
    host_out.zero_()
    sig.copyAsync(host_in.data_ptr(), sig.byteSize)
    dev.synchronize(60)

    def step():
        fft.stftTensor(sig, spec, mag)
        fft.istftTensor(spec, rec)

    warmup = max(args.warmup, 3) if S == SIGNALS_PER_GPU else max(args.warmup, 1)
    sampler = ClockSampler(local_rank)   # started here so that NVML is warm when the timed region opens
    sampler.start()
    for _ in range(warmup):
        step()
    rig.barrier()

    # ---- timed region: EXACTLY K steps between two CUDA events on the launching stream, barrier +
    # device synchronisation on both sides; clocks sampled while it runs
    K = args.steps
    sampler.recording = True
    launches0 = lib.ma_kernel_launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    t0.record(stream)
    for k in range(K):
        step()
    t1.record(stream)
    dev.synchronize(600)
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    launches = int(lib.ma_kernel_launch_count() - launches0)
    sampler.recording = False
    clocks = sampler.stop()
    if rig.dist is not None:
        rig.dist.barrier()
    total_ms = t0.elapsed_time(t1)
    # ---- per-kernel attribution: the same K steps once more with an event at every kernel boundary
    # (the extra event records lengthen a step by a few percent, so they stay out of the region above)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    for k in range(K):
        ev[k][0].record(stream)
        fft.stftTensor(sig, spec, mag)
        ev[k][1].record(stream)
        fft.istftTensor(spec, rec)
        ev[k][2].record(stream)
    dev.synchronize(600)
    torch.cuda.synchronize()
    if rig.dist is not None:
        rig.dist.barrier()
    stft_ms = float(np.mean([ev[k][0].elapsed_time(ev[k][1]) for k in range(K)]))
    istft_ms = float(np.mean([ev[k][1].elapsed_time(ev[k][2]) for k in range(K)]))
    total_ms, stft_ms, istft_ms = rig.max_ranks([total_ms, stft_ms, istft_ms])
    frames_all = S * FRAMES * world
    value = frames_all * K / (total_ms * 1e-3)

    def kernel_entry(name, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"kernel": name, "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / peak}

    kernels = [kernel_entry("r2c_kernel<2048,aligned,half_interleaved,magnitude> (STFT: frame gather + window + FFT + Hermitian + magnitude)", stft_ms,
                            S * STFT_BYTES_PER_SIGNAL),
               kernel_entry("istft_fast_kernel<2048,half_interleaved,4> (iSTFT: Hermitian + inverse FFT + window + overlap-add + normalise)", istft_ms,
                            S * ISTFT_BYTES_PER_SIGNAL)]
    dom = max(kernels, key=lambda e: e["ms"])
    traffic = measured_traffic_per_signal().get(dom["kernel"].split("<")[0])
    traffic = traffic * S if traffic is not None else None
    roofline = {"bound": "hbm", "achieved": dom["achieved_gbs"], "peak": peak, "unit": "GB/s",
                "frac": dom["frac"], "traffic": traffic, "kernel": dom["kernel"], "peak_kind": rig.peak_kind,
                "step_frac": S * (STFT_BYTES_PER_SIGNAL + ISTFT_BYTES_PER_SIGNAL) / (total_ms / K * 1e-3) / 1e9 / peak,
                "kernel_timing": "per-kernel ms from a second pass over the same K steps with a CUDA event at every kernel "
                                 "boundary; value / ms_per_step from the K steps between two events only"}

    e2e = bench_e2e(rig, args, fft, window, sig, spec, mag, rec, host_in, host_out, frames_all)

    # reconstruction sanity on the timed buffers (not part of any timed region)
    chk = host_out[0, N_FFT:SIGNAL_LEN - N_FFT] - host_in[0, N_FFT:SIGNAL_LEN - N_FFT]
    recon_err = float(chk.double().pow(2).mean().sqrt() / host_in[0].double().pow(2).mean().sqrt())

    # ---- the fixed workloads split over the ranks (strong scaling)
    strong = {}
    if not args.no_extras:
        lo, hi = shard_range(SIGNALS_PER_GPU, rank, world)
        n_loc = min(hi - lo, S)
        sg, sp, mg, rc = sig.rows(0, n_loc), spec.rows(0, n_loc), mag.rows(0, n_loc), rec.rows(0, n_loc)

        def shard_step():
            fft.stftTensor(sg, sp, mg)
            fft.istftTensor(sp, rc)

        ms = rig.timed(shard_step, reps=max(5, min(K, 20)), warm=2)
        nbytes = SIGNALS_PER_GPU * (STFT_BYTES_PER_SIGNAL + ISTFT_BYTES_PER_SIGNAL)
        strong["stft_istft"] = {
            "workload": f"the configuration's 256 signals split over {world} ranks ({n_loc} signals on rank {rank})",
            "scaling": "strong", "n_gpus": world, "ms_per_step": ms, "value": SIGNALS_PER_GPU * FRAMES / (ms * 1e-3),
            "unit": "frames/s", "frac_of_hbm_roofline": nbytes / (ms * 1e-3) / 1e9 / (peak * world)}

    for tns in (spec, mag, rec, sig):
        tns.free()
    rig.unpin(host_out)

    extra = {}
    if not args.no_extras:
        strong["conv"] = bench_conv(rig, CONV3, seed_ir=1003, seed_x=1013)
        strong["conv_low_latency"] = bench_conv(rig, CONV4, seed_ir=1004, seed_x=1014)
        extra["strong"] = strong
        if world == 1:
            os.sched_setaffinity(0, affinity_before)
            cores = len(affinity_before)
            extra["conv"] = dict(strong["conv"])
            extra["conv_low_latency"] = dict(strong["conv_low_latency"])
            extra["large_fft"] = bench_large(rig)
            if not args.no_cpu_baseline:
                extra["conv"]["cpu_baseline"] = cpu_conv_baseline(CONV3, cores)
                extra["conv_low_latency"]["cpu_baseline"] = cpu_conv_baseline(CONV4, cores)
                extra["large_fft"]["cpu_baseline"] = cpu_large_baseline(cores)
            extra["next_rows"] = bench_next_rows(dev, lib, torch, stream, peak)

    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        os.sched_setaffinity(0, affinity_before)
        cores = len(affinity_before)
        sample = max(16, cores)
        x = host_in[:sample].numpy()
        cpu_port_stft_istft(x[:cores], window, cores)
        best = min(cpu_port_stft_istft(x, window, cores) for _ in range(3))
        one = min(cpu_port_stft_istft(x[:2], window, 1) for _ in range(2))
        cpu = {"value": sample * FRAMES / best, "unit": "frames/s", "cores": cores, "kind": "port",
               "one_thread": 2 * FRAMES / one,
               "sample": f"{sample} of the 256 signals ({sample * FRAMES} frames), float32 scipy.fft + numpy port of "
                         f"the reference's stft/istft, {cores} threads, best of 3; one_thread: 2 signals on one thread, "
                         "best of 2"}
    rig.unpin(host_in)

    if rig.dist is not None:
        rig.dist.barrier()
    if rank == 0:
        line = {
            "metric": "stft_istft_frames_per_s", "value": value, "unit": "frames/s", "n_gpus": world,
            "steps": K, "warmup": warmup, "ms_per_step": total_ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world, signals=S),
            "roofline": roofline, "kernels": kernels, "e2e": e2e, "cpu_baseline": cpu,
            "gpu_launches": launches, "clocks": clocks, "reconstruction_rel_rms": recon_err,
            "stft_frames_per_s": frames_all / (stft_ms * 1e-3), "istft_frames_per_s": frames_all / (istft_ms * 1e-3),
            "wall_ms_per_step": 1e3 * t_wall / K, "host_cpus_bound_to_gpu": cpus_bound,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    fft.close()
    if rig.dist is not None:
        rig.dist.destroy_process_group()


def bench_e2e(rig, args, fft, window, sig, spec, mag, rec, host_in, host_out, frames_all):
    """End to end from and to pinned host memory, three legs on the same buffers:
      pipeline   public Tensor API: copy in, STFT, iSTFT, copy out over 16 row ranges round-robin
                 on 4 contexts (streams) of this GPU, so one range's copy-in overlaps another's
                 transforms and a third's copy-out; spectra stay device-resident (the e2e value);
      copy_only  the same copies with no kernels between them: what the host links of this box
                 allow at this many ranks;
      host_api   ma_stft_host + ma_istft_host, the calls the reference's stft() / istft() bind to:
                 complex spectra and magnitudes come back to the host and go in again."""
    import torch
    from metalaudio_b200 import AudioDevice, FFT, WindowType
    dev, lib = rig.dev, rig.lib
    S = sig.shape[0]
    K = args.steps
    e2e_steps = max(2, min(K, 5))
    n_lanes, n_ranges = 4, 16
    lanes = [AudioDevice(rig.local_rank, pinnedBytes=1 << 20) for _ in range(n_lanes)]
    lane_fft = [FFT(d, FFT.Config(size=N_FFT, windowType=WindowType.hann, hopSize=HOP), window=window) for d in lanes]
    lane_stream = [torch.cuda.ExternalStream(lib.ma_context_stream(d.handle), device=rig.device) for d in lanes]
    bounds = [(i * S) // n_ranges for i in range(n_ranges + 1)]
    ranges = [(bounds[i], bounds[i + 1] - bounds[i]) for i in range(n_ranges) if bounds[i + 1] > bounds[i]]

    def e2e_step(transform: bool):
        for i, (lo, cnt) in enumerate(ranges):
            d, ff = lanes[i % n_lanes], lane_fft[i % n_lanes]
            sg, sp, mg, rc = sig.rows(lo, cnt, d), spec.rows(lo, cnt, d), mag.rows(lo, cnt, d), rec.rows(lo, cnt, d)
            sg.copyAsync(host_in.data_ptr() + 4 * lo * SIGNAL_LEN, sg.byteSize)
            if transform:
                ff.stftTensor(sg, sp, mg)
                ff.istftTensor(sp, rc)
            rc.copyToAsync(host_out.data_ptr() + 4 * lo * SIGNAL_LEN, rc.byteSize)
        for d in lanes:
            d.synchronize(120)

    def leg(transform: bool):
        e2e_step(transform)
        rig.barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        ends = [torch.cuda.Event(enable_timing=True) for _ in lanes]
        e0.record(lane_stream[0])
        for _ in range(e2e_steps):
            e2e_step(transform)
        for ev_, st_ in zip(ends, lane_stream):
            ev_.record(st_)
        for d in lanes:
            d.synchronize(120)
        torch.cuda.synchronize()
        ms = max(e0.elapsed_time(ev_) for ev_ in ends)
        return rig.max_ranks([ms])[0] / e2e_steps

    copy_ms = leg(False)
    pipe_ms = leg(True)
    e2e = {"value": frames_all / (pipe_ms * 1e-3), "unit": "frames/s",
           "h2d_bytes_per_step": sig.byteSize, "d2h_bytes_per_step": rec.byteSize, "steps": e2e_steps,
           "ms_per_step": pipe_ms,
           "how": f"{len(ranges)} row ranges over {n_lanes} streams: copy-in, STFT, iSTFT, copy-out of different "
                  "ranges overlap; spectra and magnitudes stay in device memory",
           "copy_only_ms_per_step": copy_ms, "pipeline_over_copy_only": pipe_ms / copy_ms,
           "copy_only_gbs_each_way": sig.byteSize / (copy_ms * 1e-3) / 1e9}
    for ff in lane_fft:
        ff.close()
    for d in lanes:
        d.close()

    # host-buffer entry points on a quarter of the signals (the buffers that come back are 6x the input)
    hs = max(4, S // 4)
    h_spec = rig.pinned((hs, FRAMES, KH, 2))
    h_mag = rig.pinned((hs, FRAMES, KH))
    st = lib.ma_context_reserve_workspace(dev.handle, 2 * (256 << 20))

    def host_call():
        a = lib.ma_stft_host(fft._h, ptr(host_in), SIGNAL_LEN, SIGNAL_LEN, hs, ptr(h_spec), None, ptr(h_mag), 0, 1.0, 0)
        b = lib.ma_istft_host(fft._h, ptr(h_spec), None, FRAMES, hs, ptr(host_out), SIGNAL_LEN, 1e-8, 0)
        if a != 0 or b != 0 or st != 0:
            raise RuntimeError(f"host-buffer STFT / iSTFT failed: {st} {a} {b}")

    host_call()
    rig.barrier()
    reps = 2
    t0 = time.perf_counter()
    for _ in range(reps):
        host_call()
    host_ms = rig.max_ranks([(time.perf_counter() - t0) * 1e3 / reps])[0]
    bytes_in = 4 * hs * SIGNAL_LEN + 8 * hs * FRAMES * KH
    bytes_out = 12 * hs * FRAMES * KH + 4 * hs * SIGNAL_LEN
    e2e["host_api"] = {
        "value": hs * FRAMES * rig.world / (host_ms * 1e-3), "unit": "frames/s", "ms_per_call_pair": host_ms,
        "signals": hs, "h2d_bytes": bytes_in, "d2h_bytes": bytes_out,
        "gbs_over_the_link": (bytes_in + bytes_out) / (host_ms * 1e-3) / 1e9,
        "how": "ma_stft_host then ma_istft_host on pinned host arrays: complex spectra + magnitudes return to the "
               "host (what the reference's stft() hands back) and the spectra go in again for the inverse; chunks "
               "pipelined over three streams through the context's pre-allocated workspace; host wall clock"}
    rig.unpin(h_spec)
    rig.unpin(h_mag)
    return e2e


def bench_conv(rig, cfg, seed_ir: int, seed_x: int):
    """One partitioned-convolution configuration, its FIXED channel count split over the ranks
    (by impulse-response pair when the responses are per pair): causal streaming steps - every step
    reads the whole frequency-domain delay line of every channel once, the HBM-streaming kernel -
    and the whole-signal call (the reference's process(input:output:)), each timed with CUDA events,
    maximum over ranks.  At one rank also end to end from and to pinned host memory."""
    import torch
    from metalaudio_b200 import Convolution, Tensor
    from metalaudio_b200.sharding import shard_range
    dev, lib, stream, peak = rig.dev, rig.lib, rig.stream, rig.peak
    C_all, B, taps, L, group = cfg["channels"], cfg["block"], cfg["taps"], cfg["length"], cfg["group"]
    lo, hi = shard_range(C_all, rig.rank, rig.world, group)
    C = hi - lo
    P = taps // B
    shared = group == 1
    conv = Convolution(dev, Convolution.Mode.partitioned(blockSize=B), channels=C)
    if shared:
        conv.setKernel(decaying_irs(1, taps, seed_ir)[0])
        sharing = C
    else:
        irs = decaying_irs(C // group, taps, seed_ir, first=lo // group)
        conv.setKernel(irs, channelToKernel=[c // group for c in range(C)])
        del irs
        sharing = group
    if cfg.get("splits", 0) > 0:
        st = lib.ma_pconv_step_splits(conv._h, int(cfg["splits"]), None)
        if st != 0:
            raise RuntimeError(f"ma_pconv_step_splits failed: {st}")
    steps, warm = cfg["steps"], cfg["warm"]
    n = (steps + warm) * B
    gen = torch.Generator(device=rig.device).manual_seed(seed_x + rig.rank)
    x = torch.empty((C, n), dtype=torch.float32, device=rig.device).normal_(0.0, 0.1, generator=gen)
    y = torch.empty_like(x)
    torch.cuda.synchronize()

    def do(t):
        st = lib.ma_pconv_step_dev(conv._h, ctypes.c_void_p(x.data_ptr() + 4 * t * B), n,
                                   ctypes.c_void_p(y.data_ptr() + 4 * t * B), n)
        if st != 0:
            raise RuntimeError(f"ma_pconv_step_dev failed: {st}")

    for t in range(warm):
        do(t)
    rig.barrier()
    l0 = lib.ma_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for t in range(warm, warm + steps):
        do(t)
    e1.record(stream)
    dev.synchronize(120)
    torch.cuda.synchronize()
    launches = int(lib.ma_kernel_launch_count() - l0)
    ms = rig.max_ranks([e0.elapsed_time(e1) / steps])[0]
    if rig.dist is not None:
        rig.dist.barrier()
    bpcb = conv_bytes_per_channel_block(B, P, sharing)
    gbs_per_gpu = C * bpcb / (ms * 1e-3) / 1e9
    out = {"workload": f"partitioned convolution: {C_all} channels, "
                       + ("one shared" if shared else f"{C_all // group} per-pair") +
                       f" impulse response(s) of {taps} taps, block {B} (FFT {2 * B}, {P} partitions), split over "
                       f"{rig.world} ranks ({C} channels on rank {rig.rank})",
           "scaling": "strong", "n_gpus": rig.world, "channels_per_gpu": C,
           "metric": "conv_channel_samples_per_s", "value": C_all * B / (ms * 1e-3), "unit": "channel-samples/s",
           "ms_per_step": ms, "steps": steps, "gpu_launches": launches,
           "roofline": {"bound": "hbm", "achieved": gbs_per_gpu, "peak": peak, "unit": "GB/s", "frac": gbs_per_gpu / peak,
                        "algorithmic_bytes_per_channel_block": bpcb,
                        "kernel": "pconv_mac_kernel + r2c + c2r per step (per GPU)"}}
    del x, y
    # Whole-signal call: all block spectra exist up front, so the multiply-accumulate is tiled over
    # time and becomes FMA-bound; its rate is quoted against the same streaming byte count.
    if not rig_skip_whole(cfg, C):
        full = L + taps - 1
        st = lib.ma_pconv_reset(conv._h)
        st = st or lib.ma_pconv_reserve(conv._h, L)
        xs = torch.empty((C, L), dtype=torch.float32, device=rig.device).normal_(0.0, 0.1, generator=gen)
        ys = torch.empty((C, full), dtype=torch.float32, device=rig.device)
        torch.cuda.synchronize()

        def whole():
            nonlocal st
            st = st or lib.ma_pconv_process_dev(conv._h, ptr(xs), L, L, ptr(ys), full)

        pms = rig.timed(whole, reps=2, warm=1)
        if st != 0:
            raise RuntimeError(f"whole-signal convolution failed: {st}")
        blocks = (full + B - 1) // B
        stream_bytes = C * (L // B) * bpcb
        out["whole_signal"] = {
            "workload": f"process(): {C_all} channels x 2^{int(np.log2(L))} samples, full L+K-1 output ({blocks} blocks "
                        "per channel)",
            "value": C_all * L / (pms * 1e-3), "unit": "channel-samples/s", "ms": pms,
            "times_streaming_roofline": stream_bytes / (pms * 1e-3) / 1e9 / peak,
            "complex_macs": float(C) * blocks * P * B,
            "note": "time-tiled multiply-accumulate: delay-line spectra reused on chip, FP32-FMA-bound, so the "
                    "HBM-streaming byte count is exceeded by design"}
        if rig.world == 1:
            # end to end: pinned host rows in, the full L+K-1 rows back, copies inside the timed region
            h_in = rig.pinned((C, L))
            h_out = rig.pinned((C, full))
            h_in.normal_(0.0, 0.1, generator=torch.Generator().manual_seed(seed_x))
            lib.ma_pconv_reset(conv._h)
            times = []
            for _ in range(3):
                t0 = time.perf_counter()
                st = lib.ma_pconv_process_host(conv._h, ptr(h_in), L, L, ptr(h_out), full)
                times.append(time.perf_counter() - t0)
                if st != 0:
                    raise RuntimeError(f"ma_pconv_process_host failed: {st}")
            ems = min(times[1:]) * 1e3
            out["e2e"] = {"value": C * L / (ems * 1e-3), "unit": "channel-samples/s", "ms": ems,
                          "h2d_bytes_per_step": 4 * C * L, "d2h_bytes_per_step": 4 * C * full,
                          "how": "ma_pconv_process_host on pinned host arrays: copy in, whole-signal call, full "
                                 "L+K-1 output copied back; host wall clock, best of 2 after a warm-up"}
            rig.unpin(h_in)
            rig.unpin(h_out)
        del xs, ys
    conv.close()
    return out


def rig_skip_whole(cfg, channels: int) -> bool:
    return cfg.get("skip_whole", False) or channels < 1


def bench_large(rig):
    """65536-point forward + inverse batch (configuration 5), device-resident and end to end."""
    import torch
    from metalaudio_b200 import FFT, Tensor, WindowType
    dev, lib, peak = rig.dev, rig.lib, rig.peak
    n, batch = LARGE["n"], LARGE["batch"]
    fft = FFT(dev, FFT.Config(size=n, windowType=WindowType.none))
    host = rig.pinned((batch, n))
    host.normal_(0.0, 1.0, generator=torch.Generator().manual_seed(1005))
    x = torch.empty((batch, n), dtype=torch.float32, device=rig.device)
    x.copy_(host)
    z = torch.empty((batch, n // 2 + 1, 2), dtype=torch.float32, device=rig.device)
    y = torch.empty_like(x)
    torch.cuda.synchronize()

    def pair():
        a = lib.ma_fft_forward_dev(fft._h, ptr(x), ptr(z), None, None, 0, 1.0, batch, 0)
        b = lib.ma_fft_inverse_dev(fft._h, ptr(z), None, ptr(y), batch, 0)
        if a != 0 or b != 0:
            raise RuntimeError(f"large FFT failed: {a} {b}")

    ms = rig.timed(pair, reps=10, warm=3)
    nbytes = 2 * batch * (n * 4 + (n // 2 + 1) * 8)
    gbs = nbytes / (ms * 1e-3) / 1e9
    out = {"workload": f"{batch} x 65536-point real forward + inverse", "metric": "fft65536_pairs_per_s",
           "value": batch / (ms * 1e-3), "unit": "pairs/s", "ms_per_pair_batch": ms,
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "algorithmic_bytes": nbytes}}
    del x, y, z
    # end to end: pinned host frames in, half spectra back, then spectra in and frames back
    h_spec = rig.pinned((batch, n // 2 + 1, 2))
    h_back = rig.pinned((batch, n))
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        a = lib.ma_fft_forward_host(fft._h, ptr(host), ptr(h_spec), None, None, 0, 1.0, batch, 0)
        b = lib.ma_fft_inverse_host(fft._h, ptr(h_spec), None, ptr(h_back), batch, 0)
        times.append(time.perf_counter() - t0)
        if a != 0 or b != 0:
            raise RuntimeError(f"large FFT (host buffers) failed: {a} {b}")
    ems = min(times[1:]) * 1e3
    err = float((h_back[:64] - host[:64]).double().pow(2).mean().sqrt() / host[:64].double().pow(2).mean().sqrt())
    out["e2e"] = {"value": batch / (ems * 1e-3), "unit": "pairs/s", "ms": ems,
                  "h2d_bytes_per_step": 4 * batch * n + 8 * batch * (n // 2 + 1),
                  "d2h_bytes_per_step": 4 * batch * n + 8 * batch * (n // 2 + 1), "round_trip_rel_rms": err,
                  "how": "ma_fft_forward_host then ma_fft_inverse_host on pinned host arrays; host wall clock, best of 2 "
                         "after a warm-up"}
    for t in (host, h_spec, h_back):
        rig.unpin(t)
    fft.close()
    return out


def bench_next_rows(dev, lib, torch, stream, peak, small=False):
    """The callers either side of the hot path: STFT / iSTFT through the magnitude + phase layout
    (64 signals of configuration 2's shape), the one-shot FFT convolution (256 signals, 131072-tap
    kernel, 2^20-point transforms) and biquad cascades.  Device-resident, CUDA-event timed, best of
    5 after a warm-up."""
    from metalaudio_b200 import FFT, WindowType
    device = torch.device("cuda", dev.deviceIndex)

    def timed(fn, reps=5):
        best = None
        for i in range(reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            st = fn()
            e1.record(stream)
            dev.synchronize(120)
            torch.cuda.synchronize()
            if st != 0:
                raise RuntimeError(f"next-row workload failed: status {st}")
            if i > 0:
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
        return best

    out = {}
    # --- magnitude / phase layout
    S, L, n, hop = (16 if small else 64), SIGNAL_LEN, N_FFT, HOP
    frames = (L - n) // hop + 1
    kh = n // 2 + 1
    fft = FFT(dev, FFT.Config(size=n, windowType=WindowType.hann, hopSize=hop), window=periodic_hann(n))
    x = torch.empty((S, L), dtype=torch.float32, device=device).uniform_(-1.0, 1.0)
    mag = torch.empty((S, frames, kh), dtype=torch.float32, device=device)
    ph = torch.empty_like(mag)
    y = torch.empty((S, L), dtype=torch.float32, device=device)
    torch.cuda.synchronize()
    ms_f = timed(lambda: lib.ma_stft_dev(fft._h, ptr(x), L, L, S, ptr(mag), ptr(ph), None, 0, 1.0, 3))
    ms_i = timed(lambda: lib.ma_istft_dev(fft._h, ptr(mag), ptr(ph), frames, S, ptr(y), L, 1e-8, 3))
    keep = slice(n, L - n)
    err = float((y[:, keep] - x[:, keep]).pow(2).mean().sqrt() / x[:, keep].pow(2).mean().sqrt())
    bytes_f = S * (4 * L + frames * 8 * kh)
    out["polar_stft_istft"] = {
        "workload": f"{S} signals x 2^20 samples, N={n}, hop={hop}: STFT to magnitude+phase, iSTFT from them",
        "stft_ms": ms_f, "istft_ms": ms_i, "frames_per_s": S * frames / ((ms_f + ms_i) * 1e-3),
        "stft_frac_of_hbm_peak": bytes_f / (ms_f * 1e-3) / 1e9 / peak,
        "istft_frac_of_hbm_peak": bytes_f / (ms_i * 1e-3) / 1e9 / peak,
        "algorithmic_bytes_each": bytes_f, "reconstruction_rel_rms": err}
    fft.close()
    del x, mag, ph, y
    # --- one-shot FFT convolution: enough signals to fill the GPU several times over
    sig, taps, nfft = (8 if small else 256), 131072, 1 << 20
    length = nfft - taps + 1
    h = decaying_irs(1, taps, 1003)[0]
    fc = ctypes.c_void_p()
    st = lib.ma_fftconv_create(dev.handle, h.ctypes.data_as(ctypes.c_void_p), taps, length, sig, ctypes.byref(fc))
    if st != 0:
        raise RuntimeError(f"ma_fftconv_create failed: {st}")
    xs = torch.empty((sig, length), dtype=torch.float32, device=device).normal_(0.0, 0.1)
    ys = torch.empty((sig, nfft), dtype=torch.float32, device=device)
    torch.cuda.synchronize()
    ms_c = timed(lambda: lib.ma_fftconv_process_dev(fc, ptr(xs), length, length, sig, ptr(ys)))
    bytes_c = sig * 4 * (length + nfft)
    out["fft_convolution"] = {
        "workload": f"{sig} signals x {length} samples, one {taps}-tap kernel, {nfft}-point transforms",
        "ms": ms_c, "value": sig * length / (ms_c * 1e-3), "unit": "signal-samples/s",
        "frac_of_hbm_peak": bytes_c / (ms_c * 1e-3) / 1e9 / peak, "algorithmic_bytes": bytes_c,
        "note": "three passes per chunk (columns forward, rows forward * kernel spectrum + inverse in place, "
                "columns inverse) on L2-resident pass data: HBM sees input and output once; the passes "
                "themselves are latency / issue bound at this transform size"}
    lib.ma_fftconv_destroy(fc)
    del xs, ys
    # --- multichannel biquad: 512 channels x 2^20 samples, one low-pass section, then a 4-section cascade
    C, L = (296 if small else 512), SIGNAL_LEN
    xb = torch.empty((C, L), dtype=torch.float32, device=device).normal_(0.0, 0.1)
    yb = torch.empty_like(xb)
    torch.cuda.synchronize()
    w = 2.0 * np.pi * 1000.0 / 48000.0
    al = np.sin(w) / (2.0 * 0.7071067811865476)
    lp = (np.array([(1 - np.cos(w)) / 2, 1 - np.cos(w), (1 - np.cos(w)) / 2, -2 * np.cos(w), 1 - al]) / (1 + al)).astype(np.float32)
    res = {}
    for sections in (1, 4):
        bq = ctypes.c_void_p()
        st = lib.ma_biquad_create(dev.handle, C, sections, ctypes.byref(bq))
        coeffs = np.ascontiguousarray(np.tile(lp, (sections, 1)))
        st = st or lib.ma_biquad_set_coefficients(bq, coeffs.ctypes.data_as(ctypes.c_void_p), 1, None)
        if st != 0:
            raise RuntimeError(f"biquad set-up failed: {st}")
        ms_b = timed(lambda: lib.ma_biquad_process_dev(bq, ptr(xb), L, ptr(yb), L, L))
        res[sections] = ms_b
        lib.ma_biquad_destroy(bq)
    bytes_b = C * L * 8
    out["biquad"] = {
        "workload": f"{C} channels x 2^20 samples, Direct Form II Transposed low-pass sections, state in double",
        "ms_1_section": res[1], "ms_4_sections": res[4], "value": C * L / (res[1] * 1e-3), "unit": "channel-samples/s",
        "frac_of_hbm_peak_1_section": bytes_b / (res[1] * 1e-3) / 1e9 / peak,
        "frac_of_hbm_peak_4_sections": bytes_b / (res[4] * 1e-3) / 1e9 / peak, "algorithmic_bytes": bytes_b}
    return out


def run_only(args, local_rank: int):
    """One of the extra workloads alone, for profiler captures of its kernels."""
    import torch
    rig = Rig(local_rank, 0, 1)
    if args.only == "next":
        res = bench_next_rows(rig.dev, rig.lib, torch, rig.stream, rig.peak, small=args.small)
    elif args.only == "conv4":
        cfg = dict(CONV4, channels=256 if args.small else (args.conv4_channels or CONV4["channels"]),
                   splits=args.conv_splits, skip_whole=not args.whole)
        res = bench_conv(rig, cfg, seed_ir=1004, seed_x=1014)
    elif args.only == "conv":
        cfg = dict(CONV3, skip_whole=not (args.whole or CONV3["channels"] >= 256))
        res = bench_conv(rig, cfg, seed_ir=1003, seed_x=1013)
    else:
        res = bench_large(rig)
    print(json.dumps({args.only: res}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true", help="skip the strong-scaling, convolution and 65536-point lines")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--signals", type=int, default=SIGNALS_PER_GPU,
                    help="signals per GPU (default: the benchmark configuration's 256; smaller for profiler captures)")
    ap.add_argument("--conv-channels", type=int, default=CONV3["channels"])
    ap.add_argument("--conv-splits", type=int, default=0,
                    help="with --only conv / conv4: force the streaming step's partition splits (0: the library's choice)")
    ap.add_argument("--conv4-channels", type=int, default=0,
                    help="with --only conv4: channels of the low-latency case (0: the configuration's 1024)")
    ap.add_argument("--large-batch", type=int, default=LARGE["batch"])
    ap.add_argument("--small", action="store_true", help="with --only next / conv4: a quarter-size case for profiler captures")
    ap.add_argument("--whole", action="store_true", help="with --only conv / conv4: also run the whole-signal call")
    ap.add_argument("--only", choices=["conv", "conv4", "large", "next"], default=None,
                    help="run just one of the extra workloads (profiler captures)")
    ap.add_argument("--port-worker", nargs=4, type=int, default=None, metavar=("BLOCK", "TAPS", "BLOCKS", "SEED"),
                    help="internal: time the CPU port of the convolution block loop and print seconds per block")
    args = ap.parse_args()
    if args.port_worker is not None:
        print(_port_seconds_per_block(*args.port_worker), flush=True)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    CONV3["channels"] = args.conv_channels
    CONV3["splits"] = args.conv_splits
    LARGE["batch"] = args.large_batch
    if args.only is not None:
        run_only(args, local_rank)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
