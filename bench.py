#!/usr/bin/env python
"""Benchmark of the MetalDSP hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the hot path over one batch of synthetic input: the batched
STFT + iSTFT configuration (256 mono signals of 2^20 uniform[-1,1) samples per GPU,
n_fft 4096, hop 1024, periodic Hann; half-spectrum complex + magnitude out, COLA
overlap-add reconstruction back).  Metric: STFT frames/s, whole job over all GPUs, with the
signals already resident in HBM.  Under torchrun every rank runs its own shard of
independent signals (no collective on the data path; weak scaling), the timed region is
bracketed by barrier + device synchronisation and the maximum over ranks is reported.

The JSON line also carries
  roofline      the dominant kernel's achieved HBM GB/s (algorithmic bytes / CUDA-event time)
                against the measured copy bandwidth of this pool's B200s,
  kernels       the same for every kernel of the step,
  e2e           the same metric through the public Tensor API with pinned host buffers,
                host->device and device->host copies inside the timed region,
  cpu_baseline  the float32 CPU port of the reference path timed on the host cores (N=1 only),
  conv          the partitioned-convolution configuration (512 channels, one shared 131072-tap
                IR, block 256) as a streaming step, with its own roofline fraction,
  large_fft     the 65536-point forward + inverse batch.

`--impl reference` times the CPU port of the reference path (the reference itself is Swift +
Apple Accelerate and cannot run here) on all host cores over a bounded sample per step.
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
CONV = dict(channels=512, block=256, taps=131072, bytes_per_channel_block=1058832)
LARGE = dict(n=65536, batch=4096)


def periodic_hann(n: int) -> np.ndarray:
    """0.5(1 - cos(2 pi k/n)), computed in float64: the window the benchmark configuration names."""
    k = np.arange(n, dtype=np.float64)
    return (0.5 * (1.0 - np.cos(2.0 * np.pi * k / float(n)))).astype(np.float32)


def decaying_ir(taps: int, seed: int = 1003) -> np.ndarray:
    """Synthetic room response: Gaussian noise with an exponential decay reaching -60 dB after 1.5 s
    at 48 kHz, scaled to unit energy."""
    g = np.random.Generator(np.random.PCG64(seed))
    k = np.arange(taps, dtype=np.float64)
    h = g.standard_normal(taps) * np.exp(-6.907755278982137 * k / (1.5 * 48000.0))
    return (h / np.sqrt(np.sum(h * h))).astype(np.float32)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs
    (read-only queries)."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
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
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
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
    """`--impl reference`: the CPU port on all host cores; rank 0 only."""
    if rank != 0:
        return
    from oracle import configs, reference_path as rp
    cores = os.cpu_count() or 1
    sample = max(cores, 16)
    x = configs.c2_signals(n_signals=sample, length=SIGNAL_LEN)
    w = periodic_hann(N_FFT)
    for _ in range(min(args.warmup, 1)):
        cpu_port_stft_istft(x[:cores], w, cores)
    times = [cpu_port_stft_istft(x, w, cores) for _ in range(args.steps)]
    total = float(np.sum(times))
    frames = sample * FRAMES * args.steps
    value = frames / total
    line = {
        "impl": "reference", "metric": "stft_istft_frames_per_s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, sample_note=f"each step = {sample} signals on the host CPU"),
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} signals x 2^20 samples per step ({sample * FRAMES} frames), "
                                   f"scipy.fft float32 + numpy, {cores} threads"},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, sample_note: str | None = None, signals: int = SIGNALS_PER_GPU):
    cfg = {"workload": f"batched STFT+iSTFT: {signals} mono fp32 signals x 2^20 samples per GPU, uniform[-1,1), "
                       "n_fft=4096, hop=1024, periodic Hann, half-spectrum complex + magnitude out, "
                       "COLA overlap-add reconstruction",
           "signals_per_gpu": signals, "signal_len": SIGNAL_LEN, "n_fft": N_FFT, "hop": HOP,
           "frames_per_gpu": signals * FRAMES, "window": "periodic_hann",
           "sharding": f"independent signals per rank, no collective ({n_gpus} ranks)",
           "cache": "inputs (1.07 GB) and outputs (6.4 GB) per step exceed the 126 MB L2; no flush needed"}
    if sample_note:
        cfg["sample"] = sample_note
    return cfg


# ----------------------------------------------------------------------------- GPU arm

def run_ours(args, rank: int, local_rank: int, world: int):
    import torch
    from metalaudio_b200 import AudioDevice, Convolution, FFT, Tensor, WindowType

    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = AudioDevice(local_rank)
    lib = dev._lib
    stream = torch.cuda.ExternalStream(lib.ma_context_stream(dev.handle), device=torch.device("cuda", local_rank))
    peak, peak_kind = measured_peak_gbs()

    window = periodic_hann(N_FFT)
    fft = FFT(dev, FFT.Config(size=N_FFT, windowType=WindowType.hann, hopSize=HOP), window=window)
    S = args.signals
    sig = Tensor(dev, (S, SIGNAL_LEN))
    spec = Tensor(dev, (S, FRAMES, KH, 2))
    mag = Tensor(dev, (S, FRAMES, KH))
    rec = Tensor(dev, (S, SIGNAL_LEN))

    # Synthetic input: uniform[-1,1), seeded per global signal index, generated into pinned host
    # memory (the e2e leg copies it from there every step).
    host_in = torch.empty((S, SIGNAL_LEN), dtype=torch.float32, pin_memory=True)
    host_out = torch.empty((S, SIGNAL_LEN), dtype=torch.float32, pin_memory=True)
    gen = torch.Generator().manual_seed(1002 + rank)
    host_in.uniform_(-1.0, 1.0, generator=gen)
    sig.copyAsync(host_in.data_ptr(), sig.byteSize)
    dev.synchronize(60)

    def step():
        fft.stftTensor(sig, spec, mag)
        fft.istftTensor(spec, rec)

    def barrier():
        dev.synchronize(120)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    warmup = max(args.warmup, 3) if S == SIGNALS_PER_GPU else max(args.warmup, 1)
    for _ in range(warmup):
        step()
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream around every kernel
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = lib.ma_kernel_launch_count()
    t_wall0 = time.perf_counter()
    for k in range(K):
        ev[k][0].record(stream)
        fft.stftTensor(sig, spec, mag)
        ev[k][1].record(stream)
        fft.istftTensor(spec, rec)
        ev[k][2].record(stream)
    dev.synchronize(600)
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    launches = int(lib.ma_kernel_launch_count() - launches0)
    clocks = sampler.stop()
    if dist is not None:
        dist.barrier()
    total_ms = ev[0][0].elapsed_time(ev[K - 1][2])
    stft_ms = float(np.mean([ev[k][0].elapsed_time(ev[k][1]) for k in range(K)]))
    istft_ms = float(np.mean([ev[k][1].elapsed_time(ev[k][2]) for k in range(K)]))
    if dist is not None:
        t = torch.tensor([total_ms, stft_ms, istft_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, stft_ms, istft_ms = [float(v) for v in t.tolist()]
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
    # dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised in
    # profiles/stft_istft_n4096_hop1024.md (48-signal case), scaled by the signals of this launch.
    per_signal = {"r2c_kernel": (0.206366208e9 + 1.146860e9) / 48, "istft_fast_kernel": (0.832580608e9 + 0.184410368e9) / 48}
    traffic = per_signal.get(dom["kernel"].split("<")[0])
    traffic = traffic * S if traffic is not None else None
    roofline = {"bound": "hbm", "achieved": dom["achieved_gbs"], "peak": peak, "unit": "GB/s",
                "frac": dom["frac"], "traffic": traffic, "kernel": dom["kernel"], "peak_kind": peak_kind}

    # ---- e2e: pinned host -> device -> STFT -> iSTFT -> pinned host, through the Tensor API.
    # The signals are independent, so the step is cut into row ranges that go round-robin to a few
    # AudioDevice contexts (streams) of this GPU: one range's host->device copy overlaps another's
    # transforms and a third's device->host copy (PCIe is full duplex).  Every byte of the step's
    # input and output crosses PCIe inside the timed region.
    e2e_steps = max(2, min(K, 5))
    n_lanes, n_ranges = 4, 16
    lanes = [AudioDevice(local_rank, pinnedBytes=1 << 20) for _ in range(n_lanes)]
    lane_fft = [FFT(d, FFT.Config(size=N_FFT, windowType=WindowType.hann, hopSize=HOP), window=window) for d in lanes]
    lane_stream = [torch.cuda.ExternalStream(lib.ma_context_stream(d.handle), device=torch.device("cuda", local_rank))
                   for d in lanes]
    bounds = [(i * S) // n_ranges for i in range(n_ranges + 1)]
    ranges = [(bounds[i], bounds[i + 1] - bounds[i]) for i in range(n_ranges) if bounds[i + 1] > bounds[i]]

    def e2e_step():
        for i, (lo, cnt) in enumerate(ranges):
            d, ff = lanes[i % n_lanes], lane_fft[i % n_lanes]
            sg, sp, mg, rc = sig.rows(lo, cnt, d), spec.rows(lo, cnt, d), mag.rows(lo, cnt, d), rec.rows(lo, cnt, d)
            sg.copyAsync(host_in.data_ptr() + 4 * lo * SIGNAL_LEN, sg.byteSize)
            ff.stftTensor(sg, sp, mg)
            ff.istftTensor(sp, rc)
            rc.copyToAsync(host_out.data_ptr() + 4 * lo * SIGNAL_LEN, rc.byteSize)
        for d in lanes:
            d.synchronize(120)

    e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    ends = [torch.cuda.Event(enable_timing=True) for _ in lanes]
    e0.record(lane_stream[0])
    for _ in range(e2e_steps):
        e2e_step()
    for ev_, st_ in zip(ends, lane_stream):
        ev_.record(st_)
    for d in lanes:
        d.synchronize(120)
    torch.cuda.synchronize()
    e2e_ms = max(e0.elapsed_time(ev_) for ev_ in ends)
    if dist is not None:
        t = torch.tensor([e2e_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": frames_all * e2e_steps / (e2e_ms * 1e-3), "unit": "frames/s",
           "h2d_bytes_per_step": sig.byteSize, "d2h_bytes_per_step": rec.byteSize, "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps,
           "how": f"{len(ranges)} row ranges over {n_lanes} streams: copy-in, STFT, iSTFT, copy-out of different "
                  "ranges overlap"}
    for ff in lane_fft:
        ff.close()
    for d in lanes:
        d.close()

    # reconstruction sanity on the timed buffers (not part of any timed region)
    chk = host_out[0, N_FFT:SIGNAL_LEN - N_FFT] - host_in[0, N_FFT:SIGNAL_LEN - N_FFT]
    recon_err = float(chk.double().pow(2).mean().sqrt() / host_in[0].double().pow(2).mean().sqrt())

    for tns in (spec, mag, rec, sig):
        tns.free()
    del host_out

    extra = {}
    if not args.no_extras and rank == 0:  # single-GPU side measurements: rank 0 only, the others wait at the barrier
        extra["conv"] = bench_conv(dev, lib, torch, stream, peak)
        extra["conv_low_latency"] = bench_conv4(dev, lib, torch, stream, peak)
        extra["large_fft"] = bench_large(dev, lib, torch, stream, peak)
        extra["next_rows"] = bench_next_rows(dev, lib, torch, stream, peak)

    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        sample = max(16, cores)
        x = host_in[:sample].numpy()
        cpu_port_stft_istft(x[:cores], window, cores)
        best = min(cpu_port_stft_istft(x, window, cores) for _ in range(3))
        cpu = {"value": sample * FRAMES / best, "unit": "frames/s", "cores": cores, "kind": "port",
               "sample": f"{sample} of the 256 signals ({sample * FRAMES} frames), float32 scipy.fft + numpy port of "
                         f"the reference's stft/istft, {cores} threads, best of 3"}

    if dist is not None:
        dist.barrier()
    if rank == 0:
        line = {
            "metric": "stft_istft_frames_per_s", "value": value, "unit": "frames/s", "n_gpus": world,
            "steps": K, "warmup": warmup, "ms_per_step": total_ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world, signals=S),
            "roofline": roofline, "kernels": kernels, "e2e": e2e, "cpu_baseline": cpu,
            "gpu_launches": launches, "clocks": clocks, "reconstruction_rel_rms": recon_err,
            "stft_frames_per_s": frames_all / (stft_ms * 1e-3), "istft_frames_per_s": frames_all / (istft_ms * 1e-3),
            "wall_ms_per_step": 1e3 * t_wall / K,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    fft.close()
    if dist is not None:
        dist.destroy_process_group()


def bench_conv(dev, lib, torch, stream, peak, whole_signal=None):
    """Partitioned convolution, configuration 3 shape, as causal streaming steps: every step
    reads the whole frequency-domain delay line of every channel once."""
    from metalaudio_b200 import Convolution, Tensor
    C, B, taps = CONV["channels"], CONV["block"], CONV["taps"]
    steps, warm = (200, 16) if C >= 256 else (24, 8)
    conv = Convolution(dev, Convolution.Mode.partitioned(blockSize=B), channels=C)
    conv.setKernel(decaying_ir(taps))
    x = Tensor(dev, (C, (steps + warm) * B))
    y = Tensor(dev, (C, (steps + warm) * B))
    host = torch.empty((C, (steps + warm) * B), dtype=torch.float32, pin_memory=True)
    host.normal_(0.0, 0.1, generator=torch.Generator().manual_seed(1013))
    x.copyAsync(host.data_ptr(), x.byteSize)
    dev.synchronize(60)
    stride = (steps + warm) * B

    def do(t):
        st = lib.ma_pconv_step_dev(conv._h, ctypes.c_void_p(x.pointer + 4 * t * B), stride,
                                   ctypes.c_void_p(y.pointer + 4 * t * B), stride)
        if st != 0:
            raise RuntimeError(f"ma_pconv_step_dev failed: {st}")

    for t in range(warm):
        do(t)
    dev.synchronize(60)
    l0 = lib.ma_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for t in range(warm, warm + steps):
        do(t)
    e1.record(stream)
    dev.synchronize(120)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = int(lib.ma_kernel_launch_count() - l0)
    gbs = C * CONV["bytes_per_channel_block"] / (ms * 1e-3) / 1e9
    out = {"workload": "partitioned convolution: 512 channels, shared 131072-tap IR, block 256 (FFT 512, 512 "
                       "partitions), streaming steps",
           "metric": "conv_channel_samples_per_s", "value": C * B / (ms * 1e-3), "unit": "channel-samples/s",
           "ms_per_step": ms, "steps": steps, "gpu_launches": launches,
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "algorithmic_bytes_per_channel_block": CONV["bytes_per_channel_block"],
                        "kernel": "pconv_mac_kernel + r2c + c2r per step"}}
    x.free()
    y.free()
    # Whole-signal call (the reference's process(input:output:)): 2^20 samples per channel, full
    # L+K-1 output.  All block spectra exist up front, so the multiply-accumulate is tiled over
    # time and becomes FMA-bound; its rate is quoted against the same streaming byte count.
    if (C >= 256) if whole_signal is None else whole_signal:
        L = 1 << 20
        full = L + taps - 1
        st = lib.ma_pconv_reset(conv._h)
        st = st or lib.ma_pconv_reserve(conv._h, L)
        xs = torch.empty((C, L), dtype=torch.float32, device=f"cuda:{dev.deviceIndex}")
        xs.normal_(0.0, 0.1, generator=torch.Generator(device=xs.device).manual_seed(1013))
        ys = torch.empty((C, full), dtype=torch.float32, device=xs.device)
        torch.cuda.synchronize()
        times = []
        for _ in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            st = st or lib.ma_pconv_process_dev(conv._h, ctypes.c_void_p(xs.data_ptr()), L, L,
                                                ctypes.c_void_p(ys.data_ptr()), full)
            e1.record(stream)
            dev.synchronize(120)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        if st != 0:
            raise RuntimeError(f"whole-signal convolution failed: {st}")
        pms = min(times[1:])
        stream_bytes = C * (L // B) * CONV["bytes_per_channel_block"]
        out["whole_signal"] = {
            "workload": f"process(): {C} channels x 2^20 samples, full L+K-1 output (4608 blocks per channel)",
            "value": C * L / (pms * 1e-3), "unit": "channel-samples/s", "ms": pms,
            "times_streaming_roofline": stream_bytes / (pms * 1e-3) / 1e9 / peak,
            "note": "time-tiled multiply-accumulate: delay-line spectra reused on chip, FMA-bound "
                    "(1.24e12 FP32 FMAs), so the HBM-streaming byte count is exceeded by design"}
        del xs, ys
    conv.close()
    return out


def bench_conv4(dev, lib, torch, stream, peak, channels=1024):
    """Low-latency partitioned convolution, configuration 4 shape, as causal streaming steps: 1024
    channels, block 64 (FFT 128), 262144-tap impulse response per channel pair (512 distinct ones,
    4096 partitions): the per-pair spectra cannot be shared beyond two channels."""
    from metalaudio_b200 import Convolution, Tensor
    C, B, taps = channels, 64, 262144
    n_irs = C // 2
    bytes_per_channel_block = 4 * B + 4 * B + 8 * (B + 1) * (1 + taps // B + taps // B // 2)   # 3 195 912
    steps, warm = 40, 8
    g = np.random.Generator(np.random.PCG64(1004))
    decay = np.exp(-6.907755278982137 * np.arange(taps, dtype=np.float64) / (1.5 * 48000.0)).astype(np.float32)
    irs = g.standard_normal((n_irs, taps), dtype=np.float32) * decay
    irs /= np.sqrt(np.sum(irs.astype(np.float64) ** 2, axis=1, keepdims=True)).astype(np.float32)
    conv = Convolution(dev, Convolution.Mode.partitioned(blockSize=B), channels=C)
    conv.setKernel(irs, channelToKernel=[c // 2 for c in range(C)])
    del irs
    x = Tensor(dev, (C, (steps + warm) * B))
    y = Tensor(dev, (C, (steps + warm) * B))
    host = torch.empty((C, (steps + warm) * B), dtype=torch.float32, pin_memory=True)
    host.normal_(0.0, 0.1, generator=torch.Generator().manual_seed(1014))
    x.copyAsync(host.data_ptr(), x.byteSize)
    dev.synchronize(60)
    stride = (steps + warm) * B

    def do(t):
        st = lib.ma_pconv_step_dev(conv._h, ctypes.c_void_p(x.pointer + 4 * t * B), stride,
                                   ctypes.c_void_p(y.pointer + 4 * t * B), stride)
        if st != 0:
            raise RuntimeError(f"ma_pconv_step_dev failed: {st}")

    for t in range(warm):
        do(t)
    dev.synchronize(60)
    l0 = lib.ma_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for t in range(warm, warm + steps):
        do(t)
    e1.record(stream)
    dev.synchronize(120)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = int(lib.ma_kernel_launch_count() - l0)
    gbs = C * bytes_per_channel_block / (ms * 1e-3) / 1e9
    out = {"workload": f"partitioned convolution: {C} channels, {n_irs} impulse responses of 262144 taps (one per "
                       "channel pair), block 64 (FFT 128, 4096 partitions), streaming steps",
           "metric": "conv_channel_samples_per_s", "value": C * B / (ms * 1e-3), "unit": "channel-samples/s",
           "ms_per_step": ms, "steps": steps, "gpu_launches": launches,
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "algorithmic_bytes_per_channel_block": bytes_per_channel_block,
                        "kernel": "pconv_mac_kernel + r2c + c2r per step"}}
    x.free()
    y.free()
    conv.close()
    return out


def bench_large(dev, lib, torch, stream, peak):
    """65536-point forward + inverse batch (configuration 5)."""
    from metalaudio_b200 import FFT, Tensor, WindowType
    n, batch = LARGE["n"], LARGE["batch"]
    fft = FFT(dev, FFT.Config(size=n, windowType=WindowType.none))
    x = Tensor(dev, (batch, n))
    z = Tensor(dev, (batch, n // 2 + 1, 2))
    y = Tensor(dev, (batch, n))
    host = torch.empty((batch, n), dtype=torch.float32, pin_memory=True)
    host.normal_(0.0, 1.0, generator=torch.Generator().manual_seed(1005))
    x.copyAsync(host.data_ptr(), x.byteSize)
    dev.synchronize(60)

    def pair():
        a = lib.ma_fft_forward_dev(fft._h, ctypes.c_void_p(x.pointer), ctypes.c_void_p(z.pointer), None, None, 0,
                                   1.0, batch, 0)
        b = lib.ma_fft_inverse_dev(fft._h, ctypes.c_void_p(z.pointer), None, ctypes.c_void_p(y.pointer), batch, 0)
        if a != 0 or b != 0:
            raise RuntimeError(f"large FFT failed: {a} {b}")

    for _ in range(3):
        pair()
    dev.synchronize(60)
    reps = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        pair()
    e1.record(stream)
    dev.synchronize(120)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    nbytes = 2 * batch * (n * 4 + (n // 2 + 1) * 8)
    gbs = nbytes / (ms * 1e-3) / 1e9
    out = {"workload": "4096 x 65536-point real forward + inverse", "metric": "fft65536_pairs_per_s",
           "value": batch / (ms * 1e-3), "unit": "pairs/s", "ms_per_pair_batch": ms,
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "algorithmic_bytes": nbytes}}
    fft.close()
    for t in (x, y, z):
        t.free()
    return out


def bench_next_rows(dev, lib, torch, stream, peak, small=False):
    """The callers either side of the hot path: STFT / iSTFT through the magnitude + phase layout
    (64 signals of configuration 2's shape) and the one-shot FFT convolution (32 signals, 131072-tap
    kernel, 2^20-point transforms).  Device-resident, CUDA-event timed, best of 5 after a warm-up."""
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

    def ptr(t):
        return ctypes.c_void_p(t.data_ptr())

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
    # --- one-shot FFT convolution
    sig, taps, nfft = (8 if small else 32), 131072, 1 << 20
    length = nfft - taps + 1
    h = decaying_ir(taps)
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
    from metalaudio_b200 import AudioDevice
    dev = AudioDevice(local_rank)
    lib = dev._lib
    stream = torch.cuda.ExternalStream(lib.ma_context_stream(dev.handle), device=torch.device("cuda", local_rank))
    peak, _ = measured_peak_gbs()
    if args.only == "next":
        res = bench_next_rows(dev, lib, torch, stream, peak, small=args.small)
    elif args.only == "conv4":
        res = bench_conv4(dev, lib, torch, stream, peak, channels=256 if args.small else 1024)
    elif args.only == "conv":
        res = bench_conv(dev, lib, torch, stream, peak, whole_signal=True if args.small else None)
    else:
        res = bench_large(dev, lib, torch, stream, peak)
    print(json.dumps({args.only: res}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extras", action="store_true", help="skip the convolution and 65536-point lines")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--signals", type=int, default=SIGNALS_PER_GPU,
                    help="signals per GPU (default: the benchmark configuration's 256; smaller for profiler captures)")
    ap.add_argument("--conv-channels", type=int, default=CONV["channels"])
    ap.add_argument("--large-batch", type=int, default=LARGE["batch"])
    ap.add_argument("--small", action="store_true", help="with --only next / conv4: a quarter-size case for profiler captures; with --only conv: run the "
                         "whole-signal call at any channel count")
    ap.add_argument("--only", choices=["conv", "conv4", "large", "next"], default=None,
                    help="run just one of the extra workloads (profiler captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    CONV["channels"] = args.conv_channels
    LARGE["batch"] = args.large_batch
    if args.only is not None:
        run_only(args, local_rank)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
