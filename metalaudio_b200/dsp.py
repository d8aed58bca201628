"""Host-side mirror of the reference's public MetalDSP API for the FFT / STFT / partitioned
convolution path, over the C ABI (``include/metalaudio_cuda.h``).

Names, argument meaning and error behaviour follow the Swift API so that tests read like
the reference's XCTest suites:

* ``AudioDevice``                       Sources/MetalAudioKit/Core/AudioDevice.swift:222
* ``Tensor``                            Sources/MetalAudioKit/Buffers/Tensor.swift:12
* ``FFT``, ``FFT.Config``, ``WindowType``, ``COLACompliance``, ``FFTError``
                                        Sources/MetalDSP/FFT.swift:12-55, :155-348, :441-495, :818-919, :1780-1847
* ``FFT.stft`` / ``istft`` / ``forwardBatch`` / ``inverseBatch`` / ``STFTResult``
                                        Sources/MetalDSP/STFT.swift:10-22, :40-128, :327-527
* ``Convolution`` (``.partitioned``), ``ConvolutionError``
                                        Sources/MetalDSP/Convolution.swift:8-47, :112-125, :176-383, :529-775

Every transform runs on the CUDA backend; there is no size routing and no CPU fallback.
numpy arrays stand in for Swift ``[Float]`` / ``UnsafePointer<Float>``.
"""
from __future__ import annotations

import ctypes
import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L

_INT_MAX = (1 << 63) - 1


# --------------------------------------------------------------------------- errors

class MetalAudioError(Exception):
    """Sources/MetalAudioKit/Core/AudioDevice.swift:11-77."""

    def __init__(self, case: str, message: str = ""):
        self.case = case
        super().__init__(message or case)

    @staticmethod
    def invalidConfiguration(msg: str) -> "MetalAudioError":
        return MetalAudioError("invalidConfiguration", f"Invalid configuration: {msg}")

    @staticmethod
    def bufferSizeMismatch(expected: int, actual: int) -> "MetalAudioError":
        e = MetalAudioError("bufferSizeMismatch", f"Buffer size mismatch: expected {expected} bytes, got {actual}")
        e.expected, e.actual = expected, actual
        return e


class FFTError(Exception):
    """Sources/MetalDSP/FFT.swift:12-55; ``case`` holds the Swift case name and the payload
    is kept as attributes; ``errorDescription`` carries the same text."""

    def __init__(self, case: str, description: str, **payload):
        self.case = case
        self.errorDescription = description
        self.__dict__.update(payload)
        super().__init__(description)

    @staticmethod
    def inputTooShort(inputSize: int, requiredSize: int) -> "FFTError":
        return FFTError("inputTooShort",
                        f"Input size {inputSize} is shorter than the required FFT size {requiredSize}. "
                        f"Provide at least {requiredSize} samples, or use a smaller FFT size.",
                        inputSize=inputSize, requiredSize=requiredSize)

    @staticmethod
    def sizeTooLarge(requestedSize: int, maxSize: int) -> "FFTError":
        return FFTError("sizeTooLarge", f"FFT size {requestedSize} exceeds maximum supported size {maxSize}.",
                        requestedSize=requestedSize, maxSize=maxSize)

    @staticmethod
    def sizeNotPowerOf2(size: int) -> "FFTError":
        return FFTError("sizeNotPowerOf2",
                        f"FFT size {size} is not a power of 2. Use sizes like 256, 512, 1024, 2048, etc.", size=size)

    @staticmethod
    def invalidHopSize(hopSize: int, fftSize: int) -> "FFTError":
        return FFTError("invalidHopSize", f"Hop size {hopSize} is invalid. Must be > 0 and <= FFT size ({fftSize}).",
                        hopSize=hopSize, fftSize=fftSize)

    @staticmethod
    def batchSizeOverflow(batchSize: int, fftSize: int) -> "FFTError":
        return FFTError("batchSizeOverflow",
                        f"Batch size {batchSize} with FFT size {fftSize} would overflow buffer limits.",
                        batchSize=batchSize, fftSize=fftSize)

    @staticmethod
    def istftOutputOverflow(frameCount: int, hopSize: int, fftSize: int) -> "FFTError":
        return FFTError("istftOutputOverflow",
                        f"ISTFT output length calculation overflowed: frameCount={frameCount}, hopSize={hopSize}, "
                        f"fftSize={fftSize}. Use smaller STFT result or process in chunks.",
                        frameCount=frameCount, hopSize=hopSize, fftSize=fftSize)

    @staticmethod
    def istftFrameOverflow(frameIndex: int, hopSize: int, fftSize: int, outputLength: int) -> "FFTError":
        return FFTError("istftFrameOverflow",
                        f"ISTFT frame {frameIndex} position overflow: frameIndex*hopSize={frameIndex}*{hopSize} + "
                        f"fftSize={fftSize} exceeds outputLength={outputLength}. "
                        "STFT result may be corrupted or parameters are inconsistent.",
                        frameIndex=frameIndex, hopSize=hopSize, fftSize=fftSize, outputLength=outputLength)


class ConvolutionError(Exception):
    """Sources/MetalDSP/Convolution.swift:8-47."""

    def __init__(self, case: str, description: str, **payload):
        self.case = case
        self.errorDescription = description
        self.__dict__.update(payload)
        super().__init__(description)

    @staticmethod
    def inputSizeMismatch(inputSize: int, expectedMaxSize: int, fftSize: int) -> "ConvolutionError":
        return ConvolutionError("inputSizeMismatch",
                                f"Convolution input size {inputSize} exceeds expected maximum {expectedMaxSize} "
                                f"(FFT size: {fftSize}). This would cause circular convolution artifacts. "
                                "Call setKernel() with a larger expectedInputSize parameter.",
                                inputSize=inputSize, expectedMaxSize=expectedMaxSize, fftSize=fftSize)

    @staticmethod
    def kernelNotConfigured() -> "ConvolutionError":
        return ConvolutionError("kernelNotConfigured",
                                "Convolution kernel has not been set. Call setKernel() before processing.")

    @staticmethod
    def emptyKernel() -> "ConvolutionError":
        return ConvolutionError("emptyKernel", "Convolution kernel cannot be empty. Provide at least one sample.")

    @staticmethod
    def fftNotInitialized() -> "ConvolutionError":
        return ConvolutionError("fftNotInitialized",
                                "FFT resources failed to initialize. This may indicate a Metal device error.")

    @staticmethod
    def invalidPartitionState(reason: str) -> "ConvolutionError":
        return ConvolutionError("invalidPartitionState",
                                f"Partitioned convolution is in an invalid state: {reason}", reason=reason)

    @staticmethod
    def outputSizeOverflow(inputSize: int, kernelSize: int) -> "ConvolutionError":
        return ConvolutionError("outputSizeOverflow",
                                f"Output size would overflow: input ({inputSize}) + kernel ({kernelSize}) - 1 exceeds "
                                "Int.max. Use smaller buffers or process in chunks.",
                                inputSize=inputSize, kernelSize=kernelSize)


# FFT.swift:63: global switch of the sampled NaN / Inf check on transform outputs (the reference
# always checks in DEBUG builds and only behind this flag in release builds).  Set once at start-up.
fftValidationEnabled: bool = False
# Messages of the latest validation warnings (the reference sends them to os.log at debug level).
fftValidationLog: List[str] = []


def validateFFTOutput(buffer, count: int, context: str) -> bool:
    """FFT.swift:80-134: looks at about 50 evenly spaced values plus the last one (never the whole
    buffer), reports the first NaN and the first Inf it meets, never raises.  Returns True when
    either was found.  Does nothing unless ``fftValidationEnabled`` is set."""
    if not fftValidationEnabled or count <= 0:
        return False
    buf = np.asarray(buffer).reshape(-1)
    sample_count = min(50, count)
    stride = max(1, count // sample_count)
    nan_index = inf_index = -1
    i = 0
    while i < count and (nan_index < 0 or inf_index < 0):
        v = buf[i]
        if nan_index < 0 and np.isnan(v):
            nan_index = i
        if inf_index < 0 and np.isinf(v):
            inf_index = i
        i += stride
    if count > 1:
        last = buf[count - 1]
        if nan_index < 0 and np.isnan(last):
            nan_index = count - 1
        if inf_index < 0 and np.isinf(last):
            inf_index = count - 1
    if nan_index >= 0:
        fftValidationLog.append(f"[FFT] Warning: NaN detected in {context} near index {nan_index}")
    if inf_index >= 0:
        fftValidationLog.append(f"[FFT] Warning: Inf detected in {context} near index {inf_index}")
    del fftValidationLog[:-64]
    return nan_index >= 0 or inf_index >= 0


def _raise_status(st: int, where: str = "") -> None:
    """Map a C status onto the reference's error vocabulary."""
    if st == L.MA_OK:
        return
    lib = L.load()
    text = lib.ma_status_string(st).decode()
    if st == L.MA_ERR_DEVICE_LOST:
        raise MetalAudioError("deviceLost", f"{where}: {text}")
    if st == L.MA_ERR_TIMEOUT:
        raise MetalAudioError("gpuTimeout", f"{where}: {text}")
    if st == L.MA_ERR_ALLOC:
        raise MetalAudioError("bufferAllocationFailed", f"{where}: {text}")
    if st == L.MA_ERR_CUDA:
        raise MetalAudioError("gpuExecutionError", f"{where}: {text} (cudaError {lib.ma_last_cuda_error()})")
    if st == L.MA_ERR_KERNEL_NOT_CONFIGURED:
        raise ConvolutionError.fftNotInitialized()
    raise MetalAudioError("invalidConfiguration", f"{where}: {text}")


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# --------------------------------------------------------------------------- device / tensor

class AudioDevice:
    """CUDA device + stream context (AudioDevice.swift:222, :323; ComputeContext's
    executeSync / executeSyncWithTiming slice, ComputeContext.swift:154-297)."""

    def __init__(self, deviceIndex: int = 0, pinnedBytes: int = 0):
        self._lib = L.load()
        h = ctypes.c_void_p()
        st = self._lib.ma_context_create(int(deviceIndex), int(pinnedBytes), ctypes.byref(h))
        if st != L.MA_OK:
            if st == L.MA_ERR_DEVICE_LOST:
                raise MetalAudioError("deviceNotFound", "No CUDA device found; this library has no CPU fallback")
            _raise_status(st, "AudioDevice()")
        self._h = h
        self.deviceIndex = int(deviceIndex)

    @property
    def handle(self):
        return self._h

    @property
    def name(self) -> str:
        buf = ctypes.create_string_buffer(256)
        self._lib.ma_context_device_name(self._h, buf, 256)
        return buf.value.decode()

    @property
    def isDeviceAvailable(self) -> bool:
        v = ctypes.c_int32(0)
        self._lib.ma_context_is_available(self._h, ctypes.byref(v))
        return bool(v.value)

    def markDeviceLost(self) -> None:
        """AudioDevice.swift:434-472: every later call throws ``deviceLost``."""
        self._lib.ma_context_mark_lost(self._h)

    def ensureAvailable(self) -> None:
        if not self.isDeviceAvailable:
            raise MetalAudioError("deviceLost", "GPU device was lost")

    def synchronize(self, timeout: float = 2.0) -> None:
        """ComputeContext.executeSync's wait with its 2 s default (ComputeContext.swift:137)."""
        _raise_status(self._lib.ma_context_sync(self._h, float(timeout)), "synchronize")

    def timingBegin(self) -> None:
        _raise_status(self._lib.ma_timing_begin(self._h), "timingBegin")

    def timingEnd(self) -> float:
        """Milliseconds of device time since timingBegin (executeSyncWithTiming)."""
        ms = ctypes.c_float(0)
        _raise_status(self._lib.ma_timing_end(self._h, ctypes.byref(ms)), "timingEnd")
        return float(ms.value)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ma_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Tensor:
    """float32 device buffer with a shape (Tensor.swift:59, :272, :325, :390)."""

    def __init__(self, device: AudioDevice, shape: Sequence[int]):
        self.device = device
        self.shape = tuple(int(s) for s in shape)
        self.count = int(np.prod(self.shape)) if len(self.shape) else 1
        p = ctypes.c_void_p()
        _raise_status(device._lib.ma_buffer_alloc(device.handle, self.count * 4, ctypes.byref(p)), "Tensor()")
        self._p = p

    @property
    def pointer(self) -> int:
        return self._p.value

    @property
    def byteSize(self) -> int:
        return self.count * 4

    def copy(self, from_: np.ndarray) -> None:
        a = _f32(from_)
        if a.size != self.count:
            raise MetalAudioError("bufferSizeMismatch", f"expected {self.count} elements, got {a.size}")
        _raise_status(self.device._lib.ma_memcpy_h2d(self.device.handle, self._p, _ptr(a), a.nbytes), "Tensor.copy")

    def toArray(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=np.float32)
        _raise_status(self.device._lib.ma_memcpy_d2h(self.device.handle, _ptr(out), self._p, out.nbytes),
                      "Tensor.toArray")
        return out

    def copyAsync(self, from_ptr: int, nbytes: int) -> None:
        """Stream-ordered host->device copy from PINNED host memory at ``from_ptr``."""
        _raise_status(self.device._lib.ma_memcpy_h2d_async(self.device.handle, self._p, ctypes.c_void_p(from_ptr),
                                                          nbytes), "Tensor.copyAsync")

    def copyToAsync(self, to_ptr: int, nbytes: int) -> None:
        """Stream-ordered device->host copy into PINNED host memory at ``to_ptr``."""
        _raise_status(self.device._lib.ma_memcpy_d2h_async(self.device.handle, ctypes.c_void_p(to_ptr), self._p,
                                                          nbytes), "Tensor.copyToAsync")

    def rows(self, first: int, count: int, device: Optional["AudioDevice"] = None) -> "Tensor":
        """Non-owning view of `count` leading-dimension rows starting at `first`, optionally bound to
        another AudioDevice (stream) of the same GPU, so independent row ranges can be processed on
        different streams."""
        v = Tensor.__new__(Tensor)
        v.device = device if device is not None else self.device
        v.shape = (int(count),) + self.shape[1:]
        v.count = int(np.prod(v.shape))
        row_elems = int(np.prod(self.shape[1:])) if len(self.shape) > 1 else 1
        v._p = ctypes.c_void_p(self._p.value + 4 * row_elems * int(first))
        v._view = True
        return v

    def zero(self) -> None:
        _raise_status(self.device._lib.ma_buffer_zero(self.device.handle, self._p, self.byteSize), "Tensor.zero")

    def free(self) -> None:
        if getattr(self, "_view", False):
            self._p = None
            return
        if getattr(self, "_p", None) and self.device._h:
            self.device._lib.ma_buffer_free(self.device.handle, self._p)
        self._p = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# --------------------------------------------------------------------------- FFT

class WindowType(enum.Enum):
    """FFT.swift:260-327."""
    none = "none"
    hann = "hann"
    hamming = "hamming"
    blackman = "blackman"

    def coefficient(self, at: int, length: int) -> np.float32:
        """Symmetric window (denominator N-1) evaluated in float64 (FFT.swift:268-294)."""
        if length <= 1:
            return np.float32(1.0)
        n = float(at)
        denom = float(length) - 1.0
        if self is WindowType.none:
            return np.float32(1.0)
        if self is WindowType.hann:
            return np.float32(0.5 * (1.0 - math.cos(2.0 * math.pi * n / denom)))
        if self is WindowType.hamming:
            return np.float32(0.54 - 0.46 * math.cos(2.0 * math.pi * n / denom))
        return np.float32(0.42 - 0.5 * math.cos(2.0 * math.pi * n / denom) + 0.08 * math.cos(4.0 * math.pi * n / denom))

    def table(self, length: int) -> np.ndarray:
        if length <= 1 or self is WindowType.none:
            return np.ones(length, dtype=np.float32)
        n = np.arange(length, dtype=np.float64)
        d = float(length) - 1.0
        if self is WindowType.hann:
            w = 0.5 * (1.0 - np.cos(2.0 * np.pi * n / d))
        elif self is WindowType.hamming:
            w = 0.54 - 0.46 * np.cos(2.0 * np.pi * n / d)
        else:
            w = 0.42 - 0.5 * np.cos(2.0 * np.pi * n / d) + 0.08 * np.cos(4.0 * np.pi * n / d)
        return w.astype(np.float32)

    @property
    def colaHopDivisors(self) -> List[int]:
        return {WindowType.none: [1], WindowType.hann: [2, 4], WindowType.hamming: [], WindowType.blackman: [3, 4]}[self]

    @property
    def name_(self) -> str:
        return {WindowType.none: "rectangular", WindowType.hann: "Hann", WindowType.hamming: "Hamming",
                WindowType.blackman: "Blackman"}[self]


class COLACompliance(enum.Enum):
    """FFT.swift:330-348."""
    perfect = "perfect"
    nearPerfect = "nearPerfect"
    nonCompliant = "nonCompliant"

    @property
    def description(self) -> str:
        return {COLACompliance.perfect: "Perfect COLA - guaranteed perfect reconstruction",
                COLACompliance.nearPerfect: "Near-perfect COLA - reconstruction error typically < 0.1%",
                COLACompliance.nonCompliant: "Non-COLA - reconstruction may have artifacts"}[self]


class Backend(enum.Enum):
    """FFT.swift:1519-1550.  Kept for source compatibility; every size runs on ``cuda``."""
    vdsp = "vdsp"
    gpu = "gpu"
    mpsGraph = "mpsGraph"
    cuda = "cuda"


@dataclass
class STFTResult:
    """STFT.swift:10-22: ``real`` / ``imag`` are (frameCount, fftSize) arrays (the reference's
    array-of-arrays, full-N split layout)."""
    real: np.ndarray
    imag: np.ndarray

    @property
    def frameCount(self) -> int:
        return int(len(self.real))

    @property
    def binCount(self) -> int:
        return int(self.real.shape[1]) if self.frameCount else 0


class ToleranceProvider:
    """The two fields of ToleranceConfiguration the path reads
    (Sources/MetalAudioKit/Config/ToleranceConfiguration.swift:166-181: ``conservative()``,
    which is what an unknown GPU family maps to)."""
    windowFloorEpsilon: float = 1e-8
    fftAccuracy: float = 1e-6
    convolutionAccuracy: float = 1e-6


def validatedWindowFloor(configured: Optional[float] = None) -> float:
    """STFT.swift:491-501."""
    c = np.float32(ToleranceProvider.windowFloorEpsilon if configured is None else configured)
    if c < np.float32(1e-10):
        return 1e-6
    if c > np.float32(0.1):
        return 0.1
    return float(c)


class FFT:
    """FFT.swift:155.  One CUDA plan per object."""

    maxFFTSize = 1 << 24  # FFT.swift:422

    @dataclass
    class Config:
        """FFT.swift:158-258."""
        size: int
        inverse: bool = False
        windowType: WindowType = WindowType.hann
        hopSize: Optional[int] = None

        def __post_init__(self):
            if self.hopSize is None:
                self.hopSize = max(1, self.size // 4)

        @property
        def colaCompliance(self) -> COLACompliance:
            divs = self.windowType.colaHopDivisors
            if not divs:
                if self.windowType is WindowType.hamming and self.hopSize in (self.size // 2, self.size // 4):
                    return COLACompliance.nearPerfect
                return COLACompliance.nonCompliant
            for d in divs:
                if self.size % d == 0 and self.hopSize == self.size // d:
                    return COLACompliance.perfect
            return COLACompliance.nonCompliant

        @property
        def overlapPercent(self) -> int:
            return 100 - (self.hopSize * 100 // self.size)

        def validateCOLA(self):
            c = self.colaCompliance
            w = self.windowType.name_
            if c is COLACompliance.perfect:
                return True, c, f"{w} window with hop size {self.hopSize} (overlap {self.overlapPercent}%) satisfies COLA"
            if c is COLACompliance.nearPerfect:
                return True, c, f"{w} window with hop size {self.hopSize} is near-COLA (error < 0.1%)"
            hops = []
            for d in self.windowType.colaHopDivisors:
                if self.size % d == 0:
                    hop = self.size // d
                    hops.append(f"{hop} ({100 - (hop * 100 // self.size)}% overlap)")
            sug = ("Suggested hop sizes: " + ", ".join(hops)) if hops else \
                "Consider using Hann window for COLA-compliant STFT"
            return False, c, f"{w} window with hop size {self.hopSize} does not satisfy COLA. {sug}"

    def __init__(self, device: AudioDevice, config: "FFT.Config", window: Optional[np.ndarray] = None):
        """``window`` overrides the table built from ``config.windowType`` (e.g. a periodic
        Hann); the reference always builds the symmetric table (FFT.swift:461)."""
        n = int(config.size)
        if n <= 0 or (n & (n - 1)) != 0:
            raise FFTError.sizeNotPowerOf2(n)
        if n > FFT.maxFFTSize:
            raise FFTError.sizeTooLarge(n, FFT.maxFFTSize)
        if config.hopSize <= 0 or config.hopSize > n:
            raise FFTError.invalidHopSize(config.hopSize, n)
        if n < 2:
            raise MetalAudioError.invalidConfiguration("FFT size 1 is not served by the CUDA backend")
        self.device = device
        self.config = config
        self.size = n
        self._lib = device._lib
        self.window = _f32(window) if window is not None else config.windowType.table(n)
        if self.window.size != n:
            raise MetalAudioError.invalidConfiguration("window table must have `size` coefficients")
        has_window = window is not None or config.windowType is not WindowType.none
        h = ctypes.c_void_p()
        st = self._lib.ma_fft_plan_create(device.handle, n, _ptr(self.window) if has_window else None,
                                          int(config.hopSize), ctypes.byref(h))
        _raise_status(st, "FFT.init")
        self._h = h

    # ---- single transforms (pointer API of the reference; arrays here)
    def forward(self, input: np.ndarray, outputReal: np.ndarray, outputImag: np.ndarray) -> None:
        """FFT.swift:818-855: unnormalised DFT of N real samples into real[N], imag[N].
        Direction follows ``config.inverse`` as in the reference (one vDSP setup serves both
        methods, FFT.swift:470-482): an ``inverse: true`` object conjugates."""
        n = self.size
        x = _f32(input).reshape(-1)[:n]
        st = self._lib.ma_fft_forward_host(self._h, _ptr(x), _ptr(outputReal), _ptr(outputImag), None, 0, 1.0, 1,
                                           L.LAYOUT_FULL_SPLIT)
        if st != L.MA_OK:  # non-throwing API: outputs zeroed on failure (FFT.swift:826-835)
            outputReal[:n] = 0
            outputImag[:n] = 0
            return
        if self.config.inverse:
            outputImag[:n] *= -1.0
        validateFFTOutput(outputReal, n, "outputReal")   # FFT.swift:853-854
        validateFFTOutput(outputImag, n, "outputImag")

    def inverse(self, inputReal: np.ndarray, inputImag: np.ndarray, output: np.ndarray) -> None:
        """FFT.swift:889-919: real part of the DFT in the object's direction, times 1/N.
        With ``config.inverse == True`` this is the inverse transform; a forward-configured
        object returns the time-reversed sequence, as the reference does."""
        n = self.size
        re = _f32(inputReal).reshape(-1)[:n]
        im = _f32(inputImag).reshape(-1)[:n]
        out = np.empty(n, dtype=np.float32)
        st = self._lib.ma_fft_inverse_host(self._h, _ptr(re), _ptr(im), _ptr(out), 1, L.LAYOUT_FULL_SPLIT)
        if st != L.MA_OK:
            output[:n] = 0
            return
        if not self.config.inverse:
            out = np.concatenate([out[:1], out[1:][::-1]])
        output[:n] = out
        validateFFTOutput(output, n, "inverse.output")   # FFT.swift:917-918

    def _mag(self, real, imag, out, kind, reference=1.0):
        kh = self.size // 2 + 1
        re = _f32(real).reshape(-1)[:kh]
        im = _f32(imag).reshape(-1)[:kh]
        tmp = np.empty(kh, dtype=np.float32)
        st = self._lib.ma_fft_magnitude_host(self._h, _ptr(re), _ptr(im), _ptr(tmp), 1, kind, float(reference))
        _raise_status(st, "magnitude")
        out[:kh] = tmp

    def magnitude(self, real, imag, magnitude) -> None:
        """FFT.swift:1780-1791 (N/2+1 values)."""
        self._mag(real, imag, magnitude, L.MAG_MAGNITUDE)

    def power(self, real, imag, power) -> None:
        """FFT.swift:1804-1815."""
        self._mag(real, imag, power, L.MAG_POWER)

    def magnitudeDB(self, real, imag, magnitudeDB, reference: float = 1.0) -> None:
        """FFT.swift:1833-1847."""
        self._mag(real, imag, magnitudeDB, L.MAG_DB, reference)

    # ---- backend shims (FFT.swift:1552-1747): one backend, kept for source compatibility
    @property
    def optimalBackend(self) -> Backend:
        return Backend.cuda

    @property
    def shouldUseGPU(self) -> bool:
        return True

    @property
    def shouldUseMetal(self) -> bool:
        """FFT.swift:1537-1539: the reference's custom-kernel tier (2048 < N <= 8192).  Here the
        same sizes are the ones whose transform stays in shared memory in a single pass."""
        return 2048 < self.size <= 8192

    @property
    def shouldUseMPSGraph(self) -> bool:
        """FFT.swift:1522-1527: the reference's size class above 8192 points, served here by the
        multi-pass kernels."""
        return self.size > 8192

    def _complex(self, input, output, inverse: bool, context: str) -> Backend:
        n2 = 2 * self.size
        if len(input) < n2:
            raise MetalAudioError.bufferSizeMismatch(n2, len(input))
        x = _f32(np.asarray(input, dtype=np.float32).reshape(-1)[:n2])   # oversized inputs are truncated
        out = np.empty(n2, dtype=np.float32)
        st = self._lib.ma_fft_complex_host(self._h, _ptr(x), _ptr(out), 1, 1 if inverse else 0)
        _raise_status(st, context)
        if isinstance(output, list):          # the reference resizes its inout array
            output[:] = out.tolist()
        else:
            if len(output) < n2:
                raise MetalAudioError.bufferSizeMismatch(n2, len(output))
            output[:n2] = out
        validateFFTOutput(out, n2, context + ".output")
        return Backend.cuda

    def forwardGPU(self, input, output) -> Backend:
        """FFT.swift:945-1107: complex forward DFT of N interleaved (re, im) pairs (2N floats in,
        2N floats out, unscaled).  Inputs shorter than 2N raise bufferSizeMismatch, longer ones are
        truncated; ``output`` may be a list (resized) or an array of at least 2N floats."""
        return self._complex(input, output, False, "forwardGPU")

    def inverseGPU(self, input, output) -> Backend:
        """FFT.swift:1176-1315: complex inverse DFT with the 1/N scale, same data format."""
        return self._complex(input, output, True, "inverseGPU")

    def forwardMPSGraph(self, input, outputReal, outputImag) -> None:
        """FFT.swift:1372-1431: real input, split real / imag output of N values each.  One
        backend: the same kernels as forward()."""
        if len(input) < self.size:
            raise FFTError.inputTooShort(len(input), self.size)
        self._split_out(np.asarray(input), outputReal, outputImag, "forwardMPSGraph")

    def inverseMPSGraph(self, inputReal, inputImag, output) -> None:
        """FFT.swift:1445-1515: split spectrum in, N real samples out with the 1/N scale (a true
        inverse whatever ``config.inverse`` says, as the graph in the reference is)."""
        n = self.size
        if len(inputReal) < n or len(inputImag) < n:
            raise FFTError.inputTooShort(min(len(inputReal), len(inputImag)), n)
        out = self.inverseBatch(np.asarray(inputReal, dtype=np.float32).reshape(1, -1)[:, :n],
                                np.asarray(inputImag, dtype=np.float32).reshape(1, -1)[:, :n])[0]
        if isinstance(output, list):
            output[:] = out.tolist()
        else:
            output[:n] = out
        validateFFTOutput(out, n, "inverseMPSGraph.output")

    def _split_out(self, x, outputReal, outputImag, context: str) -> None:
        n = self.size
        re, im = self.forwardBatch(np.asarray(x, dtype=np.float32).reshape(1, -1)[:, :n])
        for dst, src in ((outputReal, re[0]), (outputImag, im[0])):
            if isinstance(dst, list):
                dst[:] = src.tolist()
            else:
                dst[:n] = src
        validateFFTOutput(re[0], n, context + ".outputReal")
        validateFFTOutput(im[0], n, context + ".outputImag")

    def warmup(self) -> None:
        x = np.zeros(self.size, dtype=np.float32)
        r = np.zeros(self.size, dtype=np.float32)
        i = np.zeros(self.size, dtype=np.float32)
        self.forward(x, r, i)

    def forwardAuto(self, input, outputReal, outputImag) -> Backend:
        if len(input) < self.size:
            raise FFTError.inputTooShort(len(input), self.size)
        self.forward(np.asarray(input), outputReal, outputImag)
        return Backend.cuda

    def inverseAuto(self, inputReal, inputImag, output) -> Backend:
        self.inverse(inputReal, inputImag, output)
        return Backend.cuda

    # ---- batches
    def forwardBatch(self, inputs: np.ndarray):
        """STFT.swift:94-128: batch of forward transforms; returns (real, imag) (B, N)."""
        n = self.size
        inputs = np.asarray(inputs, dtype=np.float32)
        if inputs.size == 0:
            return np.zeros((0, n), np.float32), np.zeros((0, n), np.float32)
        for idx, row in enumerate(inputs):
            if len(row) < n:
                raise FFTError.inputTooShort(len(row), n)
        x = _f32(inputs[:, :n])
        b = x.shape[0]
        if b * n > _INT_MAX // 8:
            raise FFTError.batchSizeOverflow(b, n)
        re = np.empty((b, n), np.float32)
        im = np.empty((b, n), np.float32)
        st = self._lib.ma_fft_forward_host(self._h, _ptr(x), _ptr(re), _ptr(im), None, 0, 1.0, b, L.LAYOUT_FULL_SPLIT)
        _raise_status(st, "forwardBatch")
        return re, im

    def inverseBatch(self, inputsReal: np.ndarray, inputsImag: np.ndarray) -> np.ndarray:
        """STFT.swift:327-373 with the true inverse transform."""
        n = self.size
        re = _f32(inputsReal)
        im = _f32(inputsImag)
        if re.size == 0:
            return np.zeros((0, n), np.float32)
        b = re.shape[0]
        out = np.empty((b, n), np.float32)
        st = self._lib.ma_fft_inverse_host(self._h, _ptr(re), _ptr(im), _ptr(out), b, L.LAYOUT_FULL_SPLIT)
        _raise_status(st, "inverseBatch")
        return out

    # ---- STFT / iSTFT
    def frameCount(self, inputLength: int) -> int:
        if inputLength < self.size:
            raise FFTError.inputTooShort(inputLength, self.size)
        return (inputLength - self.size) // self.config.hopSize + 1

    def stft(self, input: np.ndarray) -> STFTResult:
        """STFT.swift:40-81: frames at i*hop, analysis window, forward DFT, full-N split."""
        x = _f32(input).reshape(-1)
        f = self.frameCount(x.size)
        n = self.size
        re = np.empty((f, n), np.float32)
        im = np.empty((f, n), np.float32)
        st = self._lib.ma_stft_host(self._h, _ptr(x), x.size, x.size, 1, _ptr(re), _ptr(im), None, 0, 1.0,
                                    L.LAYOUT_FULL_SPLIT)
        _raise_status(st, "stft")
        return STFTResult(re, im)

    def istft(self, stft: STFTResult) -> np.ndarray:
        """STFT.swift:384-527.  Uses the true inverse transform per frame; the reference
        pushes frames through the object's forward-direction setup, which time-reverses
        them (its tests only assert loose structure)."""
        f = stft.frameCount
        if f == 0:
            return np.zeros(0, np.float32)
        n, hop = self.size, self.config.hopSize
        if (f - 1) * hop + n > _INT_MAX:
            raise FFTError.istftOutputOverflow(f, hop, n)
        if len(stft.real) < f or len(stft.imag) < f:
            raise FFTError.inputTooShort(min(len(stft.real), len(stft.imag)), f)
        out_len = (f - 1) * hop + n
        re = _f32(stft.real)
        im = _f32(stft.imag)
        out = np.empty(out_len, np.float32)
        st = self._lib.ma_istft_host(self._h, _ptr(re), _ptr(im), f, 1, _ptr(out), out_len,
                                     validatedWindowFloor(), L.LAYOUT_FULL_SPLIT)
        _raise_status(st, "istft")
        return out

    # ---- multi-signal, half-spectrum forms (device-friendly layout; not in the reference)
    def stftBatch(self, signals: np.ndarray, magnitude: bool = False):
        """STFT of (S, L) signals -> complex64 (S, F, N/2+1) [, float32 magnitudes]."""
        x = _f32(signals)
        s, length = x.shape
        f = self.frameCount(length)
        kh = self.size // 2 + 1
        spec = np.empty((s, f, kh, 2), np.float32)
        mag = np.empty((s, f, kh), np.float32) if magnitude else None
        st = self._lib.ma_stft_host(self._h, _ptr(x), length, length, s, _ptr(spec), None, _ptr(mag),
                                    L.MAG_MAGNITUDE, 1.0, L.LAYOUT_HALF_INTERLEAVED)
        _raise_status(st, "stftBatch")
        spec_c = spec.view(np.complex64).reshape(s, f, kh)
        return (spec_c, mag) if magnitude else spec_c

    def istftBatch(self, spectra: np.ndarray) -> np.ndarray:
        """Inverse of stftBatch: complex64 (S, F, N/2+1) -> (S, (F-1)*hop+N)."""
        z = np.ascontiguousarray(spectra, dtype=np.complex64)
        s, f, kh = z.shape
        out_len = (f - 1) * self.config.hopSize + self.size
        out = np.empty((s, out_len), np.float32)
        st = self._lib.ma_istft_host(self._h, _ptr(z.view(np.float32)), None, f, s, _ptr(out), out_len,
                                     validatedWindowFloor(), L.LAYOUT_HALF_INTERLEAVED)
        _raise_status(st, "istftBatch")
        return out

    def stftPolar(self, signals: np.ndarray):
        """STFT of (S, L) signals straight to magnitude and phase, float32 (S, F, N/2+1) each:
        the split HTDemucs does on the host after stft (HTDemucs.swift:726-741), fused into the
        transform so the complex spectrum never reaches memory."""
        x = _f32(signals)
        s, length = x.shape
        f = self.frameCount(length)
        kh = self.size // 2 + 1
        mag = np.empty((s, f, kh), np.float32)
        phase = np.empty((s, f, kh), np.float32)
        st = self._lib.ma_stft_host(self._h, _ptr(x), length, length, s, _ptr(mag), _ptr(phase), None,
                                    L.MAG_MAGNITUDE, 1.0, L.LAYOUT_HALF_POLAR)
        _raise_status(st, "stftPolar")
        return mag, phase

    def istftPolar(self, magnitude: np.ndarray, phase: np.ndarray) -> np.ndarray:
        """iSTFT from magnitude and phase (S, F, N/2+1): the polar -> complex rebuild with its
        conjugate mirror (HTDemucs.swift:795-812) fused into the inverse transform."""
        m = _f32(magnitude)
        ph = _f32(phase)
        if m.shape != ph.shape or m.ndim != 3:
            raise MetalAudioError.invalidConfiguration("magnitude and phase must both be (S, F, N/2+1)")
        s, f, kh = m.shape
        out_len = (f - 1) * self.config.hopSize + self.size
        out = np.empty((s, out_len), np.float32)
        st = self._lib.ma_istft_host(self._h, _ptr(m), _ptr(ph), f, s, _ptr(out), out_len,
                                     validatedWindowFloor(), L.LAYOUT_HALF_POLAR)
        _raise_status(st, "istftPolar")
        return out

    # ---- device-resident forms: Tensor in, Tensor out, nothing crosses PCIe
    def stftTensor(self, signals: "Tensor", spectrum: "Tensor", magnitude: Optional["Tensor"] = None) -> int:
        """STFT of a (S, L) signal Tensor into a (S, F, N/2+1, 2) spectrum Tensor (and a
        (S, F, N/2+1) magnitude Tensor).  Queued on the device stream; returns F."""
        s, length = signals.shape
        f = self.frameCount(length)
        st = self._lib.ma_stft_dev(self._h, ctypes.c_void_p(signals.pointer), length, length, s,
                                   ctypes.c_void_p(spectrum.pointer), None,
                                   ctypes.c_void_p(magnitude.pointer) if magnitude is not None else None,
                                   L.MAG_MAGNITUDE, 1.0, L.LAYOUT_HALF_INTERLEAVED)
        _raise_status(st, "stftTensor")
        return f

    def istftTensor(self, spectrum: "Tensor", output: "Tensor") -> None:
        """Inverse of stftTensor into a (S, out_stride) Tensor with out_stride >= (F-1)*hop+N."""
        s, f = spectrum.shape[0], spectrum.shape[1]
        st = self._lib.ma_istft_dev(self._h, ctypes.c_void_p(spectrum.pointer), None, f, s,
                                    ctypes.c_void_p(output.pointer), output.shape[1], validatedWindowFloor(),
                                    L.LAYOUT_HALF_INTERLEAVED)
        _raise_status(st, "istftTensor")

    def releaseGPUResources(self) -> None:
        """STFT.swift:537-542.  Device tables are a few KB; kept so the object stays usable."""

    def didReceiveMemoryPressure(self, level: str) -> None:
        """MemoryPressureResponder hook (STFT.swift:544-559)."""
        if level == "critical":
            self.releaseGPUResources()

    def close(self) -> None:
        if getattr(self, "_h", None) and self.device._h:
            self._lib.ma_fft_plan_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------- convolution

def spectrumToPolar(device: "AudioDevice", spectrum: "Tensor", magnitude: Optional["Tensor"],
                    phase: Optional["Tensor"]) -> None:
    """compute_magnitude + compute_phase (DSP.metal:784-813) over a Tensor of interleaved complex
    bins (last dimension 2); either output may be None."""
    st = device._lib.ma_spectrum_to_polar_dev(device.handle, ctypes.c_void_p(spectrum.pointer),
                                              ctypes.c_void_p(magnitude.pointer) if magnitude is not None else None,
                                              ctypes.c_void_p(phase.pointer) if phase is not None else None,
                                              spectrum.count // 2)
    _raise_status(st, "spectrumToPolar")


def polarToSpectrum(device: "AudioDevice", magnitude: "Tensor", phase: "Tensor", spectrum: "Tensor") -> None:
    """polar_to_complex (DSP.metal:821-834)."""
    st = device._lib.ma_polar_to_spectrum_dev(device.handle, ctypes.c_void_p(magnitude.pointer),
                                              ctypes.c_void_p(phase.pointer), ctypes.c_void_p(spectrum.pointer),
                                              magnitude.count)
    _raise_status(st, "polarToSpectrum")


def toDecibels(device: "AudioDevice", data: "Tensor", reference: float = 1.0, minDB: float = -100.0) -> None:
    """to_decibels in place (DSP.metal:861-881)."""
    st = device._lib.ma_to_decibels_dev(device.handle, ctypes.c_void_p(data.pointer), data.count, float(reference),
                                        float(minDB))
    _raise_status(st, "toDecibels")


class Convolution:
    """Convolution.swift:176.  ``Mode.partitioned`` and ``Mode.fft`` are served by this backend;
    ``Mode.direct`` (vDSP cross-correlation semantics, Convolution.swift:400-434) is not."""

    class Mode:
        """Convolution.swift:112-125."""

        def __init__(self, kind: str, blockSize: int = 0, useMPSGraphFFT: bool = False):
            self.kind = kind
            self.blockSize = blockSize
            self.useMPSGraphFFT = useMPSGraphFFT

        @staticmethod
        def partitioned(blockSize: int, useMPSGraphFFT: bool = False) -> "Convolution.Mode":
            return Convolution.Mode("partitioned", blockSize, useMPSGraphFFT)

        @staticmethod
        def fft() -> "Convolution.Mode":
            return Convolution.Mode("fft")

    def __init__(self, device: AudioDevice, mode: Optional["Convolution.Mode"] = None, channels: int = 1):
        """``channels`` > 1 runs that many independent channels through one object (the
        reference holds one object per channel).  The default mode is ``.fft``
        (Convolution.swift:176)."""
        if mode is None:
            mode = Convolution.Mode.fft()
        if mode.kind not in ("partitioned", "fft"):
            raise MetalAudioError.invalidConfiguration("only .partitioned and .fft modes are served by the CUDA backend")
        self.device = device
        self.mode = mode
        self.channels = int(channels)
        self.kernel = np.zeros(0, np.float32)
        self._lib = device._lib
        self._h = None
        self._fc = None           # .fft mode handle
        self.fftSize = 0
        self._expected = 0

    def setKernel(self, kernel: np.ndarray, expectedInputSize: Optional[int] = None,
                  channelToKernel: Optional[Sequence[int]] = None) -> None:
        """Convolution.swift:188-208 -> :250-322.  ``kernel`` may be (taps,) or (n_irs, taps)
        with ``channelToKernel`` mapping each channel to its impulse response."""
        k = _f32(kernel)
        if k.size == 0:
            raise ConvolutionError.emptyKernel()
        if self.mode.kind == "fft":
            return self._setup_fft(k, expectedInputSize)
        b = int(self.mode.blockSize)
        if b <= 0:
            raise MetalAudioError.invalidConfiguration(f"Block size must be positive, got {b}")
        if (b & (b - 1)) != 0:
            raise FFTError.sizeNotPowerOf2(2 * b)
        k2 = k.reshape(1, -1) if k.ndim == 1 else k
        self.kernel = k2[0] if k.ndim == 1 else k2
        self._taps = int(k2.shape[1])
        if self._h is None:
            h = ctypes.c_void_p()
            _raise_status(self._lib.ma_pconv_create(self.device.handle, b, self.channels, ctypes.byref(h)),
                          "Convolution.setKernel")
            self._h = h
        cmap = None
        if channelToKernel is not None:
            cmap = np.ascontiguousarray(channelToKernel, dtype=np.int32)
        st = self._lib.ma_pconv_set_kernels(self._h, _ptr(k2), self._taps, int(k2.shape[0]), _ptr(cmap))
        _raise_status(st, "Convolution.setKernel")

    def _setup_fft(self, k: np.ndarray, expectedInputSize: Optional[int]) -> None:
        """Convolution.swift:210-248: FFT size = next power of two >= expected + taps - 1."""
        if k.ndim != 1:
            raise MetalAudioError.invalidConfiguration(".fft mode takes one kernel")
        expected = int(k.size if expectedInputSize is None else expectedInputSize)
        if expected + k.size - 1 > (1 << 24):
            raise FFTError.sizeTooLarge(expected + int(k.size) - 1, 1 << 24)
        if self._fc is not None:
            self._lib.ma_fftconv_destroy(self._fc)
            self._fc = None
        h = ctypes.c_void_p()
        st = self._lib.ma_fftconv_create(self.device.handle, _ptr(k), int(k.size), expected, self.channels,
                                         ctypes.byref(h))
        _raise_status(st, "Convolution.setKernel")
        self._fc = h
        self.kernel = k
        self._taps = int(k.size)
        self._expected = expected
        n = ctypes.c_int64(0)
        self._lib.ma_fftconv_fft_size(h, ctypes.byref(n))
        self.fftSize = int(n.value)

    def _process_fft(self, x: np.ndarray, output: Optional[np.ndarray]) -> np.ndarray:
        """Convolution.swift:437-493: fftSize samples per signal, the linear convolution in the
        first len + taps - 1 of them."""
        if self._fc is None:
            raise ConvolutionError.fftNotInitialized()
        single = x.ndim == 1
        x2 = x.reshape(1, -1) if single else x
        if x2.shape[0] > self.channels:
            raise MetalAudioError.invalidConfiguration(f"expected at most {self.channels} signals, got {x2.shape[0]}")
        length = x2.shape[1]
        if length > self._expected:
            raise ConvolutionError.inputSizeMismatch(length, self._expected, self.fftSize)
        out = np.empty((x2.shape[0], self.fftSize), np.float32)
        st = self._lib.ma_fftconv_process_host(self._fc, _ptr(x2), length, length, x2.shape[0], _ptr(out))
        _raise_status(st, "Convolution.process")
        res = out[0] if single else out
        if output is not None and single and output.size >= self.fftSize:
            output[:self.fftSize] = res  # the inverse writes fftSize samples into the caller's array
            return output
        return res

    @property
    def partitionCount(self) -> int:
        v = ctypes.c_int32(0)
        if self._h is None:
            return 0
        self._lib.ma_pconv_partition_count(self._h, ctypes.byref(v))
        return int(v.value)

    @property
    def kernelTailLength(self) -> int:
        return 0 if (self._h is None and self._fc is None) else self._taps - 1

    def expectedOutputSize(self, forInputSize: int) -> int:
        return forInputSize if (self._h is None and self._fc is None) else forInputSize + self._taps - 1

    @property
    def maxInputSize(self) -> int:
        """Convolution.swift:377-383: the expected input size in .fft mode, 0 (no limit) otherwise."""
        return self._expected if self.mode.kind == "fft" else 0

    def process(self, input: np.ndarray, output: Optional[np.ndarray] = None) -> np.ndarray:
        """Convolution.swift:336-352 -> :529-758.  (L,) for one channel or (channels, L);
        returns the full L+K-1 samples per channel.  A caller-supplied ``output`` at least
        that long is zeroed and filled like the reference's ``inout`` array."""
        x = _f32(input)
        if x.size == 0:
            return np.zeros(0, np.float32)
        if self.mode.kind == "fft":
            return self._process_fft(x, output)
        if self._h is None:
            raise ConvolutionError.fftNotInitialized()
        single = x.ndim == 1
        x2 = x.reshape(1, -1) if single else x
        if x2.shape[0] != self.channels:
            raise MetalAudioError.invalidConfiguration(f"expected {self.channels} channels, got {x2.shape[0]}")
        length = x2.shape[1]
        if length + self._taps - 1 > _INT_MAX:
            raise ConvolutionError.outputSizeOverflow(length, self._taps)
        full = length + self._taps - 1
        out = np.empty((self.channels, full), np.float32)
        st = self._lib.ma_pconv_process_host(self._h, _ptr(x2), length, length, _ptr(out), full)
        _raise_status(st, "Convolution.process")
        res = out[0] if single else out
        if output is not None and single and output.size >= full:
            output[:] = 0
            output[:full] = res
            return output
        return res

    def reset(self) -> None:
        """Convolution.swift:764-775."""
        if self._h is not None:
            _raise_status(self._lib.ma_pconv_reset(self._h), "Convolution.reset")

    def releaseFFTResources(self) -> None:
        """Convolution.swift:802."""

    def close(self) -> None:
        if getattr(self, "_h", None) and self.device._h:
            self._lib.ma_pconv_destroy(self._h)
        self._h = None
        if getattr(self, "_fc", None) and self.device._h:
            self._lib.ma_fftconv_destroy(self._fc)
        self._fc = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------- filters

class FilterError(Exception):
    """Sources/MetalDSP/Filters.swift:14-26."""

    def __init__(self, case: str, description: str, **payload):
        self.case = case
        self.errorDescription = description
        self.__dict__.update(payload)
        super().__init__(description)

    @staticmethod
    def unstable(reason: str) -> "FilterError":
        return FilterError("unstable", f"Filter is unstable: {reason}", reason=reason)

    @staticmethod
    def invalidParameter(name: str, value: float, requirement: str) -> "FilterError":
        return FilterError("invalidParameter", f"Invalid parameter '{name}' with value {value}: {requirement}",
                           name=name, value=value, requirement=requirement)


class BiquadFilter:
    """Filters.swift:65.  Coefficient design (RBJ forms, float64 then rounded to float32,
    Filters.swift:226-345) and its validation (:346-490) run on the host exactly as in the
    reference; every sample is filtered on the GPU (``ma_biquad_process_*``), whatever the buffer
    size.  ``channels`` > 1 filters that many independent rows with the same coefficients."""

    class FilterType:
        """Filters.swift:68-77."""

        def __init__(self, kind: str, gainDB: float = 0.0):
            self.kind = kind
            self.gainDB = float(gainDB)

    for _k in ("lowpass", "highpass", "bandpass", "notch", "allpass"):
        setattr(FilterType, _k, FilterType(_k))
    FilterType.peaking = staticmethod(lambda gainDB: BiquadFilter.FilterType("peaking", gainDB))
    FilterType.lowshelf = staticmethod(lambda gainDB: BiquadFilter.FilterType("lowshelf", gainDB))
    FilterType.highshelf = staticmethod(lambda gainDB: BiquadFilter.FilterType("highshelf", gainDB))
    del _k

    class Coefficients:
        """Filters.swift:80-96: b0, b1, b2, a1, a2 (a0 divided out); identity by default."""

        def __init__(self, b0: float = 1.0, b1: float = 0.0, b2: float = 0.0, a1: float = 0.0, a2: float = 0.0):
            self.b0, self.b1, self.b2, self.a1, self.a2 = (np.float32(v) for v in (b0, b1, b2, a1, a2))

        def asArray(self) -> np.ndarray:
            return np.array([self.b0, self.b1, self.b2, self.a1, self.a2], np.float32)

    def __init__(self, device: AudioDevice, channels: int = 1):
        self.device = device
        self.channels = int(channels)
        self._lib = device._lib
        self.coefficients = BiquadFilter.Coefficients()
        h = ctypes.c_void_p()
        _raise_status(self._lib.ma_biquad_create(device.handle, self.channels, 1, ctypes.byref(h)), "BiquadFilter()")
        self._h = h
        self._upload()

    gpuEnabled = True

    def _upload(self) -> None:
        c = self.coefficients.asArray()
        _raise_status(self._lib.ma_biquad_set_coefficients(self._h, _ptr(c), 1, None), "BiquadFilter.configure")

    @staticmethod
    def design(type: "BiquadFilter.FilterType", frequency: float, sampleRate: float,
               q: float = 0.7071067811865476) -> "BiquadFilter.Coefficients":
        """Validated coefficients for the parameters, or FilterError (Filters.swift:346-482)."""
        frequency, sampleRate, q = np.float32(frequency), np.float32(sampleRate), np.float32(q)
        if not sampleRate > 0:
            raise FilterError.invalidParameter("sampleRate", float(sampleRate), "must be > 0")
        nyquist = np.float32(sampleRate / np.float32(2.0))
        if not (frequency > 0 and frequency < nyquist):
            raise FilterError.invalidParameter("frequency", float(frequency), f"must be > 0 and < {float(nyquist)} Hz (Nyquist)")
        if not q > 0:
            raise FilterError.invalidParameter("q", float(q), "must be > 0")
        if not (np.isfinite(frequency) and np.isfinite(sampleRate) and np.isfinite(q)):
            raise FilterError.invalidParameter("input", 0.0, "parameters must not be NaN or Infinite")
        omega = 2.0 * math.pi * float(frequency) / float(sampleRate)
        sn, cs = math.sin(omega), math.cos(omega)
        alpha = sn / (2.0 * float(q))
        k = type.kind
        if k == "lowpass":
            b = ((1.0 - cs) / 2.0, 1.0 - cs, (1.0 - cs) / 2.0)
            a = (1.0 + alpha, -2.0 * cs, 1.0 - alpha)
        elif k == "highpass":
            b = ((1.0 + cs) / 2.0, -(1.0 + cs), (1.0 + cs) / 2.0)
            a = (1.0 + alpha, -2.0 * cs, 1.0 - alpha)
        elif k == "bandpass":
            b = (alpha, 0.0, -alpha)
            a = (1.0 + alpha, -2.0 * cs, 1.0 - alpha)
        elif k == "notch":
            b = (1.0, -2.0 * cs, 1.0)
            a = (1.0 + alpha, -2.0 * cs, 1.0 - alpha)
        elif k == "allpass":
            b = (1.0 - alpha, -2.0 * cs, 1.0 + alpha)
            a = (1.0 + alpha, -2.0 * cs, 1.0 - alpha)
        elif k == "peaking":
            A = math.pow(10.0, float(np.float32(type.gainDB)) / 40.0)
            b = (1.0 + alpha * A, -2.0 * cs, 1.0 - alpha * A)
            a = (1.0 + alpha / A, -2.0 * cs, 1.0 - alpha / A)
        elif k in ("lowshelf", "highshelf"):
            A = math.pow(10.0, float(np.float32(type.gainDB)) / 40.0)
            rt = 2.0 * math.sqrt(A) * alpha
            sg = 1.0 if k == "lowshelf" else -1.0      # the two shelves mirror the cos terms
            b = (A * ((A + 1.0) - sg * (A - 1.0) * cs + rt),
                 sg * 2.0 * A * ((A - 1.0) - sg * (A + 1.0) * cs),
                 A * ((A + 1.0) - sg * (A - 1.0) * cs - rt))
            a = ((A + 1.0) + sg * (A - 1.0) * cs + rt,
                 -sg * 2.0 * ((A - 1.0) + sg * (A + 1.0) * cs),
                 (A + 1.0) + sg * (A - 1.0) * cs - rt)
        else:
            raise MetalAudioError.invalidConfiguration(f"unknown filter type {k}")
        a0f = np.float32(a[0])
        if not abs(a0f) > np.float32(1e-6):
            raise FilterError.invalidParameter("a0 (computed)", float(a0f),
                                               "denominator coefficient a0 must not be near zero (|a0| > 1e-6). This "
                                               "typically indicates frequency near 0 Hz or Nyquist, or extreme Q values")
        with np.errstate(over="ignore", invalid="ignore"):
            nb = [np.float32(v / a[0]) for v in b]
            na = [np.float32(v / a[0]) for v in a[1:]]
        if not all(np.isfinite(v) for v in nb + na):
            raise FilterError.invalidParameter("coefficients", 0.0,
                                               "normalized coefficients must not be NaN or Infinite. This typically "
                                               "indicates extreme parameter combinations (very high Q, frequency near "
                                               "0 or Nyquist)")
        if not abs(na[1]) < 1.0:
            raise FilterError.invalidParameter("a2 (stability)", float(na[1]),
                                               f"|a2| must be < 1 for filter stability. Current |a2| = {abs(float(na[1]))}. "
                                               "Try reducing Q or adjusting frequency.")
        if not abs(na[0]) < np.float32(1.0) + na[1]:
            raise FilterError.invalidParameter("a1 (stability)", float(na[0]),
                                               f"|a1| must be < 1 + a2 for filter stability. Current |a1| = "
                                               f"{abs(float(na[0]))}, 1 + a2 = {float(np.float32(1.0) + na[1])}. Try reducing Q.")
        return BiquadFilter.Coefficients(nb[0], nb[1], nb[2], na[0], na[1])

    def configure(self, type: "BiquadFilter.FilterType", frequency: float, sampleRate: float,
                  q: float = 0.7071067811865476) -> None:
        """Filters.swift:346-490: the object keeps its previous coefficients when validation fails."""
        self.coefficients = BiquadFilter.design(type, frequency, sampleRate, q)
        self._upload()

    def setCoefficients(self, coefficients: "BiquadFilter.Coefficients") -> None:
        self.coefficients = coefficients
        self._upload()

    @property
    def currentCoefficients(self) -> "BiquadFilter.Coefficients":
        return self.coefficients

    def process(self, input=None, sample: Optional[float] = None):
        """``process(input:)`` (Filters.swift:555-593) for a (L,) array or (channels, L) rows;
        ``process(sample=...)`` (:515-537) for one sample.  State carries over between calls."""
        if sample is not None:
            return float(self.process(np.array([sample], np.float32))[0])
        x = _f32(input)
        if x.size == 0:
            return np.zeros(x.shape, np.float32)
        single = x.ndim == 1
        x2 = x.reshape(1, -1) if single else x
        if x2.shape[0] != self.channels:
            raise MetalAudioError.invalidConfiguration(f"expected {self.channels} channels, got {x2.shape[0]}")
        out = np.empty_like(x2)
        n = x2.shape[1]
        _raise_status(self._lib.ma_biquad_process_host(self._h, _ptr(x2), n, _ptr(out), n, n), "BiquadFilter.process")
        return out[0] if single else out

    def processTensor(self, input: "Tensor", output: "Tensor") -> None:
        """Device-resident form: (channels, L) Tensors, queued on the device stream."""
        n = input.shape[-1]
        st = self._lib.ma_biquad_process_dev(self._h, ctypes.c_void_p(input.pointer), n,
                                             ctypes.c_void_p(output.pointer), output.shape[-1], n)
        _raise_status(st, "BiquadFilter.processTensor")

    def reset(self) -> None:
        """Filters.swift:662-672."""
        _raise_status(self._lib.ma_biquad_reset(self._h), "BiquadFilter.reset")

    @property
    def delays(self) -> np.ndarray:
        """(channels, 2) array of (z1, z2)."""
        st = np.empty((self.channels, 1, 2), np.float32)
        _raise_status(self._lib.ma_biquad_get_state(self._h, _ptr(st)), "BiquadFilter.delays")
        return st[:, 0, :]

    def validateStability(self) -> None:
        """Filters.swift:688-716."""
        a1, a2 = self.coefficients.a1, self.coefficients.a2
        if not (np.isfinite(a1) and np.isfinite(a2)):
            raise FilterError.unstable("coefficients contain NaN or Infinite values, filter is in invalid state")
        if not abs(a2) < 1.0:
            raise FilterError.unstable(f"a2 coefficient magnitude ({abs(float(a2))}) >= 1, poles outside unit circle")
        if not abs(a1) < np.float32(1.0) + a2:
            raise FilterError.unstable(f"a1 coefficient ({float(a1)}) violates stability condition |a1| < 1 + a2 = "
                                       f"{float(np.float32(1.0) + a2)}")

    @property
    def isStable(self) -> bool:
        a1, a2 = self.coefficients.a1, self.coefficients.a2
        return bool(np.isfinite(a1) and np.isfinite(a2) and abs(a2) < 1.0 and abs(a1) < np.float32(1.0) + a2)

    def close(self) -> None:
        if getattr(self, "_h", None) and self.device._h:
            self._lib.ma_biquad_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FilterBank:
    """Filters.swift:736.  ``processSeries`` runs the bands as one cascade of sections on the GPU;
    ``processParallel`` feeds one signal to every band (one channel per band) and mixes them with
    1/bandCount (:845-868).  Both run over the same per-band filters in the reference, so a band's
    (z1, z2) state carries over when a caller alternates between the two: the two device objects
    here hand their state to each other on every switch.  At most ``maxBands`` bands (the cascade
    length one kernel launch serves); the reference has no such limit."""

    maxBands = 32

    def __init__(self, device: AudioDevice, bandCount: int):
        if int(bandCount) > FilterBank.maxBands:
            raise FilterError.invalidParameter("bandCount", float(bandCount),
                                               f"must be <= {FilterBank.maxBands} on the CUDA backend (one cascade per launch)")
        self.device = device
        self.bandCount = int(bandCount)
        self._last = None
        self._lib = device._lib
        self._coeffs = [BiquadFilter.Coefficients() for _ in range(max(self.bandCount, 0))]
        self._series = None
        self._parallel = None
        self._dirty = True

    gpuEnabled = True

    def _handles(self):
        if self.bandCount <= 0:
            return
        if self._series is None:
            hs, hp = ctypes.c_void_p(), ctypes.c_void_p()
            _raise_status(self._lib.ma_biquad_create(self.device.handle, 1, self.bandCount, ctypes.byref(hs)), "FilterBank")
            _raise_status(self._lib.ma_biquad_create(self.device.handle, self.bandCount, 1, ctypes.byref(hp)), "FilterBank")
            self._series, self._parallel = hs, hp
        if self._dirty:
            c = np.stack([k.asArray() for k in self._coeffs])
            _raise_status(self._lib.ma_biquad_set_coefficients(self._series, _ptr(c), 1, None), "FilterBank")
            cmap = np.arange(self.bandCount, dtype=np.int32)
            _raise_status(self._lib.ma_biquad_set_coefficients(self._parallel, _ptr(c), self.bandCount, _ptr(cmap)), "FilterBank")
            self._dirty = False

    def _switch_to(self, which: str):
        """Makes `which` ("series" / "parallel") the object holding the bands' current state: both
        lay it out as bandCount x (z1, z2)."""
        if self._last is not None and self._last != which:
            st = np.empty((self.bandCount, 2), np.float32)
            src = self._series if self._last == "series" else self._parallel
            dst = self._series if which == "series" else self._parallel
            _raise_status(self._lib.ma_biquad_get_state(src, _ptr(st)), "FilterBank")
            _raise_status(self._lib.ma_biquad_set_state(dst, _ptr(st)), "FilterBank")
        self._last = which

    def configureAsEQ(self, lowFreq: float, highFreq: float, sampleRate: float, q: float = 1.414) -> None:
        """Logarithmically spaced 0 dB peaking bands (Filters.swift:768-812)."""
        if self.bandCount < 2:
            raise FilterError.invalidParameter("bandCount", float(self.bandCount), "must be >= 2 for logarithmic band spacing")
        lowFreq, highFreq = np.float32(lowFreq), np.float32(highFreq)
        if not lowFreq > 0:
            raise FilterError.invalidParameter("lowFreq", float(lowFreq),
                                               f"must be > 0 (got {float(lowFreq)}, log10 requires positive values)")
        if not (highFreq > 0 and highFreq > lowFreq):
            raise FilterError.invalidParameter("highFreq", float(highFreq), f"must be > 0 and > lowFreq ({float(lowFreq)})")
        log_low, log_high = np.log10(lowFreq), np.log10(highFreq)
        step = np.float32((log_high - log_low) / np.float32(self.bandCount - 1))
        new = []
        for i in range(self.bandCount):
            freq = np.power(np.float32(10.0), np.float32(log_low + np.float32(i) * step))
            new.append(BiquadFilter.design(BiquadFilter.FilterType.peaking(0.0), freq, sampleRate, q))
            # the reference configures band by band: earlier bands keep their new settings if a later one throws
            self._coeffs[i] = new[-1]
            self._dirty = True

    def setBandGain(self, band: int, gainDB: float, frequency: float, sampleRate: float, q: float = 1.414) -> None:
        """Filters.swift:822-842."""
        if not (0 <= band < self.bandCount):
            raise FilterError.invalidParameter("band", float(band), f"must be in range 0..<{self.bandCount}")
        self._coeffs[band] = BiquadFilter.design(BiquadFilter.FilterType.peaking(gainDB), frequency, sampleRate, q)
        self._dirty = True

    def processSeries(self, input) -> np.ndarray:
        x = _f32(input)
        if x.size == 0 or self.bandCount <= 0:
            return x.copy()
        self._handles()
        self._switch_to("series")
        out = np.empty_like(x)
        _raise_status(self._lib.ma_biquad_process_host(self._series, _ptr(x), x.size, _ptr(out), x.size, x.size),
                      "FilterBank.processSeries")
        return out

    def processParallel(self, input) -> np.ndarray:
        x = _f32(input)
        if x.size == 0 or self.bandCount <= 0:
            return np.zeros_like(x)
        self._handles()
        self._switch_to("parallel")
        n = x.size
        dev = self.device
        tin, bands, mix = Tensor(dev, (n,)), Tensor(dev, (self.bandCount, n)), Tensor(dev, (n,))
        try:
            tin.copy(x)
            st = self._lib.ma_biquad_process_dev(self._parallel, ctypes.c_void_p(tin.pointer), 0,
                                                 ctypes.c_void_p(bands.pointer), n, n)
            _raise_status(st, "FilterBank.processParallel")
            scale = float(np.float32(1.0) / np.float32(self.bandCount))
            st = self._lib.ma_channel_mix_dev(dev.handle, ctypes.c_void_p(bands.pointer), self.bandCount, n, n, scale,
                                              ctypes.c_void_p(mix.pointer))
            _raise_status(st, "FilterBank.processParallel")
            return mix.toArray()
        finally:
            for t in (tin, bands, mix):
                t.free()

    def reset(self) -> None:
        for h in (self._series, self._parallel):
            if h is not None:
                _raise_status(self._lib.ma_biquad_reset(h), "FilterBank.reset")
        self._last = None

    def close(self) -> None:
        for h in (getattr(self, "_series", None), getattr(self, "_parallel", None)):
            if h is not None and self.device._h:
                self._lib.ma_biquad_destroy(h)
        self._series = self._parallel = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
