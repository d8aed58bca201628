"""B200-native (sm_100a CUDA) backend for the MetalDSP hot path: batched real-input
FFT / inverse FFT, STFT / iSTFT, uniformly partitioned and one-shot FFT convolution, and the
magnitude / phase glue around the STFT, plus multichannel biquad cascades.

``metalaudio_b200.dsp`` mirrors the reference's public Swift API over the C ABI declared in
``include/metalaudio_cuda.h``; ``metalaudio_b200.build`` compiles the library in-tree.
Nothing here computes on the CPU: without the CUDA library every call raises.
"""
from .dsp import (AudioDevice, Backend, BiquadFilter, COLACompliance, Convolution, ConvolutionError, FFT, FFTError,
                  FilterBank, FilterError,
                  MetalAudioError, STFTResult, Tensor, ToleranceProvider, WindowType, polarToSpectrum,
                  spectrumToPolar, toDecibels, validatedWindowFloor)

__all__ = ["AudioDevice", "Backend", "BiquadFilter", "COLACompliance", "Convolution", "ConvolutionError", "FFT",
           "FFTError", "FilterBank", "FilterError",
           "MetalAudioError", "STFTResult", "Tensor", "ToleranceProvider", "WindowType", "polarToSpectrum",
           "spectrumToPolar", "toDecibels", "validatedWindowFloor"]
