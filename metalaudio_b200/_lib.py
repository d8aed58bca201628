"""ctypes binding of ``libmetalaudio_cuda.so`` (the C ABI in ``include/metalaudio_cuda.h``).

Loading fails loudly: there is no CPU fallback anywhere in this package.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_size_t, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmetalaudio_cuda.so")

c_float_p = POINTER(c_float)
c_int32_p = POINTER(c_int32)
c_int64_p = POINTER(c_int64)

# name -> (restype, argtypes); mirrors include/metalaudio_cuda.h one to one.
SIGNATURES = {
    "ma_status_string": (c_char_p, [c_int32]),
    "ma_last_cuda_error": (c_int32, []),
    "ma_kernel_launch_count": (c_uint64, []),
    "ma_device_count": (c_int32, []),
    "ma_context_create": (c_int32, [c_int32, c_size_t, POINTER(c_void_p)]),
    "ma_context_destroy": (c_int32, [c_void_p]),
    "ma_context_sync": (c_int32, [c_void_p, c_double]),
    "ma_context_reserve_workspace": (c_int32, [c_void_p, c_size_t]),
    "ma_context_device_name": (c_int32, [c_void_p, c_char_p, c_size_t]),
    "ma_context_stream": (c_void_p, [c_void_p]),
    "ma_context_mark_lost": (c_int32, [c_void_p]),
    "ma_context_is_available": (c_int32, [c_void_p, c_int32_p]),
    "ma_timing_begin": (c_int32, [c_void_p]),
    "ma_timing_end": (c_int32, [c_void_p, c_float_p]),
    "ma_test_inject_fault": (c_int32, [c_void_p, c_int32, c_int32]),
    "ma_test_bounded_wait": (c_int32, [c_void_p, c_int32]),
    "ma_buffer_alloc": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "ma_buffer_free": (c_int32, [c_void_p, c_void_p]),
    "ma_buffer_zero": (c_int32, [c_void_p, c_void_p, c_size_t]),
    "ma_memcpy_h2d": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ma_memcpy_d2h": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ma_memcpy_h2d_async": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ma_memcpy_d2h_async": (c_int32, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ma_host_alloc": (c_int32, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "ma_host_free": (c_int32, [c_void_p, c_void_p]),
    "ma_fft_plan_create": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, POINTER(c_void_p)]),
    "ma_fft_plan_destroy": (c_int32, [c_void_p]),
    "ma_fft_plan_scratch_bytes": (c_int32, [c_void_p, POINTER(c_size_t)]),
    "ma_fft_forward_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_float, c_int64, c_int32]),
    "ma_fft_forward_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_float, c_int64, c_int32]),
    "ma_fft_forward_static_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_float, c_int64, c_int32]),
    "ma_fft_inverse_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32]),
    "ma_fft_inverse_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32]),
    "ma_fft_complex_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int32]),
    "ma_fft_complex_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int32]),
    "ma_fft_magnitude_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_float]),
    "ma_fft_magnitude_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_float]),
    "ma_stft_frame_count": (c_int32, [c_void_p, c_int64, c_int64_p]),
    "ma_istft_output_length": (c_int32, [c_void_p, c_int64, c_int64_p]),
    "ma_stft_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_float, c_int32]),
    "ma_stft_host": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_float, c_int32]),
    "ma_istft_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_float, c_int32]),
    "ma_istft_host": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_float, c_int32]),
    "ma_pconv_create": (c_int32, [c_void_p, c_int32, c_int32, POINTER(c_void_p)]),
    "ma_pconv_destroy": (c_int32, [c_void_p]),
    "ma_pconv_set_kernels": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "ma_pconv_partition_count": (c_int32, [c_void_p, c_int32_p]),
    "ma_pconv_step_splits": (c_int32, [c_void_p, c_int32, c_int32_p]),
    "ma_pconv_reserve": (c_int32, [c_void_p, c_int64]),
    "ma_pconv_process_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64]),
    "ma_pconv_process_host": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64]),
    "ma_pconv_step_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_int64]),
    "ma_pconv_reset": (c_int32, [c_void_p]),
    "ma_spectrum_to_polar_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64]),
    "ma_polar_to_spectrum_dev": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64]),
    "ma_to_decibels_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_float, c_float]),
    "ma_biquad_create": (c_int32, [c_void_p, c_int32, c_int32, POINTER(c_void_p)]),
    "ma_biquad_destroy": (c_int32, [c_void_p]),
    "ma_biquad_set_coefficients": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p]),
    "ma_biquad_process_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64]),
    "ma_biquad_process_host": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64]),
    "ma_biquad_reset": (c_int32, [c_void_p]),
    "ma_biquad_get_state": (c_int32, [c_void_p, c_void_p]),
    "ma_biquad_set_state": (c_int32, [c_void_p, c_void_p]),
    "ma_channel_mix_dev": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_float, c_void_p]),
    "ma_fftconv_create": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, POINTER(c_void_p)]),
    "ma_fftconv_destroy": (c_int32, [c_void_p]),
    "ma_fftconv_fft_size": (c_int32, [c_void_p, POINTER(c_int64)]),
    "ma_fftconv_process_dev": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]),
    "ma_fftconv_process_host": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]),
}

# Status codes and enums (include/metalaudio_cuda.h).
MA_OK = 0
(MA_ERR_INVALID_ARGUMENT, MA_ERR_SIZE_NOT_POW2, MA_ERR_SIZE_TOO_LARGE, MA_ERR_INVALID_HOP,
 MA_ERR_INPUT_TOO_SHORT, MA_ERR_BATCH_OVERFLOW, MA_ERR_ISTFT_OVERFLOW, MA_ERR_EMPTY_KERNEL,
 MA_ERR_KERNEL_NOT_CONFIGURED, MA_ERR_INVALID_PARTITION_STATE, MA_ERR_OUTPUT_OVERFLOW, MA_ERR_ALLOC,
 MA_ERR_TIMEOUT, MA_ERR_DEVICE_LOST, MA_ERR_CUDA, MA_ERR_UNSUPPORTED, MA_ERR_SCRATCH_LIMIT,
 MA_ERR_INPUT_SIZE_MISMATCH) = range(1, 19)
LAYOUT_HALF_INTERLEAVED, LAYOUT_FULL_SPLIT, LAYOUT_HALF_PACKED, LAYOUT_HALF_POLAR = 0, 1, 2, 3
MAG_MAGNITUDE, MAG_POWER, MAG_DB = 0, 1, 2
FAULT_ALLOC, FAULT_LAUNCH, FAULT_SYNC, FAULT_DEVICE_LOST = 0, 1, 2, 3

_lib = None


def load() -> ctypes.CDLL:
    """Load the library and bind every declared symbol.  Raises if the file or a symbol is
    missing: the product never runs without its CUDA library."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m metalaudio_b200.build` (needs nvcc). "
            "There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
