/*
 * metalaudio_cuda.h - C ABI of the CUDA (sm_100a) backend for the MetalDSP hot path:
 * batched real-input FFT / inverse FFT, STFT / iSTFT and uniformly partitioned FFT
 * convolution.
 *
 * The reference (a Swift package) has no FFI of its own: its boundary for this path is
 * the public Swift API of `FFT` and `Convolution`.  Every entry point below names the
 * reference interface (file:line within the reference tree) whose arithmetic it
 * replaces; a Swift `FFT` / `Convolution` / `AudioDevice` / `Tensor` shim calls these
 * through a system-library module target.
 *
 * Conventions
 *  - plain C: opaque handles, pointers, sizes; every call returns an ma_status.
 *  - `_dev` entry points take device pointers, are ordered on the context's stream, do
 *    not allocate and do not synchronise.  `_host` entry points take host pointers,
 *    copy through the context (directly when the memory is pinned, e.g. from
 *    ma_host_alloc, through the context's pinned staging buffer otherwise) and return
 *    after the result is in the caller's buffer.
 *  - all data is float32; complex data is interleaved (re, im) unless a layout says
 *    otherwise; all index arithmetic is 64-bit and overflow-checked on the host.
 *  - there is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef METALAUDIO_CUDA_H
#define METALAUDIO_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t ma_status;

/* Status codes.  The FFT / convolution codes map 1:1 onto the reference's Swift error
 * enums: FFTError (Sources/MetalDSP/FFT.swift:12-33), ConvolutionError
 * (Sources/MetalDSP/Convolution.swift:8-27), MetalAudioError
 * (Sources/MetalAudioKit/Core/AudioDevice.swift:11-32). */
enum {
    MA_OK = 0,
    MA_ERR_INVALID_ARGUMENT = 1,       /* MetalAudioError.invalidConfiguration */
    MA_ERR_SIZE_NOT_POW2 = 2,          /* FFTError.sizeNotPowerOf2 */
    MA_ERR_SIZE_TOO_LARGE = 3,         /* FFTError.sizeTooLarge (N > 2^24) */
    MA_ERR_INVALID_HOP = 4,            /* FFTError.invalidHopSize */
    MA_ERR_INPUT_TOO_SHORT = 5,        /* FFTError.inputTooShort */
    MA_ERR_BATCH_OVERFLOW = 6,         /* FFTError.batchSizeOverflow */
    MA_ERR_ISTFT_OVERFLOW = 7,         /* FFTError.istftOutputOverflow / istftFrameOverflow */
    MA_ERR_EMPTY_KERNEL = 8,           /* invalidConfiguration("Kernel must not be empty ...") */
    MA_ERR_KERNEL_NOT_CONFIGURED = 9,  /* ConvolutionError.fftNotInitialized */
    MA_ERR_INVALID_PARTITION_STATE = 10, /* ConvolutionError.invalidPartitionState */
    MA_ERR_OUTPUT_OVERFLOW = 11,       /* ConvolutionError.outputSizeOverflow */
    MA_ERR_ALLOC = 12,                 /* MetalAudioError.bufferAllocationFailed */
    MA_ERR_TIMEOUT = 13,               /* MetalAudioError.gpuTimeout */
    MA_ERR_DEVICE_LOST = 14,           /* MetalAudioError.deviceLost / deviceNotFound */
    MA_ERR_CUDA = 15,                  /* MetalAudioError.gpuExecutionError; see ma_last_cuda_error */
    MA_ERR_UNSUPPORTED = 16,
    MA_ERR_SCRATCH_LIMIT = 17,         /* work needs more scratch than the built-in static buffer holds */
    MA_ERR_INPUT_SIZE_MISMATCH = 18    /* ConvolutionError.inputSizeMismatch */
};

/* Spectrum layouts accepted / produced by the transforms (N = FFT size). */
enum {
    MA_LAYOUT_HALF_INTERLEAVED = 0, /* N/2+1 interleaved complex bins per frame (re,im pairs) */
    MA_LAYOUT_FULL_SPLIT = 1,       /* the reference's layout: real[N] and imag[N] per frame,
                                       bins N/2+1..N-1 the conjugate mirror (FFT.swift:799-802) */
    MA_LAYOUT_HALF_PACKED = 2,      /* N/2 interleaved complex bins, bin 0 = (DC, Nyquist);
                                       internal format of the convolution delay line */
    MA_LAYOUT_HALF_POLAR = 3        /* array a = magnitude[N/2+1], array b = phase[N/2+1] (radians,
                                       atan2(im, re)) per frame: the magnitude / phase split and
                                       the polar -> complex rebuild that the reference's one STFT
                                       consumer does on the host around stft / istft
                                       (Sources/MetalNN/HTDemucs.swift:726-741, :795-812; shader
                                       forms compute_phase / polar_to_complex,
                                       Shaders/DSP.metal:806-834), fused into the transforms.
                                       Plans up to 8192 points. */
};

/* Magnitude kinds (FFT.swift:1780-1847). */
enum { MA_MAG_MAGNITUDE = 0, MA_MAG_POWER = 1, MA_MAG_DB = 2 };

/* Host-side fault injection sites (ma_test_inject_fault). */
enum { MA_FAULT_ALLOC = 0, MA_FAULT_LAUNCH = 1, MA_FAULT_SYNC = 2, MA_FAULT_DEVICE_LOST = 3 };

typedef struct ma_context ma_context;
typedef struct ma_fft_plan ma_fft_plan;
typedef struct ma_pconv ma_pconv;
typedef struct ma_fftconv ma_fftconv;
typedef struct ma_biquad ma_biquad;

/* ------------------------------------------------------------------ library */

/* Human-readable text for a status code. */
const char* ma_status_string(ma_status s);
/* Last cudaError_t seen by this thread's most recent failing call (0 if none). */
int32_t ma_last_cuda_error(void);
/* Number of kernels this library has launched in this process (all contexts). */
uint64_t ma_kernel_launch_count(void);
/* Number of visible CUDA devices; 0 when none (then every create call fails). */
int32_t ma_device_count(void);

/* ------------------------------------------------------------------ context
 * Replaces AudioDevice (device + queue ownership, AudioDevice.swift:222, :323-332) and
 * the executeSync / executeSyncWithTiming slice of ComputeContext
 * (Sources/MetalAudioKit/Core/ComputeContext.swift:154-211, :232-297). */

/* Create a context on `device_index` with its own stream and a pinned staging buffer of
 * `pinned_bytes` (0 picks 64 MiB). */
ma_status ma_context_create(int32_t device_index, size_t pinned_bytes, ma_context** out);
ma_status ma_context_destroy(ma_context* ctx);
/* Wait for all work queued on the context, at most `timeout_s` seconds (<= 0: the
 * reference's default of 2 s, ComputeContext.swift:137).  Polls an event; on expiry
 * returns MA_ERR_TIMEOUT and leaves the stream draining. */
ma_status ma_context_sync(ma_context* ctx, double timeout_s);
/* Device workspace of the pipelined *_host calls (ma_stft_host, ma_istft_host, ma_pconv_process_host,
 * and ma_fft_forward_host / ma_fft_inverse_host for batches of 16 MiB and more): `bytes` of device memory
 * in two lanes, allocated once here (or, at a default of 2 x 256 MiB, by the first such call) and
 * kept until the context is destroyed - the "pre-allocated staging" half of AudioDevice /
 * ComputeContext in this backend.  Grows only when a single signal with its results does not fit a
 * lane. */
ma_status ma_context_reserve_workspace(ma_context* ctx, size_t bytes);
/* Device name into `buf` (AudioDevice.name). */
ma_status ma_context_device_name(ma_context* ctx, char* buf, size_t buf_len);
/* The context's cudaStream_t as an opaque pointer, for callers that order their own
 * device work (e.g. event timing) against it. */
void* ma_context_stream(ma_context* ctx);
/* AudioDevice.markDeviceLost / ensureAvailable (AudioDevice.swift:434-472, :733-741):
 * after mark_lost every call on the context returns MA_ERR_DEVICE_LOST. */
ma_status ma_context_mark_lost(ma_context* ctx);
ma_status ma_context_is_available(ma_context* ctx, int32_t* available);
/* executeSyncWithTiming: bracket queued work with events; end returns elapsed ms and
 * waits for the work. */
ma_status ma_timing_begin(ma_context* ctx);
ma_status ma_timing_end(ma_context* ctx, float* milliseconds);
/* Test hook, host side only: the next call that reaches `site` fails with
 * `cuda_error` (no GPU work is disturbed). */
ma_status ma_test_inject_fault(ma_context* ctx, int32_t site, int32_t cuda_error);
/* Test hook for the device-side timeout path (the reference's gpuTimeout,
 * ComputeContext.swift:176-208): queues a one-thread kernel that waits, with the same bounded
 * wait the transform kernels use for their staged copies, on a barrier nothing will complete;
 * after `polls` polls (1..65536) it gives up and raises the context's error flag, which the next
 * ma_context_sync reports as MA_ERR_TIMEOUT and clears.  Nothing faults or hangs. */
ma_status ma_test_bounded_wait(ma_context* ctx, int32_t polls);

/* ------------------------------------------------------------------ buffers
 * Backing store of Tensor (Sources/MetalAudioKit/Buffers/Tensor.swift:59, :272, :325,
 * :390): a device allocation plus explicit host copies. */
ma_status ma_buffer_alloc(ma_context* ctx, size_t bytes, void** dptr);
ma_status ma_buffer_free(ma_context* ctx, void* dptr);
ma_status ma_buffer_zero(ma_context* ctx, void* dptr, size_t bytes);           /* Tensor.zero */
ma_status ma_memcpy_h2d(ma_context* ctx, void* dptr, const void* host, size_t bytes); /* Tensor.copy(from:) */
ma_status ma_memcpy_d2h(ma_context* ctx, void* host, const void* dptr, size_t bytes); /* Tensor.toArray / copy(to:) */
/* Stream-ordered copies that return immediately; `host` must be pinned. */
ma_status ma_memcpy_h2d_async(ma_context* ctx, void* dptr, const void* host, size_t bytes);
ma_status ma_memcpy_d2h_async(ma_context* ctx, void* host, const void* dptr, size_t bytes);
/* Pinned host memory for callers that want zero-staging transfers. */
ma_status ma_host_alloc(ma_context* ctx, size_t bytes, void** hptr);
ma_status ma_host_free(ma_context* ctx, void* hptr);

/* ------------------------------------------------------------------ FFT plan
 * Replaces FFT.init(device:config:) (FFT.swift:441-495): validates N (power of two,
 * 2 <= N <= 2^24) and 0 < hop <= N, keeps the window table on the device.
 * `window` is a host array of N coefficients computed by the caller exactly as
 * FFT.swift:461 does (symmetric, float64 then rounded) or NULL for no window;
 * forward()/inverse() never apply it, stft/istft do (FFT.swift:783-786,
 * STFT.swift:63-68, :462). */
ma_status ma_fft_plan_create(ma_context* ctx, int32_t n, const float* window, int32_t hop,
                             ma_fft_plan** out);
ma_status ma_fft_plan_destroy(ma_fft_plan* plan);
/* Bytes of device scratch the plan holds for N > 8192 (0 below): two lanes of pass data.  A batch
 * of such transforms is cut into chunks that alternate between the context's stream and a second,
 * internal stream (one lane of the scratch each); the internal stream starts behind everything
 * queued on the context's stream and is joined back to it before the call returns, so callers
 * keep seeing one stream. */
ma_status ma_fft_plan_scratch_bytes(ma_fft_plan* plan, size_t* bytes);

/* Unnormalised forward DFT of `batch` contiguous real frames of N samples.
 * Replaces FFT.forward (FFT.swift:818-855), forwardBatch (STFT.swift:94-128) and the
 * GPU / MPSGraph / auto variants (FFT.swift:945-1107, :1372-1431, :1639-1687).
 * layout HALF_INTERLEAVED / HALF_PACKED: `out_a` receives the interleaved bins, `out_b`
 * is ignored.  layout FULL_SPLIT: `out_a` = real[batch][N], `out_b` = imag[batch][N].
 * `mag` (may be NULL) receives batch x (N/2+1) magnitudes of `mag_kind` computed in the
 * same pass (db_reference used for MA_MAG_DB). */
ma_status ma_fft_forward_dev(ma_fft_plan* plan, const float* in, float* out_a, float* out_b,
                             float* mag, int32_t mag_kind, float db_reference,
                             int64_t batch, int32_t layout);
ma_status ma_fft_forward_host(ma_fft_plan* plan, const float* in, float* out_a, float* out_b,
                              float* mag, int32_t mag_kind, float db_reference,
                              int64_t batch, int32_t layout);

/* Size of the library's built-in scratch buffer used by ma_fft_forward_static_dev. */
#define MA_STATIC_SCRATCH_BYTES ((size_t)8 << 20)

/* Forward transform for callers that must not allocate device memory.  It has no counterpart in
 * the reference.  Who needs it: code running where cudaMalloc is off limits - an audio render
 * callback with a hard deadline (an allocation can block for milliseconds and synchronises the
 * device) or a process whose device-memory budget was fixed at start-up and must not grow.  Such
 * callers create the plan once at start-up and afterwards need every call to leave the
 * allocator alone.
 *
 * Same arguments and results as ma_fft_forward_dev for plans above 8192 points (smaller plans
 * need no scratch and are simply forwarded to ma_fft_forward_dev).  The difference: the
 * intermediate pass data goes through a fixed buffer of MA_STATIC_SCRATCH_BYTES that is compiled
 * into the library (a file-scope __device__ array), not through the plan's own allocation.  The
 * call itself performs no cudaMalloc / cudaFree / stream-ordered allocation of any kind.
 *  - Limit: one transform's intermediate data, (N2/2 + 1) * N1 * 8 bytes (about 4*N bytes), must fit
 *    the buffer, i.e. N <= 2^20; larger plans return MA_ERR_SCRATCH_LIMIT.  Batches larger than the
 *    buffer holds are processed in several passes.
 *  - Every GPU that loads the library carries the buffer until the process exits.
 *  - The first call on each device looks the buffer's device address up (one cheap runtime query,
 *    made with that device current).  Make that first call before starting any stream capture.
 *  - All calls, from all plans and contexts on one device, share the one buffer, and it keeps
 *    whatever the previous call left in it.  Nothing in it has to start at zero - each pass
 *    overwrites every element the next pass reads - so no clearing is done.  Two calls whose
 *    kernels overlap on the GPU (different streams / contexts) would trample each other's
 *    intermediate data: issue them on one stream, or otherwise make sure they do not overlap. */
ma_status ma_fft_forward_static_dev(ma_fft_plan* plan, const float* in, float* out_a, float* out_b,
                                    float* mag, int32_t mag_kind, float db_reference,
                                    int64_t batch, int32_t layout);

/* Inverse DFT with the 1/N scale fused.  Replaces FFT.inverse (FFT.swift:889-919),
 * inverseBatch (STFT.swift:327-373), inverseGPU / inverseMPSGraph / inverseAuto.
 * The input spectrum is taken as Hermitian: only bins 0..N/2 are read (for FULL_SPLIT
 * from in_a = real, in_b = imag). */
ma_status ma_fft_inverse_dev(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out,
                             int64_t batch, int32_t layout);
ma_status ma_fft_inverse_host(ma_fft_plan* plan, const float* in_a, const float* in_b, float* out,
                              int64_t batch, int32_t layout);

/* Complex-input transform of `batch` sequences of N interleaved (re, im) pairs, in and out
 * (2N floats per sequence, 8-byte aligned for the _dev form): the full complex DFT, forward
 * unscaled (inverse == 0) or inverse with the 1/N scale (inverse != 0).  Replaces the
 * explicit-backend calls FFT.forwardGPU / inverseGPU (FFT.swift:945-1107, :1176-1315), whose
 * data format this is, for every plan size.  Runs as split -> batched real transform -> combine
 * through a plan-owned work buffer that is allocated on the first such call. */
ma_status ma_fft_complex_dev(ma_fft_plan* plan, const float* in, float* out, int64_t batch, int32_t inverse);
ma_status ma_fft_complex_host(ma_fft_plan* plan, const float* in, float* out, int64_t batch, int32_t inverse);

/* Magnitude / power / dB over bins 0..N/2 of caller-supplied FULL_SPLIT spectra.
 * Replaces FFT.magnitude / power / magnitudeDB (FFT.swift:1780-1847). */
ma_status ma_fft_magnitude_dev(ma_fft_plan* plan, const float* re, const float* im, float* out,
                               int64_t batch, int32_t kind, float db_reference);
ma_status ma_fft_magnitude_host(ma_fft_plan* plan, const float* re, const float* im, float* out,
                                int64_t batch, int32_t kind, float db_reference);

/* ------------------------------------------------------------------ spectrum glue
 * Elementwise steps of the reference's shader library on device arrays, stream-ordered:
 * compute_magnitude + compute_phase in one pass over `count` interleaved complex bins
 * (Shaders/DSP.metal:784-813; either output may be NULL), polar_to_complex (:821-834) and the
 * in-place to_decibels with its 1e-10 ratio clamp, min_db floor and reference <= 0 fallback
 * (:861-881).  The transforms produce and consume the same quantities directly with
 * MA_LAYOUT_HALF_POLAR; these serve spectra that already exist. */
ma_status ma_spectrum_to_polar_dev(ma_context* ctx, const float* spectrum, float* magnitude, float* phase,
                                   int64_t count);
ma_status ma_polar_to_spectrum_dev(ma_context* ctx, const float* magnitude, const float* phase, float* spectrum,
                                   int64_t count);
ma_status ma_to_decibels_dev(ma_context* ctx, float* data, int64_t count, float reference, float min_db);

/* ------------------------------------------------------------------ STFT / iSTFT */

/* Frame count (L - N)/hop + 1 for a signal of `length` (STFT.swift:45-49);
 * MA_ERR_INPUT_TOO_SHORT when length < N. */
ma_status ma_stft_frame_count(ma_fft_plan* plan, int64_t length, int64_t* frames);
/* Output length (F-1)*hop + N with the overflow check of STFT.swift:393-397. */
ma_status ma_istft_output_length(ma_fft_plan* plan, int64_t frames, int64_t* length);

/* STFT of `n_signals` signals of `length` samples, signal s starting at
 * signals + s*signal_stride: frames at i*hop, analysis window, forward DFT.
 * Replaces FFT.stft (STFT.swift:40-81) run over a set of signals.  Outputs are indexed
 * by global frame g = s*F + f with the layouts of ma_fft_forward_dev; `mag` optional.
 * Plans above 8192 points read the frames straight from the signal (window applied by the
 * loader) through the two-pass transforms; their inverse (ma_istft_*) passes the frames through
 * a plan-owned buffer that is allocated on the first such call. */
ma_status ma_stft_dev(ma_fft_plan* plan, const float* signals, int64_t length,
                      int64_t signal_stride, int64_t n_signals, float* out_a, float* out_b,
                      float* mag, int32_t mag_kind, float db_reference, int32_t layout);
/* Host form: the signals are cut into chunks that fit a lane of the context's workspace; with
 * pinned host memory (ma_host_alloc) copy-in, transform and copy-out of successive chunks overlap
 * on three streams and the host waits once, at the end; nothing is allocated per call. */
ma_status ma_stft_host(ma_fft_plan* plan, const float* signals, int64_t length,
                       int64_t signal_stride, int64_t n_signals, float* out_a, float* out_b,
                       float* mag, int32_t mag_kind, float db_reference, int32_t layout);

/* iSTFT of `frames` frames per signal: inverse DFT (1/N), synthesis window, overlap-add,
 * division by max(sum of squared window, floor), all in one pass.  Replaces FFT.istft
 * (STFT.swift:384-527); uses the true inverse transform (the reference runs the object's
 * forward-direction setup, which returns frames time-reversed).  `floor` is the already
 * validated window floor (STFT.swift:491-501).  out: n_signals rows of out_stride floats,
 * each holding (frames-1)*hop + N samples. */
ma_status ma_istft_dev(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                       int64_t n_signals, float* out, int64_t out_stride, float floor,
                       int32_t layout);
ma_status ma_istft_host(ma_fft_plan* plan, const float* in_a, const float* in_b, int64_t frames,
                        int64_t n_signals, float* out, int64_t out_stride, float floor,
                        int32_t layout);

/* ------------------------------------------------------------------ partitioned convolution
 * Replaces Convolution(device:mode: .partitioned(blockSize:)) + setKernel + process +
 * reset (Convolution.swift:112-125, :188-208, :250-322, :336-352, :529-758, :764-775),
 * for `n_channels` independent channels at once (the reference holds one object per
 * channel). */
ma_status ma_pconv_create(ma_context* ctx, int32_t block_size, int32_t n_channels, ma_pconv** out);
ma_status ma_pconv_destroy(ma_pconv* pc);
/* Partition `n_irs` impulse responses of `taps` floats (host memory, row-major) into
 * P = ceil(taps/B) zero-padded blocks and transform them; channel c uses IR
 * channel_to_ir[c] (NULL: every channel uses IR 0).  Allocates the delay line
 * (n_channels x P spectra) and clears it. */
ma_status ma_pconv_set_kernels(ma_pconv* pc, const float* irs, int64_t taps, int32_t n_irs,
                               const int32_t* channel_to_ir);
ma_status ma_pconv_partition_count(ma_pconv* pc, int32_t* partitions);
/* Tuning knob of the streaming step (no counterpart in the reference): into how many ranges of
 * partitions the multiply-accumulate of one step is split (ranges run as separate CTAs and their
 * partial spectra are added up afterwards; from 16 ranges up, groups of eight ranges form thread-block
 * clusters that add their sums up on chip).  ma_pconv_set_kernels picks a count that puts about five
 * CTAs on every SM; set_to > 0 replaces it (1 <= set_to <= min(64, partitions)), set_to <= 0 only
 * reports.  Results do not depend on it beyond float32 summation order. */
ma_status ma_pconv_step_splits(ma_pconv* pc, int32_t set_to, int32_t* splits);
/* Whole-signal call, as process(input:output:): every channel receives len samples
 * (row c at in + c*in_stride) and produces the full len + taps - 1 output samples
 * (row c at out + c*out_stride), ceil((len+taps-1)/B) blocks pushed through the delay
 * line; the delay line keeps its state for the next call.  `max_len` passed to
 * ma_pconv_reserve bounds len for the _dev form, which never allocates.  The _host form sends
 * groups of channels through the context's workspace lanes; with both host arrays pinned the
 * groups' copies in, convolutions and copies out overlap on three streams (see
 * ma_context_reserve_workspace). */
ma_status ma_pconv_reserve(ma_pconv* pc, int64_t max_len);
ma_status ma_pconv_process_dev(ma_pconv* pc, const float* in, int64_t len, int64_t in_stride,
                               float* out, int64_t out_stride);
ma_status ma_pconv_process_host(ma_pconv* pc, const float* in, int64_t len, int64_t in_stride,
                                float* out, int64_t out_stride);
/* Causal streaming step: one block of B input samples per channel in (row stride
 * in_stride), one block of B output samples out; the block's second half is kept in the
 * object and added to the next step's output.  Every step reads the whole delay line:
 * this is the HBM-streaming kernel.  No reference counterpart call (the reference loops
 * blocks inside process()); the arithmetic per block is Convolution.swift:580-757.
 * Back-to-back steps on one context overlap the start of a step with the end of the previous one;
 * the library detects by itself when anything else of its own was queued in between or when a
 * step's output is fed back as the next input.  A caller that fills in_block with a kernel of its
 * OWN on the context's stream (ma_context_stream) must keep one other stream operation of this
 * library (for instance ma_buffer_zero of a scratch word) or a stream/event wait between that
 * kernel and the step. */
ma_status ma_pconv_step_dev(ma_pconv* pc, const float* in_block, int64_t in_stride,
                            float* out_block, int64_t out_stride);
/* Zero the delay line, the write index and the overlap tail (Convolution.reset). */
ma_status ma_pconv_reset(ma_pconv* pc);

/* ------------------------------------------------------------------ one-shot FFT convolution
 * Replaces Convolution(device:mode: .fft) + setKernel(_:expectedInputSize:) + process
 * (Convolution.swift:188-208, :210-248, :437-493) for up to `max_signals` signals that share one
 * kernel.  fft_size is the next power of two >= expected_input + taps - 1 (at least 2);
 * MA_ERR_EMPTY_KERNEL for taps == 0, MA_ERR_SIZE_TOO_LARGE above 2^24.  The kernel (host memory)
 * is transformed once here; every work buffer is allocated here. */
ma_status ma_fftconv_create(ma_context* ctx, const float* kernel, int64_t taps, int64_t expected_input,
                            int32_t max_signals, ma_fftconv** out);
ma_status ma_fftconv_destroy(ma_fftconv* fc);
ma_status ma_fftconv_fft_size(ma_fftconv* fc, int64_t* fft_size);
/* Signal s (len samples at in + s*in_stride) is zero-padded to fft_size, transformed, multiplied
 * by the kernel spectrum and transformed back: out receives n_signals contiguous rows of fft_size
 * samples, the linear convolution in the first len + taps - 1 of them (the reference returns the
 * same fft_size samples).  len > expected_input would wrap around and is refused with
 * MA_ERR_INPUT_SIZE_MISMATCH (Convolution.swift:461-467); n_signals > max_signals gives
 * MA_ERR_BATCH_OVERFLOW.  The _dev form allocates nothing. */
ma_status ma_fftconv_process_dev(ma_fftconv* fc, const float* in, int64_t len, int64_t in_stride,
                                 int32_t n_signals, float* out);
ma_status ma_fftconv_process_host(ma_fftconv* fc, const float* in, int64_t len, int64_t in_stride,
                                  int32_t n_signals, float* out);

/* ------------------------------------------------------------------ biquad cascades
 * Replaces the biquad_filter_multichannel shader (Shaders/DSP.metal:697-744) and the processing
 * loops of BiquadFilter / FilterBank (Filters.swift:515-660, :845-868): `n_channels` independent
 * channels in [channel][sample] layout, each a cascade of `n_sections` (<= 32) Direct Form II
 * Transposed sections, y = b0 x + z1; z1 = b1 x - a1 y + z2; z2 = b2 x - a2 y, with the (z1, z2)
 * state of every channel and section kept in the object between calls.  Coefficient design
 * (Filters.swift:226-345) stays on the host. */
ma_status ma_biquad_create(ma_context* ctx, int32_t n_channels, int32_t n_sections, ma_biquad** out);
ma_status ma_biquad_destroy(ma_biquad* bq);
/* coeffs: n_sets x n_sections x (b0, b1, b2, a1, a2), host memory, a0 already divided out.
 * Channel c uses set channel_to_set[c]; NULL means one set shared by all channels. */
ma_status ma_biquad_set_coefficients(ma_biquad* bq, const float* coeffs, int32_t n_sets,
                                     const int32_t* channel_to_set);
/* Filters `samples` samples of every channel (row c at in + c*in_stride, out + c*out_stride) and
 * advances the states.  in_stride == 0 feeds one signal to every channel (a parallel filter
 * bank).  The _dev form allocates nothing. */
ma_status ma_biquad_process_dev(ma_biquad* bq, const float* in, int64_t in_stride, float* out,
                                int64_t out_stride, int64_t samples);
ma_status ma_biquad_process_host(ma_biquad* bq, const float* in, int64_t in_stride, float* out,
                                 int64_t out_stride, int64_t samples);
/* BiquadFilter.reset (Filters.swift:662-672); state exchange with the host as
 * n_channels x n_sections x (z1, z2). */
ma_status ma_biquad_reset(ma_biquad* bq);
ma_status ma_biquad_get_state(ma_biquad* bq, float* state);
ma_status ma_biquad_set_state(ma_biquad* bq, const float* state);
/* out[n] = scale * sum over channels of in[c*stride + n], summed in channel order: the mix step of
 * FilterBank.processParallel (Filters.swift:854-868). */
ma_status ma_channel_mix_dev(ma_context* ctx, const float* in, int32_t n_channels, int64_t stride,
                             int64_t samples, float scale, float* out);

#ifdef __cplusplus
}
#endif
#endif /* METALAUDIO_CUDA_H */
