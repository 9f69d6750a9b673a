/* Entry points of libterapipe (_tp_sm100.so) that never allocate.
 *
 * This header has no counterpart in the reference project (which ships no native code).
 *
 * Who needs it: callers that must not call cudaMalloc or any allocating library routine while
 * they run -- for example code inside a real-time or latency-critical loop, a plug-in hosted by
 * a process that owns all device memory through its own pool, or a caller that runs while the
 * CUDA allocator is locked by someone else.  The regular LayerNorm backward
 * (tp_layernorm_bwd) needs a caller-provided scratch buffer for its per-CTA partial sums; such
 * callers may have nowhere to get one from.
 *
 * tp_layernorm_bwd_noalloc is the same kernel with that scratch placed in a fixed array that is
 * part of the library image: 160 slots x 2 x 4096 floats = 5 242 880 bytes of device memory on
 * every GPU that loads the library, held until the process exits.
 *
 * Limits and rules:
 *   - H (row width) at most 4096 and a multiple of 8; larger rows are rejected with
 *     status -4 ("size beyond the built-in maximum"), nothing is launched.
 *   - The first call on each device looks up the device address of the array
 *     (cudaGetSymbolAddress, with that device current).  Make that first call before starting
 *     any stream capture on the device.
 *   - All calls on a device share the one array.  Each call overwrites the slots it uses before
 *     reading them, so nothing has to be cleared between calls, but two calls that overlap on
 *     the GPU (different streams) race on it: serialise them.
 *   - Inputs and outputs are still the caller's: dy, x, gamma, dres (optional), dx are 16-bit
 *     (dtype 0 = fp16, 1 = bf16) row-major [rows][H]; mean, rstd are fp32 [rows];
 *     dgamma, dbeta are fp32 [H] and are ADDED to.
 *   - Returns 0 on success, a negative status otherwise (see common.cuh: ErrorCode).
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int tp_layernorm_bwd_noalloc(int dtype, const void* dy, const void* x, const float* mean,
                             const float* rstd, const void* gamma, const void* dres, void* dx,
                             float* dgamma, float* dbeta, int rows, int H, void* stream);

/* Size of the built-in scratch array in floats (for documentation and tests). */
long long tp_layernorm_bwd_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
