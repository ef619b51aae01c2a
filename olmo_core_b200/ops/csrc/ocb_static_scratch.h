// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it is an addition of this
// library.
//
// Who needs it: code that runs where an allocation is not possible or not wanted -- a caller that has
// handed all free device memory to a caching allocator it cannot re-enter (e.g. from inside another
// allocator's callback), a C or C++ host without a tensor library to provide scratch buffers, or a
// latency-critical loop that wants the guarantee that a call never reaches cudaMalloc / cudaFree (both
// may synchronise the whole device). The regular entry point `ocb_rmsnorm_bwd` asks the caller for a
// [ocb_norm_bwd_partials(), group] fp32 scratch buffer for the per-block weight-gradient partials and a
// second call (`ocb_reduce_partials`) to fold them; here the partials live in a fixed array inside the
// library's device image and both steps are issued by one call.
//
// Properties
//   * No allocation: the call uses neither cudaMalloc / cudaFree nor any allocating library routine.
//     The scratch is a file-scope `static __device__` array of
//         ocb_norm_bwd_partials() x OCB_STATIC_SCRATCH_MAX_GROUP fp32  (296 x 4096 x 4 B = 4.6 MiB per device).
//   * Size limit: `group` (the normalised width) must be <= OCB_STATIC_SCRATCH_MAX_GROUP when a weight
//     gradient is requested. Wider groups are rejected with OCB_ERR_STATIC_SCRATCH_TOO_SMALL before
//     anything is launched; use `ocb_rmsnorm_bwd` with a caller-provided buffer for those.
//   * Set-up: the first call on each device resolves the array's device address
//     (cudaGetSymbolAddress). That first call may initialise the CUDA module, so make it before starting
//     a stream capture; later calls on that device only enqueue work on `stream`.
//   * Device: the array that is used is the one of the CURRENT device (cudaGetDevice) at the time of the call, so
//     the current device must be the device `stream` belongs to.
//   * Empty input (rows <= 0): nothing is launched; with dw_accumulate == 0 the weight gradient is set to zero.
//   * Shared state: every call on a device uses the same array. The rows a call is going to use are
//     cleared (cudaMemsetAsync on `stream`) before its kernel runs, so consecutive calls on ONE stream
//     are safe. Calls that can overlap -- different streams, or different host threads on different
//     streams -- race on the array and produce wrong weight gradients; serialise them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OCB_STATIC_SCRATCH_MAX_GROUP 4096
#define OCB_ERR_STATIC_SCRATCH_TOO_SMALL (-6)
#define OCB_ERR_STATIC_SCRATCH_SETUP (-7)

// Largest `group` accepted together with a weight gradient (= OCB_STATIC_SCRATCH_MAX_GROUP).
int ocb_rmsnorm_bwd_static_max_group(void);

// dx = d rmsnorm(x)*w / dx given dy, and dw[c] (+)= sum over rows and groups of dy * x * rstd.
//   dy, x, dx : [rows, cols] activations (act_dtype), row strides lddy / ldx / lddx (elements)
//   w         : [group] weight (w_dtype) or null for a weightless norm
//   rstd      : [rows * cols / group] fp32, saved by ocb_rmsnorm_fwd
//   dw        : [group] fp32 or bf16 (dw_dtype), or null when no weight gradient is wanted
//   dw_accumulate : 0 = overwrite dw, 1 = add to it
// Returns 0, a negative launcher code, or one of the OCB_ERR_STATIC_SCRATCH_* codes.
int ocb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                           int dw_accumulate, int rows, int cols, int group, long long lddy, long long ldx,
                           long long lddx, int act_dtype, int w_dtype, int dw_dtype, cudaStream_t stream);

// Human-readable text for the return codes of ocb_rmsnorm_bwd_static (static storage, never null).
const char* ocb_rmsnorm_bwd_static_strerror(int code);

#ifdef __cplusplus
}
#endif
