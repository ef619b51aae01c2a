// Dynamic e4m3 quantisation for the 8-bit GEMM (ocb_gemm_fp8): every operand is scaled along its REDUCTION dimension,
// one fp32 scale per row of the K-major matrix that the tensor cores read.
//
//   rowwise      x [R, C]  ->  q [R, C],   scale[r] = amax(x[r, :]) / 448        (operand already K-major)
//   colwise^T    x [R, C]  ->  q [C, R],   scale[c] = amax(x[:, c]) / 448        (operand needed transposed: the weight
//                                                                                 in dgrad, both operands in wgrad)
//
// These stand in for the cast kernels torchao generates around Float8Linear in the reference
// (src/olmo_core/float8/__init__.py:25-162, src/olmo_core/float8/ao.py:153-239). One pass over the input each, plus a
// column-maximum pre-pass for the transposed form.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ocb_api.h"

namespace ocb {

constexpr float kE4M3Max = 448.f;

// Scale for a maximum magnitude; optionally rounded UP to a power of two, so that scaling is exact in floating point.
__device__ __forceinline__ float scale_for(float amax, int pow2) {
  const float s = fmaxf(amax, 1e-12f) / kE4M3Max;
  return pow2 ? exp2f(ceilf(log2f(s))) : s;
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// One warp per row; the row is read twice (the second time from L2 / L1).
__global__ void quantize_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                                        int rows, int cols, long long ldx, long long ldq, int pow2) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx);
  const int vecs = cols >> 3;
  float amax = 0.f;
  for (int i = lane; i < vecs; i += 32) {
    const uint4 u = in[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = scale_for(amax, pow2);
  const float inv = 1.f / s;
  if (lane == 0) scale[row] = s;
  uint2* out = reinterpret_cast<uint2*>(q + static_cast<long long>(row) * ldq);
  for (int i = lane; i < vecs; i += 32) {
    const uint4 u = in[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint8_t b[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      b[2 * k] = to_e4m3(f.x * inv);
      b[2 * k + 1] = to_e4m3(f.y * inv);
    }
    out[i] = *reinterpret_cast<const uint2*>(b);
  }
}

// Column maxima: block = 64 columns x 16 row slices; slices meet through atomicMax on the bit pattern (values >= 0).
__global__ void column_amax_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ amax, int rows, int cols,
                                   long long ldx, int rows_per_block) {
  const int c = blockIdx.x * 64 + threadIdx.x;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float m = 0.f;
  if (c < cols) {
    for (int r = r0 + threadIdx.y; r < r1; r += blockDim.y) m = fmaxf(m, fabsf(__bfloat162float(x[static_cast<long long>(r) * ldx + c])));
    atomicMax(reinterpret_cast<int*>(amax) + c, __float_as_int(m));
  }
}

// 64 x 64 tile transposed through shared memory; amax[c] becomes scale[c] in place (first row-block of each column tile).
__global__ void quantize_transpose_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ amax,
                                          uint8_t* __restrict__ qt, float* __restrict__ scale, int rows, int cols,
                                          long long ldx, long long ldq, int pow2) {
  __shared__ uint8_t tile[64][65];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 256 threads: 64 x 4
  const int c = c0 + tx;
  float inv = 0.f;
  if (c < cols) {
    const float s = scale_for(amax[c], pow2);
    inv = 1.f / s;
    if (blockIdx.y == 0 && ty == 0) scale[c] = s;
  }
  for (int r = ty; r < 64; r += 4) {
    const int row = r0 + r;
    uint8_t v = 0;
    if (row < rows && c < cols) v = to_e4m3(__bfloat162float(x[static_cast<long long>(row) * ldx + c]) * inv);
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int cc = ty; cc < 64; cc += 4) {
    const int out_row = c0 + cc, out_col = r0 + tx;
    if (out_row < cols && out_col < rows) qt[static_cast<long long>(out_row) * ldq + out_col] = tile[tx][cc];
  }
}

}  // namespace ocb

using namespace ocb;

extern "C" int ocb_quantize_e4m3_rowwise(const void* x, void* q, float* scale, int rows, int cols, long long ldx,
                                         long long ldq, int pow2, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ldx & 7) || (ldq & 7)) return -1;
  quantize_rowwise_kernel<<<(rows * 32 + 255) / 256, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scale, rows, cols, ldx, ldq, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// q_t: [cols, rows] bytes with row stride ldq; scale: [cols]; scratch: fp32 [cols].
extern "C" int ocb_quantize_e4m3_colwise_t(const void* x, void* q_t, float* scale, float* scratch, int rows, int cols,
                                           long long ldx, long long ldq, int pow2, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * cols, stream) != cudaSuccess) return -4;
  const int rows_per_block = 256;
  dim3 g1((cols + 63) / 64, (rows + rows_per_block - 1) / rows_per_block), b1(64, 16);
  column_amax_kernel<<<g1, b1, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch, rows, cols, ldx, rows_per_block);
  dim3 g2((cols + 63) / 64, (rows + 63) / 64);
  quantize_transpose_kernel<<<g2, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch,
                                                    reinterpret_cast<uint8_t*>(q_t), scale, rows, cols, ldx, ldq, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
