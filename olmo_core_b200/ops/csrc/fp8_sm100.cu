// Dynamic e4m3 quantisation for the 8-bit GEMM (ocb_gemm_fp8): every operand is scaled along its REDUCTION dimension,
// one fp32 scale per row of the K-major matrix that the tensor cores read.
//
//   rowwise      x [R, C]  ->  q [R, C],   scale[r] = amax(x[r, :]) / 448        (operand already K-major)
//   colwise^T    x [R, C]  ->  q [C, R],   scale[c] = amax(x[:, c]) / 448        (operand needed transposed: the weight
//                                                                                 in dgrad, both operands in wgrad)
//
// These stand in for the cast kernels torchao generates around Float8Linear in the reference
// (src/olmo_core/float8/__init__.py:25-162, src/olmo_core/float8/ao.py:153-239). One pass over the input each, plus a
// column-maximum pre-pass for the transposed form; every global access is 16 bytes wide (32-byte runs on the
// transposed side).

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

// Column maxima. A block of 256 threads covers 128 columns x rows_per_block rows: thread = (16-byte column group,
// one of 16 row slices), eight running maxima per thread, slices merged in shared memory, blocks through atomicMax on
// the bit pattern (values >= 0).
__global__ void __launch_bounds__(256)
column_amax_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ amax, int rows, int cols, long long ldx,
                   int rows_per_block) {
  __shared__ float part[16][129];
  const int cvec = threadIdx.x & 15, slice = threadIdx.x >> 4;
  const int c = blockIdx.x * 128 + cvec * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float m[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) m[k] = 0.f;
  if (c < cols) {
    for (int r = r0 + slice; r < r1; r += 16) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * ldx + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        m[2 * k] = fmaxf(m[2 * k], fabsf(f.x));
        m[2 * k + 1] = fmaxf(m[2 * k + 1], fabsf(f.y));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) part[slice][cvec * 8 + k] = m[k];
  __syncthreads();
  if (threadIdx.x < 128) {
    float v = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < 16; ++s2) v = fmaxf(v, part[s2][threadIdx.x]);
    const int col = blockIdx.x * 128 + threadIdx.x;
    if (col < cols) atomicMax(reinterpret_cast<int*>(amax) + col, __float_as_int(v));
  }
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// A [128 rows x 128 columns] tile of x goes through shared memory (16-byte loads, 65-word row pitch: conflict-free in
// both directions); a thread then owns two adjacent columns and 32 of the rows and writes 32 contiguous bytes to each
// of two rows of q_t. amax[c] becomes scale[c] (written by the first row-block of each column tile).
constexpr int QT_TILE = 128, QT_PITCH = 65;

__global__ void __launch_bounds__(256)
quantize_transpose_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ qt,
                          float* __restrict__ scale, int rows, int cols, long long ldx, long long ldq, int pow2) {
  __shared__ uint32_t tile[QT_TILE * QT_PITCH];
  const int c0 = blockIdx.x * QT_TILE, r0 = blockIdx.y * QT_TILE;
  const int t = threadIdx.x;
#pragma unroll
  for (int j = 0; j < (QT_TILE * QT_TILE / 8) / 256; ++j) {
    const int v = t + 256 * j;
    const int r = v >> 4, cvec = v & 15;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (r0 + r < rows && c0 + cvec * 8 < cols)
      u = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r0 + r) * ldx + c0 + cvec * 8);
    uint32_t* dst = tile + r * QT_PITCH + cvec * 4;
    dst[0] = u.x; dst[1] = u.y; dst[2] = u.z; dst[3] = u.w;
  }
  __syncthreads();
  const int cpair = t & 63, b = t >> 6;
  const int c = c0 + 2 * cpair;
  if (c >= cols) return;  // cols % 8 == 0: both columns of a live pair exist
  const float s_lo = scale_for(amax[c], pow2), s_hi = scale_for(amax[c + 1], pow2);
  const float inv_lo = 1.f / s_lo, inv_hi = 1.f / s_hi;
  if (blockIdx.y == 0 && b == 0) {
    scale[c] = s_lo;
    scale[c + 1] = s_hi;
  }
  const int rbase = r0 + b * 32;
  if (rbase >= rows) return;
  uint32_t lo[8], hi[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float fl[4], fh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = tile[(b * 32 + g * 4 + i) * QT_PITCH + cpair];
      fl[i] = __uint_as_float(w << 16) * inv_lo;
      fh[i] = __uint_as_float(w & 0xffff0000u) * inv_hi;
    }
    lo[g] = e4m3x4(fl[0], fl[1], fl[2], fl[3]);
    hi[g] = e4m3x4(fh[0], fh[1], fh[2], fh[3]);
  }
  uint8_t* out_lo = qt + static_cast<long long>(c) * ldq + rbase;
  uint8_t* out_hi = qt + static_cast<long long>(c + 1) * ldq + rbase;
  if (rbase + 32 <= rows) {
    reinterpret_cast<uint4*>(out_lo)[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    reinterpret_cast<uint4*>(out_lo)[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    reinterpret_cast<uint4*>(out_hi)[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    reinterpret_cast<uint4*>(out_hi)[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (rbase + i < rows) {
        out_lo[i] = static_cast<uint8_t>(lo[i >> 2] >> (8 * (i & 3)));
        out_hi[i] = static_cast<uint8_t>(hi[i >> 2] >> (8 * (i & 3)));
      }
    }
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
  if ((cols & 7) || (ldx & 7) || (ldq & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q_t) & 15))
    return -1;
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * cols, stream) != cudaSuccess) return -4;
  const int rows_per_block = 512;
  dim3 g1((cols + 127) / 128, (rows + rows_per_block - 1) / rows_per_block);
  column_amax_kernel<<<g1, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch, rows, cols, ldx, rows_per_block);
  dim3 g2((cols + QT_TILE - 1) / QT_TILE, (rows + QT_TILE - 1) / QT_TILE);
  quantize_transpose_kernel<<<g2, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch,
                                                    reinterpret_cast<uint8_t*>(q_t), scale, rows, cols, ldx, ldq, pow2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
