// Micro-scaling (MX) quantisation to e4m3 with one E8M0 (power-of-two) scale per 32 consecutive elements of the
// REDUCTION dimension, for the block-scaled tensor-core GEMM of gemm_mx_sm100.cu. This is the cast that torchao's
// MXLinear performs around its GEMMs in the reference (src/olmo_core/float8/ao.py:190-239, selected by
// src/olmo_core/float8/__init__.py:118-130).
//
//   rowwise      x [R, C]  ->  q   [R, C] e4m3, scale per (row, 32 columns)      operand already K-major
//   colwise^T    x [R, C]  ->  q_t [C, R] e4m3, scale per (column, 32 rows)      operand needed transposed: the weight
//                                                                                in dgrad, both operands in wgrad
//
// The scales are written directly in the layout the tensor core reads them in: 512-byte blocks that hold the 4 scales
// of 128 rows for 128 consecutive reduction elements, byte (row % 32) * 16 + (row / 32 % 4) * 4 + (block % 4), blocks
// ordered [row / 128][reduction / 128]. One 512-byte bulk copy per tile and stage then feeds tcgen05.cp unchanged.
//
// Scale rounding: mode 0 ("rceil") picks the smallest power of two s with amax / s <= 448, so nothing saturates;
// mode 1 ("floor") is the OCP MX rule s = 2^(floor(log2 amax) - 8) with a saturating cast; mode 2 ("ceil") rounds the
// exponent of amax up instead, mode 3 ("even") rounds amax to the nearest value representable with e4m3's mantissa first.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ocb_api.h"

namespace ocb {
namespace mxq {

__device__ __forceinline__ long long sf_offset(int row, int kblock, int k_atoms) {
  return (static_cast<long long>(row >> 7) * k_atoms + (kblock >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
         (kblock & 3);
}

// Biased E8M0 exponent for a block maximum.
__device__ __forceinline__ uint32_t e8m0_for(float amax, int mode) {
  uint32_t e;
  if (mode == 0) {
    const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.f));
    e = (bits >> 23) + ((bits & 0x7FFFFFu) != 0u ? 1u : 0u);
  } else {
    // floor / ceil / even: the power of two at (below, above, nearest in e4m3's 3 mantissa bits to) the maximum, then
    // 2^-8 of it, so that the maximum lands in e4m3's top binade
    uint32_t bits = __float_as_uint(amax);
    if (mode == 3) bits += 1u << 19;
    uint32_t ea = bits >> 23;
    if (mode == 2 && (bits & 0x7FFFFFu) != 0u) ea += 1u;
    e = ea > 8u ? ea - 8u : 0u;
  }
  return min(e, 253u);
}
// 1 / 2^(e - 127), exact.
__device__ __forceinline__ float inv_scale_of(uint32_t e) { return __uint_as_float((254u - e) << 23); }

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One thread per 8 consecutive elements; the 4 threads of a 32-element block meet through two shuffles.
__global__ void __launch_bounds__(256)
quantize_mx_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                           int rows, int cols, long long ldx, long long ldq, int mode) {
  const int vecs_per_row = cols >> 3;
  const long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(rows) * vecs_per_row;
  const bool live = v < total;  // cols % 32 == 0, so the 4 threads of a block are live or dead together
  const int row = live ? static_cast<int>(v / vecs_per_row) : 0;
  const int cv = live ? static_cast<int>(v - static_cast<long long>(row) * vecs_per_row) : 0;
  float f[8];
  float amax = 0.f;
  if (live) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + cv * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 p = __bfloat1622float2(h[k]);
      f[2 * k] = p.x;
      f[2 * k + 1] = p.y;
      amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
    }
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  const uint32_t e = e8m0_for(amax, mode);
  const float inv = inv_scale_of(e);
  uint2 o;
  o.x = e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
  o.y = e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
  *reinterpret_cast<uint2*>(q + static_cast<long long>(row) * ldq + cv * 8) = o;
  if ((cv & 3) == 0) sf[sf_offset(row, cv >> 2, cols >> 7)] = static_cast<uint8_t>(e);
}

// A [128 rows x 128 columns] tile of x goes through shared memory; a thread then owns two adjacent columns and one
// 32-row block of them: it reads them down the tile (conflict-free: 65-word row pitch), and writes 32 bytes to each of
// two rows of q_t.
constexpr int T_ROWS = 128, T_COLS = 128, T_PITCH = 65;  // pitch in 32-bit words (two bf16 each)

__global__ void __launch_bounds__(256)
quantize_mx_colwise_t_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q_t, uint8_t* __restrict__ sf,
                             int rows, int cols, long long ldx, long long ldq, int mode) {
  __shared__ uint32_t tile[T_ROWS * T_PITCH];
  const int c0 = blockIdx.x * T_COLS, r0 = blockIdx.y * T_ROWS;
  const int t = threadIdx.x;
#pragma unroll
  for (int j = 0; j < (T_ROWS * T_COLS / 8) / 256; ++j) {
    const int v = t + 256 * j;
    const int r = v >> 4, cvec = v & 15;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (c0 + cvec * 8 < cols) u = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r0 + r) * ldx + c0 + cvec * 8);
    uint32_t* dst = tile + r * T_PITCH + cvec * 4;
    dst[0] = u.x; dst[1] = u.y; dst[2] = u.z; dst[3] = u.w;
  }
  __syncthreads();
  const int cpair = t & 63, b = t >> 6;
  const int c = c0 + 2 * cpair;
  if (c >= cols) return;  // cols % 8 == 0: a live pair is live in both columns
  float lo[32], hi[32];
  float amax_lo = 0.f, amax_hi = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint32_t w = tile[(b * 32 + i) * T_PITCH + cpair];
    lo[i] = __uint_as_float(w << 16);
    hi[i] = __uint_as_float(w & 0xffff0000u);
    amax_lo = fmaxf(amax_lo, fabsf(lo[i]));
    amax_hi = fmaxf(amax_hi, fabsf(hi[i]));
  }
  const uint32_t e_lo = e8m0_for(amax_lo, mode), e_hi = e8m0_for(amax_hi, mode);
  const float inv_lo = inv_scale_of(e_lo), inv_hi = inv_scale_of(e_hi);
  uint4* out_lo = reinterpret_cast<uint4*>(q_t + static_cast<long long>(c) * ldq + r0 + b * 32);
  uint4* out_hi = reinterpret_cast<uint4*>(q_t + static_cast<long long>(c + 1) * ldq + r0 + b * 32);
#pragma unroll
  for (int v = 0; v < 2; ++v) {
    uint4 a, h;
    a.x = e4m3x4(lo[16 * v + 0] * inv_lo, lo[16 * v + 1] * inv_lo, lo[16 * v + 2] * inv_lo, lo[16 * v + 3] * inv_lo);
    a.y = e4m3x4(lo[16 * v + 4] * inv_lo, lo[16 * v + 5] * inv_lo, lo[16 * v + 6] * inv_lo, lo[16 * v + 7] * inv_lo);
    a.z = e4m3x4(lo[16 * v + 8] * inv_lo, lo[16 * v + 9] * inv_lo, lo[16 * v + 10] * inv_lo, lo[16 * v + 11] * inv_lo);
    a.w = e4m3x4(lo[16 * v + 12] * inv_lo, lo[16 * v + 13] * inv_lo, lo[16 * v + 14] * inv_lo, lo[16 * v + 15] * inv_lo);
    h.x = e4m3x4(hi[16 * v + 0] * inv_hi, hi[16 * v + 1] * inv_hi, hi[16 * v + 2] * inv_hi, hi[16 * v + 3] * inv_hi);
    h.y = e4m3x4(hi[16 * v + 4] * inv_hi, hi[16 * v + 5] * inv_hi, hi[16 * v + 6] * inv_hi, hi[16 * v + 7] * inv_hi);
    h.z = e4m3x4(hi[16 * v + 8] * inv_hi, hi[16 * v + 9] * inv_hi, hi[16 * v + 10] * inv_hi, hi[16 * v + 11] * inv_hi);
    h.w = e4m3x4(hi[16 * v + 12] * inv_hi, hi[16 * v + 13] * inv_hi, hi[16 * v + 14] * inv_hi, hi[16 * v + 15] * inv_hi);
    out_lo[v] = a;
    out_hi[v] = h;
  }
  const int kblock = (r0 >> 5) + b, k_atoms = rows >> 7;
  sf[sf_offset(c, kblock, k_atoms)] = static_cast<uint8_t>(e_lo);
  sf[sf_offset(c + 1, kblock, k_atoms)] = static_cast<uint8_t>(e_hi);
}

}  // namespace mxq
}  // namespace ocb

using namespace ocb::mxq;

extern "C" long long ocb_mx_scale_bytes(int rows, int k) {
  return static_cast<long long>((rows + 127) / 128) * (k / 128) * 512;
}

extern "C" int ocb_quantize_mx_rowwise(const void* x, void* q, void* sf, int rows, int cols, long long ldx, long long ldq,
                                       int mode, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 127) || (ldx & 7) || (ldq & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15))
    return -1;
  const long long total = static_cast<long long>(rows) * (cols >> 3);
  quantize_mx_rowwise_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(sf), rows, cols,
      ldx, ldq, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// q_t: [cols, rows] bytes with row pitch ldq; rows (the reduction of the product q_t feeds) must be a multiple of 128.
extern "C" int ocb_quantize_mx_colwise_t(const void* x, void* q_t, void* sf, int rows, int cols, long long ldx,
                                         long long ldq, int mode, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((rows & 127) || (cols & 7) || (ldx & 7) || (ldq & 15) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(q_t) & 15))
    return -1;
  dim3 grid((cols + T_COLS - 1) / T_COLS, rows / T_ROWS);
  quantize_mx_colwise_t_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                         reinterpret_cast<uint8_t*>(q_t), reinterpret_cast<uint8_t*>(sf),
                                                         rows, cols, ldx, ldq, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
