// Memory-bound kernels for sm_100a: RMSNorm (+residual), fused QK-norm + rotary embedding, SwiGLU,
// cross-entropy (+z-loss) with in-place gradient, embedding gather / scatter-add, SkipStep-AdamW and
// sum-of-squares. All use 128-bit accesses, fp32 math, and one pass over HBM per tensor.
//
// Numerics follow the reference formulas:
//   RMSNorm        src/olmo_core/nn/layer_norm.py:215-236   (fp32 stats, weight multiply, then cast)
//   RoPE           src/olmo_core/nn/rope.py:470-578         (rotate-half, fp32, cached sin/cos)
//   SwiGLU         src/olmo_core/nn/feed_forward.py:165-171
//   CE + z-loss    src/olmo_core/nn/functional/cross_entropy_loss.py:12-50
//   SkipStepAdamW  src/olmo_core/optim/adamw.py:12-47

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {

template <typename T>
struct Vec8;

template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  // round-trip through the storage type (used where the reference materialises an intermediate)
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};

constexpr int kNormThreads = 256;
constexpr int kNormBwdBlocks = 296;  // 2 x 148 SMs: persistent grid for the weight-gradient partials

// Sum over a group of `tpg` consecutive threads (tpg is a power of two, <= blockDim). Uses shuffles
// inside a warp and shared memory across warps. `sbuf` must hold blockDim/32 floats.
__device__ __forceinline__ float group_sum(float v, int tpg, float* sbuf) {
  if (tpg <= 32) {
    for (int o = tpg >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  }
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sbuf[warp] = v;
  __syncthreads();
  const int wpg = tpg >> 5;
  const int g0 = (warp / wpg) * wpg;
  float s = 0.f;
  for (int i = 0; i < wpg; ++i) s += sbuf[g0 + i];
  return s;
}

// ----------------------------------------------------------------------------------------------------
// RMSNorm forward. Each group of `tpg` threads owns one normalisation group; a thread walks the group
// in 8-element vectors with stride tpg. The row is re-read from L1 for the second pass.
// ----------------------------------------------------------------------------------------------------
template <typename T, typename W>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const T* __restrict__ x, const W* __restrict__ w, const T* __restrict__ resid, T* __restrict__ y,
                   float* __restrict__ rstd_out, long long n_groups, int groups_per_row, int group, int tpg,
                   long long ldx, long long ldy, long long ldr, float eps) {
  __shared__ float sbuf[kNormThreads / 32];
  const int gpb = kNormThreads / tpg;  // groups per block
  const int gi = threadIdx.x / tpg, ti = threadIdx.x % tpg;
  const int nvec = group / 8;
  for (long long g0 = static_cast<long long>(blockIdx.x) * gpb; g0 < n_groups; g0 += static_cast<long long>(gridDim.x) * gpb) {
    const long long g = g0 + gi;
    const bool active = g < n_groups;
    const long long row = active ? g / groups_per_row : 0;
    const int gcol = active ? static_cast<int>(g % groups_per_row) * group : 0;
    const T* xr = x + row * ldx + gcol;
    float ss = 0.f;
    if (active) {
      for (int v = ti; v < nvec; v += tpg) {
        float f[8];
        Vec8<T>::load(xr + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
    }
    ss = group_sum(ss, tpg, sbuf);
    const float rstd = rsqrtf(ss / static_cast<float>(group) + eps);
    if (active) {
      if (ti == 0 && rstd_out != nullptr) rstd_out[g] = rstd;
      T* yr = y + row * ldy + gcol;
      const T* rr = resid ? resid + row * ldr + gcol : nullptr;
      const W* wr = w;
      for (int v = ti; v < nvec; v += tpg) {
        float f[8], wf[8], o[8];
        Vec8<T>::load(xr + v * 8, f);
        if (wr) {
          Vec8<W>::load(wr + v * 8, wf);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) wf[j] = 1.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[j] * rstd * wf[j];
        if (rr) {
          float rf[8];
          Vec8<T>::load(rr + v * 8, rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rf[j] + Vec8<T>::round(o[j]);
        }
        Vec8<T>::store(yr + v * 8, o);
      }
    }
  }
}

// RMSNorm backward: dx and per-block partial sums of dw. Block b handles groups b, b+grid, ... with the
// same thread->column mapping every iteration so dw accumulates in registers (up to kMaxVec vectors).
constexpr int kMaxVec = 4;

// MAXV = 8-element vectors per thread: 2 covers groups up to 4096 columns with two blocks per SM (the persistent grid size); 4 covers up to
// 8192 columns at one block per SM.
template <typename T, typename W, int MAXV>
__global__ void __launch_bounds__(kNormThreads, MAXV == 2 ? 2 : 1)
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const W* __restrict__ w,
                   const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ dw_partial,
                   long long n_groups, int groups_per_row, int group, int tpg, long long lddy, long long ldx,
                   long long lddx) {
  __shared__ float sbuf[kNormThreads / 32];
  const int gpb = kNormThreads / tpg;
  const int gi = threadIdx.x / tpg, ti = threadIdx.x % tpg;
  const int nvec = group / 8;
  float dw[MAXV][8], wf[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = ti + i * tpg;  // the thread's columns are the same for every group it visits: load w once
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw[i][j] = 0.f; wf[i][j] = 1.f; }
    if (w != nullptr && v < nvec) Vec8<W>::load(w + v * 8, wf[i]);
  }

  for (long long g0 = static_cast<long long>(blockIdx.x) * gpb; g0 < n_groups; g0 += static_cast<long long>(gridDim.x) * gpb) {
    const long long g = g0 + gi;
    const bool active = g < n_groups;
    const long long row = active ? g / groups_per_row : 0;
    const int gcol = active ? static_cast<int>(g % groups_per_row) * group : 0;
    const T* xr = x + row * ldx + gcol;
    const T* dyr = dy + row * lddy + gcol;
    const float rstd = active ? rstd_in[g] : 0.f;
    // Every load of the row is issued before anything is consumed (2 * MAXV 16-byte loads in flight per thread); the
    // values stay in registers for the second phase, so global memory is read exactly once.
    float xf[MAXV][8], gf[MAXV][8];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = ti + i * tpg;
      if (active && v < nvec) {
        Vec8<T>::load(xr + v * 8, xf[i]);
        Vec8<T>::load(dyr + v * 8, gf[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xf[i][j] = gf[i][j] = 0.f;
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += gf[i][j] * wf[i][j] * xf[i][j] * rstd;
    dot = group_sum(dot, tpg, sbuf);
    const float c = dot / static_cast<float>(group);
    if (active) {
      T* dxr = dx + row * lddx + gcol;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int v = ti + i * tpg;
        if (v < nvec) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xhat = xf[i][j] * rstd;
            o[j] = rstd * (gf[i][j] * wf[i][j] - xhat * c);
            dw[i][j] += gf[i][j] * xhat;
          }
          Vec8<T>::store(dxr + v * 8, o);
        }
      }
    }
  }
  if (dw_partial != nullptr) {
    // Thread (gi, ti) holds columns {(ti + i*tpg)*8 .. +8}. Groups that share a block also share columns,
    // so they are combined with atomics on the block's private partial row (zeroed by the launcher).
    float* prow = dw_partial + static_cast<long long>(blockIdx.x) * group;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = ti + i * tpg;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (gpb == 1) prow[v * 8 + j] = dw[i][j];
          else atomicAdd(&prow[v * 8 + j], dw[i][j]);
        }
      }
    }
  }
}

// out[c] (+)= sum_p partial[p, c]. Block = 32 columns x 32 slices of the partial rows: every thread adds up its slice with
// independent loads, the slices meet in shared memory, and the summation order is fixed (deterministic).
template <typename O>
__global__ void __launch_bounds__(1024)
reduce_partials_kernel(const float* __restrict__ partial, O* __restrict__ out, int n_partial, int cols, int accumulate) {
  __shared__ float tile[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols) {
    for (int p = threadIdx.y; p < n_partial; p += 32) s += partial[static_cast<long long>(p) * cols + c];
  }
  tile[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += tile[y][threadIdx.x];
    if (accumulate) t += static_cast<float>(out[c]);
    out[c] = static_cast<O>(t);
  }
}

// ----------------------------------------------------------------------------------------------------
// Fused (optional) RMSNorm + rotary embedding. One block per token row; each thread owns "pair vectors":
// 8 channels (h, o..o+8) and their rotate-half partners (h, o+half..). norm_mode 1 = stats over the
// full row, 2 = stats per head.
// ----------------------------------------------------------------------------------------------------
constexpr int kMaxPv = 2;  // up to 2*256 pair vectors = 8192 channels per row

// PV = pair vectors per thread (1 covers rows of up to 4096 channels and leaves room for 3-4 resident blocks per SM).
template <typename T, typename W, bool BWD, int PV>
__global__ void __launch_bounds__(kNormThreads, PV == 1 ? (BWD ? 3 : 4) : 2)
norm_rope_kernel(const T* __restrict__ in, const T* __restrict__ x_saved, const W* __restrict__ w,
                 float* __restrict__ rstd_io, T* __restrict__ out, float* __restrict__ dw_partial,
                 const float* __restrict__ sin_t, const float* __restrict__ cos_t, const int* __restrict__ pos_ids,
                 int rows, int n_heads, int head_dim, int seq_len, int pos_offset, int norm_mode, long long ld_in,
                 long long ld_x, long long ld_out, float eps) {
  __shared__ float sbuf[kNormThreads / 32];
  const int half = head_dim / 2;
  const int pv_per_head = half / 8;  // power of two, <= 32 (checked by the launcher)
  const int n_pv = n_heads * pv_per_head;
  const int cols = n_heads * head_dim;
  float dwa[PV][8], dwb[PV][8];
#pragma unroll
  for (int i = 0; i < PV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwa[i][j] = dwb[i][j] = 0.f;

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int pos = pos_ids ? pos_ids[row] : (row % seq_len) + pos_offset;
    const float* sr = sin_t + static_cast<long long>(pos) * head_dim;
    const float* cr = cos_t + static_cast<long long>(pos) * head_dim;
    const T* inr = in + static_cast<long long>(row) * ld_in;
    T* outr = out + static_cast<long long>(row) * ld_out;
    if (!BWD) {
      float xa[PV][8], xb[PV][8], rstd_h[PV];
      float ss_row = 0.f;
#pragma unroll
      for (int i = 0; i < PV; ++i) {
        const int pv = threadIdx.x + i * kNormThreads;
        const bool on = pv < n_pv;
        const int h = on ? pv / pv_per_head : 0, o = on ? (pv % pv_per_head) * 8 : 0;
        float ss = 0.f;
        if (on) {
          Vec8<T>::load(inr + h * head_dim + o, xa[i]);
          Vec8<T>::load(inr + h * head_dim + half + o, xb[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += xa[i][j] * xa[i][j] + xb[i][j] * xb[i][j];
        }
        ss_row += ss;
        rstd_h[i] = 1.f;
        if (norm_mode == 2) {
          for (int s = pv_per_head >> 1; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
          rstd_h[i] = rsqrtf(ss / static_cast<float>(head_dim) + eps);
          if (on && (pv % pv_per_head) == 0 && rstd_io) rstd_io[static_cast<long long>(row) * n_heads + h] = rstd_h[i];
        }
      }
      float rstd_row = 1.f;
      if (norm_mode == 1) {
        ss_row = group_sum(ss_row, kNormThreads, sbuf);
        rstd_row = rsqrtf(ss_row / static_cast<float>(cols) + eps);
        if (threadIdx.x == 0 && rstd_io) rstd_io[row] = rstd_row;
      }
#pragma unroll
      for (int i = 0; i < PV; ++i) {
        const int pv = threadIdx.x + i * kNormThreads;
        if (pv < n_pv) {
          const int h = pv / pv_per_head, o = (pv % pv_per_head) * 8;
          float ya[8], yb[8];
          if (norm_mode != 0) {
            const float rs = norm_mode == 1 ? rstd_row : rstd_h[i];
            float wa[8], wb[8];
            const int wofs = norm_mode == 1 ? h * head_dim : 0;
            Vec8<W>::load(w + wofs + o, wa);
            Vec8<W>::load(w + wofs + half + o, wb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              ya[j] = Vec8<T>::round(xa[i][j] * rs * wa[j]);
              yb[j] = Vec8<T>::round(xb[i][j] * rs * wb[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) { ya[j] = xa[i][j]; yb[j] = xb[i][j]; }
          }
          float oa[8], ob[8], c_lo[8], s_lo[8], c_hi[8], s_hi[8];
          Vec8<float>::load(cr + o, c_lo);
          Vec8<float>::load(sr + o, s_lo);
          Vec8<float>::load(cr + half + o, c_hi);
          Vec8<float>::load(sr + half + o, s_hi);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            oa[j] = ya[j] * c_lo[j] - yb[j] * s_lo[j];
            ob[j] = yb[j] * c_hi[j] + ya[j] * s_hi[j];
          }
          Vec8<T>::store(outr + h * head_dim + o, oa);
          Vec8<T>::store(outr + h * head_dim + half + o, ob);
        }
      }
    } else {
      const T* xr = x_saved + static_cast<long long>(row) * ld_x;
      float ga[PV][8], gb[PV][8], c_h[PV];
      float dot_row = 0.f;
      const float rstd_row = norm_mode == 1 ? rstd_io[row] : 1.f;
#pragma unroll
      for (int i = 0; i < PV; ++i) {
        const int pv = threadIdx.x + i * kNormThreads;
        const bool on = pv < n_pv;
        const int h = on ? pv / pv_per_head : 0, o = on ? (pv % pv_per_head) * 8 : 0;
        float dot = 0.f;
        if (on) {
          float da[8], db[8], c_lo[8], s_lo[8], c_hi[8], s_hi[8];
          Vec8<T>::load(inr + h * head_dim + o, da);
          Vec8<T>::load(inr + h * head_dim + half + o, db);
          Vec8<float>::load(cr + o, c_lo);
          Vec8<float>::load(sr + o, s_lo);
          Vec8<float>::load(cr + half + o, c_hi);
          Vec8<float>::load(sr + half + o, s_hi);
#pragma unroll
          for (int j = 0; j < 8; ++j) {  // transpose of the rotation
            ga[i][j] = da[j] * c_lo[j] + db[j] * s_hi[j];
            gb[i][j] = db[j] * c_hi[j] - da[j] * s_lo[j];
          }
          if (norm_mode != 0) {
            float xa[8], xb[8], wa[8], wb[8];
            Vec8<T>::load(xr + h * head_dim + o, xa);
            Vec8<T>::load(xr + h * head_dim + half + o, xb);
            const int wofs = norm_mode == 1 ? h * head_dim : 0;
            Vec8<W>::load(w + wofs + o, wa);
            Vec8<W>::load(w + wofs + half + o, wb);
            const float rs = norm_mode == 1 ? rstd_row : rstd_io[static_cast<long long>(row) * n_heads + h];
#pragma unroll
            for (int j = 0; j < 8; ++j) dot += (ga[i][j] * wa[j] * xa[j] + gb[i][j] * wb[j] * xb[j]) * rs;
          }
        }
        dot_row += dot;
        c_h[i] = 0.f;
        if (norm_mode == 2) {
          for (int s = pv_per_head >> 1; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
          c_h[i] = dot / static_cast<float>(head_dim);
        }
      }
      float c_row = 0.f;
      if (norm_mode == 1) c_row = group_sum(dot_row, kNormThreads, sbuf) / static_cast<float>(cols);
#pragma unroll
      for (int i = 0; i < PV; ++i) {
        const int pv = threadIdx.x + i * kNormThreads;
        if (pv < n_pv) {
          const int h = pv / pv_per_head, o = (pv % pv_per_head) * 8;
          float oa[8], ob[8];
          if (norm_mode != 0) {
            float xa[8], xb[8], wa[8], wb[8];
            Vec8<T>::load(xr + h * head_dim + o, xa);
            Vec8<T>::load(xr + h * head_dim + half + o, xb);
            const int wofs = norm_mode == 1 ? h * head_dim : 0;
            Vec8<W>::load(w + wofs + o, wa);
            Vec8<W>::load(w + wofs + half + o, wb);
            const float rs = norm_mode == 1 ? rstd_row : rstd_io[static_cast<long long>(row) * n_heads + h];
            const float c = norm_mode == 1 ? c_row : c_h[i];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float xha = xa[j] * rs, xhb = xb[j] * rs;
              oa[j] = rs * (ga[i][j] * wa[j] - xha * c);
              ob[j] = rs * (gb[i][j] * wb[j] - xhb * c);
              dwa[i][j] += ga[i][j] * xha;
              dwb[i][j] += gb[i][j] * xhb;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) { oa[j] = ga[i][j]; ob[j] = gb[i][j]; }
          }
          Vec8<T>::store(outr + h * head_dim + o, oa);
          Vec8<T>::store(outr + h * head_dim + half + o, ob);
        }
      }
    }
  }
  if (BWD && dw_partial != nullptr && norm_mode != 0) {
    const int wcols = norm_mode == 1 ? cols : head_dim;
    // Blocks b and b + kNormBwdBlocks share a partial row (zeroed by the launcher). A row gets at most two fp32
    // addends in the full-row mode, and a sum of two is the same in either order, so the result stays reproducible.
    float* prow = dw_partial + static_cast<long long>(blockIdx.x % kNormBwdBlocks) * wcols;
#pragma unroll
    for (int i = 0; i < PV; ++i) {
      const int pv = threadIdx.x + i * kNormThreads;
      if (pv < n_pv) {
        const int h = pv / pv_per_head, o = (pv % pv_per_head) * 8;
        const int wofs = norm_mode == 1 ? h * head_dim : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (norm_mode == 1) {
            atomicAdd(&prow[wofs + o + j], dwa[i][j]);
            atomicAdd(&prow[wofs + half + o + j], dwb[i][j]);
          } else {
            atomicAdd(&prow[o + j], dwa[i][j]);
            atomicAdd(&prow[half + o + j], dwb[i][j]);
          }
        }
      }
    }
  }
}

}  // namespace ocb

#include "rownorm_pipe.cuh"

namespace ocb {

// ----------------------------------------------------------------------------------------------------
// SwiGLU
// ----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long rows,
                                  int cols, long long lda, long long ldb, long long ldo) {
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    float fa[8], fb[8], o[8];
    Vec8<T>::load(a + r * lda + c, fa);
    Vec8<T>::load(b + r * ldb + c, fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = Vec8<T>::round(fa[j] / (1.f + __expf(-fa[j])));
      o[j] = s * fb[j];
    }
    Vec8<T>::store(out + r * ldo + c, o);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ a, const T* __restrict__ b,
                                  T* __restrict__ da, T* __restrict__ db, long long rows, int cols, long long lddo,
                                  long long lda, long long ldb, long long ldda, long long lddb) {
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    float g[8], fa[8], fb[8], oa[8], ob[8];
    Vec8<T>::load(dout + r * lddo + c, g);
    Vec8<T>::load(a + r * lda + c, fa);
    Vec8<T>::load(b + r * ldb + c, fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-fa[j]));
      const float silu = fa[j] * sig;
      oa[j] = g[j] * fb[j] * (sig * (1.f + fa[j] * (1.f - sig)));
      ob[j] = g[j] * silu;
    }
    Vec8<T>::store(da + r * ldda + c, oa);
    Vec8<T>::store(db + r * lddb + c, ob);
  }
}

// ----------------------------------------------------------------------------------------------------
// Cross entropy + z-loss. One block per row; two passes over the row (the second hits L2).
// ----------------------------------------------------------------------------------------------------
constexpr int kCeThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const T* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ ce,
                     float* __restrict__ z, T* __restrict__ dlogits, int rows, int vocab, long long ld, long long ldd,
                     long long ignore_index, float z_mult, const float* __restrict__ grad_scale) {
  __shared__ float smax[kCeThreads / 32], ssum[kCeThreads / 32];
  __shared__ float s_lse, s_m;
  const int row = blockIdx.x;
  if (row >= rows) return;
  const long long label = labels[row];
  const T* lr = logits + static_cast<long long>(row) * ld;
  T* dr = dlogits ? dlogits + static_cast<long long>(row) * ldd : nullptr;
  const int nvec = vocab / 8;
  if (label == ignore_index || label < 0 || label >= vocab) {
    if (threadIdx.x == 0) { ce[row] = 0.f; if (z) z[row] = 0.f; }
    if (dr) {
      float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int v = threadIdx.x; v < nvec; v += kCeThreads) Vec8<T>::store(dr + v * 8, zero);
      for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kCeThreads) dr[c] = static_cast<T>(0.f);
    }
    return;
  }
  // pass 1: online max / sum-exp
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    Vec8<T>::load(lr + v * 8, f);
    float vm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) vm = fmaxf(vm, f[j]);
    if (vm > m) { s *= __expf(m - vm); m = vm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kCeThreads) {
    const float f = static_cast<float>(lr[c]);
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  // combine across the block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float wm = warp_max(m);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);
  s = warp_sum(s);
  if (lane == 0) { smax[warp] = wm; ssum[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = smax[0];
    for (int i = 1; i < kCeThreads / 32; ++i) bm = fmaxf(bm, smax[i]);
    float bs = 0.f;
    for (int i = 0; i < kCeThreads / 32; ++i) bs += (smax[i] == -INFINITY) ? 0.f : ssum[i] * __expf(smax[i] - bm);
    const float lse = bm + logf(bs);
    s_lse = lse;
    s_m = bm;
    ce[row] = lse - static_cast<float>(lr[label]);
    if (z) z[row] = z_mult * lse * lse;
  }
  if (dr == nullptr) return;
  __syncthreads();
  const float lse = s_lse;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float pscale = gs * (1.f + 2.f * z_mult * lse);
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8], o[8];
    Vec8<T>::load(lr + v * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = pscale * __expf(f[j] - lse);
    const long long base = static_cast<long long>(v) * 8;
    if (label >= base && label < base + 8) o[label - base] -= gs;
    Vec8<T>::store(dr + v * 8, o);
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kCeThreads) {
    float o = pscale * __expf(static_cast<float>(lr[c]) - lse);
    if (c == label) o -= gs;
    dr[c] = static_cast<T>(o);
  }
}

// ----------------------------------------------------------------------------------------------------
// Embedding
// ----------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                     int rows, int dim, long long vocab) {
  const int vpr = dim / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    long long id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + id * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * dim);
    const int n16 = vpr * static_cast<int>(sizeof(T)) / 2;  // number of 16-byte chunks
    for (int v = threadIdx.x; v < n16; v += blockDim.x) dst[v] = src[v];
  }
}

template <typename T>
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const T* __restrict__ dout, float* __restrict__ dtable,
                                     int rows, int dim, long long vocab) {
  const int vpr = dim / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long id = ids[row];
    if (id < 0 || id >= vocab) continue;
    float* dst = dtable + id * dim;
    const T* src = dout + static_cast<long long>(row) * dim;
    for (int v = threadIdx.x; v < vpr; v += blockDim.x) {
      float f[8];
      Vec8<T>::load(src + v * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + v * 8 + j, f[j]);
    }
  }
}

// ----------------------------------------------------------------------------------------------------
// SkipStep-AdamW on a flat range, 4 elements per thread.
//   p <- p*(1 - f*lr*wd); m <- lerp(m, g, f*(1-b1)); v <- v*(1 - f*(1-b2)) + f*(1-b2)*g^2
//   p <- p - f*(lr/bc1) * m / (sqrt(v)/sqrt(bc2) + eps),  bc_i = 1 - b_i^(t+1)
// ----------------------------------------------------------------------------------------------------
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ g,
                             __nv_bfloat16* __restrict__ p_lowp, long long n, float lr, float beta1, float beta2, float eps,
                             float wd, const float* __restrict__ step, const float* __restrict__ step_factor,
                             const float* __restrict__ grad_scale) {
  const float f = step_factor ? *step_factor : 1.f;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float t = (step ? *step : 0.f) + 1.f;
  const float bc1 = 1.f - powf(beta1, t);
  const float bc2 = 1.f - powf(beta2, t);
  const float step_size = f * lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - f * lr * wd;
  const float w1 = f * (1.f - beta1), w2 = f * (1.f - beta2);
  const long long n4 = n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i], mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    float gg[4];
    if (sizeof(G) == 4) {
      const float4 t4 = reinterpret_cast<const float4*>(g)[i];
      gg[0] = t4.x; gg[1] = t4.y; gg[2] = t4.z; gg[3] = t4.w;
    } else {
      const uint2 u = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    }
    float pp[4] = {pv.x, pv.y, pv.z, pv.w}, mm[4] = {mv.x, mv.y, mv.z, mv.w}, v2[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gg[j] * gs;
      pp[j] *= decay;
      mm[j] += w1 * (gj - mm[j]);
      v2[j] = v2[j] * (1.f - w2) + w2 * gj * gj;
      pp[j] -= step_size * mm[j] / (sqrtf(v2[j]) * inv_sqrt_bc2 + eps);
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(v2[0], v2[1], v2[2], v2[3]);
    if (p_lowp) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(p_lowp)[i] = o;
    }
  }
  // tail
  const long long tail0 = n4 * 4;
  for (long long i = tail0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gj = static_cast<float>(g[i]) * gs;
    float pj = p[i] * decay;
    const float mj = m[i] + w1 * (gj - m[i]);
    const float vj = v[i] * (1.f - w2) + w2 * gj * gj;
    pj -= step_size * mj / (sqrtf(vj) * inv_sqrt_bc2 + eps);
    p[i] = pj; m[i] = mj; v[i] = vj;
    if (p_lowp) p_lowp[i] = __float2bfloat16_rn(pj);
  }
}

constexpr int kSumsqBlocks = 592;  // 4 x 148
constexpr int kSumsqThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kSumsqThreads)
sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float sbuf[kSumsqThreads / 32];
  float s = 0.f;
  const long long n8 = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    Vec8<T>::load(x + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * f[j];
  }
  for (long long i = n8 * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = static_cast<float>(x[i]);
    s += f * f;
  }
  s = group_sum(s, kSumsqThreads, sbuf);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void __launch_bounds__(kSumsqThreads)
sumsq_final_kernel(const float* __restrict__ partial, int n_partial, float* __restrict__ out, int accumulate) {
  __shared__ float sbuf[kSumsqThreads / 32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n_partial; i += kSumsqThreads) s += partial[i];
  s = group_sum(s, kSumsqThreads, sbuf);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long n8 = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8];
    Vec8<float>::load(x + i * 8, f);
    Vec8<__nv_bfloat16>::store(y + i * 8, f);
  }
  for (long long i = n8 * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16_rn(x[i]);
}

static inline int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

static inline int pick_tpg(int group, int max_vec = kMaxVec) {
  // threads per normalisation group: enough that each thread sees <= kMaxVec vectors where possible
  int nvec = group / 8;
  int tpg = 1;
  while (tpg < kNormThreads && tpg * max_vec < nvec) tpg <<= 1;
  if (tpg < 8 && nvec >= 8) tpg = 8;
  while (tpg > nvec && tpg > 1) tpg >>= 1;
  return tpg;
}

#define OCB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -4)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Dynamic shared memory above 48 KB has to be requested per kernel; the request is repeated per launch because it is
// per device and costs about a microsecond.
template <typename K>
static inline bool allow_smem(K kernel, size_t bytes) {
  // the 48 KB that need no request include the kernel's static shared memory, hence the margin
  return bytes <= 40 * 1024 ||
         cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) == cudaSuccess;
}

static inline size_t pipe_bytes(int chunks_per_row, bool with_trig, int stages = kPipeStages) {
  return sizeof(uint4) * stages * chunks_per_row * kNormThreads + (with_trig ? sizeof(float) * stages * 2 * 128 : 0);
}

// The pipelined kernels can be switched off for comparison (OCB_NORM_PIPE=0).
static inline bool norm_pipe_enabled() {
  static const bool on = [] {
    const char* e = getenv("OCB_NORM_PIPE");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

}  // namespace ocb

using namespace ocb;
typedef __nv_bfloat16 bf16;

// Dispatch on (activation dtype, weight dtype)
#define OCB_DISPATCH_TW(act, wd, ...)                                 \
  if (act == OCB_BF16 && wd == OCB_BF16) { using T = bf16; using W = bf16; __VA_ARGS__ }       \
  else if (act == OCB_BF16 && wd == OCB_F32) { using T = bf16; using W = float; __VA_ARGS__ }  \
  else if (act == OCB_F32 && wd == OCB_F32) { using T = float; using W = float; __VA_ARGS__ }  \
  else if (act == OCB_F32 && wd == OCB_BF16) { using T = float; using W = bf16; __VA_ARGS__ }  \
  else { return -1; }
#define OCB_DISPATCH_T(act, ...)                       \
  if (act == OCB_BF16) { using T = bf16; __VA_ARGS__ } \
  else if (act == OCB_F32) { using T = float; __VA_ARGS__ } \
  else { return -1; }

// The copy-ring RMSNorm backward (rows of 2048 / 4096 bf16 channels, 16-byte aligned operands). Returns 1 if the
// shape is not eligible, 0 after a launch, a negative code on failure. Every block stores one whole row of `partial`.
static int launch_rmsnorm_bwd_pipe(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                   float* partial, int rows, int cols, int group, int grid, long long lddy, long long ldx,
                                   long long lddx, int act_dtype, int w_dtype, cudaStream_t stream) {
  const bool pipe = norm_pipe_enabled() && act_dtype == OCB_BF16 && group == cols && (cols == 2048 || cols == 4096) &&
                    lddy % 8 == 0 && ldx % 8 == 0 && lddx % 8 == 0 && aligned16(dy) && aligned16(x) && aligned16(dx) &&
                    aligned16(w) && aligned16(partial) && (w_dtype == OCB_BF16 || w_dtype == OCB_F32);
  if (!pipe) return 1;
  const bf16* gp = static_cast<const bf16*>(dy);
  const bf16* xp = static_cast<const bf16*>(x);
  bf16* dxp = static_cast<bf16*>(dx);
#define OCB_RMS_BWD_PIPE(WT, NV)                                                                                   \
  {                                                                                                                \
    auto kern = rmsnorm_bwd_pipe_kernel<WT, NV>;                                                                   \
    const size_t bytes = pipe_bytes(2 * NV, false, kPipeStagesBwd);                                                \
    if (!allow_smem(kern, bytes)) return -4;                                                                       \
    kern<<<grid, kNormThreads, bytes, stream>>>(gp, xp, static_cast<const WT*>(w), rstd, dxp, partial, rows, lddy, ldx, lddx); \
  }
  if (w_dtype == OCB_BF16) { if (cols == 2048) OCB_RMS_BWD_PIPE(bf16, 1) else OCB_RMS_BWD_PIPE(bf16, 2) }
  else { if (cols == 2048) OCB_RMS_BWD_PIPE(float, 1) else OCB_RMS_BWD_PIPE(float, 2) }
#undef OCB_RMS_BWD_PIPE
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_rmsnorm_fwd(const void* x, const void* w, const void* resid, void* y, float* rstd, int rows, int cols,
                               int group, long long ldx, long long ldy, long long ldr, float eps, int act_dtype,
                               int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (group <= 0 || cols % group != 0 || group % 8 != 0 || ldx % 8 != 0 || ldy % 8 != 0) return -1;
  if (norm_pipe_enabled() && act_dtype == OCB_BF16 && group == cols && (cols == 2048 || cols == 4096) && ldx % 8 == 0 &&
      ldy % 8 == 0 && (resid == nullptr || ldr % 8 == 0) && aligned16(x) && aligned16(y) && aligned16(resid) &&
      aligned16(w) && (w_dtype == OCB_BF16 || w_dtype == OCB_F32)) {
    const int grid = rows < 148 * 3 ? rows : 148 * 3;
    const bf16* xp = static_cast<const bf16*>(x);
    const bf16* rp = static_cast<const bf16*>(resid);
    bf16* yp = static_cast<bf16*>(y);
#define OCB_RMS_FWD_PIPE(WT, NV, RES)                                                                              \
    {                                                                                                              \
      auto kern = rmsnorm_fwd_pipe_kernel<WT, NV, RES>;                                                            \
      const size_t bytes = pipe_bytes((RES ? 2 : 1) * NV, false);                                                  \
      if (!allow_smem(kern, bytes)) return -4;                                                                     \
      kern<<<grid, kNormThreads, bytes, stream>>>(xp, static_cast<const WT*>(w), rp, yp, rstd, rows, ldx, ldy, ldr, eps); \
    }
    const int nv = cols / 2048;
    if (w_dtype == OCB_BF16) {
      if (nv == 1) { if (resid) OCB_RMS_FWD_PIPE(bf16, 1, true) else OCB_RMS_FWD_PIPE(bf16, 1, false) }
      else { if (resid) OCB_RMS_FWD_PIPE(bf16, 2, true) else OCB_RMS_FWD_PIPE(bf16, 2, false) }
    } else {
      if (nv == 1) { if (resid) OCB_RMS_FWD_PIPE(float, 1, true) else OCB_RMS_FWD_PIPE(float, 1, false) }
      else { if (resid) OCB_RMS_FWD_PIPE(float, 2, true) else OCB_RMS_FWD_PIPE(float, 2, false) }
    }
#undef OCB_RMS_FWD_PIPE
    return OCB_CHECK_LAUNCH();
  }
  const int gpr = cols / group;
  const long long n_groups = static_cast<long long>(rows) * gpr;
  const int tpg = pick_tpg(group);
  const int gpb = kNormThreads / tpg;
  const int grid = ew_grid((n_groups + gpb - 1) / gpb, 1);
  OCB_DISPATCH_TW(act_dtype, w_dtype, {
    rmsnorm_fwd_kernel<T, W><<<grid, kNormThreads, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const W*>(w), static_cast<const T*>(resid), static_cast<T*>(y), rstd,
        n_groups, gpr, group, tpg, ldx, ldy, ldr, eps);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_norm_bwd_partials() { return kNormBwdBlocks; }

extern "C" int ocb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* dw_partial, int rows, int cols, int group, long long lddy, long long ldx,
                               long long lddx, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (group <= 0 || cols % group != 0 || group % 8 != 0) return -1;
  const int gpr = cols / group;
  const long long n_groups = static_cast<long long>(rows) * gpr;
  const int maxv = group <= 2 * kNormThreads * 8 ? 2 : kMaxVec;
  const int tpg = pick_tpg(group, maxv);
  if ((group / 8 + tpg - 1) / tpg > maxv) return -1;  // group too wide for the register-resident row
  const int gpb = kNormThreads / tpg;
  long long want = (n_groups + gpb - 1) / gpb;
  const int grid = static_cast<int>(want < kNormBwdBlocks ? want : kNormBwdBlocks);
  // The copy-ring kernel stores one whole partial row per block: only rows without a block have to be cleared first.
  if (dw_partial != nullptr && grid < kNormBwdBlocks) {
    if (cudaMemsetAsync(dw_partial, 0, sizeof(float) * static_cast<size_t>(kNormBwdBlocks) * group, stream) != cudaSuccess)
      return -4;
  }
  {
    const int rc = launch_rmsnorm_bwd_pipe(dy, x, w, rstd, dx, dw_partial, rows, cols, group, grid, lddy, ldx, lddx,
                                           act_dtype, w_dtype, stream);
    if (rc <= 0) return rc;
  }
  if (dw_partial != nullptr && grid == kNormBwdBlocks) {  // the register kernel adds into its rows
    if (cudaMemsetAsync(dw_partial, 0, sizeof(float) * static_cast<size_t>(kNormBwdBlocks) * group, stream) != cudaSuccess)
      return -4;
  }
  OCB_DISPATCH_TW(act_dtype, w_dtype, {
    if (maxv == 2)
      rmsnorm_bwd_kernel<T, W, 2><<<grid, kNormThreads, 0, stream>>>(
          static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const W*>(w), rstd, static_cast<T*>(dx),
          dw_partial, n_groups, gpr, group, tpg, lddy, ldx, lddx);
    else
      rmsnorm_bwd_kernel<T, W, kMaxVec><<<grid, kNormThreads, 0, stream>>>(
          static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const W*>(w), rstd, static_cast<T*>(dx),
          dw_partial, n_groups, gpr, group, tpg, lddy, ldx, lddx);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_reduce_partials(const float* partial, void* out, int n_partial, int cols, int accumulate,
                                   int out_dtype, cudaStream_t stream) {
  if (cols <= 0) return 0;
  const dim3 threads(32, 32);
  const int grid = (cols + 31) / 32;
  if (out_dtype == OCB_F32)
    reduce_partials_kernel<float><<<grid, threads, 0, stream>>>(partial, static_cast<float*>(out), n_partial, cols, accumulate);
  else
    reduce_partials_kernel<bf16><<<grid, threads, 0, stream>>>(partial, static_cast<bf16*>(out), n_partial, cols, accumulate);
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_norm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* sin_t,
                                 const float* cos_t, const int* pos_ids, int rows, int n_heads, int head_dim,
                                 int seq_len, int pos_offset, int norm_mode, long long ldx, long long ldy, float eps,
                                 int act_dtype, int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int half = head_dim / 2;
  if (head_dim % 16 != 0 || (half / 8) > 32 || ((half / 8) & (half / 8 - 1)) != 0) return -1;
  if (n_heads * (half / 8) > kMaxPv * kNormThreads) return -1;
  if (norm_pipe_enabled() && act_dtype == OCB_BF16 && head_dim == 128 && n_heads * 8 <= kNormThreads && ldx % 8 == 0 &&
      ldy % 8 == 0 && aligned16(x) && aligned16(y) && aligned16(w) && aligned16(sin_t) && aligned16(cos_t) &&
      (w_dtype == OCB_BF16 || w_dtype == OCB_F32)) {
    const int pgrid = rows < 148 * 3 ? rows : 148 * 3;
    const size_t bytes = pipe_bytes(2, true);
    if (w_dtype == OCB_BF16) {
      auto kern = norm_rope_pipe_kernel<bf16, false>;
      if (!allow_smem(kern, bytes)) return -4;
      kern<<<pgrid, kNormThreads, bytes, stream>>>(static_cast<const bf16*>(x), nullptr, static_cast<const bf16*>(w), rstd,
                                                   static_cast<bf16*>(y), nullptr, sin_t, cos_t, pos_ids, rows, n_heads,
                                                   seq_len, pos_offset, norm_mode, ldx, 0, ldy, eps);
    } else {
      auto kern = norm_rope_pipe_kernel<float, false>;
      if (!allow_smem(kern, bytes)) return -4;
      kern<<<pgrid, kNormThreads, bytes, stream>>>(static_cast<const bf16*>(x), nullptr, static_cast<const float*>(w), rstd,
                                                   static_cast<bf16*>(y), nullptr, sin_t, cos_t, pos_ids, rows, n_heads,
                                                   seq_len, pos_offset, norm_mode, ldx, 0, ldy, eps);
    }
    return OCB_CHECK_LAUNCH();
  }
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  const bool one_pv = n_heads * (half / 8) <= kNormThreads;
  OCB_DISPATCH_TW(act_dtype, w_dtype, {
    auto kern = one_pv ? norm_rope_kernel<T, W, false, 1> : norm_rope_kernel<T, W, false, 2>;
    kern<<<grid, kNormThreads, 0, stream>>>(
        static_cast<const T*>(x), nullptr, static_cast<const W*>(w), rstd, static_cast<T*>(y), nullptr, sin_t, cos_t,
        pos_ids, rows, n_heads, head_dim, seq_len, pos_offset, norm_mode, ldx, 0, ldy, eps);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_norm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                 float* dw_partial, const float* sin_t, const float* cos_t, const int* pos_ids, int rows,
                                 int n_heads, int head_dim, int seq_len, int pos_offset, int norm_mode, long long lddy,
                                 long long ldx, long long lddx, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int half = head_dim / 2;
  if (head_dim % 16 != 0 || (half / 8) > 32 || ((half / 8) & (half / 8 - 1)) != 0) return -1;
  if (n_heads * (half / 8) > kMaxPv * kNormThreads) return -1;
  const bool one_pv = n_heads * (half / 8) <= kNormThreads;
  // every block must be resident at once (a persistent grid that spills into a second wave doubles the run time):
  // three blocks per SM fit with one pair vector per thread, two otherwise
  const int max_blocks = one_pv ? kNormBwdBlocks + kNormBwdBlocks / 2 : kNormBwdBlocks;
  const int grid = rows < max_blocks ? rows : max_blocks;
  const bool pipe = norm_pipe_enabled() && act_dtype == OCB_BF16 && head_dim == 128 && n_heads * 8 <= kNormThreads &&
                    lddy % 8 == 0 && lddx % 8 == 0 && (norm_mode == 0 || ldx % 8 == 0) && aligned16(dy) && aligned16(dx) &&
                    aligned16(x) && aligned16(w) && aligned16(sin_t) && aligned16(cos_t) && aligned16(dw_partial) &&
                    (w_dtype == OCB_BF16 || w_dtype == OCB_F32);
  // In the full-row mode the pipelined kernel stores one whole partial row per block: only rows
  // without a block have to be cleared. The per-head mode adds into its rows.
  const bool all_rows_written = pipe && norm_mode == 1 && rows >= kNormBwdBlocks;
  if (dw_partial != nullptr && norm_mode != 0 && !all_rows_written) {
    const int wcols = norm_mode == 1 ? n_heads * head_dim : head_dim;
    if (cudaMemsetAsync(dw_partial, 0, sizeof(float) * static_cast<size_t>(kNormBwdBlocks) * wcols, stream) != cudaSuccess)
      return -4;
  }
  if (pipe) {
    const int pgrid = rows < kNormBwdBlocks ? rows : kNormBwdBlocks;
    const size_t bytes = pipe_bytes(4, true, kPipeStagesBwd);
    if (w_dtype == OCB_BF16) {
      auto kern = norm_rope_pipe_kernel<bf16, true>;
      if (!allow_smem(kern, bytes)) return -4;
      kern<<<pgrid, kNormThreads, bytes, stream>>>(static_cast<const bf16*>(dy), static_cast<const bf16*>(x),
                                                   static_cast<const bf16*>(w), const_cast<float*>(rstd),
                                                   static_cast<bf16*>(dx), dw_partial, sin_t, cos_t, pos_ids, rows, n_heads,
                                                   seq_len, pos_offset, norm_mode, lddy, ldx, lddx, 0.f);
    } else {
      auto kern = norm_rope_pipe_kernel<float, true>;
      if (!allow_smem(kern, bytes)) return -4;
      kern<<<pgrid, kNormThreads, bytes, stream>>>(static_cast<const bf16*>(dy), static_cast<const bf16*>(x),
                                                   static_cast<const float*>(w), const_cast<float*>(rstd),
                                                   static_cast<bf16*>(dx), dw_partial, sin_t, cos_t, pos_ids, rows, n_heads,
                                                   seq_len, pos_offset, norm_mode, lddy, ldx, lddx, 0.f);
    }
    return OCB_CHECK_LAUNCH();
  }
  OCB_DISPATCH_TW(act_dtype, w_dtype, {
    auto kern = one_pv ? norm_rope_kernel<T, W, true, 1> : norm_rope_kernel<T, W, true, 2>;
    kern<<<grid, kNormThreads, 0, stream>>>(
        static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const W*>(w), const_cast<float*>(rstd),
        static_cast<T*>(dx), dw_partial, sin_t, cos_t, pos_ids, rows, n_heads, head_dim, seq_len, pos_offset, norm_mode,
        lddy, ldx, lddx, 0.f);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_swiglu_fwd(const void* a, const void* b, void* out, long long rows, int cols, long long lda,
                              long long ldb, long long ldo, int act_dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldo % 8 != 0) return -1;
  const int grid = ew_grid(rows * (cols / 8), 256);
  OCB_DISPATCH_T(act_dtype, {
    swiglu_fwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out),
                                                   rows, cols, lda, ldb, ldo);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_swiglu_bwd(const void* dout, const void* a, const void* b, void* da, void* db, long long rows, int cols,
                              long long lddo, long long lda, long long ldb, long long ldda, long long lddb, int act_dtype,
                              cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || lddo % 8 != 0 || ldda % 8 != 0 || lddb % 8 != 0) return -1;
  const int grid = ew_grid(rows * (cols / 8), 256);
  OCB_DISPATCH_T(act_dtype, {
    swiglu_bwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(dout), static_cast<const T*>(a),
                                                   static_cast<const T*>(b), static_cast<T*>(da), static_cast<T*>(db), rows,
                                                   cols, lddo, lda, ldb, ldda, lddb);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_cross_entropy_fwd_bwd(const void* logits, const long long* labels, float* ce, float* z, void* dlogits,
                                         int rows, int vocab, long long ld, long long ldd, long long ignore_index,
                                         float z_mult, const float* grad_scale, int act_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (ld % 8 != 0 || (dlogits && ldd % 8 != 0)) return -1;
  OCB_DISPATCH_T(act_dtype, {
    cross_entropy_kernel<T><<<rows, kCeThreads, 0, stream>>>(static_cast<const T*>(logits), labels, ce, z,
                                                             static_cast<T*>(dlogits), rows, vocab, ld, ldd, ignore_index,
                                                             z_mult, grad_scale);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_embedding_fwd(const long long* ids, const void* table, void* out, int rows, int dim, long long vocab,
                                 int act_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim % 8 != 0) return -1;
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  OCB_DISPATCH_T(act_dtype, {
    embedding_fwd_kernel<T><<<grid, 128, 0, stream>>>(ids, static_cast<const T*>(table), static_cast<T*>(out), rows, dim, vocab);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_embedding_bwd(const long long* ids, const void* dout, float* dtable, int rows, int dim, long long vocab,
                                 int act_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim % 8 != 0) return -1;
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  OCB_DISPATCH_T(act_dtype, {
    embedding_bwd_kernel<T><<<grid, 128, 0, stream>>>(ids, static_cast<const T*>(dout), dtable, rows, dim, vocab);
  })
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_adamw_step(float* p, float* m, float* v, const void* g, void* p_lowp, long long n, float lr, float beta1,
                              float beta2, float eps, float weight_decay, const float* step, const float* step_factor,
                              const float* grad_scale, int grad_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = ew_grid((n + 3) / 4, 256);
  if (grad_dtype == OCB_F32)
    adamw_kernel<float><<<grid, 256, 0, stream>>>(p, m, v, static_cast<const float*>(g), static_cast<bf16*>(p_lowp), n, lr,
                                                  beta1, beta2, eps, weight_decay, step, step_factor, grad_scale);
  else
    adamw_kernel<bf16><<<grid, 256, 0, stream>>>(p, m, v, static_cast<const bf16*>(g), static_cast<bf16*>(p_lowp), n, lr,
                                                 beta1, beta2, eps, weight_decay, step, step_factor, grad_scale);
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_sumsq_partials() { return kSumsqBlocks; }

extern "C" int ocb_sumsq(const void* x, long long n, float* scratch, float* out, int accumulate, int dtype,
                         cudaStream_t stream) {
  if (n <= 0) {
    if (!accumulate) cudaMemsetAsync(out, 0, sizeof(float), stream);
    return 0;
  }
  long long want = (n / 8 + kSumsqThreads - 1) / kSumsqThreads;
  const int grid = static_cast<int>(want < 1 ? 1 : (want < kSumsqBlocks ? want : kSumsqBlocks));
  if (dtype == OCB_F32)
    sumsq_partial_kernel<float><<<grid, kSumsqThreads, 0, stream>>>(static_cast<const float*>(x), n, scratch);
  else
    sumsq_partial_kernel<bf16><<<grid, kSumsqThreads, 0, stream>>>(static_cast<const bf16*>(x), n, scratch);
  sumsq_final_kernel<<<1, kSumsqThreads, 0, stream>>>(scratch, grid, out, accumulate);
  return OCB_CHECK_LAUNCH();
}

extern "C" int ocb_cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = ew_grid((n + 7) / 8, 256);
  cast_f32_bf16_kernel<<<grid, 256, 0, stream>>>(x, static_cast<bf16*>(y), n);
  return OCB_CHECK_LAUNCH();
}

// ---- RMSNorm backward without any allocation (declared and documented in ocb_static_scratch.h) ------
#include <mutex>

#include "ocb_static_scratch.h"

// Weight-gradient partials of one call: one row per block of the persistent backward grid. Shared by all
// calls on the device, which is why the launcher clears the rows it is about to use on the caller's stream.
static __device__ __align__(256) float g_static_norm_partials[ocb::kNormBwdBlocks * OCB_STATIC_SCRATCH_MAX_GROUP];

namespace {
constexpr int kStaticMaxDevices = 64;
float* g_static_partials_ptr[kStaticMaxDevices] = {};
std::mutex g_static_partials_mutex;

// Device address of the scratch array on the current device; resolved once per device.
int static_partials(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return OCB_ERR_STATIC_SCRATCH_SETUP;
  std::lock_guard<std::mutex> lock(g_static_partials_mutex);
  if (g_static_partials_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_norm_partials) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();  // leave no sticky error behind for the caller's next launch check
      return OCB_ERR_STATIC_SCRATCH_SETUP;
    }
    g_static_partials_ptr[dev] = p;
  }
  *out = g_static_partials_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int ocb_rmsnorm_bwd_static_max_group() { return OCB_STATIC_SCRATCH_MAX_GROUP; }

extern "C" const char* ocb_rmsnorm_bwd_static_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case -1: return "invalid argument: group must divide cols, be a multiple of 8 and at most 8192";
    case -4: return "CUDA launch or memset failed";
    case OCB_ERR_STATIC_SCRATCH_TOO_SMALL:
      return "group exceeds OCB_STATIC_SCRATCH_MAX_GROUP (4096): the built-in scratch array is too small; "
             "use ocb_rmsnorm_bwd with a caller-provided partials buffer";
    case OCB_ERR_STATIC_SCRATCH_SETUP:
      return "could not resolve the device address of the built-in scratch array on the current device";
    default: return "unknown error code";
  }
}

extern "C" int ocb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                      void* dw, int dw_accumulate, int rows, int cols, int group, long long lddy,
                                      long long ldx, long long lddx, int act_dtype, int w_dtype, int dw_dtype,
                                      cudaStream_t stream) {
  using namespace ocb;
  if (group <= 0 || cols % group != 0 || group % 8 != 0) return -1;
  if (dw != nullptr && group > OCB_STATIC_SCRATCH_MAX_GROUP) return OCB_ERR_STATIC_SCRATCH_TOO_SMALL;
  if (rows <= 0) {
    // an empty batch contributes nothing: "overwrite" still has to leave zeros behind, "accumulate" leaves dw as it is
    if (dw != nullptr && !dw_accumulate &&
        cudaMemsetAsync(dw, 0, static_cast<size_t>(group) * (dw_dtype == OCB_F32 ? 4 : 2), stream) != cudaSuccess)
      return -4;
    return 0;
  }
  const int gpr = cols / group;
  const long long n_groups = static_cast<long long>(rows) * gpr;
  const int maxv = group <= 2 * kNormThreads * 8 ? 2 : kMaxVec;
  const int tpg = pick_tpg(group, maxv);
  if ((group / 8 + tpg - 1) / tpg > maxv) return -1;
  const int gpb = kNormThreads / tpg;
  const long long want = (n_groups + gpb - 1) / gpb;
  const int grid = static_cast<int>(want < kNormBwdBlocks ? want : kNormBwdBlocks);
  float* partial = nullptr;
  if (dw != nullptr) {
    const int rc = static_partials(&partial);
    if (rc != 0) return rc;
  }
  // Same kernel selection as ocb_rmsnorm_bwd, so that both entry points give bit-identical dx. The copy-ring kernel
  // overwrites the `grid` partial rows that are folded below; the register kernel adds into them.
  int launched = launch_rmsnorm_bwd_pipe(dy, x, w, rstd, dx, partial, rows, cols, group, grid, lddy, ldx, lddx, act_dtype,
                                         w_dtype, stream);
  if (launched < 0) return launched;
  if (launched == 1 && dw != nullptr) {
    // Only the `grid` rows this call accumulates into (and later folds) have to start at zero.
    if (cudaMemsetAsync(partial, 0, sizeof(float) * static_cast<size_t>(grid) * group, stream) != cudaSuccess) return -4;
  }
  if (launched == 1) {
    OCB_DISPATCH_TW(act_dtype, w_dtype, {
      if (maxv == 2)
        rmsnorm_bwd_kernel<T, W, 2><<<grid, kNormThreads, 0, stream>>>(
            static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const W*>(w), rstd, static_cast<T*>(dx),
            partial, n_groups, gpr, group, tpg, lddy, ldx, lddx);
      else
        rmsnorm_bwd_kernel<T, W, kMaxVec><<<grid, kNormThreads, 0, stream>>>(
            static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const W*>(w), rstd, static_cast<T*>(dx),
            partial, n_groups, gpr, group, tpg, lddy, ldx, lddx);
    })
  }
  if (cudaGetLastError() != cudaSuccess) return -4;
  if (dw != nullptr) {
    const dim3 threads(32, 32);
    const int rgrid = (group + 31) / 32;
    if (dw_dtype == OCB_F32)
      reduce_partials_kernel<float><<<rgrid, threads, 0, stream>>>(partial, static_cast<float*>(dw), grid, group, dw_accumulate);
    else
      reduce_partials_kernel<bf16><<<rgrid, threads, 0, stream>>>(partial, static_cast<bf16*>(dw), grid, group, dw_accumulate);
  }
  return OCB_CHECK_LAUNCH();
}
