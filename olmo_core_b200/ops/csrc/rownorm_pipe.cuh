// Row-wise normalisation kernels with a shared-memory copy pipeline (included by elementwise.cu).
//
// One block owns one token row at a time. The kernels it replaces loaded a row, reduced it across the block and
// only then could ask for the next row, so a block had one row in flight and the step was a chain of memory
// latencies (0.30-0.36 of the copy bandwidth). Here every thread copies the 16-byte pieces IT will consume with
// cp.async into a ring of kPipeStages rows, three rows ahead of the arithmetic; a thread waits only for its own
// copies (cp.async.wait_group, a hardware wait, not a spin on another thread), so the only block-wide barrier left
// is the one of the reduction. That barrier also publishes the row's sin/cos values, which 64 threads copy for the
// whole block (every head uses the same 2 x 128 values), and releases the ring slot of the previous row.
//
// bf16 activations only; anything else takes the register kernels in elementwise.cu.

#pragma once

namespace ocb {

constexpr int kPipeStages = 4;     // forward kernels: three blocks per SM
constexpr int kPipeStagesBwd = 4;  // backward kernels: two blocks per SM (six stages measured no faster)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void lds8(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Sum over the block's 8 warps through one of two alternating scratch rows: one barrier per call. A scratch row is
// rewritten two calls later, by which time every thread has passed the barrier of the call in between.
__device__ __forceinline__ float block_sum_alt(float v, float (*sbuf)[kNormThreads / 32], int it) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sbuf[it & 1][threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) s += sbuf[it & 1][i];
  return s;
}

// ----------------------------------------------------------------------------------------------------------------
// (optional RMSNorm) + rotate-half RoPE, head_dim 128, up to 32 heads per row. Thread t owns 8 channels of head t/8
// at offset (t%8)*8 and their partners 64 channels further on. Same arithmetic, in the same order, as
// norm_rope_kernel.
// ----------------------------------------------------------------------------------------------------------------
template <typename W, bool BWD>
__global__ void __launch_bounds__(kNormThreads, BWD ? 2 : 3)
norm_rope_pipe_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ x_saved,
                      const W* __restrict__ w, float* __restrict__ rstd_io, __nv_bfloat16* __restrict__ out,
                      float* __restrict__ dw_partial, const float* __restrict__ sin_t, const float* __restrict__ cos_t,
                      const int* __restrict__ pos_ids, int rows, int n_heads, int seq_len, int pos_offset,
                      int norm_mode, long long ld_in, long long ld_x, long long ld_out, float eps) {
  constexpr int HD = 128, HALF = 64, S = BWD ? kPipeStagesBwd : kPipeStages, NCH = BWD ? 4 : 2;
  extern __shared__ __align__(16) unsigned char pipe_smem[];
  uint4* data = reinterpret_cast<uint4*>(pipe_smem);                                        // [S][NCH][256]
  float* trig = reinterpret_cast<float*>(pipe_smem + sizeof(uint4) * S * NCH * kNormThreads);  // [S][cos, sin][HD]
  __shared__ float sbuf[2][kNormThreads / 32];

  const int t = threadIdx.x;
  const bool on = t < n_heads * 8;
  const int h = t >> 3, o = (t & 7) * 8;
  const int cols = n_heads * HD;
  const bool need_x = BWD && norm_mode != 0;

  float wa[8], wb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) wa[j] = wb[j] = 1.f;
  if (norm_mode != 0 && on) {
    const int wofs = norm_mode == 1 ? h * HD : 0;
    Vec8<W>::load(w + wofs + o, wa);
    Vec8<W>::load(w + wofs + HALF + o, wb);
  }
  float dwa[8], dwb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) dwa[j] = dwb[j] = 0.f;

  auto issue = [&](long long row, int st) {
    if (row < rows) {
      if (on) {
        const __nv_bfloat16* src = in + row * ld_in + h * HD + o;
        cp_async16(&data[(st * NCH + 0) * kNormThreads + t], src);
        cp_async16(&data[(st * NCH + 1) * kNormThreads + t], src + HALF);
        if (need_x) {
          const __nv_bfloat16* xs = x_saved + row * ld_x + h * HD + o;
          cp_async16(&data[(st * NCH + 2) * kNormThreads + t], xs);
          cp_async16(&data[(st * NCH + 3) * kNormThreads + t], xs + HALF);
        }
      }
      if (t < 64) {  // warp 0: the cos row, warp 1: the sin row, 16 bytes per lane
        // 32-bit arithmetic: `rows` is an int, and a 64-bit remainder costs these two warps over a hundred instructions
        const int pos = pos_ids ? pos_ids[row] : static_cast<int>(row) % seq_len + pos_offset;
        const float* tab = (t < 32 ? cos_t : sin_t) + static_cast<long long>(pos) * HD + (t & 31) * 4;
        cp_async16(&trig[(st * 2 + (t >> 5)) * HD + (t & 31) * 4], tab);
      }
    }
    cp_async_commit();  // one group per call, empty or not, so that the group count below stays fixed
  };

  const long long stride = gridDim.x;
  for (int s = 0; s < S - 1; ++s) issue(blockIdx.x + s * stride, s);

  // backward: the saved statistic of a row is requested one iteration before it is needed
  auto saved_rstd = [&](long long row) -> float {
    if (!BWD || row >= rows) return 1.f;
    if (norm_mode == 1) return rstd_io[row];
    if (norm_mode == 2 && on) return rstd_io[row * n_heads + h];
    return 1.f;
  };
  float rs_bwd = saved_rstd(blockIdx.x);

  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += stride, ++it) {
    const int st = it % S;
    const float rs_next = saved_rstd(row + stride);
    cp_async_wait<S - 2>();  // all but the newest S-2 groups are complete: this thread's pieces of `row` have landed
    float a[8], b[8], xa[8], xb[8];
    if (on) {
      unpack8(data[(st * NCH + 0) * kNormThreads + t], a);
      unpack8(data[(st * NCH + 1) * kNormThreads + t], b);
      if (need_x) {
        unpack8(data[(st * NCH + 2) * kNormThreads + t], xa);
        unpack8(data[(st * NCH + 3) * kNormThreads + t], xb);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
    }
    if (!need_x) {
#pragma unroll
      for (int j = 0; j < 8; ++j) xa[j] = xb[j] = 0.f;
    }
    const float* cs = trig + (st * 2 + 0) * HD;
    const float* sn = trig + (st * 2 + 1) * HD;

    if (!BWD) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
      float rs = 1.f;
      if (norm_mode == 2) {
        float hs = ss;
        for (int s2 = 4; s2 > 0; s2 >>= 1) hs += __shfl_xor_sync(0xffffffffu, hs, s2);
        rs = rsqrtf(hs / static_cast<float>(HD) + eps);
        if (on && (t & 7) == 0 && rstd_io) rstd_io[row * n_heads + h] = rs;
      }
      const float total = block_sum_alt(ss, sbuf, it);  // the barrier: sin/cos of `row` visible, previous slot free
      issue(row + (S - 1) * stride, (it + S - 1) % S);
      if (norm_mode == 1) {
        rs = rsqrtf(total / static_cast<float>(cols) + eps);
        if (t == 0 && rstd_io) rstd_io[row] = rs;
      }
      if (on) {
        float c_lo[8], s_lo[8], c_hi[8], s_hi[8], oa[8], ob[8];
        lds8(cs + o, c_lo);
        lds8(sn + o, s_lo);
        lds8(cs + HALF + o, c_hi);
        lds8(sn + HALF + o, s_hi);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ya = norm_mode != 0 ? round_bf16(a[j] * rs * wa[j]) : a[j];
          const float yb = norm_mode != 0 ? round_bf16(b[j] * rs * wb[j]) : b[j];
          oa[j] = ya * c_lo[j] - yb * s_lo[j];
          ob[j] = yb * c_hi[j] + ya * s_hi[j];
        }
        __nv_bfloat16* dst = out + row * ld_out + h * HD + o;
        *reinterpret_cast<uint4*>(dst) = pack8(oa);
        *reinterpret_cast<uint4*>(dst + HALF) = pack8(ob);
      }
    } else {
      // The rotation's transpose needs sin/cos, which other threads copied: the barrier comes first here.
      const float rs = rs_bwd;
      __syncthreads();
      issue(row + (S - 1) * stride, (it + S - 1) % S);
      float ga[8], gb[8];
      {
        float c_lo[8], s_lo[8], c_hi[8], s_hi[8];
        lds8(cs + o, c_lo);
        lds8(sn + o, s_lo);
        lds8(cs + HALF + o, c_hi);
        lds8(sn + HALF + o, s_hi);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ga[j] = a[j] * c_lo[j] + b[j] * s_hi[j];
          gb[j] = b[j] * c_hi[j] - a[j] * s_lo[j];
        }
      }
      float c = 0.f;
      if (norm_mode != 0) {
        float dot = 0.f;
        if (on) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dot += (ga[j] * wa[j] * xa[j] + gb[j] * wb[j] * xb[j]) * rs;
        }
        if (norm_mode == 2) {
          for (int s2 = 4; s2 > 0; s2 >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s2);
          c = dot / static_cast<float>(HD);
        } else {
          // second barrier of the row; its scratch row alternates like the forward kernel's
          c = block_sum_alt(dot, sbuf, it) / static_cast<float>(cols);
        }
      }
      if (on) {
        float oa[8], ob[8];
        if (norm_mode != 0) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xha = xa[j] * rs, xhb = xb[j] * rs;
            oa[j] = rs * (ga[j] * wa[j] - xha * c);
            ob[j] = rs * (gb[j] * wb[j] - xhb * c);
            dwa[j] += ga[j] * xha;
            dwb[j] += gb[j] * xhb;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { oa[j] = ga[j]; ob[j] = gb[j]; }
        }
        __nv_bfloat16* dst = out + row * ld_out + h * HD + o;
        *reinterpret_cast<uint4*>(dst) = pack8(oa);
        *reinterpret_cast<uint4*>(dst + HALF) = pack8(ob);
      }
    }
    rs_bwd = rs_next;
  }
  cp_async_wait<0>();  // nothing may still be writing into shared memory when the block retires

  if (BWD && dw_partial != nullptr && norm_mode != 0 && on) {
    // One partial row per block (the grid never exceeds kNormBwdBlocks). Full-row mode: every thread owns its
    // columns, plain stores. Per-head mode: the 32 heads of a block meet in the same head_dim columns.
    const int wcols = norm_mode == 1 ? cols : HD;
    float* prow = dw_partial + static_cast<long long>(blockIdx.x) * wcols;
    if (norm_mode == 1) {
      Vec8<float>::store(prow + h * HD + o, dwa);
      Vec8<float>::store(prow + h * HD + HALF + o, dwb);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&prow[o + j], dwa[j]);
        atomicAdd(&prow[HALF + o + j], dwb[j]);
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------------------------
// RMSNorm over whole rows of NV * 2048 bf16 channels (NV = 1, 2): thread t owns the 8-channel vectors t, t + 256, ...
// Forward: y = x * rstd * w (+ residual after rounding, as the register kernel does). Backward: dx and one row of
// weight-gradient partials per block.
// ----------------------------------------------------------------------------------------------------------------
template <typename W, int NV, bool RESID>
__global__ void __launch_bounds__(kNormThreads, 3)
rmsnorm_fwd_pipe_kernel(const __nv_bfloat16* __restrict__ x, const W* __restrict__ w,
                        const __nv_bfloat16* __restrict__ resid, __nv_bfloat16* __restrict__ y,
                        float* __restrict__ rstd_out, int rows, long long ldx, long long ldy, long long ldr, float eps) {
  constexpr int S = kPipeStages, NCH = (RESID ? 2 : 1) * NV, COLS = NV * kNormThreads * 8;
  extern __shared__ __align__(16) unsigned char pipe_smem[];
  uint4* data = reinterpret_cast<uint4*>(pipe_smem);  // [S][NCH][256]
  __shared__ float sbuf[2][kNormThreads / 32];
  const int t = threadIdx.x;

  float wf[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) wf[i][j] = 1.f;
    if (w != nullptr) Vec8<W>::load(w + (t + i * kNormThreads) * 8, wf[i]);
  }

  auto issue = [&](long long row, int st) {
    if (row < rows) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        cp_async16(&data[(st * NCH + i) * kNormThreads + t], x + row * ldx + (t + i * kNormThreads) * 8);
        if (RESID) cp_async16(&data[(st * NCH + NV + i) * kNormThreads + t], resid + row * ldr + (t + i * kNormThreads) * 8);
      }
    }
    cp_async_commit();
  };
  const long long stride = gridDim.x;
  for (int s = 0; s < S - 1; ++s) issue(blockIdx.x + s * stride, s);

  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += stride, ++it) {
    const int st = it % S;
    cp_async_wait<S - 2>();
    float f[NV][8], rf[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      unpack8(data[(st * NCH + i) * kNormThreads + t], f[i]);
      if (RESID) unpack8(data[(st * NCH + NV + i) * kNormThreads + t], rf[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[i][j] * f[i][j];
    }
    // A thread reads only what it copied itself, so the slot of the previous row is free once every thread has
    // reached this barrier.
    const float total = block_sum_alt(ss, sbuf, it);
    issue(row + (S - 1) * stride, (it + S - 1) % S);
    const float rstd = rsqrtf(total / static_cast<float>(COLS) + eps);
    if (t == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = f[i][j] * rstd * wf[i][j];
        if (RESID) o[j] = rf[i][j] + round_bf16(o[j]);
      }
      *reinterpret_cast<uint4*>(y + row * ldy + (t + i * kNormThreads) * 8) = pack8(o);
    }
  }
  cp_async_wait<0>();
}

template <typename W, int NV>
__global__ void __launch_bounds__(kNormThreads, 2)
rmsnorm_bwd_pipe_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const W* __restrict__ w, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw_partial, int rows, long long lddy, long long ldx, long long lddx) {
  constexpr int S = kPipeStagesBwd, NCH = 2 * NV, COLS = NV * kNormThreads * 8;
  extern __shared__ __align__(16) unsigned char pipe_smem[];
  uint4* data = reinterpret_cast<uint4*>(pipe_smem);  // [S][NCH][256]
  __shared__ float sbuf[2][kNormThreads / 32];
  const int t = threadIdx.x;

  float wf[NV][8], dw[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { wf[i][j] = 1.f; dw[i][j] = 0.f; }
    if (w != nullptr) Vec8<W>::load(w + (t + i * kNormThreads) * 8, wf[i]);
  }

  auto issue = [&](long long row, int st) {
    if (row < rows) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        cp_async16(&data[(st * NCH + i) * kNormThreads + t], x + row * ldx + (t + i * kNormThreads) * 8);
        cp_async16(&data[(st * NCH + NV + i) * kNormThreads + t], dy + row * lddy + (t + i * kNormThreads) * 8);
      }
    }
    cp_async_commit();
  };
  const long long stride = gridDim.x;
  for (int s = 0; s < S - 1; ++s) issue(blockIdx.x + s * stride, s);

  int it = 0;
  float rstd = blockIdx.x < rows ? rstd_in[blockIdx.x] : 0.f;
  for (long long row = blockIdx.x; row < rows; row += stride, ++it) {
    const int st = it % S;
    // the next row's statistic is requested a whole iteration before it is needed
    const float rstd_next = row + stride < rows ? rstd_in[row + stride] : 0.f;
    cp_async_wait<S - 2>();
    float xf[NV][8], gf[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      unpack8(data[(st * NCH + i) * kNormThreads + t], xf[i]);
      unpack8(data[(st * NCH + NV + i) * kNormThreads + t], gf[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += gf[i][j] * wf[i][j] * xf[i][j] * rstd;
    }
    const float c = block_sum_alt(dot, sbuf, it) / static_cast<float>(COLS);
    issue(row + (S - 1) * stride, (it + S - 1) % S);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = xf[i][j] * rstd;
        o[j] = rstd * (gf[i][j] * wf[i][j] - xhat * c);
        dw[i][j] += gf[i][j] * xhat;
      }
      *reinterpret_cast<uint4*>(dx + row * lddx + (t + i * kNormThreads) * 8) = pack8(o);
    }
    rstd = rstd_next;
  }
  cp_async_wait<0>();
  if (dw_partial != nullptr) {
    float* prow = dw_partial + static_cast<long long>(blockIdx.x) * COLS;
#pragma unroll
    for (int i = 0; i < NV; ++i) Vec8<float>::store(prow + (t + i * kNormThreads) * 8, dw[i]);
  }
}

}  // namespace ocb
