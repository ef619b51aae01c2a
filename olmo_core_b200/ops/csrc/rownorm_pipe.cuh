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

// Eight fp32 values as four packed pairs: sm_100 executes mul / add / sub / fma on both halves of a pair in one
// instruction, which halves the arithmetic instruction count of these kernels (they are close to issue-bound).
struct V8 {
  uint64_t p[4];
};
__device__ __forceinline__ V8 v8_from_bf16(const uint4& u) {
  V8 r;
  r.p[0] = bf16x2_to_f32x2(u.x); r.p[1] = bf16x2_to_f32x2(u.y);
  r.p[2] = bf16x2_to_f32x2(u.z); r.p[3] = bf16x2_to_f32x2(u.w);
  return r;
}
__device__ __forceinline__ V8 v8_from_floats(const float (&f)[8]) {
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = pack_f32x2(f[2 * k], f[2 * k + 1]);
  return r;
}
__device__ __forceinline__ V8 v8_splat(float s) {
  V8 r;
  r.p[0] = r.p[1] = r.p[2] = r.p[3] = pack_f32x2(s, s);
  return r;
}
__device__ __forceinline__ V8 v8_lds(const float* smem) {
  float f[8];
  lds8(smem, f);
  return v8_from_floats(f);
}
__device__ __forceinline__ uint64_t sub_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ V8 v8_mul(const V8& a, const V8& b) {
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = mul_f32x2(a.p[k], b.p[k]);
  return r;
}
__device__ __forceinline__ V8 v8_mul(const V8& a, uint64_t s2) {
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = mul_f32x2(a.p[k], s2);
  return r;
}
__device__ __forceinline__ V8 v8_add(const V8& a, const V8& b) {
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = add_f32x2(a.p[k], b.p[k]);
  return r;
}
__device__ __forceinline__ V8 v8_sub(const V8& a, const V8& b) {
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = sub_f32x2(a.p[k], b.p[k]);
  return r;
}
__device__ __forceinline__ V8 v8_fma(const V8& a, const V8& b, const V8& c) {  // a * b + c
  V8 r;
#pragma unroll
  for (int k = 0; k < 4; ++k) r.p[k] = fma_f32x2(a.p[k], b.p[k], c.p[k]);
  return r;
}
__device__ __forceinline__ float v8_hsum(const V8& a) {
  const uint64_t s = add_f32x2(add_f32x2(a.p[0], a.p[1]), add_f32x2(a.p[2], a.p[3]));
  float lo, hi;
  unpack_f32x2(s, lo, hi);
  return lo + hi;
}
__device__ __forceinline__ uint4 v8_to_bf16(const V8& a) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float lo, hi;
    unpack_f32x2(a.p[k], lo, hi);
    w[k] = pack_bf16x2(lo, hi);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ V8 v8_round_bf16(const V8& a) { return v8_from_bf16(v8_to_bf16(a)); }
__device__ __forceinline__ void v8_store_f32(float* dst, const V8& a) {
  float f[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) unpack_f32x2(a.p[k], f[2 * k], f[2 * k + 1]);
  Vec8<float>::store(dst, f);
}
template <typename W>
__device__ __forceinline__ V8 v8_load_w(const W* w) {
  float f[8];
  Vec8<W>::load(w, f);
  return v8_from_floats(f);
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

  V8 wa = v8_splat(1.f), wb = v8_splat(1.f);
  if (norm_mode != 0 && on) {
    const int wofs = norm_mode == 1 ? h * HD : 0;
    wa = v8_load_w<W>(w + wofs + o);
    wb = v8_load_w<W>(w + wofs + HALF + o);
  }
  V8 dwa = v8_splat(0.f), dwb = v8_splat(0.f);

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
    V8 a = v8_splat(0.f), b = a, xa = a, xb = a;
    if (on) {
      a = v8_from_bf16(data[(st * NCH + 0) * kNormThreads + t]);
      b = v8_from_bf16(data[(st * NCH + 1) * kNormThreads + t]);
      if (need_x) {
        xa = v8_from_bf16(data[(st * NCH + 2) * kNormThreads + t]);
        xb = v8_from_bf16(data[(st * NCH + 3) * kNormThreads + t]);
      }
    }
    const float* cs = trig + (st * 2 + 0) * HD;
    const float* sn = trig + (st * 2 + 1) * HD;

    if (!BWD) {
      const float ss = v8_hsum(v8_fma(b, b, v8_mul(a, a)));
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
        V8 ya = a, yb = b;
        if (norm_mode != 0) {  // (x * rstd) * w, rounded to bf16 as the unfused modules would
          const uint64_t rs2 = pack_f32x2(rs, rs);
          ya = v8_round_bf16(v8_mul(v8_mul(a, rs2), wa));
          yb = v8_round_bf16(v8_mul(v8_mul(b, rs2), wb));
        }
        const V8 oa = v8_sub(v8_mul(ya, v8_lds(cs + o)), v8_mul(yb, v8_lds(sn + o)));
        const V8 ob = v8_fma(ya, v8_lds(sn + HALF + o), v8_mul(yb, v8_lds(cs + HALF + o)));
        __nv_bfloat16* dst = out + row * ld_out + h * HD + o;
        *reinterpret_cast<uint4*>(dst) = v8_to_bf16(oa);
        *reinterpret_cast<uint4*>(dst + HALF) = v8_to_bf16(ob);
      }
    } else {
      // The rotation's transpose needs sin/cos, which other threads copied: the barrier comes first here.
      const float rs = rs_bwd;
      __syncthreads();
      issue(row + (S - 1) * stride, (it + S - 1) % S);
      const V8 ga = v8_fma(b, v8_lds(sn + HALF + o), v8_mul(a, v8_lds(cs + o)));
      const V8 gb = v8_sub(v8_mul(b, v8_lds(cs + HALF + o)), v8_mul(a, v8_lds(sn + o)));
      if (norm_mode != 0) {
        const V8 gwa = v8_mul(ga, wa), gwb = v8_mul(gb, wb);
        float dot = on ? rs * v8_hsum(v8_fma(gwb, xb, v8_mul(gwa, xa))) : 0.f;
        float c;
        if (norm_mode == 2) {
          for (int s2 = 4; s2 > 0; s2 >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s2);
          c = dot / static_cast<float>(HD);
        } else {
          // second barrier of the row; its scratch row alternates like the forward kernel's
          c = block_sum_alt(dot, sbuf, it) / static_cast<float>(cols);
        }
        if (on) {
          const uint64_t rs2 = pack_f32x2(rs, rs);
          const V8 c8 = v8_splat(c);
          const V8 xha = v8_mul(xa, rs2), xhb = v8_mul(xb, rs2);
          const V8 oa = v8_mul(v8_sub(gwa, v8_mul(xha, c8)), rs2);
          const V8 ob = v8_mul(v8_sub(gwb, v8_mul(xhb, c8)), rs2);
          dwa = v8_fma(ga, xha, dwa);
          dwb = v8_fma(gb, xhb, dwb);
          __nv_bfloat16* dst = out + row * ld_out + h * HD + o;
          *reinterpret_cast<uint4*>(dst) = v8_to_bf16(oa);
          *reinterpret_cast<uint4*>(dst + HALF) = v8_to_bf16(ob);
        }
      } else if (on) {
        __nv_bfloat16* dst = out + row * ld_out + h * HD + o;
        *reinterpret_cast<uint4*>(dst) = v8_to_bf16(ga);
        *reinterpret_cast<uint4*>(dst + HALF) = v8_to_bf16(gb);
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
      v8_store_f32(prow + h * HD + o, dwa);
      v8_store_f32(prow + h * HD + HALF + o, dwb);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a0, a1, b0, b1;
        unpack_f32x2(dwa.p[k], a0, a1);
        unpack_f32x2(dwb.p[k], b0, b1);
        atomicAdd(&prow[o + 2 * k], a0);
        atomicAdd(&prow[o + 2 * k + 1], a1);
        atomicAdd(&prow[HALF + o + 2 * k], b0);
        atomicAdd(&prow[HALF + o + 2 * k + 1], b1);
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

  V8 wf[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) wf[i] = w != nullptr ? v8_load_w<W>(w + (t + i * kNormThreads) * 8) : v8_splat(1.f);

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
    V8 f[NV], rf[NV];
    V8 sq = v8_splat(0.f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      f[i] = v8_from_bf16(data[(st * NCH + i) * kNormThreads + t]);
      if (RESID) rf[i] = v8_from_bf16(data[(st * NCH + NV + i) * kNormThreads + t]);
      sq = v8_fma(f[i], f[i], sq);
    }
    const float ss = v8_hsum(sq);
    // A thread reads only what it copied itself, so the slot of the previous row is free once every thread has
    // reached this barrier.
    const float total = block_sum_alt(ss, sbuf, it);
    issue(row + (S - 1) * stride, (it + S - 1) % S);
    const float rstd = rsqrtf(total / static_cast<float>(COLS) + eps);
    if (t == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    const uint64_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      V8 o = v8_mul(v8_mul(f[i], rstd2), wf[i]);
      if (RESID) o = v8_add(rf[i], v8_round_bf16(o));
      *reinterpret_cast<uint4*>(y + row * ldy + (t + i * kNormThreads) * 8) = v8_to_bf16(o);
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

  V8 wf[NV], dw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    wf[i] = w != nullptr ? v8_load_w<W>(w + (t + i * kNormThreads) * 8) : v8_splat(1.f);
    dw[i] = v8_splat(0.f);
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
    V8 xf[NV], gf[NV], gw[NV];
    V8 acc = v8_splat(0.f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xf[i] = v8_from_bf16(data[(st * NCH + i) * kNormThreads + t]);
      gf[i] = v8_from_bf16(data[(st * NCH + NV + i) * kNormThreads + t]);
      gw[i] = v8_mul(gf[i], wf[i]);
      acc = v8_fma(gw[i], xf[i], acc);
    }
    const float c = block_sum_alt(rstd * v8_hsum(acc), sbuf, it) / static_cast<float>(COLS);
    issue(row + (S - 1) * stride, (it + S - 1) % S);
    const uint64_t rstd2 = pack_f32x2(rstd, rstd);
    const V8 c8 = v8_splat(c);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const V8 xhat = v8_mul(xf[i], rstd2);
      const V8 o = v8_mul(v8_sub(gw[i], v8_mul(xhat, c8)), rstd2);
      dw[i] = v8_fma(gf[i], xhat, dw[i]);
      *reinterpret_cast<uint4*>(dx + row * lddx + (t + i * kNormThreads) * 8) = v8_to_bf16(o);
    }
    rstd = rstd_next;
  }
  cp_async_wait<0>();
  if (dw_partial != nullptr) {
    float* prow = dw_partial + static_cast<long long>(blockIdx.x) * COLS;
#pragma unroll
    for (int i = 0; i < NV; ++i) v8_store_f32(prow + (t + i * kNormThreads) * 8, dw[i]);
  }
}

}  // namespace ocb
