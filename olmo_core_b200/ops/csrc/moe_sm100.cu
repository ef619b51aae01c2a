// Mixture-of-experts routing and token permutation for sm_100a.
//
//   router     logits [N, E] -> softmax scores, top-k (weights, expert ids), tokens per expert      (one pass)
//   sort       expert ids [N*k] -> stable counting sort: row of every routed copy, copy of every row, group offsets
//   gather     expert-sorted activation matrix  xs[r] = (w[src[r]] *) x[src[r] / k]
//   scatter    y[t] = sum_j w[t, j] * ys[dest[t*k + j]]      (fp32 accumulation, fixed order: deterministic)
//   rowdot     dw[t, j] = <ys[dest[t*k + j]], dy[t]>         (gradient of the routing weights)
//
// These replace the Triton copy kernels and the torch.sort / topk / histc calls of the reference
// (src/olmo_core/kernels/moe.py:31-536, src/olmo_core/ops/moe.py:52-304, src/olmo_core/nn/moe/router.py:416-512,
// src/olmo_core/nn/moe/parallel_mlp.py:102-125). All kernels are memory bound: rows move with 16-byte accesses and
// every byte is touched once. Nothing here waits on another CTA or on the host.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ocb_api.h"

namespace ocb {

constexpr int SORT_CHUNK = 2048;  // routed copies ranked by one warp
constexpr int MAX_EXPERTS = 1024;

__device__ __forceinline__ float ld_act(const void* p, long long i, int dtype) {
  return dtype == OCB_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                           : reinterpret_cast<const float*>(p)[i];
}

// ------------------------------------------------------------------------------------------------ router
// One warp per token. Each lane keeps E/32 logits in registers (E <= 1024); the top-k are extracted by k rounds of a
// warp arg-max (ties go to the lower expert id, like torch.topk on a stable sort). mode: 0 = softmax then top-k,
// 1 = sigmoid scores then top-k. normalize: weights / sum(weights). counts: int32 [E], must be zero on entry.
template <int PER_LANE>
__global__ void router_topk_kernel(const void* __restrict__ logits, float* __restrict__ scores, float* __restrict__ weights,
                                   int* __restrict__ experts, int* __restrict__ counts, int n_tokens, int n_experts,
                                   int top_k, int mode, int normalize, long long ld, int dtype) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_tokens) return;
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < n_experts ? ld_act(logits, warp * ld + e, dtype) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  if (mode == 0) {
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      v[i] = (i * 32 + lane) < n_experts ? __expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) v[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) v[i] = (i * 32 + lane) < n_experts ? 1.f / (1.f + __expf(-v[i])) : 0.f;
  }
  if (scores != nullptr) {
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts) scores[static_cast<long long>(warp) * n_experts + e] = v[i];
    }
  }
  float total = 0.f;
  float picked_w = 0.f;  // lane j keeps the j-th pick (top_k <= 32)
  int picked_e = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts && v[i] > best) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {  // remove the winner (scores are >= 0); static indexing keeps v[] in registers
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) v[i] = -2.f;
    }
    if (lane == j) { picked_w = best; picked_e = best_e; }
    total += best;
  }
  if (lane < top_k) {
    if (normalize) picked_w /= fmaxf(total, 1e-20f);
    weights[static_cast<long long>(warp) * top_k + lane] = picked_w;
    experts[static_cast<long long>(warp) * top_k + lane] = picked_e;
    if (counts != nullptr) atomicAdd(&counts[picked_e], 1);
  }
}

// -------------------------------------------------------------------------------------------------- sort
// Pass 1: one warp per chunk of SORT_CHUNK routed copies. rank[j] = how many earlier copies of the chunk go to the same
// expert; hist[chunk, e] = copies of the chunk going to e.
__global__ void sort_rank_kernel(const int* __restrict__ experts, int* __restrict__ rank, int* __restrict__ hist,
                                 int n, int n_experts) {
  extern __shared__ int counters[];  // [n_experts]
  const int lane = threadIdx.x;
  const int chunk = blockIdx.x;
  for (int e = lane; e < n_experts; e += 32) counters[e] = 0;
  __syncwarp();
  const int begin = chunk * SORT_CHUNK;
  const int end = min(n, begin + SORT_CHUNK);
  for (int base = begin; base < end; base += 32) {
    const int j = base + lane;
    const bool live = j < end;
    const int e = live ? experts[j] : -1 - lane;  // dead lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    int start = 0;
    if (live && lane == leader) {
      start = counters[e];
      counters[e] = start + __popc(peers);
    }
    start = __shfl_sync(0xffffffffu, start, leader);
    if (live) rank[j] = start + before;
    __syncwarp();
  }
  for (int e = lane; e < n_experts; e += 32) hist[chunk * n_experts + e] = counters[e];
}

// Pass 2: one thread per expert turns hist[:, e] into exclusive prefix sums over the chunks and writes the expert total;
// thread 0 then scans the totals into offsets[0..E].
__global__ void sort_scan_kernel(int* __restrict__ hist, int* __restrict__ offsets, int n_chunks, int n_experts) {
  __shared__ int totals[MAX_EXPERTS];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int h = hist[c * n_experts + e];
      hist[c * n_experts + e] = run;
      run += h;
    }
    totals[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = run;
      run += totals[e];
    }
    offsets[n_experts] = run;
  }
}

// Pass 3: dest[j] = offsets[e] + chunk base + rank; src[dest[j]] = j; sorted_experts[dest[j]] = e.
__global__ void sort_place_kernel(const int* __restrict__ experts, const int* __restrict__ rank, const int* __restrict__ hist,
                                  const int* __restrict__ offsets, int* __restrict__ dest, int* __restrict__ src,
                                  int* __restrict__ sorted_experts, int n, int n_experts) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const int e = experts[j];
  const int d = offsets[e] + hist[(j / SORT_CHUNK) * n_experts + e] + rank[j];
  dest[j] = d;
  src[d] = j;
  if (sorted_experts != nullptr) sorted_experts[d] = e;
}

// ------------------------------------------------------------------------------------------- row movement
// One warp per output row, 16-byte accesses (cols % 8 == 0 for bf16).
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int n_rows, int cols,
                                   int top_k, long long ldx, long long ldo) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int j = src[row];
  const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<long long>(j / top_k) * ldx);
  uint4* o = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * ldo);
  const int vecs = cols >> 3;
  if (w == nullptr) {
    for (int i = lane; i < vecs; i += 32) o[i] = in[i];
  } else {
    const float s = w[j];
    for (int i = lane; i < vecs; i += 32) {
      uint4 u = in[i];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        h[q] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
      o[i] = u;
    }
  }
}

// One warp per token: y[t] = sum_j w[t, j] * ys[dest[t*k + j]].
__global__ void scatter_rows_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ dest,
                                    const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int n_tokens, int cols,
                                    int top_k, long long lds, long long ldy) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const int vecs = cols >> 3;
  for (int i = lane; i < vecs; i += 32) {
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int r = dest[t * top_k + j];
      const float s = w == nullptr ? 1.f : w[t * top_k + j];
      const uint4 u = reinterpret_cast<const uint4*>(ys + static_cast<long long>(r) * lds)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += s * f.x;
        acc[2 * q + 1] += s * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(y + static_cast<long long>(t) * ldy)[i] = o;
  }
}

// One warp per routed copy: dw[j] = <ys[dest[j]], dy[j / k]>.
__global__ void rowdot_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ dest,
                              const __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, int n_copies, int cols,
                              int top_k, long long lds, long long ldd) {
  const int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (j >= n_copies) return;
  const uint4* a = reinterpret_cast<const uint4*>(ys + static_cast<long long>(dest[j]) * lds);
  const uint4* b = reinterpret_cast<const uint4*>(dy + static_cast<long long>(j / top_k) * ldd);
  float acc = 0.f;
  for (int i = lane; i < (cols >> 3); i += 32) {
    const uint4 ua = a[i], ub = b[i];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ua);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 fa = __bfloat1622float2(ha[q]), fb = __bfloat1622float2(hb[q]);
      acc += fa.x * fb.x + fa.y * fb.y;
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dw[j] = acc;
}

}  // namespace ocb

using namespace ocb;

static inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? 0 : -4; }

extern "C" int ocb_moe_router_topk(const void* logits, float* scores, float* weights, int* experts, int* counts,
                                   int n_tokens, int n_experts, int top_k, int mode, int normalize, long long ld,
                                   int act_dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_experts <= 0 || n_experts > MAX_EXPERTS || top_k <= 0 || top_k > 32 || top_k > n_experts) return -1;
  if (counts != nullptr && cudaMemsetAsync(counts, 0, sizeof(int) * n_experts, stream) != cudaSuccess) return -4;
  const int threads = 256;
  const int blocks = (n_tokens * 32 + threads - 1) / threads;
#define OCB_ROUTER(PL)                                                                                              \
  router_topk_kernel<PL><<<blocks, threads, 0, stream>>>(logits, scores, weights, experts, counts, n_tokens, n_experts, \
                                                         top_k, mode, normalize, ld, act_dtype)
  if (n_experts <= 32) OCB_ROUTER(1);
  else if (n_experts <= 64) OCB_ROUTER(2);
  else if (n_experts <= 128) OCB_ROUTER(4);
  else if (n_experts <= 256) OCB_ROUTER(8);
  else if (n_experts <= 512) OCB_ROUTER(16);
  else OCB_ROUTER(32);
#undef OCB_ROUTER
  return launch_ok();
}

// Scratch: int32 [ocb_moe_sort_scratch_ints(n, n_experts)].
extern "C" long long ocb_moe_sort_scratch_ints(int n, int n_experts) {
  const long long chunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
  return static_cast<long long>(n) + chunks * n_experts;
}

extern "C" int ocb_moe_sort(const int* experts, int* dest, int* src, int* sorted_experts, int* offsets, int* scratch, int n,
                            int n_experts, cudaStream_t stream) {
  if (n_experts <= 0 || n_experts > MAX_EXPERTS) return -1;
  if (n <= 0) return cudaMemsetAsync(offsets, 0, sizeof(int) * (n_experts + 1), stream) == cudaSuccess ? 0 : -4;
  const int chunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
  int* rank = scratch;
  int* hist = scratch + n;
  sort_rank_kernel<<<chunks, 32, sizeof(int) * n_experts, stream>>>(experts, rank, hist, n, n_experts);
  sort_scan_kernel<<<1, 256, 0, stream>>>(hist, offsets, chunks, n_experts);
  sort_place_kernel<<<(n + 255) / 256, 256, 0, stream>>>(experts, rank, hist, offsets, dest, src, sorted_experts, n,
                                                         n_experts);
  return launch_ok();
}

extern "C" int ocb_moe_gather(const void* x, const int* src, const float* w, void* out, int n_rows, int cols, int top_k,
                              long long ldx, long long ldo, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if ((cols & 7) || (ldx & 7) || (ldo & 7)) return -1;
  gather_rows_kernel<<<(n_rows * 32 + 255) / 256, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), src, w, reinterpret_cast<__nv_bfloat16*>(out), n_rows, cols, top_k, ldx, ldo);
  return launch_ok();
}

extern "C" int ocb_moe_scatter(const void* ys, const int* dest, const float* w, void* y, int n_tokens, int cols, int top_k,
                               long long lds, long long ldy, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((cols & 7) || (lds & 7) || (ldy & 7)) return -1;
  scatter_rows_kernel<<<(n_tokens * 32 + 255) / 256, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(ys), dest, w, reinterpret_cast<__nv_bfloat16*>(y), n_tokens, cols, top_k, lds, ldy);
  return launch_ok();
}

extern "C" int ocb_moe_rowdot(const void* ys, const int* dest, const void* dy, float* dw, int n_copies, int cols, int top_k,
                              long long lds, long long ldd, cudaStream_t stream) {
  if (n_copies <= 0) return 0;
  if ((cols & 7) || (lds & 7) || (ldd & 7)) return -1;
  rowdot_kernel<<<(n_copies * 32 + 255) / 256, 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(ys), dest, reinterpret_cast<const __nv_bfloat16*>(dy), dw, n_copies, cols, top_k,
      lds, ldd);
  return launch_ok();
}
