// Optimizer step fused with its collectives over NVLink peer memory (sharded data parallelism).
//
// The reference reduce-scatters gradients and all-gathers parameters with NCCL around a separate optimizer step
// (FSDP2 inside src/olmo_core/nn/transformer/model.py:859-968, optimizer in src/olmo_core/optim/adamw.py). Here every
// rank keeps its full fp32 gradient buffer and its full bf16 parameter buffer in symmetric memory (the same virtual
// layout on every GPU, mapped into every peer), and two kernels do all of the work for the rows a rank owns:
//
//   ocb_peer_reduce_sumsq  : g[i] = (1/W) * sum_r grad_r[i]   read straight from the W peers' buffers (P2P loads over
//                            NVLink), or with ONE multimem.ld_reduce per 16 bytes when the buffers are bound to an
//                            NVSwitch multicast object (the switch adds the W copies in flight); the squared norm of
//                            the reduced shard is accumulated on the way (gradient clipping needs the global norm
//                            before any parameter may move);
//   ocb_adamw_peer_scatter : SkipStep-AdamW on the fp32 master shard, then the bf16 copy of every updated element is
//                            stored into all W peers' parameter buffers (P2P stores, or one multimem.st) -- the
//                            "all-gather" happens as the values are produced.
//
// Ordering across ranks is the caller's job: a barrier on the stream before the reduce (all ranks finished writing
// gradients) and after the scatter (all stores have landed; the kernel ends with a system-scope fence).
// No TMA and no cluster multicast is involved anywhere in this file: peers are reached with plain ld/st.global and
// multimem instructions only.

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {
namespace {

constexpr int kPeerMax = 16;
constexpr int kFusedThreads = 256;
constexpr int kFusedBlocks = 592;  // 4 x 148

struct PeerPtrs {
  const void* p[kPeerMax];
};
struct PeerPtrsMut {
  void* p[kPeerMax];
};

__device__ __forceinline__ float4 ld_nc_f4(const float* ptr) {
  float4 v;
  // peer memory changes between steps: bypass L1, which is not coherent across GPUs
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b64(void* mc_ptr, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_ptr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y))
               : "memory");
}

// out[i] = scale * sum_r grads_r[offset + i]; partial[blockIdx] = sum over the block's elements of out[i]^2.
// n is a multiple of 4 and all pointers are 16-byte aligned (the runtime aligns every slot).
template <bool MULTIMEM>
__global__ void __launch_bounds__(kFusedThreads)
peer_reduce_sumsq_kernel(PeerPtrs grads, const float* __restrict__ mc_grad, int world, long long offset, long long n,
                         float scale, float* __restrict__ out, float* __restrict__ partial) {
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s;
    if (MULTIMEM) {
      s = multimem_ld_reduce_f4(mc_grad + offset + 4 * i);
    } else {
      s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 v = ld_nc_f4(static_cast<const float*>(grads.p[r]) + offset + 4 * i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  __shared__ float red[kFusedThreads / 32];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kFusedThreads / 32 ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) partial[blockIdx.x] = v;
  }
}

__global__ void add_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out) {
  float v = 0.f;
  for (int i = threadIdx.x; i < n; i += 32) v += partial[i];
  v = warp_sum(v);
  if (threadIdx.x == 0) out[0] += v;
}

// SkipStep-AdamW (same update as adamw_kernel in elementwise.cu) on n elements of the fp32 master shard; the bf16
// result goes to element lowp_offset + i of every peer's parameter buffer.
template <bool MULTIMEM>
__global__ void __launch_bounds__(kFusedThreads)
adamw_peer_scatter_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                          PeerPtrsMut lowp, __nv_bfloat16* __restrict__ mc_lowp, int world, long long lowp_offset,
                          long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                          const float* __restrict__ step_ptr, const float* __restrict__ step_factor_ptr,
                          const float* __restrict__ grad_scale_ptr) {
  // `step` counts the updates already applied; `factor` is 1, or 0 for a skipped step (everything stays unchanged)
  const float factor = step_factor_ptr != nullptr ? step_factor_ptr[0] : 1.f;
  const float gscale = grad_scale_ptr != nullptr ? grad_scale_ptr[0] : 1.f;
  const float t = (step_ptr != nullptr ? step_ptr[0] : 0.f) + 1.f;
  const float bc1 = 1.f - powf(beta1, t);
  const float bc2 = 1.f - powf(beta2, t);
  const float step_size = factor * lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - factor * lr * weight_decay;
  const float w1 = factor * (1.f - beta1), w2 = factor * (1.f - beta2);
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float* pe = &pv.x;
    float* me = &mv.x;
    float* ve = &vv.x;
    const float* ge = &gv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float grad = ge[k] * gscale;
      pe[k] *= decay;
      me[k] += w1 * (grad - me[k]);
      ve[k] = ve[k] * (1.f - w2) + w2 * grad * grad;
      pe[k] -= step_size * me[k] / (sqrtf(ve[k]) * inv_sqrt_bc2 + eps);
    }
    reinterpret_cast<float4*>(p)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    const uint2 packed = make_uint2(pack_bf16x2(pv.x, pv.y), pack_bf16x2(pv.z, pv.w));
    if (MULTIMEM) {
      multimem_st_b64(mc_lowp + lowp_offset + 4 * i, packed);
    } else {
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(lowp.p[r]) + lowp_offset + 4 * i) = packed;
    }
  }
  __threadfence_system();  // peers read these parameters after the caller's barrier
}

int pick_grid(long long n4) {
  long long blocks = (n4 + kFusedThreads - 1) / kFusedThreads;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < kFusedBlocks ? blocks : kFusedBlocks);
}

}  // namespace
}  // namespace ocb

using namespace ocb;

extern "C" int ocb_fused_partials() { return kFusedBlocks; }

// peer_grads: host array of `world` device pointers (each rank's fp32 gradient buffer, same layout); mc_grad: multicast
// address of the same buffer or null. Writes the averaged gradients of [offset, offset+n) to out (local, fp32) and
// ADDS their squared norm to sumsq[0]. scratch: fp32 [ocb_fused_partials()].
extern "C" int ocb_peer_reduce_sumsq(const void* const* peer_grads, const void* mc_grad, int world, long long offset,
                                     long long n, float scale, float* out, float* scratch, float* sumsq,
                                     cudaStream_t stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kPeerMax || (n & 3) || (offset & 3) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  PeerPtrs ptrs;
  for (int r = 0; r < kPeerMax; ++r) ptrs.p[r] = r < world ? peer_grads[r] : nullptr;
  const int grid = pick_grid(n >> 2);
  if (mc_grad != nullptr)
    peer_reduce_sumsq_kernel<true><<<grid, kFusedThreads, 0, stream>>>(ptrs, static_cast<const float*>(mc_grad), world,
                                                                      offset, n, scale, out, scratch);
  else
    peer_reduce_sumsq_kernel<false><<<grid, kFusedThreads, 0, stream>>>(ptrs, nullptr, world, offset, n, scale, out, scratch);
  add_partials_kernel<<<1, 32, 0, stream>>>(scratch, grid, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// p, m, v, g: this rank's fp32 shard (n elements, n % 4 == 0). peer_lowp: host array of `world` device pointers to the
// peers' bf16 parameter buffers; element lowp_offset + i of each receives bf16(p[i]). mc_lowp: multicast address or null.
extern "C" int ocb_adamw_peer_scatter(float* p, float* m, float* v, const float* g, void* const* peer_lowp, void* mc_lowp,
                                      int world, long long lowp_offset, long long n, float lr, float beta1, float beta2,
                                      float eps, float weight_decay, const float* step, const float* step_factor,
                                      const float* grad_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kPeerMax || (n & 3) || (lowp_offset & 3)) return -1;
  PeerPtrsMut ptrs;
  for (int r = 0; r < kPeerMax; ++r) ptrs.p[r] = r < world ? peer_lowp[r] : nullptr;
  const int grid = pick_grid(n >> 2);
  if (mc_lowp != nullptr)
    adamw_peer_scatter_kernel<true><<<grid, kFusedThreads, 0, stream>>>(
        p, m, v, g, ptrs, static_cast<__nv_bfloat16*>(mc_lowp), world, lowp_offset, n, lr, beta1, beta2, eps, weight_decay,
        step, step_factor, grad_scale);
  else
    adamw_peer_scatter_kernel<false><<<grid, kFusedThreads, 0, stream>>>(p, m, v, g, ptrs, nullptr, world, lowp_offset, n,
                                                                        lr, beta1, beta2, eps, weight_decay, step,
                                                                        step_factor, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
