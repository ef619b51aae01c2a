// Per-block parameter gather and gradient reduce-scatter of the streamed sharded-parameter mode, over NVLink peer
// memory (the reference gets both from FSDP2's per-block NCCL all-gather / reduce-scatter:
// src/olmo_core/nn/transformer/model.py:859-935).
//
// Every rank keeps only its rows of every parameter: bf16 in `param_shard`, fp32 gradients in `grad_shard`, both in
// symmetric memory with the same layout on every rank. A block's parameters are needed in full only while the block
// computes, so they are assembled into a small local ring just in time:
//
//   ocb_peer_gather_segments       full[seg.full_off + r * seg.n + i] = param_shard_r[seg.shard_off + i]   for all ranks r
//                                  (plain loads from the owners' memory; runs on a side stream one block ahead of
//                                  the GEMMs that consume the assembled weights)
//   ocb_peer_scatter_add_segments  grad_shard_r[seg.shard_off + i] += scale * grad_full[seg.full_off + r * seg.n + i]
//                                  with fire-and-forget fp32 reductions performed at the owner's L2, then the local
//                                  full-size gradient block is cleared for the next block that uses the ring slot.
//                                  No rank waits for any other: one barrier before the optimizer step is enough.
//
// fp32 additions from different ranks arrive in no fixed order, so a reduced gradient is reproducible up to the rounding
// of a `world`-term fp32 sum. Plain ld / st / red only: no TMA, no multimem.

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {
namespace {

constexpr int kStreamMaxRanks = 16;
constexpr int kStreamThreads = 256;

struct StreamPeers {
  void* p[kStreamMaxRanks];
};

// One parameter of the block: n elements per rank at shard_off of every rank's shard, the full copy at full_off.
struct StreamSegment {
  long long shard_off, full_off, n;
};

__global__ void __launch_bounds__(kStreamThreads)
peer_gather_segments_kernel(StreamPeers shards, int world, const StreamSegment* __restrict__ segs, int nseg,
                            __nv_bfloat16* __restrict__ full) {
  for (int s = 0; s < nseg; ++s) {
    const StreamSegment seg = segs[s];
    const long long n8 = seg.n >> 3;  // 16-byte pieces (the runtime aligns every offset to 8 elements)
    const long long total = n8 * world;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const int r = static_cast<int>(i / n8);
      const long long j = i - r * n8;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(shards.p[r]) + seg.shard_off) + j;
      uint4 v;
      asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
      reinterpret_cast<uint4*>(full + seg.full_off + r * seg.n)[j] = v;
    }
    const long long tail = seg.n & 7;
    if (tail != 0 && blockIdx.x == 0) {
      for (long long i = threadIdx.x; i < tail * world; i += blockDim.x) {
        const int r = static_cast<int>(i / tail);
        const long long j = (seg.n - tail) + (i - r * tail);
        full[seg.full_off + r * seg.n + j] = static_cast<const __nv_bfloat16*>(shards.p[r])[seg.shard_off + j];
      }
    }
  }
}

__global__ void __launch_bounds__(kStreamThreads)
peer_scatter_add_segments_kernel(StreamPeers grad_shards, int world, const StreamSegment* __restrict__ segs, int nseg,
                                 float* __restrict__ grad_full, float scale) {
  for (int s = 0; s < nseg; ++s) {
    const StreamSegment seg = segs[s];
    const long long n4 = seg.n >> 2;
    const long long total = n4 * world;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const int r = static_cast<int>(i / n4);
      const long long j = i - r * n4;
      float4* src = reinterpret_cast<float4*>(grad_full + seg.full_off + r * seg.n) + j;
      const float4 v = *src;
      *src = make_float4(0.f, 0.f, 0.f, 0.f);
      float* dst = static_cast<float*>(grad_shards.p[r]) + seg.shard_off + 4 * j;
      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x * scale), "f"(v.y * scale),
                   "f"(v.z * scale), "f"(v.w * scale)
                   : "memory");
    }
    const long long tail = seg.n & 3;
    if (tail != 0 && blockIdx.x == 0) {
      for (long long i = threadIdx.x; i < tail * world; i += blockDim.x) {
        const int r = static_cast<int>(i / tail);
        const long long j = (seg.n - tail) + (i - r * tail);
        float* src = grad_full + seg.full_off + r * seg.n + j;
        const float v = *src;
        *src = 0.f;
        asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(static_cast<float*>(grad_shards.p[r]) + seg.shard_off + j),
                     "f"(v * scale)
                     : "memory");
      }
    }
  }
}

}  // namespace
}  // namespace ocb

using namespace ocb;

// segs: DEVICE array of nseg {shard_off, full_off, n} triples (int64). shard_ptrs[r]: rank r's bf16 parameter shard as
// mapped on this GPU. full: this GPU's assembled copy. All offsets are multiples of 8 elements.
extern "C" int ocb_peer_gather_segments(void* const* shard_ptrs, int world, const void* segs, int nseg, void* full,
                                        cudaStream_t stream) {
  if (world < 1 || world > kStreamMaxRanks || nseg < 0) return -1;
  if (nseg == 0) return 0;
  StreamPeers p;
  for (int r = 0; r < world; ++r) p.p[r] = shard_ptrs[r];
  peer_gather_segments_kernel<<<296, kStreamThreads, 0, stream>>>(p, world, static_cast<const StreamSegment*>(segs), nseg,
                                                                  static_cast<__nv_bfloat16*>(full));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// grad_shard_ptrs[r]: rank r's fp32 gradient shard as mapped on this GPU; grad_full: this GPU's full-size gradient
// block, cleared by the kernel. scale: 1 / world for an average.
extern "C" int ocb_peer_scatter_add_segments(void* const* grad_shard_ptrs, int world, const void* segs, int nseg,
                                             void* grad_full, float scale, cudaStream_t stream) {
  if (world < 1 || world > kStreamMaxRanks || nseg < 0) return -1;
  if (nseg == 0) return 0;
  StreamPeers p;
  for (int r = 0; r < world; ++r) p.p[r] = grad_shard_ptrs[r];
  peer_scatter_add_segments_kernel<<<296, kStreamThreads, 0, stream>>>(p, world, static_cast<const StreamSegment*>(segs), nseg,
                                                                       static_cast<float*>(grad_full), scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
