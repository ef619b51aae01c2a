// Per-block parameter gather and gradient reduce-scatter of the streamed sharded-parameter mode, over NVLink peer
// memory (the reference gets both from FSDP2's per-block NCCL all-gather / reduce-scatter:
// src/olmo_core/nn/transformer/model.py:859-935).
//
// Every rank keeps only its rows of every parameter: bf16 in `param_shard` (symmetric memory, the same layout on every
// rank) and fp32 gradients in `grad_shard` (local). A block's parameters are needed in full only while the block computes,
// so they are assembled into a small local ring just in time, and the block's full-size gradients sit in a ring slot
// (symmetric memory again) only until the owners of the rows have collected them:
//
//   ocb_peer_gather_segments       full[seg.full_off + r * seg.n + i] = param_shard_r[seg.shard_off + i]   for all ranks r
//                                  (plain loads from the owners' memory; runs on a side stream one block ahead of
//                                  the GEMMs that consume the assembled weights)
//   ocb_peer_pull_reduce_segments  grad_shard[seg.shard_off + i] += scale * sum_r grad_full_r[seg.full_off + me * seg.n + i]
//                                  every rank pulls ITS rows of the block's gradient out of all ranks' ring slots (plain
//                                  loads, summed in rank order in registers: reproducible bit for bit) and accumulates
//                                  them into its shard. The caller brackets the kernel with two stream barriers across
//                                  the ranks (all ranks have finished the block's backward / all ranks have finished
//                                  pulling, so the slots may be cleared and reused); both run on the side stream, behind
//                                  the next block's backward. Pushing with fp32 reductions instead needs no barrier but
//                                  reached only 165 GB/s here (reductions of 16 bytes at the owner's L2), against
//                                  785 GB/s for plain loads.
//
// Plain ld / st only: no TMA, no multimem, no atomics.

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
peer_pull_reduce_segments_kernel(StreamPeers grad_fulls, int world, int rank, const StreamSegment* __restrict__ segs, int nseg,
                                 float* __restrict__ grad_shard, float scale) {
  for (int s = 0; s < nseg; ++s) {
    const StreamSegment seg = segs[s];
    const long long n4 = seg.n >> 2;
    const long long src_off = seg.full_off + static_cast<long long>(rank) * seg.n;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float* src = static_cast<const float*>(grad_fulls.p[r]) + src_off + 4 * i;
        float4 v;
        asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src) : "memory");
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float4* dst = reinterpret_cast<float4*>(grad_shard + seg.shard_off) + i;
      float4 o = *dst;
      o.x += acc.x * scale; o.y += acc.y * scale; o.z += acc.z * scale; o.w += acc.w * scale;
      *dst = o;
    }
    const long long tail = seg.n & 3;
    if (tail != 0 && blockIdx.x == 0 && threadIdx.x < tail) {
      const long long j = (seg.n - tail) + threadIdx.x;
      float acc = 0.f;
      for (int r = 0; r < world; ++r) {
        float v;
        asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(v) : "l"(static_cast<const float*>(grad_fulls.p[r]) + src_off + j) : "memory");
        acc += v;
      }
      grad_shard[seg.shard_off + j] += acc * scale;
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

// grad_full_ptrs[r]: rank r's full-size fp32 gradient block (its ring slot) as mapped on this GPU; grad_shard: this
// rank's shard, accumulated into. scale: 1 / world for an average. The slots are not modified.
extern "C" int ocb_peer_pull_reduce_segments(void* const* grad_full_ptrs, int world, int rank, const void* segs, int nseg,
                                             void* grad_shard, float scale, cudaStream_t stream) {
  if (world < 1 || world > kStreamMaxRanks || rank < 0 || rank >= world || nseg < 0) return -1;
  if (nseg == 0) return 0;
  StreamPeers p;
  for (int r = 0; r < world; ++r) p.p[r] = grad_full_ptrs[r];
  peer_pull_reduce_segments_kernel<<<296, kStreamThreads, 0, stream>>>(p, world, rank, static_cast<const StreamSegment*>(segs),
                                                                       nseg, static_cast<float*>(grad_shard), scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
