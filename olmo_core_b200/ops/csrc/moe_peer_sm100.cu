// Expert-parallel token exchange over peer memory: one kernel that permutes rows AND delivers them to the GPU that owns
// their expert (or back to the GPU that owns the token), with plain stores through the NVLink peer mappings of a
// symmetric buffer. It replaces "gather into a send buffer, NCCL all-to-all, re-sort by local expert" of the reference's
// dropless expert-parallel path (src/olmo_core/nn/moe/parallel_mlp.py, parallel_forward_once) by a single pass whose
// destination layout is already grouped by local expert.
//
// The transfer is described by a table of segments computed on the device from the all-gathered routing counts: segment s
// moves rows [src_start[s], src_start[s] + count[s]) of the (optionally gathered) source to rows dst_start[s]... of rank
// dst_rank[s]'s buffer. Dispatch uses one segment per global expert, combine one per (local expert, source rank).
// Completion is a stream-ordered cross-rank barrier issued by the caller after the launch; nothing in here waits.

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {
namespace {

constexpr int PUSH_MAX_PEERS = 16;
constexpr int PUSH_WARPS = 8;
constexpr int PUSH_BLOCKS_PER_SEGMENT = 24;

struct PushParams {
  const uint4* src;             // [rows, ld_src] bf16, viewed as 16-byte vectors
  const int* gather_idx;        // nullable: source row of sorted row i is gather_idx[i] / gather_div
  int gather_div;
  const int* seg_src_start;     // [S]
  const int* seg_count;         // [S]
  const int* seg_dst_rank;      // [S]
  const long long* seg_dst_start;  // [S]
  const int* seg_src_col;       // nullable [S]: first 16-byte vector of the segment inside a source row
  const int* seg_dst_col;       // nullable [S]: first 16-byte vector inside a destination row
  uint4* peer[PUSH_MAX_PEERS];  // base of every rank's destination buffer
  long long dst_capacity_rows;
  int vecs_per_row;             // cols / 8
  long long ld_src_vec, ld_dst_vec;
  int* status;
};

__global__ void __launch_bounds__(PUSH_WARPS * 32) moe_push_rows_kernel(const PushParams p) {
  const int s = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int count = p.seg_count[s];
  if (count <= 0) return;
  const int src0 = p.seg_src_start[s];
  const long long dst0 = p.seg_dst_start[s];
  uint4* dst_base = p.peer[p.seg_dst_rank[s]];
  for (int r = blockIdx.x * PUSH_WARPS + warp; r < count; r += gridDim.x * PUSH_WARPS) {
    const long long dst_row = dst0 + r;
    if (dst_row < 0 || dst_row >= p.dst_capacity_rows) {  // more rows than the receive buffer holds: report, skip
      if (lane == 0) atomicCAS(p.status, 0, kStatusBadArgument);
      continue;
    }
    const int sorted_row = src0 + r;
    const long long src_row = p.gather_idx ? p.gather_idx[sorted_row] / p.gather_div : sorted_row;
    const uint4* src = p.src + src_row * p.ld_src_vec + (p.seg_src_col ? p.seg_src_col[s] : 0);
    uint4* dst = dst_base + dst_row * p.ld_dst_vec + (p.seg_dst_col ? p.seg_dst_col[s] : 0);
    // two vectors in flight per lane: the loads of the second overlap the NVLink stores of the first
    int v = lane;
    for (; v + 32 < p.vecs_per_row; v += 64) {
      const uint4 a = src[v], b = src[v + 32];
      dst[v] = a;
      dst[v + 32] = b;
    }
    if (v < p.vecs_per_row) dst[v] = src[v];
  }
}


// Sum of row ranges over peers: segment s produces rows [dst_start[s], +count[s]) of the local output as the fp32 sum,
// over the ranks set in peer_mask[s], of rows [src_start[s], +count[s]) of that rank's buffer (bf16, read over NVLink
// with 16-byte loads, four peers' loads in flight per lane). The fixed rank order makes the sum reproducible.
struct ReduceParams {
  const uint4* peer[PUSH_MAX_PEERS];
  uint4* out;
  const long long* seg_src_start;
  const long long* seg_dst_start;
  const int* seg_count;
  const int* seg_peer_mask;
  int world;
  int vecs_per_row;
  long long ld_src_vec, ld_dst_vec;
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__global__ void __launch_bounds__(PUSH_WARPS * 32) peer_reduce_rows_kernel(const ReduceParams p) {
  const int s = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int count = p.seg_count[s];
  const int mask = p.seg_peer_mask[s];
  int ranks[PUSH_MAX_PEERS];
  int n = 0;
  for (int r = 0; r < p.world; ++r)
    if (mask & (1 << r)) ranks[n++] = r;
  const long long src0 = p.seg_src_start[s], dst0 = p.seg_dst_start[s];
  for (int r = blockIdx.x * PUSH_WARPS + warp; r < count; r += gridDim.x * PUSH_WARPS) {
    for (int v = lane; v < p.vecs_per_row; v += 32) {
      const long long off = (src0 + r) * p.ld_src_vec + v;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      int i = 0;
      for (; i + 4 <= n; i += 4) {
        const uint4 a = p.peer[ranks[i]][off], b = p.peer[ranks[i + 1]][off];
        const uint4 c = p.peer[ranks[i + 2]][off], d = p.peer[ranks[i + 3]][off];
        add_bf16x8(acc, a);
        add_bf16x8(acc, b);
        add_bf16x8(acc, c);
        add_bf16x8(acc, d);
      }
      for (; i < n; ++i) add_bf16x8(acc, p.peer[ranks[i]][off]);
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      p.out[(dst0 + r) * p.ld_dst_vec + v] = o;
    }
  }
}

}  // namespace
}  // namespace ocb

using namespace ocb;

// src: [*, ld_src] bf16 rows of `cols` elements (cols % 8 == 0, row starts 16-byte aligned). peer_ptrs: host array of
// `world` device pointers (each rank's destination base, already offset to the half of the double buffer in use).
static int push_rows(const void* src, const int* gather_idx, int gather_div, const int* seg_src_start,
                     const int* seg_count, const int* seg_dst_rank, const long long* seg_dst_start,
                     const int* seg_src_col, const int* seg_dst_col, int num_segments, void* const* peer_ptrs, int world,
                     long long dst_capacity_rows, int cols, long long ld_src, long long ld_dst, int* status,
                     cudaStream_t stream) {
  if (num_segments <= 0) return 0;
  if (world < 1 || world > PUSH_MAX_PEERS || (cols % 8) || (ld_src % 8) || (ld_dst % 8) || gather_div < 1 || status == nullptr)
    return -5;
  PushParams p;
  p.src = static_cast<const uint4*>(src);
  p.gather_idx = gather_idx;
  p.gather_div = gather_div;
  p.seg_src_start = seg_src_start;
  p.seg_count = seg_count;
  p.seg_dst_rank = seg_dst_rank;
  p.seg_dst_start = seg_dst_start;
  p.seg_src_col = seg_src_col;
  p.seg_dst_col = seg_dst_col;
  for (int i = 0; i < PUSH_MAX_PEERS; ++i) p.peer[i] = static_cast<uint4*>(i < world ? peer_ptrs[i] : nullptr);
  p.dst_capacity_rows = dst_capacity_rows;
  p.vecs_per_row = cols / 8;
  p.ld_src_vec = ld_src / 8;
  p.ld_dst_vec = ld_dst / 8;
  p.status = status;
  moe_push_rows_kernel<<<dim3(PUSH_BLOCKS_PER_SEGMENT, num_segments), PUSH_WARPS * 32, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ocb_moe_push_rows(const void* src, const int* gather_idx, int gather_div, const int* seg_src_start,
                                 const int* seg_count, const int* seg_dst_rank, const long long* seg_dst_start,
                                 int num_segments, void* const* peer_ptrs, int world, long long dst_capacity_rows, int cols,
                                 long long ld_src, long long ld_dst, int* status, cudaStream_t stream) {
  return push_rows(src, gather_idx, gather_div, seg_src_start, seg_count, seg_dst_rank, seg_dst_start, nullptr, nullptr,
                   num_segments, peer_ptrs, world, dst_capacity_rows, cols, ld_src, ld_dst, status, stream);
}

// The same transfer for row SLICES: segment s reads `cols` elements from column seg_src_col_vec[s] * 8 of its source
// rows and writes them from column seg_dst_col_vec[s] * 8 of its destination rows (both in 16-byte vectors). This is the
// sequence <-> head exchange of Ulysses context parallelism as one kernel: a head group of every local token goes to
// the rank that owns the group (or comes back), with no packing copy on either side.
extern "C" int ocb_push_row_slices(const void* src, const int* seg_src_start, const int* seg_count, const int* seg_dst_rank,
                                   const long long* seg_dst_start, const int* seg_src_col_vec, const int* seg_dst_col_vec,
                                   int num_segments, void* const* peer_ptrs, int world, long long dst_capacity_rows,
                                   int cols, long long ld_src, long long ld_dst, int* status, cudaStream_t stream) {
  return push_rows(src, nullptr, 1, seg_src_start, seg_count, seg_dst_rank, seg_dst_start, seg_src_col_vec, seg_dst_col_vec,
                   num_segments, peer_ptrs, world, dst_capacity_rows, cols, ld_src, ld_dst, status, stream);
}

// out rows [seg_dst_start[s], +seg_count[s]) = sum over the ranks in seg_peer_mask[s] of rows [seg_src_start[s], ...) of
// peer_ptrs[rank] (bf16 rows of `cols` elements, fp32 accumulation in rank order). The caller's barrier orders this
// kernel behind the peers' writes. Used to bring key / value gradients of context-parallel attention to their owners.
extern "C" int ocb_peer_reduce_rows(void* const* peer_ptrs, int world, void* out, const long long* seg_src_start,
                                    const long long* seg_dst_start, const int* seg_count, const int* seg_peer_mask,
                                    int num_segments, int cols, long long ld_src, long long ld_dst, cudaStream_t stream) {
  if (num_segments <= 0) return 0;
  if (world < 1 || world > PUSH_MAX_PEERS || (cols % 8) || (ld_src % 8) || (ld_dst % 8)) return -5;
  ReduceParams p;
  for (int i = 0; i < PUSH_MAX_PEERS; ++i) p.peer[i] = static_cast<const uint4*>(i < world ? peer_ptrs[i] : nullptr);
  p.out = static_cast<uint4*>(out);
  p.seg_src_start = seg_src_start;
  p.seg_dst_start = seg_dst_start;
  p.seg_count = seg_count;
  p.seg_peer_mask = seg_peer_mask;
  p.world = world;
  p.vecs_per_row = cols / 8;
  p.ld_src_vec = ld_src / 8;
  p.ld_dst_vec = ld_dst / 8;
  peer_reduce_rows_kernel<<<dim3(PUSH_BLOCKS_PER_SEGMENT, num_segments), PUSH_WARPS * 32, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
