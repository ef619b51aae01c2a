// How the attention kernels find their rows when the sequence is sharded over a context-parallel group
// (role of the ring / all-gather KV exchange of src/olmo_core/nn/attention/ring.py and
// src/olmo_core/nn/attention/backend.py:446-640, done here by the kernels themselves).
//
// Queries are local: [B, Tq] rows in one or two chunks of `q_chunk_tiles` 128-row tiles; chunk c starts at global tile
// q_tile0[c] (contiguous layout: one chunk; zig-zag layout: chunks r and 2 cp - 1 - r). Keys are addressed in GLOBAL
// order, Tk per batch entry, cut into chunks of `kv_chunk_tiles` tiles; chunk c lives in source buffer kv_src[c] (this
// GPU's or a peer's [B, kv_rows_src, Hkv, D] buffer, mapped into this GPU's address space) from its tile kv_tile0[c]
// on. The kernels fetch key / value tiles from the owner's memory with plain (non-multicast) TMA loads through
// per-source tensor maps kept in global memory, so no gathered copy of K / V exists anywhere.
// Without sharding everything is one chunk of one source and q_tile0[0] = (Tk - Tq) / 128 aligns the causal diagonal
// at the end (a query sees keys up to its own global position).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace ocb {

constexpr int ATTN_MAX_KV_CHUNKS = 32;
constexpr int ATTN_MAX_SOURCES = 16;

struct AttnSeqMap {
  int Tq, Tk;
  int q_chunk_tiles;
  int q_tile0[2];
  int kv_chunk_tiles;
  int kv_rows_src;
  unsigned char kv_src[ATTN_MAX_KV_CHUNKS];
  short kv_tile0[ATTN_MAX_KV_CHUNKS];
  const CUtensorMap* kv_maps;  // [2 * n_src]: K maps, then V maps; nullptr = the kernel's own K / V map arguments
  int n_src;
};

// global tile of local query tile `lt`
__device__ __forceinline__ int attn_q_gtile(const AttnSeqMap& m, int lt) {
  return lt < m.q_chunk_tiles ? m.q_tile0[0] + lt : m.q_tile0[1] + lt - m.q_chunk_tiles;
}

// row (in the source's [B * kv_rows_src] row space) and source of global key tile `j` of batch entry `b`
__device__ __forceinline__ int attn_kv_row0(const AttnSeqMap& m, int b, int j, int& src) {
  if (m.kv_maps == nullptr) {  // unsharded: one chunk of one source, no division on the producer's path
    src = 0;
    return b * m.kv_rows_src + j * 128;
  }
  const int c = j / m.kv_chunk_tiles;
  src = m.kv_src[c];
  return b * m.kv_rows_src + (m.kv_tile0[c] + j - c * m.kv_chunk_tiles) * 128;
}

__device__ __forceinline__ const CUtensorMap* attn_k_map(const AttnSeqMap& m, const CUtensorMap* own, int src) {
  return m.kv_maps ? m.kv_maps + src : own;
}
__device__ __forceinline__ const CUtensorMap* attn_v_map(const AttnSeqMap& m, const CUtensorMap* own, int src) {
  return m.kv_maps ? m.kv_maps + m.n_src + src : own;
}

// Host side: the map of an unsharded call.
inline AttnSeqMap attn_plain_map(int Tq, int Tk) {
  AttnSeqMap m = {};
  m.Tq = Tq;
  m.Tk = Tk;
  m.q_chunk_tiles = Tq / 128;
  m.q_tile0[0] = (Tk - Tq) / 128;
  m.q_tile0[1] = 0;
  m.kv_chunk_tiles = Tk / 128;
  m.kv_rows_src = Tk;
  m.kv_maps = nullptr;
  m.n_src = 1;
  return m;
}

// Host side (attention_sm100.cu): fills `m` for a sharded call and uploads the per-source K / V tensor maps.
// `layout` = {q_chunk_tiles, q_tile0[0], q_tile0[1], kv_chunk_tiles, n_chunks, then per chunk: source, first tile}.
int attn_sharded_map(AttnSeqMap* m, int B, int Tq, int Tk, int Hkv, const void* const* k_srcs, const void* const* v_srcs,
                     int n_src, int kv_rows_src, long long ldk, long long ldv, const int* layout, cudaStream_t stream);

}  // namespace ocb
