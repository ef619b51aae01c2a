// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) ->
// tcgen05.mma with fp32 accumulators in tensor memory -> epilogue warps (tcgen05.ld) -> global.
//
//   C[M,N] (=|+=) opA(A) * opB(B)
//
// Operand majors cover the three products a linear layer needs without any transposes in memory:
//   forward   Y  = X  * W^T   A = X  [M,K] K-major,  B = W [N,K] K-major
//   dgrad     dX = dY * W     A = dY [M,K] K-major,  B = W [K,N] stored row-major  -> MN-major
//   wgrad     dW = dY^T * X   A = dY [K,M] stored row-major -> MN-major, B = X [K,N] -> MN-major
// (replaces the cuBLAS calls behind nn.Linear in the reference: src/olmo_core/nn/feed_forward.py:161-171,
//  src/olmo_core/nn/attention/__init__.py:379-390, src/olmo_core/nn/lm_head.py:174)
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (one TMEM lane quadrant each). Tile 128 x 256 x 64, 4-stage smem ring,
// two 256-column fp32 accumulators in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
// All waits are bounded (see common.cuh).

#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;

enum : int { EPI_BF16 = 0, EPI_F32_ACC = 1, EPI_F32 = 2, EPI_BF16_ACC = 3, EPI_F32_RED_PEER = 4 };
constexpr int MAX_PEERS = 8;

struct GemmParams {
  void* C;
  long long ldc;
  int M, N, K;
  int group_m;  // rasterisation group size (in M tiles)
  int* status;
  // Grouped modes (see ocb_grouped_gemm_bf16): row prefix sums of the groups and per-group operand strides.
  const int* offsets;
  int num_groups;
  int b_group_rows;  // rows of the stacked B operand per group (outer TMA coordinate)
  int c_group_rows;  // rows of the stacked C per group (reduction-grouped mode)
  // Tensor-parallel modes: A gathered from the peers' row shards (GROUP_GATHER) and / or C reduced into the row shard of
  // its owner (EPI_F32_RED_PEER). m_local = rows per rank.
  const CUtensorMap* peer_a_maps;  // [world] tensor maps of the peers' A shards, in global memory
  float* peer_c[MAX_PEERS];        // the peers' fp32 output shards
  int world, rank, m_local;
  // 8-bit operands: elements per 128-byte line of a tile (BK for bf16, 2 * BK for e4m3) and the de-quantisation scales.
  int bk;
  const float* scale_a;  // [M] one per row of A
  const float* scale_b;  // [N] one per row of B (= output column)
  // Split of the last wave's tiles along the reduction (plain mode only): tiles >= split_first are cut into split_parts
  // parts; partial tiles go to split_ws [slot][part][BM][BN] fp32 and arrivals are counted in split_counters [slot].
  int split_first, split_parts;
  float* split_ws;
  int* split_counters;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gm = min(tiles_m - first_m, group_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

enum : int { GROUP_NONE = 0, GROUP_ROWS = 1, GROUP_REDUCTION = 2, GROUP_GATHER = 3 };

// Everything a role needs to know about one output tile.
struct TileInfo {
  int m0, n0;     // tile origin: A rows (or A columns when A is MN-major) and B columns
  int m_end;      // first row that must not be stored
  int k0;         // first reduction index
  int num_kb;     // number of BK-deep blocks of the reduction (0: the tile is all zeros)
  int k_tail;     // valid reduction rows in the last block (BK when it is full)
  int b_off;      // added to the outer coordinate of B
  int c_row_off;  // added to the output row
  int a_map;      // GROUP_GATHER: whose shard of A the tile reads
  int a_row0;     // GROUP_GATHER: first row inside that shard
  int split_parts, split_part, split_slot;  // reduction split of a last-wave tile (split_parts == 1: not split)
};

// Walks the tiles of one CTA (tile = blockIdx.x, += gridDim.x) and resolves them to coordinates. In the grouped modes the
// group boundaries live in device memory, so the mapping is computed here and not on the host.
template <int GROUPED>
struct TileWalker {
  const GemmParams& p;
  int tiles_n, tiles_m, tile;
  int g, base;  // GROUP_ROWS: current group and the index of its first tile
  __device__ TileWalker(const GemmParams& params) : p(params), g(0), base(0) {
    tiles_n = (p.N + BN - 1) / BN;
    tiles_m = (p.M + BM - 1) / BM;
    tile = blockIdx.x;
  }
  __device__ bool next(TileInfo& t) {
    t.split_parts = 1;
    t.split_part = 0;
    t.split_slot = 0;
    if (GROUPED == GROUP_NONE || GROUPED == GROUP_GATHER) {
      // `tile` walks work units: whole tiles below split_first, then split_parts units per remaining tile
      int out_tile = tile, part = 0;
      const bool in_split = GROUPED == GROUP_NONE && p.split_parts > 1 && tile >= p.split_first;
      if (in_split) {
        out_tile = p.split_first + (tile - p.split_first) / p.split_parts;
        part = (tile - p.split_first) % p.split_parts;
      }
      if (out_tile >= tiles_m * tiles_n) return false;
      int tm, tn;
      tile_coords(out_tile, tiles_m, tiles_n, p.group_m, tm, tn);
      if (p.world > 1) {
        // Every rank starts at a different row shard (its own when gathering, its neighbour's when scattering), so that
        // at any moment the ranks pull from / push to different peers.
        const int per_shard = p.m_local / BM;
        const int shift = (GROUPED == GROUP_GATHER ? p.rank : p.rank + 1) * per_shard;
        tm = (tm + shift) % tiles_m;
      }
      if (GROUPED == GROUP_GATHER) {
        t.a_map = (tm * BM) / p.m_local;
        t.a_row0 = tm * BM - t.a_map * p.m_local;
      }
      t.m0 = tm * BM; t.n0 = tn * BN; t.m_end = p.M; t.k0 = 0;
      t.num_kb = (p.K + p.bk - 1) / p.bk; t.k_tail = BK; t.b_off = 0; t.c_row_off = 0;
      if (in_split) {
        const int per_part = (t.num_kb + p.split_parts - 1) / p.split_parts;  // the host keeps every part non-empty
        const int kb0 = part * per_part;
        t.k0 = kb0 * p.bk;
        t.num_kb = min(per_part, t.num_kb - kb0);
        t.split_parts = p.split_parts;
        t.split_part = part;
        t.split_slot = out_tile - p.split_first;
      }
    } else if (GROUPED == GROUP_ROWS) {
      int lo, rows, tm_g;
      while (true) {
        if (g >= p.num_groups) return false;
        lo = p.offsets[g];
        rows = p.offsets[g + 1] - lo;
        tm_g = (rows + BM - 1) / BM;
        if (tile < base + tm_g * tiles_n) break;
        base += tm_g * tiles_n;
        ++g;
      }
      const int local = tile - base;
      t.m0 = lo + (local % tm_g) * BM; t.n0 = (local / tm_g) * BN; t.m_end = lo + rows; t.k0 = 0;
      t.num_kb = (p.K + p.bk - 1) / p.bk; t.k_tail = BK; t.b_off = g * p.b_group_rows; t.c_row_off = 0;
    } else {
      const int per_group = tiles_m * tiles_n;
      if (tile >= per_group * p.num_groups) return false;
      const int grp = tile / per_group, local = tile - grp * per_group;
      const int lo = p.offsets[grp], rows = p.offsets[grp + 1] - lo;
      t.m0 = (local % tiles_m) * BM; t.n0 = (local / tiles_m) * BN; t.m_end = p.M; t.k0 = lo;
      t.num_kb = (rows + BK - 1) / BK; t.k_tail = rows - (t.num_kb - 1) * BK; t.b_off = 0;
      t.c_row_off = grp * p.c_group_rows;
    }
    tile += gridDim.x;
    return true;
  }
};

template <int A_MN, int B_MN, int EPI, int GROUPED, int FP8>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* split_flag = abort_flag + 1;  // epilogue warps: "this CTA completes a split tile"

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileWalker<GROUPED> walker(p);
      TileInfo t;
      while (ok && walker.next(t)) {
        const int m0 = t.m0, n0 = t.n0;
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = t.k0 + kb * p.bk;  // in elements: 64 two-byte or 128 one-byte elements fill the 128-byte line
          // The innermost TMA coordinate is k0 for K-major operands (a multiple of 64 there: k0 starts at 0) and
          // m0 / n0 for MN-major ones (multiples of 64); the group offsets only ever enter an OUTER coordinate.
          if (GROUPED == GROUP_GATHER) {
            // A tile of a peer's shard, read straight from that GPU's memory (a plain TMA load, no multicast).
            tma_load_2d(sa, &p.peer_a_maps[t.a_map], &full_bar[stage], k0, t.a_row0);
          } else if (A_MN == 0) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (64 * BK * 2), &tma_a, &full_bar[stage], m0 + j * 64, k0);
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], k0, t.b_off + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tma_b, &full_bar[stage], n0 + j * 64, t.b_off + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA's shared memory goes away.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // In the reduction-grouped mode the whole warp runs the loop (all lanes help to blank the ragged tail of a group);
    // otherwise only the issuing lane does.
    if (lane == 0 || GROUPED == GROUP_REDUCTION) {
      constexpr uint32_t idesc = FP8 ? make_idesc_e4m3(BM, BN) : make_idesc_bf16(BM, BN, A_MN, B_MN);
      // K-major: rows are 128 B apart inside an 8-row swizzle atom, atoms 1024 B apart (SBO); LBO unused (=1).
      // MN-major: 64-element column chunks are one [64 x BK] TMA box apart (LBO); 8 k-rows = 1024 B (SBO).
      constexpr uint32_t a_lbo = A_MN ? 64 * BK * 2 : 16, b_lbo = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t a_kstep = A_MN ? 2048 : 32, b_kstep = B_MN ? 2048 : 32;  // bytes per UMMA_K = 16
      constexpr uint32_t kDescHi = desc_hi_sw128(1024);
      const uint32_t a_lo0 = desc_lo_sw128(smem_u32(smem), a_lbo);
      const uint32_t b_lo0 = desc_lo_sw128(smem_u32(smem) + A_STAGE_BYTES, b_lbo);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      TileWalker<GROUPED> walker(p);
      TileInfo t;
      for (; ok && walker.next(t); ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, kStatusTimeoutMma);
        if (GROUPED == GROUP_REDUCTION) ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.num_kb; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kStatusTimeoutMma);
          if (GROUPED == GROUP_REDUCTION) ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          if (GROUPED == GROUP_REDUCTION && A_MN == 1 && kb == t.num_kb - 1 && t.k_tail < BK) {
            // The last block reaches into the next group's rows (or, past the last group, into rows nobody wrote). A
            // reduction row is one 128-byte line of each [BK x 64] box (the swizzle only permutes within a line), so
            // blanking the lines [k_tail, BK) of BOTH operands makes those rows contribute exactly zero; blanking only
            // one side would still let a NaN or infinity on the other side through (0 x NaN).
            const int first = t.k_tail * 8, count = (BK - t.k_tail) * 8;  // in 16-byte units
            uint8_t* sa_ptr = smem + stage * STAGE_BYTES;
#pragma unroll
            for (int j = 0; j < (BM + BN) / 64; ++j) {  // the A boxes, then (B_MN == 1 in this mode) the B boxes
              uint4* box = reinterpret_cast<uint4*>(sa_ptr + j * (64 * BK * 2)) + first;
              for (int i = lane; i < count; i += 32) box[i] = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            // descriptor low words of this stage: the stage offset and the k-step land in the start-address field
            const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
            umma_ss_lean<FP8 ? 1 : 0>(d_tmem, a_lo, b_lo, kDescHi, idesc, kb != 0);
#pragma unroll
            for (int k = 1; k < BK / 16; ++k)
              umma_ss_lean<FP8 ? 1 : 0>(d_tmem, a_lo + ((k * a_kstep) >> 4), b_lo + ((k * b_kstep) >> 4), kDescHi, idesc, 1);
            umma_commit(&empty_bar[stage]);
          }
          if (GROUPED == GROUP_REDUCTION) __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok && lane == 0) {
          if (t.num_kb > 0) umma_commit(&tfull_bar[acc]);
          else mbar_arrive(&tfull_bar[acc]);  // nothing was issued for a group without rows
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    bool ok = true;
    int it = 0;
    TileWalker<GROUPED> walker(p);
    TileInfo t;
    for (; ok && walker.next(t); ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row_in = t.m0 + quad * 32 + lane;
      const long long row = static_cast<long long>(t.c_row_off) + row_in;
      const int n0 = t.n0;
      const bool row_ok = row_in < t.m_end;
      const bool empty = t.num_kb == 0;  // a group without rows: the accumulator was never written
      // Writes 32 consecutive output columns of this thread's row: chunk c of the tile, values in r.
      auto store_chunk = [&](uint32_t(&r)[32], int c) {
        const int col = n0 + c * 32;
        if (!row_ok || col >= p.N) return;
        if (FP8) {
          // De-quantise: the operands were scaled per row of A and per row of B (per output column).
          const float sa = p.scale_a[row_in];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float sb = col + j < p.N ? p.scale_b[col + j] : 0.f;
            r[j] = __float_as_uint(__uint_as_float(r[j]) * sa * sb);
          }
        }
        if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
          if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              if (EPI == EPI_BF16_ACC) {
                const uint4 old = reinterpret_cast<const uint4*>(dst)[v];
                const float2 a0 = unpack_bf16x2(old.x), a1 = unpack_bf16x2(old.y), a2 = unpack_bf16x2(old.z),
                             a3 = unpack_bf16x2(old.w);
                o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]) + a0.x, __uint_as_float(r[8 * v + 1]) + a0.y);
                o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) + a1.x, __uint_as_float(r[8 * v + 3]) + a1.y);
                o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) + a2.x, __uint_as_float(r[8 * v + 5]) + a2.y);
                o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) + a3.x, __uint_as_float(r[8 * v + 7]) + a3.y);
              } else {
                o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              }
              reinterpret_cast<uint4*>(dst)[v] = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                float v = __uint_as_float(r[j]);
                if (EPI == EPI_BF16_ACC) v += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16_rn(v);
              }
            }
          }
        } else if (EPI == EPI_F32_RED_PEER) {
          // The row belongs to the shard of rank `owner`: add the partial product into that GPU's buffer with fire-and-
          // forget fp32 reductions over NVLink (no reply is awaited, so the next tile's loads are not held up).
          const int owner = row_in / p.m_local;
          float* dst = p.peer_c[owner] + static_cast<long long>(row_in - owner * p.m_local) * p.ldc + col;
          if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * v),
                           "f"(__uint_as_float(r[4 * v + 0])), "f"(__uint_as_float(r[4 * v + 1])),
                           "f"(__uint_as_float(r[4 * v + 2])), "f"(__uint_as_float(r[4 * v + 3]))
                           : "memory");
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(dst + j), "f"(__uint_as_float(r[j])) : "memory");
              }
            }
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
          if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 o = make_float4(__uint_as_float(r[4 * v + 0]), __uint_as_float(r[4 * v + 1]),
                                     __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              if (EPI == EPI_F32_ACC) {
                const float4 old = reinterpret_cast<const float4*>(dst)[v];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              reinterpret_cast<float4*>(dst)[v] = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                float v = __uint_as_float(r[j]);
                if (EPI == EPI_F32_ACC) v += dst[j];
                dst[j] = v;
              }
            }
          }
        }
      };
      // A tile of the last, partly filled wave may be split along the reduction over several CTAs (t.split_parts > 1):
      // each part leaves its fp32 partial tile in the workspace, and the part that arrives last adds them up in part
      // order and runs the epilogue. Nobody waits for anybody, and the order of the additions is fixed.
      const bool split = t.split_parts > 1;
      float* ws_row = nullptr;
      if (split) {
        ws_row = p.split_ws + (static_cast<long long>(t.split_slot) * t.split_parts + t.split_part) * (BM * BN) +
                 (quad * 32 + lane) * BN;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (GROUPED == GROUP_REDUCTION && empty) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (split) {
          uint4* dst = reinterpret_cast<uint4*>(ws_row + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v) dst[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        } else {
          store_chunk(r, c);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (split) {
        __threadfence();  // this thread's partials are visible device-wide before the arrival is counted
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const int before = atomicAdd(&p.split_counters[t.split_slot], 1);
          *split_flag = (before == t.split_parts - 1) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = *split_flag != 0;
        if (last) {
          __threadfence();
          const float* base = p.split_ws + static_cast<long long>(t.split_slot) * t.split_parts * (BM * BN) +
                              (quad * 32 + lane) * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
            for (int q = 0; q < t.split_parts; ++q) {
              const float4* src = reinterpret_cast<const float4*>(base + static_cast<long long>(q) * (BM * BN) + c * 32);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                const float4 x = __ldcg(src + v);
                r[4 * v + 0] = __float_as_uint(__uint_as_float(r[4 * v + 0]) + x.x);
                r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + x.y);
                r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + x.z);
                r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + x.w);
              }
            }
            store_chunk(r, c);
          }
          if (warp == 2 && lane == 0) p.split_counters[t.split_slot] = 0;  // ready for the next launch on this stream
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// Host side: tensor-map construction (cached) and launch.
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

static thread_local int g_last_tmap_error = 0;

struct TmapKey {
  const void* ptr;
  uint64_t d0, d1, d2, stride1, stride2;
  uint32_t b0, b1, b2;
  uint32_t dtype;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && stride1 == o.stride1 && stride2 == o.stride2 &&
           b0 == o.b0 && b1 == o.b1 && b2 == o.b2 && dtype == o.dtype;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.stride1); mix(k.stride2); mix(k.b0); mix(k.b1); mix(k.b2); mix(k.dtype);
    return h;
  }
};

// Builds (or fetches) a tiled tensor map with 128-byte swizzle. rank 2 or 3; inner box must span 128 bytes.
bool get_tensor_map(CUtensorMap* out, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int elem_bytes) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{ptr, dims[0], dims[1], rank > 2 ? dims[2] : 1, strides_bytes[0], rank > 2 ? strides_bytes[1] : 0,
              box[0], box[1], rank > 2 ? box[2] : 1, static_cast<uint32_t>(elem_bytes)};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t gdim[3] = {dims[0], dims[1], rank > 2 ? dims[2] : 1};
  cuuint64_t gstr[2] = {strides_bytes[0], rank > 2 ? strides_bytes[1] : 0};
  cuuint32_t bdim[3] = {box[0], box[1], rank > 2 ? box[2] : 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
  CUresult r = enc(out, dt, rank, const_cast<void*>(ptr), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    // A thread that has not touched the runtime yet (e.g. an autograd worker) may have no context bound.
    cudaFree(nullptr);
    r = enc(out, dt, rank, const_cast<void*>(ptr), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  g_last_tmap_error = static_cast<int>(r);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return true;
}

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Workspace of the last-wave reduction split, one per stream (GEMMs on different streams may run at the same time):
// num_sms partial tiles of BM x BN fp32 and as many arrival counters (zero between launches).
struct SplitWorkspace {
  float* tiles = nullptr;
  int* counters = nullptr;
};

static bool split_workspace(cudaStream_t stream, SplitWorkspace* out) {
  static std::mutex mu;
  static std::unordered_map<cudaStream_t, SplitWorkspace> per_stream;
  std::lock_guard<std::mutex> g(mu);
  auto it = per_stream.find(stream);
  if (it == per_stream.end()) {
    if (per_stream.size() >= 8) return false;  // unusual: many streams issue GEMMs; those run without the split
    SplitWorkspace w;
    const size_t n = static_cast<size_t>(num_sms());
    if (cudaMalloc(&w.tiles, n * BM * BN * sizeof(float)) != cudaSuccess) return false;
    if (cudaMalloc(&w.counters, n * sizeof(int)) != cudaSuccess || cudaMemset(w.counters, 0, n * sizeof(int)) != cudaSuccess) {
      cudaFree(w.tiles);
      return false;
    }
    it = per_stream.emplace(stream, w).first;
  }
  *out = it->second;
  return true;
}

static bool split_enabled() {
  static const bool on = [] {
    const char* v = getenv("OCB_GEMM_SPLIT_LAST_WAVE");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <int A_MN, int B_MN, int EPI, int GROUPED = GROUP_NONE, int FP8 = 0>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p_in, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI, GROUPED, FP8>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  GemmParams p = p_in;
  p.split_first = 0;
  p.split_parts = 1;
  p.split_ws = nullptr;
  p.split_counters = nullptr;
  // Upper bound of the tile count (the exact count of the row-grouped mode depends on device data: every group may
  // add one partly filled row of tiles).
  long long tiles_m = (p.M + BM - 1) / BM;
  if (GROUPED == GROUP_ROWS) tiles_m += p.num_groups;
  if (GROUPED == GROUP_REDUCTION) tiles_m *= p.num_groups;
  long long units = tiles_m * ((p.N + BN - 1) / BN);
  const int sms = num_sms();
  if (GROUPED == GROUP_NONE && EPI != EPI_F32_RED_PEER && p.world == 1 && split_enabled()) {
    // The persistent grid runs floor(tiles / SMs) full waves and then a wave that fills only `rest` SMs. When that wave
    // is at most half full, its tiles are cut along the reduction so that it keeps (nearly) all SMs busy for a fraction
    // of a tile's time.
    const int full = static_cast<int>(units / sms), rest = static_cast<int>(units % sms);
    const int num_kb = (p.K + p.bk - 1) / p.bk;
    if (full >= 1 && rest > 0 && 2 * rest <= sms) {
      int parts = sms / rest;
      if (parts > 4) parts = 4;
      while (parts > 1 && (num_kb / parts < 8 || (parts - 1) * ((num_kb + parts - 1) / parts) >= num_kb)) --parts;
      SplitWorkspace w;
      if (parts > 1 && split_workspace(stream, &w)) {
        p.split_first = full * sms;
        p.split_parts = parts;
        p.split_ws = w.tiles;
        p.split_counters = w.counters;
        units = static_cast<long long>(full) * sms + static_cast<long long>(rest) * parts;
      }
    }
  }
  const int grid = units < sms ? static_cast<int>(units) : sms;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ocb

using namespace ocb;

extern "C" int ocb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int epilogue, int* status,
                                  cudaStream_t stream);

// Which kernel serves ocb_gemm_bf16: 1 = CTA pairs (gemm_pair_sm100.cu) whenever the problem fills at least one wave of
// 256 x 256 pair tiles, 0 = always the one-CTA-per-tile kernel of this file. Initial value from OCB_GEMM_PAIR (default 1).
static int g_pair_mode = [] {
  const char* v = getenv("OCB_GEMM_PAIR");
  return (v == nullptr || v[0] != '0') ? 1 : 0;
}();
extern "C" int ocb_gemm_set_pair_mode(int mode) {
  const int old = g_pair_mode;
  g_pair_mode = mode ? 1 : 0;
  return old;
}

// Returns 0 on success, negative on a host-side failure (bad argument, tensor-map error, launch error).
extern "C" int ocb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, int a_mn_major, int b_mn_major, int epilogue, int* status,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // the pair kernel moves its output in 16-byte pieces
  const long long c_elem = (epilogue == EPI_BF16 || epilogue == EPI_BF16_ACC) ? 2 : 4;
  if (g_pair_mode && epilogue <= EPI_BF16_ACC && (ldc * c_elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) >= num_sms() / 2)
    return ocb_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, epilogue, status, stream);
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  CUtensorMap ta, tb;
  {
    // Stored layout of A: K-major -> [M rows, K inner]; MN-major -> [K rows, M inner].
    uint64_t dims[2] = {static_cast<uint64_t>(a_mn_major ? M : K), static_cast<uint64_t>(a_mn_major ? K : M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(a_mn_major ? BK : BM)};
    if (!get_tensor_map(&ta, A, 2, dims, str, box, 2)) return -(1000 + g_last_tmap_error);
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(b_mn_major ? N : K), static_cast<uint64_t>(b_mn_major ? K : N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(b_mn_major ? BK : BN)};
    if (!get_tensor_map(&tb, B, 2, dims, str, box, 2)) return -(2000 + g_last_tmap_error);
  }
  GemmParams p;
  p.C = C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.group_m = 8;
  p.bk = BK;
  p.scale_a = nullptr;
  p.scale_b = nullptr;
  p.status = status;
  p.offsets = nullptr;
  p.num_groups = 0;
  p.b_group_rows = 0;
  p.c_group_rows = 0;
  p.peer_a_maps = nullptr;
  p.world = 1;
  p.rank = 0;
  p.m_local = M;

#define OCB_DISPATCH_EPI(AM, BMJ)                                                       \
  switch (epilogue) {                                                                   \
    case EPI_BF16: return launch_gemm<AM, BMJ, EPI_BF16>(ta, tb, p, stream);            \
    case EPI_F32_ACC: return launch_gemm<AM, BMJ, EPI_F32_ACC>(ta, tb, p, stream);      \
    case EPI_F32: return launch_gemm<AM, BMJ, EPI_F32>(ta, tb, p, stream);              \
    case EPI_BF16_ACC: return launch_gemm<AM, BMJ, EPI_BF16_ACC>(ta, tb, p, stream);    \
    default: return -1;                                                                 \
  }
  if (!a_mn_major && !b_mn_major) { OCB_DISPATCH_EPI(0, 0) }
  if (!a_mn_major && b_mn_major) { OCB_DISPATCH_EPI(0, 1) }
  if (a_mn_major && b_mn_major) { OCB_DISPATCH_EPI(1, 1) }
  OCB_DISPATCH_EPI(1, 0)
#undef OCB_DISPATCH_EPI
}

// Grouped GEMM over rows sorted by group (the experts of a mixture-of-experts layer), one launch for all groups.
// offsets: int32 [num_groups + 1] DEVICE array of row prefix sums (offsets[0] = 0, offsets[G] <= total_rows); it is read
// by the kernel, so no host synchronisation is needed to know the group sizes.
//   mode 1, rows grouped:       C[r, :N] = A[r, :K] * op(B_g) for the rows r of group g.
//       A: [total_rows, K] K-major. B: the G operands stacked along the outer dimension, K-major ([G*N, K], y = x W^T)
//       or MN-major ([G*K, N], y = x W). C: [total_rows, N].
//   mode 2, reduction grouped:  C_g[M, N] (=|+=) A[rows of g, :M]^T * B[rows of g, :N]   (weight gradients)
//       A: [total_rows, M] and B: [total_rows, N], both MN-major. C: [G*M, N].
// epilogue as in ocb_gemm_bf16. Groups without rows produce zeros (mode 2) or nothing (mode 1).
extern "C" int ocb_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* offsets, int num_groups, int mode,
                                     int total_rows, int M, int N, int K, long long lda, long long ldb, long long ldc,
                                     int b_mn_major, int epilogue, int* status, cudaStream_t stream) {
  if (num_groups <= 0 || total_rows <= 0 || N <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  if (mode != GROUP_ROWS && mode != GROUP_REDUCTION) return -1;
  CUtensorMap ta, tb;
  GemmParams p;
  p.C = C;
  p.ldc = ldc;
  p.N = N;
  p.group_m = 8;
  p.bk = BK;
  p.scale_a = nullptr;
  p.scale_b = nullptr;
  p.status = status;
  p.offsets = offsets;
  p.num_groups = num_groups;
  p.b_group_rows = 0;
  p.c_group_rows = 0;
  p.peer_a_maps = nullptr;
  p.world = 1;
  p.rank = 0;
  p.m_local = 0;
  if (mode == GROUP_ROWS) {
    if (K <= 0) return 0;
    p.M = total_rows;
    p.K = K;
    p.b_group_rows = b_mn_major ? K : N;
    uint64_t adims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(total_rows)};
    uint64_t astr[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t abox[2] = {64, static_cast<uint32_t>(BM)};
    if (!get_tensor_map(&ta, A, 2, adims, astr, abox, 2)) return -(1000 + g_last_tmap_error);
    uint64_t bdims[2] = {static_cast<uint64_t>(b_mn_major ? N : K),
                         static_cast<uint64_t>(num_groups) * static_cast<uint64_t>(b_mn_major ? K : N)};
    uint64_t bstr[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t bbox[2] = {64, static_cast<uint32_t>(b_mn_major ? BK : BN)};
    if (!get_tensor_map(&tb, B, 2, bdims, bstr, bbox, 2)) return -(2000 + g_last_tmap_error);
    if (epilogue != EPI_BF16) return -1;
    return b_mn_major ? launch_gemm<0, 1, EPI_BF16, GROUP_ROWS>(ta, tb, p, stream)
                      : launch_gemm<0, 0, EPI_BF16, GROUP_ROWS>(ta, tb, p, stream);
  }
  if (M <= 0) return 0;
  p.M = M;
  p.K = total_rows;
  p.c_group_rows = M;
  uint64_t adims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(total_rows)};
  uint64_t astr[1] = {static_cast<uint64_t>(lda) * 2};
  uint32_t abox[2] = {64, static_cast<uint32_t>(BK)};
  if (!get_tensor_map(&ta, A, 2, adims, astr, abox, 2)) return -(1000 + g_last_tmap_error);
  uint64_t bdims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(total_rows)};
  uint64_t bstr[1] = {static_cast<uint64_t>(ldb) * 2};
  uint32_t bbox[2] = {64, static_cast<uint32_t>(BK)};
  if (!get_tensor_map(&tb, B, 2, bdims, bstr, bbox, 2)) return -(2000 + g_last_tmap_error);
  switch (epilogue) {
    case EPI_F32_ACC: return launch_gemm<1, 1, EPI_F32_ACC, GROUP_REDUCTION>(ta, tb, p, stream);
    case EPI_F32: return launch_gemm<1, 1, EPI_F32, GROUP_REDUCTION>(ta, tb, p, stream);
    case EPI_BF16: return launch_gemm<1, 1, EPI_BF16, GROUP_REDUCTION>(ta, tb, p, stream);
    default: return -1;
  }
}

// Device copies of the per-peer tensor maps of ocb_gemm_bf16_tp: a ring of slots, one per call. A slot is rewritten only
// after 64 further calls, and the copy into it is ordered on the caller's stream behind the kernels that read it.
static CUtensorMap* peer_map_slot(const CUtensorMap* host_maps, int world, cudaStream_t stream) {
  constexpr int kSlots = 64;
  static CUtensorMap* ring = nullptr;
  static int next = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  if (ring == nullptr && cudaMalloc(&ring, sizeof(CUtensorMap) * MAX_PEERS * kSlots) != cudaSuccess) return nullptr;
  CUtensorMap* slot = ring + static_cast<size_t>(next) * MAX_PEERS;
  next = (next + 1) % kSlots;
  if (cudaMemcpyAsync(slot, host_maps, sizeof(CUtensorMap) * world, cudaMemcpyHostToDevice, stream) != cudaSuccess)
    return nullptr;
  return slot;
}

// Tensor-parallel GEMMs that move their operand / result over NVLink from inside the kernel, tile by tile.
//   gather_a != 0 (all-gather -> GEMM):  C[world*m_local, N] = [A_0; ...; A_{world-1}] * op(B), where A_r ([m_local, K],
//       K-major, row stride lda) lives on rank r: a_ptrs[r] is its address as mapped on this GPU. Every tile loads its
//       A block straight from the owner's memory with a plain (non-multicast) TMA load. C is local (epilogue bf16/fp32).
//   scatter_c != 0 (GEMM -> reduce-scatter):  A ([world*m_local, K] local, K-major) * op(B) is a partial sum; rows
//       [r*m_local, (r+1)*m_local) are added into c_ptrs[r] (fp32 [m_local, N], row stride ldc, zeroed by the owner
//       beforehand) with vector reductions over NVLink. The sum is complete after a barrier across the ranks.
// m_local must be a multiple of 128. The callers order these kernels against the peers with their own barriers.
extern "C" int ocb_gemm_bf16_tp(const void* const* a_ptrs, const void* B, void* const* c_ptrs, int m_local, int N, int K,
                                long long lda, long long ldb, long long ldc, int world, int rank, int gather_a,
                                int scatter_c, int b_mn_major, int epilogue, int* status, cudaStream_t stream) {
  if (m_local <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || (m_local % BM) != 0) return -1;
  if (gather_a == scatter_c) return -1;  // exactly one of the two fusions per call
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
  const int M = world * m_local;
  GemmParams p;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.group_m = 8;
  p.bk = BK;
  p.scale_a = nullptr;
  p.scale_b = nullptr;
  p.status = status;
  p.offsets = nullptr;
  p.num_groups = 0;
  p.b_group_rows = 0;
  p.c_group_rows = 0;
  p.peer_a_maps = nullptr;
  p.world = world;
  p.rank = rank;
  p.m_local = m_local;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(b_mn_major ? N : K), static_cast<uint64_t>(b_mn_major ? K : N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(b_mn_major ? BK : BN)};
    if (!get_tensor_map(&tb, B, 2, dims, str, box, 2)) return -(2000 + g_last_tmap_error);
  }
  if (gather_a) {
    CUtensorMap maps[MAX_PEERS];
    for (int r = 0; r < world; ++r) {
      if (reinterpret_cast<uintptr_t>(a_ptrs[r]) & 15) return -1;
      uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(m_local)};
      uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
      uint32_t box[2] = {64, static_cast<uint32_t>(BM)};
      if (!get_tensor_map(&maps[r], a_ptrs[r], 2, dims, str, box, 2)) return -(1000 + g_last_tmap_error);
    }
    ta = maps[rank];
    p.peer_a_maps = peer_map_slot(maps, world, stream);
    if (p.peer_a_maps == nullptr) return -3;
    p.C = c_ptrs[0];
    if (b_mn_major) {
      switch (epilogue) {
        case EPI_BF16: return launch_gemm<0, 1, EPI_BF16, GROUP_GATHER>(ta, tb, p, stream);
        case EPI_F32: return launch_gemm<0, 1, EPI_F32, GROUP_GATHER>(ta, tb, p, stream);
        default: return -1;
      }
    }
    switch (epilogue) {
      case EPI_BF16: return launch_gemm<0, 0, EPI_BF16, GROUP_GATHER>(ta, tb, p, stream);
      case EPI_F32: return launch_gemm<0, 0, EPI_F32, GROUP_GATHER>(ta, tb, p, stream);
      default: return -1;
    }
  }
  if (reinterpret_cast<uintptr_t>(a_ptrs[0]) & 15) return -1;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(BM)};
    if (!get_tensor_map(&ta, a_ptrs[0], 2, dims, str, box, 2)) return -(1000 + g_last_tmap_error);
  }
  p.C = nullptr;
  for (int r = 0; r < world; ++r) p.peer_c[r] = static_cast<float*>(c_ptrs[r]);
  return b_mn_major ? launch_gemm<0, 1, EPI_F32_RED_PEER, GROUP_NONE>(ta, tb, p, stream)
                    : launch_gemm<0, 0, EPI_F32_RED_PEER, GROUP_NONE>(ta, tb, p, stream);
}

// C[M, N] = (A_q * B_q^T) .* (scale_a[m] * scale_b[n]) with e4m3 operands on the tensor cores (kind::f8f6f4) and fp32
// accumulation. A_q: [M, K], B_q: [N, K], both K-major bytes with row strides lda / ldb (multiples of 16); K % 16 == 0.
// epilogue: 0 = bf16 store, 1 = fp32 accumulate, 2 = fp32 store.
extern "C" int ocb_gemm_fp8(const void* A, const void* B, void* C, const float* scale_a, const float* scale_b, int M, int N,
                            int K, long long lda, long long ldb, long long ldc, int epilogue, int* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  if (scale_a == nullptr || scale_b == nullptr) return -1;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda)};
    uint32_t box[2] = {128, static_cast<uint32_t>(BM)};
    if (!get_tensor_map(&ta, A, 2, dims, str, box, 1)) return -(1000 + g_last_tmap_error);
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb)};
    uint32_t box[2] = {128, static_cast<uint32_t>(BN)};
    if (!get_tensor_map(&tb, B, 2, dims, str, box, 1)) return -(2000 + g_last_tmap_error);
  }
  GemmParams p;
  p.C = C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.group_m = 8;
  p.bk = 2 * BK;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.status = status;
  p.offsets = nullptr;
  p.num_groups = 0;
  p.b_group_rows = 0;
  p.c_group_rows = 0;
  p.peer_a_maps = nullptr;
  p.world = 1;
  p.rank = 0;
  p.m_local = M;
  switch (epilogue) {
    case EPI_BF16: return launch_gemm<0, 0, EPI_BF16, GROUP_NONE, 1>(ta, tb, p, stream);
    case EPI_F32_ACC: return launch_gemm<0, 0, EPI_F32_ACC, GROUP_NONE, 1>(ta, tb, p, stream);
    case EPI_F32: return launch_gemm<0, 0, EPI_F32, GROUP_NONE, 1>(ta, tb, p, stream);
    default: return -1;
  }
}
