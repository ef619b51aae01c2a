// Dense bf16 GEMM on CTA pairs (tcgen05.mma.cta_group::2): two CTAs on the two SMs of one TPC compute one
// 256 x 256 output tile together.
//
//   C[M,N] (=|+=) opA(A) * opB(B)          (same operand-major conventions as gemm_sm100.cu)
//
// Why pairs: with one CTA per tile (gemm_sm100.cu) every CTA stages a 128-row A block and a 256-row B block per
// 64-deep reduction step, 48 KB per 512 tensor-core cycles, and the kernel waits for operands for a quarter to a third
// of its time. In a pair each CTA stages its own 128 rows of A and only HALF of the B block (128 rows); the tensor
// cores of both SMs read both halves. That is 32 KB per SM for the same 512 cycles of math, and the shared memory
// that frees up holds a deeper ring (6 stages instead of 4).
//
// Roles per CTA (192 threads): warp 0 = TMA producer for this CTA's operand halves, warp 1 = TMEM owner and, in the
// pair's leader (cluster rank 0) only, the MMA issuer; warps 2..5 = epilogue for this CTA's 128 accumulator rows.
// Barriers: the "stage full" barrier of the leader counts the bytes of BOTH CTAs' loads (the follower's TMA loads
// name the leader's barrier); "stage empty" and "accumulator full" are signalled in both CTAs by two tcgen05.commit
// instructions, one per CTA; "accumulator empty" lives in the leader and counts the eight epilogue warps of the pair.
// No load in this file is a cluster broadcast: each CTA fetches its own half with a plain tiled TMA load.
// All waits are bounded (common.cuh); a wait that runs out sets the status word and the kernel drains and returns.
//
// Fused epilogues for the gated MLP (reference: src/olmo_core/nn/feed_forward.py:161-171):
//   EPI_SWIGLU_FWD  B is [w1; w3] stacked ([2H, K]); the pair tile covers 128 columns of H: the leader stages the w1
//                   rows, the follower the w3 rows, so every accumulator row holds a = x w1^T in columns 0..127 and
//                   b = x w3^T in columns 128..255. The epilogue stores a and b (for the backward pass) into
//                   C [M, 2H] and h = silu(a) * b into C2 [M, H].
//   EPI_SWIGLU_BWD  the GEMM computes dh = dy W2 ([M, H]); the epilogue reads a and b from AB [M, 2H] and stores
//                   da = dh * b * silu'(a), db = dh * silu(a) into C [M, 2H] and the recomputed h into C2 [M, H]
//                   (when C2 is given), so dh never reaches memory.

#include <mutex>

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {

bool get_tensor_map(CUtensorMap* out, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int elem_bytes);

namespace pairgemm {

constexpr int BM = 128;   // accumulator rows per CTA (the pair tile has 2 * BM rows)
constexpr int BN = 256;   // columns of the pair tile
constexpr int BNH = 128;  // B rows staged per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_STAGING_BYTES = 4 * 2 * 32 * 128;  // four epilogue warps, two 32-row x 128-byte buffers each
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;

enum : int { EPI_BF16 = 0, EPI_F32_ACC = 1, EPI_F32 = 2, EPI_BF16_ACC = 3, EPI_SWIGLU_FWD = 5, EPI_SWIGLU_BWD = 6 };

struct Params {
  void* C;
  long long ldc;
  void* C2;  // fused gated-MLP epilogues: h [M, H]
  long long ldc2;
  const void* AB;  // EPI_SWIGLU_BWD: saved a | b, [M, 2H]
  long long ldab;
  int M, N, K;  // N: columns walked by the tiles (H for the fused epilogues)
  int H;        // fused epilogues: row offset of w3 inside B and column offset of b / db inside C
  int group_m;
  int* status;
};

// ---- cluster helpers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of any CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled TMA load of a CTA pair: the destination is this CTA's shared memory, the completion bytes are counted on
// `bar_cluster_addr`, which may belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* desc, uint32_t bar_cluster_addr,
                                                 int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B with M = 256 (128 rows from each CTA's shared memory) and N = 256 (128 B rows from
// each CTA). Issued by one thread of the leader; the descriptors are shared-memory offsets valid in both CTAs.
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// `bar_cluster_addr` observes the completion of every tcgen05.mma this thread has issued so far.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gm = min(tiles_m - first_m, group_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}


// ---- epilogue staging ------------------------------------------------------------------------------------------------
constexpr int STG_BYTES = 32 * 128;  // one warp's 32 rows x 128 bytes
enum : int { ST_PLAIN = 0, ST_BF16_ADD = 1, ST_F32_ADD = 2 };

// 16-byte slot `chunk` (0..7) of staged row `row` (0..31); the XOR keeps both the row-per-thread and the
// 8-lanes-per-row access patterns free of bank conflicts.
__device__ __forceinline__ uint4* stg_slot(uint8_t* stg, int row, int chunk) {
  return reinterpret_cast<uint4*>(stg + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Moves a staged block to global memory: 8 lanes cover the 128 bytes of one row, 4 rows per instruction.
// gbase: address of (first row, first byte); valid_bytes per row may be short of 128 at the matrix edge (a multiple of
// the element size). MODE adds to what is in memory (bf16: read-modify-write; fp32: reductions performed in L2).
template <int MODE>
__device__ __forceinline__ void stg_store(uint8_t* stg, uint8_t* gbase, long long ld_bytes, int rows_valid, int valid_bytes,
                                          int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    if (rr >= rows_valid || cc * 16 >= valid_bytes) continue;
    const uint4 v = *stg_slot(stg, rr, cc);
    uint8_t* dst = gbase + rr * ld_bytes + cc * 16;
    if (cc * 16 + 16 <= valid_bytes) {
      if (MODE == ST_PLAIN) {
        *reinterpret_cast<uint4*>(dst) = v;
      } else if (MODE == ST_F32_ADD) {
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x)),
                     "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                     : "memory");
      } else {
        const uint4 old = *reinterpret_cast<const uint4*>(dst);
        const uint32_t nw[4] = {v.x, v.y, v.z, v.w}, ow[4] = {old.x, old.y, old.z, old.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16x2(nw[j]), b = unpack_bf16x2(ow[j]);
          o[j] = pack_bf16x2(a.x + b.x, a.y + b.y);
        }
        *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
      // ragged end of a row: element by element
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      if (MODE == ST_F32_ADD) {
        for (int j = 0; j < 4 && cc * 16 + 4 * j < valid_bytes; ++j) atomicAdd(reinterpret_cast<float*>(dst) + j, __uint_as_float(w[j]));
      } else {
        for (int j = 0; j < 8 && cc * 16 + 2 * j < valid_bytes; ++j) {
          // (fp32 plain stores reach here with 4-byte elements: two 2-byte halves per element, both inside valid_bytes)
          uint16_t e = (j & 1) ? static_cast<uint16_t>(w[j >> 1] >> 16) : static_cast<uint16_t>(w[j >> 1] & 0xffffu);
          if (MODE == ST_BF16_ADD) {
            const __nv_bfloat16 old = reinterpret_cast<const __nv_bfloat16*>(dst)[j];
            const __nv_bfloat16 nv = __float2bfloat16_rn(__bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&e)) + __bfloat162float(old));
            e = *reinterpret_cast<const uint16_t*>(&nv);
          }
          reinterpret_cast<uint16_t*>(dst)[j] = e;
        }
      }
    }
  }
}

// The reverse for two blocks at once (the a and b chunks of the gated-MLP backward): 32 x 128 bytes of global memory each
// into a staging buffer, zeros where the matrix ends.
__device__ __forceinline__ uint4 load_16b_edge(const uint8_t* src, int bytes_left) {
  if (bytes_left >= 16) return __ldg(reinterpret_cast<const uint4*>(src));
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  for (int j = 0; j < 8 && 2 * j < bytes_left; ++j)
    w[j >> 1] |= static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(src)[j]) << ((j & 1) * 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
// Issues the sixteen loads of a lane (a and b chunk); ab_stash moves them into the staging buffers later, so other work
// can be placed between the two.
__device__ __forceinline__ void ab_fetch(uint4 (&va)[8], uint4 (&vb)[8], const uint8_t* ga, const uint8_t* gb,
                                         long long ld_bytes, int rows_valid, int valid_bytes, int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    va[i] = make_uint4(0u, 0u, 0u, 0u);
    vb[i] = va[i];
    if (rr < rows_valid && cc * 16 < valid_bytes) {
      const long long off = rr * ld_bytes + cc * 16;
      va[i] = load_16b_edge(ga + off, valid_bytes - cc * 16);
      vb[i] = load_16b_edge(gb + off, valid_bytes - cc * 16);
    }
  }
}
__device__ __forceinline__ void ab_stash(const uint4 (&va)[8], const uint4 (&vb)[8], uint8_t* stg_a, uint8_t* stg_b, int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    *stg_slot(stg_a, rr, cc) = va[i];
    *stg_slot(stg_b, rr, cc) = vb[i];
  }
}

__device__ __forceinline__ float silu_f(float a) { return __fdividef(a, 1.f + __expf(-a)); }

template <int A_MN, int B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Params p) {
  constexpr int TILE_N = EPI == EPI_SWIGLU_FWD ? BNH : BN;  // columns of p.N one pair tile covers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EPI_STAGING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader of the pair
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers are initialised before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
        const int m0 = tm * (2 * BM) + static_cast<int>(cta) * BM;
        // B rows of this CTA: its half of the 256 columns, or (fused forward) the same 128 columns of w1 / w3
        const int n0 = EPI == EPI_SWIGLU_FWD ? tn * BNH + static_cast<int>(cta) * p.H : tn * BN + static_cast<int>(cta) * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cta == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tma_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (64 * BK * 2), &tma_a, bar, m0 + j * 64, k0);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sb, &tma_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * (64 * BK * 2), &tma_b, bar, n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? 64 * BK * 2 : 16, b_lbo = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t a_kstep = A_MN ? 2048 : 32, b_kstep = B_MN ? 2048 : 32;  // bytes per UMMA_K = 16
      constexpr uint32_t kDescHi = desc_hi_sw128(1024);
      const uint32_t a_lo0 = desc_lo_sw128(smem_u32(smem), a_lbo);
      const uint32_t b_lo0 = desc_lo_sw128(smem_u32(smem) + A_STAGE_BYTES, b_lbo);
      // the follower's barriers sit at the same offsets of its shared memory
      const uint32_t empty_peer0 = map_to_cta(smem_u32(&empty_bar[0]), 1);
      const uint32_t tfull_peer0 = map_to_cta(smem_u32(&tfull_bar[0]), 1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kStatusTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
          umma_pair(d_tmem, a_lo, b_lo, kDescHi, idesc, kb != 0);
#pragma unroll
          for (int k = 1; k < BK / 16; ++k)
            umma_pair(d_tmem, a_lo + ((k * a_kstep) >> 4), b_lo + ((k * b_kstep) >> 4), kDescHi, idesc, 1);
          // free the stage in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&empty_bar[stage]));
          umma_commit_pair(empty_peer0 + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          umma_commit_pair(smem_u32(&tfull_bar[acc]));
          umma_commit_pair(tfull_peer0 + acc * 8);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    // A thread owns one accumulator row (tcgen05.ld 32x32b). Writing rows straight to memory would make every warp
    // store touch 32 different lines, so each warp turns its 32 x 128-byte block through two staging buffers in shared
    // memory (16-byte slots, XOR-swizzled by row) and moves it to / from global memory with 8 lanes per 128-byte line.
    const int quad = warp & 3;
    uint8_t* stg0 = smem + STAGES * STAGE_BYTES + (warp - 2) * (2 * STG_BYTES);
    uint8_t* stg1 = stg0 + STG_BYTES;
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(&tempty_bar[0]), 0);
    bool ok = true;
    int it = 0;
    uint4 va[8], vb[8];  // EPI_SWIGLU_BWD: the a | b chunk requested ahead of its use
    if (EPI == EPI_SWIGLU_BWD && pair < num_tiles) {
      int tm, tn;
      tile_coords(pair, tiles_m, tiles_n, p.group_m, tm, tn);
      const int frow0 = tm * (2 * BM) + static_cast<int>(cta) * BM + quad * 32, fh0 = tn * BN;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.AB) + (static_cast<long long>(frow0) * p.ldab + fh0) * 2;
      ab_fetch(va, vb, src, src + static_cast<long long>(p.H) * 2, p.ldab * 2, min(32, p.M - frow0), min(64, p.N - fh0) * 2, lane);
    }
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
      const int row0 = tm * (2 * BM) + static_cast<int>(cta) * BM + quad * 32;  // first row of this warp
      const int rows_valid = min(32, p.M - row0);                               // <= 0: nothing to store
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      // hands the accumulator back to the MMA issuer as soon as its last column has been read into registers
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader0 + acc * 8);
      };
      if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
        const int n0 = tn * BN;
        uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(row0) * p.ldc + n0) * 2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          tmem_ld_wait();
          if (c == BN / 64 - 1) release_acc();
          const int cols_valid = min(64, p.N - (n0 + c * 64));
          if (rows_valid <= 0 || cols_valid <= 0) continue;
          uint8_t* stg = (c & 1) ? stg1 : stg0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            *stg_slot(stg, lane, v) = make_uint4(pack_bf16x2(__uint_as_float(r0[8 * v + 0]), __uint_as_float(r0[8 * v + 1])),
                                                 pack_bf16x2(__uint_as_float(r0[8 * v + 2]), __uint_as_float(r0[8 * v + 3])),
                                                 pack_bf16x2(__uint_as_float(r0[8 * v + 4]), __uint_as_float(r0[8 * v + 5])),
                                                 pack_bf16x2(__uint_as_float(r0[8 * v + 6]), __uint_as_float(r0[8 * v + 7])));
            *stg_slot(stg, lane, 4 + v) = make_uint4(pack_bf16x2(__uint_as_float(r1[8 * v + 0]), __uint_as_float(r1[8 * v + 1])),
                                                     pack_bf16x2(__uint_as_float(r1[8 * v + 2]), __uint_as_float(r1[8 * v + 3])),
                                                     pack_bf16x2(__uint_as_float(r1[8 * v + 4]), __uint_as_float(r1[8 * v + 5])),
                                                     pack_bf16x2(__uint_as_float(r1[8 * v + 6]), __uint_as_float(r1[8 * v + 7])));
          }
          __syncwarp();
          stg_store<EPI == EPI_BF16_ACC ? ST_BF16_ADD : ST_PLAIN>(stg, c_base + c * 128, p.ldc * 2, rows_valid, cols_valid * 2, lane);
          // the other buffer serves the next chunk; this one is rewritten two chunks later, after the syncwarp above
        }
        __syncwarp();
      } else if (EPI == EPI_F32 || EPI == EPI_F32_ACC) {
        const int n0 = tn * BN;
        uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(row0) * p.ldc + n0) * 4;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          if (c == BN / 32 - 1) release_acc();
          const int cols_valid = min(32, p.N - (n0 + c * 32));
          if (rows_valid <= 0 || cols_valid <= 0) continue;
          uint8_t* stg = (c & 1) ? stg1 : stg0;
#pragma unroll
          for (int v = 0; v < 8; ++v) *stg_slot(stg, lane, v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          __syncwarp();
          stg_store<EPI == EPI_F32_ACC ? ST_F32_ADD : ST_PLAIN>(stg, c_base + c * 128, p.ldc * 4, rows_valid, cols_valid * 4, lane);
        }
        __syncwarp();
      } else if (EPI == EPI_SWIGLU_FWD) {
        // accumulator columns [0,128): a for H-columns tn*128.., [128,256): b for the same columns
        const int h0 = tn * BNH;
        uint8_t* a_base = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(row0) * p.ldc + h0) * 2;
        uint8_t* b_base = a_base + static_cast<long long>(p.H) * 2;
        uint8_t* h_base = reinterpret_cast<uint8_t*>(p.C2) + (static_cast<long long>(row0) * p.ldc2 + h0) * 2;
#pragma unroll 1
        for (int c = 0; c < BNH / 64; ++c) {
          uint32_t oh[32];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t ra[32], rb[32];
            tmem_ld_32x32(t_row + c * 64 + half * 32, ra);
            tmem_ld_32x32(t_row + BNH + c * 64 + half * 32, rb);
            tmem_ld_wait();
            if (c == BNH / 64 - 1 && half == 1) release_acc();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t wa[4], wb[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                // a and b are rounded to bf16 first so that h is exactly what the backward pass recomputes from them
                wa[j] = pack_bf16x2(__uint_as_float(ra[8 * v + 2 * j]), __uint_as_float(ra[8 * v + 2 * j + 1]));
                wb[j] = pack_bf16x2(__uint_as_float(rb[8 * v + 2 * j]), __uint_as_float(rb[8 * v + 2 * j + 1]));
                const float2 fa = unpack_bf16x2(wa[j]), fb = unpack_bf16x2(wb[j]);
                oh[half * 16 + v * 4 + j] = pack_bf16x2(silu_f(fa.x) * fb.x, silu_f(fa.y) * fb.y);
              }
              *stg_slot(stg0, lane, half * 4 + v) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
              *stg_slot(stg1, lane, half * 4 + v) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
            }
          }
          const int cols_valid = min(64, p.N - (h0 + c * 64));
          const bool live = rows_valid > 0 && cols_valid > 0;
          __syncwarp();
          if (live) {
            stg_store<ST_PLAIN>(stg0, a_base + c * 128, p.ldc * 2, rows_valid, cols_valid * 2, lane);
            stg_store<ST_PLAIN>(stg1, b_base + c * 128, p.ldc * 2, rows_valid, cols_valid * 2, lane);
          }
          __syncwarp();
#pragma unroll
          for (int v = 0; v < 8; ++v) *stg_slot(stg0, lane, v) = make_uint4(oh[4 * v], oh[4 * v + 1], oh[4 * v + 2], oh[4 * v + 3]);
          __syncwarp();
          if (live) stg_store<ST_PLAIN>(stg0, h_base + c * 128, p.ldc2 * 2, rows_valid, cols_valid * 2, lane);
          __syncwarp();
        }
      } else {
        // EPI_SWIGLU_BWD: the accumulator is dh for H-columns tn*256..; a | b come from memory. Their loads do not
        // depend on the accumulator: the first chunk was requested before the wait above, and every further chunk is
        // requested before the stores of the chunk in front of it.
        const int h0 = tn * BN;
        uint8_t* da_base = reinterpret_cast<uint8_t*>(p.C) + (static_cast<long long>(row0) * p.ldc + h0) * 2;
        uint8_t* db_base = da_base + static_cast<long long>(p.H) * 2;
        uint8_t* h_base = p.C2 == nullptr ? nullptr
                                          : reinterpret_cast<uint8_t*>(p.C2) + (static_cast<long long>(row0) * p.ldc2 + h0) * 2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int cols_valid = min(64, p.N - (h0 + c * 64));
          const bool live = rows_valid > 0 && cols_valid > 0;
          ab_stash(va, vb, stg0, stg1, lane);
          uint32_t oh[32];
          __syncwarp();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t rd[32];
            tmem_ld_32x32(t_row + c * 64 + half * 32, rd);
            tmem_ld_wait();
            if (c == BN / 64 - 1 && half == 1) release_acc();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4* sa = stg_slot(stg0, lane, half * 4 + v);
              uint4* sb = stg_slot(stg1, lane, half * 4 + v);
              const uint4 xa = *sa, xb = *sb;
              const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wb[4] = {xb.x, xb.y, xb.z, xb.w};
              uint32_t oda[4], odb[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 fa = unpack_bf16x2(wa[j]), fb = unpack_bf16x2(wb[j]);
                const float d0 = __uint_as_float(rd[8 * v + 2 * j]), d1 = __uint_as_float(rd[8 * v + 2 * j + 1]);
                const float s0 = __fdividef(1.f, 1.f + __expf(-fa.x)), s1 = __fdividef(1.f, 1.f + __expf(-fa.y));
                const float si0 = fa.x * s0, si1 = fa.y * s1;  // silu(a)
                // d silu(a) / da = s (1 + a (1 - s))
                oda[j] = pack_bf16x2(d0 * fb.x * s0 * (1.f + fa.x * (1.f - s0)), d1 * fb.y * s1 * (1.f + fa.y * (1.f - s1)));
                odb[j] = pack_bf16x2(d0 * si0, d1 * si1);
                oh[half * 16 + v * 4 + j] = pack_bf16x2(si0 * fb.x, si1 * fb.y);
              }
              *sa = make_uint4(oda[0], oda[1], oda[2], oda[3]);  // in place: the slot belongs to this thread's row
              *sb = make_uint4(odb[0], odb[1], odb[2], odb[3]);
            }
          }
          __syncwarp();
          // request the next chunk (of this tile, or the first one of this CTA's next tile) before storing this one
          {
            int nrow0 = row0, nh0 = h0 + (c + 1) * 64;
            bool more = true;
            if (c == BN / 64 - 1) {
              const int ntile = tile + num_pairs;
              more = ntile < num_tiles;
              if (more) {
                int ntm, ntn;
                tile_coords(ntile, tiles_m, tiles_n, p.group_m, ntm, ntn);
                nrow0 = ntm * (2 * BM) + static_cast<int>(cta) * BM + quad * 32;
                nh0 = ntn * BN;
              }
            }
            const int nrows = more ? min(32, p.M - nrow0) : 0, ncols = min(64, p.N - nh0);
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.AB) + (static_cast<long long>(nrow0) * p.ldab + nh0) * 2;
            ab_fetch(va, vb, src, src + static_cast<long long>(p.H) * 2, p.ldab * 2, ncols > 0 ? nrows : 0, ncols * 2, lane);
          }
          if (live) {
            stg_store<ST_PLAIN>(stg0, da_base + c * 128, p.ldc * 2, rows_valid, cols_valid * 2, lane);
            stg_store<ST_PLAIN>(stg1, db_base + c * 128, p.ldc * 2, rows_valid, cols_valid * 2, lane);
          }
          __syncwarp();
          if (h_base != nullptr) {
#pragma unroll
            for (int v = 0; v < 8; ++v) *stg_slot(stg0, lane, v) = make_uint4(oh[4 * v], oh[4 * v + 1], oh[4 * v + 2], oh[4 * v + 3]);
            __syncwarp();
            if (live) stg_store<ST_PLAIN>(stg0, h_base + c * 128, p.ldc2 * 2, rows_valid, cols_valid * 2, lane);
            __syncwarp();
          }
        }
      }
    }
  }

  // Neither CTA may leave while the other can still read its shared memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

static int max_pairs(const void* kern) {
  // Number of CTA pairs that can be resident at once (a pair occupies the two SMs of one TPC).
  static std::mutex mu;
  static int cached = 0;
  std::lock_guard<std::mutex> g(mu);
  if (cached > 0) return cached;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    n = sms / 2;
  }
  cached = n;
  return cached;
}

template <int A_MN, int B_MN, int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  constexpr int TILE_N = EPI == EPI_SWIGLU_FWD ? BNH : BN;
  const long long tiles = static_cast<long long>((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + TILE_N - 1) / TILE_N);
  const int pairs_max = max_pairs(reinterpret_cast<const void*>(kern));
  const int pairs = tiles < pairs_max ? static_cast<int>(tiles) : pairs_max;
  kern<<<2 * pairs, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

static bool operand_maps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N, int K, long long lda,
                         long long ldb, int a_mn, int b_mn) {
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a_mn ? M : K), static_cast<uint64_t>(a_mn ? K : M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(a_mn ? BK : BM)};
    if (!get_tensor_map(ta, A, 2, dims, str, box, 2)) return false;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(b_mn ? N : K), static_cast<uint64_t>(b_mn ? K : N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(b_mn ? BK : BNH)};
    if (!get_tensor_map(tb, B, 2, dims, str, box, 2)) return false;
  }
  return true;
}

}  // namespace pairgemm
}  // namespace ocb

using namespace ocb;
using namespace ocb::pairgemm;

// Same contract as ocb_gemm_bf16 (gemm_sm100.cu), computed by CTA pairs.
extern "C" int ocb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int epilogue, int* status,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  CUtensorMap ta, tb;
  if (!operand_maps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn_major, b_mn_major)) return -1000;
  Params p = {};
  p.C = C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.group_m = 8;
  p.status = status;
#define OCB_PAIR_EPI(AM, BMJ)                                                      \
  switch (epilogue) {                                                              \
    case EPI_BF16: return launch<AM, BMJ, EPI_BF16>(ta, tb, p, stream);            \
    case EPI_F32_ACC: return launch<AM, BMJ, EPI_F32_ACC>(ta, tb, p, stream);      \
    case EPI_F32: return launch<AM, BMJ, EPI_F32>(ta, tb, p, stream);              \
    case EPI_BF16_ACC: return launch<AM, BMJ, EPI_BF16_ACC>(ta, tb, p, stream);    \
    default: return -1;                                                            \
  }
  if (!a_mn_major && !b_mn_major) { OCB_PAIR_EPI(0, 0) }
  if (!a_mn_major && b_mn_major) { OCB_PAIR_EPI(0, 1) }
  if (a_mn_major && b_mn_major) { OCB_PAIR_EPI(1, 1) }
  OCB_PAIR_EPI(1, 0)
#undef OCB_PAIR_EPI
}

// Gated-MLP up-projection with the activation in the epilogue: W13 = [w1; w3] ([2H, K], K-major, row stride ldw).
//   AB[M, 2H] = x W13^T  (a | b, bf16),  Hout[M, H] = silu(a) * b.
extern "C" int ocb_gemm_swiglu_fwd(const void* X, const void* W13, void* AB, void* Hout, int M, int H, int K, long long ldx,
                                   long long ldw, long long ldab, long long ldh, int* status, cudaStream_t stream) {
  if (M <= 0 || H <= 0 || K <= 0) return 0;
  if ((ldx % 8) != 0 || (ldw % 8) != 0 || (ldab % 8) != 0 || (ldh % 8) != 0 || (H % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W13) & 15) ||
      (reinterpret_cast<uintptr_t>(AB) & 15) || (reinterpret_cast<uintptr_t>(Hout) & 15))
    return -1;
  CUtensorMap ta, tb;
  if (!operand_maps(&ta, &tb, X, W13, M, 2 * H, K, ldx, ldw, 0, 0)) return -1000;
  Params p = {};
  p.C = AB;
  p.ldc = ldab;
  p.C2 = Hout;
  p.ldc2 = ldh;
  p.M = M;
  p.N = H;
  p.K = K;
  p.H = H;
  p.group_m = 8;
  p.status = status;
  return launch<0, 0, EPI_SWIGLU_FWD>(ta, tb, p, stream);
}

// Gated-MLP backward through the activation inside the dgrad GEMM of the down-projection:
//   dh = dY W2 (W2: [K, H] row-major = MN-major B), never stored;  dAB[M, 2H] = (dh b silu'(a) | dh silu(a)),
//   Hout[M, H] = silu(a) b recomputed (optional; the weight gradient of the down-projection needs it).
extern "C" int ocb_gemm_swiglu_bwd(const void* dY, const void* W2, const void* AB, void* dAB, void* Hout, int M, int H, int K,
                                   long long lddy, long long ldw, long long ldab, long long lddab, long long ldh, int* status,
                                   cudaStream_t stream) {
  if (M <= 0 || H <= 0 || K <= 0) return 0;
  if ((lddy % 8) != 0 || (ldw % 8) != 0 || (ldab % 8) != 0 || (lddab % 8) != 0 || (ldh % 8) != 0 || (H % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(dY) & 15) || (reinterpret_cast<uintptr_t>(W2) & 15) ||
      (reinterpret_cast<uintptr_t>(AB) & 15) || (reinterpret_cast<uintptr_t>(dAB) & 15) ||
      (reinterpret_cast<uintptr_t>(Hout) & 15))
    return -1;
  CUtensorMap ta, tb;
  if (!operand_maps(&ta, &tb, dY, W2, M, H, K, lddy, ldw, 0, 1)) return -1000;
  Params p = {};
  p.C = dAB;
  p.ldc = lddab;
  p.C2 = Hout;
  p.ldc2 = ldh;
  p.AB = AB;
  p.ldab = ldab;
  p.M = M;
  p.N = H;
  p.K = K;
  p.H = H;
  p.group_m = 8;
  p.status = status;
  return launch<0, 1, EPI_SWIGLU_BWD>(ta, tb, p, stream);
}
