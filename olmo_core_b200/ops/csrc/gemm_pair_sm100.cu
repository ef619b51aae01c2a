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
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
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

__device__ __forceinline__ float silu_f(float a) { return a / (1.f + __expf(-a)); }

template <int A_MN, int B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Params p) {
  constexpr bool kFused = EPI == EPI_SWIGLU_FWD || EPI == EPI_SWIGLU_BWD;
  constexpr int TILE_N = EPI == EPI_SWIGLU_FWD ? BNH : BN;  // columns of p.N one pair tile covers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
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
    const int quad = warp & 3;
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = map_to_cta(smem_u32(&tempty_bar[1]), 0);
    bool ok = true;
    int it = 0;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
      const int row = tm * (2 * BM) + static_cast<int>(cta) * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (!kFused) {
        const int n0 = tn * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col;
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
          } else {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col;
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
        }
      } else if (EPI == EPI_SWIGLU_FWD) {
        // accumulator columns [0,128): a for H-columns tn*128.., [128,256): b for the same columns
        const int h0 = tn * BNH;
        __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
        __nv_bfloat16* h_row = reinterpret_cast<__nv_bfloat16*>(p.C2) + static_cast<long long>(row) * p.ldc2;
#pragma unroll 1
        for (int c = 0; c < BNH / 16; ++c) {
          uint32_t ra[16], rb[16];
          tmem_ld_32x16(t_row + c * 16, ra);
          tmem_ld_32x16(t_row + BNH + c * 16, rb);
          tmem_ld_wait();
          const int col = h0 + c * 16;
          if (!row_ok || col >= p.N) continue;
          uint32_t oa[8], ob[8], oh[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            // a and b are rounded to bf16 first so that h is exactly what the backward pass recomputes from them
            oa[j] = pack_bf16x2(__uint_as_float(ra[2 * j]), __uint_as_float(ra[2 * j + 1]));
            ob[j] = pack_bf16x2(__uint_as_float(rb[2 * j]), __uint_as_float(rb[2 * j + 1]));
            const float2 fa = unpack_bf16x2(oa[j]), fb = unpack_bf16x2(ob[j]);
            oh[j] = pack_bf16x2(silu_f(fa.x) * fb.x, silu_f(fa.y) * fb.y);
          }
          if (col + 16 <= p.N) {
            uint4* da = reinterpret_cast<uint4*>(c_row + col);
            uint4* db = reinterpret_cast<uint4*>(c_row + p.H + col);
            uint4* dh = reinterpret_cast<uint4*>(h_row + col);
            da[0] = make_uint4(oa[0], oa[1], oa[2], oa[3]); da[1] = make_uint4(oa[4], oa[5], oa[6], oa[7]);
            db[0] = make_uint4(ob[0], ob[1], ob[2], ob[3]); db[1] = make_uint4(ob[4], ob[5], ob[6], ob[7]);
            dh[0] = make_uint4(oh[0], oh[1], oh[2], oh[3]); dh[1] = make_uint4(oh[4], oh[5], oh[6], oh[7]);
          } else {
            for (int j = 0; j < 16 && col + j < p.N; ++j) {
              const uint32_t wa = oa[j >> 1], wb = ob[j >> 1], wh = oh[j >> 1];
              const uint16_t sa16 = (j & 1) ? (wa >> 16) : (wa & 0xffffu), sb16 = (j & 1) ? (wb >> 16) : (wb & 0xffffu),
                             sh16 = (j & 1) ? (wh >> 16) : (wh & 0xffffu);
              reinterpret_cast<uint16_t*>(c_row)[col + j] = sa16;
              reinterpret_cast<uint16_t*>(c_row)[p.H + col + j] = sb16;
              reinterpret_cast<uint16_t*>(h_row)[col + j] = sh16;
            }
          }
        }
      } else {
        // EPI_SWIGLU_BWD: the accumulator is dh for H-columns tn*256..; a | b come from memory
        const int h0 = tn * BN;
        const __nv_bfloat16* ab_row = reinterpret_cast<const __nv_bfloat16*>(p.AB) + static_cast<long long>(row) * p.ldab;
        __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
        __nv_bfloat16* h_row = p.C2 == nullptr ? nullptr
                                               : reinterpret_cast<__nv_bfloat16*>(p.C2) + static_cast<long long>(row) * p.ldc2;
#pragma unroll 1
        for (int c = 0; c < BN / 16; ++c) {
          uint32_t rd[16];
          tmem_ld_32x16(t_row + c * 16, rd);
          const int col = h0 + c * 16;
          const bool live = row_ok && col < p.N;
          uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0, b0 = a0, b1 = a0;
          const bool vec = col + 16 <= p.N;
          if (live && vec) {
            a0 = __ldg(reinterpret_cast<const uint4*>(ab_row + col));
            a1 = __ldg(reinterpret_cast<const uint4*>(ab_row + col) + 1);
            b0 = __ldg(reinterpret_cast<const uint4*>(ab_row + p.H + col));
            b1 = __ldg(reinterpret_cast<const uint4*>(ab_row + p.H + col) + 1);
          }
          tmem_ld_wait();
          if (!live) continue;
          uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          if (!vec) {
            for (int j = 0; j < 16; ++j) {
              uint32_t ea = 0, eb = 0;
              if (col + j < p.N) {
                ea = reinterpret_cast<const uint16_t*>(ab_row)[col + j];
                eb = reinterpret_cast<const uint16_t*>(ab_row)[p.H + col + j];
              }
              if (j & 1) { wa[j >> 1] |= ea << 16; wb[j >> 1] |= eb << 16; }
              else { wa[j >> 1] = ea; wb[j >> 1] = eb; }
            }
          }
          uint32_t oda[8], odb[8], oh[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 fa = unpack_bf16x2(wa[j]), fb = unpack_bf16x2(wb[j]);
            const float d0 = __uint_as_float(rd[2 * j]), d1 = __uint_as_float(rd[2 * j + 1]);
            const float s0 = 1.f / (1.f + __expf(-fa.x)), s1 = 1.f / (1.f + __expf(-fa.y));
            const float si0 = fa.x * s0, si1 = fa.y * s1;  // silu(a)
            // d silu(a) / da = s (1 + a (1 - s))
            oda[j] = pack_bf16x2(d0 * fb.x * s0 * (1.f + fa.x * (1.f - s0)), d1 * fb.y * s1 * (1.f + fa.y * (1.f - s1)));
            odb[j] = pack_bf16x2(d0 * si0, d1 * si1);
            oh[j] = pack_bf16x2(si0 * fb.x, si1 * fb.y);
          }
          if (vec) {
            uint4* da = reinterpret_cast<uint4*>(c_row + col);
            uint4* db = reinterpret_cast<uint4*>(c_row + p.H + col);
            da[0] = make_uint4(oda[0], oda[1], oda[2], oda[3]); da[1] = make_uint4(oda[4], oda[5], oda[6], oda[7]);
            db[0] = make_uint4(odb[0], odb[1], odb[2], odb[3]); db[1] = make_uint4(odb[4], odb[5], odb[6], odb[7]);
            if (h_row != nullptr) {
              uint4* dh = reinterpret_cast<uint4*>(h_row + col);
              dh[0] = make_uint4(oh[0], oh[1], oh[2], oh[3]); dh[1] = make_uint4(oh[4], oh[5], oh[6], oh[7]);
            }
          } else {
            for (int j = 0; j < 16 && col + j < p.N; ++j) {
              const uint32_t xa = oda[j >> 1], xb = odb[j >> 1], xh = oh[j >> 1];
              reinterpret_cast<uint16_t*>(c_row)[col + j] = (j & 1) ? (xa >> 16) : (xa & 0xffffu);
              reinterpret_cast<uint16_t*>(c_row)[p.H + col + j] = (j & 1) ? (xb >> 16) : (xb & 0xffffu);
              if (h_row != nullptr) reinterpret_cast<uint16_t*>(h_row)[col + j] = (j & 1) ? (xh >> 16) : (xh & 0xffffu);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
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
