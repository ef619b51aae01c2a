// Flash attention backward for sm_100a (tcgen05 / TMEM / TMA), head_dim 128, 128-row tiles.
//
// Math (per head; P = softmax(scale * Q K^T + mask), O = P V, delta_i = sum_d O_id dO_id):
//     dV = P^T dO            dP = dO V^T            dS = P o (dP - delta) * scale
//     dK = dS^T Q            dQ = dS K
// as in the reference's flash backends (src/olmo_core/nn/attention/backend.py) -- P is recomputed from Q, K and the
// saved log-sum-exp instead of being stored.
//
// Three launches, none of which needs atomics or a cross-CTA reduction:
//   1. attn_delta_kernel : delta = rowsum(O o dO)                                  (memory bound)
//   2. attn_dkdv_kernel  : one CTA per (K/V tile, kv head, batch) walks the query tiles (and the query heads of its
//      group); S and dP are tcgen05.mma results in TMEM, the softmax warps turn them into bf16 P and dS tiles in
//      shared memory laid out so that the SAME tile serves as a K-major and as an MN-major UMMA operand, and
//      dV += P^T dO, dK += dS^T Q accumulate in TMEM (4 x 128 columns = all of TMEM);
//   3. attn_dq_kernel    : one CTA per (query tile, head, batch) walks the K/V tiles; dS goes back to TMEM as packed
//      bf16 and is the A operand of dQ += dS K straight from tensor memory.
// In both, every query row is shared by two softmax threads (columns [0,64) and [64,128)) in warps whose rank modulo
// four -- the TMEM lane quadrant a warp may access -- is the same.
// Recomputing S and dP in both kernels costs two extra tile products (7 instead of 5) and buys independence.

#include "common.cuh"
#include "ocb_api.h"
#include "tmap.h"

namespace ocb {
namespace {

// Optional cycle accounting of one CTA's roles (compile with -DOCB_ATTN_PROFILE; read with ocb_attention_prof_read).
#ifdef OCB_ATTN_PROFILE
__device__ long long g_attn_prof[32];
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = clock64()
#define PROF_LAP(i) do { const long long now_ = clock64(); prof_acc[i] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_STORE(base, n, cond) do { if (cond) for (int i_ = 0; i_ < (n); ++i_) g_attn_prof[(base) + i_] = prof_acc[i_]; } while (0)
#else
#define PROF_DECL(n) do {} while (0)
#define PROF_LAP(i) do {} while (0)
#define PROF_STORE(base, n, cond) do {} while (0)
#endif

constexpr int BT = 128;                    // tile rows (queries and keys)
constexpr int BD = 128;                    // head dim
constexpr int TILE_BYTES = BT * BD * 2;    // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int BWD_THREADS = 320;  // TMA warp + MMA warp + 8 softmax warps (two threads per query row)
constexpr float LOG2E = 1.4426950408889634f;

struct AttnBwdParams {
  const float* lse;    // [B, H, T] natural log
  const float* delta;  // [B, H, T]
  __nv_bfloat16* dq;   // [B, T, H, D]
  __nv_bfloat16* dk;   // [B, T, Hkv, D]
  __nv_bfloat16* dv;
  long long ld_dq, ld_dk, ld_dv;
  int T, H, Hkv;
  float scale, scale_log2;
  int causal;
  // Optional visibility bounds (sliding windows and document boundaries), as indices inside the sequence, int32 [B * T],
  // both non-decreasing: query i sees key j iff row_lo[i] <= j <= i; col_hi[j] is the last query that sees key j.
  const int* row_lo;
  const int* col_hi;
  int* status;
};

// [128 rows x 128 cols] bf16 tile stored as two [128 x 64] boxes with 128-byte swizzle.
// K-major view (contraction over the columns): k-step k = columns [16k, 16k+16).
__device__ __forceinline__ uint64_t desc_k(uint32_t tile, int k) {
  return make_smem_desc_sw128(tile + (k >> 2) * HALF_BYTES + (k & 3) * 32, 16, 1024);
}
// MN-major view (contraction over the rows): k-step k = rows [16k, 16k+16).
__device__ __forceinline__ uint64_t desc_mn(uint32_t tile, int k) {
  return make_smem_desc_sw128(tile + k * 2048, HALF_BYTES, 1024);
}

// Store 32 consecutive bf16 pairs... i.e. columns [32c, 32c+32) of row `row` (16 packed words) into a swizzled tile.
__device__ __forceinline__ void store_tile_row_chunk(uint8_t* tile, int row, int c, const uint32_t (&w)[16]) {
  uint8_t* base = tile + (c >> 1) * HALF_BYTES + row * 128;
  const int slot0 = (c & 1) * 4;  // 16-byte slot of the first 8 columns of this chunk inside the 128-byte row
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int slot = (slot0 + v) ^ (row & 7);
    *reinterpret_cast<uint4*>(base + slot * 16) = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
  }
}

__device__ __forceinline__ void store_acc_row(__nv_bfloat16* dst, uint32_t tmem_addr, int c_begin) {
#pragma unroll 1
  for (int c = c_begin; c < c_begin + 2; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(tmem_addr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 o;
      o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
      o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
      o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
      o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
      reinterpret_cast<uint4*>(dst + c * 32)[v] = o;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// 1. delta[b, h, t] = sum_d O[b, t, h, d] * dO[b, t, h, d]      (one warp per (token, head))
// ------------------------------------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, long long rows, int T, int H, long long ld_o, long long ld_do) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows * H) return;
  const long long token = w / H;
  const int h = static_cast<int>(w % H);
  const uint2 a = *reinterpret_cast<const uint2*>(o + token * ld_o + h * BD + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(dout + token * ld_do + h * BD + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
  float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
  s = warp_sum(s);
  if (lane == 0) delta[(token / T * H + h) * T + token % T] = s;
}

// ------------------------------------------------------------------------------------------------------------
// 2. dK, dV
// ------------------------------------------------------------------------------------------------------------
constexpr int DKDV_SMEM = 7 * TILE_BYTES + 1024 + 256;  // K, V, two Q stages, dO, P, dS

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do,
                 const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + 1 * TILE_BYTES;
  // Q is double-buffered and loaded one query tile ahead; dO has one buffer that is refilled as soon as dV += P^T dO has
  // read it (that product is issued before dK += dS^T Q for this reason). S and dP are signalled separately, so the
  // exponentials of a tile run while its dO is still in flight.
  uint8_t* sQ = smem + 2 * TILE_BYTES;   // stage s at sQ + s * TILE_BYTES
  uint8_t* sdO = smem + 4 * TILE_BYTES;
  uint8_t* sP = smem + 5 * TILE_BYTES;   // [q rows x kv cols]
  uint8_t* sdS = smem + 6 * TILE_BYTES;  // [q rows x kv cols]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * TILE_BYTES);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* q_empty = bars + 3;    // [2] dK += dS^T Q has read the stage
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;   // dV += P^T dO has read dO
  uint64_t* s_full = bars + 7;     // S is in TMEM
  uint64_t* dp_full = bars + 8;    // dP is in TMEM
  uint64_t* pds_full = bars + 9;   // P and dS tiles are in shared memory (8 warp arrivals)
  uint64_t* pds_empty = bars + 10; // the MMAs that read P / dS have finished
  uint64_t* acc_full = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // K/V tile
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  // query tiles [i_first, n_q) can see this key tile: up to the tile of the last query that sees its last key
  const int n_q = p.col_hi ? p.col_hi[b * p.T + jt * BT + BT - 1] / BT + 1 : p.T / BT;
  const int i_first = p.causal ? jt : 0;
  const int iters = (n_q - i_first) * group;  // (query head of the group, query tile) pairs
  const int kv_row0 = b * p.T + jt * BT;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int st = 0; st < 2; ++st) {
      mbar_init(&q_full[st], 1);
      mbar_init(&q_empty[st], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_2d(sK, &tma_k, kv_full, hk * BD, kv_row0);
      tma_load_2d(sK + HALF_BYTES, &tma_k, kv_full, hk * BD + 64, kv_row0);
      tma_load_2d(sV, &tma_v, kv_full, hk * BD, kv_row0);
      tma_load_2d(sV + HALF_BYTES, &tma_v, kv_full, hk * BD + 64, kv_row0);
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int h = hk * group + it / (n_q - i_first);
        const int q_row0 = b * p.T + (i_first + it % (n_q - i_first)) * BT;
        const int st = it & 1;
        uint8_t* q_dst = sQ + st * TILE_BYTES;
        ok = mbar_wait_bounded(&q_empty[st], ((it >> 1) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&q_full[st], TILE_BYTES);
        tma_load_2d(q_dst, &tma_q, &q_full[st], h * BD, q_row0);
        tma_load_2d(q_dst + HALF_BYTES, &tma_q, &q_full[st], h * BD + 64, q_row0);
        ok = mbar_wait_bounded(do_empty, (it & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(do_full, TILE_BYTES);
        tma_load_2d(sdO, &tma_do, do_full, h * BD, q_row0);
        tma_load_2d(sdO + HALF_BYTES, &tma_do, do_full, h * BD + 64, q_row0);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BT, BT, 0, 0);  // both operands contracted over their columns
      constexpr uint32_t idesc_mm = make_idesc_bf16(BT, BD, 1, 1);  // both operands contracted over their rows
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), adO = smem_u32(sdO), aP = smem_u32(sP), adS = smem_u32(sdS);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, p.status, kStatusTimeoutMma);
      for (int it = 0; it < iters && ok; ++it) {
        const uint32_t ph = it & 1;
        const int st = it & 1;
        const uint32_t aQ = smem_u32(sQ + st * TILE_BYTES);
        ok = mbar_wait_bounded(&q_full[st], (it >> 1) & 1, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        // S = Q K^T (S / dP of the previous pair were consumed before P / dS were published)
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tS, desc_k(aQ, k), desc_k(aK, k), idesc_kk, k != 0);
        umma_commit(s_full);
        ok = mbar_wait_bounded(do_full, ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        // dP = dO V^T
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tdP, desc_k(adO, k), desc_k(aV, k), idesc_kk, k != 0);
        umma_commit(dp_full);
        ok = mbar_wait_bounded(pds_full, ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        // dV += P^T dO first: its completion frees the dO buffer for the next tile's load
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tdV, desc_mn(aP, k), desc_mn(adO, k), idesc_mm, (it | k) != 0);
        umma_commit(do_empty);
        // dK += dS^T Q
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tdK, desc_mn(adS, k), desc_mn(aQ, k), idesc_mm, (it | k) != 0);
        umma_commit(&q_empty[st]);
        umma_commit(pds_empty);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // query row within the tile
    const int c_begin = ((warp - 2) >> 2) * 2;  // warps 2-5 take columns [0,64), warps 6-9 columns [64,128)
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const uint32_t ph = it & 1;
      const int h = hk * group + it / (n_q - i_first);
      const int qi = i_first + it % (n_q - i_first);
      const long long stat = (static_cast<long long>(b) * p.H + h) * p.T + qi * BT + row;
      const float lse2 = p.lse[stat] * LOG2E;
      const float dl = p.delta[stat];
      const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nl2 = pack_f32x2(-lse2, -lse2);
      const uint64_t scl2 = pack_f32x2(p.scale, p.scale), nds2 = pack_f32x2(-dl * p.scale, -dl * p.scale);
      const bool on_diag = p.causal && qi == jt;
      const int my_lo = p.row_lo ? p.row_lo[b * p.T + qi * BT + row] : 0;
      const int lo_last = p.row_lo ? p.row_lo[b * p.T + qi * BT + BT - 1] : 0;
      const bool diag = on_diag || jt * BT < lo_last;  // the tile needs the element-wise mask
      const int hi_col = on_diag ? row : BT - 1;       // visible key columns of this query row: [lo_col, hi_col]
      const int lo_col = my_lo - jt * BT;
      ok = mbar_wait_bounded(s_full, ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (it > 0) {
        ok = mbar_wait_bounded(pds_empty, ph ^ 1u, abort_flag, p.status, kStatusTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after();
      // phase 1, needs S only: probabilities of this thread's 64 columns (kept in registers for phase 2), P tile
      uint32_t t0[32], t1[32];
      uint64_t pv[2][16];  // the probabilities as packed fp32 pairs
      tmem_ld_32x32(tS + lane_addr + c_begin * 32, t0);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c_begin + cc;
        uint32_t(&s)[32] = cc ? t1 : t0;
        tmem_ld_wait();
        if (cc == 0) tmem_ld_32x32(tS + lane_addr + (c + 1) * 32, t1);  // flies while the first chunk is processed
        uint32_t pw[16];
        float p0[16], p1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          unpack_f32x2(fma_f32x2(pack_u32x2(s[2 * i], s[2 * i + 1]), sc2, nl2), p0[i], p1[i]);
          p0[i] = fast_exp2(p0[i]);
          p1[i] = fast_exp2(p1[i]);
        }
        if (diag) {  // warp-uniform: only tiles on the diagonal or on a window / document edge pay for the mask
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (c * 32 + 2 * i > hi_col || c * 32 + 2 * i < lo_col) p0[i] = 0.f;
            if (c * 32 + 2 * i + 1 > hi_col || c * 32 + 2 * i + 1 < lo_col) p1[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pv[cc][i] = pack_f32x2(p0[i], p1[i]);
          pw[i] = pack_bf16x2(p0[i], p1[i]);
        }
        store_tile_row_chunk(sP, row, c, pw);
      }
      // phase 2, once dP = dO V^T has landed: dS = P (dP - delta) scale
      ok = mbar_wait_bounded(dp_full, ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      tmem_ld_32x32(tdP + lane_addr + c_begin * 32, t0);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c_begin + cc;
        uint32_t(&g)[32] = cc ? t1 : t0;
        tmem_ld_wait();
        if (cc == 0) tmem_ld_32x32(tdP + lane_addr + (c + 1) * 32, t1);
        uint32_t dw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t t = fma_f32x2(pack_u32x2(g[2 * i], g[2 * i + 1]), scl2, nds2);  // (dP - delta) scale
          float d0, d1;
          unpack_f32x2(mul_f32x2(t, pv[cc][i]), d0, d1);
          dw[i] = pack_bf16x2(d0, d1);
        }
        store_tile_row_chunk(sdS, row, c, dw);
      }
      fence_proxy_async_smem();  // make the tiles visible to the tensor core (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (ok) {
      ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const long long token = static_cast<long long>(kv_row0) + row;  // accumulator row = key row
      store_acc_row(p.dv + token * p.ld_dv + hk * BD, tdV + lane_addr, c_begin);
      store_acc_row(p.dk + token * p.ld_dk + hk * BD, tdK + lane_addr, c_begin);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------
// 3. dQ
//
// One CTA per (query tile, head, batch) walks the key/value tiles with TWO tiles in flight: softmax warps 2-5 own the
// even tiles, warps 6-9 the odd ones (one thread per query row, all 128 columns), so that while one group turns its S
// into P and dS the tensor core works on the other group's tile. Tensor memory: R[0], R[1] (S of the even / odd tile,
// later its dS as packed bf16, the A operand of dQ += dS K), X (dP of either tile, handed back as soon as it has been
// read) and the dQ accumulator. The issue order  S(0) S(1) dP(0) | dP(j+1) dQ(j) S(j+2) ...  needs no wait between an
// MMA and a later MMA that overwrites what it read: tcgen05.mma operations of one thread execute in order.
// P stays in registers between the two phases as packed bf16 -- the same rounding the dV product sees.
// ------------------------------------------------------------------------------------------------------------
constexpr int DQ_KST = 3;  // K stages: a tile's K is read by S and again, much later, by dQ
constexpr int DQ_VST = 2;  // V stages: read by dP only
constexpr int DQ_SMEM = (2 + DQ_KST + DQ_VST) * TILE_BYTES + 1024 + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
               const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do,
               const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + 1 * TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;             // stage s at sK + s * TILE_BYTES
  uint8_t* sV = smem + (2 + DQ_KST) * TILE_BYTES;  // stage s at sV + s * TILE_BYTES
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + DQ_KST + DQ_VST) * TILE_BYTES);
  uint64_t* qdo_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [3]
  uint64_t* k_empty = bars + 4;   // [3] dQ += dS K has read the stage
  uint64_t* v_full = bars + 7;    // [2]
  uint64_t* v_empty = bars + 9;   // [2] dP = dO V^T has read the stage
  uint64_t* s_full = bars + 11;   // [2] S of an even / odd tile is in R[0] / R[1]
  uint64_t* dp_full = bars + 13;  // [2] dP of an even / odd tile is in X
  uint64_t* x_free = bars + 15;   // [2] the even / odd group has read X (4 warp arrivals)
  uint64_t* ds_full = bars + 17;  // [2] dS of an even / odd tile is in R[0] / R[1] (4 warp arrivals)
  uint64_t* acc_full = bars + 19;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q_row0 = b * p.T + qt * BT;
  const int lo_first = p.row_lo ? p.row_lo[q_row0] : 0;
  const int lo_last = p.row_lo ? p.row_lo[q_row0 + BT - 1] : 0;
  const int j_lo = lo_first / BT;  // first key tile any row of this query tile can see; `j` counts tiles from there
  const int n_kv = (p.causal ? qt + 1 : p.T / BT) - j_lo;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int st = 0; st < DQ_KST; ++st) {
      mbar_init(&k_full[st], 1);
      mbar_init(&k_empty[st], 1);
    }
    for (int st = 0; st < 2; ++st) {
      mbar_init(&v_full[st], 1);
      mbar_init(&v_empty[st], 1);
      mbar_init(&s_full[st], 1);
      mbar_init(&dp_full[st], 1);
      mbar_init(&x_free[st], 4);
      mbar_init(&ds_full[st], 4);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tR = tmem_base /* R[r] at tR + 128 r */, tX = tmem_base + 256, tdQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(qdo_full, 2 * TILE_BYTES);
      tma_load_2d(sQ, &tma_q, qdo_full, h * BD, q_row0);
      tma_load_2d(sQ + HALF_BYTES, &tma_q, qdo_full, h * BD + 64, q_row0);
      tma_load_2d(sdO, &tma_do, qdo_full, h * BD, q_row0);
      tma_load_2d(sdO + HALF_BYTES, &tma_do, qdo_full, h * BD + 64, q_row0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int kv_row0 = b * p.T + (j_lo + j) * BT;
        const int ks = j % DQ_KST, vs = j & 1;
        uint8_t* dK_ = sK + ks * TILE_BYTES;
        uint8_t* dV_ = sV + vs * TILE_BYTES;
        ok = mbar_wait_bounded(&k_empty[ks], ((j / DQ_KST) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[ks], TILE_BYTES);
        tma_load_2d(dK_, &tma_k, &k_full[ks], hk * BD, kv_row0);
        tma_load_2d(dK_ + HALF_BYTES, &tma_k, &k_full[ks], hk * BD + 64, kv_row0);
        ok = mbar_wait_bounded(&v_empty[vs], ((j >> 1) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[vs], TILE_BYTES);
        tma_load_2d(dV_, &tma_v, &v_full[vs], hk * BD, kv_row0);
        tma_load_2d(dV_ + HALF_BYTES, &tma_v, &v_full[vs], hk * BD + 64, kv_row0);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BT, BD, 0, 1);  // A = dS from TMEM, B = K contracted over its rows
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK0 = smem_u32(sK), aV0 = smem_u32(sV);
      bool ok = mbar_wait_bounded(qdo_full, 0, abort_flag, p.status, kStatusTimeoutMma);
      // S(j) = Q K_j^T into R[j & 1]
      auto issue_s = [&](int j) -> bool {
        const int ks = j % DQ_KST;
        if (!mbar_wait_bounded(&k_full[ks], (j / DQ_KST) & 1, abort_flag, p.status, kStatusTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t aK = aK0 + ks * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tR + (j & 1) * 128, desc_k(aQ, k), desc_k(aK, k), idesc_kk, k != 0);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      // dP(j) = dO V_j^T into X (the caller has made sure that X was read)
      auto issue_dp = [&](int j) -> bool {
        const int vs = j & 1;
        if (!mbar_wait_bounded(&v_full[vs], (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t aV = aV0 + vs * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tX, desc_k(adO, k), desc_k(aV, k), idesc_kk, k != 0);
        umma_commit(&dp_full[j & 1]);
        umma_commit(&v_empty[vs]);
        return true;
      };
      ok = ok && issue_s(0);
      if (n_kv > 1) ok = ok && issue_s(1);
      ok = ok && issue_dp(0);
      PROF_DECL(4);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int r = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        PROF_LAP(3);
        if (j + 1 < n_kv) {
          ok = mbar_wait_bounded(&x_free[r], ph, abort_flag, p.status, kStatusTimeoutMma);
          if (!ok) break;
          PROF_LAP(0);
          ok = issue_dp(j + 1);
          if (!ok) break;
          PROF_LAP(1);
        }
        ok = mbar_wait_bounded(&ds_full[r], ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        PROF_LAP(2);
        tc_fence_after();
        const int ks = j % DQ_KST;
        const uint32_t aK = aK0 + ks * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ts(tdQ, tR + r * 128 + k * 8, desc_mn(aK, k), idesc_dq, (j | k) != 0);
        umma_commit(&k_empty[ks]);
        if (j + 2 < n_kv) ok = issue_s(j + 2);  // overwrites dS(j) only after dQ(j): same thread, in order
      }
      if (ok) umma_commit(acc_full);
      PROF_LAP(3);
      PROF_STORE(8, 4, blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    }
  } else {
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;  // 0: even tiles (and dQ columns [0,64) at the end), 1: odd tiles ([64,128))
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const long long stat = (static_cast<long long>(b) * p.H + h) * p.T + qt * BT + row;
    const float lse2 = p.lse[stat] * LOG2E;
    const float dl = p.delta[stat];
    const int my_lo = p.row_lo ? p.row_lo[q_row0 + row] : 0;
    const uint32_t tRg = tR + grp * 128 + lane_addr;
    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nl2 = pack_f32x2(-lse2, -lse2);
    const uint64_t scl2 = pack_f32x2(p.scale, p.scale), nds2 = pack_f32x2(-dl * p.scale, -dl * p.scale);
    bool ok = true;
    PROF_DECL(8);
    for (int j = grp; j < n_kv; j += 2) {
      PROF_LAP(4);
      const uint32_t ph = (j >> 1) & 1;
      const int kv0 = (j_lo + j) * BT;
      const bool on_diag = p.causal && j_lo + j == qt;
      const bool diag = on_diag || kv0 < lo_last;
      const int hi_col = on_diag ? row : BT - 1;
      const int lo_col = my_lo - kv0;
      ok = mbar_wait_bounded(&s_full[grp], ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      PROF_LAP(0);
      tc_fence_after();
      // phase 1: P of the whole row, kept as packed bf16
      uint32_t ppk[64];
      uint32_t g0[16], g1[16];  // 16-column pieces keep the live set under the register limit
      tmem_ld_32x16(tRg, g0);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t(&s)[16] = (c & 1) ? g1 : g0;
        PROF_LAP(1);
        tmem_ld_wait();
        PROF_LAP(5);
        if (c < 7) tmem_ld_32x16(tRg + (c + 1) * 16, (c & 1) ? g0 : g1);
        uint64_t e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = fma_f32x2(pack_u32x2(s[2 * i], s[2 * i + 1]), sc2, nl2);
        float p0[8], p1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          unpack_f32x2(e[i], p0[i], p1[i]);
          p0[i] = fast_exp2(p0[i]);
          p1[i] = fast_exp2(p1[i]);
        }
        if (diag) {  // warp-uniform: only tiles on the diagonal or on a window / document edge pay for the mask
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (c * 16 + 2 * i > hi_col || c * 16 + 2 * i < lo_col) p0[i] = 0.f;
            if (c * 16 + 2 * i + 1 > hi_col || c * 16 + 2 * i + 1 < lo_col) p1[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ppk[c * 8 + i] = pack_bf16x2(p0[i], p1[i]);
      }
      // phase 2: dS = P (dP - delta) scale, written over S as packed bf16
      PROF_LAP(1);
      ok = mbar_wait_bounded(&dp_full[grp], ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      PROF_LAP(2);
      tc_fence_after();
      tmem_ld_32x16(tX + lane_addr, g0);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t dw[16];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t(&g)[16] = hh ? g1 : g0;
          PROF_LAP(3);
          tmem_ld_wait();
          PROF_LAP(6);
          if (c < 3 || hh == 0) {
            tmem_ld_32x16(tX + lane_addr + (2 * c + hh + 1) * 16, hh ? g0 : g1);
          } else {
            tc_fence_before();  // X has been read: the next tile's dP may overwrite it
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_free[grp]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint64_t t = fma_f32x2(pack_u32x2(g[2 * i], g[2 * i + 1]), scl2, nds2);  // (dP - delta) scale
            float d0, d1;
            unpack_f32x2(mul_f32x2(t, bf16x2_to_f32x2(ppk[c * 16 + hh * 8 + i])), d0, d1);
            dw[hh * 8 + i] = pack_bf16x2(d0, d1);
          }
        }
        tmem_st_32x16(tRg + c * 16, dw);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[grp]);
      PROF_LAP(3);
    }
    PROF_STORE(0, 8, warp == 2 && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const long long token = static_cast<long long>(q_row0) + row;
      store_acc_row(p.dq + token * p.ld_dq + h * BD, tdQ + lane_addr, grp * 2);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

bool make_map(CUtensorMap* map, const void* ptr, long long rows, int heads, long long ld) {
  uint64_t dims[2] = {static_cast<uint64_t>(heads) * BD, static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(ld) * 2};
  uint32_t box[2] = {64, BT};
  return get_tensor_map(map, ptr, 2, dims, str, box, 2);
}

}  // namespace
}  // namespace ocb

using namespace ocb;

#ifdef OCB_ATTN_PROFILE
extern "C" int ocb_attention_prof_read(long long* host32) {
  return cudaMemcpyFromSymbol(host32, g_attn_prof, sizeof(long long) * 32) == cudaSuccess ? 0 : -1;
}
#endif

// Gradients of ocb_attention_fwd. dout/out/q/dq: [B, T, H, D]; k, v, dk, dv: [B, T, Hkv, D]; lse: [B, H, T] from the
// forward pass; delta: [B, H, T] fp32 scratch (written here). dq/dk/dv are written densely (row stride heads * D).
extern "C" int ocb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                 const float* lse, void* dq, void* dk, void* dv, const int* bounds, float* delta, int B,
                                 int Tq, int Tk, int H, int Hkv, int D, long long ldq, long long ldk, long long ldv,
                                 long long ldo, float scale, int causal, int window, int* status, cudaStream_t stream) {
  if (B <= 0 || Tq <= 0) return 0;
  (void)window;  // folded into `bounds` (int32 [2, B * T]: row_lo then col_hi, see ocb_attention_fwd) by the caller
  if (D != BD || Tq != Tk || (Tq % BT) != 0 || (bounds != nullptr && !causal) || Hkv <= 0 || (H % Hkv) != 0 ||
      delta == nullptr)
    return -5;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -1;
  const long long rows = static_cast<long long>(B) * Tq;
  const long long ld_do = static_cast<long long>(H) * BD;  // dout is dense
  CUtensorMap mq, mk, mv, mdo;
  if (!make_map(&mq, q, rows, H, ldq)) return -1001;
  if (!make_map(&mk, k, rows, Hkv, ldk)) return -1002;
  if (!make_map(&mv, v, rows, Hkv, ldv)) return -1003;
  if (!make_map(&mdo, dout, rows, H, ld_do)) return -1004;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKDV_SMEM) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM) != cudaSuccess) return -3;
    configured = true;
  }
  {
    const long long warps = rows * H;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), delta, rows, Tq, H, ldo, ld_do);
  }
  AttnBwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.ld_dq = static_cast<long long>(H) * BD;
  p.ld_dk = p.ld_dv = static_cast<long long>(Hkv) * BD;
  p.T = Tq;
  p.H = H;
  p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.causal = causal;
  p.row_lo = bounds;
  p.col_hi = bounds ? bounds + static_cast<long long>(B) * Tq : nullptr;
  p.status = status;
  attn_dkdv_kernel<<<dim3(Tq / BT, Hkv, B), BWD_THREADS, DKDV_SMEM, stream>>>(mq, mk, mv, mdo, p);
  attn_dq_kernel<<<dim3(Tq / BT, H, B), BWD_THREADS, DQ_SMEM, stream>>>(mq, mk, mv, mdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
