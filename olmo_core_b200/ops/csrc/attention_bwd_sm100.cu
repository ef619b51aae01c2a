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
//   2. attn_dkdv_kernel  : one CTA per (K/V tile, kv head, batch) walks 64-row query sub-tiles, computing S^T and dP^T
//      so that P^T and dS^T stay in tensor memory as the A operands of dV += P^T dO and dK += dS^T Q;
//   3. attn_dq_kernel    : one CTA per (query tile, head, batch) walks the K/V tiles; dS goes back to TMEM as packed
//      bf16 and is the A operand of dQ += dS K.
// Both keep TWO tiles in flight: two groups of four softmax warps alternate, so the exponentials of one tile run while
// the tensor core works on the other. The softmax loops use packed fp32-pair arithmetic (fma/mul.f32x2) and take the
// element-wise mask only on tiles that touch the diagonal or a window / document edge.
// Recomputing S and dP in both kernels costs two extra tile products (7 instead of 5) and buys independence.

#include "common.cuh"
#include "attn_seq_map.cuh"
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
  AttnSeqMap m;  // where query tiles sit in the global sequence and where key / value tiles are fetched from
  int H, Hkv;
  float scale, scale_log2;
  int causal;
  // Optional visibility bounds (sliding windows and document boundaries), both non-decreasing: row_lo int32 [B * Tq] is
  // the lowest key index a query sees, col_hi int32 [B * Tk] the position of the last query that sees a key (key indices
  // and query positions in the global sequence): the query at position i sees key j iff row_lo[i] <= j <= i.
  const int* row_lo;
  const int* col_hi;
  int* status;
};

// [128 rows x 128 cols] bf16 tile stored as two [128 x 64] boxes with 128-byte swizzle (sub-tiles: two [64 x 64] boxes).
// K-major view (contraction over the columns): k-step k = columns [16k, 16k+16), LBO field unused (16).
// MN-major view (contraction over the rows): k-step k = rows [16k, 16k+16), LBO = distance between the two boxes.
// Both as descriptor low words (see desc_lo_sw128 / umma_ss_lean): stepping costs one integer add per instruction.
constexpr uint32_t kHi = desc_hi_sw128(1024);
__device__ __forceinline__ constexpr uint32_t koff_k(int k, uint32_t box_bytes) {  // K-major k-step, in 16-byte units
  return ((k >> 2) * box_bytes + (k & 3) * 32) >> 4;
}
__device__ __forceinline__ constexpr uint32_t koff_mn(int k) { return (k * 2048) >> 4; }  // MN-major k-step
// All k-step descriptors of a tile, materialised in registers BEFORE the issuing thread waits for the tile: once the
// wait returns, nothing but the tcgen05.mma instructions themselves stands between the tensor core and its work.
template <int STEPS>
__device__ __forceinline__ void descs_k(uint64_t (&d)[STEPS], uint32_t lo, uint32_t box_bytes) {
#pragma unroll
  for (int k = 0; k < STEPS; ++k) {
    d[k] = pack_u32x2(lo + koff_k(k, box_bytes), kHi);
    asm volatile("" : "+l"(d[k]));
  }
}
template <int STEPS>
__device__ __forceinline__ void descs_mn(uint64_t (&d)[STEPS], uint32_t lo) {
#pragma unroll
  for (int k = 0; k < STEPS; ++k) {
    d[k] = pack_u32x2(lo + koff_mn(k), kHi);
    asm volatile("" : "+l"(d[k]));
  }
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
// 1. delta[b, h, t] = sum_d O[b, t, h, d] * dO[b, t, h, d]
//    Sixteen lanes per (token, head) row with 16-byte loads; a warp takes 2 x kDeltaUnroll rows and issues all of
//    its loads before the first sum, so that every thread has 128 bytes in flight.
// ------------------------------------------------------------------------------------------------------------
constexpr int kDeltaUnroll = 4;

__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                  float* __restrict__ delta, long long rows, int T, int H, long long ld_o, long long ld_do) {
  // 32-bit row arithmetic (the launcher checks that rows * H fits): 64-bit divisions would dominate the kernel
  const int n = static_cast<int>(rows) * H;
  const int warp = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31, half = lane >> 4, l = lane & 15;
  uint4 a[kDeltaUnroll], g[kDeltaUnroll];
  int w[kDeltaUnroll];
#pragma unroll
  for (int k = 0; k < kDeltaUnroll; ++k) {
    w[k] = (warp * kDeltaUnroll + k) * 2 + half;
    a[k] = g[k] = make_uint4(0u, 0u, 0u, 0u);
    if (w[k] < n) {
      const int token = w[k] / H, h = w[k] - token * H;
      a[k] = *reinterpret_cast<const uint4*>(o + static_cast<long long>(token) * ld_o + h * BD + l * 8);
      g[k] = *reinterpret_cast<const uint4*>(dout + static_cast<long long>(token) * ld_do + h * BD + l * 8);
    }
  }
#pragma unroll
  for (int k = 0; k < kDeltaUnroll; ++k) {
    const float2 a0 = unpack_bf16x2(a[k].x), a1 = unpack_bf16x2(a[k].y), a2 = unpack_bf16x2(a[k].z), a3 = unpack_bf16x2(a[k].w);
    const float2 g0 = unpack_bf16x2(g[k].x), g1 = unpack_bf16x2(g[k].y), g2 = unpack_bf16x2(g[k].z), g3 = unpack_bf16x2(g[k].w);
    float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y + a3.x * g3.x + a3.y * g3.y;
#pragma unroll
    for (int sh = 8; sh > 0; sh >>= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);  // stays inside the 16 lanes of a row
    if (l == 0 && w[k] < n) {
      const int token = w[k] / H, h = w[k] - token * H;
      const int b = token / T, tq = token - b * T;
      delta[(static_cast<long long>(b) * H + h) * T + tq] = s;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// 2. dK, dV
//
// One CTA per (K/V tile, kv head, batch) walks 64-row query sub-tiles ("units": the query heads of the group, their
// query tiles, two halves each) with TWO units in flight: softmax warps 2-5 own the even units, warps 6-9 the odd ones.
// Everything is computed transposed so that the probabilities never leave tensor memory:
//     S^T = K Q^T, dP^T = V dO^T           [128 keys x 64 queries], SS products with N = 64
//     P^T, dS^T                            packed bf16 written over S^T / dP^T (one thread per key row, 64 columns)
//     dV += P^T dO,  dK += dS^T Q          A operand straight from tensor memory, B = the 64-row dO / Q sub-tile
// Tensor memory: dV, dK (2 x 128 columns) and, per unit parity, S^T | dP^T (2 x (64 + 64) columns). The row statistics
// are per COLUMN here; the producer brings lse and delta of the 64 queries into shared memory with the sub-tiles.
// Issue order  S(0) dP(0) S(1) dP(1) | dV(u) dK(u) S(u+2) dP(u+2) ...: an MMA that overwrites what an earlier MMA of
// the same thread reads needs no wait, they execute in order.
// ------------------------------------------------------------------------------------------------------------
constexpr int SUB = 64;                   // query rows per unit
constexpr int SUB_BYTES = SUB * BD * 2;   // 16 KB: two [64 x 64] boxes
constexpr int SUB_BOX = SUB_BYTES / 2;
constexpr int KV_NST = 4;                 // stages of (Q sub-tile, dO sub-tile, lse, delta)
constexpr int STAT_BYTES = 2 * SUB * 4;   // lse then delta of the 64 queries
constexpr int DKDV_SMEM = 2 * TILE_BYTES + KV_NST * (2 * SUB_BYTES + STAT_BYTES) + 1024 + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tma_q /* 64-row boxes */, const __grid_constant__ CUtensorMap tma_k,
                 const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do /* 64-row boxes */,
                 const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQdO = smem + 2 * TILE_BYTES;  // stage s: Q sub-tile at sQdO + 2 s SUB_BYTES, dO one sub-tile after it
  float* sStat = reinterpret_cast<float*>(smem + 2 * TILE_BYTES + KV_NST * 2 * SUB_BYTES);  // stage s: [lse 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * TILE_BYTES + KV_NST * (2 * SUB_BYTES + STAT_BYTES));
  uint64_t* kv_full = bars + 0;
  uint64_t* full = bars + 1;      // [4] Q, dO, lse, delta of a unit have landed
  uint64_t* empty = bars + 5;     // [4] dK += dS^T Q of the unit has finished
  uint64_t* s_full = bars + 9;    // [2] S^T of an even / odd unit is in TMEM
  uint64_t* dp_full = bars + 11;  // [2] dP^T
  uint64_t* p_full = bars + 13;   // [2] P^T is in TMEM (4 warp arrivals)
  uint64_t* ds_full = bars + 15;  // [2] dS^T is in TMEM (4 warp arrivals)
  uint64_t* acc_full = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // K/V tile
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  // LOCAL query tiles [i_first, n_q) can see this key tile: from the first one at or after the key tile's place in the
  // global sequence up to the tile of the last query that sees its last key (local tiles are in global order)
  const int kv_g0 = b * p.m.Tk + jt * BT;  // the tile's first key in the global [B * Tk] key space (bounds, outputs)
  int i_first = 0, n_q = p.m.Tq / BT;
  if (p.causal)
    while (i_first < n_q && attn_q_gtile(p.m, i_first) < jt) ++i_first;
  if (p.col_hi) {
    const int hi_last = p.col_hi[kv_g0 + BT - 1];
    while (n_q > i_first && attn_q_gtile(p.m, n_q - 1) * BT > hi_last) --n_q;
  }
  const int per_head = (n_q - i_first) * 2;  // units per query head
  const int units = per_head * group;
  int kv_src;
  const int kv_row0 = attn_kv_row0(p.m, b, jt, kv_src);  // the tile's first row in its source buffer
  // last query that sees the FIRST key of the tile: units that reach beyond it need the element-wise mask
  const int hi_first = p.col_hi ? p.col_hi[kv_g0] : p.m.Tk - 1;
  if (units == 0) {
    // no local query sees this tile (possible only when the queries are a shard of the sequence): its gradients are zero
    for (int i = threadIdx.x; i < BT * (BD / 8); i += BWD_THREADS) {
      const long long token = static_cast<long long>(kv_g0) + i / (BD / 8);
      const int c = (i % (BD / 8)) * 8;
      *reinterpret_cast<uint4*>(p.dk + token * p.ld_dk + hk * BD + c) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(p.dv + token * p.ld_dv + hk * BD + c) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int st = 0; st < KV_NST; ++st) {
      mbar_init(&full[st], 1);
      mbar_init(&empty[st], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&s_full[r], 1);
      mbar_init(&dp_full[r], 1);
      mbar_init(&p_full[r], 4);
      mbar_init(&ds_full[r], 4);
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
  const uint32_t tdV = tmem_base, tdK = tmem_base + 128, tReg = tmem_base + 256;  // unit parity r: tReg + 128 r

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      const CUtensorMap* mk = attn_k_map(p.m, &tma_k, kv_src);
      const CUtensorMap* mv = attn_v_map(p.m, &tma_v, kv_src);
      tma_load_2d(sK, mk, kv_full, hk * BD, kv_row0);
      tma_load_2d(sK + HALF_BYTES, mk, kv_full, hk * BD + 64, kv_row0);
      tma_load_2d(sV, mv, kv_full, hk * BD, kv_row0);
      tma_load_2d(sV + HALF_BYTES, mv, kv_full, hk * BD + 64, kv_row0);
      bool ok = true;
      for (int u = 0; u < units && ok; ++u) {
        const int h = hk * group + u / per_head;
        const int rem = u % per_head;
        const int q0 = (i_first + (rem >> 1)) * BT + (rem & 1) * SUB;  // local row of the unit's first query
        const int q_row0 = b * p.m.Tq + q0;
        const int st = u % KV_NST;
        uint8_t* q_dst = sQdO + st * 2 * SUB_BYTES;
        uint8_t* do_dst = q_dst + SUB_BYTES;
        float* stat_dst = sStat + st * 2 * SUB;
        const long long stat = (static_cast<long long>(b) * p.H + h) * p.m.Tq + q0;
        ok = mbar_wait_bounded(&empty[st], ((u / KV_NST) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&full[st], 2 * SUB_BYTES + STAT_BYTES);
        tma_load_2d(q_dst, &tma_q, &full[st], h * BD, q_row0);
        tma_load_2d(q_dst + SUB_BOX, &tma_q, &full[st], h * BD + 64, q_row0);
        tma_load_2d(do_dst, &tma_do, &full[st], h * BD, q_row0);
        tma_load_2d(do_dst + SUB_BOX, &tma_do, &full[st], h * BD + 64, q_row0);
        bulk_load_1d(stat_dst, p.lse + stat, SUB * 4, &full[st]);
        bulk_load_1d(stat_dst + SUB, p.delta + stat, SUB * 4, &full[st]);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(BT, SUB, 0, 0);  // [128 keys x 64 queries], both contracted over d
      constexpr uint32_t idesc_acc = make_idesc_bf16(BT, BD, 0, 1);  // A from TMEM, B contracted over its rows
      const uint32_t aQdO = smem_u32(sQdO);
      uint64_t dK_[8], dV_[8];  // K and V never move
      descs_k(dK_, desc_lo_sw128(smem_u32(sK), 16), HALF_BYTES);
      descs_k(dV_, desc_lo_sw128(smem_u32(sV), 16), HALF_BYTES);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, p.status, kStatusTimeoutMma);
      PROF_DECL(5);
      // S^T and dP^T of unit u into the region of its parity
      auto issue_sp = [&](int u) -> bool {
        const int st = u % KV_NST;
        const uint32_t q_lo = desc_lo_sw128(aQdO + st * 2 * SUB_BYTES, 16);
        uint64_t dQ_[8], ddO_[8];
        descs_k(dQ_, q_lo, SUB_BOX);
        descs_k(ddO_, q_lo + (SUB_BYTES >> 4), SUB_BOX);
        const uint32_t tS = tReg + (u & 1) * 128, tP = tS + SUB;
        PROF_LAP(3);
        if (!mbar_wait_bounded(&full[st], (u / KV_NST) & 1, abort_flag, p.status, kStatusTimeoutMma)) return false;
        PROF_LAP(4);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tS, dK_[k], dQ_[k], idesc_st, k != 0);
        umma_commit(&s_full[u & 1]);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tP, dV_[k], ddO_[k], idesc_st, k != 0);
        umma_commit(&dp_full[u & 1]);
        return true;
      };
      ok = ok && issue_sp(0);
      if (units > 1) ok = ok && issue_sp(1);
      for (int u = 0; u < units && ok; ++u) {
        PROF_LAP(3);
        const int r = u & 1;
        const uint32_t ph = (u >> 1) & 1;
        const int st = u % KV_NST;
        // MN-major views of the unit's Q / dO sub-tiles (the box distance is the LBO field of the low word)
        const uint32_t qmn_lo = desc_lo_sw128(aQdO + st * 2 * SUB_BYTES, SUB_BOX);
        uint64_t dQmn[SUB / 16], ddOmn[SUB / 16];
        descs_mn(dQmn, qmn_lo);
        descs_mn(ddOmn, qmn_lo + (SUB_BYTES >> 4));
        const uint32_t tPT = tReg + r * 128, tdST = tPT + SUB;  // packed bf16 over the first 32 columns of S^T / dP^T
        const uint32_t acc0 = u != 0;
        ok = mbar_wait_bounded(&p_full[r], ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        PROF_LAP(0);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < SUB / 16; ++k)
          umma_f16_ts(tdV, tPT + k * 8, ddOmn[k], idesc_acc, k == 0 ? acc0 : 1u);
        PROF_LAP(3);
        ok = mbar_wait_bounded(&ds_full[r], ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        PROF_LAP(1);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < SUB / 16; ++k)
          umma_f16_ts(tdK, tdST + k * 8, dQmn[k], idesc_acc, k == 0 ? acc0 : 1u);
        umma_commit(&empty[st]);
        PROF_LAP(3);
        if (u + 2 < units) ok = issue_sp(u + 2);  // overwrites P^T / dS^T of unit u only after the products above
        PROF_LAP(2);
      }
      if (ok) umma_commit(acc_full);
      PROF_STORE(24, 5, blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    }
  } else {
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;  // 0: even units (and columns [0,64) of dV / dK at the end), 1: odd units
    const int row = quad * 32 + lane;  // key row within the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int kv_pos = jt * BT + row;  // position of this thread's key in the sequence
    const int vis_lo = p.causal ? kv_pos : 0;                               // first and
    const int vis_hi = p.col_hi ? p.col_hi[b * p.m.Tk + kv_pos] : p.m.Tk - 1;  // last query that sees the key
    const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nlog2 = pack_f32x2(-LOG2E, -LOG2E);
    const uint64_t scl2 = pack_f32x2(p.scale, p.scale), nscl2 = pack_f32x2(-p.scale, -p.scale);
    const uint32_t tS = tReg + grp * 128 + lane_addr, tP = tS + SUB;
    bool ok = true;
    PROF_DECL(5);
    for (int u = grp; u < units; u += 2) {
      PROF_LAP(4);
      const uint32_t ph = (u >> 1) & 1;
      const int rem = u % per_head;
      const int q0 = attn_q_gtile(p.m, i_first + (rem >> 1)) * BT + (rem & 1) * SUB;  // global position
      const int st = u % KV_NST;
      const float* st_lse = sStat + st * 2 * SUB;
      const float* st_dl = st_lse + SUB;
      const bool edge = (p.causal && q0 < jt * BT + BT - 1) || q0 + SUB - 1 > hi_first;  // uniform over the CTA
      const int c_lo = vis_lo - q0, c_hi = vis_hi - q0;  // visible columns of this key row: [c_lo, c_hi]
      ok = mbar_wait_bounded(&full[st], (u / KV_NST) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);  // lse, delta
      ok = ok && mbar_wait_bounded(&s_full[grp], ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      PROF_LAP(0);
      tc_fence_after();
      // phase 1: P^T of this key row for the 64 queries, kept as packed bf16 and written over S^T
      uint32_t ppk[32];
      uint32_t t0[32], t1[32];
      tmem_ld_32x32(tS, t0);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t(&s)[32] = cc ? t1 : t0;
        tmem_ld_wait();
        if (cc == 0) tmem_ld_32x32(tS + 32, t1);
        float p0[16], p1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t nl2 = mul_f32x2(*reinterpret_cast<const uint64_t*>(st_lse + cc * 32 + 2 * i), nlog2);
          unpack_f32x2(fma_f32x2(pack_u32x2(s[2 * i], s[2 * i + 1]), sc2, nl2), p0[i], p1[i]);
          p0[i] = fast_exp2(p0[i]);
          p1[i] = fast_exp2(p1[i]);
        }
        if (edge) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (cc * 32 + 2 * i < c_lo || cc * 32 + 2 * i > c_hi) p0[i] = 0.f;
            if (cc * 32 + 2 * i + 1 < c_lo || cc * 32 + 2 * i + 1 > c_hi) p1[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) ppk[cc * 16 + i] = pack_bf16x2(p0[i], p1[i]);
      }
      {
        uint32_t(&lo)[16] = *reinterpret_cast<uint32_t(*)[16]>(&ppk[0]);
        uint32_t(&hi)[16] = *reinterpret_cast<uint32_t(*)[16]>(&ppk[16]);
        tmem_st_32x16(tS, lo);
        tmem_st_32x16(tS + 16, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[grp]);
      // phase 2: dS^T = P^T (dP^T - delta) scale, written over dP^T
      PROF_LAP(1);
      ok = mbar_wait_bounded(&dp_full[grp], ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      PROF_LAP(2);
      tc_fence_after();
      uint32_t dw[32];
      tmem_ld_32x32(tP, t0);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t(&g)[32] = cc ? t1 : t0;
        tmem_ld_wait();
        if (cc == 0) tmem_ld_32x32(tP + 32, t1);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t nds2 = mul_f32x2(*reinterpret_cast<const uint64_t*>(st_dl + cc * 32 + 2 * i), nscl2);
          const uint64_t t = fma_f32x2(pack_u32x2(g[2 * i], g[2 * i + 1]), scl2, nds2);  // (dP - delta) scale
          float d0, d1;
          unpack_f32x2(mul_f32x2(t, bf16x2_to_f32x2(ppk[cc * 16 + i])), d0, d1);
          dw[cc * 16 + i] = pack_bf16x2(d0, d1);
        }
      }
      {
        uint32_t(&lo)[16] = *reinterpret_cast<uint32_t(*)[16]>(&dw[0]);
        uint32_t(&hi)[16] = *reinterpret_cast<uint32_t(*)[16]>(&dw[16]);
        tmem_st_32x16(tP, lo);
        tmem_st_32x16(tP + 16, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[grp]);
      PROF_LAP(3);
    }
    PROF_STORE(16, 5, warp == 2 && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const long long token = static_cast<long long>(kv_g0) + row;  // accumulator row = key row
      store_acc_row(p.dv + token * p.ld_dv + hk * BD, tdV + lane_addr, grp * 2);
      store_acc_row(p.dk + token * p.ld_dk + hk * BD, tdK + lane_addr, grp * 2);
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
  const int gt = attn_q_gtile(p.m, qt);  // the tile's place in the global sequence
  const int q_row0 = b * p.m.Tq + qt * BT;
  const int lo_first = p.row_lo ? p.row_lo[q_row0] : 0;
  const int lo_last = p.row_lo ? p.row_lo[q_row0 + BT - 1] : 0;
  const int j_lo = lo_first / BT;  // first key tile any row of this query tile can see; `j` counts tiles from there
  const int n_kv = (p.causal ? gt + 1 : p.m.Tk / BT) - j_lo;

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
        int src;
        const int kv_row0 = attn_kv_row0(p.m, b, j_lo + j, src);
        const CUtensorMap* mk = attn_k_map(p.m, &tma_k, src);
        const CUtensorMap* mv = attn_v_map(p.m, &tma_v, src);
        const int ks = j % DQ_KST, vs = j & 1;
        uint8_t* dK_ = sK + ks * TILE_BYTES;
        uint8_t* dV_ = sV + vs * TILE_BYTES;
        ok = mbar_wait_bounded(&k_empty[ks], ((j / DQ_KST) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[ks], TILE_BYTES);
        tma_load_2d(dK_, mk, &k_full[ks], hk * BD, kv_row0);
        tma_load_2d(dK_ + HALF_BYTES, mk, &k_full[ks], hk * BD + 64, kv_row0);
        ok = mbar_wait_bounded(&v_empty[vs], ((j >> 1) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[vs], TILE_BYTES);
        tma_load_2d(dV_, mv, &v_full[vs], hk * BD, kv_row0);
        tma_load_2d(dV_ + HALF_BYTES, mv, &v_full[vs], hk * BD + 64, kv_row0);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BT, BD, 0, 1);  // A = dS from TMEM, B = K contracted over its rows
      uint64_t dQ_[8], ddO_[8];  // Q and dO never move
      descs_k(dQ_, desc_lo_sw128(smem_u32(sQ), 16), HALF_BYTES);
      descs_k(ddO_, desc_lo_sw128(smem_u32(sdO), 16), HALF_BYTES);
      const uint32_t k_lo0 = desc_lo_sw128(smem_u32(sK), 16), v_lo0 = desc_lo_sw128(smem_u32(sV), 16);
      const uint32_t kmn_lo0 = desc_lo_sw128(smem_u32(sK), HALF_BYTES);  // MN-major view of the K stages
      bool ok = mbar_wait_bounded(qdo_full, 0, abort_flag, p.status, kStatusTimeoutMma);
      PROF_DECL(6);
      // S(j) = Q K_j^T into R[j & 1]
      auto issue_s = [&](int j) -> bool {
        const int ks = j % DQ_KST;
        uint64_t dK_[8];
        descs_k(dK_, k_lo0 + ks * (TILE_BYTES >> 4), HALF_BYTES);
        PROF_LAP(3);
        if (!mbar_wait_bounded(&k_full[ks], (j / DQ_KST) & 1, abort_flag, p.status, kStatusTimeoutMma)) return false;
        PROF_LAP(4);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tR + (j & 1) * 128, dQ_[k], dK_[k], idesc_kk, k != 0);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      // dP(j) = dO V_j^T into X (the caller has made sure that X was read)
      auto issue_dp = [&](int j) -> bool {
        const int vs = j & 1;
        uint64_t dV_[8];
        descs_k(dV_, v_lo0 + vs * (TILE_BYTES >> 4), HALF_BYTES);
        PROF_LAP(1);
        if (!mbar_wait_bounded(&v_full[vs], (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutMma)) return false;
        PROF_LAP(5);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ss(tX, ddO_[k], dV_[k], idesc_kk, k != 0);
        umma_commit(&dp_full[j & 1]);
        umma_commit(&v_empty[vs]);
        return true;
      };
      ok = ok && issue_s(0);
      if (n_kv > 1) ok = ok && issue_s(1);
      ok = ok && issue_dp(0);
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
        const int ks = j % DQ_KST;
        uint64_t dKmn[8];
        descs_mn(dKmn, kmn_lo0 + ks * (TILE_BYTES >> 4));
        const uint32_t acc0 = j != 0;
        ok = mbar_wait_bounded(&ds_full[r], ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        PROF_LAP(2);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ts(tdQ, tR + r * 128 + k * 8, dKmn[k], idesc_dq, k == 0 ? acc0 : 1u);
        umma_commit(&k_empty[ks]);
        if (j + 2 < n_kv) ok = issue_s(j + 2);  // overwrites dS(j) only after dQ(j): same thread, in order
      }
      if (ok) umma_commit(acc_full);
      PROF_LAP(3);
      PROF_STORE(8, 6, blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    }
  } else {
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;  // 0: even tiles (and dQ columns [0,64) at the end), 1: odd tiles ([64,128))
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const long long stat = (static_cast<long long>(b) * p.H + h) * p.m.Tq + qt * BT + row;
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
      const bool on_diag = p.causal && j_lo + j == gt;
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

bool make_map(CUtensorMap* map, const void* ptr, long long rows, int heads, long long ld, int box_rows = BT) {
  uint64_t dims[2] = {static_cast<uint64_t>(heads) * BD, static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(ld) * 2};
  uint32_t box[2] = {64, static_cast<uint32_t>(box_rows)};
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

// Shared by the two entry points below: `mk` / `mv` are the tensor maps of the caller's own K / V (ignored by the
// kernels when m.kv_maps is set). dk / dv cover ALL Tk keys of the global sequence, densely.
static int attn_bwd_launch(const void* q, const CUtensorMap& mk, const CUtensorMap& mv, const void* out, const void* dout,
                           const float* lse, void* dq, void* dk, void* dv, const int* bounds, float* delta, int B, int H,
                           int Hkv, long long ldq, long long ldo, float scale, int causal, const AttnSeqMap& m, int* status,
                           cudaStream_t stream) {
  const int Tq = m.Tq, Tk = m.Tk;
  const long long rows = static_cast<long long>(B) * Tq;
  const long long ld_do = static_cast<long long>(H) * BD;  // dout is dense
  CUtensorMap mq, mdo, mq_sub, mdo_sub;  // *_sub: 64-row boxes for the dK/dV kernel's query sub-tiles
  if (!make_map(&mq_sub, q, rows, H, ldq, SUB)) return -1005;
  if (!make_map(&mdo_sub, dout, rows, H, ld_do, SUB)) return -1006;
  if (!make_map(&mq, q, rows, H, ldq)) return -1001;
  if (!make_map(&mdo, dout, rows, H, ld_do)) return -1004;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKDV_SMEM) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM) != cudaSuccess) return -3;
    configured = true;
  }
  if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dout) & 15u) != 0) return -1;  // 16-byte loads
  if (rows * H > 0x3fffffffLL) return -1;  // the delta kernel indexes (token, head) rows with 32-bit integers
  {
    const long long warps = (rows * H + 2 * kDeltaUnroll - 1) / (2 * kDeltaUnroll);
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
  p.m = m;
  p.H = H;
  p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.causal = causal;
  p.row_lo = bounds;
  p.col_hi = bounds ? bounds + static_cast<long long>(B) * Tq : nullptr;
  p.status = status;
  attn_dkdv_kernel<<<dim3(Tk / BT, Hkv, B), BWD_THREADS, DKDV_SMEM, stream>>>(mq_sub, mk, mv, mdo_sub, p);
  attn_dq_kernel<<<dim3(Tq / BT, H, B), BWD_THREADS, DQ_SMEM, stream>>>(mq, mk, mv, mdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Gradients of ocb_attention_fwd. dout/out/q/dq: [B, Tq, H, D]; k, v, dk, dv: [B, Tk, Hkv, D]; lse: [B, H, Tq] from the
// forward pass; delta: [B, H, Tq] fp32 scratch (written here). dq/dk/dv are written densely (row stride heads * D).
// `bounds` as for ocb_attention_fwd (int32: [B * Tq] row_lo, then [B * Tk] col_hi).
extern "C" int ocb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                 const float* lse, void* dq, void* dk, void* dv, const int* bounds, float* delta, int B,
                                 int Tq, int Tk, int H, int Hkv, int D, long long ldq, long long ldk, long long ldv,
                                 long long ldo, float scale, int causal, int window, int* status, cudaStream_t stream) {
  if (B <= 0 || Tq <= 0) return 0;
  (void)window;
  if (D != BD || Tq > Tk || (Tq % BT) != 0 || (Tk % BT) != 0 || (bounds != nullptr && !causal) || Hkv <= 0 ||
      (H % Hkv) != 0 || delta == nullptr)
    return -5;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -1;
  CUtensorMap mk, mv;
  if (!make_map(&mk, k, static_cast<long long>(B) * Tk, Hkv, ldk)) return -1002;
  if (!make_map(&mv, v, static_cast<long long>(B) * Tk, Hkv, ldv)) return -1003;
  return attn_bwd_launch(q, mk, mv, out, dout, lse, dq, dk, dv, bounds, delta, B, H, Hkv, ldq, ldo, scale, causal,
                         attn_plain_map(Tq, Tk), status, stream);
}

// Gradients of ocb_attention_fwd_sharded (same description of the key / value sources). dk / dv: [B, Tk, Hkv, D] in GLOBAL
// key order on this GPU: the local queries' contribution to every key of the sequence (zero where no local query sees
// a key); the caller sums them over the ranks onto the owners.
extern "C" int ocb_attention_bwd_sharded(const void* q, const void* const* k_srcs, const void* const* v_srcs, int n_src,
                                         int kv_rows_src, const int* layout, const void* out, const void* dout,
                                         const float* lse, void* dq, void* dk, void* dv, const int* bounds, float* delta,
                                         int B, int Tq, int Tk, int H, int Hkv, int D, long long ldq, long long ldk,
                                         long long ldv, long long ldo, float scale, int causal, int* status,
                                         cudaStream_t stream) {
  if (B <= 0 || Tq <= 0) return 0;
  if (D != BD || (Tq % BT) != 0 || (Tk % BT) != 0 || (bounds != nullptr && !causal) || Hkv <= 0 || (H % Hkv) != 0 ||
      delta == nullptr)
    return -5;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -1;
  AttnSeqMap m;
  const int rc = attn_sharded_map(&m, B, Tq, Tk, Hkv, k_srcs, v_srcs, n_src, kv_rows_src, ldk, ldv, layout, stream);
  if (rc != 0) return rc;
  CUtensorMap mk, mv;
  if (!make_map(&mk, k_srcs[0], static_cast<long long>(B) * kv_rows_src, Hkv, ldk)) return -1002;
  if (!make_map(&mv, v_srcs[0], static_cast<long long>(B) * kv_rows_src, Hkv, ldv)) return -1003;
  return attn_bwd_launch(q, mk, mv, out, dout, lse, dq, dk, dv, bounds, delta, B, H, Hkv, ldq, ldo, scale, causal, m, status,
                         stream);
}
