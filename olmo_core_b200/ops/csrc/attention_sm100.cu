// Flash attention for sm_100a: tcgen05 tensor-core tiles with TMEM accumulators, operands staged by TMA.
//
// Semantics follow the reference's attention (src/olmo_core/nn/attention/__init__.py:560-640 with the flash
// backends of src/olmo_core/nn/attention/backend.py): softmax(scale * Q K^T + causal mask) V over
// [batch, seq, heads, head_dim] tensors, grouped-query heads, fp32 softmax statistics, bf16 in/out, and the
// per-row log-sum-exp kept for the backward pass.
//
// Forward design (head_dim 128, 128-row tiles):
//   * one CTA per (128 query rows, head, batch); 192 threads = TMA warp + MMA warp + 4 softmax warps (one query
//     row per thread = one TMEM lane per thread, so no cross-thread reductions);
//   * S = Q K^T is a 128x128x128 tcgen05.mma from shared memory into TMEM columns [0,128); the softmax warps read
//     their rows with tcgen05.ld, and write P = exp2(S*scale - m) as packed bf16 back into TMEM columns [0,64)
//     (over the part of S already consumed), from where it is the A operand of the O += P V tcgen05.mma
//     (accumulator in TMEM columns [128,256)) -- P never touches shared memory;
//   * the running maximum is only refreshed when it grows by more than 2^8 (a stale maximum keeps exp2 within range
//     and makes rescaling O, a TMEM read-modify-write, rare);
//   * K and V tiles are single-buffered; overlap comes from two CTAs per SM (96 KB shared memory and 256 TMEM
//     columns each), so one CTA's softmax runs under the other's tensor-core work.
// Every wait is bounded (see common.cuh); a kernel that gives up sets the status word and frees its TMEM.

#include "common.cuh"

#include <mutex>
#include "attn_seq_map.cuh"
#include "ocb_api.h"
#include "tmap.h"

namespace ocb {

// Optional cycle accounting of one CTA's softmax warp (compile with -DOCB_ATTN_PROFILE; read with ocb_attention_fwd_prof_read).
#ifdef OCB_ATTN_PROFILE
__device__ long long g_attn_fwd_prof[16];
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = clock64()
#define PROF_LAP(i) do { const long long now_ = clock64(); prof_acc[i] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_STORE(base, n, cond) do { if (cond) for (int i_ = 0; i_ < (n); ++i_) g_attn_fwd_prof[(base) + i_] = prof_acc[i_]; } while (0)
#else
#define PROF_DECL(n) do {} while (0)
#define PROF_LAP(i) do {} while (0)
#define PROF_STORE(base, n, cond) do {} while (0)
#endif

constexpr int AT_TILE = 128;                       // rows of a Q tile and of a K/V tile
constexpr int AT_D = 128;                          // head dim
constexpr int AT_TILE_BYTES = AT_TILE * AT_D * 2;  // 32 KB
constexpr int AT_HALF_BYTES = AT_TILE_BYTES / 2;   // one [128 x 64] TMA box
constexpr int AT_THREADS = 192;
constexpr int AT_FWD_SMEM = 3 * AT_TILE_BYTES + 1024 + 256;
constexpr uint32_t AT_FWD_TMEM_COLS = 256;
constexpr float AT_RESCALE_THRESHOLD = 8.0f;  // log2 units

struct AttnFwdParams {
  __nv_bfloat16* out;
  float* lse;
  long long ld_out;  // elements between consecutive tokens of `out`
  AttnSeqMap m;  // where query tiles sit in the global sequence and where key / value tiles are fetched from
  int H, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  // Optional per-query lower bound of the visible keys (global key index, int32 [B * Tq], non-decreasing along
  // the sequence): key j is visible to query i iff row_lo[i] <= j (and j <= position of i when causal). It encodes sliding windows
  // and document boundaries at once. nullptr = no lower bound.
  const int* row_lo;
  int* status;
};

// Operand tiles are [128 rows x 128 cols] held as two [128 x 64] boxes. Descriptors are handled as low words (see
// desc_lo_sw128 / umma_ss_lean): stepping through a tile costs the issuing thread one integer add per instruction.
// K-major view (contraction over the columns): k-step k = columns [16k, 16k+16); LBO field unused.
// MN-major view (V: contraction over the kv rows): k-step k = rows [16k, 16k+16); LBO = distance between the two boxes.
constexpr uint32_t kHi = desc_hi_sw128(1024);
__device__ __forceinline__ constexpr uint32_t koff_k(int k) { return ((k >> 2) * AT_HALF_BYTES + (k & 3) * 32) >> 4; }
__device__ __forceinline__ constexpr uint32_t koff_mn(int k) { return (k * 2048) >> 4; }

__global__ void __launch_bounds__(AT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + AT_TILE_BYTES;
  uint8_t* sV = smem + 2 * AT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * AT_TILE_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int gt = attn_q_gtile(p.m, qt);  // the tile's place in the global sequence
  const int q_row0 = b * p.m.Tq + qt * AT_TILE;
  // The bounds are non-decreasing, so the tile's first row has the smallest one (where the key loop starts) and its last
  // row the largest (tiles that start below it need the element-wise mask). `j` below counts tiles from j_lo.
  const int lo_first = p.row_lo ? p.row_lo[q_row0] : 0;
  const int lo_last = p.row_lo ? p.row_lo[q_row0 + AT_TILE - 1] : 0;
  const int j_lo = lo_first / AT_TILE;
  const int n_kv = (p.causal ? gt + 1 : p.m.Tk / AT_TILE) - j_lo;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_FWD_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;        // fp32 scores, columns [0,128)
  const uint32_t tmem_P = tmem_base;        // bf16 probabilities packed two per column, columns [0,64)
  const uint32_t tmem_O = tmem_base + 128;  // fp32 output accumulator, columns [128,256)

  if (warp == 0) {
    // ---------------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_2d(sQ, &tma_q, q_full, h * AT_D, q_row0);
      tma_load_2d(sQ + AT_HALF_BYTES, &tma_q, q_full, h * AT_D + 64, q_row0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t ph = j & 1;
        int src;
        const int kv_row0 = attn_kv_row0(p.m, b, j_lo + j, src);
        const CUtensorMap* mk = attn_k_map(p.m, &tma_k, src);
        const CUtensorMap* mv = attn_v_map(p.m, &tma_v, src);
        ok = mbar_wait_bounded(k_empty, ph ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(k_full, AT_TILE_BYTES);
        tma_load_2d(sK, mk, k_full, hk * AT_D, kv_row0);
        tma_load_2d(sK + AT_HALF_BYTES, mk, k_full, hk * AT_D + 64, kv_row0);
        ok = mbar_wait_bounded(v_empty, ph ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(v_full, AT_TILE_BYTES);
        tma_load_2d(sV, mv, v_full, hk * AT_D, kv_row0);
        tma_load_2d(sV + AT_HALF_BYTES, mv, v_full, hk * AT_D + 64, kv_row0);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(AT_TILE, AT_TILE, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(AT_TILE, AT_D, 0, 1);
      // every k-step descriptor lives in registers: Q, K and V tiles have fixed places in shared memory
      uint64_t dQ_[8], dK_[8], dV_[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        dQ_[k] = pack_u32x2(desc_lo_sw128(smem_u32(sQ), 16) + koff_k(k), kHi);
        dK_[k] = pack_u32x2(desc_lo_sw128(smem_u32(sK), 16) + koff_k(k), kHi);
        dV_[k] = pack_u32x2(desc_lo_sw128(smem_u32(sV), AT_HALF_BYTES) + koff_mn(k), kHi);
      }
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kStatusTimeoutMma);
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t ph = j & 1;
        ok = mbar_wait_bounded(k_full, ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        if (j > 0) {
          // P of the previous tile lives where S is about to be written: wait until O += P V has read it.
          ok = mbar_wait_bounded(o_full, ph ^ 1u, abort_flag, p.status, kStatusTimeoutMma);
          if (!ok) break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k)
          umma_f16_ss(tmem_S, dQ_[k], dK_[k], idesc_qk, k != 0);
        umma_commit(k_empty);
        umma_commit(s_full);
        ok = mbar_wait_bounded(p_full, ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        ok = mbar_wait_bounded(v_full, ph, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc0 = j != 0;
#pragma unroll
        for (int k = 0; k < AT_TILE / 16; ++k)
          umma_f16_ts(tmem_O, tmem_P + k * 8, dV_[k], idesc_pv, k == 0 ? acc0 : 1u);
        umma_commit(v_empty);
        umma_commit(o_full);
      }
    }
  } else {
    // ---------------------------------------------------------------------------------- softmax + epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // query row within the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int my_lo = p.row_lo ? p.row_lo[q_row0 + row] : 0;
    float m_ref = -INFINITY;  // reference maximum (log2 units) the stored probabilities are relative to
    float l = 0.f;
    bool ok = true;
    PROF_DECL(5);
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t ph = j & 1;
      PROF_LAP(4);
      ok = mbar_wait_bounded(s_full, ph, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      PROF_LAP(0);
      tc_fence_after();
      const int kv0 = (j_lo + j) * AT_TILE;
      const bool on_diag = p.causal && j_lo + j == gt;
      const bool diag = on_diag || kv0 < lo_last;  // the tile needs the element-wise mask
      const int hi_col = on_diag ? row : AT_TILE - 1;  // visible columns of this row: [lo_col, hi_col]
      const int lo_col = my_lo - kv0;
      // pass 1: row maximum. The next chunk's TMEM load is in flight while the current chunk is processed.
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;  // four chains instead of one
      uint32_t ra[32], rb[32];
      tmem_ld_32x32(tmem_S + lane_addr, ra);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        tmem_ld_wait();
        if (c < 3) tmem_ld_32x32(tmem_S + lane_addr + (c + 1) * 32, nxt);
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mx0 = fmaxf(mx0, (c * 32 + i > hi_col || c * 32 + i < lo_col) ? -INFINITY : __uint_as_float(cur[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(cur[i]));
            mx1 = fmaxf(mx1, __uint_as_float(cur[i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(cur[i + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(cur[i + 3]));
          }
        }
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      PROF_LAP(1);
      mx *= p.scale_log2;  // the scale is positive, so it commutes with the maximum
      const bool grow = mx > m_ref + AT_RESCALE_THRESHOLD;  // also true for the first tile (m_ref = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_ref;
        const float alpha = grow ? exp2f(m_ref - m_new) : 1.f;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_O + lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tmem_O + lane_addr + c * 32, r);
          }
        }
        l *= alpha;
        m_ref = m_new;
      }
      // pass 2: probabilities relative to m_ref, written as bf16 pairs over the consumed part of S
      PROF_LAP(2);
      const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nm2 = pack_f32x2(-m_ref, -m_ref);
      uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;  // packed fp32 pairs: two adds per instruction, two chains
      tmem_ld_32x32(tmem_S + lane_addr, ra);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        tmem_ld_wait();
        if (c < 3) tmem_ld_32x32(tmem_S + lane_addr + (c + 1) * 32, nxt);
        uint32_t pk[16];
        float p0[16], p1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          unpack_f32x2(fma_f32x2(pack_u32x2(cur[2 * i], cur[2 * i + 1]), sc2, nm2), p0[i], p1[i]);
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
        for (int i = 0; i < 16; i += 2) {
          sum_a = add_f32x2(sum_a, pack_f32x2(p0[i], p1[i]));
          sum_b = add_f32x2(sum_b, pack_f32x2(p0[i + 1], p1[i + 1]));
          pk[i] = pack_bf16x2(p0[i], p1[i]);
          pk[i + 1] = pack_bf16x2(p0[i + 1], p1[i + 1]);
        }
        // P chunk c lands on S columns [16c, 16c+16): all of them were loaded (chunks <= c+1 are in registers)
        tmem_st_32x16(tmem_P + lane_addr + c * 16, pk);
      }
      float sum;
      {
        float s0, s1;
        unpack_f32x2(add_f32x2(sum_a, sum_b), s0, s1);
        sum = s0 + s1;
      }
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      PROF_LAP(3);
    }
    PROF_STORE(0, 5, warp == 2 && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
    if (ok) {
      ok = mbar_wait_bounded(o_full, (n_kv - 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const long long token = static_cast<long long>(q_row0) + row;
      __nv_bfloat16* dst = p.out + token * p.ld_out + h * AT_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_O + lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]) * inv_l, __uint_as_float(r[8 * v + 1]) * inv_l);
          o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) * inv_l, __uint_as_float(r[8 * v + 3]) * inv_l);
          o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) * inv_l, __uint_as_float(r[8 * v + 5]) * inv_l);
          o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) * inv_l, __uint_as_float(r[8 * v + 7]) * inv_l);
          reinterpret_cast<uint4*>(dst + c * 32)[v] = o;
        }
      }
      // natural-log log-sum-exp of the scaled scores
      p.lse[(static_cast<long long>(b) * p.H + h) * p.m.Tq + qt * AT_TILE + row] = m_ref * 0.6931471805599453f + logf(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, AT_FWD_TMEM_COLS);
  }
}

static bool make_qkv_map(CUtensorMap* map, const void* ptr, long long rows, int heads, long long ld) {
  uint64_t dims[2] = {static_cast<uint64_t>(heads) * AT_D, static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(ld) * 2};
  uint32_t box[2] = {64, AT_TILE};
  return get_tensor_map(map, ptr, 2, dims, str, box, 2);
}

}  // namespace ocb

using namespace ocb;

#ifdef OCB_ATTN_PROFILE
extern "C" int ocb_attention_fwd_prof_read(long long* host16) {
  return cudaMemcpyFromSymbol(host16, g_attn_fwd_prof, sizeof(long long) * 16) == cudaSuccess ? 0 : -1;
}
#endif

namespace ocb {

// Device copies of per-source tensor maps: a ring of slots, one per call. A slot is rewritten only after 64 further
// calls, and the copy into it is ordered on the caller's stream behind the kernels that read it.
CUtensorMap* attn_map_ring_slot(const CUtensorMap* host_maps, int count, cudaStream_t stream) {
  constexpr int kSlots = 64, kPerSlot = 2 * ATTN_MAX_SOURCES;
  static CUtensorMap* ring = nullptr;
  static int next = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  if (count > kPerSlot) return nullptr;
  if (ring == nullptr && cudaMalloc(&ring, sizeof(CUtensorMap) * kPerSlot * kSlots) != cudaSuccess) return nullptr;
  CUtensorMap* slot = ring + static_cast<size_t>(next) * kPerSlot;
  next = (next + 1) % kSlots;
  if (cudaMemcpyAsync(slot, host_maps, sizeof(CUtensorMap) * count, cudaMemcpyHostToDevice, stream) != cudaSuccess)
    return nullptr;
  return slot;
}

// Fills `m` from the flat description the C entry points take and builds the per-source K / V maps. Returns 0, or a
// negative code. `layout` = {q_chunk_tiles, q_tile0[0], q_tile0[1], kv_chunk_tiles, n_chunks, then per chunk: source,
// first tile}.
int attn_sharded_map(AttnSeqMap* m, int B, int Tq, int Tk, int Hkv, const void* const* k_srcs, const void* const* v_srcs,
                     int n_src, int kv_rows_src, long long ldk, long long ldv, const int* layout, cudaStream_t stream) {
  if (n_src <= 0 || n_src > ATTN_MAX_SOURCES || layout == nullptr) return -1;
  const int n_chunks = layout[4];
  if (n_chunks <= 0 || n_chunks > ATTN_MAX_KV_CHUNKS || layout[0] <= 0 || layout[3] <= 0) return -1;
  if (layout[3] * n_chunks * AT_TILE != Tk || (kv_rows_src % AT_TILE) != 0) return -1;
  const int q_tiles = Tq / AT_TILE;
  if (q_tiles != layout[0] && q_tiles != 2 * layout[0]) return -1;
  *m = attn_plain_map(Tq, Tk);
  m->q_chunk_tiles = layout[0];
  m->q_tile0[0] = layout[1];
  m->q_tile0[1] = layout[2];
  m->kv_chunk_tiles = layout[3];
  m->kv_rows_src = kv_rows_src;
  for (int c = 0; c < n_chunks; ++c) {
    const int src = layout[5 + 2 * c], t0 = layout[6 + 2 * c];
    if (src < 0 || src >= n_src || t0 < 0 || (t0 + layout[3]) * AT_TILE > kv_rows_src) return -1;
    m->kv_src[c] = static_cast<unsigned char>(src);
    m->kv_tile0[c] = static_cast<short>(t0);
  }
  CUtensorMap maps[2 * ATTN_MAX_SOURCES];
  for (int r = 0; r < n_src; ++r) {
    if (!make_qkv_map(&maps[r], k_srcs[r], static_cast<long long>(B) * kv_rows_src, Hkv, ldk)) return -1002;
    if (!make_qkv_map(&maps[n_src + r], v_srcs[r], static_cast<long long>(B) * kv_rows_src, Hkv, ldv)) return -1003;
  }
  m->n_src = n_src;
  m->kv_maps = attn_map_ring_slot(maps, 2 * n_src, stream);
  return m->kv_maps ? 0 : -3;
}

static int attn_fwd_launch(const void* q, const CUtensorMap& mk, const CUtensorMap& mv, void* out, float* lse,
                           const int* bounds, int B, int H, int Hkv, long long ldq, long long ldo, float scale, int causal,
                           const AttnSeqMap& m, int* status, cudaStream_t stream) {
  CUtensorMap mq;
  if (!make_qkv_map(&mq, q, static_cast<long long>(B) * m.Tq, H, ldq)) return -1001;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_FWD_SMEM) != cudaSuccess) return -3;
    configured = true;
  }
  AttnFwdParams p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.ld_out = ldo;
  p.m = m;
  p.H = H;
  p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.row_lo = bounds;
  p.status = status;
  dim3 grid(m.Tq / AT_TILE, H, B);
  attn_fwd_kernel<<<grid, AT_THREADS, AT_FWD_SMEM, stream>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ocb

// q,out: [B, Tq, H, D]; k,v: [B, Tk, Hkv, D]; bf16, D contiguous, heads contiguous (stride D), tokens `ld*` elements
// apart and batches Tq*ld (Tk*ld) apart. lse: [B, H, Tq] fp32. Supported: D == 128, Tq and Tk multiples of 128 with
// Tq <= Tk (the queries are the LAST Tq positions of the sequence: causal masking is aligned at the end); other cases
// return -5 so that the caller can take another path. Sliding windows and document boundaries are passed as `bounds`:
// int32 [B * Tq] per-query lowest visible key, then [B * Tk] per-key position of the last query that sees it (key indices
// and query positions inside the Tk-long sequence, non-decreasing); they need causal != 0. `window` is unused (folded
// into the bounds by the caller).
extern "C" int ocb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* bounds,
                                 int B, int Tq, int Tk, int H, int Hkv, int D, long long ldq, long long ldk, long long ldv,
                                 long long ldo, float scale, int causal, int window, int* status, cudaStream_t stream) {
  if (B <= 0 || Tq <= 0) return 0;
  (void)window;
  if (D != AT_D || Tq > Tk || (Tq % AT_TILE) != 0 || (Tk % AT_TILE) != 0 || (bounds != nullptr && !causal) || Hkv <= 0 ||
      (H % Hkv) != 0)
    return -5;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -1;
  CUtensorMap mk, mv;
  if (!make_qkv_map(&mk, k, static_cast<long long>(B) * Tk, Hkv, ldk)) return -1002;
  if (!make_qkv_map(&mv, v, static_cast<long long>(B) * Tk, Hkv, ldv)) return -1003;
  return attn_fwd_launch(q, mk, mv, out, lse, bounds, B, H, Hkv, ldq, ldo, scale, causal, attn_plain_map(Tq, Tk), status,
                         stream);
}

// Context-parallel forward: the local queries attend to a sequence whose keys and values are sharded over `n_src`
// buffers (k_srcs[r] / v_srcs[r]: [B, kv_rows_src, Hkv, D] on rank r, as mapped into this GPU's address space; the
// caller's own buffer included). Key / value tiles are read from their owners' memory inside the kernel; the caller
// orders the kernel behind the peers' writes with its own barrier. `layout` is described at attn_sharded_map.
extern "C" int ocb_attention_fwd_sharded(const void* q, const void* const* k_srcs, const void* const* v_srcs, int n_src,
                                         int kv_rows_src, const int* layout, void* out, float* lse, const int* bounds, int B,
                                         int Tq, int Tk, int H, int Hkv, int D, long long ldq, long long ldk, long long ldv,
                                         long long ldo, float scale, int causal, int* status, cudaStream_t stream) {
  if (B <= 0 || Tq <= 0) return 0;
  if (D != AT_D || (Tq % AT_TILE) != 0 || (Tk % AT_TILE) != 0 || (bounds != nullptr && !causal) || Hkv <= 0 || (H % Hkv) != 0)
    return -5;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -1;
  AttnSeqMap m;
  const int rc = attn_sharded_map(&m, B, Tq, Tk, Hkv, k_srcs, v_srcs, n_src, kv_rows_src, ldk, ldv, layout, stream);
  if (rc != 0) return rc;
  CUtensorMap mk, mv;  // unused by the kernel when m.kv_maps is set, but must be valid maps
  if (!make_qkv_map(&mk, k_srcs[0], static_cast<long long>(B) * kv_rows_src, Hkv, ldk)) return -1002;
  if (!make_qkv_map(&mv, v_srcs[0], static_cast<long long>(B) * kv_rows_src, Hkv, ldv)) return -1003;
  return attn_fwd_launch(q, mk, mv, out, lse, bounds, B, H, Hkv, ldq, ldo, scale, causal, m, status, stream);
}
