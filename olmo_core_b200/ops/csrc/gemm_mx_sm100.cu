// Block-scaled (MX) e4m3 GEMM for sm_100a: tcgen05.mma.kind::mxf8f6f4.block_scale with the E8M0 scale factors of both
// operands in tensor memory, so the 32-element scales are applied by the tensor core itself and not in an epilogue.
//
//   C[M, N] (=|+=) sum_k  A_q[m, k] 2^(sa[m, k/32] - 127)  *  B_q[n, k] 2^(sb[n, k/32] - 127)
//
// A_q [M, K] and B_q [N, K] are e4m3 bytes, K-major (K % 128 == 0); the scales arrive in the 512-byte block layout that
// mx_quant_sm100.cu writes. This is the GEMM behind the reference's MXLinear (torchao, cuBLAS MXFP8 kernels:
// src/olmo_core/float8/ao.py:190-239); the three products of a linear layer use it with operands quantised along their
// own reduction dimension (see ops/mx.py).
//
// CTA layout (192 threads): warp 0 = producer (two TMA tile loads and three 512-byte bulk copies of scales per stage),
// warp 1 = issuer (per stage: three tcgen05.cp of the scales from shared to tensor memory, four K=32 MMAs whose
// instruction descriptors select scale byte 0..3), warps 2..5 = epilogue. Tile 128 x 192 x 128: two 192-column fp32
// accumulators leave tensor-memory columns for the scales (4 for A, 8 for the two 128-row blocks that a 192-row B tile
// can touch), and the epilogue of one tile overlaps the main loop of the next. Copies and MMAs issued by one thread
// execute in issue order, so one set of scale columns serves every stage. All waits are bounded (common.cuh).

#include "common.cuh"
#include "ocb_api.h"
#include "tmap.h"

namespace ocb {
namespace mxg {

constexpr int BM = 128;
constexpr int BN = 192;
constexpr int BKE = 128;  // reduction elements (= bytes) per stage: one 128-byte swizzle line per row
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BKE;
constexpr int B_BYTES = BN * BKE;
constexpr int TILE_BYTES = A_BYTES + B_BYTES;  // 40 KB, a multiple of 1024
constexpr int SF_BLOCK = 512;                  // scales of 128 rows x 128 reduction elements
constexpr int SF_BYTES = 3 * SF_BLOCK;         // A block, two B blocks
constexpr int SMEM_BYTES = STAGES * (TILE_BYTES + SF_BYTES) + 1024 + 256;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SFA_COL = 2 * BN;       // 384
constexpr uint32_t SFB_COL = SFA_COL + 4;  // 388..395

enum : int { EPI_BF16 = 0, EPI_F32_ACC = 1, EPI_F32 = 2 };

struct Params {
  void* C;
  long long ldc;
  int M, N, K;
  int group_m;
  const uint8_t* sfa;  // [ceil(M/128)][K/128][512]
  const uint8_t* sfb;  // [ceil(N/128)][K/128][512]
  int* status;
};

// kind::mxf8f6f4 instruction descriptor: e4m3 A and B (format 0), both K-major, N >> 3 at bit 17, E8M0 scales (bit 23),
// M >> 4 at bit 24; the scale byte used by this K=32 step goes to bits [29,31) for A and [4,6) for B.
__host__ __device__ constexpr uint32_t idesc_mx(int m, int n, uint32_t sf_id) {
  return (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24) | (sf_id << 29) |
         (sf_id << 4);
}

// Shared-memory descriptor of one 512-byte scale block for tcgen05.cp: no swizzle, 8-row x 16-byte core matrices that
// follow each other every 128 bytes (SBO); a single 16-byte column, so the leading offset is unused.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(128u >> 4) << 32) | (1ull << 46);
}
// 32 rows x 16 bytes from shared memory into 4 tensor-memory columns, replicated to the four 32-lane quadrants.
__device__ __forceinline__ void sf_copy(uint32_t tmem_dst, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                        uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %7, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %4, [%5], [%6], p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ bool next_tile(int tile, const Params& p, int& m0, int& n0) {
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  if (tile >= tiles_m * tiles_n) return false;
  const int per_group = p.group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gm = min(tiles_m - first_m, p.group_m);
  const int r = tile - g * per_group;
  m0 = (first_m + r % gm) * BM;
  n0 = (r / gm) * BN;
  return true;
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + STAGES * TILE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sf_smem + STAGES * SF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = p.K / BKE;
  const int n_blocks = (p.N + 127) >> 7;

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
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int m0, n0;
      for (int tile = blockIdx.x; ok && next_tile(tile, p, m0, n0); tile += gridDim.x) {
        const uint8_t* sfa_row = p.sfa + static_cast<long long>(m0 >> 7) * num_kb * SF_BLOCK;
        const int nb0 = n0 >> 7, nb1 = min(nb0 + 1, n_blocks - 1);  // past the end: any block (those columns are not stored)
        const uint8_t* sfb_row0 = p.sfb + static_cast<long long>(nb0) * num_kb * SF_BLOCK;
        const uint8_t* sfb_row1 = p.sfb + static_cast<long long>(nb1) * num_kb * SF_BLOCK;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer);
          if (!ok) break;
          uint8_t* sa = smem + stage * TILE_BYTES;
          uint8_t* ss = sf_smem + stage * SF_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], TILE_BYTES + SF_BYTES);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * BKE, m0);
          tma_load_2d(sa + A_BYTES, &tma_b, &full_bar[stage], kb * BKE, n0);
          bulk_load_1d(ss, sfa_row + kb * SF_BLOCK, SF_BLOCK, &full_bar[stage]);
          bulk_load_1d(ss + SF_BLOCK, sfb_row0 + kb * SF_BLOCK, SF_BLOCK, &full_bar[stage]);
          bulk_load_1d(ss + 2 * SF_BLOCK, sfb_row1 + kb * SF_BLOCK, SF_BLOCK, &full_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      constexpr uint32_t kDescHi = desc_hi_sw128(1024);
      const uint32_t a_lo0 = desc_lo_sw128(smem_u32(smem), 16);
      const uint32_t b_lo0 = desc_lo_sw128(smem_u32(smem) + A_BYTES, 16);
      const uint32_t sf0 = smem_u32(sf_smem);
      const uint32_t tsfa = tmem_base + SFA_COL;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0, m0, n0;
      for (int tile = blockIdx.x; ok && next_tile(tile, p, m0, n0); tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // the tile starts 0 or 64 rows into its first 128-row scale block: 32 rows per tensor-memory column
        const uint32_t tsfb = tmem_base + SFB_COL + static_cast<uint32_t>((n0 & 127) >> 5);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kStatusTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ss = sf0 + stage * SF_BYTES;
          sf_copy(tmem_base + SFA_COL, sf_desc(ss));
          sf_copy(tmem_base + SFB_COL, sf_desc(ss + SF_BLOCK));
          sf_copy(tmem_base + SFB_COL + 4, sf_desc(ss + 2 * SF_BLOCK));
          const uint32_t a_lo = a_lo0 + stage * (TILE_BYTES >> 4), b_lo = b_lo0 + stage * (TILE_BYTES >> 4);
#pragma unroll
          for (uint32_t k = 0; k < BKE / 32; ++k) {
            // K = 32 elements = 32 bytes of the swizzled line per step; scale byte k of the stage's columns
            umma_mx(d_tmem, a_lo + 2 * k, b_lo + 2 * k, kDescHi, idesc_mx(BM, BN, k), tsfa | (k << 30), tsfb | (k << 30),
                    (kb | static_cast<int>(k)) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    bool ok = true;
    int it = 0, m0, n0;
    for (int tile = blockIdx.x; ok && next_tile(tile, p, m0, n0); tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (!row_ok || col >= p.N) continue;
        if (EPI == EPI_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col;
          if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              reinterpret_cast<uint4*>(dst)[v] = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
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

template <int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_mx_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_mx_kernel<EPI><<<grid, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace mxg
}  // namespace ocb

using namespace ocb;

extern "C" int ocb_gemm_mx(const void* A, const void* B, void* C, const void* sfa, const void* sfb, int M, int N, int K,
                           long long lda, long long ldb, long long ldc, int epilogue, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % mxg::BKE) != 0 || (lda % 16) != 0 || (ldb % 16) != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    return -1;
  if (sfa == nullptr || sfb == nullptr) return -1;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda)};
    uint32_t box[2] = {128, static_cast<uint32_t>(mxg::BM)};
    if (!get_tensor_map(&ta, A, 2, dims, str, box, 1)) return -1001;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb)};
    uint32_t box[2] = {128, static_cast<uint32_t>(mxg::BN)};
    if (!get_tensor_map(&tb, B, 2, dims, str, box, 1)) return -2001;
  }
  mxg::Params p;
  p.C = C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.group_m = 8;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa);
  p.sfb = reinterpret_cast<const uint8_t*>(sfb);
  p.status = status;
  switch (epilogue) {
    case mxg::EPI_BF16: return mxg::launch<mxg::EPI_BF16>(ta, tb, p, stream);
    case mxg::EPI_F32_ACC: return mxg::launch<mxg::EPI_F32_ACC>(ta, tb, p, stream);
    case mxg::EPI_F32: return mxg::launch<mxg::EPI_F32>(ta, tb, p, stream);
    default: return -1;
  }
}
