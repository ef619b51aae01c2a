// Cross-GPU barrier on a CUDA stream over symmetric (peer-mapped) memory, with a deadline.
//
// Every rank owns one row of 32-bit flags per channel in a symmetric buffer: flags[channel][r] is the last epoch
// that rank r has announced to this GPU. A barrier at epoch e is one tiny kernel: thread r publishes e into
// rank r's copy of flags[channel][my_rank] with a system-scope release store (so everything this GPU wrote before the
// barrier is visible to a peer that acquires the flag), then polls its own flags[channel][r] with system-scope acquire
// loads until it holds e or a later epoch. Epochs only grow, so a fast peer that has already announced e + 1 is fine.
//
// The wait is bounded: after `timeout_ns` of %globaltimer the kernel records kStatusTimeoutPeerFlag in the status word
// and returns normally. The context stays usable; the host sees the failure in check_device_status() (the reference
// has no counterpart: its NCCL collectives hang until the process-group watchdog kills the job).
// Plain ld / st only: no multimem and no TMA, so a rank that has left the job cannot raise faults on its peers.

#include "common.cuh"
#include "ocb_api.h"

namespace ocb {
namespace {

constexpr int kBarrierMaxRanks = 16;

struct FlagPtrs {
  uint32_t* p[kBarrierMaxRanks];  // base of every rank's flag array, as mapped on this GPU
};

__device__ __forceinline__ void st_release_sys(uint32_t* ptr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* ptr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}

// skip_signal_rank: a rank that must NOT be signalled (-1: none). Only the tests use it, to let a wait run out.
__global__ void peer_barrier_kernel(FlagPtrs flags, int world, int rank, int channel, uint32_t epoch,
                                    unsigned long long timeout_ns, int skip_signal_rank, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const int slot = channel * kBarrierMaxRanks;
  __threadfence_system();
  if (r != skip_signal_rank) st_release_sys(flags.p[r] + slot + rank, epoch);
  const uint32_t* mine = flags.p[rank] + slot + r;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
    if ((++spins & 0x3Fu) == 0) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status != nullptr) atomicCAS(status, 0, kStatusTimeoutPeerFlag);
        return;
      }
      __nanosleep(200);
    }
  }
}

}  // namespace
}  // namespace ocb

using namespace ocb;

// Number of 32-bit words a rank's flag array needs (channels x ranks).
extern "C" int ocb_peer_barrier_flag_words(void) { return 8 * kBarrierMaxRanks; }

// flag_ptrs: `world` pointers, entry r = rank r's flag array (zero-initialised, ocb_peer_barrier_flag_words() words) as
// mapped on this GPU. epoch: 1, 2, 3, ... identical on all ranks for one barrier. Returns 0 or a negative launch error;
// a wait that ran out is reported through `status` (code 4), not here.
extern "C" int ocb_peer_barrier(void* const* flag_ptrs, int world, int rank, int channel, unsigned int epoch,
                                long long timeout_ms, int skip_signal_rank, int* status, cudaStream_t stream) {
  if (world < 1 || world > kBarrierMaxRanks || rank < 0 || rank >= world || channel < 0 || channel >= 8) return -1;
  FlagPtrs f;
  for (int r = 0; r < world; ++r) f.p[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  const unsigned long long ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 1) * 1000000ull;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(f, world, rank, channel, epoch, ns, skip_signal_rank, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
