// Shared-memory staging by bulk asynchronous copies (the copy engine behind TMA, 1-D form, one CTA, no
// multicast), used by the persistent kernels of the library: a CTA walks over tiles, and while it computes
// tile n out of one shared-memory buffer the copy engine fills the other with tile n + 1. Bytes in flight cost
// no registers and a tile's load latency hides behind the arithmetic of the tile before it.
//
// Completion is counted on an mbarrier per buffer. EVERY wait is bounded: stage_wait() polls at most
// kStageSpinLimit times, with a 256 ns sleep between polls once the first 4096 have failed (about a second
// in all). A kernel whose wait ran out counts it (its translation unit's g_stage_timeouts), gives the copies
// it still has in flight one more bounded wait so that no copy lands in shared memory the SM has handed to
// another CTA, and returns without writing its remaining tiles. That has never been observed; a non-zero
// count (halo_b200_stage_timeouts) means the outputs of the calls made before it are invalid.
#ifndef HALO_B200_STAGE_CUH_
#define HALO_B200_STAGE_CUH_

#include <cstdint>

namespace halo_b200 {

constexpr unsigned kStageSpinLimit = 1u << 22;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

// One thread: both barriers of a double buffer, one arrival each (the thread that posts the byte count).
__device__ __forceinline__ void stage_init(unsigned long long* bars, int n) {
  for (int i = 0; i < n; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[i])) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One thread: announce `bytes` for the barrier's current phase (and arrive).
__device__ __forceinline__ void stage_expect(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One thread: copy `bytes` (a multiple of 16, both addresses 16-byte aligned) from global memory into this CTA's
// shared memory, completion counted on `bar`.
__device__ __forceinline__ void stage_copy(unsigned smem_dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Bounded wait for phase `parity` of the mbarrier at shared address `bar`; returns 1 when the phase completed.
__device__ __forceinline__ unsigned stage_wait(unsigned bar, unsigned parity) {
  unsigned done = 0;
  for (unsigned spin = 0; spin < kStageSpinLimit && !done; ++spin) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (!done && spin >= 4096) __nanosleep(256);  // the fast path never sleeps; the limit is about a second
  }
  return done;
}

}  // namespace halo_b200

#endif  // HALO_B200_STAGE_CUH_
