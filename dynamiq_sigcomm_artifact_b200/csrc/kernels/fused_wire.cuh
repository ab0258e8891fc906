// Flags, bounded waits and work-split helpers shared by the bodies of the persistent all-reduce kernel.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "../common/tcgen05.cuh"
#include "fused_allreduce.cuh"

namespace dq {

constexpr int kWireBlock = 1024;  // elements of a codec block

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const uint32_t* p) { return __ldcg(p); }

// Wait until *flag reaches `epoch`; false when the budget ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long budget_ns) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = now_ns();
  unsigned spins = 0;
  for (;;) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((++spins & 63u) == 0) {
      if (now_ns() - t0 > budget_ns) return false;
      __nanosleep(64);
    }
  }
}

// ---- per-warp bulk prefetch (TMA engine, 1-D form) of the next raw block --------------------
// Lane 0 arms the warp's mbarrier with the byte count and issues one cp.async.bulk of a whole
// block (4 KiB fp32 / 2 KiB bf16) from this GPU's own bucket into the warp's staging buffer; the
// warp later waits on the barrier's phase (bounded) and reads the block from shared memory.

using tc::mbar_init;
using tc::mbar_wait;
__device__ __forceinline__ void bulk_prefetch(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  tc::bulk_load(dst_smem, src_gmem, bytes, bar);
}

// [lo, hi) of CTA `cta` inside the shard of step s, and the shard's first block
__device__ __forceinline__ void step_range(const ARParams& p, int s, int cta, int per_cta, int& shard_lo, int& lo,
                                           int& hi) {
  const int shard = p.steps[s][0];
  shard_lo = min(shard * p.blocks_per_shard, p.nblocks);
  const int shard_hi = min(shard_lo + p.blocks_per_shard, p.nblocks);
  lo = min(shard_lo + cta * per_cta, shard_hi);
  hi = min(lo + per_cta, shard_hi);
}

// first writer wins: (code, step, CTA, slot) in the status words
__device__ __forceinline__ void report_failure(const ARParams& p, uint32_t code, int s, int slot) {
  if (atomicCAS(p.status, kOk, code) == kOk) {
    p.status[1] = (static_cast<uint32_t>(s) << 16) | static_cast<uint32_t>(blockIdx.x);
    p.status[2] = static_cast<uint32_t>(slot);
  }
}

// Debug mode: true if this thread found a slot index of step s outside the set, or a block of the CTA's range
// [lo, hi) whose encoded bytes would leave its slot.  Fixed-width codecs: block i of the shard sits at
// i * block_bytes.  Plan-driven codecs (PLAN_UNIT = 8: superchunk records of mixed width, 128: rotation codes
// of mixed width) read offsets from device memory, which no host-side check sees.  Threads stride the range.
template <int PLAN_UNIT, bool HAS_SCALES>
__device__ __forceinline__ bool debug_step_out_of_bounds(const ARParams& p, int s, int shard_lo, int lo, int hi,
                                                         int& bad_slot) {
  const int recv_slot = p.steps[s][2], nrecv = p.steps[s][3], out = p.steps[s][4], send_slot = p.steps[s][6];
  bool bad = false;
  bad_slot = -1;
  if (nrecv > 0 && (recv_slot < 0 || recv_slot + nrecv > p.nslots)) bad = true, bad_slot = recv_slot;
  if ((out == kOutSend || out == kOutFinal) && (send_slot < 0 || send_slot >= p.nslots)) bad = true, bad_slot = send_slot;
  if (static_cast<unsigned long long>(p.nslots) * p.slot_stride > p.set_bytes) bad = true;
  const unsigned long long payload_end = HAS_SCALES ? p.scales_off : p.slot_stride;
  for (int blk = lo + static_cast<int>(threadIdx.x); blk < hi && !bad; blk += static_cast<int>(blockDim.x)) {
    unsigned long long off, bytes;
    if constexpr (PLAN_UNIT > 0) {
      const uint32_t base = __ldg(p.sc_plan + shard_lo), o0 = __ldg(p.sc_plan + blk), o1 = __ldg(p.sc_plan + blk + 1);
      if (o0 < base || o1 < o0) bad = true;
      off = static_cast<unsigned long long>(o0 - base) * PLAN_UNIT;
      bytes = static_cast<unsigned long long>(o1 - o0) * PLAN_UNIT;
      if constexpr (PLAN_UNIT == 128) {  // one width (2..8) per block, 128 bytes per bit of width
        const uint32_t wb = __ldg(p.sc_plan + p.nblocks + 1 + blk);
        if (wb < 2u || wb > 8u || o1 - o0 != wb) bad = true;
      }
    } else {
      off = static_cast<unsigned long long>(blk - shard_lo) * p.block_bytes;
      bytes = p.block_bytes;
    }
    if (off + bytes > payload_end) bad = true;
    if (HAS_SCALES && p.scales_off + 4ull * static_cast<unsigned long long>(blk - shard_lo + 1) > p.slot_stride) bad = true;
  }
  return bad;
}

}  // namespace dq
