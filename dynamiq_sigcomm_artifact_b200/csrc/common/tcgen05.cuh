// tcgen05 / TMEM / mbarrier / bulk-copy primitives shared by the Hadamard operator
// (kernels/fwht_tcgen05.cu) and the fused collective kernel (kernels/fused_rht_tc.cuh).
//
// Two operand layouts in shared memory, both without swizzle:
//  * K-major: 8-row x 16-byte core matrices; core matrices that are neighbours along K are kLbo bytes
//    apart, 8-row groups kSbo bytes apart.  kLbo = 144 (not 128) staggers the banks so that transposed
//    scalar stores are conflict-free.  A thread that holds four consecutive K values of a row stores them
//    with one 16-byte store.
//  * MN-major (A operand only).  For 32-bit operands the tensor core accepts exactly one MN-major form, the
//    128-byte swizzle with 32-byte atomicity (layout type 1): atoms of 4 K-values x 32 rows, one 128-byte line
//    per K-value, 512 bytes per atom; inside an atom the 32-byte chunk c (rows 8 c .. 8 c + 7) of K-value r sits
//    at r * 128 + ((c ^ r) * 32).  Element (m, k) is at
//        (m / 32) * kMnLbo + (k / 4) * kMnSbo + (k % 4) * 128 + (((m % 32) / 8) ^ (k % 4)) * 32 + (m % 8) * 4.
//    A thread that holds the 32 values of one k for 32 consecutive rows stores them with eight 16-byte stores:
//    this is how an accumulator row read back from TMEM becomes the TRANSPOSED operand of the next pass
//    without scalar stores.  (The unswizzled and the 16-byte-atomicity MN-major forms give all-zero
//    accumulators for TF32 on B200.)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace dq {
namespace tc {

constexpr uint32_t kLbo = 144, kSbo = 8 * kLbo;             // 8 K-chunks of 16 bytes per 8-row group
constexpr uint32_t kOperandBytes = (128 / 8) * kSbo;        // 18432: A operand, 128 rows x 32 tf32
constexpr uint32_t kHBytes = (32 / 8) * kSbo;               // 4608: B operand, 32 rows x 32 tf32
constexpr uint32_t kPollLimit = 1u << 22;

// instruction descriptor: D = F32, A = B = TF32, both K-major, N = 32, M = 128, dense
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescMnA = kIdesc | (1u << 15);         // the same with an MN-major A operand
constexpr uint32_t kMnSbo = 512, kMnLbo = 8 * kMnSbo;       // stride between atoms along K (4 K-values) and along M (32 rows)
constexpr uint32_t kMnOperandBytes = 4 * kMnLbo;            // 16384: A operand, 128 rows x 32 tf32, MN-major

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);   // start address
  d |= static_cast<uint64_t>((kLbo >> 4) & 0x3FFFu) << 16;  // leading (K) byte offset
  d |= static_cast<uint64_t>((kSbo >> 4) & 0x3FFFu) << 32;  // stride (M/N) byte offset
  d |= 1ull << 46;                                          // descriptor version for sm_100
  return d;                                                 // layout type 0: no swizzle
}

// MN-major A operand: leading (M-atom) offset kMnLbo, stride (K-atom) offset kMnSbo, 128-byte swizzle with
// 32-byte atomicity
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((kMnLbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((kMnSbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 1ull << 61;  // layout type 1: 128-byte swizzle, 32-byte atomicity
  return d;
}
// byte offset of the 16-byte chunk that holds rows m .. m+3 (m a multiple of 4) of column k
__device__ __forceinline__ uint32_t mn_chunk_offset(int m, int k) {
  return static_cast<uint32_t>(m >> 5) * kMnLbo + static_cast<uint32_t>(k >> 2) * kMnSbo + (k & 3) * 128 +
         ((((m & 31) >> 3) ^ (k & 3)) << 5) + ((m >> 2) & 1) * 16;
}

// byte offset of element (row, k) of a K-major operand
__device__ __forceinline__ uint32_t operand_offset(int row, int k) {
  return static_cast<uint32_t>(row >> 3) * kSbo + static_cast<uint32_t>(k >> 2) * kLbo + (row & 7) * 16 + (k & 3) * 4;
}

// H_32 (entry (n, k) = +-1 by the parity of popc(n & k)) as a K-major B operand
__device__ __forceinline__ void fill_hadamard32(uint8_t* hmat, int tid, int nthreads) {
  for (int i = tid; i < 32 * 32; i += nthreads) {
    const int n = i >> 5, k = i & 31;
    *reinterpret_cast<float*>(hmat + operand_offset(n, k)) = (__popc(n & k) & 1) ? -1.0f : 1.0f;
  }
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// true when the phase with the given parity has completed; gives up after kPollLimit polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < kPollLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// one bulk (TMA, 1-D) copy from this GPU's global memory into shared memory, completing on `bar`
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier generic accesses of dst precede the copy
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate,
                                         uint32_t idesc = kIdesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
        "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
        "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
        "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
      : "r"(taddr)
      : "memory");
}
// The same load split in two, so that several loads can be in flight under one wait: `tmem_load32_issue`
// starts the load, `tmem_load32_fence` waits for all loads issued so far and ties the registers to the
// wait (a use of r[] cannot be scheduled above it).
__device__ __forceinline__ void tmem_load32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load32_fence(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                 "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {  // one converged warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {  // the warp that allocated
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[128 x 32] (+)= A[128 x 32] . H_32 for one TF32 operand: 4 K-steps of 8 (two core matrices each)
__device__ __forceinline__ void mma_tile_k32(uint32_t tmem_d, uint32_t a, uint32_t b, bool accumulate_first) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    mma_tf32(tmem_d, make_desc(a + ks * 2 * kLbo), make_desc(b + ks * 2 * kLbo), (accumulate_first || ks) ? 1u : 0u);
}

// the same product with A stored MN-major: two K atoms (8 K-values) per step
__device__ __forceinline__ void mma_tile_k32_mn(uint32_t tmem_d, uint32_t a, uint32_t b) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    mma_tf32(tmem_d, make_desc_mn(a + ks * 2 * kMnSbo), make_desc(b + ks * 2 * kLbo), ks ? 1u : 0u, kIdescMnA);
}

}  // namespace tc
}  // namespace dq
