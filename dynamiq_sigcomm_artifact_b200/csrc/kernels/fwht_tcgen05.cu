// Randomized Walsh-Hadamard transform of 1024-element blocks on the 5th-generation tensor
// cores (tcgen05 + TMEM), fed by bulk (TMA) copies.
//
// H_1024 = H_32 (x) H_32, so a block seen as a 32 x 32 matrix X transforms as Z = H X H.
// Four blocks form one 128 x 32 tile.  Two tcgen05.mma passes with the same constant B = H_32:
//   pass 1:  D1 = A1 . H,  A1[row, k] = s * X[row][k]          (rows of the tile, K-major)
//   pass 2:  D2 = A2 . H,  A2[(b, c), k] = D1[(b, k)][c]       (each block transposed)
// so that thread (b, c) ends with Z_b[n][c], n = 0..31, read back from TMEM with tcgen05.ld.
// fp32 inputs are split into two TF32 terms (hi = x with the low 13 mantissa bits cleared,
// lo = x - hi), each pass accumulating both in fp32: H has entries +-1, exact in TF32.
//
// Stands where the reference has its shared-memory / radix-8 global Hadamard kernels
// (cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hadamard.cu:66-274), used by its THC hook
// (testbed_evaluation/new_comm_hooks/thc_hooks.py:124-149).
//
// Every wait (bulk-copy barrier, MMA-commit barrier) is bounded; on expiry the CTA records an
// error, skips its remaining tiles, frees its TMEM columns and returns.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include "../common/philox.cuh"
#include "../common/tcgen05.cuh"

namespace dq {
namespace {

using namespace tc;

constexpr int kTileRows = 128, kTileCols = 32, kTileElems = kTileRows * kTileCols;  // 4 blocks
constexpr int kThreads = 128;
constexpr uint32_t kStageBytes = kTileElems * 4;                 // 16384
constexpr uint32_t kTmemCols = 64;                               // D1 in columns 0..31, D2 in 32..63

enum : int { kFwhtOk = 0, kFwhtCopyTimeout = 1, kFwhtMmaTimeout = 2 };

// One pass: 4 K-steps for the hi operand, 4 for lo.
__device__ __forceinline__ void issue_pass(uint32_t tmem_d, uint32_t a_hi, uint32_t a_lo, uint32_t b, uint64_t* bar) {
  mma_tile_k32(tmem_d, a_hi, b, false);
  mma_tile_k32(tmem_d, a_lo, b, true);
  mma_commit(bar);
}

__global__ void __launch_bounds__(kThreads) fwht1024_tcgen05_kernel(const float* __restrict__ in,
                                                                    float* __restrict__ out, long long ntiles,
                                                                    uint32_t seed_lo, uint32_t seed_hi, uint32_t step,
                                                                    uint32_t bucket, int apply_signs, float scale,
                                                                    int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* a_hi = smem;
  uint8_t* a_lo = a_hi + kOperandBytes;
  uint8_t* hmat = a_lo + kOperandBytes;
  float* stage = reinterpret_cast<float*>(hmat + kHBytes);  // 2 x 16 KiB
  uint32_t* sign_words = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(stage) + 2 * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sign_words + 32);  // [0,1]: stage full, [2]: mma done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // constants: H_32 and the sign words
  fill_hadamard32(hmat, tid, kThreads);
  if (tid < 32) sign_words[tid] = apply_signs ? sign_word(tid, step, bucket, seed_lo, seed_hi) : 0u;
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    s_abort = 0;
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (warp == 0) tmem_alloc(tmem_slot, kTmemCols);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // H_32 written by threads, read by the MMA
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  uint32_t full_parity[2] = {0, 0}, mma_parity = 0;
  long long tile = blockIdx.x;
  int buf = 0;
  if (tid == 0 && tile < ntiles) bulk_load(stage, in + tile * kTileElems, kStageBytes, &bars[0]);

  for (; tile < ntiles; tile += gridDim.x, buf ^= 1) {
    const long long next = tile + gridDim.x;
    if (tid == 0 && next < ntiles)
      bulk_load(stage + (buf ^ 1) * kTileElems, in + next * kTileElems, kStageBytes, &bars[buf ^ 1]);
    bool ok = mbar_wait(&bars[buf], full_parity[buf]);
    full_parity[buf] ^= 1u;
    if (!ok) atomicExch(&s_abort, kFwhtCopyTimeout);
    __syncthreads();
    if (s_abort) break;

    // ---- pass 1 operand: signed, sanitised, split input in K-major core matrices ----
    const float* st = stage + buf * kTileElems;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + kThreads * i;  // float4 index inside the tile: coalesced, conflict-free
      const int row = idx >> 3, c4 = idx & 7;
      float4 x = *reinterpret_cast<const float4*>(st + idx * 4);
      const uint32_t sw = sign_words[(row & 31)];  // element (row % 32) * 32 + col -> word row % 32, bit col
      float v[4] = {x.x, x.y, x.z, x.w}, hi[4], lo[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f = (fabsf(v[k]) <= 3.402823466e38f) ? v[k] : 0.0f;
        f = __uint_as_float(__float_as_uint(f) ^ (((sw >> (c4 * 4 + k)) & 1u) << 31));
        hi[k] = __uint_as_float(__float_as_uint(f) & 0xFFFFE000u);
        lo[k] = f - hi[k];
      }
      const uint32_t off = operand_offset(row, c4 * 4);
      *reinterpret_cast<float4*>(a_hi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<float4*>(a_lo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_pass(tmem_base, smem_u32(a_hi), smem_u32(a_lo), smem_u32(hmat), &bars[2]);
    }
    ok = mbar_wait(&bars[2], mma_parity);
    mma_parity ^= 1u;
    if (!ok) atomicExch(&s_abort, kFwhtMmaTimeout);
    __syncthreads();
    if (s_abort) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- pass 2 operand: D1 read back, each block transposed: A2[(b, c), k = r] = D1[(b, r)][c] ----
    float d[32];
    tmem_load32(tmem_lane, d);
    {
      const int b32 = warp * 32, r = lane;  // this thread holds row (b, r) of D1
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float hi = __uint_as_float(__float_as_uint(d[c]) & 0xFFFFE000u);
        const uint32_t off = operand_offset(b32 + c, r);
        *reinterpret_cast<float*>(a_hi + off) = hi;
        *reinterpret_cast<float*>(a_lo + off) = d[c] - hi;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_pass(tmem_base + 32, smem_u32(a_hi), smem_u32(a_lo), smem_u32(hmat), &bars[2]);
    }
    ok = mbar_wait(&bars[2], mma_parity);
    mma_parity ^= 1u;
    if (!ok) atomicExch(&s_abort, kFwhtMmaTimeout);
    __syncthreads();
    if (s_abort) break;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- result: thread (b, c) holds Z_b[n][c]; element index inside the block = 32 n + c ----
    tmem_load32(tmem_lane + 32, d);
    float* o = out + tile * kTileElems + warp * 1024 + lane;
#pragma unroll
    for (int n = 0; n < 32; ++n) o[n * 32] = d[n] * scale;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // TMEM and the operand buffers are free for the next tile
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  if (s_abort) {
    if (tid == 0) atomicCAS(status, kFwhtOk, s_abort);
    // the other stage buffer may still have a copy in flight: give it a bounded chance to land
    if (tid == 0) mbar_wait(&bars[buf ^ 1], full_parity[buf ^ 1]);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

constexpr size_t kSmemBytes = 2 * kOperandBytes + kHBytes + 2 * kStageBytes + 32 * 4 + 3 * 8 + 16;

}  // namespace

// y = H_1024 (s * x) * scale for every 1024-element block of x (fp32, numel a multiple of 4096).
// With apply_signs the Rademacher diagonal of (seed, step, bucket) is applied first.
// Returns (y, status) - status is a one-element int32 tensor, 0 when every wait completed.
std::tuple<at::Tensor, at::Tensor> fwht1024_tcgen05(at::Tensor x, int64_t seed, int64_t step, int64_t bucket,
                                                    bool apply_signs, double scale, int64_t ctas) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kFloat, "fwht: contiguous fp32 CUDA tensor");
  TORCH_CHECK(x.numel() % kTileElems == 0, "fwht: numel must be a multiple of 4096 (four 1024-element blocks)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "fwht: input must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  at::Tensor status = at::zeros({1}, x.options().dtype(at::kInt));
  const long long ntiles = x.numel() / kTileElems;
  if (ntiles == 0) return {y, status};
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(fwht1024_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemBytes)));
    configured = true;
  }
  int dev = 0, sms = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long want = ctas > 0 ? ctas : 3LL * sms;
  const int grid = static_cast<int>(std::min<long long>(ntiles, want));
  auto stream = at::cuda::getCurrentCUDAStream();
  const uint64_t s = static_cast<uint64_t>(seed);
  fwht1024_tcgen05_kernel<<<grid, kThreads, kSmemBytes, stream>>>(
      x.data_ptr<float>(), y.data_ptr<float>(), ntiles, static_cast<uint32_t>(s & 0xFFFFFFFFull),
      static_cast<uint32_t>(s >> 32), static_cast<uint32_t>(step), static_cast<uint32_t>(bucket), apply_signs ? 1 : 0,
      static_cast<float>(scale), status.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, status};
}

}  // namespace dq
