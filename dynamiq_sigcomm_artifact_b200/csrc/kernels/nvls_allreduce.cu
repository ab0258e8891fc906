// Uncompressed all-reduce through the NVSwitch's in-switch reduction (NVLS): multimem.ld_reduce pulls one value
// from every rank's copy and adds them inside the switch, multimem.st writes the result to every rank's copy.
//
// One cooperative launch per bucket:
//   1. bucket (fp32 or bf16) -> this rank's staging buffer S in wire precision (bf16 or fp32)
//   2. barrier over the ranks (release / acquire flags in peer memory, bounded waits)
//   3. this rank's 1/W slice of S: multimem.ld_reduce (sum over the ranks, fp32 accumulation) -> multimem.st (to all)
//   4. barrier over the ranks
//   5. S -> bucket, times the post-scale (1 / W for the mean)
// S, the flags and the multicast mapping of S come from the caller (torch.distributed symmetric memory).  Per
// rank the switch moves ~2 x the wire size of the bucket, against 2 (W - 1) / W x for a ring plus its hops.
//
// The reference has no counterpart: its uncompressed baselines are the library all-reduce
// (testbed_evaluation/new_comm_hooks/comm_hooks.py:175-212 runs bf16 through its own ring).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

#include "../common/rht_codec.cuh"
#include "fused_wire.cuh"

namespace dq {
namespace {

namespace cg = cooperative_groups;

struct NvlsParams {
  void* bucket;
  long long n;             // elements of the bucket
  long long n_pad;         // elements of S in use: n rounded up to 8 * world
  uint8_t* stage;          // this rank's S
  uint8_t* mc;             // multicast address of S
  uint32_t* flags[kMaxWorld];  // every rank's flag words (peer mapped); flags[rank] is local
  int world, rank;
  uint32_t epoch;          // this call uses epoch and epoch + 1
  float post_scale;
  unsigned long long timeout_ns;
  uint32_t* status;        // local, 4 words
};

__device__ __forceinline__ void mm_ld_reduce_f32(const void* addr, float (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3])
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void mm_st_f32(void* addr, const float (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v[0]), "f"(v[1]),
               "f"(v[2]), "f"(v[3])
               : "memory");
}
__device__ __forceinline__ void mm_ld_reduce_bf16(const void* addr, uint32_t (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void mm_st_bf16(void* addr, const uint32_t (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

// All ranks have reached this point and their earlier writes are visible.  CTA 0 talks to the peers; the
// grid-wide syncs around it hold the other CTAs.  Returns false (on every thread of the grid) after a timeout.
__device__ bool rank_barrier(const NvlsParams& p, uint32_t epoch, cg::grid_group& grid, uint32_t* abort_word) {
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    const int t = threadIdx.x;
    if (t < p.world && t != p.rank) st_release_sys(p.flags[t] + p.rank, epoch);
    if (t < p.world && t != p.rank && !wait_flag(p.flags[p.rank] + t, epoch, p.timeout_ns)) {
      if (atomicCAS(p.status, kOk, kErrWaitTimeout) == kOk) {
        p.status[1] = 0;
        p.status[2] = static_cast<uint32_t>(t);
      }
      atomicExch(abort_word, 1u);
    }
  }
  grid.sync();
  __threadfence_system();
  return *reinterpret_cast<volatile uint32_t*>(abort_word) == 0u;
}

template <typename T, int WIRE>
__global__ void __launch_bounds__(512, 1) nvls_allreduce_kernel(const __grid_constant__ NvlsParams p) {
  cg::grid_group grid = cg::this_grid();
  uint32_t* abort_word = p.status + 3;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const T* in = static_cast<const T*>(p.bucket);
  T* out = static_cast<T*>(p.bucket);
  constexpr int kWireBytes = WIRE / 8;

  // 1. bucket -> S, eight elements per thread and step
  for (long long i = tid * 8; i < p.n_pad; i += nthreads * 8) {
    float v[8];
    if (i + 8 <= p.n) {  // the bucket is 16-byte aligned (checked by the host)
      if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(in + i), b = *reinterpret_cast<const float4*>(in + i + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
      } else {
        const uint4 q = *reinterpret_cast<const uint4*>(in + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = __uint_as_float(w[k] << 16);
          v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = (i + k < p.n) ? Elem<T>::to_float(in[i + k]) : 0.0f;
    }
    if constexpr (WIRE == 16) {
      uint4 q;
      __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
      __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
      q.x = *reinterpret_cast<uint32_t*>(&a), q.y = *reinterpret_cast<uint32_t*>(&b);
      q.z = *reinterpret_cast<uint32_t*>(&c), q.w = *reinterpret_cast<uint32_t*>(&d);
      *reinterpret_cast<uint4*>(p.stage + i * kWireBytes) = q;
    } else {
      *reinterpret_cast<float4*>(p.stage + i * kWireBytes) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(p.stage + (i + 4) * kWireBytes) = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  bool ok = rank_barrier(p, p.epoch, grid, abort_word);

  // 3. this rank's slice: in-switch sum, result to every rank
  if (ok) {
    const long long per = p.n_pad / p.world;  // a multiple of 8
    const long long lo = p.rank * per, hi = lo + per;
    constexpr int kPer16 = 16 / kWireBytes;  // elements per 16-byte access
    constexpr int kUnroll = 4;               // reductions in flight per thread: the round trip through the switch is long
    const long long stride = nthreads * kPer16;
    for (long long i0 = lo + tid * kPer16; i0 < hi; i0 += stride * kUnroll) {
      if constexpr (WIRE == 16) {
        uint32_t v[kUnroll][4];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i0 + u * stride < hi) mm_ld_reduce_bf16(p.mc + (i0 + u * stride) * kWireBytes, v[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i0 + u * stride < hi) mm_st_bf16(p.mc + (i0 + u * stride) * kWireBytes, v[u]);
      } else {
        float v[kUnroll][4];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i0 + u * stride < hi) mm_ld_reduce_f32(p.mc + (i0 + u * stride) * kWireBytes, v[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i0 + u * stride < hi) mm_st_f32(p.mc + (i0 + u * stride) * kWireBytes, v[u]);
      }
    }
  }
  ok = rank_barrier(p, p.epoch + 1, grid, abort_word) && ok;

  // 5. S -> bucket
  if (ok) {
    for (long long i = tid * 8; i < p.n; i += nthreads * 8) {
      float v[8];
      if constexpr (WIRE == 16) {
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(p.stage + i * kWireBytes));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = __uint_as_float(w[k] << 16);
          v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
      } else {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.stage + i * kWireBytes));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(p.stage + (i + 4) * kWireBytes));
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= p.post_scale;
      if (i + 8 <= p.n) {
        if constexpr (sizeof(T) == 4) {
          *reinterpret_cast<float4*>(out + i) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(out + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          uint4 q;
          __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
          __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
          q.x = *reinterpret_cast<uint32_t*>(&a), q.y = *reinterpret_cast<uint32_t*>(&b);
          q.z = *reinterpret_cast<uint32_t*>(&c), q.w = *reinterpret_cast<uint32_t*>(&d);
          *reinterpret_cast<uint4*>(out + i) = q;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (i + k < p.n) out[i + k] = Elem<T>::from_float(v[k]);
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *abort_word = 0u;  // the word is per call; the error code stays
}

template <typename T, int WIRE>
void launch_nvls(const NvlsParams& p, int ctas, cudaStream_t stream) {
  const void* fn = reinterpret_cast<const void*>(&nvls_allreduce_kernel<T, WIRE>);
  int dev = 0, sms = 0, per_sm = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  C10_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, 512, 0));
  TORCH_CHECK(ctas >= 1 && ctas <= sms * per_sm, "nvls all-reduce: ", ctas, " CTAs cannot be co-resident");
  void* args[] = {const_cast<NvlsParams*>(&p)};
  C10_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, dim3(ctas), dim3(512), args, 0, stream));
}

}  // namespace

// In-place all-reduce of `bucket` (fp32 or bf16, contiguous).  `stage_ptr` / `mc_ptr`: this rank's staging buffer
// and its multicast address; `flag_ptrs`: every rank's flag array as mapped here (world uint32 words each);
// `stage_bytes`: capacity of the staging buffer; `status_ptr`: 4 local uint32 words.
void nvls_allreduce(at::Tensor bucket, int64_t stage_ptr, int64_t mc_ptr, std::vector<int64_t> flag_ptrs,
                    int64_t stage_bytes, int64_t status_ptr, int64_t rank, int64_t world, int64_t wire_bits, int64_t epoch,
                    double post_scale, int64_t timeout_ns, int64_t ctas) {
  TORCH_CHECK(bucket.is_cuda() && bucket.is_contiguous(), "nvls all-reduce: contiguous CUDA bucket");
  TORCH_CHECK(bucket.scalar_type() == at::kFloat || bucket.scalar_type() == at::kBFloat16, "bucket: fp32 or bf16");
  TORCH_CHECK(wire_bits == 16 || wire_bits == 32, "the wire carries bf16 (16) or fp32 (32) values");
  TORCH_CHECK(world >= 2 && world <= kMaxWorld && rank >= 0 && rank < world, "bad rank / world");
  TORCH_CHECK(static_cast<int64_t>(flag_ptrs.size()) == world, "one flag pointer per rank");
  TORCH_CHECK(mc_ptr != 0 && (mc_ptr % 16) == 0 && (stage_ptr % 16) == 0, "staging buffer / multicast address missing or misaligned");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(bucket.data_ptr()) % 16 == 0, "nvls all-reduce: the bucket must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(bucket.device());
  NvlsParams p{};
  p.bucket = bucket.data_ptr();
  p.n = bucket.numel();
  const long long unit = 8 * world;
  p.n_pad = (p.n + unit - 1) / unit * unit;
  TORCH_CHECK(p.n_pad * (wire_bits / 8) <= stage_bytes, "bucket of ", p.n, " elements does not fit the staging buffer");
  p.stage = reinterpret_cast<uint8_t*>(stage_ptr);
  p.mc = reinterpret_cast<uint8_t*>(mc_ptr);
  for (int r = 0; r < world; ++r) p.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  p.world = static_cast<int>(world);
  p.rank = static_cast<int>(rank);
  p.epoch = static_cast<uint32_t>(epoch);
  p.post_scale = static_cast<float>(post_scale);
  p.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  p.status = reinterpret_cast<uint32_t*>(status_ptr);
  if (p.n == 0) return;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const bool f32 = bucket.scalar_type() == at::kFloat;
  if (f32 && wire_bits == 16) launch_nvls<float, 16>(p, static_cast<int>(ctas), stream);
  else if (f32) launch_nvls<float, 32>(p, static_cast<int>(ctas), stream);
  else if (wire_bits == 16) launch_nvls<__nv_bfloat16, 16>(p, static_cast<int>(ctas), stream);
  else launch_nvls<__nv_bfloat16, 32>(p, static_cast<int>(ctas), stream);
}

}  // namespace dq
