// Device code of the persistent compressed all-reduce; included by the per-bit-width
// translation units (fused_allreduce_b*.cu) so that they compile in parallel.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <cuda_runtime.h>

#include "../common/rht_codec.cuh"
#include "fused_allreduce.cuh"

namespace dq {

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

template <int BITS, typename T>
__device__ __forceinline__ void fused_allreduce_body(const ARParams& p) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  float* tile = smem + warp * kBlock;
  uint32_t* sign_words = reinterpret_cast<uint32_t*>(smem + nwarps * kBlock);

  if (tid < 32) sign_words[tid] = sign_word(tid, p.step, p.bucket_id, p.seed_lo, p.seed_hi);
  __syncthreads();
  const uint32_t sign_mask = lane_sign_mask(sign_words, lane);

  T* bucket = static_cast<T*>(p.bucket);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(bucket) & 15u) == 0;
  const int per_cta = (p.blocks_per_shard + G - 1) / G;
  uint8_t* my_mail = p.mail[p.rank];
  const uint32_t* my_flags = p.flags[p.rank];
  const int tail_block = (p.n % kBlock) ? p.nblocks - 1 : -1;

  for (int s = 0; s < p.nsteps; ++s) {
    const int shard = p.steps[s][0], local = p.steps[s][1], recv_slot = p.steps[s][2], nrecv = p.steps[s][3];
    const int out = p.steps[s][4], dst = p.steps[s][5], send_slot = p.steps[s][6];
    const uint32_t tag = stream_tag(p.bucket_id, static_cast<uint32_t>(p.steps[s][7]));

    const int shard_lo = min(shard * p.blocks_per_shard, p.nblocks);
    const int shard_hi = min(shard_lo + p.blocks_per_shard, p.nblocks);
    const int lo = min(shard_lo + cta * per_cta, shard_hi);
    const int hi = min(lo + per_cta, shard_hi);
    if (hi <= lo) continue;  // producer and consumer agree on empty ranges: no flag traffic

    if (nrecv > 0) {
      bool timed_out = false;
      int bad_slot = 0;
      if (tid < nrecv) {
        const uint32_t* f = my_flags + p.flag_base + static_cast<uint32_t>(recv_slot + tid) * G + cta;
        timed_out = !wait_flag(f, p.epoch, p.timeout_ns);
        bad_slot = recv_slot + tid;
      }
      if (__syncthreads_or(timed_out)) {
        if (timed_out) {
          if (atomicCAS(p.status, kOk, kErrWaitTimeout) == kOk) {
            p.status[1] = (static_cast<uint32_t>(s) << 16) | static_cast<uint32_t>(cta);
            p.status[2] = static_cast<uint32_t>(bad_slot);
          }
        }
        return;  // the whole CTA gives up; peers that depend on it time out the same way
      }
    }

    for (int blk = lo + warp; blk < hi; blk += nwarps) {
      const int bs = blk - shard_lo;  // block index inside the shard = inside the message
      const long long e0 = static_cast<long long>(blk) * kBlock;
      const int valid = static_cast<int>(min(static_cast<long long>(kBlock), p.n - e0));
      float v[32];

      if (out != kOutDecode) {
        if (local == kLocalRaw) {
          load_block<T>(bucket + e0, valid, vec_ok, lane, v);
          rotate_forward(v, sign_mask, tile, lane);
        } else if (blk == tail_block) {
          load_block<float>(p.tail_ws, kBlock, true, lane, v);
        } else {
          load_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
        }
        for (int r = 0; r < nrecv; ++r) {
          const uint8_t* slot = my_mail + static_cast<unsigned long long>(recv_slot + r) * p.slot_stride;
          const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
          uint32_t w[BITS];
#pragma unroll
          for (int j = 0; j < BITS; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
          const float scale = __ldcg(reinterpret_cast<const float*>(slot + p.scales_off) + bs);
          dequantize_add_block<BITS>(w, scale, v);
        }
      }

      if (out == kOutStore) {
        if (blk == tail_block) store_block<float>(p.tail_ws, kBlock, true, lane, v);
        else store_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
      } else if (out == kOutSend) {
        uint32_t w[BITS];
        const float scale = quantize_block<BITS>(v, w, static_cast<uint32_t>(blk), tag, p.step, p.seed_lo, p.seed_hi, lane);
        if (!p.no_transmit) {
          uint8_t* slot = p.mail[dst] + static_cast<unsigned long long>(send_slot) * p.slot_stride;
          uint32_t* codes = reinterpret_cast<uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
          for (int j = 0; j < BITS; ++j) codes[j * 32 + lane] = w[j];
          if (lane == 0) reinterpret_cast<float*>(slot + p.scales_off)[bs] = scale;
        }
      } else {
        uint32_t w[BITS];
        float scale;
        if (out == kOutFinal) {
          scale = quantize_block<BITS>(v, w, static_cast<uint32_t>(blk), tag, p.step, p.seed_lo, p.seed_hi, lane);
          if (!p.no_transmit) {
            for (int peer = 0; peer < p.world; ++peer) {
              if (peer == p.rank) continue;
              uint8_t* slot = p.mail[peer] + static_cast<unsigned long long>(send_slot) * p.slot_stride;
              uint32_t* codes = reinterpret_cast<uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
              for (int j = 0; j < BITS; ++j) codes[j * 32 + lane] = w[j];
              if (lane == 0) reinterpret_cast<float*>(slot + p.scales_off)[bs] = scale;
            }
          }
        } else {  // kOutDecode
          const uint8_t* slot = my_mail + static_cast<unsigned long long>(recv_slot) * p.slot_stride;
          const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
          for (int j = 0; j < BITS; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
          scale = __ldcg(reinterpret_cast<const float*>(slot + p.scales_off) + bs);
        }
        dequantize_block<BITS>(w, scale, v);
        rotate_inverse(v, sign_mask, p.finish_scale, tile, lane);
        store_block<T>(bucket + e0, valid, vec_ok, lane, v);
      }
    }

    if (out == kOutSend || out == kOutFinal) {
      __syncthreads();  // every warp's payload stores precede the flag
      if (out == kOutSend) {
        if (tid == 0) {
          __threadfence_system();
          st_release_sys(p.flags[dst] + p.flag_base + static_cast<uint32_t>(send_slot) * G + cta, p.epoch);
        }
      } else if (tid < p.world && tid != p.rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + p.flag_base + static_cast<uint32_t>(send_slot) * G + cta, p.epoch);
      }
    }
  }
}

template <int BITS, typename T>
__global__ void __launch_bounds__(512, 1) fused_allreduce_kernel(const __grid_constant__ ARParams p) {
  fused_allreduce_body<BITS, T>(p);
}

// Several ranks in one launch on one GPU (blockIdx.y = rank): the single-GPU form of the
// collective used by the standalone codec ops and by tests.  Cooperative, so that CTAs that
// wait on one another are co-resident.
template <int BITS, typename T>
__global__ void __launch_bounds__(512, 1) fused_allreduce_multi_kernel(const ARParams* __restrict__ plist) {
  fused_allreduce_body<BITS, T>(plist[blockIdx.y]);
}

template <int BITS, typename T>
void launch_one(const ARParams* host_params, const ARParams* dev_params, int nranks, int ctas, int threads,
                       cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(threads / 32) * kBlock * sizeof(float) + 32 * sizeof(uint32_t);
  const void* fn = nranks == 1 ? reinterpret_cast<const void*>(&fused_allreduce_kernel<BITS, T>)
                               : reinterpret_cast<const void*>(&fused_allreduce_multi_kernel<BITS, T>);
  C10_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int dev = 0, sms = 0, per_sm = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  C10_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem));
  TORCH_CHECK(static_cast<long long>(ctas) * nranks <= static_cast<long long>(sms) * per_sm,
              "fused all-reduce: ", ctas, " CTAs x ", nranks, " ranks do not fit co-resident on ", sms, " SMs x ",
              per_sm);
  dim3 grid(ctas, nranks), block(threads);
  if (nranks == 1) {
    void* args[] = {const_cast<ARParams*>(host_params)};
    C10_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, grid, block, args, smem, stream));
  } else {
    void* args[] = {&dev_params};
    C10_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, grid, block, args, smem, stream));
  }
}


#define DQ_INSTANTIATE_FUSED_ALLREDUCE(BITS)                                                                   \
  template void launch_one<BITS, float>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<BITS, __nv_bfloat16>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

}  // namespace dq
