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

// ---- per-warp bulk prefetch (TMA engine, 1-D form) of the next raw block --------------------
// Lane 0 arms the warp's mbarrier with the byte count and issues one cp.async.bulk of a whole
// block (4 KiB fp32 / 2 KiB bf16) from this GPU's own bucket into the warp's staging buffer; the
// warp later waits on the barrier's phase (bounded) and reads the block from shared memory.

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bulk_prefetch(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier generic reads of dst precede the copy
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// true when the phase with the given parity has completed; gives up after ~2^22 polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
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

struct RawItem {
  int s, blk;  // program step and block index; s < 0: none
};

// [lo, hi) of CTA `cta` inside the shard of step s, and the shard's first block
__device__ __forceinline__ void step_range(const ARParams& p, int s, int cta, int per_cta, int& shard_lo, int& lo,
                                           int& hi) {
  const int shard = p.steps[s][0];
  shard_lo = min(shard * p.blocks_per_shard, p.nblocks);
  const int shard_hi = min(shard_lo + p.blocks_per_shard, p.nblocks);
  lo = min(shard_lo + cta * per_cta, shard_hi);
  hi = min(lo + per_cta, shard_hi);
}

// the next block after (s, blk) that this warp will read as raw gradients (blk < 0: start of step s)
__device__ __forceinline__ RawItem next_raw_item(const ARParams& p, int s, int blk, int cta, int per_cta, int warp,
                                                 int nwarps) {
  for (; s < p.nsteps; ++s, blk = -1) {
    if (p.steps[s][1] != kLocalRaw || p.steps[s][4] == kOutDecode) continue;
    int shard_lo, lo, hi;
    step_range(p, s, cta, per_cta, shard_lo, lo, hi);
    const int cand = blk < 0 ? lo + warp : blk + nwarps;
    if (cand < hi) return RawItem{s, cand};
  }
  return RawItem{-1, -1};
}

template <int BITS, typename T>
__device__ __forceinline__ void fused_allreduce_body(const ARParams& p) {
  extern __shared__ __align__(128) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  float* tile = smem + warp * kBlock;
  float* stage = smem + (nwarps + warp) * kBlock;
  uint32_t* sign_words = reinterpret_cast<uint32_t*>(smem + 2 * nwarps * kBlock);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sign_words + 32);
  uint64_t* bar = bars + warp;

  if (tid < 32) sign_words[tid] = sign_word(tid, p.step, p.bucket_id, p.seed_lo, p.seed_hi);
  if (lane == 0) mbar_init(bar, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  const uint32_t sign_mask = lane_sign_mask(sign_words, lane);

  T* bucket = static_cast<T*>(p.bucket);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(bucket) & 15u) == 0;
  const int per_cta = (p.blocks_per_shard + G - 1) / G;
  uint8_t* my_mail = p.mail[p.rank];
  const uint32_t* my_flags = p.flags[p.rank];
  const int tail_block = (p.n % kBlock) ? p.nblocks - 1 : -1;
  constexpr uint32_t kBlockBytes = kBlock * sizeof(T);

  // prefetch state (warp-uniform): the item whose data is in flight or resident in `stage`
  RawItem pf = RawItem{-1, -1};
  uint32_t pf_parity = 0;
  bool prefetch_ok = true;
  auto issue_prefetch = [&](RawItem it) {
    pf = RawItem{-1, -1};
    if (!prefetch_ok || it.s < 0 || !vec_ok || it.blk == tail_block) return;
    pf = it;
    if (lane == 0) bulk_prefetch(stage, bucket + static_cast<long long>(it.blk) * kBlock, kBlockBytes, bar);
  };
  issue_prefetch(next_raw_item(p, 0, -1, cta, per_cta, warp, nwarps));

  auto fail = [&](uint32_t code, int s, int slot) {
    if (atomicCAS(p.status, kOk, code) == kOk) {
      p.status[1] = (static_cast<uint32_t>(s) << 16) | static_cast<uint32_t>(cta);
      p.status[2] = static_cast<uint32_t>(slot);
    }
  };

  for (int s = 0; s < p.nsteps; ++s) {
    const int local = p.steps[s][1], recv_slot = p.steps[s][2], nrecv = p.steps[s][3];
    const int out = p.steps[s][4], dst = p.steps[s][5], send_slot = p.steps[s][6];
    const uint32_t tag = stream_tag(p.bucket_id, static_cast<uint32_t>(p.steps[s][7]) & ~kTagStratified);
    const int strat_world = (static_cast<uint32_t>(p.steps[s][7]) & kTagStratified) ? p.world : 1;
    int shard_lo, lo, hi;
    step_range(p, s, cta, per_cta, shard_lo, lo, hi);
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
        if (timed_out) fail(kErrWaitTimeout, s, bad_slot);
        if (pf.s >= 0) mbar_wait(bar, pf_parity);  // let this warp's copy in flight land before leaving
        return;  // the whole CTA gives up; peers that depend on it time out the same way
      }
    }

    for (int blk = lo + warp; blk < hi; blk += nwarps) {
      const int bs = blk - shard_lo;  // block index inside the shard = inside the message
      const long long e0 = static_cast<long long>(blk) * kBlock;
      const int valid = static_cast<int>(min(static_cast<long long>(kBlock), p.n - e0));
      float v[32];
      uint32_t w[BITS];
      float scale = 0.f;

      if (nrecv > 0) {  // first incoming message: issue its loads before the local work
        const uint8_t* slot = my_mail + static_cast<unsigned long long>(recv_slot) * p.slot_stride;
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
        for (int j = 0; j < BITS; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
        scale = __ldcg(reinterpret_cast<const float*>(slot + p.scales_off) + bs);
      }

      if (out != kOutDecode) {
        if (local == kLocalRaw) {
          if (pf.s == s && pf.blk == blk && mbar_wait(bar, pf_parity)) {
            pf_parity ^= 1u;
            load_block<T>(reinterpret_cast<const T*>(stage), kBlock, true, lane, v);
            __syncwarp();
          } else {
            if (pf.s == s && pf.blk == blk) {  // the copy never completed: report it, read directly,
              fail(kErrCopyTimeout, s, -1);    // and stop prefetching (the warp stays in step with its CTA)
              prefetch_ok = false;
            }
            load_block<T>(bucket + e0, valid, vec_ok, lane, v);
          }
          issue_prefetch(next_raw_item(p, s, blk, cta, per_cta, warp, nwarps));
          rotate_forward(v, sign_mask, tile, lane);
        } else if (blk == tail_block) {
          load_block<float>(p.tail_ws, kBlock, true, lane, v);
        } else {
          load_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
        }
        if (nrecv > 0) dequantize_add_block<BITS>(w, scale, v);
        for (int r = 1; r < nrecv; ++r) {
          const uint8_t* slot = my_mail + static_cast<unsigned long long>(recv_slot + r) * p.slot_stride;
          const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
          for (int j = 0; j < BITS; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
          scale = __ldcg(reinterpret_cast<const float*>(slot + p.scales_off) + bs);
          dequantize_add_block<BITS>(w, scale, v);
        }
      }

      if (out == kOutStore) {
        if (blk == tail_block) store_block<float>(p.tail_ws, kBlock, true, lane, v);
        else store_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
      } else if (out == kOutSend) {
        scale = quantize_block<BITS>(v, w, static_cast<uint32_t>(blk), tag, p.step, p.seed_lo, p.seed_hi, lane, p.rank,
                                     strat_world);
        if (!p.no_transmit) {
          uint8_t* slot = p.mail[dst] + static_cast<unsigned long long>(send_slot) * p.slot_stride;
          uint32_t* codes = reinterpret_cast<uint32_t*>(slot) + static_cast<size_t>(bs) * (BITS * 32);
#pragma unroll
          for (int j = 0; j < BITS; ++j) codes[j * 32 + lane] = w[j];
          if (lane == 0) reinterpret_cast<float*>(slot + p.scales_off)[bs] = scale;
        }
      } else {
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
        }
        // kOutDecode: w / scale were loaded from the all-gather slot above
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
  const size_t smem = static_cast<size_t>(threads / 32) * (2 * kBlock * sizeof(float) + sizeof(uint64_t)) + 32 * sizeof(uint32_t);
  const void* fn = nranks == 1 ? reinterpret_cast<const void*>(&fused_allreduce_kernel<BITS, T>)
                               : reinterpret_cast<const void*>(&fused_allreduce_multi_kernel<BITS, T>);
  // attribute and occupancy are queried once per (kernel, device, block size) and cached
  struct Cache {
    int dev = -1, threads = -1, capacity = 0;
  };
  static thread_local Cache cache[2];
  Cache& c = cache[nranks == 1 ? 0 : 1];
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  if (c.dev != dev || c.threads != threads) {
    int sms = 0, per_sm = 0;
    C10_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    C10_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem));
    c.dev = dev, c.threads = threads, c.capacity = sms * per_sm;
  }
  TORCH_CHECK(static_cast<long long>(ctas) * nranks <= c.capacity, "fused all-reduce: ", ctas, " CTAs x ", nranks,
              " ranks do not fit co-resident (capacity ", c.capacity, " CTAs of ", threads, " threads)");
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
