// Device code of the persistent compressed all-reduce; included by the per-bit-width
// translation units (fused_allreduce_b*.cu) so that they compile in parallel.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "../common/rht_codec.cuh"
#include "../common/sc_codec.cuh"
#include "../common/mx_codec.cuh"
#include "fused_allreduce.cuh"
#include "fused_wire.cuh"
#include "fused_rht_tc.cuh"

namespace dq {

struct RawItem {
  int s, blk;  // program step and block index; s < 0: none
};

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

// Shared-memory layout of a CTA of the SIMT bodies (nwarps warps):
//   [tile: nwarps x 4 KiB][stage: nwarps x 4 KiB (optional)][sign table fwd][sign table inv][sign words]
//   [prefetch barriers][pending flags: 2 x kMaxWorld ints]
// The tensor-core rotation has its own layout (fused_rht_tc.cuh).
template <bool TC>
__host__ __device__ constexpr size_t fused_smem_bytes(int threads, bool stage = true) {
  if (TC) return rht_tc_smem_bytes(threads, stage);
  const size_t nwarps = threads / 32;
  return nwarps * kBlock * 4 + (stage ? nwarps * kBlock * 4 : 0) + 2 * 4096 + 32 * 4 + nwarps * 8 + 64 + 128;
}

template <int BITS, typename T, int CODEC>
__device__ __forceinline__ void fused_simt_body(const ARParams& p) {
  constexpr bool MX = CODEC == kCodecMx;      // block-float codes (8 / 6 / 4 bit) with native conversions
  constexpr bool CAST = CODEC == kCodecCast;  // identity wire: bf16 (16) or fp32 (32) values
  constexpr bool MIX = CODEC == kCodecScMixAee || CODEC == kCodecScMixMee;  // superchunk records of per-superchunk width
  constexpr bool SC = CODEC == kCodecScAee || CODEC == kCodecScMee || MX || CAST || MIX;  // lane-contiguous record codecs
  constexpr int CB = BITS == 32 ? 32 : 16;
  constexpr bool MEE = CODEC == kCodecScMee || CODEC == kCodecScMixMee;
  constexpr int SCB = (BITS == 2 || BITS == 4 || BITS == 8) ? BITS : 4;  // superchunk code width (2, 4, 8 only)
  constexpr int MXB = (BITS == 4 || BITS == 6 || BITS == 8) ? BITS : 8;  // block-float code width (4, 6, 8 only)
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int cta = blockIdx.x, G = gridDim.x;

  uint8_t* cursor = smem_raw;
  float* tile = reinterpret_cast<float*>(cursor) + warp * kBlock;
  cursor += static_cast<size_t>(nwarps) * kBlock * 4;
  const bool use_stage = p.prefetch != 0;
  float* stage = reinterpret_cast<float*>(cursor) + warp * kBlock;
  if (use_stage) cursor += static_cast<size_t>(nwarps) * kBlock * 4;
  float* sgn_fwd = reinterpret_cast<float*>(cursor);
  cursor += 4096;
  float* sgn_inv = reinterpret_cast<float*>(cursor);
  cursor += 4096;
  uint32_t* sign_words = reinterpret_cast<uint32_t*>(cursor);
  cursor += 32 * 4;
  uint64_t* bar = reinterpret_cast<uint64_t*>(cursor) + warp;

  if (tid < 32) sign_words[tid] = sign_word(tid, p.step, p.bucket_id, p.seed_lo, p.seed_hi);
  if (lane == 0) mbar_init(bar, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  if (!SC) fill_sign_tables(sgn_fwd, sgn_inv, sign_words, p.finish_scale, tid, blockDim.x);
  __syncthreads();

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
  // the rotation codec and the identity wire read raw blocks in the coalesced load layout, which a bulk copy into
  // the warp's staging buffer can prefetch; the other record codecs use that buffer to form lane-contiguous runs
  bool prefetch_ok = (!SC || CAST) && use_stage;
  const ScParams scp{p.sc_lattice_max, p.sc_c1, p.sc_c2, p.sc_lut};
  uint8_t* rec_tile = reinterpret_cast<uint8_t*>(tile);  // superchunk codec: the warp's record staging area
  auto issue_prefetch = [&](RawItem it) {
    pf = RawItem{-1, -1};
    if (!prefetch_ok || it.s < 0 || !vec_ok || it.blk == tail_block) return;
    pf = it;
    if (lane == 0) bulk_prefetch(stage, bucket + static_cast<long long>(it.blk) * kBlock, kBlockBytes, bar);
  };
  issue_prefetch(next_raw_item(p, 0, -1, cta, per_cta, warp, nwarps));

  auto fail = [&](uint32_t code, int s, int slot) { report_failure(p, code, s, slot); };

  // Flags of consecutive sending steps that receive nothing (the scatter of the direct topology: W - 1 of them)
  // are published together: one block barrier and one system-scope fence for the run instead of one per step.
  // A consumer needs all of its incoming shards before it can start anyway, so nothing is delayed.
  int* pend = reinterpret_cast<int*>(reinterpret_cast<uint64_t*>(cursor) + nwarps);  // 2 * kMaxWorld ints behind the barriers
  int npend = 0;  // CTA-uniform
  auto flush_flags = [&]() {
    if (npend == 0) return;
    __syncthreads();  // every warp's payload stores of the pending steps precede their flags
    if (tid < npend) {
      __threadfence_system();
      st_release_sys(p.flags[pend[2 * tid]] + p.flag_base + static_cast<uint32_t>(pend[2 * tid + 1]) * G + cta, p.epoch);
    }
    npend = 0;
    __syncthreads();  // `pend` may be rewritten from here on
  };

  bool aborted = false;
  for (int s = 0; s < p.nsteps && !aborted; ++s) {
    const int local = p.steps[s][1], recv_slot = p.steps[s][2], nrecv = p.steps[s][3];
    const int out = p.steps[s][4], dst = p.steps[s][5], send_slot = p.steps[s][6];
    if (!(nrecv == 0 && out == kOutSend)) flush_flags();  // before this step waits for anybody
    const uint32_t tag = stream_tag(p.bucket_id, static_cast<uint32_t>(p.steps[s][7]) & ~kTagStratified);
    const int strat_world = (static_cast<uint32_t>(p.steps[s][7]) & kTagStratified) ? p.world : 1;
    int shard_lo, lo, hi;
    step_range(p, s, cta, per_cta, shard_lo, lo, hi);
    if (hi <= lo) continue;  // producer and consumer agree on empty ranges: no flag traffic

    if (p.debug) {  // CTA-uniform: a step with an access outside its slots is not run at all
      int bad_slot;
      constexpr int kPlanUnit = (CODEC == kCodecScMixAee || CODEC == kCodecScMixMee) ? 8 : (CODEC == kCodecRhtMix ? 128 : 0);
      const bool bad = debug_step_out_of_bounds<kPlanUnit, !SC>(p, s, shard_lo, lo, hi, bad_slot);
      if (__syncthreads_or(bad)) {
        if (bad) fail(kErrBounds, s, bad_slot);
        aborted = true;
        break;
      }
    }

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
        aborted = true;  // the whole CTA gives up; peers that depend on it time out the same way
        break;
      }
    }
    const bool rotate_in = (out != kOutDecode) && (local == kLocalRaw);
    const bool rotate_out = (out == kOutFinal) || (out == kOutDecode);

    for (int blk = lo + warp; blk < hi; blk += nwarps) {
      constexpr bool active = true;
      const int bs = blk - shard_lo;  // block index inside the shard = inside the message
      const long long e0 = static_cast<long long>(blk) * kBlock;
      const int valid = static_cast<int>(min(static_cast<long long>(kBlock), p.n - e0));
      float v[32];
      if constexpr (SC) {
        // ---- record codecs (superchunk AEE / MEE, block-float): no rotation, one record area per block ----
        constexpr unsigned kBB = CAST ? CastGeom<CB>::kBlockBytes : (MX ? MxGeom<MXB>::kBlockBytes : ScGeom<SCB>::kBlockBytes);
        unsigned long long boff = static_cast<unsigned long long>(bs) * kBB;
        uint32_t wpack = 0;
        int mix_n8 = 0;
        if constexpr (MIX) {  // per-block offset and widths from the plan
          const uint32_t o0 = __ldg(p.sc_plan + blk), o1 = __ldg(p.sc_plan + blk + 1);
          boff = static_cast<unsigned long long>(o0 - __ldg(p.sc_plan + shard_lo)) * 8ull;
          mix_n8 = static_cast<int>(o1 - o0);
          wpack = __ldg(p.sc_plan + p.nblocks + 1 + blk);
        }
        const uint32_t first_call = static_cast<uint32_t>(blk) * 64u;  // Philox call index = element / 16
        auto rec_in = [&](const uint8_t* src) {
          if constexpr (MIX) sc_copy_in_n(rec_tile, src, mix_n8, lane);
          else if constexpr (CAST) bytes_copy_in<CastGeom<CB>::kBlockBytes>(rec_tile, src, lane);
          else if constexpr (MX) mx_copy_in<MXB>(rec_tile, src, lane);
          else sc_copy_in<SCB>(rec_tile, src, lane);
          __syncwarp();
        };
        auto rec_out = [&](uint8_t* dstp) {
          if constexpr (MIX) sc_copy_out_n(dstp, rec_tile, mix_n8, lane);
          else if constexpr (CAST) bytes_copy_out<CastGeom<CB>::kBlockBytes>(dstp, rec_tile, lane);
          else if constexpr (MX) mx_copy_out<MXB>(dstp, rec_tile, lane);
          else sc_copy_out<SCB>(dstp, rec_tile, lane);
        };
        auto rec_encode = [&]() {
          if constexpr (MIX) sc_encode_block_mix<MEE>(v, rec_tile, p.sc_lut, wpack, first_call, tag, p.step, p.seed_lo, p.seed_hi, lane);
          else if constexpr (CAST) cast_encode_block<CB>(v, rec_tile, lane);
          else if constexpr (MX) mx_encode_block<MXB>(v, rec_tile, lane);
          else sc_encode_block<SCB, MEE>(v, rec_tile, scp, first_call, tag, p.step, p.seed_lo, p.seed_hi, lane);
          __syncwarp();
        };
        if constexpr (CAST) {
          // identity wire: values move between global memory and registers in the coalesced load layout,
          // nothing is staged (csrc/common/mx_codec.cuh, cast_msg_*)
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
              issue_prefetch(blk + nwarps < hi ? RawItem{s, blk + nwarps}  // the common case needs no search
                                              : next_raw_item(p, s + 1, -1, cta, per_cta, warp, nwarps));
            }
            else if (blk == tail_block) load_block<float>(p.tail_ws, kBlock, true, lane, v);
            else load_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
            for (int r = 0; r < nrecv; ++r)
              cast_msg_load<CB, true>(v, my_mail + static_cast<unsigned long long>(recv_slot + r) * p.slot_stride + boff, lane);
          }
          if (out == kOutStore) {
            if (blk == tail_block) store_block<float>(p.tail_ws, kBlock, true, lane, v);
            else store_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
          } else if (out == kOutSend) {
            cast_round<CB>(v);
            if (!p.no_transmit)
              cast_msg_store<CB>(p.mail[dst] + static_cast<unsigned long long>(send_slot) * p.slot_stride + boff, v, lane);
          } else {
            if (out == kOutFinal) {
              cast_round<CB>(v);  // this rank keeps what its peers will decode
              if (!p.no_transmit) {
                for (int peer = 0; peer < p.world; ++peer) {
                  if (peer == p.rank) continue;
                  cast_msg_store<CB>(p.mail[peer] + static_cast<unsigned long long>(send_slot) * p.slot_stride + boff, v, lane);
                }
              }
            } else {
              cast_msg_load<CB, false>(v, my_mail + static_cast<unsigned long long>(recv_slot) * p.slot_stride + boff, lane);
            }
            const float wf = static_cast<float>(p.world), ps = p.finish_scale * 1024.0f;
            if (ps == __fdiv_rn(1.0f, wf)) {
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __fdiv_rn(v[k], wf);
            } else {
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __fmul_rn(v[k], ps);
            }
            store_block<T>(bucket + e0, valid, vec_ok, lane, v);
          }
        } else {
        // whole fp32 blocks go through the warp's (otherwise unused) staging buffer with coalesced accesses
        auto raw_in = [&](const T* src, int nvalid) {
          if constexpr (std::is_same<T, float>::value) {
            if (use_stage && vec_ok && nvalid == kBlock) return sc_load_block_coalesced(src, stage, lane, v);
          }
          sc_load_block<T>(src, nvalid, vec_ok, lane, v);
        };
        auto raw_out = [&](T* dstp, int nvalid) {
          if constexpr (std::is_same<T, float>::value) {
            if (use_stage && vec_ok && nvalid == kBlock) return sc_store_block_coalesced(dstp, stage, lane, v);
          }
          sc_store_block<T>(dstp, nvalid, vec_ok, lane, v);
        };
        if (out != kOutDecode) {
            if (local == kLocalRaw) raw_in(bucket + e0, valid);
            else if (blk == tail_block) sc_load_block<float>(p.tail_ws, kBlock, true, lane, v);
            else raw_in(bucket + e0, kBlock);
            for (int r = 0; r < nrecv; ++r) {
              const uint8_t* slot = my_mail + static_cast<unsigned long long>(recv_slot + r) * p.slot_stride;
              rec_in(slot + boff);
              if constexpr (MIX) sc_decode_block_mix<MEE, true>(v, rec_tile, p.sc_lut, wpack, lane);
              else if constexpr (CAST) cast_decode_block<CB, true>(v, rec_tile, lane);
              else if constexpr (MX) mx_decode_block<MXB, true>(v, rec_tile, lane);
              else sc_decode_block<SCB, MEE, true>(v, rec_tile, scp, lane);
              __syncwarp();
            }
          }
          if (out == kOutStore) {
            if (blk == tail_block) sc_store_block<float>(p.tail_ws, kBlock, true, lane, v);
            else raw_out(bucket + e0, kBlock);
          } else if (out == kOutSend) {
            rec_encode();
            if (!p.no_transmit) rec_out(p.mail[dst] + static_cast<unsigned long long>(send_slot) * p.slot_stride + boff);
            __syncwarp();
          } else {
            if (out == kOutFinal) {
              rec_encode();
              if (!p.no_transmit) {
                for (int peer = 0; peer < p.world; ++peer) {
                  if (peer == p.rank) continue;
                  rec_out(p.mail[peer] + static_cast<unsigned long long>(send_slot) * p.slot_stride + boff);
                }
              }
            } else {
              rec_in(my_mail + static_cast<unsigned long long>(recv_slot) * p.slot_stride + boff);
            }
            if constexpr (MIX) sc_decode_block_mix<MEE, false>(v, rec_tile, p.sc_lut, wpack, lane);
            else if constexpr (CAST) cast_decode_block<CB, false>(v, rec_tile, lane);
            else if constexpr (MX) mx_decode_block<MXB, false>(v, rec_tile, lane);
            else sc_decode_block<SCB, MEE, false>(v, rec_tile, scp, lane);
            __syncwarp();
            // the mean divides by the world size, as the tensor-operator codecs do; any other post-scale
            // (1 for a plain sum) multiplies
            const float wf = static_cast<float>(p.world), ps = p.finish_scale * 1024.0f;
            if (ps == __fdiv_rn(1.0f, wf)) {
  #pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __fdiv_rn(v[k], wf);
            } else {
  #pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __fmul_rn(v[k], ps);
            }
            raw_out(bucket + e0, valid);
          }
        }
      } else {
      // ---- rotation codec ----
      constexpr bool MIXR = CODEC == kCodecRhtMix;  // a code width per block, from the plan
      constexpr int RB = MIXR ? 8 : ((BITS >= 2 && BITS <= 8) ? BITS : 8);  // (largest) code width
      uint32_t w[RB];
      float scale = 0.f;
      int wb = RB;                                             // this block's width
      size_t code_word = static_cast<size_t>(bs) * (RB * 32);  // first code word of the block inside a message
      if constexpr (MIXR) {
        wb = static_cast<int>(__ldg(p.sc_plan + p.nblocks + 1 + blk));
        code_word = static_cast<size_t>(__ldg(p.sc_plan + blk) - __ldg(p.sc_plan + shard_lo)) * 32;
      }
      auto with_width = [&](auto&& fn) {  // fn(width as a compile-time constant)
        if constexpr (!MIXR) {
          fn(std::integral_constant<int, RB>{});
        } else {
          switch (wb) {
            case 2: fn(std::integral_constant<int, 2>{}); break;
            case 3: fn(std::integral_constant<int, 3>{}); break;
            case 4: fn(std::integral_constant<int, 4>{}); break;
            case 5: fn(std::integral_constant<int, 5>{}); break;
            case 6: fn(std::integral_constant<int, 6>{}); break;
            case 7: fn(std::integral_constant<int, 7>{}); break;
            default: fn(std::integral_constant<int, 8>{}); break;
          }
        }
      };
      auto load_codes = [&](const uint8_t* slot) {
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + code_word;
#pragma unroll
        for (int j = 0; j < RB; ++j)
          if (!MIXR || j < wb) w[j] = ld_cg_u32(codes + j * 32 + lane);
        scale = __ldcg(reinterpret_cast<const float*>(slot + p.scales_off) + bs);
      };
      auto store_codes = [&](uint8_t* slot) {
        uint32_t* codes = reinterpret_cast<uint32_t*>(slot) + code_word;
#pragma unroll
        for (int j = 0; j < RB; ++j)
          if (!MIXR || j < wb) codes[j * 32 + lane] = w[j];
        if (lane == 0) reinterpret_cast<float*>(slot + p.scales_off)[bs] = scale;
      };

      if (active && nrecv > 0)  // first incoming message: issue its loads before the local work
        load_codes(my_mail + static_cast<unsigned long long>(recv_slot) * p.slot_stride);

      if (active && out != kOutDecode) {
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
          issue_prefetch(blk + nwarps < hi ? RawItem{s, blk + nwarps}  // the common case needs no search
                                              : next_raw_item(p, s + 1, -1, cta, per_cta, warp, nwarps));
        } else if (blk == tail_block) {
          load_block<float>(p.tail_ws, kBlock, true, lane, v);
        } else {
          load_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
        }
      }
      if (rotate_in) rotate_forward(v, sgn_fwd, tile, lane);

      if (active && out != kOutDecode) {
        for (int r = 0; r < nrecv; ++r) {
          if (r > 0) load_codes(my_mail + static_cast<unsigned long long>(recv_slot + r) * p.slot_stride);
          with_width([&](auto B) {
            dequantize_add_block<B.value>(reinterpret_cast<const uint32_t(&)[B.value]>(w), scale, v);
          });
        }
      }

      if (out == kOutStore) {
        if (active) {
          if (blk == tail_block) store_block<float>(p.tail_ws, kBlock, true, lane, v);
          else store_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
        }
      } else if (out == kOutSend) {
        if (active) {
          with_width([&](auto B) {
            scale = quantize_block<B.value>(v, reinterpret_cast<uint32_t(&)[B.value]>(w), static_cast<uint32_t>(blk), tag,
                                            p.step, p.seed_lo, p.seed_hi, lane, p.rank, strat_world);
          });
          if (!p.no_transmit) store_codes(p.mail[dst] + static_cast<unsigned long long>(send_slot) * p.slot_stride);
        }
      } else {
        if (active) {
          if (out == kOutFinal) {
            with_width([&](auto B) {
              scale = quantize_block<B.value>(v, reinterpret_cast<uint32_t(&)[B.value]>(w), static_cast<uint32_t>(blk),
                                              tag, p.step, p.seed_lo, p.seed_hi, lane);
            });
            if (!p.no_transmit) {
              for (int peer = 0; peer < p.world; ++peer) {
                if (peer == p.rank) continue;
                store_codes(p.mail[peer] + static_cast<unsigned long long>(send_slot) * p.slot_stride);
              }
            }
            // the width policy of the next step reads the scale of every block from this rank's own slots
            if (MIXR && lane == 0)
              reinterpret_cast<float*>(my_mail + static_cast<unsigned long long>(send_slot) * p.slot_stride +
                                       p.scales_off)[bs] = scale;
          }
          // kOutDecode: w / scale were loaded from the all-gather slot above
          with_width([&](auto B) {
            dequantize_block<B.value>(reinterpret_cast<const uint32_t(&)[B.value]>(w), scale, v);
          });
        }
        if (rotate_out) rotate_inverse(v, sgn_inv, tile, lane);
        store_block<T>(bucket + e0, valid, vec_ok, lane, v);
      }
      }  // rotation codec
    }

    if (out == kOutSend) {
      if (tid == 0) pend[2 * npend] = dst, pend[2 * npend + 1] = send_slot;
      ++npend;
      const bool next_is_pure_send = s + 1 < p.nsteps && p.steps[s + 1][3] == 0 && p.steps[s + 1][4] == kOutSend;
      if (!next_is_pure_send || npend == kMaxWorld) flush_flags();
    } else if (out == kOutFinal) {
      __syncthreads();  // every warp's payload stores precede the flags
      if (tid < p.world && tid != p.rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + p.flag_base + static_cast<uint32_t>(send_slot) * G + cta, p.epoch);
      }
    }
  }
  flush_flags();  // a run of sends that ends the program, or an abort

  if (aborted && pf.s >= 0) mbar_wait(bar, pf_parity);  // let this warp's copy in flight land before leaving
}

template <int BITS, typename T, int CODEC>
__device__ __forceinline__ void fused_allreduce_body(const ARParams& p) {
  if constexpr (CODEC == kCodecRhtTc) rht_tc_body<BITS, T>(p);
  else fused_simt_body<BITS, T, CODEC>(p);
}

// largest CTA of a codec's kernels (the tensor-core body trades a warpgroup for registers)
template <int CODEC>
constexpr int max_cta_threads() { return CODEC == kCodecRhtTc ? 512 : 512; }

template <int BITS, typename T, int CODEC>
__global__ void __launch_bounds__(max_cta_threads<CODEC>(), 1) fused_allreduce_kernel(const __grid_constant__ ARParams p) {
  fused_allreduce_body<BITS, T, CODEC>(p);
}

// Several ranks in one launch on one GPU (blockIdx.y = rank): the single-GPU form of the
// collective used by the standalone codec ops and by tests.  Cooperative, so that CTAs that
// wait on one another are co-resident.
template <int BITS, typename T, int CODEC>
__global__ void __launch_bounds__(max_cta_threads<CODEC>(), 1) fused_allreduce_multi_kernel(const ARParams* __restrict__ plist) {
  fused_allreduce_body<BITS, T, CODEC>(plist[blockIdx.y]);
}

template <int BITS, typename T, int CODEC>
void launch_one(const ARParams* host_params, const ARParams* dev_params, int nranks, int ctas, int threads,
                cudaStream_t stream) {
  constexpr bool TC = CODEC == kCodecRhtTc;
  TORCH_CHECK(!TC || (threads % 128 == 0 && threads >= 128 && threads <= 512),
              "the tensor-core rotation runs with 1 to 4 whole warpgroups (128, 256, 384 or 512 threads)");
  const bool stage = host_params == nullptr || host_params->prefetch != 0;
  const size_t smem = fused_smem_bytes<TC>(threads, stage);
  const void* fn = nranks == 1 ? reinterpret_cast<const void*>(&fused_allreduce_kernel<BITS, T, CODEC>)
                               : reinterpret_cast<const void*>(&fused_allreduce_multi_kernel<BITS, T, CODEC>);
  // attribute and occupancy are queried once per (kernel, device, block size) and cached
  struct Cache {
    int dev = -1, threads = -1, capacity = 0;
  };
  static thread_local Cache cache[4];
  Cache& c = cache[(nranks == 1 ? 0 : 1) + (stage ? 0 : 2)];
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  if (c.dev != dev || c.threads != threads) {
    int sms = 0, per_sm = 0, optin = 0;
    // the limit is a property of the kernel, shared by every (block size, staging) combination that launches it:
    // raise it to the device's opt-in maximum once instead of to this combination's need
    C10_CUDA_CHECK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    TORCH_CHECK(static_cast<size_t>(optin) >= smem, "fused all-reduce: ", smem, " bytes of shared memory per CTA exceed the device limit ", optin);
    C10_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, optin));
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
  template void launch_one<BITS, float, kCodecRht>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);           \
  template void launch_one<BITS, __nv_bfloat16, kCodecRht>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);   \
  template void launch_one<BITS, float, kCodecRhtTc>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<BITS, __nv_bfloat16, kCodecRhtTc>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

#define DQ_INSTANTIATE_FUSED_ALLREDUCE_CAST(BITS)                                                                       \
  template void launch_one<BITS, float, kCodecCast>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<BITS, __nv_bfloat16, kCodecCast>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

#define DQ_INSTANTIATE_FUSED_ALLREDUCE_MX(BITS)                                                                         \
  template void launch_one<BITS, float, kCodecMx>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);           \
  template void launch_one<BITS, __nv_bfloat16, kCodecMx>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

#define DQ_INSTANTIATE_FUSED_ALLREDUCE_SC(BITS)                                                                         \
  template void launch_one<BITS, float, kCodecScAee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<BITS, __nv_bfloat16, kCodecScAee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t); \
  template void launch_one<BITS, float, kCodecScMee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<BITS, __nv_bfloat16, kCodecScMee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

// rotation codec with a width per block: the BITS parameter is a placeholder (8, the widest block)
#define DQ_INSTANTIATE_FUSED_ALLREDUCE_RHTMIX                                                                           \
  template void launch_one<8, float, kCodecRhtMix>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<8, __nv_bfloat16, kCodecRhtMix>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

// mixed-width superchunk codec: the BITS parameter is a placeholder (8, the widest record)
#define DQ_INSTANTIATE_FUSED_ALLREDUCE_SCMIX                                                                              \
  template void launch_one<8, float, kCodecScMixAee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<8, __nv_bfloat16, kCodecScMixAee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t); \
  template void launch_one<8, float, kCodecScMixMee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);         \
  template void launch_one<8, __nv_bfloat16, kCodecScMixMee>(const ARParams*, const ARParams*, int, int, int, cudaStream_t);

}  // namespace dq
