// Rotation codec of the persistent all-reduce kernel with the Hadamard rotation on the tensor cores
// (tcgen05.mma kind::tf32, accumulators in TMEM), software-pipelined per warpgroup.
//
// Work unit: a QUAD = four consecutive 1024-element blocks, one per warp of a warpgroup, i.e. one
// 128 x 32 MMA tile.  H_1024 = H_32 (x) H_32: a block seen as a 32 x 32 matrix X transforms as H X H,
// computed as two passes D = A . H_32 with a transposition of every block in between:
//
//   forward  pass 1   A1[(b, i), k = j ]  = s * X[i][j]      K-major, written from the staged raw block
//            pass 2   A2[(b, j'), k = i]  = D1[(b, i)][j']   MN-major: the thread that read accumulator
//                                                            row i back stores it as column i
//            result   D2[(b, j')][i']     = Y[i'][j']        lane j', register i'  <->  coefficient 32 i' + j'
//   inverse  pass 1   A1[(b, i'), k = j'] = W[i'][j']        MN-major, written from the dequantised codes
//            pass 2   A2[(b, j), k = i']  = D1[(b, i')][j]   MN-major
//            result   D2[(b, j)][i]       = X[i][j]          lane j, register i  <->  element 32 i + j
//
// The MN-major operand layout (common/tcgen05.cuh) turns every transposition into eight 16-byte
// shared-memory stores per thread.  Operands are single TF32: H_32 is exact, the data loses the low 13
// mantissa bits, a relative error of 2^-11 per value - three orders of magnitude below the rounding noise
// of an 8-bit code.  The rotation is exact whenever the inputs and the 32-term partial sums fit 11
// significant bits (small integers times a power of two); the tests use such inputs to compare the wire
// bytes with the CPU oracle, and otherwise compare the rotation with a float64 product.
//
// Pipeline (per warpgroup, all four warps in step; `consume` is what the block loop calls):
//   consume(q):  wait MMA2(q)        -> coefficients of q in registers (tcgen05.ld)
//                wait MMA1(q+1)      -> read D1, store A2, named barrier, one thread issues MMA2(q+1)
//                stage(q+2) -> A1, named barrier, one thread issues MMA1(q+2); bulk copy of q+3's raw block
//                then the caller quantises / packs / sends q while both MMAs run.
// A1, A2, D1 and D2 are single-buffered: each is rewritten only after the wait that proves its last
// reader done.  The forward pipeline runs across step boundaries (raw gradients of later shards are
// already in the bucket); it never looks past a step that decodes, so the decode pipeline, which is
// drained at the end of every step, finds the operands free.
//
// The owner's last reduce-scatter step (kOutFinal) writes its encoded shard to every peer's all-gather
// slot AND to its own, then decodes its own slot like any other all-gather message: one decode path.
//
// Register budget: the body keeps a block's 32 coefficients, its codes in the making, the random bytes and the
// pipeline state live at once; it is compiled for CTAs of at most 384 threads (three warpgroups, 168
// registers per thread), where it does not spill.
//
// Every wait is bounded (mbarrier polls, flag waits by %globaltimer); a wait that gives up sets an error
// word, lets copies in flight land, frees the TMEM columns and the CTA returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../common/rht_codec.cuh"
#include "../common/tcgen05.cuh"
#include "fused_allreduce.cuh"
#include "fused_wire.cuh"

namespace dq {

struct Quad {
  int s, base;  // program step and first block; s < 0: none
};
// compile-time tags of a pipeline tick: hand a finished quad to the caller, or only fill the pipeline
struct ReadTag { static constexpr bool value = true; };
struct FillTag { static constexpr bool value = false; };
__device__ __forceinline__ bool same_quad(Quad a, Quad b) { return a.s == b.s && a.base == b.base; }

// Shared memory of a CTA of `threads` threads (nwg = threads / 128 warpgroups, nwarps = threads / 32):
//   [A1: nwg x 18 KiB][A2: nwg x 18 KiB][stage: nwarps x 4 KiB (optional)][H_32][sign table fwd][sign table inv]
//   [sign words][step table][stage barriers: nwarps][MMA barriers: 2 nwg][TMEM slot][error flag]
__host__ __device__ constexpr size_t rht_tc_smem_bytes(int threads, bool stage) {
  const size_t nwarps = threads / 32, nwg = threads / 128;
  return nwg * 2 * tc::kOperandBytes + (stage ? nwarps * 4096 : 0) + tc::kHBytes + 2 * 4096 + 32 * 4 +
         kMaxSteps * 16 + nwarps * 8 + nwg * 16 + 16 + 1024;
}

__device__ __forceinline__ void wg_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

// 32 registers of a lane -> column k = lane of an MN-major operand, rows row0 .. row0 + 31
__device__ __forceinline__ void store_mn_column(uint8_t* a, int row0, int lane, const float (&d)[32]) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(a + tc::mn_chunk_offset(row0 + 4 * c, lane)) =
        make_float4(d[4 * c], d[4 * c + 1], d[4 * c + 2], d[4 * c + 3]);
}

// 1024 elements in the column layout: register m of a lane is element 32 m + lane
template <typename T>
__device__ __forceinline__ void store_block_cols(T* base, int valid, int lane, const float (&v)[32]) {
  if (valid == kBlock) {
#pragma unroll
    for (int m = 0; m < 32; ++m) base[32 * m + lane] = Elem<T>::from_float(v[m]);
  } else {
#pragma unroll
    for (int m = 0; m < 32; ++m) {
      const int e = 32 * m + lane;
      if (e < valid) base[e] = Elem<T>::from_float(v[m]);
    }
  }
}

template <int BITS, typename T>
__device__ __forceinline__ void rht_tc_body(const ARParams& p) {
  constexpr int RB = (BITS >= 2 && BITS <= 8) ? BITS : 8;
  extern __shared__ __align__(1024) uint8_t smem_tc[];
  // swizzled operand atoms must be 1024-byte aligned in the shared address space: align by hand (the size
  // computed by rht_tc_smem_bytes has the slack)
  uint8_t* smem_raw = smem_tc + ((1024u - (tc::smem_u32(smem_tc) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  const int nwg = nwarps >> 2, wg = warp >> 2, wi = warp & 3;
  const bool use_stage = p.prefetch != 0;

  // ---- shared memory ----
  uint8_t* cursor = smem_raw;
  uint8_t* a1 = cursor + static_cast<size_t>(wg) * tc::kOperandBytes;
  cursor += static_cast<size_t>(nwg) * tc::kOperandBytes;
  uint8_t* a2 = cursor + static_cast<size_t>(wg) * tc::kOperandBytes;
  cursor += static_cast<size_t>(nwg) * tc::kOperandBytes;
  T* stage = reinterpret_cast<T*>(cursor + static_cast<size_t>(warp) * 4096);
  if (use_stage) cursor += static_cast<size_t>(nwarps) * 4096;
  uint8_t* hmat = cursor;
  cursor += tc::kHBytes;
  float* sgn_fwd = reinterpret_cast<float*>(cursor);
  cursor += 4096;
  float* sgn_inv = reinterpret_cast<float*>(cursor);  // column layout, swizzled: see below
  cursor += 4096;
  uint32_t* sign_words = reinterpret_cast<uint32_t*>(cursor);
  cursor += 32 * 4;
  int4* tab = reinterpret_cast<int4*>(cursor);  // per step: {lo, hi, shard_lo, flags}
  cursor += kMaxSteps * 16;
  uint64_t* sbar = reinterpret_cast<uint64_t*>(cursor) + warp;  // this warp's bulk-copy barrier
  cursor += static_cast<size_t>(nwarps) * 8;
  uint64_t* bar1 = reinterpret_cast<uint64_t*>(cursor) + 2 * wg;  // MMA1 / MMA2 completion of the warpgroup
  uint64_t* bar2 = bar1 + 1;
  cursor += static_cast<size_t>(nwg) * 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cursor);
  int* tc_error = reinterpret_cast<int*>(cursor + 8);

  enum : int { kFwd = 1, kDec = 2, kFin = 4 };
  const int per_cta = (p.blocks_per_shard + G - 1) / G;
  if (tid < 32) sign_words[tid] = sign_word(tid, p.step, p.bucket_id, p.seed_lo, p.seed_hi);
  if (tid < p.nsteps) {
    int shard_lo, lo, hi;
    step_range(p, tid, cta, per_cta, shard_lo, lo, hi);
    const int out = p.steps[tid][4];
    const int flags = ((p.steps[tid][1] == kLocalRaw && out != kOutDecode) ? kFwd : 0) | (out == kOutDecode ? kDec : 0) |
                      (out == kOutFinal ? kFin : 0);
    tab[tid] = make_int4(lo, hi, shard_lo, flags);
  }
  tc::fill_hadamard32(hmat, tid, blockDim.x);
  if (lane == 0) mbar_init(sbar, 1);
  if (wi == 0 && lane == 0) {
    mbar_init(bar1, 1);
    mbar_init(bar2, 1);
  }
  if (tid == 0) *tc_error = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  const uint32_t tmem_cols = nwg == 1 ? 64u : nwg == 2 ? 128u : 256u;  // D1 | D2 (64 columns) per warpgroup, a power of two
  if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
  __syncthreads();
  // Sign tables.  Forward: +-1 in element order (the staged raw block is read in element order).
  // Inverse: +-c for the column layout, where lane j holds elements 32 i + j in registers i = 0..31: the
  // 16-byte chunk of registers 4 q .. 4 q + 3 of lane j sits at float index 32 j + 4 (q ^ (j & 7)), so the eight
  // lanes of a quarter warp read eight different bank groups.
  for (int e = tid; e < 1024; e += blockDim.x) {
    const bool neg = (sign_words[e >> 5] >> (e & 31)) & 1u;
    sgn_fwd[e] = neg ? -1.0f : 1.0f;
    const int i = e >> 5, j = e & 31;
    sgn_inv[32 * j + 4 * ((i >> 2) ^ (j & 7)) + (i & 3)] = neg ? -p.finish_scale : p.finish_scale;
  }
  tc::fence_async_smem();  // H_32 was written by threads and is read by the tensor core
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_wg = tmem_base + static_cast<uint32_t>(wg) * 64u;         // D1; D2 is 32 columns further
  const uint32_t tmem_row = tmem_wg + (static_cast<uint32_t>(wi * 32) << 16);  // this warp's 32 lanes
  const uint32_t hmat_u32 = tc::smem_u32(hmat), a1_u32 = tc::smem_u32(a1), a2_u32 = tc::smem_u32(a2);
  const bool leader = (wi == 0 && lane == 0);
  const int barrier_id = 1 + wg;

  T* bucket = static_cast<T*>(p.bucket);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(bucket) & 15u) == 0;
  uint8_t* my_mail = p.mail[p.rank];
  const uint32_t* my_flags = p.flags[p.rank];
  const int tail_block = (p.n % kBlock) ? p.nblocks - 1 : -1;
  constexpr uint32_t kBlockBytes = kBlock * sizeof(T);
  const int qstride = 4 * nwg;  // blocks between consecutive quads of a warpgroup
  const int nsteps = p.nsteps;
  const long long n_elems = p.n;

  // ---- pipeline state: uniform over the warpgroup except `pf_blk`, which is per warp ----
  bool in1 = false, in2 = false;          // an MMA1 / MMA2 is in flight
  Quad sc{-1, -1};                        // forward: the next quad to stage
  int sc_hi = 0;                          // end of sc's step
  uint32_t par1 = 0, par2 = 0, spar = 0;
  int pf_blk = -1;                        // raw block in (or on its way into) this warp's stage
  bool prefetch_ok = use_stage && vec_ok;

  // first quad of this warpgroup at or after step s among the steps that rotate forward; none past a step
  // that decodes
  auto seek = [&](int s, int& hi) -> Quad {
    for (; s < nsteps; ++s) {
      const int4 t = tab[s];
      if (t.w & kDec) break;
      if ((t.w & kFwd) && t.x + 4 * wg < t.y) {
        hi = t.y;
        return Quad{s, t.x + 4 * wg};
      }
      if (t.w & kFin) break;
    }
    return Quad{-1, -1};
  };
  auto advance = [&](Quad q, int& hi) -> Quad {
    if (q.base + qstride < hi) return Quad{q.s, q.base + qstride};
    if (tab[q.s].w & kFin) return Quad{-1, -1};
    return seek(q.s + 1, hi);
  };
  auto prefetch_block = [&](Quad q, int hi) {  // this warp's block of quad q -> stage
    pf_blk = -1;
    const int blk = q.base + wi;
    if (!prefetch_ok || q.s < 0 || blk >= hi || blk == tail_block) return;
    pf_blk = blk;
    if (lane == 0) bulk_prefetch(stage, bucket + static_cast<long long>(blk) * kBlock, kBlockBytes, sbar);
  };
  auto mma_wait = [&](uint64_t* bar, uint32_t& parity) {
    if (!mbar_wait(bar, parity)) atomicExch(tc_error, 1);
    parity ^= 1u;
  };

  // One tick of the pipeline (see the file comment).  `read` (a compile-time tag): hand the coefficients of
  // the quad whose MMA2 is in flight to the caller in v.  `stage_next`: write the next quad's first operand
  // through `do_stage` (which fills A1).  `a1_mn`: that operand is MN-major (decode) or K-major (forward).
  auto tick = [&](auto read, float (&v)[32], bool stage_next, bool a1_mn, auto&& do_stage) {
    const bool transpose = in1;
    if constexpr (decltype(read)::value) mma_wait(bar2, par2);
    if (transpose) mma_wait(bar1, par1);
    tc::tc_fence_after();
    if (transpose) {
      float rd[32];
      tc::tmem_load32(tmem_row, rd);
      store_mn_column(a2, 32 * wi, lane, rd);
    }
    if (stage_next) do_stage();
    if constexpr (decltype(read)::value) tc::tmem_load32(tmem_row + 32, v);
    tc::fence_async_smem();
    tc::tc_fence_before();
    wg_sync(barrier_id);
    if (leader) {
      tc::tc_fence_after();
      if (transpose) {
        tc::mma_tile_k32_mn(tmem_wg + 32, a2_u32, hmat_u32);
        tc::mma_commit(bar2);
      }
      if (stage_next) {
        if (a1_mn) tc::mma_tile_k32_mn(tmem_wg, a1_u32, hmat_u32);
        else tc::mma_tile_k32(tmem_wg, a1_u32, hmat_u32, false);
        tc::mma_commit(bar1);
      }
    }
    in2 = transpose;
    in1 = stage_next;
  };
  // forward staging of quad `sc`: raw block -> signs -> A1 (K-major); then the bulk copy of the quad after it
  auto stage_forward = [&]() {
    const int blk = sc.base + wi;
    int nhi = sc_hi;
    const Quad nq = advance(sc, nhi);
    if (blk < sc_hi) {
      float x[32];
      const long long e0 = static_cast<long long>(blk) * kBlock;
      if (pf_blk == blk && mbar_wait(sbar, spar)) {
        spar ^= 1u;
        load_block<T>(stage, kBlock, true, lane, x);
        __syncwarp();  // every lane has read the stage before the next copy overwrites it
      } else {
        if (pf_blk == blk) {  // the copy never completed: report it, read directly and stop prefetching
          report_failure(p, kErrCopyTimeout, sc.s, -1);
          prefetch_ok = false;
        }
        const int valid = static_cast<int>(min(static_cast<long long>(kBlock), n_elems - e0));
        load_block<T>(bucket + e0, valid, vec_ok, lane, x);
      }
      prefetch_block(nq, nhi);
      scale_by_table(x, sgn_fwd, lane);
#pragma unroll
      for (int j = 0; j < 8; ++j)  // element 128 j + 4 lane + k = row 4 j + lane / 8, column 4 (lane % 8) + k
        *reinterpret_cast<float4*>(a1 + tc::operand_offset(32 * wi + 4 * j + (lane >> 3), (lane & 7) * 4)) =
            make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
    } else {
      prefetch_block(nq, nhi);
    }
    sc = nq;
    sc_hi = nhi;
  };
  // rotated coefficients of quad q (lane j', register i' <-> coefficient 32 i' + j'); pipeline advanced
  auto consume_forward = [&](Quad q, int hi, float (&v)[32]) {
    if (!in1 && !in2 && !same_quad(sc, q)) {  // the pipeline ran dry before q (after a decode phase)
      sc = q;
      sc_hi = hi;
      pf_blk = -1;
    }
    // Quads enter and leave the pipeline in cursor order and are asked for in that order, so the oldest
    // quad in flight is always the one wanted.  A dry pipeline takes two ticks to fill; after that every
    // call is one straight-line tick.
    if (!in2) {
      float none[32];
      for (int fill = 0; fill < 2 && !in2; ++fill) tick(FillTag{}, none, sc.s >= 0, false, stage_forward);
      if (!in2) {  // cannot happen while the cursor and the block loop agree; not a hang
        atomicExch(tc_error, 2);
        return;
      }
    }
    tick(ReadTag{}, v, sc.s >= 0, false, stage_forward);
  };

  // ---- decode: message in `slot` -> dequantise -> inverse rotation -> bucket, blocks [lo, hi) ----
  const unsigned long long scales_off_dec = p.scales_off;
  auto decode_range = [&](const uint8_t* slot, int shard_lo, int lo, int hi) {
    const int b0 = lo + 4 * wg;
    if (b0 >= hi) return;
    const int nq = (hi - b0 + qstride - 1) / qstride;
    uint32_t wc[RB];
    float sc_w = 0.f;
    auto load_codes = [&](int k) {  // codes of this warp's block of quad k into wc / sc_w
      const int blk = b0 + k * qstride + wi;
      if (blk < hi) {
        const int bs = blk - shard_lo;
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (RB * 32);
#pragma unroll
        for (int j = 0; j < RB; ++j) wc[j] = ld_cg_u32(codes + j * 32 + lane);
        sc_w = __ldcg(reinterpret_cast<const float*>(slot + scales_off_dec) + bs);
      }
    };
    int ks = 0;  // quad staged by the next tick
    auto stage_inverse = [&]() {  // dequantised coefficients of quad ks -> A1 (MN-major)
      const int blk = b0 + ks * qstride + wi;
      if (blk < hi) {
        float y[32];
        dequantize_block<RB>(wc, sc_w, y);
        store_mn_column(a1, 32 * wi, lane, y);
      }
      ++ks;
    };
    load_codes(0);
    for (int k = 0; k < 2; ++k) {  // two ticks fill the pipeline
      float none[32];
      tick(FillTag{}, none, k < nq, true, stage_inverse);
      if (k + 1 < nq) load_codes(k + 1);
    }
    for (int k = 0; k < nq; ++k) {  // then one quad comes out per tick
      float v[32];
      tick(ReadTag{}, v, k + 2 < nq, true, stage_inverse);
      if (k + 3 < nq) load_codes(k + 3);
      const int blk = b0 + k * qstride + wi;
      if (blk < hi) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // x (+-c): registers 4 q .. 4 q + 3 of this lane's column
          const float4 t = *reinterpret_cast<const float4*>(sgn_inv + 32 * lane + 4 * (q ^ (lane & 7)));
          const float2 a = __fmul2_rn(make_float2(v[4 * q], v[4 * q + 1]), make_float2(t.x, t.y));
          const float2 b = __fmul2_rn(make_float2(v[4 * q + 2], v[4 * q + 3]), make_float2(t.z, t.w));
          v[4 * q] = a.x, v[4 * q + 1] = a.y, v[4 * q + 2] = b.x, v[4 * q + 3] = b.y;
        }
        const long long e0 = static_cast<long long>(blk) * kBlock;
        const int valid = static_cast<int>(min(static_cast<long long>(kBlock), n_elems - e0));
        store_block_cols<T>(bucket + e0, valid, lane, v);
      }
    }
  };

  sc = seek(0, sc_hi);
  prefetch_block(sc, sc_hi);

  // kernel parameters used inside the block loops, read once
  const unsigned long long slot_stride = p.slot_stride, scales_off = p.scales_off;
  const uint32_t rng_step = p.step, seed_lo = p.seed_lo, seed_hi = p.seed_hi, epoch = p.epoch;
  const int world = p.world, rank = p.rank;
  const bool transmit = p.no_transmit == 0;

  bool aborted = false;
  for (int s = 0; s < nsteps && !aborted; ++s) {
    const int local = p.steps[s][1], recv_slot = p.steps[s][2], nrecv = p.steps[s][3];
    const int out = p.steps[s][4], dst = p.steps[s][5], send_slot = p.steps[s][6];
    const uint32_t tag = stream_tag(p.bucket_id, static_cast<uint32_t>(p.steps[s][7]) & ~kTagStratified);
    const int strat_world = (static_cast<uint32_t>(p.steps[s][7]) & kTagStratified) ? world : 1;
    const int4 range = tab[s];
    const int lo = range.x, hi = range.y, shard_lo = range.z;
    if (hi <= lo) continue;  // producer and consumer agree on empty ranges: no flag traffic

    if (p.debug) {  // CTA-uniform: a step with an access outside its slots is not run at all
      int bad_slot;
      const bool bad = debug_step_out_of_bounds<0, true>(p, s, shard_lo, lo, hi, bad_slot);
      if (__syncthreads_or(bad)) {
        if (bad) report_failure(p, kErrBounds, s, bad_slot);
        aborted = true;
        break;
      }
    }

    if (nrecv > 0) {
      bool timed_out = false;
      int bad_slot = 0;
      if (tid < nrecv) {
        const uint32_t* f = my_flags + p.flag_base + static_cast<uint32_t>(recv_slot + tid) * G + cta;
        timed_out = !wait_flag(f, epoch, p.timeout_ns);
        bad_slot = recv_slot + tid;
      }
      if (__syncthreads_or(timed_out)) {
        if (timed_out) report_failure(p, kErrWaitTimeout, s, bad_slot);
        aborted = true;  // the whole CTA gives up; peers that depend on it time out the same way
        break;
      }
    }

    if (out == kOutDecode) {
      decode_range(my_mail + static_cast<unsigned long long>(recv_slot) * slot_stride, shard_lo, lo, hi);
      continue;
    }

    const uint8_t* recv0 = my_mail + static_cast<unsigned long long>(recv_slot < 0 ? 0 : recv_slot) * slot_stride;
    const bool to_one = out == kOutSend;
    const int strat_rank = to_one ? rank : 0, strat_w = to_one ? strat_world : 1;
    const unsigned long long send_off = static_cast<unsigned long long>(send_slot < 0 ? 0 : send_slot) * slot_stride;
    uint8_t* const send_one = p.mail[to_one ? dst : rank] + send_off;  // the single destination, or the owner's own slot
    for (int base = lo + 4 * wg; base < hi; base += qstride) {
      const int blk = base + wi;
      const bool active = blk < hi;  // warps past the end still join the warpgroup's barrier
      const int bs = blk - shard_lo;
      const long long e0 = static_cast<long long>(blk) * kBlock;
      uint32_t w[RB];
      float scale = 0.f;
      if (active && nrecv > 0) {  // first incoming message: issue its loads before the local work
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(recv0) + static_cast<size_t>(bs) * (RB * 32);
#pragma unroll
        for (int j = 0; j < RB; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
        scale = __ldcg(reinterpret_cast<const float*>(recv0 + scales_off) + bs);
      }
      float v[32];
      if (local == kLocalRaw) {
        consume_forward(Quad{s, base}, hi, v);
      } else if (active) {
        if (blk == tail_block) load_block<float>(p.tail_ws, kBlock, true, lane, v);
        else load_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
      }
      if (!active) continue;
      if (nrecv > 0) dequantize_add_block<RB>(w, scale, v);
      for (int r = 1; r < nrecv; ++r) {
        const uint8_t* slot = recv0 + static_cast<unsigned long long>(r) * slot_stride;
        const uint32_t* codes = reinterpret_cast<const uint32_t*>(slot) + static_cast<size_t>(bs) * (RB * 32);
#pragma unroll
        for (int j = 0; j < RB; ++j) w[j] = ld_cg_u32(codes + j * 32 + lane);
        scale = __ldcg(reinterpret_cast<const float*>(slot + scales_off) + bs);
        dequantize_add_block<RB>(w, scale, v);
      }
      if (out == kOutStore) {
        if (blk == tail_block) store_block<float>(p.tail_ws, kBlock, true, lane, v);
        else store_block<T>(bucket + e0, kBlock, vec_ok, lane, v);
        continue;
      }
      scale = quantize_block<RB>(v, w, static_cast<uint32_t>(blk), tag, rng_step, seed_lo, seed_hi, lane, strat_rank,
                                 strat_w);
      auto put = [&](uint8_t* slot) {  // every lane stores the (same) scale: one transaction, no branch
        uint32_t* codes = reinterpret_cast<uint32_t*>(slot) + static_cast<size_t>(bs) * (RB * 32);
#pragma unroll
        for (int j = 0; j < RB; ++j) codes[j * 32 + lane] = w[j];
        reinterpret_cast<float*>(slot + scales_off)[bs] = scale;
      };
      if (to_one) {
        if (transmit) put(send_one);
      } else {
        put(send_one);  // the owner decodes its own all-gather slot below
        if (transmit) {
          for (int k = 1; k < world; ++k) put(p.mail[(rank + k) % world] + send_off);
        }
      }
    }

    __syncthreads();  // every warp's payload stores precede the flags (and the owner's own decode)
    if (out == kOutSend) {
      if (tid == 0) {
        __threadfence_system();
        st_release_sys(p.flags[dst] + p.flag_base + static_cast<uint32_t>(send_slot) * G + cta, epoch);
      }
    } else if (out == kOutFinal) {
      if (tid < world && tid != rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + p.flag_base + static_cast<uint32_t>(send_slot) * G + cta, epoch);
      }
      decode_range(my_mail + send_off, shard_lo, lo, hi);
    }
  }

  // leaving: let whatever is still in flight land before the TMEM columns and the CTA's memory go away
  if (pf_blk >= 0) mbar_wait(sbar, spar);
  if (in1) mbar_wait(bar1, par1);
  if (in2) mbar_wait(bar2, par2);
  if (tid == 0 && *tc_error) report_failure(p, kErrMmaTimeout, *tc_error, -1);
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace dq
