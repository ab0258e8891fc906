// Device-side bit allocation for the superchunk codec: per-superchunk code widths, the message plan of
// the mixed-width collective, and the dynamic-bitrate controller.  Nothing here reads a value back to
// the host, so a bucket's widths are chosen, packed and consumed on the stream that produced its energies.
//
// Counterparts in the reference (all host-driven torch chains with device-to-host syncs):
//   widths      _dynamic_bitrate_qbits, testbed_evaluation/new_comm_hooks/comm_hooks.py:64-70
//   plan        argsort / nonzero / index_select / index_copy_ per width group, comm_hooks.py:718-764
//   controller  _bisect_dynamic_bitrate_u / _adjust_dynamic_bitrate_u, comm_hooks.py:72-139
//
// Controller state (fp64, device): [0] u, [1] initialised (0 / 1), [2] last average width, [3] last delta.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

namespace dq {
namespace {

constexpr float kNormScale = 4.0f / (512.0f / 17.0f);
constexpr double kUMin = -10.0, kUMax = 60.0, kTol = 0.1;
constexpr int kMaxIters = 32;

// width of a superchunk from its score s + u: 8 from 8 up, 4 from 4 up, else 2
// (= 2 ** clamp(floor(log2(score)), 1, 3) with the comparisons done on the score itself)
__device__ __forceinline__ int width_of(float s, float u) {
  const float score = __fadd_rn(s, u);
  return score >= 8.0f ? 8 : (score >= 4.0f ? 4 : 2);
}

__global__ void __launch_bounds__(256) sc_widths_kernel(const float* __restrict__ stats, const double* __restrict__ state,
                                                        float* __restrict__ s_out, uint8_t* __restrict__ widths,
                                                        long long nsc) {
  const float u = static_cast<float>(state[0]);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nsc;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float s = __fmul_rn(log2f(fmaxf(stats[2 * i + 1], 1e-20f)), kNormScale);
    s_out[i] = s;
    widths[i] = static_cast<uint8_t>(width_of(s, u));
  }
}

// plan[0] = 0, plan[1 + b] = bytes of block b / 8 (turned into offsets by a prefix sum afterwards),
// plan[nb + 1 + b] = packed widths of block b; superchunks past the end count as 2-bit
__global__ void __launch_bounds__(256) sc_plan_pack_kernel(const uint8_t* __restrict__ widths, long long nsc, int nb,
                                                           int* __restrict__ plan) {
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < nb; b += gridDim.x * blockDim.x) {
    uint32_t pack = 0;
    int bytes = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = 4ll * b + j;
      int w = i < nsc ? widths[i] : 2;
      if (w != 2 && w != 4 && w != 8) w = 2;  // never index outside the tables on a malformed input
      pack |= static_cast<uint32_t>(w) << (8 * j);
      bytes += 16 * (2 * w + 1) + 2;
    }
    plan[1 + b] = bytes >> 3;
    plan[nb + 1 + b] = static_cast<int>(pack);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) plan[0] = 0;
}

// number of i with s[i] + u >= t, s ascending (s + u is monotone in s under round-to-nearest)
__device__ long long count_at_least(const float* s, long long n, float u, float t) {
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (__fadd_rn(s[mid], u) >= t) hi = mid; else lo = mid + 1;
  }
  return n - lo;
}

__device__ double average_width(const float* s, long long n, double u) {
  const float uf = static_cast<float>(u);
  const long long c4 = count_at_least(s, n, uf, 4.0f), c8 = count_at_least(s, n, uf, 8.0f);
  return (2.0 * n + 2.0 * c4 + 4.0 * c8) / static_cast<double>(n);
}

__global__ void sc_bitrate_update_kernel(const float* __restrict__ s, long long n, double* __restrict__ state,
                                         double target) {
  if (threadIdx.x != 0 || blockIdx.x != 0 || n <= 0) return;
  double out_u, out_avg, out_delta;
  if (state[1] == 0.0) {  // first compressed step: bisect on [u_min, u_max]
    double low = kUMin, high = kUMax;
    out_u = high;
    out_avg = average_width(s, n, out_u);
    out_delta = target - out_avg;
    for (int it = 0; it < kMaxIters; ++it) {
      const double mid = 0.5 * (low + high);
      const double avg = average_width(s, n, mid), delta = target - avg;
      if (fabs(delta) < fabs(out_delta)) out_u = mid, out_avg = avg, out_delta = delta;
      if (fabs(delta) <= kTol) {
        out_u = mid, out_avg = avg, out_delta = delta;
        break;
      }
      if (delta > 0) low = mid; else high = mid;
    }
  } else {  // later steps: nudge u by the shortfall, halving until the sign holds
    const double prev = fmin(kUMax, fmax(kUMin, state[0]));
    const double old_avg = average_width(s, n, prev), old_delta = target - old_avg;
    out_u = prev, out_avg = old_avg, out_delta = old_delta;
    if (fabs(old_delta) > kTol) {
      double step = old_delta;
      for (int it = 0; it < kMaxIters; ++it) {
        const double cand = fmin(kUMax, fmax(kUMin, prev + step));
        const double avg = average_width(s, n, cand), delta = target - avg;
        if (fabs(delta) <= kTol || old_delta * delta >= 0) {
          out_u = cand, out_avg = avg, out_delta = delta;
          break;
        }
        if (fabs(delta) < fabs(out_delta)) out_u = cand, out_avg = avg, out_delta = delta;
        step *= 0.5;
      }
    }
  }
  state[0] = out_u;
  state[1] = 1.0;
  state[2] = out_avg;
  state[3] = out_delta;
}

}  // namespace

// stats [nsc, 2] (energy in column 1) + controller state -> s_out [nsc] (score without u), widths [nsc] (uint8)
void superchunk_widths(at::Tensor stats, at::Tensor state, at::Tensor s_out, at::Tensor widths) {
  TORCH_CHECK(stats.is_cuda() && stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.dim() == 2 &&
                  stats.size(1) == 2, "superchunk_widths: stats must be a contiguous CUDA fp32 [nsc, 2] tensor");
  const long long nsc = stats.size(0);
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kDouble && state.numel() >= 4 && state.is_contiguous(),
              "superchunk_widths: controller state must be 4 CUDA doubles");
  TORCH_CHECK(s_out.is_cuda() && s_out.scalar_type() == at::kFloat && s_out.is_contiguous() && s_out.numel() >= nsc &&
                  widths.is_cuda() && widths.scalar_type() == at::kByte && widths.is_contiguous() && widths.numel() >= nsc,
              "superchunk_widths: outputs must be CUDA fp32 / uint8 tensors of nsc elements");
  if (nsc == 0) return;
  c10::cuda::CUDAGuard guard(stats.device());
  const int grid = static_cast<int>(std::min<long long>((nsc + 255) / 256, 148LL * 8));
  sc_widths_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      stats.data_ptr<float>(), state.data_ptr<double>(), s_out.data_ptr<float>(), widths.data_ptr<uint8_t>(), nsc);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// widths [nsc] uint8 in {2, 4, 8} -> plan int32 [2 nb + 1]: nb + 1 block offsets (8-byte units), nb packed widths
at::Tensor superchunk_plan(at::Tensor widths) {
  TORCH_CHECK(widths.is_cuda() && widths.scalar_type() == at::kByte && widths.is_contiguous(),
              "superchunk_plan: widths must be a contiguous CUDA uint8 tensor");
  c10::cuda::CUDAGuard guard(widths.device());
  const long long nsc = widths.numel();
  const int nb = static_cast<int>((nsc + 3) / 4);
  at::Tensor plan = at::empty({2ll * nb + 1}, widths.options().dtype(at::kInt));
  if (nb == 0) return plan.zero_();
  const int grid = std::min((nb + 255) / 256, 148 * 8);
  sc_plan_pack_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(widths.data_ptr<uint8_t>(), nsc, nb,
                                                                           plan.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  at::Tensor sizes = plan.slice(0, 1, nb + 1);
  sizes.copy_(at::cumsum(sizes, 0, at::kInt));
  return plan;
}

// sorted_s: ascending scores of every superchunk of the step; updates the controller state in place
void superchunk_bitrate_update(at::Tensor sorted_s, at::Tensor state, double target) {
  TORCH_CHECK(sorted_s.is_cuda() && sorted_s.scalar_type() == at::kFloat && sorted_s.is_contiguous(),
              "superchunk_bitrate_update: scores must be a contiguous CUDA fp32 tensor");
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kDouble && state.numel() >= 4 && state.is_contiguous(),
              "superchunk_bitrate_update: controller state must be 4 CUDA doubles");
  if (sorted_s.numel() == 0) return;
  c10::cuda::CUDAGuard guard(sorted_s.device());
  sc_bitrate_update_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(sorted_s.data_ptr<float>(), sorted_s.numel(),
                                                                          state.data_ptr<double>(), target);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ---- rotation codec: a code width per 1024-element block ---------------------------------------------------
//
// width_k = clamp(round(c + log2(absmax_k)), 2, 8), one offset c per bucket, the largest whose total width
// stays within the budget (reverse water-filling; host twin and rationale: bitalloc.py, rht_block_widths).
// absmax_k = scale_k * R(previous width_k), where scale_k is what the last collective left in this rank's
// own all-gather slots - identical on every rank, so the widths need no communication and no host read.
// All arithmetic is on integers: logarithms quantised to 1/8 bit from the exponent field and seven
// comparisons, a 2048-bin histogram, a bisection on the histogram, a block-wide prefix sum.

namespace {

constexpr int kLogBins = 2048, kLogBias = 1016;  // floor(8 log2 x) + 1016 for fp32 x > 0 lies in [0, 2040]

__device__ __forceinline__ int quantised_log2(float x) {
  if (!(x > 0.0f) || x > 3.402823466e38f) return -kLogBias;
  const uint32_t bits = __float_as_uint(x);
  const int expo = static_cast<int>((bits >> 23) & 0xFFu) - 127;
  const float mant = __uint_as_float((bits & 0x007FFFFFu) | 0x3F800000u);
  const int frac = (mant >= 1.0905077f) + (mant >= 1.1892071f) + (mant >= 1.2968396f) + (mant >= 1.4142135f) +
                   (mant >= 1.5422108f) + (mant >= 1.6817929f) + (mant >= 1.8340080f);
  return 8 * expo + frac;
}

__device__ __forceinline__ int rht_width_at(int lq, int c8) { return max(2, min(8, (lq + c8 + 4) >> 3)); }

// Sum over the thread block of one long long per thread (blockDim.x a multiple of 32, at most 1024).
__device__ long long block_sum(long long v, long long* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  long long t = 0;
  for (int i = 0; i < nwarps; ++i) t += scratch[i];
  return t;
}

// The update runs as four small launches so that every pass over the blocks is spread over the whole GPU (a bucket
// of 1.2 G elements has 1.2 M blocks): (1) quantised log2 of every block's absmax + histogram, (2) bisection on the
// histogram for the offset c (one CTA), (3) new widths and their prefix sum inside tiles of 1024 blocks, (4) tile
// bases added.  Scratch (int32): [kLogBins histogram][1 offset][ntiles tile totals][nblocks logs].

__global__ void __launch_bounds__(256) rht_log_hist_kernel(const uint8_t* __restrict__ mail, const int* __restrict__ plan,
                                                           int nblocks, int blocks_per_shard, long long slot_stride,
                                                           long long scales_off, int first_ag_slot,
                                                           int* __restrict__ hist, int* __restrict__ logs) {
  __shared__ int local[kLogBins];
  const int* widths = plan + nblocks + 1;
  for (int i = threadIdx.x; i < kLogBins; i += blockDim.x) local[i] = 0;
  __syncthreads();
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < nblocks; k += gridDim.x * blockDim.x) {
    const int shard = k / blocks_per_shard, bs = k - shard * blocks_per_shard;
    const float scale = *reinterpret_cast<const float*>(mail + (first_ag_slot + shard) * slot_stride + scales_off + 4ll * bs);
    const int wprev = max(2, min(8, widths[k]));
    const int lq = quantised_log2(__fmul_rn(scale, static_cast<float>((1 << (wprev - 1)) - 1)));
    logs[k] = lq;
    atomicAdd(&local[lq + kLogBias], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kLogBins; i += blockDim.x)
    if (local[i] != 0) atomicAdd(&hist[i], local[i]);
}

__global__ void __launch_bounds__(1024, 1) rht_offset_kernel(const int* __restrict__ hist, long long budget,
                                                             int* __restrict__ offset) {
  __shared__ long long scratch[32];
  const int tid = threadIdx.x, nt = blockDim.x;
  auto total_at = [&](int c8) {
    long long v = 0;
    for (int b = tid; b < kLogBins; b += nt) v += static_cast<long long>(hist[b]) * rht_width_at(b - kLogBias, c8);
    return block_sum(v, scratch);
  };
  int lo = -2048, hi = 2048;
  if (total_at(hi) <= budget) {
    lo = hi;
  } else {
    while (hi - lo > 1) {  // total_at(lo) <= budget (or lo is the floor), total_at(hi) > budget
      const int m = (lo + hi) >> 1;  // floor, also for negative sums, like the host twin's //
      if (total_at(m) <= budget) lo = m; else hi = m;
    }
  }
  if (tid == 0) *offset = lo;
}

// tile = 1024 consecutive blocks, one per thread: new width, exclusive prefix inside the tile, tile total
__global__ void __launch_bounds__(1024, 1) rht_widths_tiles_kernel(const int* __restrict__ logs, const int* __restrict__ offset,
                                                                   int nblocks, int* __restrict__ plan,
                                                                   int* __restrict__ tile_totals) {
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int k = blockIdx.x * 1024 + tid;
  int* widths = plan + nblocks + 1;
  const int w = k < nblocks ? rht_width_at(logs[k], *offset) : 0;
  int incl = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, v, o);
      if (lane >= o) v += up;
    }
    warp_sums[lane] = v;  // inclusive over warps
  }
  __syncthreads();
  const int before = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - w;
  if (k < nblocks) {
    plan[k] = before;  // offset inside the tile; the tile's base is added by the next launch
    widths[k] = w;
  }
  if (tid == 1023) tile_totals[blockIdx.x] = warp_sums[31];
}

__global__ void __launch_bounds__(1024, 1) rht_add_tile_base_kernel(const int* __restrict__ tile_totals, int nblocks,
                                                                    int* __restrict__ plan) {
  __shared__ long long scratch[32];
  long long mine = 0;
  for (int t = threadIdx.x; t < static_cast<int>(blockIdx.x); t += blockDim.x) mine += tile_totals[t];
  const int base = static_cast<int>(block_sum(mine, scratch));
  const int k = blockIdx.x * 1024 + threadIdx.x;
  if (k < nblocks) plan[k] += base;
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) plan[nblocks] = base + tile_totals[blockIdx.x];
}

}  // namespace

// In-place update of a rotation-codec plan (int32 [2 nblocks + 1]: offsets in 128-byte units, then widths) from
// the scales that the last collective left in `mailbox` (this rank's slot set, uint8): the widths of the next
// collective of this bucket.  `budget` = total width allowed, round(target bits per value * nblocks).
void rht_widths_update(at::Tensor mailbox, at::Tensor plan, int64_t nblocks, int64_t blocks_per_shard,
                       int64_t slot_stride, int64_t scales_off, int64_t first_ag_slot, int64_t budget) {
  TORCH_CHECK(mailbox.is_cuda() && mailbox.scalar_type() == at::kByte && mailbox.is_contiguous(), "mailbox: uint8 CUDA");
  TORCH_CHECK(plan.is_cuda() && plan.scalar_type() == at::kInt && plan.is_contiguous() && plan.numel() >= 2 * nblocks + 1,
              "plan: int32 CUDA tensor of 2 nblocks + 1 entries");
  TORCH_CHECK(nblocks > 0 && blocks_per_shard > 0, "empty bucket");
  const int64_t nshards = (nblocks + blocks_per_shard - 1) / blocks_per_shard;
  TORCH_CHECK((first_ag_slot + nshards - 1) * slot_stride + scales_off + 4 * blocks_per_shard <= mailbox.numel(),
              "the all-gather slots lie outside the mailbox");
  TORCH_CHECK(scales_off % 4 == 0 && slot_stride % 4 == 0, "misaligned scales");
  c10::cuda::CUDAGuard guard(plan.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int nb = static_cast<int>(nblocks), ntiles = (nb + 1023) / 1024;
  at::Tensor scratch = at::zeros({kLogBins + 1 + ntiles + nblocks}, plan.options());
  int* hist = scratch.data_ptr<int>();
  int* offset = hist + kLogBins;
  int* tile_totals = offset + 1;
  int* logs = tile_totals + ntiles;
  const int grid = std::min((nb + 255) / 256, 148 * 4);
  rht_log_hist_kernel<<<grid, 256, 0, stream>>>(mailbox.data_ptr<uint8_t>(), plan.data_ptr<int>(), nb,
                                                static_cast<int>(blocks_per_shard), slot_stride, scales_off,
                                                static_cast<int>(first_ag_slot), hist, logs);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  rht_offset_kernel<<<1, 1024, 0, stream>>>(hist, budget, offset);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  rht_widths_tiles_kernel<<<ntiles, 1024, 0, stream>>>(logs, offset, nb, plan.data_ptr<int>(), tile_totals);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  rht_add_tile_base_kernel<<<ntiles, 1024, 0, stream>>>(tile_totals, nb, plan.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace dq
