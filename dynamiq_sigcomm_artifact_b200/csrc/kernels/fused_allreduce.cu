#include <atomic>
// Persistent compressed all-reduce over peer-mapped NVLink memory (sm_100a).
//
// One cooperative launch per bucket performs the whole collective: rotation, scaling,
// stochastic quantisation, packing, the reduce-scatter hops (decode + add + re-encode), the
// all-gather and the inverse rotation.  Payloads are written straight into the consumer
// GPU's mailbox with peer stores, followed by a release store of a sequence flag; consumers
// poll the flag with acquire loads under a time budget.  No library collective is called.
//
// Replaces, in the reference: the compress / hop / decompress kernels
// (cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hierarchical_mee.cu:203-696), the Python ring
// and butterfly schedulers around them (testbed_evaluation/new_comm_hooks/utils.py:78-226,
// ring_rdma.py:565-832) and the staged host transport
// (rdma_comm_compress/ring_allreduce_ext/ring_allreduce_backend.cu:685-1766).
//
// Work split: CTA c owns the same contiguous range of blocks of every shard on every rank,
// so step s of CTA c on one GPU depends only on step s-1 of CTA c on another GPU; one flag
// per (slot, CTA).  Every message has its own slot, so nothing is reused inside a collective;
// consecutive collectives alternate between two slot sets.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cuda_bf16.h>
#include "fused_allreduce.cuh"

namespace dq {

static constexpr int kBlock = 1024;  // codec block, elements

// defined in fused_allreduce_b{2..8}.cu
template <int BITS, typename T, int CODEC>
void launch_one(const ARParams* host_params, const ARParams* dev_params, int nranks, int ctas, int threads,
                cudaStream_t stream);

template <typename T, int CODEC>
static void launch_rht(int bits, const ARParams* hp, const ARParams* dp, int nranks, int ctas, int threads,
                       cudaStream_t stream) {
  switch (bits) {
    case 2: launch_one<2, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 3: launch_one<3, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 4: launch_one<4, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 5: launch_one<5, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 6: launch_one<6, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 7: launch_one<7, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 8: launch_one<8, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    default: TORCH_CHECK(false, "bits must be in 2..8, got ", bits);
  }
}

template <typename T, int CODEC>
static void launch_sc(int bits, const ARParams* hp, const ARParams* dp, int nranks, int ctas, int threads,
                      cudaStream_t stream) {
  switch (bits) {
    case 2: launch_one<2, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 4: launch_one<4, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    case 8: launch_one<8, T, CODEC>(hp, dp, nranks, ctas, threads, stream); break;
    default: TORCH_CHECK(false, "the superchunk codec has 2, 4 and 8 bit codes, got ", bits);
  }
}

template <typename T>
static void launch_mx(int bits, const ARParams* hp, const ARParams* dp, int nranks, int ctas, int threads,
                      cudaStream_t stream) {
  switch (bits) {
    case 4: launch_one<4, T, kCodecMx>(hp, dp, nranks, ctas, threads, stream); break;
    case 6: launch_one<6, T, kCodecMx>(hp, dp, nranks, ctas, threads, stream); break;
    case 8: launch_one<8, T, kCodecMx>(hp, dp, nranks, ctas, threads, stream); break;
    default: TORCH_CHECK(false, "the block-float codec has 4, 6 and 8 bit codes, got ", bits);
  }
}

template <typename T>
static void launch_cast(int bits, const ARParams* hp, const ARParams* dp, int nranks, int ctas, int threads,
                        cudaStream_t stream) {
  switch (bits) {
    case 16: launch_one<16, T, kCodecCast>(hp, dp, nranks, ctas, threads, stream); break;
    case 32: launch_one<32, T, kCodecCast>(hp, dp, nranks, ctas, threads, stream); break;
    default: TORCH_CHECK(false, "the identity wire carries bf16 (16) or fp32 (32) values, got ", bits);
  }
}

// `codec`: kCodecRht (SIMT rotation), kCodecRhtTc (tcgen05 rotation), kCodecScAee, kCodecScMee, kCodecMx
template <typename T>
static void launch_bits(int bits, const ARParams* hp, const ARParams* dp, int nranks, int ctas, int threads,
                        cudaStream_t stream, int codec) {
  switch (codec) {
    case kCodecRht: launch_rht<T, kCodecRht>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecRhtTc: launch_rht<T, kCodecRhtTc>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecScAee: launch_sc<T, kCodecScAee>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecScMee: launch_sc<T, kCodecScMee>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecMx: launch_mx<T>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecCast: launch_cast<T>(bits, hp, dp, nranks, ctas, threads, stream); break;
    case kCodecScMixAee: launch_one<8, T, kCodecScMixAee>(hp, dp, nranks, ctas, threads, stream); break;
    case kCodecScMixMee: launch_one<8, T, kCodecScMixMee>(hp, dp, nranks, ctas, threads, stream); break;
    case kCodecRhtMix: launch_one<8, T, kCodecRhtMix>(hp, dp, nranks, ctas, threads, stream); break;
    default: TORCH_CHECK(false, "unknown codec ", codec);
  }
}

static unsigned block_bytes_of(int codec, int bits) {
  if (codec == kCodecScAee || codec == kCodecScMee) return 4u * (16u * (2u * bits + 1u) + 2u);
  if (codec == kCodecScMixAee || codec == kCodecScMixMee) return 4u * 274u;  // the widest block: four 8-bit records
  if (codec == kCodecMx) return 128u * bits + 32u;
  if (codec == kCodecCast) return 128u * bits;
  if (codec == kCodecRhtMix) return 128u * 8u;  // slots are sized for the widest block
  return 128u * bits;
}

// superchunk codec constants; `lut` holds the 2^bits decode levels (device, fp32)
static void fill_sc(ARParams& p, int64_t codec, int64_t bits, double lattice_max, double c1, double c2,
                    const c10::optional<at::Tensor>& lut, const c10::optional<at::Tensor>& plan) {
  p.codec = static_cast<int>(codec);
  p.tensor_rotation = codec == kCodecRhtTc;
  p.block_bytes = block_bytes_of(static_cast<int>(codec), static_cast<int>(bits));
  p.sc_lattice_max = static_cast<float>(lattice_max);
  p.sc_c1 = static_cast<float>(c1);
  p.sc_c2 = static_cast<float>(c2);
  p.sc_lut = nullptr;
  if (codec == kCodecScMee) {
    TORCH_CHECK(lut.has_value() && lut->is_cuda() && lut->scalar_type() == at::kFloat && lut->is_contiguous() &&
                    lut->numel() >= (1 << bits),
                "the MEE codec needs a CUDA fp32 table of 2^bits decode levels");
    p.sc_lut = lut->data_ptr<float>();
  }
  if (codec == kCodecScAee || codec == kCodecScMee) TORCH_CHECK(lattice_max > 0, "lattice_max must be positive");
  p.sc_plan = nullptr;
  if (codec == kCodecScMixAee || codec == kCodecScMixMee) {
    TORCH_CHECK(lut.has_value() && lut->is_cuda() && lut->scalar_type() == at::kFloat && lut->is_contiguous() &&
                    lut->numel() >= 292,
                "the mixed-width codec needs its CUDA fp32 constant table (292 values)");
    TORCH_CHECK(plan.has_value() && plan->is_cuda() && plan->scalar_type() == at::kInt && plan->is_contiguous() &&
                    plan->numel() >= 2 * static_cast<int64_t>(p.nblocks) + 1,
                "the mixed-width codec needs an int32 CUDA plan of nblocks + 1 offsets and nblocks packed widths");
    p.sc_lut = lut->data_ptr<float>();
    p.sc_plan = reinterpret_cast<const uint32_t*>(plan->data_ptr<int>());
  }
  if (codec == kCodecRhtMix) {
    TORCH_CHECK(plan.has_value() && plan->is_cuda() && plan->scalar_type() == at::kInt && plan->is_contiguous() &&
                    plan->numel() >= 2 * static_cast<int64_t>(p.nblocks) + 1,
                "the mixed-width rotation codec needs an int32 CUDA plan of nblocks + 1 offsets and nblocks widths");
    p.sc_plan = reinterpret_cast<const uint32_t*>(plan->data_ptr<int>());
  }
}

// Process-wide switch of the kernels' debug mode (ARParams::debug), set from Python (`set_debug`).
static std::atomic<int> g_debug{0};
void set_debug(bool on) { g_debug.store(on ? 1 : 0); }

static void fill_common(ARParams& p, const at::Tensor& bucket, const at::Tensor& steps, int64_t rank, int64_t world,
                        int64_t blocks_per_shard, int64_t slot_stride, int64_t scales_off, int64_t flag_base,
                        int64_t epoch, int64_t seed, int64_t step, int64_t bucket_id, double post_scale,
                        int64_t timeout_ns, int64_t status_ptr, int64_t tail_ws_ptr, bool no_transmit) {
  TORCH_CHECK(bucket.is_cuda() && bucket.is_contiguous(), "bucket must be a contiguous CUDA tensor");
  TORCH_CHECK(bucket.scalar_type() == at::kFloat || bucket.scalar_type() == at::kBFloat16,
              "bucket must be float32 or bfloat16");
  TORCH_CHECK(steps.device().is_cpu() && steps.scalar_type() == at::kInt && steps.dim() == 2 &&
                  steps.size(1) == kStepInts && steps.is_contiguous(),
              "steps must be a CPU int32 [nsteps, 8] tensor");
  TORCH_CHECK(steps.size(0) <= kMaxSteps, "program too long");
  TORCH_CHECK(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "bad rank/world");
  p.bucket = bucket.data_ptr();
  p.n = bucket.numel();
  p.nblocks = static_cast<int>((p.n + kBlock - 1) / kBlock);
  p.blocks_per_shard = static_cast<int>(blocks_per_shard);
  TORCH_CHECK(p.blocks_per_shard * world >= p.nblocks, "shards do not cover the bucket");
  p.world = static_cast<int>(world);
  p.rank = static_cast<int>(rank);
  p.nsteps = static_cast<int>(steps.size(0));
  p.slot_stride = static_cast<unsigned long long>(slot_stride);
  p.scales_off = static_cast<unsigned long long>(scales_off);
  p.flag_base = static_cast<uint32_t>(flag_base);
  p.epoch = static_cast<uint32_t>(epoch);
  p.seed_lo = static_cast<uint32_t>(static_cast<uint64_t>(seed) & 0xFFFFFFFFull);
  p.seed_hi = static_cast<uint32_t>(static_cast<uint64_t>(seed) >> 32);
  p.step = static_cast<uint32_t>(step);
  p.bucket_id = static_cast<uint32_t>(bucket_id);
  p.finish_scale = static_cast<float>(post_scale / 1024.0);
  p.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  p.status = reinterpret_cast<uint32_t*>(status_ptr);
  p.tail_ws = reinterpret_cast<float*>(tail_ws_ptr);
  p.no_transmit = no_transmit ? 1 : 0;
  p.debug = g_debug.load();
  const int* sp = steps.data_ptr<int>();
  for (int s = 0; s < p.nsteps; ++s)
    for (int k = 0; k < kStepInts; ++k) p.steps[s][k] = sp[s * kStepInts + k];
}

static void check_layout(ARParams& p, int bits, int64_t mailbox_bytes, int64_t nslots, int64_t flag_words,
                         int ctas) {
  (void)bits;
  p.nslots = static_cast<int>(nslots);
  p.set_bytes = static_cast<unsigned long long>(mailbox_bytes);
  const unsigned long long need = static_cast<unsigned long long>(p.blocks_per_shard) * p.block_bytes;
  const bool has_scales = p.codec == kCodecRht || p.codec == kCodecRhtTc || p.codec == kCodecRhtMix;  // fp32 scales after the codes
  TORCH_CHECK(p.scales_off >= need && (p.scales_off % 16) == 0, "scales overlap the codes of a slot");
  TORCH_CHECK(p.slot_stride >= p.scales_off + (has_scales ? 4ull * p.blocks_per_shard : 0ull) &&
                  (p.slot_stride % 16) == 0,
              "slot stride too small");
  TORCH_CHECK(static_cast<unsigned long long>(nslots) * p.slot_stride <= static_cast<unsigned long long>(mailbox_bytes),
              "mailbox too small for ", nslots, " slots");
  TORCH_CHECK(static_cast<long long>(p.flag_base) + nslots * ctas <= flag_words, "flag array too small");
  for (int s = 0; s < p.nsteps; ++s) {
    const int* st = p.steps[s];
    TORCH_CHECK(st[0] >= 0 && st[0] < p.world, "step ", s, ": bad shard");
    TORCH_CHECK(st[3] == 0 || (st[2] >= 0 && st[2] + st[3] <= nslots), "step ", s, ": bad receive slots");
    if (st[4] == kOutSend) TORCH_CHECK(st[5] >= 0 && st[5] < p.world && st[6] >= 0 && st[6] < nslots, "step ", s, ": bad send");
    if (st[4] == kOutFinal) TORCH_CHECK(st[6] >= 0 && st[6] < nslots, "step ", s, ": bad final slot");
  }
}

// One rank of a real multi-GPU collective.  mail_ptrs / flag_ptrs: device addresses of every
// rank's mailbox and flag array as mapped into this process.
void fused_allreduce(at::Tensor bucket, at::Tensor steps, std::vector<int64_t> mail_ptrs,
                     std::vector<int64_t> flag_ptrs, int64_t mailbox_bytes, int64_t flag_words, int64_t nslots,
                     int64_t status_ptr, int64_t tail_ws_ptr, int64_t rank, int64_t world, int64_t bits, int64_t ctas,
                     int64_t threads, int64_t blocks_per_shard, int64_t slot_stride, int64_t scales_off,
                     int64_t flag_base, int64_t epoch, int64_t seed, int64_t step, int64_t bucket_id,
                     double post_scale, int64_t timeout_ns, bool no_transmit, int64_t codec, double sc_lattice_max, double sc_c1, double sc_c2,
                     c10::optional<at::Tensor> sc_lut, c10::optional<at::Tensor> sc_plan, bool prefetch) {
  c10::cuda::CUDAGuard guard(bucket.device());
  TORCH_CHECK(static_cast<int64_t>(mail_ptrs.size()) == world && static_cast<int64_t>(flag_ptrs.size()) == world,
              "need one mailbox and one flag pointer per rank");
  TORCH_CHECK(threads % 32 == 0 && threads >= 32 && threads <= 512, "threads must be a multiple of 32, at most 512");
  ARParams p{};
  fill_common(p, bucket, steps, rank, world, blocks_per_shard, slot_stride, scales_off, flag_base, epoch, seed, step,
              bucket_id, post_scale, timeout_ns, status_ptr, tail_ws_ptr, no_transmit);
  fill_sc(p, codec, bits, sc_lattice_max, sc_c1, sc_c2, sc_lut, sc_plan);
  p.prefetch = prefetch ? 1 : 0;
  for (int r = 0; r < world; ++r) {
    p.mail[r] = reinterpret_cast<uint8_t*>(mail_ptrs[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  check_layout(p, static_cast<int>(bits), mailbox_bytes, nslots, flag_words, static_cast<int>(ctas));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  if (bucket.scalar_type() == at::kFloat)
    launch_bits<float>(static_cast<int>(bits), &p, nullptr, 1, static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
  else
    launch_bits<__nv_bfloat16>(static_cast<int>(bits), &p, nullptr, 1, static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
}

// All ranks of a collective in one launch on one GPU.  buckets[r], mailboxes[r] (uint8),
// flags[r] (int32) and steps[r] belong to rank r; status is a 4-word int32 tensor and
// tail_ws a [world, 1024] float tensor.
void fused_allreduce_local(std::vector<at::Tensor> buckets, at::Tensor steps, std::vector<at::Tensor> mailboxes,
                           std::vector<at::Tensor> flags, at::Tensor status, at::Tensor tail_ws, int64_t nslots,
                           int64_t bits, int64_t ctas, int64_t threads, int64_t blocks_per_shard, int64_t slot_stride,
                           int64_t scales_off, int64_t flag_base, int64_t epoch, int64_t seed, int64_t step,
                           int64_t bucket_id, double post_scale, int64_t timeout_ns, bool no_transmit, int64_t codec, double sc_lattice_max, double sc_c1, double sc_c2,
                     c10::optional<at::Tensor> sc_lut, c10::optional<at::Tensor> sc_plan, bool prefetch) {
  const int64_t world = static_cast<int64_t>(buckets.size());
  TORCH_CHECK(world >= 1 && world <= kMaxWorld, "1..8 ranks");
  TORCH_CHECK(steps.dim() == 3 && steps.size(0) == world, "steps must be [world, nsteps, 8]");
  TORCH_CHECK(static_cast<int64_t>(mailboxes.size()) == world && static_cast<int64_t>(flags.size()) == world,
              "one mailbox and one flag array per rank");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 4, "status: 4 int32 words");
  TORCH_CHECK(tail_ws.is_cuda() && tail_ws.scalar_type() == at::kFloat && tail_ws.numel() >= world * kBlock,
              "tail_ws: [world, 1024] float32");
  TORCH_CHECK(threads % 32 == 0 && threads >= 32 && threads <= 512, "threads must be a multiple of 32, at most 512");
  c10::cuda::CUDAGuard guard(buckets[0].device());
  std::vector<ARParams> hp(world);
  for (int64_t r = 0; r < world; ++r) {
    TORCH_CHECK(buckets[r].numel() == buckets[0].numel() && buckets[r].scalar_type() == buckets[0].scalar_type(),
                "buckets must agree in size and dtype");
    TORCH_CHECK(mailboxes[r].is_cuda() && mailboxes[r].is_contiguous() && flags[r].is_cuda() &&
                    flags[r].scalar_type() == at::kInt,
                "mailboxes / flags must be CUDA tensors");
    hp[r] = ARParams{};
    fill_common(hp[r], buckets[r], steps[r].contiguous(), r, world, blocks_per_shard, slot_stride, scales_off,
                flag_base, epoch, seed, step, bucket_id, post_scale, timeout_ns,
                reinterpret_cast<int64_t>(status.data_ptr()),
                reinterpret_cast<int64_t>(tail_ws.data_ptr<float>() + r * kBlock), no_transmit);
    fill_sc(hp[r], codec, bits, sc_lattice_max, sc_c1, sc_c2, sc_lut, sc_plan);
    hp[r].prefetch = prefetch ? 1 : 0;
    for (int64_t q = 0; q < world; ++q) {
      hp[r].mail[q] = static_cast<uint8_t*>(mailboxes[q].data_ptr());
      hp[r].flags[q] = reinterpret_cast<uint32_t*>(flags[q].data_ptr());
    }
    check_layout(hp[r], static_cast<int>(bits), mailboxes[r].numel() * mailboxes[r].element_size(), nslots,
                 flags[r].numel(), static_cast<int>(ctas));
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  if (world == 1) {
    if (buckets[0].scalar_type() == at::kFloat)
      launch_bits<float>(static_cast<int>(bits), hp.data(), nullptr, 1, static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
    else
      launch_bits<__nv_bfloat16>(static_cast<int>(bits), hp.data(), nullptr, 1, static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
    return;
  }
  at::Tensor dev = at::empty({static_cast<int64_t>(world * sizeof(ARParams))},
                             at::TensorOptions().dtype(at::kByte).device(buckets[0].device()));
  C10_CUDA_CHECK(cudaMemcpyAsync(dev.data_ptr(), hp.data(), world * sizeof(ARParams), cudaMemcpyHostToDevice, stream));
  C10_CUDA_CHECK(cudaStreamSynchronize(stream));  // hp is pageable host memory
  const ARParams* dp = reinterpret_cast<const ARParams*>(dev.data_ptr());
  if (buckets[0].scalar_type() == at::kFloat)
    launch_bits<float>(static_cast<int>(bits), hp.data(), dp, static_cast<int>(world), static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
  else
    launch_bits<__nv_bfloat16>(static_cast<int>(bits), hp.data(), dp, static_cast<int>(world), static_cast<int>(ctas), static_cast<int>(threads), stream, static_cast<int>(codec));
  C10_CUDA_CHECK(cudaStreamSynchronize(stream));  // keep `dev` alive until the kernel has read it
}

}  // namespace dq
