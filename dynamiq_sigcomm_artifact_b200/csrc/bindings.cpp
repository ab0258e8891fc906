// Operator registration: every native entry point is a torch.ops.dq.* operator, loaded from
// the in-tree shared library by dynamiq_sigcomm_artifact_b200/ops/__init__.py.
// Reference counterpart: the pybind modules eden_utils
// (cuda_kernels/src/srrcomp/eden_utils/eden_utils.cpp:417-433) and ring_allreduce_native
// (rdma_comm_compress/ring_allreduce_ext/ring_allreduce_bindings.cpp:7-156).
#include <torch/extension.h>
#include <torch/library.h>

namespace dq {
at::Tensor topology();
std::tuple<int64_t, at::Tensor> symm_alloc(int64_t device, int64_t bytes);
int64_t symm_open(int64_t device, at::Tensor handle);
void symm_close(int64_t ptr);
void symm_free(int64_t ptr);
at::Tensor wrap_ptr(int64_t ptr, int64_t bytes, int64_t device);

void set_debug(bool on);
void fused_allreduce(at::Tensor bucket, at::Tensor steps, std::vector<int64_t> mail_ptrs,
                     std::vector<int64_t> flag_ptrs, int64_t mailbox_bytes, int64_t flag_words, int64_t nslots,
                     int64_t status_ptr, int64_t tail_ws_ptr, int64_t rank, int64_t world, int64_t bits, int64_t ctas,
                     int64_t threads, int64_t blocks_per_shard, int64_t slot_stride, int64_t scales_off,
                     int64_t flag_base, int64_t epoch, int64_t seed, int64_t step, int64_t bucket_id,
                     double post_scale, int64_t timeout_ns, bool no_transmit, int64_t codec, double sc_lattice_max, double sc_c1, double sc_c2,
                     c10::optional<at::Tensor> sc_lut, c10::optional<at::Tensor> sc_plan, bool prefetch);
void fused_allreduce_local(std::vector<at::Tensor> buckets, at::Tensor steps, std::vector<at::Tensor> mailboxes,
                           std::vector<at::Tensor> flags, at::Tensor status, at::Tensor tail_ws, int64_t nslots,
                           int64_t bits, int64_t ctas, int64_t threads, int64_t blocks_per_shard, int64_t slot_stride,
                           int64_t scales_off, int64_t flag_base, int64_t epoch, int64_t seed, int64_t step,
                           int64_t bucket_id, double post_scale, int64_t timeout_ns, bool no_transmit, int64_t codec, double sc_lattice_max, double sc_c1, double sc_c2,
                     c10::optional<at::Tensor> sc_lut, c10::optional<at::Tensor> sc_plan, bool prefetch);
std::tuple<at::Tensor, at::Tensor, at::Tensor> norm_fwd(at::Tensor x, at::Tensor w, c10::optional<at::Tensor> b,
                                                        double eps, bool rms);
std::tuple<at::Tensor, at::Tensor, at::Tensor> norm_bwd(at::Tensor dy, at::Tensor x, at::Tensor w, at::Tensor mean,
                                                        at::Tensor rstd, bool rms, c10::optional<at::Tensor> dw_out,
                                                        c10::optional<at::Tensor> db_out);
std::tuple<at::Tensor, at::Tensor> ce_fwd(at::Tensor logits, at::Tensor labels, int64_t vocab, int64_t ignore_index);
at::Tensor ce_bwd(at::Tensor logits, at::Tensor labels, at::Tensor lse, at::Tensor gout, at::Tensor n_valid,
                  int64_t vocab, int64_t ignore_index);
std::tuple<at::Tensor, at::Tensor> fwht1024_tcgen05(at::Tensor x, int64_t seed, int64_t step, int64_t bucket,
                                                    bool apply_signs, double scale, int64_t ctas);
at::Tensor bins_to_bits(at::Tensor bins, int64_t nbits);
at::Tensor bits_to_bins(at::Tensor words, int64_t nbits, int64_t n);
at::Tensor colsum(at::Tensor x, c10::optional<at::Tensor> out);
void scatter_add_rows(at::Tensor grad, at::Tensor ids, at::Tensor rows, double scale);
at::Tensor swiglu_fwd(at::Tensor in);
at::Tensor swiglu_bwd(at::Tensor dy, at::Tensor in);
std::tuple<at::Tensor, at::Tensor> superchunk_center(at::Tensor x, int64_t world);
void superchunk_add_mean(at::Tensor resid, at::Tensor mean, at::Tensor out);
void fwht_levels_(at::Tensor x, int64_t first, int64_t nlevels, double scale);
void superchunk_widths(at::Tensor stats, at::Tensor state, at::Tensor s_out, at::Tensor widths);
at::Tensor superchunk_plan(at::Tensor widths);
void superchunk_bitrate_update(at::Tensor sorted_s, at::Tensor state, double target);
void nvls_allreduce(at::Tensor bucket, int64_t stage_ptr, int64_t mc_ptr, std::vector<int64_t> flag_ptrs,
                    int64_t stage_bytes, int64_t status_ptr, int64_t rank, int64_t world, int64_t wire_bits, int64_t epoch,
                    double post_scale, int64_t timeout_ns, int64_t ctas);
void thc_quantize_(at::Tensor y, at::Tensor stats, int64_t world, double t_over_sqrt_d, int64_t levels, int64_t stream,
                   int64_t step, int64_t seed);
void thc_dequantize_(at::Tensor total, at::Tensor stats, int64_t world, double t_over_sqrt_d, int64_t levels);
void rht_widths_update(at::Tensor mailbox, at::Tensor plan, int64_t nblocks, int64_t blocks_per_shard,
                       int64_t slot_stride, int64_t scales_off, int64_t first_ag_slot, int64_t budget);
at::Tensor rope(at::Tensor x, at::Tensor cos, at::Tensor sin, bool backward);
void adamw_step(at::Tensor table, at::Tensor numel, at::Tensor chunk_start, int64_t total_chunks, bool param_bf16,
                bool grad_bf16, double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step,
                double grad_scale);
}  // namespace dq

TORCH_LIBRARY(dq, m) {
  m.def("norm_fwd(Tensor x, Tensor w, Tensor? b, float eps, bool rms) -> (Tensor, Tensor, Tensor)", &dq::norm_fwd);
  m.def("norm_bwd(Tensor dy, Tensor x, Tensor w, Tensor mean, Tensor rstd, bool rms, Tensor(a!)? dw_out=None, Tensor(b!)? db_out=None) -> (Tensor, Tensor, Tensor)", &dq::norm_bwd);
  m.def("ce_fwd(Tensor logits, Tensor labels, int vocab, int ignore_index) -> (Tensor, Tensor)", &dq::ce_fwd);
  m.def("ce_bwd(Tensor(a!) logits, Tensor labels, Tensor lse, Tensor gout, Tensor n_valid, int vocab, int ignore_index) -> Tensor(a!)", &dq::ce_bwd);
  m.def("fwht1024_tcgen05(Tensor x, int seed, int step, int bucket, bool apply_signs, float scale, int ctas) -> (Tensor, Tensor)", &dq::fwht1024_tcgen05);
  m.def("bins_to_bits(Tensor bins, int nbits) -> Tensor", &dq::bins_to_bits);
  m.def("bits_to_bins(Tensor words, int nbits, int n) -> Tensor", &dq::bits_to_bins);
  m.def("colsum(Tensor x, Tensor(a!)? out=None) -> Tensor(a!)", &dq::colsum);
  m.def("scatter_add_rows(Tensor(a!) grad, Tensor ids, Tensor rows, float scale) -> ()", &dq::scatter_add_rows);
  m.def("swiglu_fwd(Tensor x) -> Tensor", &dq::swiglu_fwd);
  m.def("swiglu_bwd(Tensor dy, Tensor x) -> Tensor", &dq::swiglu_bwd);
  m.def("superchunk_center(Tensor x, int world) -> (Tensor, Tensor)", &dq::superchunk_center);
  m.def("superchunk_add_mean(Tensor resid, Tensor mean, Tensor(a!) out) -> ()", &dq::superchunk_add_mean);
  m.def("fwht_levels_(Tensor(a!) x, int first, int nlevels, float scale) -> ()", &dq::fwht_levels_);
  m.def("superchunk_widths(Tensor stats, Tensor state, Tensor(a!) s_out, Tensor(b!) widths) -> ()", &dq::superchunk_widths);
  m.def("superchunk_plan(Tensor widths) -> Tensor", &dq::superchunk_plan);
  m.def("superchunk_bitrate_update(Tensor sorted_s, Tensor(a!) state, float target) -> ()", &dq::superchunk_bitrate_update);
  m.def("rht_widths_update(Tensor mailbox, Tensor(a!) plan, int nblocks, int blocks_per_shard, int slot_stride, "
        "int scales_off, int first_ag_slot, int budget) -> ()", &dq::rht_widths_update);
  m.def("nvls_allreduce(Tensor(a!) bucket, int stage_ptr, int mc_ptr, int[] flag_ptrs, int stage_bytes, int status_ptr, "
        "int rank, int world, int wire_bits, int epoch, float post_scale, int timeout_ns, int ctas) -> ()",
        &dq::nvls_allreduce);
  m.def("thc_quantize_(Tensor(a!) y, Tensor stats, int world, float t_over_sqrt_d, int levels, int stream, int step, "
        "int seed) -> ()", &dq::thc_quantize_);
  m.def("thc_dequantize_(Tensor(a!) total, Tensor stats, int world, float t_over_sqrt_d, int levels) -> ()",
        &dq::thc_dequantize_);
  m.def("rope(Tensor x, Tensor cos, Tensor sin, bool backward) -> Tensor", &dq::rope);
  m.def("adamw_step(Tensor table, Tensor numel, Tensor chunk_start, int total_chunks, bool param_bf16, bool grad_bf16, "
        "float lr, float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale) -> ()", &dq::adamw_step);
  m.def("topology() -> Tensor", &dq::topology);
  m.def("symm_alloc(int device, int bytes) -> (int, Tensor)", &dq::symm_alloc);
  m.def("symm_open(int device, Tensor handle) -> int", &dq::symm_open);
  m.def("symm_close(int ptr) -> ()", &dq::symm_close);
  m.def("symm_free(int ptr) -> ()", &dq::symm_free);
  m.def("wrap_ptr(int ptr, int bytes, int device) -> Tensor", &dq::wrap_ptr);
  m.def("set_debug(bool on) -> ()", &dq::set_debug);
  m.def(
      "fused_allreduce(Tensor(a!) bucket, Tensor steps, int[] mail_ptrs, int[] flag_ptrs, int mailbox_bytes, "
      "int flag_words, int nslots, int status_ptr, int tail_ws_ptr, int rank, int world, int bits, int ctas, "
      "int threads, int blocks_per_shard, int slot_stride, int scales_off, int flag_base, int epoch, int seed, "
      "int step, int bucket_id, float post_scale, int timeout_ns, bool no_transmit, int codec, float sc_lattice_max, float sc_c1, float sc_c2, Tensor? sc_lut, Tensor? sc_plan=None, bool prefetch=True) -> ()",
      &dq::fused_allreduce);
  m.def(
      "fused_allreduce_local(Tensor[] buckets, Tensor steps, Tensor[] mailboxes, Tensor[] flags, Tensor status, "
      "Tensor tail_ws, int nslots, int bits, int ctas, int threads, int blocks_per_shard, int slot_stride, "
      "int scales_off, int flag_base, int epoch, int seed, int step, int bucket_id, float post_scale, "
      "int timeout_ns, bool no_transmit, int codec, float sc_lattice_max, float sc_c1, float sc_c2, Tensor? sc_lut, Tensor? sc_plan=None, bool prefetch=True) -> ()",
      &dq::fused_allreduce_local);
}
