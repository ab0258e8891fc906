// Identity-wire (bf16 / fp32) instantiations of the persistent all-reduce kernel: the custom
// point-to-point all-reduce of uncompressed gradients.
#include "fused_allreduce_impl.cuh"
namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE_CAST(16)
DQ_INSTANTIATE_FUSED_ALLREDUCE_CAST(32)
}  // namespace dq
