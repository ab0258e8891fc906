// Block-float (MXFP8 / FP6 / FP4) instantiations of the persistent compressed all-reduce kernel.
#include "fused_allreduce_impl.cuh"
namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE_MX(8)
DQ_INSTANTIATE_FUSED_ALLREDUCE_MX(6)
DQ_INSTANTIATE_FUSED_ALLREDUCE_MX(4)
}  // namespace dq
