// 2-bit superchunk (AEE / MEE) instantiation of the persistent compressed all-reduce kernel.
#include "fused_allreduce_impl.cuh"
namespace dq {
DQ_INSTANTIATE_FUSED_ALLREDUCE_SC(2)
}  // namespace dq
