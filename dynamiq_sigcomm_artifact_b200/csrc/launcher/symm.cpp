// NVLink transport bring-up: topology discovery and peer-mapped ("symmetric") buffers.
//
// Stands where the reference has its RDMA connection set-up (rdma_cm listen/connect, pinned
// host rings registered as memory regions, a RemoteInfo handshake;
// rdma_comm_compress/ring_allreduce_ext/ring_allreduce_backend.cu:436-528,861-887) and its
// NVLink pair check through `nvidia-smi topo -m`
// (testbed_evaluation/new_comm_hooks/ring_rdma.py:386-494).  On one NVSwitch box the
// "connection" is a device allocation whose IPC handle every other rank opens; after that the
// collective kernels address peers by pointer.  Handles travel through torch.distributed
// (see parallel/symm.py), so this file needs no sockets.
#include <c10/cuda/CUDAException.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace dq {

namespace {
std::mutex g_mu;
std::unordered_map<int64_t, int> g_owned;   // pointer -> device, allocations made here
std::unordered_map<int64_t, int> g_opened;  // pointer -> device, peer mappings opened here
}  // namespace

// [ndev, ndev, 3] int32: (can access peer, performance rank, native atomics) for every ordered pair.
at::Tensor topology() {
  int n = 0;
  C10_CUDA_CHECK(cudaGetDeviceCount(&n));
  at::Tensor t = at::zeros({n, n, 3}, at::kInt);
  auto a = t.accessor<int, 3>();
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      if (i == j) {
        a[i][j][0] = 1;
        continue;
      }
      int v = 0;
      if (cudaDeviceCanAccessPeer(&v, i, j) != cudaSuccess) {
        cudaGetLastError();
        v = 0;
      }
      a[i][j][0] = v;
      if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrPerformanceRank, i, j) == cudaSuccess) a[i][j][1] = v;
      else cudaGetLastError();
      if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrNativeAtomicSupported, i, j) == cudaSuccess) a[i][j][2] = v;
      else cudaGetLastError();
    }
  return t;
}

// Allocate `bytes` of zeroed device memory outside the caching allocator (IPC needs a whole
// allocation) and return (address, 64-byte IPC handle).
std::tuple<int64_t, at::Tensor> symm_alloc(int64_t device, int64_t bytes) {
  TORCH_CHECK(bytes > 0, "symm_alloc: bytes must be positive");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  void* p = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  C10_CUDA_CHECK(cudaMemset(p, 0, static_cast<size_t>(bytes)));
  C10_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    TORCH_CHECK(false, "cudaIpcGetMemHandle failed: ", cudaGetErrorString(e));
  }
  at::Tensor handle = at::empty({static_cast<int64_t>(sizeof(h))}, at::kByte);
  std::memcpy(handle.data_ptr(), &h, sizeof(h));
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_owned[reinterpret_cast<int64_t>(p)] = static_cast<int>(device);
  }
  return {reinterpret_cast<int64_t>(p), handle};
}

// Map a peer's allocation into this process (enables peer access on first use).
int64_t symm_open(int64_t device, at::Tensor handle) {
  TORCH_CHECK(handle.device().is_cpu() && handle.scalar_type() == at::kByte &&
                  handle.numel() == static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)) && handle.is_contiguous(),
              "symm_open: handle must be a 64-byte CPU uint8 tensor");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    TORCH_CHECK(false, "cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e));
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_opened[reinterpret_cast<int64_t>(p)] = static_cast<int>(device);
  return reinterpret_cast<int64_t>(p);
}

void symm_close(int64_t ptr) {
  int dev = -1;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_opened.find(ptr);
    if (it == g_opened.end()) return;
    dev = it->second;
    g_opened.erase(it);
  }
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(dev));
  cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
  cudaGetLastError();
}

void symm_free(int64_t ptr) {
  int dev = -1;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_owned.find(ptr);
    if (it == g_owned.end()) return;
    dev = it->second;
    g_owned.erase(it);
  }
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(dev));
  cudaFree(reinterpret_cast<void*>(ptr));
  cudaGetLastError();
}

// View `bytes` at a raw device address as a uint8 tensor (no ownership).
at::Tensor wrap_ptr(int64_t ptr, int64_t bytes, int64_t device) {
  return at::from_blob(reinterpret_cast<void*>(ptr), {bytes},
                       at::TensorOptions().dtype(at::kByte).device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
}

}  // namespace dq
