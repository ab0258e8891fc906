/* Allocation-free C entry point of the native library (dq_native.so).
 *
 * This entry point has no counterpart in the reference implementation.
 *
 * Who it is for: code that must not (or cannot) allocate device memory at the moment it needs
 * the RMSNorm backward pass - a host without the PyTorch caching allocator (a plain C/C++ or
 * ctypes caller), a caller running under a fixed memory budget that was carved up in advance,
 * or a real-time loop where a cudaMalloc (which synchronises the device) is not acceptable.
 * The regular operator (torch.ops.dq.norm_bwd) asks the allocator for its per-warp partial-sum
 * scratch on every call; this variant keeps that scratch in a fixed array inside the library.
 *
 * The scratch is a file-scope device array of DQ_NOALLOC_MAX_PARTS x DQ_NOALLOC_MAX_HIDDEN
 * floats (4 MiB).  Every GPU on which the library is loaded holds it until the process exits.
 * All calls share it and it keeps the previous call's contents; the kernel overwrites every
 * word it later reads, so nothing needs clearing, but two calls that overlap on the GPU
 * (different streams, or different host threads) race on it: serialise them.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 * caches it; make that first call outside of any stream capture.
 */
#ifndef DQ_NOALLOC_H_
#define DQ_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define DQ_NOALLOC_MAX_HIDDEN 2048 /* largest hidden size (elements per row) */
#define DQ_NOALLOC_MAX_PARTS 512   /* partial-sum rows held in the scratch array */

enum {
  DQ_NOALLOC_OK = 0,
  DQ_NOALLOC_BAD_HIDDEN = -1,  /* hidden > DQ_NOALLOC_MAX_HIDDEN, or not a multiple of 8, or <= 0 */
  DQ_NOALLOC_BAD_ROWS = -2,    /* rows <= 0 */
  DQ_NOALLOC_BAD_POINTER = -3, /* null or not 16-byte aligned */
  DQ_NOALLOC_CUDA_ERROR = -4   /* a CUDA call failed; see dq_noalloc_last_cuda_error() */
};

/* RMSNorm backward.  dy, x, dx: [rows, hidden] row-major, bf16 (is_bf16 != 0) or fp32;
 * w, dw: [hidden] fp32; rstd: [rows] fp32 as saved by the forward pass.  Writes dx and dw.
 * Launches on `stream` (a cudaStream_t passed as void*; NULL is the default stream) of the
 * current device and returns without synchronising.  Calls no cudaMalloc / cudaFree and no
 * allocating library routine. */
int dq_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* dw,
                           int rows, int hidden, int is_bf16, void* stream);

/* Text for a return code of dq_rmsnorm_bwd_noalloc. */
const char* dq_noalloc_strerror(int code);

/* The cudaError_t (as int) behind the last DQ_NOALLOC_CUDA_ERROR of the calling thread. */
int dq_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* DQ_NOALLOC_H_ */
