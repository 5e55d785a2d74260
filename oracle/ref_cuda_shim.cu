// C entry points around the reference's own XLA custom-call handlers, so that the unmodified reference kernels can
// be timed and checked beside this library.  Test / benchmark infrastructure only: compiled by
// oracle/build_ref_cuda.py together with the reference's rwkv_kernel/jax_kernel/rwkv_kernels.cu, taken from where it
// lies in the reference tree (never copied), into oracle/_ref/.  The handler prototypes are those of the reference's
// kernels.h:44-53; the buffer orders are in rwkv_kernels.cu:451-508.
#include <cuda_runtime_api.h>

#include <cstddef>

namespace gpu_ops {
void rwkv_forward_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len);
void rwkv_backward_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len);
}  // namespace gpu_ops

extern "C" {
__attribute__((visibility("default"))) void ref_wkv6_forward(void *stream, void **buffers, const char *opaque, size_t len) {
    gpu_ops::rwkv_forward_fn(static_cast<cudaStream_t>(stream), buffers, opaque, len);
}
__attribute__((visibility("default"))) void ref_wkv6_backward(void *stream, void **buffers, const char *opaque, size_t len) {
    gpu_ops::rwkv_backward_fn(static_cast<cudaStream_t>(stream), buffers, opaque, len);
}
__attribute__((visibility("default"))) int ref_wkv6_last_cuda_error(void) { return (int)cudaGetLastError(); }
}
