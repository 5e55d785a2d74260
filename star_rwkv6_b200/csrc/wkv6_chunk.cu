// Chunked tensor-core variant: placeholder until the tcgen05 kernels land.
#include "wkv6_internal.h"

namespace wkv6 {
bool chunk_supported(const wkv6_problem *) { return false; }
size_t chunk_ckpt_bytes(const wkv6_problem *) { return 0; }
size_t chunk_backward_workspace(const wkv6_problem *, const Dims &, int) { return 0; }
int chunk_forward(const wkv6_problem *, const Dims &, const void *, const void *, const void *, const void *,
                  const void *, void *, const void *, const int64_t *, int, void *, void *, cudaStream_t) {
    return fail(WKV6_ERR_UNSUPPORTED, "chunked variant not built");
}
int chunk_backward(const wkv6_problem *, const Dims &, const void *, const void *, const void *, const void *,
                   const void *, const void *, void *, void *, void *, void *, void *, const void *, void *, size_t,
                   cudaStream_t) {
    return fail(WKV6_ERR_UNSUPPORTED, "chunked variant not built");
}
}  // namespace wkv6
