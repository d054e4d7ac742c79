// Peer-visible buffers for the fused GEMM + gather (one node, one process per GPU).
//
// A buffer that other processes' GPUs will store into is allocated with cudaMalloc (so that the
// pointer is the base of its allocation) and exported as a CUDA IPC handle.  A peer process opens the
// handle WITH ITS OWN DEVICE CURRENT and cudaIpcMemLazyEnablePeerAccess: that is what maps the memory
// into the address space of the context whose kernels will touch it (opening it under the exporting
// device's context, as tensor-sharing between processes does, leaves kernels of the importing GPU
// without a valid mapping).  The reference project has no multi-GPU code; nothing here replaces any
// of its interfaces.
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/peakgemm.h"

namespace {
thread_local int t_peer_cuda_error = 0;
int fail(cudaError_t e) {
    t_peer_cuda_error = static_cast<int>(e);
    cudaGetLastError();
    return PG_ERR_CUDA;
}
static_assert(sizeof(cudaIpcMemHandle_t) == PG_PEER_HANDLE_BYTES, "IPC handle size");
}  // namespace

extern "C" {

int pg_peer_last_cuda_error(void) { return t_peer_cuda_error; }

int pg_peer_alloc(size_t bytes, void **ptr, void *handle_out) {
    if (!ptr || !handle_out || bytes == 0) return PG_ERR_BAD_ARG;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return fail(e);
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(e);
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr = p;
    return PG_OK;
}

int pg_peer_open(const void *handle, void **ptr) {
    if (!ptr || !handle) return PG_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(e);
    *ptr = p;
    return PG_OK;
}

int pg_peer_close(void *ptr) {
    if (!ptr) return PG_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? PG_OK : fail(e);
}

int pg_peer_free(void *ptr) {
    if (!ptr) return PG_OK;
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? PG_OK : fail(e);
}

}  // extern "C"
