/* Status strings and the device/pinned buffer helpers of the C ABI
 * (reference contracts: include/s2pro/status.h:23, include/s2pro/tensor.h:23-43;
 * reference behaviour: src/core/tensor.c:60-127 — host buffers are pinned so
 * stream copies are asynchronous, device buffers are plain cudaMalloc). */
#include <string.h>
#include "s2p_b200_abi.h"

const char* s2p_status_str(s2p_status s) {
    static const char* const names[] = {
        "ok", "invalid argument", "cuda error", "i/o error", "out of memory",
        "format/parse error", "invalid state", "unsupported",
        "internal invariant violated", "capacity exhausted"};
    const int i = -(int)s;
    return (i >= 0 && i < 10) ? names[i] : "unknown status";
}

size_t s2p_dtype_size(s2p_dtype dt) {
    static const unsigned char sz[] = {2, 4, 2, 1, 4, 8, 1};
    return ((unsigned)dt < sizeof(sz)) ? sz[dt] : 0;
}

int64_t s2p_tensor_numel(const s2p_tensor* t) {
    if (!t || t->ndim < 0 || t->ndim > 4) return 0;
    int64_t n = 1;
    for (int i = 0; i < t->ndim; i++) n *= t->shape[i];
    return n;
}

static s2p_status describe(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape) {
    if (!t || !shape || ndim < 1 || ndim > 4) return S2P_ERR_INVALID;
    const size_t esz = s2p_dtype_size(dt);
    if (!esz) return S2P_ERR_INVALID;
    int64_t numel = 1;
    for (int i = 0; i < ndim; i++) {
        if (shape[i] <= 0 || numel > INT64_MAX / shape[i]) return S2P_ERR_INVALID;
        numel *= shape[i];
    }
    if ((uint64_t)numel > SIZE_MAX / esz) return S2P_ERR_INVALID;
    memset(t, 0, sizeof(*t));
    t->dtype = dt;
    t->ndim = ndim;
    for (int i = 0; i < 4; i++) t->shape[i] = i < ndim ? shape[i] : 1;
    t->bytes = (size_t)numel * esz;
    return S2P_OK;
}

static s2p_status alloc_common(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape, int dev) {
    S2P_TRY(describe(t, dt, ndim, shape));
    const cudaError_t e = dev ? cudaMalloc(&t->data, t->bytes) : cudaMallocHost(&t->data, t->bytes);
    if (e != cudaSuccess) {
        fprintf(stderr, "[s2pro] %s(%zu) failed: %s\n", dev ? "cudaMalloc" : "cudaMallocHost", t->bytes,
                cudaGetErrorString(e));
        t->data = NULL;
        return e == cudaErrorMemoryAllocation ? S2P_ERR_OOM : S2P_ERR_CUDA;
    }
    t->on_device = dev;
    return S2P_OK;
}

s2p_status s2p_tensor_device_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape) {
    return alloc_common(t, dt, ndim, shape, 1);
}
s2p_status s2p_tensor_host_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape) {
    return alloc_common(t, dt, ndim, shape, 0);
}

s2p_status s2p_tensor_upload(s2p_tensor* dst, const void* src, size_t bytes, cudaStream_t stream) {
    if (!dst || !dst->data || !dst->on_device || bytes > dst->bytes || (!src && bytes)) return S2P_ERR_INVALID;
    if (bytes) S2P_CUDA_TRY(cudaMemcpyAsync(dst->data, src, bytes, cudaMemcpyHostToDevice, stream));
    return S2P_OK;
}
s2p_status s2p_tensor_download(void* dst, const s2p_tensor* src, size_t bytes, cudaStream_t stream) {
    if (!src || !src->data || !src->on_device || bytes > src->bytes || (!dst && bytes)) return S2P_ERR_INVALID;
    if (bytes) S2P_CUDA_TRY(cudaMemcpyAsync(dst, src->data, bytes, cudaMemcpyDeviceToHost, stream));
    return S2P_OK;
}

void s2p_tensor_free(s2p_tensor* t) {
    if (!t) return;
    if (t->data) {
        const cudaError_t e = t->on_device ? cudaFree(t->data) : cudaFreeHost(t->data);
        if (e != cudaSuccess) fprintf(stderr, "[s2pro] tensor free failed: %s\n", cudaGetErrorString(e));
    }
    memset(t, 0, sizeof(*t));
}
