/* Status strings and the buffer helpers of the C ABI.
 *
 * Contract (include/s2pro/status.h:23, include/s2pro/tensor.h:23-43 of the reference): an
 * s2p_tensor describes up to four dimensions of one element type and owns either device memory
 * or pinned host memory; a freed or never-allocated descriptor is all zero.  Host buffers are
 * pinned so that copies on a stream are asynchronous (the reference's choice too,
 * src/core/tensor.c:60-127).
 */
#include <string.h>
#include "s2p_b200_abi.h"

/* ---- status --------------------------------------------------------------------------- */

const char* s2p_status_str(s2p_status s) {
    switch (s) {
    case S2P_OK: return "ok";
    case S2P_ERR_INVALID: return "invalid argument";
    case S2P_ERR_CUDA: return "cuda error";
    case S2P_ERR_IO: return "i/o error";
    case S2P_ERR_OOM: return "out of memory";
    case S2P_ERR_FORMAT: return "format/parse error";
    case S2P_ERR_STATE: return "invalid state";
    case S2P_ERR_UNSUPPORTED: return "unsupported";
    case S2P_ERR_INTERNAL: return "internal invariant violated";
    case S2P_ERR_FULL: return "capacity exhausted";
    }
    return "unknown status";
}

/* ---- element types ---------------------------------------------------------------------- */

size_t s2p_dtype_size(s2p_dtype dt) {
    switch (dt) {
    case S2P_DT_BF16: case S2P_DT_F16: return 2;
    case S2P_DT_F32: case S2P_DT_I32: return 4;
    case S2P_DT_I64: return 8;
    case S2P_DT_I8: case S2P_DT_U8: return 1;
    }
    return 0;
}

int64_t s2p_tensor_numel(const s2p_tensor* t) {
    if (!t || t->ndim < 0 || t->ndim > 4) return 0;
    int64_t n = 1;
    for (int d = 0; d < t->ndim; d++) n *= t->shape[d];
    return n;
}

/* ---- allocation --------------------------------------------------------------------------
 * Both kinds of buffer go through one routine: the byte count is formed with checked
 * multiplications (a shape that overflows is an invalid argument, not a small allocation), the
 * memory is obtained, and only then is the caller's descriptor written - so a failed call
 * leaves whatever the caller had there untouched except for the documented zeroing. */

static int shape_bytes(s2p_dtype dt, int ndim, const int64_t* shape, size_t* bytes_out) {
    size_t bytes = s2p_dtype_size(dt);
    if (!bytes || !shape || ndim < 1 || ndim > 4) return 0;
    for (int d = 0; d < ndim; d++) {
        if (shape[d] <= 0) return 0;
        if (__builtin_mul_overflow(bytes, (size_t)shape[d], &bytes)) return 0;
    }
    if (bytes > (size_t)INT64_MAX) return 0; /* the element count must fit the signed count the ABI reports */
    *bytes_out = bytes;
    return 1;
}

static s2p_status tensor_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape, int on_device) {
    size_t bytes = 0;
    if (!t || !shape_bytes(dt, ndim, shape, &bytes)) return S2P_ERR_INVALID;
    void* mem = NULL;
    const cudaError_t e = on_device ? cudaMalloc(&mem, bytes) : cudaMallocHost(&mem, bytes);
    memset(t, 0, sizeof(*t));
    if (e != cudaSuccess) {
        fprintf(stderr, "[s2pro] %s(%zu) failed: %s\n", on_device ? "cudaMalloc" : "cudaMallocHost", bytes, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? S2P_ERR_OOM : S2P_ERR_CUDA;
    }
    t->data = mem;
    t->dtype = dt;
    t->ndim = ndim;
    t->bytes = bytes;
    t->on_device = on_device;
    for (int d = 0; d < 4; d++) t->shape[d] = d < ndim ? shape[d] : 1;
    return S2P_OK;
}

s2p_status s2p_tensor_device_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape) {
    return tensor_alloc(t, dt, ndim, shape, 1);
}
s2p_status s2p_tensor_host_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape) {
    return tensor_alloc(t, dt, ndim, shape, 0);
}

void s2p_tensor_free(s2p_tensor* t) {
    if (!t) return;
    void* mem = t->data;
    const int on_device = t->on_device;
    memset(t, 0, sizeof(*t));
    if (!mem) return;
    const cudaError_t e = on_device ? cudaFree(mem) : cudaFreeHost(mem);
    if (e != cudaSuccess) fprintf(stderr, "[s2pro] tensor free failed: %s\n", cudaGetErrorString(e));
}

/* ---- copies: a device tensor on one side, caller memory on the other, in stream order ------ */

static s2p_status device_copy(const s2p_tensor* dev, void* dev_ptr_side, const void* other, size_t bytes, int to_device,
                              cudaStream_t stream) {
    if (!dev || !dev->data || !dev->on_device || bytes > dev->bytes) return S2P_ERR_INVALID;
    if (!bytes) return S2P_OK;
    if (!other) return S2P_ERR_INVALID;
    if (to_device) S2P_CUDA_TRY(cudaMemcpyAsync(dev->data, other, bytes, cudaMemcpyHostToDevice, stream));
    else S2P_CUDA_TRY(cudaMemcpyAsync(dev_ptr_side, dev->data, bytes, cudaMemcpyDeviceToHost, stream));
    return S2P_OK;
}

s2p_status s2p_tensor_upload(s2p_tensor* dst, const void* src, size_t bytes, cudaStream_t stream) {
    return device_copy(dst, NULL, src, bytes, 1, stream);
}
s2p_status s2p_tensor_download(void* dst, const s2p_tensor* src, size_t bytes, cudaStream_t stream) {
    return device_copy(src, dst, dst, bytes, 0, stream);
}
