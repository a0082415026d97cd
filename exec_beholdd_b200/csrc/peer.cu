// Peer-visible device buffers for the multi-GPU paths (one process per GPU, all GPUs of one
// node behind NVSwitch): a buffer is allocated by its owner, exported as an opaque 64-byte
// handle, and opened by the other ranks' processes, which then read and write it with ordinary
// loads and stores over NVLink. The handles travel between the processes however the host
// likes (the Python host uses its process group's all-gather).
//
// The reference is single-process and has no counterpart.
#include "common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle crosses the C ABI as 64 opaque bytes");

static bool ctx_ok(const bhd_ctx* c) { return c && c->magic == BHD_CTX_MAGIC; }

extern "C" int32_t bhd_peer_alloc(bhd_ctx* ctx, uint64_t n_bytes, void** out_dev, uint8_t* handle64) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!out_dev || !handle64 || n_bytes == 0) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "peer_alloc: null output or empty buffer");
    *out_dev = nullptr;
    bhd_device_guard guard(ctx);
    void* p = nullptr;
    if (cudaMalloc(&p, n_bytes) != cudaSuccess) {
        cudaGetLastError();
        return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %llu bytes for %s", bhd_device_name(),
                        (unsigned long long)n_bytes, "a peer-visible buffer");
    }
    BHD_CUDA(ctx, cudaMemset(p, 0, n_bytes), "clearing a peer-visible buffer");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return bhd_cuda_fail(ctx, e, "exporting a peer-visible buffer");
    }
    memcpy(handle64, &h, 64);
    *out_dev = p;
    return BHD_OK;
}

extern "C" int32_t bhd_peer_open(bhd_ctx* ctx, const uint8_t* handle64, void** out_dev) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!out_dev || !handle64) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "peer_open: null argument");
    *out_dev = nullptr;
    bhd_device_guard guard(ctx);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    BHD_CUDA(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "opening a peer's buffer");
    *out_dev = p;
    return BHD_OK;
}

extern "C" int32_t bhd_peer_close(bhd_ctx* ctx, void* dev) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!dev) return BHD_OK;
    bhd_device_guard guard(ctx);
    BHD_CUDA(ctx, cudaDeviceSynchronize(), "synchronising before closing a peer's buffer");
    BHD_CUDA(ctx, cudaIpcCloseMemHandle(dev), "closing a peer's buffer");
    return BHD_OK;
}

extern "C" int32_t bhd_peer_free(bhd_ctx* ctx, void* dev) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!dev) return BHD_OK;
    bhd_device_guard guard(ctx);
    BHD_CUDA(ctx, cudaDeviceSynchronize(), "synchronising before freeing a peer-visible buffer");
    BHD_CUDA(ctx, cudaFree(dev), "freeing a peer-visible buffer");
    return BHD_OK;
}
