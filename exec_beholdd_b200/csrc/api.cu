// C ABI of the library: contexts, resident weights, validation and dispatch.
//
// Validation mirrors the reference CPU device (crates/beholdd-backend/src/cpu.rs:55-97,
// 415-452): shapes and the exact packed byte count are checked before anything touches an
// output, and a refused call leaves its outputs unmodified.
#include <cuda.h>
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>

#include <new>

#include "common.cuh"

int32_t bhd_launch_matvec_fast(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                               uint64_t batch, float scale, int accumulate, cudaStream_t s, bool* handled);
void bhd_weight_build_tensor_map(bhd_ctx* ctx, bhd_weight* w);
void bhd_weight_build_tensor_map16(bhd_ctx* ctx, bhd_weight* w);
int32_t bhd_launch_gemm_q8_tcgen05(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y, uint64_t m,
                                   cudaStream_t s, bool* handled);
int32_t bhd_launch_matvec_decode(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                 uint32_t batch, float scale, int accumulate, cudaStream_t s, bool* handled);
int32_t bhd_launch_matvec_decode_i8(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                    uint32_t batch, float scale, int accumulate, cudaStream_t s, bool* handled);
int32_t bhd_launch_stage_copy(bhd_ctx* ctx, const float* src_mapped, float* dst_dev, size_t n16, cudaStream_t s);

int32_t bhd_fail(bhd_ctx* ctx, int32_t status, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return status;
}

int32_t bhd_cuda_fail(bhd_ctx* ctx, cudaError_t e, const char* what) {
    const int32_t st = (e == cudaErrorMemoryAllocation) ? BHD_ERR_ALLOCATION : BHD_ERR_BACKEND;
    return bhd_fail(ctx, st, "%s backend error: %s: %s", bhd_device_name(), what, cudaGetErrorString(e));
}

const char* bhd_kind_name(uint32_t kind) {
    switch (kind) {
        case BHD_TYPE_F32: return "F32";
        case BHD_TYPE_F16: return "F16";
        case BHD_TYPE_Q8_0: return "Q8_0";
        case BHD_TYPE_Q4_K: return "Q4_K";
        case BHD_TYPE_Q5_K: return "Q5_K";
        case BHD_TYPE_Q6_K: return "Q6_K";
        case BHD_TYPE_BF16: return "BF16";
        default: return "unknown";
    }
}

// crates/beholdd-core/src/quant.rs:79-118 restricted to the formats this library decodes.
bool bhd_block_geometry(uint32_t kind, uint64_t* elems, uint64_t* bytes) {
    switch (kind) {
        case BHD_TYPE_F32: *elems = 1; *bytes = 4; return true;
        case BHD_TYPE_F16: *elems = 1; *bytes = 2; return true;
        case BHD_TYPE_Q8_0: *elems = 32; *bytes = 34; return true;
        case BHD_TYPE_Q4_K: *elems = 256; *bytes = 144; return true;
        case BHD_TYPE_Q5_K: *elems = 256; *bytes = 176; return true;
        case BHD_TYPE_Q6_K: *elems = 256; *bytes = 210; return true;
        case BHD_TYPE_BF16: *elems = 1; *bytes = 2; return true;
        default: return false;
    }
}

int32_t bhd_ensure_workspace(bhd_ctx* ctx, size_t bytes, cudaStream_t stream) {
    if (bytes <= ctx->workspace_bytes) return BHD_OK;
    // Growing is rare (first call of a new size). Earlier work may still use the old block.
    BHD_CUDA(ctx, cudaDeviceSynchronize(), "synchronising before growing the workspace");
    if (ctx->workspace) cudaFree(ctx->workspace);
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    const size_t want = (bytes + (bytes >> 2) + 0xFFFFF) & ~size_t(0xFFFFF);
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %zu bytes for %s", bhd_device_name(), want,
                        "kernel workspace");
    }
    (void)stream;
    ctx->workspace = static_cast<uint8_t*>(p);
    ctx->workspace_bytes = want;
    return BHD_OK;
}

static bool valid_ctx(const bhd_ctx* c) { return c && c->magic == BHD_CTX_MAGIC; }
static bool valid_w(const bhd_ctx* c, const bhd_weight* w) { return w && w->magic == BHD_WEIGHT_MAGIC && w->ctx == c; }

extern "C" {

const char* bhd_error_text(int32_t status) {
    switch (status) {
        case BHD_OK: return "ok";
        case BHD_ERR_UNSUPPORTED_FORMAT: return "the device has no decoder for this weight format";
        case BHD_ERR_SHAPE: return "shape mismatch";
        case BHD_ERR_ALLOCATION: return "device storage could not be reserved";
        case BHD_ERR_BACKEND: return "a CUDA call failed";
        case BHD_ERR_INVALID_ARGUMENT: return "invalid argument or foreign handle";
        case BHD_ERR_DEVICE_STATUS: return "a kernel reported a problem through the device status word";
        default: return "unknown status";
    }
}

int32_t bhd_last_error_message(const bhd_ctx* ctx, char* buffer, int32_t capacity) {
    if (!valid_ctx(ctx)) return 0;
    const int32_t len = int32_t(strlen(ctx->err));
    if (buffer && capacity > 0) {
        const int32_t n = len < capacity - 1 ? len : capacity - 1;
        memcpy(buffer, ctx->err, size_t(n));
        buffer[n] = 0;
    }
    return len;
}

const char* bhd_device_name(void) { return "cuda-b200"; }

int32_t bhd_supports(uint32_t ggml_type) {
    uint64_t e, b;
    return bhd_block_geometry(ggml_type, &e, &b) ? 1 : 0;
}

int32_t bhd_ctx_create(int32_t device, bhd_ctx** out_ctx) {
    if (!out_ctx) return BHD_ERR_INVALID_ARGUMENT;
    *out_ctx = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count || device >= BHD_MAX_DEVICES) {
        cudaGetLastError();
        return BHD_ERR_BACKEND;
    }
    bhd_ctx* c = new (std::nothrow) bhd_ctx();
    if (!c) return BHD_ERR_ALLOCATION;
    memset(c, 0, sizeof(*c));
    c->magic = BHD_CTX_MAGIC;
    c->device = device;
    bhd_device_guard guard(c);  // the caller's current device is put back when this call returns
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return BHD_ERR_BACKEND; }
    c->sm_count = prop.multiProcessorCount;
    if (prop.major != 10) {
        // Built for sm_100a only; there is no other code path to fall back to.
        delete c;
        return BHD_ERR_BACKEND;
    }
    if (cudaMalloc(reinterpret_cast<void**>(&c->status_dev), 256) != cudaSuccess ||
        cudaMemset(c->status_dev, 0, 256) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void**>(&c->status_host), 256) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&c->counters), 65536 * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(c->counters, 0, 65536 * sizeof(uint32_t)) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return BHD_ERR_ALLOCATION;
    }
    // streams and events of the routed experts' side-by-side size classes: made now, not on first use, which may be
    // inside a stream capture
    bool side_ok = cudaEventCreateWithFlags(&c->fork_event, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 3 && side_ok; ++i)
        side_ok = cudaStreamCreateWithFlags(&c->side_stream[i], cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&c->join_event[i], cudaEventDisableTiming) == cudaSuccess;
    if (!side_ok) {
        cudaGetLastError();
        bhd_ctx_destroy(c);
        return BHD_ERR_ALLOCATION;
    }
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
        c->tmap_encode = fn;
    else
        cudaGetLastError();
    *out_ctx = c;
    return BHD_OK;
}

int32_t bhd_ctx_destroy(bhd_ctx* ctx) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    {
    bhd_device_guard guard(ctx);
    cudaDeviceSynchronize();
    if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
    for (int i = 0; i < 3; ++i) {
        if (ctx->side_stream[i]) cudaStreamDestroy(ctx->side_stream[i]);
        if (ctx->join_event[i]) cudaEventDestroy(ctx->join_event[i]);
    }
    if (ctx->fork_event) cudaEventDestroy(ctx->fork_event);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->stage_x) cudaFree(ctx->stage_x);
    if (ctx->stage_y) cudaFree(ctx->stage_y);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    }
    ctx->magic = 0;
    delete ctx;
    return BHD_OK;
}

// Exact storage validation, crates/beholdd-backend/src/cpu.rs:55-97.
static int32_t validate_storage(bhd_ctx* ctx, uint64_t n_bytes, uint32_t kind, uint64_t rows, uint64_t cols,
                                uint64_t slabs, uint64_t* row_bytes_out) {
    uint64_t n;
    if (__builtin_mul_overflow(rows, cols, &n))
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: weight element count overflows for %llux%llu",
                        (unsigned long long)rows, (unsigned long long)cols);
    uint64_t be, bb;
    if (!bhd_block_geometry(kind, &be, &bb))
        return bhd_fail(ctx, BHD_ERR_UNSUPPORTED_FORMAT, "%s cannot decode ggml type %u (weight %llux%llu)",
                        bhd_device_name(), kind, (unsigned long long)rows, (unsigned long long)cols);
    if (cols % be != 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE,
                        "shape mismatch: %llux%llu %s weight has %llu elements per row, not a whole number of "
                        "%llu-element blocks",
                        (unsigned long long)rows, (unsigned long long)cols, bhd_kind_name(kind),
                        (unsigned long long)cols, (unsigned long long)be);
    const uint64_t bpr = cols / be;
    uint64_t row_bytes, slab_bytes, expect;
    if (__builtin_mul_overflow(bpr, bb, &row_bytes) || __builtin_mul_overflow(rows, row_bytes, &slab_bytes) ||
        __builtin_mul_overflow(slab_bytes, slabs, &expect))
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: weight byte count overflows for %llux%llu %s",
                        (unsigned long long)rows, (unsigned long long)cols, bhd_kind_name(kind));
    if (n_bytes != expect)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: %llux%llu %s weight needs %llu bytes, got %llu",
                        (unsigned long long)rows, (unsigned long long)cols, bhd_kind_name(kind),
                        (unsigned long long)expect, (unsigned long long)n_bytes);
    *row_bytes_out = row_bytes;
    return BHD_OK;
}

static int32_t make_weight(bhd_ctx* ctx, const void* src, bool src_is_device, uint64_t n_bytes, uint32_t kind,
                           uint64_t rows, uint64_t cols, uint64_t slabs, bhd_weight** out) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!out) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "weight upload: null output handle");
    *out = nullptr;
    if (slabs == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: a weight needs at least one slab");
    uint64_t row_bytes = 0;
    const int32_t st = validate_storage(ctx, n_bytes, kind, rows, cols, slabs, &row_bytes);
    if (st != BHD_OK) return st;
    if (n_bytes > 0 && !src) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "weight upload: null bytes");
    bhd_device_guard guard(ctx);
    bhd_weight* w = new (std::nothrow) bhd_weight();
    if (!w) return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate host memory for a weight handle", bhd_device_name());
    memset(w, 0, sizeof(*w));
    w->magic = BHD_WEIGHT_MAGIC;
    w->ctx = ctx;
    w->device = ctx->device;
    w->kind = kind;
    w->rows = rows;
    w->cols = cols;
    w->slabs = slabs;
    w->row_bytes = row_bytes;
    w->slab_bytes = rows * row_bytes;
    if (src_is_device) {
        if (reinterpret_cast<uintptr_t>(src) % 16 != 0) {
            delete w;
            return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "weight wrap: device bytes must be 16-byte aligned");
        }
        w->dev = const_cast<uint8_t*>(static_cast<const uint8_t*>(src));
        w->owned = false;
    } else {
        void* p = nullptr;
        const cudaError_t e = cudaMalloc(&p, n_bytes ? n_bytes : 16);
        if (e != cudaSuccess) {
            cudaGetLastError();
            delete w;
            return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %llu bytes for %s", bhd_device_name(),
                            (unsigned long long)n_bytes, "resident weight");
        }
        w->dev = static_cast<uint8_t*>(p);
        w->owned = true;
        if (n_bytes) {
            const cudaError_t c = cudaMemcpy(p, src, n_bytes, cudaMemcpyHostToDevice);
            if (c != cudaSuccess) {
                cudaFree(p);
                delete w;
                return bhd_cuda_fail(ctx, c, "uploading weight bytes");
            }
        }
    }
    bhd_weight_build_tensor_map(ctx, w);
    bhd_weight_build_tensor_map16(ctx, w);
    *out = w;
    return BHD_OK;
}

int32_t bhd_weight_upload(bhd_ctx* ctx, const uint8_t* bytes_host, uint64_t n_bytes, uint32_t ggml_type, uint64_t rows,
                          uint64_t cols, uint64_t n_slabs, bhd_weight** out_weight) {
    return make_weight(ctx, bytes_host, false, n_bytes, ggml_type, rows, cols, n_slabs, out_weight);
}

int32_t bhd_weight_wrap_device(bhd_ctx* ctx, const void* bytes_dev, uint64_t n_bytes, uint32_t ggml_type, uint64_t rows,
                               uint64_t cols, uint64_t n_slabs, bhd_weight** out_weight) {
    return make_weight(ctx, bytes_dev, true, n_bytes, ggml_type, rows, cols, n_slabs, out_weight);
}

int32_t bhd_weight_free(bhd_weight* w) {
    if (!w || w->magic != BHD_WEIGHT_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (w->owned && w->dev) {
        bhd_device_guard guard(w->device);
        cudaDeviceSynchronize();
        cudaFree(w->dev);
    }
    w->magic = 0;
    delete w;
    return BHD_OK;
}

int32_t bhd_dequantize(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, float* out_dev, uint64_t out_len,
                       void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!valid_w(ctx, w)) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "dequantize: not a weight of this context");
    if (slab >= w->slabs) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: slab %llu of %llu", (unsigned long long)slab, (unsigned long long)w->slabs);
    if (out_len != w->rows * w->cols)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: expected %llu floats, got %llu",
                        (unsigned long long)(w->rows * w->cols), (unsigned long long)out_len);
    if (out_len == 0) return BHD_OK;
    if (!out_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "dequantize: null output");
    bhd_device_guard guard(ctx);
    return bhd_launch_dequantize(ctx, w, slab, out_dev, cudaStream_t(stream));
}

static int32_t check_matvec_args(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x, const void* y,
                                 uint64_t batch, float scale, const char* who) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!valid_w(ctx, w)) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "%s: not a weight of this context", who);
    if (slab >= w->slabs)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: slab %llu of %llu", (unsigned long long)slab,
                        (unsigned long long)w->slabs);
    if (!isfinite(scale)) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "%s: scale must be finite", who);
    if (batch > 0 && ((w->cols > 0 && !x) || (w->rows > 0 && !y)))
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "%s: null buffer", who);
    return BHD_OK;
}

int32_t bhd_matvec(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x_dev, float* y_dev, uint32_t batch,
                   float scale, int32_t accumulate, void* stream) {
    const int32_t st = check_matvec_args(ctx, w, slab, x_dev, y_dev, batch, scale, "matvec");
    if (st != BHD_OK) return st;
    if (batch == 0 || w->rows == 0) return BHD_OK;
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
    bool handled = false;
    if (batch <= 2) {
        const int32_t is = bhd_launch_matvec_decode_i8(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s, &handled);
        if (is != BHD_OK || handled) return is;
    }
    if (batch <= 4) {
        const int32_t ds = bhd_launch_matvec_decode(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s, &handled);
        if (ds != BHD_OK || handled) return ds;
    }
    const int32_t fs = bhd_launch_matvec_fast(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s, &handled);
    if (fs != BHD_OK || handled) return fs;
    return bhd_launch_matvec_general(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s);
}

int32_t bhd_matmul(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x_dev, float* y_dev, uint64_t m,
                   void* stream) {
    const int32_t st = check_matvec_args(ctx, w, slab, x_dev, y_dev, m, 1.0f, "matmul");
    if (st != BHD_OK) return st;
    if (m == 0 || w->rows == 0) return BHD_OK;
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
    bool handled = false;
    const int32_t gs = bhd_launch_gemm_q8_tcgen05(ctx, w, slab, x_dev, y_dev, m, s, &handled);
    if (gs != BHD_OK || handled) return gs;
    const int32_t fs = bhd_launch_matvec_fast(ctx, w, slab, x_dev, y_dev, m, 1.0f, 0, s, &handled);
    if (fs != BHD_OK || handled) return fs;
    return bhd_launch_matvec_general(ctx, w, slab, x_dev, y_dev, m, 1.0f, 0, s);
}

static int32_t ensure_stage(bhd_ctx* ctx, float** buf, size_t* have, size_t bytes, const char* purpose) {
    if (bytes <= *have) return BHD_OK;
    cudaDeviceSynchronize();
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %zu bytes for %s", bhd_device_name(), bytes, purpose);
    }
    *buf = static_cast<float*>(p);
    *have = bytes;
    return BHD_OK;
}

// The device address of a page-locked host buffer (unified addressing), or nullptr for pageable memory.
static float* mapped_address(const void* host) {
    cudaPointerAttributes a;
    float* dev = nullptr;
    if (cudaPointerGetAttributes(&a, host) == cudaSuccess && a.type == cudaMemoryTypeHost && a.devicePointer)
        dev = static_cast<float*>(a.devicePointer);
    cudaGetLastError();  // a pageable pointer is reported as an error by older drivers: not ours to keep
    return dev;
}

// Reports what the kernels of the host-buffer stream flagged. `bits` was copied by the stream itself.
static int32_t report_status_bits(bhd_ctx* ctx, uint32_t bits) {
    if (bits == 0) return BHD_OK;
    return bhd_fail(ctx, BHD_ERR_DEVICE_STATUS, "device status 0x%x:%s%s%s%s%s", bits,
                    (bits & BHD_DEV_NAN_IN_SOFTMAX) ? " softmax input cannot contain NaN;" : "",
                    (bits & BHD_DEV_BAD_EXPERT_ID) ? " expert id out of range;" : "",
                    (bits & BHD_DEV_WAIT_TIMEOUT) ? " a bounded wait gave up;" : "",
                    (bits & BHD_DEV_BAD_ROUTE_PROB) ? " router probabilities not finite, non-negative with a positive sum;" : "",
                    (bits & BHD_DEV_ACTIVATION_RANGE) ? " an activation is NaN or infinite, or beyond the fp16 range (|x| > 65504) on a path with fp16 operands;" : "");
}

// Waits for the host-buffer stream and reports the status word (read and cleared in stream order).
static int32_t finish_host_stream(bhd_ctx* ctx) {
    cudaStream_t s = ctx->host_stream;
    BHD_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, 4, cudaMemcpyDeviceToHost, s), "reading the status word");
    BHD_CUDA(ctx, cudaStreamSynchronize(s), "waiting for the host-buffer stream");
    const uint32_t bits = ctx->status_host[0];
    if (bits == 0) return BHD_OK;
    BHD_CUDA(ctx, cudaMemsetAsync(ctx->status_dev, 0, 4, s), "clearing the status word");
    BHD_CUDA(ctx, cudaStreamSynchronize(s), "waiting for the host-buffer stream");
    return report_status_bits(ctx, bits);
}

// Enqueues one host-buffer matvec on the context's own stream, without waiting for it.
static int32_t enqueue_matvec_host(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x_host, float* y_host,
                                   uint32_t batch, float scale, int32_t accumulate) {
    const size_t xb = size_t(batch) * w->cols * sizeof(float), yb = size_t(batch) * w->rows * sizeof(float);
    cudaStream_t s = ctx->host_stream;
    int32_t st;
    // A page-locked output buffer is addressable from the device (unified addressing): the
    // kernel then writes y across PCIe itself, which saves one copy operation per call. x is
    // always staged in device memory, because every cluster of CTAs reads all of it; a
    // page-locked x is staged by a small kernel chained to the matvec by programmatic dependent
    // launch (the fetch across PCIe hides behind the previous matvec), a pageable one by a copy.
    float* y_direct = accumulate ? nullptr : mapped_address(y_host);
    const float* x_mapped = mapped_address(x_host);
    if ((st = ensure_stage(ctx, &ctx->stage_x, &ctx->stage_x_bytes, xb ? xb : 16, "activation staging")) != BHD_OK) return st;
    if (!y_direct && (st = ensure_stage(ctx, &ctx->stage_y, &ctx->stage_y_bytes, yb, "output staging")) != BHD_OK) return st;
    if (xb) {
        if (x_mapped && (reinterpret_cast<uintptr_t>(x_mapped) & 15) == 0 && xb % 16 == 0) {
            if ((st = bhd_launch_stage_copy(ctx, x_mapped, ctx->stage_x, xb / 16, s)) != BHD_OK) return st;
        } else {
            BHD_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, x_host, xb, cudaMemcpyHostToDevice, s), "copying activations in");
        }
    }
    if (accumulate) BHD_CUDA(ctx, cudaMemcpyAsync(ctx->stage_y, y_host, yb, cudaMemcpyHostToDevice, s), "copying outputs in");
    st = bhd_matvec(ctx, w, slab, ctx->stage_x, y_direct ? y_direct : ctx->stage_y, batch, scale, accumulate, s);
    if (st != BHD_OK) return st;
    if (!y_direct) BHD_CUDA(ctx, cudaMemcpyAsync(y_host, ctx->stage_y, yb, cudaMemcpyDeviceToHost, s), "copying outputs back");
    return BHD_OK;
}

int32_t bhd_matvec_host(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x_host, float* y_host,
                        uint32_t batch, float scale, int32_t accumulate) {
    int32_t st = check_matvec_args(ctx, w, slab, x_host, y_host, batch, scale, "matvec_host");
    if (st != BHD_OK) return st;
    if (batch == 0 || w->rows == 0) return BHD_OK;
    bhd_device_guard guard(ctx);
    if ((st = enqueue_matvec_host(ctx, w, slab, x_host, y_host, batch, scale, accumulate)) != BHD_OK) return st;
    return finish_host_stream(ctx);
}

int32_t bhd_matvec_host_async(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x_host, float* y_host,
                              uint32_t batch, float scale, int32_t accumulate) {
    int32_t st = check_matvec_args(ctx, w, slab, x_host, y_host, batch, scale, "matvec_host_async");
    if (st != BHD_OK) return st;
    if (batch == 0 || w->rows == 0) return BHD_OK;
    bhd_device_guard guard(ctx);
    return enqueue_matvec_host(ctx, w, slab, x_host, y_host, batch, scale, accumulate);
}

int32_t bhd_sync(bhd_ctx* ctx) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_device_guard guard(ctx);
    return finish_host_stream(ctx);
}

int32_t bhd_moe_layer_host(bhd_ctx* ctx, const bhd_weight* router, const bhd_weight* gate_exps,
                           const bhd_weight* up_exps, const bhd_weight* down_exps, const float* x_host, float* y_host,
                           uint64_t n_positions, uint32_t top_k, int32_t* experts_host, float* weights_host,
                           int32_t* counts_host, int32_t accumulate) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!valid_w(ctx, router) || !valid_w(ctx, gate_exps))
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_layer_host: tensors are not weights of this context");
    if (n_positions == 0) return BHD_OK;
    if (!x_host || !y_host) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_layer_host: null buffer");
    bhd_device_guard guard(ctx);
    const uint64_t dim = router->cols, ne = router->rows;
    const size_t xb = size_t(n_positions) * dim * sizeof(float);
    const size_t rb = size_t(n_positions) * top_k * 4;
    // y staging holds: y [T*dim] f32 | experts [T*k] i32 | weights [T*k] f32 | counts [ne] i32
    const size_t yb = xb + 2 * rb + ne * 4;
    int32_t st;
    if ((st = ensure_stage(ctx, &ctx->stage_x, &ctx->stage_x_bytes, xb, "activation staging")) != BHD_OK) return st;
    if ((st = ensure_stage(ctx, &ctx->stage_y, &ctx->stage_y_bytes, yb, "output staging")) != BHD_OK) return st;
    cudaStream_t s = ctx->host_stream;
    float* y_dev = ctx->stage_y;
    int32_t* e_dev = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(y_dev) + xb);
    float* w_dev = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(e_dev) + rb);
    int32_t* c_dev = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(w_dev) + rb);
    BHD_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, x_host, xb, cudaMemcpyHostToDevice, s), "copying activations in");
    if (accumulate) BHD_CUDA(ctx, cudaMemcpyAsync(y_dev, y_host, xb, cudaMemcpyHostToDevice, s), "copying outputs in");
    st = bhd_moe_layer(ctx, router, gate_exps, up_exps, down_exps, ctx->stage_x, y_dev, n_positions, top_k, e_dev, w_dev,
                       c_dev, accumulate, s);
    if (st != BHD_OK) return st;
    BHD_CUDA(ctx, cudaMemcpyAsync(y_host, y_dev, xb, cudaMemcpyDeviceToHost, s), "copying outputs back");
    if (experts_host) BHD_CUDA(ctx, cudaMemcpyAsync(experts_host, e_dev, rb, cudaMemcpyDeviceToHost, s), "copying experts back");
    if (weights_host) BHD_CUDA(ctx, cudaMemcpyAsync(weights_host, w_dev, rb, cudaMemcpyDeviceToHost, s), "copying route weights back");
    if (counts_host) BHD_CUDA(ctx, cudaMemcpyAsync(counts_host, c_dev, ne * 4, cudaMemcpyDeviceToHost, s), "copying counts back");
    return finish_host_stream(ctx);
}

int32_t bhd_check_status(bhd_ctx* ctx, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
    BHD_CUDA(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, 4, cudaMemcpyDeviceToHost, s), "reading the status word");
    BHD_CUDA(ctx, cudaMemsetAsync(ctx->status_dev, 0, 4, s), "clearing the status word");
    BHD_CUDA(ctx, cudaStreamSynchronize(s), "waiting for the status word");
    return report_status_bits(ctx, ctx->status_host[0]);
}

int32_t bhd_debug_wait_test(bhd_ctx* ctx, uint32_t spin_limit, uint32_t drop_one_copy) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    ctx->spin_limit = spin_limit;
    ctx->debug_drop = drop_one_copy ? 1u : 0u;
    return BHD_OK;
}

int32_t bhd_debug_option(bhd_ctx* ctx, uint32_t key, uint32_t value) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    switch (key) {
        case BHD_OPTION_MOE_TC_MIN_CLASS: ctx->moe_tc_min_cls = value; return BHD_OK;
        case BHD_OPTION_MOE_TC_PLAIN: ctx->moe_tc_plain = value; return BHD_OK;
        case BHD_OPTION_GEMM_IMPL: ctx->gemm_impl = value; return BHD_OK;
        case BHD_OPTION_ROUTER_TILING: ctx->router_variant = value; return BHD_OK;
        case BHD_OPTION_PLAIN_LAUNCHES: ctx->plain_launches = value; return BHD_OK;
        default: return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "debug_option: unknown key %u", key);
    }
}

uint64_t bhd_launch_count(const bhd_ctx* ctx) { return valid_ctx(ctx) ? ctx->launches : 0; }

}  // extern "C"
