// General kernels of the path: whole-weight decode, the order-exact matvec, the
// shape-agnostic warp-per-row matvec, and the small elementwise operators.
//
// The fast TMA-staged tensor-core matvec lives in matvec_mma.cu; the kernels here accept
// every supported format and every shape (any row pitch, any column count) and are what
// the library uses when a shape does not meet the fast path's alignment rules.
#include "common.cuh"

namespace {

template <uint32_t KIND>
__global__ void k_dequantize(const uint8_t* __restrict__ w, uint64_t row_bytes, uint64_t rows, uint64_t cols,
                             float* __restrict__ out) {
    const uint64_t n = rows * cols;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t r = i / cols, k = i - r * cols;
        out[i] = bhd_decode_elem<KIND>(w + r * row_bytes, k);
    }
}

// One thread per (row, batch column): a single f32 accumulator walked left to right with a
// separately rounded product and sum, i.e. exactly the CPU reference's order
// (crates/beholdd-backend/src/cpu.rs:198-218; crates/beholdd-kernel/src/kquant.rs:61-79).
// Results are bit-identical to the CPU path. Used for the router logits, whose ranking
// must match the CPU's, and as the on-device cross-check of the fast kernels.
template <uint32_t KIND>
__global__ void k_matvec_strict(const uint8_t* __restrict__ w, uint64_t row_bytes, uint64_t rows, uint64_t cols,
                                const float* __restrict__ x, float* __restrict__ y, uint32_t batch, float scale,
                                int accumulate) {
    const uint64_t idx = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (idx >= rows * batch) return;
    const uint64_t b = idx / rows, r = idx - b * rows;
    const uint8_t* row = w + r * row_bytes;
    const float* xv = x + b * cols;
    float acc = 0.0f;
    for (uint64_t k = 0; k < cols; ++k) acc = __fadd_rn(acc, __fmul_rn(bhd_decode_elem<KIND>(row, k), xv[k]));
    const float v = __fmul_rn(acc, scale);
    float* out = y + b * rows + r;
    *out = accumulate ? __fadd_rn(*out, v) : v;
}

// One warp per row, lanes stride the columns (coalesced bytes), up to 8 batch columns per
// pass, fixed-order shuffle reduction (deterministic).
template <uint32_t KIND, int NB>
__global__ void k_matvec_warp(const uint8_t* __restrict__ w, uint64_t row_bytes, uint64_t rows, uint64_t cols,
                              const float* __restrict__ x, float* __restrict__ y, uint64_t b0, float scale,
                              int accumulate) {
    const uint64_t r = (blockIdx.x * uint64_t(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const uint8_t* row = w + r * row_bytes;
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[b] = 0.0f;
    for (uint64_t k = lane; k < cols; k += 32) {
        const float wv = bhd_decode_elem<KIND>(row, k);
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[b] = fmaf(wv, x[(b0 + b) * cols + k], acc[b]);
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        float v = acc[b];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) {
            const float s = __fmul_rn(v, scale);
            float* out = y + (b0 + b) * rows + r;
            *out = accumulate ? __fadd_rn(*out, s) : s;
        }
    }
}

__global__ void k_fill_scaled_zero(float* y, uint64_t n, float scale, int accumulate) {
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const float v = __fmul_rn(0.0f, scale);
    y[i] = accumulate ? __fadd_rn(y[i], v) : v;
}

}  // namespace

int32_t bhd_launch_dequantize(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, float* out, cudaStream_t s) {
    const uint64_t n = w->rows * w->cols;
    if (n == 0) return BHD_OK;
    const int threads = 256;
    const uint64_t want = (n + threads - 1) / threads;
    const int blocks = int(want < uint64_t(ctx->sm_count) * 16 ? want : uint64_t(ctx->sm_count) * 16);
    const uint8_t* base = w->dev + slab * w->slab_bytes;
#define LAUNCH(K) k_dequantize<K><<<blocks, threads, 0, s>>>(base, w->row_bytes, w->rows, w->cols, out)
    BHD_DISPATCH_KIND(w->kind, LAUNCH)
#undef LAUNCH
    BHD_LAUNCHED(ctx, "dequantize kernel");
    return BHD_OK;
}

static int32_t launch_zero_width(bhd_ctx* ctx, float* y, uint64_t n, float scale, int accumulate, cudaStream_t s) {
    if (n == 0) return BHD_OK;
    k_fill_scaled_zero<<<unsigned((n + 255) / 256), 256, 0, s>>>(y, n, scale, accumulate);
    BHD_LAUNCHED(ctx, "zero-width matvec kernel");
    return BHD_OK;
}

int32_t bhd_launch_matvec_strict(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                 uint32_t batch, float scale, int accumulate, cudaStream_t s) {
    if (w->rows == 0 || batch == 0) return BHD_OK;
    if (w->cols == 0) return launch_zero_width(ctx, y, w->rows * batch, scale, accumulate, s);
    const uint64_t n = w->rows * batch;
    const int threads = 64;  // few rows per CTA: every thread streams its own row
    const uint8_t* base = w->dev + slab * w->slab_bytes;
#define LAUNCH(K)                                                                                           \
    k_matvec_strict<K><<<unsigned((n + threads - 1) / threads), threads, 0, s>>>(base, w->row_bytes, w->rows, \
                                                                                  w->cols, x, y, batch, scale, accumulate)
    BHD_DISPATCH_KIND(w->kind, LAUNCH)
#undef LAUNCH
    BHD_LAUNCHED(ctx, "order-exact matvec kernel");
    return BHD_OK;
}

template <int NB>
static void launch_warp(const bhd_weight* w, const uint8_t* base, const float* x, float* y, uint64_t b0, float scale,
                        int accumulate, cudaStream_t s) {
    const int threads = 128;
    const unsigned blocks = unsigned((w->rows * 32 + threads - 1) / threads);
#define LAUNCH(K) \
    k_matvec_warp<K, NB><<<blocks, threads, 0, s>>>(base, w->row_bytes, w->rows, w->cols, x, y, b0, scale, accumulate)
    BHD_DISPATCH_KIND(w->kind, LAUNCH)
#undef LAUNCH
}

int32_t bhd_launch_matvec_general(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                  uint64_t batch, float scale, int accumulate, cudaStream_t s) {
    if (w->rows == 0 || batch == 0) return BHD_OK;
    if (w->cols == 0) return launch_zero_width(ctx, y, w->rows * batch, scale, accumulate, s);
    const uint8_t* base = w->dev + slab * w->slab_bytes;
    uint64_t b0 = 0;
    while (b0 < batch) {
        const uint64_t left = batch - b0;
        if (left >= 8) { launch_warp<8>(w, base, x, y, b0, scale, accumulate, s); b0 += 8; }
        else if (left >= 4) { launch_warp<4>(w, base, x, y, b0, scale, accumulate, s); b0 += 4; }
        else if (left >= 2) { launch_warp<2>(w, base, x, y, b0, scale, accumulate, s); b0 += 2; }
        else { launch_warp<1>(w, base, x, y, b0, scale, accumulate, s); b0 += 1; }
        BHD_LAUNCHED(ctx, "warp-per-row matvec kernel");
    }
    return BHD_OK;
}

// ---- staging of page-locked host activations --------------------------------------------
namespace {

// Copies n16 16-byte words from a page-locked host buffer (addressed through unified addressing)
// into device memory. Launched with programmatic stream serialization: the words are fetched
// across PCIe before the wait, while the previous kernel of the stream (which may still read
// dst) is running, and written after it has finished. Nothing on the GPU writes the source.
__global__ void k_stage_copy(const uint4* src, uint4* __restrict__ dst, size_t n16) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (i < n16) v = __ldcv(src + i);  // never a cached copy: the host rewrites this buffer between calls
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (i < n16) dst[i] = v;
}

}  // namespace

int32_t bhd_launch_stage_copy(bhd_ctx* ctx, const float* src_mapped, float* dst_dev, size_t n16, cudaStream_t s) {
    if (n16 == 0) return BHD_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned((n16 + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_stage_copy, reinterpret_cast<const uint4*>(src_mapped), reinterpret_cast<uint4*>(dst_dev), n16),
             "launching the activation staging kernel");
    ctx->launches += 1;
    return BHD_OK;
}

// ---- elementwise operators --------------------------------------------------------------

namespace {

// SiLU gating, crates/beholdd-kernel/src/vecops.rs:91-111.
__global__ void k_swiglu(float* __restrict__ gate, const float* __restrict__ up, uint64_t n, float limit) {
    bhd_wait_for_prior_kernels();
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    float g = gate[i], u = up[i];
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fmaxf(-limit, fminf(u, limit));
    }
    gate[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

__global__ void k_add_in_place(float* __restrict__ out, const float* __restrict__ res, uint64_t n) {
    bhd_wait_for_prior_kernels();
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], res[i]);
}

}  // namespace

extern "C" int32_t bhd_swiglu(bhd_ctx* ctx, float* gate_dev, const float* up_dev, uint64_t n, float limit,
                              void* stream) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return BHD_OK;
    if (!gate_dev || !up_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "swiglu: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_swiglu, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), gate_dev, up_dev, n, limit);
    BHD_LAUNCHED(ctx, "swiglu kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_add_in_place(bhd_ctx* ctx, float* output_dev, const float* residual_dev, uint64_t n,
                                    void* stream) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return BHD_OK;
    if (!output_dev || !residual_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "add_in_place: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_add_in_place, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), output_dev, residual_dev, n);
    BHD_LAUNCHED(ctx, "add_in_place kernel");
    return BHD_OK;
}
