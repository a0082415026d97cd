// The qwen3moe routed-expert block: router softmax + stable top-k + renormalisation,
// per-expert route counts, and the general (any shape) expert kernels.
//
// Follows crates/beholdd-model/src/qwen3moe/forward.rs:1299-1407 and :1886-1924 of the
// reference; the arithmetic that decides expert *indices* is kept in the CPU's exact
// order so that the selection is the CPU's selection.
#include "common.cuh"
#include "expf_exact.h"

namespace {

constexpr int NEAR_MISS_WINDOW = 8;  // forward.rs NEAR_MISS_WINDOW

// One CTA per position; thread e owns expert e (n_experts <= 1024).
// Input: logits (bit-identical to the CPU's router matvec, computed by the order-exact
// matvec kernel) in probs[t][e]; output: probabilities in place plus the selection.
__global__ void k_route_select(float* __restrict__ probs, uint32_t n_experts, uint32_t top_k,
                               int32_t* __restrict__ experts_out, float* __restrict__ weights_out,
                               int32_t* __restrict__ counts, int32_t* __restrict__ near_out, uint32_t near_per,
                               uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    extern __shared__ float sh[];  // [n_experts] values, then selection scratch
    float* val = sh;
    float* psel = sh + n_experts;                                   // [top_k]
    int32_t* isel = reinterpret_cast<int32_t*>(psel + top_k);       // [top_k]
    __shared__ float s_red[32];
    __shared__ float s_max, s_inv;
    __shared__ double s_sum64;

    const uint32_t t = blockIdx.x, e = threadIdx.x;
    float* row = probs + uint64_t(t) * n_experts;
    const bool live = e < n_experts;
    float v = live ? row[e] : -INFINITY;
    if (live && isnan(v)) atomicOr(status, BHD_DEV_NAN_IN_SOFTMAX);  // Device::softmax refuses NaN (cpu.rs:576-580)

    // max (order-independent); vecops.rs:71
    float m = v;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((e & 31) == 0) s_red[e >> 5] = m;
    __syncthreads();
    if (e < 32) {
        float mm = e < (blockDim.x >> 5) ? s_red[e] : -INFINITY;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
        if (e == 0) s_max = mm;
    }
    __syncthreads();
    m = s_max;
    const bool all_masked = !isfinite(m);  // vecops.rs:72-77: every entry -inf (or +inf max) -> zeros
    float ev = 0.0f;
    if (live && !all_masked) ev = isfinite(v) ? bhd_expf_exact(__fsub_rn(v, m)) : 0.0f;
    if (live) val[e] = ev;
    __syncthreads();
    if (e == 0) {
        // Sequential f32 sum in index order, vecops.rs:78-83.
        float sum = 0.0f;
        for (uint32_t i = 0; i < n_experts; ++i) sum = __fadd_rn(sum, val[i]);
        s_inv = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    const float p = all_masked ? 0.0f : __fmul_rn(ev, s_inv);
    __syncthreads();
    if (live) {
        val[e] = p;
        row[e] = p;
    }
    if (top_k == 0) return;  // softmax only
    __syncthreads();
    if (live) {
        // Rank of expert e under (probability descending, index ascending): forward.rs:1902-1906.
        if (!(isfinite(p) && p >= 0.0f)) atomicOr(status, BHD_DEV_BAD_ROUTE_PROB);  // forward.rs:1893-1898
        uint32_t rank = 0;
        for (uint32_t j = 0; j < n_experts; ++j) {
            const float pj = val[j];
            rank += (pj > p || (pj == p && j < e)) ? 1u : 0u;
        }
        if (rank < top_k) {
            psel[rank] = p;
            isel[rank] = int32_t(e);
        } else if (near_out && rank < top_k + near_per) {
            near_out[uint64_t(t) * near_per + (rank - top_k)] = int32_t(e);
        }
    }
    __syncthreads();
    if (e == 0) {
        // f64 sum of the selected probabilities in selection order, forward.rs:1910-1916.
        double sum = 0.0;
        for (uint32_t i = 0; i < top_k; ++i) sum = __dadd_rn(sum, double(psel[i]));
        if (!(isfinite(sum) && sum > 0.0)) atomicOr(status, BHD_DEV_BAD_ROUTE_PROB);
        s_sum64 = sum;
    }
    __syncthreads();
    if (e < top_k) {
        const uint64_t o = uint64_t(t) * top_k + e;
        experts_out[o] = isel[e];
        weights_out[o] = __double2float_rn(__ddiv_rn(double(psel[e]), s_sum64));  // forward.rs:1918-1922
        if (counts) atomicAdd(&counts[isel[e]], 1);
    }
}

// Router logits in the reference's summation order: logits[t][e] = ((0 + w[e][0]*x[t][0]) +
// w[e][1]*x[t][1]) + ..., every product and every sum rounded to f32 (forward.rs:1330-1336 ->
// cpu.rs:198-218). The chain of 'dim' dependent additions per (position, expert) is the floor
// (about 4 us for 2048 columns); everything else is arranged to stay out of its way:
//   * CTA = 8 experts x 8 positions = two warps (8 experts x 4 positions each), one chain per
//     lane; small CTAs, so that a single position already spreads over 16 SMs;
//   * 128-column tiles of w and x staged by 16-byte cp.async, six tiles in flight (a tile is
//     consumed in about 0.27 us, its fetch takes over 1 us);
//   * rows padded to 132 floats: the eight experts of a quarter-warp read 16 bytes each from
//     disjoint banks, the position's x is a broadcast.
// Two shapes (measured): up to 128 positions, CTAs of 8 positions with seven tiles in flight;
// beyond, CTAs of 32 positions with three.
constexpr int RT_EXP = 8, RT_COLS = 128, RT_LD = RT_COLS + 4, RT_W_FLOATS = RT_EXP * RT_LD;
constexpr size_t rt_smem_bytes(int tok, int buf) { return size_t(buf) * (RT_W_FLOATS + tok * RT_LD) * sizeof(float); }

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

// Requires dim % 4 == 0 and 16-byte aligned w and x.
template <int RT_TOK, int RT_BUF>
__global__ void __launch_bounds__(RT_TOK * RT_EXP) k_router_logits_f32(const float* __restrict__ w, uint32_t n_experts, uint32_t dim,
                                                           const float* __restrict__ x, uint32_t n_positions,
                                                           float* __restrict__ out, int32_t* __restrict__ counts) {
    bhd_wait_for_prior_kernels();
    // the per-expert route counts start at zero; the selection kernel that follows adds to them
    if (counts && blockIdx.y == 0) {
        const uint32_t e = blockIdx.x * RT_EXP + threadIdx.x;
        if (threadIdx.x < RT_EXP && e < n_experts) counts[e] = 0;
    }
    constexpr int RT_THREADS = RT_TOK * RT_EXP, RT_X_FLOATS = RT_TOK * RT_LD;
    extern __shared__ __align__(16) float rt_smem[];
    float* ws = rt_smem;                          // [buf][expert][RT_LD]
    float* xs = rt_smem + RT_BUF * RT_W_FLOATS;   // [buf][position][RT_LD]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t e0 = blockIdx.x * RT_EXP, t0 = blockIdx.y * RT_TOK;
    const uint32_t tiles = (dim + RT_COLS - 1) / RT_COLS;
    auto load = [&](uint32_t tile, int buf) {
        const uint32_t c0 = tile * RT_COLS;
#pragma unroll
        for (int i = 0; i < RT_EXP * 32 / RT_THREADS; ++i) {  // w: 8 experts x 32 float4
            const uint32_t idx = threadIdx.x + RT_THREADS * i, e = idx >> 5, c = (idx & 31) * 4;
            float* dst = ws + buf * RT_W_FLOATS + e * RT_LD + c;
            if (e0 + e < n_experts && c0 + c < dim) cp_async16(dst, w + uint64_t(e0 + e) * dim + c0 + c);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < RT_TOK * 32 / RT_THREADS; ++i) {  // x: positions x 32 float4
            const uint32_t idx = threadIdx.x + RT_THREADS * i, t = idx >> 5, c = (idx & 31) * 4;
            float* dst = xs + buf * RT_X_FLOATS + t * RT_LD + c;
            if (t0 + t < n_positions && c0 + c < dim) cp_async16(dst, x + uint64_t(t0 + t) * dim + c0 + c);
            else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    for (uint32_t i = 0; i < RT_BUF - 1; ++i) {
        if (i < tiles) load(i, i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc = 0.0f;
    const uint32_t el = lane & 7, tl = uint32_t(warp) * 4 + (lane >> 3);  // this lane's expert and position within the CTA
    const bool chain = t0 + uint32_t(warp) * 4 < n_positions;            // whole warps skip tiles they have no position for
    for (uint32_t tile = 0; tile < tiles; ++tile) {
        const int buf = tile % RT_BUF;
        asm volatile("cp.async.wait_group %0;" ::"n"(RT_BUF - 2) : "memory");
        __syncthreads();  // tile is visible to everyone, and everyone is done with the buffer refilled below
        if (tile + RT_BUF - 1 < tiles) load(tile + RT_BUF - 1, (tile + RT_BUF - 1) % RT_BUF);
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (chain) {
            const uint32_t n = min(uint32_t(RT_COLS), dim - tile * RT_COLS);  // a multiple of 4
            const float4* wt = reinterpret_cast<const float4*>(ws + buf * RT_W_FLOATS + el * RT_LD);
            const float4* xt = reinterpret_cast<const float4*>(xs + buf * RT_X_FLOATS + tl * RT_LD);
            const uint32_t n4 = n / 4;
            float4 a[8], b[8];
            float pr[32];
            if (n == RT_COLS) {
                // The chain of dependent additions is the critical path of a warp, so everything
                // else is placed in its shadow, in program order (measured: 14.9 -> 9.5 us for one
                // position): between
                // the 32 additions of one 32-column group sit the 32 products of the next group
                // and the shared-memory loads of the one after.
                float npr[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) { a[i] = wt[i]; b[i] = xt[i]; }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    pr[4 * i] = __fmul_rn(a[i].x, b[i].x);
                    pr[4 * i + 1] = __fmul_rn(a[i].y, b[i].y);
                    pr[4 * i + 2] = __fmul_rn(a[i].z, b[i].z);
                    pr[4 * i + 3] = __fmul_rn(a[i].w, b[i].w);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) { a[i] = wt[8 + i]; b[i] = xt[8 + i]; }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc = __fadd_rn(acc, pr[4 * i]);
                        if (g < 3) npr[4 * i] = __fmul_rn(a[i].x, b[i].x);
                        acc = __fadd_rn(acc, pr[4 * i + 1]);
                        if (g < 3) npr[4 * i + 1] = __fmul_rn(a[i].y, b[i].y);
                        acc = __fadd_rn(acc, pr[4 * i + 2]);
                        if (g < 3) npr[4 * i + 2] = __fmul_rn(a[i].z, b[i].z);
                        acc = __fadd_rn(acc, pr[4 * i + 3]);
                        if (g < 3) npr[4 * i + 3] = __fmul_rn(a[i].w, b[i].w);
                        if (g < 2) { a[i] = wt[(g + 2) * 8 + i]; b[i] = xt[(g + 2) * 8 + i]; }
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) pr[i] = npr[i];
                }
            } else {
                // Ragged last tile: 32 columns at a time, the loads of the next 32 issued before
                // the 32 dependent additions of the current ones.
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    a[i] = uint32_t(i) < n4 ? wt[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                    b[i] = uint32_t(i) < n4 ? xt[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                for (uint32_t c = 0; c < n4; c += 8) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        pr[4 * i] = __fmul_rn(a[i].x, b[i].x);
                        pr[4 * i + 1] = __fmul_rn(a[i].y, b[i].y);
                        pr[4 * i + 2] = __fmul_rn(a[i].z, b[i].z);
                        pr[4 * i + 3] = __fmul_rn(a[i].w, b[i].w);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t cn = c + 8 + i;
                        if (cn < n4) { a[i] = wt[cn]; b[i] = xt[cn]; }
                    }
                    const uint32_t live = min(32u, (n4 - c) * 4);  // 32 except in a ragged last tile
                    if (live == 32) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc = __fadd_rn(acc, pr[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (uint32_t(i) < live) acc = __fadd_rn(acc, pr[i]);
                    }
                }
            }
        }
    }
    if (t0 + tl < n_positions && e0 + el < n_experts) out[uint64_t(t0 + tl) * n_experts + e0 + el] = acc;
}

// ---- general expert kernels (any dim / expert_ff that are whole Q8_0 blocks) -----------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One warp per (route, ff row): gate and up dot products of the route's expert with the
// route's position, then SiLU gating (vecops.rs:91-111 with limit 0).
__global__ void k_moe_gate_up_warp(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                                   uint64_t slab_bytes, uint64_t row_bytes, uint32_t dim, uint32_t ff,
                                   const float* __restrict__ x, const int32_t* __restrict__ experts, uint32_t top_k,
                                   uint32_t first_expert, uint32_t n_local, uint32_t n_experts_total,
                                   float* __restrict__ act, uint32_t* __restrict__ status) {
    const uint32_t route = blockIdx.x;
    const uint32_t f = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (f >= ff) return;
    const int32_t e = experts[route];
    if (e < 0 || uint32_t(e) >= n_experts_total) {
        if (lane == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
        return;
    }
    if (uint32_t(e) < first_expert || uint32_t(e) >= first_expert + n_local) return;
    const uint64_t off = uint64_t(uint32_t(e) - first_expert) * slab_bytes + uint64_t(f) * row_bytes;
    const uint8_t* grow = gate + off;
    const uint8_t* urow = up + off;
    const float* xv = x + uint64_t(route / top_k) * dim;
    float g = 0.0f, u = 0.0f;
    for (uint32_t k = lane; k < dim; k += 32) {
        const float xk = xv[k];
        g = fmaf(bhd_decode_elem<BHD_TYPE_Q8_0>(grow, k), xk, g);
        u = fmaf(bhd_decode_elem<BHD_TYPE_Q8_0>(urow, k), xk, u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) act[uint64_t(route) * ff + f] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

// One warp per (position, output row): the down projections of the position's routes,
// scaled by the route weight and added in selection order into a zero accumulator
// (forward.rs:1385-1398; cpu.rs:280-284: out += acc * scale, product and sum rounded apart).
__global__ void k_moe_down_warp(const uint8_t* __restrict__ down, uint64_t slab_bytes, uint64_t row_bytes,
                                uint32_t dim, uint32_t ff, const float* __restrict__ act,
                                const int32_t* __restrict__ experts, const float* __restrict__ weights,
                                uint32_t top_k, uint32_t first_expert, uint32_t n_local, float* __restrict__ y,
                                int accumulate) {
    const uint32_t t = blockIdx.x;
    const uint32_t h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= dim) return;
    float out = 0.0f;
    for (uint32_t j = 0; j < top_k; ++j) {
        const uint32_t route = t * top_k + j;
        const int32_t e = experts[route];
        if (e < 0 || uint32_t(e) < first_expert || uint32_t(e) >= first_expert + n_local) continue;
        const uint8_t* drow = down + uint64_t(uint32_t(e) - first_expert) * slab_bytes + uint64_t(h) * row_bytes;
        const float* a = act + uint64_t(route) * ff;
        float d = 0.0f;
        for (uint32_t k = lane; k < ff; k += 32) d = fmaf(bhd_decode_elem<BHD_TYPE_Q8_0>(drow, k), a[k], d);
        d = warp_sum(d);
        out = __fadd_rn(out, __fmul_rn(d, weights[route]));
    }
    if (lane == 0) {
        float* dst = y + uint64_t(t) * dim + h;
        *dst = accumulate ? __fadd_rn(*dst, out) : out;
    }
}

__global__ void k_moe_combine(const float* __restrict__ per_route, float* __restrict__ y, uint64_t n, uint32_t top_k,
                              int accumulate) {
    bhd_wait_for_prior_kernels();
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    float out = 0.0f;
    for (uint32_t j = 0; j < top_k; ++j) out = __fadd_rn(out, per_route[uint64_t(j) * n + i]);
    y[i] = accumulate ? __fadd_rn(y[i], out) : out;
}

bool valid_ctx(const bhd_ctx* c) { return c && c->magic == BHD_CTX_MAGIC; }
bool valid_w(const bhd_ctx* c, const bhd_weight* w) { return w && w->magic == BHD_WEIGHT_MAGIC && w->ctx == c; }

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

namespace {
__global__ void k_expf_exact(const float* __restrict__ in, float* __restrict__ out, uint64_t n) {
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i < n) out[i] = bhd_expf_exact(in[i]);
}
}  // namespace

extern "C" int32_t bhd_debug_expf(bhd_ctx* ctx, const float* in_dev, float* out_dev, uint64_t n, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return BHD_OK;
    if (!in_dev || !out_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "debug_expf: null buffer");
    bhd_device_guard guard(ctx);
    k_expf_exact<<<unsigned((n + 255) / 256), 256, 0, cudaStream_t(stream)>>>(in_dev, out_dev, n);
    BHD_LAUNCHED(ctx, "expf kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_softmax(bhd_ctx* ctx, float* v_dev, uint64_t n_rows, uint64_t n, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: softmax input cannot be empty");
    if (n > 1024) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: softmax rows longer than 1024 are not supported");
    if (n_rows == 0) return BHD_OK;
    if (!v_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "softmax: null buffer");
    bhd_device_guard guard(ctx);
    // Reuses the router kernel with top_k = 0: softmax only.
    const unsigned threads = unsigned((n + 31) / 32 * 32);
    const size_t smem = n * sizeof(float) + 16;
    bhd_launch_dependent(ctx, k_route_select, dim3(unsigned(n_rows)), dim3(threads), smem, cudaStream_t(stream), v_dev, uint32_t(n), 0, nullptr, nullptr,
                                                                               nullptr, nullptr, 0, ctx->status_dev);
    BHD_LAUNCHED(ctx, "softmax kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_moe_route(bhd_ctx* ctx, const bhd_weight* router, const float* x_dev, uint64_t n_positions,
                                 uint32_t top_k, int32_t* experts_dev, float* weights_dev, int32_t* counts_dev,
                                 int32_t* near_dev, float* probs_dev, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!valid_w(ctx, router)) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_route: router is not a weight of this context");
    const uint64_t n_experts = router->rows;
    if (top_k == 0 || top_k > n_experts)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: top-k must be between 1 and %llu, got %u",
                        (unsigned long long)n_experts, top_k);
    if (n_experts > 1024) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: more than 1024 experts are not supported");
    if (n_positions == 0) return BHD_OK;
    if (!x_dev || !experts_dev || !weights_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_route: null buffer");
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
    float* probs = probs_dev;
    if (!probs) {
        const int32_t st = bhd_ensure_workspace(ctx, n_positions * n_experts * sizeof(float), s);
        if (st != BHD_OK) return st;
        probs = reinterpret_cast<float*>(ctx->workspace);
    }
    const bool fast_router = router->kind == BHD_TYPE_F32 && n_positions <= 65535ull * 8 && router->cols % 4 == 0 &&
                             (reinterpret_cast<uintptr_t>(router->dev) & 15) == 0 && (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0;
    if (counts_dev && !fast_router)  // the fast router kernel clears them itself
        BHD_CUDA(ctx, cudaMemsetAsync(counts_dev, 0, n_experts * sizeof(int32_t), s), "clearing expert counts");
    // Router logits in the CPU's summation order (forward.rs:1330-1336 -> cpu.rs:198-218).
    if (fast_router) {
        static bhd_once_per_device once;
        if (once.pending(ctx)) {
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_f32<8, 7>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rt_smem_bytes(8, 7))),
                     "raising the shared memory limit");
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_f32<32, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rt_smem_bytes(32, 3))),
                     "raising the shared memory limit");
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_f32<32, 5>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rt_smem_bytes(32, 5))),
                     "raising the shared memory limit");
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_router_logits_f32<16, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rt_smem_bytes(16, 6))),
                     "raising the shared memory limit");
            once.mark(ctx);
        }
        const float* rw = reinterpret_cast<const float*>(router->dev);
        const unsigned gx = unsigned((n_experts + RT_EXP - 1) / RT_EXP);
        const uint32_t variant = ctx->router_variant;
        if (n_positions <= 128 || variant == 3)  // measured: 18.5 us against 24.7 us at 128 positions; 46 against 41 at 512
            bhd_launch_dependent(ctx, k_router_logits_f32<8, 7>, dim3(gx, unsigned((n_positions + 7) / 8)), dim3(64), rt_smem_bytes(8, 7), s, 
                rw, uint32_t(n_experts), uint32_t(router->cols), x_dev, uint32_t(n_positions), probs, counts_dev);
        else if (variant == 1)
            bhd_launch_dependent(ctx, k_router_logits_f32<32, 5>, dim3(gx, unsigned((n_positions + 31) / 32)), dim3(256), rt_smem_bytes(32, 5), s, 
                rw, uint32_t(n_experts), uint32_t(router->cols), x_dev, uint32_t(n_positions), probs, counts_dev);
        else if (variant == 2)
            bhd_launch_dependent(ctx, k_router_logits_f32<16, 6>, dim3(gx, unsigned((n_positions + 15) / 16)), dim3(128), rt_smem_bytes(16, 6), s, 
                rw, uint32_t(n_experts), uint32_t(router->cols), x_dev, uint32_t(n_positions), probs, counts_dev);
        else
            bhd_launch_dependent(ctx, k_router_logits_f32<32, 3>, dim3(gx, unsigned((n_positions + 31) / 32)), dim3(256), rt_smem_bytes(32, 3), s, 
                rw, uint32_t(n_experts), uint32_t(router->cols), x_dev, uint32_t(n_positions), probs, counts_dev);
        BHD_LAUNCHED(ctx, "router logits kernel");
    } else {
        const int32_t st = bhd_launch_matvec_strict(ctx, router, 0, x_dev, probs, uint32_t(n_positions), 1.0f, 0, s);
        if (st != BHD_OK) return st;
    }
    const uint32_t near_per = uint32_t(n_experts - top_k < NEAR_MISS_WINDOW ? n_experts - top_k : NEAR_MISS_WINDOW);
    const unsigned threads = unsigned((n_experts + 31) / 32 * 32);
    const size_t smem = (n_experts + 2 * top_k) * sizeof(float) + 16;
    bhd_launch_dependent(ctx, k_route_select, dim3(unsigned(n_positions)), dim3(threads), smem, s, probs, uint32_t(n_experts), top_k, experts_dev,
                                                                 weights_dev, counts_dev, near_dev, near_per,
                                                                 ctx->status_dev);
    BHD_LAUNCHED(ctx, "route selection kernel");
    return BHD_OK;
}

namespace {

// Everything bhd_moe_experts checks before it touches an output; bhd_moe_layer runs the same
// checks before it routes, so that a refused call leaves the routing outputs alone too.
int32_t validate_experts(bhd_ctx* ctx, const bhd_weight* gate_exps, const bhd_weight* up_exps, const bhd_weight* down_exps,
                         const float* x_dev, uint64_t n_positions, uint32_t top_k, const int32_t* experts_dev,
                         const float* weights_dev, uint32_t n_local, const float* y_dev) {
    if (!valid_w(ctx, gate_exps) || !valid_w(ctx, up_exps) || !valid_w(ctx, down_exps))
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_experts: expert tensors are not weights of this context");
    if (gate_exps->kind != BHD_TYPE_Q8_0 || up_exps->kind != BHD_TYPE_Q8_0 || down_exps->kind != BHD_TYPE_Q8_0)
        return bhd_fail(ctx, BHD_ERR_UNSUPPORTED_FORMAT, "%s cannot decode %s routed experts (Q8_0 only)",
                        bhd_device_name(), bhd_kind_name(gate_exps->kind != BHD_TYPE_Q8_0 ? gate_exps->kind
                                                         : (up_exps->kind != BHD_TYPE_Q8_0 ? up_exps->kind : down_exps->kind)));
    const uint64_t ff = gate_exps->rows, dim = gate_exps->cols;
    if (up_exps->rows != ff || up_exps->cols != dim || down_exps->rows != dim || down_exps->cols != ff ||
        gate_exps->slabs != up_exps->slabs || gate_exps->slabs != down_exps->slabs)
        return bhd_fail(ctx, BHD_ERR_SHAPE,
                        "shape mismatch: experts gate %llux%llux%llu, up %llux%llux%llu, down %llux%llux%llu",
                        (unsigned long long)gate_exps->rows, (unsigned long long)gate_exps->cols,
                        (unsigned long long)gate_exps->slabs, (unsigned long long)up_exps->rows,
                        (unsigned long long)up_exps->cols, (unsigned long long)up_exps->slabs,
                        (unsigned long long)down_exps->rows, (unsigned long long)down_exps->cols,
                        (unsigned long long)down_exps->slabs);
    if (n_local != gate_exps->slabs)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: %u local experts but the tensors hold %llu slabs", n_local,
                        (unsigned long long)gate_exps->slabs);
    if (top_k == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: top-k must be positive");
    if (n_positions == 0) return BHD_OK;
    if (!x_dev || !experts_dev || !weights_dev || !y_dev)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_experts: null buffer");
    if (n_positions * top_k > 0x7fffffffull || dim > 0x7fffffffull || ff > 0x7fffffffull)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: routed block too large");
    return BHD_OK;
}

int32_t run_experts(bhd_ctx* ctx, const bhd_weight* gate_exps, const bhd_weight* up_exps, const bhd_weight* down_exps,
                    const float* x_dev, uint64_t n_positions, uint32_t top_k, const int32_t* experts_dev,
                    const float* weights_dev, uint32_t first_expert, uint32_t n_local, uint32_t n_total, float* y_dev,
                    int32_t accumulate, cudaStream_t s) {
    const uint64_t ff = gate_exps->rows, dim = gate_exps->cols;
    bool handled = false;
    int32_t st = bhd_moe_experts_fast(ctx, gate_exps, up_exps, down_exps, x_dev, n_positions, top_k, experts_dev,
                                      weights_dev, first_expert, n_local, n_total, y_dev, accumulate, s, &handled, nullptr);
    if (st != BHD_OK || handled) return st;

    // General kernels: one warp per (route, row). Grids put the large dimension on x.
    const uint64_t routes = n_positions * top_k;
    st = bhd_ensure_workspace(ctx, align_up(routes * ff * sizeof(float), 256), s);
    if (st != BHD_OK) return st;
    float* act = reinterpret_cast<float*>(ctx->workspace);
    const int warps = 8;
    const uint32_t ff_blocks = uint32_t((ff + warps - 1) / warps), dim_blocks = uint32_t((dim + warps - 1) / warps);
    if (ff_blocks > 65535u || dim_blocks > 65535u)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: expert matrices of %llu x %llu are beyond the general kernels",
                        (unsigned long long)ff, (unsigned long long)dim);
    k_moe_gate_up_warp<<<dim3(unsigned(routes), ff_blocks), warps * 32, 0, s>>>(
        gate_exps->dev, up_exps->dev, gate_exps->slab_bytes, gate_exps->row_bytes, uint32_t(dim), uint32_t(ff), x_dev,
        experts_dev, top_k, first_expert, n_local, n_total, act, ctx->status_dev);
    BHD_LAUNCHED(ctx, "expert gate/up kernel");
    k_moe_down_warp<<<dim3(unsigned(n_positions), dim_blocks), warps * 32, 0, s>>>(
        down_exps->dev, down_exps->slab_bytes, down_exps->row_bytes, uint32_t(dim), uint32_t(ff), act, experts_dev,
        weights_dev, top_k, first_expert, n_local, y_dev, accumulate);
    BHD_LAUNCHED(ctx, "expert down kernel");
    return BHD_OK;
}

}  // namespace

extern "C" int32_t bhd_moe_experts(bhd_ctx* ctx, const bhd_weight* gate_exps, const bhd_weight* up_exps,
                                   const bhd_weight* down_exps, const float* x_dev, uint64_t n_positions,
                                   uint32_t top_k, const int32_t* experts_dev, const float* weights_dev,
                                   uint32_t first_expert, uint32_t n_local, uint32_t n_experts, float* y_dev,
                                   int32_t accumulate, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    const int32_t st = validate_experts(ctx, gate_exps, up_exps, down_exps, x_dev, n_positions, top_k, experts_dev,
                                        weights_dev, n_local, y_dev);
    if (st != BHD_OK || n_positions == 0) return st;
    if (n_experts != 0 && uint64_t(first_expert) + n_local > n_experts)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: local experts %u..%llu exceed the %u experts of the layer",
                        first_expert, (unsigned long long)first_expert + n_local, n_experts);
    bhd_device_guard guard(ctx);
    // n_experts == 0: the caller does not know the layer's expert count; only negative ids can then be told from
    // ids that belong to another rank.
    return run_experts(ctx, gate_exps, up_exps, down_exps, x_dev, n_positions, top_k, experts_dev, weights_dev,
                       first_expert, n_local, n_experts ? n_experts : 0x7fffffffu, y_dev, accumulate, cudaStream_t(stream));
}

// bhd_moe_route for callers inside the library (validated arguments, no probabilities or near misses).
int32_t bhd_moe_route_internal(bhd_ctx* ctx, const bhd_weight* router, const float* x_dev, uint64_t n_positions, uint32_t top_k,
                               int32_t* experts_dev, float* weights_dev, int32_t* counts_dev, cudaStream_t s) {
    return bhd_moe_route(ctx, router, x_dev, n_positions, top_k, experts_dev, weights_dev, counts_dev, nullptr, nullptr, s);
}

extern "C" int32_t bhd_moe_combine(bhd_ctx* ctx, const float* per_route_dev, float* y_dev, uint64_t n_positions,
                                   uint32_t top_k, uint64_t dim, int32_t accumulate, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    const uint64_t n = n_positions * dim;
    if (n == 0) return BHD_OK;
    if (!per_route_dev || !y_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_combine: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_moe_combine, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), per_route_dev, y_dev, n, top_k, accumulate);
    BHD_LAUNCHED(ctx, "route combine kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_moe_layer(bhd_ctx* ctx, const bhd_weight* router, const bhd_weight* gate_exps,
                                 const bhd_weight* up_exps, const bhd_weight* down_exps, const float* x_dev,
                                 float* y_dev, uint64_t n_positions, uint32_t top_k, int32_t* experts_dev,
                                 float* weights_dev, int32_t* counts_dev, int32_t accumulate, void* stream) {
    if (!valid_ctx(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!valid_w(ctx, router) || !valid_w(ctx, gate_exps))
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_layer: tensors are not weights of this context");
    if (router->cols != gate_exps->cols || router->rows != gate_exps->slabs)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: router %llux%llu against %llu experts of width %llu",
                        (unsigned long long)router->rows, (unsigned long long)router->cols,
                        (unsigned long long)gate_exps->slabs, (unsigned long long)gate_exps->cols);
    if (!experts_dev || !weights_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "moe_layer: null routing buffers");
    // every refusal of the expert half happens before the router writes anything
    int32_t st = validate_experts(ctx, gate_exps, up_exps, down_exps, x_dev, n_positions, top_k, experts_dev, weights_dev,
                                  uint32_t(gate_exps->slabs), y_dev);
    if (st != BHD_OK) return st;
    bhd_device_guard guard(ctx);
    st = bhd_moe_route(ctx, router, x_dev, n_positions, top_k, experts_dev, weights_dev, counts_dev, nullptr, nullptr, stream);
    if (st != BHD_OK || n_positions == 0) return st;
    return run_experts(ctx, gate_exps, up_exps, down_exps, x_dev, n_positions, top_k, experts_dev, weights_dev, 0,
                       uint32_t(gate_exps->slabs), uint32_t(gate_exps->slabs), y_dev, accumulate, cudaStream_t(stream));
}
