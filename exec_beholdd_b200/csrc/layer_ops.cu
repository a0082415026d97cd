// The operators of a transformer layer around the quantised projections and the routed experts:
// RMSNorm (also the per-head QK-norm), rotary embedding in both pair layouts, causal /
// incremental attention over an f32 key-value cache, and embedding-row decoding.
//
// Each follows the reference's CPU arithmetic step by step, in the same order and at the same
// widths, so the results are the CPU's bits (up to the order of one f64 sum in RMSNorm):
//   RMSNorm    crates/beholdd-kernel/src/vecops.rs:54-64   f64 sum of squares, one f32 factor
//   rope       vecops.rs:163-197                           a*c - b*s, a*s + b*c, each product and sum rounded to f32
//   attention  crates/beholdd-backend/src/cpu.rs:585-837   f64 dot products, f32 softmax (host expf), f64 value sums
//   embedding  crates/beholdd-model/src/qwen3moe/forward.rs:954-972  Device::dequantize of one row
// These are HBM- or latency-bound helpers, not hot kernels: one CTA per row / per (position, head).
#include "common.cuh"
#include "expf_exact.h"

namespace {

bool ctx_ok(const bhd_ctx* c) { return c && c->magic == BHD_CTX_MAGIC; }

// One row by one CTA of 256 threads (y may be x).
__device__ __forceinline__ void rmsnorm_row(float* yr, const float* xr, const float* __restrict__ w, uint64_t n, float eps,
                                            double* s_part, float* s_inv) {
    double ss = 0.0;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const double v = double(xr[i]);
        ss = __dadd_rn(ss, __dmul_rn(v, v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (unsigned i = 0; i < (blockDim.x >> 5); ++i) t += s_part[i];
        *s_inv = float(1.0 / sqrt(t / double(n) + double(eps)));
    }
    __syncthreads();
    const float inv = *s_inv;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __fmul_rn(xr[i], inv);
        yr[i] = w ? __fmul_rn(v, w[i]) : v;
    }
}

__global__ void __launch_bounds__(256) k_rmsnorm(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w, uint64_t n,
                                                 float eps) {
    bhd_wait_for_prior_kernels();
    __shared__ double s_part[8];
    __shared__ float s_inv;
    rmsnorm_row(y + blockIdx.x * n, x + blockIdx.x * n, w, n, eps, s_part, &s_inv);
}

// What a decode step does to the new position's query, key and value heads between the projections and attention, in one
// launch instead of six: per-head RMSNorm of q and k (k_rmsnorm's arithmetic), rope with the table row of position
// *pos_dev (k_rope's arithmetic), and the key and value rows appended to their caches at that position. One CTA per head
// vector: n_heads query heads, n_kv_heads key heads, n_kv_heads value heads.
__global__ void __launch_bounds__(256) k_qk_norm_rope_store(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                                                            const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                                            const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                                            float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                            const int32_t* __restrict__ pos_dev, uint32_t max_positions, uint32_t n_heads,
                                                            uint32_t n_kv_heads, uint32_t head_dim, float eps, int layout,
                                                            uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    __shared__ double s_part[8];
    __shared__ float s_inv;
    const int32_t pos = *pos_dev;
    if (pos < 0 || uint32_t(pos) >= max_positions) {
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
        return;
    }
    const uint32_t c = blockIdx.x;
    const uint64_t cache_row = uint64_t(pos) * n_kv_heads * head_dim;
    if (c >= n_heads + n_kv_heads) {   // a value head: copy
        const uint32_t j = c - n_heads - n_kv_heads;
        for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) v_cache[cache_row + uint64_t(j) * head_dim + i] = v[uint64_t(j) * head_dim + i];
        return;
    }
    const bool is_q = c < n_heads;
    float* xv = is_q ? q + uint64_t(c) * head_dim : k + uint64_t(c - n_heads) * head_dim;
    rmsnorm_row(xv, xv, is_q ? q_norm : k_norm, head_dim, eps, s_part, &s_inv);
    __syncthreads();
    const uint32_t n_pairs = head_dim / 2;
    float a = 0.f, b = 0.f;
    const uint32_t i = threadIdx.x;
    const uint32_t ia = layout == 0 ? 2 * i : i, ib = layout == 0 ? 2 * i + 1 : i + n_pairs;
    if (i < n_pairs) {   // head_dim <= 512: one pair per thread
        const float x0 = xv[ia], x1 = xv[ib];
        const float cs = cos_table[uint64_t(pos) * n_pairs + i], sn = sin_table[uint64_t(pos) * n_pairs + i];
        a = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        b = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        xv[ia] = a;
        xv[ib] = b;
        if (!is_q) {
            float* kc = k_cache + cache_row + uint64_t(c - n_heads) * head_dim;
            kc[ia] = a;
            kc[ib] = b;
        }
    }
}

// x [n_positions][vectors_per_position][2 * n_pairs]; cos / sin [n_positions][n_pairs].
// With pos_dev, the first position's table row is read from device memory (a decode step replayed as a CUDA graph).
__global__ void k_rope(float* __restrict__ x, const float* __restrict__ cos, const float* __restrict__ sin, uint64_t n_vectors,
                       uint32_t vectors_per_position, uint32_t n_pairs, int layout, int inverse, const int32_t* __restrict__ pos_dev) {
    bhd_wait_for_prior_kernels();
    const uint64_t idx = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (idx >= n_vectors * n_pairs) return;
    const uint64_t vec = idx / n_pairs, i = idx - vec * n_pairs, pos = vec / vectors_per_position + (pos_dev ? uint64_t(*pos_dev) : 0ull);
    float* xv = x + vec * 2 * n_pairs;
    const uint64_t ia = layout == 0 ? 2 * i : i, ib = layout == 0 ? 2 * i + 1 : i + n_pairs;
    const float a = xv[ia], b = xv[ib];
    const float c = cos[pos * n_pairs + i], s = inverse ? -sin[pos * n_pairs + i] : sin[pos * n_pairs + i];
    xv[ia] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    xv[ib] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}

// One CTA per (query position, head). scores in shared memory (f32, one per visible key position).
__global__ void __launch_bounds__(128) k_attention(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k_cache,
                                                   const float* __restrict__ v_cache, uint32_t query_start, uint32_t n_heads,
                                                   uint32_t n_kv_heads, uint32_t head_dim, float scale, const int32_t* __restrict__ start_dev,
                                                   uint32_t max_positions, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    extern __shared__ float scores[];
    __shared__ float s_max, s_inv;
    const uint32_t qp = blockIdx.x, head = blockIdx.y, kv_head = head / (n_heads / n_kv_heads);
    if (start_dev) {  // the query's position is read from device memory; the score buffer holds max_positions entries
        const int32_t sd = *start_dev;
        if (sd < 0 || uint32_t(sd) + qp >= max_positions) {
            if (threadIdx.x == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
            return;
        }
        query_start = uint32_t(sd);
    }
    const uint32_t visible = query_start + qp + 1;
    const float* query = q + (uint64_t(qp) * n_heads + head) * head_dim;
    // scores: f64 dot product in element order, scaled in f64, rounded to f32
    for (uint32_t kp = threadIdx.x; kp < visible; kp += blockDim.x) {
        const float* key = k_cache + (uint64_t(kp) * n_kv_heads + kv_head) * head_dim;
        double dot = 0.0;
        for (uint32_t d = 0; d < head_dim; ++d) dot = __dadd_rn(dot, __dmul_rn(double(query[d]), double(key[d])));
        scores[kp] = float(__dmul_rn(dot, double(scale)));
    }
    __syncthreads();
    // softmax as vecops::softmax: max, exp(v - max) (0 for -inf), sequential f32 sum, multiply by 1 / sum
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (uint32_t i = threadIdx.x; i < visible; i += 32) m = fmaxf(m, scores[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) s_max = m;
    }
    __syncthreads();
    const float m = s_max;
    const bool all_masked = !isfinite(m);
    for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) {
        const float v = scores[i];
        scores[i] = all_masked ? 0.0f : (isfinite(v) ? bhd_expf_exact(__fsub_rn(v, m)) : 0.0f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t i = 0; i < visible; ++i) sum = __fadd_rn(sum, scores[i]);
        s_inv = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    if (!all_masked) {
        const float inv = s_inv;
        for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) scores[i] = __fmul_rn(scores[i], inv);
    }
    __syncthreads();
    // values: per output dimension an f64 sum over the visible positions, in position order
    float* o = out + (uint64_t(qp) * n_heads + head) * head_dim;
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        double sum = 0.0;
        for (uint32_t vp = 0; vp < visible; ++vp)
            sum = __dadd_rn(sum, __dmul_rn(double(scores[vp]), double(v_cache[(uint64_t(vp) * n_kv_heads + kv_head) * head_dim + d])));
        o[d] = float(sum);
    }
}

// The f64 with the value of f, without the conversion unit (16 lanes per clock and SM, a quarter of the FP64 pipe's rate: with
// one conversion per operand in front of every multiply-add it was 54 % busy in the block kernel below and a third of that
// kernel's instructions): re-biased exponent and shifted mantissa for normal numbers and zeros; subnormals, infinities and
// NaNs take the instruction. For staging loops, not for use inside a dependent chain (its branch splits the schedule).
__device__ __forceinline__ double f32_to_f64(float f) {
    const uint32_t b = __float_as_uint(f), e = b & 0x7f800000u;
    if (e == 0u || e == 0x7f800000u) {
        if ((b << 1) == 0u) return __hiloint2double(int(b), 0);
        return double(f);
    }
    return __hiloint2double(int((b & 0x80000000u) | (((b & 0x7fffffffu) >> 3) + 0x38000000u)), int(b << 29));
}

// The same arithmetic in the same order, arranged so that memory latency stays off the dependent f64 chains (a decode
// step has only one CTA per head, so nothing else hides it): 256 threads; a thread forms the dot products of its keys
// from 16-byte loads, one 32-element batch ahead of the chain; the value rows are staged through shared memory in tiles
// of 8192 floats, the next tile's loads in flight (in registers) while thread d runs the position-ordered chain of
// output dimension d over the current tile. head_dim a multiple of 4, 32..256.
constexpr int ATT_THREADS = 256, ATT_TILE_FLOATS = 8192;
__global__ void __launch_bounds__(ATT_THREADS) k_attention_tiled(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                 const float* __restrict__ v_cache, uint32_t query_start, uint32_t n_heads,
                                                                 uint32_t n_kv_heads, uint32_t head_dim, float scale,
                                                                 const int32_t* __restrict__ start_dev, uint32_t max_positions,
                                                                 uint32_t score_slots, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    extern __shared__ __align__(16) float att_smem[];
    __shared__ float s_max, s_inv;
    const uint32_t qp = blockIdx.x, head = blockIdx.y, kv_head = head / (n_heads / n_kv_heads);
    if (start_dev) {
        const int32_t sd = *start_dev;
        if (sd < 0 || uint32_t(sd) + qp >= max_positions) {
            if (threadIdx.x == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
            return;
        }
        query_start = uint32_t(sd);
    }
    const uint32_t visible = query_start + qp + 1;
    float* tile = att_smem;                                              // ATT_TILE_FLOATS
    double* qd = reinterpret_cast<double*>(att_smem + ATT_TILE_FLOATS);  // head_dim: the query, widened once
    double* pd = qd + head_dim;                                          // one per visible position: the probabilities, widened once
    float* scores = reinterpret_cast<float*>(pd + score_slots);          // one per visible position
    const float* query = q + (uint64_t(qp) * n_heads + head) * head_dim;
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) qd[d] = f32_to_f64(query[d]);
    __syncthreads();
    const uint64_t row_stride = uint64_t(n_kv_heads) * head_dim;
    // scores: f64 dot product in element order, scaled in f64, rounded to f32
    for (uint32_t kp = threadIdx.x; kp < visible; kp += blockDim.x) {
        const float4* key = reinterpret_cast<const float4*>(k_cache + uint64_t(kp) * row_stride + uint64_t(kv_head) * head_dim);
        double dot = 0.0;
        float4 cur[8], nxt[8];
        const uint32_t n4 = head_dim / 4;
#pragma unroll
        for (int j = 0; j < 8; ++j) cur[j] = j < int(n4) ? key[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t b0 = 0; b0 < n4; b0 += 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) nxt[j] = (b0 + 8 + j < n4) ? key[b0 + 8 + j] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (b0 + j < n4) {
                    const double2 qa = *reinterpret_cast<const double2*>(qd + 4 * (b0 + j)), qb = *reinterpret_cast<const double2*>(qd + 4 * (b0 + j) + 2);
                    dot = __dadd_rn(dot, __dmul_rn(qa.x, double(cur[j].x)));
                    dot = __dadd_rn(dot, __dmul_rn(qa.y, double(cur[j].y)));
                    dot = __dadd_rn(dot, __dmul_rn(qb.x, double(cur[j].z)));
                    dot = __dadd_rn(dot, __dmul_rn(qb.y, double(cur[j].w)));
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
        }
        scores[kp] = float(__dmul_rn(dot, double(scale)));
    }
    __syncthreads();
    // softmax as vecops::softmax: max, exp(v - max) (0 for -inf), sequential f32 sum, multiply by 1 / sum
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (uint32_t i = threadIdx.x; i < visible; i += 32) m = fmaxf(m, scores[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) s_max = m;
    }
    __syncthreads();
    const float m = s_max;
    const bool all_masked = !isfinite(m);
    for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) {
        const float v = scores[i];
        scores[i] = all_masked ? 0.0f : (isfinite(v) ? bhd_expf_exact(__fsub_rn(v, m)) : 0.0f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        uint32_t i = 0;
        for (; i + 8 <= visible; i += 8) {
            float e[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = scores[i + j];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum = __fadd_rn(sum, e[j]);
        }
        for (; i < visible; ++i) sum = __fadd_rn(sum, scores[i]);
        s_inv = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    {
        const float inv = s_inv;
        for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) pd[i] = f32_to_f64(all_masked ? scores[i] : __fmul_rn(scores[i], inv));
    }
    __syncthreads();
    // values: per output dimension an f64 sum over the visible positions, in position order
    const uint32_t tp = ATT_TILE_FLOATS / head_dim;              // positions per tile
    const uint32_t per_thread = ATT_TILE_FLOATS / 4 / ATT_THREADS;  // float4 per thread per tile: 8
    const uint32_t row4 = head_dim / 4;
    float4 stage[ATT_TILE_FLOATS / 4 / ATT_THREADS];
    auto fetch = [&](uint32_t p0) {   // tile of positions p0 .. p0 + tp into registers (rows beyond `visible` are not read)
#pragma unroll
        for (uint32_t j = 0; j < per_thread; ++j) {
            const uint32_t idx = threadIdx.x + j * ATT_THREADS, pr = idx / row4, c4 = idx - pr * row4;
            stage[j] = (p0 + pr < visible) ? reinterpret_cast<const float4*>(v_cache + uint64_t(p0 + pr) * row_stride + uint64_t(kv_head) * head_dim)[c4]
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    double sum = 0.0;
    fetch(0);
    for (uint32_t p0 = 0; p0 < visible; p0 += tp) {
#pragma unroll
        for (uint32_t j = 0; j < per_thread; ++j) reinterpret_cast<float4*>(tile)[threadIdx.x + j * ATT_THREADS] = stage[j];
        __syncthreads();
        if (p0 + tp < visible) fetch(p0 + tp);       // in flight while the chain below runs
        if (threadIdx.x < head_dim) {
            const uint32_t n = min(tp, visible - p0);
            uint32_t pr = 0;
            for (; pr + 8 <= n; pr += 8) {   // the eight products do not depend on the chain: formed ahead of it
                double prod[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) prod[j] = __dmul_rn(pd[p0 + pr + j], double(tile[(pr + j) * head_dim + threadIdx.x]));
#pragma unroll
                for (int j = 0; j < 8; ++j) sum = __dadd_rn(sum, prod[j]);
            }
            for (; pr < n; ++pr) sum = __dadd_rn(sum, __dmul_rn(pd[p0 + pr], double(tile[pr * head_dim + threadIdx.x])));
        }
        __syncthreads();
    }
    if (threadIdx.x < head_dim) out[(uint64_t(qp) * n_heads + head) * head_dim + threadIdx.x] = float(sum);
}

// Decode form (one query position, head_dim 128): a cluster of four CTAs per head, because a decode step has only one CTA's
// worth of work per head in the kernel above and leaves most SMs idle while its thread-per-key reads of the cache wait on
// memory. Same sums, same order:
//   scores  CTA r of the cluster takes the r-th quarter of the visible keys, in tiles of 128 keys copied asynchronously
//           (16-byte cp.async, coalesced, two tiles in flight) into padded shared-memory rows; a thread runs the element-ordered
//           chain of one key, the 256 threads covering two tiles a pass. Every score is stored into all four CTAs' score arrays through distributed shared
//           memory; one cluster barrier.
//   softmax by every CTA for itself (the same operations on the same values: the same bits).
//   values  CTA r owns output dimensions 32r .. 32r + 31: warp 0 runs their position-ordered chains over tiles of 128
//           positions x 32 dimensions, which all threads keep copying one tile ahead (the first two during the score phase).
constexpr int AD_THREADS = 256, AD_CLUSTER = 4, AD_HD = 128, AD_KT = 128, AD_KROW = AD_HD + 4, AD_VT = 128, AD_VD = AD_HD / AD_CLUSTER;
__host__ __device__ constexpr size_t attention_decode_smem(uint32_t score_slots) {
    return 2 * size_t(AD_KT) * AD_KROW * sizeof(float) + 2 * size_t(AD_VT) * AD_VD * sizeof(float) + size_t(AD_HD) * sizeof(double) +
           size_t(score_slots) * (sizeof(double) + sizeof(float)) + 16;
}
__device__ __forceinline__ uint32_t ad_smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ad_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ad_smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ad_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ad_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__global__ void __launch_bounds__(AD_THREADS) k_attention_decode4(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                  const float* __restrict__ v_cache, uint32_t query_start, uint32_t n_heads,
                                                                  uint32_t n_kv_heads, float scale, const int32_t* __restrict__ start_dev,
                                                                  uint32_t max_positions, uint32_t score_slots, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    extern __shared__ __align__(16) uint8_t ad_smem[];
    __shared__ float s_max, s_inv;
    float* kbuf = reinterpret_cast<float*>(ad_smem);                                   // [2][128 keys][132]
    float* vbuf = kbuf + 2 * AD_KT * AD_KROW;                                          // [2][128 positions][32]
    double* qd = reinterpret_cast<double*>(vbuf + 2 * AD_VT * AD_VD);                  // [128]
    double* pd = qd + AD_HD;                                                           // [score_slots]
    float* scores = reinterpret_cast<float*>(pd + score_slots);                        // [score_slots]
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const uint32_t head = blockIdx.y, kv_head = head / (n_heads / n_kv_heads);
    if (start_dev) {   // the same value in all four CTAs: they leave together, before any cluster barrier
        const int32_t sd = *start_dev;
        if (sd < 0 || uint32_t(sd) >= max_positions) {
            if (threadIdx.x == 0 && rank == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
            return;
        }
        query_start = uint32_t(sd);
    }
    // every CTA of the cluster must be running before a peer stores into its shared memory: arrive now, wait before the stores
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const uint32_t visible = query_start + 1;
    const uint64_t row_stride = uint64_t(n_kv_heads) * AD_HD;
    const float* kbase = k_cache + uint64_t(kv_head) * AD_HD;
    const float* vbase = v_cache + uint64_t(kv_head) * AD_HD + rank * AD_VD;
    const uint32_t kq = (visible + AD_CLUSTER - 1) / AD_CLUSTER, k0 = min(visible, rank * kq), k1 = min(visible, k0 + kq);   // this CTA's keys
    const uint32_t k_tiles = (k1 - k0 + AD_KT - 1) / AD_KT, v_tiles = (visible + AD_VT - 1) / AD_VT;
    auto copy_k = [&](uint32_t t) {   // keys k0 + 128 t .. of this CTA into buffer t & 1 (one commit group, possibly empty)
        float* dst = kbuf + (t & 1) * AD_KT * AD_KROW;
        const uint32_t base = k0 + t * AD_KT;
#pragma unroll 4
        for (uint32_t i = 0; i < AD_KT * (AD_HD / 4) / AD_THREADS; ++i) {
            const uint32_t c = threadIdx.x + i * AD_THREADS, key = c >> 5, part = c & 31;
            if (t < k_tiles && base + key < k1) ad_cp16(dst + key * AD_KROW + 4 * part, kbase + uint64_t(base + key) * row_stride + 4 * part);
        }
        ad_commit();
    };
    auto copy_v = [&](uint32_t t) {   // positions 128 t .. x this CTA's 32 dimensions into buffer t & 1
        float* dst = vbuf + (t & 1) * AD_VT * AD_VD;
#pragma unroll
        for (uint32_t i = 0; i < AD_VT * (AD_VD / 4) / AD_THREADS; ++i) {
            const uint32_t c = threadIdx.x + i * AD_THREADS, pos = c >> 3, part = c & 7;
            if (t < v_tiles && t * AD_VT + pos < visible) ad_cp16(dst + pos * AD_VD + 4 * part, vbase + uint64_t(t * AD_VT + pos) * row_stride + 4 * part);
        }
        ad_commit();
    };
    // groups in flight, oldest first: K0, K1, V0, V1
    copy_k(0);
    copy_k(1);
    copy_v(0);
    copy_v(1);
    const float* query = q + uint64_t(head) * AD_HD;
    if (threadIdx.x < AD_HD) qd[threadIdx.x] = f32_to_f64(query[threadIdx.x]);
    // ---- scores of this CTA's keys ----
    uint32_t peer_scores[AD_CLUSTER];
#pragma unroll
    for (uint32_t r = 0; r < AD_CLUSTER; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_scores[r]) : "r"(ad_smem_u32(scores)), "r"(r));
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    for (uint32_t tp = 0; tp < k_tiles; tp += 2) {   // two tiles a pass: threads 0..127 on the even tile, 128..255 on the odd one
        // first pass: the two groups behind the pair (V0, V1) may still be in flight; later passes: the pair is the newest
        if (tp == 0) ad_wait_group<2>(); else ad_wait_group<0>();
        __syncthreads();
        const uint32_t t = tp + (threadIdx.x >> 7), krow_i = threadIdx.x & (AD_KT - 1);
        const uint32_t kp = k0 + t * AD_KT + krow_i;
        if (t < k_tiles && kp < k1) {
            const float4* key = reinterpret_cast<const float4*>(kbuf + (t & 1) * AD_KT * AD_KROW + krow_i * AD_KROW);
            double dot = 0.0;
#pragma unroll 2
            for (uint32_t b0 = 0; b0 < AD_HD / 4; b0 += 8) {
                double prod[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 kf = key[b0 + j];
                    const double2 qa = *reinterpret_cast<const double2*>(qd + 4 * (b0 + j)), qb = *reinterpret_cast<const double2*>(qd + 4 * (b0 + j) + 2);
                    prod[4 * j] = __dmul_rn(qa.x, double(kf.x));
                    prod[4 * j + 1] = __dmul_rn(qa.y, double(kf.y));
                    prod[4 * j + 2] = __dmul_rn(qb.x, double(kf.z));
                    prod[4 * j + 3] = __dmul_rn(qb.y, double(kf.w));
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) dot = __dadd_rn(dot, prod[j]);
            }
            const float sc = float(__dmul_rn(dot, double(scale)));
#pragma unroll
            for (uint32_t r = 0; r < AD_CLUSTER; ++r)
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer_scores[r] + 4u * kp), "f"(sc) : "memory");
        }
        __syncthreads();                       // the buffers' readers are done
        copy_k(tp + 2);                        // one group each, empty beyond the last tile
        copy_k(tp + 3);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // ---- softmax (vecops::softmax: max, exp(v - max) (0 for -inf), sequential f32 sum, multiply by 1 / sum) ----
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (uint32_t i = threadIdx.x; i < visible; i += 32) m = fmaxf(m, scores[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) s_max = m;
    }
    __syncthreads();
    const float m = s_max;
    const bool all_masked = !isfinite(m);
    for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) {
        const float v = scores[i];
        scores[i] = all_masked ? 0.0f : (isfinite(v) ? bhd_expf_exact(__fsub_rn(v, m)) : 0.0f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        uint32_t i = 0;
        for (; i + 8 <= visible; i += 8) {
            float e[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = scores[i + j];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum = __fadd_rn(sum, e[j]);
        }
        for (; i < visible; ++i) sum = __fadd_rn(sum, scores[i]);
        s_inv = __fdiv_rn(1.0f, sum);
    }
    __syncthreads();
    {
        const float inv = s_inv;
        for (uint32_t i = threadIdx.x; i < visible; i += blockDim.x) pd[i] = f32_to_f64(all_masked ? scores[i] : __fmul_rn(scores[i], inv));
    }
    // ---- values: warp 0, lane = output dimension 32 rank + lane ----
    double sum = 0.0;
    for (uint32_t t = 0; t < v_tiles; ++t) {
        ad_wait_group<1>();                    // all but the newest group: tile t has landed
        __syncthreads();                       // ... for every thread's copies (first pass: pd is complete)
        if (threadIdx.x < 32) {
            const float* vt = vbuf + (t & 1) * AD_VT * AD_VD + threadIdx.x;
            const uint32_t p0 = t * AD_VT, n = min(uint32_t(AD_VT), visible - p0);
            uint32_t pr = 0;
            for (; pr + 8 <= n; pr += 8) {   // the eight products do not depend on the chain: formed ahead of it
                double prod[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) prod[j] = __dmul_rn(pd[p0 + pr + j], double(vt[(pr + j) * AD_VD]));
#pragma unroll
                for (int j = 0; j < 8; ++j) sum = __dadd_rn(sum, prod[j]);
            }
            for (; pr < n; ++pr) sum = __dadd_rn(sum, __dmul_rn(pd[p0 + pr], double(vt[pr * AD_VD])));
        }
        __syncthreads();
        if (t + 2 < v_tiles) copy_v(t + 2); else ad_commit();
    }
    ad_wait_group<0>();
    if (threadIdx.x < 32) out[uint64_t(head) * AD_HD + rank * AD_VD + threadIdx.x] = float(sum);
    // no CTA may leave while a peer can still store scores into it: all stores precede the barrier above
}

// Prefill form (head_dim 128, several query positions): the same sums in the same order, with the keys and values of a
// kv head read once for a block of queries instead of once per (query, head). A CTA owns 32 (query, head) pairs: the G
// query heads of one kv head for 32 / G consecutive positions; warp w owns pairs 4w .. 4w + 3. Keys and values pass through
// shared memory in tiles of 32 positions (the next tile's loads in flight in registers), **as f64**: every element is
// widened once per tile, with integer operations (f32_to_f64), instead of once per use inside the chains.
//   scores  tiles of 64 keys, a lane takes keys lane and lane + 32: eight chains a lane (its keys against the warp's four
//           queries, which sit in shared memory as f64 and are read as broadcasts). One fused multiply-add per element: the product of two f32 values is exact in
//           f64, so fma(q, k, dot) rounds once, to the same value as the reference's add of the product.
//   softmax per pair by its warp: max, exact exp, the sequential f32 sum by one lane per pair, 1 / sum.
//   values  lane = output dimensions lane, lane + 32, lane + 64, lane + 96: sixteen chains a lane over the positions in order;
//           the tile's probabilities are widened once per warp into a small f64 table.
// Blocks of late queries (the long ones) are scheduled first. The scores of the block's pairs sit in shared memory while they
// fit (about 760 positions); for longer caches (SCRATCH) the CTAs are persistent, take (query block, kv head) items
// round-robin and keep their scores in a row per pair of a device-memory scratch area (each warp's own rows: they stay in L2).
constexpr int AB_THREADS = 256, AB_PAIRS = 32, AB_TILE = 32, AB_KTILE = 64, AB_HD = 128, AB_KSTRIDE = AB_HD + 2;   // in doubles: rows 1040 bytes apart
__host__ __device__ constexpr size_t attention_block_smem(uint32_t score_stride) {
    return size_t(AB_PAIRS) * AB_HD * sizeof(double) + size_t(AB_KTILE) * AB_KSTRIDE * sizeof(double) + size_t(AB_PAIRS) * AB_TILE * sizeof(double) +
           size_t(AB_PAIRS) * score_stride * sizeof(float);
}
template <bool SCRATCH>
__global__ void __launch_bounds__(AB_THREADS) k_attention_block(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                const float* __restrict__ v_cache, uint32_t query_start, uint32_t n_query,
                                                                uint32_t n_heads, uint32_t n_kv_heads, float scale, uint32_t score_stride,
                                                                float* __restrict__ scratch) {
    bhd_wait_for_prior_kernels();
    extern __shared__ __align__(16) uint8_t ab_smem[];
    double* qs = reinterpret_cast<double*>(ab_smem);             // [32 pairs][128]
    double* tile = qs + AB_PAIRS * AB_HD;                        // [64 keys][130] or [32 positions][128] (values)
    double* pt = tile + AB_KTILE * AB_KSTRIDE;                   // [32 pairs][32 positions]: the tile's probabilities
    float* scores = SCRATCH ? scratch + uint64_t(blockIdx.x) * AB_PAIRS * score_stride   // [32 pairs][score_stride], this CTA's own
                            : reinterpret_cast<float*>(pt + AB_PAIRS * AB_TILE);
    const uint32_t G = n_heads / n_kv_heads, QB = AB_PAIRS / G, q_blocks = (n_query + QB - 1) / QB, n_items = q_blocks * n_kv_heads;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x) {   // one item per CTA unless SCRATCH
    const uint32_t kv_head = item % n_kv_heads, q0 = (q_blocks - 1 - item / n_kv_heads) * QB;
    const uint32_t n_here = min(QB, n_query - q0);            // queries of this block
    const uint32_t max_vis = query_start + q0 + n_here;       // positions the block's last query sees
    const uint64_t row_stride = uint64_t(n_kv_heads) * AB_HD;
    // pair pi = (query q0 + pi / G, head kv_head * G + pi % G)
    for (uint32_t i = threadIdx.x; i < AB_PAIRS * AB_HD; i += AB_THREADS) {
        const uint32_t pi = i / AB_HD, d = i - pi * AB_HD, qi = pi / G;
        qs[i] = qi < n_here ? f32_to_f64(q[(uint64_t(q0 + qi) * n_heads + kv_head * G + (pi - qi * G)) * AB_HD + d]) : 0.0;
    }
    uint32_t vis[4];   // visible positions of the warp's pairs (0: no such query)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t qi = (4 * warp + j) / G;
        vis[j] = qi < n_here ? query_start + q0 + qi + 1 : 0u;
    }
    float4 stage[4];
    auto fetch = [&](const float* cache, uint32_t p0) {   // rows p0 .. p0 + 31 of this kv head; rows from max_vis on are not read
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t idx = threadIdx.x + j * AB_THREADS, r = idx >> 5, c4 = idx & 31;
            stage[j] = (p0 + r < max_vis) ? reinterpret_cast<const float4*>(cache + uint64_t(p0 + r) * row_stride + uint64_t(kv_head) * AB_HD)[c4]
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto put = [&](uint32_t stride) {   // widened
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t idx = threadIdx.x + j * AB_THREADS, r = idx >> 5, c4 = idx & 31;
            double2* dst = reinterpret_cast<double2*>(tile + r * stride + 4 * c4);
            dst[0] = make_double2(f32_to_f64(stage[j].x), f32_to_f64(stage[j].y));
            dst[1] = make_double2(f32_to_f64(stage[j].z), f32_to_f64(stage[j].w));
        }
    };
    // ---- scores: tiles of 64 keys, a lane takes keys lane and lane + 32 of the tile (eight chains, and every broadcast
    // query read serves two keys) ----
    float4 kstage[8];
    auto fetch_keys = [&](uint32_t p0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t idx = threadIdx.x + j * AB_THREADS, r = idx >> 5, c4 = idx & 31;
            kstage[j] = (p0 + r < max_vis) ? reinterpret_cast<const float4*>(k_cache + uint64_t(p0 + r) * row_stride + uint64_t(kv_head) * AB_HD)[c4]
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto put_keys = [&]() {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t idx = threadIdx.x + j * AB_THREADS, r = idx >> 5, c4 = idx & 31;
            double2* dst = reinterpret_cast<double2*>(tile + r * AB_KSTRIDE + 4 * c4);
            dst[0] = make_double2(f32_to_f64(kstage[j].x), f32_to_f64(kstage[j].y));
            dst[1] = make_double2(f32_to_f64(kstage[j].z), f32_to_f64(kstage[j].w));
        }
    };
    fetch_keys(0);
    for (uint32_t p0 = 0; p0 < max_vis; p0 += AB_KTILE) {
        __syncthreads();                     // the tile's previous readers are done (first pass: qs is complete)
        put_keys();
        __syncthreads();
        if (p0 + AB_KTILE < max_vis) fetch_keys(p0 + AB_KTILE);
        const double* krow0 = tile + lane * AB_KSTRIDE;
        const double* krow1 = krow0 + 32 * AB_KSTRIDE;
        double dot[2][4] = {{0.0, 0.0, 0.0, 0.0}, {0.0, 0.0, 0.0, 0.0}};
#pragma unroll 4
        for (uint32_t d4 = 0; d4 < AB_HD / 4; ++d4) {
            const double2 ka0 = *reinterpret_cast<const double2*>(krow0 + 4 * d4), kb0 = *reinterpret_cast<const double2*>(krow0 + 4 * d4 + 2);
            const double2 ka1 = *reinterpret_cast<const double2*>(krow1 + 4 * d4), kb1 = *reinterpret_cast<const double2*>(krow1 + 4 * d4 + 2);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const double2* qq = reinterpret_cast<const double2*>(qs + (4 * warp + j) * AB_HD + 4 * d4);
                const double2 a = qq[0], b = qq[1];
                dot[0][j] = __fma_rn(a.x, ka0.x, dot[0][j]);
                dot[1][j] = __fma_rn(a.x, ka1.x, dot[1][j]);
                dot[0][j] = __fma_rn(a.y, ka0.y, dot[0][j]);
                dot[1][j] = __fma_rn(a.y, ka1.y, dot[1][j]);
                dot[0][j] = __fma_rn(b.x, kb0.x, dot[0][j]);
                dot[1][j] = __fma_rn(b.x, kb1.x, dot[1][j]);
                dot[0][j] = __fma_rn(b.y, kb0.y, dot[0][j]);
                dot[1][j] = __fma_rn(b.y, kb1.y, dot[1][j]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t kp = p0 + 32 * h + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (kp < vis[j]) scores[(4 * warp + j) * score_stride + kp] = float(__dmul_rn(dot[h][j], double(scale)));
        }
    }
    __syncwarp();
    // ---- softmax of the warp's four pairs (vecops::softmax: max, exp(v - max), sequential f32 sum, times 1 / sum) ----
    bool scaled[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float* sc = scores + (4 * warp + j) * score_stride;
        const uint32_t n = vis[j];
        float m = -INFINITY;
        for (uint32_t i = lane; i < n; i += 32) m = fmaxf(m, sc[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const bool all_masked = !isfinite(m);
        scaled[j] = !all_masked;             // a row without a finite maximum stays all zero (no multiplication by 1 / 0)
        for (uint32_t i = lane; i < n; i += 32) {
            const float v = sc[i];
            sc[i] = all_masked ? 0.0f : (isfinite(v) ? bhd_expf_exact(__fsub_rn(v, m)) : 0.0f);
        }
    }
    __syncwarp();
    float inv = 0.0f;
    if (lane < 4) {   // lane j adds pair j's terms in position order
        const float* sc = scores + (4 * warp + lane) * score_stride;
        const uint32_t n = lane == 0 ? vis[0] : (lane == 1 ? vis[1] : (lane == 2 ? vis[2] : vis[3]));
        float sum = 0.0f;
        uint32_t i = 0;
        for (; i + 8 <= n; i += 8) {
            float e[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) e[t] = sc[i + t];
#pragma unroll
            for (int t = 0; t < 8; ++t) sum = __fadd_rn(sum, e[t]);
        }
        for (; i < n; ++i) sum = __fadd_rn(sum, sc[i]);
        inv = __fdiv_rn(1.0f, sum);
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float* sc = scores + (4 * warp + j) * score_stride;
        const float inv_j = __shfl_sync(0xffffffffu, inv, j);
        if (scaled[j])
            for (uint32_t i = lane; i < vis[j]; i += 32) sc[i] = __fmul_rn(sc[i], inv_j);
    }
    __syncwarp();
    // ---- values ----
    double acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.0;
    fetch(v_cache, 0);
    for (uint32_t p0 = 0; p0 < max_vis; p0 += AB_TILE) {
        __syncthreads();
        put(AB_HD);
#pragma unroll
        for (int j = 0; j < 4; ++j)   // the warp's own rows of the probability table
            pt[(4 * warp + j) * AB_TILE + lane] = (p0 + lane < vis[j]) ? f32_to_f64(scores[(4 * warp + j) * score_stride + p0 + lane]) : 0.0;
        __syncthreads();
        if (p0 + AB_TILE < max_vis) fetch(v_cache, p0 + AB_TILE);
        const uint32_t n = min(uint32_t(AB_TILE), max_vis - p0);
#pragma unroll 4
        for (uint32_t r = 0; r < n; ++r) {
            const double* vrow = tile + r * AB_HD + lane;
            const double v0 = vrow[0], v1 = vrow[32], v2 = vrow[64], v3 = vrow[96];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (p0 + r < vis[j]) {   // uniform in the warp; a position a query does not see adds nothing, whatever its values
                    const double pj = pt[(4 * warp + j) * AB_TILE + r];
                    acc[j][0] = __fma_rn(pj, v0, acc[j][0]);
                    acc[j][1] = __fma_rn(pj, v1, acc[j][1]);
                    acc[j][2] = __fma_rn(pj, v2, acc[j][2]);
                    acc[j][3] = __fma_rn(pj, v3, acc[j][3]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t pi = 4 * warp + j, qi = pi / G;
        if (qi < n_here) {
            float* o = out + (uint64_t(q0 + qi) * n_heads + kv_head * G + (pi - qi * G)) * AB_HD;
#pragma unroll
            for (int c = 0; c < 4; ++c) o[lane + 32 * c] = float(acc[j][c]);
        }
    }
    }   // items
}

// Launches the tiled kernel when the head shape allows, else the plain one. `score_slots` bounds the visible positions.
static int32_t launch_attention(bhd_ctx* ctx, float* out, const float* q, const float* k, const float* v, uint32_t n_query, uint32_t query_start,
                                uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, float scale, const int32_t* start_dev,
                                uint32_t max_positions, uint64_t score_slots, cudaStream_t s) {
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_attention, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_attention_tiled, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "raising the shared memory limit");
        once.mark(ctx);
    }
    const bool aligned = ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    // several query positions of 128-wide heads: blocks of queries that share the keys and values of their kv head
    const uint32_t group = n_heads / n_kv_heads, score_stride = uint32_t((score_slots + 3) / 4 * 4);
    if (!start_dev && n_query >= 8 && head_dim == AB_HD && aligned && group <= 32 && (group & (group - 1)) == 0) {
        static bhd_once_per_device once_block;
        static int per_sm[BHD_MAX_DEVICES] = {};
        const size_t smem_scratch = attention_block_smem(0);
        if (once_block.pending(ctx)) {
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_attention_block<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "raising the shared memory limit");
            BHD_CUDA(ctx, cudaFuncSetAttribute(k_attention_block<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_scratch)), "raising the shared memory limit");
            BHD_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm[ctx->device], k_attention_block<true>, AB_THREADS, smem_scratch), "querying occupancy");
            once_block.mark(ctx);
        }
        const uint32_t qb = AB_PAIRS / group, n_items = (n_query + qb - 1) / qb * n_kv_heads;
        if (attention_block_smem(score_stride) <= 200 * 1024) {
            bhd_launch_dependent(ctx, k_attention_block<false>, dim3(n_items), dim3(AB_THREADS), attention_block_smem(score_stride), s, out, q, k, v,
                                 query_start, n_query, n_heads, n_kv_heads, scale, score_stride, static_cast<float*>(nullptr));
        } else {
            const uint32_t slots = uint32_t(ctx->sm_count) * uint32_t(per_sm[ctx->device] > 0 ? per_sm[ctx->device] : 1);
            const uint32_t grid = n_items < slots ? n_items : slots;
            const int32_t st = bhd_ensure_workspace(ctx, size_t(grid) * AB_PAIRS * score_stride * sizeof(float), s);
            if (st != BHD_OK) return st;
            bhd_launch_dependent(ctx, k_attention_block<true>, dim3(grid), dim3(AB_THREADS), smem_scratch, s, out, q, k, v, query_start, n_query, n_heads,
                                 n_kv_heads, scale, score_stride, reinterpret_cast<float*>(ctx->workspace));
        }
        BHD_LAUNCHED(ctx, "attention kernel");
        return BHD_OK;
    }
    // one query position of 128-wide heads: a cluster of four CTAs per head
    static bool clusters_fit[BHD_MAX_DEVICES] = {};   // a cluster of four CTAs with the largest shared-memory size can be resident
    static bhd_once_per_device once_decode;
    if (n_query == 1 && head_dim == AD_HD && aligned && attention_decode_smem(uint32_t(score_slots)) <= 200 * 1024 && once_decode.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_attention_decode4, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "raising the shared memory limit");
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(AD_CLUSTER, 1);
        probe.blockDim = dim3(AD_THREADS);
        probe.dynamicSmemBytes = 200 * 1024;
        cudaLaunchAttribute pa[1];
        pa[0].id = cudaLaunchAttributeClusterDimension;
        pa[0].val.clusterDim.x = AD_CLUSTER;
        pa[0].val.clusterDim.y = 1;
        pa[0].val.clusterDim.z = 1;
        probe.attrs = pa;
        probe.numAttrs = 1;
        int n_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, k_attention_decode4, &probe) != cudaSuccess) {
            cudaGetLastError();
            n_clusters = 0;
        }
        clusters_fit[ctx->device] = n_clusters > 0;
        once_decode.mark(ctx);
    }
    if (n_query == 1 && head_dim == AD_HD && aligned && attention_decode_smem(uint32_t(score_slots)) <= 200 * 1024 && clusters_fit[ctx->device]) {
        const size_t dyn = attention_decode_smem(uint32_t(score_slots));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(AD_CLUSTER, n_heads);
        cfg.blockDim = dim3(AD_THREADS);
        cfg.dynamicSmemBytes = dyn;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = AD_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->plain_launches ? 1 : 2;
        BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_attention_decode4, out, q, k, v, query_start, n_heads, n_kv_heads, scale, start_dev, max_positions,
                                         uint32_t(score_slots), ctx->status_dev), "launching the attention kernel");
        ctx->launches += 1;
        return BHD_OK;
    }
    const size_t tiled_smem = size_t(ATT_TILE_FLOATS) * sizeof(float) + (size_t(head_dim) + score_slots) * sizeof(double) + score_slots * sizeof(float);
    if (aligned && head_dim % 4 == 0 && head_dim >= 32 && head_dim <= 256 && ATT_TILE_FLOATS % head_dim == 0 && tiled_smem <= 200 * 1024) {
        bhd_launch_dependent(ctx, k_attention_tiled, dim3(n_query, n_heads), dim3(ATT_THREADS), tiled_smem, s, out, q, k, v, query_start, n_heads, n_kv_heads,
                             head_dim, scale, start_dev, max_positions, uint32_t(score_slots), ctx->status_dev);
    } else {
        bhd_launch_dependent(ctx, k_attention, dim3(n_query, n_heads), dim3(128), size_t(score_slots) * sizeof(float), s, out, q, k, v, query_start, n_heads, n_kv_heads, head_dim,
                                                                                              scale, start_dev, max_positions, ctx->status_dev);
    }
    BHD_LAUNCHED(ctx, "attention kernel");
    return BHD_OK;
}

// Command::SigmoidGate (crates/beholdd-backend/src/execution.rs:1425-1441): out = in * sigmoid(gate), the sigmoid in its
// overflow-free form.
__global__ void k_sigmoid_gate(float* __restrict__ out, const float* __restrict__ in, const float* __restrict__ gate, uint64_t n) {
    bhd_wait_for_prior_kernels();
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i];
    const float tail = bhd_expf_exact(-fabsf(g));
    const float sig = g >= 0.0f ? __fdiv_rn(1.0f, __fadd_rn(1.0f, tail)) : __fdiv_rn(tail, __fadd_rn(1.0f, tail));
    out[i] = __fmul_rn(in[i], sig);
}

// dst[*pos_dev][0 .. row_floats) = src: appends one row to a cache at a position read from device memory.
__global__ void k_store_row_at(float* __restrict__ dst, const float* __restrict__ src, const int32_t* __restrict__ pos_dev, uint64_t row_floats,
                               uint64_t max_rows, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    const int32_t pos = *pos_dev;
    if (pos < 0 || uint64_t(pos) >= max_rows) {
        if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
        return;
    }
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i < row_floats) dst[uint64_t(pos) * row_floats + i] = src[i];
}

template <uint32_t KIND>
__global__ void k_embedding_rows(const uint8_t* __restrict__ w, uint64_t row_bytes, uint64_t rows, uint64_t cols, const int32_t* __restrict__ ids,
                                 float* __restrict__ out, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    const int32_t id = ids[blockIdx.x];
    if (id < 0 || uint64_t(id) >= rows) {
        if (threadIdx.x == 0) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
        return;
    }
    const uint8_t* row = w + uint64_t(id) * row_bytes;
    for (uint64_t k = threadIdx.x; k < cols; k += blockDim.x) out[blockIdx.x * cols + k] = bhd_decode_elem<KIND>(row, k);
}

}  // namespace

extern "C" int32_t bhd_rmsnorm(bhd_ctx* ctx, float* y_dev, const float* x_dev, const float* weight_dev, uint64_t n_rows, uint64_t n, float eps,
                               void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: RMSNorm input cannot be empty");
    if (!isfinite(eps) || eps < 0.0f) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: RMSNorm epsilon must be finite and non-negative, got %g", double(eps));
    if (n_rows == 0) return BHD_OK;
    if (n_rows > 0x7fffffffull) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: too many RMSNorm rows");
    if (!y_dev || !x_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rmsnorm: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_rmsnorm, dim3(unsigned(n_rows)), dim3(256), 0, cudaStream_t(stream), y_dev, x_dev, weight_dev, n, eps);
    BHD_LAUNCHED(ctx, "RMSNorm kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_rope(bhd_ctx* ctx, float* x_dev, const float* cos_dev, const float* sin_dev, uint64_t n_positions,
                            uint32_t vectors_per_position, uint32_t n_pairs, int32_t layout, int32_t inverse, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (layout != 0 && layout != 1) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rope: layout must be 0 (interleaved) or 1 (split half)");
    const uint64_t n_vectors = n_positions * vectors_per_position;
    if (n_vectors == 0 || n_pairs == 0) return BHD_OK;
    if (!x_dev || !cos_dev || !sin_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rope: null buffer");
    bhd_device_guard guard(ctx);
    const uint64_t n = n_vectors * n_pairs;
    bhd_launch_dependent(ctx, k_rope, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), x_dev, cos_dev, sin_dev, n_vectors, vectors_per_position, n_pairs, layout,
                                                                         inverse, nullptr);
    BHD_LAUNCHED(ctx, "rotary embedding kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_rope_at(bhd_ctx* ctx, float* x_dev, const float* cos_table_dev, const float* sin_table_dev, const int32_t* pos_dev,
                               uint32_t n_vectors, uint32_t n_pairs, int32_t layout, int32_t inverse, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (layout != 0 && layout != 1) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rope: layout must be 0 (interleaved) or 1 (split half)");
    if (n_vectors == 0 || n_pairs == 0) return BHD_OK;
    if (!x_dev || !cos_table_dev || !sin_table_dev || !pos_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rope: null buffer");
    bhd_device_guard guard(ctx);
    const uint64_t n = uint64_t(n_vectors) * n_pairs;
    bhd_launch_dependent(ctx, k_rope, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), x_dev, cos_table_dev, sin_table_dev, n_vectors, n_vectors, n_pairs, layout,
                                                                         inverse, pos_dev);
    BHD_LAUNCHED(ctx, "rotary embedding kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_qk_norm_rope_store_at(bhd_ctx* ctx, float* q_dev, float* k_dev, const float* v_dev, const float* q_norm_dev,
                                             const float* k_norm_dev, const float* cos_table_dev, const float* sin_table_dev, float* k_cache_dev,
                                             float* v_cache_dev, const int32_t* pos_dev, uint64_t max_positions, uint32_t n_heads,
                                             uint32_t n_kv_heads, uint32_t head_dim, float eps, int32_t layout, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (layout != 0 && layout != 1) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rope: layout must be 0 (interleaved) or 1 (split half)");
    if (n_heads == 0 || n_kv_heads == 0 || head_dim == 0 || head_dim % 2 != 0 || head_dim > 512 || max_positions == 0 || max_positions > 0x7fffffffull)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: heads=%u kv_heads=%u head_dim=%u positions=%llu", n_heads, n_kv_heads, head_dim,
                        (unsigned long long)max_positions);
    if (!isfinite(eps) || eps < 0.0f) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: RMSNorm epsilon must be finite and non-negative, got %g", double(eps));
    if (!q_dev || !k_dev || !v_dev || !cos_table_dev || !sin_table_dev || !k_cache_dev || !v_cache_dev || !pos_dev)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "qk_norm_rope_store: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_qk_norm_rope_store, dim3(n_heads + 2 * n_kv_heads), dim3(256), 0, cudaStream_t(stream), q_dev, k_dev, v_dev, q_norm_dev, k_norm_dev, cos_table_dev,
                                                                                      sin_table_dev, k_cache_dev, v_cache_dev, pos_dev,
                                                                                      uint32_t(max_positions), n_heads, n_kv_heads, head_dim, eps, layout,
                                                                                      ctx->status_dev);
    BHD_LAUNCHED(ctx, "query/key norm, rope and cache append kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_store_row_at(bhd_ctx* ctx, float* dst_dev, const float* src_dev, const int32_t* pos_dev, uint64_t row_floats,
                                    uint64_t max_rows, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (row_floats == 0) return BHD_OK;
    if (!dst_dev || !src_dev || !pos_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "store_row_at: null buffer");
    if (row_floats > (1ull << 38)) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: row too long");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_store_row_at, dim3(unsigned((row_floats + 255) / 256)), dim3(256), 0, cudaStream_t(stream), dst_dev, src_dev, pos_dev, row_floats, max_rows,
                                                                                          ctx->status_dev);
    BHD_LAUNCHED(ctx, "cache append kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_incremental_attention_at(bhd_ctx* ctx, float* out_dev, const float* q_dev, const float* k_cache_dev,
                                                const float* v_cache_dev, const int32_t* pos_dev, uint64_t max_positions, uint32_t n_heads,
                                                uint32_t n_kv_heads, uint32_t head_dim, float scale, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (max_positions == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention requires at least one cached position");
    if (n_heads == 0 || n_kv_heads == 0 || head_dim == 0 || n_heads % n_kv_heads != 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention got heads=%u kv_heads=%u head_dim=%u", n_heads, n_kv_heads, head_dim);
    if (!isfinite(scale) || scale <= 0.0f)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention scale must be positive and finite, got %g", double(scale));
    if (n_heads > 65535u || max_positions > (200u * 1024u) / 4u)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: attention over %llu positions and %u heads is beyond this kernel",
                        (unsigned long long)max_positions, n_heads);
    if (!out_dev || !q_dev || !k_cache_dev || !v_cache_dev || !pos_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "attention: null buffer");
    bhd_device_guard guard(ctx);
    return launch_attention(ctx, out_dev, q_dev, k_cache_dev, v_cache_dev, 1, 0, n_heads, n_kv_heads, head_dim, scale, pos_dev, uint32_t(max_positions),
                            max_positions, cudaStream_t(stream));
}

extern "C" int32_t bhd_incremental_attention(bhd_ctx* ctx, float* out_dev, const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                             uint64_t n_query_positions, uint64_t query_start, uint64_t n_kv_positions, uint32_t n_heads,
                                             uint32_t n_kv_heads, uint32_t head_dim, float scale, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (n_query_positions == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention requires at least one query position");
    if (n_kv_positions == 0) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention requires at least one cached position");
    if (n_heads == 0 || n_kv_heads == 0 || head_dim == 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention dimensions must be non-zero, got heads=%u kv_heads=%u head_dim=%u",
                        n_heads, n_kv_heads, head_dim);
    if (n_heads % n_kv_heads != 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention needs query heads divisible by kv heads, got %u and %u",
                        n_heads, n_kv_heads);
    if (!isfinite(scale) || scale <= 0.0f)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention scale must be positive and finite, got %g", double(scale));
    if (query_start + n_query_positions > n_kv_positions)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: incremental causal attention query range %llu..%llu exceeds %llu cached positions",
                        (unsigned long long)query_start, (unsigned long long)(query_start + n_query_positions), (unsigned long long)n_kv_positions);
    if (n_query_positions > 0x7fffffffull || n_heads > 65535u || n_kv_positions > (200u * 1024u) / 4u)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: attention over %llu positions and %u heads is beyond this kernel",
                        (unsigned long long)n_kv_positions, n_heads);
    if (!out_dev || !q_dev || !k_cache_dev || !v_cache_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "attention: null buffer");
    bhd_device_guard guard(ctx);
    return launch_attention(ctx, out_dev, q_dev, k_cache_dev, v_cache_dev, uint32_t(n_query_positions), uint32_t(query_start), n_heads, n_kv_heads,
                            head_dim, scale, nullptr, 0, query_start + n_query_positions, cudaStream_t(stream));
}

extern "C" int32_t bhd_embedding_rows(bhd_ctx* ctx, const bhd_weight* table, const int32_t* ids_dev, uint64_t n_ids, float* out_dev,
                                      void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (!table || table->magic != BHD_WEIGHT_MAGIC || table->ctx != ctx) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "embedding_rows: not a weight of this context");
    if (n_ids == 0 || table->cols == 0) return BHD_OK;
    if (n_ids > 0x7fffffffull) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: too many embedding rows");
    if (!ids_dev || !out_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "embedding_rows: null buffer");
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
#define LAUNCH(K) \
    bhd_launch_dependent(ctx, k_embedding_rows<K>, dim3(unsigned(n_ids)), dim3(256), 0, s, table->dev, table->row_bytes, table->rows * table->slabs, table->cols, ids_dev, out_dev, ctx->status_dev)
    BHD_DISPATCH_KIND(table->kind, LAUNCH)
#undef LAUNCH
    BHD_LAUNCHED(ctx, "embedding row kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_sigmoid_gate(bhd_ctx* ctx, float* out_dev, const float* in_dev, const float* gate_dev, uint64_t n, void* stream) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return BHD_OK;
    if (!out_dev || !in_dev || !gate_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "sigmoid_gate: null buffer");
    bhd_device_guard guard(ctx);
    bhd_launch_dependent(ctx, k_sigmoid_gate, dim3(unsigned((n + 255) / 256)), dim3(256), 0, cudaStream_t(stream), out_dev, in_dev, gate_dev, n);
    BHD_LAUNCHED(ctx, "sigmoid gate kernel");
    return BHD_OK;
}

// Grows the context's workspace to at least n_bytes now, so that later calls (a CUDA graph capture in particular, during
// which nothing may be allocated) find it large enough.
// The workspace's current size. It only changes when the workspace is replaced by a larger one, so a host that holds
// CUDA graphs compares it with the size at capture time to know whether the graphs still point into live memory.
extern "C" uint64_t bhd_workspace_bytes(const bhd_ctx* ctx) { return ctx_ok(ctx) ? uint64_t(ctx->workspace_bytes) : 0ull; }

extern "C" int32_t bhd_workspace_reserve(bhd_ctx* ctx, uint64_t n_bytes) {
    if (!ctx_ok(ctx)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_device_guard guard(ctx);
    return bhd_ensure_workspace(ctx, size_t(n_bytes), nullptr);
}
