// Grouped routed-expert matmul for packed Q8_0 experts on sm_100a, integer tensor-core variant.
//
// One CTA = one group (up to 32 routes of one expert, sorted by the plan kernel) x one 64- or
// 128-row tile of the expert matrix, streaming all columns once. With at most 32 routes per expert the
// layer is bound by weight traffic, so the goal is the decode kernel's: as few issue slots per
// weight byte as possible.
//   * Q8_0 quants go to mma.sync m16n8k32 (s8 x s8 -> s32) exactly as they lie in memory; no
//     conversion. One MMA covers one 32-column block of 16 rows for four routes.
//   * Activations are block-scaled integers per (route, 256-column chunk): X = round(x * 32639 / max|x|)
//     split into two signed bytes, X = 256 * d0 + d1. The two digits of a route sit in adjacent
//     MMA columns (column = 2 * route + digit), so the lane that owns accumulator columns
//     (2t, 2t+1) combines them without any exchange: v = 256 * c0 + c1, exact in s32.
//   * Per block the lane adds d_block(row) * v into a per-chunk f32 sum; per chunk it folds in
//     the route's chunk factor max|x| / 32639. Relative error 2^-16 of the largest activation of the chunk.
//   * Four or eight consumer warps (16 rows each) share the staged activations; one producer
//     warp keeps a 2-3 stage ring full: one tiled TMA copy per 64 x 272-byte weight box, one bulk
//     copy for the group's packed activations (contiguous, because slots are sorted by expert).
// Every wait is bounded and reports through the status word.
//
// Reference semantics: crates/beholdd-model/src/qwen3moe/forward.rs:1363-1400 (gate/up matvec,
// SwiGLU, down matvec_add scaled by the route weight) with kquant::q8_0::dot
// (crates/beholdd-kernel/src/kquant.rs:61-79).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int CHUNK_K = 256;
constexpr int BOX = 272;        // packed bytes per row per chunk
constexpr int BOX_ROWS = 64;    // rows of the weight tensor map's box
// Packed activations of one (slot, chunk): 8 blocks x 2 digits x 32 bytes in fragment order,
// then the chunk factor as f32; padded to 576 bytes so that the eight routes a warp reads at once fall
// into different shared-memory banks (144 words = 16 mod 32).
constexpr int SLOT_BYTES = 576, SLOT_SCALE_OFF = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half(uint16_t(h))); }
__device__ __forceinline__ void imma_s8(int (&c)[4], const uint32_t (&a)[4], uint2 b) {
    c[0] = c[1] = c[2] = c[3] = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b.x), "r"(b.y));
}

// ---- activations of the routed experts as block-floating bytes, in slot order ----------------
// mode 0: row of slot = x[position of the slot's route] (the token-to-expert gather);
// mode 1: row of slot = silu(g[slot]) * u[slot] (crates/beholdd-kernel/src/vecops.rs:91-111, limit 0).
// One warp per (slot, chunk); lane l holds columns 8l..8l+7 of the chunk (block l / 4).
// out[(chunk * n_slots + slot) * SLOT_BYTES ...]: per block 32 bytes of digit 0 then 32 of digit
// 1, byte order [t][half][i] for k-slot 16 * half + 4 * t + i (what lane-in-quad t loads as one
// 8-byte B fragment), then the chunk's factor max|x| / 32639.
__global__ void k_moe_slots_i8(int mode, const MoeHeader* __restrict__ hdr, const int32_t* __restrict__ slot_route,
                               const uint8_t* __restrict__ slot_cls, uint32_t max_cls, uint32_t top_k,
                               const float* __restrict__ src, const float* __restrict__ src2, uint32_t K, uint32_t n_slots,
                               uint8_t* __restrict__ out, uint32_t* __restrict__ status) {
    bhd_wait_for_prior_kernels();
    const uint32_t chunk = blockIdx.y, slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (slot >= hdr->local_routes || slot >= n_slots) return;  // whole warps
    if (slot_cls[slot] > max_cls) return;                       // a group the tensor-core kernel takes (fp16 rows)
    const uint32_t k0 = chunk * CHUNK_K + 8 * lane;
    const uint64_t row = mode == 0 ? uint64_t(uint32_t(slot_route[slot]) / top_k) : uint64_t(slot);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (k0 + 7 < K) {
        const float4 a = *reinterpret_cast<const float4*>(src + row * K + k0), b = *reinterpret_cast<const float4*>(src + row * K + k0 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (mode == 1) {
            const float4 c = *reinterpret_cast<const float4*>(src2 + row * K + k0), d = *reinterpret_cast<const float4*>(src2 + row * K + k0 + 4);
            const float u[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fdiv_rn(v[i], __fadd_rn(1.0f, expf(-v[i]))), u[i]);
        }
    } else {
        for (int i = 0; i < 8; ++i)
            if (k0 + i < K) {
                float a = src[row * K + k0 + i];
                if (mode == 1) a = __fmul_rn(__fdiv_rn(a, __fadd_rn(1.0f, expf(-a))), src2[row * K + k0 + i]);
                v[i] = a;
            }
    }
    float mx = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (!(fabsf(v[i]) <= 3.0e38f)) { bad = true; v[i] = 0.f; }  // NaN or infinity
        mx = fmaxf(mx, fabsf(v[i]));
    }
    if (bad) atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // The chunk's largest magnitude maps to 32639 = 127 * 256 + 127, the largest integer whose two balanced digits
    // both fit a signed byte; chunks below 2^-100 pack as zero.
    // When a power-of-two factor already makes every value of the chunk an integer within that range (small
    // integers, dyadic fractions), it is used instead: such inputs then pass through exactly.
    const uint32_t eb = __float_as_uint(mx) >> 23;
    const bool tiny = eb < 27u;
    float up = tiny ? 0.f : __fdiv_rn(32639.0f, mx);
    float down = tiny ? 0.f : __fdiv_rn(mx, 32639.0f);
    {
        const float up2 = tiny ? 0.f : __uint_as_float((268u - eb) << 23);  // |x * up2| < 2^15
        bool lossless = !tiny;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = v[i] * up2;
            lossless = lossless && t == rintf(t) && fabsf(t) <= 32639.0f;
        }
        if (__all_sync(0xffffffffu, lossless)) {
            up = up2;
            down = __uint_as_float((eb - 14u) << 23);
        }
    }
    uint32_t w0[2] = {0u, 0u}, w1[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int X = __float2int_rn(v[i] * up);           // |X| <= 32639
        const int d0 = (X + 128) >> 8, d1 = X - d0 * 256;  // X = 256 * d0 + d1, d0 in [-127, 127], d1 in [-128, 127]
        w0[i >> 2] |= (uint32_t(d0) & 0xffu) << (8 * (i & 3));
        w1[i >> 2] |= (uint32_t(d1) & 0xffu) << (8 * (i & 3));
    }
    uint8_t* dst = out + (uint64_t(chunk) * n_slots + slot) * SLOT_BYTES;
    const uint32_t blk = lane >> 2, m = lane & 3;  // columns 8m..8m+7 of block blk: k-slots 8m + i
    // k = 8m + i: half = m / 2, t = 2 * (m % 2) + i / 4 -> byte position t * 8 + half * 4 + i % 4
    uint8_t* b0 = dst + blk * 64 + (2 * (m & 1)) * 8 + (m >> 1) * 4;
    *reinterpret_cast<uint32_t*>(b0) = w0[0];
    *reinterpret_cast<uint32_t*>(b0 + 8) = w0[1];
    *reinterpret_cast<uint32_t*>(b0 + 32) = w1[0];
    *reinterpret_cast<uint32_t*>(b0 + 40) = w1[1];
    if (lane < 16) *reinterpret_cast<float*>(dst + SLOT_SCALE_OFF + 4 * lane) = lane == 0 ? down : 0.f;
}

struct GroupedI8Params {
    const MoeHeader* hdr;
    const MoeGroup* groups;
    const int32_t* glist;      // the class's group indices
    const uint8_t* xq;         // [chunk][slot][SLOT_BYTES]
    float* out0;               // [slot][rows] of matrix 0 (gate, or down)
    float* out1;               // [slot][rows] of matrix 1 (up)
    float* const* slot_dst;    // optional: where the output row of a slot starts (instead of out0 + slot * rows)
    const float* slot_weight;  // down only: route weight per slot
    uint32_t* status;
    uint32_t rows, chunks, n_slots, cls, ring;
};

// NT MMAs per block: routes 4j..4j+3 in MMA j (NT = 1, 2, 4, 8 for groups of up to 4, 8, 16, 32 routes).
// CW consumer warps (4 or 8) = 16 * CW rows per CTA.
template <int NT, int CW>
__global__ void __launch_bounds__((CW + 1) * 32) k_moe_grouped_i8(const __grid_constant__ CUtensorMap tmap0,
                                                            const __grid_constant__ CUtensorMap tmap1, const GroupedI8Params p) {
    constexpr int TILE_ROWS = 16 * CW, CONSUMERS = CW, W_BYTES = TILE_ROWS * BOX;
    constexpr int X_MAX = NT * 4 * SLOT_BYTES;
    constexpr int STAGE = (W_BYTES + X_MAX + 127) / 128 * 128;
    bhd_wait_for_prior_kernels();
    if (blockIdx.y >= p.hdr->gcount[p.cls]) return;  // whole CTA, before anything is set up
    const MoeGroup grp = p.groups[p.glist[blockIdx.y]];
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 127u) & ~127u;
    __shared__ uint64_t full[4], empty[4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t nb = uint32_t(grp.nb), slot0 = uint32_t(grp.slot0), tile = blockIdx.x, R = p.ring;
    const CUtensorMap* tmap = blockIdx.z ? &tmap1 : &tmap0;
    float* const out = blockIdx.z ? p.out1 : p.out0;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < R; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], CONSUMERS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // ---- producer ----
        if (lane == 0) {
            const int y = int(uint32_t(grp.expert_local) * p.rows + tile * TILE_ROWS);
            for (uint32_t c = 0; c < p.chunks; ++c) {
                const uint32_t s = c % R;
                if (!mbar_wait(&empty[s], ((c / R) & 1) ^ 1)) { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); break; }
                const uint32_t dst = smem0 + s * STAGE;
                mbar_arrive_expect_tx(&full[s], W_BYTES + nb * SLOT_BYTES);
#pragma unroll
                for (int h = 0; h < TILE_ROWS / BOX_ROWS; ++h)
                    tma_load_2d(dst + h * BOX_ROWS * BOX, tmap, int(c * (BOX / 2)), y + h * BOX_ROWS, &full[s]);
                bulk_load_1d(dst + W_BYTES, p.xq + (uint64_t(c) * p.n_slots + slot0) * SLOT_BYTES, nb * SLOT_BYTES, &full[s]);
            }
        }
        return;
    }

    // ---- consumers: warp w owns rows 16w..16w+15 of the tile ----
    const uint32_t r0 = uint32_t(warp) * 16 + g, r1 = r0 + 8;
    float acc[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = 0.f;
    // B fragment of MMA j: lane g supplies column g = (route 4j + g / 2, digit g % 2)
    const uint32_t b_off = uint32_t(g >> 1) * SLOT_BYTES + uint32_t(g & 1) * 32 + uint32_t(t) * 8;
    for (uint32_t c = 0; c < p.chunks; ++c) {
        const uint32_t s = c % R;
        if (!mbar_wait(&full[s], (c / R) & 1)) {
            if (lane == 0) atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT);
            break;
        }
        const uint32_t st = smem0 + s * STAGE, w0 = st + r0 * BOX, w1 = st + r1 * BOX, xb = st + W_BYTES;
        float part[NT][2];  // sum over the chunk's blocks of d_block * (integer dot product)
#pragma unroll
        for (int j = 0; j < NT; ++j) part[j][0] = part[j][1] = 0.f;
        // Operands of one 32-column block: the lane's A fragment (rows r0 / r1, two halves of
        // k), the two block scales, and its B fragment for each of the NT MMAs. The loads of
        // block b + 1 are issued between the MMAs of block b and the arithmetic on their
        // results, so neither the shared-memory nor the MMA latency is ever waited for alone
        // (the asm statements keep program order, so the order below is the issue order).
        struct Ops { uint32_t raw[6]; uint32_t a[4]; uint32_t d0, d1; uint2 b[NT]; };
        auto load_block = [&](int blk, Ops& o) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int off = 34 * blk + 2 + 16 * h + 4 * t;  // this lane's four quants of the half block
                if (blk & 1) {
                    o.a[2 * h] = lds32(w0 + off);
                    o.a[2 * h + 1] = lds32(w1 + off);
                } else {  // 2 mod 4: two aligned words, stitched when they are used
                    o.raw[3 * h] = lds32(w0 + off - 2);
                    o.raw[3 * h + 1] = lds32(w0 + off + 2);
                    o.raw[3 * h + 2] = lds32(w1 + off - 2);
                    o.a[2 * h + 1] = lds32(w1 + off + 2);
                }
            }
            o.d0 = lds16(w0 + 34 * blk);
            o.d1 = lds16(w1 + 34 * blk);
#pragma unroll
            for (int j = 0; j < NT; ++j) o.b[j] = lds64(xb + uint32_t(4 * j) * SLOT_BYTES + b_off + blk * 64);
        };
        auto finish_a = [&](int blk, Ops& o) {
            if (!(blk & 1)) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    o.a[2 * h] = __funnelshift_r(o.raw[3 * h], o.raw[3 * h + 1], 16);
                    o.a[2 * h + 1] = __funnelshift_r(o.raw[3 * h + 2], o.a[2 * h + 1], 16);
                }
            }
        };
        Ops cur, nxt;
        load_block(0, cur);
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            finish_a(blk, cur);
            int ci[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) imma_s8(ci[j], cur.a, cur.b[j]);
            if (blk < 7) load_block(blk + 1, nxt);
            const float d0 = h2f(cur.d0), d1 = h2f(cur.d1);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                // accumulator columns (2t, 2t+1) = route 4j + t, digits 0 and 1
                part[j][0] = fmaf(d0, float(ci[j][0] * 256 + ci[j][1]), part[j][0]);
                part[j][1] = fmaf(d1, float(ci[j][2] * 256 + ci[j][3]), part[j][1]);
            }
            if (blk < 7) cur = nxt;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const float xs = __uint_as_float(lds32(xb + uint32_t(4 * j + t) * SLOT_BYTES + SLOT_SCALE_OFF));
            acc[j][0] = fmaf(xs, part[j][0], acc[j][0]);
            acc[j][1] = fmaf(xs, part[j][1], acc[j][1]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    const uint32_t row_a = tile * TILE_ROWS + r0, row_b = tile * TILE_ROWS + r1;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint32_t route = uint32_t(4 * j + t);
        if (route >= nb) continue;  // columns beyond the group hold whatever was in shared memory
        const uint32_t slot = slot0 + route;
        const float sc = p.slot_weight ? p.slot_weight[slot] : 1.0f;
        float* dst = p.slot_dst ? p.slot_dst[slot] : out + uint64_t(slot) * p.rows;
        if (row_a < p.rows) dst[row_a] = __fmul_rn(acc[j][0], sc);
        if (row_b < p.rows) dst[row_b] = __fmul_rn(acc[j][1], sc);
    }
}

template <int NT, int CW>
int32_t launch_nt(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, GroupedI8Params p, uint32_t group_bound, cudaStream_t s) {
    constexpr int TILE_ROWS = 16 * CW, W_BYTES = TILE_ROWS * BOX, THREADS = (CW + 1) * 32;
    constexpr int STAGE = (W_BYTES + NT * 4 * SLOT_BYTES + 127) / 128 * 128;
    constexpr int RING = NT >= 4 ? 2 : 3;  // several CTAs per SM cover the latency the short ring leaves open
    constexpr size_t DYN = size_t(RING) * STAGE + 128;
    const uint32_t tiles = uint32_t((w0->rows + TILE_ROWS - 1) / TILE_ROWS);
    auto kern = k_moe_grouped_i8<NT, CW>;
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(DYN)), "raising the shared memory limit");
        once.mark(ctx);
    }
    if (group_bound == 0) return BHD_OK;
    CUtensorMap m0, m1;
    memcpy(&m0, w0->tmap, sizeof(m0));
    memcpy(&m1, (w1 ? w1 : w0)->tmap, sizeof(m1));
    p.ring = RING;
    bhd_launch_dependent(ctx, kern, dim3(tiles, group_bound, w1 ? 2 : 1), dim3(THREADS), DYN, s, m0, m1, p);
    BHD_LAUNCHED(ctx, "integer grouped expert kernel");
    return BHD_OK;
}

}  // namespace

bool bhd_moe_i8_usable(const bhd_weight* w) { return w->kind == BHD_TYPE_Q8_0 && w->tmap_ok && w->cols % 8 == 0; }

size_t bhd_moe_slots_i8_bytes(uint32_t K, uint32_t n_slots) {
    return size_t((K + CHUNK_K - 1) / CHUNK_K) * n_slots * SLOT_BYTES;
}

int32_t bhd_launch_moe_slots_i8(bhd_ctx* ctx, int mode, const void* hdr, const int32_t* slot_route, const uint8_t* slot_cls,
                                uint32_t max_cls, uint32_t top_k, const float* src, const float* src2, uint32_t K, uint32_t n_slots,
                                void* out, cudaStream_t s) {
    if (n_slots == 0) return BHD_OK;
    bhd_launch_dependent(ctx, k_moe_slots_i8, dim3((n_slots + 3) / 4, (K + CHUNK_K - 1) / CHUNK_K), dim3(128), 0, s, mode, static_cast<const MoeHeader*>(hdr), slot_route, slot_cls, max_cls, top_k,
                                                                                         src, src2, K, n_slots, static_cast<uint8_t*>(out),
                                                                                         ctx->status_dev);
    BHD_LAUNCHED(ctx, mode ? "expert gating kernel" : "token gather kernel");
    return BHD_OK;
}

// Groups of one size class (cls 0..3: up to 4, 8, 16, 32 routes): one CTA per (group, 64-row tile[, gate|up]).
int32_t bhd_launch_moe_grouped_i8(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                  const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* xq, uint32_t n_slots,
                                  float* out0, float* out1, float* const* slot_dst, const float* slot_weight, cudaStream_t s) {
    GroupedI8Params p;
    p.slot_dst = slot_dst;
    p.hdr = static_cast<const MoeHeader*>(hdr);
    p.groups = static_cast<const MoeGroup*>(groups);
    p.glist = glist;
    p.xq = static_cast<const uint8_t*>(xq);
    p.out0 = out0;
    p.out1 = out1;
    p.slot_weight = slot_weight;
    p.status = ctx->status_dev;
    p.rows = uint32_t(w0->rows);
    p.chunks = uint32_t((w0->cols + CHUNK_K - 1) / CHUNK_K);
    p.n_slots = n_slots;
    p.cls = cls;
    p.ring = 0;
    switch (cls) {
        case 0: return launch_nt<1, 4>(ctx, w0, w1, p, group_bound, s);
        case 1: return launch_nt<2, 4>(ctx, w0, w1, p, group_bound, s);
        case 2: return launch_nt<4, 4>(ctx, w0, w1, p, group_bound, s);
        default: return launch_nt<8, 8>(ctx, w0, w1, p, group_bound, s);
    }
}
