// Decode matvec (1 or 2 activation vectors) for packed Q8_0 / Q4_K / Q6_K on sm_100a, integer
// tensor-core variant. Same structure as matvec_decode.cu (16 rows per CTA, four warps on
// alternating 256-column chunks, one private TMA ring per warp, diagonal B operand, fixed-order
// reduction), but the quants go to mma.sync m16n8k32 as 8-bit integers:
//
//   * Q8_0 quants are fed as they lie in memory (s8), Q4_K nibbles cost one AND (and one shift
//     for the high ones) per four weights, Q6_K codes one OR of two masked planes. There is no
//     conversion to a floating-point bit pattern and no constant offset to undo, and one
//     instruction covers 32 columns instead of 16 -- about half the issue slots per byte of
//     the fp16 variant, which was issue-bound.
//   * Activations are block floating point: per scale group (32 columns, 16 for Q6_K) a power
//     of two 2^e and a 15-bit integer X = round(x * 2^(14 - e)) split into two signed bytes,
//     X = 256 * d0 + d1. The two digits sit in adjacent MMA columns; the s32 accumulators are
//     combined exactly (256 * c0 + c1) and scaled by 2^(e - 14) and the block scale in f32.
//     Relative error 2^-15 of the largest activation of the group; any finite f32 is accepted.
//
// Reference semantics: crates/beholdd-backend/src/cpu.rs:398-507; block formats:
// crates/beholdd-kernel/src/kquant.rs:29-241.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int ROWS = 16, WARPS = 4, CHUNK_K = 256;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

template <uint32_t KIND> struct Geo;
// RING: stages per warp. Four stages of Q4_K hold all 4096 columns of a projection, so a CTA
// that starts early (programmatic dependent launch) has requested all its weights before the
// activations exist; the wider formats keep two stages to leave room for six CTAs per SM.
template <> struct Geo<BHD_TYPE_Q8_0> { static constexpr int BOX = 272, GROUPS = 8, RING = 2; };
template <> struct Geo<BHD_TYPE_Q4_K> { static constexpr int BOX = 144, GROUPS = 8, RING = 4; };
template <> struct Geo<BHD_TYPE_Q6_K> { static constexpr int BOX = 240, GROUPS = 16, RING = 2; };
__host__ __device__ constexpr int igroups(uint32_t kind) { return kind == BHD_TYPE_Q6_K ? 16 : 8; }

// Packed activations of one chunk: [group][vector][digit][t] 8-byte B fragments (b0, b1), then
// [group][vector] f32 pairs (2^(e-14), sum of the dequantised activations of the group).
__host__ __device__ constexpr int iblob_frag_bytes(uint32_t kind, int nb) { return igroups(kind) * nb * 64; }
__host__ __device__ constexpr int iblob_bytes(uint32_t kind, int nb) {
    return (iblob_frag_bytes(kind, nb) + igroups(kind) * nb * 8 + 127) / 128 * 128;
}

// Column (within the chunk) behind k-slot `slot` (0..31) of the MMA that covers scale group
// `grp`. Q8_0: the block's bytes in order. Q4_K: a lane's eight bytes are split over the two
// halves of the k range. Q6_K: a k32 MMA spans two 16-column groups, the even one in slots
// 0..15 and the odd one in slots 16..31 (slot is then relative to the pair).
__host__ __device__ __forceinline__ int slot_column(uint32_t kind, int grp, int slot) {
    if (kind == BHD_TYPE_Q8_0) return 32 * grp + slot;
    if (kind == BHD_TYPE_Q4_K) {
        const int t = (slot & 15) >> 2, i = slot & 3, hi = slot >> 4;
        return 64 * (grp >> 1) + 32 * (grp & 1) + 8 * t + 4 * hi + i;
    }
    return 16 * grp + (slot & 15);  // caller passes slots 0..15 for even groups, 16..31 for odd ones
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// A unsigned (nibbles, 6-bit codes) or signed (Q8_0 quants); B always signed digits.
template <bool A_SIGNED, bool FIRST>
__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    if (FIRST) c[0] = c[1] = c[2] = c[3] = 0;
    if (A_SIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
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
__device__ __forceinline__ float2 ldsf2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// Packed activations are rewritten by every launch while CTAs of the next one may already be
// resident, so they are read past L1.
__device__ __forceinline__ uint2 ldg64_cg(const void* p) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// Programmatic dependent launch (a no-op when the kernel was launched without the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half(uint16_t(h))); }
__device__ __forceinline__ float u2f(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.0f; }

// ---- activation packer ----------------------------------------------------------------------
// One CTA per chunk, one warp per scale group (looping when there are more groups than warps).
// Lane l holds column slot l of its group (Q6_K: lanes 0..15). x [nvec x K] f32.
__global__ void k_pack_x_i8(uint32_t kind, const float* __restrict__ x, uint32_t nvec, uint32_t nb, uint32_t K,
                            uint8_t* __restrict__ blob, uint32_t* __restrict__ status) {
    const int chunk = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = igroups(kind), per = 256 / groups;  // columns per group: 32 or 16
    // Programmatic dependent launch: let the matvec kernel that follows start its weight
    // prefetch now; wait for whatever preceded this launch (it may have produced x, and the
    // previous matvec may still be reading the blob) before touching memory.
    pdl_launch_dependents();
    pdl_wait();
    uint8_t* cb = blob + uint64_t(chunk) * iblob_bytes(kind, nb);
    float2* meta = reinterpret_cast<float2*>(cb + iblob_frag_bytes(kind, nb));
    for (int item = warp; item < groups * int(nb); item += blockDim.x >> 5) {
        const int grp = item / int(nb), v = item % int(nb);
        // the slot this lane fills: Q6_K odd groups live in slots 16..31 of their MMA
        const bool live = lane < per;
        const int slot = (kind == BHD_TYPE_Q6_K && (grp & 1)) ? 16 + lane : lane;
        const uint32_t k = uint32_t(chunk) * CHUNK_K + uint32_t(slot_column(kind, grp, slot));
        float val = 0.f;
        if (live && uint32_t(v) < nvec && k < K) val = x[uint64_t(v) * K + k];
        if (!(fabsf(val) <= 3.0e38f)) { atomicOr(status, BHD_DEV_ACTIVATION_RANGE); val = 0.f; }  // NaN or infinity
        float mx = fabsf(val);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        int ex = 0;
        if (mx > 0.f) frexpf(mx, &ex);              // mx = m * 2^ex, m in [0.5, 1)
        // Groups whose largest magnitude is below 2^-100 pack as zero (their power of two would overflow).
        const float up = ex < -100 ? 0.f : ldexpf(1.0f, 14 - ex), down = ex < -100 ? 0.f : ldexpf(1.0f, ex - 14);
        const int X = __float2int_rn(val * up);      // |X| <= 2^14
        const int d0 = (X + 128) >> 8, d1 = X - d0 * 256;  // X = 256 * d0 + d1, both in [-128, 127]
        float sum = float(X) * down;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        // fragment [grp][v][digit][t]: bytes 0..3 = slots 4t..4t+3 (b0), bytes 4..7 = slots 16+4t.. (b1)
        uint8_t* frag = cb + (grp * nb + v) * 64;
        const int t = (slot & 15) >> 2, i = slot & 3, half_ = slot >> 4;
        if (live) {
            frag[t * 8 + half_ * 4 + i] = uint8_t(int8_t(d0));
            frag[32 + t * 8 + half_ * 4 + i] = uint8_t(int8_t(d1));
            if (kind == BHD_TYPE_Q6_K) {  // the other half of the k range belongs to the neighbouring group: zero here
                frag[t * 8 + (half_ ^ 1) * 4 + i] = 0;
                frag[32 + t * 8 + (half_ ^ 1) * 4 + i] = 0;
            }
        }
        if (lane == 0) meta[grp * nb + v] = make_float2(down, sum);
    }
}

struct DecodeI8Params {
    const uint8_t* blob;
    float* y;
    uint32_t* status;
    uint32_t rows, row_base, chunks, batch;
    float scale;
    int accumulate;
};

template <uint32_t KIND>
__device__ __forceinline__ int tile_row(int m) {
    if (KIND == BHD_TYPE_Q4_K) return m < 8 ? 2 * m : 2 * (m - 8) + 1;  // keeps 8-byte reads conflict-free
    return m;
}

// NB vectors; GPT = 4 / NB scale groups share one accumulator tile; lane-in-quad t owns tile
// columns (2t, 2t+1) = (group gl = t / NB, vector v = t % NB) x (digit 0, digit 1).
template <uint32_t KIND, int NB, int RING>
__global__ void __launch_bounds__(WARPS * 32) k_matvec_decode_i8(const __grid_constant__ CUtensorMap tmap, const DecodeI8Params p) {
    constexpr int BOX = Geo<KIND>::BOX, GROUPS = Geo<KIND>::GROUPS, GPT = 4 / NB, TILES = GROUPS / GPT;
    constexpr int W_BYTES = ROWS * BOX, X_BYTES = iblob_bytes(KIND, NB), FRAG = iblob_frag_bytes(KIND, NB);
    constexpr int STAGE = (W_BYTES + 127) / 128 * 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    __shared__ uint64_t bars[WARPS][RING];
    __shared__ float red[WARPS][ROWS][NB];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t tile = blockIdx.x;
    if (lane == 0) {
        for (int i = 0; i < RING; ++i) mbar_init(&bars[warp][i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint8_t* ring = smem + warp * (RING * STAGE);
    const uint32_t ring32 = smem_u32(ring);
    const uint32_t my_chunks = p.chunks > uint32_t(warp) ? (p.chunks - warp + WARPS - 1) / WARPS : 0;
    // lane 0 only: stage the weights of the warp's i-th chunk.
    auto issue_w = [&](uint32_t i) {
        const uint32_t chunk = warp + i * WARPS, slot = i % RING;
        mbar_arrive_expect_tx(&bars[warp][slot], W_BYTES);
        const uint32_t byte0 = (KIND == BHD_TYPE_Q6_K) ? ((210u * chunk) & ~15u) : uint32_t(BOX) * chunk;
        tma_load_2d(ring + slot * STAGE, &tmap, int(byte0 >> 1), int(p.row_base + tile * ROWS), &bars[warp][slot]);
    };
    // Weights are never written by a preceding kernel, so their first stages are requested
    // before waiting for the grids this launch depends on (the packer, and before it whatever
    // produced x and y); everything else happens after the wait.
    if (lane == 0)
        for (uint32_t i = 0; i < my_chunks && i < RING; ++i) issue_w(i);
    pdl_launch_dependents();
    pdl_wait();

    const int r0 = tile_row<KIND>(g), r1 = tile_row<KIND>(g + 8);
    const int gl = t / NB, v = t % NB;                  // what this lane's accumulator columns mean
    const int bv = (g >> 1) % NB, bgl = (g >> 1) / NB;  // what this lane's B column (n = g) means
    const int boff = bv * 64 + (g & 1) * 32 + t * 8;    // fragment offset within a group
    float tot0 = 0.f, tot1 = 0.f;

    // The lane's share of a chunk's packed activations, straight from global memory (L2): the
    // B fragments of the TILES groups its MMA column stands for, and (2^(e-14), sum) of the
    // TILES groups its accumulator columns stand for. Loaded one chunk ahead.
    uint2 bq[TILES], bq_next[TILES];
    float2 mq[TILES], mq_next[TILES];
    auto load_x = [&](uint32_t chunk, uint2 (&q)[TILES], float2 (&m)[TILES]) {
        const uint8_t* cb = p.blob + uint64_t(chunk) * X_BYTES;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
            q[tl] = ldg64_cg(cb + (tl * GPT + bgl) * (64 * NB) + boff);
            const uint2 mm = ldg64_cg(cb + FRAG + 8 * ((tl * GPT + gl) * NB + v));
            m[tl] = make_float2(__uint_as_float(mm.x), __uint_as_float(mm.y));
        }
    };
    if (my_chunks > 0) load_x(warp, bq_next, mq_next);

    for (uint32_t i = 0; i < my_chunks; ++i) {
        const uint32_t slot = i % RING, chunk = warp + i * WARPS;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
            bq[tl] = bq_next[tl];
            mq[tl] = mq_next[tl];
        }
        if (i + 1 < my_chunks) load_x(chunk + WARPS, bq_next, mq_next);
        if (!mbar_wait(&bars[warp][slot], (i / RING) & 1)) {
            if (lane == 0) atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT);
            break;
        }
        const uint32_t st = ring32 + slot * STAGE;
        const uint32_t w0 = st + r0 * BOX, w1 = st + r1 * BOX;
        // real fragment when the group is one this lane's MMA column stands for, zeros otherwise
        auto bfrag = [&](int grp) -> uint2 {
            const bool on = (grp % GPT) == bgl;
            return make_uint2(on ? bq[grp / GPT].x : 0u, on ? bq[grp / GPT].y : 0u);
        };
        int acc[TILES][4];

        if constexpr (KIND == BHD_TYPE_Q8_0) {
#pragma unroll
            for (int blk = 0; blk < 8; ++blk) {
                uint32_t a[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int off = 34 * blk + 2 + 16 * h + 4 * t;  // this lane's four quants of the half block
                    if (blk & 1) {
                        a[2 * h] = lds32(w0 + off);
                        a[2 * h + 1] = lds32(w1 + off);
                    } else {  // 2 mod 4: stitch two aligned words
                        a[2 * h] = __funnelshift_r(lds32(w0 + off - 2), lds32(w0 + off + 2), 16);
                        a[2 * h + 1] = __funnelshift_r(lds32(w1 + off - 2), lds32(w1 + off + 2), 16);
                    }
                }
                if (blk % GPT == 0) imma<true, true>(acc[blk / GPT], a[0], a[1], a[2], a[3], bfrag(blk));
                else imma<true, false>(acc[blk / GPT], a[0], a[1], a[2], a[3], bfrag(blk));
            }
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const int blk = tl * GPT + gl;
                const float2 m = mq[tl];
                const float d0 = h2f(lds16(w0 + 34 * blk)) * m.x, d1 = h2f(lds16(w1 + 34 * blk)) * m.x;
                tot0 = fmaf(d0, float(acc[tl][0] * 256 + acc[tl][1]), tot0);
                tot1 = fmaf(d1, float(acc[tl][2] * 256 + acc[tl][3]), tot1);
            }
        } else if constexpr (KIND == BHD_TYPE_Q4_K) {
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                const uint2 q0 = lds64(w0 + 16 + 32 * pp + 8 * t), q1 = lds64(w1 + 16 + 32 * pp + 8 * t);
                // low nibbles: sub-block 2pp, high nibbles: sub-block 2pp + 1
                {
                    const int j = 2 * pp;
                    const uint32_t a0 = q0.x & 0x0F0F0F0Fu, a1 = q1.x & 0x0F0F0F0Fu, a2 = q0.y & 0x0F0F0F0Fu, a3 = q1.y & 0x0F0F0F0Fu;
                    if (j % GPT == 0) imma<false, true>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                    else imma<false, false>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                }
                {
                    const int j = 2 * pp + 1;
                    const uint32_t a0 = (q0.x >> 4) & 0x0F0F0F0Fu, a1 = (q1.x >> 4) & 0x0F0F0F0Fu;
                    const uint32_t a2 = (q0.y >> 4) & 0x0F0F0F0Fu, a3 = (q1.y >> 4) & 0x0F0F0F0Fu;
                    if (j % GPT == 0) imma<false, true>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                    else imma<false, false>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                }
            }
            const uint4 h0 = lds128(w0), h1 = lds128(w1);
            const float d0 = h2f(h0.x & 0xffffu), m0 = h2f(h0.x >> 16), d1 = h2f(h1.x & 0xffffu), m1 = h2f(h1.x >> 16);
            // Packed 6-bit fields (crates/beholdd-kernel/src/kquant.rs:176-185), four per word:
            // scales 0-3, mins 0-3, scales 4-7, mins 4-7.
            auto fields = [](const uint4& h, uint32_t (&f)[4]) {
                f[0] = h.y & 0x3F3F3F3Fu;
                f[1] = h.z & 0x3F3F3F3Fu;
                f[2] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                f[3] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            };
            uint32_t f0[4], f1[4];
            fields(h0, f0);
            fields(h1, f1);
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const int j = tl * GPT + gl;        // runtime (depends on the lane)
                const int hi4 = (tl * GPT) >> 2;    // compile-time: which half of the eight sub-blocks
                const uint32_t sh = 8u * uint32_t(j & 3);
                const float sc0 = u2f((f0[2 * hi4] >> sh) & 0xffu), mn0 = u2f((f0[2 * hi4 + 1] >> sh) & 0xffu);
                const float sc1 = u2f((f1[2 * hi4] >> sh) & 0xffu), mn1 = u2f((f1[2 * hi4 + 1] >> sh) & 0xffu);
                const float2 m = mq[tl];
                tot0 += fmaf(d0 * sc0 * m.x, float(acc[tl][0] * 256 + acc[tl][1]), -(m0 * mn0) * m.y);
                tot1 += fmaf(d1 * sc1 * m.x, float(acc[tl][2] * 256 + acc[tl][3]), -(m1 * mn1) * m.y);
            }
        } else {  // Q6_K
            const uint32_t q6_off = (210u * chunk) & 15u;  // where the superblock starts in the staged window
            const uint32_t shb = 8u * (q6_off & 3u);
            const uint32_t b0 = w0 + (q6_off & ~3u), b1 = w1 + (q6_off & ~3u);
            auto word = [&](uint32_t base, int byte_off) -> uint32_t {
                return __funnelshift_r(lds32(base + byte_off), lds32(base + byte_off + 4), shb);
            };
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) acc[tl][0] = acc[tl][1] = acc[tl][2] = acc[tl][3] = 0;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                // high-plane words of this lane for the two 16-lane halves
                const uint32_t qhA0 = word(b0, 128 + 32 * hf + 4 * t), qhA1 = word(b1, 128 + 32 * hf + 4 * t);
                const uint32_t qhB0 = word(b0, 128 + 32 * hf + 16 + 4 * t), qhB1 = word(b1, 128 + 32 * hf + 16 + 4 * t);
#pragma unroll
                for (int gp = 0; gp < 2; ++gp) {  // low-plane byte range shared by groups gp and gp + 2 of the half
                    const uint32_t qlA0 = word(b0, 64 * hf + 32 * gp + 4 * t), qlA1 = word(b1, 64 * hf + 32 * gp + 4 * t);
                    const uint32_t qlB0 = word(b0, 64 * hf + 32 * gp + 16 + 4 * t), qlB1 = word(b1, 64 * hf + 32 * gp + 16 + 4 * t);
#pragma unroll
                    for (int up = 0; up < 2; ++up) {
                        const int grp = gp + 2 * up;         // 32-element group within the half: 0..3
                        const int G = 8 * hf + 2 * grp;      // scale groups G (slots 0..15) and G + 1 (slots 16..31)
                        const uint32_t a0 = ((qlA0 >> (4 * up)) & 0x0F0F0F0Fu) | (((qhA0 >> (2 * grp)) & 0x03030303u) << 4);
                        const uint32_t a1 = ((qlA1 >> (4 * up)) & 0x0F0F0F0Fu) | (((qhA1 >> (2 * grp)) & 0x03030303u) << 4);
                        const uint32_t a2 = ((qlB0 >> (4 * up)) & 0x0F0F0F0Fu) | (((qhB0 >> (2 * grp)) & 0x03030303u) << 4);
                        const uint32_t a3 = ((qlB1 >> (4 * up)) & 0x0F0F0F0Fu) | (((qhB1 >> (2 * grp)) & 0x03030303u) << 4);
                        // The lane feeds group G through b0 or group G + 1 through b1, whichever its column stands for.
                        const uint2 fa = bfrag(G), fb = bfrag(G + 1);
                        imma<false, false>(acc[G / GPT], a0, a1, a2, a3, make_uint2(fa.x | fb.x, fa.y | fb.y));
                    }
                }
            }
            const float d0 = h2f(word(b0, 208) & 0xffffu), d1 = h2f(word(b1, 208) & 0xffffu);
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const int s = tl * GPT + gl;  // scale group
                const uint32_t sw0 = word(b0, 192 + (s & ~3)), sw1 = word(b1, 192 + (s & ~3));
                const float s0 = d0 * float(int8_t((sw0 >> (8 * (s & 3))) & 0xffu));
                const float s1 = d1 * float(int8_t((sw1 >> (8 * (s & 3))) & 0xffu));
                const float2 m = mq[tl];
                // codes are unsigned 0..63; the value is code - 32
                tot0 = fmaf(s0, fmaf(m.x, float(acc[tl][0] * 256 + acc[tl][1]), -32.f * m.y), tot0);
                tot1 = fmaf(s1, fmaf(m.x, float(acc[tl][2] * 256 + acc[tl][3]), -32.f * m.y), tot1);
            }
        }
        __syncwarp();
        if (lane == 0 && i + RING < my_chunks) issue_w(i + RING);
    }

    // Sum over the groups handled by different lanes of the quad (same vector v), then over warps.
#pragma unroll
    for (int m = NB; m < 4; m <<= 1) {
        tot0 += __shfl_xor_sync(0xffffffffu, tot0, m);
        tot1 += __shfl_xor_sync(0xffffffffu, tot1, m);
    }
    if (t < NB) {
        red[warp][r0][t] = tot0;
        red[warp][r1][t] = tot1;
    }
    __syncthreads();
    if (threadIdx.x < ROWS * NB) {
        const int r = threadIdx.x / NB, vv = threadIdx.x % NB;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) sum += red[w][r][vv];
        const uint32_t row = tile * ROWS + r;
        if (row < p.rows && uint32_t(vv) < p.batch) {
            const float val = __fmul_rn(sum, p.scale);
            float* o = p.y + uint64_t(vv) * p.rows + row;
            *o = p.accumulate ? __fadd_rn(*o, val) : val;
        }
    }
}

template <uint32_t KIND, int NB, int RING = Geo<KIND>::RING>
int32_t launch_i8(bhd_ctx* ctx, const bhd_weight* w, const DecodeI8Params& p, uint32_t tiles, cudaStream_t s) {
    constexpr int W_BYTES = ROWS * Geo<KIND>::BOX;
    constexpr int STAGE = (W_BYTES + 127) / 128 * 128;
    constexpr size_t DYN = size_t(WARPS) * RING * STAGE + 128;
    auto kern = k_matvec_decode_i8<KIND, NB, RING>;
    static int cached_device = -1;
    if (cached_device != ctx->device) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(DYN)), "raising the shared memory limit");
        cached_device = ctx->device;
    }
    CUtensorMap map;
    memcpy(&map, w->tmap16, sizeof(map));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = DYN;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, map, p), "launching the integer decode matvec kernel");
    ctx->launches += 1;
    return BHD_OK;
}

}  // namespace

// Decode path of bhd_matvec for one or two activation vectors.
int32_t bhd_launch_matvec_decode_i8(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                    uint32_t batch, float scale, int accumulate, cudaStream_t s, bool* handled) {
    *handled = false;
    if (!w->tmap16_ok || batch == 0 || batch > 2 || w->cols == 0 || w->rows > 0x7fffffffull) return BHD_OK;
    if (w->kind != BHD_TYPE_Q8_0 && w->kind != BHD_TYPE_Q4_K && w->kind != BHD_TYPE_Q6_K) return BHD_OK;
    const uint32_t chunks = uint32_t((w->cols + CHUNK_K - 1) / CHUNK_K);
    const uint32_t tiles = uint32_t((w->rows + ROWS - 1) / ROWS);
    const int nb = int(batch);
    int32_t st = bhd_ensure_workspace(ctx, size_t(chunks) * iblob_bytes(w->kind, nb), s);
    if (st != BHD_OK) return st;
    uint8_t* blob = ctx->workspace;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(chunks);
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_pack_x_i8, w->kind, x, batch, uint32_t(nb), uint32_t(w->cols), blob, ctx->status_dev),
                 "launching the activation packing kernel");
        ctx->launches += 1;
    }
    DecodeI8Params p;
    p.blob = blob;
    p.y = y;
    p.status = ctx->status_dev;
    p.rows = uint32_t(w->rows);
    p.row_base = uint32_t(slab * w->rows);
    p.chunks = chunks;
    p.batch = batch;
    p.scale = scale;
    p.accumulate = accumulate;
#define BHD_CASE(K)                                                 \
    case K:                                                         \
        if (nb == 1) st = launch_i8<K, 1>(ctx, w, p, tiles, s);     \
        else st = launch_i8<K, 2>(ctx, w, p, tiles, s);             \
        break;
    switch (w->kind) {
        BHD_CASE(BHD_TYPE_Q8_0)
        BHD_CASE(BHD_TYPE_Q4_K)
        BHD_CASE(BHD_TYPE_Q6_K)
        default: return BHD_OK;
    }
#undef BHD_CASE
    if (st != BHD_OK) return st;
    *handled = true;
    return BHD_OK;
}
