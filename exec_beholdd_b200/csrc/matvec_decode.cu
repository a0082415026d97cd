// Decode matvec (1, 2 or 4 activation vectors) for packed Q8_0 / Q4_K / Q6_K on sm_100a.
//
// HBM-bound by design; the job of the kernel is to spend as few issue slots per packed byte
// as possible while keeping many bytes in flight.
//
//   * One CTA owns 16 rows and ALL columns; its four warps take every fourth 256-column
//     chunk. Nothing is exchanged between CTAs: the warps add their partial sums through
//     shared memory in a fixed order, so results are bit-identical from run to run.
//   * Every warp runs its own ring: lane 0 issues one TMA copy of the warp's next
//     16-row x 256-column chunk (272 / 144 / 240 bytes per row, checkpoint layout, via a 2-D
//     tensor map) plus one bulk copy of that chunk's packed activations, and the warp waits on
//     its own mbarrier. No producer warp, no CTA-wide synchronisation in the loop.
//   * Quants become fp16 bit patterns with logic ops only (0x6400 | q = 1024 + q) and go to
//     mma.sync m16n8k16 as the 16-row operand.
//   * The B operand is "diagonal": the 8 MMA columns are (scale group, vector, hi/lo half)
//     and a k-step only feeds the columns of its own scale group. The accumulator tile
//     therefore holds one partial sum per scale group, and the block scales, mins and the
//     1024-offset are applied ONCE per superblock, each lane of a quad handling the groups
//     whose columns it owns -- no per-group post-processing, no redundant scale decoding.
//   * Activations are split x = hi + lo in fp16 (relative error 2^-22), products are exact,
//     accumulation is f32.
//
// Reference semantics: crates/beholdd-backend/src/cpu.rs:398-507; block formats:
// crates/beholdd-kernel/src/kquant.rs:29-241.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int ROWS = 16;        // rows per CTA
constexpr int WARPS = 4;        // warps per CTA, each on its own column chunks
constexpr int CHUNK_K = 256;
constexpr int STEPS = 16;
constexpr int RING = 2;         // stages in flight per warp (many small CTAs per SM keep the total deep)
constexpr uint32_t SPIN_LIMIT = 1u << 22;

template <uint32_t KIND> struct Geo;
template <> struct Geo<BHD_TYPE_Q8_0> { static constexpr int BOX = 272, GROUPS = 8; };
template <> struct Geo<BHD_TYPE_Q4_K> { static constexpr int BOX = 144, GROUPS = 8; };
template <> struct Geo<BHD_TYPE_Q6_K> { static constexpr int BOX = 240, GROUPS = 16; };

__host__ __device__ constexpr int dgroups(uint32_t kind) { return kind == BHD_TYPE_Q6_K ? 16 : 8; }
// Packed activations of one chunk: [step][vector][hi|lo][t] 8-byte fragments, then
// [group][vector] f32 sums of (hi + lo), then 64 zero bytes that inactive lanes read.
__host__ __device__ constexpr int dblob_frag_bytes(int nb) { return STEPS * nb * 64; }
__host__ __device__ constexpr int dblob_bytes(uint32_t kind, int nb) {
    return (dblob_frag_bytes(nb) + dgroups(kind) * nb * 4 + 64 + 127) / 128 * 128;
}

// Columns (within a chunk) that lane-in-quad t supplies to k-step s: four consecutive ones
// starting here. Must match the byte positions the unpackers read.
__host__ __device__ __forceinline__ int chunk_k4(uint32_t kind, int s, int t) {
    if (kind == BHD_TYPE_Q8_0) return 32 * (s >> 1) + 16 * (s & 1) + 4 * t;
    if (kind == BHD_TYPE_Q4_K) {
        const int j = s >> 1, hs = s & 1;
        return 64 * (j >> 1) + 32 * (j & 1) + 8 * t + 4 * hs;
    }
    return 128 * (s >> 3) + 32 * ((s & 7) >> 1) + 16 * (s & 1) + 4 * t;
}
// Scale group of k-step s.
__host__ __device__ __forceinline__ int step_group(uint32_t kind, int s) { return kind == BHD_TYPE_Q6_K ? s : (s >> 1); }

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
__device__ __forceinline__ void mma_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}
__device__ __forceinline__ void mma_new(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y), "f"(0.0f));
}
// Shared-memory loads by 32-bit shared address: keeps all address arithmetic in 32 bits.
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
__device__ __forceinline__ float ldsf(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float h2f(uint32_t h) { return __half2float(__ushort_as_half(uint16_t(h))); }
// Small unsigned integer (< 2^23) in the low bits of v -> float, without the conversion pipe.
__device__ __forceinline__ float u2f(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.0f; }

// ---- activation packer ----------------------------------------------------------------------
// One CTA per chunk. x [nb x K] f32 -> fragments [step][v][hi|lo][t] and per-(group, v) sums.
// Programmatic dependent launch (no-ops when the kernel was launched without the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__global__ void k_pack_x_decode(uint32_t kind, const float* __restrict__ x, uint32_t nvec, uint32_t nb, uint32_t K,
                                uint8_t* __restrict__ blob, uint32_t* __restrict__ status) {
    __shared__ float stepsum[STEPS][4];
    // let the matvec kernel start its weight prefetch; wait for whatever produced x and for the
    // previous matvec, which may still be reading the blob
    pdl_launch_dependents();
    pdl_wait();
    const int chunk = blockIdx.x;
    const int s = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = lane & 3, v = lane >> 2;  // lanes 4v..4v+3 handle vector v (v < nb <= 4); other lanes idle
    uint8_t* cb = blob + uint64_t(chunk) * dblob_bytes(kind, nb);
    float sum = 0.f;
    if (v < int(nb)) {
        const uint32_t k4 = uint32_t(chunk) * CHUNK_K + chunk_k4(kind, s, t);
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k4 < K && v < int(nvec)) f = *reinterpret_cast<const float4*>(x + uint64_t(v) * K + k4);
        const float e[4] = {f.x, f.y, f.z, f.w};
        uint32_t hi[4], lo[4];
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half h = __float2half_rn(e[i]);
            const float hf = __half2float(h);
            bad |= !(fabsf(hf) <= 65504.0f);
            const __half l = __float2half_rn(e[i] - hf);
            hi[i] = __half_as_ushort(h);
            lo[i] = __half_as_ushort(l);
            sum += hf + __half2float(l);
        }
        if (bad) atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
        uint2 fh, fl;
        if (kind == BHD_TYPE_Q4_K) {  // its unpacking yields the four columns in the order 0,2,1,3
            fh = make_uint2(hi[0] | (hi[2] << 16), hi[1] | (hi[3] << 16));
            fl = make_uint2(lo[0] | (lo[2] << 16), lo[1] | (lo[3] << 16));
        } else {
            fh = make_uint2(hi[0] | (hi[1] << 16), hi[2] | (hi[3] << 16));
            fl = make_uint2(lo[0] | (lo[1] << 16), lo[2] | (lo[3] << 16));
        }
        uint8_t* dst = cb + (s * nb + v) * 64 + t * 8;
        *reinterpret_cast<uint2*>(dst) = fh;
        *reinterpret_cast<uint2*>(dst + 32) = fl;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (t == 0 && v < 4) stepsum[s][v] = sum;
    __syncthreads();
    const int groups = dgroups(kind), per = STEPS / groups;
    float* sums = reinterpret_cast<float*>(cb + dblob_frag_bytes(nb));
    if (int(threadIdx.x) < groups * int(nb)) {
        const int grp = threadIdx.x / nb, vv = threadIdx.x % nb;
        float acc = 0.f;
        for (int i = 0; i < per; ++i) acc += stepsum[grp * per + i][vv];
        sums[grp * nb + vv] = acc;
    }
    if (threadIdx.x < 16) reinterpret_cast<uint32_t*>(cb + dblob_frag_bytes(nb) + groups * nb * 4)[threadIdx.x] = 0u;
}

struct DecodeParams {
    const uint8_t* blob;
    float* y;
    uint32_t* status;
    uint32_t rows, row_base, chunks, batch;
    float scale;
    int accumulate;
    int pdl;  // launch with programmatic stream serialization (host-side switch only)
};

template <uint32_t KIND>
__device__ __forceinline__ int tile_row(int m) {
    if (KIND == BHD_TYPE_Q4_K) return m < 8 ? 2 * m : 2 * (m - 8) + 1;  // keeps 8-byte reads conflict-free
    return m;
}

// NB vectors; GPT = 4 / NB scale groups share one accumulator tile; lane-in-quad t owns
// tile columns (2t, 2t+1) = (group gl = t / NB, vector v = t % NB) x (hi, lo).
template <uint32_t KIND, int NB>
__global__ void __launch_bounds__(WARPS * 32) k_matvec_decode(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
    constexpr int BOX = Geo<KIND>::BOX, GROUPS = Geo<KIND>::GROUPS, GPT = 4 / NB, TILES = GROUPS / GPT;
    constexpr int W_BYTES = ROWS * BOX, X_BYTES = dblob_bytes(KIND, NB);
    constexpr int STAGE = (W_BYTES + X_BYTES + 127) / 128 * 128;
    constexpr int FRAG = dblob_frag_bytes(NB);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    __shared__ uint64_t bars[WARPS][RING];
    __shared__ float red[WARPS][ROWS][NB];
    __shared__ __align__(16) uint8_t zero_area[STEPS * NB * 64 + 64];  // what inactive lanes feed the MMA

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t tile = blockIdx.x;
    for (int i = threadIdx.x; i < int(sizeof(zero_area) / 4); i += blockDim.x) reinterpret_cast<uint32_t*>(zero_area)[i] = 0u;
    if (lane == 0) {
        for (int i = 0; i < RING; ++i) mbar_init(&bars[warp][i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint8_t* ring = smem + warp * (RING * STAGE);
    const uint32_t ring32 = smem_u32(ring);
    const uint32_t zeros32 = smem_u32(zero_area);
    const uint32_t my_chunks = p.chunks > uint32_t(warp) ? (p.chunks - warp + WARPS - 1) / WARPS : 0;
    // lane 0 only: stage the warp's i-th chunk; weights and packed activations are separate
    // copies on the same barrier, so that the first weights can be requested before the
    // activation packer has finished (weights are never written by a preceding kernel).
    auto issue_w = [&](uint32_t i) {
        const uint32_t chunk = warp + i * WARPS, slot = i % RING;
        mbar_arrive_expect_tx(&bars[warp][slot], W_BYTES + X_BYTES);
        const uint32_t byte0 = (KIND == BHD_TYPE_Q6_K) ? ((210u * chunk) & ~15u) : uint32_t(BOX) * chunk;
        tma_load_2d(ring + slot * STAGE, &tmap, int(byte0 >> 1), int(p.row_base + tile * ROWS), &bars[warp][slot]);
    };
    auto issue_x = [&](uint32_t i) {
        const uint32_t chunk = warp + i * WARPS, slot = i % RING;
        bulk_load_1d(ring + slot * STAGE + W_BYTES, p.blob + uint64_t(chunk) * X_BYTES, X_BYTES, &bars[warp][slot]);
    };
    if (lane == 0)
        for (uint32_t i = 0; i < my_chunks && i < RING; ++i) issue_w(i);
    pdl_launch_dependents();
    pdl_wait();  // the packer (and before it whatever produced x and y) has finished
    if (lane == 0)
        for (uint32_t i = 0; i < my_chunks && i < RING; ++i) issue_x(i);

    const int r0 = tile_row<KIND>(g), r1 = tile_row<KIND>(g + 8);
    const int gl = t / NB, v = t % NB;            // what this lane's accumulator columns mean
    const int bv = (g >> 1) % NB, bgl = (g >> 1) / NB;  // what this lane's B column (n = g) means
    const int boff = bv * 64 + (g & 1) * 32 + t * 8;    // fragment offset within a step
    float tot0 = 0.f, tot1 = 0.f;                 // rows r0 / r1, vector v, groups handled by this lane

    for (uint32_t i = 0; i < my_chunks; ++i) {
        const uint32_t slot = i % RING, chunk = warp + i * WARPS;
        if (!mbar_wait(&bars[warp][slot], (i / RING) & 1)) {
            if (lane == 0) atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT);
            break;
        }
        const uint32_t st = ring32 + slot * STAGE;
        const uint32_t w0 = st + r0 * BOX, w1 = st + r1 * BOX;
        const uint32_t xb = st + W_BYTES;
        const uint32_t sums = xb + FRAG + 4 * v;  // + 4 * NB * group
        // Where this lane reads its B fragments: the staged activations when the step's group
        // is the one its column stands for, an all-zero area otherwise. Steps add a constant.
        uint32_t bsrc[GPT];
#pragma unroll
        for (int c = 0; c < GPT; ++c) bsrc[c] = (c == bgl) ? xb + boff : zeros32;
        auto bfrag = [&](int s) -> uint2 { return lds64(bsrc[step_group(KIND, s) % GPT] + s * (64 * NB)); };
        float acc[TILES][4];

        if constexpr (KIND == BHD_TYPE_Q8_0) {
#pragma unroll
            for (int blk = 0; blk < 8; ++blk) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int off = 34 * blk + 2 + 16 * h + 4 * t;
                    uint32_t q0, q1;
                    if (blk & 1) {
                        q0 = lds32(w0 + off);
                        q1 = lds32(w1 + off);
                    } else {
                        q0 = __funnelshift_r(lds32(w0 + off - 2), lds32(w0 + off + 2), 16);
                        q1 = __funnelshift_r(lds32(w1 + off - 2), lds32(w1 + off + 2), 16);
                    }
                    q0 ^= 0x80808080u;  // 0x6400 | (q + 128) is the fp16 q + 1152
                    q1 ^= 0x80808080u;
                    const uint32_t a0 = __byte_perm(q0, 0x64646464u, 0x4140), a2 = __byte_perm(q0, 0x64646464u, 0x4342);
                    const uint32_t a1 = __byte_perm(q1, 0x64646464u, 0x4140), a3 = __byte_perm(q1, 0x64646464u, 0x4342);
                    const int s = 2 * blk + h, tl = blk / GPT;
                    if (h == 0 && blk % GPT == 0) mma_new(acc[tl], a0, a1, a2, a3, bfrag(s));
                    else mma_acc(acc[tl], a0, a1, a2, a3, bfrag(s));
                }
            }
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const int blk = tl * GPT + gl;  // the block whose sums sit in this lane's columns
                const float d0 = h2f(lds16(w0 + 34 * blk));
                const float d1 = h2f(lds16(w1 + 34 * blk));
                const float sx = ldsf(sums + 4 * NB * blk);
                tot0 = fmaf(d0, fmaf(-1152.f, sx, acc[tl][0] + acc[tl][1]), tot0);
                tot1 = fmaf(d1, fmaf(-1152.f, sx, acc[tl][2] + acc[tl][3]), tot1);
            }
        } else if constexpr (KIND == BHD_TYPE_Q4_K) {
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                const uint2 q0 = lds64(w0 + 16 + 32 * pp + 8 * t);
                const uint2 q1 = lds64(w1 + 16 + 32 * pp + 8 * t);
#pragma unroll
                for (int nib = 0; nib < 2; ++nib) {
                    const int j = 2 * pp + nib, tl = j / GPT;
#pragma unroll
                    for (int hs = 0; hs < 2; ++hs) {
                        const uint32_t u0 = hs ? q0.y : q0.x, u1 = hs ? q1.y : q1.x;
                        uint32_t a0, a1, a2, a3;
                        if (nib == 0) {  // 0x6400 | q = 1024 + q
                            a0 = (u0 & 0x000F000Fu) | 0x64006400u; a2 = ((u0 >> 8) & 0x000F000Fu) | 0x64006400u;
                            a1 = (u1 & 0x000F000Fu) | 0x64006400u; a3 = ((u1 >> 8) & 0x000F000Fu) | 0x64006400u;
                        } else {         // 0x5400 | (q << 4) = 64 + q
                            a0 = (u0 & 0x00F000F0u) | 0x54005400u; a2 = ((u0 >> 8) & 0x00F000F0u) | 0x54005400u;
                            a1 = (u1 & 0x00F000F0u) | 0x54005400u; a3 = ((u1 >> 8) & 0x00F000F0u) | 0x54005400u;
                        }
                        const int s = 2 * j + hs;
                        if (hs == 0 && j % GPT == 0) mma_new(acc[tl], a0, a1, a2, a3, bfrag(s));
                        else mma_acc(acc[tl], a0, a1, a2, a3, bfrag(s));
                    }
                }
            }
            // Scales and mins of the sub-blocks this lane owns: j = tl * GPT + gl.
            const uint4 h0 = lds128(w0);
            const uint4 h1 = lds128(w1);
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
                const int j = tl * GPT + gl;          // runtime (depends on the lane)
                const int hi4 = (tl * GPT) >> 2;      // compile-time: which half of the eight sub-blocks
                const uint32_t sh = 8u * uint32_t(j & 3);
                const float sc0 = u2f((f0[2 * hi4] >> sh) & 0xffu), mn0 = u2f((f0[2 * hi4 + 1] >> sh) & 0xffu);
                const float sc1 = u2f((f1[2 * hi4] >> sh) & 0xffu), mn1 = u2f((f1[2 * hi4 + 1] >> sh) & 0xffu);
                const float off = (j & 1) ? 64.f : 1024.f;
                const float ds0 = d0 * sc0, ds1 = d1 * sc1;
                const float sx = ldsf(sums + 4 * NB * j);
                tot0 += fmaf(ds0, acc[tl][0] + acc[tl][1], -fmaf(ds0, off, m0 * mn0) * sx);
                tot1 += fmaf(ds1, acc[tl][2] + acc[tl][3], -fmaf(ds1, off, m1 * mn1) * sx);
            }
        } else {  // Q6_K
            const uint32_t q6_off = (210u * chunk) & 15u;  // where the superblock starts in the staged window
            const uint32_t shb = 8u * (q6_off & 3u);
            const uint32_t b0 = w0 + (q6_off & ~3u);
            const uint32_t b1 = w1 + (q6_off & ~3u);
            auto word = [&](uint32_t base, int byte_off) -> uint32_t {
                return __funnelshift_r(lds32(base + byte_off), lds32(base + byte_off + 4), shb);
            };
            // The loop below follows the packed planes, not the tile order, so tiles start at zero.
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) acc[tl][0] = acc[tl][1] = acc[tl][2] = acc[tl][3] = 0.f;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                for (int lam = 0; lam < 2; ++lam) {
                    const uint32_t qh0 = word(b0, 128 + 32 * hf + 16 * lam + 4 * t), qh1 = word(b1, 128 + 32 * hf + 16 * lam + 4 * t);
#pragma unroll
                    for (int gp = 0; gp < 2; ++gp) {
                        const uint32_t ql0 = word(b0, 64 * hf + 32 * gp + 16 * lam + 4 * t), ql1 = word(b1, 64 * hf + 32 * gp + 16 * lam + 4 * t);
#pragma unroll
                        for (int up = 0; up < 2; ++up) {
                            const int grp = gp + 2 * up, s = 8 * hf + 2 * grp + lam, tl = s / GPT;
                            const uint32_t c0 = ((ql0 >> (4 * up)) & 0x0F0F0F0Fu) | (((qh0 >> (2 * grp)) & 0x03030303u) << 4);
                            const uint32_t c1 = ((ql1 >> (4 * up)) & 0x0F0F0F0Fu) | (((qh1 >> (2 * grp)) & 0x03030303u) << 4);
                            const uint32_t a0 = __byte_perm(c0, 0x64646464u, 0x4140), a2 = __byte_perm(c0, 0x64646464u, 0x4342);
                            const uint32_t a1 = __byte_perm(c1, 0x64646464u, 0x4140), a3 = __byte_perm(c1, 0x64646464u, 0x4342);
                            mma_acc(acc[tl], a0, a1, a2, a3, bfrag(s));
                        }
                    }
                }
            }
            const float d0 = h2f(word(b0, 208) & 0xffffu), d1 = h2f(word(b1, 208) & 0xffffu);
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const int s = tl * GPT + gl;  // scale group == step index
                const uint32_t sw0 = word(b0, 192 + (s & ~3)), sw1 = word(b1, 192 + (s & ~3));
                const float s0 = d0 * float(int8_t((sw0 >> (8 * (s & 3))) & 0xffu));
                const float s1 = d1 * float(int8_t((sw1 >> (8 * (s & 3))) & 0xffu));
                const float sx = ldsf(sums + 4 * NB * s);
                tot0 = fmaf(s0, fmaf(-1056.f, sx, acc[tl][0] + acc[tl][1]), tot0);  // codes carry 1024 + c; value is c - 32
                tot1 = fmaf(s1, fmaf(-1056.f, sx, acc[tl][2] + acc[tl][3]), tot1);
            }
        }
        __syncwarp();
        if (lane == 0 && i + RING < my_chunks) {
            issue_w(i + RING);
            issue_x(i + RING);
        }
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int box_of(uint32_t kind) {
    switch (kind) {
        case BHD_TYPE_Q8_0: return Geo<BHD_TYPE_Q8_0>::BOX;
        case BHD_TYPE_Q4_K: return Geo<BHD_TYPE_Q4_K>::BOX;
        case BHD_TYPE_Q6_K: return Geo<BHD_TYPE_Q6_K>::BOX;
        default: return 0;
    }
}

template <uint32_t KIND, int NB>
int32_t launch_decode(bhd_ctx* ctx, const bhd_weight* w, const DecodeParams& p, uint32_t tiles, cudaStream_t s) {
    constexpr int W_BYTES = ROWS * Geo<KIND>::BOX, X_BYTES = dblob_bytes(KIND, NB);
    constexpr int STAGE = (W_BYTES + X_BYTES + 127) / 128 * 128;
    constexpr size_t DYN = size_t(WARPS) * RING * STAGE + 128;
    auto kern = k_matvec_decode<KIND, NB>;
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(DYN)), "raising the shared memory limit");
        once.mark(ctx);
    }
    CUtensorMap map;
    memcpy(&map, w->tmap16, sizeof(map));
    if (p.pdl) {
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
        BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, map, p), "launching the decode matvec kernel");
        ctx->launches += 1;
        return BHD_OK;
    }
    kern<<<tiles, WARPS * 32, DYN, s>>>(map, p);
    BHD_LAUNCHED(ctx, "decode matvec kernel");
    return BHD_OK;
}

}  // namespace

// Tensor map with a 16-row box for the decode kernel.
void bhd_weight_build_tensor_map16(bhd_ctx* ctx, bhd_weight* w) {
    w->tmap16_ok = false;
    const int box = box_of(w->kind);
    if (!box || !ctx->tmap_encode || w->rows == 0 || w->cols == 0) return;
    if (w->row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(w->dev) & 15) != 0) return;
    const uint64_t total_rows = w->rows * w->slabs;
    if (total_rows > 0x7fffffffull || w->row_bytes / 2 > 0x7fffffffull) return;
    CUtensorMap map;
    const cuuint64_t dims[2] = {w->row_bytes / 2, total_rows};
    const cuuint64_t strides[1] = {w->row_bytes};
    const cuuint32_t boxdim[2] = {cuuint32_t(box / 2), cuuint32_t(ROWS)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode)(
        &map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, boxdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return;
    memcpy(w->tmap16, &map, sizeof(map));
    w->tmap16_ok = true;
}

// Decode path of bhd_matvec for 1..4 activation vectors (3 runs as 4 with a zero vector).
int32_t bhd_launch_matvec_decode(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                 uint32_t batch, float scale, int accumulate, cudaStream_t s, bool* handled) {
    *handled = false;
    if (!w->tmap16_ok || batch == 0 || batch > 4 || w->cols == 0 || w->cols % 4 != 0) return BHD_OK;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || w->rows > 0x7fffffffull) return BHD_OK;
    const uint32_t chunks = uint32_t((w->cols + CHUNK_K - 1) / CHUNK_K);
    const uint32_t tiles = uint32_t((w->rows + ROWS - 1) / ROWS);
    // Two Q8_0 vectors run faster through the four-vector variant (measured), as do three of any format.
    const int nb = (batch == 3 || (batch == 2 && w->kind == BHD_TYPE_Q8_0)) ? 4 : int(batch);
    const size_t blob_bytes = size_t(chunks) * dblob_bytes(w->kind, nb);
    int32_t st = bhd_ensure_workspace(ctx, blob_bytes, s);
    if (st != BHD_OK) return st;
    uint8_t* blob = ctx->workspace;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(chunks);
        cfg.blockDim = dim3(STEPS * 32);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_pack_x_decode, w->kind, x, batch, uint32_t(nb), uint32_t(w->cols), blob, ctx->status_dev),
                 "launching the activation packing kernel");
        ctx->launches += 1;
    }
    DecodeParams p;
    p.pdl = 1;
    p.blob = blob;
    p.y = y;
    p.status = ctx->status_dev;
    p.rows = uint32_t(w->rows);
    p.row_base = uint32_t(slab * w->rows);
    p.chunks = chunks;
    p.batch = batch;
    p.scale = scale;
    p.accumulate = accumulate;
#define BHD_CASE(K)                                                      \
    case K:                                                              \
        if (nb == 1) st = launch_decode<K, 1>(ctx, w, p, tiles, s);      \
        else if (nb == 2) st = launch_decode<K, 2>(ctx, w, p, tiles, s); \
        else st = launch_decode<K, 4>(ctx, w, p, tiles, s);              \
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

// ---- decode matvec for callers that must not allocate ------------------------------------------
// Some embedders of this library run where device allocation is off the table once serving has
// started: a real-time decode loop that may not take the allocator's locks or its implicit
// synchronisation, a process whose whole HBM budget was handed to a weight/KV-cache arena at
// start-up, or a host that calls in from inside a stream capture. For them this entry point
// keeps the one piece of scratch the decode matvec needs -- the packed fp16 activations -- in
// a fixed array that is part of the library image instead of the context's growable workspace.
//
// The array costs BHD_NOALLOC_SCRATCH_BYTES of HBM on every GPU that loads the library, for the
// life of the process. It always suffices for cols <= 16384 with up to 4 activation vectors;
// requests whose packed activations do not fit are refused with BHD_ERR_SHAPE rather than
// served some other way.
constexpr size_t BHD_NOALLOC_SCRATCH_BYTES = 288 * 1024;
static __device__ __align__(256) uint8_t g_noalloc_scratch[BHD_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = BHD_MAX_DEVICES;
// Device address of g_noalloc_scratch per CUDA device. In host code the symbol's name is only a
// handle for the runtime, not a device pointer, so the address is looked up once per device.
uint8_t* g_noalloc_ptr[MAX_DEVICES] = {};
}  // namespace

extern "C" __attribute__((visibility("default"))) int32_t bhd_matvec_noalloc(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab,
                                                                             const float* x_dev, float* y_dev, uint32_t batch,
                                                                             float scale, int32_t accumulate, void* stream) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (!w || w->magic != BHD_WEIGHT_MAGIC || w->ctx != ctx)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "matvec_noalloc: not a weight of this context");
    if (slab >= w->slabs)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: slab %llu of %llu", (unsigned long long)slab,
                        (unsigned long long)w->slabs);
    if (!isfinite(scale)) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "matvec_noalloc: scale must be finite");
    if (batch == 0 || w->rows == 0) return BHD_OK;
    if (!x_dev || !y_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "matvec_noalloc: null buffer");
    if (batch > 4)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: matvec_noalloc serves at most 4 activation vectors, got %u", batch);
    bhd_device_guard guard(ctx);  // the context's GPU is current for the rest of the call, the caller's afterwards
    cudaStream_t s = cudaStream_t(stream);
    const bool tma_path = w->tmap16_ok && w->cols != 0 && w->cols % 4 == 0 && (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0 &&
                          w->rows <= 0x7fffffffull;
    if (!tma_path)  // the general kernels need no scratch at all
        return bhd_launch_matvec_general(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s);
    const uint32_t chunks = uint32_t((w->cols + CHUNK_K - 1) / CHUNK_K);
    const uint32_t tiles = uint32_t((w->rows + ROWS - 1) / ROWS);
    const int nb = batch == 3 ? 4 : int(batch);
    const size_t need = size_t(chunks) * dblob_bytes(w->kind, nb);
    if (need > BHD_NOALLOC_SCRATCH_BYTES)
        return bhd_fail(ctx, BHD_ERR_SHAPE,
                        "shape mismatch: matvec_noalloc needs %zu bytes of scratch for %llu columns x %u vectors, the fixed "
                        "array holds %zu (cols <= 16384)",
                        need, (unsigned long long)w->cols, batch, BHD_NOALLOC_SCRATCH_BYTES);
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "matvec_noalloc: device index %d out of range", ctx->device);
    if (!g_noalloc_ptr[ctx->device]) {
        // First call on this device: resolve the array's device address (the guard above made the device current).
        void* p = nullptr;
        BHD_CUDA(ctx, cudaGetSymbolAddress(&p, g_noalloc_scratch), "resolving the fixed scratch array");
        g_noalloc_ptr[ctx->device] = static_cast<uint8_t*>(p);
    }
    uint8_t* blob = g_noalloc_ptr[ctx->device];
    // The packer rewrites every byte the matvec reads (fragments, sums and zero padding), so the
    // previous call's contents never leak into this one.
    k_pack_x_decode<<<chunks, STEPS * 32, 0, s>>>(w->kind, x_dev, batch, uint32_t(nb), uint32_t(w->cols), blob, ctx->status_dev);
    BHD_LAUNCHED(ctx, "activation packing kernel");
    DecodeParams p;
    p.pdl = 0;
    p.blob = blob;
    p.y = y_dev;
    p.status = ctx->status_dev;
    p.rows = uint32_t(w->rows);
    p.row_base = uint32_t(slab * w->rows);
    p.chunks = chunks;
    p.batch = batch;
    p.scale = scale;
    p.accumulate = accumulate;
    int32_t st = BHD_OK;
#define BHD_CASE(K)                                                      \
    case K:                                                              \
        if (nb == 1) st = launch_decode<K, 1>(ctx, w, p, tiles, s);      \
        else if (nb == 2) st = launch_decode<K, 2>(ctx, w, p, tiles, s); \
        else st = launch_decode<K, 4>(ctx, w, p, tiles, s);              \
        break;
    switch (w->kind) {
        BHD_CASE(BHD_TYPE_Q8_0)
        BHD_CASE(BHD_TYPE_Q4_K)
        BHD_CASE(BHD_TYPE_Q6_K)
        default: return bhd_launch_matvec_general(ctx, w, slab, x_dev, y_dev, batch, scale, accumulate, s);
    }
#undef BHD_CASE
    return st;
}
