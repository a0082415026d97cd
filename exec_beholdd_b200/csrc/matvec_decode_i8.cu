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
//     of two s and a 15- to 16-bit integer X = round(x / s), |X| <= 32639, split into two signed
//     bytes, X = 256 * d0 + d1. The two digits sit in adjacent MMA columns; the s32 accumulators
//     are combined exactly (256 * c0 + c1) and scaled by s and the block scale in f32. Relative
//     error at most 2^-15 of the largest activation of the group; any finite f32 is accepted.
//
// Reference semantics: crates/beholdd-backend/src/cpu.rs:398-507; block formats:
// crates/beholdd-kernel/src/kquant.rs:29-241.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int ROWS = 16, WARPS = 4, CHUNK_K = 256;
constexpr int MAX_X_SMEM = 16 * 1024; // packed activations a CTA may hold
constexpr uint32_t SPIN_LIMIT = 1u << 22;

template <uint32_t KIND> struct Geo;
// RING: stages per warp. Four stages of Q4_K hold all 4096 columns of a projection, so a CTA
// that starts early (programmatic dependent launch) has requested all its weights before the
// activations exist; the wider formats keep two stages to leave room for six CTAs per SM.
// CLUSTER: CTAs that share one packing of the activations. Two measured fastest for Q4_K (8.6 us
// against 9.0 with four and 9.2 with eight per 12288x4096 matvec); the wider formats keep four
// and two vectors keep four so that the packed activations leave room for six CTAs per SM.
template <> struct Geo<BHD_TYPE_Q8_0> { static constexpr int BOX = 272, GROUPS = 8, RING = 2; };
template <> struct Geo<BHD_TYPE_Q4_K> { static constexpr int BOX = 144, GROUPS = 8, RING = 3; };
template <> struct Geo<BHD_TYPE_Q6_K> { static constexpr int BOX = 240, GROUPS = 16, RING = 2; };
__host__ __device__ constexpr int cluster_of(uint32_t kind, int nb) { return (kind == BHD_TYPE_Q4_K && nb == 1) ? 2 : 4; }
__host__ __device__ constexpr int igroups(uint32_t kind) { return kind == BHD_TYPE_Q6_K ? 16 : 8; }

// Packed activations of one chunk: [group][vector][digit][t] 8-byte B fragments (b0, b1), then
// [group][vector] f32 pairs (the group's factor s, sum of the dequantised activations of the group).
__host__ __device__ constexpr int iblob_frag_bytes(uint32_t kind, int nb) { return igroups(kind) * nb * 64; }
__host__ __device__ constexpr int iblob_bytes(uint32_t kind, int nb) {
    return (iblob_frag_bytes(kind, nb) + igroups(kind) * nb * 8 + 127) / 128 * 128;
}

// Column (within the chunk) behind k-slot `slot` (0..31) of the MMA that covers scale group
// `grp`:
//   Q8_0: 32 * grp + slot (the block's bytes in order);
//   Q4_K: 64 * (grp / 2) + 32 * (grp % 2) + 8 * t + 4 * hi + i with t = (slot % 16) / 4,
//         i = slot % 4, hi = slot / 16 (a lane's eight bytes are split over the two halves of k);
//   Q6_K: a k32 MMA spans two 16-column groups, the even one in slots 0..15 and the odd one in
//         slots 16..31: 16 * grp + slot % 16.
// In every format the bytes behind B-fragment registers b0 (slots 4t..4t+3) and b1 (slots
// 16+4t..16+4t+3) of lane-in-quad t are runs of four consecutive columns.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = SPIN_LIMIT) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < limit; ++spin) {
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
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
// Distributed shared memory: the address of `local` (a shared-memory address of this CTA) in
// the CTA of rank `rank` of the cluster, and an 8-byte load from such an address.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ uint2 ld_cluster64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared::cluster.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Publishes this CTA's shared-memory writes to the cluster and waits for everyone else's. The
// CTA barrier makes all threads' writes visible to thread 0, whose single cluster-scope fence
// then covers them (cumulativity); one fence per CTA is much cheaper than one per thread.
__device__ __forceinline__ void cluster_sync() {
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("fence.acq_rel.cluster;" ::: "memory");
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Rendezvous that publishes nothing (no fence): used only to keep shared memory alive until
// every CTA of the cluster has finished reading it.
__device__ __forceinline__ void cluster_rendezvous() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
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

// ---- activation packer (runs inside the matvec kernel, once per cluster) --------------------
// The CTAs of a cluster split the chunks between them; each packs its share into its own shared
// memory and every CTA of the cluster reads the fragments it needs through distributed shared
// memory. One quad of lanes packs one (group, vector) item: lane t of the quad holds exactly
// the columns behind its own B-fragment registers (see slot_column), so no bytes cross lanes.
// x [nvec x K] f32; dst = this CTA's packed chunks [n_local][iblob_bytes].
template <uint32_t KIND, int NB>
__device__ __forceinline__ void pack_chunks(const float* __restrict__ x, uint32_t nvec, uint32_t K, uint32_t chunk0,
                                            uint32_t chunk_stride, uint32_t run, uint32_t n_local, uint32_t chunks,
                                            uint8_t* dst, uint32_t* status) {
    constexpr int GROUPS = igroups(KIND), X_BYTES = iblob_bytes(KIND, NB), FRAG = iblob_frag_bytes(KIND, NB);
    constexpr int ITEMS = GROUPS * NB;  // per chunk
    static_assert(ITEMS % 8 == 0, "whole warps must run the same number of passes (full-mask shuffles below)");
    const int quad = threadIdx.x >> 2, t = threadIdx.x & 3, nquads = blockDim.x >> 2;
    const bool vec_ok = (K & 3u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    for (uint32_t it = quad; it < n_local * ITEMS; it += nquads) {
        // local chunk lc -> chunk: runs of `run` consecutive chunks, `chunk_stride` apart
        const uint32_t lc = it / ITEMS, item = it % ITEMS, chunk = chunk0 + (lc / run) * chunk_stride + lc % run;
        const int grp = int(item) / NB, v = int(item) % NB;
        // columns (within the chunk) behind b0 and b1 of this lane
        int c0, c1;
        if (KIND == BHD_TYPE_Q8_0) { c0 = 32 * grp + 4 * t; c1 = c0 + 16; }
        else if (KIND == BHD_TYPE_Q4_K) { c0 = 64 * (grp >> 1) + 32 * (grp & 1) + 8 * t; c1 = c0 + 4; }
        else { c0 = 16 * grp + 4 * t; c1 = -1; }  // Q6_K: the other half of the k range is the neighbouring group
        float val[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) val[i] = 0.f;
        const uint32_t k0 = chunk * CHUNK_K + uint32_t(c0), k1 = chunk * CHUNK_K + uint32_t(c1);
        const bool live = chunk < chunks && uint32_t(v) < nvec;
        const float* xr = x + uint64_t(v) * K;
        if (live && k0 + 3 < K && vec_ok) {
            const float4 f = *reinterpret_cast<const float4*>(xr + k0);
            val[0] = f.x; val[1] = f.y; val[2] = f.z; val[3] = f.w;
        } else if (live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) if (k0 + i < K) val[i] = xr[k0 + i];
        }
        if (c1 >= 0) {
            if (live && k1 + 3 < K && vec_ok) {
                const float4 f = *reinterpret_cast<const float4*>(xr + k1);
                val[4] = f.x; val[5] = f.y; val[6] = f.z; val[7] = f.w;
            } else if (live) {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k1 + i < K) val[4 + i] = xr[k1 + i];
            }
        }
        float mx = 0.f;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (!(fabsf(val[i]) <= 3.0e38f)) { bad = true; val[i] = 0.f; }  // NaN or infinity
            mx = fmaxf(mx, fabsf(val[i]));
        }
        if (bad) atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        // mx = m * 2^ex with m in [0.5, 1): ex = biased exponent - 126. The factor is the power of two that brings the
        // group's largest magnitude just below 2^15, or below 2^14 when that would pass 32639 = 127 * 256 + 127, the
        // largest integer whose two balanced digits both fit a signed byte. A power of two keeps small integers and
        // dyadic fractions exact. Groups whose largest magnitude is below 2^-100 (denormals included) pack as zero.
        const int eb = int(__float_as_uint(mx) >> 23);
        const bool tiny = eb < 27;
        const float up16 = __uint_as_float(uint32_t(268 - eb) << 23);               // 2^(15 - ex)
        const bool wide = !tiny && mx * up16 <= 32639.0f;
        const float up = tiny ? 0.f : (wide ? up16 : __uint_as_float(uint32_t(267 - eb) << 23));
        const float down = tiny ? 0.f : __uint_as_float(uint32_t(wide ? eb - 14 : eb - 13) << 23);
        uint32_t w0[2] = {0u, 0u}, w1[2] = {0u, 0u};  // digit 0 / digit 1 words for b0, b1
        int sumX = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int X = __float2int_rn(val[i] * up);          // |X| <= 32639
            const int d0 = (X + 128) >> 8, d1 = X - d0 * 256;   // X = 256 * d0 + d1, d0 in [-127, 127], d1 in [-128, 127]
            w0[i >> 2] |= (uint32_t(d0) & 0xffu) << (8 * (i & 3));
            w1[i >> 2] |= (uint32_t(d1) & 0xffu) << (8 * (i & 3));
            sumX += X;
        }
        sumX += __shfl_xor_sync(0xffffffffu, sumX, 1);
        sumX += __shfl_xor_sync(0xffffffffu, sumX, 2);
        uint8_t* cb = dst + size_t(lc) * X_BYTES;
        uint2* frag = reinterpret_cast<uint2*>(cb + (grp * NB + v) * 64);
        if (KIND == BHD_TYPE_Q6_K && (grp & 1)) {  // odd groups sit in slots 16..31 of their MMA: b1
            frag[t] = make_uint2(0u, w0[0]);
            frag[4 + t] = make_uint2(0u, w1[0]);
        } else {
            frag[t] = make_uint2(w0[0], w0[1]);
            frag[4 + t] = make_uint2(w1[0], w1[1]);
        }
        if (t == 0) reinterpret_cast<float2*>(cb + FRAG)[grp * NB + v] = make_float2(down, float(sumX) * down);
    }
}

struct DecodeI8Params {
    const float* x;
    float* y;
    uint32_t* status;
    uint32_t rows, row_base, chunks, batch, cols, tiles, chunks_per_cta;
    float scale;
    int accumulate;
    uint32_t spin_limit;  // polls a wait makes before it gives up
    uint32_t drop_copy;   // test hook: warp 0 of tile 0 leaves its first weight copy unrequested, so its wait runs out
};

template <uint32_t KIND>
__device__ __forceinline__ int tile_row(int m) {
    if (KIND == BHD_TYPE_Q4_K) return m < 8 ? 2 * m : 2 * (m - 8) + 1;  // keeps 8-byte reads conflict-free
    return m;
}

// NB vectors; GPT = 4 / NB scale groups share one accumulator tile; lane-in-quad t owns tile
// columns (2t, 2t+1) = (group gl = t / NB, vector v = t % NB) x (digit 0, digit 1).
// KS = 1: a cluster is CLUSTER row tiles sharing one packing of x. KS = 4 (wide rows, few of
// them): a cluster is one row tile cut four ways along the columns -- rank r takes chunks
// c with (c / WARPS) % 4 == r, packs exactly those itself, and rank 0 adds the four partial
// sums in rank order, so the result is as deterministic as without the split.
template <uint32_t KIND, int NB, int RING, int KS>
__global__ void __launch_bounds__(WARPS * 32) k_matvec_decode_i8(const __grid_constant__ CUtensorMap tmap, const DecodeI8Params p) {
    constexpr int BOX = Geo<KIND>::BOX, GROUPS = Geo<KIND>::GROUPS, CLUSTER = KS > 1 ? 1 : cluster_of(KIND, NB), GPT = 4 / NB, TILES = GROUPS / GPT;
    constexpr uint32_t CSTEP = WARPS * KS;  // distance between consecutive chunks of one warp
    constexpr int W_BYTES = ROWS * BOX, X_BYTES = iblob_bytes(KIND, NB), FRAG = iblob_frag_bytes(KIND, NB);
    constexpr int STAGE = (W_BYTES + 127) / 128 * 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    __shared__ uint64_t bars[WARPS][RING];
    __shared__ float red[WARPS][ROWS][NB];
    __shared__ float part[KS][ROWS * NB];  // rank 0's copy receives the partial sums of all ranks

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t rank = cluster_rank();
    const uint32_t tile = blockIdx.x / KS;  // KS = 1: the grid is padded to whole clusters, tiles beyond the matrix only pack
    const uint32_t first = uint32_t(warp) + (KS > 1 ? WARPS * rank : 0u);  // this warp's first chunk
    if (lane == 0) {
        for (int i = 0; i < RING; ++i) mbar_init(&bars[warp][i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint8_t* ring = smem + warp * (RING * STAGE);
    const uint32_t ring32 = smem_u32(ring);
    const uint32_t my_chunks = (tile < p.tiles && p.chunks > first) ? (p.chunks - first + CSTEP - 1) / CSTEP : 0;
    // lane 0 only: stage the weights of the warp's i-th chunk.
    auto issue_w = [&](uint32_t i) {
        const uint32_t chunk = first + i * CSTEP, slot = i % RING;
        mbar_arrive_expect_tx(&bars[warp][slot], W_BYTES);
        if (p.drop_copy && i == 0 && warp == 0 && blockIdx.x == 0) return;
        const uint32_t byte0 = (KIND == BHD_TYPE_Q6_K) ? ((210u * chunk) & ~15u) : uint32_t(BOX) * chunk;
        tma_load_2d(ring + slot * STAGE, &tmap, int(byte0 >> 1), int(p.row_base + tile * ROWS), &bars[warp][slot]);
    };
    // Weights are never written by a preceding kernel, so their first stages are requested
    // before waiting for the grids this launch depends on (whatever produced x and y);
    // everything else happens after the wait.
    if (lane == 0)
        for (uint32_t i = 0; i < my_chunks && i < RING; ++i) issue_w(i);
    pdl_launch_dependents();
    pdl_wait();

    uint8_t* xs = smem + WARPS * RING * STAGE;
    if (KS == 1) {
        // Chunk c is packed by the CTA of cluster rank c % CLUSTER, as its local chunk c / CLUSTER.
        pack_chunks<KIND, NB>(p.x, p.batch, p.cols, rank, CLUSTER, 1, p.chunks_per_cta, p.chunks, xs, p.status);
        cluster_sync();
    } else {
        // This CTA packs its own chunks: WARPS consecutive ones every CSTEP; local index = i * WARPS + warp.
        pack_chunks<KIND, NB>(p.x, p.batch, p.cols, WARPS * rank, CSTEP, WARPS, p.chunks_per_cta, p.chunks, xs, p.status);
        __syncthreads();
    }

    const int r0 = tile_row<KIND>(g), r1 = tile_row<KIND>(g + 8);
    const int gl = t / NB, v = t % NB;                  // what this lane's accumulator columns mean
    const int bv = (g >> 1) % NB, bgl = (g >> 1) / NB;  // what this lane's B column (n = g) means
    const int boff = bv * 64 + (g & 1) * 32 + t * 8;    // fragment offset within a group
    float tot0 = 0.f, tot1 = 0.f;

    // The lane's share of a chunk's packed activations, from the shared memory of the CTA that
    // packed it: the B fragments of the TILES groups its MMA column stands for, and
    // (factor, sum) of the TILES groups its accumulator columns stand for. Loaded one chunk ahead.
    uint2 bq[TILES], bq_next[TILES];
    float2 mq[TILES], mq_next[TILES];
    const uint32_t xs32 = smem_u32(xs);
    auto load_x = [&](uint32_t chunk, uint2 (&q)[TILES], float2 (&m)[TILES]) {
        const uint32_t cb = KS == 1 ? map_to_rank(xs32 + (chunk / CLUSTER) * X_BYTES, chunk % CLUSTER)
                                    : map_to_rank(xs32 + ((chunk / CSTEP) * WARPS + chunk % WARPS) * X_BYTES, rank);
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
            q[tl] = ld_cluster64(cb + (tl * GPT + bgl) * (64 * NB) + boff);
            const uint2 mm = ld_cluster64(cb + FRAG + 8 * ((tl * GPT + gl) * NB + v));
            m[tl] = make_float2(__uint_as_float(mm.x), __uint_as_float(mm.y));
        }
    };
    if (my_chunks > 0) load_x(first, bq_next, mq_next);

    for (uint32_t i = 0; i < my_chunks; ++i) {
        const uint32_t slot = i % RING, chunk = first + i * CSTEP;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
            bq[tl] = bq_next[tl];
            mq[tl] = mq_next[tl];
        }
        if (i + 1 < my_chunks) load_x(chunk + CSTEP, bq_next, mq_next);
        if (!mbar_wait(&bars[warp][slot], (i / RING) & 1, p.spin_limit)) {
            if (lane == 0) atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT);
            // Give up on this warp's rows, but not before the copies it has already requested into the other
            // slots of its ring have landed (bounded again): the CTA must not end with copies in flight.
            for (uint32_t j = i + 1; j < my_chunks && j < i + RING; ++j) mbar_wait(&bars[warp][j % RING], (j / RING) & 1, p.spin_limit);
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
            // block scales first (the asm statements keep program order)
            uint32_t dq0[TILES], dq1[TILES];
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                dq0[tl] = lds16(w0 + 34 * (tl * GPT + gl));
                dq1[tl] = lds16(w1 + 34 * (tl * GPT + gl));
            }
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
                const float2 m = mq[tl];
                const float d0 = h2f(dq0[tl]) * m.x, d1 = h2f(dq1[tl]) * m.x;
                tot0 = fmaf(d0, float(acc[tl][0] * 256 + acc[tl][1]), tot0);
                tot1 = fmaf(d1, float(acc[tl][2] * 256 + acc[tl][3]), tot1);
            }
        } else if constexpr (KIND == BHD_TYPE_Q4_K) {
            // the superblock headers are requested first: the asm statements keep program order,
            // so loads placed after the MMAs would be waited for on their own
            const uint4 h0 = lds128(w0), h1 = lds128(w1);
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
                    // high nibbles stay where they are (16 * q, still a u8); the 1/16 is folded into the group's factor below
                    const uint32_t a0 = q0.x & 0xF0F0F0F0u, a1 = q1.x & 0xF0F0F0F0u;
                    const uint32_t a2 = q0.y & 0xF0F0F0F0u, a3 = q1.y & 0xF0F0F0F0u;
                    if (j % GPT == 0) imma<false, true>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                    else imma<false, false>(acc[j / GPT], a0, a1, a2, a3, bfrag(j));
                }
            }
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
                const float mx = (j & 1) ? m.x * 0.0625f : m.x;  // odd sub-blocks were fed as 16 * q
                tot0 += fmaf(d0 * sc0 * mx, float(acc[tl][0] * 256 + acc[tl][1]), -(m0 * mn0) * m.y);
                tot1 += fmaf(d1 * sc1 * mx, float(acc[tl][2] * 256 + acc[tl][3]), -(m1 * mn1) * m.y);
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
    float sum = 0.f;
    const int r = threadIdx.x / NB, vv = threadIdx.x % NB;
    if (threadIdx.x < ROWS * NB) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) sum += red[w][r][vv];
    }
    if (KS > 1) {
        // every rank stores its partial sums into rank 0's `part`, then rank 0 adds them in rank order
        if (threadIdx.x < ROWS * NB) {
            const uint32_t dst = map_to_rank(smem_u32(&part[rank][threadIdx.x]), 0);
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(sum) : "memory");
        }
        cluster_sync();
        if (rank != 0) return;
        sum = 0.f;
        if (threadIdx.x < ROWS * NB) {
#pragma unroll
            for (int k = 0; k < KS; ++k) sum += part[k][threadIdx.x];
        }
    }
    if (threadIdx.x < ROWS * NB) {
        const uint32_t row = tile * ROWS + r;
        if (row < p.rows && uint32_t(vv) < p.batch) {
            const float val = __fmul_rn(sum, p.scale);
            float* o = p.y + uint64_t(vv) * p.rows + row;
            *o = p.accumulate ? __fadd_rn(*o, val) : val;
        }
    }
    if (KS == 1) cluster_rendezvous();  // no CTA may leave while another still reads its packed activations
}

template <uint32_t KIND, int NB, int KS, int RING = Geo<KIND>::RING>
int32_t launch_i8(bhd_ctx* ctx, const bhd_weight* w, const DecodeI8Params& p, cudaStream_t s) {
    constexpr int W_BYTES = ROWS * Geo<KIND>::BOX, CLUSTER = KS > 1 ? KS : cluster_of(KIND, NB);
    constexpr int STAGE = (W_BYTES + 127) / 128 * 128;
    constexpr size_t RING_BYTES = size_t(WARPS) * RING * STAGE + 128;
    auto kern = k_matvec_decode_i8<KIND, NB, RING, KS>;
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(RING_BYTES + MAX_X_SMEM)),
                 "raising the shared memory limit");
        once.mark(ctx);
    }
    CUtensorMap map;
    memcpy(&map, w->tmap16, sizeof(map));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(KS > 1 ? p.tiles * KS : (p.tiles + CLUSTER - 1) / CLUSTER * CLUSTER);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = RING_BYTES + size_t(p.chunks_per_cta) * iblob_bytes(KIND, NB);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CLUSTER;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, map, p), "launching the integer decode matvec kernel");
    ctx->launches += 1;
    return BHD_OK;
}

}  // namespace

// Decode path of bhd_matvec for one or two activation vectors. One launch: the activations are
// packed inside the kernel, once per cluster.
int32_t bhd_launch_matvec_decode_i8(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                    uint32_t batch, float scale, int accumulate, cudaStream_t s, bool* handled) {
    *handled = false;
    if (!w->tmap16_ok || batch == 0 || batch > 2 || w->cols == 0 || w->rows > 0x7fffffffull) return BHD_OK;
    if (w->kind != BHD_TYPE_Q8_0 && w->kind != BHD_TYPE_Q4_K && w->kind != BHD_TYPE_Q6_K) return BHD_OK;
    const uint32_t chunks = uint32_t((w->cols + CHUNK_K - 1) / CHUNK_K);
    const uint32_t tiles = uint32_t((w->rows + ROWS - 1) / ROWS);
    const int nb = int(batch);
    // Three and four vectors (one 8-column MMA per block, measured): 19 us against the fp16 decode kernel's 13 us
    // per 12288x4096 matvec, so they stay there. Where this kernel wins, by measurement on B200: one vector
    // of Q4_K or Q8_0 at every shape tried; one vector of Q6_K, or two of Q4_K, only for tall
    // matrices of up to 4096 columns (rows are not split over CTAs here, so wide rows leave
    // too few CTAs, and the wider operand sets of those variants cost occupancy).
    const bool tall = w->rows >= 8192 && w->cols <= 4096;
    if (nb == 1 && w->kind == BHD_TYPE_Q6_K && !tall) return BHD_OK;
    if (nb == 2 && !(w->kind == BHD_TYPE_Q4_K && tall)) return BHD_OK;
    // Few row tiles and long rows (a down projection, [4096 x 12288]): four CTAs per tile, each a
    // quarter of the columns, so that the grid still fills the GPU.
    // Measured: Q4_K 4096x12288 12.8 -> 11.7 us, 4096x4096 7.1 -> 6.2 us; Q8_0 gains only below
    // about 160 row tiles (2048x8192 7.6 -> 5.8 us, but 4096x12288 13.4 -> 14.5 us).
    const uint32_t ks_tiles = w->kind == BHD_TYPE_Q4_K ? 384u : (w->kind == BHD_TYPE_Q8_0 ? 160u : 0u);
    const bool ksplit = nb == 1 && tiles <= ks_tiles && chunks >= 16;
    const uint32_t cluster = uint32_t(cluster_of(w->kind, nb));
    const uint32_t per_cta = ksplit ? WARPS * ((chunks + WARPS * 4 - 1) / (WARPS * 4)) : (chunks + cluster - 1) / cluster;
    if (size_t(per_cta) * iblob_bytes(w->kind, nb) > size_t(MAX_X_SMEM)) return BHD_OK;  // very wide rows: other paths
    DecodeI8Params p;
    p.x = x;
    p.y = y;
    p.status = ctx->status_dev;
    p.rows = uint32_t(w->rows);
    p.row_base = uint32_t(slab * w->rows);
    p.chunks = chunks;
    p.batch = batch;
    p.cols = uint32_t(w->cols);
    p.tiles = tiles;
    p.chunks_per_cta = per_cta;
    p.scale = scale;
    p.accumulate = accumulate;
    p.spin_limit = ctx->spin_limit ? ctx->spin_limit : SPIN_LIMIT;
    p.drop_copy = ctx->debug_drop;
    ctx->debug_drop = 0;  // one launch only
    int32_t st = BHD_OK;
#define BHD_CASE(K)                                          \
    case K:                                                  \
        if (nb == 1) st = launch_i8<K, 1, 1>(ctx, w, p, s);  \
        else st = launch_i8<K, 2, 1>(ctx, w, p, s);          \
        break;
    if (ksplit && w->kind == BHD_TYPE_Q4_K) st = launch_i8<BHD_TYPE_Q4_K, 1, 4>(ctx, w, p, s);
    else if (ksplit) st = launch_i8<BHD_TYPE_Q8_0, 1, 4>(ctx, w, p, s);
    else switch (w->kind) {
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
