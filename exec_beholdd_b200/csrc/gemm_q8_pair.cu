// Prefill matmul for packed Q8_0, Q4_K and Q6_K weights: persistent CTA pairs (tcgen05 cta_group::2).
//
//   Y[m][n] = sum_k X[m][k] * W[n][k],   W packed Q8_0, Q4_K or Q6_K [N x K], X fp16 [M x K] (converted once per call), Y f32.
//
// A cluster of two CTAs on neighbouring SMs works on one 256-row x 256-token tile at a time. Each CTA converts its
// own 128 weight rows (packed chunk by TMA -> fp16 K-major 128B-swizzled tile in its shared memory, block scale
// folded in) and loads only ITS HALF of the token tile (128 tokens x 64 columns = 16 KB per slice instead of 32);
// one thread of the even CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), for which the hardware
// reads both halves of the token tile out of both shared memories, and each SM accumulates its 128 rows x 256
// tokens in its own tensor memory. Halving the token bytes per SM is what buys ring depth: the token ring holds
// six slices and the weight ring three (one CTA per tile had three of both), which is what the load latency of
// a token tile needs to stay off the critical path.
//
// Schedule as in gemm_q8_persistent.cu: one cluster per SM pair walks a list of tiles; producers run ahead across
// tile boundaries; two accumulators in tensor memory so that eight write-back warps per CTA drain one tile while
// the MMAs of the next fill the other; waits on the critical path poll with mbarrier.test_wait. The two rings
// are released by ONE tcgen05.commit per slice onto a ring of "slice done" barriers (multicast to both CTAs)
// that every producer watches at its own distance.
//
// Cross-CTA signals: converters and write-back warps of both CTAs arrive on the even CTA's barriers
// (mapa + mbarrier.arrive.shared::cluster); token tiles of both CTAs complete their bytes on the even CTA's
// barrier (TMA load with .cta_group::2, no multicast); commits reach both CTAs through the commit's own
// multicast. Every wait is bounded; a wait that gives up sets the status word, the roles drain, the two CTAs
// meet at a cluster barrier and free their tensor memory.
//
// Reference semantics: a loop of Device::matvec over positions
// (crates/beholdd-model/src/qwen3moe/forward.rs:1086-1127) with kquant::q8_0::dot
// (crates/beholdd-kernel/src/kquant.rs:61-79); fp16 operands with f32 accumulation keep the result within the
// path's 2e-3 tolerance.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;            // weight rows per CTA (the pair's MMA has M = 256)
constexpr int TOK = 256;               // tokens per tile
constexpr int HALF_TOK = 128;          // tokens each CTA loads
constexpr int CHUNK_K = 256;           // columns per packed chunk
constexpr int SLICE_K = 64;            // columns per fp16 stage (one 128-byte swizzle row)
constexpr int PACK_ROW = 272;          // packed bytes per row per chunk: Q8_0 (eight blocks of 34 bytes); Q4_K: 144 (one superblock)
constexpr int PACK_BYTES = TILE_N * PACK_ROW;   // 34816, a multiple of 1024: the size of a chunk buffer for either format
// Q6_K: a 240-byte window that starts at the 16-byte boundary at or below the row's 210-byte superblock (a TMA copy must
// start on one) and so holds it at an even offset of 0..14 bytes.
__host__ __device__ constexpr int pack_row_of(uint32_t kind) { return kind == BHD_TYPE_Q4_K ? 144 : (kind == BHD_TYPE_Q6_K ? 240 : 272); }
constexpr int A_BYTES = TILE_N * SLICE_K * 2;   // 16384
constexpr int B_BYTES = HALF_TOK * SLICE_K * 2; // 16384
constexpr int THREADS = 20 * 32;       // warps 0-11: producers, issuers, converters; warps 12-19: write-back
constexpr int SA = 3;                  // weight-tile stages
constexpr int SB_BYTES = 6 * B_BYTES;  // token ring: six slices of one 256-token tile, or three of a 512-token tile
constexpr int DONE = 16;               // "slice done" barriers; more than either ring's depth
constexpr int FULL = 6;                // "slice ready" barriers; at least either ring's depth
constexpr uint32_t SPIN_LIMIT = 1u << 24;       // polls, roughly a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {  // a barrier of either CTA
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Polling wait (critical path).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// Polling wait with a short pause between polls, for the producers: they run ahead of the MMAs, and every poll they
// spare leaves the shared-memory pipe to the MMA issuer, whose own barrier reads queue behind them.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < (SPIN_LIMIT >> 2); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        __nanosleep(40);
    }
    return false;
}
// Sleeping wait (long waits off the critical path: leaves the issue slots to the converters).
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < (1u << 20); ++spin) {
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
// The same load with its bytes counted on a barrier that may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- tcgen05 wrappers (cta_group::2) --------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {  // one whole warp of each CTA, same warp index
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on the barrier at this shared-memory offset in BOTH CTAs when the MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(uint16_t(3))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major, 128B-swizzled fp16 tile (rows of 128 bytes, 8-row groups 1024
// bytes apart): start address >> 4 (bits 0-13), stride byte offset >> 4 (32-45) = 1024 >> 4, descriptor
// version 1 (46-47), layout type 2 = SWIZZLE_128B (61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return uint64_t(lo) | (uint64_t(hi) << 32);
}
// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = f16 (0), both K-major, N >> 3 at bits
// 17-22, M >> 4 at bits 24-28 (M counts the rows of both CTAs).
__device__ __forceinline__ uint32_t umma_idesc(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

struct PairParams {
    float* y;            // [M x N]
    uint32_t* status;
    uint32_t n_rows;     // N: weight rows of the slab
    uint32_t row_base;   // tensor-map row of the slab's first row
    uint32_t m;          // tokens
    uint32_t k;          // columns
    uint32_t tok_tiles;  // ceil(M / tokens per tile); tile t = (row pair t / tok_tiles, token tile t % tok_tiles)
    uint32_t tiles;      // row pairs * token tiles
};

// WIDE = false: 256-token tiles, one issuer, the two accumulators alternate between consecutive tiles (the write-back
// of one tile overlaps the MMAs of the next). WIDE = true: 512-token tiles, every converted weight slice is used
// twice: two issuer threads (warps 1 and 11) each own one accumulator and one 256-token half of the tile, so the
// per-slice cost of an issuer (two barrier reads, four MMAs, a commit: about as long as the four MMAs run) is
// paid in parallel and half as much weight conversion is done per flop; the write-back is not overlapped.
// KIND: BHD_TYPE_Q8_0, or BHD_TYPE_Q4_K (crates/beholdd-kernel/src/kquant.rs:176-241): the converter then forms
// fp16((d * sc) * q - dmin * m), computed in f32, from a sub-block's nibbles; a 64-column slice is the pair of sub-blocks that shares 32
// quant bytes (low nibbles, high nibbles), so a thread still converts one 32-column block of one row.
template <uint32_t KIND, bool WIDE>
__global__ void __launch_bounds__(THREADS, 1) k_gemm_q8_pair(const __grid_constant__ CUtensorMap tmap_w,
                                                             const __grid_constant__ CUtensorMap tmap_x, const PairParams p) {
    constexpr uint32_t TOKT = WIDE ? 2 * TOK : TOK;              // tokens per tile
    constexpr uint32_t BS_BYTES = WIDE ? 2 * B_BYTES : B_BYTES;  // token bytes per stage and CTA
    constexpr uint32_t SB = SB_BYTES / BS_BYTES;
    constexpr int PROW = pack_row_of(KIND), PBYTES = TILE_N * PROW;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t pk_full[2], pk_empty[2], full[FULL], done[DONE], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t pack_addr = smem0, a_addr = smem0 + 2 * PACK_BYTES, b_addr = a_addr + SA * A_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();            // 0: issues the MMAs and owns the pair's barriers
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t slices = (p.k + SLICE_K - 1) / SLICE_K, chunks = (p.k + CHUNK_K - 1) / CHUNK_K;
    const uint32_t n_my = pair < p.tiles ? (p.tiles - pair + n_pairs - 1) / n_pairs : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&pk_full[i], 1);
            mbar_init(&pk_empty[i], 8);
            mbar_init(&tmem_full[i], WIDE ? 2 : 1);   // WIDE: both issuers (only barrier 0 is used)
            mbar_init(&tmem_empty[i], 16);            // eight write-back warps of each CTA
        }
        // Slice g is ready when the sixteen converter warps of the pair have arrived and the token bytes of both CTAs have
        // landed: ONE barrier per slice (full[g % FULL]) for both rings, so the issuer reads one barrier per slice. No
        // arrival for slice g + FULL can come before slice g's phase is complete: both producers first wait for a slice
        // >= g to be done (FULL is at least either ring's depth), and its MMAs are issued after the phase completed.
        for (int i = 0; i < FULL; ++i) mbar_init(&full[i], 17);
        for (int i = 0; i < DONE; ++i) mbar_init(&done[i], WIDE ? 2 : 1);  // one commit per issuer
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(&tmem_base_slot, 512);  // two accumulators of 256 columns
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the other CTA's barriers exist before anything here signals them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    auto give_up = [&]() { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); *(volatile int*)&abort_flag = 1; };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };
    // g counts the pair's slices over all its tiles. The MMAs of slice g arrive on done[g % DONE]; a stage of a ring
    // of depth D is free for slice g once slice g - D is done.
    auto slice_done = [&](uint32_t g) { return mbar_wait_relaxed(&done[g % DONE], (g / DONE) & 1); };

    if (warp == 0) {
        // ---- packed weight chunks of this CTA's 128 rows: two in flight ----
        if (lane == 0) {
            uint32_t gc = 0;
            for (uint32_t i = 0; i < n_my && !aborted(); ++i) {
                const uint32_t t = pair + i * n_pairs, n0 = (t / p.tok_tiles) * (2 * TILE_N) + rank * TILE_N;
                for (uint32_t c = 0; c < chunks; ++c, ++gc) {
                    const uint32_t pb = gc & 1;
                    if (aborted() || !mbar_wait_relaxed(&pk_empty[pb], ((gc >> 1) & 1) ^ 1)) { give_up(); break; }
                    mbar_arrive_expect_tx(&pk_full[pb], PBYTES);
                    const uint32_t byte0 = KIND == BHD_TYPE_Q6_K ? ((210u * c) & ~15u) : uint32_t(PROW) * c;
                    tma_load_2d(pack_addr + pb * PACK_BYTES, &tmap_w, int(byte0 / 2), int(p.row_base + n0), &pk_full[pb]);
                }
            }
        }
    } else if (warp == 10) {
        // ---- this CTA's half of the token tiles; the bytes of both halves are counted on the even CTA's barrier ----
        if (lane == 0) {
            // The kernel is launched as a programmatic dependent of the fp16 conversion of the tokens: everything up to
            // here (and the weight side) runs while that kernel drains; the tokens are read only after it has finished.
            bhd_wait_for_prior_kernels();
            uint32_t g = 0;
            for (uint32_t i = 0; i < n_my && !aborted(); ++i) {
                const uint32_t t = pair + i * n_pairs, m_tile = (t % p.tok_tiles) * TOKT, m0 = m_tile + rank * HALF_TOK;
                const bool two = WIDE && m_tile + TOK < p.m;   // the tile's second 256 tokens exist
                for (uint32_t it = 0; it < slices; ++it, ++g) {
                    const uint32_t s = g % SB;
                    if (aborted() || (g >= SB && !slice_done(g - SB))) { give_up(); break; }
                    const uint32_t bar = in_cta(smem_u32(&full[g % FULL]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&full[g % FULL], (two ? 4 : 2) * B_BYTES);
                    tma_load_2d_pair(b_addr + s * BS_BYTES, &tmap_x, int(it * SLICE_K), int(m0), bar);
                    if (two) tma_load_2d_pair(b_addr + s * BS_BYTES + B_BYTES, &tmap_x, int(it * SLICE_K), int(m0 + TOK), bar);
                }
            }
        }
    } else if (warp == 1 || (WIDE && warp == 11)) {
        // ---- MMA issuers (even CTA only). Narrow: warp 1, tile i accumulates into buffer i & 1 of both CTAs' tensor
        // memory. Wide: warp 1 owns accumulator 0 and the tile's first 256 tokens, warp 11 accumulator 1 and the rest. ----
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(2 * TILE_N, TOK);
            const uint32_t which = warp == 1 ? 0u : 1u;
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t i = 0; i < n_my && ok; ++i) {
                const uint32_t buf = WIDE ? which : (i & 1), acc = tmem_base + buf * TOK;
                const uint32_t t = pair + i * n_pairs, m_tile = (t % p.tok_tiles) * TOKT;
                const bool mine = !WIDE || which == 0 || m_tile + TOK < p.m;   // this issuer's tokens exist
                if (WIDE ? i >= 1 : i >= 2) {  // both CTAs' write-back must have emptied the accumulator
                    const uint32_t par = WIDE ? ((i - 1) & 1) : (((i >> 1) & 1) ^ 1);
                    if (aborted() || !mbar_wait(&tmem_empty[WIDE ? 0 : buf], par)) { give_up(); break; }
                    tc_fence_after();
                }
                for (uint32_t it = 0; it < slices; ++it, ++g) {
                    const uint32_t sa = g % SA, sb = g % SB;
                    if (!mbar_wait(&full[g % FULL], (g / FULL) & 1)) { give_up(); ok = false; break; }
                    tc_fence_after();
                    if (mine) {
                        const uint64_t da = umma_desc(a_addr + sa * A_BYTES), db = umma_desc(b_addr + sb * BS_BYTES + (WIDE ? which * B_BYTES : 0u));
#pragma unroll
                        for (uint32_t k16 = 0; k16 < 4; ++k16)  // 32 bytes (16 fp16) further along the swizzled row per step
                            tc_mma_pair(acc, da + 2 * k16, db + 2 * k16, idesc, (it | k16) ? 1u : 0u);
                    }
                    tc_commit_pair(&done[g % DONE]);  // both CTAs: this issuer's MMAs have finished reading slice g's stages
                }
                if (ok) tc_commit_pair(&tmem_full[WIDE ? 0 : buf]);  // both CTAs: every MMA of this issuer for the tile is complete
            }
        }
    } else if (warp >= 2 && warp < 10) {
        // ---- converters: thread = (weight row, one of the slice's two Q8_0 blocks) ----
        const uint32_t ct = threadIdx.x - 64;   // 0..255
        const uint32_t row = ct & 127, blk = ct >> 7;  // blk is uniform per warp
        const uint32_t sw = row & 7, a_row_off = (row >> 3) * 1024 + sw * 128;
        const __half2 off = __half2half2(__ushort_as_half(uint16_t(0x6480)));  // 1152
        uint32_t g = 0, gc = 0;
        bool ok = true;
        for (uint32_t i = 0; i < n_my && ok; ++i) {
            for (uint32_t c = 0; c < chunks && ok; ++c, ++gc) {
                const uint32_t pb = gc & 1;
                if (aborted() || !mbar_wait_relaxed(&pk_full[pb], (gc >> 1) & 1)) { give_up(); ok = false; break; }
                const uint32_t src_row = pack_addr + pb * PACK_BYTES + row * PROW + (KIND == BHD_TYPE_Q8_0 ? blk * 32 : 0u);
#pragma unroll
                for (uint32_t kb = 0; kb < 4; ++kb) {  // unrolled: the register indices below are constants
                    if (c * 4 + kb >= slices) break;
                    const uint32_t s = g % SA;
                    if (aborted() || (g >= SA && !slice_done(g - SA))) { give_up(); ok = false; break; }
                    const uint32_t a_dst = a_addr + s * A_BYTES + a_row_off;
                    if constexpr (KIND == BHD_TYPE_Q8_0) {
                        // Two Q8_0 blocks = 68 bytes = 17 words [d0 | q0..q31 | d1 | q32..q63] from word 17 * kb of the row;
                        // this thread's block is words 0..8 (block 0: d in the low half of word 0, quants straddling words)
                        // or 8..16 (block 1: d in the high half of word 8, quants word-aligned). Read as three aligned
                        // 16-byte loads from word 16 * kb: rows are 272 bytes apart, so the eight lanes of a quarter-warp
                        // hit eight different 16-byte bank groups, and the nine words are v[kb .. kb + 8].
                        uint32_t v[12];
#pragma unroll
                        for (int j = 0; j < 3; ++j) {
                            const uint4 q4 = lds128(src_row + kb * 64 + 16 * j);
                            v[4 * j] = q4.x; v[4 * j + 1] = q4.y; v[4 * j + 2] = q4.z; v[4 * j + 3] = q4.w;
                        }
                        const uint32_t* w = v + kb;
                        const uint32_t dbits = blk == 0 ? (w[0] & 0xffffu) : (w[0] >> 16);
                        const __half2 d2 = __half2half2(__ushort_as_half(uint16_t(dbits)));
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {  // 8 quants -> one 16-byte chunk of the swizzled row
                            uint32_t h[4];
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const int q = 2 * ch + j;
                                const uint32_t quad = blk == 0 ? __funnelshift_r(w[q], w[q + 1], 16) : w[q + 1];
                                const uint32_t u = quad ^ 0x80808080u;  // 0x6400 | (q + 128) is the fp16 q + 1152
                                const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140), hi = __byte_perm(u, 0x64646464u, 0x4342);
                                const __half2 qa = __hsub2(*reinterpret_cast<const __half2*>(&lo), off);
                                const __half2 qb = __hsub2(*reinterpret_cast<const __half2*>(&hi), off);
                                const __half2 a = __hmul2(qa, d2), b = __hmul2(qb, d2);
                                h[2 * j] = *reinterpret_cast<const uint32_t*>(&a);
                                h[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                            }
                            const uint32_t chunk16 = (blk * 4 + uint32_t(ch)) ^ sw;  // 128B swizzle: chunk index XOR row mod 8
                            sts128(a_dst + chunk16 * 16, make_uint4(h[0], h[1], h[2], h[3]));
                        }
                    } else if constexpr (KIND == BHD_TYPE_Q4_K) {
                        // Q4_K superblock of the row (144 bytes: d, dmin, 12 scale bytes, 128 quant bytes). Slice kb is the
                        // pair of sub-blocks (2kb, 2kb + 1) = the low and the high nibbles of quant bytes 32kb .. 32kb + 31.
                        // Rows are 144 bytes apart: the 16-byte loads of a quarter-warp fall into eight different bank groups.
                        const uint4 hd = lds128(src_row);
                        const uint4 qa = lds128(src_row + 16 + 32 * kb), qb = lds128(src_row + 32 + 32 * kb);
                        const uint32_t sc_w[3] = {hd.y, hd.z, hd.w};
                        auto sbyte = [&](uint32_t i) { return (sc_w[i >> 2] >> (8 * (i & 3))) & 0xffu; };  // i is uniform in the warp
                        const uint32_t sb = 2 * kb + blk;
                        uint32_t sc, mn;   // scale_min_k4 (kquant.rs:176-185)
                        if (sb < 4) {
                            sc = sbyte(sb) & 63u;
                            mn = sbyte(sb + 4) & 63u;
                        } else {
                            sc = (sbyte(sb + 4) & 0xFu) | ((sbyte(sb - 4) >> 6) << 4);
                            mn = (sbyte(sb + 4) >> 4) | ((sbyte(sb) >> 6) << 4);
                        }
                        const float d = __half2float(__ushort_as_half(uint16_t(hd.x & 0xffffu))), dmin = __half2float(__ushort_as_half(uint16_t(hd.x >> 16)));
                        // The value is formed in f32 and rounded to fp16 once: d * sc * q and dmin * m usually cancel to a large
                        // part, so rounding the two terms to fp16 first would double the error of the difference.
                        const float dsc = __fmul_rn(d, float(sc)), ndm = -__fmul_rn(dmin, float(mn));
                        const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                        // byte k of u under the exponent of 2^23: the f32 8388608 + n, from which n by one subtraction
                        auto nib = [](uint32_t u, uint32_t sel) { return __uint_as_float(__byte_perm(u, 0x4B000000u, sel)) - 8388608.0f; };
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t h[4];
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const uint32_t u = (blk == 0 ? qw[2 * ch + j] : (qw[2 * ch + j] >> 4)) & 0x0F0F0F0Fu;
                                const __half2 a = __floats2half2_rn(fmaf(nib(u, 0x7440), dsc, ndm), fmaf(nib(u, 0x7441), dsc, ndm));
                                const __half2 b = __floats2half2_rn(fmaf(nib(u, 0x7442), dsc, ndm), fmaf(nib(u, 0x7443), dsc, ndm));
                                h[2 * j] = *reinterpret_cast<const uint32_t*>(&a);
                                h[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                            }
                            const uint32_t chunk16 = (blk * 4 + uint32_t(ch)) ^ sw;
                            sts128(a_dst + chunk16 * 16, make_uint4(h[0], h[1], h[2], h[3]));
                        }
                    } else {
                        // Q6_K superblock (crates/beholdd-kernel/src/kquant.rs:115-162; 210 bytes: ql[128], qh[64], 16 int8 scales, d)
                        // at byte `o` of the row's window. Slice kb covers two of the four 32-element groups of the 128-element half
                        // kb / 2; this thread's group gi takes the low (gi < 2) or high nibbles of 32 ql bytes and two bits of 32
                        // qh bytes: value = d * scale * (code - 32), one scale per 16 elements. Both byte fields start `o` bytes after
                        // a 32-byte boundary: three aligned 16-byte loads each (rows 240 bytes apart: no bank conflicts), then the
                        // words are moved down by o / 4 words with two layers of selects and by the odd half-word with funnel shifts.
                        const uint32_t o = (210u * c) & 15u, o4 = o >> 2, ob = (o & 2u) * 8u;   // uniform in the CTA
                        const uint32_t half = kb >> 1, gi = 2 * (kb & 1) + blk;
                        auto field = [&](uint32_t addr, uint32_t (&w)[8]) {
                            uint32_t v[12];
#pragma unroll
                            for (int j = 0; j < 3; ++j) {
                                const uint4 q4 = lds128(addr + 16 * j);
                                v[4 * j] = q4.x; v[4 * j + 1] = q4.y; v[4 * j + 2] = q4.z; v[4 * j + 3] = q4.w;
                            }
#pragma unroll
                            for (int i = 0; i < 11; ++i) v[i] = (o4 & 1u) ? v[i + 1] : v[i];
#pragma unroll
                            for (int i = 0; i < 9; ++i) v[i] = (o4 & 2u) ? v[i + 2] : v[i];
#pragma unroll
                            for (int i = 0; i < 8; ++i) w[i] = __funnelshift_r(v[i], v[i + 1], ob);
                        };
                        uint32_t wl[8], wh[8];
                        field(src_row + 64 * half + 32 * (gi & 1), wl);
                        field(src_row + 128 + 32 * half, wh);
                        const uint32_t meta = src_row + o;
                        int sc0, sc1;
                        uint32_t dbits;
                        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sc0) : "r"(meta + 192 + 8 * half + 2 * gi));
                        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sc1) : "r"(meta + 193 + 8 * half + 2 * gi));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits) : "r"(meta + 208));
                        const float d = __half2float(__ushort_as_half(uint16_t(dbits)));
                        const float ds[2] = {__fmul_rn(d, float(sc0)), __fmul_rn(d, float(sc1))};
                        // byte k of the codes under the exponent of 2^23: the f32 8388608 + code, from which code - 32 by one subtraction
                        auto code = [](uint32_t u, uint32_t sel) { return __uint_as_float(__byte_perm(u, 0x4B000000u, sel)) - 8388640.0f; };
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t h[4];
                            const float dsc = ds[ch >> 1];   // elements 8ch .. 8ch + 7: scale 0 for the first sixteen
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const uint32_t lo4 = ((gi & 2u) ? (wl[2 * ch + j] >> 4) : wl[2 * ch + j]) & 0x0F0F0F0Fu;
                                const uint32_t u = lo4 | (((wh[2 * ch + j] >> (2 * gi)) & 0x03030303u) << 4);
                                const __half2 a = __floats2half2_rn(__fmul_rn(code(u, 0x7440), dsc), __fmul_rn(code(u, 0x7441), dsc));
                                const __half2 b = __floats2half2_rn(__fmul_rn(code(u, 0x7442), dsc), __fmul_rn(code(u, 0x7443), dsc));
                                h[2 * j] = *reinterpret_cast<const uint32_t*>(&a);
                                h[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                            }
                            const uint32_t chunk16 = (blk * 4 + uint32_t(ch)) ^ sw;
                            sts128(a_dst + chunk16 * 16, make_uint4(h[0], h[1], h[2], h[3]));
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(in_cta(smem_u32(&full[g % FULL]), 0));  // one arrival per converter warp
                    ++g;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&pk_empty[pb]);
            }
        }
    } else if (warp >= 12) {
        // ---- write-back of this CTA's 128 rows: TMEM lane = weight row, column = token. A warp may read the lane quarter
        // warp % 4; the two warps of a quarter each take half of the tile's columns. ----
        const uint32_t q = uint32_t(warp) & 3u, part = uint32_t(warp - 12) >> 2;
        constexpr uint32_t COLS = TOKT / 2;   // columns per warp
        for (uint32_t i = 0; i < n_my; ++i) {
            const uint32_t t = pair + i * n_pairs, n0 = (t / p.tok_tiles) * (2 * TILE_N) + rank * TILE_N, m0 = (t % p.tok_tiles) * TOKT;
            const uint32_t buf = WIDE ? 0u : (i & 1), par = WIDE ? (i & 1) : ((i >> 1) & 1);
            if (aborted() || !mbar_wait_sleep(&tmem_full[buf], par)) { give_up(); break; }
            tc_fence_after();
            const uint32_t n = n0 + q * 32 + lane;
            for (uint32_t col = part * COLS; col < (part + 1) * COLS; col += 32) {
                if (m0 + col >= p.m) break;            // uniform across the warp
                uint32_t r[32];
                tc_ld32(tmem_base + ((q * 32u) << 16) + buf * TOK + col, r);
                if (n < p.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t m = m0 + col + j;
                        if (m < p.m) p.y[uint64_t(m) * p.n_rows + n] = __uint_as_float(r[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(in_cta(smem_u32(&tmem_empty[buf]), 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA frees tensor memory or leaves while the other may still signal it
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// Dense prefill on CTA pairs (Q8_0, Q4_K or Q6_K weights), M >= 256: Y[m][n] = sum_k fp16(X[m][k]) * fp16(W[n][k]); x16 is the fp16 copy of X.
// wide: 512-token tiles with two issuers (see the kernel); else 256-token tiles with an overlapped write-back.
int32_t bhd_launch_gemm_q8_pair(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M, bool wide,
                                cudaStream_t s) {
    const uint32_t K = uint32_t(w->cols), N = uint32_t(w->rows);
    static int sm_count[BHD_MAX_DEVICES] = {};
    static bhd_once_per_device once;
    const size_t dyn = 1024 + 2 * size_t(PACK_BYTES) + size_t(SA) * A_BYTES + size_t(SB_BYTES);
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q8_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q8_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q4_K, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q4_K, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q6_K, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_pair<BHD_TYPE_Q6_K, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        BHD_CUDA(ctx, cudaDeviceGetAttribute(&sm_count[ctx->device], cudaDevAttrMultiProcessorCount, ctx->device), "reading the SM count");
        once.mark(ctx);
    }
    const uint32_t sms = uint32_t(sm_count[ctx->device] > 1 ? sm_count[ctx->device] : 148);
    const uint32_t tokt = wide ? 2 * TOK : TOK;
    const uint32_t row_pairs = (N + 2 * TILE_N - 1) / (2 * TILE_N), tok_tiles = (M + tokt - 1) / tokt, tiles = row_pairs * tok_tiles;
    const uint32_t n_pairs = tiles < sms / 2 ? tiles : sms / 2;

    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode);
    CUtensorMap map_w, map_x;
    {
        const cuuint64_t dims[2] = {w->row_bytes / 2, w->rows * w->slabs};
        const cuuint64_t strides[1] = {w->row_bytes};
        const cuuint32_t box[2] = {cuuint32_t(pack_row_of(w->kind) / 2), TILE_N};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the weight tensor map", bhd_device_name());
    }
    {
        const cuuint64_t dims[2] = {K, M};
        const cuuint64_t strides[1] = {uint64_t(K) * 2};
        const cuuint32_t box[2] = {SLICE_K, HALF_TOK};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the activation tensor map", bhd_device_name());
    }
    PairParams p = {};
    p.y = y;
    p.status = ctx->status_dev;
    p.n_rows = N;
    p.row_base = uint32_t(slab * w->rows);
    p.m = M;
    p.k = K;
    p.tok_tiles = tok_tiles;
    p.tiles = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * n_pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = dyn;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->plain_launches ? 1 : 2;
    const bool q4 = w->kind == BHD_TYPE_Q4_K, q6 = w->kind == BHD_TYPE_Q6_K;
    if (q6 && wide) BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q6_K, true>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    else if (q6) BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q6_K, false>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    else if (q4 && wide) BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q4_K, true>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    else if (q4) BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q4_K, false>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    else if (wide) BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q8_0, true>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    else BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_gemm_q8_pair<BHD_TYPE_Q8_0, false>, map_w, map_x, p), "launching the paired tcgen05 matmul kernel");
    ctx->launches += 1;
    return BHD_OK;
}
