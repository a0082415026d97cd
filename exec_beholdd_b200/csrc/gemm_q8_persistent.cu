// Prefill matmul for packed Q8_0 weights: persistent CTAs on the 5th-generation tensor cores.
//
//   Y[m][n] = sum_k X[m][k] * W[n][k],   W packed Q8_0 [N x K], X fp16 [M x K] (converted once per call), Y f32.
//
// Same operand mapping as gemm_q8_tcgen05.cu (the 128 weight rows of a tile are the MMA's M operand, built in
// shared memory as a K-major 128B-swizzled fp16 tile with the block scale folded in; TN tokens are the N operand,
// loaded by TMA; the f32 accumulator lives in tensor memory), with the schedule changed in the three places
// where that kernel loses its time:
//   * One CTA per SM walks a list of tiles. Barriers, tensor memory and the rings are set up once, and the
//     producers (weight chunks, token tiles, converters) run ahead across tile boundaries, so the rings are full
//     when a tile's first MMA is issued.
//   * Two accumulators in tensor memory. Four dedicated warps drain one (tcgen05.ld -> global) while the MMAs of
//     the next tile fill the other: the 128 x TN x 4-byte write-back, which nothing overlapped before, leaves
//     the critical path.
//   * Every wait polls with mbarrier.test_wait instead of sleeping in try_wait (the wake-up after a sleep cost
//     more than the work between two barriers), and all eight converter warps work on every slice (a thread
//     converts one 32-column block of one row), which halves the latency of a slice's conversion and lets every
//     waiter see every phase of every barrier.
// Roles: warp 0 weight chunks (TMA), warp 1 MMA issue + tensor-memory allocation, warps 2-9 converters, warp 10
// token tiles (TMA), warps 12-15 write-back. Every wait is bounded; a wait that gives up sets the status word,
// the roles drain and the CTA frees its tensor memory before it returns.
//
// Reference semantics: a loop of Device::matvec over positions
// (crates/beholdd-model/src/qwen3moe/forward.rs:1086-1127) with kquant::q8_0::dot
// (crates/beholdd-kernel/src/kquant.rs:61-79); fp16 operands with f32 accumulation keep the result within the
// path's 2e-3 tolerance.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;            // weight rows per tile (MMA M)
constexpr int CHUNK_K = 256;           // columns per packed chunk
constexpr int SLICE_K = 64;            // columns per fp16 stage (one 128-byte swizzle row)
constexpr int PACK_ROW = 272;          // packed bytes per row per chunk
constexpr int PACK_BYTES = TILE_N * PACK_ROW;   // 34816, a multiple of 1024
constexpr int A_BYTES = TILE_N * SLICE_K * 2;   // 16384
constexpr int THREADS = 16 * 32;
constexpr int MAX_STAGES = 8;
constexpr uint32_t SPIN_LIMIT = 1u << 24;       // polls, roughly a second

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
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
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
// 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

struct PersistentParams {
    float* y;            // [M x N]
    uint32_t* status;
    uint32_t n_rows;     // N: weight rows of the slab
    uint32_t row_base;   // tensor-map row of the slab's first row
    uint32_t m;          // tokens
    uint32_t k;          // columns
    uint32_t tn;         // tokens per tile: 64, 128 or 256
    uint32_t stages;     // fp16 stages in the ring
    uint32_t tok_tiles;  // ceil(M / tn); tile t = (row tile t / tok_tiles, token tile t % tok_tiles)
    uint32_t tiles;      // row tiles * token tiles
};

__global__ void __launch_bounds__(THREADS, 1) k_gemm_q8_persistent(const __grid_constant__ CUtensorMap tmap_w,
                                                                   const __grid_constant__ CUtensorMap tmap_x,
                                                                   const PersistentParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t pk_full[2], pk_empty[2], a_full[MAX_STAGES], b_full[MAX_STAGES], st_empty[MAX_STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t bn = p.tn;  // MMA N = rows of the token tile
    const uint32_t stage_bytes = A_BYTES + bn * 128u;
    const uint32_t pack_addr = smem0, stage_addr = smem0 + 2 * PACK_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t slices = (p.k + SLICE_K - 1) / SLICE_K, chunks = (p.k + CHUNK_K - 1) / CHUNK_K;
    const uint32_t S = p.stages;
    const uint32_t n_my = blockIdx.x < p.tiles ? (p.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&pk_full[i], 1);
            mbar_init(&pk_empty[i], 8);
            mbar_init(&tmem_full[i], 1);
            mbar_init(&tmem_empty[i], 4);
        }
        for (uint32_t i = 0; i < S; ++i) {
            mbar_init(&a_full[i], 8);
            mbar_init(&b_full[i], 1);
            mbar_init(&st_empty[i], 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, 2 * bn);  // two accumulators; 128, 256 or 512 columns
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    auto give_up = [&]() { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); *(volatile int*)&abort_flag = 1; };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };
    // g counts this CTA's slices over all its tiles; slice g lives in stage g % S. Before a stage is refilled,
    // the MMAs of its previous use must have finished reading it.
    auto stage_free = [&](uint32_t g) { return g < S || mbar_wait(&st_empty[g % S], (g / S - 1) & 1); };

    if (warp == 0) {
        // ---- packed weight chunks: two in flight, requested as soon as a buffer is released ----
        if (lane == 0) {
            uint32_t gc = 0;
            for (uint32_t i = 0; i < n_my && !aborted(); ++i) {
                const uint32_t t = blockIdx.x + i * gridDim.x, n0 = (t / p.tok_tiles) * TILE_N;
                for (uint32_t c = 0; c < chunks; ++c, ++gc) {
                    const uint32_t pb = gc & 1;
                    if (aborted() || !mbar_wait(&pk_empty[pb], ((gc >> 1) & 1) ^ 1)) { give_up(); break; }
                    mbar_arrive_expect_tx(&pk_full[pb], PACK_BYTES);
                    tma_load_2d(pack_addr + pb * PACK_BYTES, &tmap_w, int(c * (PACK_ROW / 2)), int(p.row_base + n0), &pk_full[pb]);
                }
            }
        }
    } else if (warp == 10) {
        // ---- token tiles ----
        if (lane == 0) {
            uint32_t g = 0;
            for (uint32_t i = 0; i < n_my && !aborted(); ++i) {
                const uint32_t t = blockIdx.x + i * gridDim.x, m0 = (t % p.tok_tiles) * p.tn;
                for (uint32_t it = 0; it < slices; ++it, ++g) {
                    const uint32_t s = g % S;
                    if (aborted() || !stage_free(g)) { give_up(); break; }
                    mbar_arrive_expect_tx(&b_full[s], bn * 128u);
                    tma_load_2d(stage_addr + s * stage_bytes + A_BYTES, &tmap_x, int(it * SLICE_K), int(m0), &b_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: tile i accumulates into buffer i & 1 ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(TILE_N, bn);
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t i = 0; i < n_my && ok; ++i) {
                const uint32_t buf = i & 1, acc = tmem_base + buf * bn;
                if (i >= 2) {  // the write-back of tile i - 2 must have emptied this accumulator
                    if (aborted() || !mbar_wait(&tmem_empty[buf], ((i >> 1) & 1) ^ 1)) { give_up(); break; }
                    tc_fence_after();
                }
                for (uint32_t it = 0; it < slices; ++it, ++g) {
                    const uint32_t s = g % S, par = (g / S) & 1;
                    if (aborted() || !mbar_wait(&b_full[s], par) || !mbar_wait(&a_full[s], par)) { give_up(); ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = umma_desc(stage_addr + s * stage_bytes), db = umma_desc(stage_addr + s * stage_bytes + A_BYTES);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < 4; ++k16)  // 32 bytes (16 fp16) further along the swizzled row per step
                        tc_mma_f16(acc, da + 2 * k16, db + 2 * k16, idesc, (it | k16) ? 1u : 0u);
                    tc_commit(&st_empty[s]);  // arrives when these MMAs have finished reading the stage
                }
                if (ok) tc_commit(&tmem_full[buf]);  // arrives when every MMA of the tile is complete
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
                if (aborted() || !mbar_wait(&pk_full[pb], (gc >> 1) & 1)) { give_up(); ok = false; break; }
                const uint32_t src_row = pack_addr + pb * PACK_BYTES + row * PACK_ROW;
                for (uint32_t kb = 0; kb < 4; ++kb, ++g) {
                    if (c * 4 + kb >= slices) break;
                    const uint32_t s = g % S;
                    if (aborted() || !stage_free(g)) { give_up(); ok = false; break; }
                    // Two Q8_0 blocks = 68 bytes = 17 words [d0 | q0..q31 | d1 | q32..q63] from word 17 * kb of the
                    // row. Block 0 is words 0..8 (d in the low half of word 0, quants straddling words), block 1
                    // words 8..16 (d in the high half of word 8, quants word-aligned in 9..16).
                    uint32_t w[9];
#pragma unroll
                    for (int j = 0; j < 9; ++j) w[j] = lds32(src_row + kb * 68 + blk * 32 + 4 * j);
                    const uint32_t dbits = blk == 0 ? (w[0] & 0xffffu) : (w[0] >> 16);
                    const __half2 d2 = __half2half2(__ushort_as_half(uint16_t(dbits)));
                    const uint32_t a_dst = stage_addr + s * stage_bytes + a_row_off;
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
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[s]);  // one arrival per converter warp
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&pk_empty[pb]);
            }
        }
    } else if (warp >= 12) {
        // ---- write-back: TMEM lane = weight row, column = token. A warp may read the lane quarter warp % 4. ----
        const uint32_t q = uint32_t(warp) & 3u;
        for (uint32_t i = 0; i < n_my; ++i) {
            const uint32_t t = blockIdx.x + i * gridDim.x, n0 = (t / p.tok_tiles) * TILE_N, m0 = (t % p.tok_tiles) * p.tn;
            const uint32_t buf = i & 1;
            if (aborted() || !mbar_wait(&tmem_full[buf], (i >> 1) & 1)) { give_up(); break; }
            tc_fence_after();
            const uint32_t n = n0 + q * 32 + lane;
            for (uint32_t col = 0; col < p.tn; col += 32) {
                if (m0 + col >= p.m) break;            // uniform across the warp
                uint32_t r[32];
                tc_ld32(tmem_base + ((q * 32u) << 16) + buf * bn + col, r);
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
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * bn);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// Dense prefill: Y[m][n] = sum_k fp16(X[m][k]) * fp16(W[n][k]); x16 is the fp16 copy of X [M x K].
int32_t bhd_launch_gemm_q8_persistent(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M,
                                      cudaStream_t s) {
    const uint32_t K = uint32_t(w->cols), N = uint32_t(w->rows);
    static int sm_count[BHD_MAX_DEVICES] = {};
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_persistent, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
                 "raising the shared memory limit");
        BHD_CUDA(ctx, cudaDeviceGetAttribute(&sm_count[ctx->device], cudaDevAttrMultiProcessorCount, ctx->device), "reading the SM count");
        once.mark(ctx);
    }
    const uint32_t sms = uint32_t(sm_count[ctx->device] > 0 ? sm_count[ctx->device] : 148);
    const uint32_t row_tiles = (N + TILE_N - 1) / TILE_N;
    // Tokens per tile: the wider the tile, the fewer times a weight tile is converted; but the tiles are dealt to the
    // SMs in whole rounds, so a narrower tile wins when it leaves fewer SMs idle in the last round. Cost of a tile
    // relative to a 256-token one, measured: 0.56 (128 tokens), 0.36 (64).
    uint32_t tn = 64;
    if (M >= 128) {
        float best = 1e30f;
        const uint32_t cand[3] = {256, 128, 64};
        const float cost[3] = {1.0f, 0.56f, 0.36f};
        for (int i = 0; i < 3; ++i) {
            if (cand[i] > M && cand[i] != 128) continue;
            const uint32_t tiles = row_tiles * ((M + cand[i] - 1) / cand[i]);
            const float t = float((tiles + sms - 1) / sms) * cost[i];
            if (t < best - 1e-6f) { best = t; tn = cand[i]; }
        }
    }
    const uint32_t tok_tiles = (M + tn - 1) / tn, tiles = row_tiles * tok_tiles;
    const uint32_t stage_bytes = A_BYTES + tn * 128u;
    uint32_t stages = (226u * 1024u - 1024u - 2u * PACK_BYTES) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const size_t dyn = 1024 + 2 * size_t(PACK_BYTES) + size_t(stages) * stage_bytes;

    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode);
    CUtensorMap map_w, map_x;
    {
        const cuuint64_t dims[2] = {w->row_bytes / 2, w->rows * w->slabs};
        const cuuint64_t strides[1] = {w->row_bytes};
        const cuuint32_t box[2] = {PACK_ROW / 2, TILE_N};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the weight tensor map", bhd_device_name());
    }
    {
        const cuuint64_t dims[2] = {K, M};
        const cuuint64_t strides[1] = {uint64_t(K) * 2};
        const cuuint32_t box[2] = {SLICE_K, tn};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the activation tensor map", bhd_device_name());
    }
    PersistentParams p = {};
    p.y = y;
    p.status = ctx->status_dev;
    p.n_rows = N;
    p.row_base = uint32_t(slab * w->rows);
    p.m = M;
    p.k = K;
    p.tn = tn;
    p.stages = stages;
    p.tok_tiles = tok_tiles;
    p.tiles = tiles;
    k_gemm_q8_persistent<<<tiles < sms ? tiles : sms, THREADS, dyn, s>>>(map_w, map_x, p);
    BHD_LAUNCHED(ctx, "tcgen05 persistent matmul kernel");
    return BHD_OK;
}
