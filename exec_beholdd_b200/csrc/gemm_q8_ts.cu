// Q8_0 matmul on the 5th-generation tensor cores with the weight operand in tensor memory.
//
//   out[m][n] = scale[m] * sum_k X[m][k] * W[n][k],   W packed Q8_0, X fp16 (row-scaled), f32 out.
//
// Same mapping as gemm_q8_tcgen05.cu (weights are the 128-row operand A, tokens the N operand B,
// accumulator in TMEM) with one change that removes most of the kernel's shared-memory traffic,
// which is what bounds the shared-memory-operand form: the converter warps write the fp16 weight
// tile straight from registers into tensor memory (tcgen05.st) and the MMAs read A from there
// (tcgen05.mma with a TMEM A operand); only the token tiles (B) pass through shared memory.
//
// EXACT form (routed experts): both operands are carried as fp16 pairs, w = hi + lo and x = hi + lo
// with exact residuals (d*q has 19 significant bits, hi + lo holds 22), so the products lose
// nothing and the result matches an f32 computation to accumulation order. The token tile then
// holds 2 * tn rows (hi rows, lo rows), each K-step issues two MMAs (A_hi, A_lo) and the
// epilogue adds the two halves of the accumulator. Plain form (prefill): one rounding per
// operand, one MMA per K-step.
//
// Roles per CTA: warp 0 requests packed weight chunks (TMA, 2 in flight), warp 1 issues the MMAs
// and owns the TMEM allocation, warps 2-9 convert (two groups of four warps on alternating
// 64-column slices; thread = weight row = TMEM lane) and group 0 is the epilogue, warp 10
// requests the token tiles (TMA, 128B swizzle). Every wait is bounded; a wait that gives up sets
// the status word, the roles drain and the CTA frees its tensor memory before it returns.
//
// Reference semantics: a loop of Device::matvec over positions / routes
// (crates/beholdd-model/src/qwen3moe/forward.rs:1086-1127, 1363-1400) with kquant::q8_0::dot
// (crates/beholdd-kernel/src/kquant.rs:61-79).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;            // weight rows per CTA (MMA M)
constexpr int CHUNK_K = 256;           // columns per packed chunk
constexpr int SLICE_K = 64;            // columns per stage
constexpr int PACK_ROW = 272;          // packed bytes per row per chunk
constexpr int PACK_BYTES = TILE_N * PACK_ROW;   // 34816
constexpr int THREADS = 11 * 32;
constexpr uint32_t SPIN_LIMIT = 1u << 20;

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
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
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
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
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
// 32 consecutive 32-bit columns of this thread's TMEM lane, from registers.
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major, 128B-swizzled fp16 tile (rows of 128 bytes, 8-row groups
// 1024 bytes apart): start address >> 4 (bits 0-13), stride byte offset >> 4 (32-45) = 1024 >> 4,
// descriptor version 1 (46-47), layout type 2 = SWIZZLE_128B (61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return uint64_t(lo) | (uint64_t(hi) << 32);
}
// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = f16 (0), both K-major, N >> 3 at bits 17-22, M >> 4 at 24-28.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

struct TsParams {
    float* y;            // [M x N]; grouped: [slot][N] of matrix 0
    float* y1;           // grouped: matrix 1 (blockIdx.z == 1), or null
    float* const* row_dst;  // optional: where the output row of activation row m starts (instead of y + m * N)
    uint32_t* status;
    uint32_t n_rows;     // N: weight rows of one slab
    uint32_t row_base;   // tensor-map row of the slab's first row (dense mode)
    uint32_t m;          // activation rows (dense mode)
    uint32_t k;          // columns
    uint32_t tn;         // activation rows per tile: 16 .. 256
    uint32_t stages;     // stages in the ring (even)
    const MoeHeader* hdr;  // grouped mode when groups != null: blockIdx.y walks the groups of one size class
    const MoeGroup* groups;
    const int32_t* glist;
    uint32_t cls;
    const float* col_scale;  // optional factor per activation row
};

template <bool EXACT>
__global__ void __launch_bounds__(THREADS, 1) k_gemm_q8_ts(const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1,
                                                           const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_xlo,
                                                           const TsParams p) {
    uint32_t m0, m_end, row_base;
    if (p.groups) {
        if (blockIdx.y >= p.hdr->gcount[p.cls]) return;  // the whole CTA, before any barrier or tensor memory exists
        const MoeGroup grp = p.groups[p.glist[blockIdx.y]];
        m0 = uint32_t(grp.slot0);
        m_end = m0 + uint32_t(grp.nb);
        row_base = uint32_t(grp.expert_local) * p.n_rows;
    } else {
        m0 = blockIdx.y * p.tn;
        m_end = p.m;
        row_base = p.row_base;
    }
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t pk_full[2], pk_empty[2], a_full[8], b_full[8], st_empty[8], tmem_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    constexpr uint32_t A_COLS = EXACT ? 64u : 32u;          // TMEM columns of one stage's weight tile(s): 64 fp16 per row, hi (and lo)
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t bn = EXACT ? 2u * p.tn : p.tn;           // MMA N = rows of the token tile
    const uint32_t stage_bytes = bn * 128u;
    const uint32_t pack_addr = smem0, stage_addr = smem0 + 2 * PACK_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const CUtensorMap* tmap_w = blockIdx.z ? &tmap_w1 : &tmap_w0;
    float* const yout = blockIdx.z ? p.y1 : p.y;
    const uint32_t n0 = blockIdx.x * TILE_N;
    const uint32_t slices = (p.k + SLICE_K - 1) / SLICE_K, chunks = (p.k + CHUNK_K - 1) / CHUNK_K;
    const uint32_t S = p.stages;
    // tensor memory: accumulator (bn columns), then the stages' weight tiles
    uint32_t tmem_cols = 32;
    while (tmem_cols < bn + S * A_COLS) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(&pk_full[i], 1); mbar_init(&pk_empty[i], 8); }
        for (uint32_t i = 0; i < S; ++i) {
            mbar_init(&a_full[i], 4);
            mbar_init(&b_full[i], 1);
            mbar_init(&st_empty[i], 1);
        }
        mbar_init(&tmem_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_a = tmem_base + bn;
    auto give_up = [&]() { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); *(volatile int*)&abort_flag = 1; };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };
    // wait until the MMAs of the previous use of slice it's stage are done with it (true at once for the first use)
    auto stage_free = [&](uint32_t it) {
        const uint32_t use = it / S;
        if (use == 0) return true;
        return mbar_wait(&st_empty[it % S], (use - 1) & 1);
    };

    if (warp == 0) {
        // ---- packed weight chunks: requested as soon as a buffer is released ----
        if (lane == 0) {
            for (uint32_t c = 0; c < chunks && !aborted(); ++c) {
                const uint32_t pb = c & 1;
                if (!mbar_wait(&pk_empty[pb], ((c >> 1) & 1) ^ 1)) { give_up(); break; }
                mbar_arrive_expect_tx(&pk_full[pb], PACK_BYTES);
                tma_load_2d(pack_addr + pb * PACK_BYTES, tmap_w, int(c * (PACK_ROW / 2)), int(row_base + n0), &pk_full[pb]);
            }
        }
    } else if (warp == 10) {
        // ---- token tiles ----
        if (lane == 0) {
            for (uint32_t it = 0; it < slices && !aborted(); ++it) {
                const uint32_t s = it % S;
                if (!stage_free(it)) { give_up(); break; }
                mbar_arrive_expect_tx(&b_full[s], bn * 128u);
                tma_load_2d(stage_addr + s * stage_bytes, &tmap_x, int(it * SLICE_K), int(m0), &b_full[s]);
                if (EXACT) tma_load_2d(stage_addr + s * stage_bytes + p.tn * 128u, &tmap_xlo, int(it * SLICE_K), int(m0), &b_full[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(TILE_N, bn);
            for (uint32_t it = 0; it < slices; ++it) {
                const uint32_t s = it % S, par = (it / S) & 1;
                if (aborted() || !mbar_wait(&b_full[s], par) || !mbar_wait(&a_full[s], par)) { give_up(); break; }
                tc_fence_after();
                const uint64_t db = umma_desc(stage_addr + s * stage_bytes);
                const uint32_t ta = tmem_a + s * A_COLS;
#pragma unroll
                for (uint32_t k16 = 0; k16 < 4; ++k16) {  // 16 fp16 = 8 TMEM columns of A, 32 bytes along the swizzled rows of B
                    tc_mma_ts(tmem_base, ta + 8 * k16, db + 2 * k16, idesc, (it | k16) ? 1u : 0u);
                    if (EXACT) tc_mma_ts(tmem_base, ta + 32 + 8 * k16, db + 2 * k16, idesc, 1u);
                }
                tc_commit(&st_empty[s]);  // arrives when these MMAs have finished reading the stage
            }
            tc_commit(&tmem_full);        // arrives when every MMA issued is complete
        }
    } else {
        // ---- converters: two groups of four warps take alternating 64-column slices; thread = weight row = TMEM lane.
        // A warp may only touch the TMEM lanes of its quarter (warp index mod 4), which fixes the row of every thread. ----
        const uint32_t grp = uint32_t(warp - 2) >> 2;          // 0: warps 2-5, 1: warps 6-9
        const uint32_t quarter = uint32_t(warp) & 3u;
        const uint32_t row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16;       // TMEM address: lane in bits 16-31, column in bits 0-15
        bool ok = true;
        for (uint32_t c = 0; c < chunks && ok; ++c) {
            const uint32_t pb = c & 1;
            if (aborted() || !mbar_wait(&pk_full[pb], (c >> 1) & 1)) { give_up(); ok = false; break; }
            const uint32_t src_row = pack_addr + pb * PACK_BYTES + row * PACK_ROW;
#pragma unroll
            for (uint32_t kb = 0; kb < 4; ++kb) {  // unrolled so that the register indices below are constants
                if ((kb & 1u) != grp) continue;     // uniform per warp
                const uint32_t it = c * 4 + kb;
                if (it >= slices) break;
                const uint32_t s = it % S;
                if (!stage_free(it)) { give_up(); ok = false; break; }
                // Two Q8_0 blocks = 68 bytes = 17 words [d0 | q0..q31 | d1 | q32..q63], starting at word 17 * kb of
                // the row: five aligned 16-byte loads from word 16 * kb (rows are 272 bytes apart, so the eight
                // lanes of a quarter-warp hit eight different 16-byte bank groups), the slice's words are v[kb ..].
                uint32_t v[20];
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    const uint4 q4 = lds128(src_row + kb * 64 + 16 * i);
                    v[4 * i] = q4.x; v[4 * i + 1] = q4.y; v[4 * i + 2] = q4.z; v[4 * i + 3] = q4.w;
                }
                const uint32_t* w = v + kb;
                uint32_t hi[32], lo[EXACT ? 32 : 1];
                const __half2 off = __half2half2(__ushort_as_half(uint16_t(0x6480)));  // 1152
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    const uint32_t dbits = blk == 0 ? (w[0] & 0xffffu) : (w[8] >> 16);
                    const __half2 d2 = __half2half2(__ushort_as_half(uint16_t(dbits)));
#pragma unroll
                    for (int j = 0; j < 8; ++j) {  // word j of the block: quants 4j .. 4j+3
                        const uint32_t q = blk == 0 ? __funnelshift_r(w[j], w[j + 1], 16) : w[9 + j];
                        const uint32_t u = q ^ 0x80808080u;  // 0x6400 | (q + 128) is the fp16 q + 1152
                        const uint32_t p0 = __byte_perm(u, 0x64646464u, 0x4140), p1 = __byte_perm(u, 0x64646464u, 0x4342);
                        const __half2 qa = __hsub2(*reinterpret_cast<const __half2*>(&p0), off);
                        const __half2 qb = __hsub2(*reinterpret_cast<const __half2*>(&p1), off);
                        const __half2 a = __hmul2(qa, d2), b = __hmul2(qb, d2);
                        hi[blk * 16 + 2 * j] = *reinterpret_cast<const uint32_t*>(&a);
                        hi[blk * 16 + 2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                        if (EXACT) {  // exact residual of the rounded product (it has at most 8 significant bits)
                            const __half2 ra = __hfma2(qa, d2, __hneg2(a)), rb = __hfma2(qb, d2, __hneg2(b));
                            lo[blk * 16 + 2 * j] = *reinterpret_cast<const uint32_t*>(&ra);
                            lo[blk * 16 + 2 * j + 1] = *reinterpret_cast<const uint32_t*>(&rb);
                        }
                    }
                }
                const uint32_t ta = tmem_a + s * A_COLS + lane_addr;
                tc_st32(ta, hi);
                if (EXACT) tc_st32(ta + 32, reinterpret_cast<const uint32_t(&)[32]>(lo));
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[s]);  // one arrival per converter warp
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pk_empty[pb]);
        }
        // ---- epilogue (group 0): TMEM lane = weight row, column = activation row ----
        if (grp == 0) {
            if (ok && !aborted() && mbar_wait(&tmem_full, 0)) {
                tc_fence_after();
                const uint32_t n = n0 + row;
                for (uint32_t col = 0; col < p.tn; col += 32) {
                    if (m0 + col >= m_end) break;  // uniform across the warp
                    uint32_t r[32];
                    tc_ld32(tmem_base + lane_addr + col, r);
                    if (EXACT) {  // the columns of the lo rows
                        uint32_t r2[32];
                        tc_ld32(tmem_base + lane_addr + p.tn + col, r2);
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
                    }
                    if (n < p.n_rows) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t m = m0 + col + j;
                            if (m < m_end) {
                                const float sc = p.col_scale ? p.col_scale[m] : 1.0f;
                                float* dst = p.row_dst ? p.row_dst[m] : yout + uint64_t(m) * p.n_rows;
                                dst[n] = __fmul_rn(__uint_as_float(r[j]), sc);
                            }
                        }
                    }
                }
            } else if (ok) {
                give_up();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool encode_weight_map(bhd_ctx* ctx, const bhd_weight* w, CUtensorMap* map) {
    const cuuint64_t dims[2] = {w->row_bytes / 2, w->rows * w->slabs};
    const cuuint64_t strides[1] = {w->row_bytes};
    const cuuint32_t box[2] = {PACK_ROW / 2, TILE_N};
    const cuuint32_t estr[2] = {1, 1};
    return reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, box, estr,
                                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool encode_x_map(bhd_ctx* ctx, const void* x16, uint64_t rows, uint64_t K, uint32_t tn, CUtensorMap* map) {
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K * 2};
    const cuuint32_t box[2] = {SLICE_K, tn};
    const cuuint32_t estr[2] = {1, 1};
    return reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box,
                                                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t ts_smem_bytes(bool exact, uint32_t tn, uint32_t stages) { return 1024 + 2 * size_t(PACK_BYTES) + size_t(stages) * (exact ? 2u : 1u) * tn * 128u; }

template <bool EXACT>
int32_t launch_ts(bhd_ctx* ctx, dim3 grid, size_t dyn, const CUtensorMap& w0, const CUtensorMap& w1, const CUtensorMap& x, const CUtensorMap& xlo,
                  const TsParams& p, cudaStream_t s) {
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_ts<EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024), "raising the shared memory limit");
        once.mark(ctx);
    }
    k_gemm_q8_ts<EXACT><<<grid, THREADS, dyn, s>>>(w0, w1, x, xlo, p);
    BHD_LAUNCHED(ctx, EXACT ? "tcgen05 grouped expert kernel" : "tcgen05 matmul kernel (TMEM operand)");
    return BHD_OK;
}

}  // namespace

bool bhd_gemm_q8_ts_usable(const bhd_ctx* ctx, const bhd_weight* w) {
    return ctx->tmap_encode && w->kind == BHD_TYPE_Q8_0 && w->row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(w->dev) & 15) == 0 &&
           w->cols % 32 == 0 && w->cols != 0 && w->rows * w->slabs <= 0x7fffffffull;
}

// Grouped, exact form for the routed experts: every group of size class `cls` (consecutive rows of the
// fp16 activation arrays x_hi / x_lo [n_slots x K]) against its expert's slab of w0 (and of w1 for
// blockIdx.z == 1): out[slot][row] = col_scale[slot] * sum_k (x_hi + x_lo)[slot][k] * W[expert][row][k].
// `group_bound` bounds the class's group count (the grid's y extent); classes 2..5 = tiles of 16..128 rows.
int32_t bhd_launch_gemm_q8_ts_grouped(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                      const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* x_hi, const void* x_lo,
                                      uint32_t n_slots, float* out0, float* out1, float* const* row_dst, const float* col_scale,
                                      cudaStream_t s) {
    if (group_bound == 0) return BHD_OK;
    if (cls < 2 || cls > 5) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "grouped matmul: size class %u has no tensor-core form", cls);
    const uint32_t K = uint32_t(w0->cols), N = uint32_t(w0->rows), tn = 4u << cls;
    // Narrow tiles are bound by weight traffic: two stages leave shared and tensor memory for a second CTA per SM,
    // which covers the first one's start-up and drain.
    const uint32_t stages = tn <= 64 ? 2u : 4u;
    CUtensorMap mw0, mw1, mx, mxlo;
    if (!encode_weight_map(ctx, w0, &mw0) || !encode_weight_map(ctx, w1 ? w1 : w0, &mw1) || !encode_x_map(ctx, x_hi, n_slots, K, tn, &mx) ||
        !encode_x_map(ctx, x_lo, n_slots, K, tn, &mxlo))
        return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode a tensor map", bhd_device_name());
    TsParams p = {};
    p.y = out0;
    p.y1 = out1;
    p.row_dst = row_dst;
    p.status = ctx->status_dev;
    p.n_rows = N;
    p.k = K;
    p.tn = tn;
    p.stages = stages;
    p.hdr = static_cast<const MoeHeader*>(hdr);
    p.groups = static_cast<const MoeGroup*>(groups);
    p.glist = glist;
    p.cls = cls;
    p.col_scale = col_scale;
    return launch_ts<true>(ctx, dim3((N + TILE_N - 1) / TILE_N, group_bound, w1 ? 2 : 1), ts_smem_bytes(true, tn, stages), mw0, mw1, mx, mxlo, p, s);
}

// Dense, plain form (prefill): Y[m][n] = sum_k fp16(X[m][k]) * fp16(W[n][k]); x16 is the fp16 copy of X.
int32_t bhd_launch_gemm_q8_ts_dense(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M, cudaStream_t s) {
    const uint32_t K = uint32_t(w->cols), N = uint32_t(w->rows);
    const uint32_t tn = M >= 256 ? 256u : (M >= 128 ? 128u : 64u);
    const uint32_t stages = 4;
    CUtensorMap mw, mx;
    if (!encode_weight_map(ctx, w, &mw) || !encode_x_map(ctx, x16, M, K, tn, &mx))
        return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode a tensor map", bhd_device_name());
    TsParams p = {};
    p.y = y;
    p.status = ctx->status_dev;
    p.n_rows = N;
    p.row_base = uint32_t(slab * w->rows);
    p.m = M;
    p.k = K;
    p.tn = tn;
    p.stages = stages;
    return launch_ts<false>(ctx, dim3((N + TILE_N - 1) / TILE_N, (M + tn - 1) / tn), ts_smem_bytes(false, tn, stages), mw, mw, mx, mx, p, s);
}
