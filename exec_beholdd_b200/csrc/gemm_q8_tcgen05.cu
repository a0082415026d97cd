// Prefill matmul for packed Q8_0 weights on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   Y[m][n] = sum_k X[m][k] * W[n][k],   W packed Q8_0 [N x K], X f32 [M x K], M >= 64.
//
// A dense contraction (2*M*N*K flops against N*K*1.0625 weight bytes), bound by the tensor
// pipe once M is a few hundred. Mapping:
//   * The WEIGHTS are the 128-row MMA operand (A), the tokens are the N operand (B, 64/128/256
//     per tile), so one CTA produces a [128 weight rows x TN tokens] tile whose f32 accumulator
//     lives in TMEM (128 lanes x TN columns).
//   * Weights stay packed in HBM. One TMA copy stages a 128-row x 256-column chunk (272 B per
//     row); four converter warps (one thread per weight row) turn each 64-column slice into a
//     K-major, 128B-swizzled fp16 tile, folding the block scale in: a = fp16(d * q), one
//     rounding (q and d are exact in fp16).
//   * Activations are converted to fp16 once per call; TMA loads [TN x 64] slices with the
//     128B swizzle straight into the B tiles.
//   * Two elected threads (in different warps) issue tcgen05.mma (kind::f16, M = 128, N = TN,
//     K = 16) four times per 64-column slice, on alternate slices and into separate TMEM
//     accumulators, and commit to the stage's mbarrier; one thread alone needs about 0.6 us per
//     slice for its waits, issues and commit, which bounded the kernel at every tile width. The
//     first converter group then becomes the epilogue: tcgen05.ld both accumulators, add, and
//     store Y coalesced along n.
// Rings: 2 packed chunks, 3-4 fp16 stages. Every wait is bounded; a wait that gives up sets
// the status word, the roles drain and the CTA frees its TMEM before it returns.
//
// Reference semantics: a loop of Device::matvec over positions
// (crates/beholdd-model/src/qwen3moe/forward.rs:1086-1127) with kquant::q8_0::dot
// (crates/beholdd-kernel/src/kquant.rs:61-79); fp16 operands with f32 accumulation keep the
// result within the path's 2e-3 tolerance (measured in tests/test_gpu_parity.py).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;            // weight rows per CTA (MMA M)
constexpr int CHUNK_K = 256;           // columns per packed chunk
constexpr int SLICE_K = 64;            // columns per fp16 stage (one 128-byte swizzle row)
constexpr int PACK_ROW = 272;          // packed bytes per row per chunk
constexpr int PACK_BYTES = TILE_N * PACK_ROW;   // 34816, a multiple of 1024
constexpr int A_BYTES = TILE_N * SLICE_K * 2;   // 16384
// warp 0 weight-chunk TMA, warp 1 MMA (even slices) + TMEM, then NG groups of four converter warps (one thread
// per weight row) that take alternating slices; the first group is also the epilogue.
// after the converters: one warp that requests the activation tiles and the second MMA issuer
__host__ __device__ constexpr int gemm_threads(int ng) { return 64 + 128 * ng + 64; }
constexpr uint32_t SPIN_LIMIT = 1u << 24;

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
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
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

// Shared-memory matrix descriptor of a K-major, 128B-swizzled fp16 tile (rows of 128 bytes,
// 8-row groups 1024 bytes apart). Fields: start address >> 4 (bits 0-13), leading byte offset
// >> 4 (16-29, unused for this layout), stride byte offset >> 4 (32-45) = 1024 >> 4,
// descriptor version 1 (46-47), layout type 2 = SWIZZLE_128B (61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return uint64_t(lo) | (uint64_t(hi) << 32);
}
// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = f16 (0), both K-major,
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

// f32 -> f16 for the activations, flagging values fp16 cannot hold.
__global__ void k_f32_to_f16(const float* __restrict__ x, __half* __restrict__ out, uint64_t n, uint32_t* __restrict__ status) {
    // The matmul kernel behind this one may be scheduled as soon as every CTA here has started: it sets up and converts
    // its first weight slices meanwhile, and waits for this grid to finish before it loads a token.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint64_t i = (blockIdx.x * uint64_t(blockDim.x) + threadIdx.x) * 4;
    if (i >= n) return;
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    if (!(fabsf(fa.x) <= 65504.f && fabsf(fa.y) <= 65504.f && fabsf(fb.x) <= 65504.f && fabsf(fb.y) <= 65504.f))
        atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
    *reinterpret_cast<__half2*>(out + i) = a;
    *reinterpret_cast<__half2*>(out + i + 2) = b;
}

constexpr int PLAIN_NG = 2;  // converter groups: one cannot feed two MMA issuers

struct GemmParams {
    float* y;            // [M x N]; grouped: [slot][N] of matrix 0
    float* y1;           // grouped: [slot][N] of matrix 1 (blockIdx.z == 1), or null
    uint32_t* status;
    uint32_t n_rows;     // N: weight rows of one slab
    uint32_t row_base;   // tensor-map row of the slab's first row (dense mode)
    uint32_t m;          // tokens (dense mode)
    uint32_t k;          // columns
    uint32_t tn;         // tokens per tile: 32, 64, 128 or 256
    uint32_t stages;     // fp16 stages in the ring
    // Grouped mode (groups != null): blockIdx.y walks the groups of one size class; a group is `nb`
    // consecutive rows of the activation array (slots slot0 .. slot0 + nb) against the slab of its expert.
    const MoeHeader* hdr;
    const MoeGroup* groups;
    const int32_t* glist;
    uint32_t cls;
    const float* col_scale;  // optional factor per activation row, applied to its outputs
};

template <int NG>
__global__ void __launch_bounds__(gemm_threads(NG), 1) k_gemm_q8_tcgen05(const __grid_constant__ CUtensorMap tmap_w0,
                                                                const __grid_constant__ CUtensorMap tmap_w1,
                                                                const __grid_constant__ CUtensorMap tmap_x,
                                                                const GemmParams p) {
    // Which tokens and which slab this CTA works on. A CTA beyond the class's group count leaves at once
    // (the whole CTA, before any barrier or tensor memory exists).
    uint32_t m0, m_end, row_base;
    if (p.groups) {
        if (blockIdx.y >= p.hdr->gcount[p.cls]) return;
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
    // st_empty[s][k & 1]: the MMAs of the k-th use of stage s have finished reading it. Two barriers per
    // stage, alternating by use, because a converter group sees only every other use of a stage and the two
    // MMA issuers are not ordered with each other: on a single barrier a parity wait could be a whole phase
    // early. On its own barrier every waiter sees every phase.
    // a_full / b_full follow the same rule for the same reason: with an odd number of stages an MMA issuer
    // (alternate slices) meets only every other use of a stage.
    __shared__ uint64_t pk_full[2], pk_empty[2], a_full[8][2], b_full[8][2], st_empty[8][2], tmem_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t bn = p.tn;  // MMA N = rows of the B tile
    const uint32_t a_bytes = A_BYTES;
    const uint32_t stage_bytes = a_bytes + bn * 128u;
    const uint32_t pack_addr = smem0, stage_addr = smem0 + 2 * PACK_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int XW = 2 + 4 * NG, MW = 3 + 4 * NG;  // activation-tile producer warp, second MMA issuer warp
    const CUtensorMap* tmap_w = blockIdx.z ? &tmap_w1 : &tmap_w0;
    float* const yout = blockIdx.z ? p.y1 : p.y;
    const uint32_t n0 = blockIdx.x * TILE_N;
    const uint32_t slices = (p.k + SLICE_K - 1) / SLICE_K, chunks = (p.k + CHUNK_K - 1) / CHUNK_K;
    const uint32_t S = p.stages;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(&pk_full[i], 1); mbar_init(&pk_empty[i], 4 * NG); }
        for (uint32_t i = 0; i < S; ++i) {
            mbar_init(&a_full[i][0], 4);
            mbar_init(&a_full[i][1], 4);
            mbar_init(&b_full[i][0], 1);
            mbar_init(&b_full[i][1], 1);
            mbar_init(&st_empty[i][0], 1);
            mbar_init(&st_empty[i][1], 1);
        }
        mbar_init(&tmem_full, 2);  // both MMA issuers
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, 2 * bn);  // two accumulators; a power of two >= 32
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    auto give_up = [&]() { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); *(volatile int*)&abort_flag = 1; };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };
    // wait until the previous user of slice it's stage is done with it (true at once for the first use)
    auto stage_free = [&](uint32_t it) {
        const uint32_t use = it / S;
        if (use == 0) return true;
        const uint32_t k = use - 1;
        return mbar_wait(&st_empty[it % S][k & 1], (k >> 1) & 1);
    };

    if (warp == 0) {
        // ---- TMA producers: two independent request streams in two warps. This one keeps the two packed
        // weight chunks in flight (a chunk is requested as soon as its buffer is released); warp XW fetches the
        // activation tile of each slice as its stage frees up. ----
        if (lane == 0) {
            for (uint32_t c = 0; c < chunks && !aborted(); ++c) {
                const uint32_t pb = c & 1;
                if (!mbar_wait(&pk_empty[pb], ((c >> 1) & 1) ^ 1)) { give_up(); break; }
                mbar_arrive_expect_tx(&pk_full[pb], PACK_BYTES);
                tma_load_2d(pack_addr + pb * PACK_BYTES, tmap_w, int(c * (PACK_ROW / 2)), int(row_base + n0), &pk_full[pb]);
            }
        }
    } else if (warp == XW) {
        if (lane == 0) {
            for (uint32_t it = 0; it < slices && !aborted(); ++it) {
                const uint32_t s = it % S;
                if (!stage_free(it)) { give_up(); break; }
                uint64_t* bf = &b_full[s][(it / S) & 1];
                mbar_arrive_expect_tx(bf, bn * 128u);
                tma_load_2d(stage_addr + s * stage_bytes + a_bytes, &tmap_x, int(it * SLICE_K), int(m0), bf);
            }
        }
    } else if (warp == 1 || warp == MW) {
        // ---- MMA issuers. One thread needs about 0.6 us per slice just to get through its two barrier
        // waits, four tcgen05.mma and the commit, whatever the tile width; so two threads take alternate
        // slices, each accumulating into its own TMEM columns (no ordering is needed between them), and
        // the epilogue adds the two accumulators. ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(TILE_N, bn);
            const uint32_t first = warp == 1 ? 0u : 1u, acc = tmem_base + first * bn;
            bool ok = true;
            for (uint32_t it = first; it < slices && ok; it += 2) {
                const uint32_t s = it % S, use = it / S, par = (use >> 1) & 1;
                if (aborted() || !mbar_wait(&b_full[s][use & 1], par) || !mbar_wait(&a_full[s][use & 1], par)) { give_up(); ok = false; break; }
                tc_fence_after();
                const uint64_t da = umma_desc(stage_addr + s * stage_bytes), db = umma_desc(stage_addr + s * stage_bytes + a_bytes);
#pragma unroll
                for (uint32_t k16 = 0; k16 < 4; ++k16)  // 32 bytes (16 fp16) further along the swizzled row per step
                    tc_mma_f16(acc, da + 2 * k16, db + 2 * k16, idesc, (it != first || k16) ? 1u : 0u);
                tc_commit(&st_empty[s][(it / S) & 1]);  // arrives when these MMAs have finished reading the stage
            }
            tc_commit(&tmem_full);        // arrives when every MMA this thread issued is complete
        }
    } else {
        // ---- converters: NG groups of four warps take alternating 64-column slices; thread = one weight row ----
        const uint32_t ct = threadIdx.x - 64;   // 0..255
        const uint32_t row = ct & 127, grp = ct >> 7;  // grp is uniform per warp
        const uint32_t sw = row & 7, a_row_off = (row >> 3) * 1024 + sw * 128;
        bool ok = true;
        for (uint32_t c = 0; c < chunks && ok; ++c) {
            const uint32_t pb = c & 1;
            if (aborted() || !mbar_wait(&pk_full[pb], (c >> 1) & 1)) { give_up(); ok = false; break; }
            const uint32_t src_row = pack_addr + pb * PACK_BYTES + row * PACK_ROW;
#pragma unroll
            for (uint32_t kb = 0; kb < 4; ++kb) {  // unrolled so that the register indices below are constants
                if (kb % NG != grp) continue;      // uniform per warp
                const uint32_t it = c * 4 + kb;
                if (it >= slices) break;
                const uint32_t s = it % S;
                if (!stage_free(it)) { give_up(); ok = false; break; }
                // Two Q8_0 blocks = 68 bytes = 17 words [d0 | q0..q31 | d1 | q32..q63], starting at word 17 * kb of
                // the row. Read as five aligned 16-byte loads from word 16 * kb: rows are 272 bytes apart, so the
                // eight lanes of a quarter-warp hit eight different 16-byte bank groups (no conflicts), and the
                // slice's words are v[kb .. kb + 16].
                uint32_t v[20];
#pragma unroll
                for (int i = 0; i < 5; ++i) {
                    const uint4 q4 = lds128(src_row + kb * 64 + 16 * i);
                    v[4 * i] = q4.x; v[4 * i + 1] = q4.y; v[4 * i + 2] = q4.z; v[4 * i + 3] = q4.w;
                }
                const uint32_t* w = v + kb;
                const uint32_t a_dst = stage_addr + s * stage_bytes + a_row_off;
                const __half2 off = __half2half2(__ushort_as_half(uint16_t(0x6480)));  // 1152
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    const uint32_t dbits = blk == 0 ? (w[0] & 0xffffu) : (w[8] >> 16);
                    const __half2 d2 = __half2half2(__ushort_as_half(uint16_t(dbits)));
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {  // 8 quants -> one 16-byte chunk of the swizzled row
                        uint32_t q[2];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int i = 2 * ch + j;
                            q[j] = blk == 0 ? __funnelshift_r(w[i], w[i + 1], 16) : w[9 + i];
                        }
                        uint32_t h[4];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t u = q[j] ^ 0x80808080u;  // 0x6400 | (q + 128) is the fp16 q + 1152
                            const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140), hi = __byte_perm(u, 0x64646464u, 0x4342);
                            const __half2 qa = __hsub2(*reinterpret_cast<const __half2*>(&lo), off);
                            const __half2 qb = __hsub2(*reinterpret_cast<const __half2*>(&hi), off);
                            const __half2 a = __hmul2(qa, d2), b = __hmul2(qb, d2);
                            h[2 * j] = *reinterpret_cast<const uint32_t*>(&a);
                            h[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                        }
                        const uint32_t chunk16 = uint32_t(blk * 4 + ch) ^ sw;  // 128B swizzle: chunk index XOR row mod 8
                        sts128(a_dst + chunk16 * 16, make_uint4(h[0], h[1], h[2], h[3]));
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[s][(it / S) & 1]);  // one arrival per converter warp
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pk_empty[pb]);
        }
        // ---- epilogue: TMEM lane = weight row, column = token ------------------------------------
        if (warp >= 6) {
            // warps 6-9 only convert
        } else if (ok && !aborted() && mbar_wait(&tmem_full, 0)) {
            tc_fence_after();
            const uint32_t q = warp & 3;                 // the TMEM lane quarter this warp may read
            const uint32_t n = n0 + q * 32 + lane;
            for (uint32_t col = 0; col < p.tn; col += 32) {
                if (m0 + col >= m_end) break;            // uniform across the warp
                uint32_t r[32];
                tc_ld32(tmem_base + ((q * 32u) << 16) + col, r);
                if (slices > 1) {  // the odd slices' accumulator
                    uint32_t r2[32];
                    tc_ld32(tmem_base + ((q * 32u) << 16) + bn + col, r2);
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
                }
                if (n < p.n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t m = m0 + col + j;
                        if (m < m_end) {
                            const float sc = p.col_scale ? p.col_scale[m] : 1.0f;
                            yout[uint64_t(m) * p.n_rows + n] = __fmul_rn(__uint_as_float(r[j]), sc);
                        }
                    }
                }
            }
        } else if (ok) {
            give_up();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * bn);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

// Grouped form for the routed experts: every group of size class `cls` (17 or more routes of one expert,
// consecutive rows of the fp16 activation array x16 [n_slots x K]) against its expert's slab of w0 (and
// of w1 for blockIdx.z == 1): out[slot][row] = col_scale[slot] * sum_k x16[slot][k] * W[expert][row][k].
// `group_bound` is an upper bound of the class's group count (the grid's y extent); tn = the class's
// largest group, 32 to 256 tokens per tile.
int32_t bhd_launch_gemm_q8_grouped(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                   const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* x16, uint32_t n_slots,
                                   float* out0, float* out1, const float* col_scale, cudaStream_t s) {
    if (group_bound == 0) return BHD_OK;
    const uint32_t K = uint32_t(w0->cols), N = uint32_t(w0->rows);
    const uint32_t tn = 4u << cls;  // classes 2..6 -> 16, 32, 64, 128, 256
    if (cls < 2 || cls > 6) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "grouped matmul: size class %u has no tensor-core form", cls);
    // Two stages leave room for two CTAs per SM at the narrow tiles, where the kernel is bound by weight traffic
    // and a second CTA covers the first one's start-up and drain; the wide tiles keep deeper rings.
    const uint32_t stages = tn == 256 ? 3u : (tn <= 32 ? 2u : 4u);
    const size_t dyn = 1024 + 2 * size_t(PACK_BYTES) + size_t(stages) * (A_BYTES + tn * 128u);
    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode);
    CUtensorMap map_w[2], map_x;
    for (int i = 0; i < 2; ++i) {
        const bhd_weight* w = (i == 1 && w1) ? w1 : w0;
        const cuuint64_t dims[2] = {w->row_bytes / 2, w->rows * w->slabs};
        const cuuint64_t strides[1] = {w->row_bytes};
        const cuuint32_t box[2] = {PACK_ROW / 2, TILE_N};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the expert tensor map", bhd_device_name());
    }
    {
        const cuuint64_t dims[2] = {K, n_slots};
        const cuuint64_t strides[1] = {uint64_t(K) * 2};
        const cuuint32_t box[2] = {SLICE_K, tn};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the activation tensor map", bhd_device_name());
    }
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_tcgen05<PLAIN_NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024),
                 "raising the shared memory limit");
        once.mark(ctx);
    }
    GemmParams p = {};
    p.y = out0;
    p.y1 = out1;
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
    k_gemm_q8_tcgen05<PLAIN_NG><<<dim3((N + TILE_N - 1) / TILE_N, group_bound, w1 ? 2 : 1), gemm_threads(PLAIN_NG), dyn, s>>>(
        map_w[0], map_w[1], map_x, p);
    BHD_LAUNCHED(ctx, "tcgen05 grouped expert kernel");
    return BHD_OK;
}

bool bhd_gemm_q8_grouped_usable(const bhd_ctx* ctx, const bhd_weight* w) {
    return ctx->tmap_encode && w->kind == BHD_TYPE_Q8_0 && w->row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(w->dev) & 15) == 0 &&
           w->cols % 32 == 0 && w->cols != 0 && w->rows * w->slabs <= 0x7fffffffull;
}

// Tensor-core path of bhd_matmul: Q8_0 weights, M >= 64 tokens. Sets *handled = false when the
// shape does not qualify (the caller then uses the batched matvec kernels).
int32_t bhd_launch_gemm_q8_tcgen05(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y, uint64_t m,
                                   cudaStream_t s, bool* handled) {
    *handled = false;
    // Q8_0 from 64 tokens on; Q4_K and Q6_K from 256 tokens on (the CTA-pair kernel converts all three, the per-tile kernels
    // Q8_0 only)
    const bool q4 = (w->kind == BHD_TYPE_Q4_K || w->kind == BHD_TYPE_Q6_K) && m >= 256 && w->cols % 256 == 0 && w->row_bytes % 16 == 0 &&
                    (ctx->gemm_impl == 0 || ctx->gemm_impl == 3 || ctx->gemm_impl == 5);
    if ((w->kind != BHD_TYPE_Q8_0 && !q4) || !ctx->tmap_encode || m < 64 || m > 0x7fffffffull) return BHD_OK;
    if (w->row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(w->dev) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return BHD_OK;
    if (w->cols == 0 || w->cols % 32 != 0 || w->rows > 0x7fffffffull || w->rows * w->slabs > 0x7fffffffull) return BHD_OK;
    const uint32_t K = uint32_t(w->cols), N = uint32_t(w->rows), M = uint32_t(m);
    const uint32_t tn = M >= 256 ? 256u : (M >= 128 ? 128u : 64u);
    const uint32_t stages = tn == 256 ? 3u : 4u;
    const size_t dyn = 1024 + 2 * size_t(PACK_BYTES) + size_t(stages) * (A_BYTES + tn * 128u);

    // fp16 copy of the activations in the workspace
    const size_t x16_bytes = align_up(size_t(M) * K * 2, 256);
    int32_t st = bhd_ensure_workspace(ctx, x16_bytes, s);
    if (st != BHD_OK) return st;
    __half* x16 = reinterpret_cast<__half*>(ctx->workspace);
    const uint64_t n_elems = uint64_t(M) * K;
    k_f32_to_f16<<<unsigned((n_elems / 4 + 255) / 256), 256, 0, s>>>(x, x16, n_elems, ctx->status_dev);
    BHD_LAUNCHED(ctx, "activation fp16 conversion kernel");
    // 0: the library's choice, 1: one CTA per tile, 2: the same with the weight operand in tensor memory, 3: CTA pairs on
    // 256-token tiles, 4: persistent single CTAs, 5: CTA pairs on 512-token tiles.
    // The choice: pairs from 256 tokens on. A 512-token tile takes about 1.6 times as long as a 256-token tile (its
    // write-back is not overlapped) for twice the work, and tiles are dealt to the SM pairs in whole rounds.
    uint32_t impl = ctx->gemm_impl;
    if (impl == 0) {
        impl = 1;
        if (M >= 256) {
            int sms = 148;
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device);
            const uint32_t pairs = uint32_t(sms > 1 ? sms / 2 : 1), row_pairs = (N + 255) / 256;
            const uint32_t rounds_narrow = (row_pairs * ((M + 255) / 256) + pairs - 1) / pairs, rounds_wide = (row_pairs * ((M + 511) / 512) + pairs - 1) / pairs;
            impl = (M > 256 && 1.6f * float(rounds_wide) <= float(rounds_narrow)) ? 5u : 3u;
        }
    }
    if (impl != 1) {
        if ((impl == 3 || impl == 5) && M >= 256) st = bhd_launch_gemm_q8_pair(ctx, w, slab, x16, y, M, impl == 5, s);
        else if (impl == 2) st = bhd_launch_gemm_q8_ts_dense(ctx, w, slab, x16, y, M, s);
        else st = bhd_launch_gemm_q8_persistent(ctx, w, slab, x16, y, M, s);
        *handled = st == BHD_OK;
        return st;
    }
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
        if (encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: cannot encode the activation tensor map", bhd_device_name());
    }
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        BHD_CUDA(ctx, cudaFuncSetAttribute(k_gemm_q8_tcgen05<PLAIN_NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024),
                 "raising the shared memory limit");
        once.mark(ctx);
    }
    GemmParams p = {};
    p.y = y;
    p.status = ctx->status_dev;
    p.n_rows = N;
    p.row_base = uint32_t(slab * w->rows);
    p.m = M;
    p.k = K;
    p.tn = tn;
    p.stages = stages;
    k_gemm_q8_tcgen05<PLAIN_NG><<<dim3((N + TILE_N - 1) / TILE_N, (M + tn - 1) / tn), gemm_threads(PLAIN_NG), dyn, s>>>(map_w, map_w, map_x, p);
    BHD_LAUNCHED(ctx, "tcgen05 matmul kernel");
    *handled = true;
    return BHD_OK;
}
