// Batched dequant-fused matvec for packed Q8_0 / Q4_K / Q6_K weights on sm_100a.
//
// The operation is HBM-bound (0.56 - 1.06 bytes per weight, a handful of activation vectors),
// so the kernel is built around keeping many bytes in flight and spending as few issue slots
// per byte as possible:
//
//   * Packed rows stay in their checkpoint layout. A 2-D tensor map over [rows][row_bytes]
//     lets one TMA instruction per stage stage a 64-row x 256-column chunk (272 / 144 / 240
//     bytes per row) into shared memory; a 3-4 deep mbarrier ring per CTA keeps the copies
//     ahead of the math. The chunk widths happen to shift consecutive rows by 16 bytes
//     modulo 128, so the unpacking reads are free of bank conflicts.
//   * Unpacking never converts to f32. Quants are turned into fp16 bit patterns with one or
//     two logic ops per pair ("0x6400 | q" is 1024 + q) and fed to mma.sync m16n8k16 with the
//     weights as the 16-row operand and the activation vectors as the 8 columns. The constant
//     offset and the block scales are applied in f32 to the per-block partial sums, using
//     per-block activation sums prepared once.
//   * Activations are split into two fp16 halves (x = hi + lo, relative error 2^-22) that sit
//     in adjacent MMA columns, so the products are exact and accumulation is f32.
//   * Work is cut into (row tile, column chunk) stages and dealt to the resident CTAs as
//     equal contiguous ranges. A row tile whose stages straddle CTAs is finished by the last
//     CTA to arrive, which adds the partial sums in column order: results do not depend on
//     scheduling and are bit-identical from run to run.
//
// Reference semantics: crates/beholdd-backend/src/cpu.rs:398-507 (y = acc*scale or
// y += acc*scale); block formats: crates/beholdd-kernel/src/kquant.rs:29-241.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TILE_ROWS = 64;     // rows per CTA stage: 4 consumer warps x one 16-row MMA tile
constexpr int CHUNK_K = 256;      // columns per stage
constexpr int STEPS = 16;         // k16 MMA steps per stage
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

template <uint32_t KIND> struct Fmt;
template <> struct Fmt<BHD_TYPE_Q8_0> { static constexpr int BOX = 272, CHUNK_BYTES = 272, GROUPS = 8; };
template <> struct Fmt<BHD_TYPE_Q4_K> { static constexpr int BOX = 144, CHUNK_BYTES = 144, GROUPS = 8; };
template <> struct Fmt<BHD_TYPE_Q6_K> { static constexpr int BOX = 240, CHUNK_BYTES = 210, GROUPS = 16; };

__host__ __device__ constexpr int groups_of(uint32_t kind) { return kind == BHD_TYPE_Q6_K ? 16 : 8; }

// Size of one chunk of packed activations: STEPS x NT MMA B-fragments (32 lanes x 8 bytes)
// followed by GROUPS x NT x 8 f32 column sums.
__host__ __device__ constexpr int xblob_bytes(uint32_t kind, int nt) { return STEPS * nt * 256 + groups_of(kind) * nt * 32; }

// First of the four consecutive columns (within a chunk) that lane-in-quad t supplies to MMA
// step s. Consumers read the matching packed bytes; the activation packer uses the same map.
__host__ __device__ __forceinline__ int chunk_k4(uint32_t kind, int s, int t) {
    if (kind == BHD_TYPE_Q8_0) return 32 * (s >> 1) + 16 * (s & 1) + 4 * t;          // block s/2, half s%2
    if (kind == BHD_TYPE_Q4_K) {                                                     // sub-block s/2
        const int j = s >> 1, hs = s & 1;
        return 64 * (j >> 1) + 32 * (j & 1) + 8 * t + 4 * hs;
    }
    return 128 * (s >> 3) + 32 * ((s & 7) >> 1) + 16 * (s & 1) + 4 * t;              // Q6_K: half, group, 16-lane half
}

// ---- PTX wrappers -------------------------------------------------------------------------

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
// Bounded wait: returns false when the phase did not complete within the spin limit.
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
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint2 lds64(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half(uint16_t(h))); }

// ---- activation packer ------------------------------------------------------------------
// Builds, for one 256-column chunk and one n-tile j, the MMA B-fragments of up to 8 columns.
// Split mode: column n is activation vector 4j + n/2, its fp16 high part (n even) or the fp16
// remainder (n odd), so x = hi + lo to 2^-22. Plain mode: column n is vector 8j + n rounded to
// fp16. `row` is this lane's source row (nullptr: the column is padding and packs as zero);
// with `row2` the value packed is silu(row[i]) * row2[i] (crates/beholdd-kernel/src/vecops.rs:
// 91-111, limit 0). Must be called by all 512 threads of the CTA (16 steps x 32 lanes).
__device__ __forceinline__ void pack_tile(uint32_t kind, const float* row, const float* row2, bool lo_part, uint32_t chunk,
                                          uint32_t K, int nt, int j, uint8_t* cb, float (*stepsum)[8], uint32_t* status) {
    const int s = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t k4 = chunk * CHUNK_K + chunk_k4(kind, s, t);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row && k4 < K) {
        v = *reinterpret_cast<const float4*>(row + k4);
        if (row2) {
            const float4 u = *reinterpret_cast<const float4*>(row2 + k4);
            v.x = __fmul_rn(__fdiv_rn(v.x, __fadd_rn(1.0f, expf(-v.x))), u.x);
            v.y = __fmul_rn(__fdiv_rn(v.y, __fadd_rn(1.0f, expf(-v.y))), u.y);
            v.z = __fmul_rn(__fdiv_rn(v.z, __fadd_rn(1.0f, expf(-v.z))), u.z);
            v.w = __fmul_rn(__fdiv_rn(v.w, __fadd_rn(1.0f, expf(-v.w))), u.w);
        }
    }
    float e[4] = {v.x, v.y, v.z, v.w};
    uint32_t hbits[4];
    float part[4];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half hi = __float2half_rn(e[i]);
        const float hif = __half2float(hi);
        bad |= !(fabsf(hif) <= 65504.0f);  // overflow to inf, or NaN input
        const __half sel = lo_part ? __float2half_rn(e[i] - hif) : hi;
        hbits[i] = __half_as_ushort(sel);
        part[i] = __half2float(sel);
    }
    if (bad) atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
    // Q4_K's unpacking yields the four columns in the order 0,2,1,3.
    uint2 frag;
    if (kind == BHD_TYPE_Q4_K) frag = make_uint2(hbits[0] | (hbits[2] << 16), hbits[1] | (hbits[3] << 16));
    else frag = make_uint2(hbits[0] | (hbits[1] << 16), hbits[2] | (hbits[3] << 16));
    *reinterpret_cast<uint2*>(cb + (s * nt + j) * 256 + lane * 8) = frag;
    float sum = (part[0] + part[1]) + (part[2] + part[3]);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    __syncthreads();  // stepsum may still be read for the previous n-tile
    if (t == 0) stepsum[s][g] = sum;
    __syncthreads();
    const int groups = groups_of(kind), per = STEPS / groups;
    if (int(threadIdx.x) < groups * 8) {
        const int grp = threadIdx.x >> 3, n = threadIdx.x & 7;
        float acc = 0.f;
        for (int i = 0; i < per; ++i) acc += stepsum[grp * per + i][n];
        reinterpret_cast<float*>(cb + STEPS * nt * 256)[(grp * nt + j) * 8 + n] = acc;
    }
}

// Programmatic dependent launch (no-ops when the kernel was launched without the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// x [batch x K] f32 -> one blob per chunk, split mode. grid (chunks, nt), 512 threads.
__global__ void k_pack_x(uint32_t kind, const float* __restrict__ x, uint64_t ldx, uint32_t batch, uint32_t K, int nt,
                         uint8_t* __restrict__ blob, uint32_t* __restrict__ status) {
    __shared__ float stepsum[STEPS][8];
    // let the matvec kernel start its weight prefetch; wait for whatever produced x and for the
    // previous matvec, which may still be reading the blob
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.y, g = (threadIdx.x & 31) >> 2;
    const uint32_t b = 4 * j + (g >> 1);
    pack_tile(kind, b < batch ? x + uint64_t(b) * ldx : nullptr, nullptr, g & 1, blockIdx.x, K, nt, j,
              blob + uint64_t(blockIdx.x) * xblob_bytes(kind, nt), stepsum, status);
}

// ---- main kernel ------------------------------------------------------------------------------

struct MatvecParams {
    const uint8_t* xblob;   // packed activations, one blob per chunk
    float* y;               // [batch x rows]
    float* partial;         // stream-K partial sums
    uint32_t* counters;     // one per (row tile, warp), zero between launches
    uint32_t* status;
    uint32_t rows;          // rows of this slab
    uint32_t row_base;      // tensor-map row of the slab's first row
    uint32_t batch;
    uint32_t chunks;        // chunks per row (ceil(K / 256))
    uint32_t total_stages;  // row tiles * chunks
    uint32_t per_cta;       // stages per CTA
    float scale;
    int accumulate;
    const float* vec_scale; // optional per-vector factor (replaces `scale`)
};

template <uint32_t KIND, int NT>
struct Smem {
    static constexpr int W_BYTES = TILE_ROWS * Fmt<KIND>::BOX;
    static constexpr int X_BYTES = xblob_bytes(KIND, NT);
    static constexpr int STAGE = (W_BYTES + X_BYTES + 127) / 128 * 128;
    static constexpr int X_OFF = (W_BYTES + 15) / 16 * 16;
};

// MMA row m (0..15) of a warp's tile -> row within the warp's 16 rows. Q4_K reads 8 bytes per
// lane, so rows are interleaved to keep each half-warp's accesses on distinct banks.
template <uint32_t KIND>
__device__ __forceinline__ int tile_row(int m) {
    if (KIND == BHD_TYPE_Q4_K) return m < 8 ? 2 * m : 2 * (m - 8) + 1;
    return m;
}

template <uint32_t KIND, int NT>
__device__ __forceinline__ void consume_stage(const uint8_t* __restrict__ wrow0, const uint8_t* __restrict__ wrow1,
                                              const uint8_t* __restrict__ xb, int lane, uint32_t q6_off,
                                              float (&tot)[NT][4]) {
    const int t = lane & 3;
    const uint8_t* bfrag = xb + lane * 8;
    const float* sx = reinterpret_cast<const float*>(xb + STEPS * NT * 256) + 2 * t;

    if constexpr (KIND == BHD_TYPE_Q8_0) {
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            float raw[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) raw[j][0] = raw[j][1] = raw[j][2] = raw[j][3] = 0.f;
            const float d0 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(wrow0 + 34 * blk));
            const float d1 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(wrow1 + 34 * blk));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int off = 34 * blk + 2 + 16 * h + 4 * t;  // quant bytes of this lane
                uint32_t w0, w1;
                if (blk & 1) {  // 4-byte aligned
                    w0 = lds32(wrow0 + off);
                    w1 = lds32(wrow1 + off);
                } else {        // 2 mod 4: stitch two aligned words
                    w0 = __funnelshift_r(lds32(wrow0 + off - 2), lds32(wrow0 + off + 2), 16);
                    w1 = __funnelshift_r(lds32(wrow1 + off - 2), lds32(wrow1 + off + 2), 16);
                }
                w0 ^= 0x80808080u;  // int8 -> biased uint8; 0x6400 | u is the fp16 1024 + u = q + 1152
                w1 ^= 0x80808080u;
                const uint32_t a0 = __byte_perm(w0, 0x64646464u, 0x4140), a2 = __byte_perm(w0, 0x64646464u, 0x4342);
                const uint32_t a1 = __byte_perm(w1, 0x64646464u, 0x4140), a3 = __byte_perm(w1, 0x64646464u, 0x4342);
                const int s = 2 * blk + h;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint2 b = lds64(bfrag + (s * NT + j) * 256);
                    mma_f16(raw[j], a0, a1, a2, a3, b.x, b.y);
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const float2 sxv = *reinterpret_cast<const float2*>(sx + (blk * NT + j) * 8);
                tot[j][0] = fmaf(d0, fmaf(-1152.f, sxv.x, raw[j][0]), tot[j][0]);
                tot[j][1] = fmaf(d0, fmaf(-1152.f, sxv.y, raw[j][1]), tot[j][1]);
                tot[j][2] = fmaf(d1, fmaf(-1152.f, sxv.x, raw[j][2]), tot[j][2]);
                tot[j][3] = fmaf(d1, fmaf(-1152.f, sxv.y, raw[j][3]), tot[j][3]);
            }
        }
    } else if constexpr (KIND == BHD_TYPE_Q4_K) {
        // Header: d, dmin (f16) and twelve bytes of packed 6-bit scales / mins.
        const uint4 h0 = *reinterpret_cast<const uint4*>(wrow0);
        const uint4 h1 = *reinterpret_cast<const uint4*>(wrow1);
        const float d0 = half_bits_to_float(h0.x & 0xffffu), m0 = half_bits_to_float(h0.x >> 16);
        const float d1 = half_bits_to_float(h1.x & 0xffffu), m1 = half_bits_to_float(h1.x >> 16);
        auto scale_min = [](const uint4& h, int j, uint32_t& sc, uint32_t& mn) {
            // bytes q[0..11] live in h.y, h.z, h.w (crates/beholdd-kernel/src/kquant.rs:176-185)
            auto byte = [&](int i) -> uint32_t { const uint32_t w = i < 4 ? h.y : (i < 8 ? h.z : h.w); return (w >> (8 * (i & 3))) & 0xffu; };
            if (j < 4) { sc = byte(j) & 63u; mn = byte(j + 4) & 63u; }
            else { sc = (byte(j + 4) & 0xFu) | ((byte(j - 4) >> 6) << 4); mn = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4); }
        };
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 q0 = lds64(wrow0 + 16 + 32 * p + 8 * t);
            const uint2 q1 = lds64(wrow1 + 16 + 32 * p + 8 * t);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int j = 2 * p + nib;
                float raw[NT][4];
#pragma unroll
                for (int jj = 0; jj < NT; ++jj) raw[jj][0] = raw[jj][1] = raw[jj][2] = raw[jj][3] = 0.f;
#pragma unroll
                for (int hs = 0; hs < 2; ++hs) {
                    const uint32_t w0 = hs ? q0.y : q0.x, w1 = hs ? q1.y : q1.x;
                    uint32_t a0, a1, a2, a3;
                    if (nib == 0) {  // low nibbles: 0x6400 | q = 1024 + q
                        a0 = (w0 & 0x000F000Fu) | 0x64006400u; a2 = ((w0 >> 8) & 0x000F000Fu) | 0x64006400u;
                        a1 = (w1 & 0x000F000Fu) | 0x64006400u; a3 = ((w1 >> 8) & 0x000F000Fu) | 0x64006400u;
                    } else {         // high nibbles in place: 0x5400 | (q << 4) = 64 + q
                        a0 = (w0 & 0x00F000F0u) | 0x54005400u; a2 = ((w0 >> 8) & 0x00F000F0u) | 0x54005400u;
                        a1 = (w1 & 0x00F000F0u) | 0x54005400u; a3 = ((w1 >> 8) & 0x00F000F0u) | 0x54005400u;
                    }
                    const int s = 2 * j + hs;
#pragma unroll
                    for (int jj = 0; jj < NT; ++jj) {
                        const uint2 b = lds64(bfrag + (s * NT + jj) * 256);
                        mma_f16(raw[jj], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                uint32_t sc0, mn0, sc1, mn1;
                scale_min(h0, j, sc0, mn0);
                scale_min(h1, j, sc1, mn1);
                const float off = nib ? 64.f : 1024.f;
                const float ds0 = d0 * float(sc0), ds1 = d1 * float(sc1);
                const float c0 = fmaf(ds0, off, m0 * float(mn0)), c1 = fmaf(ds1, off, m1 * float(mn1));
#pragma unroll
                for (int jj = 0; jj < NT; ++jj) {
                    const float2 sxv = *reinterpret_cast<const float2*>(sx + (j * NT + jj) * 8);
                    tot[jj][0] += fmaf(ds0, raw[jj][0], -c0 * sxv.x);
                    tot[jj][1] += fmaf(ds0, raw[jj][1], -c0 * sxv.y);
                    tot[jj][2] += fmaf(ds1, raw[jj][2], -c1 * sxv.x);
                    tot[jj][3] += fmaf(ds1, raw[jj][3], -c1 * sxv.y);
                }
            }
        }
    } else {  // Q6_K: the superblock starts q6_off bytes into the staged 240-byte window
        const uint32_t sh = 8u * (q6_off & 3u);
        const uint8_t* b0 = wrow0 + (q6_off & ~3u);
        const uint8_t* b1 = wrow1 + (q6_off & ~3u);
        auto word = [&](const uint8_t* base, int byte_off) -> uint32_t {  // unaligned 32-bit read at base + byte_off
            return __funnelshift_r(lds32(base + byte_off), lds32(base + byte_off + 4), sh);
        };
        const float d0 = half_bits_to_float(word(b0, 208) & 0xffffu), d1 = half_bits_to_float(word(b1, 208) & 0xffffu);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
            for (int lam = 0; lam < 2; ++lam) {
                const uint32_t qh0 = word(b0, 128 + 32 * hf + 16 * lam + 4 * t), qh1 = word(b1, 128 + 32 * hf + 16 * lam + 4 * t);
#pragma unroll
                for (int gp = 0; gp < 2; ++gp) {  // low-plane byte range shared by groups gp and gp + 2
                    const uint32_t ql0 = word(b0, 64 * hf + 32 * gp + 16 * lam + 4 * t), ql1 = word(b1, 64 * hf + 32 * gp + 16 * lam + 4 * t);
#pragma unroll
                    for (int up = 0; up < 2; ++up) {
                        const int grp = gp + 2 * up;          // group within the half: 0..3
                        const int s = 8 * hf + 2 * grp + lam;  // MMA step == 16-element scale group
                        const uint32_t c0 = ((ql0 >> (4 * up)) & 0x0F0F0F0Fu) | (((qh0 >> (2 * grp)) & 0x03030303u) << 4);
                        const uint32_t c1 = ((ql1 >> (4 * up)) & 0x0F0F0F0Fu) | (((qh1 >> (2 * grp)) & 0x03030303u) << 4);
                        const uint32_t a0 = __byte_perm(c0, 0x64646464u, 0x4140), a2 = __byte_perm(c0, 0x64646464u, 0x4342);
                        const uint32_t a1 = __byte_perm(c1, 0x64646464u, 0x4140), a3 = __byte_perm(c1, 0x64646464u, 0x4342);
                        // int8 sub-block scales: byte s of the 16 scale bytes
                        const uint32_t sw0 = word(b0, 192 + (s & ~3)), sw1 = word(b1, 192 + (s & ~3));
                        const float s0 = d0 * float(int8_t((sw0 >> (8 * (s & 3))) & 0xffu));
                        const float s1 = d1 * float(int8_t((sw1 >> (8 * (s & 3))) & 0xffu));
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            float raw[4] = {0.f, 0.f, 0.f, 0.f};
                            const uint2 b = lds64(bfrag + (s * NT + j) * 256);
                            mma_f16(raw, a0, a1, a2, a3, b.x, b.y);
                            const float2 sxv = *reinterpret_cast<const float2*>(sx + (s * NT + j) * 8);
                            // codes carry 1024 + c; the value is c - 32
                            tot[j][0] = fmaf(s0, fmaf(-1056.f, sxv.x, raw[0]), tot[j][0]);
                            tot[j][1] = fmaf(s0, fmaf(-1056.f, sxv.y, raw[1]), tot[j][1]);
                            tot[j][2] = fmaf(s1, fmaf(-1056.f, sxv.x, raw[2]), tot[j][2]);
                            tot[j][3] = fmaf(s1, fmaf(-1056.f, sxv.y, raw[3]), tot[j][3]);
                        }
                    }
                }
            }
        }
    }
}

// The body shared by the plain and the grouped kernel: CTA `cta_index` streams stages
// [cta_index * per_cta, +per_cta) of the (row tile, chunk) sequence described by p.
// SPLIT says what the 8 columns of an n-tile are (see pack_tile).
template <uint32_t KIND, int NT, bool SPLIT>
__device__ __forceinline__ void run_stage_range(const CUtensorMap* tmap_ptr, const MatvecParams& p, uint32_t cta_index,
                                                int n_stages_ring) {
    using S = Smem<KIND, NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);  // TMA destinations need 128-byte alignment
    __shared__ uint64_t full_bar[8], empty_bar[8];
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t s_begin = cta_index * p.per_cta;
    const uint32_t s_end = min(s_begin + p.per_cta, p.total_stages);
    if (s_begin >= s_end) return;

    if (threadIdx.x == 0) {
        for (int i = 0; i < n_stages_ring; ++i) {
            mbar_init(&full_bar[i], 1);
            mbar_init(&empty_bar[i], CONSUMER_WARPS);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    pdl_launch_dependents();
    if (warp == CONSUMER_WARPS) {
        // ---- producer: one lane issues the copies of every stage. The weights of the first
        // ring of stages are requested before waiting for the grids this launch depends on
        // (weights are never written by a preceding kernel); the packed activations after. ----
        if (lane == 0) {
            auto copy_w = [&](uint32_t s, uint32_t slot) {
                const uint32_t tile = s / p.chunks, chunk = s - tile * p.chunks;
                mbar_arrive_expect_tx(&full_bar[slot], S::W_BYTES + S::X_BYTES);
                // Inner coordinate in 2-byte elements; its byte offset is a multiple of 16.
                const uint32_t byte0 = (KIND == BHD_TYPE_Q6_K) ? ((210u * chunk) & ~15u) : Fmt<KIND>::CHUNK_BYTES * chunk;
                tma_load_2d(smem + slot * S::STAGE, tmap_ptr, int(byte0 >> 1), int(p.row_base + tile * TILE_ROWS), &full_bar[slot]);
            };
            auto copy_x = [&](uint32_t s, uint32_t slot) {
                const uint32_t chunk = s % p.chunks;
                bulk_load_1d(smem + slot * S::STAGE + S::X_OFF, p.xblob + uint64_t(chunk) * S::X_BYTES, S::X_BYTES, &full_bar[slot]);
            };
            const uint32_t head = min(uint32_t(n_stages_ring), s_end - s_begin);
            for (uint32_t it = 0; it < head; ++it) copy_w(s_begin + it, it);
            pdl_wait();
            for (uint32_t it = 0; it < head; ++it) copy_x(s_begin + it, it);
            for (uint32_t s = s_begin + head; s < s_end; ++s) {
                const uint32_t it = s - s_begin, slot = it % n_stages_ring;
                if (!mbar_wait(&empty_bar[slot], ((it / n_stages_ring) & 1) ^ 1) || *(volatile int*)&abort_flag) {
                    atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT);
                    abort_flag = 1;
                    break;
                }
                copy_w(s, slot);
                copy_x(s, slot);
            }
        }
        return;
    }
    pdl_wait();  // consumers touch y, the partial sums and the tile counters

    // ---- consumers: warp w owns rows [16w, 16w+16) of every tile --------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16 + tile_row<KIND>(g), r1 = warp * 16 + tile_row<KIND>(g + 8);
    float tot[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) tot[j][0] = tot[j][1] = tot[j][2] = tot[j][3] = 0.f;

    uint32_t seg_first_chunk = s_begin % p.chunks;
    for (uint32_t s = s_begin; s < s_end; ++s) {
        const uint32_t it = s - s_begin, slot = it % n_stages_ring;
        const uint32_t tile = s / p.chunks, chunk = s - tile * p.chunks;
        if (!mbar_wait(&full_bar[slot], (it / n_stages_ring) & 1)) {
            if (lane == 0) { atomicOr(p.status, BHD_DEV_WAIT_TIMEOUT); abort_flag = 1; }
            return;
        }
        const uint8_t* st = smem + slot * S::STAGE;
        const uint32_t q6_off = (KIND == BHD_TYPE_Q6_K) ? ((210u * chunk) & 15u) : 0u;
        consume_stage<KIND, NT>(st + r0 * Fmt<KIND>::BOX, st + r1 * Fmt<KIND>::BOX, st + S::X_OFF, lane, q6_off, tot);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[slot]);

        const bool tile_done = (chunk + 1 == p.chunks) || (s + 1 == s_end);
        if (!tile_done) continue;

        // ---- finish this (tile, segment) -----------------------------------------------------
        const bool whole = (seg_first_chunk == 0) && (chunk + 1 == p.chunks);
        const uint32_t row_a = tile * TILE_ROWS + r0, row_b = tile * TILE_ROWS + r1;
        bool write_out = whole;
        if (!whole) {
            // Partial sums of this segment go to scratch; the last segment to arrive adds all
            // segments of the tile in column order.
            const uint32_t first_cta = (tile * p.chunks) / p.per_cta;
            const uint32_t last_cta = (tile * p.chunks + p.chunks - 1) / p.per_cta;
            const uint32_t nseg = last_cta - first_cta + 1;
            float* mine = p.partial + (uint64_t(tile + cta_index) * CONSUMER_WARPS + warp) * (NT * 4 * 32);
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) __stcg(mine + (j * 4 + i) * 32 + lane, tot[j][i]);
            __threadfence();
            __syncwarp();
            uint32_t old = 0;
            if (lane == 0) old = atomicAdd(&p.counters[tile * CONSUMER_WARPS + warp], 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == nseg - 1) {
                __threadfence();
#pragma unroll
                for (int j = 0; j < NT; ++j) tot[j][0] = tot[j][1] = tot[j][2] = tot[j][3] = 0.f;
                for (uint32_t c = first_cta; c <= last_cta; ++c) {
                    const float* seg = p.partial + (uint64_t(tile + c) * CONSUMER_WARPS + warp) * (NT * 4 * 32);
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) tot[j][i] += __ldcg(seg + (j * 4 + i) * 32 + lane);
                }
                if (lane == 0) p.counters[tile * CONSUMER_WARPS + warp] = 0;  // ready for the next launch
                write_out = true;
            }
        }
        if (write_out) {
            auto store = [&](uint32_t b, float va, float vb) {
                if (b >= p.batch) return;
                const float sc = p.vec_scale ? p.vec_scale[b] : p.scale;
                va = __fmul_rn(va, sc);
                vb = __fmul_rn(vb, sc);
                if (row_a < p.rows) {
                    float* o = p.y + uint64_t(b) * p.rows + row_a;
                    *o = p.accumulate ? __fadd_rn(*o, va) : va;
                }
                if (row_b < p.rows) {
                    float* o = p.y + uint64_t(b) * p.rows + row_b;
                    *o = p.accumulate ? __fadd_rn(*o, vb) : vb;
                }
            };
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (SPLIT) {  // columns 2t (hi) and 2t+1 (lo) of vector 4j + t
                    store(4 * j + t, tot[j][0] + tot[j][1], tot[j][2] + tot[j][3]);
                } else {      // columns 2t and 2t+1 are vectors 8j + 2t and 8j + 2t + 1
                    store(8 * j + 2 * t, tot[j][0], tot[j][2]);
                    store(8 * j + 2 * t + 1, tot[j][1], tot[j][3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) tot[j][0] = tot[j][1] = tot[j][2] = tot[j][3] = 0.f;
        seg_first_chunk = 0;
    }
}

template <uint32_t KIND, int NT>
__global__ void __launch_bounds__(THREADS) k_matvec_mma(const __grid_constant__ CUtensorMap tmap, const MatvecParams p,
                                                        int n_stages_ring) {
    run_stage_range<KIND, NT, true>(&tmap, p, blockIdx.x, n_stages_ring);
}

// ---- grouped experts (qwen3moe routed block) ---------------------------------------------------
// Routes are sorted by expert (moe_plan.cu); every expert's routes are cut into groups and each
// (group, row tile) of an expert matrix is one CTA of a grouped kernel streaming all columns: the
// integer kernel (moe_grouped_i8.cu) for groups of few routes, the tensor-core kernel
// (gemm_q8_tcgen05.cu) for groups of many. The size class of a group picks the kernel instance.

// y[t] (+)= ((0 + d[slot(t,0)]) + d[slot(t,1)]) + ...: the reference's accumulation order
// (crates/beholdd-model/src/qwen3moe/forward.rs:1385-1398); routes of other ranks are skipped.
__global__ void k_moe_combine_slots(const float* __restrict__ d, const int32_t* __restrict__ route_slot,
                                    float* __restrict__ y, uint64_t n, uint32_t dim, uint32_t top_k, int accumulate) {
    bhd_wait_for_prior_kernels();
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const uint64_t t = i / dim, h = i - t * dim;
    float out = 0.0f;
    for (uint32_t j = 0; j < top_k; ++j) {
        const int32_t slot = route_slot[t * top_k + j];
        if (slot >= 0) out = __fadd_rn(out, d[uint64_t(slot) * dim + h]);
    }
    y[i] = accumulate ? __fadd_rn(y[i], out) : out;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int box_bytes_of(uint32_t kind) {
    switch (kind) {
        case BHD_TYPE_Q8_0: return Fmt<BHD_TYPE_Q8_0>::BOX;
        case BHD_TYPE_Q4_K: return Fmt<BHD_TYPE_Q4_K>::BOX;
        case BHD_TYPE_Q6_K: return Fmt<BHD_TYPE_Q6_K>::BOX;
        default: return 0;
    }
}

template <uint32_t KIND, int NT>
int32_t launch_one(bhd_ctx* ctx, const bhd_weight* w, const MatvecParams& base, cudaStream_t s) {
    using S = Smem<KIND, NT>;
    auto kern = k_matvec_mma<KIND, NT>;
    static int ring = 0, per_sm = 0;  // per instantiation; every GPU this library accepts is the same part
    static bhd_once_per_device once;
    if (once.pending(ctx)) {
        int r = 4;
        size_t dyn = size_t(r) * S::STAGE + 128;
        if (dyn > 200 * 1024) { r = 3; dyn = size_t(r) * S::STAGE + 128; }
        BHD_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn)), "raising the shared memory limit");
        int occ = 0;
        BHD_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, THREADS, dyn), "querying occupancy");
        if (occ < 1) return bhd_fail(ctx, BHD_ERR_BACKEND, "%s backend error: matvec kernel does not fit on an SM", bhd_device_name());
        per_sm = occ > 4 ? 4 : occ;
        ring = r;
        once.mark(ctx);
    }
    MatvecParams p = base;
    const uint32_t slots = uint32_t(ctx->sm_count) * per_sm;
    const uint32_t grid = p.total_stages < slots ? p.total_stages : slots;
    p.per_cta = (p.total_stages + grid - 1) / grid;
    const uint32_t ctas = (p.total_stages + p.per_cta - 1) / p.per_cta;
    CUtensorMap map;
    memcpy(&map, w->tmap, sizeof(map));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = size_t(ring) * S::STAGE + 128;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, map, p, ring), "launching the tensor-core matvec kernel");
    ctx->launches += 1;
    return BHD_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

void bhd_weight_build_tensor_map(bhd_ctx* ctx, bhd_weight* w) {
    w->tmap_ok = false;
    const int box = box_bytes_of(w->kind);
    if (!box || !ctx->tmap_encode || w->rows == 0 || w->cols == 0) return;
    if (w->row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(w->dev) & 15) != 0) return;
    const uint64_t total_rows = w->rows * w->slabs;
    if (total_rows > 0x7fffffffull || w->row_bytes / 2 > 0x7fffffffull) return;
    CUtensorMap map;
    const cuuint64_t dims[2] = {w->row_bytes / 2, total_rows};      // inner dimension in 2-byte elements
    const cuuint64_t strides[1] = {w->row_bytes};
    const cuuint32_t boxdim[2] = {cuuint32_t(box / 2), cuuint32_t(TILE_ROWS)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode)(
        &map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w->dev, dims, strides, boxdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return;
    memcpy(w->tmap, &map, sizeof(map));
    w->tmap_ok = true;
    w->tmap_box_rows = TILE_ROWS;
    w->tmap_box_bytes = uint32_t(box);
}

// Fast path of bhd_matvec / bhd_matmul. Sets *handled = false (and launches nothing) when the
// weight or the buffers do not meet the path's alignment rules; the caller then uses the
// general kernels.
int32_t bhd_launch_matvec_fast(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                               uint64_t batch, float scale, int accumulate, cudaStream_t s, bool* handled) {
    *handled = false;
    if (!w->tmap_ok || w->cols == 0 || w->cols % 4 != 0) return BHD_OK;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || w->rows > 0x7fffffffull || batch > 0x7fffffffull) return BHD_OK;
    const uint32_t chunks = uint32_t((w->cols + CHUNK_K - 1) / CHUNK_K);
    const uint32_t tiles = uint32_t((w->rows + TILE_ROWS - 1) / TILE_ROWS);
    if (uint64_t(tiles) * CONSUMER_WARPS > 65536 || uint64_t(tiles) * chunks > 0x7fffffffull) return BHD_OK;

    // Activation vectors are processed up to 32 at a time (NT <= 8 n-tiles of four).
    uint64_t b0 = 0;
    while (b0 < batch) {
        const uint32_t nb = uint32_t(batch - b0 < 32 ? batch - b0 : 32);
        const int nt = nb <= 4 ? 1 : (nb <= 8 ? 2 : (nb <= 16 ? 4 : 8));
        const size_t blob_bytes = align_up(size_t(chunks) * xblob_bytes(w->kind, nt), 256);
        const uint32_t max_ctas = uint32_t(ctx->sm_count) * 4;
        const size_t partial_bytes = size_t(tiles + max_ctas + 1) * CONSUMER_WARPS * nt * 4 * 32 * sizeof(float);
        // workspace: [activation blob] [partial sums]
        int32_t st = bhd_ensure_workspace(ctx, blob_bytes + partial_bytes, s);
        if (st != BHD_OK) return st;
        uint8_t* blob = ctx->workspace;

        {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(chunks, nt);
            cfg.blockDim = dim3(STEPS * 32);
            cfg.stream = s;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            BHD_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_pack_x, w->kind, x + b0 * w->cols, uint64_t(w->cols), uint32_t(nb), uint32_t(w->cols),
                                             int(nt), blob, ctx->status_dev),
                     "launching the activation packing kernel");
            ctx->launches += 1;
        }

        MatvecParams p;
        p.xblob = blob;
        p.y = y + b0 * w->rows;
        p.partial = reinterpret_cast<float*>(blob + blob_bytes);
        p.counters = ctx->counters;
        p.status = ctx->status_dev;
        p.rows = uint32_t(w->rows);
        p.row_base = uint32_t(slab * w->rows);
        p.batch = nb;
        p.chunks = chunks;
        p.total_stages = tiles * chunks;
        p.per_cta = 0;
        p.scale = scale;
        p.accumulate = accumulate;
        p.vec_scale = nullptr;
#define BHD_CASE(K)                                                 \
    case K:                                                         \
        switch (nt) {                                               \
            case 1: st = launch_one<K, 1>(ctx, w, p, s); break;     \
            case 2: st = launch_one<K, 2>(ctx, w, p, s); break;     \
            case 4: st = launch_one<K, 4>(ctx, w, p, s); break;     \
            default: st = launch_one<K, 8>(ctx, w, p, s); break;    \
        }                                                           \
        break;
        switch (w->kind) {
            BHD_CASE(BHD_TYPE_Q8_0)
            BHD_CASE(BHD_TYPE_Q4_K)
            BHD_CASE(BHD_TYPE_Q6_K)
            default: return BHD_OK;
        }
#undef BHD_CASE
        if (st != BHD_OK) return st;
        b0 += nb;
    }
    *handled = true;
    return BHD_OK;
}

namespace {

// One launch per size class that can occur (a class only exists when there are enough routes and enough
// positions for its smallest group: an expert has at most one route per position): the integer kernel below `tc_min`, the tensor-core kernel from there on.
int32_t launch_grouped_all(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const MoePlanBuffers& pb, uint32_t n_routes,
                           uint32_t n_positions, uint32_t n_local, uint32_t cap, uint32_t tc_min, const void* xq, const void* x16, const void* x16_lo, float* out0,
                           float* out1, float* const* slot_dst, const float* i8_scale, const float* tc_scale, cudaStream_t s) {
    const uint32_t small = n_local < n_routes ? n_local : n_routes;
    uint32_t n_cls = 0;
    for (uint32_t cls = 0; cls < uint32_t(BHD_MOE_CLASSES); ++cls) {
        const uint32_t least = bhd_moe_cls_least(int(cls));
        if (n_routes < least || least > cap || least > n_positions) break;  // an expert has at most one route per position
        ++n_cls;
    }
    // The classes work on disjoint groups, so their kernels need not wait for one another: with the integer kernels
    // (at most four classes) every class after the first runs on a side stream forked from the caller's stream and joined
    // to it again, which also holds inside a stream capture (the side streams join the capture and leave it at the join).
    // A class that turns out to be empty then costs the chain nothing.
    const bool side_by_side = n_cls > 1 && n_cls <= 4 && tc_min >= n_cls;
    if (side_by_side) BHD_CUDA(ctx, cudaEventRecord(ctx->fork_event, s), "forking the size classes");
    for (uint32_t cls = 0; cls < n_cls; ++cls) {
        const uint32_t least = bhd_moe_cls_least(int(cls));
        // An expert cut into several groups only yields groups of more than cap / 2 routes, so the classes below hold
        // at most one group per expert; every class holds at most routes / (its smallest group) groups.
        const uint32_t by_size = n_routes / least;
        const uint32_t bound = (2 * (4u << cls) >= cap) ? by_size : (small < by_size ? small : by_size);
        cudaStream_t cs = s;
        if (side_by_side && cls > 0) {
            cs = ctx->side_stream[cls - 1];
            BHD_CUDA(ctx, cudaStreamWaitEvent(cs, ctx->fork_event, 0), "forking the size classes");
        }
        int32_t st;
        if (cls < tc_min)
            st = bhd_launch_moe_grouped_i8(ctx, w0, w1, pb.hdr, pb.groups, pb.glist + uint64_t(cls) * pb.gmax, cls, bound, xq, n_routes, out0,
                                           out1, slot_dst, i8_scale, cs);
        else if (ctx->moe_tc_plain && !slot_dst)
            st = bhd_launch_gemm_q8_grouped(ctx, w0, w1, pb.hdr, pb.groups, pb.glist + uint64_t(cls) * pb.gmax, cls, bound, x16, n_routes,
                                            out0, out1, tc_scale, cs);
        else
            st = bhd_launch_gemm_q8_ts_grouped(ctx, w0, w1, pb.hdr, pb.groups, pb.glist + uint64_t(cls) * pb.gmax, cls, bound, x16, x16_lo,
                                               n_routes, out0, out1, slot_dst, tc_scale, cs);
        if (side_by_side && cls > 0) {  // joined even after a failed launch, so that a capture in progress stays well-formed
            cudaEventRecord(ctx->join_event[cls - 1], cs);
            cudaStreamWaitEvent(s, ctx->join_event[cls - 1], 0);
        }
        if (st != BHD_OK) return st;
    }
    return BHD_OK;
}

}  // namespace

// Fast path of bhd_moe_experts: plan (sort routes by expert, cut into groups), token gather +
// packing of the activations (block-floating bytes for the integer kernel, row-scaled fp16 for the
// tensor-core kernel), grouped gate/up, SiLU gating fused into the packing of the down input,
// grouped down scaled by the route weight, combine in route order. Sets *handled = false when the
// tensors do not meet the rules of the TMA path (Q8_0, 16-byte aligned rows).
int32_t bhd_moe_experts_fast(bhd_ctx* ctx, const bhd_weight* gate, const bhd_weight* up, const bhd_weight* down,
                             const float* x, uint64_t T, uint32_t top_k, const int32_t* experts, const float* weights,
                             uint32_t first_expert, uint32_t n_local, uint32_t n_total, float* y, int accumulate,
                             cudaStream_t s, bool* handled, const MoePeerOut* peer) {
    *handled = false;
    if (!bhd_moe_i8_usable(gate) || !bhd_moe_i8_usable(up) || !bhd_moe_i8_usable(down)) return BHD_OK;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return BHD_OK;
    const uint64_t ff = gate->rows, dim = gate->cols;
    if (dim % 8 != 0 || ff % 8 != 0) return BHD_OK;
    const uint64_t R64 = T * top_k;
    // 2^20 routes keep every grid dimension of the grouped kernels (at most routes / 5 groups of a
    // class on grid.y would not fit, but a class of groups that small holds at most one group per
    // expert) within 65535; more routes take the general kernels.
    if (R64 > (1u << 20) || n_local > 1024) return BHD_OK;
    const uint32_t R = uint32_t(R64), E = n_local;
    // Groups of many routes can go to the tensor-core kernel (BHD_OPTION_MOE_TC_MIN_CLASS). It is not the default:
    // measured on B200, its per-slice pipeline latency makes it slower than the integer kernel at every group size
    // met so far (17 to 160 routes per expert).
    const uint32_t opt = ctx->moe_tc_min_cls;
    const bool tc_ok = opt != 0 && opt < uint32_t(BHD_MOE_CLASSES) && bhd_gemm_q8_grouped_usable(ctx, gate) &&
                       bhd_gemm_q8_grouped_usable(ctx, up) && bhd_gemm_q8_grouped_usable(ctx, down);
    uint32_t tc_min = opt;
    if (tc_min < 2) tc_min = 2;
    if (tc_min > 4) tc_min = 4;
    const uint32_t cap = tc_ok ? ((ctx->moe_tc_plain && !peer) ? 256u : 128u) : 32u;  // the exact form holds hi and lo rows: 128 routes per tile
    if (!tc_ok) tc_min = uint32_t(BHD_MOE_CLASSES);
    const uint32_t gmax = E + R / 32 + 1;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_hdr = take(sizeof(MoeHeader)), o_counts = take(4 * size_t(E)), o_offsets = take(4 * size_t(E + 1));
    const size_t o_rslot = take(4 * size_t(R)), o_sroute = take(4 * size_t(R)), o_sweight = take(4 * size_t(R)), o_scls = take(size_t(R));
    const size_t o_groups = take(sizeof(MoeGroup) * size_t(gmax)), o_glist = take(4 * size_t(BHD_MOE_CLASSES) * size_t(gmax));
    const size_t o_whist = take(4 * bhd_moe_plan_scratch_words(R, E));
    const size_t o_g = take(4 * size_t(R) * ff), o_u = take(4 * size_t(R) * ff), o_d = take(4 * size_t(R) * dim);
    const size_t o_xq = take(bhd_moe_slots_i8_bytes(uint32_t(dim), R)), o_aq = take(bhd_moe_slots_i8_bytes(uint32_t(ff), R));
    const size_t o_x16 = take(tc_ok ? 2 * size_t(R) * dim : 0), o_a16 = take(tc_ok ? 2 * size_t(R) * ff : 0);
    const size_t o_x16l = take(tc_ok ? 2 * size_t(R) * dim : 0), o_a16l = take(tc_ok ? 2 * size_t(R) * ff : 0);
    const size_t o_xs = take(4 * size_t(R)), o_as = take(4 * size_t(R)), o_sdst = take(peer ? sizeof(float*) * size_t(R) : 0);
    int32_t st = bhd_ensure_workspace(ctx, off, s);
    if (st != BHD_OK) return st;
    uint8_t* ws = ctx->workspace;
    MoePlanBuffers pb;
    pb.hdr = reinterpret_cast<MoeHeader*>(ws + o_hdr);
    pb.counts = reinterpret_cast<uint32_t*>(ws + o_counts);
    pb.offsets = reinterpret_cast<uint32_t*>(ws + o_offsets);
    pb.route_slot = reinterpret_cast<int32_t*>(ws + o_rslot);
    pb.slot_route = reinterpret_cast<int32_t*>(ws + o_sroute);
    pb.slot_weight = reinterpret_cast<float*>(ws + o_sweight);
    pb.slot_cls = ws + o_scls;
    pb.groups = reinterpret_cast<MoeGroup*>(ws + o_groups);
    pb.glist = reinterpret_cast<int32_t*>(ws + o_glist);
    pb.whist = reinterpret_cast<uint32_t*>(ws + o_whist);
    pb.gmax = gmax;
    pb.slot_dst = peer ? reinterpret_cast<float**>(ws + o_sdst) : nullptr;
    pb.peer_rows = peer ? peer->peer_rows : nullptr;
    pb.t_per_rank = peer ? peer->t_per_rank : 0u;
    pb.dim = uint32_t(dim);
    pb.top_k = top_k;
    float* gbuf = reinterpret_cast<float*>(ws + o_g);
    float* ubuf = reinterpret_cast<float*>(ws + o_u);
    float* dbuf = reinterpret_cast<float*>(ws + o_d);
    float* xscale = reinterpret_cast<float*>(ws + o_xs);
    float* ascale = reinterpret_cast<float*>(ws + o_as);
    const bool tc_possible = tc_ok && R >= bhd_moe_cls_least(int(tc_min));

    if ((st = bhd_launch_moe_plan(ctx, experts, weights, R, first_expert, E, n_total, cap, uint32_t(T), pb, s)) != BHD_OK) return st;
    // gate and up: [ff x dim] per expert, both matrices in one launch per size class
    if ((st = bhd_launch_moe_slots_i8(ctx, 0, pb.hdr, pb.slot_route, pb.slot_cls, tc_min - 1, top_k, x, nullptr, uint32_t(dim), R, ws + o_xq, s)) != BHD_OK) return st;
    if (tc_possible && (st = bhd_launch_moe_rows_f16(ctx, 0, pb.hdr, pb.slot_route, pb.slot_cls, tc_min, top_k, x, nullptr, uint32_t(dim), R,
                                                      ws + o_x16, ws + o_x16l, nullptr, xscale, s)) != BHD_OK) return st;
    if ((st = launch_grouped_all(ctx, gate, up, pb, R, uint32_t(T), E, cap, tc_min, ws + o_xq, ws + o_x16, ws + o_x16l, gbuf, ubuf, nullptr, nullptr, xscale, s)) != BHD_OK) return st;
    // down: [dim x ff] per expert, each output row scaled by its route weight
    if ((st = bhd_launch_moe_slots_i8(ctx, 1, pb.hdr, pb.slot_route, pb.slot_cls, tc_min - 1, top_k, gbuf, ubuf, uint32_t(ff), R, ws + o_aq, s)) != BHD_OK) return st;
    if (tc_possible && (st = bhd_launch_moe_rows_f16(ctx, 1, pb.hdr, pb.slot_route, pb.slot_cls, tc_min, top_k, gbuf, ubuf, uint32_t(ff), R,
                                                      ws + o_a16, ws + o_a16l, pb.slot_weight, ascale, s)) != BHD_OK) return st;
    if ((st = launch_grouped_all(ctx, down, nullptr, pb, R, uint32_t(T), E, cap, tc_min, ws + o_aq, ws + o_a16, ws + o_a16l, dbuf, nullptr, pb.slot_dst, pb.slot_weight, ascale, s)) != BHD_OK) return st;
    if (peer) {  // the rows went to their owners; the caller signals them and combines what it received
        *handled = true;
        return BHD_OK;
    }
    const uint64_t n = T * dim;
    bhd_launch_dependent(ctx, k_moe_combine_slots, dim3(unsigned((n + 255) / 256)), dim3(256), 0, s, dbuf, pb.route_slot, y, n, uint32_t(dim), top_k, accumulate);
    BHD_LAUNCHED(ctx, "route combine kernel");
    *handled = true;
    return BHD_OK;
}
