// Activations of the routed experts as row-scaled fp16, in slot order, for the tensor-core grouped
// kernel (groups of many routes per expert, gemm_q8_tcgen05.cu).
//
//   mode 0: row of a slot = x[position of the slot's route]           (the token-to-expert gather)
//   mode 1: row of a slot = silu(g[slot]) * u[slot]                    (crates/beholdd-kernel/src/vecops.rs:91-111, limit 0)
//
// With `out_lo` the fp16 remainder of every element is written to a second array (the exact form of
// the tensor-core kernel carries activations as hi + lo pairs).
// Every row is scaled by a power of two so that its largest magnitude lands in [2^14, 2^15) before
// the conversion: fp16 then keeps 11 significant bits of every element down to 2^-28 of the row's
// maximum, whatever the row's magnitude (a hidden state with one 1e4 spike, a gated activation of
// 1e7), and nothing overflows. The power of two goes out with the row (`scale_out`, multiplied by
// the route weight in mode 1) and the matmul's epilogue multiplies it back in.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_mul(float g, float u) { return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u); }

__global__ void __launch_bounds__(128) k_moe_rows_f16(int mode, const MoeHeader* __restrict__ hdr, const int32_t* __restrict__ slot_route,
                                                      const uint8_t* __restrict__ slot_cls, uint32_t min_cls, uint32_t top_k,
                                                      const float* __restrict__ src, const float* __restrict__ src2, uint32_t K,
                                                      uint32_t n_slots, __half* __restrict__ out, __half* __restrict__ out_lo,
                                                      const float* __restrict__ slot_weight,
                                                      float* __restrict__ scale_out, uint32_t* __restrict__ status) {
    const uint32_t slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (slot >= hdr->local_routes || slot >= n_slots) return;  // whole warps
    if (slot_cls[slot] < min_cls) return;                       // a group the integer kernels take
    const uint64_t row = mode == 0 ? uint64_t(uint32_t(slot_route[slot]) / top_k) : uint64_t(slot);
    const float4* a = reinterpret_cast<const float4*>(src + row * K);
    const float4* b = mode == 1 ? reinterpret_cast<const float4*>(src2 + row * K) : nullptr;
    const uint32_t n4 = K / 4;
    auto value = [&](uint32_t i) -> float4 {
        float4 v = a[i];
        if (mode == 1) {
            const float4 u = b[i];
            v.x = silu_mul(v.x, u.x); v.y = silu_mul(v.y, u.y); v.z = silu_mul(v.z, u.z); v.w = silu_mul(v.w, u.w);
        }
        return v;
    };
    float mx = 0.f;
    bool bad = false;
    for (uint32_t i = lane; i < n4; i += 32) {
        const float4 v = value(i);
        const float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        if (!(m <= 3.0e38f)) bad = true;  // NaN or infinity
        else mx = fmaxf(mx, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (bad) atomicOr(status, BHD_DEV_ACTIVATION_RANGE);
    // mx = m * 2^(eb - 127), m in [1, 2). Rows whose largest magnitude is below 2^-100 convert to zeros.
    const int eb = int(__float_as_uint(mx) >> 23);
    const bool tiny = eb < 27;
    const float down = tiny ? 0.f : __uint_as_float(uint32_t(268 - eb) << 23);  // 2^(14 - (eb - 127))
    const float up = tiny ? 0.f : __uint_as_float(uint32_t(eb - 14) << 23);     // its inverse
    uint2* o = reinterpret_cast<uint2*>(out + uint64_t(slot) * K);
    uint2* ol = out_lo ? reinterpret_cast<uint2*>(out_lo + uint64_t(slot) * K) : nullptr;
    for (uint32_t i = lane; i < n4; i += 32) {
        float4 v = value(i);
        if (!(fabsf(v.x) <= 3.0e38f)) v.x = 0.f;
        if (!(fabsf(v.y) <= 3.0e38f)) v.y = 0.f;
        if (!(fabsf(v.z) <= 3.0e38f)) v.z = 0.f;
        if (!(fabsf(v.w) <= 3.0e38f)) v.w = 0.f;
        const float sx = v.x * down, sy = v.y * down, sz = v.z * down, sw = v.w * down;  // exact: a power of two
        const __half2 h0 = __floats2half2_rn(sx, sy), h1 = __floats2half2_rn(sz, sw);
        o[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        if (ol) {  // the fp16 remainders: hi + lo holds 22 significant bits of the value
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(sx - f0.x, sy - f0.y), l1 = __floats2half2_rn(sz - f1.x, sw - f1.y);
            ol[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&l0), *reinterpret_cast<const uint32_t*>(&l1));
        }
    }
    if (lane == 0) scale_out[slot] = slot_weight ? __fmul_rn(up, slot_weight[slot]) : up;
}

}  // namespace

int32_t bhd_launch_moe_rows_f16(bhd_ctx* ctx, int mode, const void* hdr, const int32_t* slot_route, const uint8_t* slot_cls,
                                uint32_t min_cls, uint32_t top_k, const float* src, const float* src2, uint32_t K, uint32_t n_slots,
                                void* out16, void* out16_lo, const float* slot_weight, float* scale_out, cudaStream_t s) {
    if (n_slots == 0) return BHD_OK;
    k_moe_rows_f16<<<(n_slots + 3) / 4, 128, 0, s>>>(mode, static_cast<const MoeHeader*>(hdr), slot_route, slot_cls, min_cls, top_k, src, src2,
                                                       K, n_slots, static_cast<__half*>(out16), static_cast<__half*>(out16_lo), slot_weight, scale_out,
                                                       ctx->status_dev);
    BHD_LAUNCHED(ctx, mode ? "expert gating kernel (fp16 rows)" : "token gather kernel (fp16 rows)");
    return BHD_OK;
}
