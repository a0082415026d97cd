// Seeded synthetic tensors generated on the device, for workloads whose weights are too large to
// generate on the host in reasonable time (a 48-layer mixture-of-experts model is 32 GB of packed
// blocks). The Q8_0 generator reproduces the host generator byte for byte (one counter-based
// splitmix64 stream per field: an f16 scale uniform in [1e-3, 1e-2] and 32 int8 quants uniform in
// [-127, 127] per block), so a test can compare the two; the normal generator has the same
// distribution as the host's (Box-Muller on two uniform streams) but uses the device's math
// functions, so its bits are its own.
#include "common.cuh"

namespace {

constexpr uint64_t GAMMA = 0x9E3779B97F4A7C15ull;

__host__ __device__ inline uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return seed * 0x2545F4914F6CDD1Dull + stream * 0xD6E8FEB86659FD93ull;
}
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ double uniform01(uint64_t key, uint64_t index) {  // 53 random bits in [0, 1)
    return double(mix64(key + (index + 1) * GAMMA) >> 11) * (1.0 / 9007199254740992.0);
}

// binary16 bits of a positive double in the normal binary16 range, rounded to nearest even, in integer arithmetic
// (the same rounding as the host generator's float64 -> float16 cast).
__device__ __forceinline__ uint16_t f16_bits_of(double d) {
    const uint64_t b = uint64_t(__double_as_longlong(d));
    int e = int((b >> 52) & 0x7ff) - 1023 + 15;
    const uint64_t m = b & ((1ull << 52) - 1);
    uint64_t keep = m >> 42;
    const uint64_t rest = m & ((1ull << 42) - 1), half = 1ull << 41;
    if (rest > half || (rest == half && (keep & 1))) ++keep;
    if (keep == 1024) { keep = 0; ++e; }
    return uint16_t((uint32_t(e) << 10) | uint32_t(keep));
}

// Slab s uses field streams (stream0 + s * stream_step) * 16 + 1 (scales) and * 16 + 2 (quants); block indices restart per slab.
__global__ void k_fill_q8_0(uint8_t* __restrict__ out, uint64_t blocks_per_slab, uint64_t n_slabs, uint64_t seed, uint64_t stream0,
                            uint64_t stream_step) {
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= blocks_per_slab * n_slabs) return;
    const uint64_t slab = i / blocks_per_slab, b = i - slab * blocks_per_slab;
    const uint64_t stream = stream0 + slab * stream_step;
    const uint64_t key_d = stream_key(seed, stream * 16 + 1), key_q = stream_key(seed, stream * 16 + 2);
    uint8_t* blk = out + i * 34;
    const double d = 1e-3 + (1e-2 - 1e-3) * uniform01(key_d, b);
    const uint16_t dbits = f16_bits_of(d);
    blk[0] = uint8_t(dbits & 0xff);
    blk[1] = uint8_t(dbits >> 8);
    for (int j = 0; j < 32; ++j) {
        const uint64_t z = mix64(key_q + (b * 32 + j + 1) * GAMMA);
        blk[2 + j] = uint8_t(int8_t(int(z % 255ull) - 127));
    }
}

__global__ void k_fill_normal(float* __restrict__ out, uint64_t n, uint64_t seed, uint64_t stream, float std) {
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const double u1 = 1.0 - uniform01(stream_key(seed, stream * 2 + 1000003), i);  // (0, 1]
    const double u2 = uniform01(stream_key(seed, stream * 2 + 1000004), i);
    out[i] = float(sqrt(-2.0 * log(u1)) * cospi(2.0 * u2) * double(std));
}

}  // namespace

extern "C" int32_t bhd_debug_fill_q8_0(bhd_ctx* ctx, uint8_t* out_dev, uint64_t blocks_per_slab, uint64_t n_slabs, uint64_t seed,
                                       uint64_t stream0, uint64_t stream_step, void* cuda_stream) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    const uint64_t n = blocks_per_slab * n_slabs;
    if (n == 0) return BHD_OK;
    if (!out_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "fill_q8_0: null buffer");
    if ((n + 255) / 256 > 0x7fffffffull) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: too many blocks to fill");
    bhd_device_guard guard(ctx);
    k_fill_q8_0<<<unsigned((n + 255) / 256), 256, 0, cudaStream_t(cuda_stream)>>>(out_dev, blocks_per_slab, n_slabs, seed, stream0, stream_step);
    BHD_LAUNCHED(ctx, "Q8_0 fill kernel");
    return BHD_OK;
}

extern "C" int32_t bhd_debug_fill_normal(bhd_ctx* ctx, float* out_dev, uint64_t n, uint64_t seed, uint64_t stream, float std, void* cuda_stream) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (n == 0) return BHD_OK;
    if (!out_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "fill_normal: null buffer");
    if ((n + 255) / 256 > 0x7fffffffull) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: too many values to fill");
    bhd_device_guard guard(ctx);
    k_fill_normal<<<unsigned((n + 255) / 256), 256, 0, cudaStream_t(cuda_stream)>>>(out_dev, n, seed, stream, std);
    BHD_LAUNCHED(ctx, "normal fill kernel");
    return BHD_OK;
}
