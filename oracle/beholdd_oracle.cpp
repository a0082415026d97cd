// TEST INFRASTRUCTURE ONLY -- CPU oracle for the quantised-matvec / qwen3moe routed-expert path.
//
// This file is a C++17 restatement of the reference's *CPU* arithmetic for that path. It is
// the checker the CUDA kernels are compared against and the "port" CPU baseline a benchmark
// may time. It is never linked into, loaded by, or called from the product library.
//
// Parity status: PINNED. The reference is Rust and cannot be compiled in this environment
// (no cargo/rustc), so the oracle is pinned two ways instead:
//   * every known-answer test the reference's own unit tests hold for this path is replayed
//     against this file (tests/test_oracle_kat.py), and
//   * the reference's independent f64 NumPy implementation (tools/qwen3moe_ref.py) was run
//     on a synthetic checkpoint and its outputs are committed as golden vectors
//     (tests/golden/), which this file must reproduce.
// Bit-level results of expf-based steps (softmax, SiLU) depend on the host libm, exactly as
// they do for the reference (Rust f32::exp lowers to the platform libm).
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fPIC -shared (Rust never contracts a*b+c into
// an FMA; gcc would on FMA targets unless told not to).
//
// Each function cites the reference file:line it follows (paths relative to the reference
// repository root).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <limits>
#include <thread>
#include <vector>

namespace {

// ---- status codes shared with the tests ------------------------------------------------
constexpr int32_t ORC_OK = 0;
constexpr int32_t ORC_UNSUPPORTED = -1;  // DeviceError::UnsupportedFormat
constexpr int32_t ORC_SHAPE = -2;        // DeviceError::Shape
constexpr int32_t ORC_INVALID = -3;      // anyhow bail! in the model layer

// crates/beholdd-core/src/quant.rs:259-278 -- IEEE binary16 to f32 including subnormals.
inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t(h) & 0x8000u) << 16;
    const uint32_t exp = (uint32_t(h) >> 10) & 0x1Fu;
    const uint32_t man = uint32_t(h) & 0x3FFu;
    uint32_t bits;
    if (exp == 0 && man == 0) {
        bits = sign;
    } else if (exp == 0) {
        // value = man * 2^-24; renormalise around the leading one at bit p.
        const uint32_t p = 31u - uint32_t(__builtin_clz(man));
        bits = sign | ((p + 103u) << 23) | ((man - (1u << p)) << (23u - p));
    } else if (exp == 0x1Fu) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127u - 15u) << 23) | (man << 13);
    }
    float out;
    std::memcpy(&out, &bits, 4);
    return out;
}

// crates/beholdd-core/src/quant.rs:253-255
inline float bf16_to_f32(uint16_t h) {
    const uint32_t bits = uint32_t(h) << 16;
    float out;
    std::memcpy(&out, &bits, 4);
    return out;
}

inline uint16_t le16(const uint8_t* p) { return uint16_t(p[0]) | (uint16_t(p[1]) << 8); }

// crates/beholdd-kernel/src/kquant.rs:311-316 with crates/beholdd-core/src/quant.rs:79-118:
// the formats the CPU device can decode, as (elements, bytes) per block.
bool block_geometry(uint32_t kind, uint64_t* elems, uint64_t* bytes) {
    switch (kind) {
        case 0: *elems = 1; *bytes = 4; return true;       // F32
        case 1: *elems = 1; *bytes = 2; return true;       // F16
        case 8: *elems = 32; *bytes = 34; return true;     // Q8_0
        case 12: *elems = 256; *bytes = 144; return true;  // Q4_K
        case 13: *elems = 256; *bytes = 176; return true;  // Q5_K
        case 14: *elems = 256; *bytes = 210; return true;  // Q6_K
        case 30: *elems = 1; *bytes = 2; return true;      // BF16
        default: return false;
    }
}

// crates/beholdd-kernel/src/kquant.rs:39-54
void q8_0_dequant(const uint8_t* src, float* out, uint64_t n) {
    const uint64_t nb = n / 32;
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 34;
        const float d = f16_to_f32(le16(blk));
        for (int i = 0; i < 32; ++i) out[b * 32 + i] = d * float(int8_t(blk[2 + i]));
    }
}

// crates/beholdd-kernel/src/kquant.rs:61-79 -- one accumulator, left to right,
// (d*q) then (*x) then (+): three roundings per element, no FMA.
float q8_0_dot(const uint8_t* src, const float* x, uint64_t cols) {
    const uint64_t nb = cols / 32;
    float acc = 0.0f;
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 34;
        const float d = f16_to_f32(le16(blk));
        const float* xv = x + b * 32;
        for (int i = 0; i < 32; ++i) {
            const float decoded = d * float(int8_t(blk[2 + i]));
            acc += decoded * xv[i];
        }
    }
    return acc;
}

// crates/beholdd-kernel/src/kquant.rs:143-162
template <int LOW_SHIFT, int HIGH_SHIFT>
void q6_k_group(const uint8_t* low, const uint8_t* high, const uint8_t* scales, float d, float* out) {
    for (int sg = 0; sg < 2; ++sg) {
        const float scaled_d = d * float(int8_t(scales[sg]));
        for (int i = 0; i < 16; ++i) {
            const int l = sg * 16 + i;
            const uint8_t code = uint8_t(((low[l] >> LOW_SHIFT) & 0x0F) | (((high[l] >> HIGH_SHIFT) & 0x03) << 4));
            out[l] = scaled_d * float(int32_t(code) - 32);
        }
    }
}

// crates/beholdd-kernel/src/kquant.rs:115-139
void q6_k_dequant(const uint8_t* src, float* out, uint64_t n) {
    const uint64_t nb = n / 256;
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 210;
        float* values = out + b * 256;
        const float d = f16_to_f32(le16(blk + 208));
        for (int half = 0; half < 2; ++half) {
            const uint8_t* low = blk + half * 64;
            const uint8_t* high = blk + 128 + half * 32;
            const uint8_t* scales = blk + 192 + half * 8;
            float* o = values + half * 128;
            q6_k_group<0, 0>(low, high, scales, d, o);
            q6_k_group<0, 2>(low + 32, high, scales + 2, d, o + 32);
            q6_k_group<4, 4>(low, high, scales + 4, d, o + 64);
            q6_k_group<4, 6>(low + 32, high, scales + 6, d, o + 96);
        }
    }
}

// crates/beholdd-kernel/src/kquant.rs:176-185
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = uint8_t((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = uint8_t((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// crates/beholdd-kernel/src/kquant.rs:209-241
void q4_k_dequant(const uint8_t* src, float* out, uint64_t n) {
    const uint64_t nb = n / 256;
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 144;
        const float d = f16_to_f32(le16(blk));
        const float dmin = f16_to_f32(le16(blk + 2));
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        float* y = out + b * 256;
        for (int pass = 0; pass < 4; ++pass) {
            const uint8_t* q = qs + pass * 32;
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(pass * 2, scales, &sc1, &m1);
            scale_min_k4(pass * 2 + 1, scales, &sc2, &m2);
            const float d1 = d * float(sc1), off1 = dmin * float(m1);
            const float d2 = d * float(sc2), off2 = dmin * float(m2);
            const int base = pass * 64;
            for (int l = 0; l < 32; ++l) {
                y[base + l] = d1 * float(q[l] & 0xF) - off1;
                y[base + 32 + l] = d2 * float(q[l] >> 4) - off2;
            }
        }
    }
}

// crates/beholdd-kernel/src/kquant.rs:268-303
void q5_k_dequant(const uint8_t* src, float* out, uint64_t n) {
    const uint64_t nb = n / 256;
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 176;
        const float d = f16_to_f32(le16(blk));
        const float dmin = f16_to_f32(le16(blk + 2));
        const uint8_t* scales = blk + 4;
        const uint8_t* qh = blk + 16;
        const uint8_t* qs = blk + 48;
        float* y = out + b * 256;
        for (int pass = 0; pass < 4; ++pass) {
            const uint8_t* q = qs + pass * 32;
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(pass * 2, scales, &sc1, &m1);
            scale_min_k4(pass * 2 + 1, scales, &sc2, &m2);
            const float d1 = d * float(sc1), off1 = dmin * float(m1);
            const float d2 = d * float(sc2), off2 = dmin * float(m2);
            const uint8_t u1 = uint8_t(1u << (pass * 2)), u2 = uint8_t(2u << (pass * 2));
            const int base = pass * 64;
            for (int l = 0; l < 32; ++l) {
                const int hi1 = (qh[l] & u1) ? 16 : 0;
                const int hi2 = (qh[l] & u2) ? 16 : 0;
                y[base + l] = d1 * float(int(q[l] & 0xF) + hi1) - off1;
                y[base + 32 + l] = d2 * float(int(q[l] >> 4) + hi2) - off2;
            }
        }
    }
}

// crates/beholdd-backend/src/cpu.rs:55-97 -- exact storage validation; returns the element
// count or a negative status.
int32_t validate_storage(uint64_t n_bytes, uint32_t kind, uint64_t rows, uint64_t cols, uint64_t* n_out) {
    uint64_t n;
    if (__builtin_mul_overflow(rows, cols, &n)) return ORC_SHAPE;
    uint64_t be, bb;
    if (!block_geometry(kind, &be, &bb)) return ORC_UNSUPPORTED;
    if (cols % be != 0) return ORC_SHAPE;
    const uint64_t bpr = cols / be;
    uint64_t blocks, expect;
    if (__builtin_mul_overflow(rows, bpr, &blocks) || __builtin_mul_overflow(blocks, bb, &expect)) return ORC_SHAPE;
    if (n_bytes != expect) return ORC_SHAPE;
    *n_out = n;
    return ORC_OK;
}

// crates/beholdd-backend/src/cpu.rs:99-130
int32_t dequant_any(const uint8_t* bytes, uint64_t n_bytes, uint32_t kind, uint64_t rows, uint64_t cols,
                    float* out, uint64_t out_len) {
    uint64_t n;
    const int32_t st = validate_storage(n_bytes, kind, rows, cols, &n);
    if (st != ORC_OK) return st;
    if (out_len != n) return ORC_SHAPE;
    switch (kind) {
        case 0:
            for (uint64_t i = 0; i < n; ++i) std::memcpy(out + i, bytes + 4 * i, 4);
            break;
        case 1:
            for (uint64_t i = 0; i < n; ++i) out[i] = f16_to_f32(le16(bytes + 2 * i));
            break;
        case 30:
            for (uint64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(le16(bytes + 2 * i));
            break;
        case 8: q8_0_dequant(bytes, out, n); break;
        case 12: q4_k_dequant(bytes, out, n); break;
        case 13: q5_k_dequant(bytes, out, n); break;
        case 14: q6_k_dequant(bytes, out, n); break;
        default: return ORC_UNSUPPORTED;
    }
    return ORC_OK;
}

// crates/beholdd-kernel/src/vecops.rs:44-46 and crates/beholdd-backend/src/cpu.rs:164,178-190
uint64_t worker_count(uint64_t rows, uint64_t cols, uint64_t available) {
    uint64_t total;
    if (__builtin_mul_overflow(rows, cols, &total)) total = std::numeric_limits<uint64_t>::max();
    if (!(rows > 1 && total >= (1ull << 16))) return 1;
    return std::min<uint64_t>(std::min<uint64_t>(std::max<uint64_t>(available, 1), std::max<uint64_t>(rows, 1)), 8);
}

// crates/beholdd-backend/src/cpu.rs:198-218
void dot_row_range(float* y, uint64_t rows, const float* x, const float* tmp, uint64_t cols, float scale, bool accumulate) {
    for (uint64_t r = 0; r < rows; ++r) {
        const float* row = tmp + r * cols;
        float acc = 0.0f;
        for (uint64_t i = 0; i < cols; ++i) acc += row[i] * x[i];
        if (accumulate) y[r] += acc * scale; else y[r] = acc * scale;
    }
}

// crates/beholdd-backend/src/cpu.rs:270-286
void q8_0_dot_row_range(float* y, uint64_t rows, const float* x, const uint8_t* packed, uint64_t row_bytes,
                        uint64_t cols, float scale, bool accumulate) {
    for (uint64_t r = 0; r < rows; ++r) {
        const float acc = q8_0_dot(packed + r * row_bytes, x, cols);
        if (accumulate) y[r] += acc * scale; else y[r] = acc * scale;
    }
}

// Row-chunk threading shared by cpu.rs:232-267 (dot_rows) and :291-330 (q8_0_dot_rows): at
// most `threads` contiguous chunks whose sizes differ by at most one row; fresh OS threads on
// every call; the calling thread runs the last chunk.
template <class F>
void for_row_chunks(uint64_t rows, uint64_t threads, F&& body) {
    threads = std::min<uint64_t>(std::max<uint64_t>(threads, 1), std::max<uint64_t>(rows, 1));
    if (threads <= 1) {
        body(0, rows);
        return;
    }
    const uint64_t base = rows / threads, extra = rows % threads;
    std::vector<std::thread> pool;
    pool.reserve(threads - 1);
    uint64_t start = 0;
    for (uint64_t chunk = 0; chunk + 1 < threads; ++chunk) {
        const uint64_t take = base + (chunk < extra ? 1 : 0);
        pool.emplace_back([=, &body] { body(start, take); });
        start += take;
    }
    body(start, rows - start);
    for (auto& t : pool) t.join();
}

// crates/beholdd-backend/src/cpu.rs:415-507 -- the shared body of matvec / matvec_add.
int32_t run_with_threads(float* y, uint64_t y_len, const float* x, uint64_t x_len, const uint8_t* bytes,
                         uint64_t n_bytes, uint32_t kind, uint64_t rows, uint64_t cols, float scale,
                         bool accumulate, uint64_t threads) {
    if (x_len != cols || y_len != rows) return ORC_SHAPE;
    uint64_t n;
    const int32_t st = validate_storage(n_bytes, kind, rows, cols, &n);
    if (st != ORC_OK) return st;
    if (cols == 0) {
        const float result = 0.0f * scale;
        for (uint64_t r = 0; r < rows; ++r) {
            if (accumulate) y[r] += result; else y[r] = result;
        }
        return ORC_OK;
    }
    if (kind == 8) {
        const uint64_t row_bytes = cols / 32 * 34;
        for_row_chunks(rows, threads, [&](uint64_t r0, uint64_t take) {
            q8_0_dot_row_range(y + r0, take, x, bytes + r0 * row_bytes, row_bytes, cols, scale, accumulate);
        });
        return ORC_OK;
    }
    if (kind == 30) {
        // cpu.rs:470-477 uses an AVX-512 BF16 dot whose summation order is not the scalar one;
        // that format is outside the path this oracle pins.
        return ORC_UNSUPPORTED;
    }
    // Dequantise the whole matrix, then sequential f32 dot per row (cpu.rs:488-506).
    std::vector<float> tmp(n);
    const int32_t dq = dequant_any(bytes, n_bytes, kind, rows, cols, tmp.data(), n);
    if (dq != ORC_OK) return dq;
    for_row_chunks(rows, threads, [&](uint64_t r0, uint64_t take) {
        dot_row_range(y + r0, take, x, tmp.data() + r0 * cols, cols, scale, accumulate);
    });
    return ORC_OK;
}

uint64_t available_parallelism() {
    const unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : n;
}

// crates/beholdd-kernel/src/vecops.rs:70-87
void softmax_inplace(float* v, uint64_t n) {
    float m = -std::numeric_limits<float>::infinity();
    for (uint64_t i = 0; i < n; ++i) m = std::fmax(m, v[i]);  // f32::max ignores NaN like fmax
    if (!std::isfinite(m)) {
        for (uint64_t i = 0; i < n; ++i) v[i] = 0.0f;
        return;
    }
    float sum = 0.0f;
    for (uint64_t i = 0; i < n; ++i) {
        v[i] = std::isfinite(v[i]) ? expf(v[i] - m) : 0.0f;
        sum += v[i];
    }
    const float inv = 1.0f / sum;
    for (uint64_t i = 0; i < n; ++i) v[i] *= inv;
}

// crates/beholdd-kernel/src/vecops.rs:91-93
inline float silu(float x) { return x / (1.0f + expf(-x)); }

// crates/beholdd-kernel/src/vecops.rs:101-111
void swiglu_inplace(float* gate, const float* up, uint64_t n, float limit) {
    for (uint64_t i = 0; i < n; ++i) {
        float gv = gate[i], uv = up[i];
        if (limit > 0.0f) {
            gv = std::fmin(gv, limit);
            uv = std::fmax(-limit, std::fmin(uv, limit));
        }
        gate[i] = silu(gv) * uv;
    }
}

// crates/beholdd-kernel/src/vecops.rs:54-64
void rmsnorm(float* y, const float* x, const float* w, uint64_t n, float eps) {
    double ss = 0.0;
    for (uint64_t i = 0; i < n; ++i) ss += double(x[i]) * double(x[i]);
    const float inv = float(1.0 / std::sqrt(ss / double(n) + double(eps)));
    for (uint64_t i = 0; i < n; ++i) y[i] = x[i] * inv * (w ? w[i] : 1.0f);
}

constexpr uint64_t NEAR_MISS_WINDOW = 8;  // crates/beholdd-model/src/qwen3moe/forward.rs (NEAR_MISS_WINDOW)

// crates/beholdd-model/src/qwen3moe/forward.rs:1886-1924
int32_t stable_top_k(const float* p, uint64_t n, uint64_t k, int32_t* idx_out, float* w_out,
                     int32_t* near_out, uint64_t* near_len_out) {
    if (k == 0 || k > n) return ORC_INVALID;
    for (uint64_t i = 0; i < n; ++i)
        if (!std::isfinite(p[i]) || p[i] < 0.0f) return ORC_INVALID;
    std::vector<uint64_t> order(n);
    for (uint64_t i = 0; i < n; ++i) order[i] = i;
    // total_cmp on finite non-negative floats equals the integer order of their bit patterns,
    // which also puts -0.0 below +0.0 the way total_cmp does.
    auto key = [&](uint64_t i) {
        int32_t bits;
        std::memcpy(&bits, p + i, 4);
        return bits < 0 ? int32_t(bits ^ 0x7FFFFFFF) : bits;
    };
    std::stable_sort(order.begin(), order.end(), [&](uint64_t l, uint64_t r) {
        const int32_t kl = key(l), kr = key(r);
        if (kl != kr) return kl > kr;
        return l < r;
    });
    const uint64_t near_len = std::min<uint64_t>(NEAR_MISS_WINDOW, n - k);
    if (near_out)
        for (uint64_t i = 0; i < near_len; ++i) near_out[i] = int32_t(order[k + i]);
    if (near_len_out) *near_len_out = near_len;
    double sum = 0.0;
    for (uint64_t i = 0; i < k; ++i) sum += double(p[order[i]]);
    if (!std::isfinite(sum) || sum <= 0.0) return ORC_INVALID;
    for (uint64_t i = 0; i < k; ++i) {
        idx_out[i] = int32_t(order[i]);
        w_out[i] = float(double(p[order[i]]) / sum);
    }
    return ORC_OK;
}

}  // namespace

extern "C" {

float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

int32_t orc_block_geometry(uint32_t kind, uint64_t* elems, uint64_t* bytes) {
    return block_geometry(kind, elems, bytes) ? ORC_OK : ORC_UNSUPPORTED;
}

// Device::dequantize (crates/beholdd-backend/src/cpu.rs:519-521).
int32_t orc_dequantize(const uint8_t* bytes, uint64_t n_bytes, uint32_t kind, uint64_t rows, uint64_t cols,
                       float* out, uint64_t out_len) {
    return dequant_any(bytes, n_bytes, kind, rows, cols, out, out_len);
}

float orc_q8_0_dot(const uint8_t* row, const float* x, uint64_t cols) { return q8_0_dot(row, x, cols); }

void orc_scale_min_k4(int32_t j, const uint8_t* q, uint8_t* sc, uint8_t* m) { scale_min_k4(j, q, sc, m); }

uint64_t orc_worker_count(uint64_t rows, uint64_t cols, uint64_t available) { return worker_count(rows, cols, available); }

uint64_t orc_available_parallelism() { return available_parallelism(); }

// Device::matvec / Device::matvec_add (cpu.rs:523-535). threads == 0 means "decide like
// Cpu::run" (cpu.rs:398-408); any other value is Cpu::matvec_with_threads.
int32_t orc_matvec(float* y, uint64_t y_len, const float* x, uint64_t x_len, const uint8_t* bytes, uint64_t n_bytes,
                   uint32_t kind, uint64_t rows, uint64_t cols, float scale, int32_t accumulate, uint64_t threads) {
    if (threads == 0) threads = worker_count(rows, cols, available_parallelism());
    return run_with_threads(y, y_len, x, x_len, bytes, n_bytes, kind, rows, cols, scale, accumulate != 0, threads);
}

// The serial "increasing-column F32" matvec the reference's native-kernel specification
// uses for Q4_K/Q6_K (crates/beholdd-backend/src/hag/kernels/kquant.rs:233-256): decode,
// then product and sum as two separately rounded steps.
int32_t orc_serial_matvec(float* y, const float* x, const uint8_t* bytes, uint64_t n_bytes, uint32_t kind,
                          uint64_t rows, uint64_t cols) {
    return run_with_threads(y, rows, x, cols, bytes, n_bytes, kind, rows, cols, 1.0f, false, 1);
}

// Device::softmax (cpu.rs:572-583): refuses empty input and NaN.
int32_t orc_softmax(float* v, uint64_t n) {
    if (n == 0) return ORC_SHAPE;
    for (uint64_t i = 0; i < n; ++i)
        if (std::isnan(v[i])) return ORC_SHAPE;
    softmax_inplace(v, n);
    return ORC_OK;
}

// Device::swiglu (vecops.rs:101-111).
int32_t orc_swiglu(float* gate, const float* up, uint64_t n, float limit) {
    swiglu_inplace(gate, up, n, limit);
    return ORC_OK;
}

int32_t orc_rmsnorm(float* y, const float* x, const float* w, uint64_t n, float eps) {
    if (n == 0 || !std::isfinite(eps) || eps < 0.0f) return ORC_SHAPE;
    rmsnorm(y, x, w, n, eps);
    return ORC_OK;
}

int32_t orc_stable_top_k(const float* p, uint64_t n, uint64_t k, int32_t* idx_out, float* w_out, int32_t* near_out,
                         uint64_t* near_len_out) {
    return stable_top_k(p, n, k, idx_out, w_out, near_out, near_len_out);
}

// Router half of the routed block (forward.rs:1327-1345): per position F32 router matvec
// (the dequantise-then-dot fallback of cpu.rs:488-506), softmax, stable top-k. Also derives
// the per-expert route counts (count[e] = number of (t, j) with experts[t*k+j] == e).
int32_t orc_moe_route(const float* router, uint64_t n_experts, uint64_t dim, const float* x, uint64_t n_positions,
                      uint64_t top_k, float* probs_out, int32_t* experts_out, float* weights_out,
                      int32_t* near_out, int32_t* counts_out) {
    std::vector<float> probs(n_experts);
    const uint64_t near_per = std::min<uint64_t>(NEAR_MISS_WINDOW, n_experts > top_k ? n_experts - top_k : 0);
    if (counts_out)
        for (uint64_t e = 0; e < n_experts; ++e) counts_out[e] = 0;
    for (uint64_t t = 0; t < n_positions; ++t) {
        const uint64_t threads = worker_count(n_experts, dim, available_parallelism());
        int32_t st = run_with_threads(probs.data(), n_experts, x + t * dim, dim,
                                      reinterpret_cast<const uint8_t*>(router), n_experts * dim * 4, 0, n_experts,
                                      dim, 1.0f, false, threads);
        if (st != ORC_OK) return st;
        st = orc_softmax(probs.data(), n_experts);
        if (st != ORC_OK) return st;
        if (probs_out) std::memcpy(probs_out + t * n_experts, probs.data(), n_experts * 4);
        uint64_t near_len = 0;
        st = stable_top_k(probs.data(), n_experts, top_k, experts_out + t * top_k, weights_out + t * top_k,
                          near_out ? near_out + t * near_per : nullptr, &near_len);
        if (st != ORC_OK) return st;
        if (counts_out)
            for (uint64_t j = 0; j < top_k; ++j) counts_out[experts_out[t * top_k + j]] += 1;
    }
    return ORC_OK;
}

// Expert half of the routed block (forward.rs:1360-1400): for each position, for each route
// in selection order: gate matvec, up matvec, swiglu(limit 0), down matvec_add scaled by the
// route weight into a zero-initialised output row. Expert slabs are contiguous Q8_0 matrices
// (forward.rs:1619-1636,1668-1690). `threads` == 0 applies the reference's worker rule.
int32_t orc_moe_experts(const uint8_t* gate_exps, const uint8_t* up_exps, const uint8_t* down_exps, uint64_t n_experts,
                        uint64_t dim, uint64_t expert_ff, const float* x, uint64_t n_positions, uint64_t top_k,
                        const int32_t* experts, const float* expert_weights, float* out, uint64_t threads) {
    if (dim % 32 != 0 || expert_ff % 32 != 0) return ORC_SHAPE;
    const uint64_t gu_slab = expert_ff * (dim / 32) * 34;
    const uint64_t down_slab = dim * (expert_ff / 32) * 34;
    std::vector<float> gate(expert_ff), up(expert_ff);
    for (uint64_t i = 0; i < n_positions * dim; ++i) out[i] = 0.0f;
    for (uint64_t t = 0; t < n_positions; ++t) {
        const float* input = x + t * dim;
        float* out_row = out + t * dim;
        for (uint64_t j = 0; j < top_k; ++j) {
            const int32_t e = experts[t * top_k + j];
            if (e < 0 || uint64_t(e) >= n_experts) return ORC_INVALID;
            const uint64_t tg = threads ? threads : worker_count(expert_ff, dim, available_parallelism());
            const uint64_t td = threads ? threads : worker_count(dim, expert_ff, available_parallelism());
            int32_t st = run_with_threads(gate.data(), expert_ff, input, dim, gate_exps + uint64_t(e) * gu_slab, gu_slab, 8,
                                          expert_ff, dim, 1.0f, false, tg);
            if (st != ORC_OK) return st;
            st = run_with_threads(up.data(), expert_ff, input, dim, up_exps + uint64_t(e) * gu_slab, gu_slab, 8, expert_ff,
                                  dim, 1.0f, false, tg);
            if (st != ORC_OK) return st;
            swiglu_inplace(gate.data(), up.data(), expert_ff, 0.0f);
            st = run_with_threads(out_row, dim, gate.data(), expert_ff, down_exps + uint64_t(e) * down_slab, down_slab, 8,
                                  dim, expert_ff, expert_weights[t * top_k + j], true, td);
            if (st != ORC_OK) return st;
        }
    }
    return ORC_OK;
}

// The whole routed feed-forward of one layer (forward.rs:1299-1407): route, run experts,
// then `hidden += output` (cpu.rs:839-851) when `accumulate` is set, else `y = output`.
int32_t orc_moe_layer(const float* router, const uint8_t* gate_exps, const uint8_t* up_exps, const uint8_t* down_exps,
                      uint64_t n_experts, uint64_t dim, uint64_t expert_ff, const float* x, uint64_t n_positions,
                      uint64_t top_k, float* y, int32_t accumulate, int32_t* experts_out, float* weights_out,
                      int32_t* counts_out, uint64_t threads) {
    int32_t st = orc_moe_route(router, n_experts, dim, x, n_positions, top_k, nullptr, experts_out, weights_out, nullptr,
                               counts_out);
    if (st != ORC_OK) return st;
    std::vector<float> out(n_positions * dim);
    st = orc_moe_experts(gate_exps, up_exps, down_exps, n_experts, dim, expert_ff, x, n_positions, top_k, experts_out,
                         weights_out, out.data(), threads);
    if (st != ORC_OK) return st;
    for (uint64_t i = 0; i < n_positions * dim; ++i) {
        if (accumulate) y[i] += out[i]; else y[i] = out[i];
    }
    return ORC_OK;
}

// ---- the rest of a transformer layer (rotary embedding, causal attention) ----------------------

// crates/beholdd-kernel/src/vecops.rs:118-150 (rope_freqs with optional YaRN interpolation) and :153-161
// (rope_at): cos / sin of one position, f64 angle arithmetic rounded to f32 at the end.
int32_t orc_rope_table(double theta, uint64_t dim, uint64_t orig_seq_len, double factor, double beta_fast, double beta_slow,
                       uint64_t pos, float* cos_out, float* sin_out) {
    if (dim == 0 || dim % 2 != 0 || !cos_out || !sin_out) return ORC_SHAPE;
    const uint64_t half = dim / 2;
    std::vector<double> freqs(half);
    for (uint64_t i = 0; i < half; ++i) freqs[i] = 1.0 / std::pow(theta, double(2 * i) / double(dim));
    if (orig_seq_len > 0) {
        auto corr = [&](double rot) { return double(dim) * std::log(double(orig_seq_len) / (rot * 2.0 * M_PI)) / (2.0 * std::log(theta)); };
        double lo = std::floor(corr(beta_fast)), hi = std::ceil(corr(beta_slow));
        lo = std::max(lo, 0.0);
        hi = std::min(hi, double(dim) - 1.0);
        if (lo == hi) hi += 0.001;
        for (uint64_t i = 0; i < half; ++i) {
            const double ramp = std::min(1.0, std::max(0.0, (double(i) - lo) / (hi - lo)));
            freqs[i] = freqs[i] / factor * ramp + freqs[i] * (1.0 - ramp);
        }
    }
    for (uint64_t i = 0; i < half; ++i) {
        const double a = double(pos) * freqs[i];
        cos_out[i] = float(std::cos(a));
        sin_out[i] = float(std::sin(a));
    }
    return ORC_OK;
}

// Device::rope (crates/beholdd-backend/src/cpu.rs:870-905) over vecops::rope_apply (interleaved pairs,
// vecops.rs:163-178) and rope_apply_split_half (vecops.rs:180-197). layout 0 = interleaved, 1 = split half.
int32_t orc_rope(float* x, uint64_t x_len, const float* cos, const float* sin, uint64_t n_pairs, int32_t layout, int32_t inverse) {
    if (x_len != 2 * n_pairs) return ORC_SHAPE;
    const float sgn = inverse ? -1.0f : 1.0f;
    for (uint64_t i = 0; i < n_pairs; ++i) {
        const uint64_t ia = layout == 0 ? 2 * i : i, ib = layout == 0 ? 2 * i + 1 : i + n_pairs;
        const float a = x[ia], b = x[ib];
        const float c = cos[i], s = sgn * sin[i];
        x[ia] = a * c - b * s;
        x[ib] = a * s + b * c;
    }
    return ORC_OK;
}

// Device::incremental_causal_attention (cpu.rs:693-837); Device::causal_attention (cpu.rs:585-691) is the case
// query_start = 0, n_kv_positions = n_query_positions. f64 dot products and f64 value sums, f32 softmax.
int32_t orc_incremental_attention(float* out, const float* q, const float* k_cache, const float* v_cache, uint64_t n_query_positions,
                                  uint64_t query_start, uint64_t n_kv_positions, uint64_t n_heads, uint64_t n_kv_heads,
                                  uint64_t head_dim, float scale) {
    if (n_query_positions == 0 || n_kv_positions == 0 || n_heads == 0 || n_kv_heads == 0 || head_dim == 0) return ORC_SHAPE;
    if (n_heads % n_kv_heads != 0 || !std::isfinite(scale) || scale <= 0.0f) return ORC_SHAPE;
    if (query_start + n_query_positions > n_kv_positions) return ORC_SHAPE;
    const uint64_t group = n_heads / n_kv_heads;
    std::vector<float> scores(query_start + n_query_positions);
    for (uint64_t qp = 0; qp < n_query_positions; ++qp) {
        const uint64_t abs_pos = query_start + qp;
        for (uint64_t head = 0; head < n_heads; ++head) {
            const uint64_t kv_head = head / group;
            const float* query = q + (qp * n_heads + head) * head_dim;
            for (uint64_t kp = 0; kp <= abs_pos; ++kp) {
                const float* key = k_cache + (kp * n_kv_heads + kv_head) * head_dim;
                double dot = 0.0;
                for (uint64_t d = 0; d < head_dim; ++d) dot += double(query[d]) * double(key[d]);
                scores[kp] = float(dot * double(scale));
            }
            softmax_inplace(scores.data(), abs_pos + 1);
            float* o = out + (qp * n_heads + head) * head_dim;
            for (uint64_t d = 0; d < head_dim; ++d) {
                double sum = 0.0;
                for (uint64_t vp = 0; vp <= abs_pos; ++vp) sum += double(scores[vp]) * double(v_cache[(vp * n_kv_heads + kv_head) * head_dim + d]);
                o[d] = float(sum);
            }
        }
    }
    return ORC_OK;
}

// The host libm's expf over an array: what the reference's softmax and SiLU call through Rust's
// f32::exp (crates/beholdd-kernel/src/vecops.rs:70-93). Lets a test compare the device's expf with it.
void orc_expf_array(const float* in, float* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = expf(in[i]);
}

}  // extern "C"
