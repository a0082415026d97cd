// Shared declarations of the beholdd_b200 library: context and weight handles, error
// plumbing, and the per-element decoders of the packed GGUF block formats.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/beholdd_b200.h"

#define BHD_CTX_MAGIC 0x62686443u  // "bhdC"
#define BHD_MAX_DEVICES 64  // contexts are refused on device indices beyond this
#define BHD_WEIGHT_MAGIC 0x62686457u  // "bhdW"

// Device status word bits (kernels OR them in; bhd_check_status reports and clears them).
#define BHD_DEV_NAN_IN_SOFTMAX 1u
#define BHD_DEV_BAD_EXPERT_ID 2u
#define BHD_DEV_WAIT_TIMEOUT 4u
#define BHD_DEV_BAD_ROUTE_PROB 8u
#define BHD_DEV_ACTIVATION_RANGE 16u

struct bhd_ctx {
    uint32_t magic;
    int device;
    int sm_count;
    char err[512];
    uint8_t* workspace;     // grown on demand; used by calls in stream order
    size_t workspace_bytes;
    uint32_t* status_dev;   // device status word (+ spare words)
    uint32_t* status_host;  // pinned mirror
    uint32_t* counters;     // 65536 tile counters of the split-column reduction; zero between launches
    float* stage_x;         // device staging for the host-buffer entry points
    float* stage_y;
    size_t stage_x_bytes, stage_y_bytes;
    void* pinned;           // pinned bounce buffer for host entry points
    size_t pinned_bytes;
    cudaStream_t host_stream;  // non-blocking stream of the host-buffer entry points
    cudaStream_t side_stream[3];  // the routed experts' size classes run side by side: forked from and joined to the caller's stream
    cudaEvent_t fork_event, join_event[3];
    uint32_t spin_limit;    // polls a bounded wait makes before it gives up (0: the kernel's default)
    uint32_t debug_drop;    // test hook: the next decode matvec leaves this many copies unrequested
    uint32_t moe_tc_min_cls; // smallest group size class the tensor-core grouped kernel takes (0: the default)
    uint32_t moe_tc_plain;   // 1: the tensor-core grouped kernel with singly rounded fp16 operands in shared memory
    uint32_t router_variant; // tiling of the router-logits kernel for more than 64 positions (0: default)
    uint32_t plain_launches; // 1: no programmatic dependent launches (every kernel starts after the one before it ended)
    uint32_t gemm_impl;      // prefill matmul: 0 the library's choice, 1 one CTA per tile, 2 the same with the weight operand in tensor memory, 3 CTA pairs, 4 persistent CTAs, 5 CTA pairs on 512-token tiles
    uint64_t launches;
    void* tmap_encode;      // cuTensorMapEncodeTiled, resolved once at creation
};

struct bhd_weight {
    uint32_t magic;
    bhd_ctx* ctx;
    int device;           // the context's GPU, kept here so that a weight can be freed after its context
    uint8_t* dev;
    bool owned;
    uint32_t kind;
    uint64_t rows, cols, slabs;
    uint64_t row_bytes;   // packed bytes of one row
    uint64_t slab_bytes;  // rows * row_bytes
    // 2-D tensor map over all rows of all slabs ([slabs*rows][row_bytes] bytes) for the
    // TMA-staged kernels; valid only when `tmap_ok`.
    alignas(64) unsigned char tmap[128];
    bool tmap_ok;
    uint32_t tmap_box_rows, tmap_box_bytes;
    alignas(64) unsigned char tmap16[128];  // same view with a 16-row box (decode kernel)
    bool tmap16_ok;
};

// Makes the context's GPU the calling thread's current device for the duration of one exported
// call and puts the caller's device back afterwards, so a host with several GPUs (or a current
// device that differs from the context's) launches on the right one. It also empties the
// thread's "last error" slot: an error another library left there must not be mistaken for a
// failure of the launch that follows.
struct bhd_device_guard {
    int prev = -1;
    bool switched = false;
    explicit bhd_device_guard(const bhd_ctx* ctx) : bhd_device_guard(ctx->device) {}
    explicit bhd_device_guard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != device) {
            cudaSetDevice(device);
            switched = true;
        }
        cudaGetLastError();
    }
    ~bhd_device_guard() {
        if (switched && prev >= 0) cudaSetDevice(prev);
    }
    bhd_device_guard(const bhd_device_guard&) = delete;
    bhd_device_guard& operator=(const bhd_device_guard&) = delete;
};

// Work that must happen once per GPU (kernel attributes are per device): `static bhd_once_per_device once;`
// at the launch site, then `if (once.first(ctx)) { ... }`.
struct bhd_once_per_device {
    bool done[BHD_MAX_DEVICES] = {};
    bool pending(const bhd_ctx* ctx) const { return !done[ctx->device]; }
    void mark(const bhd_ctx* ctx) { done[ctx->device] = true; }
};

int32_t bhd_fail(bhd_ctx* ctx, int32_t status, const char* fmt, ...);
int32_t bhd_cuda_fail(bhd_ctx* ctx, cudaError_t e, const char* what);
int32_t bhd_ensure_workspace(bhd_ctx* ctx, size_t bytes, cudaStream_t stream);
const char* bhd_kind_name(uint32_t kind);
bool bhd_block_geometry(uint32_t kind, uint64_t* elems, uint64_t* bytes);

#define BHD_CUDA(ctx, call, what)                                   \
    do {                                                            \
        cudaError_t _e = (call);                                    \
        if (_e != cudaSuccess) return bhd_cuda_fail(ctx, _e, what); \
    } while (0)

#define BHD_LAUNCHED(ctx, what)                                     \
    do {                                                            \
        cudaError_t _e = cudaGetLastError();                        \
        if (_e != cudaSuccess) return bhd_cuda_fail(ctx, _e, what); \
        (ctx)->launches += 1;                                       \
    } while (0)

// ---- dependent launches -----------------------------------------------------------------
// A kernel launched through bhd_launch_dependent may be scheduled while the kernel before it in the stream is still
// draining (programmatic dependent launch), which hides most of the launch latency of a chain of short kernels. Such a
// kernel executes bhd_wait_for_prior_kernels() as its first statement: that returns once every kernel before it in
// the stream has finished and its writes are visible, so the ordering is that of a plain launch. Never give the
// attribute to a kernel that does not wait: its successor would only wait for it, not for the kernels before it.
__device__ __forceinline__ void bhd_wait_for_prior_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void bhd_launch_dependent(const bhd_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->plain_launches ? 0 : 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);  // the caller reads the outcome with BHD_LAUNCHED
}

// ---- per-element decoders -------------------------------------------------------------
// Each returns exactly the f32 the reference's CPU decoder produces for element k of a
// packed row (crates/beholdd-kernel/src/kquant.rs:39-54, 115-162, 209-241, 268-303): the
// same multiplications in the same order, each rounded to f32 (no FMA contraction).

__device__ __forceinline__ float bhd_f16_bits_to_f32(uint16_t h) {
    // Exact for every bit pattern including subnormals, like
    // crates/beholdd-core/src/quant.rs:259-278.
    return __half2float(__ushort_as_half(h));
}

// Every 16-bit field of every supported block format sits at an even offset of an even-sized
// block, and weight bases are at least 16-byte aligned, so this load is always aligned.
__device__ __forceinline__ uint16_t bhd_ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}

__device__ __forceinline__ void bhd_scale_min_k4(int j, const uint8_t* q, uint32_t* sc, uint32_t* m) {
    if (j < 4) {
        *sc = q[j] & 63u;
        *m = q[j + 4] & 63u;
    } else {
        *sc = (q[j + 4] & 0xFu) | ((uint32_t(q[j - 4]) >> 6) << 4);
        *m = (uint32_t(q[j + 4]) >> 4) | ((uint32_t(q[j]) >> 6) << 4);
    }
}

template <uint32_t KIND>
__device__ __forceinline__ float bhd_decode_elem(const uint8_t* row, uint64_t k);

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_F32>(const uint8_t* row, uint64_t k) {
    return *reinterpret_cast<const float*>(row + 4 * k);
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_F16>(const uint8_t* row, uint64_t k) {
    return bhd_f16_bits_to_f32(bhd_ld_u16(row + 2 * k));
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_BF16>(const uint8_t* row, uint64_t k) {
    // the upper half of an f32 (crates/beholdd-core/src/quant.rs bf16_to_f32; cpu.rs:113-122)
    return __uint_as_float(uint32_t(bhd_ld_u16(row + 2 * k)) << 16);
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_Q8_0>(const uint8_t* row, uint64_t k) {
    const uint8_t* blk = row + (k >> 5) * 34;
    const float d = bhd_f16_bits_to_f32(bhd_ld_u16(blk));
    return __fmul_rn(d, float(int8_t(blk[2 + (k & 31)])));
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_Q4_K>(const uint8_t* row, uint64_t k) {
    const uint8_t* blk = row + (k >> 8) * 144;
    const uint32_t i = uint32_t(k & 255), pass = i >> 6, hi = (i >> 5) & 1, l = i & 31;
    const float d = bhd_f16_bits_to_f32(bhd_ld_u16(blk));
    const float dmin = bhd_f16_bits_to_f32(bhd_ld_u16(blk + 2));
    uint32_t sc, m;
    bhd_scale_min_k4(int(pass * 2 + hi), blk + 4, &sc, &m);
    const uint32_t q = (uint32_t(blk[16 + pass * 32 + l]) >> (4 * hi)) & 15u;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, float(sc)), float(q)), __fmul_rn(dmin, float(m)));
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_Q5_K>(const uint8_t* row, uint64_t k) {
    const uint8_t* blk = row + (k >> 8) * 176;
    const uint32_t i = uint32_t(k & 255), pass = i >> 6, hi = (i >> 5) & 1, l = i & 31;
    const float d = bhd_f16_bits_to_f32(bhd_ld_u16(blk));
    const float dmin = bhd_f16_bits_to_f32(bhd_ld_u16(blk + 2));
    uint32_t sc, m;
    bhd_scale_min_k4(int(pass * 2 + hi), blk + 4, &sc, &m);
    const uint32_t bit = (uint32_t(blk[16 + l]) >> (pass * 2 + hi)) & 1u;
    const uint32_t q = ((uint32_t(blk[48 + pass * 32 + l]) >> (4 * hi)) & 15u) + 16u * bit;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, float(sc)), float(q)), __fmul_rn(dmin, float(m)));
}

template <>
__device__ __forceinline__ float bhd_decode_elem<BHD_TYPE_Q6_K>(const uint8_t* row, uint64_t k) {
    const uint8_t* blk = row + (k >> 8) * 210;
    const uint32_t i = uint32_t(k & 255), half_i = i >> 7, within = i & 127, group = within >> 5, lane = within & 31;
    const uint32_t low = (uint32_t(blk[half_i * 64 + (group & 1) * 32 + lane]) >> (4 * (group >> 1))) & 15u;
    const uint32_t high = (uint32_t(blk[128 + half_i * 32 + lane]) >> (2 * group)) & 3u;
    const int code = int(low | (high << 4)) - 32;
    const float d = bhd_f16_bits_to_f32(bhd_ld_u16(blk + 208));
    const float scale = float(int8_t(blk[192 + (i >> 4)]));
    return __fmul_rn(__fmul_rn(d, scale), float(code));
}

// Dispatch a template on the weight kind.
#define BHD_DISPATCH_KIND(kind, MACRO)                   \
    switch (kind) {                                      \
        case BHD_TYPE_F32: MACRO(BHD_TYPE_F32); break;   \
        case BHD_TYPE_F16: MACRO(BHD_TYPE_F16); break;   \
        case BHD_TYPE_Q8_0: MACRO(BHD_TYPE_Q8_0); break; \
        case BHD_TYPE_Q4_K: MACRO(BHD_TYPE_Q4_K); break; \
        case BHD_TYPE_Q5_K: MACRO(BHD_TYPE_Q5_K); break; \
        case BHD_TYPE_Q6_K: MACRO(BHD_TYPE_Q6_K); break; \
        case BHD_TYPE_BF16: MACRO(BHD_TYPE_BF16); break; \
        default: break;                                  \
    }

// ---- routed-expert plan records (written by the plan kernels, read by the grouped kernels) ------
// Routes are sorted by (expert, route index) into "slots"; an expert's slots are cut into groups of at
// most `cap` routes and every group belongs to the size class of its route count.
constexpr int BHD_MOE_CLASSES = 7;  // groups of up to 4, 8, 16, 32, 64, 128, 256 routes
__host__ __device__ constexpr int bhd_moe_cls(int nb) {
    return nb <= 4 ? 0 : (nb <= 8 ? 1 : (nb <= 16 ? 2 : (nb <= 32 ? 3 : (nb <= 64 ? 4 : (nb <= 128 ? 5 : 6)))));
}
__host__ __device__ constexpr uint32_t bhd_moe_cls_least(int cls) { return cls == 0 ? 1u : (4u << (cls - 1)) + 1u; }  // 1, 5, 9, 17, 33, 65, 129
struct MoeGroup {
    int32_t expert_local, slot0, nb, cls;
    uint32_t pad0, pad1, pad2, pad3;
};
struct MoeHeader {
    uint32_t gcount[8];  // groups per size class
    uint32_t total_groups, local_routes, pad0, pad1;
};

extern "C" int32_t bhd_peer_alloc(bhd_ctx* ctx, uint64_t n_bytes, void** out_dev, uint8_t* handle64);
extern "C" int32_t bhd_peer_open(bhd_ctx* ctx, const uint8_t* handle64, void** out_dev);
extern "C" int32_t bhd_peer_close(bhd_ctx* ctx, void* dev);
extern "C" int32_t bhd_peer_free(bhd_ctx* ctx, void* dev);

// ---- kernel launchers implemented across the .cu files --------------------------------
int32_t bhd_launch_dequantize(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, float* out, cudaStream_t s);
int32_t bhd_launch_matvec_strict(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                 uint32_t batch, float scale, int accumulate, cudaStream_t s);
int32_t bhd_launch_matvec_general(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const float* x, float* y,
                                  uint64_t batch, float scale, int accumulate, cudaStream_t s);
int32_t bhd_launch_moe_grouped_i8(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                  const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* xq, uint32_t n_slots,
                                  float* out0, float* out1, float* const* slot_dst, const float* slot_weight, cudaStream_t s);

int32_t bhd_launch_moe_slots_i8(bhd_ctx* ctx, int mode, const void* hdr, const int32_t* slot_route, const uint8_t* slot_cls,
                                uint32_t max_cls, uint32_t top_k, const float* src, const float* src2, uint32_t K, uint32_t n_slots,
                                void* out, cudaStream_t s);
int32_t bhd_launch_moe_rows_f16(bhd_ctx* ctx, int mode, const void* hdr, const int32_t* slot_route, const uint8_t* slot_cls,
                                uint32_t min_cls, uint32_t top_k, const float* src, const float* src2, uint32_t K, uint32_t n_slots,
                                void* out16, void* out16_lo, const float* slot_weight, float* scale_out, cudaStream_t s);
int32_t bhd_launch_gemm_q8_ts_grouped(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                      const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* x_hi, const void* x_lo,
                                      uint32_t n_slots, float* out0, float* out1, float* const* row_dst, const float* col_scale,
                                      cudaStream_t s);
int32_t bhd_launch_gemm_q8_ts_dense(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M, cudaStream_t s);
int32_t bhd_launch_gemm_q8_pair(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M, bool wide, cudaStream_t s);
int32_t bhd_launch_gemm_q8_persistent(bhd_ctx* ctx, const bhd_weight* w, uint64_t slab, const void* x16, float* y, uint32_t M, cudaStream_t s);
bool bhd_gemm_q8_ts_usable(const bhd_ctx* ctx, const bhd_weight* w);
int32_t bhd_launch_gemm_q8_grouped(bhd_ctx* ctx, const bhd_weight* w0, const bhd_weight* w1, const void* hdr, const void* groups,
                                   const int32_t* glist, uint32_t cls, uint32_t group_bound, const void* x16, uint32_t n_slots,
                                   float* out0, float* out1, const float* col_scale, cudaStream_t s);
bool bhd_gemm_q8_grouped_usable(const bhd_ctx* ctx, const bhd_weight* w);
int32_t bhd_launch_stage_copy(bhd_ctx* ctx, const float* src_mapped, float* dst_dev, size_t n16, cudaStream_t s);
size_t bhd_moe_slots_i8_bytes(uint32_t K, uint32_t n_slots);
// Sorts the routes of the local experts by (expert, route index) and lists the groups: see moe_plan.cu.
struct MoePlanBuffers {
    MoeHeader* hdr;
    uint32_t *counts, *offsets;     // [n_local], [n_local + 1]
    int32_t *route_slot;            // [routes]: slot of a local route, -1 for a route of another rank
    int32_t *slot_route;            // [routes]: route of a slot
    float* slot_weight;             // [routes]: route weight of a slot
    uint8_t* slot_cls;              // [routes]: size class of the group the slot belongs to
    MoeGroup* groups;               // [gmax]
    int32_t* glist;                 // [BHD_MOE_CLASSES][gmax]: group indices per class, in expert order
    uint32_t* whist;                // [route blocks * 8][n_local] scratch
    uint32_t gmax;
    // Expert parallel: where the weighted output row of each slot goes. Route r = (p * top_k + j) of global
    // position p belongs to rank p / t_per_rank, whose buffer of returned rows [top_k][t_per_rank][dim] starts at
    // peer_rows[that rank] (as mapped in this process). Null peer_rows: rows stay in the local scratch.
    float** slot_dst;               // [routes]
    float* const* peer_rows;
    uint32_t t_per_rank, dim, top_k;
};
struct MoePeerOut {                 // argument of the fast expert path when it runs as one rank of an expert-parallel group
    float* const* peer_rows;
    uint32_t t_per_rank;
};
int32_t bhd_moe_experts_fast(bhd_ctx* ctx, const bhd_weight* gate, const bhd_weight* up, const bhd_weight* down,
                             const float* x, uint64_t T, uint32_t top_k, const int32_t* experts, const float* weights,
                             uint32_t first_expert, uint32_t n_local, uint32_t n_total, float* y, int accumulate,
                             cudaStream_t s, bool* handled, const MoePeerOut* peer);
size_t bhd_moe_plan_scratch_words(uint32_t n_routes, uint32_t n_local);
int32_t bhd_launch_moe_plan(bhd_ctx* ctx, const int32_t* experts, const float* weights, uint32_t n_routes, uint32_t first_expert,
                            uint32_t n_local, uint32_t n_total, uint32_t cap, uint32_t n_positions, const MoePlanBuffers& b, cudaStream_t s);
bool bhd_moe_i8_usable(const bhd_weight* w);

