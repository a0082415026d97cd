// Expert-parallel execution of the routed-expert layer over the GPUs of one node, with the exchange
// done by the kernels themselves over peer memory (NVLink / NVSwitch): no collective library on the
// data path, no host round trip, and the whole layer can be captured into a CUDA graph.
//
// Rank r holds experts [r * E / W, (r + 1) * E / W) and owns T positions per call (the same T on
// every rank). One layer:
//   1. route the own positions (bit-exact selection, moe.cu);
//   2. dispatch: copy the own x rows, expert ids and route weights into slot `rank` of EVERY rank's
//      exchange block (a position's 8 routes reach most ranks anyway, and each row travels once per
//      rank instead of once per route), then raise this rank's flag in every block;
//   3. wait for all W flags, then run the grouped expert kernels over all W * T positions for
//      the local experts only. The down-projection epilogues store each route's weighted output
//      row straight into the block of the rank that owns the position, at [route j][position t];
//   4. raise this rank's second flag everywhere, wait for all W of them, and add the k returned
//      rows of every own position in selection order: ((0 + r0) + r1) + ..., the reference's order
//      (crates/beholdd-model/src/qwen3moe/forward.rs:1385-1398). Each row is computed by the same
//      arithmetic as on one GPU, so the result is bit-identical to the single-GPU layer run on
//      the W * T positions, for every W.
// Flags carry a call counter that only grows (kept on the device, so a captured graph replays
// correctly); every wait is bounded and reports through the status word. Loads and stores to
// peer memory are ordinary ones; nothing here uses multicast.
//
// The reference is single-process and has no counterpart (its routed block is forward.rs:1299-1407).
#include <new>

#include "common.cuh"

#define BHD_EP_MAGIC 0x62686445u  // "bhdE"
constexpr int EP_MAX_WORLD = 8;
constexpr uint32_t EP_SPIN_LIMIT = 1u << 21;  // polls of a flag in this GPU's own memory: about a second

int32_t bhd_moe_route_internal(bhd_ctx* ctx, const bhd_weight* router, const float* x_dev, uint64_t n_positions, uint32_t top_k,
                               int32_t* experts_dev, float* weights_dev, int32_t* counts_dev, cudaStream_t s);

struct EpLayout {  // byte offsets inside every rank's exchange block
    size_t x, experts, weights, rows, flags, total;
};
struct EpPeers {
    uint8_t* base[EP_MAX_WORLD];
};

struct bhd_ep {
    uint32_t magic;
    bhd_ctx* ctx;
    uint32_t rank, world, n_experts, dim, top_k, max_t;
    EpLayout lay;
    uint8_t* local;
    EpPeers peers;       // peers.base[r]: rank r's block as mapped in this process (own block at [rank])
    float** rows_table;  // device array [world]: the rows buffer of every rank
    bool connected;
};

namespace {

EpLayout ep_layout(uint32_t world, uint32_t max_t, uint32_t dim, uint32_t top_k) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    EpLayout l;
    size_t off = 0;
    l.x = off; off = up(off + size_t(world) * max_t * dim * 4);
    l.experts = off; off = up(off + size_t(world) * max_t * top_k * 4);
    l.weights = off; off = up(off + size_t(world) * max_t * top_k * 4);
    l.rows = off; off = up(off + size_t(top_k) * max_t * dim * 4);
    l.flags = off; off = up(off + 64 * 4);
    l.total = off;
    return l;
}
// words of the flag area
constexpr int FLAG_DISPATCH = 0, FLAG_RETURN = 8, FLAG_EPOCH = 16, FLAG_TICKET = 17;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Copies this rank's positions and routes into every rank's block; the last CTA to finish starts a new
// call (epoch + 1) and raises this rank's dispatch flag in every block.
__global__ void __launch_bounds__(256) k_ep_dispatch(const float* __restrict__ x, const int32_t* __restrict__ experts,
                                                     const float* __restrict__ weights, uint32_t T, uint32_t dim, uint32_t top_k,
                                                     uint32_t rank, uint32_t world, EpPeers peers, EpLayout lay) {
    __shared__ bool s_last;
    const size_t n4 = size_t(T) * dim / 4, nr = size_t(T) * top_k;
    const size_t tid = blockIdx.x * size_t(blockDim.x) + threadIdx.x, step = size_t(gridDim.x) * blockDim.x;
    for (size_t i = tid; i < n4; i += step) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        for (uint32_t r = 0; r < world; ++r) reinterpret_cast<float4*>(peers.base[r] + lay.x)[size_t(rank) * n4 + i] = v;
    }
    for (size_t i = tid; i < nr; i += step) {
        const int32_t e = experts[i];
        const float w = weights[i];
        for (uint32_t r = 0; r < world; ++r) {
            reinterpret_cast<int32_t*>(peers.base[r] + lay.experts)[size_t(rank) * nr + i] = e;
            reinterpret_cast<float*>(peers.base[r] + lay.weights)[size_t(rank) * nr + i] = w;
        }
    }
    __threadfence_system();
    __syncthreads();
    uint32_t* flags = reinterpret_cast<uint32_t*>(peers.base[rank] + lay.flags);
    if (threadIdx.x == 0) s_last = atomicAdd(flags + FLAG_TICKET, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    const uint32_t e = flags[FLAG_EPOCH] + 1u;
    if (threadIdx.x < world) st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + lay.flags) + FLAG_DISPATCH + rank, e);
    __syncthreads();
    if (threadIdx.x == 0) {
        flags[FLAG_EPOCH] = e;
        flags[FLAG_TICKET] = 0u;
    }
}

// One warp. With `raise`: publishes this rank's earlier stores to peer memory and raises its flag `which` in every
// block first. Then waits until all ranks' flags in the own block have reached the current call.
__global__ void k_ep_sync(int raise, int which, uint32_t rank, uint32_t world, EpPeers peers, EpLayout lay, uint32_t* status) {
    const uint32_t lane = threadIdx.x;
    uint32_t* flags = reinterpret_cast<uint32_t*>(peers.base[rank] + lay.flags);
    const uint32_t e = flags[FLAG_EPOCH];
    if (raise) {
        __threadfence_system();
        if (lane < world) st_release_sys(reinterpret_cast<uint32_t*>(peers.base[lane] + lay.flags) + which + rank, e);
    }
    if (lane < world) {
        bool ok = false;
        for (uint32_t spin = 0; spin < EP_SPIN_LIMIT; ++spin) {
            if (int32_t(ld_acquire_sys(flags + which + lane) - e) >= 0) { ok = true; break; }
            __nanosleep(200);
        }
        if (!ok) atomicOr(status, BHD_DEV_WAIT_TIMEOUT);
    }
}

__global__ void k_ep_combine(const float* __restrict__ rows, float* __restrict__ y, uint64_t n, uint32_t top_k, int accumulate) {
    const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    float out = 0.0f;
    for (uint32_t j = 0; j < top_k; ++j) out = __fadd_rn(out, __ldcg(rows + uint64_t(j) * n + i));  // written by peers: not through L1
    y[i] = accumulate ? __fadd_rn(y[i], out) : out;
}

bool ep_ok(const bhd_ep* ep) { return ep && ep->magic == BHD_EP_MAGIC && ep->ctx && ep->ctx->magic == BHD_CTX_MAGIC; }

}  // namespace

extern "C" int32_t bhd_ep_create(bhd_ctx* ctx, uint32_t rank, uint32_t world, uint32_t n_experts, uint32_t dim, uint32_t top_k,
                                 uint32_t max_positions, bhd_ep** out_ep, uint8_t* handle64) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (!out_ep || !handle64) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_create: null output");
    *out_ep = nullptr;
    if (world < 1 || world > EP_MAX_WORLD || rank >= world || n_experts == 0 || n_experts % world != 0 || dim == 0 || dim % 4 != 0 ||
        top_k == 0 || max_positions == 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: expert-parallel group of %u ranks (at most %d), rank %u, %u experts, width %u",
                        world, EP_MAX_WORLD, rank, n_experts, dim);
    bhd_ep* ep = new (std::nothrow) bhd_ep();
    if (!ep) return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate host memory for an exchange handle", bhd_device_name());
    memset(ep, 0, sizeof(*ep));
    ep->ctx = ctx;
    ep->rank = rank; ep->world = world; ep->n_experts = n_experts; ep->dim = dim; ep->top_k = top_k; ep->max_t = max_positions;
    ep->lay = ep_layout(world, max_positions, dim, top_k);
    void* p = nullptr;
    int32_t st = bhd_peer_alloc(ctx, ep->lay.total, &p, handle64);
    if (st != BHD_OK) { delete ep; return st; }
    ep->local = static_cast<uint8_t*>(p);
    ep->peers.base[rank] = ep->local;
    bhd_device_guard guard(ctx);
    if (cudaMalloc(reinterpret_cast<void**>(&ep->rows_table), sizeof(float*) * EP_MAX_WORLD) != cudaSuccess) {
        cudaGetLastError();
        bhd_peer_free(ctx, p);
        delete ep;
        return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %zu bytes for %s", bhd_device_name(), sizeof(float*) * EP_MAX_WORLD, "an exchange table");
    }
    ep->magic = BHD_EP_MAGIC;
    ep->connected = world == 1;
    if (world == 1) {
        float* rows = reinterpret_cast<float*>(ep->local + ep->lay.rows);
        cudaMemcpy(ep->rows_table, &rows, sizeof(float*), cudaMemcpyHostToDevice);
    }
    *out_ep = ep;
    return BHD_OK;
}

extern "C" int32_t bhd_ep_connect(bhd_ep* ep, const uint8_t* handles) {
    if (!ep_ok(ep)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = ep->ctx;
    if (!handles) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_connect: null handles");
    bhd_device_guard guard(ctx);
    float* table[EP_MAX_WORLD] = {};
    for (uint32_t r = 0; r < ep->world; ++r) {
        if (r != ep->rank && !ep->peers.base[r]) {
            void* p = nullptr;
            const int32_t st = bhd_peer_open(ctx, handles + 64 * size_t(r), &p);
            if (st != BHD_OK) return st;
            ep->peers.base[r] = static_cast<uint8_t*>(p);
        }
        table[r] = reinterpret_cast<float*>(ep->peers.base[r] + ep->lay.rows);
    }
    BHD_CUDA(ctx, cudaMemcpy(ep->rows_table, table, sizeof(float*) * ep->world, cudaMemcpyHostToDevice), "writing the exchange table");
    ep->connected = true;
    return BHD_OK;
}

extern "C" int32_t bhd_ep_destroy(bhd_ep* ep) {
    if (!ep_ok(ep)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = ep->ctx;
    {
        bhd_device_guard guard(ctx);
        cudaDeviceSynchronize();
        for (uint32_t r = 0; r < ep->world; ++r)
            if (r != ep->rank && ep->peers.base[r]) cudaIpcCloseMemHandle(ep->peers.base[r]);
        if (ep->rows_table) cudaFree(ep->rows_table);
        if (ep->local) cudaFree(ep->local);
        cudaGetLastError();
    }
    ep->magic = 0;
    delete ep;
    return BHD_OK;
}

extern "C" int32_t bhd_ep_layer(bhd_ep* ep, const bhd_weight* router, const bhd_weight* gate_exps, const bhd_weight* up_exps,
                                const bhd_weight* down_exps, const float* x_dev, float* y_dev, uint64_t n_positions,
                                int32_t* experts_dev, float* weights_dev, int32_t* counts_dev, int32_t accumulate, void* stream) {
    if (!ep_ok(ep)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = ep->ctx;
    if (!ep->connected) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_layer: the group is not connected yet");
    if (!router || router->magic != BHD_WEIGHT_MAGIC || router->ctx != ctx || !gate_exps || gate_exps->magic != BHD_WEIGHT_MAGIC ||
        gate_exps->ctx != ctx || !up_exps || up_exps->magic != BHD_WEIGHT_MAGIC || up_exps->ctx != ctx || !down_exps ||
        down_exps->magic != BHD_WEIGHT_MAGIC || down_exps->ctx != ctx)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_layer: tensors are not weights of this context");
    const uint32_t W = ep->world, k = ep->top_k, dim = ep->dim, per = ep->n_experts / W;
    if (router->rows != ep->n_experts || router->cols != dim || gate_exps->cols != dim || gate_exps->slabs != per ||
        up_exps->slabs != per || down_exps->slabs != per || down_exps->rows != dim || up_exps->rows != gate_exps->rows ||
        up_exps->cols != dim || down_exps->cols != gate_exps->rows)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: router %llux%llu, %llu local experts of %llux%llu against a group of %u experts of width %u on %u ranks",
                        (unsigned long long)router->rows, (unsigned long long)router->cols, (unsigned long long)gate_exps->slabs,
                        (unsigned long long)gate_exps->rows, (unsigned long long)gate_exps->cols, ep->n_experts, dim, W);
    if (n_positions == 0) return BHD_OK;
    if (n_positions > ep->max_t)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: %llu positions, the exchange was created for at most %u per rank",
                        (unsigned long long)n_positions, ep->max_t);
    if (!x_dev || !y_dev || !experts_dev || !weights_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_layer: null buffer");
    if ((reinterpret_cast<uintptr_t>(x_dev) & 15) != 0) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "ep_layer: x must be 16-byte aligned");
    bhd_device_guard guard(ctx);
    cudaStream_t s = cudaStream_t(stream);
    const uint32_t T = uint32_t(n_positions);

    int32_t st = bhd_moe_route_internal(ctx, router, x_dev, T, k, experts_dev, weights_dev, counts_dev, s);
    if (st != BHD_OK) return st;
    const size_t work = size_t(T) * dim / 4;
    const unsigned grid = unsigned(work / 256 < 1 ? 1 : (work / 256 > 128 ? 128 : work / 256));
    k_ep_dispatch<<<grid, 256, 0, s>>>(x_dev, experts_dev, weights_dev, T, dim, k, ep->rank, W, ep->peers, ep->lay);
    BHD_LAUNCHED(ctx, "expert-parallel dispatch kernel");
    k_ep_sync<<<1, 32, 0, s>>>(0, FLAG_DISPATCH, ep->rank, W, ep->peers, ep->lay, ctx->status_dev);
    BHD_LAUNCHED(ctx, "expert-parallel wait kernel");

    MoePeerOut peer;
    peer.peer_rows = ep->rows_table;
    peer.t_per_rank = T;
    bool handled = false;
    st = bhd_moe_experts_fast(ctx, gate_exps, up_exps, down_exps, reinterpret_cast<const float*>(ep->local + ep->lay.x), uint64_t(W) * T, k,
                              reinterpret_cast<const int32_t*>(ep->local + ep->lay.experts),
                              reinterpret_cast<const float*>(ep->local + ep->lay.weights), ep->rank * per, per, ep->n_experts, nullptr, 0, s,
                              &handled, &peer);
    if (st != BHD_OK) return st;
    if (!handled)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: the expert-parallel layer needs Q8_0 experts whose packed rows are multiples of 16 bytes");
    k_ep_sync<<<1, 32, 0, s>>>(1, FLAG_RETURN, ep->rank, W, ep->peers, ep->lay, ctx->status_dev);
    BHD_LAUNCHED(ctx, "expert-parallel signal kernel");
    const uint64_t n = uint64_t(T) * dim;
    k_ep_combine<<<unsigned((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const float*>(ep->local + ep->lay.rows), y_dev, n, k, accumulate);
    BHD_LAUNCHED(ctx, "route combine kernel");
    return BHD_OK;
}

// ---- a large projection with its rows split over the ranks -----------------------------------------
// Rank r holds rows [r * N / W, (r + 1) * N / W) of the packed weight (whole packed rows, so no sum
// crosses a GPU and the order of every row's summation is the single-GPU order), computes its slice
// of y with the ordinary matvec kernels, and one more kernel stores the slice into every rank's copy
// of y over peer memory, raises this rank's flag everywhere, waits (bounded) for the other ranks'
// flags and hands the assembled y to the caller. Two buffers alternate between calls: a rank that
// runs ahead writes the next call's slice into the other buffer while a slower rank still reads
// this call's. The reference's counterpart is a plain Device::matvec (crates/beholdd-backend/src/lib.rs:182-198).

#define BHD_RS_MAGIC 0x62686452u  // "bhdR"

struct RsLayout {
    size_t y[2], flags, total;
};

struct bhd_rowsplit {
    uint32_t magic;
    bhd_ctx* ctx;
    uint32_t rank, world, rows, max_batch;
    RsLayout lay;
    uint8_t* local;
    EpPeers peers;
    float* slice;  // [max_batch x rows / world] local scratch
    bool connected;
};

namespace {

constexpr int RS_FLAG = 0, RS_EPOCH = 16;

// One CTA. slice [batch x per] -> rows [rank * per, +per) of y in every rank's block; flags; wait; y -> out.
__global__ void __launch_bounds__(1024) k_rs_exchange(const float* __restrict__ slice, uint32_t batch, uint32_t per, uint32_t rows,
                                                      uint32_t rank, uint32_t world, EpPeers peers, RsLayout lay, float* __restrict__ out,
                                                      uint32_t* status) {
    uint32_t* flags = reinterpret_cast<uint32_t*>(peers.base[rank] + lay.flags);
    const uint32_t e = flags[RS_EPOCH] + 1u;
    const size_t yoff = lay.y[e & 1u];
    const uint32_t n = batch * per;
    if ((per & 3u) == 0) {
        const uint32_t per4 = per / 4;
        for (uint32_t i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const uint32_t b = i / per4, c = i - b * per4;
            const float4 v = reinterpret_cast<const float4*>(slice)[i];
            for (uint32_t r = 0; r < world; ++r)
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(peers.base[r] + yoff) + size_t(b) * rows + size_t(rank) * per + 4 * c) = v;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            const uint32_t b = i / per, c = i - b * per;
            const float v = slice[i];
            for (uint32_t r = 0; r < world; ++r) reinterpret_cast<float*>(peers.base[r] + yoff)[size_t(b) * rows + size_t(rank) * per + c] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + lay.flags) + RS_FLAG + rank, e);
        bool ok = false;
        for (uint32_t spin = 0; spin < EP_SPIN_LIMIT; ++spin) {
            if (int32_t(ld_acquire_sys(flags + RS_FLAG + threadIdx.x) - e) >= 0) { ok = true; break; }
            __nanosleep(100);
        }
        if (!ok) atomicOr(status, BHD_DEV_WAIT_TIMEOUT);
    }
    __syncthreads();
    if (threadIdx.x == 0) flags[RS_EPOCH] = e;
    const float* y = reinterpret_cast<const float*>(peers.base[rank] + yoff);
    for (uint32_t i = threadIdx.x; i < batch * rows; i += blockDim.x) out[i] = __ldcg(y + i);  // written by peers: not through L1
}

bool rs_ok(const bhd_rowsplit* rs) { return rs && rs->magic == BHD_RS_MAGIC && rs->ctx && rs->ctx->magic == BHD_CTX_MAGIC; }

}  // namespace

extern "C" int32_t bhd_rowsplit_create(bhd_ctx* ctx, uint32_t rank, uint32_t world, uint32_t rows, uint32_t max_batch,
                                       bhd_rowsplit** out_rs, uint8_t* handle64) {
    if (!ctx || ctx->magic != BHD_CTX_MAGIC) return BHD_ERR_INVALID_ARGUMENT;
    if (!out_rs || !handle64) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rowsplit_create: null output");
    *out_rs = nullptr;
    if (world < 1 || world > EP_MAX_WORLD || rank >= world || rows == 0 || rows % world != 0 || max_batch == 0)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: %u rows do not split over %u ranks (at most %d), rank %u", rows, world,
                        EP_MAX_WORLD, rank);
    bhd_rowsplit* rs = new (std::nothrow) bhd_rowsplit();
    if (!rs) return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate host memory for an exchange handle", bhd_device_name());
    memset(rs, 0, sizeof(*rs));
    rs->ctx = ctx;
    rs->rank = rank; rs->world = world; rs->rows = rows; rs->max_batch = max_batch;
    const size_t ybytes = (size_t(max_batch) * rows * 4 + 255) / 256 * 256;
    rs->lay.y[0] = 0; rs->lay.y[1] = ybytes; rs->lay.flags = 2 * ybytes; rs->lay.total = 2 * ybytes + 256;
    void* p = nullptr;
    int32_t st = bhd_peer_alloc(ctx, rs->lay.total, &p, handle64);
    if (st != BHD_OK) { delete rs; return st; }
    rs->local = static_cast<uint8_t*>(p);
    rs->peers.base[rank] = rs->local;
    bhd_device_guard guard(ctx);
    if (cudaMalloc(reinterpret_cast<void**>(&rs->slice), size_t(max_batch) * (rows / world) * 4) != cudaSuccess) {
        cudaGetLastError();
        bhd_peer_free(ctx, p);
        delete rs;
        return bhd_fail(ctx, BHD_ERR_ALLOCATION, "%s could not allocate %zu bytes for %s", bhd_device_name(),
                        size_t(max_batch) * (rows / world) * 4, "a row-split slice");
    }
    rs->magic = BHD_RS_MAGIC;
    rs->connected = world == 1;
    *out_rs = rs;
    return BHD_OK;
}

extern "C" int32_t bhd_rowsplit_connect(bhd_rowsplit* rs, const uint8_t* handles) {
    if (!rs_ok(rs)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = rs->ctx;
    if (!handles) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rowsplit_connect: null handles");
    bhd_device_guard guard(ctx);
    for (uint32_t r = 0; r < rs->world; ++r) {
        if (r == rs->rank || rs->peers.base[r]) continue;
        void* p = nullptr;
        const int32_t st = bhd_peer_open(ctx, handles + 64 * size_t(r), &p);
        if (st != BHD_OK) return st;
        rs->peers.base[r] = static_cast<uint8_t*>(p);
    }
    rs->connected = true;
    return BHD_OK;
}

extern "C" int32_t bhd_rowsplit_destroy(bhd_rowsplit* rs) {
    if (!rs_ok(rs)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = rs->ctx;
    {
        bhd_device_guard guard(ctx);
        cudaDeviceSynchronize();
        for (uint32_t r = 0; r < rs->world; ++r)
            if (r != rs->rank && rs->peers.base[r]) cudaIpcCloseMemHandle(rs->peers.base[r]);
        if (rs->slice) cudaFree(rs->slice);
        if (rs->local) cudaFree(rs->local);
        cudaGetLastError();
    }
    rs->magic = 0;
    delete rs;
    return BHD_OK;
}

extern "C" int32_t bhd_rowsplit_matvec(bhd_rowsplit* rs, const bhd_weight* shard, uint64_t slab, const float* x_dev, float* y_dev,
                                       uint32_t batch, float scale, void* stream) {
    if (!rs_ok(rs)) return BHD_ERR_INVALID_ARGUMENT;
    bhd_ctx* ctx = rs->ctx;
    if (!rs->connected) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rowsplit_matvec: the group is not connected yet");
    if (!shard || shard->magic != BHD_WEIGHT_MAGIC || shard->ctx != ctx)
        return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rowsplit_matvec: not a weight of this context");
    const uint32_t per = rs->rows / rs->world;
    if (shard->rows != per)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: the shard has %llu rows, a rank of this group holds %u", (unsigned long long)shard->rows, per);
    if (batch == 0) return BHD_OK;
    if (batch > rs->max_batch)
        return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: %u activation vectors, the exchange was created for at most %u", batch, rs->max_batch);
    if (!x_dev || !y_dev) return bhd_fail(ctx, BHD_ERR_INVALID_ARGUMENT, "rowsplit_matvec: null buffer");
    bhd_device_guard guard(ctx);
    int32_t st = batch <= 8 ? bhd_matvec(ctx, shard, slab, x_dev, rs->slice, batch, scale, 0, stream)
                            : bhd_matmul(ctx, shard, slab, x_dev, rs->slice, batch, stream);
    if (st != BHD_OK) return st;
    k_rs_exchange<<<1, 1024, 0, cudaStream_t(stream)>>>(rs->slice, batch, per, rs->rows, rs->rank, rs->world, rs->peers, rs->lay, y_dev,
                                                         ctx->status_dev);
    BHD_LAUNCHED(ctx, "row-split exchange kernel");
    return BHD_OK;
}
