// Route planning for the routed-expert block: a stable counting sort of the local routes by expert,
// and the list of expert groups the grouped kernels work through.
//
// The reference visits routes per (position, route) and has no such step
// (crates/beholdd-model/src/qwen3moe/forward.rs:1363-1400); sorting by expert is what lets every
// expert's weights be read once for all the routes that selected it. The order inside an expert
// is the route index, so the plan (and with it every sum downstream) is the same from run to
// run and does not depend on how the work was spread over CTAs.
//
// Two launches, both spread over the routes:
//   k_moe_hist    route block b (2048 routes) = 8 warps x 256 consecutive routes; every warp
//                 counts its routes per local expert. The last CTA to finish turns the counts into
//                 exclusive prefixes over (block, warp) per expert, expert offsets, and the
//                 group records and per-class group lists (in expert order).
//   k_moe_scatter the same walk again: slot = expert offset + prefix of (block, warp) + rank
//                 inside the warp's range, by warp-wide matching of equal experts. With a single
//                 route block (up to 2048 routes) the first launch does this step as well.
// All integer work; ids outside [0, n_total) are reported through the status word, ids of other
// ranks' experts are skipped.
#include "common.cuh"

namespace {

constexpr int PLAN_THREADS = 256, PLAN_WARPS = PLAN_THREADS / 32, WARP_ROUTES = 256, BLOCK_ROUTES = PLAN_WARPS * WARP_ROUTES;
constexpr int NQ = 2 + BHD_MOE_CLASSES;  // scanned per expert: routes, groups, groups per class

__device__ __forceinline__ uint32_t lanemask_lt() {
    uint32_t m;
    asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Local expert index of route r, or -1 (another rank's expert, a bad id, or beyond the routes).
__device__ __forceinline__ int32_t local_expert(const int32_t* __restrict__ experts, uint32_t r, uint32_t n_routes, uint32_t first,
                                                uint32_t n_local, uint32_t n_total, uint32_t* status) {
    if (r >= n_routes) return -1;
    const int32_t e = experts[r];
    if (e < 0 || uint32_t(e) >= n_total) {
        if (status) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
        return -1;
    }
    if (uint32_t(e) < first || uint32_t(e) >= first + n_local) return -1;
    return int32_t(uint32_t(e) - first);
}

// Parts an expert with n routes is cut into: equal sizes (+-1), `big` of them one route larger.
struct Parts { uint32_t parts, small_nb, big; };
__device__ __forceinline__ Parts cut(uint32_t n, uint32_t cap) {
    Parts p;
    p.parts = (n + cap - 1) / cap;
    p.small_nb = p.parts ? n / p.parts : 0u;
    p.big = p.parts ? n % p.parts : 0u;
    return p;
}

// The second walk over the routes of block `block`: slot = expert offset + prefix of (block, warp) + rank inside
// the warp's range. `run` [PLAN_WARPS][n_local] is shared-memory scratch.
__device__ __forceinline__ void scatter_block(const int32_t* __restrict__ experts, const float* __restrict__ weights, uint32_t n_routes,
                                              uint32_t first, uint32_t n_local, uint32_t n_total, uint32_t cap, const MoePlanBuffers& b,
                                              uint32_t block, uint32_t* run) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = threadIdx.x; i < PLAN_WARPS * n_local; i += PLAN_THREADS) run[i] = 0u;
    __syncthreads();
    const uint32_t r0 = block * BLOCK_ROUTES + warp * WARP_ROUTES;
    const uint32_t* prefix = b.whist + (uint64_t(block) * PLAN_WARPS + warp) * n_local;
    for (int it = 0; it < WARP_ROUTES / 32; ++it) {
        const uint32_t r = r0 + it * 32 + lane;
        const int32_t el = local_expert(experts, r, n_routes, first, n_local, n_total, nullptr);
        const uint32_t mask = __match_any_sync(0xffffffffu, el >= 0 ? uint32_t(el) : 0x80000000u + lane);
        uint32_t seen = 0;
        if (el >= 0) seen = run[warp * n_local + el];
        __syncwarp();
        if (el >= 0) {
            const uint32_t in_expert = __ldcg(prefix + el) + seen + __popc(mask & lanemask_lt());  // rank among the expert's routes
            const uint32_t slot = __ldcg(b.offsets + el) + in_expert;
            if ((mask & lanemask_lt()) == 0) run[warp * n_local + el] = seen + __popc(mask);
            // size class of the group this slot falls into (the cut of the histogram step, recomputed)
            const Parts pt = cut(__ldcg(b.counts + el), cap);
            const uint32_t in_big = pt.big * (pt.small_nb + 1);
            const uint32_t nb = in_expert < in_big ? pt.small_nb + 1 : pt.small_nb;
            b.route_slot[r] = int32_t(slot);
            b.slot_route[slot] = int32_t(r);
            b.slot_weight[slot] = weights[r];
            b.slot_cls[slot] = uint8_t(bhd_moe_cls(int(nb)));
            if (b.peer_rows) {
                const uint32_t pos = r / b.top_k, j = r - pos * b.top_k, owner = pos / b.t_per_rank, t = pos - owner * b.t_per_rank;
                b.slot_dst[slot] = b.peer_rows[owner] + (uint64_t(j) * b.t_per_rank + t) * b.dim;
            }
        } else if (r < n_routes) {
            b.route_slot[r] = -1;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(PLAN_THREADS) k_moe_hist(const int32_t* __restrict__ experts, const float* __restrict__ weights,
                                                           uint32_t n_routes, uint32_t first, uint32_t n_local, uint32_t n_total,
                                                           uint32_t cap, uint32_t n_positions, MoePlanBuffers b, uint32_t* ticket,
                                                           uint32_t* status) {
    bhd_wait_for_prior_kernels();
    extern __shared__ uint32_t hist[];  // [PLAN_WARPS][n_local], later the per-expert totals
    __shared__ uint32_t s_warp[PLAN_WARPS][NQ], s_carry[NQ];
    __shared__ bool s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_blocks = gridDim.x;
    for (uint32_t i = threadIdx.x; i < PLAN_WARPS * n_local; i += PLAN_THREADS) hist[i] = 0u;
    __syncthreads();
    const uint32_t r0 = blockIdx.x * BLOCK_ROUTES + warp * WARP_ROUTES;
    for (int it = 0; it < WARP_ROUTES / 32; ++it) {
        const int32_t el = local_expert(experts, r0 + it * 32 + lane, n_routes, first, n_local, n_total, status);
        const uint32_t mask = __match_any_sync(0xffffffffu, el >= 0 ? uint32_t(el) : 0x80000000u + lane);
        if (el >= 0 && (mask & lanemask_lt()) == 0) hist[warp * n_local + el] += __popc(mask);  // one leader per expert, own row
        __syncwarp();
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < PLAN_WARPS * n_local; i += PLAN_THREADS)
        b.whist[uint64_t(blockIdx.x) * PLAN_WARPS * n_local + i] = hist[i];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1u) == n_blocks - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- the last CTA: prefixes, offsets, groups ----
    uint32_t* total = hist;  // [n_local]
    for (uint32_t e = threadIdx.x; e < n_local; e += PLAN_THREADS) {
        uint32_t run = 0;
        for (uint32_t i = 0; i < n_blocks * PLAN_WARPS; ++i) {
            uint32_t* p = b.whist + uint64_t(i) * n_local + e;
            const uint32_t c = __ldcg(p);
            __stcg(p, run);
            run += c;
        }
        total[e] = run;
        // A position names an expert at most once (the selection is a top-k of distinct experts), so no expert has more
        // routes than there are positions; the grouped kernels are only launched for the size classes that rule allows.
        if (run > n_positions) atomicOr(status, BHD_DEV_BAD_EXPERT_ID);
    }
    if (threadIdx.x < NQ) s_carry[threadIdx.x] = 0u;
    __syncthreads();
    // Experts in chunks of one per thread: a block-wide exclusive scan of (routes, groups, groups per
    // class) gives every expert its first slot, its first group index and its place in each class
    // list, exactly as a sequential walk over the experts would assign them.
    for (uint32_t e0 = 0; e0 < n_local; e0 += PLAN_THREADS) {
        const uint32_t e = e0 + threadIdx.x;
        const uint32_t n = e < n_local ? total[e] : 0u;
        const Parts pt = cut(n, cap);
        const int cls_small = pt.small_nb ? bhd_moe_cls(int(pt.small_nb)) : 0, cls_big = bhd_moe_cls(int(pt.small_nb + 1));
        uint32_t v[NQ], incl[NQ];
        v[0] = n;
        v[1] = pt.parts;
#pragma unroll
        for (int c = 0; c < BHD_MOE_CLASSES; ++c)
            v[2 + c] = ((pt.big && cls_big == c) ? pt.big : 0u) + ((pt.small_nb && cls_small == c) ? pt.parts - pt.big : 0u);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            incl[q] = v[q];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t o = __shfl_up_sync(0xffffffffu, incl[q], d);
                if (lane >= d) incl[q] += o;
            }
            if (lane == 31) s_warp[warp][q] = incl[q];
        }
        __syncthreads();
        uint32_t base[NQ], chunk_total[NQ];
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            base[q] = s_carry[q];
            chunk_total[q] = 0;
            for (int w = 0; w < PLAN_WARPS; ++w) {
                const uint32_t t = s_warp[w][q];
                if (w < warp) base[q] += t;
                chunk_total[q] += t;
            }
            base[q] += incl[q] - v[q];
        }
        if (e < n_local) {
            b.offsets[e] = base[0];
            b.counts[e] = n;
            uint32_t s0 = base[0], ng = base[1];
            uint32_t gc[BHD_MOE_CLASSES];
#pragma unroll
            for (int c = 0; c < BHD_MOE_CLASSES; ++c) gc[c] = base[2 + c];
            for (uint32_t part = 0; part < pt.parts && ng < b.gmax; ++part) {
                const uint32_t nb = pt.small_nb + (part < pt.big ? 1u : 0u);
                const int cls = bhd_moe_cls(int(nb));
                MoeGroup g;
                g.expert_local = int32_t(e); g.slot0 = int32_t(s0); g.nb = int32_t(nb); g.cls = cls;
                g.pad0 = g.pad1 = g.pad2 = g.pad3 = 0;
                uint32_t at = 0;
#pragma unroll
                for (int c = 0; c < BHD_MOE_CLASSES; ++c)
                    if (c == cls) at = gc[c]++;
                b.glist[uint64_t(cls) * b.gmax + at] = int32_t(ng);
                b.groups[ng++] = g;
                s0 += nb;
            }
        }
        __syncthreads();
        if (threadIdx.x < NQ) s_carry[threadIdx.x] += chunk_total[threadIdx.x];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        b.offsets[n_local] = s_carry[0];
#pragma unroll
        for (int c = 0; c < 8; ++c) b.hdr->gcount[c] = c < BHD_MOE_CLASSES ? s_carry[2 + c] : 0u;
        b.hdr->total_groups = s_carry[1];
        b.hdr->local_routes = s_carry[0];
        b.hdr->pad0 = b.hdr->pad1 = 0;
        *ticket = 0u;  // ready for the next launch
    }
    // A single route block needs no second launch: this CTA has everything the scatter step reads.
    if (n_blocks == 1) {
        __threadfence();
        __syncthreads();
        scatter_block(experts, weights, n_routes, first, n_local, n_total, cap, b, 0, hist);
    }
}

__global__ void __launch_bounds__(PLAN_THREADS) k_moe_scatter(const int32_t* __restrict__ experts, const float* __restrict__ weights,
                                                              uint32_t n_routes, uint32_t first, uint32_t n_local, uint32_t n_total,
                                                              uint32_t cap, MoePlanBuffers b) {
    bhd_wait_for_prior_kernels();
    extern __shared__ uint32_t run[];  // [PLAN_WARPS][n_local]: routes of the expert already seen by this warp
    scatter_block(experts, weights, n_routes, first, n_local, n_total, cap, b, blockIdx.x, run);
}

}  // namespace

size_t bhd_moe_plan_scratch_words(uint32_t n_routes, uint32_t n_local) {
    const size_t blocks = (size_t(n_routes) + BLOCK_ROUTES - 1) / BLOCK_ROUTES;
    return blocks * PLAN_WARPS * n_local;
}

int32_t bhd_launch_moe_plan(bhd_ctx* ctx, const int32_t* experts, const float* weights, uint32_t n_routes, uint32_t first_expert,
                            uint32_t n_local, uint32_t n_total, uint32_t cap, uint32_t n_positions, const MoePlanBuffers& b, cudaStream_t s) {
    if (n_routes == 0 || n_local == 0 || n_local > 1024) return bhd_fail(ctx, BHD_ERR_SHAPE, "shape mismatch: route plan for %u routes, %u experts", n_routes, n_local);
    const unsigned blocks = unsigned((n_routes + BLOCK_ROUTES - 1) / BLOCK_ROUTES);
    const size_t smem = size_t(PLAN_WARPS) * n_local * sizeof(uint32_t);  // at most 32 KB
    uint32_t* ticket = ctx->status_dev + 1;  // a spare word next to the status word; zero between launches
    bhd_launch_dependent(ctx, k_moe_hist, dim3(blocks), dim3(PLAN_THREADS), smem, s, experts, weights, n_routes, first_expert, n_local, n_total, cap, n_positions, b, ticket,
                                                  ctx->status_dev);
    BHD_LAUNCHED(ctx, "route histogram kernel");
    if (blocks > 1) {  // a single block scatters inside the first launch
        bhd_launch_dependent(ctx, k_moe_scatter, dim3(blocks), dim3(PLAN_THREADS), smem, s, experts, weights, n_routes, first_expert, n_local, n_total, cap, b);
        BHD_LAUNCHED(ctx, "route scatter kernel");
    }
    return BHD_OK;
}
