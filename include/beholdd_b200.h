/*
 * beholdd_b200 -- C ABI of the B200 (sm_100a) implementation of beholdd's quantised-matvec
 * and qwen3moe routed-expert hot path.
 *
 * Conventions (the same ones beholdd's existing native transport uses,
 * vendor/exec-hag/include/exec_hag.h:13-66): every call returns an int32_t status, 0 on
 * success and negative on refusal or failure; handles are opaque; buffers are owned by the
 * caller; calls on one context are serialised by the caller; nothing unwinds across this
 * boundary. A refused call never touches its outputs and never falls back to another path
 * (crates/beholdd-backend/src/lib.rs:62-66).
 *
 * Pointers named *_dev are device pointers on the context's GPU; pointers named *_host are
 * host pointers. `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 * Device-pointer calls are asynchronous on `stream`; host-pointer calls synchronise before
 * they return.
 *
 * Paths in comments are relative to the reference repository root.
 */
#ifndef BEHOLDD_B200_H
#define BEHOLDD_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Status codes. The first four mirror DeviceError (crates/beholdd-backend/src/lib.rs:60-101). */
#define BHD_OK 0
#define BHD_ERR_UNSUPPORTED_FORMAT (-1) /* DeviceError::UnsupportedFormat */
#define BHD_ERR_SHAPE (-2)              /* DeviceError::Shape */
#define BHD_ERR_ALLOCATION (-3)         /* DeviceError::Allocation */
#define BHD_ERR_BACKEND (-4)            /* DeviceError::Backend (a CUDA call failed) */
#define BHD_ERR_INVALID_ARGUMENT (-5)   /* null handle, foreign handle, non-finite scale */
#define BHD_ERR_DEVICE_STATUS (-6)      /* a kernel reported a problem through its status word */

/* ggml type codes of the weight formats (crates/beholdd-core/src/quant.rs:79-118). */
#define BHD_TYPE_F32 0u
#define BHD_TYPE_F16 1u
#define BHD_TYPE_Q8_0 8u
#define BHD_TYPE_Q4_K 12u
#define BHD_TYPE_Q5_K 13u
#define BHD_TYPE_Q6_K 14u
#define BHD_TYPE_BF16 30u

typedef struct bhd_ctx bhd_ctx;       /* one per GPU; owns the stream-ordered workspace */
/* Device and workspace rules of a context:
 *  - Every call makes the context's GPU the calling thread's current device while it runs and
 *    restores the caller's device before it returns; the caller's current device need not match.
 *  - The workspace grows on demand (first call of a larger size): growing synchronises the device,
 *    frees the old block and allocates a new one. A CUDA graph captured earlier keeps the old
 *    block's addresses, so capture only after one eager call of the largest shape, and never
 *    during a capture call a shape larger than any eager call before it. */
typedef struct bhd_weight bhd_weight; /* a packed weight resident in HBM */

/* Static text for a status code (like exec_hag_error_text). */
const char* bhd_error_text(int32_t status);

/* Detailed message of the last failed call on this context (DeviceError's Display text).
 * Copies at most `capacity` bytes including the terminator; returns the full length. */
int32_t bhd_last_error_message(const bhd_ctx* ctx, char* buffer, int32_t capacity);

/* Device::name (crates/beholdd-backend/src/lib.rs:166). */
const char* bhd_device_name(void);

/* Create / destroy a context on CUDA device `device`. Replaces constructing the backend
 * object (Cpu::new, crates/beholdd-backend/src/cpu.rs:46-49; a resident backend is created
 * like crates/beholdd-backend/src/execution.rs:1143-1154). */
int32_t bhd_ctx_create(int32_t device, bhd_ctx** out_ctx);
int32_t bhd_ctx_destroy(bhd_ctx* ctx);

/* Device::supports (crates/beholdd-backend/src/lib.rs:172; cpu.rs:515-517): 1 if the
 * library decodes this ggml type, else 0. */
int32_t bhd_supports(uint32_t ggml_type);

/* ExecutionDevice::upload_weight + prepare_weight (crates/beholdd-backend/src/execution.rs:
 * 1066-1070): validates the exact byte count like Cpu::validate_storage (cpu.rs:55-97) and
 * copies the packed bytes to HBM unchanged. A weight may hold `n_slabs` equally shaped
 * matrices back to back (a 3-D expert tensor, crates/beholdd-model/src/qwen3moe/forward.rs:
 * 1668-1690); `rows` is then the row count of ONE slab. */
int32_t bhd_weight_upload(bhd_ctx* ctx, const uint8_t* bytes_host, uint64_t n_bytes, uint32_t ggml_type,
                          uint64_t rows, uint64_t cols, uint64_t n_slabs, bhd_weight** out_weight);
/* Same, but the packed bytes already sit in device memory owned by the caller, which must
 * keep them alive and unchanged while the handle exists (no copy is made). */
int32_t bhd_weight_wrap_device(bhd_ctx* ctx, const void* bytes_dev, uint64_t n_bytes, uint32_t ggml_type,
                               uint64_t rows, uint64_t cols, uint64_t n_slabs, bhd_weight** out_weight);
int32_t bhd_weight_free(bhd_weight* weight);

/* Device::dequantize (crates/beholdd-backend/src/lib.rs:179; cpu.rs:99-130): decode slab
 * `slab` into rows*cols floats. */
int32_t bhd_dequantize(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, float* out_dev, uint64_t out_len,
                       void* stream);

/* Device::matvec / Device::matvec_add (crates/beholdd-backend/src/lib.rs:182-198;
 * cpu.rs:398-507) on resident operands, for `batch` activation vectors at once:
 *   accumulate == 0:  y[b][r]  = (sum_i W[r][i] * x[b][i]) * scale
 *   accumulate != 0:  y[b][r] += (sum_i W[r][i] * x[b][i]) * scale
 * x is [batch x cols], y is [batch x rows], both row-major f32. The reference has no batched
 * form (it loops matvec per position, forward.rs:1091-1100); batch > 1 reads the weights
 * once. Device::matvec is scale = 1, accumulate = 0. A non-finite scale is refused
 * (execution.rs:616-622). cols == 0 gives 0*scale (cpu.rs:439-452). */
int32_t bhd_matvec(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, const float* x_dev, float* y_dev,
                   uint32_t batch, float scale, int32_t accumulate, void* stream);

/* The same operation through host buffers, the shape of the immediate Device trait whose
 * slices live in host memory: copies x in, runs, copies y back, synchronises. When y_host is
 * page-locked and accumulate == 0 the kernel writes y into it directly (unified addressing)
 * and the copy back is skipped; x is always staged through device memory. */
int32_t bhd_matvec_host(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, const float* x_host, float* y_host,
                        uint32_t batch, float scale, int32_t accumulate);

/* bhd_matvec_host without the wait: the copies and the kernel are queued on the context's own
 * (non-blocking) stream and the call returns. Results are in y_host, and problems the kernels
 * flagged are reported, once bhd_sync has returned. A page-locked x_host is read by the GPU
 * when the queued work runs, so it must stay unchanged until then; a pageable x_host is copied
 * before the call returns. Calls are executed in the order they were made. This is the shape of
 * ExecutionDevice::submit / wait (crates/beholdd-backend/src/execution.rs:1101-1114) for a single
 * Linear command on host-visible buffers. */
int32_t bhd_matvec_host_async(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, const float* x_host,
                              float* y_host, uint32_t batch, float scale, int32_t accumulate);

/* Waits for everything the host-buffer entry points queued on this context
 * (ExecutionDevice::wait, execution.rs:1111-1114) and returns BHD_ERR_DEVICE_STATUS if a kernel
 * flagged a problem (the word is cleared). */
int32_t bhd_sync(bhd_ctx* ctx);

/* No counterpart in the reference. A decode matvec (the operation of bhd_matvec for batch <= 4;
 * results agree with it within the path's tolerance, not to the bit, because bhd_matvec may pick
 * a different kernel for the same shape) for hosts that may not allocate device memory once they are serving: real-time
 * decode loops that cannot take the allocator's locks or implicit synchronisation, processes
 * that gave all of HBM to their own arena at start-up. Its scratch (the packed fp16
 * activations) is a fixed 288 KiB array inside the library image, held by every GPU that loads
 * the library until the process exits, instead of the context workspace; the call performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *   - Limit: batch <= 4, and the packed activations must fit the array (always true for
 *     cols <= 16384); anything larger is refused with BHD_ERR_SHAPE, outputs untouched.
 *   - The first call on a device also looks up the array's device address; make that call
 *     before starting any stream capture.
 *   - All calls on a GPU share the one array (from any context or stream): calls whose kernels
 *     can overlap on the GPU race on it. Issue them on one stream, or order them yourself. */
int32_t bhd_matvec_noalloc(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, const float* x_dev, float* y_dev,
                           uint32_t batch, float scale, int32_t accumulate, void* stream);

/* Prefill: Y[m][n] = sum_k X[m][k] * W[n][k] for m < M, a loop of Device::matvec over
 * positions in the reference (crates/beholdd-model/src/qwen3moe/forward.rs:1086-1127).
 * Tensor-core forms (fp16 operands, f32 accumulation, max relative error about 2e-3): Q8_0 from 64 positions on;
 * Q4_K and Q6_K from 256 positions on, Q6_K only when a packed row is a multiple of 16 bytes (columns a multiple
 * of 2048). Everything else runs on the integer kernels in batches of at most 8 positions. */
int32_t bhd_matmul(bhd_ctx* ctx, const bhd_weight* weight, uint64_t slab, const float* x_dev, float* y_dev,
                   uint64_t m, void* stream);

/* Device::softmax over `n_rows` rows of `n` floats in place (lib.rs:208; cpu.rs:572-583;
 * vecops.rs:70-87). NaN input is reported through BHD_ERR_DEVICE_STATUS by
 * bhd_check_status. */
int32_t bhd_softmax(bhd_ctx* ctx, float* v_dev, uint64_t n_rows, uint64_t n, void* stream);

/* Device::swiglu: gate[i] = silu(gate[i]) * up[i] with the asymmetric clamp when limit > 0
 * (lib.rs:258; vecops.rs:101-111). */
int32_t bhd_swiglu(bhd_ctx* ctx, float* gate_dev, const float* up_dev, uint64_t n, float limit, void* stream);

/* Device::add_in_place: output[i] += residual[i] (lib.rs:255; cpu.rs:839-851). */
int32_t bhd_add_in_place(bhd_ctx* ctx, float* output_dev, const float* residual_dev, uint64_t n, void* stream);

/* Router half of the routed block (forward.rs:1327-1345 with stable_top_k :1886-1924):
 * F32 router matvec in the CPU's summation order, softmax, stable top-k with lower-index
 * tie-break, renormalisation in f64. Outputs (any may be NULL except experts/weights):
 *   experts_dev  [T x top_k] int32   expert ids in selection order
 *   weights_dev  [T x top_k] f32     renormalised route weights
 *   counts_dev   [n_experts] int32   routes per expert
 *   near_dev     [T x min(8, n_experts - top_k)] int32  ranks top_k.. (near misses)
 *   probs_dev    [T x n_experts] f32 softmax probabilities
 * `router` must be an F32 weight [n_experts x dim]. */
int32_t bhd_moe_route(bhd_ctx* ctx, const bhd_weight* router, const float* x_dev, uint64_t n_positions,
                      uint32_t top_k, int32_t* experts_dev, float* weights_dev, int32_t* counts_dev,
                      int32_t* near_dev, float* probs_dev, void* stream);

/* Expert half (forward.rs:1360-1400): for every position and every route in selection
 * order, gate and up matvec, SiLU gating (vecops.rs:101-111, limit 0), down matvec scaled
 * by the route weight and added in route order into a zeroed row. gate/up weights hold
 * n_experts slabs [expert_ff x dim], down holds n_experts slabs [dim x expert_ff], all Q8_0.
 * Only experts e with first_expert <= e < first_expert + n_local are applied (the others
 * contribute nothing), which is what one rank of an expert-parallel group computes; the
 * slabs of `gate/up/down` are then the local experts only. With first_expert = 0 and
 * n_local = n_experts this is the whole layer. `n_experts` is the layer's expert count over all
 * ranks: an id outside [0, n_experts) is reported through the status word (pass 0 if unknown; only
 * negative ids can then be told from another rank's). The experts of one position must be distinct, as the
 * reference's stable top-k yields them: the grouped kernels (Q8_0 experts with 16-byte aligned rows) report an
 * expert named by more routes than there are positions through the status word; the general kernels compute
 * any assignment.
 *   accumulate == 0: y[t] = out[t];  accumulate != 0: y[t] += out[t]  (forward.rs:1405-1407) */
int32_t bhd_moe_experts(bhd_ctx* ctx, const bhd_weight* gate_exps, const bhd_weight* up_exps,
                        const bhd_weight* down_exps, const float* x_dev, uint64_t n_positions, uint32_t top_k,
                        const int32_t* experts_dev, const float* weights_dev, uint32_t first_expert,
                        uint32_t n_local, uint32_t n_experts, float* y_dev, int32_t accumulate, void* stream);

/* Weighted combine of per-route outputs (forward.rs:1385-1398; cpu.rs:280-284): per_route is
 * [top_k][T][dim], each row already scaled by its route weight; for every position the rows
 * are added in selection order into a zero accumulator, ((0 + r0) + r1) + ..., then stored
 * (accumulate == 0) or added to y (accumulate != 0). This is the owner-side half of the
 * expert-parallel layer, where the rows come back from the ranks that hold the experts. */
int32_t bhd_moe_combine(bhd_ctx* ctx, const float* per_route_dev, float* y_dev, uint64_t n_positions, uint32_t top_k,
                        uint64_t dim, int32_t accumulate, void* stream);

/* ---- the rest of a transformer layer (what config "full forward" needs around the projections and the experts) ----
 *
 * Device::rmsnorm (lib.rs:200-206; cpu.rs:537-570; vecops.rs:54-64) over n_rows rows of n floats:
 * y = x / sqrt(mean(x^2) + eps) * w with an f64 sum of squares; weight_dev may be NULL. With n = head_dim and
 * one row per (position, head) this is the per-head QK-norm (forward.rs:1131-1160). */
int32_t bhd_rmsnorm(bhd_ctx* ctx, float* y_dev, const float* x_dev, const float* weight_dev, uint64_t n_rows, uint64_t n,
                    float eps, void* stream);

/* Device::rope (lib.rs:260-272; cpu.rs:870-905; vecops.rs:163-197) in place on n_positions * vectors_per_position
 * vectors of 2 * n_pairs floats; cos/sin are [n_positions][n_pairs] (vecops::rope_at per position, computed by the
 * host in f64). layout 0 = interleaved pairs, 1 = split half (Qwen); inverse != 0 negates the sine. */
int32_t bhd_rope(bhd_ctx* ctx, float* x_dev, const float* cos_dev, const float* sin_dev, uint64_t n_positions,
                 uint32_t vectors_per_position, uint32_t n_pairs, int32_t layout, int32_t inverse, void* stream);

/* Device::incremental_causal_attention (lib.rs:228-253; cpu.rs:693-837): q [n_query][n_heads][head_dim] at absolute
 * positions query_start.., caches [n_kv_positions][n_kv_heads][head_dim] f32; position p attends to cache entries
 * 0..p. Device::causal_attention (cpu.rs:585-691) is query_start = 0 with the sequence itself as the cache. f64 dot
 * products and value sums, f32 softmax, as the CPU computes them: every kernel form gives the CPU's bits. Forms: one
 * query of 128-wide heads over up to about 2600 positions runs on a cluster of four CTAs per head; 8 or more queries of
 * 128-wide heads run in blocks of 32 (query, head) pairs that share a kv head (the query heads per kv head a power of
 * two, at most 32; over more than about 760 positions the blocks keep their scores in the context workspace);
 * everything else one CTA per (query, head). */
int32_t bhd_incremental_attention(bhd_ctx* ctx, float* out_dev, const float* q_dev, const float* k_cache_dev,
                                  const float* v_cache_dev, uint64_t n_query_positions, uint64_t query_start,
                                  uint64_t n_kv_positions, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                  float scale, void* stream);

/* Command::SigmoidGate of the recorded IR (crates/beholdd-backend/src/execution.rs:441-445, 1425-1441):
 * out[i] = in[i] * sigmoid(gate[i]). */
int32_t bhd_sigmoid_gate(bhd_ctx* ctx, float* out_dev, const float* in_dev, const float* gate_dev, uint64_t n, void* stream);

/* Grows the context's workspace to at least n_bytes now. Nothing may be allocated while a stream is being captured
 * into a CUDA graph, so a host that records graphs reserves the largest workspace its commands need first. */
int32_t bhd_workspace_reserve(bhd_ctx* ctx, uint64_t n_bytes);
/* The workspace's current size in bytes. The workspace is only ever replaced by a larger one, so a graph captured when
 * this returned v is valid exactly as long as it still returns v. */
uint64_t bhd_workspace_bytes(const bhd_ctx* ctx);

/* The same operators for a decode step replayed as a CUDA graph, where the position may not be a launch parameter:
 * it is read from device memory (*pos_dev, an int32 the host or a kernel advances between replays). No counterpart in
 * the reference, which records one batch per position (execution.rs:1093-1099).
 *   bhd_rope_at                  rotates n_vectors vectors of the one position *pos_dev with row *pos_dev of the tables
 *                                [max_positions][n_pairs]
 *   bhd_store_row_at             dst[*pos_dev][0 .. row_floats) = src (appends a key or value row to its cache)
 *   bhd_incremental_attention_at one query at position *pos_dev against cache rows 0 .. *pos_dev; max_positions sizes
 *                                the score buffer
 *   bhd_qk_norm_rope_store_at    what a decode step does between the projections and attention in one launch: per-head
 *                                RMSNorm of q [n_heads][head_dim] and k [n_kv_heads][head_dim] in place (null weights:
 *                                plain normalisation), rope of both with row *pos_dev of the tables, k and v appended to
 *                                their caches [max_positions][n_kv_heads][head_dim] at *pos_dev; same bits as the
 *                                separate calls
 * A position outside [0, max) is reported through the status word and the kernel writes nothing. */
int32_t bhd_qk_norm_rope_store_at(bhd_ctx* ctx, float* q_dev, float* k_dev, const float* v_dev, const float* q_norm_dev,
                                  const float* k_norm_dev, const float* cos_table_dev, const float* sin_table_dev, float* k_cache_dev,
                                  float* v_cache_dev, const int32_t* pos_dev, uint64_t max_positions, uint32_t n_heads, uint32_t n_kv_heads,
                                  uint32_t head_dim, float eps, int32_t layout, void* stream);
int32_t bhd_rope_at(bhd_ctx* ctx, float* x_dev, const float* cos_table_dev, const float* sin_table_dev, const int32_t* pos_dev,
                    uint32_t n_vectors, uint32_t n_pairs, int32_t layout, int32_t inverse, void* stream);
int32_t bhd_store_row_at(bhd_ctx* ctx, float* dst_dev, const float* src_dev, const int32_t* pos_dev, uint64_t row_floats,
                         uint64_t max_rows, void* stream);
int32_t bhd_incremental_attention_at(bhd_ctx* ctx, float* out_dev, const float* q_dev, const float* k_cache_dev,
                                     const float* v_cache_dev, const int32_t* pos_dev, uint64_t max_positions, uint32_t n_heads,
                                     uint32_t n_kv_heads, uint32_t head_dim, float scale, void* stream);

/* Embedding lookup (forward.rs:954-972): rows ids[i] of `table` decoded to f32, out [n_ids][cols]; an id outside the
 * table is reported through the status word. */
int32_t bhd_embedding_rows(bhd_ctx* ctx, const bhd_weight* table, const int32_t* ids_dev, uint64_t n_ids, float* out_dev,
                           void* stream);

/* ---- several GPUs of one node (one process per GPU); the reference is single-process and has no counterpart ----
 *
 * Peer-visible buffers: allocated (and zeroed) by their owner, exported as 64 opaque bytes, opened by the
 * other ranks' processes, which then address them with ordinary loads and stores over NVLink. How the 64
 * bytes travel between the processes is the host's business. Close every opened mapping before its owner
 * frees the buffer. */
int32_t bhd_peer_alloc(bhd_ctx* ctx, uint64_t n_bytes, void** out_dev, uint8_t* handle64);
int32_t bhd_peer_open(bhd_ctx* ctx, const uint8_t* handle64, void** out_dev);
int32_t bhd_peer_close(bhd_ctx* ctx, void* dev);
int32_t bhd_peer_free(bhd_ctx* ctx, void* dev);

/* The routed layer with the experts split over `world` ranks (at most 8): rank r holds experts
 * [r * n_experts / world, (r + 1) * n_experts / world) as the slabs of its gate/up/down weights, the router is
 * replicated, and every rank owns `n_positions` positions per call (the same number on every rank). The ranks
 * exchange rows through peer memory inside the kernels (dispatch: every position to every rank; return: each
 * route's weighted output row straight from the down-projection epilogue into the owner's buffer), flags with a
 * bounded wait order the steps, and the owner adds the returned rows in selection order
 * (forward.rs:1385-1398): the result equals bhd_moe_layer over all world * n_positions positions on one GPU,
 * bit for bit. No host synchronisation, no collective library; the call can be captured into a CUDA graph.
 *   bhd_ep_create   allocates this rank's exchange block for at most `max_positions` positions per rank and
 *                   returns its 64-byte handle;
 *   bhd_ep_connect  takes the handles of all ranks in rank order (world * 64 bytes; the own entry is ignored);
 *   bhd_ep_layer    one layer; all ranks must call it the same number of times with the same n_positions. A
 *                   rank that never arrives makes the others' waits run out (about a second), which they
 *                   report through BHD_ERR_DEVICE_STATUS at the next bhd_check_status. */
typedef struct bhd_ep bhd_ep;
int32_t bhd_ep_create(bhd_ctx* ctx, uint32_t rank, uint32_t world, uint32_t n_experts, uint32_t dim, uint32_t top_k,
                      uint32_t max_positions, bhd_ep** out_ep, uint8_t* handle64);
int32_t bhd_ep_connect(bhd_ep* ep, const uint8_t* handles);
int32_t bhd_ep_layer(bhd_ep* ep, const bhd_weight* router, const bhd_weight* gate_exps, const bhd_weight* up_exps,
                     const bhd_weight* down_exps, const float* x_dev, float* y_dev, uint64_t n_positions,
                     int32_t* experts_dev, float* weights_dev, int32_t* counts_dev, int32_t accumulate, void* stream);
int32_t bhd_ep_destroy(bhd_ep* ep);

/* One large projection with its rows split over `world` ranks: rank r holds whole packed rows
 * [r * rows / world, (r + 1) * rows / world) as `shard`; every rank has the full x and ends with the full
 * y [batch x rows] in y_dev. The slices travel through peer memory inside one kernel after the matvec (stores
 * into every rank's copy, flags, bounded wait); no row's summation crosses a GPU, so y does not depend on
 * `world` beyond the kernel the shard's shape selects. Capturable into a CUDA graph. All ranks must make the
 * same sequence of calls. Device::matvec is the reference's form (crates/beholdd-backend/src/lib.rs:182-198). */
typedef struct bhd_rowsplit bhd_rowsplit;
int32_t bhd_rowsplit_create(bhd_ctx* ctx, uint32_t rank, uint32_t world, uint32_t rows, uint32_t max_batch,
                            bhd_rowsplit** out_rs, uint8_t* handle64);
int32_t bhd_rowsplit_connect(bhd_rowsplit* rs, const uint8_t* handles);
int32_t bhd_rowsplit_matvec(bhd_rowsplit* rs, const bhd_weight* shard, uint64_t slab, const float* x_dev, float* y_dev,
                            uint32_t batch, float scale, void* stream);
int32_t bhd_rowsplit_destroy(bhd_rowsplit* rs);

/* The whole routed feed-forward of one layer (forward.rs:1299-1407): bhd_moe_route then
 * bhd_moe_experts over all experts. The operator shape follows the reference's only
 * resident routed-MoE entry point, VulkanDevice::routed_moe_bf16 / RoutedMoeProgram::
 * execute_batch (crates/beholdd-backend/src/vulkan.rs:1792-1799, 2699-2706), with Q8_0
 * experts and routing done on the device. */
int32_t bhd_moe_layer(bhd_ctx* ctx, const bhd_weight* router, const bhd_weight* gate_exps, const bhd_weight* up_exps,
                      const bhd_weight* down_exps, const float* x_dev, float* y_dev, uint64_t n_positions,
                      uint32_t top_k, int32_t* experts_dev, float* weights_dev, int32_t* counts_dev,
                      int32_t accumulate, void* stream);

/* The routed layer through host buffers: x [T x dim] in, y [T x dim] (+ routing) out. */
int32_t bhd_moe_layer_host(bhd_ctx* ctx, const bhd_weight* router, const bhd_weight* gate_exps,
                           const bhd_weight* up_exps, const bhd_weight* down_exps, const float* x_host,
                           float* y_host, uint64_t n_positions, uint32_t top_k, int32_t* experts_host,
                           float* weights_host, int32_t* counts_host, int32_t accumulate);

/* Synchronise `stream` and read the context's device status word: BHD_OK, or
 * BHD_ERR_DEVICE_STATUS with the detail in bhd_last_error_message (NaN fed to softmax,
 * an out-of-range expert id, a bounded wait that gave up). Clears the word. */
int32_t bhd_check_status(bhd_ctx* ctx, void* stream);

/* Test hook, no counterpart in the reference. Every wait inside the kernels is bounded; this lets a
 * test watch one run out without any fault: `spin_limit` (0 = default) replaces the number of polls
 * the single-vector decode matvec makes before it gives up, and a non-zero `drop_one_copy` makes the
 * next such matvec leave one weight copy unrequested, so that one warp's wait cannot complete. The
 * kernel then sets the status word, lets the copies it did request land, and returns normally
 * (the rows of that warp's tile are wrong, which is why the status word is set); the context
 * stays usable. bhd_check_status reports BHD_ERR_DEVICE_STATUS once. */
int32_t bhd_debug_wait_test(bhd_ctx* ctx, uint32_t spin_limit, uint32_t drop_one_copy);

/* Tuning hook, no counterpart in the reference. Keys:
 *   BHD_OPTION_MOE_TC_MIN_CLASS  smallest expert-group size class the tensor-core (tcgen05) grouped kernel takes
 *                                in bhd_moe_experts / bhd_moe_layer / bhd_ep_layer: 2 = groups of 9+ routes,
 *                                3 = 17+, 4 = 33+; smaller groups run on the integer kernel. 0 (default): integer
 *                                kernels only (experts are then cut into groups of at most 32 routes).
 *   BHD_OPTION_MOE_TC_PLAIN      1: those groups run with singly rounded fp16 operands staged in shared memory
 *                                (faster, about 1e-3 less accurate); 0: exact hi + lo operands (default).
 *   BHD_OPTION_GEMM_IMPL         prefill matmul: 0 = the library's choice (persistent CTA pairs from 256 tokens on, one CTA
 *                                per tile below), 1 = one CTA per tile, 2 = one CTA per tile with the weight operand in
 *                                tensor memory, 3 = persistent CTA pairs (tcgen05 cta_group::2) on 256-token tiles,
 *                                4 = persistent single CTAs, 5 = CTA pairs on 512-token tiles with two MMA issuers.
 *   BHD_OPTION_ROUTER_TILING     router-logits kernel for more than 64 positions: 0 = 32 positions per CTA and 3
 *                                tiles in flight, 1 = 32 and 5, 2 = 16 and 6, 3 = 8 and 7 (the small-batch tiling).
 *   BHD_OPTION_PLAIN_LAUNCHES    1: the short kernels of a layer (norms, rope, attention, routing, expert staging and
 *                                combination) start only after the kernel before them has ended; 0 (default): they are
 *                                launched as programmatic dependents, scheduled while their predecessor drains, and wait
 *                                for it on the device before touching memory. Results are identical. */
#define BHD_OPTION_MOE_TC_MIN_CLASS 1u
#define BHD_OPTION_MOE_TC_PLAIN 2u
#define BHD_OPTION_GEMM_IMPL 3u
#define BHD_OPTION_ROUTER_TILING 5u
#define BHD_OPTION_PLAIN_LAUNCHES 6u
int32_t bhd_debug_option(bhd_ctx* ctx, uint32_t key, uint32_t value);

/* Test hook, no counterpart in the reference: out[i] = the library's expf(in[i]), the function the
 * router softmax uses on the device. The reference calls the host libm (Rust f32::exp,
 * crates/beholdd-kernel/src/vecops.rs:70-87); expert selection is the CPU's only if both give
 * the same floats, which a test checks over a sweep of arguments. */
int32_t bhd_debug_expf(bhd_ctx* ctx, const float* in_dev, float* out_dev, uint64_t n, void* stream);

/* Benchmark helpers, no counterpart in the reference: seeded synthetic tensors generated on the device.
 * bhd_debug_fill_q8_0 writes n_slabs * blocks_per_slab Q8_0 blocks (34 bytes each; an f16 scale uniform in
 * [1e-3, 1e-2] and 32 int8 quants uniform in [-127, 127]), byte for byte what the host generator of this
 * package produces for (seed, stream0 + slab * stream_step); bhd_debug_fill_normal writes f32 N(0, std). */
int32_t bhd_debug_fill_q8_0(bhd_ctx* ctx, uint8_t* out_dev, uint64_t blocks_per_slab, uint64_t n_slabs, uint64_t seed,
                            uint64_t stream0, uint64_t stream_step, void* stream);
int32_t bhd_debug_fill_normal(bhd_ctx* ctx, float* out_dev, uint64_t n, uint64_t seed, uint64_t stream, float std,
                              void* cuda_stream);

/* How many kernels this library has launched on the context since it was created. */
uint64_t bhd_launch_count(const bhd_ctx* ctx);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* BEHOLDD_B200_H */
