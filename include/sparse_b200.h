/*
 * sparse_b200 — C ABI of the B200 (sm_100a) MoE-layer hot path.
 *
 * The reference project is pure Python and has no foreign-function interface;
 * every entry point below replaces a span of Python/ATen calls inside
 * `DistributedSparseMoeBlock` (file utils/eval_core.py of the reference), named
 * in the comment above it.  A host program binds these symbols with ctypes
 * (or cgo/JNI/N-API, the signatures are plain C) and passes raw device
 * pointers, sizes and a CUDA stream.
 *
 * Conventions
 *   - every function returns 0 on success and a negative SB_E_* code on
 *     failure; `sb_last_error_string()` describes the last failure of the
 *     calling thread;
 *   - nothing here allocates or frees device memory, synchronises the host
 *     with the device, or keeps a pointer after the call returns, unless the
 *     function's comment says otherwise;
 *   - `stream` is a `cudaStream_t` passed as `void *` (NULL = legacy default);
 *   - activations and weights are bf16, row-major, nn.Linear layout
 *     ([out_features, in_features]); indices are int32;
 *   - all device pointers must be 16-byte aligned; matrices handed to the
 *     grouped GEMM must be 128-byte aligned.
 */
#ifndef SPARSE_B200_H_
#define SPARSE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_OK                 0
#define SB_E_INVALID_ARG     -1
#define SB_E_WORKSPACE       -2   /* workspace too small */
#define SB_E_CUDA            -3   /* a CUDA runtime/driver call failed */
#define SB_E_UNSUPPORTED     -4   /* shape outside what the kernels cover */
#define SB_E_DEVICE_TIMEOUT  -5   /* a bounded device-side wait gave up */

#define SB_DTYPE_BF16 0
#define SB_DTYPE_F32  1

#define SB_COPY_HOST_TO_DEVICE 0   /* pinned host -> cache slot */
#define SB_COPY_PEER_TO_DEVICE 1   /* peer GPU    -> cache slot */
#define SB_COPY_DEVICE_LOCAL   2

/* Rows per GEMM tile; `sb_permute` cuts every expert segment into tiles of
 * this many rows and the grouped GEMM consumes that table. */
#define SB_TILE_M 128

/* ABI version of this header (bumped on any signature change). */
int32_t sb_abi_version(void);

/* Text for the calling thread's last non-zero status. */
const char *sb_last_error_string(void);

/* Number of SMs of the current device (grid sizing on the host side). */
int32_t sb_device_sm_count(void);

/* Once per device, before the first sb_moe_layer_forward on it: creates the
 * layer driver's side stream and events for `device` (the only resources the
 * library owns; they live until the process exits).  Idempotent and
 * thread-safe; no entry point creates them lazily.  The reference has no
 * counterpart: its block creates its prefetch and EPIPE streams in __init__
 * (utils/eval_core.py:4939-4968). */
int32_t sb_init(int32_t device);

/* Process-wide scheduling knobs of the kernels, read at every launch; results
 * are bit-identical under every setting, only the time changes.
 *   "sched"          0 = walk the tile table in order with a fixed stride
 *                        (default), 1 = rank the row chunks by the size of
 *                        their expert and deal them out boustrophedon, 2 = as
 *                        1 with odd CTA pairs walking their list backwards
 *   "dense_group"    row chunks per raster block of a dense (shared-expert)
 *                    pass, 1..64 (default 1)
 *   "kslabs"         K steps (64 deep) of a full tile per pipeline stage where
 *                    the caller leaves the depth open: 2 (default, half the
 *                    barrier round trips) or 1
 *   "dispatch_ctas"  CTAs per SM of sb_ep_dispatch, 1..8 (default 1: the kernel
 *                    runs beside the shared expert's GEMM, and fewer resident
 *                    warps leave that GEMM its issue slots)
 *   "router_overlap" 1 = sb_moe_layer_forward runs the router beside the shared
 *                    expert's gate/up pass (default), 0 = in front of it
 * Unknown keys and out-of-range values are SB_E_INVALID_ARG.  No counterpart in
 * the reference (its knobs are environment variables read by the block). */
int32_t sb_set_tuning(const char *key, int32_t value);

/* Rows per tile of the tile tables this library writes and consumes (256: the
 * token extent of one tensor-core tile of a CTA pair), and whether the gate/up
 * slab `w13` is expected with gate and up rows interleaved (row 2j = gate_j,
 * row 2j+1 = up_j; always 1) instead of stacked (I gate rows, then I up rows). */
int32_t sb_tile_rows(void);
int32_t sb_w13_interleaved(void);

/*
 * Router: logits = x . Wg^T (+ bias) rounded to the model dtype, softmax in
 * fp32, top-k (larger probability first, then smaller expert id), optional
 * renormalisation, weights cast to the model dtype.  Optionally also the
 * shared expert's scalar gate sigmoid(x . wsg) in the model dtype.
 * Replaces `_routing_router` (utils/eval_core.py:9519-9520, 9591-9595) and the
 * gate half of `_shared_expert_forward` (utils/eval_core.py:9461-9462).
 *
 *   x            [T,H]   model dtype (bf16 or f32 per `dtype`)
 *   wg           [E,H]   same dtype
 *   bias         [E]     f32 values already rounded to the model dtype, or NULL
 *   w_shared_gate[H]     same dtype as x, or NULL
 *   out_idx      [T,K]   int32
 *   out_w        [T,K]   model dtype
 *   fp32_logits  0: logits are rounded to the model dtype before the softmax
 *                (Qwen-MoE gate, an nn.Linear in the model dtype);
 *                1: logits stay fp32 (DeepSeek-V2 gate, which casts its inputs
 *                to fp32; that gate is third-party remote code the reference
 *                only calls, utils/eval_core.py:9503-9517)
 *   out_logits   [T,E]   model dtype (f32 if fp32_logits), or NULL
 *   out_shared_scale [T] model dtype, or NULL (required iff w_shared_gate)
 * Limits: H % 8 == 0, 1 <= K <= 8, K <= E <= 256.
 */
int32_t sb_router_topk(const void *x, const void *wg, const float *bias,
                       const void *w_shared_gate, int32_t T, int32_t H, int32_t E,
                       int32_t K, int32_t renorm, int32_t dtype, int32_t fp32_logits,
                       int32_t *out_idx, void *out_w, void *out_logits,
                       void *out_shared_scale, void *stream);

/* Same stage, but starting from given model-dtype logits [T,E] (softmax +
 * top-k only).  Used to check the tie rule in isolation. */
int32_t sb_softmax_topk(const void *logits, int32_t T, int32_t E, int32_t K,
                        int32_t renorm, int32_t dtype, int32_t *out_idx,
                        void *out_w, void *stream);

/* Bytes of scratch `sb_permute` needs for `n_items` items over E experts. */
size_t sb_permute_workspace_bytes(int32_t n_items, int32_t E);

/* Number of int32 the tile table needs for `n_items` items over E experts. */
size_t sb_tile_table_ints(int32_t n_items, int32_t E);

/*
 * Expert-sorted permutation: stable counting sort of the flat items by expert
 * id, gather of the activation rows into that order, and the row-tile table
 * the grouped GEMM walks.  Item i reads source row i / items_per_row.
 * Replaces the expand/argsort/gather/bincount sequence of the reference
 * (utils/eval_core.py:14873-14882) and the local re-sort by expert
 * (utils/eval_core.py:13240-13253); the EP=1 loop of `_experts_world1_exact`
 * (utils/eval_core.py:14690-14700) needs the same grouping.
 *
 *   x              [n_items/items_per_row, H] bf16
 *   item_expert    [n_items] int32 in [0,E); a negative id drops the item
 *   item_scale     [n_items] bf16 route weight per item, or NULL
 *   ws             scratch of sb_permute_workspace_bytes()
 *   out_rows       [n_items,H] bf16, rows in expert-sorted order; NULL = sort
 *                  only, no rows are gathered (x may then be NULL too)
 *   expert_offsets [E+1] int32
 *   slot_of_item   [n_items] int32 (-1 for dropped items)
 *   item_of_slot   [n_items] int32
 *   slot_scale     [n_items] bf16 = item_scale[item_of_slot], or NULL
 *   tile_table     [sb_tile_table_ints()] int32: [0] = number of row tiles,
 *                  then from int 4 on one (expert, row_begin, row_end, 0)
 *                  quadruple per tile, tiles of one expert adjacent.
 */
int32_t sb_permute(const void *x, const int32_t *item_expert, const void *item_scale,
                   int32_t n_items, int32_t items_per_row, int32_t H, int32_t E,
                   void *ws, size_t ws_bytes, void *out_rows, int32_t *expert_offsets,
                   int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale,
                   int32_t *tile_table, void *stream);

/*
 * sb_permute for callers that cannot hand over scratch memory.  (No counterpart
 * in the reference: it has no allocation-free mode.)
 *
 * Some hosts of this library must not allocate device memory on the serving
 * path: a decode loop in which cudaMalloc would stall every stream of the
 * device, or a process whose memory pool (PyTorch's caching allocator, a
 * framework arena) already owns all of HBM so that a raw allocation fails or
 * fragments it.  sb_permute asks such a caller for a workspace it may have no
 * way to get.  This variant takes none: the per-chunk histograms live in a
 * 512 KiB array inside the library's device image, which every GPU that loads
 * the library holds until the process exits.  Inputs and outputs are still the
 * caller's; the call itself runs no cudaMalloc, cudaFree or other allocating
 * routine.  Results are identical to sb_permute.
 *
 * Limit: ceil(n_items/128) * E <= 131072 (e.g. 262144 items over 64 experts);
 * larger problems are refused with SB_E_WORKSPACE and a message.
 * The first call on each device looks up the array's device address (with that
 * device current); make that first call before starting any stream capture.
 * All calls on a device share the one array and nothing in it needs clearing
 * between calls, but two calls that overlap on the GPU (different streams)
 * race on it: keep calls on one stream or order them with events.
 */
int32_t sb_permute_noalloc(const void *x, const int32_t *item_expert,
                           const void *item_scale, int32_t n_items,
                           int32_t items_per_row, int32_t H, int32_t E,
                           void *out_rows, int32_t *expert_offsets,
                           int32_t *slot_of_item, int32_t *item_of_slot,
                           void *slot_scale, int32_t *tile_table, void *stream);

/*
 * Grouped SwiGLU expert MLP on the tensor cores (tcgen05, TMEM accumulators,
 * TMA-fed): for every row tile of `tile_table`
 *     h   = bf16( bf16(silu(bf16(x.Wg^T))) * bf16(x.Wu^T) )
 *     out = bf16( bf16(h.Wd^T) * row_scale )
 * with the same rounding points as the reference's three `F.linear` calls and
 * the `* cur_w` that follows (utils/eval_core.py:11787-11790, 11765).
 *
 *   rows          [R_cap,H] bf16, expert-sorted (out_rows of sb_permute)
 *   tile_table    as written by sb_permute; NULL = one dense group of
 *                 `dense_rows` rows using weight slot 0 (shared expert)
 *   w13           [S, 2*I, H] bf16 weight slab, per slot gate and up rows
 *                 interleaved (row 2j = gate_j, row 2j+1 = up_j)
 *   w2            [S, H, I]   bf16 weight slab
 *   slot_of_expert[E] int32 expert id -> weight slot, or NULL for identity;
 *                 -2 = skip this expert's tiles in this launch (they are left
 *                 for a later launch, e.g. once its weights have arrived);
 *                 any other negative value, or one >= S, raises status 2
 *                 and the expert's rows are left uncomputed (never run
 *                 with another expert's weights)
 *   row_scale     [R_cap] bf16 per-row factor, or NULL for none
 *   hbuf          [R_cap, I] bf16 scratch for the intermediate
 *   out           [R_cap, H] bf16
 *   status        device int32; set non-zero if a bounded wait gave up
 * Limits: H % 64 == 0, I % 64 == 0, H,I >= 64.
 */
int32_t sb_grouped_swiglu(const void *rows, const int32_t *tile_table,
                          int32_t dense_rows, const void *w13, const void *w2,
                          const int32_t *slot_of_expert, const void *row_scale,
                          int32_t R_cap, int32_t H, int32_t I, int32_t S,
                          void *hbuf, void *out, int32_t *status, void *stream);

/* The routed part of sb_decode_experts with every result row stored at its own
 * address (`row_dst` uint64 [rows of the tile table], 0 = drop) instead of into
 * a dense output buffer: rows of the local expert sort go straight to the rows
 * of a return buffer that a later sb_combine reads (see
 * sb_ep_exchange_dispatch_local).  Groups of any size (swept 16 rows at a time).
 * `T` is the caller's token count of this step (it selects the same K split,
 * hence the same summation order, as the step's other launches). */
int32_t sb_decode_experts_to(const void *x, const int32_t *item_of_slot, int32_t items_per_row,
                             const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                             const void *w2, const void *row_scale, int32_t H, int32_t I, int32_t n_slots,
                             void *hbuf, const uint64_t *row_dst, int32_t T, int32_t *status, void *stream);

/* sb_grouped_swiglu restricted to one of its two passes: `passes` 1 = gate/up +
 * SwiGLU into `hbuf`, 2 = down projection from `hbuf` into `out`, 3 = both.
 * Lets a caller put other work (a transfer on another stream) between the
 * passes of the shared expert.  `stages` names the kernel's shared-memory
 * pipeline: 0 = the library's choice (three 64 KB stages of two K steps each),
 * 2..6 = that many 36 KB stages of one K step, -1 = whichever layout leaves an
 * SM enough shared memory and registers for one CTA of sb_router_topk launched
 * on another stream, which is how the router is hidden behind the shared
 * expert's gate/up pass. */
int32_t sb_grouped_swiglu_passes(const void *rows, const int32_t *tile_table, int32_t dense_rows,
                                 const void *w13, const void *w2, const int32_t *slot_of_expert,
                                 const void *row_scale, int32_t R_cap, int32_t H, int32_t I, int32_t S,
                                 void *hbuf, void *out, int32_t passes, int32_t stages, int32_t *status,
                                 void *stream);

/* Token counts up to this use the weight-streaming kernels below inside
 * sb_moe_layer_forward instead of the tensor-core grouped GEMM. */
#define SB_DECODE_MAX_TOKENS 16

/*
 * Decode-sized expert MLPs (a few tokens against whole expert matrices): the
 * same arithmetic as sb_grouped_swiglu for the routed groups of `tile_table`
 * AND the shared expert, as two weight-streaming launches (each warp streams
 * 16 weight rows through registers into warp-level MMAs).  Replaces the same
 * reference spans as sb_grouped_swiglu (utils/eval_core.py:11767-11793, 11765,
 * 9455-9463) for decode steps.  Routed token rows are read through
 * `item_of_slot` (row = item / items_per_row of `x`), so sb_permute may be
 * called with out_rows == NULL; with item_of_slot == NULL the rows of `x` are
 * taken as already expert-sorted (row = position in the tile table's range).
 *
 *   x [T,H]; hbuf [n_items, I]; y [n_items, H]; shared_h [T, I_shared];
 *   shared_out [T, H]; row_scale [n_items] and shared_scale [T] bf16 or NULL;
 *   shared_w13 / shared_w2 NULL = no shared expert; tile_table NULL = no
 *   routed groups.  w13 row order as sb_w13_interleaved() says.
 * Limits: H, I, I_shared multiples of 32; T <= SB_DECODE_MAX_TOKENS when there
 * is a shared expert; routed groups of more than SB_DECODE_MAX_TOKENS rows are
 * left untouched (sb_grouped_swiglu_mixed finishes those).
 */
int32_t sb_decode_experts(const void *x, const int32_t *item_of_slot, int32_t items_per_row,
                          const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                          const void *w2, const void *row_scale, int32_t H, int32_t I, int32_t n_slots,
                          void *hbuf, void *y, const void *shared_w13, const void *shared_w2,
                          const void *shared_scale, int32_t I_shared, int32_t T, void *shared_h,
                          void *shared_out, int32_t *status, void *stream);

/*
 * Expert MLPs for FEW rows per expert (decode-sized expert-parallel steps, where
 * a rank receives a handful of rows for each of its experts): the routed groups
 * of `tile_table` over already expert-sorted `rows`, plus (optionally) the shared
 * expert over the rank's own `shared_x` [T,H], in the two weight-streaming
 * launches of sb_decode_experts.  Groups are swept 16 rows at a time.
 * `max_group_rows` is the caller's upper bound on the rows of any group (for an
 * expert-parallel decode step: ep * tokens per rank); with 0 (unknown) only
 * groups of at most SB_DECODE_MAX_TOKENS rows are streamed and the tensor-core
 * kernel of sb_grouped_swiglu is launched for the rest.  Results as
 * sb_grouped_swiglu up to fp32 summation order.  With `row_dst` (see
 * sb_ep_resolve_return; may be NULL) routed result rows go to those addresses
 * instead of `out`.  Replaces
 * `_plain_ep_compute_segment` over the received segments and
 * `_shared_expert_forward` (utils/eval_core.py:11700-11765, 13156-13372,
 * 9455-9463) in decode.
 */
int32_t sb_grouped_swiglu_mixed(const void *rows, const int32_t *tile_table, const void *w13, const void *w2,
                                const int32_t *slot_of_expert, const void *row_scale, int32_t R_cap,
                                int32_t H, int32_t I, int32_t S, void *hbuf, void *out,
                                int32_t max_group_rows, const void *shared_x, const void *shared_w13,
                                const void *shared_w2, const void *shared_scale, int32_t I_shared, int32_t T,
                                void *shared_h, void *shared_out, const uint64_t *row_dst, int32_t *status,
                                void *stream);

/*
 * Decode-sized routing (T <= SB_DECODE_MAX_TOKENS, bf16): sb_router_topk and the
 * sort half of sb_permute in two launches -- one warp per (token, router row),
 * then softmax/top-k and the stable expert sort of the T*K items in a single
 * CTA.  Same bits as sb_router_topk + sb_permute.  Replaces
 * utils/eval_core.py:9519-9520, 9591-9595 and 14873-14882 for decode steps.
 *   ws: T*E fp32 scratch; slot_scale [>= T*K] bf16 (route weight per sorted row);
 *   the remaining outputs as in sb_router_topk / sb_permute.
 */
int32_t sb_route_decode(const void *x, const void *w_router, const float *router_bias, const void *w_shared_gate,
                        int32_t T, int32_t H, int32_t E, int32_t K, int32_t renorm, int32_t fp32_logits,
                        float *ws, int32_t *out_idx, void *out_w, void *out_logits, void *out_shared_scale,
                        int32_t *expert_offsets, int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale,
                        int32_t *tile_table, void *stream);

/*
 * Un-permute and combine: for each token add its K expert rows in ascending
 * expert id, every add rounding to bf16, then add the shared expert's row.
 * Replaces the unsort + `combine_expert_outputs` + final add
 * (utils/eval_core.py:15058-15060, 523-538, 16547).
 *
 *   rows_out     [n_items,H] bf16 expert-sorted rows (already route-weighted)
 *   slot_of_item [T*K] int32 (-1 = contributes nothing)
 *   idx          [T,K] int32 expert ids (ordering key)
 *   shared_out   [T,H] bf16 or NULL
 *   out          [T,H] bf16
 * Limits: H % 8 == 0, K <= 8.
 */
int32_t sb_combine(const void *rows_out, const int32_t *slot_of_item,
                   const int32_t *idx, const void *shared_out, int32_t T, int32_t H,
                   int32_t K, void *out, void *stream);

/* sb_combine that also applies the shared expert's scalar gate: the row added is
 * bf16(shared_out[t] * shared_scale[t]) (`shared_scale` [T] bf16 as written by
 * sb_router_topk, NULL = as sb_combine).  Same bits as letting the shared
 * expert's down pass scale its rows (row_scale of sb_grouped_swiglu), but that
 * pass then needs nothing from the router
 * (utils/eval_core.py:9455-9463: gate multiply, then the add). */
int32_t sb_combine_gated(const void *rows_out, const int32_t *slot_of_item, const int32_t *idx,
                         const void *shared_out, const void *shared_scale, int32_t T, int32_t H, int32_t K,
                         void *out, void *stream);

/*
 * Asynchronous copy of one expert payload into a preallocated cache slot on
 * `stream` (pinned host memory, a peer GPU, or this GPU).  Callable from a
 * second host thread while kernels are launched on other streams; `device` is
 * made current for the call.  Replaces the `.to(device, non_blocking=True)`
 * weight copies (utils/eval_core.py:11379-11380, 11427-11429, 9975-9982,
 * 11626-11633; utils/rs_overlap.py:245-248).
 */
int32_t sb_slot_copy_async(void *dst_slot, const void *src, size_t bytes,
                           int32_t kind, int32_t device, void *stream);

/* ------------------------------------------------------------------------
 * Expert parallelism over NVLink peer memory (one process per GPU).
 * Together these replace `_experts_ep_group`'s dispatch and return halves:
 * expand/argsort/bincount, the count all-to-all with its two host syncs, the
 * three payload all-to-alls, the local re-sort, the return all-to-all and the
 * unsort (utils/eval_core.py:14865-14900, 14999-15019, 13240-13253,
 * 15048-15060), and `_resolve_dest_for_flat_experts` (6736-6769) through the
 * `owner` table.
 *
 * Set-up calls (these DO allocate / synchronise; call them once, outside the
 * serving loop):
 *   sb_peer_alloc   zero-filled device buffer that can be exported
 *   sb_ipc_export   64-byte handle of such a buffer, to send to the other ranks
 *   sb_ipc_import   peer's buffer mapped into this process (peer access enabled)
 * Every rank then holds, per shared buffer, an array of `ep` device pointers
 * indexed by rank (its own entry is the local pointer); these arrays are HOST
 * arrays, passed by value into the kernels.
 * ------------------------------------------------------------------------ */
int32_t sb_peer_alloc(size_t bytes, void **out_ptr);
int32_t sb_peer_free(void *ptr);
int32_t sb_ipc_export(const void *ptr, void *handle64);
int32_t sb_ipc_import(const void *handle64, void **out_ptr);
int32_t sb_ipc_close(void *ptr);

/* Write this rank's per-expert item counts (differences of `local_offsets`
 * [E+1], as produced by sb_permute) into row `rank` of every rank's counts
 * matrix int32 [ep][E]. */
int32_t sb_ep_publish_counts(const int32_t *local_offsets, int32_t E, int32_t rank,
                             int32_t ep, void *const *peer_counts, void *stream);

/* Stream-ordered barrier across the ranks: flags are uint32 [ep] per rank in
 * peer memory, `epoch` increases by one per call on every rank.  The wait is
 * bounded (2 s); on expiry `status` (device int32, may be NULL) becomes 3. */
int32_t sb_ep_barrier(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t epoch,
                      int32_t *status, void *stream);

/* The same barrier with the epoch taken from (and advanced in) this rank's own
 * device counter `epoch_counter` (uint32, zero at set-up, touched by nobody
 * else): every rank issues the same sequence of barriers, so the counters move
 * in step and no per-call value is baked into the launch -- a captured CUDA
 * graph of a layer step can be replayed.  Do not mix with sb_ep_barrier on the
 * same flags. */
int32_t sb_ep_barrier_seq(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t *epoch_counter,
                          int32_t *status, void *stream);
/* sb_ep_barrier_seq with the wait limit given by the caller (nanoseconds of the
 * device's global timer, > 0) instead of the default 2 s: a host that polls
 * peer liveness can keep a lost rank from holding the stream for seconds.  On
 * expiry `status` becomes 3, the kernel returns and the context stays usable.
 * The reference's counterpart is the process-group timeout of its collectives
 * (utils/eval_core.py:7041-7056). */
int32_t sb_ep_barrier_timed(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t *epoch_counter,
                            uint64_t limit_ns, int32_t *status, void *stream);

/* From the complete counts matrix: where this rank's items of each expert start
 * in the destination's receive buffer (`dst_base` [E]), and this rank's own
 * receive-side segments (`recv_offsets` [E+1], tile table as in sb_permute,
 * sized by sb_tile_table_ints(recv_cap, E)).  `owner` is int32 [ep][E]:
 * owner[s][e] = rank that executes expert e for tokens on rank s (identical
 * rows for plain ownership; different rows when experts are replicated, as in
 * the reference's dest_rank_table, utils/eval_core.py:672-717).  Receive
 * buffers are laid out by expert id, then source rank, then the source's
 * stable item order.  sb_ep_dispatch takes row `rank` of the same table. */
int32_t sb_ep_plan(const int32_t *counts_all, const int32_t *owner, int32_t E, int32_t rank,
                   int32_t ep, int32_t recv_cap, int32_t *dst_base, int32_t *recv_offsets,
                   int32_t *tile_table, void *stream);

/* The whole send side of a decode-sized step as ONE single-CTA launch:
 * sb_ep_publish_counts, barrier, sb_ep_plan, sb_ep_dispatch, barrier ("every
 * rank's rows have landed"); arguments as in those calls, `owner` the full
 * [ep][E] table, two epochs taken from `epoch_counter`.  With `peer_meta`
 * (may be NULL; then `peer_ret`, `row_dst` are unused) the rows carry return
 * addresses and sb_ep_resolve_return is done at the end of the same launch.
 * Meant for at most a few hundred items (one CTA copies the rows). */
int32_t sb_ep_exchange_dispatch(const int32_t *local_offsets, void *const *peer_counts, void *const *peer_flags,
                                uint32_t *epoch_counter, const int32_t *owner, int32_t E, int32_t rank,
                                int32_t ep, int32_t recv_cap, int32_t *dst_base, int32_t *recv_offsets,
                                int32_t *tile_table, const void *x, const int32_t *item_expert,
                                const void *item_scale, const int32_t *slot_of_item, int32_t n_items,
                                int32_t items_per_row, int32_t H, void *const *peer_rows,
                                void *const *peer_scale, int32_t *item_rank, int32_t *item_row,
                                void *const *peer_meta, void *const *peer_ret, int32_t ret_rows,
                                uint64_t *row_dst, int32_t *status, void *stream);

/* sb_ep_exchange_dispatch for a rank that executes some experts it does not own
 * out of its own cache slots ("run locally if the weights are here, else at the
 * owner": the idea of the reference's _light_destinations,
 * utils/eval_core.py:6396-6411).  `local_map` (int32 [E], NULL = none): >= 0
 * for an expert whose items stay here.  Their counts are published as 0, their
 * rows are not sent, `item_rank[i]` = this rank and `item_row[i]` = i, and
 * `local_dst[s]` (uint64 [n_items]) receives, for every row s of the local
 * expert sort, the address of row `item_of_slot[s]` of this rank's own return
 * buffer: what sb_decode_experts takes as `row_dst` to put locally computed
 * rows where the combine expects them.  Needs `peer_meta` (return addresses). */
int32_t sb_ep_exchange_dispatch_local(const int32_t *local_offsets, void *const *peer_counts,
                                      void *const *peer_flags, uint32_t *epoch_counter, const int32_t *owner,
                                      int32_t E, int32_t rank, int32_t ep, int32_t recv_cap, int32_t *dst_base,
                                      int32_t *recv_offsets, int32_t *tile_table, const void *x,
                                      const int32_t *item_expert, const void *item_scale,
                                      const int32_t *slot_of_item, int32_t n_items, int32_t items_per_row,
                                      int32_t H, void *const *peer_rows, void *const *peer_scale,
                                      int32_t *item_rank, int32_t *item_row, void *const *peer_meta,
                                      void *const *peer_ret, int32_t ret_rows, uint64_t *row_dst,
                                      const int32_t *local_map, const int32_t *item_of_slot, uint64_t *local_dst,
                                      int32_t *status, void *stream);

/* Copy every item's activation row and route weight into its row of the
 * owner's receive buffers (`peer_rows[d]` [recv_cap,H] bf16, `peer_scale[d]`
 * [recv_cap] bf16) and remember where it went (`item_rank`, `item_row` [n_items]).
 * `slot_of_item` / `local_offsets` come from sb_permute on the local items.
 * With `peer_meta` (int32 [recv_cap] per rank, may be NULL) every row also
 * carries its return address: (rank << 24) | item index, n_items < 2^24, and
 * `item_row[i]` is then the item's row in this rank's own return buffer (= i)
 * instead of its row at the owner.  Either way an item that was not sent
 * (expert id outside [0,E), no room) has item_rank = item_row = -1. */
int32_t sb_ep_dispatch(const void *x, const int32_t *item_expert, const void *item_scale,
                       const int32_t *slot_of_item, const int32_t *local_offsets,
                       const int32_t *dst_base, const int32_t *owner, int32_t n_items,
                       int32_t items_per_row, int32_t H, int32_t ep, int32_t recv_cap,
                       void *const *peer_rows, void *const *peer_scale, int32_t *item_rank,
                       int32_t *item_row, int32_t rank, void *const *peer_meta, void *stream);

/* Fused compute + return transfer of the routed experts.  sb_ep_resolve_return
 * turns the return addresses of the received rows (`recv_meta`, written by the
 * senders' sb_ep_dispatch) into device addresses of rows in the senders'
 * return buffers `peer_ret[s]` ([ret_rows,H] bf16, item order) as mapped on
 * this GPU; sb_grouped_swiglu_scatter is sb_grouped_swiglu whose down pass
 * stores every result row to that address (a peer store over NVLink when the
 * sender is another GPU) while the GEMM is still running, instead of to a
 * local buffer that the senders read afterwards.  After the next barrier each
 * sender combines its own return buffer with sb_combine (slot_of_item =
 * the `item_row` that sb_ep_dispatch wrote: the item's own index, or -1 for an
 * item that was never sent, which the combine skips).  Replaces the output all-to-all of utils/eval_core.py:15048-15054
 * together with the segment compute of 13156-13372. */
int32_t sb_ep_resolve_return(const int32_t *recv_meta, const int32_t *recv_offsets, int32_t E,
                             void *const *peer_ret, int32_t ep, int32_t ret_rows, int32_t H, int32_t recv_cap,
                             uint64_t *row_dst, void *stream);
/* The alternative to the fused scatter: after a plain sb_grouped_swiglu into the
 * local output buffer `y` [recv_cap,H], copy every received row to its return
 * address (whole rows, 512-byte warp stores).  Runs on a side stream beside the
 * shared expert's down pass, which is how the return transfer is hidden when
 * the fused store pattern would make the down GEMM NVLink-bound. */
int32_t sb_ep_return_rows(const void *y, const uint64_t *row_dst, const int32_t *recv_offsets, int32_t E,
                          int32_t H, int32_t recv_cap, void *stream);
int32_t sb_grouped_swiglu_scatter(const void *rows, const int32_t *tile_table, const void *w13, const void *w2,
                                  const int32_t *slot_of_expert, const void *row_scale, int32_t R_cap,
                                  int32_t H, int32_t I, int32_t S, void *hbuf, const uint64_t *row_dst,
                                  int32_t *status, void *stream);

/* sb_combine with the K rows of a token read from the owners' output buffers
 * (`peer_y[d]` [recv_cap,H] bf16). */
int32_t sb_ep_combine(void *const *peer_y, const int32_t *item_rank, const int32_t *item_row,
                      const int32_t *idx, const void *shared_out, int32_t T, int32_t H,
                      int32_t K, int32_t ep, void *out, void *stream);

/* Everything one single-GPU layer pass needs; all pointers are device
 * pointers owned by the caller. */
typedef struct sb_moe_layer {
  int32_t T, H, E, K, I, I_shared, renorm, n_slots;
  int32_t router_fp32_logits;    /* see sb_router_topk */
  int32_t reserved_;
  const void *x;                 /* [T,H] bf16 */
  const void *router_w;          /* [E,H] bf16 */
  const float *router_bias;      /* [E] or NULL */
  const void *shared_gate_w;     /* [H] bf16 or NULL */
  const void *w13, *w2;          /* routed slabs [S,2I,H], [S,H,I] */
  const int32_t *slot_of_expert; /* [E] or NULL */
  const void *shared_w13, *shared_w2; /* [1,2Is,H], [1,H,Is] or NULL */
  /* outputs */
  void *out;                     /* [T,H] bf16 */
  void *logits;                  /* [T,E] bf16 (f32 if router_fp32_logits) or NULL */
  int32_t *topk_idx;             /* [T,K] */
  void *topk_w;                  /* [T,K] bf16 */
  /* scratch, sized for T*K items */
  void *ws; size_t ws_bytes;     /* sb_moe_layer_workspace_bytes() */
} sb_moe_layer;

/* sizeof(sb_moe_layer) as this library was compiled, so a binding can check
 * its mirror of the struct. */
size_t sb_moe_layer_struct_bytes(void);

size_t sb_moe_layer_workspace_bytes(int32_t T, int32_t H, int32_t E, int32_t K,
                                    int32_t I, int32_t I_shared);

/*
 * One whole single-GPU layer pass: router -> permute -> routed grouped SwiGLU
 * -> shared expert -> combine, without a host sync; ordered on `stream` (with
 * a shared expert, router and sort run on the library's side stream between a
 * fork from and a join back into `stream`, so the call can be captured in a
 * CUDA graph).  Needs sb_init(device) once per device.
 * Replaces `DistributedSparseMoeBlock.forward` at world=1
 * (utils/eval_core.py:16418-16563 with 14690-14721 and 9455-9463).
 * `status` is a device int32 (may be NULL) as in sb_grouped_swiglu.
 */
int32_t sb_moe_layer_forward(const sb_moe_layer *layer, int32_t *status, void *stream);

/*
 * The small kernels of a decode step around the MoE layers (the reference runs
 * these through the Transformers model classes it loads at
 * utils/eval_core.py:17807-17829 and calls once per generated token from the
 * loop at 18464-18607).  All tensors bf16, row-major.
 *
 * sb_add_rmsnorm   residual [T,H] += delta (+ delta2), rounded to bf16 after each
 *                  add and written back (delta NULL: no add, no write-back);
 *                  out = weight * bf16(h * rsqrt(mean(h^2) + eps)).  out NULL:
 *                  only the residual update.
 * sb_rope_append   rotary embedding (pairs (i, i + rope_dim/2) of the first
 *                  rope_dim elements, angle pos * theta^(-2i/rope_dim), cos/sin
 *                  rounded to bf16) on q [T,n_q,dk] in place and on k
 *                  [T,n_kv,dk]; rotated k and v [T,n_kv,dv] are stored into the
 *                  cache rows (seq_of_token[t], pos_of_token[t]) of cache_k
 *                  [B,s_max,n_kv,dk] / cache_v [B,s_max,n_kv,dv].  q_stride,
 *                  k_stride, v_stride: elements between consecutive tokens
 *                  (0 = densely packed), so q, k, v may be column slices of
 *                  one fused projection output.
 * sb_attn_decode   one query per sequence, q [B,n_q,dk] (q_stride elements
 *                  between sequences, 0 = packed), against the first
 *                  seq_lens[b] (device int32) cached positions; softmax in fp32;
 *                  out [B,n_q,dv].  The keys are split `n_split` ways over CTAs
 *                  and merged by a second kernel; ws needs
 *                  sb_attn_decode_workspace_bytes.  Built for (dk,dv) =
 *                  (128,128), (192,128), (64,64).
 */
int32_t sb_add_rmsnorm(void *residual, const void *delta, const void *delta2, const void *weight, float eps,
                       int32_t T, int32_t H, void *out, void *stream);
int32_t sb_rope_append(void *q, const void *k, const void *v, const int32_t *seq_of_token,
                       const int32_t *pos_of_token, int32_t T, int32_t n_q, int32_t n_kv, int32_t dk, int32_t dv,
                       int32_t rope_dim, float theta, int32_t s_max, void *cache_k, void *cache_v, int32_t q_stride,
                       int32_t k_stride, int32_t v_stride, void *stream);
size_t sb_attn_decode_workspace_bytes(int32_t B, int32_t n_q, int32_t dv, int32_t n_split);
int32_t sb_attn_decode(const void *q, int32_t q_stride, const void *cache_k, const void *cache_v,
                       const int32_t *seq_lens, int32_t B, int32_t n_q, int32_t n_kv, int32_t dk, int32_t dv,
                       int32_t s_max, float scale, int32_t n_split, void *ws, size_t ws_bytes, void *out,
                       void *stream);

/* Number of kernels the last sb_moe_layer_forward of this thread launched. */
int32_t sb_last_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SPARSE_B200_H_ */
