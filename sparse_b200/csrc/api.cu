// extern "C" surface of libsparse_b200: argument checks, error text, the
// whole-layer driver and the cache-slot copy.  Declarations and the reference
// spans they replace are in include/sparse_b200.h.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "sb_common.cuh"

namespace sb {

static thread_local char g_err[512] = "";
static thread_local int g_launches = 0;

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int32_t fail(int32_t code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void count_launch(int n) { g_launches += n; }
void reset_launch_count() { g_launches = 0; }

static inline size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Side stream and fork/join events of the layer driver, one set per device,
// created by sb_init.  Holding the mutex over a fork..join enqueue keeps two
// host threads from interleaving their records on the shared events.
struct SideLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, mid = nullptr, join = nullptr;
};
static std::recursive_mutex g_side_mu;
static SideLane g_side[64];

static SideLane *side_lane() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  SideLane &l = g_side[dev];
  return l.stream != nullptr ? &l : nullptr;
}

static int32_t create_side_lane(int dev) {
  std::lock_guard<std::recursive_mutex> lock(g_side_mu);
  SideLane &l = g_side[dev];
  if (l.stream != nullptr) return SB_OK;
  cudaStream_t st = nullptr;
  SB_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
  for (int i = 0; i < 3; ++i) {
    if (cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(ev[j]);
      cudaStreamDestroy(st);
      return fail(SB_E_CUDA, "sb_init: cannot create the layer driver's events");
    }
  }
  l.fork = ev[0]; l.mid = ev[1]; l.join = ev[2];
  l.stream = st;
  return SB_OK;
}

static int env_int(const char *name, int fallback) {
  const char *e = getenv(name);
  return (e && *e) ? atoi(e) : fallback;
}
// Router and sort beside the shared expert's gate/up pass (1, default) or the
// router in front of everything and only the sort beside the shared expert (0).
static std::atomic<int> g_router_overlap{1};
static int router_overlap() { return g_router_overlap.load(std::memory_order_relaxed); }
// Largest batch for which the shared and the routed GEMM share the SMs by grid
// size, and how many CTA pairs the shared expert gets then.
static int split_tokens() {
  static const int v = env_int("SPARSE_B200_SPLIT_TOKENS", 1024);
  return v;
}
static int shared_pairs() {
  static const int v = env_int("SPARSE_B200_SHARED_PAIRS", 16);
  return v;
}

// "Depth" of a GEMM launch that should leave room for a router CTA on every SM
// (the launcher picks the stage layout, see grouped_swiglu_pair.cu).
constexpr int kStagesBesideRouter = -1;

int32_t launch_grouped_swiglu_any(const void *rows, const int32_t *tile_table, int dense_rows,
                                  const void *w13, const void *w2, const int32_t *slot_of_expert,
                                  const void *row_scale, int R_cap, int H, int I, int S, void *hbuf,
                                  void *out, int32_t *status, cudaStream_t stream, int max_pairs = 0,
                                  int passes = 3, int stages = 0) {
  return launch_grouped_swiglu_pair(rows, tile_table, dense_rows, w13, w2, slot_of_expert, row_scale,
                                    R_cap, H, I, S, hbuf, out, status, 0, max_pairs, nullptr, stream, passes,
                                    stages);
}

// Carves the caller's workspace; the same walk gives the required size.
struct LayerScratch {
  char *permute_ws; size_t permute_ws_bytes;
  int32_t *tile_table, *expert_offsets, *slot_of_item, *item_of_slot;
  void *slot_scale, *shared_scale, *xs, *hbuf, *y, *shared_h, *shared_out;
  float *router_ws;
  size_t total;
  int r_cap, t_cap;
};

static LayerScratch carve(char *base, int T, int H, int E, int K, int I, int I_shared) {
  LayerScratch s;
  const size_t al = 1024;
  const int n_items = T * K;
  s.r_cap = (int)up((size_t)(n_items > 0 ? n_items : 1), SB_TILE_M);
  s.t_cap = (int)up((size_t)(T > 0 ? T : 1), SB_TILE_M);
  size_t off = 0;
  auto take = [&](size_t bytes) { char *p = base + off; off += up(bytes, al); return p; };
  s.permute_ws_bytes = sb_permute_workspace_bytes(n_items, E);
  s.permute_ws = take(s.permute_ws_bytes);
  s.tile_table = (int32_t *)take(sb_tile_table_ints(n_items, E) * 4);
  s.expert_offsets = (int32_t *)take((size_t)(E + 1) * 4);
  s.slot_of_item = (int32_t *)take((size_t)s.r_cap * 4);
  s.item_of_slot = (int32_t *)take((size_t)s.r_cap * 4);
  s.slot_scale = take((size_t)s.r_cap * 2);
  s.shared_scale = take((size_t)s.t_cap * 2);
  s.router_ws = (float *)take((size_t)SB_DECODE_MAX_TOKENS * (size_t)E * 4);
  s.xs = take((size_t)s.r_cap * H * 2);
  s.hbuf = take((size_t)s.r_cap * I * 2);
  s.y = take((size_t)s.r_cap * H * 2);
  s.shared_h = I_shared > 0 ? take((size_t)s.t_cap * I_shared * 2) : nullptr;
  s.shared_out = I_shared > 0 ? take((size_t)s.t_cap * H * 2) : nullptr;
  s.total = off;
  return s;
}

// Layer pass above the decode size.  The shared expert's gate/up pass needs
// nothing from the routing and its down pass only the scalar gate, so with a
// shared expert the work is split over two streams:
//
//   caller's stream   shared gate/up (5-stage pipeline) . shared down .        . routed GEMMs . combine
//   side stream       router . count/scan/scatter/gather ^(mid)        ^(join)
//
// The gate/up launch goes first and takes one CTA per SM with a pipeline one
// stage shorter than usual; what it leaves free on each SM (shared memory,
// registers) is what one router CTA needs, so the router's CUDA-core dot
// products run under the tensor-core pass instead of in front of it.  Up to
// split_tokens() rows, where both GEMMs stream weights and neither fills the
// machine, the routed GEMM follows on the side stream too and the two share
// the SMs by grid size.  Without a shared expert everything runs in order on
// the caller's stream.
static int32_t layer_forward_large(const sb_moe_layer *L, const LayerScratch &s, int32_t *status,
                                   cudaStream_t stream) {
  const int T = L->T, H = L->H, E = L->E, K = L->K, I = L->I, Is = L->I_shared;
  void *shared_scale = L->shared_gate_w ? s.shared_scale : nullptr;
  int32_t rc;
  if (Is == 0) {
    rc = launch_router(L->x, L->router_w, L->router_bias, nullptr, T, H, E, K, L->renorm, SB_DTYPE_BF16,
                       L->router_fp32_logits, L->topk_idx, L->topk_w, L->logits, nullptr, stream);
    if (rc != SB_OK) return rc;
    rc = launch_permute(L->x, L->topk_idx, L->topk_w, T * K, K, H, E, s.permute_ws, s.permute_ws_bytes, s.xs,
                        s.expert_offsets, s.slot_of_item, s.item_of_slot, s.slot_scale, s.tile_table, stream);
    if (rc != SB_OK) return rc;
    rc = launch_grouped_swiglu_any(s.xs, s.tile_table, 0, L->w13, L->w2, L->slot_of_expert, s.slot_scale, s.r_cap,
                                   H, I, L->n_slots, s.hbuf, s.y, status, stream);
    if (rc != SB_OK) return rc;
    return launch_combine(s.y, s.slot_of_item, L->topk_idx, nullptr, nullptr, T, H, K, L->out, stream);
  }
  std::unique_lock<std::recursive_mutex> lock(g_side_mu);
  SideLane *lane = side_lane();
  if (lane == nullptr)
    return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: call sb_init(device) once for this device first");
  const bool beside = router_overlap() != 0;
  const int all_pairs = sb_device_sm_count() / 2;
  const bool split = T <= split_tokens() && all_pairs > 2 * shared_pairs();
  cudaStream_t side = lane->stream;
  if (!beside) {
    rc = launch_router(L->x, L->router_w, L->router_bias, L->shared_gate_w, T, H, E, K, L->renorm, SB_DTYPE_BF16,
                       L->router_fp32_logits, L->topk_idx, L->topk_w, L->logits, shared_scale, stream);
    if (rc != SB_OK) return rc;
  }
  SB_CUDA_CHECK(cudaEventRecord(lane->fork, stream));
  SB_CUDA_CHECK(cudaStreamWaitEvent(side, lane->fork, 0));
  // From here on the side stream is forked from the caller's: every path below
  // records `mid` and `join` and makes the caller's stream wait for both, so a
  // stream capture always ends joined, whatever failed in between.
  int32_t rc_shared = SB_OK;
  if (beside)
    rc_shared = launch_grouped_swiglu_any(L->x, nullptr, T, L->shared_w13, L->shared_w2, nullptr, nullptr, T, H, Is,
                                          1, s.shared_h, s.shared_out, status, stream,
                                          split ? shared_pairs() : 0, 1, kStagesBesideRouter);
  rc = SB_OK;
  if (beside)
    rc = launch_router(L->x, L->router_w, L->router_bias, L->shared_gate_w, T, H, E, K, L->renorm, SB_DTYPE_BF16,
                       L->router_fp32_logits, L->topk_idx, L->topk_w, L->logits, shared_scale, side);
  SB_CUDA_CHECK(cudaEventRecord(lane->mid, side));
  if (rc == SB_OK)
    rc = launch_permute(L->x, L->topk_idx, L->topk_w, T * K, K, H, E, s.permute_ws, s.permute_ws_bytes, s.xs,
                        s.expert_offsets, s.slot_of_item, s.item_of_slot, s.slot_scale, s.tile_table, side);
  if (rc == SB_OK && split)
    rc = launch_grouped_swiglu_any(s.xs, s.tile_table, 0, L->w13, L->w2, L->slot_of_expert, s.slot_scale, s.r_cap,
                                   H, I, L->n_slots, s.hbuf, s.y, status, side, all_pairs - shared_pairs());
  SB_CUDA_CHECK(cudaEventRecord(lane->join, side));
  // The shared expert's down pass leaves the scalar gate to the combine kernel, so
  // it does not wait for the router (which takes 190 us instead of 73 us while it
  // shares the SMs with the gate/up pass).
  if (rc_shared == SB_OK)
    rc_shared = launch_grouped_swiglu_any(L->x, nullptr, T, L->shared_w13, L->shared_w2, nullptr, nullptr, T,
                                          H, Is, 1, s.shared_h, s.shared_out, status, stream,
                                          split ? shared_pairs() : 0, beside ? 2 : 3, 0);
  SB_CUDA_CHECK(cudaStreamWaitEvent(stream, lane->mid, 0));
  SB_CUDA_CHECK(cudaStreamWaitEvent(stream, lane->join, 0));
  lock.unlock();
  if (rc != SB_OK) return rc;
  if (rc_shared != SB_OK) return rc_shared;
  if (!split) {
    rc = launch_grouped_swiglu_any(s.xs, s.tile_table, 0, L->w13, L->w2, L->slot_of_expert, s.slot_scale, s.r_cap,
                                   H, I, L->n_slots, s.hbuf, s.y, status, stream);
    if (rc != SB_OK) return rc;
  }
  return launch_combine(s.y, s.slot_of_item, L->topk_idx, s.shared_out, shared_scale, T, H, K, L->out, stream);
}

}  // namespace sb

using namespace sb;

extern "C" {

int32_t sb_abi_version(void) { return 2; }

int32_t sb_init(int32_t device) {
  int count = 0;
  SB_CUDA_CHECK(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count || device >= 64)
    return fail(SB_E_INVALID_ARG, "sb_init: device %d outside [0,%d)", device, count < 64 ? count : 64);
  int prev = -1;
  SB_CUDA_CHECK(cudaGetDevice(&prev));
  SB_CUDA_CHECK(cudaSetDevice(device));
  int32_t rc = create_side_lane(device);
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  return rc;
}

int32_t sb_set_tuning(const char *key, int32_t value) {
  if (!key) return fail(SB_E_INVALID_ARG, "sb_set_tuning: null key");
  if (strcmp(key, "router_overlap") == 0) {
    if (value != 0 && value != 1) return fail(SB_E_INVALID_ARG, "sb_set_tuning: router_overlap must be 0 or 1");
    g_router_overlap.store(value);
    return SB_OK;
  }
  int32_t rc = set_gemm_tuning(key, value);
  if (rc == SB_E_UNSUPPORTED) rc = set_ep_tuning(key, value);
  if (rc == SB_E_UNSUPPORTED) return fail(SB_E_INVALID_ARG, "sb_set_tuning: unknown key '%s'", key);
  return rc;
}

/* Rows per tile-table entry and the row order of w13: constants of the CTA-pair GEMM. */
int32_t sb_tile_rows(void) { return 256; }

int32_t sb_w13_interleaved(void) { return 1; }

const char *sb_last_error_string(void) { return g_err; }

int32_t sb_last_launch_count(void) { return g_launches; }

int32_t sb_device_sm_count(void) {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

int32_t sb_router_topk(const void *x, const void *wg, const float *bias, const void *w_shared_gate,
                       int32_t T, int32_t H, int32_t E, int32_t K, int32_t renorm, int32_t dtype,
                       int32_t fp32_logits, int32_t *out_idx, void *out_w, void *out_logits,
                       void *out_shared_scale, void *stream) {
  return launch_router(x, wg, bias, w_shared_gate, T, H, E, K, renorm, dtype, fp32_logits, out_idx,
                       out_w, out_logits, out_shared_scale, static_cast<cudaStream_t>(stream));
}

int32_t sb_softmax_topk(const void *logits, int32_t T, int32_t E, int32_t K, int32_t renorm,
                        int32_t dtype, int32_t *out_idx, void *out_w, void *stream) {
  return launch_softmax_topk(logits, T, E, K, renorm, dtype, out_idx, out_w,
                             static_cast<cudaStream_t>(stream));
}

int32_t sb_permute(const void *x, const int32_t *item_expert, const void *item_scale,
                   int32_t n_items, int32_t items_per_row, int32_t H, int32_t E, void *ws,
                   size_t ws_bytes, void *out_rows, int32_t *expert_offsets, int32_t *slot_of_item,
                   int32_t *item_of_slot, void *slot_scale, int32_t *tile_table, void *stream) {
  return launch_permute(x, item_expert, item_scale, n_items, items_per_row, H, E, ws, ws_bytes,
                        out_rows, expert_offsets, slot_of_item, item_of_slot, slot_scale, tile_table,
                        static_cast<cudaStream_t>(stream));
}

int32_t sb_grouped_swiglu(const void *rows, const int32_t *tile_table, int32_t dense_rows,
                          const void *w13, const void *w2, const int32_t *slot_of_expert,
                          const void *row_scale, int32_t R_cap, int32_t H, int32_t I, int32_t S,
                          void *hbuf, void *out, int32_t *status, void *stream) {
  return launch_grouped_swiglu_any(rows, tile_table, dense_rows, w13, w2, slot_of_expert, row_scale,
                                   R_cap, H, I, S, hbuf, out, status, static_cast<cudaStream_t>(stream));
}

int32_t sb_decode_experts(const void *x, const int32_t *item_of_slot, int32_t items_per_row,
                          const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                          const void *w2, const void *row_scale, int32_t H, int32_t I, int32_t n_slots,
                          void *hbuf, void *y, const void *shared_w13, const void *shared_w2,
                          const void *shared_scale, int32_t I_shared, int32_t T, void *shared_h,
                          void *shared_out, int32_t *status, void *stream) {
  if (shared_w13 && T > SB_DECODE_MAX_TOKENS)
    return fail(SB_E_UNSUPPORTED, "sb_decode_experts: at most %d rows for the shared expert", SB_DECODE_MAX_TOKENS);
  return launch_decode_experts(x, item_of_slot, items_per_row, tile_table, slot_of_expert, w13, w2, row_scale,
                               H, I, n_slots, hbuf, y, shared_w13, shared_w2, shared_scale, I_shared, T,
                               shared_h, shared_out, status, 2, 0, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int32_t sb_decode_experts_to(const void *x, const int32_t *item_of_slot, int32_t items_per_row,
                             const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                             const void *w2, const void *row_scale, int32_t H, int32_t I, int32_t n_slots,
                             void *hbuf, const uint64_t *row_dst, int32_t T, int32_t *status, void *stream) {
  if (!tile_table || !row_dst || T < 1) return fail(SB_E_INVALID_ARG, "sb_decode_experts_to: bad arguments");
  return launch_decode_experts(x, item_of_slot, items_per_row, tile_table, slot_of_expert, w13, w2, row_scale, H,
                               I, n_slots, hbuf, nullptr, nullptr, nullptr, nullptr, 0, T, nullptr, nullptr, status,
                               2, 1 << 30, nullptr, reinterpret_cast<const unsigned long long *>(row_dst),
                               static_cast<cudaStream_t>(stream));
}

int32_t sb_grouped_swiglu_passes(const void *rows, const int32_t *tile_table, int32_t dense_rows,
                                 const void *w13, const void *w2, const int32_t *slot_of_expert,
                                 const void *row_scale, int32_t R_cap, int32_t H, int32_t I, int32_t S,
                                 void *hbuf, void *out, int32_t passes, int32_t stages, int32_t *status,
                                 void *stream) {
  if (passes < 1 || passes > 3) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu_passes: passes=%d", passes);
  return launch_grouped_swiglu_pair(rows, tile_table, dense_rows, w13, w2, slot_of_expert, row_scale, R_cap, H, I,
                                    S, hbuf, out, status, 0, 0, nullptr, static_cast<cudaStream_t>(stream), passes,
                                    stages);
}

int32_t sb_grouped_swiglu_scatter(const void *rows, const int32_t *tile_table, const void *w13, const void *w2,
                                  const int32_t *slot_of_expert, const void *row_scale, int32_t R_cap,
                                  int32_t H, int32_t I, int32_t S, void *hbuf, const uint64_t *row_dst,
                                  int32_t *status, void *stream) {
  if (!tile_table || !row_dst) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu_scatter: null pointer");
  return launch_grouped_swiglu_pair(rows, tile_table, 0, w13, w2, slot_of_expert, row_scale, R_cap, H, I, S, hbuf,
                                    nullptr, status, 0, 0, reinterpret_cast<const unsigned long long *>(row_dst),
                                    static_cast<cudaStream_t>(stream));
}

int32_t sb_grouped_swiglu_mixed(const void *rows, const int32_t *tile_table, const void *w13, const void *w2,
                                const int32_t *slot_of_expert, const void *row_scale, int32_t R_cap,
                                int32_t H, int32_t I, int32_t S, void *hbuf, void *out,
                                int32_t max_group_rows, const void *shared_x, const void *shared_w13,
                                const void *shared_w2, const void *shared_scale, int32_t I_shared, int32_t T,
                                void *shared_h, void *shared_out, const uint64_t *row_dst, int32_t *status,
                                void *stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!tile_table) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu_mixed: needs a tile table");
  const unsigned long long *dst = reinterpret_cast<const unsigned long long *>(row_dst);
  const bool with_shared = shared_w13 != nullptr && T > 0;
  if (with_shared && (!shared_x || !shared_w2 || !shared_h || !shared_out || I_shared <= 0))
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu_mixed: shared expert arguments go together");
  if (H % 32 != 0 || I % 32 != 0 || (with_shared && I_shared % 32 != 0)) {
    if (dst != nullptr)
      return fail(SB_E_UNSUPPORTED, "sb_grouped_swiglu_mixed: row_dst needs H, I, I_shared to be multiples of 32");
    int32_t rc = launch_grouped_swiglu_any(rows, tile_table, 0, w13, w2, slot_of_expert, row_scale, R_cap, H, I, S,
                                           hbuf, out, status, st);
    if (rc != SB_OK || !with_shared) return rc;
    return launch_grouped_swiglu_any(shared_x, nullptr, T, shared_w13, shared_w2, nullptr, shared_scale, T, H,
                                     I_shared, 1, shared_h, shared_out, status, st);
  }
  const int limit = max_group_rows > 0 ? max_group_rows : SB_DECODE_MAX_TOKENS;
  int32_t rc = launch_decode_experts(rows, nullptr, 1, tile_table, slot_of_expert, w13, w2, row_scale, H, I, S,
                                     hbuf, out, with_shared ? shared_w13 : nullptr,
                                     with_shared ? shared_w2 : nullptr, with_shared ? shared_scale : nullptr,
                                     with_shared ? I_shared : 0, with_shared ? T : 1, shared_h, shared_out,
                                     status, 2, limit, shared_x, dst, st);
  if (rc != SB_OK || max_group_rows > 0) return rc;     // the caller's bound says no group is left over
  return launch_grouped_swiglu_pair(rows, tile_table, 0, w13, w2, slot_of_expert, row_scale, R_cap, H, I, S,
                                    hbuf, out, status, limit, 0, dst, st);
}

int32_t sb_route_decode(const void *x, const void *w_router, const float *router_bias, const void *w_shared_gate,
                        int32_t T, int32_t H, int32_t E, int32_t K, int32_t renorm, int32_t fp32_logits,
                        float *ws, int32_t *out_idx, void *out_w, void *out_logits, void *out_shared_scale,
                        int32_t *expert_offsets, int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale,
                        int32_t *tile_table, void *stream) {
  if (T < 0 || T > SB_DECODE_MAX_TOKENS)
    return fail(SB_E_INVALID_ARG, "sb_route_decode: T=%d outside [0,%d]", T, SB_DECODE_MAX_TOKENS);
  if (!x || !w_router || !out_idx || !out_w || !tile_table)
    return fail(SB_E_INVALID_ARG, "sb_route_decode: null pointer");
  if ((w_shared_gate != nullptr) != (out_shared_scale != nullptr))
    return fail(SB_E_INVALID_ARG, "sb_route_decode: w_shared_gate and out_shared_scale go together");
  return launch_router_decode(x, w_router, router_bias, w_shared_gate, T, H, E, K, renorm, fp32_logits, ws,
                              out_idx, out_w, out_logits, out_shared_scale, expert_offsets, slot_of_item,
                              item_of_slot, slot_scale, tile_table, static_cast<cudaStream_t>(stream));
}

int32_t sb_combine(const void *rows_out, const int32_t *slot_of_item, const int32_t *idx,
                   const void *shared_out, int32_t T, int32_t H, int32_t K, void *out, void *stream) {
  return launch_combine(rows_out, slot_of_item, idx, shared_out, nullptr, T, H, K, out,
                        static_cast<cudaStream_t>(stream));
}

int32_t sb_combine_gated(const void *rows_out, const int32_t *slot_of_item, const int32_t *idx,
                         const void *shared_out, const void *shared_scale, int32_t T, int32_t H, int32_t K,
                         void *out, void *stream) {
  return launch_combine(rows_out, slot_of_item, idx, shared_out, shared_scale, T, H, K, out,
                        static_cast<cudaStream_t>(stream));
}

int32_t sb_slot_copy_async(void *dst_slot, const void *src, size_t bytes, int32_t kind,
                           int32_t device, void *stream) {
  if (!dst_slot || !src) return fail(SB_E_INVALID_ARG, "sb_slot_copy_async: null pointer");
  if (bytes == 0) return SB_OK;
  cudaMemcpyKind k;
  switch (kind) {
    case SB_COPY_HOST_TO_DEVICE: k = cudaMemcpyHostToDevice; break;
    case SB_COPY_PEER_TO_DEVICE: k = cudaMemcpyDefault; break;     // unified addressing finds the peer
    case SB_COPY_DEVICE_LOCAL: k = cudaMemcpyDeviceToDevice; break;
    default: return fail(SB_E_INVALID_ARG, "sb_slot_copy_async: unknown kind %d", kind);
  }
  if (device >= 0) SB_CUDA_CHECK(cudaSetDevice(device));
  SB_CUDA_CHECK(cudaMemcpyAsync(dst_slot, src, bytes, k, static_cast<cudaStream_t>(stream)));
  return SB_OK;
}

size_t sb_moe_layer_struct_bytes(void) { return sizeof(sb_moe_layer); }

size_t sb_moe_layer_workspace_bytes(int32_t T, int32_t H, int32_t E, int32_t K, int32_t I,
                                    int32_t I_shared) {
  if (T < 0 || H <= 0 || E <= 0 || K <= 0 || I <= 0 || I_shared < 0) return 0;
  return carve(nullptr, T, H, E, K, I, I_shared).total;
}

int32_t sb_moe_layer_forward(const sb_moe_layer *L, int32_t *status, void *stream_) {
  reset_launch_count();
  if (!L) return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: null layer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int T = L->T, H = L->H, E = L->E, K = L->K, I = L->I, Is = L->I_shared;
  if (T < 0 || H <= 0 || E <= 0 || K <= 0 || I <= 0 || Is < 0)
    return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: bad shape T=%d H=%d E=%d K=%d I=%d Is=%d", T, H,
                E, K, I, Is);
  if (T == 0) return SB_OK;
  if (!L->x || !L->router_w || !L->w13 || !L->w2 || !L->out || !L->topk_idx || !L->topk_w || !L->ws)
    return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: null pointer");
  if ((Is > 0) != (L->shared_w13 != nullptr && L->shared_w2 != nullptr))
    return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: shared weights and I_shared go together");
  if (L->shared_gate_w && Is == 0)
    return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: shared gate without shared expert");
  if (!aligned(L->ws, 1024)) return fail(SB_E_INVALID_ARG, "sb_moe_layer_forward: ws must be 1024-byte aligned");
  LayerScratch s = carve(static_cast<char *>(L->ws), T, H, E, K, I, Is);
  if (L->ws_bytes < s.total)
    return fail(SB_E_WORKSPACE, "sb_moe_layer_forward: workspace %zu < %zu bytes", L->ws_bytes, s.total);

  if (T <= SB_DECODE_MAX_TOKENS) {
    int32_t rc = launch_router_decode(L->x, L->router_w, L->router_bias, L->shared_gate_w, T, H, E, K, L->renorm,
                                      L->router_fp32_logits, s.router_ws, L->topk_idx, L->topk_w, L->logits,
                                      L->shared_gate_w ? s.shared_scale : nullptr, s.expert_offsets,
                                      s.slot_of_item, s.item_of_slot, s.slot_scale, s.tile_table, stream);
    if (rc != SB_OK) return rc;
    // decode-sized pass: the router launch already sorted the items (no gathered copy of x)
    rc = launch_decode_experts(L->x, s.item_of_slot, K, s.tile_table, L->slot_of_expert, L->w13, L->w2,
                               s.slot_scale, H, I, L->n_slots, s.hbuf, s.y, Is > 0 ? L->shared_w13 : nullptr,
                               Is > 0 ? L->shared_w2 : nullptr, L->shared_gate_w ? s.shared_scale : nullptr,
                               Is, T, s.shared_h, s.shared_out, status, 2, 0, nullptr, nullptr, stream);
    if (rc != SB_OK) return rc;
    return launch_combine(s.y, s.slot_of_item, L->topk_idx, Is > 0 ? s.shared_out : nullptr, nullptr, T, H, K,
                          L->out, stream);
  }
  return layer_forward_large(L, s, status, stream);
}

}  // extern "C"
