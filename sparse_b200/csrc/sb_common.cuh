// Shared helpers for the sparse_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sparse_b200.h"

namespace sb {

// Thread-local error text behind sb_last_error_string().
void set_error(const char *fmt, ...);
int32_t fail(int32_t code, const char *fmt, ...);
// Kernel-launch counter behind sb_last_launch_count().
void count_launch(int n = 1);
void reset_launch_count();

#define SB_CUDA_CHECK(expr)                                                          \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess)                                                           \
      return ::sb::fail(SB_E_CUDA, "%s failed: %s (%s:%d)", #expr,                   \
                        cudaGetErrorString(_e), __FILE__, __LINE__);                 \
  } while (0)

// Programmatic dependent launch: a kernel launched with launch_pdl may start
// (be scheduled, run its index set-up) while the previous kernel of the stream is
// still draining, once all of that kernel's CTAs have executed
// pdl_launch_dependents(); pdl_wait() then blocks until the previous kernel has
// completed and its writes are visible.  Both are no-ops in a plain launch.
// Rule for kernels using them: no global memory access before pdl_wait().
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define SB_LAUNCH_CHECK()                                                            \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess)                                                           \
      return ::sb::fail(SB_E_CUDA, "kernel launch failed: %s (%s:%d)",               \
                        cudaGetErrorString(_e), __FILE__, __LINE__);                 \
    ::sb::count_launch();                                                            \
  } while (0)

static inline bool aligned(const void *p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// ---- bf16 helpers --------------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// round-to-nearest-even fp32 -> bf16 bits, then back to fp32
__device__ __forceinline__ float round_bf16(float f) {
  return __bfloat162float(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);   // .x = lo, .y = hi
  return *reinterpret_cast<uint32_t *>(&v);
}

// Tile table layout shared by sb_permute and the grouped GEMM.
constexpr int kTileHeaderInts = 4;   // [0] = number of row tiles
constexpr int kTileEntryInts = 4;    // expert, row_begin, row_end, 0

}  // namespace sb

// Internal launchers (one per .cu file), all asynchronous on `stream`.
namespace sb {
int32_t launch_router(const void *x, const void *wg, const float *bias, const void *wsg,
                      int T, int H, int E, int K, int renorm, int dtype, int fp32_logits,
                      int32_t *out_idx, void *out_w, void *out_logits, void *out_shared_scale,
                      cudaStream_t stream);
int32_t launch_router_decode(const void *x, const void *wg, const float *bias, const void *wsg, int T, int H,
                             int E, int K, int renorm, int fp32_logits, float *ws, int32_t *out_idx,
                             void *out_w, void *out_logits, void *out_shared_scale, int32_t *expert_offsets,
                             int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale, int32_t *tile_table,
                             cudaStream_t stream);
int32_t launch_softmax_topk(const void *logits, int T, int E, int K, int renorm, int dtype,
                            int32_t *out_idx, void *out_w, cudaStream_t stream);
int32_t launch_permute(const void *x, const int32_t *item_expert, const void *item_scale,
                       int n_items, int items_per_row, int H, int E, void *ws,
                       size_t ws_bytes, void *out_rows, int32_t *expert_offsets,
                       int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale,
                       int32_t *tile_table, cudaStream_t stream);
int32_t launch_grouped_swiglu_pair(const void *rows, const int32_t *tile_table, int dense_rows,
                                   const void *w13, const void *w2, const int32_t *slot_of_expert,
                                   const void *row_scale, int R_cap, int H, int I, int S,
                                   void *hbuf, void *out, int32_t *status, int skip_rows_upto, int max_pairs,
                                   const unsigned long long *row_dst, cudaStream_t stream, int passes = 3,
                                   int stages = 0);
int32_t set_gemm_tuning(const char *key, int value);
int32_t set_ep_tuning(const char *key, int value);       // SB_E_UNSUPPORTED: not one of its keys
int32_t launch_decode_experts(const void *x, const int32_t *item_of_slot, int items_per_row,
                              const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                              const void *w2, const void *row_scale, int H, int I, int n_slots, void *hbuf,
                              void *y, const void *shared_w13, const void *shared_w2,
                              const void *shared_scale, int I_sh, int T, void *shared_h, void *shared_out,
                              int32_t *status, int ctas_per_sm, int max_rows, const void *shared_x,
                              const unsigned long long *row_dst, cudaStream_t stream);
int32_t launch_combine(const void *rows_out, const int32_t *slot_of_item, const int32_t *idx,
                       const void *shared_out, const void *shared_scale, int T, int H, int K, void *out,
                       cudaStream_t stream);
}  // namespace sb
