// Decode-sized expert MLPs: a handful of tokens against whole expert matrices.
//
// With 1..16 tokens the layer is a pure weight-streaming problem (138 MB of
// bf16 weights for 4 routed experts plus the shared expert of the Qwen block,
// ~21 us at HBM speed): a 256-row tcgen05 tile per CTA pair leaves most SMs
// without a stream of their own.  Here every warp streams 16 weight rows
// straight from global memory into registers with 16-byte loads (16 in flight
// per lane) and multiplies them with warp-level m16n8k16 MMAs against the
// token rows, which stay L1-resident.  No conversion instructions, no shared
// memory staging: the k index inside each 32-element chunk is permuted the same
// way for both operands (lane c of a quad owns elements c*8..c*8+7 of the
// chunk), so a 16-byte load is directly two MMAs' worth of fragments.  A CTA of
// 8 warps splits a task's K range between warps and adds the partial sums
// through shared memory.
//
// Same arithmetic contract as the grouped GEMM (fp32 accumulation, bf16
// rounding after gate, up, silu, product, down and the route-weight scaling;
// utils/eval_core.py:11787-11790, 11765 of the reference); only the fp32
// summation order differs, as it does between any two GEMM kernels.
//
// Two launches per layer, each covering the routed groups AND the shared
// expert:  pass 1  h = bf16(bf16(silu(bf16 x.Wg)) * bf16 x.Wu)
//          pass 2  y = bf16(bf16(h.Wd) * scale)
// Routed token rows are read through `item_of_slot` (no gathered copy of x), or
// directly when the rows are already expert-sorted (`item_of_slot` null).
// Groups of more than 16 rows are left alone: next to the tile kernel this
// pair of launches serves the light groups of a large batch.
#include <stdlib.h>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSlotSkip = -2;
constexpr int kMaxTok = 16;          // two 8-token MMA column tiles

struct Group { int slot, begin, end; };

__device__ __forceinline__ Group read_group(const int32_t *tile_table, const int32_t *slot_of_expert, int c) {
  const int4 e = __ldg(reinterpret_cast<const int4 *>(tile_table + kTileHeaderInts) + c);
  Group g;
  g.slot = slot_of_expert ? __ldg(slot_of_expert + e.x) : e.x;
  g.begin = e.y; g.end = e.z;
  return g;
}

// weights are read once: keep them out of L1 so the token rows stay there
__device__ __forceinline__ uint4 ld_stream(const __nv_bfloat16 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[nt] += W[16 rows, chunks) . X[tokens nt*8.., chunks)^T for one warp.
// Lane (g = lane/4, c = lane%4): row_lo/row_hi point at element c*8 of weight
// rows g and g+8 of the warp's 16, tok[nt] at element c*8 of token g of column
// tile nt.  acc[nt] = {lo row x tokens 2c, 2c+1; hi row x tokens 2c, 2c+1}.
template <int NT>
__device__ __forceinline__ void stream_rows(const __nv_bfloat16 *row_lo, const __nv_bfloat16 *row_hi,
                                            const __nv_bfloat16 *const (&tok)[2], int chunk_begin, int chunk_end,
                                            float (&acc)[2][4]) {
  constexpr int U = NT == 1 ? 8 : 4;
  for (int ch = chunk_begin; ch < chunk_end; ch += U) {
    uint4 lo[U], hi[U], xb[NT][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = ch + u < chunk_end;
      const size_t off = (size_t)(ch + u) * 32;
      lo[u] = ok ? ld_stream(row_lo + off) : make_uint4(0, 0, 0, 0);
      hi[u] = ok ? ld_stream(row_hi + off) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        xb[nt][u] = ok ? __ldg(reinterpret_cast<const uint4 *>(tok[nt] + off)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma16816(acc[nt], lo[u].x, hi[u].x, lo[u].y, hi[u].y, xb[nt][u].x, xb[nt][u].y);
        mma16816(acc[nt], lo[u].z, hi[u].z, lo[u].w, hi[u].w, xb[nt][u].z, xb[nt][u].w);
      }
    }
  }
}

// Adds the partial sums of the `ks_n` warps that share a row group; the warp
// with k-slice 0 ends up with the totals.  Block-wide call.
__device__ __forceinline__ void reduce_k_slices(float (&acc)[2][4], int warp, int lane, int ks, int ks_n,
                                                float (*red)[8][32]) {
  if (ks != 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[warp][i][lane] = acc[i >> 2][i & 3];
  }
  __syncthreads();
  if (ks == 0) {
    for (int j = 1; j < ks_n; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i >> 2][i & 3] += red[warp + j][i][lane];
  }
  __syncthreads();
}

// pass 1.  Block task = (group, 8/ks_n x 8 intermediate features); a warp owns
// 8 features (gate row g in the low half of its MMA rows, up row g in the high
// half) over one of ks_n slices of H.
__global__ void __launch_bounds__(kThreads, 2)
decode_gate_up_kernel(const __nv_bfloat16 *__restrict__ x, const int32_t *__restrict__ item_of_slot,
                      int items_per_row, const int32_t *__restrict__ tile_table,
                      const int32_t *__restrict__ slot_of_expert, const __nv_bfloat16 *__restrict__ w13,
                      int H, int I, int n_slots, int interleaved, __nv_bfloat16 *__restrict__ hbuf,
                      const __nv_bfloat16 *__restrict__ shared_x,
                      const __nv_bfloat16 *__restrict__ shared_w13, int I_sh, int T,
                      __nv_bfloat16 *__restrict__ shared_h, int ks_n, int max_rows,
                      int32_t *__restrict__ status) {
  __shared__ float red[kWarps][8][32];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rg_n = kWarps / ks_n, rg = warp / ks_n, ks = warp % ks_n;
  const int feats = rg_n * 8;
  const int n_groups = tile_table ? __ldg(tile_table) : 0;
  const int fb_routed = (I + feats - 1) / feats;
  const int fb_shared = shared_w13 ? (I_sh + feats - 1) / feats : 0;
  const long total = (long)n_groups * fb_routed + fb_shared;
  const int chunks = H / 32, per = (chunks + ks_n - 1) / ks_n;
  const int ch0 = min(chunks, ks * per), ch1 = min(chunks, ch0 + per);
  for (long task_id = blockIdx.x; task_id < total; task_id += gridDim.x) {
    const bool is_shared = task_id < fb_shared;          // the shared expert's tasks first
    int fb, begin, end, inter;
    const __nv_bfloat16 *wbase;
    __nv_bfloat16 *out;
    if (!is_shared) {
      const long rt = task_id - fb_shared;
      const int grp = (int)(rt / fb_routed);
      fb = (int)(rt - (long)grp * fb_routed);
      Group gr = read_group(tile_table, slot_of_expert, grp);
      if (gr.slot == kSlotSkip || gr.end - gr.begin > max_rows) continue;   // larger groups belong to the tile kernel
      if (gr.slot < 0 || gr.slot >= n_slots) { if (status && threadIdx.x == 0) atomicExch(status, 2); continue; }
      begin = gr.begin; end = gr.end; inter = I;
      wbase = w13 + (size_t)gr.slot * 2 * I * H;
      out = hbuf;
    } else {
      fb = (int)task_id;
      begin = 0; end = T; inter = I_sh;
      wbase = shared_w13;
      out = shared_h;
    }
    const int f0 = fb * feats + rg * 8;
    const int f = min(f0 + g, inter - 1);
    const __nv_bfloat16 *row_lo = wbase + (size_t)(interleaved ? 2 * f : f) * H + c * 8;
    const __nv_bfloat16 *row_hi = wbase + (size_t)(interleaved ? 2 * f + 1 : inter + f) * H + c * 8;
    const __nv_bfloat16 *xrows = is_shared ? shared_x : x;
    // groups of more than 16 rows are swept 16 rows at a time (the weights of
    // the later sweeps come from L2)
    const int group_end = end;
    for (; begin < group_end; begin += kMaxTok) {
    end = min(group_end, begin + kMaxTok);
    const int n_tok = end - begin;
    const bool live = f0 < inter && n_tok > 0;
    const __nv_bfloat16 *tok[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = begin + max(0, min(nt * 8 + g, n_tok - 1));
      const int row = (is_shared || item_of_slot == nullptr) ? t : (__ldg(item_of_slot + t) / items_per_row);
      tok[nt] = xrows + (size_t)row * H + c * 8;
    }
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (live) {
      if (n_tok > 8) stream_rows<2>(row_lo, row_hi, tok, ch0, ch1, acc);
      else stream_rows<1>(row_lo, row_hi, tok, ch0, ch1, acc);
    }
    reduce_k_slices(acc, warp, lane, ks, ks_n, red);
    if (live && ks == 0 && f0 + g < inter) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int t = nt * 8 + 2 * c + i;
          if (t < n_tok) {
            const float gv = round_bf16(acc[nt][i]), uv = round_bf16(acc[nt][2 + i]);
            const float sv = round_bf16(gv / (1.0f + expf(-gv)));
            out[(size_t)(begin + t) * inter + f0 + g] = __float2bfloat16_rn(sv * uv);
          }
        }
    }
    }
  }
}

// pass 2.  Block task = (group, 8/ks_n x 16 output features) over ks_n slices
// of the intermediate dimension; ks_n differs between routed and shared tasks
// because the shared expert's rows are longer.
__global__ void __launch_bounds__(kThreads, 2)
decode_down_kernel(const __nv_bfloat16 *__restrict__ hbuf, const int32_t *__restrict__ tile_table,
                   const int32_t *__restrict__ slot_of_expert, const __nv_bfloat16 *__restrict__ w2,
                   const __nv_bfloat16 *__restrict__ row_scale, int H, int I, int n_slots,
                   __nv_bfloat16 *__restrict__ y, const __nv_bfloat16 *__restrict__ shared_h,
                   const __nv_bfloat16 *__restrict__ shared_w2, const __nv_bfloat16 *__restrict__ shared_scale,
                   int I_sh, int T, __nv_bfloat16 *__restrict__ shared_out, int ks_routed, int ks_shared,
                   int max_rows, const unsigned long long *__restrict__ row_dst) {
  __shared__ float red[kWarps][8][32];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n_groups = tile_table ? __ldg(tile_table) : 0;
  const int rows_routed = (kWarps / ks_routed) * 16, rows_shared = (kWarps / ks_shared) * 16;
  const int fb_routed = (H + rows_routed - 1) / rows_routed;
  const int fb_shared = shared_w2 ? (H + rows_shared - 1) / rows_shared : 0;
  const long total = (long)n_groups * fb_routed + fb_shared;
  for (long task_id = blockIdx.x; task_id < total; task_id += gridDim.x) {
    const bool is_shared = task_id < fb_shared;
    int fb, begin, end, inter, ks_n;
    const __nv_bfloat16 *wmat, *hin, *scale;
    __nv_bfloat16 *out;
    if (!is_shared) {
      const long rt = task_id - fb_shared;
      const int grp = (int)(rt / fb_routed);
      fb = (int)(rt - (long)grp * fb_routed);
      Group gr = read_group(tile_table, slot_of_expert, grp);
      if (gr.slot < 0 || gr.slot >= n_slots || gr.end - gr.begin > max_rows) continue;   // skipped, or flagged by pass 1
      begin = gr.begin; end = gr.end; inter = I; ks_n = ks_routed;
      wmat = w2 + (size_t)gr.slot * H * I;
      hin = hbuf; scale = row_scale; out = y;
    } else {
      fb = (int)task_id;
      begin = 0; end = T; inter = I_sh; ks_n = ks_shared;
      wmat = shared_w2;
      hin = shared_h; scale = shared_scale; out = shared_out;
    }
    const int rg = warp / ks_n, ks = warp % ks_n;
    const int n0 = (fb * (kWarps / ks_n) + rg) * 16;
    const int chunks = inter / 32, per = (chunks + ks_n - 1) / ks_n;
    const int ch0 = min(chunks, ks * per), ch1 = min(chunks, ch0 + per);
    const int r_lo = min(n0 + g, H - 1), r_hi = min(n0 + 8 + g, H - 1);
    const __nv_bfloat16 *row_lo = wmat + (size_t)r_lo * inter + c * 8;
    const __nv_bfloat16 *row_hi = wmat + (size_t)r_hi * inter + c * 8;
    const int group_end = end;
    for (; begin < group_end; begin += kMaxTok) {
    end = min(group_end, begin + kMaxTok);
    const int n_tok = end - begin;
    const bool live = n0 < H && n_tok > 0;
    const __nv_bfloat16 *tok[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = begin + max(0, min(nt * 8 + g, n_tok - 1));
      tok[nt] = hin + (size_t)t * inter + c * 8;
    }
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (live) {
      if (n_tok > 8) stream_rows<2>(row_lo, row_hi, tok, ch0, ch1, acc);
      else stream_rows<1>(row_lo, row_hi, tok, ch0, ch1, acc);
    }
    reduce_k_slices(acc, warp, lane, ks, ks_n, red);
    if (live && ks == 0) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int t = nt * 8 + 2 * c + i;
          if (t < n_tok) {
            const float sc = scale != nullptr ? __bfloat162float(scale[begin + t]) : 1.0f;
            // routed rows may have a destination of their own (the sender's return buffer)
            __nv_bfloat16 *orow = out + (size_t)(begin + t) * H;
            if (!is_shared && row_dst != nullptr) orow = reinterpret_cast<__nv_bfloat16 *>(row_dst[begin + t]);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int n = n0 + half * 8 + g;
              if (n < H && orow != nullptr) {
                float v = round_bf16(acc[nt][half * 2 + i]);
                if (scale != nullptr) v *= sc;
                orow[n] = __float2bfloat16_rn(v);
              }
            }
          }
        }
    }
    }
  }
}

}  // namespace

int32_t launch_decode_experts(const void *x, const int32_t *item_of_slot, int items_per_row,
                              const int32_t *tile_table, const int32_t *slot_of_expert, const void *w13,
                              const void *w2, const void *row_scale, int H, int I, int n_slots, void *hbuf,
                              void *y, const void *shared_w13, const void *shared_w2, const void *shared_scale,
                              int I_sh, int T, void *shared_h, void *shared_out, int32_t *status,
                              int ctas_per_sm, int max_rows, const void *shared_x,
                              const unsigned long long *row_dst, cudaStream_t stream) {
  if (H % 32 != 0 || I % 32 != 0 || I_sh % 32 != 0)
    return fail(SB_E_UNSUPPORTED, "sb_decode_experts: H, I, I_shared must be multiples of 32");
  if (max_rows <= 0) max_rows = kMaxTok;
  if (shared_x == nullptr) shared_x = x;
  if (T <= 0) return SB_OK;
  if (!x || (tile_table && (!w13 || !w2 || !hbuf || (!y && !row_dst))))
    return fail(SB_E_INVALID_ARG, "sb_decode_experts: null pointer");
  if ((shared_w13 != nullptr) != (shared_w2 != nullptr) || (shared_w13 && (!shared_h || !shared_out)))
    return fail(SB_E_INVALID_ARG, "sb_decode_experts: shared expert arguments go together");
  const int sms = sb_device_sm_count();
  if (sms <= 0) return fail(SB_E_CUDA, "sb_decode_experts: no CUDA device");
  const int grid = sms * (ctas_per_sm == 1 ? 1 : 2);       // grid-stride over the block tasks
  // K slices per row group (measured on B200: 2 slices for 64 chunks of 32
  // elements, 1 for 44, 4 for 176 beat finer splits by up to 8 % at 8 tokens)
  auto slices = [](int k) { const int ch = k / 32; return ch > 128 ? 4 : ch > 48 ? 2 : 1; };
  const int ks1 = slices(H), ks2_routed = slices(I), ks2_shared = slices(I_sh > 0 ? I_sh : I);
  // (Splitting K finer at one or two tokens, so that the 352 pass-1 / 128 pass-2
  // tasks of a single token spread over all CTAs in several small rounds, was
  // measured slower on B200: 50 us against 45 us per layer at one token.  The
  // per-task reduction and synchronisation cost more than the emptier round.)
  // Next to the tile kernel (ctas_per_sm == 1) the SM must already be in the
  // large-shared-memory configuration that kernel needs, or the two could not
  // share an SM; alone, the default split leaves more L1 for the token rows.
  const int carveout = ctas_per_sm == 1 ? (int)cudaSharedmemCarveoutMaxShared : (int)cudaSharedmemCarveoutDefault;
  SB_CUDA_CHECK(cudaFuncSetAttribute(decode_gate_up_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, carveout));
  SB_CUDA_CHECK(cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, carveout));
  SB_CUDA_CHECK(launch_pdl(
      decode_gate_up_kernel, dim3(grid), dim3(kThreads), 0, stream,
      static_cast<const __nv_bfloat16 *>(x), item_of_slot, items_per_row, tile_table, slot_of_expert,
      static_cast<const __nv_bfloat16 *>(w13), H, I, n_slots, sb_w13_interleaved(),
      static_cast<__nv_bfloat16 *>(hbuf), static_cast<const __nv_bfloat16 *>(shared_x),
      static_cast<const __nv_bfloat16 *>(shared_w13), I_sh, T,
      static_cast<__nv_bfloat16 *>(shared_h), ks1, max_rows, status));
  SB_LAUNCH_CHECK();
  SB_CUDA_CHECK(launch_pdl(
      decode_down_kernel, dim3(grid), dim3(kThreads), 0, stream,
      static_cast<const __nv_bfloat16 *>(hbuf), tile_table, slot_of_expert,
      static_cast<const __nv_bfloat16 *>(w2), static_cast<const __nv_bfloat16 *>(row_scale), H, I, n_slots,
      static_cast<__nv_bfloat16 *>(y), static_cast<const __nv_bfloat16 *>(shared_h),
      static_cast<const __nv_bfloat16 *>(shared_w2), static_cast<const __nv_bfloat16 *>(shared_scale), I_sh, T,
      static_cast<__nv_bfloat16 *>(shared_out), ks2_routed, ks2_shared, max_rows, row_dst));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // namespace sb
