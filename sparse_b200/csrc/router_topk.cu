// Router: logits (fixed fp32 summation order) -> softmax (fp32) -> top-k.
//
// Replaces `_routing_router` of the reference (utils/eval_core.py:9519-9520,
// 9591-9595) plus the scalar gate of the shared expert
// (utils/eval_core.py:9461-9462).
//
// Summation order of one logit (bit-exact contract with the CPU oracle): the H
// inputs are cut into groups of 8; lane l of a warp takes groups l, l+32, l+64,
// ... in increasing order and keeps two partial sums, one over the even and one
// over the odd elements of its groups, elements in increasing order, each step
// p = fl(p + fl(x*w)) (for bf16 inputs the product is exact, so a fused
// multiply-add gives the same bits); the lane sum is fl(p_even + p_odd); the 32
// lane sums are combined by an xor-butterfly with offsets 16, 8, 4, 2, 1; the
// bias is added in fp32 and the result is rounded once to the model dtype.
//
// Work split: one CTA owns TB tokens whose activations sit in shared memory;
// each of its 8 warps streams pairs of router rows from L2 and dots them with
// all TB tokens, so a weight row is fetched once per CTA.  HBM traffic is one
// read of x plus the outputs; the kernel is bound by the fp32 FMA pipe
// (2*T*E*H flops on CUDA cores), not by DRAM.
#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kRouterThreads = 256;
constexpr int kRouterWarps = kRouterThreads / 32;
constexpr int kMaxExperts = 256;
constexpr int kMaxK = 8;

template <typename IN> struct Load8;

template <> struct Load8<__nv_bfloat16> {
  static constexpr bool kExactProduct = true;
  __device__ static void from(const uint4 *p, float (&v)[8]) {
    uint4 r = *p;
    v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
    v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z); v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
  }
  __device__ static void from_global(const __nv_bfloat16 *base, size_t elem, float (&v)[8]) {
    uint4 r = __ldg(reinterpret_cast<const uint4 *>(base + elem));
    v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
    v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z); v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
  }
  __device__ static float round_model(float f) { return round_bf16(f); }
  __device__ static void store(__nv_bfloat16 *p, float f) { *p = __float2bfloat16_rn(f); }
  __device__ static float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
};

template <> struct Load8<float> {
  static constexpr bool kExactProduct = false;
  __device__ static void from(const uint4 *p, float (&v)[8]) {
    uint4 a = p[0], b = p[1];
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y);
    v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y);
    v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
  __device__ static void from_global(const float *base, size_t elem, float (&v)[8]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(base + elem);
    uint4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y);
    v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y);
    v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
  __device__ static float round_model(float f) { return f; }
  __device__ static void store(float *p, float f) { *p = f; }
  __device__ static float load(const float *p) { return *p; }
};

__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
__device__ __forceinline__ float butterfly_max(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// Sums of 32 values over the 32 lanes at once: lane i returns the warp-wide sum of
// v[i].  Each step halves the values a lane still carries (it keeps the half that
// its lane-id bit selects and hands the other half to its partner), so this takes
// 31 shuffles instead of 32 x 5.  The additions pair the same lanes at the same
// offsets (16, 8, 4, 2, 1) as butterfly_sum, and fp32 addition is commutative:
// the result has the bits butterfly_sum gives for that value on every lane.
__device__ __forceinline__ float warp_sum_each(float (&v)[32], int lane) {
#pragma unroll
  for (int half = 16; half >= 1; half >>= 1) {
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float keep = upper ? v[i + half] : v[i];
      const float send = upper ? v[i] : v[i + half];
      v[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, half));
    }
  }
  return v[0];
}

// One warp: softmax over E model-dtype logits (given as fp32 values) and top-k.
// `lg` points at this token's E logits in shared memory.
template <typename IN>
__device__ void warp_softmax_topk(const float *lg, int E, int K, int renorm, int lane,
                                  int32_t *out_idx, IN *out_w) {
  constexpr int kPerLane = kMaxExperts / 32;
  float p[kPerLane];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    int e = lane + 32 * i;
    p[i] = (e < E) ? lg[e] : -INFINITY;
    m = fmaxf(m, p[i]);
  }
  m = butterfly_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    int e = lane + 32 * i;
    if (e < E) { p[i] = expf(p[i] - m); s = __fadd_rn(s, p[i]); } else { p[i] = -1.f; }
  }
  s = butterfly_sum(s);
#pragma unroll
  for (int i = 0; i < kPerLane; ++i)
    if (p[i] >= 0.f) p[i] = __fdiv_rn(p[i], s);
  // A row with a NaN or an infinite logit has NaN probabilities.  torch.topk ranks
  // NaN above every number (utils/eval_core.py:9591-9595 calls it); here NaN gets
  // the key 3 for the selection, so that the indices written are always expert
  // ids, and the weight written for it is NaN again.
#pragma unroll
  for (int i = 0; i < kPerLane; ++i)
    if (p[i] != p[i]) p[i] = 3.f;

  float sel_v[kMaxK];
  int sel_i[kMaxK];
#pragma unroll
  for (int k = 0; k < kMaxK; ++k) {
    if (k >= K) break;
    // lane-local best: larger probability, then smaller expert id
    float bv = -2.f; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      int e = lane + 32 * i;
      if (p[i] > bv) { bv = p[i]; bi = e; }   // ascending e: first max wins
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    sel_v[k] = bv > 2.f ? __int_as_float(0x7fc00000) : bv; sel_i[k] = bi;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (lane + 32 * i == bi) p[i] = -1.f;
  }
  if (lane == 0) {
    float denom = 1.f;
    if (renorm) {
      float t = 0.f;
      for (int k = 0; k < K; ++k) t = __fadd_rn(t, sel_v[k]);
      denom = fmaxf(t, 1e-12f);
    }
#pragma unroll
    for (int k = 0; k < kMaxK; ++k) {
      if (k >= K) break;
      float v = renorm ? __fdiv_rn(sel_v[k], denom) : sel_v[k];
      out_idx[k] = sel_i[k];
      Load8<IN>::store(out_w + k, v);
    }
  }
}

// Two running partial sums (even / odd elements) packed for the two-wide FMA.
struct Acc2 {
  unsigned long long v;
  __device__ static Acc2 zero() { Acc2 a; a.v = 0ull; return a; }
  __device__ float lane_sum() const {
    return __fadd_rn(__uint_as_float((uint32_t)v), __uint_as_float((uint32_t)(v >> 32)));
  }
  template <typename P> __device__ void fma(const P &x, const P &w, int i) { x.fma_into(v, w, i); }
};

// Eight consecutive elements as four (even, odd) pairs.
template <typename IN> struct Pair4;

template <> struct Pair4<__nv_bfloat16> {
  unsigned long long p[4];
  __device__ static unsigned long long widen(uint32_t word) {      // bf16x2 -> {f32 lo, f32 hi}
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(word << 16), "r"(word & 0xffff0000u));
    return r;
  }
  __device__ void load(const uint4 *src) {
    const uint4 q = *src;
    p[0] = widen(q.x); p[1] = widen(q.y); p[2] = widen(q.z); p[3] = widen(q.w);
  }
  // products of bf16 values are exact in fp32, so the fused form equals mul-then-add
  __device__ void fma_into(unsigned long long &acc, const Pair4 &w, int i) const {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(p[i]), "l"(w.p[i]));
  }
};

template <> struct Pair4<float> {
  float e[8];
  __device__ void load(const uint4 *src) {
    const uint4 a = src[0], b = src[1];
    e[0] = __uint_as_float(a.x); e[1] = __uint_as_float(a.y); e[2] = __uint_as_float(a.z);
    e[3] = __uint_as_float(a.w); e[4] = __uint_as_float(b.x); e[5] = __uint_as_float(b.y);
    e[6] = __uint_as_float(b.z); e[7] = __uint_as_float(b.w);
  }
  // fp32 inputs: multiply and add round separately (the order the CPU check emulates)
  __device__ void fma_into(unsigned long long &acc, const Pair4 &w, int i) const {
    float lo = __uint_as_float((uint32_t)acc), hi = __uint_as_float((uint32_t)(acc >> 32));
    lo = __fadd_rn(lo, __fmul_rn(e[2 * i], w.e[2 * i]));
    hi = __fadd_rn(hi, __fmul_rn(e[2 * i + 1], w.e[2 * i + 1]));
    acc = ((unsigned long long)__float_as_uint(hi) << 32) | (unsigned long long)__float_as_uint(lo);
  }
};

template <typename IN, int TB>
__global__ void __launch_bounds__(kRouterThreads, 2)
router_kernel(const IN *__restrict__ x, const IN *__restrict__ wg, const float *__restrict__ bias,
              const IN *__restrict__ wsg, int T, int H, int E, int K, int renorm, int fp32_logits,
              int tb_eff, int32_t *__restrict__ out_idx, IN *__restrict__ out_w,
              void *__restrict__ out_logits, IN *__restrict__ out_shared) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kVecPerGroup = sizeof(IN) == 2 ? 1 : 2;      // uint4 per 8 elements
  const int G = H / 8;
  uint4 *sx = reinterpret_cast<uint4 *>(smem_raw);            // [TB][G*kVecPerGroup]
  float *slog = reinterpret_cast<float *>(sx + (size_t)TB * G * kVecPerGroup);  // [TB][E+1]
  const int NR = E + (wsg != nullptr ? 1 : 0);
  const int ldl = E + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * tb_eff;      // this CTA's tokens: t0 .. t0 + tb_eff - 1 (tb_eff <= TB)

  // stage the activation tile
  const int vec_per_tok = G * kVecPerGroup;
  for (int i = threadIdx.x; i < tb_eff * vec_per_tok; i += kRouterThreads) {
    int t = i / vec_per_tok, v = i - t * vec_per_tok;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t0 + t < T)
      val = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(t0 + t) * H) + v);
    sx[i] = val;
  }
  __syncthreads();

  // Four router rows per warp pass: one shared-memory read of a token's 8
  // activations feeds 32 multiply-adds, issued as 16 two-wide fp32 FMAs
  // (`fma.rn.f32x2`: two independent IEEE FMAs per instruction, so the bits are
  // those of scalar FMAs).  Each lane therefore keeps TWO partial sums per logit,
  // one over the even and one over the odd elements of its groups.  The next
  // step's weight vectors are fetched before the current step's math.
  constexpr int RW = 4;
  const int steps = (G + 31) / 32;
  const int groups = (NR + RW - 1) / RW;
  for (int grp = warp; grp < groups; grp += kRouterWarps) {
    const IN *wp[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int row = grp * RW + r;
      wp[r] = (row < E) ? wg + (size_t)row * H : ((row < NR) ? wsg : nullptr);
    }
    Acc2 acc[TB][RW];
#pragma unroll
    for (int t = 0; t < TB; ++t)
#pragma unroll
      for (int r = 0; r < RW; ++r) acc[t][r] = Acc2::zero();
    uint4 cur[RW][kVecPerGroup], nxt[RW][kVecPerGroup];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int v = 0; v < kVecPerGroup; ++v) {
        cur[r][v] = make_uint4(0, 0, 0, 0);
        if (lane < G && wp[r] != nullptr)
          cur[r][v] = __ldg(reinterpret_cast<const uint4 *>(wp[r] + (size_t)lane * 8) + v);
      }
    // Full token tile and a hidden size of whole 256-element steps (the usual
    // case): the same arithmetic without the per-token and per-row guards.  Rows
    // past the last one read row 0's weights; their sums are never stored.
    if (TB < 8 && tb_eff == TB && (G & 31) == 0) {      // (the 8-token tile has no registers to spare for a second loop)
      const IN *wq[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r) wq[r] = wp[r] != nullptr ? wp[r] : wg;
#pragma unroll
      for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int v = 0; v < kVecPerGroup; ++v)
          cur[r][v] = __ldg(reinterpret_cast<const uint4 *>(wq[r] + (size_t)lane * 8) + v);
#pragma unroll 1
      for (int j = 0; j < steps; ++j) {
        const int g = j * 32 + lane;
        if (j + 1 < steps) {
#pragma unroll
          for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int v = 0; v < kVecPerGroup; ++v)
              nxt[r][v] = __ldg(reinterpret_cast<const uint4 *>(wq[r] + (size_t)(g + 32) * 8) + v);
        }
        Pair4<IN> w[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) w[r].load(&cur[r][0]);
#pragma unroll
        for (int t = 0; t < TB; ++t) {
          Pair4<IN> xv;
          xv.load(sx + ((size_t)t * G + g) * kVecPerGroup);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < RW; ++r) acc[t][r].fma(xv, w[r], i);
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
          for (int v = 0; v < kVecPerGroup; ++v) cur[r][v] = nxt[r][v];
      }
    } else
    for (int j = 0; j < steps; ++j) {
      const int g = j * 32 + lane;
      const int gn = g + 32;
#pragma unroll
      for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int v = 0; v < kVecPerGroup; ++v) {
          nxt[r][v] = make_uint4(0, 0, 0, 0);
          if (gn < G && wp[r] != nullptr)
            nxt[r][v] = __ldg(reinterpret_cast<const uint4 *>(wp[r] + (size_t)gn * 8) + v);
        }
      if (g < G) {
        Pair4<IN> w[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) w[r].load(&cur[r][0]);
#pragma unroll
        for (int t = 0; t < TB; ++t) {
          if (t < tb_eff) {
            Pair4<IN> xv;
            xv.load(sx + ((size_t)t * G + g) * kVecPerGroup);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int r = 0; r < RW; ++r) acc[t][r].fma(xv, w[r], i);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int v = 0; v < kVecPerGroup; ++v) cur[r][v] = nxt[r][v];
    }
    if (TB * RW < 32) {                 // (a full 32 would need every register the loop above holds)
      // lane t*RW + r ends up with the logit of (token t, row r of this group)
      float part[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) part[i] = 0.f;
#pragma unroll
      for (int t = 0; t < TB; ++t)
#pragma unroll
        for (int r = 0; r < RW; ++r) part[t * RW + r] = acc[t][r].lane_sum();
      float sum = warp_sum_each(part, lane);
      const int t = lane / RW, row = grp * RW + lane % RW;
      if (t < tb_eff && row < NR) {
        if (row < E && bias != nullptr) sum = __fadd_rn(sum, bias[row]);
        // the shared gate's logit (row E) is always a model-dtype linear output
        slog[t * ldl + row] = (fp32_logits && row < E) ? sum : Load8<IN>::round_model(sum);
      }
    } else {
#pragma unroll
      for (int t = 0; t < TB; ++t) {
        if (t < tb_eff) {
#pragma unroll
          for (int r = 0; r < RW; ++r) {
            const int row = grp * RW + r;
            float sum = butterfly_sum(acc[t][r].lane_sum());
            if (lane == 0 && row < NR) {
              if (row < E && bias != nullptr) sum = __fadd_rn(sum, bias[row]);
              slog[t * ldl + row] = (fp32_logits && row < E) ? sum : Load8<IN>::round_model(sum);
            }
          }
        }
      }
    }
  }
  __syncthreads();

  for (int t = warp; t < tb_eff; t += kRouterWarps) {
    const int tok = t0 + t;
    if (tok >= T) continue;
    const float *lg = slog + t * ldl;
    if (out_logits != nullptr) {
      if (fp32_logits)
        for (int e = lane; e < E; e += 32) static_cast<float *>(out_logits)[(size_t)tok * E + e] = lg[e];
      else
        for (int e = lane; e < E; e += 32)
          Load8<IN>::store(static_cast<IN *>(out_logits) + (size_t)tok * E + e, lg[e]);
    }
    if (wsg != nullptr && lane == 0) {
      float v = lg[E];
      float sg = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
      Load8<IN>::store(out_shared + tok, sg);
    }
    warp_softmax_topk<IN>(lg, E, K, renorm, lane, out_idx + (size_t)tok * K,
                          out_w + (size_t)tok * K);
  }
}

template <typename LT, typename IN>
__global__ void __launch_bounds__(kRouterThreads)
softmax_topk_kernel(const LT *__restrict__ logits, int ld_logits, int T, int E, int K, int renorm,
                    int32_t *__restrict__ out_idx, IN *__restrict__ out_w) {
  __shared__ float slog[kRouterWarps][kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kRouterWarps + warp;
  if (tok >= T) return;
  for (int e = lane; e < E; e += 32) slog[warp][e] = Load8<LT>::load(logits + (size_t)tok * ld_logits + e);
  __syncwarp();
  warp_softmax_topk<IN>(slog[warp], E, K, renorm, lane, out_idx + (size_t)tok * K,
                        out_w + (size_t)tok * K);
}

// Decode-sized router: one warp per (token, router row), so a single token's 61
// rows are streamed by 61 warps on 8 SMs instead of by one CTA.  Same per-lane
// summation order as router_kernel (groups lane, lane+32, ...; even/odd partial
// sums; butterfly), hence the same bits.  Logits go to `ws` as fp32 values
// already rounded to the model dtype (unless fp32_logits); softmax_topk_kernel
// finishes the job.
template <typename IN>
__global__ void __launch_bounds__(kRouterThreads)
router_rows_kernel(const IN *__restrict__ x, const IN *__restrict__ wg, const float *__restrict__ bias,
                   const IN *__restrict__ wsg, int T, int H, int E, int fp32_logits,
                   float *__restrict__ ws, void *__restrict__ out_logits, IN *__restrict__ out_shared) {
  constexpr int kVecPerGroup = sizeof(IN) == 2 ? 1 : 2;
  pdl_launch_dependents();
  pdl_wait();
  const int NR = E + (wsg != nullptr ? 1 : 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x;
  const int row = blockIdx.y * kRouterWarps + warp;
  if (row >= NR) return;
  const IN *wrow = (row < E) ? wg + (size_t)row * H : wsg;
  const IN *xrow = x + (size_t)tok * H;
  const int G = H / 8;
  Acc2 acc = Acc2::zero();
  for (int g0 = 0; g0 < G; g0 += 32 * 4) {
    uint4 wq[4][kVecPerGroup], xq[4][kVecPerGroup];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int v = 0; v < kVecPerGroup; ++v) {
        const int g = g0 + u * 32 + lane;
        wq[u][v] = make_uint4(0, 0, 0, 0); xq[u][v] = make_uint4(0, 0, 0, 0);
        if (g < G) {
          wq[u][v] = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)g * 8) + v);
          xq[u][v] = __ldg(reinterpret_cast<const uint4 *>(xrow + (size_t)g * 8) + v);
        }
      }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (g0 + u * 32 + lane < G) {
        Pair4<IN> wv, xv;
        wv.load(&wq[u][0]);
        xv.load(&xq[u][0]);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc.fma(xv, wv, i);
      }
    }
  }
  float sum = butterfly_sum(acc.lane_sum());
  if (lane == 0) {
    if (row < E) {
      if (bias != nullptr) sum = __fadd_rn(sum, bias[row]);
      const float lg = fp32_logits ? sum : Load8<IN>::round_model(sum);
      ws[(size_t)tok * E + row] = lg;
      if (out_logits != nullptr) {
        if (fp32_logits) static_cast<float *>(out_logits)[(size_t)tok * E + row] = lg;
        else Load8<IN>::store(static_cast<IN *>(out_logits) + (size_t)tok * E + row, lg);
      }
    } else {
      const float v = Load8<IN>::round_model(sum);
      Load8<IN>::store(out_shared + tok, __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v))));
    }
  }
}

template <typename IN, int TB>
int32_t launch_router_tb(const void *x, const void *wg, const float *bias, const void *wsg, int T,
                         int H, int E, int K, int renorm, int fp32_logits, int32_t *out_idx,
                         void *out_w, void *out_logits, void *out_shared, cudaStream_t stream) {
  const size_t smem_max = (size_t)TB * H * sizeof(IN) + (size_t)TB * (E + 1) * sizeof(float);
  auto kern = router_kernel<IN, TB>;
  if (smem_max > 48 * 1024)
    SB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
  // tokens per CTA: as few as keeps the grid within four CTAs per SM, so the
  // last wave is full (4096 tokens on 148 SMs -> 7 per CTA, 586 CTAs)
  const int slots = 4 * (sb_device_sm_count() > 0 ? sb_device_sm_count() : 148);
  int tb_eff = (T + slots - 1) / slots;
  if (tb_eff < 1) tb_eff = 1;
  if (tb_eff > TB) tb_eff = TB;
  int blocks = (T + tb_eff - 1) / tb_eff;
  kern<<<blocks, kRouterThreads, smem_max, stream>>>(
      static_cast<const IN *>(x), static_cast<const IN *>(wg), bias, static_cast<const IN *>(wsg),
      T, H, E, K, renorm, fp32_logits, tb_eff, out_idx, static_cast<IN *>(out_w), out_logits,
      static_cast<IN *>(out_shared));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

template <typename IN>
int32_t launch_router_t(const void *x, const void *wg, const float *bias, const void *wsg, int T,
                        int H, int E, int K, int renorm, int fp32_logits, int32_t *out_idx,
                        void *out_w, void *out_logits, void *out_shared, cudaStream_t stream) {
  // Fewer tokens per CTA when there are few tokens, so decode-sized calls still
  // spread over the SMs; 16 per CTA at prefill sizes to amortise the weight reads.
  const size_t tile8 = (size_t)8 * H * sizeof(IN) + 8 * (size_t)(E + 1) * 4;
  // 7 when that is all a CTA takes anyway (4096 tokens over four CTAs per SM on
  // 148 SMs): the tile is sized by the template, and the less shared memory a
  // router CTA asks for, the more of the SM a GEMM CTA of another stream keeps
  const int sms = sb_device_sm_count() > 0 ? sb_device_sm_count() : 148;
  if (T >= 1024 && tile8 <= 100 * 1024 && (T + 4 * sms - 1) / (4 * sms) <= 7)
    return launch_router_tb<IN, 7>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx,
                                    out_w, out_logits, out_shared, stream);
  if (T >= 1024 && tile8 <= 100 * 1024)
    return launch_router_tb<IN, 8>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx,
                                    out_w, out_logits, out_shared, stream);
  if (T >= 256)
    return launch_router_tb<IN, 4>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx,
                                   out_w, out_logits, out_shared, stream);
  return launch_router_tb<IN, 1>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx, out_w,
                                 out_logits, out_shared, stream);
}

}  // namespace

int32_t launch_router(const void *x, const void *wg, const float *bias, const void *wsg, int T,
                      int H, int E, int K, int renorm, int dtype, int fp32_logits, int32_t *out_idx,
                      void *out_w, void *out_logits, void *out_shared_scale, cudaStream_t stream) {
  if (T < 0 || H <= 0 || H % 8 != 0 || E < 1 || E > kMaxExperts || K < 1 || K > kMaxK || K > E)
    return fail(SB_E_INVALID_ARG, "sb_router_topk: need H%%8==0, 1<=K<=8, K<=E<=256 (T=%d H=%d E=%d K=%d)",
                T, H, E, K);
  if (T == 0) return SB_OK;
  if (!x || !wg || !out_idx || !out_w) return fail(SB_E_INVALID_ARG, "sb_router_topk: null pointer");
  if ((wsg != nullptr) != (out_shared_scale != nullptr))
    return fail(SB_E_INVALID_ARG, "sb_router_topk: w_shared_gate and out_shared_scale go together");
  if (!aligned(x, 16) || !aligned(wg, 16) || (wsg && !aligned(wsg, 16)))
    return fail(SB_E_INVALID_ARG, "sb_router_topk: x, wg, w_shared_gate must be 16-byte aligned");
  if ((size_t)H * (dtype == SB_DTYPE_F32 ? 4 : 2) + (E + 1) * 4 > 200 * 1024)
    return fail(SB_E_UNSUPPORTED, "sb_router_topk: hidden size %d too large for the token tile", H);
  if (dtype == SB_DTYPE_BF16)
    return launch_router_t<__nv_bfloat16>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx,
                                          out_w, out_logits, out_shared_scale, stream);
  if (dtype == SB_DTYPE_F32)
    return launch_router_t<float>(x, wg, bias, wsg, T, H, E, K, renorm, fp32_logits, out_idx, out_w,
                                  out_logits, out_shared_scale, stream);
  return fail(SB_E_INVALID_ARG, "sb_router_topk: unknown dtype %d", dtype);
}

namespace {

// Decode-sized softmax/top-k AND expert sort in one CTA: warp t finishes token
// t (same arithmetic as softmax_topk_kernel), then the T*K items (at most 128)
// are ranked by (expert id, item index) with an all-pairs count, which yields
// the same stable expert-sorted order, offsets and tile table as the permute
// kernels.
constexpr int kSmallMaxItems = 16 * kMaxK;

__global__ void __launch_bounds__(512)
route_sort_small_kernel(const float *__restrict__ logits, int T, int E, int K, int renorm, int tile_rows,
                        int tile_cap, int32_t *__restrict__ out_idx, __nv_bfloat16 *__restrict__ out_w,
                        int32_t *__restrict__ expert_offsets, int32_t *__restrict__ slot_of_item,
                        int32_t *__restrict__ item_of_slot, __nv_bfloat16 *__restrict__ slot_scale,
                        int32_t *__restrict__ tile_table) {
  __shared__ float slog[16][kMaxExperts];
  __shared__ int s_exp[kSmallMaxItems];
  __shared__ int s_off[kMaxExperts + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < T) {
    for (int e = lane; e < E; e += 32) slog[warp][e] = logits[(size_t)warp * E + e];
    __syncwarp();
    warp_softmax_topk<__nv_bfloat16>(slog[warp], E, K, renorm, lane, out_idx + (size_t)warp * K,
                                     out_w + (size_t)warp * K);
  }
  __syncthreads();                       // this CTA's global writes are visible to all its threads
  const int n = T * K;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = out_idx[i];
    s_exp[i] = (e >= 0 && e < E) ? e : -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    int below = 0;
    for (int j = 0; j < n; ++j) below += (s_exp[j] >= 0 && s_exp[j] < e) ? 1 : 0;
    s_off[e] = below;
    expert_offsets[e] = below;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = s_exp[i];
    int slot = -1;
    if (e >= 0) {
      slot = 0;
      for (int j = 0; j < n; ++j) slot += (s_exp[j] >= 0 && (s_exp[j] < e || (s_exp[j] == e && j < i))) ? 1 : 0;
      item_of_slot[slot] = i;
      slot_scale[slot] = out_w[i];
    }
    slot_of_item[i] = slot;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int ts = 0;                          // tiles of the experts below e
    for (int j = 0; j < e; ++j) ts += (s_off[j + 1] - s_off[j] + tile_rows - 1) / tile_rows;
    const int cnt = s_off[e + 1] - s_off[e];
    const int nt = (cnt + tile_rows - 1) / tile_rows;
    for (int m = 0; m < nt; ++m) {
      const int ti = ts + m;
      if (ti >= tile_cap) break;
      int32_t *ent = tile_table + kTileHeaderInts + (size_t)ti * kTileEntryInts;
      const int rb = s_off[e] + m * tile_rows;
      ent[0] = e; ent[1] = rb; ent[2] = min(s_off[e + 1], rb + tile_rows); ent[3] = 0;
    }
    if (e == E - 1) {
      const int all = ts + nt;
      tile_table[0] = all < tile_cap ? all : tile_cap;
      tile_table[1] = s_off[E];
      tile_table[2] = tile_rows; tile_table[3] = 0;
    }
  }
}

}  // namespace

int32_t launch_router_decode(const void *x, const void *wg, const float *bias, const void *wsg, int T, int H,
                             int E, int K, int renorm, int fp32_logits, float *ws, int32_t *out_idx,
                             void *out_w, void *out_logits, void *out_shared_scale, int32_t *expert_offsets,
                             int32_t *slot_of_item, int32_t *item_of_slot, void *slot_scale, int32_t *tile_table,
                             cudaStream_t stream) {
  if (T <= 0) return SB_OK;
  if (H % 8 != 0 || E < 1 || E > kMaxExperts || K < 1 || K > kMaxK || K > E || !ws)
    return fail(SB_E_INVALID_ARG, "router (decode): bad arguments");
  const int NR = E + (wsg ? 1 : 0);
  dim3 grid(T, (NR + kRouterWarps - 1) / kRouterWarps);
  SB_CUDA_CHECK(launch_pdl(router_rows_kernel<__nv_bfloat16>, grid, dim3(kRouterThreads), 0, stream,
                           static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(wg), bias,
                           static_cast<const __nv_bfloat16 *>(wsg), T, H, E, fp32_logits, ws, out_logits,
                           static_cast<__nv_bfloat16 *>(out_shared_scale)));
  SB_LAUNCH_CHECK();
  if (tile_table != nullptr) {
    // softmax/top-k and the expert sort in one single-CTA launch
    if (T > 16 || !expert_offsets || !slot_of_item || !item_of_slot || !slot_scale)
      return fail(SB_E_INVALID_ARG, "router (decode): sort outputs need T <= 16 and all tables");
    const int warps = T > 4 ? 16 : 4;
    SB_CUDA_CHECK(launch_pdl(route_sort_small_kernel, dim3(1), dim3(warps * 32), 0, stream,
                             static_cast<const float *>(ws), T, E, K, renorm, sb_tile_rows(),
                             T * K / SB_TILE_M + E, out_idx, static_cast<__nv_bfloat16 *>(out_w), expert_offsets,
                             slot_of_item, item_of_slot, static_cast<__nv_bfloat16 *>(slot_scale), tile_table));
    SB_LAUNCH_CHECK();
    return SB_OK;
  }
  softmax_topk_kernel<float, __nv_bfloat16><<<(T + kRouterWarps - 1) / kRouterWarps, kRouterThreads, 0, stream>>>(
      ws, E, T, E, K, renorm, out_idx, static_cast<__nv_bfloat16 *>(out_w));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t launch_softmax_topk(const void *logits, int T, int E, int K, int renorm, int dtype,
                            int32_t *out_idx, void *out_w, cudaStream_t stream) {
  if (T < 0 || E < 1 || E > kMaxExperts || K < 1 || K > kMaxK || K > E)
    return fail(SB_E_INVALID_ARG, "sb_softmax_topk: need 1<=K<=8, K<=E<=256 (T=%d E=%d K=%d)", T, E, K);
  if (T == 0) return SB_OK;
  if (!logits || !out_idx || !out_w) return fail(SB_E_INVALID_ARG, "sb_softmax_topk: null pointer");
  int blocks = (T + kRouterWarps - 1) / kRouterWarps;
  if (dtype == SB_DTYPE_BF16)
    softmax_topk_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, kRouterThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(logits), E, T, E, K, renorm, out_idx,
        static_cast<__nv_bfloat16 *>(out_w));
  else if (dtype == SB_DTYPE_F32)
    softmax_topk_kernel<float, float><<<blocks, kRouterThreads, 0, stream>>>(
        static_cast<const float *>(logits), E, T, E, K, renorm, out_idx, static_cast<float *>(out_w));
  else
    return fail(SB_E_INVALID_ARG, "sb_softmax_topk: unknown dtype %d", dtype);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // namespace sb
