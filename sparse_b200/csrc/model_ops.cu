// The small kernels of the decode loop around the MoE layers: RMSNorm with the
// residual add folded in, rotary embedding + KV-cache append, and decode-time
// attention (one query per sequence against the cache).
//
// The reference runs these through the Transformers model classes
// (utils/eval_core.py:17807-17829 loads them, the loop at 18464-18607 calls
// them once per generated token); here they are plain CUDA so that one decode
// step -- every layer's attention, norms and MoE block -- can be captured in a
// single CUDA graph.  All three are HBM-bound: the norm reads and writes its
// rows once, the attention reads each cached key and value exactly once.
//
// Arithmetic contract (matched by the fp32 PyTorch restatement in the tests
// within bf16 tolerance): sums and softmax in fp32; bf16 rounding of the
// residual sum, of the normalised row before the weight multiply, and of the
// outputs.
#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

template <int E>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16 *p, float (&out)[E]) {
  static_assert(E % 2 == 0, "pairs");
#pragma unroll
  for (int e = 0; e < E; e += 2) {
    const uint32_t w = *reinterpret_cast<const uint32_t *>(p + e);
    out[e] = bf16_lo(w);
    out[e + 1] = bf16_hi(w);
  }
}

// One CTA per row.  h = bf16(residual + delta) (or residual alone); the row is
// written back to `residual` when a delta was added; out = weight * bf16(h * rsqrt(mean(h^2) + eps)).
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(__nv_bfloat16 *__restrict__ residual, const __nv_bfloat16 *__restrict__ delta,
                   const __nv_bfloat16 *__restrict__ delta2, const __nv_bfloat16 *__restrict__ weight, float eps,
                   int H, __nv_bfloat16 *__restrict__ out) {
  extern __shared__ float row[];                 // H floats
  __shared__ float part[kNormThreads / 32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += kNormThreads) {
    float v = __bfloat162float(residual[base + i]);
    if (delta != nullptr) {
      v = round_bf16(v + __bfloat162float(delta[base + i]));
      if (delta2 != nullptr) v = round_bf16(v + __bfloat162float(delta2[base + i]));
      residual[base + i] = __float2bfloat16_rn(v);
    }
    row[i] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) tot += part[w];
  const float inv = rsqrtf(tot / (float)H + eps);
  if (out != nullptr)
    for (int i = threadIdx.x; i < H; i += kNormThreads)
      out[base + i] = __float2bfloat16_rn(__bfloat162float(weight[i]) * round_bf16(row[i] * inv));
}

// One CTA per token.  Rotates the first `rope_dim` elements of every q and k
// head (pairs (i, i + rope_dim/2), angle pos * theta^(-2i/rope_dim)), writes q
// back in place and k, v into the cache row of (sequence, position).
__global__ void __launch_bounds__(128)
rope_append_kernel(__nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ k,
                   const __nv_bfloat16 *__restrict__ v, const int32_t *__restrict__ seq_of_token,
                   const int32_t *__restrict__ pos_of_token, int n_q, int n_kv, int dk, int dv, int rope_dim,
                   float theta, int s_max, __nv_bfloat16 *__restrict__ cache_k, __nv_bfloat16 *__restrict__ cache_v,
                   int q_stride, int k_stride, int v_stride) {
  const int t = blockIdx.x;
  const int pos = pos_of_token[t], seq = seq_of_token[t];
  const int half = rope_dim >> 1;
  const float log_theta = __logf(theta);
  // q heads, in place
  for (int i = threadIdx.x; i < n_q * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const float ang = (float)pos * __expf(-log_theta * (2.0f * (float)j / (float)rope_dim));
    float sn, cs;
    sincosf(ang, &sn, &cs);
    sn = round_bf16(sn); cs = round_bf16(cs);
    __nv_bfloat16 *p = q + (size_t)t * q_stride + (size_t)h * dk;
    const float a = __bfloat162float(p[j]), b = __bfloat162float(p[j + half]);
    p[j] = __float2bfloat16_rn(round_bf16(a * cs) + round_bf16(-b * sn));
    p[j + half] = __float2bfloat16_rn(round_bf16(b * cs) + round_bf16(a * sn));
  }
  if (pos < 0 || pos >= s_max) return;
  __nv_bfloat16 *ck = cache_k + ((size_t)seq * s_max + pos) * n_kv * dk;
  __nv_bfloat16 *cv = cache_v + ((size_t)seq * s_max + pos) * n_kv * dv;
  for (int i = threadIdx.x; i < n_kv * dk; i += blockDim.x) {
    const int h = i / dk, j = i - h * dk;
    const __nv_bfloat16 *p = k + (size_t)t * k_stride + (size_t)h * dk;
    float val = __bfloat162float(p[j]);
    if (j < rope_dim) {
      const int jj = j < half ? j : j - half;
      const float ang = (float)pos * __expf(-log_theta * (2.0f * (float)jj / (float)rope_dim));
      float sn, cs;
      sincosf(ang, &sn, &cs);
      sn = round_bf16(sn); cs = round_bf16(cs);
      const float other = __bfloat162float(j < half ? p[j + half] : p[j - half]);
      val = round_bf16(val * cs) + round_bf16((j < half ? -other : other) * sn);
    }
    ck[i] = __float2bfloat16_rn(val);
  }
  for (int i = threadIdx.x; i < n_kv * dv; i += blockDim.x) cv[i] = v[(size_t)t * v_stride + i];
}

// Decode attention, split over the keys.  grid = (sequences * query heads,
// splits); a CTA of 4 warps walks its slice of the cached keys, each warp every
// fourth key, lanes owning DK/32 (DV/32) consecutive elements, online softmax
// per warp; the warps and then the splits are merged by their running maxima.
template <int DK, int DV>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const __nv_bfloat16 *__restrict__ q, int q_stride, const __nv_bfloat16 *__restrict__ cache_k,
                   const __nv_bfloat16 *__restrict__ cache_v, const int32_t *__restrict__ seq_lens, int n_q,
                   int n_kv, int s_max, float scale, int n_split, float *__restrict__ part) {
  constexpr int EK = DK / 32, EV = DV / 32;
  constexpr int U = 4;                        // keys a warp has in flight per iteration
  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / n_q, h = bh - b * n_q;
  const int hk = h / (n_q / n_kv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = min(seq_lens[b], s_max);
  const int per = (len + n_split - 1) / n_split;
  const int j0 = split * per, j1 = min(len, j0 + per);
  float qv[EK];
#pragma unroll
  for (int e = 0; e < EK; ++e)
    qv[e] = __bfloat162float(q[(size_t)b * q_stride + (size_t)h * DK + lane * EK + e]) * scale;
  float m = -INFINITY, l = 0.f, acc[EV];
#pragma unroll
  for (int e = 0; e < EV; ++e) acc[e] = 0.f;
  const __nv_bfloat16 *kb = cache_k + ((size_t)b * s_max * n_kv + hk) * DK + lane * EK;
  const __nv_bfloat16 *vb = cache_v + ((size_t)b * s_max * n_kv + hk) * DV + lane * EV;
  for (int j = j0 + warp * U; j < j1; j += 4 * U) {
    float kv[U][EK], vv[U][EV], s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int jj = min(j + u, j1 - 1);       // clamped: the duplicate is masked below
      load_bf16<EK>(kb + (size_t)jj * n_kv * DK, kv[u]);
      load_bf16<EV>(vb + (size_t)jj * n_kv * DV, vv[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      s[u] = 0.f;
#pragma unroll
      for (int e = 0; e < EK; ++e) s[u] += qv[e] * kv[u][e];
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], off);
    float m_new = m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (j + u >= j1) s[u] = -INFINITY;
      m_new = fmaxf(m_new, s[u]);
    }
    const float corr = __expf(m - m_new);
    l *= corr;
#pragma unroll
    for (int e = 0; e < EV; ++e) acc[e] *= corr;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float p = __expf(s[u] - m_new);    // exp(-inf) = 0 for the masked keys
      l += p;
#pragma unroll
      for (int e = 0; e < EV; ++e) acc[e] += p * vv[u][e];
    }
    m = m_new;
  }
  // merge the four warps
  __shared__ float sm[4], sl[4], sacc[4][DV];
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < EV; ++e) sacc[warp][lane * EV + e] = acc[e];
  __syncthreads();
  if (warp == 0) {
    float mm = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
    float ll = 0.f, out[EV];
#pragma unroll
    for (int e = 0; e < EV; ++e) out[e] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = sm[w] == -INFINITY ? 0.f : __expf(sm[w] - mm);
      ll += sl[w] * c;
#pragma unroll
      for (int e = 0; e < EV; ++e) out[e] += sacc[w][lane * EV + e] * c;
    }
    float *dst = part + ((size_t)bh * n_split + split) * (DV + 2);
    if (lane == 0) { dst[0] = mm; dst[1] = ll; }
#pragma unroll
    for (int e = 0; e < EV; ++e) dst[2 + lane * EV + e] = out[e];
  }
}

template <int DV>
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float *__restrict__ part, int n_split, __nv_bfloat16 *__restrict__ out) {
  const int bh = blockIdx.x;
  const float *src = part + (size_t)bh * n_split * (DV + 2);
  float mm = -INFINITY;
  for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, src[(size_t)s * (DV + 2)]);
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float *p = src + (size_t)s * (DV + 2);
      const float c = p[0] == -INFINITY ? 0.f : __expf(p[0] - mm);
      ll += p[1] * c;
      acc += p[2 + d] * c;
    }
    out[(size_t)bh * DV + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
  }
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

int32_t sb_add_rmsnorm(void *residual, const void *delta, const void *delta2, const void *weight, float eps,
                       int32_t T, int32_t H, void *out, void *stream) {
  if (T < 0 || H <= 0 || H > 16384) return fail(SB_E_INVALID_ARG, "sb_add_rmsnorm: bad shape (T=%d H=%d)", T, H);
  if (T == 0) return SB_OK;
  if (!residual || (!out && !delta) || (out && !weight) || (delta2 && !delta))
    return fail(SB_E_INVALID_ARG, "sb_add_rmsnorm: null pointer");
  add_rmsnorm_kernel<<<T, kNormThreads, (size_t)H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(residual), static_cast<const __nv_bfloat16 *>(delta),
      static_cast<const __nv_bfloat16 *>(delta2), static_cast<const __nv_bfloat16 *>(weight), eps, H,
      static_cast<__nv_bfloat16 *>(out));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_rope_append(void *q, const void *k, const void *v, const int32_t *seq_of_token,
                       const int32_t *pos_of_token, int32_t T, int32_t n_q, int32_t n_kv, int32_t dk, int32_t dv,
                       int32_t rope_dim, float theta, int32_t s_max, void *cache_k, void *cache_v, int32_t q_stride,
                       int32_t k_stride, int32_t v_stride, void *stream) {
  if (q_stride == 0) q_stride = n_q * dk;
  if (k_stride == 0) k_stride = n_kv * dk;
  if (v_stride == 0) v_stride = n_kv * dv;
  if (q_stride < n_q * dk || k_stride < n_kv * dk || v_stride < n_kv * dv)
    return fail(SB_E_INVALID_ARG, "sb_rope_append: a token stride is smaller than the token");
  if (T < 0 || n_q < 1 || n_kv < 1 || dk < 2 || dv < 1 || rope_dim < 0 || rope_dim > dk || (rope_dim & 1) || s_max < 1)
    return fail(SB_E_INVALID_ARG, "sb_rope_append: bad shape");
  if (T == 0) return SB_OK;
  if (!q || !k || !v || !seq_of_token || !pos_of_token || !cache_k || !cache_v)
    return fail(SB_E_INVALID_ARG, "sb_rope_append: null pointer");
  rope_append_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k), static_cast<const __nv_bfloat16 *>(v),
      seq_of_token, pos_of_token, n_q, n_kv, dk, dv, rope_dim, theta, s_max,
      static_cast<__nv_bfloat16 *>(cache_k), static_cast<__nv_bfloat16 *>(cache_v), q_stride, k_stride, v_stride);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

size_t sb_attn_decode_workspace_bytes(int32_t B, int32_t n_q, int32_t dv, int32_t n_split) {
  if (B < 0 || n_q < 1 || dv < 1 || n_split < 1) return 0;
  return (size_t)B * n_q * n_split * (dv + 2) * sizeof(float);
}

int32_t sb_attn_decode(const void *q, int32_t q_stride, const void *cache_k, const void *cache_v,
                       const int32_t *seq_lens, int32_t B, int32_t n_q, int32_t n_kv, int32_t dk, int32_t dv,
                       int32_t s_max, float scale, int32_t n_split, void *ws, size_t ws_bytes, void *out,
                       void *stream) {
  if (q_stride == 0) q_stride = n_q * dk;
  if (q_stride < n_q * dk) return fail(SB_E_INVALID_ARG, "sb_attn_decode: q_stride smaller than a token's heads");
  if (B < 0 || n_q < 1 || n_kv < 1 || n_q % n_kv != 0 || s_max < 1 || n_split < 1 || n_split > 256)
    return fail(SB_E_INVALID_ARG, "sb_attn_decode: bad shape");
  if (B == 0) return SB_OK;
  if (!q || !cache_k || !cache_v || !seq_lens || !ws || !out) return fail(SB_E_INVALID_ARG, "sb_attn_decode: null pointer");
  if (ws_bytes < sb_attn_decode_workspace_bytes(B, n_q, dv, n_split))
    return fail(SB_E_WORKSPACE, "sb_attn_decode: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(B * n_q, n_split);
  const __nv_bfloat16 *qq = static_cast<const __nv_bfloat16 *>(q);
  const __nv_bfloat16 *kk = static_cast<const __nv_bfloat16 *>(cache_k);
  const __nv_bfloat16 *vv = static_cast<const __nv_bfloat16 *>(cache_v);
  float *part = static_cast<float *>(ws);
  __nv_bfloat16 *oo = static_cast<__nv_bfloat16 *>(out);
  if (dk == 128 && dv == 128) {
    attn_decode_kernel<128, 128><<<grid, 128, 0, st>>>(qq, q_stride, kk, vv, seq_lens, n_q, n_kv, s_max, scale, n_split, part);
    SB_LAUNCH_CHECK();
    attn_merge_kernel<128><<<B * n_q, 128, 0, st>>>(part, n_split, oo);
  } else if (dk == 192 && dv == 128) {
    attn_decode_kernel<192, 128><<<grid, 128, 0, st>>>(qq, q_stride, kk, vv, seq_lens, n_q, n_kv, s_max, scale, n_split, part);
    SB_LAUNCH_CHECK();
    attn_merge_kernel<128><<<B * n_q, 128, 0, st>>>(part, n_split, oo);
  } else if (dk == 64 && dv == 64) {
    attn_decode_kernel<64, 64><<<grid, 128, 0, st>>>(qq, q_stride, kk, vv, seq_lens, n_q, n_kv, s_max, scale, n_split, part);
    SB_LAUNCH_CHECK();
    attn_merge_kernel<64><<<B * n_q, 128, 0, st>>>(part, n_split, oo);
  } else {
    return fail(SB_E_UNSUPPORTED, "sb_attn_decode: head dims (%d,%d) not built (128/128, 192/128, 64/64)", dk, dv);
  }
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // extern "C"
