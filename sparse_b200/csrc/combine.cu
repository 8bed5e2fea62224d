// Un-permute + combine: out[t] = bf16-sequential sum of the token's K expert
// rows in ascending expert id, then + the shared expert's row (times the
// token's scalar gate when the caller hands it over here, rounded to bf16
// first: utils/eval_core.py:9455-9463 multiplies before the add).
//
// Replaces `unsorted[sort_idx] = gathered; combine_expert_outputs(...)` and the
// final `expert_out + shared_out` of the reference
// (utils/eval_core.py:15058-15060, 523-538, 16547).  The reference adds in the
// activation dtype, so every partial sum is rounded to bf16 before the next
// add; the first add is onto zeros and therefore exact.
//
// HBM-bound: reads K+1 rows and writes one row per token, 16-byte vectors,
// one CTA per token (H/8 vectors spread over the threads).
#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kMaxK = 8;

__device__ __forceinline__ uint32_t add_bf16x2_rn(uint32_t a, uint32_t b) {
  return pack_bf16x2(__fadd_rn(bf16_lo(a), bf16_lo(b)), __fadd_rn(bf16_hi(a), bf16_hi(b)));
}
__device__ __forceinline__ uint4 add_bf16x8_rn(uint4 a, uint4 b) {
  return make_uint4(add_bf16x2_rn(a.x, b.x), add_bf16x2_rn(a.y, b.y), add_bf16x2_rn(a.z, b.z),
                    add_bf16x2_rn(a.w, b.w));
}

// v * s per element with one rounding (the product of two bf16 values is exact in
// fp32, so this is the fp32 multiply followed by the rounding to bf16)
__device__ __forceinline__ uint32_t mul_bf16x2_rn(uint32_t v, uint32_t s2) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&v),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&s2));
  return *reinterpret_cast<const uint32_t *>(&r);
}

__global__ void __launch_bounds__(256)
combine_kernel(const uint4 *__restrict__ rows, const int32_t *__restrict__ slot_of_item,
               const int32_t *__restrict__ idx, const uint4 *__restrict__ shared_out,
               const unsigned short *__restrict__ shared_scale, int T,
               int vec_per_row, int K, uint4 *__restrict__ out) {
  __shared__ int s_slot[kMaxK];
  pdl_launch_dependents();
  pdl_wait();
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    if (threadIdx.x == 0) {
      // insertion sort of the K (expert id, slot) pairs, stable in slot order
      int eid[kMaxK], sl[kMaxK];
      for (int k = 0; k < K; ++k) {
        int e = idx[(size_t)t * K + k], s = slot_of_item[(size_t)t * K + k];
        int j = k;
        while (j > 0 && eid[j - 1] > e) { eid[j] = eid[j - 1]; sl[j] = sl[j - 1]; --j; }
        eid[j] = e; sl[j] = s;
      }
      for (int k = 0; k < K; ++k) s_slot[k] = sl[k];
    }
    __syncthreads();
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      uint4 acc = make_uint4(0, 0, 0, 0);   // the reference starts from zeros
      for (int k = 0; k < K; ++k) {
        int s = s_slot[k];
        if (s < 0) continue;
        acc = add_bf16x8_rn(acc, __ldg(rows + (size_t)s * vec_per_row + v));
      }
      if (shared_out != nullptr) {
        uint4 sh = __ldg(shared_out + (size_t)t * vec_per_row + v);
        if (shared_scale != nullptr) {      // the shared expert's scalar gate, applied here instead of by its GEMM
          const uint32_t g = (uint32_t)__ldg(shared_scale + t) * 0x10001u;
          sh = make_uint4(mul_bf16x2_rn(sh.x, g), mul_bf16x2_rn(sh.y, g), mul_bf16x2_rn(sh.z, g), mul_bf16x2_rn(sh.w, g));
        }
        acc = add_bf16x8_rn(acc, sh);
      }
      out[(size_t)t * vec_per_row + v] = acc;
    }
    __syncthreads();
  }
}

}  // namespace

int32_t launch_combine(const void *rows_out, const int32_t *slot_of_item, const int32_t *idx,
                       const void *shared_out, const void *shared_scale, int T, int H, int K, void *out,
                       cudaStream_t stream) {
  if (T < 0 || H <= 0 || H % 8 != 0 || K < 1 || K > kMaxK)
    return fail(SB_E_INVALID_ARG, "sb_combine: need H%%8==0 and 1<=K<=8 (T=%d H=%d K=%d)", T, H, K);
  if (T == 0) return SB_OK;
  if (!rows_out || !slot_of_item || !idx || !out)
    return fail(SB_E_INVALID_ARG, "sb_combine: null pointer");
  if (!aligned(rows_out, 16) || !aligned(out, 16) || (shared_out && !aligned(shared_out, 16)))
    return fail(SB_E_INVALID_ARG, "sb_combine: rows must be 16-byte aligned");
  int blocks = T;
  int max_blocks = sb_device_sm_count() * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  int threads = H / 8 >= 256 ? 256 : ((H / 8 + 31) / 32) * 32;
  SB_CUDA_CHECK(launch_pdl(combine_kernel, dim3(blocks), dim3(threads), 0, stream,
                           static_cast<const uint4 *>(rows_out), slot_of_item, idx,
                           static_cast<const uint4 *>(shared_out),
                           static_cast<const unsigned short *>(shared_out ? shared_scale : nullptr), T, H / 8, K,
                           static_cast<uint4 *>(out)));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // namespace sb
