// Kernels of the sparsely-gated ("MRN" / SGMoE) layer that the FastMoELayer path does not have:
// the token normalisation in front of the router and the experts, and the load / loss summary.
// They stand in, forward only, for the eager PyTorch of OrigSGMoEImpl
// (kernels/pytorch/mrn.py:186-189, :253-277, :301-333 of the reference). Both are HBM-bound or
// tiny; the router itself is the gate kernel in its normalised-logit mode (routing.cu) and the
// experts are the grouped GEMMs.
#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ void st_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One warp per (token, group): mean and biased variance over the group's `n` features in fp32
// (two passes over values that stay in L1), then (x - mean) * rsqrt(var + eps) * w + b.
// Layer norm: one group of n = d features, weight / bias per feature. Group norm of x viewed as
// [L, groups, n]: weight / bias per group (F.group_norm with num_channels == num_groups).
template <typename T>
__global__ void __launch_bounds__(256)
token_norm_kernel(const T* __restrict__ x, long long ldx, long long L, int groups, int n, const float* __restrict__ w,
                  const float* __restrict__ b, int per_group_affine, float eps, T* __restrict__ out, long long ldo) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = L * groups;
  for (long long seg = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; seg < total; seg += warps) {
    const long long t = seg / groups;
    const int g = static_cast<int>(seg - t * groups);
    const T* row = x + t * ldx + static_cast<long long>(g) * n;
    float s = 0.f;
    for (int c = lane; c < n; c += 32) s += ld_as_float<T>(row + c);
    const float mean = warp_sum(s) / n;
    float v = 0.f;
    for (int c = lane; c < n; c += 32) {
      const float dlt = ld_as_float<T>(row + c) - mean;
      v = fmaf(dlt, dlt, v);
    }
    const float rstd = rsqrtf(warp_sum(v) / n + eps);
    T* orow = out + t * ldo + static_cast<long long>(g) * n;
    for (int c = lane; c < n; c += 32) {
      const int a = per_group_affine ? g : c;
      const float y = (ld_as_float<T>(row + c) - mean) * rstd * (w ? w[a] : 1.f) + (b ? b[a] : 0.f);
      st_from_float(orow + c, y);
    }
  }
}

// Importance (sum of the gate values routed to each expert), load (rows per expert), the load
// fractions and loss = coef * (cv2(importance) + cv2(load)), cv2(v) = var(v) / (mean(v)^2 + 1e-6)
// with the unbiased variance, 0 for a single expert. One block; warp w sums the experts w, w + 8, ...
// in the fixed order of the expert-sorted rows, so the result is reproducible.
__global__ void __launch_bounds__(256)
sg_load_loss_kernel(const long long* __restrict__ offsets, const long long* __restrict__ gate_index,
                    const float* __restrict__ score, int E, int round_bf16, float loss_coef, int want_loss,
                    float* __restrict__ load_frac, float* __restrict__ loss) {
  extern __shared__ float s_imp[];                 // [E] importance, then [E] load
  float* s_load = s_imp + E;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += 8) {
    const long long p0 = offsets[e], p1 = offsets[e + 1];
    float acc = 0.f;
    for (long long p = p0 + lane; p < p1; p += 32) {
      float g = score[gate_index[p]];
      if (round_bf16) g = __bfloat162float(__float2bfloat16_rn(g));      // gates are cast to the token dtype first
      acc += g;
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      s_imp[e] = round_bf16 ? __bfloat162float(__float2bfloat16_rn(acc)) : acc;   // Tensor.sum returns the token dtype
      s_load[e] = static_cast<float>(p1 - p0);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const float total = static_cast<float>(offsets[E]);
    float cv[2] = {0.f, 0.f};
    for (int which = 0; which < 2; ++which) {
      const float* v = which == 0 ? s_imp : s_load;
      if (E > 1) {
        float mean = 0.f;
        for (int e = 0; e < E; ++e) mean += v[e];
        mean /= E;
        float var = 0.f;
        for (int e = 0; e < E; ++e) var += (v[e] - mean) * (v[e] - mean);
        var /= (E - 1);
        cv[which] = var / (mean * mean + 1e-6f);
      }
    }
    if (loss) *loss = want_loss ? (cv[0] + cv[1]) * loss_coef : 0.f;
    if (load_frac) {
      for (int e = 0; e < E; ++e) load_frac[e] = s_load[e] / total;
    }
  }
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_token_norm(const void* x, int dtype, int64_t L, int d, int64_t ldx, int num_groups,
                               const float* weight, const float* bias, int per_group_affine, float eps, void* out,
                               int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "token_norm: dtype must be bf16 or f32");
  FMOE_REQUIRE(L >= 0 && d >= 1 && num_groups >= 1 && d % num_groups == 0, "token_norm: d=%d must split into %d groups", d,
               num_groups);
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(x && out, "token_norm: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long segs = L * num_groups;
  long long blocks = (segs * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const int n = d / num_groups;
  if (dtype == FMOE_BF16) {
    token_norm_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, L, num_groups, n, weight, bias, per_group_affine, eps,
        static_cast<__nv_bfloat16*>(out), ldo);
  } else {
    token_norm_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const float*>(x), ldx, L, num_groups, n, weight, bias, per_group_affine, eps, static_cast<float*>(out), ldo);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_sg_load_loss(const int64_t* offsets, const int64_t* gate_index, const float* topk_score, int E,
                                 int round_bf16, float loss_coef, int want_loss, float* load_frac, float* loss,
                                 void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 4096, "sg_load_loss: E=%d outside [1, 4096]", E);
  FMOE_REQUIRE(offsets && gate_index && topk_score, "sg_load_loss: NULL pointer argument");
  sg_load_loss_kernel<<<1, 256, 2 * static_cast<size_t>(E) * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(gate_index), topk_score, E, round_bf16,
      loss_coef, want_loss, load_frac, loss);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}
