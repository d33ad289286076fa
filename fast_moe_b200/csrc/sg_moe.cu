// Kernels of the sparsely-gated ("MRN" / SGMoE) layer that the FastMoELayer path does not have:
// the token normalisation in front of the router and the experts, the training-time noise on the
// router logits with its smooth load estimate, and the load / loss summary.
// They stand in for the eager PyTorch of OrigSGMoEImpl (kernels/pytorch/mrn.py:186-189, :191-219,
// :221-277, :301-333 of the reference) and, further down, for what autograd makes of it. All are
// HBM-bound or tiny; the router itself is the gate kernel in its normalised-logit mode (routing.cu) and the
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

// Noisy gating while training (OrigSGMoEImpl._orig_noisy_gating, kernels/pytorch/mrn.py:229-237):
// logits2 holds, per token, the clean logits x @ w_gate in columns [0, E) and x @ w_noise in
// columns [E, 2E). stddev = softplus(x @ w_noise) + eps, noisy = clean + noise * stddev.
__global__ void __launch_bounds__(256)
noisy_logits_kernel(const float* __restrict__ logits2, long long ld, const float* __restrict__ noise, long long L, int E,
                    float eps, float* __restrict__ noisy, float* __restrict__ stddev) {
  const long long total = L * E;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / E;
    const int e = static_cast<int>(i - t * E);
    const float clean = logits2[t * ld + e];
    const float raw = logits2[t * ld + E + e];
    const float sp = raw > 20.f ? raw : log1pf(expf(raw));        // F.softplus (beta 1, threshold 20)
    const float sd = sp + eps;
    stddev[i] = sd;
    noisy[i] = __fadd_rn(clean, __fmul_rn(noise[i], sd));       // separate multiply and add, as the eager reference
  }
}

// Smooth load of the noisy router (OrigSGMoEImpl._prob_in_top_k, kernels/pytorch/mrn.py:191-219):
// for every token, the probability of each expert landing in the top k under a fresh noise draw,
//   Phi((clean - threshold) / stddev), threshold = the (k+1)-th largest L2-normalised noisy logit
// when the expert's noisy logit (compared un-normalised, as the reference does) exceeds it, else the
// k-th largest; summed over the tokens. One warp per token, lane l holds experts l, l + 32, ...;
// block b writes its sums to partials[b][E]. The sums run in a fixed order (tokens of a warp in
// sequence, then the warps of a block in sequence), so a result repeats bit for bit.
template <int VPL>
__global__ void __launch_bounds__(256)
noisy_load_kernel(const float* __restrict__ logits2, long long ld, const float* __restrict__ noisy,
                  const float* __restrict__ stddev, long long L, int E, int k, float* __restrict__ partials) {
  extern __shared__ float s_acc[];                 // [8 warps][E]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  float acc[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
  for (long long t = static_cast<long long>(blockIdx.x) * 8 + warp; t < L; t += static_cast<long long>(gridDim.x) * 8) {
    float v[VPL], nv[VPL];
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? noisy[t * E + e] : 0.f;
      sq = fmaf(v[j], v[j], sq);
    }
    const float nrm = fmaxf(sqrtf(warp_sum(sq)), 1e-12f);      // F.normalize: v / max(||v||, eps)
#pragma unroll
    for (int j = 0; j < VPL; ++j) nv[j] = (lane + 32 * j) < E ? v[j] / nrm : -INFINITY;
    // the k-th and (k+1)-th largest normalised values: k + 1 rounds of arg-max with removal
    unsigned removed = 0u;
    float thr_out = 0.f, thr_in = 0.f;
    for (int r = 0; r <= k; ++r) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int e = lane + 32 * j;
        if (e < E && !((removed >> j) & 1u) && (nv[j] > best || (nv[j] == best && e < best_e))) {
          best = nv[j];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if (best_e != 0x7fffffff && (best_e & 31) == lane) removed |= 1u << (best_e >> 5);
      if (r == k - 1) thr_out = best;
      if (r == k) thr_in = best;
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        const float clean = logits2[t * ld + e];
        const float thr = v[j] > thr_in ? thr_in : thr_out;
        const float z = (clean - thr) / stddev[t * E + e];
        acc[j] += 0.5f * (1.f + erff(z / 1.41421356237309515f));      // Normal(0, 1).cdf
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int e = lane + 32 * j;
    if (e < E) s_acc[warp * E + e] = acc[j];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += s_acc[w * E + e];
    partials[static_cast<long long>(blockIdx.x) * E + e] = s;
  }
}

// Importance (sum of the gate values routed to each expert), load (rows per expert), the load
// fractions and loss = coef * (cv2(importance) + cv2(load)), cv2(v) = var(v) / (mean(v)^2 + 1e-6)
// with the unbiased variance, 0 for a single expert. With noisy gating the loss uses the smooth
// load (per-block sums of noisy_load_kernel) instead of the row counts. One block; warp w sums the experts w, w + 8, ...
// in the fixed order of the expert-sorted rows, so the result is reproducible.
__global__ void __launch_bounds__(256)
sg_load_loss_kernel(const long long* __restrict__ offsets, const long long* __restrict__ gate_index,
                    const float* __restrict__ score, int E, int round_bf16, float loss_coef, int want_loss,
                    const float* __restrict__ load_partials, int n_partials, float* __restrict__ load_frac,
                    float* __restrict__ loss) {
  extern __shared__ float s_imp[];                 // [E] importance, [E] rows per expert, [E] the load the loss uses
  float* s_load = s_imp + E;
  float* s_cvload = s_load + E;
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
      float smooth = static_cast<float>(p1 - p0);
      if (load_partials) {                         // noisy gating: the smooth load, block sums in order
        smooth = 0.f;
        for (int b = 0; b < n_partials; ++b) smooth += load_partials[static_cast<long long>(b) * E + e];
      }
      s_cvload[e] = smooth;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const float total = static_cast<float>(offsets[E]);
    float cv[2] = {0.f, 0.f};
    for (int which = 0; which < 2; ++which) {
      const float* v = which == 0 ? s_imp : s_cvload;
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

// ---------------------------------------------------------------------------------------------
// Backward of the layer's own pieces (the reference gets them from torch autograd through its eager
// code, kernels/pytorch/mrn.py:221-333; its test compares them, kernels/tests/mrn_test.py:816-860).

// Token norm: one warp per (token, group). With xh = (x - mean) * rstd and g = d_out * w,
//   d_x = rstd * (g - mean(g) - xh * mean(g * xh)).
// Also leaves (mean, rstd) per segment in `stats` for the parameter-gradient pass.
template <typename T>
__global__ void __launch_bounds__(256)
token_norm_backward_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ dy, long long lddy, long long L,
                           int groups, int n, const float* __restrict__ w, int per_group_affine, float eps,
                           T* __restrict__ dx, long long lddx, float* __restrict__ stats) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long total = L * groups;
  for (long long seg = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; seg < total; seg += warps) {
    const long long t = seg / groups;
    const int g = static_cast<int>(seg - t * groups);
    const T* row = x + t * ldx + static_cast<long long>(g) * n;
    const T* drow = dy + t * lddy + static_cast<long long>(g) * n;
    float s = 0.f;
    for (int c = lane; c < n; c += 32) s += ld_as_float<T>(row + c);
    const float mean = warp_sum(s) / n;
    float v = 0.f;
    for (int c = lane; c < n; c += 32) {
      const float dlt = ld_as_float<T>(row + c) - mean;
      v = fmaf(dlt, dlt, v);
    }
    const float rstd = rsqrtf(warp_sum(v) / n + eps);
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < n; c += 32) {
      const int a = per_group_affine ? g : static_cast<int>(static_cast<long long>(g) * n + c);
      const float gg = ld_as_float<T>(drow + c) * (w ? w[a] : 1.f);
      const float xh = (ld_as_float<T>(row + c) - mean) * rstd;
      s1 += gg;
      s2 = fmaf(gg, xh, s2);
    }
    s1 = warp_sum(s1) / n;
    s2 = warp_sum(s2) / n;
    T* orow = dx + t * lddx + static_cast<long long>(g) * n;
    for (int c = lane; c < n; c += 32) {
      const int a = per_group_affine ? g : static_cast<int>(static_cast<long long>(g) * n + c);
      const float gg = ld_as_float<T>(drow + c) * (w ? w[a] : 1.f);
      const float xh = (ld_as_float<T>(row + c) - mean) * rstd;
      st_from_float(orow + c, rstd * (gg - s1 - xh * s2));
    }
    if (lane == 0 && stats) {
      stats[2 * seg] = mean;
      stats[2 * seg + 1] = rstd;
    }
  }
}

// Parameter gradients of the norm, first stage: thread c of chunk q sums, over the chunk's tokens,
// d_out[t, c] * xh[t, c] (weight) and d_out[t, c] (bias) -> partial[q][0 / 1][c]. Fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
norm_param_partial_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ dy, long long lddy, long long L, int d,
                          int groups, int n, const float* __restrict__ stats, int chunks, float* __restrict__ partial) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int q = blockIdx.y;
  if (c >= d) return;
  const long long per = (L + chunks - 1) / chunks;
  const long long t0 = q * per, t1 = min(L, t0 + per);
  const int g = c / n;
  float aw = 0.f, ab = 0.f;
  for (long long t = t0; t < t1; ++t) {
    const float mean = stats[2 * (t * groups + g)], rstd = stats[2 * (t * groups + g) + 1];
    const float go = ld_as_float<T>(dy + t * lddy + c);
    aw = fmaf(go, (ld_as_float<T>(x + t * ldx + c) - mean) * rstd, aw);
    ab += go;
  }
  partial[(static_cast<long long>(q) * 2 + 0) * d + c] = aw;
  partial[(static_cast<long long>(q) * 2 + 1) * d + c] = ab;
}

// Second stage: parameter a (a feature, or a whole group when the affine is per group) sums its
// partials over chunks and, per group, over the group's features. One warp per parameter.
__global__ void __launch_bounds__(256)
norm_param_reduce_kernel(const float* __restrict__ partial, int chunks, int d, int n_params, int span,
                         float* __restrict__ d_weight, float* __restrict__ d_bias) {
  const int lane = threadIdx.x & 31;
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (a >= n_params) return;
  float sw = 0.f, sb = 0.f;
  const int total = chunks * span;
  for (int i = lane; i < total; i += 32) {
    const int q = i / span;
    const int c = a * span + (i - q * span);
    sw += partial[(static_cast<long long>(q) * 2 + 0) * d + c];
    sb += partial[(static_cast<long long>(q) * 2 + 1) * d + c];
  }
  sw = warp_sum(sw);
  sb = warp_sum(sb);
  if (lane == 0) {
    if (d_weight) d_weight[a] = sw;
    if (d_bias) d_bias[a] = sb;
  }
}

// Router backward: scores = softmax(l / max(||l||, eps)) at the k chosen experts, not renormalised.
// One warp per token, lane j holds experts j, j + 32, ...
template <int VPL>
__global__ void __launch_bounds__(256)
sg_router_backward_kernel(const float* __restrict__ logits, const long long* __restrict__ idx,
                          const float* __restrict__ d_score, long long L, int E, int k, float* __restrict__ d_logits) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < L; t += warps) {
    float l[VPL], nv[VPL], p[VPL], dp[VPL];
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      l[j] = e < E ? logits[t * E + e] : 0.f;
      sq = fmaf(l[j], l[j], sq);
    }
    const float nrm = fmaxf(sqrtf(warp_sum(sq)), 1e-12f);
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      nv[j] = l[j] / nrm;
      if (lane + 32 * j < E) mx = fmaxf(mx, nv[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      p[j] = (lane + 32 * j) < E ? expf(nv[j] - mx) : 0.f;
      z += p[j];
    }
    z = warp_sum(z);
    float sdot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      p[j] /= z;
      dp[j] = 0.f;
      for (int s = 0; s < k; ++s)
        if (idx[t * k + s] == e) dp[j] += d_score[t * k + s];
      sdot = fmaf(p[j], dp[j], sdot);
    }
    sdot = warp_sum(sdot);
    float ndot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      dp[j] = p[j] * (dp[j] - sdot);            // d_n
      ndot = fmaf(nv[j], dp[j], ndot);
    }
    ndot = warp_sum(ndot);
    const bool clamped = nrm <= 1e-12f;         // F.normalize divides by the constant eps then
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      if (e < E) d_logits[t * E + e] = (clamped ? dp[j] : (dp[j] - nv[j] * ndot)) / nrm;
    }
  }
}

// Router backward with noisy gating (training): the logits that were routed on are
//   noisy = clean + noise * stddev,  stddev = softplus(raw) + eps,  clean = x @ w_gate, raw = x @ w_noise,
// and the loss also holds the smooth load  sum_t Phi((clean - thr) / stddev)  whose thresholds are
// the k-th / (k+1)-th largest normalised noisy logits of the token (kernels/pytorch/mrn.py:191-252).
// Per token: d_n from the k scores (softmax over all experts) plus the thresholds' share of the
// load gradient, the normalisation's backward, then d_clean and d_raw. `g_load` [E] is
// d loss / d load (NULL: the load takes no part, e.g. k == E). One warp per token.
template <int VPL>
__global__ void __launch_bounds__(256)
sg_noisy_router_backward_kernel(const float* __restrict__ logits2, long long ld, const float* __restrict__ noise,
                                const float* __restrict__ noisy, const float* __restrict__ stddev,
                                const long long* __restrict__ idx, const float* __restrict__ d_score,
                                const float* __restrict__ g_load, long long L, int E, int k,
                                float* __restrict__ d_logits2, long long ldd) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < L; t += warps) {
    float l[VPL], nv[VPL], p[VPL], dn[VPL];
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      l[j] = e < E ? noisy[t * E + e] : 0.f;
      sq = fmaf(l[j], l[j], sq);
    }
    const float nrm = fmaxf(sqrtf(warp_sum(sq)), 1e-12f);
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      nv[j] = (lane + 32 * j) < E ? l[j] / nrm : -INFINITY;
      mx = fmaxf(mx, nv[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      p[j] = (lane + 32 * j) < E ? expf(nv[j] - mx) : 0.f;
      z += p[j];
    }
    z = warp_sum(z);
    float sdot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      p[j] /= z;
      dn[j] = 0.f;
      for (int s = 0; s < k; ++s)
        if (idx[t * k + s] == e) dn[j] += d_score[t * k + s];
      sdot = fmaf(p[j], dn[j], sdot);
    }
    sdot = warp_sum(sdot);
#pragma unroll
    for (int j = 0; j < VPL; ++j) dn[j] = p[j] * (dn[j] - sdot);
    // ---- the smooth load's share
    float dc[VPL], dsd[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) dc[j] = dsd[j] = 0.f;
    if (g_load != nullptr && k < E) {
      unsigned removed = 0u;
      float thr_out = 0.f, thr_in = 0.f;
      int e_out = -1, e_in = -1;
      for (int r = 0; r <= k; ++r) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          const int e = lane + 32 * j;
          if (e < E && !((removed >> j) & 1u) && (nv[j] > best || (nv[j] == best && e < best_e))) {
            best = nv[j];
            best_e = e;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
          if (ob > best || (ob == best && oe < best_e)) {
            best = ob;
            best_e = oe;
          }
        }
        if (best_e != 0x7fffffff && (best_e & 31) == lane) removed |= 1u << (best_e >> 5);
        if (r == k - 1) { thr_out = best; e_out = best_e; }
        if (r == k) { thr_in = best; e_in = best_e; }
      }
      float d_in = 0.f, d_out = 0.f;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int e = lane + 32 * j;
        if (e < E) {
          const float clean = logits2[t * ld + e];
          const float sd = stddev[t * E + e];
          const bool in = l[j] > thr_in;
          const float zz = (clean - (in ? thr_in : thr_out)) / sd;
          const float c = g_load[e] * expf(-0.5f * zz * zz) * 0.3989422804014327f / sd;   // G * pdf(z) / stddev
          dc[j] = c;
          dsd[j] = -c * zz;
          if (in) d_in -= c; else d_out -= c;
        }
      }
      d_in = warp_sum(d_in);
      d_out = warp_sum(d_out);
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int e = lane + 32 * j;
        if (e == e_in) dn[j] += d_in;
        if (e == e_out) dn[j] += d_out;
      }
    }
    float ndot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
      if (lane + 32 * j < E) ndot = fmaf(nv[j], dn[j], ndot);
    ndot = warp_sum(ndot);
    const bool clamped = nrm <= 1e-12f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        const float dl = (clamped ? dn[j] : (dn[j] - nv[j] * ndot)) / nrm;      // d loss / d noisy
        const float raw = logits2[t * ld + E + e];
        const float sig = raw > 20.f ? 1.f : 1.f / (1.f + expf(-raw));          // softplus'
        d_logits2[t * ldd + e] = dl + dc[j];
        d_logits2[t * ldd + E + e] = (dl * noise[t * E + e] + dsd[j]) * sig;
      }
    }
  }
}

// d loss / d scores: loss = coef * (cv2(importance) + cv2(load)); only the importance (sum of the
// gate values per expert) depends on the scores. One block: importance as the forward sums it, its
// cv2 derivative per expert, then every chosen (token, slot) receives its expert's value.
__global__ void __launch_bounds__(256)
sg_loss_backward_kernel(const long long* __restrict__ offsets, const long long* __restrict__ gate_index,
                        const float* __restrict__ score, int E, int round_bf16, float loss_coef,
                        const float* __restrict__ d_loss, float* __restrict__ d_score,
                        const float* __restrict__ load_partials, int n_partials, float* __restrict__ d_load) {
  extern __shared__ float s_imp[];                 // [E] importance, then its gradient
  // with noisy gating the loss's second term is cv2 of the smooth load: its derivative per expert
  if (load_partials != nullptr && d_load != nullptr && threadIdx.x == 0) {
    float mean = 0.f;
    for (int e = 0; e < E; ++e) {
      float v = 0.f;
      for (int b = 0; b < n_partials; ++b) v += load_partials[static_cast<long long>(b) * E + e];
      d_load[e] = v;                               // the load itself for now
      mean += v;
    }
    mean /= E;
    float var = 0.f;
    for (int e = 0; e < E; ++e) var += (d_load[e] - mean) * (d_load[e] - mean);
    var = E > 1 ? var / (E - 1) : 0.f;
    const float den = mean * mean + 1e-6f;
    const float sc = loss_coef * (d_loss ? *d_loss : 1.f);
    for (int e = 0; e < E; ++e) {
      const float g = E > 1 ? (2.f * (d_load[e] - mean) / ((E - 1) * den) - var * 2.f * mean / (E * den * den)) : 0.f;
      d_load[e] = g * sc;
    }
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += 8) {
    float acc = 0.f;
    for (long long p = offsets[e] + lane; p < offsets[e + 1]; p += 32) {
      float g = score[gate_index[p]];
      if (round_bf16) g = __bfloat162float(__float2bfloat16_rn(g));
      acc += g;
    }
    acc = warp_sum(acc);
    if (lane == 0) s_imp[e] = round_bf16 ? __bfloat162float(__float2bfloat16_rn(acc)) : acc;
  }
  __syncthreads();
  __shared__ float s_mean, s_var;
  if (threadIdx.x == 0) {
    float mean = 0.f;
    for (int e = 0; e < E; ++e) mean += s_imp[e];
    mean /= E;
    float var = 0.f;
    for (int e = 0; e < E; ++e) var += (s_imp[e] - mean) * (s_imp[e] - mean);
    s_mean = mean;
    s_var = E > 1 ? var / (E - 1) : 0.f;
  }
  __syncthreads();
  const float scale = loss_coef * (d_loss ? *d_loss : 1.f);
  const float den = s_mean * s_mean + 1e-6f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float g = E > 1 ? (2.f * (s_imp[e] - s_mean) / ((E - 1) * den) - s_var * 2.f * s_mean / (E * den * den)) : 0.f;
    s_imp[e] = g * scale;
  }
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    const float g = s_imp[e];
    for (long long p = offsets[e] + threadIdx.x; p < offsets[e + 1]; p += blockDim.x) d_score[gate_index[p]] = g;
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

extern "C" int fmoe_sg_noisy_logits(const float* logits2, int64_t ld_logits, const float* noise, int64_t L, int E,
                                    float noise_eps, float* noisy, float* stddev, void* stream) {
  FMOE_REQUIRE(E >= 1 && L >= 0 && ld_logits >= 2ll * E, "sg_noisy_logits: logits must hold 2 * E = %d columns per token", 2 * E);
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(logits2 && noise && noisy && stddev, "sg_noisy_logits: NULL pointer argument");
  long long blocks = (L * E + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  noisy_logits_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      logits2, ld_logits, noise, L, E, noise_eps, noisy, stddev);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_sg_noisy_load(const float* logits2, int64_t ld_logits, const float* noisy, const float* stddev,
                                  int64_t L, int E, int k, float* partials, int n_partials, void* stream) {
  FMOE_REQUIRE(E >= 2 && E <= 256, "sg_noisy_load: E=%d outside [2, 256]", E);
  FMOE_REQUIRE(k >= 1 && k < E, "sg_noisy_load: k=%d must be in [1, E) (with k = E every expert is picked)", k);
  FMOE_REQUIRE(n_partials >= 1 && n_partials <= 1024, "sg_noisy_load: n_partials=%d outside [1, 1024]", n_partials);
  FMOE_REQUIRE(L >= 0 && ld_logits >= E, "sg_noisy_load: bad L or row stride");
  FMOE_REQUIRE(partials && (L == 0 || (logits2 && noisy && stddev)), "sg_noisy_load: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = 8 * static_cast<size_t>(E) * sizeof(float);
  const int vpl = (E + 31) / 32;
#define FMOE_NOISY_LOAD(V) \
  noisy_load_kernel<V><<<n_partials, 256, smem, st>>>(logits2, ld_logits, noisy, stddev, L, E, k, partials)
  if (vpl <= 1) FMOE_NOISY_LOAD(1);
  else if (vpl <= 2) FMOE_NOISY_LOAD(2);
  else if (vpl <= 4) FMOE_NOISY_LOAD(4);
  else FMOE_NOISY_LOAD(8);
#undef FMOE_NOISY_LOAD
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_sg_load_loss(const int64_t* offsets, const int64_t* gate_index, const float* topk_score, int E,
                                 int round_bf16, float loss_coef, int want_loss, const float* load_partials,
                                 int n_partials, float* load_frac, float* loss, void* stream) {
  FMOE_REQUIRE(load_partials == nullptr || n_partials >= 1, "sg_load_loss: load_partials given with n_partials=%d", n_partials);
  FMOE_REQUIRE(E >= 1 && E <= 4096, "sg_load_loss: E=%d outside [1, 4096]", E);
  FMOE_REQUIRE(offsets && gate_index && topk_score, "sg_load_loss: NULL pointer argument");
  sg_load_loss_kernel<<<1, 256, 3 * static_cast<size_t>(E) * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(gate_index), topk_score, E, round_bf16,
      loss_coef, want_loss, load_partials, n_partials, load_frac, loss);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_token_norm_backward(const void* x, const void* d_out, int dtype, int64_t L, int d, int64_t ldx,
                                        int64_t ld_dout, int num_groups, const float* weight, int per_group_affine,
                                        float eps, void* d_x, int64_t ld_dx, float* stats, float* partial, int chunks,
                                        float* d_weight, float* d_bias, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "token_norm_backward: dtype must be bf16 or f32");
  FMOE_REQUIRE(L >= 0 && d >= 1 && num_groups >= 1 && d % num_groups == 0, "token_norm_backward: d=%d must split into %d groups",
               d, num_groups);
  const bool params = d_weight != nullptr || d_bias != nullptr;
  FMOE_REQUIRE(!params || (stats && partial && chunks >= 1 && chunks <= 1024),
               "token_norm_backward: parameter gradients need the stats and partial scratch and 1..1024 chunks");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = d / num_groups;
  const int n_params = per_group_affine ? num_groups : d;
  if (L == 0) {
    if (d_weight) FMOE_CUDA_OK(cudaMemsetAsync(d_weight, 0, n_params * sizeof(float), st));
    if (d_bias) FMOE_CUDA_OK(cudaMemsetAsync(d_bias, 0, n_params * sizeof(float), st));
    return FMOE_OK;
  }
  FMOE_REQUIRE(x && d_out && d_x, "token_norm_backward: NULL pointer argument");
  const long long segs = L * num_groups;
  long long blocks = (segs * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dim3 pgrid((d + 255) / 256, chunks > 0 ? chunks : 1);
  if (dtype == FMOE_BF16) {
    using T = __nv_bfloat16;
    token_norm_backward_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const T*>(x), ldx, static_cast<const T*>(d_out), ld_dout, L, num_groups, n, weight, per_group_affine, eps,
        static_cast<T*>(d_x), ld_dx, stats);
    if (params)
      norm_param_partial_kernel<T><<<pgrid, 256, 0, st>>>(static_cast<const T*>(x), ldx, static_cast<const T*>(d_out), ld_dout,
                                                          L, d, num_groups, n, stats, chunks, partial);
  } else {
    token_norm_backward_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const float*>(x), ldx, static_cast<const float*>(d_out), ld_dout, L, num_groups, n, weight,
        per_group_affine, eps, static_cast<float*>(d_x), ld_dx, stats);
    if (params)
      norm_param_partial_kernel<float><<<pgrid, 256, 0, st>>>(static_cast<const float*>(x), ldx,
                                                              static_cast<const float*>(d_out), ld_dout, L, d, num_groups, n,
                                                              stats, chunks, partial);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  if (params) {
    ++g_misc_launches;                                   // the partial-sum launch above
    norm_param_reduce_kernel<<<(n_params * 32 + 255) / 256, 256, 0, st>>>(partial, chunks, d, n_params,
                                                                         per_group_affine ? n : 1, d_weight, d_bias);
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
  }
  return FMOE_OK;
}

extern "C" int fmoe_sg_router_backward(const float* logits, const int64_t* topk_idx, const float* d_score, int64_t L, int E,
                                       int k, float* d_logits, void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 256 && k >= 1 && k <= E && L >= 0, "sg_router_backward: E=%d (<= 256), k=%d out of range", E, k);
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(logits && topk_idx && d_score && d_logits, "sg_router_backward: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (L * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const long long* idx = reinterpret_cast<const long long*>(topk_idx);
  const int vpl = (E + 31) / 32;
#define FMOE_SG_RB(V) sg_router_backward_kernel<V><<<static_cast<unsigned>(blocks), 256, 0, st>>>(logits, idx, d_score, L, E, k, d_logits)
  if (vpl <= 1) FMOE_SG_RB(1);
  else if (vpl <= 2) FMOE_SG_RB(2);
  else if (vpl <= 4) FMOE_SG_RB(4);
  else FMOE_SG_RB(8);
#undef FMOE_SG_RB
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_sg_loss_backward(const int64_t* offsets, const int64_t* gate_index, const float* topk_score, int E,
                                     int round_bf16, float loss_coef, const float* d_loss, float* d_score,
                                     const float* load_partials, int n_partials, float* d_load, void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 4096, "sg_loss_backward: E=%d outside [1, 4096]", E);
  FMOE_REQUIRE(offsets && gate_index && topk_score && d_score, "sg_loss_backward: NULL pointer argument");
  FMOE_REQUIRE((load_partials == nullptr) == (d_load == nullptr) && (load_partials == nullptr || n_partials >= 1),
               "sg_loss_backward: load_partials and d_load go together");
  sg_loss_backward_kernel<<<1, 256, static_cast<size_t>(E) * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(gate_index), topk_score, E, round_bf16,
      loss_coef, d_loss, d_score, load_partials, n_partials, d_load);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_sg_noisy_router_backward(const float* logits2, int64_t ld_logits, const float* noise,
                                             const float* noisy, const float* stddev, const int64_t* topk_idx,
                                             const float* d_score, const float* d_load, int64_t L, int E, int k,
                                             float* d_logits2, int64_t ld_d, void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 256 && k >= 1 && k <= E && L >= 0, "sg_noisy_router_backward: E=%d (<= 256), k=%d out of range", E, k);
  FMOE_REQUIRE(ld_logits >= 2ll * E && ld_d >= 2ll * E, "sg_noisy_router_backward: rows must hold 2 * E columns");
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(logits2 && noise && noisy && stddev && topk_idx && d_score && d_logits2,
               "sg_noisy_router_backward: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (L * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const long long* idx = reinterpret_cast<const long long*>(topk_idx);
  const int vpl = (E + 31) / 32;
#define FMOE_SG_NRB(V)                                                                                                  \
  sg_noisy_router_backward_kernel<V><<<static_cast<unsigned>(blocks), 256, 0, st>>>(logits2, ld_logits, noise, noisy, stddev, \
                                                                                    idx, d_score, d_load, L, E, k, d_logits2, ld_d)
  if (vpl <= 1) FMOE_SG_NRB(1);
  else if (vpl <= 2) FMOE_SG_NRB(2);
  else if (vpl <= 4) FMOE_SG_NRB(4);
  else FMOE_SG_NRB(8);
#undef FMOE_SG_NRB
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}
