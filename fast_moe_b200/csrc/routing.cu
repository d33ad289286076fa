// Routing kernels: gate logits -> softmax -> top-k -> renormalised scores, and the stable
// counting sort that turns the [L, k] expert choices into per-expert jagged offsets and the
// permutation tensors the expert GEMMs and the combine consume.
//
// Replaces the eager ATen sequence of the reference (modules/fast_moe_module.py:93-144:
// softmax, topk, scatter_, mul, normalize, two stable sorts, floor-divide, sum, gather, cumsum,
// max + device-to-host sync). All of this is integer / HBM-bound work: one pass over x for the
// logits, one pass over the [L, k] indices for the histogram and one for the placement.
#include <atomic>

#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

constexpr int kGateWarps = 8;
constexpr int kMaxGateExperts = 256;
constexpr int kRouteBlock = 256;   // tokens per block in the counting sort

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Eight consecutive fp32 values of a row starting at element c (c a multiple of 8).
__device__ __forceinline__ void load8(const float* row, int c, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(row + c);
  const float4 b = *reinterpret_cast<const float4*>(row + c + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* row, int c, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

constexpr int kGateEC = 8;       // experts per pass over the rows

// What happens between the logits and the k scores:
//   kRouterSoftmaxRenorm  softmax over the experts, top-k, the k scores renormalised to sum 1
//                         (FastMoELayer._select_top_k_experts, modules/fast_moe_module.py:93-105)
//   kRouterNormalised     logits divided by their L2 norm, softmax over the experts, top-k, the k
//                         probabilities kept as they are (OrigSGMoEImpl._orig_noisy_gating without
//                         noise, kernels/pytorch/mrn.py:236-252; utils/utils.py:139-164)
constexpr int kRouterSoftmaxRenorm = 0;
constexpr int kRouterNormalised = 1;

// One warp per kGateTokens tokens (4, 2 or 1: as many as still leave every SM a few warps per
// scheduler). Logits are accumulated in fp32 with the reduction order fixed by the lane layout, so
// the same input always routes the same way. x is read in 16-byte pieces and each gate-weight
// piece is used for all the warp's tokens; HBM traffic is one pass over x.
// W_SMEM: the block first copies the gate weights into shared memory and reads them from there.
// Every token needs all of them, and read through L1 they were evicted by the streaming x rows
// and came from L2 again and again (the kernel ran at a tenth of the HBM rate).
template <typename XT, int kGateTokens, bool W_SMEM>
__global__ void __launch_bounds__(kGateWarps * 32)
gate_topk_kernel(const XT* __restrict__ x, long long ldx, const float* __restrict__ gw,
                 const float* __restrict__ gb, const float* __restrict__ logits_in, long long ld_logits, int split,
                 long long L, int d, int E, int k, int vec_ok, float* __restrict__ logits_out, long long* __restrict__ topk_idx,
                 float* __restrict__ topk_score, int router_mode) {
  __shared__ float s_logit[kGateWarps][kGateTokens][kMaxGateExperts];
  extern __shared__ __align__(16) float s_gw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if constexpr (W_SMEM) {
    const int n4 = (E * d) >> 2;     // the host checked: E * d a multiple of 4, gw 16-byte aligned
    for (int i = threadIdx.x; i < n4; i += kGateWarps * 32) {
      reinterpret_cast<float4*>(s_gw)[i] = reinterpret_cast<const float4*>(gw)[i];
    }
    __syncthreads();
    gw = s_gw;
  }
  const long long num_groups = (L + kGateTokens - 1) / kGateTokens;
  for (long long grp = static_cast<long long>(blockIdx.x) * kGateWarps + warp; grp < num_groups;
       grp += static_cast<long long>(gridDim.x) * kGateWarps) {
  const long long t0 = grp * kGateTokens;
  const int nt = static_cast<int>(min(static_cast<long long>(kGateTokens), L - t0));

  if (logits_in != nullptr) {
    // logits computed elsewhere (tensor-core product): row stride ld_logits; with `split` the
    // product was done on a two-term bf16 expansion of the gate weights and the halves are summed
    for (int j = 0; j < nt; ++j)
      for (int e = lane; e < E; e += 32) {
        const float* row = logits_in + (t0 + j) * ld_logits;
        float v = row[e];
        if (split) v += row[E + e];
        s_logit[warp][j][e] = v + (gb ? gb[e] : 0.f);
      }
  } else {
    const int d8 = vec_ok ? (d & ~7) : 0;
    for (int e0 = 0; e0 < E; e0 += kGateEC) {
      float acc[kGateTokens][kGateEC];
#pragma unroll
      for (int j = 0; j < kGateTokens; ++j)
#pragma unroll
        for (int i = 0; i < kGateEC; ++i) acc[j][i] = 0.f;
      for (int c = lane * 8; c < d8; c += 256) {
        float xv[kGateTokens][8];
#pragma unroll
        for (int j = 0; j < kGateTokens; ++j) {
          if (j < nt) {
            load8(x + (t0 + j) * ldx, c, xv[j]);
          } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) xv[j][u] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < kGateEC; ++i) {
          if (e0 + i < E) {
            float wv[8];
            load8(gw + static_cast<long long>(e0 + i) * d, c, wv);
#pragma unroll
            for (int j = 0; j < kGateTokens; ++j)
#pragma unroll
              for (int u = 0; u < 8; ++u) acc[j][i] = fmaf(xv[j][u], wv[u], acc[j][i]);
          }
        }
      }
      for (int c = d8 + lane; c < d; c += 32) {   // tail, or everything when rows are not 16-byte aligned
#pragma unroll
        for (int i = 0; i < kGateEC; ++i) {
          if (e0 + i < E) {
            const float w = gw[static_cast<long long>(e0 + i) * d + c];
#pragma unroll
            for (int j = 0; j < kGateTokens; ++j)
              if (j < nt) acc[j][i] = fmaf(to_f<XT>(x[(t0 + j) * ldx + c]), w, acc[j][i]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kGateTokens; ++j) {
#pragma unroll
        for (int i = 0; i < kGateEC; ++i) {
          float v = acc[j][i];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0 && e0 + i < E) s_logit[warp][j][e0 + i] = v + (gb ? gb[e0 + i] : 0.f);
        }
      }
    }
  }
  __syncwarp();
  for (int j = 0; j < nt; ++j) {
    const long long t = t0 + j;
    float* lg = s_logit[warp][j];
    if (logits_out != nullptr) {
      for (int e = lane; e < E; e += 32) logits_out[t * E + e] = lg[e];
    }
    if (router_mode == kRouterNormalised) {
      // F.normalize(logits, dim=1): divide by max(||logits||_2, 1e-12)
      float sq = 0.f;
      for (int e = lane; e < E; e += 32) sq = fmaf(lg[e], lg[e], sq);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
      for (int e = lane; e < E; e += 32) lg[e] *= inv;
      __syncwarp();
    }
    // softmax over E
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float pr = expf(lg[e] - mx);
      lg[e] = pr;
      sum += pr;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    // top-k by repeated arg-max; a taken entry is marked with -1 (scores are >= 0)
    float norm = 0.f;
    for (int s = 0; s < k; ++s) {
      float best = -2.f;
      int best_e = E;
      for (int e = lane; e < E; e += 32) {
        const float v = lg[e];
        if (v > best) {   // ascending e within the lane: first maximum wins
          best = v;
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ov > best || (ov == best && oe < best_e)) {
          best = ov;
          best_e = oe;
        }
      }
      const float sc = best / sum;
      norm += sc;
      if (lane == 0) {
        topk_idx[t * k + s] = best_e;
        topk_score[t * k + s] = sc;
        lg[best_e] = -1.f;
      }
      __syncwarp();
    }
    // F.normalize(p=1, eps=1e-12) over the k kept scores (the normalised-logit router keeps the
    // softmax probabilities as they are)
    const float denom = fmaxf(norm, 1e-12f);
    if (lane == 0 && router_mode == kRouterSoftmaxRenorm) {
      for (int s = 0; s < k; ++s) topk_score[t * k + s] = topk_score[t * k + s] / denom;
    }
  }
  __syncwarp();      // s_logit is reused by this warp's next group
  }
}

// ---- gate logits on the warp-level tensor cores ---------------------------------------------
// bf16 tokens, few experts: the logits are a skinny product [L, d] x [d, E] whose CUDA-core form
// issues ~1200 instructions per token. Here a block of 8 warps takes 32 tokens: warp w multiplies
// the 16 tokens of tile (w >> 2) by the quarter (w & 3) of the columns with mma.sync m16n8k16,
// the four partial sums meet in shared memory, and 32 threads finish one token each (softmax,
// top-k, renormalisation - the same arithmetic, in the same order, as gate_topk_kernel).
// The fp32 gate weights are split on the fly into three bf16 terms (hi + mid + lo reproduces
// every weight to 2^-24), so the products are exact and only the fp32 accumulation order
// differs from the CUDA-core kernel.
//
// Fragment layout trick: the reduction index of an MMA may be any permutation of the columns as
// long as both operands use the same one. Lane (g = lane / 4, q = lane % 4) therefore loads 16
// contiguous bytes of token row g (and g + 8) at column k0 + 8 q, and 16 bytes of each weight
// term of expert g at the same column: registers 0,1 feed one MMA, registers 2,3 the next.
constexpr int kMmaGateWarps = 8;
constexpr int kMmaGateTokens = 32;            // per block
constexpr int kMmaGatePadBytes = 64;          // row padding of the weight terms: conflict-free 16-byte reads

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>   // experts handled = 8 * NT (E rounded up; the padding experts have zero weights)
__global__ void __launch_bounds__(kMmaGateWarps * 32, 2)
gate_topk_mma_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ gw,
                     const float* __restrict__ gb, long long L, int d, int E, int k,
                     float* __restrict__ logits_out, long long* __restrict__ topk_idx,
                     float* __restrict__ topk_score, int* __restrict__ group_counts, int router_mode,
                     uint8_t* __restrict__ zero_rows, long long ldz_bytes, int zero_row_bytes) {
  constexpr int EP = 8 * NT;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel's set-up may start
  extern __shared__ __align__(16) uint8_t smem_gate[];
  const int row_bytes = d * 2 + kMmaGatePadBytes;
  uint8_t* s_w = smem_gate;                                            // [3 terms][EP][row_bytes]
  float* s_part = reinterpret_cast<float*>(smem_gate + 3 * EP * row_bytes);   // [4][32][EP + 1]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int q = lane & 3;
  const int tile = warp >> 2;
  const int kc = warp & 3;
  // this warp's columns: a quarter of d, rounded up to whole 32-column steps
  const int chunk = ((d + 3) / 4 + 31) & ~31;
  const int c_begin = kc * chunk;
  const int c_end = min(d, c_begin + chunk);
  const int steps = c_begin < c_end ? (c_end - c_begin + 31) >> 5 : 0;
  const long long num_tiles = (L + kMmaGateTokens - 1) / kMmaGateTokens;

  // Token rows of a block's 32-token tile, 16 bytes per lane and row, kDepth steps at a time.
  constexpr int kDepth = 8;                       // 32-column steps held in registers at once
  uint4 xa[kDepth], xb[kDepth];
  auto load_rows = [&](long long tile_id, int s0) {
    const long long r0 = tile_id * kMmaGateTokens + tile * 16 + g;
    const __nv_bfloat16* row0 = x + r0 * ldx;
    const __nv_bfloat16* row1 = x + (r0 + 8) * ldx;
    const bool ok0 = r0 < L;
    const bool ok1 = r0 + 8 < L;
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
      const int c = c_begin + (s0 + i) * 32 + q * 8;
      const bool in = (s0 + i) < steps && c < c_end;
      xa[i] = (in && ok0) ? *reinterpret_cast<const uint4*>(row0 + c) : make_uint4(0, 0, 0, 0);
      xb[i] = (in && ok1) ? *reinterpret_cast<const uint4*>(row1 + c) : make_uint4(0, 0, 0, 0);
    }
  };
  // the first tile's rows go out first (HBM latency); the weight staging runs underneath them
  load_rows(blockIdx.x, 0);
  // Optional side job: clear one row per token of a caller's buffer (the accumulator a fused
  // combine adds into). Stores only, issued while the loads above are in flight.
  if (zero_rows != nullptr) {
    const int vec = zero_row_bytes >> 4;
    for (long long tile_id = blockIdx.x; tile_id < num_tiles; tile_id += gridDim.x) {
      for (int r = warp; r < kMmaGateTokens; r += kMmaGateWarps) {
        const long long t = tile_id * kMmaGateTokens + r;
        if (t >= L) break;
        uint4* z = reinterpret_cast<uint4*>(zero_rows + t * ldz_bytes);
        for (int c = lane; c < vec; c += 32) z[c] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  // gate weights -> three bf16 terms in shared memory (zero rows for the padding experts),
  // four weights per thread and step, four steps in flight
  {
    const int quads_per_row = d >> 2;
    const int quads = EP * quads_per_row;
    constexpr int kUnroll = 4;
    for (int i0 = threadIdx.x; i0 < quads; i0 += kMmaGateWarps * 32 * kUnroll) {
      float4 w[kUnroll];
      int ee[kUnroll], cc[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = i0 + u * kMmaGateWarps * 32;
        ee[u] = i / quads_per_row;
        cc[u] = (i - ee[u] * quads_per_row) * 4;
        w[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < quads && ee[u] < E) w[u] = *reinterpret_cast<const float4*>(gw + static_cast<long long>(ee[u]) * d + cc[u]);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (i0 + u * kMmaGateWarps * 32 < quads) {
          const float wf[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
          uint32_t t3[3][2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const __nv_bfloat162 hi = __floats2bfloat162_rn(wf[2 * h], wf[2 * h + 1]);
            const float2 hf = __bfloat1622float2(hi);
            const float2 r1 = make_float2(wf[2 * h] - hf.x, wf[2 * h + 1] - hf.y);
            const __nv_bfloat162 mid = __floats2bfloat162_rn(r1.x, r1.y);
            const float2 mf = __bfloat1622float2(mid);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(r1.x - mf.x, r1.y - mf.y);
            t3[0][h] = *reinterpret_cast<const uint32_t*>(&hi);
            t3[1][h] = *reinterpret_cast<const uint32_t*>(&mid);
            t3[2][h] = *reinterpret_cast<const uint32_t*>(&lo);
          }
          uint8_t* dst = s_w + ee[u] * row_bytes + cc[u] * 2;
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            *reinterpret_cast<uint2*>(dst + term * EP * row_bytes) = make_uint2(t3[term][0], t3[term][1]);
          }
        }
      }
    }
  }
  __syncthreads();

  for (long long tile_id = blockIdx.x; tile_id < num_tiles; tile_id += gridDim.x) {
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
  for (int s0 = 0; s0 < steps; s0 += kDepth) {
    if (s0 > 0) load_rows(tile_id, s0);
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
      if (s0 + i < steps) {       // warp-uniform: mma.sync needs all 32 lanes
        // Lanes whose 8 columns lie past the end hold zero token values; they read the last
        // valid weight columns instead (finite numbers, multiplied by zero) and take part in
        // the MMA like every other lane.
        const int c = min(c_begin + (s0 + i) * 32 + q * 8, d - 8);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint8_t* wrow = s_w + (n * 8 + g) * row_bytes + c * 2;
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const uint4 wv = *reinterpret_cast<const uint4*>(wrow + term * EP * row_bytes);
            mma_bf16_16816(acc[n], xa[i].x, xb[i].x, xa[i].y, xb[i].y, wv.x, wv.y);
            mma_bf16_16816(acc[n], xa[i].z, xb[i].z, xa[i].w, xb[i].w, wv.z, wv.w);
          }
        }
      }
    }
  }
  // the next tile's rows travel while this one is finished
  if (tile_id + gridDim.x < num_tiles) load_rows(tile_id + gridDim.x, 0);
  // accumulator fragment: acc[n][0..1] = token row g, experts 8 n + 2 q + {0, 1}; acc[n][2..3] = row g + 8
  {
    float* part = s_part + (kc * kMmaGateTokens + tile * 16) * (EP + 1);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      part[g * (EP + 1) + n * 8 + 2 * q] = acc[n][0];
      part[g * (EP + 1) + n * 8 + 2 * q + 1] = acc[n][1];
      part[(g + 8) * (EP + 1) + n * 8 + 2 * q] = acc[n][2];
      part[(g + 8) * (EP + 1) + n * 8 + 2 * q + 1] = acc[n][3];
    }
  }
  __syncthreads();
  // all threads: sum the four partial logits of every (token, expert), add the bias
  {
    const long long t_first = tile_id * kMmaGateTokens;
    for (int i = threadIdx.x; i < kMmaGateTokens * E; i += kMmaGateWarps * 32) {
      const int tok = i / E;
      const int e = i - tok * E;
      float v = s_part[tok * (EP + 1) + e];
#pragma unroll
      for (int c = 1; c < 4; ++c) v += s_part[(c * kMmaGateTokens + tok) * (EP + 1) + e];
      v += gb ? gb[e] : 0.f;
      s_part[tok * (EP + 1) + e] = v;          // quarter 0's rows now hold the logits
      if (logits_out && t_first + tok < L) logits_out[(t_first + tok) * E + e] = v;
    }
  }
  __syncthreads();
  // one thread per token: softmax / top-k / renormalise
  if (threadIdx.x < kMmaGateTokens) {
    const long long t = tile_id * kMmaGateTokens + threadIdx.x;
    unsigned picked = 0u;                      // bit e: this token chose expert e (E <= 32 here)
    if (t < L) {
      float* lg = s_part + threadIdx.x * (EP + 1);
      float* sel = s_part + (kMmaGateTokens + threadIdx.x) * (EP + 1);   // quarter 1's row: the chosen scores
      if (router_mode == kRouterNormalised) {
        // same order of operations as gate_topk_kernel: one value per lane, butterfly sum
        float sqv[32];
#pragma unroll
        for (int l = 0; l < 32; ++l) sqv[l] = l < E ? lg[l] * lg[l] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int l = 0; l < o; ++l) sqv[l] += sqv[l + o];
        const float inv = 1.0f / fmaxf(sqrtf(sqv[0]), 1e-12f);
        for (int e = 0; e < E; ++e) lg[e] *= inv;
      }
      float mx = -INFINITY;
      for (int e = 0; e < E; ++e) mx = fmaxf(mx, lg[e]);
      for (int e = 0; e < E; ++e) lg[e] = expf(lg[e] - mx);
      // Sum in the order gate_topk_kernel uses (one value per lane, then a butterfly), so that
      // both kernels give bit-identical scores for the same logits (E <= 32 here).
      float v[32];
#pragma unroll
      for (int l = 0; l < 32; ++l) v[l] = l < E ? lg[l] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int l = 0; l < o; ++l) v[l] += v[l + o];
      const float sum = v[0];
      float norm = 0.f;
      for (int s = 0; s < k; ++s) {
        float best = -2.f;
        int best_e = E;
        for (int e = 0; e < E; ++e) {
          const float pv = lg[e];
          if (pv > best) {     // ascending e: the first maximum wins
            best = pv;
            best_e = e;
          }
        }
        const float sc = best / sum;
        norm += sc;
        topk_idx[t * k + s] = best_e;
        sel[s] = sc;
        lg[best_e] = -1.f;
        if (best_e < E) picked |= 1u << best_e;
      }
      const float denom = router_mode == kRouterSoftmaxRenorm ? fmaxf(norm, 1e-12f) : 1.0f;
      for (int s = 0; s < k; ++s) topk_score[t * k + s] = sel[s] / denom;
    }
    if (group_counts != nullptr) {
      // Rows per expert in each group of 16 tokens (the first stage of the counting sort, which
      // then needs no pass of its own over the indices): the 32 finishing threads are one warp.
      int c_lo = 0, c_hi = 0;
      for (int e = 0; e < E; ++e) {
        const unsigned b = __ballot_sync(0xffffffffu, (picked >> e) & 1u);
        if (static_cast<int>(threadIdx.x) == e) {
          c_lo = __popc(b & 0xffffu);
          c_hi = __popc(b >> 16);
        }
      }
      if (static_cast<int>(threadIdx.x) < E) {
        group_counts[(2 * tile_id) * E + threadIdx.x] = c_lo;
        group_counts[(2 * tile_id + 1) * E + threadIdx.x] = c_hi;
      }
    }
  }
  __syncthreads();      // the partial sums are overwritten by the next tile
  }
}

// ---- counting sort -------------------------------------------------------------------------
// Pass 1: per block of kRouteBlock tokens, how many of its rows go to each expert.
// A token never picks the same expert twice, so the stable order inside one expert is simply
// ascending token id; per-warp bit masks of "which lanes picked e" give every row its rank.
__device__ __forceinline__ void build_masks(const long long* __restrict__ topk_idx, long long L, int E, int k,
                                            unsigned* masks /*[8][E]*/, int* status) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kRouteBlock / 32) * E; i += kRouteBlock) masks[i] = 0u;
  __syncthreads();
  const long long t = static_cast<long long>(blockIdx.x) * kRouteBlock + threadIdx.x;
  if (t < L) {
    for (int s = 0; s < k; ++s) {
      const long long e = topk_idx[t * k + s];
      if (e < 0 || e >= E) {
        atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
        continue;
      }
      atomicOr(&masks[warp * E + static_cast<int>(e)], 1u << lane);
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kRouteBlock)
route_count_kernel(const long long* __restrict__ topk_idx, long long L, int E, int k, int* __restrict__ block_cnt,
                   int* status) {
  extern __shared__ unsigned masks[];
  build_masks(topk_idx, L, E, k, masks, status);
  for (int e = threadIdx.x; e < E; e += kRouteBlock) {
    int c = 0;
#pragma unroll
    for (int w = 0; w < kRouteBlock / 32; ++w) c += __popc(masks[w * E + e]);
    block_cnt[static_cast<long long>(blockIdx.x) * E + e] = c;
  }
}

// Pass 2 (one block): turn block_cnt[b][e] into the exclusive prefix over b, and produce
// lengths, offsets and max_len.
__global__ void __launch_bounds__(1024)
route_scan_kernel(int* __restrict__ block_cnt, int nb, int E, long long* __restrict__ lengths,
                  long long* __restrict__ offsets, long long* __restrict__ max_len) {
  __shared__ long long s_part[1024];
  __shared__ long long s_carry;
  __shared__ long long s_max;
  if (threadIdx.x == 0) {
    s_carry = 0;
    s_max = 0;
  }
  for (int base = 0; base < E; base += 1024) {
    const int e = base + threadIdx.x;
    long long total = 0;
    if (e < E) {
      for (int b = 0; b < nb; ++b) {
        const long long i = static_cast<long long>(b) * E + e;
        const int c = block_cnt[i];
        block_cnt[i] = static_cast<int>(total);
        total += c;
      }
      if (lengths) lengths[e] = total;
    }
    s_part[threadIdx.x] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
      long long run = s_carry;
      long long mx = s_max;
      const int n = min(1024, E - base);
      for (int i = 0; i < n; ++i) {
        const long long v = s_part[i];
        offsets[base + i] = run;
        run += v;
        mx = v > mx ? v : mx;
      }
      s_carry = run;
      s_max = mx;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    offsets[E] = s_carry;
    if (max_len) *max_len = s_max;
  }
}

// Pass 3: placement.
__global__ void __launch_bounds__(kRouteBlock)
route_place_kernel(const long long* __restrict__ topk_idx, long long L, int E, int k,
                   const int* __restrict__ block_base, const long long* __restrict__ offsets,
                   long long* __restrict__ gate_index, long long* __restrict__ token_index,
                   long long* __restrict__ reverse_index, int* status) {
  extern __shared__ unsigned masks[];
  build_masks(topk_idx, L, E, k, masks, status);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * kRouteBlock + threadIdx.x;
  if (t >= L) return;
  const unsigned lt = (1u << lane) - 1u;
  for (int s = 0; s < k; ++s) {
    const long long e64 = topk_idx[t * k + s];
    if (e64 < 0 || e64 >= E) continue;
    const int e = static_cast<int>(e64);
    int rank = block_base[static_cast<long long>(blockIdx.x) * E + e];
    for (int w = 0; w < warp; ++w) rank += __popc(masks[w * E + e]);
    rank += __popc(masks[warp * E + e] & lt);
    const long long pos = offsets[e] + rank;
    if (gate_index) gate_index[pos] = t * k + s;
    if (token_index) token_index[pos] = t;
    if (reverse_index) {
      // position among this token's rows = number of its picks with a smaller expert id
      int j = 0;
      for (int s2 = 0; s2 < k; ++s2) {
        const long long e2 = topk_idx[t * k + s2];
        j += (e2 < e64) ? 1 : 0;
      }
      reverse_index[t * k + j] = pos;
    }
  }
}

// Passes 2 and 3 in one launch, for tables of block counts small enough that every block can
// afford to read all of them (nb * E entries): each block sums the counts of the blocks before it
// (its base) and of all blocks (the lengths), scans the lengths into offsets itself, and places
// its rows. Block 0 also publishes lengths, offsets and max_len. Same results as the scan kernel
// followed by route_place_kernel; one launch and no single-block serial pass.
constexpr long long kPlaceScanMaxEntries = 32 * 1024;

__global__ void __launch_bounds__(kRouteBlock)
route_place_scan_kernel(const long long* __restrict__ topk_idx, long long L, int E, int k, int nb,
                        const int* __restrict__ block_cnt, long long* __restrict__ lengths,
                        long long* __restrict__ offsets, long long* __restrict__ max_len,
                        long long* __restrict__ gate_index, long long* __restrict__ token_index,
                        long long* __restrict__ reverse_index, int* status) {
  extern __shared__ unsigned masks[];                         // [8][E]
  int* s_base = reinterpret_cast<int*>(masks + (kRouteBlock / 32) * E);   // [E] rows of e in earlier blocks
  int* s_off = s_base + E;                                    // [E + 1] lengths, then offsets
  for (int e = threadIdx.x; e <= E; e += kRouteBlock) {
    if (e < E) s_base[e] = 0;
    s_off[e] = 0;
  }
  build_masks(topk_idx, L, E, k, masks, status);              // starts and ends with __syncthreads
  const int entries = nb * E;
  const int mine = static_cast<int>(blockIdx.x) * E;          // entries below this belong to earlier blocks
  for (int i = threadIdx.x; i < entries; i += kRouteBlock) {
    const int c = block_cnt[i];
    if (c != 0) {
      const int e = i % E;
      atomicAdd(&s_off[e + 1], c);
      if (i < mine) atomicAdd(&s_base[e], c);
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // lengths -> offsets (inclusive scan, 32 experts per step) and the longest segment
    const int lane = threadIdx.x;
    int carry = 0;
    int mx = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int len = e < E ? s_off[e + 1] : 0;
      if (blockIdx.x == 0 && e < E && lengths) lengths[e] = len;
      mx = max(mx, len);
      int v = len;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (e < E) s_off[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (blockIdx.x == 0 && lane == 0 && max_len) *max_len = mx;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e <= E; e += kRouteBlock) offsets[e] = s_off[e];
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * kRouteBlock + threadIdx.x;
  if (t >= L || (!gate_index && !token_index && !reverse_index)) return;
  const unsigned lt = (1u << lane) - 1u;
  for (int s = 0; s < k; ++s) {
    const long long e64 = topk_idx[t * k + s];
    if (e64 < 0 || e64 >= E) continue;
    const int e = static_cast<int>(e64);
    int rank = s_base[e];
    for (int w = 0; w < warp; ++w) rank += __popc(masks[w * E + e]);
    rank += __popc(masks[warp * E + e] & lt);
    const long long pos = static_cast<long long>(s_off[e]) + rank;
    if (gate_index) gate_index[pos] = t * k + s;
    if (token_index) token_index[pos] = t;
    if (reverse_index) {
      int j = 0;
      for (int s2 = 0; s2 < k; ++s2) j += (topk_idx[t * k + s2] < e64) ? 1 : 0;
      reverse_index[t * k + j] = pos;
    }
  }
}

// Placement for small batches, fused with the two memory passes that follow it in the layers:
// one block per group of 16 tokens. The per-group counts come from the gate kernel, so the
// indices are read once. Every block reads the whole table of group counts (at most 16 k entries:
// beyond that the per-block scan costs more than the separate counting sort it replaces),
// derives its own base and the offsets, places its rows, and then
//   - copies each of its tokens' rows to the k expert-sorted positions it has just computed
//     (the index_select of the up projection: x is read once, each row written k times), and
//   - clears its tokens' rows of the buffer the down projection's epilogue accumulates into.
// Same tensors, bit for bit, as route_count_kernel + route_place_scan_kernel followed by the row
// gather kernel and a memset.
constexpr int kGroupTokens = 16;

__global__ void __launch_bounds__(512)
route_place_gather_kernel(const long long* __restrict__ topk_idx, long long L, int E, int k, int ng,
                          const int* __restrict__ group_counts, long long* __restrict__ lengths,
                          long long* __restrict__ offsets, long long* __restrict__ max_len,
                          long long* __restrict__ gate_index, long long* __restrict__ token_index,
                          long long* __restrict__ reverse_index, const uint8_t* __restrict__ x, long long ldx_bytes,
                          int row_bytes, uint8_t* __restrict__ x_sorted, long long lds_bytes,
                          uint8_t* __restrict__ zero_rows, long long ldz_bytes, int zero_row_bytes, int* status) {
  extern __shared__ int s_int[];
  int* s_base = s_int;                         // [E] rows of expert e in earlier groups
  int* s_off = s_base + E;                     // [E + 1] lengths, then offsets
  unsigned* s_mask = reinterpret_cast<unsigned*>(s_off + E + 1);   // [E] which of the 16 tokens picked e
  int* s_dst = reinterpret_cast<int*>(s_mask + E);                 // [16 * k] sorted position of (token, slot)
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    if (e < E) {
      s_base[e] = 0;
      s_mask[e] = 0u;
    }
    s_off[e] = 0;
  }
  for (int i = threadIdx.x; i < kGroupTokens * k; i += blockDim.x) s_dst[i] = -1;
  // programmatic dependent launch: the gate kernel's outputs are read from here on
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncthreads();
  const long long t0 = static_cast<long long>(blockIdx.x) * kGroupTokens;
  if (threadIdx.x < kGroupTokens && t0 + threadIdx.x < L) {
    const long long t = t0 + threadIdx.x;
    for (int s = 0; s < k; ++s) {
      const long long e = topk_idx[t * k + s];
      if (e < 0 || e >= E) {
        atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
        continue;
      }
      atomicOr(&s_mask[static_cast<int>(e)], 1u << threadIdx.x);
    }
  }
  const int entries = ng * E;
  const int mine = static_cast<int>(blockIdx.x) * E;
  if ((E & (E - 1)) == 0) {
    // E a power of two (it divides the block size): a thread only ever meets one expert, keeps
    // its two sums in registers, lanes of a warp that share the expert combine by shuffle, and
    // one lane per (warp, expert) touches shared memory - instead of one contended shared-memory
    // atomic per table entry.
    const int e = threadIdx.x & (E - 1);
    int all = 0, before = 0;
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
      const int c = group_counts[i];
      all += c;
      if (i < mine) before += c;
    }
    for (int o = E; o < 32; o <<= 1) {
      all += __shfl_xor_sync(0xffffffffu, all, o);
      before += __shfl_xor_sync(0xffffffffu, before, o);
    }
    if ((threadIdx.x & 31) < E) {
      if (all != 0) atomicAdd(&s_off[e + 1], all);
      if (before != 0) atomicAdd(&s_base[e], before);
    }
  } else {
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
      const int c = group_counts[i];
      if (c != 0) {
        const int e = i % E;
        atomicAdd(&s_off[e + 1], c);
        if (i < mine) atomicAdd(&s_base[e], c);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    int mx = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int len = e < E ? s_off[e + 1] : 0;
      if (blockIdx.x == 0 && e < E && lengths) lengths[e] = len;
      mx = max(mx, len);
      int v = len;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (e < E) s_off[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (blockIdx.x == 0 && lane == 0 && max_len) *max_len = mx;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  }
  if (threadIdx.x < kGroupTokens && t0 + threadIdx.x < L) {
    const long long t = t0 + threadIdx.x;
    const unsigned lt = (1u << threadIdx.x) - 1u;
    for (int s = 0; s < k; ++s) {
      const long long e64 = topk_idx[t * k + s];
      if (e64 < 0 || e64 >= E) continue;
      const int e = static_cast<int>(e64);
      const long long pos = static_cast<long long>(s_off[e]) + s_base[e] + __popc(s_mask[e] & lt);
      if (gate_index) gate_index[pos] = t * k + s;
      if (token_index) token_index[pos] = t;
      if (reverse_index) {
        int j = 0;
        for (int s2 = 0; s2 < k; ++s2) j += (topk_idx[t * k + s2] < e64) ? 1 : 0;
        reverse_index[t * k + j] = pos;
      }
      s_dst[threadIdx.x * k + s] = static_cast<int>(pos);
    }
  }
  if (x_sorted == nullptr && zero_rows == nullptr) return;
  __syncthreads();
  // memory passes: one warp per token of the group
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int tt = warp; tt < kGroupTokens; tt += static_cast<int>(blockDim.x >> 5)) {
    const long long t = t0 + tt;
    if (t >= L) break;
    if (x_sorted != nullptr) {
      const uint4* a = reinterpret_cast<const uint4*>(x + t * ldx_bytes);
      const int vec = row_bytes >> 4;
      for (int c0 = lane; c0 < vec; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + 32 * u < vec) v[u] = a[c0 + 32 * u];
        for (int s = 0; s < k; ++s) {
          const int pos = s_dst[tt * k + s];
          if (pos < 0) continue;
          uint4* d = reinterpret_cast<uint4*>(x_sorted + static_cast<long long>(pos) * lds_bytes);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + 32 * u < vec) d[c0 + 32 * u] = v[u];
        }
      }
    }
    if (zero_rows != nullptr) {
      uint4* z = reinterpret_cast<uint4*>(zero_rows + t * ldz_bytes);
      const int vec = zero_row_bytes >> 4;
      for (int c = lane; c < vec; c += 32) z[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

constexpr long long kGroupTableMaxEntries = 16 * 1024;

}  // namespace
}  // namespace fmoe

using namespace fmoe;

namespace {
int gate_topk_impl(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                   const float* logits_in, int64_t ld_logits, int logits_split, int64_t L, int d, int E, int k,
                   float* logits_out, int64_t* topk_idx, float* topk_score, int* group_counts, int router_mode,
                   void* stream, void* zero_rows = nullptr, long long ldz_bytes = 0, int zero_row_bytes = 0);

// Conditions under which the tensor-core gate kernel runs (and with it the per-group counts).
bool gate_mma_path(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* logits_in, int d, int E,
                   size_t* smem_out) {
  if (logits_in != nullptr || x_dtype != FMOE_BF16 || E > 32 || d < 8 || d % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (ldx * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(gate_w) & 15) != 0)
    return false;
  const int nt = E <= 8 ? 1 : (E <= 16 ? 2 : 4);
  const size_t smem = 3 * static_cast<size_t>(8 * nt) * (static_cast<size_t>(d) * 2 + kMmaGatePadBytes) +
                      4 * static_cast<size_t>(kMmaGateTokens) * (8 * nt + 1) * sizeof(float);
  if (smem_out) *smem_out = smem;
  return smem <= 200 * 1024;
}
}  // namespace

extern "C" int fmoe_gate_topk(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                              const float* logits_in, int64_t ld_logits, int logits_split, int64_t L, int d, int E,
                              int k, float* logits_out, int64_t* topk_idx, float* topk_score, void* stream) {
  return gate_topk_impl(x, x_dtype, ldx, gate_w, gate_b, logits_in, ld_logits, logits_split, L, d, E, k, logits_out,
                        topk_idx, topk_score, nullptr, kRouterSoftmaxRenorm, stream);
}

extern "C" int fmoe_gate_topk_normalized(const void* x, int x_dtype, int64_t ldx, const float* gate_w,
                                         const float* gate_b, const float* logits_in, int64_t ld_logits, int64_t L,
                                         int d, int E, int k, float* logits_out, int64_t* topk_idx, float* topk_score,
                                         void* stream) {
  return gate_topk_impl(x, x_dtype, ldx, gate_w, gate_b, logits_in, ld_logits, 0, L, d, E, k, logits_out, topk_idx,
                        topk_score, nullptr, kRouterNormalised, stream);
}

extern "C" size_t fmoe_route_group_counts_bytes(int64_t L, int E) {
  if (L < 0 || E < 1) return 0;
  const int64_t tiles = (L + kMmaGateTokens - 1) / kMmaGateTokens;
  return static_cast<size_t>((tiles > 0 ? tiles : 1) * 2 * E) * sizeof(int);
}

extern "C" int fmoe_gate_topk_counts_supported(const void* x, int x_dtype, int64_t ldx, const float* gate_w, int64_t L,
                                               int d, int E) {
  if (L <= 0 || E < 1) return 0;
  const int64_t tiles = (L + kMmaGateTokens - 1) / kMmaGateTokens;
  if (tiles * 2 * E > kGroupTableMaxEntries) return 0;
  return gate_mma_path(x, x_dtype, ldx, gate_w, nullptr, d, E, nullptr) ? 1 : 0;
}

extern "C" int fmoe_gate_topk_counts(const void* x, int x_dtype, int64_t ldx, const float* gate_w,
                                     const float* gate_b, int64_t L, int d, int E, int k, float* logits_out,
                                     int64_t* topk_idx, float* topk_score, int* group_counts, void* zero_rows,
                                     int zero_dtype, int64_t ld_zero, int zero_cols, void* stream) {
  FMOE_REQUIRE(group_counts != nullptr, "gate_topk_counts: group_counts is NULL");
  long long ldz_bytes = 0;
  int zero_row_bytes = 0;
  if (zero_rows != nullptr) {
    const int zs = zero_dtype == FMOE_BF16 ? 2 : (zero_dtype == FMOE_F32 ? 4 : 0);
    FMOE_REQUIRE(zs != 0 && zero_cols >= 1, "gate_topk_counts: zero fill needs a dtype (bf16 / f32) and a column count");
    zero_row_bytes = zero_cols * zs;
    ldz_bytes = static_cast<long long>(ld_zero) * zs;
    FMOE_REQUIRE(zero_row_bytes % 16 == 0 && ldz_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(zero_rows) & 15) == 0,
                 "gate_topk_counts: rows to clear must be 16-byte aligned and a multiple of 16 bytes long");
  }
  if (!fmoe_gate_topk_counts_supported(x, x_dtype, ldx, gate_w, L, d, E)) {
    return fail(FMOE_ERR_UNSUPPORTED,
                "gate_topk_counts: needs bf16 tokens with 16-byte aligned rows, E <= 32, d a multiple of 8 and a "
                "small batch (L=%lld, d=%d, E=%d); use fmoe_gate_topk + fmoe_route_metadata", (long long)L, d, E);
  }
  return gate_topk_impl(x, x_dtype, ldx, gate_w, gate_b, nullptr, 0, 0, L, d, E, k, logits_out, topk_idx, topk_score,
                        group_counts, kRouterSoftmaxRenorm, stream, zero_rows, ldz_bytes, zero_row_bytes);
}

namespace {
int gate_topk_impl(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                   const float* logits_in, int64_t ld_logits, int logits_split, int64_t L, int d, int E,
                   int k, float* logits_out, int64_t* topk_idx, float* topk_score, int* group_counts, int router_mode,
                   void* stream, void* zero_rows, long long ldz_bytes, int zero_row_bytes) {
  FMOE_REQUIRE(L >= 0 && E >= 1 && E <= kMaxGateExperts, "gate_topk: E=%d outside [1, %d]", E, kMaxGateExperts);
  FMOE_REQUIRE(k >= 1 && k <= E, "gate_topk: k=%d must be in [1, E=%d]", k, E);
  if (L == 0) return FMOE_OK;   // an empty batch is valid input (its tensors have NULL data pointers)
  FMOE_REQUIRE(topk_idx && topk_score, "gate_topk: output pointers must not be NULL");
  FMOE_REQUIRE(logits_in || (x && gate_w && d >= 1), "gate_topk: need either logits_in or x and gate_w");
  FMOE_REQUIRE(!logits_in || ld_logits >= (logits_split ? 2 : 1) * static_cast<int64_t>(E),
               "gate_topk: ld_logits=%lld too small for E=%d", (long long)ld_logits, E);
  FMOE_REQUIRE(logits_in || x_dtype == FMOE_BF16 || x_dtype == FMOE_F32, "gate_topk: x must be bf16 or f32");
  if (L == 0) return FMOE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 16-byte loads need aligned rows of x and of the gate weights
  const int xs = x_dtype == FMOE_BF16 ? 2 : 4;
  const int vec_ok = (logits_in == nullptr) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ldx * xs) % 16 == 0) &&
                     ((reinterpret_cast<uintptr_t>(gate_w) & 15) == 0) && (d % 8 == 0);
  // bf16 tokens and few experts: logits on the warp-level tensor cores
  if (!logits_in && x_dtype == FMOE_BF16 && vec_ok && E <= 32) {
    const int nt = E <= 8 ? 1 : (E <= 16 ? 2 : 4);
    const size_t smem = 3 * static_cast<size_t>(8 * nt) * (static_cast<size_t>(d) * 2 + kMmaGatePadBytes) +
                        4 * static_cast<size_t>(kMmaGateTokens) * (8 * nt + 1) * sizeof(float);
    if (smem <= 200 * 1024) {
      // persistent blocks (the weights are staged once per block), two per SM: with the next
      // tile's rows prefetched into registers each block holds 64 KB of loads in flight
      long long nblk = (L + kMmaGateTokens - 1) / kMmaGateTokens;
      int dev = 0, sms = 148;
      if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (nblk > 2ll * sms) nblk = 2ll * sms;
      const unsigned blocks = static_cast<unsigned>(nblk);
#define FMOE_GATE_MMA(NT)                                                                                          \
  do {                                                                                                             \
    auto kern = gate_topk_mma_kernel<NT>;                                                                          \
    if (smem > 48 * 1024) {                                                                                        \
      FMOE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));          \
    }                                                                                                              \
    kern<<<blocks, kMmaGateWarps * 32, smem, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, gate_w, gate_b, L, d, \
                                                   E, k, logits_out, reinterpret_cast<long long*>(topk_idx),      \
                                                   topk_score, group_counts, router_mode,                          \
                                                   static_cast<uint8_t*>(zero_rows), ldz_bytes, zero_row_bytes);   \
  } while (0)
      if (nt == 1) FMOE_GATE_MMA(1); else if (nt == 2) FMOE_GATE_MMA(2); else FMOE_GATE_MMA(4);
#undef FMOE_GATE_MMA
      FMOE_CUDA_OK(cudaGetLastError());
      ++g_misc_launches;
      return FMOE_OK;
    }
  }
  if (group_counts != nullptr || zero_rows != nullptr) {
    return fail(FMOE_ERR_UNSUPPORTED, "gate_topk_counts: the per-group counts come from the tensor-core gate kernel only");
  }
  // Gate weights in shared memory when they fit beside the logits scratch (and a few blocks per SM)
  const size_t w_bytes = logits_in ? 0 : static_cast<size_t>(E) * d * sizeof(float);
  const bool w_smem = !logits_in && vec_ok && w_bytes <= 96 * 1024;
  // Several tokens per warp amortise the gate-weight reads, but only pay off when that still
  // leaves a few warps per scheduler on every SM
  const long long warps_full = 148ll * kGateWarps * 2;
  const int tok = (L >= warps_full * 4) ? 4 : ((w_smem && L >= warps_full) ? 2 : 1);
  const long long per_block = static_cast<long long>(kGateWarps) * tok;
  long long blocks = (L + per_block - 1) / per_block;
  if (w_smem && blocks > 148 * 4) blocks = 148 * 4;     // persistent blocks: the weights are staged once per block
  const unsigned grid = static_cast<unsigned>(blocks);
  long long* idx = reinterpret_cast<long long*>(topk_idx);
#define FMOE_GATE(XT, TOK, WS)                                                                                      \
  do {                                                                                                              \
    auto kern = gate_topk_kernel<XT, TOK, WS>;                                                                      \
    if (WS && w_bytes > 16 * 1024) {                                                                                 \
      FMOE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));            \
    }                                                                                                               \
    kern<<<grid, kGateWarps * 32, WS ? w_bytes : 0, st>>>(static_cast<const XT*>(x), ldx, gate_w, gate_b, logits_in, \
                                                          ld_logits, logits_split, L, d, E, k, vec_ok, logits_out,  \
                                                          idx, topk_score, router_mode);                            \
  } while (0)
#define FMOE_GATE_T(XT)                                      \
  do {                                                       \
    if (w_smem) {                                            \
      if (tok == 4) FMOE_GATE(XT, 4, true);                  \
      else if (tok == 2) FMOE_GATE(XT, 2, true);             \
      else FMOE_GATE(XT, 1, true);                           \
    } else {                                                 \
      if (tok == 4) FMOE_GATE(XT, 4, false);                 \
      else FMOE_GATE(XT, 1, false);                          \
    }                                                        \
  } while (0)
  if (logits_in || x_dtype == FMOE_F32) {
    FMOE_GATE_T(float);
  } else {
    FMOE_GATE_T(__nv_bfloat16);
  }
#undef FMOE_GATE_T
#undef FMOE_GATE
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

}  // namespace

extern "C" size_t fmoe_route_workspace_bytes(int64_t L, int E, int k) {
  (void)k;
  if (L < 0 || E < 1) return 0;
  const int64_t nb = (L + kRouteBlock - 1) / kRouteBlock;
  return static_cast<size_t>((nb > 0 ? nb : 1) * E) * sizeof(int);
}

extern "C" int fmoe_route_metadata(const int64_t* topk_idx, int64_t L, int E, int k, int64_t* lengths,
                                   int64_t* offsets, int64_t* gate_index, int64_t* token_index,
                                   int64_t* reverse_index, int64_t* max_len, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 4096, "route_metadata: E=%d outside [1, 4096]", E);
  FMOE_REQUIRE(k >= 1 && k <= E, "route_metadata: k=%d must be in [1, E=%d]", k, E);
  FMOE_REQUIRE(L >= 0 && L * k < (1ll << 31), "route_metadata: L*k must be below 2^31");
  FMOE_REQUIRE(offsets != nullptr && (L == 0 || topk_idx != nullptr), "route_metadata: NULL offsets or topk_idx");
  FMOE_REQUIRE(workspace != nullptr && workspace_bytes >= fmoe_route_workspace_bytes(L, E, k),
               "route_metadata: workspace of %zu bytes is smaller than the %zu needed", workspace_bytes,
               fmoe_route_workspace_bytes(L, E, k));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  const int nb = static_cast<int>((L + kRouteBlock - 1) / kRouteBlock);
  int* block_cnt = static_cast<int*>(workspace);
  const size_t smem = static_cast<size_t>(kRouteBlock / 32) * E * sizeof(unsigned);
  const long long* idx = reinterpret_cast<const long long*>(topk_idx);
  if (smem > 48 * 1024) {
    FMOE_CUDA_OK(cudaFuncSetAttribute(route_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FMOE_CUDA_OK(cudaFuncSetAttribute(route_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  if (nb > 0) {
    route_count_kernel<<<nb, kRouteBlock, smem, st>>>(idx, L, E, k, block_cnt, status);
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
  }
  if (nb > 0 && static_cast<long long>(nb) * E <= kPlaceScanMaxEntries) {
    // small table of block counts: every placement block scans it itself, no separate scan launch
    const size_t smem2 = smem + (2 * static_cast<size_t>(E) + 1) * sizeof(int);
    if (smem2 > 48 * 1024) {
      FMOE_CUDA_OK(cudaFuncSetAttribute(route_place_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
    }
    route_place_scan_kernel<<<nb, kRouteBlock, smem2, st>>>(
        idx, L, E, k, nb, block_cnt, reinterpret_cast<long long*>(lengths), reinterpret_cast<long long*>(offsets),
        reinterpret_cast<long long*>(max_len), reinterpret_cast<long long*>(gate_index),
        reinterpret_cast<long long*>(token_index), reinterpret_cast<long long*>(reverse_index), status);
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
    return FMOE_OK;
  }
  route_scan_kernel<<<1, 1024, 0, st>>>(block_cnt, nb, E, reinterpret_cast<long long*>(lengths),
                                        reinterpret_cast<long long*>(offsets), reinterpret_cast<long long*>(max_len));
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  if (nb > 0 && (gate_index || token_index || reverse_index)) {
    route_place_kernel<<<nb, kRouteBlock, smem, st>>>(idx, L, E, k, block_cnt, reinterpret_cast<long long*>(offsets),
                                                      reinterpret_cast<long long*>(gate_index),
                                                      reinterpret_cast<long long*>(token_index),
                                                      reinterpret_cast<long long*>(reverse_index), status);
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
  }
  return FMOE_OK;
}

extern "C" int fmoe_route_metadata_gather(const int64_t* topk_idx, int64_t L, int E, int k, const int* group_counts,
                                          int64_t* lengths, int64_t* offsets, int64_t* gate_index,
                                          int64_t* token_index, int64_t* reverse_index, int64_t* max_len,
                                          const void* x, int x_dtype, int64_t ldx, int cols, void* x_sorted,
                                          int64_t ld_sorted, void* zero_rows, int zero_dtype, int64_t ld_zero,
                                          int zero_cols, void* stream) {
  FMOE_REQUIRE(E >= 1 && E <= 32, "route_metadata_gather: E=%d outside [1, 32]", E);
  FMOE_REQUIRE(k >= 1 && k <= E, "route_metadata_gather: k=%d must be in [1, E=%d]", k, E);
  FMOE_REQUIRE(L >= 0 && L * k < (1ll << 31), "route_metadata_gather: L*k must be below 2^31");
  FMOE_REQUIRE(offsets != nullptr, "route_metadata_gather: NULL offsets");
  const int64_t ng = 2 * ((L + kMmaGateTokens - 1) / kMmaGateTokens);
  FMOE_REQUIRE(ng * E <= kGroupTableMaxEntries,
               "route_metadata_gather: table of %lld group counts exceeds %lld; use fmoe_route_metadata",
               (long long)(ng * E), (long long)kGroupTableMaxEntries);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (L == 0) {
    FMOE_CUDA_OK(cudaMemsetAsync(offsets, 0, (E + 1) * sizeof(int64_t), st));
    if (lengths) FMOE_CUDA_OK(cudaMemsetAsync(lengths, 0, E * sizeof(int64_t), st));
    if (max_len) FMOE_CUDA_OK(cudaMemsetAsync(max_len, 0, sizeof(int64_t), st));
    return FMOE_OK;
  }
  FMOE_REQUIRE(topk_idx && group_counts, "route_metadata_gather: NULL topk_idx or group_counts");
  int row_bytes = 0, zero_row_bytes = 0;
  const int xs = dtype_size(x_dtype), zs = dtype_size(zero_dtype);
  if (x_sorted != nullptr) {
    FMOE_REQUIRE(x != nullptr && xs != 0 && cols >= 1, "route_metadata_gather: gather needs x, its dtype and cols");
    row_bytes = cols * xs;
    const bool ok = (row_bytes % 16 == 0) && ((ldx * xs) % 16 == 0) && ((ld_sorted * xs) % 16 == 0) &&
                    ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(x_sorted) & 15) == 0);
    if (!ok) return fail(FMOE_ERR_UNSUPPORTED, "route_metadata_gather: rows must be 16-byte aligned multiples of 16 bytes");
  }
  if (zero_rows != nullptr) {
    FMOE_REQUIRE(zs != 0 && zero_cols >= 1, "route_metadata_gather: zero fill needs a dtype and a column count");
    zero_row_bytes = zero_cols * zs;
    const bool ok = (zero_row_bytes % 16 == 0) && ((ld_zero * zs) % 16 == 0) &&
                    ((reinterpret_cast<uintptr_t>(zero_rows) & 15) == 0);
    if (!ok) return fail(FMOE_ERR_UNSUPPORTED, "route_metadata_gather: cleared rows must be 16-byte aligned multiples of 16 bytes");
  }
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  const size_t smem = (static_cast<size_t>(3 * E + 1) + static_cast<size_t>(kGroupTokens) * k) * sizeof(int);
  const int64_t blocks = (L + kGroupTokens - 1) / kGroupTokens;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    cfg.blockDim = dim3(512, 1, 1);     // 16 warps: one per token in the copy phase
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
    FMOE_CUDA_OK(cudaLaunchKernelEx(
        &cfg, route_place_gather_kernel, reinterpret_cast<const long long*>(topk_idx), static_cast<long long>(L), E, k,
        static_cast<int>(ng), group_counts, reinterpret_cast<long long*>(lengths), reinterpret_cast<long long*>(offsets),
        reinterpret_cast<long long*>(max_len), reinterpret_cast<long long*>(gate_index),
        reinterpret_cast<long long*>(token_index), reinterpret_cast<long long*>(reverse_index),
        static_cast<const uint8_t*>(x), static_cast<long long>(ldx * xs), row_bytes, static_cast<uint8_t*>(x_sorted),
        static_cast<long long>(ld_sorted * xs), static_cast<uint8_t*>(zero_rows), static_cast<long long>(ld_zero * zs),
        zero_row_bytes, status));
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

// ------------------------------------------------------------------------------------------------
// Routing metadata for callers that cannot allocate device memory.
//
// Some callers of this library run where cudaMalloc is off the table: code executing inside a
// framework's memory-planned region where every byte was reserved up front, plugins that are only
// handed their input and output buffers, or services that run with a fixed device-memory budget.
// fmoe_route_metadata needs a small scratch table (rows per expert for every block of 256 tokens)
// that such callers have nowhere to put. This variant keeps that table in a file-scope device
// array instead, so the caller passes inputs and outputs only.
//
// The array is part of the loaded library image: every GPU that loads the library holds these
// 256 KiB until the process exits, whether or not this entry point is ever called.
namespace fmoe {
namespace {

constexpr long long kStaticRouteInts = 1ll << 16;   // 65536 ints = 256 KiB
static __device__ __align__(256) int g_route_scratch[kStaticRouteInts];

// Device address of g_route_scratch on the current device. In host code the array's name is only
// a handle for the runtime, not a device address, so the address is looked up once per device
// (with that device current) and cached.
int* static_route_scratch(int* err) {
  // atomic slots: two host threads making the first call together store the same address
  static std::atomic<int*> ptrs[kMaxDevices];
  int dev = 0;
  if ((*err = current_device_slot(&dev)) != FMOE_OK) return nullptr;
  int* p = ptrs[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_route_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = cuda_fail(e, "cudaGetSymbolAddress(route scratch)");
      return nullptr;
    }
    ptrs[dev].store(p, std::memory_order_release);
  }
  return p;
}

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_route_metadata_static(const int64_t* topk_idx, int64_t L, int E, int k, int64_t* lengths,
                                          int64_t* offsets, int64_t* gate_index, int64_t* token_index,
                                          int64_t* reverse_index, int64_t* max_len, void* stream) {
  FMOE_REQUIRE(L >= 0 && E >= 1, "route_metadata_static: L=%lld E=%d", (long long)L, E);
  const size_t need = fmoe_route_workspace_bytes(L, E, k);
  if (need > static_cast<size_t>(kStaticRouteInts) * sizeof(int)) {
    return fail(FMOE_ERR_UNSUPPORTED,
                "route_metadata_static: ceil(L/256)*E = %zu scratch entries exceed the built-in %lld "
                "(L=%lld, E=%d); use fmoe_route_metadata with a caller-provided workspace",
                need / sizeof(int), kStaticRouteInts, (long long)L, E);
  }
  int err = 0;
  int* scratch = static_route_scratch(&err);
  if (!scratch) return err;
  // Nothing in the table has to start at zero: the counting pass overwrites every entry the scan
  // and the placement pass read. The previous call's contents are simply left behind.
  return fmoe_route_metadata(topk_idx, L, E, k, lengths, offsets, gate_index, token_index, reverse_index, max_len,
                             scratch, static_cast<size_t>(kStaticRouteInts) * sizeof(int), stream);
}
