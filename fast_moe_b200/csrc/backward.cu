// Backward-pass helpers around the grouped GEMM. The reference implements the backward of its
// operators as Triton kernels of their own (kernels/triton/triton_moe.py:62-106 SwiGLU,
// :290-516 d_jagged / d_weight of the up projection, :922-983 combine, :1576-1976 jagged x jagged
// products, :3474-3559 SiLU + down projection); here every matrix product of the backward pass is
// the forward's grouped GEMM run on differently laid out operands, and this file holds the
// HBM-bound passes that produce those layouts and the elementwise derivatives:
//   d_x of a projection   rows of d_out times W[e]^T: the grouped GEMM on the transposed weight
//                         (batched_transpose_kernel), then the k rows of a token are summed by
//                         the combine kernel;
//   d_W of a projection   dW[e] = X_e^T dOut_e, a product whose reduction runs over the rows of an
//                         expert: both operands are transposed into [features, padded rows]
//                         (jagged_transpose_pad_kernel; each expert's row range padded with zeros
//                         to whole K steps) and the grouped GEMM runs in its reduction-over-rows mode;
//   d_bias                column sums per expert (jagged_colsum_kernel);
//   combine backward      d_rows[p] = d_out[token(p)] * gate[p] (gather_scale_rows_kernel) and
//                         d_gate[p] = <d_out[token(p)], rows[p]> (row_dot_kernel);
//   activations           SiLU' and the SwiGLU derivative (elementwise).
#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// kseg[0] = 0, kseg[e + 1] = kseg[e] + max(unit, len_e rounded up to unit): every expert owns at
// least one (all-zero) K step, so its weight-gradient tile is always written.
__global__ void pad_offsets_kernel(const long long* __restrict__ offsets, int E, int unit, long long* __restrict__ kseg) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    long long run = 0;
    kseg[0] = 0;
    for (int e = 0; e < E; ++e) {
      long long len = offsets[e + 1] - offsets[e];
      if (len < 0) len = 0;
      long long padded = (len + unit - 1) / unit * unit;
      if (padded < unit) padded = unit;
      run += padded;
      kseg[e + 1] = run;
    }
  }
}

// out[c, kseg[e] + j] = in[offsets[e] + j, c] for j < len_e, 0 for the padding. 32 x 32 tiles
// through shared memory; a tile of 32 padded positions never straddles two experts (unit is a
// multiple of 32). `index` (optional) names the source row of every sorted row: in[index[r] / div].
template <typename T>
__global__ void __launch_bounds__(256)
jagged_transpose_pad_kernel(const T* __restrict__ in, long long ld_in, long long in_rows, const long long* __restrict__ index,
                            int index_div, const long long* __restrict__ offsets, const long long* __restrict__ kseg, int E,
                            int cols, T* __restrict__ out, long long ld_out, int* status) {
  __shared__ T tile[32][33];
  const long long q0 = static_cast<long long>(blockIdx.x) * 32;      // padded position
  if (q0 >= kseg[E]) return;
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (kseg[mid] <= q0) lo = mid; else hi = mid;
  }
  const int e = lo;
  const long long len = offsets[e + 1] - offsets[e];
  const long long j0 = q0 - kseg[e];
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;             // 32 x 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int jr = ty + 8 * i;
    const long long j = j0 + jr;
    T v = T(0.f);
    if (j < len && c0 + tx < cols) {
      long long r = offsets[e] + j;
      if (index != nullptr) {
        r = index[r] / index_div;
        if (r < 0 || r >= in_rows) {
          atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
          r = -1;
        }
      }
      if (r >= 0) v = in[r * ld_in + c0 + tx];
    }
    tile[jr][tx] = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int cr = ty + 8 * i;
    if (c0 + cr < cols) out[static_cast<long long>(c0 + cr) * ld_out + q0 + tx] = tile[tx][cr];
  }
}

// 64 x 64 tiles of 2-byte elements with 16-byte global accesses on both sides (the 32 x 32
// tiles above move 64-byte row pieces). Shared tile: 64 rows of 33 words; the load phase stores
// four words per 16-byte vector, the store phase reads eight words of one column pair.
constexpr int kT16Pitch = 66;    // elements per tile row (33 words: conflict-free word stores)

__device__ __forceinline__ void tile16_put(__nv_bfloat16 (*tile)[kT16Pitch], int r, int v, uint4 x) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&tile[r][8 * v]);
  w[0] = x.x; w[1] = x.y; w[2] = x.z; w[3] = x.w;
}
// Store phase: thread (warp w, lane l) takes the column pair cp = (w / 2) * 8 + l / 4 and the 8 tile
// rows 8 v .. 8 v + 7 with v = (w % 2) * 4 + l % 4. It reads 8 words (two neighbouring columns of
// one row each; the 32 lanes of a warp hit 32 different banks) and splits them into the two output
// vectors: column 2 cp from the low halves, column 2 cp + 1 from the high halves.
__device__ __forceinline__ void tile16_column_pair(__nv_bfloat16 (*tile)[kT16Pitch], int r0, int cp, uint4& lo, uint4& hi) {
  const uint32_t* t = reinterpret_cast<const uint32_t*>(&tile[0][0]);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = t[(r0 + i) * (kT16Pitch / 2) + cp];
  lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
  lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
  lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
  lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
}
__device__ __forceinline__ void tile16_store_map(int& cp, int& v) {
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  cp = (w >> 1) * 8 + (l >> 2);
  v = (w & 1) * 4 + (l & 3);
}

// jagged_transpose_pad_kernel for bf16 with cols a multiple of 8 and 16-byte aligned rows on both
// sides: a block owns 64 padded positions (one K step: never straddles two experts) x 64 columns.
__global__ void __launch_bounds__(256)
jagged_transpose_pad_bf16_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, long long in_rows,
                                 const long long* __restrict__ index, int index_div, const long long* __restrict__ offsets,
                                 const long long* __restrict__ kseg, int E, int cols, __nv_bfloat16* __restrict__ out,
                                 long long ld_out, int* status) {
  __shared__ __align__(16) __nv_bfloat16 tile[64][kT16Pitch];
  const long long q0 = static_cast<long long>(blockIdx.x) * 64;
  if (q0 >= kseg[E]) return;
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (kseg[mid] <= q0) lo = mid; else hi = mid;
  }
  const int e = lo;
  const long long len = offsets[e + 1] - offsets[e];
  const long long j0 = q0 - kseg[e];
  const int c0 = blockIdx.y * 64;
  const int v = threadIdx.x & 7, rr = threadIdx.x >> 3;      // 8 vectors x 32 rows per pass
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int jr = rr + 32 * i;
    const long long j = j0 + jr;
    uint4 x = make_uint4(0, 0, 0, 0);
    if (j < len && c0 + 8 * v < cols) {
      long long r = offsets[e] + j;
      if (index != nullptr) {
        r = index[r] / index_div;
        if (r < 0 || r >= in_rows) {
          atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
          r = -1;
        }
      }
      if (r >= 0) x = *reinterpret_cast<const uint4*>(in + r * ld_in + c0 + 8 * v);
    }
    tile16_put(tile, jr, v, x);
  }
  __syncthreads();
  int cp, sv;
  tile16_store_map(cp, sv);
  uint4 even, odd;
  tile16_column_pair(tile, 8 * sv, cp, even, odd);
  const int cr = c0 + 2 * cp;                 // cols is a multiple of 8: the pair is inside or outside together
  if (cr < cols) {
    *reinterpret_cast<uint4*>(out + static_cast<long long>(cr) * ld_out + q0 + 8 * sv) = even;
    *reinterpret_cast<uint4*>(out + static_cast<long long>(cr + 1) * ld_out + q0 + 8 * sv) = odd;
  }
}

// batched_transpose_kernel for bf16 with rows and cols multiples of 8 and 16-byte aligned rows.
__global__ void __launch_bounds__(256)
batched_transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, long long in_sb, long long ld_in, int rows, int cols,
                              __nv_bfloat16* __restrict__ out, long long out_sb, long long ld_out) {
  __shared__ __align__(16) __nv_bfloat16 tile[64][kT16Pitch];
  const __nv_bfloat16* src = in + static_cast<long long>(blockIdx.z) * in_sb;
  __nv_bfloat16* dst = out + static_cast<long long>(blockIdx.z) * out_sb;
  const int r0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  const int v = threadIdx.x & 7, rr = threadIdx.x >> 3;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + rr + 32 * i;
    uint4 x = make_uint4(0, 0, 0, 0);
    if (r < rows && c0 + 8 * v < cols) x = *reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * ld_in + c0 + 8 * v);
    tile16_put(tile, rr + 32 * i, v, x);
  }
  __syncthreads();
  int cp, sv;
  tile16_store_map(cp, sv);
  uint4 lo, hi;
  tile16_column_pair(tile, 8 * sv, cp, lo, hi);
  const int c = c0 + 2 * cp;
  if (c < cols && r0 + 8 * sv < rows) {
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(c) * ld_out + r0 + 8 * sv) = lo;
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(c + 1) * ld_out + r0 + 8 * sv) = hi;
  }
}

// out[b, c, r] = in[b, r, c]: plain batched transpose (weights [E, N, K] -> [E, K, N]).
template <typename T>
__global__ void __launch_bounds__(256)
batched_transpose_kernel(const T* __restrict__ in, long long in_sb, long long ld_in, int rows, int cols, T* __restrict__ out,
                         long long out_sb, long long ld_out) {
  __shared__ T tile[32][33];
  const T* src = in + static_cast<long long>(blockIdx.z) * in_sb;
  T* dst = out + static_cast<long long>(blockIdx.z) * out_sb;
  const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty + 8 * i;
    tile[ty + 8 * i][tx] = (r < rows && c0 + tx < cols) ? src[static_cast<long long>(r) * ld_in + c0 + tx] : T(0.f);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i;
    if (c < cols && r0 + tx < rows) dst[static_cast<long long>(c) * ld_out + r0 + tx] = tile[tx][ty + 8 * i];
  }
}

// out[e, n] = sum over the rows of expert e of x[r, n], fp32 accumulation. A block owns 32 columns
// of one expert: its 8 warps take the rows r0 + w, r0 + w + 8, ... (lane = column, 4 rows in flight
// per warp), then the 8 partial sums of a column are added in warp order. The order is fixed, so
// a result repeats bit for bit.
template <typename T, typename OT>
__global__ void __launch_bounds__(256)
jagged_colsum_kernel(const T* __restrict__ x, long long ldx, const long long* __restrict__ offsets, int N, OT* __restrict__ out) {
  __shared__ float part[8][33];
  const int e = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 32 + lane;
  const long long r0 = offsets[e], r1 = offsets[e + 1];
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (n < N) {
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] += ldf<T>(x + (r + 8 * u) * ldx + n);
    }
    for (; r < r1; r += 8) acc[0] += ldf<T>(x + r * ldx + n);
  }
  part[warp][lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  __syncthreads();
  if (warp == 0 && n < N) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][lane];
    stf(out + static_cast<long long>(e) * N + n, s);
  }
}

// out[p, :] = src[index[p] / div, :] * weight[weight_index[p]]; the product is rounded to the
// output type (what Tensor.mul gives). One warp per row.
template <typename T, typename WT>
__global__ void __launch_bounds__(256)
gather_scale_rows_kernel(const T* __restrict__ src, long long src_rows, long long lds, const long long* __restrict__ index,
                         int div, const WT* __restrict__ weight, const long long* __restrict__ weight_index,
                         long long weight_count, long long rows, int cols, T* __restrict__ out, long long ldo, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long p = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    long long s = index[p];
    if (div != 1) s /= div;
    const long long wi = weight_index ? weight_index[p] : p;
    if (s < 0 || s >= src_rows || (weight && (wi < 0 || wi >= weight_count))) {
      if (lane == 0) atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      for (int c = lane; c < cols; c += 32) stf(out + p * ldo + c, 0.f);
      continue;
    }
    const float w = weight ? ldf<WT>(weight + wi) : 1.f;
    for (int c = lane; c < cols; c += 32) stf(out + p * ldo + c, ldf<T>(src + s * lds + c) * w);
  }
}

// out[p] = sum_c a[p, c] * b[index[p] / div, c] in fp32. One warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
row_dot_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ b, long long b_rows, long long ldb,
               const long long* __restrict__ index, int div, long long rows, int cols, float* __restrict__ out, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long p = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; p < rows; p += warps) {
    long long s = index ? index[p] : p;
    if (div != 1) s /= div;
    if (s < 0 || s >= b_rows) {
      if (lane == 0) {
        atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
        out[p] = 0.f;
      }
      continue;
    }
    float acc = 0.f;
    for (int c = lane; c < cols; c += 32) acc = fmaf(ldf<T>(a + p * lda + c), ldf<T>(b + s * ldb + c), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[p] = acc;
  }
}

// mode 0: d_x = d_y * silu'(x), silu'(x) = s (1 + x (1 - s)), s = sigmoid(x)
// mode 1 (SwiGLU, out = silu(alpha) * beta): d_alpha = d_out * beta * silu'(alpha), d_beta = d_out * silu(alpha)
template <typename T>
__global__ void __launch_bounds__(256)
activation_backward_kernel(int mode, const T* __restrict__ d_out, long long ldd, const T* __restrict__ alpha, long long lda,
                           const T* __restrict__ beta, long long ldb, long long rows, int cols, T* __restrict__ d_alpha,
                           long long ldda, T* __restrict__ d_beta, long long lddb) {
  const long long total = rows * cols;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    const float g = ldf<T>(d_out + r * ldd + c);
    const float a = ldf<T>(alpha + r * lda + c);
    const float sg = 1.0f / (1.0f + expf(-a));
    const float dsilu = sg * (1.0f + a * (1.0f - sg));
    if (mode == 0) {
      stf(d_alpha + r * ldda + c, g * dsilu);
    } else {
      const float bt = ldf<T>(beta + r * ldb + c);
      stf(d_alpha + r * ldda + c, g * bt * dsilu);
      stf(d_beta + r * lddb + c, g * a * sg);
    }
  }
}

// The same for bf16 with 8 elements (16 bytes) per thread and step: cols a multiple of 8, row
// strides multiples of 8, 16-byte aligned bases.
__global__ void __launch_bounds__(256)
activation_backward_bf16x8_kernel(int mode, const __nv_bfloat16* __restrict__ d_out, long long ldd,
                                  const __nv_bfloat16* __restrict__ alpha, long long lda,
                                  const __nv_bfloat16* __restrict__ beta, long long ldb, long long rows, int cols,
                                  __nv_bfloat16* __restrict__ d_alpha, long long ldda, __nv_bfloat16* __restrict__ d_beta,
                                  long long lddb) {
  const int vec = cols >> 3;
  const long long total = rows * vec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec) << 3;
    const uint4 gv = *reinterpret_cast<const uint4*>(d_out + r * ldd + c);
    const uint4 av = *reinterpret_cast<const uint4*>(alpha + r * lda + c);
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (mode != 0) bv = *reinterpret_cast<const uint4*>(beta + r * ldb + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
    uint4 oa, ob;
    __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]);
      const float2 a = __bfloat1622float2(a2[j]);
      const float2 b = __bfloat1622float2(b2[j]);
      const float sx = 1.0f / (1.0f + expf(-a.x)), sy = 1.0f / (1.0f + expf(-a.y));
      const float dx = sx * (1.0f + a.x * (1.0f - sx)), dy = sy * (1.0f + a.y * (1.0f - sy));
      if (mode == 0) {
        oa2[j] = __floats2bfloat162_rn(g.x * dx, g.y * dy);
      } else {
        oa2[j] = __floats2bfloat162_rn(g.x * b.x * dx, g.y * b.y * dy);
        ob2[j] = __floats2bfloat162_rn(g.x * a.x * sx, g.y * a.y * sy);
      }
    }
    *reinterpret_cast<uint4*>(d_alpha + r * ldda + c) = oa;
    if (mode != 0) *reinterpret_cast<uint4*>(d_beta + r * lddb + c) = ob;
  }
}

// Router backward. The forward keeps the k largest softmax probabilities of a token and
// renormalises them to sum 1 (modules/fast_moe_module.py:93-105): y_j = p_j / sum_sel p, which is
// the softmax over the k selected logits alone. So d_logit_j = y_j (dy_j - sum_i y_i dy_i) for the
// selected experts and 0 for the others. One thread per token (k is small).
__global__ void __launch_bounds__(256)
router_backward_kernel(const long long* __restrict__ topk_idx, const float* __restrict__ y, const float* __restrict__ dy,
                       long long L, int E, int k, float* __restrict__ d_logits, int* status) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= L) return;
  float* row = d_logits + t * E;
  for (int e = 0; e < E; ++e) row[e] = 0.f;
  float dot = 0.f;
  for (int s = 0; s < k; ++s) dot = fmaf(y[t * k + s], dy[t * k + s], dot);
  for (int s = 0; s < k; ++s) {
    const long long e = topk_idx[t * k + s];
    if (e < 0 || e >= E) {
      atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      continue;
    }
    row[e] = y[t * k + s] * (dy[t * k + s] - dot);
  }
}

// d_x[t, c] = sum_e d_logits[t, e] * W[e, c]: one block per token, threads over the columns.
template <typename T>
__global__ void __launch_bounds__(256)
gate_dx_kernel(const float* __restrict__ d_logits, const float* __restrict__ w, long long L, int d, int E, T* __restrict__ dx,
               long long lddx) {
  extern __shared__ float s_dl[];
  const long long t = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_dl[e] = d_logits[t * E + e];
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int e = 0; e < E; ++e) acc = fmaf(s_dl[e], w[static_cast<long long>(e) * d + c], acc);
    stf(dx + t * lddx + c, acc);
  }
}

// d_W[e, c] += sum over a chunk of tokens of d_logits[t, e] * x[t, c]; d_b[e] += sum of d_logits[t, e].
// A block owns 64 columns (two per lane) and a chunk of kGateDwChunk tokens; its 8 warps take the
// tokens t0 + w, t0 + w + 8, ..., keep up to 32 experts' partial sums per lane in registers, fold
// them into one shared [experts][64] table and add that to the fp32 result (cleared beforehand) with
// one global atomic per entry and block.
constexpr int kGateDwChunk = 256;
template <typename T>
__global__ void __launch_bounds__(256)
gate_dw_kernel(const float* __restrict__ d_logits, const T* __restrict__ x, long long ldx, long long L, int d, int E,
               float* __restrict__ dw, float* __restrict__ db) {
  __shared__ float s_acc[32][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + 2 * lane;
  const long long t0 = static_cast<long long>(blockIdx.y) * kGateDwChunk;
  const long long t1 = min(L, t0 + kGateDwChunk);
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int ne = min(32, E - e0);
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * 64; i += blockDim.x) (&s_acc[0][0])[i] = 0.f;
    __syncthreads();
    float a0[32], a1[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) a0[i] = a1[i] = 0.f;
    float bsum = 0.f;                    // lane i of the first column block also sums expert e0 + i's bias gradient
    for (long long t = t0 + warp; t < t1; t += 8) {
      const float x0 = c < d ? ldf<T>(x + t * ldx + c) : 0.f;
      const float x1 = c + 1 < d ? ldf<T>(x + t * ldx + c + 1) : 0.f;
      const float dl = lane < ne ? d_logits[t * E + e0 + lane] : 0.f;
      bsum += dl;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < ne) {
          const float g = __shfl_sync(0xffffffffu, dl, i);
          a0[i] = fmaf(g, x0, a0[i]);
          a1[i] = fmaf(g, x1, a1[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < ne) {
        atomicAdd(&s_acc[i][2 * lane], a0[i]);
        atomicAdd(&s_acc[i][2 * lane + 1], a1[i]);
      }
    }
    if (db != nullptr && blockIdx.x == 0 && lane < ne) atomicAdd(db + e0 + lane, bsum);
    __syncthreads();
    for (int i = threadIdx.x; i < ne * 64; i += blockDim.x) {
      const int ee = i >> 6, cc = blockIdx.x * 64 + (i & 63);
      if (cc < d) atomicAdd(dw + static_cast<long long>(e0 + ee) * d + cc, s_acc[ee][i & 63]);
    }
  }
}

int grid_for(long long work, int per_block) {
  long long b = (work + per_block - 1) / per_block;
  if (b > 148 * 32) b = 148 * 32;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_jagged_pad_offsets(const int64_t* offsets, int E, int dtype, int64_t* kseg, void* stream) {
  const int es = dtype_size(dtype);
  FMOE_REQUIRE(es != 0 && E >= 1 && offsets && kseg, "jagged_pad_offsets: bad arguments");
  pad_offsets_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const long long*>(offsets), E, 128 / es,
                                                                       reinterpret_cast<long long*>(kseg));
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_jagged_transpose_pad(const void* in, int dtype, int64_t in_rows, int64_t ld_in, const int64_t* index,
                                         int index_div, const int64_t* offsets, const int64_t* kseg, int E, int64_t rows,
                                         int cols, void* out, int64_t ld_out, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "jagged_transpose_pad: dtype must be bf16 or f32");
  FMOE_REQUIRE(E >= 1 && rows >= 0 && cols >= 1 && offsets && kseg && out, "jagged_transpose_pad: bad arguments");
  FMOE_REQUIRE(index == nullptr || index_div >= 1, "jagged_transpose_pad: index_div must be >= 1");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  const int unit = 128 / dtype_size(dtype);
  // upper bound of the padded length: every expert adds less than one unit, empty ones exactly one
  const long long padded_max = rows + static_cast<long long>(E) * unit;
  FMOE_REQUIRE(ld_out >= padded_max, "jagged_transpose_pad: ld_out=%lld is below rows + E * %d = %lld", (long long)ld_out,
               unit, padded_max);
  dim3 grid(static_cast<unsigned>((padded_max + 31) / 32), static_cast<unsigned>((cols + 31) / 32), 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto aligned16 = [](const void* p_) { return (reinterpret_cast<uintptr_t>(p_) & 15) == 0; };
  if (dtype == FMOE_BF16 && cols % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && aligned16(in) && aligned16(out)) {
    dim3 grid64(static_cast<unsigned>((padded_max + 63) / 64), static_cast<unsigned>((cols + 63) / 64), 1);
    jagged_transpose_pad_bf16_kernel<<<grid64, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(in), ld_in, in_rows, reinterpret_cast<const long long*>(index), index_div,
        reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(kseg), E, cols,
        static_cast<__nv_bfloat16*>(out), ld_out, status);
  } else if (dtype == FMOE_BF16) {
    jagged_transpose_pad_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(in), ld_in, in_rows, reinterpret_cast<const long long*>(index), index_div,
        reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(kseg), E, cols,
        static_cast<__nv_bfloat16*>(out), ld_out, status);
  } else {
    jagged_transpose_pad_kernel<float><<<grid, 256, 0, st>>>(
        static_cast<const float*>(in), ld_in, in_rows, reinterpret_cast<const long long*>(index), index_div,
        reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(kseg), E, cols,
        static_cast<float*>(out), ld_out, status);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_batched_transpose(const void* in, int dtype, int batch, int64_t in_sb, int64_t ld_in, int rows, int cols,
                                      void* out, int64_t out_sb, int64_t ld_out, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "batched_transpose: dtype must be bf16 or f32");
  FMOE_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, "batched_transpose: negative size");
  if (batch == 0 || rows == 0 || cols == 0) return FMOE_OK;
  FMOE_REQUIRE(in && out && batch <= 65535, "batched_transpose: bad arguments");
  dim3 grid((rows + 31) / 32, (cols + 31) / 32, batch);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto aligned16 = [](const void* p_) { return (reinterpret_cast<uintptr_t>(p_) & 15) == 0; };
  if (dtype == FMOE_BF16 && rows % 8 == 0 && cols % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && in_sb % 8 == 0 &&
      out_sb % 8 == 0 && aligned16(in) && aligned16(out)) {
    dim3 grid64((rows + 63) / 64, (cols + 63) / 64, batch);
    batched_transpose_bf16_kernel<<<grid64, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), in_sb, ld_in, rows, cols,
                                                          static_cast<__nv_bfloat16*>(out), out_sb, ld_out);
  } else if (dtype == FMOE_BF16) {
    batched_transpose_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), in_sb, ld_in, rows, cols,
                                                                   static_cast<__nv_bfloat16*>(out), out_sb, ld_out);
  } else {
    batched_transpose_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(in), in_sb, ld_in, rows, cols,
                                                           static_cast<float*>(out), out_sb, ld_out);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_jagged_jagged_bmm(const int64_t* group_offsets, const int64_t* kseg, int64_t padded_rows,
                                      const void* a_t, int64_t lda, const void* b_t, int64_t ldb, int dtype, int E, int M,
                                      int N, void* out, int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "jagged_jagged_bmm: dtype must be bf16 or f32");
  FMOE_REQUIRE(group_offsets && kseg && M >= 1 && N >= 1 && padded_rows >= 1, "jagged_jagged_bmm: bad arguments");
  GemmDesc g = {};
  g.dtype = dtype;
  g.E = E; g.N = N;
  g.K = static_cast<int>(padded_rows);
  g.offsets = group_offsets;
  g.total_rows = static_cast<int64_t>(E) * M;
  g.a = a_t; g.a_rows = M; g.lda = lda;
  g.b0 = b_t; g.b_se = 0; g.b_sn = ldb;
  g.kseg = kseg;
  g.epilogue = FMOE_EPI_NONE;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  FMOE_REQUIRE(padded_rows < (1ll << 31), "jagged_jagged_bmm: more than 2^31 padded rows");
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_jagged_colsum(const void* x, int dtype, int64_t ldx, const int64_t* offsets, int E, int N, void* out,
                                  int out_dtype, void* stream) {
  FMOE_REQUIRE((dtype == FMOE_BF16 || dtype == FMOE_F32) && (out_dtype == FMOE_BF16 || out_dtype == FMOE_F32),
               "jagged_colsum: dtypes must be bf16 or f32");
  FMOE_REQUIRE(E >= 1 && E <= 65535 && N >= 1 && offsets && out, "jagged_colsum: bad arguments");
  dim3 grid((N + 31) / 32, E, 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long* off = reinterpret_cast<const long long*>(offsets);
#define FMOE_COLSUM(T, OT) jagged_colsum_kernel<T, OT><<<grid, 256, 0, st>>>(static_cast<const T*>(x), ldx, off, N, static_cast<OT*>(out))
  if (dtype == FMOE_BF16 && out_dtype == FMOE_BF16) FMOE_COLSUM(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == FMOE_BF16) FMOE_COLSUM(__nv_bfloat16, float);
  else if (out_dtype == FMOE_F32) FMOE_COLSUM(float, float);
  else FMOE_COLSUM(float, __nv_bfloat16);
#undef FMOE_COLSUM
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_gather_scale_rows(const void* src, int dtype, int64_t src_rows, int64_t lds, const int64_t* index,
                                      int index_div, const void* weight, int w_dtype, const int64_t* weight_index,
                                      int64_t weight_count, int64_t rows, int cols, void* out, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "gather_scale_rows: dtype must be bf16 or f32");
  FMOE_REQUIRE(weight == nullptr || w_dtype == FMOE_BF16 || w_dtype == FMOE_F32, "gather_scale_rows: weight must be bf16 or f32");
  FMOE_REQUIRE(rows >= 0 && cols >= 1 && index_div >= 1, "gather_scale_rows: bad sizes");
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(src && index && out, "gather_scale_rows: NULL pointer argument");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * 32, 256);
  const long long* idx = reinterpret_cast<const long long*>(index);
  const long long* widx = reinterpret_cast<const long long*>(weight_index);
#define FMOE_GS(T, WT)                                                                                                  \
  gather_scale_rows_kernel<T, WT><<<grid, 256, 0, st>>>(static_cast<const T*>(src), src_rows, lds, idx, index_div,      \
                                                        static_cast<const WT*>(weight), widx, weight_count, rows, cols, \
                                                        static_cast<T*>(out), ldo, status)
  if (dtype == FMOE_BF16 && w_dtype == FMOE_F32) FMOE_GS(__nv_bfloat16, float);
  else if (dtype == FMOE_BF16) FMOE_GS(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == FMOE_BF16) FMOE_GS(float, __nv_bfloat16);
  else FMOE_GS(float, float);
#undef FMOE_GS
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_row_dot(const void* a, int64_t lda, const void* b, int64_t b_rows, int64_t ldb, int dtype,
                            const int64_t* index, int index_div, int64_t rows, int cols, float* out, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "row_dot: dtype must be bf16 or f32");
  FMOE_REQUIRE(rows >= 0 && cols >= 1 && index_div >= 1, "row_dot: bad sizes");
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(a && b && out, "row_dot: NULL pointer argument");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * 32, 256);
  const long long* idx = reinterpret_cast<const long long*>(index);
  if (dtype == FMOE_BF16) {
    row_dot_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a), lda,
                                                         static_cast<const __nv_bfloat16*>(b), b_rows, ldb, idx, index_div, rows,
                                                         cols, out, status);
  } else {
    row_dot_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(a), lda, static_cast<const float*>(b), b_rows, ldb,
                                                 idx, index_div, rows, cols, out, status);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_activation_backward(int mode, const void* d_out, int64_t ldd, const void* alpha, int64_t lda,
                                        const void* beta, int64_t ldb, int dtype, int64_t rows, int cols, void* d_alpha,
                                        int64_t ldda, void* d_beta, int64_t lddb, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "activation_backward: dtype must be bf16 or f32");
  FMOE_REQUIRE(mode == 0 || mode == 1, "activation_backward: mode must be 0 (SiLU) or 1 (SwiGLU)");
  FMOE_REQUIRE(rows >= 0 && cols >= 1, "activation_backward: bad sizes");
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(d_out && alpha && d_alpha && (mode == 0 || (beta && d_beta)), "activation_backward: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(rows * cols, 256);
  const auto vec_ok = [](const void* p_, long long ld_) { return p_ == nullptr || ((reinterpret_cast<uintptr_t>(p_) & 15) == 0 && ld_ % 8 == 0); };
  if (dtype == FMOE_BF16 && cols % 8 == 0 && vec_ok(d_out, ldd) && vec_ok(alpha, lda) && vec_ok(beta, ldb) &&
      vec_ok(d_alpha, ldda) && vec_ok(d_beta, lddb)) {
    using T = __nv_bfloat16;
    activation_backward_bf16x8_kernel<<<grid_for(rows * (cols / 8), 256), 256, 0, st>>>(
        mode, static_cast<const T*>(d_out), ldd, static_cast<const T*>(alpha), lda, static_cast<const T*>(beta), ldb, rows, cols,
        static_cast<T*>(d_alpha), ldda, static_cast<T*>(d_beta), lddb);
  } else if (dtype == FMOE_BF16) {
    using T = __nv_bfloat16;
    activation_backward_kernel<T><<<grid, 256, 0, st>>>(mode, static_cast<const T*>(d_out), ldd, static_cast<const T*>(alpha), lda,
                                                        static_cast<const T*>(beta), ldb, rows, cols, static_cast<T*>(d_alpha),
                                                        ldda, static_cast<T*>(d_beta), lddb);
  } else {
    using T = float;
    activation_backward_kernel<T><<<grid, 256, 0, st>>>(mode, static_cast<const T*>(d_out), ldd, static_cast<const T*>(alpha), lda,
                                                        static_cast<const T*>(beta), ldb, rows, cols, static_cast<T*>(d_alpha),
                                                        ldda, static_cast<T*>(d_beta), lddb);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_router_backward(const int64_t* topk_idx, const float* topk_score, const float* d_score, int64_t L, int E,
                                    int k, float* d_logits, void* stream) {
  FMOE_REQUIRE(L >= 0 && E >= 1 && k >= 1 && k <= E, "router_backward: L=%lld E=%d k=%d", (long long)L, E, k);
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(topk_idx && topk_score && d_score && d_logits, "router_backward: NULL pointer argument");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  router_backward_kernel<<<static_cast<unsigned>((L + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(topk_idx), topk_score, d_score, L, E, k, d_logits, status);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_gate_linear_backward(const float* d_logits, const void* x, int x_dtype, int64_t ldx,
                                         const float* gate_w, int64_t L, int d, int E, void* d_x, int64_t lddx,
                                         float* d_gate_w, float* d_gate_b, void* stream) {
  FMOE_REQUIRE(x_dtype == FMOE_BF16 || x_dtype == FMOE_F32, "gate_linear_backward: x must be bf16 or f32");
  FMOE_REQUIRE(L >= 0 && d >= 1 && E >= 1, "gate_linear_backward: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d_gate_w) FMOE_CUDA_OK(cudaMemsetAsync(d_gate_w, 0, static_cast<size_t>(E) * d * sizeof(float), st));
  if (d_gate_b) FMOE_CUDA_OK(cudaMemsetAsync(d_gate_b, 0, static_cast<size_t>(E) * sizeof(float), st));
  if (L == 0) return FMOE_OK;
  FMOE_REQUIRE(d_logits && x && gate_w, "gate_linear_backward: NULL pointer argument");
  if (d_x != nullptr) {
    const size_t smem = static_cast<size_t>(E) * sizeof(float);
    if (x_dtype == FMOE_BF16) {
      gate_dx_kernel<__nv_bfloat16><<<static_cast<unsigned>(L), 256, smem, st>>>(d_logits, gate_w, L, d, E,
                                                                               static_cast<__nv_bfloat16*>(d_x), lddx);
    } else {
      gate_dx_kernel<float><<<static_cast<unsigned>(L), 256, smem, st>>>(d_logits, gate_w, L, d, E, static_cast<float*>(d_x), lddx);
    }
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
  }
  if (d_gate_w != nullptr) {
    FMOE_REQUIRE(L <= 65535ll * kGateDwChunk, "gate_linear_backward: L=%lld exceeds %lld tokens", (long long)L,
                 65535ll * kGateDwChunk);
    dim3 grid((d + 63) / 64, static_cast<unsigned>((L + kGateDwChunk - 1) / kGateDwChunk), 1);
    if (x_dtype == FMOE_BF16) {
      gate_dw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(d_logits, static_cast<const __nv_bfloat16*>(x), ldx, L, d, E,
                                                           d_gate_w, d_gate_b);
    } else {
      gate_dw_kernel<float><<<grid, 256, 0, st>>>(d_logits, static_cast<const float*>(x), ldx, L, d, E, d_gate_w, d_gate_b);
    }
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
  }
  return FMOE_OK;
}
