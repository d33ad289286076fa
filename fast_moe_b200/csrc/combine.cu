// Gate-weighted k-way combine (mul_merge_k_add) and the elementwise SiLU pass.
//
// out[t, :] = sum_j value[p_j, :] * weight[weight_index[p_j]],  p_j = reverse_index[t, j]
//
// Replaces pytorch_mul_merge_k_add (kernels/pytorch/moe.py:14-37: gather of the gate weights,
// mul, fp32 upcast, index_add, cast = about five passes over [L*k, D]) and the Triton gather form
// _mul_merge_k_add_fwd (kernels/triton/triton_moe.py:864-914) with one pass: HBM-bound, reads
// L*k*D values once and writes L*D. The sum runs in fp32 in ascending row order, which is the
// order index_add visits the rows of one token, so the result is reproducible bit for bit.
#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

constexpr int kCombineThreads = 256;

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename VT, typename WT, typename OT, int VEC>
__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const long long* __restrict__ reverse_index, const VT* __restrict__ value, long long ldv,
               const WT* __restrict__ weight, const long long* __restrict__ weight_index, long long L, int k, int D,
               OT* __restrict__ out, long long ldo, long long n_rows, int* status) {
  // both bf16: Tensor.mul rounds the product to bf16 before the fp32 accumulation
  constexpr bool kRoundProduct = (sizeof(VT) == 2 && sizeof(WT) == 2);
  const int vec_per_row = (D + VEC - 1) / VEC;
  const long long total = L * vec_per_row;
  for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total;
       w += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = w / vec_per_row;
    const int c0 = static_cast<int>(w - t * vec_per_row) * VEC;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    // Rows are handled in groups of up to 4: first all their indices, then all gate weights and
    // values, so that the loads of a group are in flight together instead of one dependent chain
    // per row. The accumulation order stays ascending j.
    constexpr int kGroup = 4;
    for (int j0 = 0; j0 < k; j0 += kGroup) {
      long long prow[kGroup];
      float g[kGroup];
      bool ok[kGroup];
#pragma unroll
      for (int jj = 0; jj < kGroup; ++jj) {
        ok[jj] = j0 + jj < k;
        prow[jj] = ok[jj] ? reverse_index[t * k + j0 + jj] : 0;
        if (ok[jj] && (prow[jj] < 0 || prow[jj] >= n_rows)) {
          atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
          ok[jj] = false;
        }
      }
      if (weight != nullptr) {
        long long wi[kGroup];
#pragma unroll
        for (int jj = 0; jj < kGroup; ++jj) {
          wi[jj] = ok[jj] ? (weight_index ? weight_index[prow[jj]] : prow[jj]) : 0;
          if (ok[jj] && (wi[jj] < 0 || wi[jj] >= n_rows)) {
            atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
            ok[jj] = false;
          }
        }
#pragma unroll
        for (int jj = 0; jj < kGroup; ++jj) g[jj] = ok[jj] ? ldf(weight + wi[jj]) : 0.f;
      } else {
#pragma unroll
        for (int jj = 0; jj < kGroup; ++jj) g[jj] = 1.f;
      }
      float v[kGroup][VEC];
#pragma unroll
      for (int jj = 0; jj < kGroup; ++jj) {
        if (!ok[jj]) continue;
        const VT* src = value + prow[jj] * ldv + c0;
        if (c0 + VEC <= D) {
          if constexpr (sizeof(VT) * VEC == 16) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const VT* e = reinterpret_cast<const VT*>(&raw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[jj][i] = ldf(e + i);
          } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[jj][i] = ldf(src + i);
          }
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) v[jj][i] = (c0 + i < D) ? ldf(src + i) : 0.f;
        }
      }
#pragma unroll
      for (int jj = 0; jj < kGroup; ++jj) {
        if (!ok[jj]) continue;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float prod = weight != nullptr ? __fmul_rn(v[jj][i], g[jj]) : v[jj][i];
          if (kRoundProduct && weight != nullptr) prod = __bfloat162float(__float2bfloat16_rn(prod));
          acc[i] = __fadd_rn(acc[i], prod);
        }
      }
    }
    OT* dst = out + t * ldo + c0;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (c0 + i < D) {
        if constexpr (sizeof(OT) == 2) {
          dst[i] = __float2bfloat16_rn(acc[i]);
        } else {
          dst[i] = acc[i];
        }
      }
    }
  }
}

// The same sum with one warp per token (16-byte-aligned rows, k <= 32, D a multiple of the vector
// width): lane j fetches row index, weight index and gate weight of the token's j-th row once and
// the warp shares them by shuffle, so the only loads left in the inner loop are the value pieces,
// k x kPieces of them in flight per lane. combine_kernel runs four dependent loads per 16-byte
// piece per thread and reached 1.2-1.5 TB/s; same arithmetic, same order, same bits.
template <typename VT, typename WT, typename OT, int VEC>
__global__ void __launch_bounds__(kCombineThreads)
combine_warp_kernel(const long long* __restrict__ reverse_index, const VT* __restrict__ value, long long ldv,
                    const WT* __restrict__ weight, const long long* __restrict__ weight_index, long long L, int k,
                    int D, OT* __restrict__ out, long long ldo, long long n_rows, int* status) {
  constexpr bool kRoundProduct = (sizeof(VT) == 2 && sizeof(WT) == 2);
  constexpr int kPieces = 2;                       // 16-byte pieces per lane and trip
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < L; t += warps) {
    long long prow = -1;
    float g = 1.f;
    if (lane < k) {
      prow = reverse_index[t * k + lane];
      if (prow < 0 || prow >= n_rows) {
        atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
        prow = -1;
      } else if (weight != nullptr) {
        const long long wi = weight_index ? weight_index[prow] : prow;
        if (wi < 0 || wi >= n_rows) {
          atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
          prow = -1;
        } else {
          g = ldf(weight + wi);
        }
      }
    }
    // trip count uniform across the warp (the shuffles below need all 32 lanes); lanes whose
    // piece lies past the end of the row just skip their loads and stores
    for (int base = 0; base < D; base += 32 * VEC * kPieces) {
      const int c0 = base + lane * VEC;
      float acc[kPieces][VEC];
#pragma unroll
      for (int u = 0; u < kPieces; ++u)
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[u][i] = 0.f;
      // rows in groups of four: all their value loads go out before the first sum, so a lane has
      // up to 4 x kPieces loads in flight; the sums stay in ascending j order
      constexpr int kGroup = 4;
      for (int j0 = 0; j0 < k; j0 += kGroup) {
        uint4 raw[kGroup][kPieces];
        float gj[kGroup];
        bool use[kGroup];
#pragma unroll
        for (int jj = 0; jj < kGroup; ++jj) {
          const long long pj = __shfl_sync(0xffffffffu, prow, (j0 + jj) & 31);
          gj[jj] = __shfl_sync(0xffffffffu, g, (j0 + jj) & 31);
          use[jj] = (j0 + jj < k) && pj >= 0;          // warp-uniform
          if (use[jj]) {
            const VT* src = value + pj * ldv + c0;
#pragma unroll
            for (int u = 0; u < kPieces; ++u) {
              if (c0 + u * 32 * VEC < D) raw[jj][u] = *reinterpret_cast<const uint4*>(src + u * 32 * VEC);
            }
          }
        }
#pragma unroll
        for (int jj = 0; jj < kGroup; ++jj) {
          if (!use[jj]) continue;
#pragma unroll
          for (int u = 0; u < kPieces; ++u) {
            if (c0 + u * 32 * VEC < D) {
              const VT* e = reinterpret_cast<const VT*>(&raw[jj][u]);
#pragma unroll
              for (int i = 0; i < VEC; ++i) {
                const float v = ldf(e + i);
                float prod = weight != nullptr ? __fmul_rn(v, gj[jj]) : v;
                if (kRoundProduct && weight != nullptr) prod = __bfloat162float(__float2bfloat16_rn(prod));
                acc[u][i] = __fadd_rn(acc[u][i], prod);
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kPieces; ++u) {
        const int c = c0 + u * 32 * VEC;
        if (c < D) {
          OT* dst = out + t * ldo + c;
          if constexpr (sizeof(OT) == 2) {
            uint32_t w[VEC / 2];
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(acc[u][2 * i], acc[u][2 * i + 1]);
              w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            if constexpr (VEC == 8) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
              *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < VEC; i += 4) {
              *reinterpret_cast<float4*>(dst + i) = make_float4(acc[u][i], acc[u][i + 1], acc[u][i + 2], acc[u][i + 3]);
            }
          }
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_kernel(const T* __restrict__ in, long long ldi, T* __restrict__ out, long long ldo, long long rows, int cols) {
  const long long total = rows * cols;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const int c = static_cast<int>(i - r * cols);
    const float x = ldf(in + r * ldi + c);
    const float y = x / (1.0f + expf(-x));
    if constexpr (sizeof(T) == 2) {
      out[r * ldo + c] = __float2bfloat16_rn(y);
    } else {
      out[r * ldo + c] = y;
    }
  }
}

// The same for bf16 rows that allow 16-byte accesses (cols a multiple of 8, aligned rows): 8 values
// per thread and step. Same arithmetic as silu_kernel (expf, IEEE division).
__global__ void __launch_bounds__(256)
silu_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, long long ldi, __nv_bfloat16* __restrict__ out, long long ldo,
                   long long rows, int cols) {
  const int vec = cols >> 3;
  const long long total = rows * vec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec;
    const int c = static_cast<int>(i - r * vec) << 3;
    const uint4 xv = *reinterpret_cast<const uint4*>(in + r * ldi + c);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
    uint4 yv;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&yv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(x2[j]);
      y2[j] = __floats2bfloat162_rn(x.x / (1.0f + expf(-x.x)), x.y / (1.0f + expf(-x.y)));
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) = yv;
  }
}

// fp32 -> three bf16 terms, hi + mid + lo = x to about 2^-24 relative (hi = bf16(x), mid =
// bf16(x - hi), lo = bf16(x - hi - mid); the subtractions are exact in fp32). The six partial
// products a_i * b_j with i + j <= 2 reproduce a * b to fp32 accuracy, and each of them is exact
// in the tensor core's fp32 accumulator, so an fp32 product can run as ONE bf16 GEMM over a
// reduction dimension six times as long: the left operand's row is laid out as
// [hi | hi | mid | hi | lo | mid] (pattern 0), the right operand's as [hi | mid | hi | lo | hi | mid]
// (pattern 1). This is the path fp32 callers get when TF32 is not allowed, which is the
// default of torch.backends.cuda.matmul.allow_tf32 that the reference's kernels follow
// (kernels/triton/triton_moe.py:592).
__global__ void __launch_bounds__(256)
split_bf16x3_kernel(const float* __restrict__ in, long long ldi, long long rows, int cols, int cols_out, int pattern,
                    int apply_silu, __nv_bfloat16* __restrict__ out, long long ldo) {
  const long long total = rows * cols_out;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols_out;
    const int c = static_cast<int>(i - r * cols_out);
    float x = c < cols ? in[r * ldi + c] : 0.f;          // columns beyond `cols` are zero padding
    if (apply_silu) x = x / (1.0f + expf(-x));
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* o = out + r * ldo + c;
    const long long s = cols_out;
    if (pattern == 0) {
      o[0] = hi; o[s] = hi; o[2 * s] = mid; o[3 * s] = hi; o[4 * s] = lo; o[5 * s] = mid;
    } else {
      o[0] = hi; o[s] = mid; o[2 * s] = hi; o[3 * s] = lo; o[4 * s] = hi; o[5 * s] = mid;
    }
  }
}

// Row index of index_select_jagged_bmm_3D: sorted row p of expert e reads slice e of its token,
// i.e. row token * E + e of the [L * E, K] view: out[p] = (index[p] / A) * E + e(p), where e(p) is
// the expert whose segment [offsets[e], offsets[e+1]) holds p.
__global__ void __launch_bounds__(256)
expand_3d_index_kernel(const long long* __restrict__ offsets, const long long* __restrict__ index, int A, int E,
                       long long rows, long long* __restrict__ out) {
  for (long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; p < rows;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= p) lo = mid; else hi = mid;
    }
    out[p] = (index[p] / A) * E + lo;
  }
}

// dst[r, :] = src[index[r] / div, :] in 16-byte pieces (or bytes when rows are not 16-byte
// aligned). One warp-sized group of threads walks a row, so reads and writes are coalesced.
template <typename V>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ src, long long src_rows, long long lds_bytes,
                   const long long* __restrict__ index, int div, long long rows, int row_bytes,
                   uint8_t* __restrict__ dst, long long ldd_bytes, int* status) {
  const int vec_per_row = row_bytes / static_cast<int>(sizeof(V));
  const long long total = rows * vec_per_row;
  for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total;
       w += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = w / vec_per_row;
    const int c = static_cast<int>(w - r * vec_per_row);
    long long s = index[r];
    if (div != 1) s /= div;
    if (s < 0 || s >= src_rows) {
      atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      reinterpret_cast<V*>(dst + r * ldd_bytes)[c] = V{};      // a row that does not exist reads as zeros
      continue;
    }
    reinterpret_cast<V*>(dst + r * ldd_bytes)[c] = reinterpret_cast<const V*>(src + s * lds_bytes)[c];
  }
}

// 16-byte-aligned rows of at least 512 bytes: one warp per row. The row index is read once per
// row (no division per 16-byte piece), and a lane has up to four loads in flight before its
// first store. No warp-level primitives: lanes are independent.
__global__ void __launch_bounds__(256)
gather_rows_warp_kernel(const uint8_t* __restrict__ src, long long src_rows, long long lds_bytes,
                        const long long* __restrict__ index, int div, long long rows, int vec_per_row,
                        uint8_t* __restrict__ dst, long long ldd_bytes, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    long long s = index[r];
    if (div != 1) s /= div;
    uint4* d = reinterpret_cast<uint4*>(dst + r * ldd_bytes);
    if (s < 0 || s >= src_rows) {
      if (lane == 0) atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      for (int c = lane; c < vec_per_row; c += 32) d[c] = make_uint4(0, 0, 0, 0);   // a row that does not exist reads as zeros
      continue;
    }
    const uint4* a = reinterpret_cast<const uint4*>(src + s * lds_bytes);
    for (int c0 = lane; c0 < vec_per_row; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < vec_per_row) v[u] = a[c0 + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < vec_per_row) d[c0 + 32 * u] = v[u];
    }
  }
}

template <typename VT, typename WT, typename OT>
int launch_combine(const long long* rev, const void* value, long long ldv, const void* weight, const long long* widx,
                   long long L, int k, int D, void* out, long long ldo, int* status, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(VT);
  // vector loads need every row start 16-byte aligned
  const bool aligned = ((ldv * sizeof(VT)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(value) & 15) == 0);
  const long long n_rows = L * k;
  const long long work = L * ((D + VEC - 1) / VEC);
  long long blocks = (work + kCombineThreads - 1) / kCombineThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  const bool out_aligned = ((ldo * sizeof(OT)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (aligned && out_aligned && k <= 32 && D % VEC == 0) {
    long long wb = (L * 32 + kCombineThreads - 1) / kCombineThreads;     // one warp per token
    if (wb > 148 * 16) wb = 148 * 16;
    if (wb < 1) wb = 1;
    combine_warp_kernel<VT, WT, OT, VEC><<<static_cast<unsigned>(wb), kCombineThreads, 0, st>>>(
        rev, static_cast<const VT*>(value), ldv, static_cast<const WT*>(weight), widx, L, k, D,
        static_cast<OT*>(out), ldo, n_rows, status);
  } else if (aligned) {
    combine_kernel<VT, WT, OT, VEC><<<static_cast<unsigned>(blocks), kCombineThreads, 0, st>>>(
        rev, static_cast<const VT*>(value), ldv, static_cast<const WT*>(weight), widx, L, k, D,
        static_cast<OT*>(out), ldo, n_rows, status);
  } else {
    const long long work1 = L * static_cast<long long>(D);
    long long b1 = (work1 + kCombineThreads - 1) / kCombineThreads;
    if (b1 > 148 * 16) b1 = 148 * 16;
    if (b1 < 1) b1 = 1;
    combine_kernel<VT, WT, OT, 1><<<static_cast<unsigned>(b1), kCombineThreads, 0, st>>>(
        rev, static_cast<const VT*>(value), ldv, static_cast<const WT*>(weight), widx, L, k, D,
        static_cast<OT*>(out), ldo, n_rows, status);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

}  // namespace

int launch_silu(const void* in, int dtype, long long ldi, void* out, long long ldo, long long rows, int cols,
                cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return FMOE_OK;
  long long blocks = (rows * cols + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  const bool vec8 = dtype == FMOE_BF16 && cols % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 &&
                    (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  if (vec8) {
    long long b8 = (rows * (cols / 8) + 255) / 256;
    if (b8 > 148 * 32) b8 = 148 * 32;
    silu_bf16x8_kernel<<<static_cast<unsigned>(b8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), ldi,
                                                                  static_cast<__nv_bfloat16*>(out), ldo, rows, cols);
  } else if (dtype == FMOE_BF16) {
    silu_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(in), ldi, static_cast<__nv_bfloat16*>(out), ldo, rows, cols);
  } else if (dtype == FMOE_F32) {
    silu_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const float*>(in), ldi,
                                                                       static_cast<float*>(out), ldo, rows, cols);
  } else {
    return fail(FMOE_ERR_BAD_ARG, "silu: dtype %d not supported", dtype);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_gather_rows(const void* src, int dtype, int64_t src_rows, int64_t lds, const int64_t* index,
                                int index_div, int64_t rows, int cols, void* dst, int64_t ldd, void* stream) {
  const int es = dtype_size(dtype);
  FMOE_REQUIRE(es != 0, "gather_rows: unknown dtype %d", dtype);
  FMOE_REQUIRE(rows >= 0 && cols >= 1 && index_div >= 1, "gather_rows: rows=%lld cols=%d div=%d", (long long)rows, cols,
               index_div);
  FMOE_REQUIRE(rows == 0 || (src && index && dst), "gather_rows: NULL pointer argument");
  if (rows == 0) return FMOE_OK;
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int row_bytes = cols * es;
  const bool v16 = (row_bytes % 16 == 0) && ((lds * es) % 16 == 0) && ((ldd * es) % 16 == 0) &&
                   ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  const long long work = rows * (v16 ? row_bytes / 16 : row_bytes);
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const long long* idx = reinterpret_cast<const long long*>(index);
  if (v16 && row_bytes >= 512) {
    long long wb = (rows * 32 + 255) / 256;     // one warp per row
    if (wb > 148 * 16) wb = 148 * 16;
    gather_rows_warp_kernel<<<static_cast<unsigned>(wb), 256, 0, st>>>(
        static_cast<const uint8_t*>(src), src_rows, lds * es, idx, index_div, rows, row_bytes / 16,
        static_cast<uint8_t*>(dst), ldd * es, status);
  } else if (v16)
    gather_rows_kernel<uint4><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint8_t*>(src), src_rows, lds * es, idx, index_div, rows, row_bytes,
        static_cast<uint8_t*>(dst), ldd * es, status);
  else
    gather_rows_kernel<uint8_t><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint8_t*>(src), src_rows, lds * es, idx, index_div, rows, row_bytes,
        static_cast<uint8_t*>(dst), ldd * es, status);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_mul_merge_k_add(const int64_t* reverse_index, const void* value, int v_dtype, int64_t ldv,
                                    const void* weight, int w_dtype, const int64_t* weight_index, int64_t L, int k,
                                    int D, void* out, int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(L >= 0 && k >= 1 && D >= 1, "mul_merge_k_add: L=%lld k=%d D=%d", (long long)L, k, D);
  FMOE_REQUIRE(L == 0 || (reverse_index && value && out), "mul_merge_k_add: NULL pointer argument");
  FMOE_REQUIRE(v_dtype == FMOE_BF16 || v_dtype == FMOE_F32, "mul_merge_k_add: value must be bf16 or f32");
  FMOE_REQUIRE(weight == nullptr || w_dtype == FMOE_BF16 || w_dtype == FMOE_F32,
               "mul_merge_k_add: weight must be bf16 or f32");
  // Tensor.mul promotes bf16 x f32 to f32; with no weight the value type is kept.
  const int expect_out = (weight != nullptr && (v_dtype == FMOE_F32 || w_dtype == FMOE_F32)) ? FMOE_F32 : v_dtype;
  FMOE_REQUIRE(out_dtype == expect_out, "mul_merge_k_add: out dtype %d, expected %d (type promotion of value*weight)",
               out_dtype, expect_out);
  if (L == 0) return FMOE_OK;
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long* rev = reinterpret_cast<const long long*>(reverse_index);
  const long long* widx = reinterpret_cast<const long long*>(weight_index);
  const bool wf32 = (weight == nullptr) ? (v_dtype == FMOE_F32) : (w_dtype == FMOE_F32);
  if (v_dtype == FMOE_BF16 && !wf32)
    return launch_combine<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(rev, value, ldv, weight, widx, L, k, D, out, ldo, status, st);
  if (v_dtype == FMOE_BF16 && wf32)
    return launch_combine<__nv_bfloat16, float, float>(rev, value, ldv, weight, widx, L, k, D, out, ldo, status, st);
  if (v_dtype == FMOE_F32 && wf32)
    return launch_combine<float, float, float>(rev, value, ldv, weight, widx, L, k, D, out, ldo, status, st);
  return launch_combine<float, __nv_bfloat16, float>(rev, value, ldv, weight, widx, L, k, D, out, ldo, status, st);
}

extern "C" int fmoe_split_f32_bf16x3(const float* in, int64_t rows, int cols, int64_t ldi, int cols_padded, int pattern,
                                     int apply_silu, void* out, int64_t ldo, void* stream) {
  FMOE_REQUIRE(rows >= 0 && cols >= 1 && cols_padded >= cols, "split_f32_bf16x3: rows=%lld cols=%d cols_padded=%d",
               (long long)rows, cols, cols_padded);
  FMOE_REQUIRE(pattern == 0 || pattern == 1, "split_f32_bf16x3: pattern must be 0 (left operand) or 1 (right operand)");
  FMOE_REQUIRE(ldo >= 6ll * cols_padded, "split_f32_bf16x3: output rows need 6 * cols_padded = %lld elements",
               6ll * cols_padded);
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(in && out, "split_f32_bf16x3: NULL pointer argument");
  long long blocks = (rows * cols_padded + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  split_bf16x3_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      in, ldi, rows, cols, cols_padded, pattern, apply_silu, static_cast<__nv_bfloat16*>(out), ldo);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_expand_3d_index(const int64_t* offsets, const int64_t* index, int A, int E, int64_t rows,
                                    int64_t* out, void* stream) {
  FMOE_REQUIRE(A >= 1 && E >= 1 && rows >= 0, "expand_3d_index: A=%d E=%d rows=%lld", A, E, (long long)rows);
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(offsets && index && out, "expand_3d_index: NULL pointer argument");
  long long blocks = (rows + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  expand_3d_index_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(offsets), reinterpret_cast<const long long*>(index), A, E, rows,
      reinterpret_cast<long long*>(out));
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}
