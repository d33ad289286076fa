// Rowwise FP8 (e4m3fn) quantisation with a power-of-two scale per row.
//
//   amax  = max |row|
//   scale = 2^floor(log2(448 / amax)), replaced by 2^127 when that is inf or NaN
//   q     = e4m3fn(row * scale)
//
// Follows calculate_scale / pytorch_rowwise_quant_fp8 (kernels/pytorch/quant_fp8.py:13-34),
// pytorch_silu_jagged_fp8 and pytorch_bmm_weight_rowwise_quant_fp8
// (kernels/pytorch/moe_fp8.py:17-43); replaces the two-pass Triton kernels
// (kernels/triton/triton_quant_fp8.py:130-302, triton_moe_fp8.py:142-219, :292-348).
// HBM-bound: each row is read once from DRAM (the second pass hits L1/L2) and written once at
// one byte per element.
#include <math.h>

#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

// 448 / amax is evaluated in the type of amax (the reference divides a Python scalar by a
// tensor, which keeps the tensor's type), then widened to fp32 for log2/floor/exp2.
__device__ __forceinline__ float calc_scale(float amax, bool amax_is_bf16) {
  float x = __fdiv_rn(448.0f, amax);
  if (amax_is_bf16) x = __bfloat162float(__float2bfloat16_rn(x));
  // Common case without any logarithm: for a normal positive x = m * 2^e (1 <= m < 2) the fp32
  // log2 is e + log2(m), and it can only round up to e + 1 when m is within a few ulps of 2.
  // With the top ten fraction bits of m not all ones, 1 - log2(m) > 7e-4, far above half an ulp
  // of any fp32 in [-150, 129], so floor(log2(x)) = e and the scale is x with its fraction
  // cleared. Everything else (m next to 2, zero, subnormal, inf, NaN, negative) takes the exact
  // path below; the double-precision log2 there is slow on this part and used to sit on the
  // critical path of every row.
  {
    const uint32_t bits = __float_as_uint(x);
    const uint32_t ex = (bits >> 23) & 0xFFu;
    if ((bits >> 31) == 0u && ex != 0u && ex != 255u && ((bits >> 13) & 0x3FFu) != 0x3FFu) {
      return __uint_as_float(bits & 0x7F800000u);
    }
  }
  // fp32 log2 rounded correctly (computed in double, then rounded once). floor() of it decides
  // the exponent, so values of x a hair below a power of two behave as they do in fp32 log2.
  const float y = static_cast<float>(log2(static_cast<double>(x)));
  const float two127 = 1.7014118346046923e38f;
  if (isnan(y) || y == INFINITY) return two127;
  if (y == -INFINITY) return 0.0f;          // amax = inf: exp2(-inf) = 0 is finite and is kept
  const int f = static_cast<int>(floorf(y));
  if (f >= 128) return two127;              // exp2 overflows to inf -> fallback
  return ldexpf(1.0f, f);
}

// Two floats -> two e4m3fn bytes (low byte = a). Hardware conversion rounds to nearest even
// and saturates; the reference cast does not saturate: anything that rounds beyond 448
// (|v| > 464) and NaN become 0x7F with the sign kept.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float a, float b) {
  uint16_t pk;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(pk) : "f"(a), "f"(b));
  uint32_t r = pk;
  if (!(fabsf(a) <= 464.0f)) r = (r & 0xFF00u) | 0x7Fu | ((__float_as_uint(a) >> 24) & 0x80u);
  if (!(fabsf(b) <= 464.0f)) r = (r & 0x00FFu) | ((0x7Fu | ((__float_as_uint(b) >> 24) & 0x80u)) << 8);
  return r;
}

template <typename T>
__device__ __forceinline__ float ld_act(const T* p, bool apply_silu) {
  float v;
  if constexpr (sizeof(T) == 2) {
    v = __bfloat162float(*p);
    if (apply_silu) v = __bfloat162float(__float2bfloat16_rn(v / (1.0f + expf(-v))));
  } else {
    v = *p;
    if (apply_silu) v = v / (1.0f + expf(-v));
  }
  return v;
}

// TPR threads cooperate on one row; a block holds 256 / TPR rows.
template <typename T, int TPR>
__global__ void __launch_bounds__(256)
rowwise_quant_kernel(const T* __restrict__ in, long long ldi, long long rows, int cols, int apply_silu,
                     int store_reciprocal, uint8_t* __restrict__ q, long long ldq, float* __restrict__ scale_out) {
  constexpr int kRowsPerBlock = 256 / TPR;
  __shared__ float s_red[256 / 32];
  __shared__ int s_nan[256 / 32];
  const int sub = threadIdx.x / TPR;
  const int lane_in_row = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * kRowsPerBlock + sub;
  const bool active = row < rows;
  const T* src = in + (active ? row : 0) * ldi;
  const bool silu = apply_silu != 0;

  float amax = 0.f;
  int has_nan = 0;
  if (active) {
    for (int c = lane_in_row; c < cols; c += TPR) {
      const float v = fabsf(ld_act<T>(src + c, silu));
      has_nan |= isnan(v) ? 1 : 0;
      amax = fmaxf(amax, v);
    }
  }
  // reduce over the TPR threads of the row
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (o < TPR) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      has_nan |= __shfl_xor_sync(0xffffffffu, has_nan, o);
    }
  }
  if constexpr (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) {
      s_red[warp] = amax;
      s_nan[warp] = has_nan;
    }
    __syncthreads();
    amax = 0.f;
    has_nan = 0;
#pragma unroll
    for (int w = 0; w < 256 / 32; ++w) {
      amax = fmaxf(amax, s_red[w]);
      has_nan |= s_nan[w];
    }
  }
  if (has_nan) amax = NAN;   // torch.max propagates NaN
  // after SiLU the reference holds fp32 values, so the division is fp32 there
  const float scale = calc_scale(amax, sizeof(T) == 2 && !silu);
  if (active && lane_in_row == 0 && scale_out != nullptr) {
    scale_out[row] = store_reciprocal ? __fdiv_rn(1.0f, scale) : scale;
  }
  if (!active) return;
  uint8_t* dst = q + row * ldq;
  const int pairs = cols >> 1;
  const bool dst_even = (reinterpret_cast<uintptr_t>(dst) & 1) == 0;
  if (dst_even) {
    for (int pidx = lane_in_row; pidx < pairs; pidx += TPR) {
      const float a = ld_act<T>(src + 2 * pidx, silu) * scale;
      const float b = ld_act<T>(src + 2 * pidx + 1, silu) * scale;
      *reinterpret_cast<uint16_t*>(dst + 2 * pidx) = static_cast<uint16_t>(f32x2_to_e4m3x2(a, b));
    }
    if ((cols & 1) && lane_in_row == 0) {
      const float a = ld_act<T>(src + cols - 1, silu) * scale;
      dst[cols - 1] = static_cast<uint8_t>(f32x2_to_e4m3x2(a, 0.f) & 0xFF);
    }
  } else {
    for (int c = lane_in_row; c < cols; c += TPR) {
      const float a = ld_act<T>(src + c, silu) * scale;
      dst[c] = static_cast<uint8_t>(f32x2_to_e4m3x2(a, 0.f) & 0xFF);
    }
  }
}

// Wide bf16 rows (the activations of the FP8 layer: 4096 or 14336 columns) in ONE pass: a block
// of 256 threads owns a row, every thread keeps up to kRegVecs 16-byte pieces of it in registers
// between the absmax reduction and the cast, and writes 8 payload bytes per piece. Same
// arithmetic per element as rowwise_quant_kernel (bit-identical results); the row is read from
// HBM once instead of once from HBM and once from L2, with 16-byte instead of 2-byte accesses.
constexpr int kRegVecsMax = 8;  // 256 threads x 8 pieces x 8 values: rows up to 16384 columns

__device__ __forceinline__ float act_bf16(float v, bool apply_silu) {
  if (apply_silu) v = __bfloat162float(__float2bfloat16_rn(v / (1.0f + expf(-v))));
  return v;
}

// kRegVecs = 2 serves rows up to 4096 columns with a quarter of the registers, so that eight
// blocks fit on an SM: short rows need more rows in flight to cover the HBM latency.
template <int kRegVecs>
__global__ void __launch_bounds__(256, kRegVecs <= 2 ? 8 : 1)
rowwise_quant_bf16_regs_kernel(const __nv_bfloat16* __restrict__ in, long long ldi, long long rows, int cols,
                               int apply_silu, int store_reciprocal, uint8_t* __restrict__ q, long long ldq,
                               float* __restrict__ scale_out) {
  __shared__ float s_red[256 / 32];
  __shared__ int s_nan[256 / 32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* src = in + row * ldi;
  const bool silu = apply_silu != 0;
  const int nvec = cols >> 3;                  // the host checked: cols a multiple of 8, nvec <= 256 * kRegVecs
  uint4 buf[kRegVecs];
#pragma unroll
  for (int i = 0; i < kRegVecs; ++i) {
    const int v = i * 256 + threadIdx.x;
    buf[i] = v < nvec ? *reinterpret_cast<const uint4*>(src + 8 * v) : make_uint4(0, 0, 0, 0);
  }
  float amax = 0.f;
  int has_nan = 0;
  if (!silu) {
    // |bf16| orders like its 15 magnitude bits, and NaN is any magnitude above 0x7F80: one
    // packed max per pair of values instead of unpack / fabs / isnan / fmax
    uint32_t m2 = 0u;
#pragma unroll
    for (int i = 0; i < kRegVecs; ++i) {
      m2 = __vmaxu2(m2, buf[i].x & 0x7FFF7FFFu);
      m2 = __vmaxu2(m2, buf[i].y & 0x7FFF7FFFu);
      m2 = __vmaxu2(m2, buf[i].z & 0x7FFF7FFFu);
      m2 = __vmaxu2(m2, buf[i].w & 0x7FFF7FFFu);
    }
    const uint32_t m = max(m2 & 0xFFFFu, m2 >> 16);
    has_nan = m > 0x7F80u ? 1 : 0;
    amax = __uint_as_float(m << 16);
  } else {
#pragma unroll
    for (int i = 0; i < kRegVecs; ++i) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&buf[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        const float a = fabsf(act_bf16(f.x, true));
        const float b = fabsf(act_bf16(f.y, true));
        has_nan |= (isnan(a) || isnan(b)) ? 1 : 0;
        amax = fmaxf(amax, fmaxf(a, b));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    has_nan |= __shfl_xor_sync(0xffffffffu, has_nan, o);
  }
  if ((threadIdx.x & 31) == 0) {
    s_red[threadIdx.x >> 5] = amax;
    s_nan[threadIdx.x >> 5] = has_nan;
  }
  __syncthreads();
  amax = 0.f;
  has_nan = 0;
#pragma unroll
  for (int w = 0; w < 256 / 32; ++w) {
    amax = fmaxf(amax, s_red[w]);
    has_nan |= s_nan[w];
  }
  if (has_nan) amax = NAN;
  const float scale = calc_scale(amax, !silu);
  if (threadIdx.x == 0 && scale_out != nullptr) scale_out[row] = store_reciprocal ? __fdiv_rn(1.0f, scale) : scale;
  uint8_t* dst = q + row * ldq;
  // No element of a clean row can leave the e4m3 range after scaling (|v| * scale <= 448 by the
  // choice of scale), so the non-saturating fix-up of f32x2_to_e4m3x2 is only needed for rows
  // with NaN / inf or a degenerate scale.
  const bool clean = !silu && !has_nan && amax * scale <= 464.0f;
#pragma unroll
  for (int i = 0; i < kRegVecs; ++i) {
    const int v = i * 256 + threadIdx.x;
    if (v < nvec) {
      const uint32_t raw[4] = {buf[i].x, buf[i].y, buf[i].z, buf[i].w};
      uint32_t w[2];
      if (clean) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint16_t lo, hi;
          const float a0 = __uint_as_float(raw[2 * j] << 16) * scale, a1 = __uint_as_float(raw[2 * j] & 0xFFFF0000u) * scale;
          const float b0 = __uint_as_float(raw[2 * j + 1] << 16) * scale, b1 = __uint_as_float(raw[2 * j + 1] & 0xFFFF0000u) * scale;
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a0), "f"(a1));
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(b0), "f"(b1));
          w[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        }
      } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(raw);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float2 f0 = __bfloat1622float2(h[2 * j]);
          const float2 f1 = __bfloat1622float2(h[2 * j + 1]);
          const uint32_t lo = f32x2_to_e4m3x2(act_bf16(f0.x, silu) * scale, act_bf16(f0.y, silu) * scale);
          const uint32_t hi = f32x2_to_e4m3x2(act_bf16(f1.x, silu) * scale, act_bf16(f1.y, silu) * scale);
          w[j] = lo | (hi << 16);
        }
      }
      *reinterpret_cast<uint2*>(dst + 8 * v) = make_uint2(w[0], w[1]);
    }
  }
}

// weight [E, K, D]: one thread per (e, d) column, reduction over K.
template <typename T>
__global__ void __launch_bounds__(256)
colwise_quant_kernel(const T* __restrict__ w, int E, int K, int D, uint8_t* __restrict__ q,
                     float* __restrict__ scale_out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(E) * D) return;
  const int e = static_cast<int>(i / D);
  const int d = static_cast<int>(i - static_cast<long long>(e) * D);
  const T* src = w + static_cast<long long>(e) * K * D + d;
  float amax = 0.f;
  int has_nan = 0;
  for (int kk = 0; kk < K; ++kk) {
    const float v = fabsf(ld_act<T>(src + static_cast<long long>(kk) * D, false));
    has_nan |= isnan(v) ? 1 : 0;
    amax = fmaxf(amax, v);
  }
  if (has_nan) amax = NAN;
  const float scale = calc_scale(amax, sizeof(T) == 2);
  if (scale_out) scale_out[i] = scale;
  uint8_t* dst = q + static_cast<long long>(e) * K * D + d;
  for (int kk = 0; kk < K; ++kk) {
    const float a = ld_act<T>(src + static_cast<long long>(kk) * D, false) * scale;
    dst[static_cast<long long>(kk) * D] = static_cast<uint8_t>(f32x2_to_e4m3x2(a, 0.f) & 0xFF);
  }
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_rowwise_quant_fp8(const void* in, int in_dtype, int64_t rows, int cols, int64_t ldi,
                                      int apply_silu, int store_reciprocal, void* q, int64_t ldq, float* scale_out,
                                      void* stream) {
  FMOE_REQUIRE(rows >= 0 && cols >= 1, "rowwise_quant_fp8: rows=%lld cols=%d", (long long)rows, cols);
  FMOE_REQUIRE(in_dtype == FMOE_BF16 || in_dtype == FMOE_F32, "rowwise_quant_fp8: input must be bf16 or f32");
  FMOE_REQUIRE(rows == 0 || (in && q), "rowwise_quant_fp8: NULL pointer argument");
  if (rows == 0) return FMOE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* qq = static_cast<uint8_t*>(q);
  const bool wide = cols > 1024;
  const long long blocks = wide ? rows : (rows + 7) / 8;
  FMOE_REQUIRE(blocks < (1ll << 31), "rowwise_quant_fp8: too many rows");
  const unsigned g = static_cast<unsigned>(blocks);
  if (in_dtype == FMOE_BF16 && wide && cols % 8 == 0 && cols <= 256 * 8 * kRegVecsMax && (ldi * 2) % 16 == 0 &&
      (reinterpret_cast<uintptr_t>(in) & 15) == 0 && ldq % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(in);
    if (cols <= 256 * 8 * 2) {
      rowwise_quant_bf16_regs_kernel<2><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq, scale_out);
    } else {
      rowwise_quant_bf16_regs_kernel<kRegVecsMax><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq,
                                                                    scale_out);
    }
  } else if (in_dtype == FMOE_BF16) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(in);
    if (wide) rowwise_quant_kernel<__nv_bfloat16, 256><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq, scale_out);
    else rowwise_quant_kernel<__nv_bfloat16, 32><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq, scale_out);
  } else {
    const float* p = static_cast<const float*>(in);
    if (wide) rowwise_quant_kernel<float, 256><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq, scale_out);
    else rowwise_quant_kernel<float, 32><<<g, 256, 0, st>>>(p, ldi, rows, cols, apply_silu, store_reciprocal, qq, ldq, scale_out);
  }
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_bmm_weight_quant_fp8(const void* weight, int dtype, int E, int K, int D, void* q,
                                         float* scale_out, void* stream) {
  FMOE_REQUIRE(E >= 1 && K >= 1 && D >= 1, "bmm_weight_quant_fp8: E=%d K=%d D=%d", E, K, D);
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "bmm_weight_quant_fp8: weight must be bf16 or f32");
  FMOE_REQUIRE(weight && q, "bmm_weight_quant_fp8: NULL pointer argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long n = static_cast<long long>(E) * D;
  const unsigned g = static_cast<unsigned>((n + 255) / 256);
  if (dtype == FMOE_BF16)
    colwise_quant_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(weight), E, K, D,
                                                           static_cast<uint8_t*>(q), scale_out);
  else
    colwise_quant_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(weight), E, K, D,
                                                   static_cast<uint8_t*>(q), scale_out);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}
