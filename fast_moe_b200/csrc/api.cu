// C ABI glue: error reporting, the device status word, and the operator-level entry points that
// map the reference's operator arguments onto the grouped GEMM / combine / SiLU launchers.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace fmoe {

long long g_misc_launches = 0;
int launch_silu(const void* in, int dtype, long long ldi, void* out, long long ldo, long long rows, int cols,
                cudaStream_t st);

namespace {
thread_local char g_err[512] = "";
// First problem a kernel met on this device since the last reset (FMOE_DEV_*).
__device__ int g_dev_status = 0;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(FMOE_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
}

bool programmatic_launch_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FMOE_PDL");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

int current_device_slot(int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    return fail(FMOE_ERR_UNSUPPORTED, "device ordinal %d is outside the %d per-device slots this library keeps", dev,
                kMaxDevices);
  }
  *dev_out = dev;
  return FMOE_OK;
}

int* device_status_ptr(int* err) {
  // One address per device; a process drives one device in practice, but look it up per device
  // to stay correct when it does not. Two host threads that make the first call together both
  // look the address up and store the same value: the slot is atomic, the lookup idempotent.
  static std::atomic<int*> ptrs[kMaxDevices];
  int dev = 0;
  if ((*err = current_device_slot(&dev)) != FMOE_OK) return nullptr;
  int* p = ptrs[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_dev_status);
    if (e != cudaSuccess || sym == nullptr) {
      *err = cuda_fail(e, "cudaGetSymbolAddress(status word)");
      return nullptr;
    }
    p = static_cast<int*>(sym);
    ptrs[dev].store(p, std::memory_order_release);
  }
  return p;
}

namespace {

// Fills the weight part of a GemmDesc; rejects layouts the tensor-core path cannot read.
int set_weight(GemmDesc& g, const char* op, int64_t w_se, int64_t w_sk, int64_t w_sn) {
  g.b_sk = 1;
  if (g.K > 1 && w_sk != 1) {
    // N contiguous instead (a plain [E, K, N] tensor): read in place as an MN-major operand where
    // the tensor cores allow it
    const bool mn_ok = w_sn == 1 && g.dtype == FMOE_BF16 && g.N % 64 == 0 && (w_sk * 2) % 16 == 0;
    if (!mn_ok) {
      return fail(FMOE_ERR_UNSUPPORTED,
                  "%s: weight must have K contiguous (stride_k == 1, got %lld), or - bf16 with N a multiple of 64 - N "
                  "contiguous with 16-byte aligned rows; pass the [E, N, K]-stored view",
                  op, (long long)w_sk);
    }
    g.b_sk = w_sk;
  }
  g.b_se = w_se;
  g.b_sn = w_sn;
  return FMOE_OK;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_version(void) { return 100; }

extern "C" const char* fmoe_last_error(void) { return g_err; }

extern "C" long long fmoe_kernel_launch_count(void) { return g_misc_launches + grouped_gemm_launch_count(); }

extern "C" int fmoe_device_status(int* status_out, int reset, void* stream) {
  FMOE_REQUIRE(status_out != nullptr, "device_status: status_out is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int err = 0;
  int* p = device_status_ptr(&err);
  if (!p) return err;
  FMOE_CUDA_OK(cudaMemcpyAsync(status_out, p, sizeof(int), cudaMemcpyDeviceToHost, st));
  if (reset) FMOE_CUDA_OK(cudaMemsetAsync(p, 0, sizeof(int), st));
  FMOE_CUDA_OK(cudaStreamSynchronize(st));
  return FMOE_OK;
}

extern "C" int fmoe_selftest_bounded_wait(int64_t limit_us, void* stream) {
  FMOE_REQUIRE(limit_us >= 1 && limit_us <= 1000000, "selftest_bounded_wait: limit must be 1 us .. 1 s");
  return launch_selftest_wait(static_cast<unsigned long long>(limit_us) * 1000ull, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_index_select_jagged_bmm(const int64_t* offsets, const int64_t* index, int index_div,
                                            int64_t total_rows, const void* jagged, int dtype, int64_t L,
                                            int64_t ldj, const void* weight, int64_t w_se, int64_t w_sk,
                                            int64_t w_sn, const void* bias, int64_t bias_se, int E, int K, int N,
                                            int epilogue, void* out, int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "index_select_jagged_bmm: dtype must be bf16 or f32");
  FMOE_REQUIRE(epilogue == FMOE_EPI_NONE || epilogue == FMOE_EPI_SILU, "index_select_jagged_bmm: bad epilogue %d",
               epilogue);
  FMOE_REQUIRE(index == nullptr || index_div >= 1, "index_select_jagged_bmm: index_div must be >= 1");
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = jagged; g.a_rows = L; g.lda = ldj;
  g.index = index; g.index_div = index_div;
  g.b0 = weight;
  int rc = set_weight(g, "index_select_jagged_bmm", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias_se = bias_se;
  g.epilogue = epilogue;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_index_select_jagged_bmm_mul(const int64_t* offsets, const int64_t* index, int index_div,
                                                int64_t total_rows, const void* jagged, int dtype, int64_t L,
                                                int64_t ldj, const void* weight, int64_t w_se, int64_t w_sk,
                                                int64_t w_sn, const void* bias, int64_t bias_se, int E, int K, int N,
                                                const void* multiplier, int64_t ld_mul, void* out, int out_dtype,
                                                int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "index_select_jagged_bmm_mul: dtype must be bf16 or f32");
  FMOE_REQUIRE(index == nullptr || index_div >= 1, "index_select_jagged_bmm_mul: index_div must be >= 1");
  FMOE_REQUIRE(total_rows == 0 || (multiplier != nullptr && ld_mul >= N), "index_select_jagged_bmm_mul: bad multiplier");
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = jagged; g.a_rows = L; g.lda = ldj;
  g.index = index; g.index_div = index_div;
  g.b0 = weight;
  int rc = set_weight(g, "index_select_jagged_bmm_mul", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias_se = bias_se;
  g.epilogue = FMOE_EPI_NONE;
  g.mul_in = multiplier; g.ld_mul = ld_mul;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_index_select_jagged_bmm_swiglu(const int64_t* offsets, const int64_t* index, int index_div,
                                                   int64_t total_rows, const void* jagged, int dtype, int64_t L,
                                                   int64_t ldj, const void* weight, const void* weight_p,
                                                   int64_t w_se, int64_t w_sk, int64_t w_sn, const void* bias,
                                                   const void* bias_p, int64_t bias_se, int E, int K, int N,
                                                   void* out, int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "index_select_jagged_bmm_swiglu: dtype must be bf16 or f32");
  FMOE_REQUIRE(index == nullptr || index_div >= 1, "index_select_jagged_bmm_swiglu: index_div must be >= 1");
  FMOE_REQUIRE(weight_p != nullptr, "index_select_jagged_bmm_swiglu: weight_p is NULL");
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = jagged; g.a_rows = L; g.lda = ldj;
  g.index = index; g.index_div = index_div;
  g.b0 = weight; g.b1 = weight_p;
  int rc = set_weight(g, "index_select_jagged_bmm_swiglu", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias1 = bias_p; g.bias_se = bias_se;
  g.epilogue = FMOE_EPI_SWIGLU;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_index_select_jagged_bmm_fp8(const int64_t* offsets, const int64_t* index, int index_div,
                                                int64_t total_rows, const void* jagged_q, const float* jagged_scale,
                                                int64_t L, int64_t ldj, const void* weight_q,
                                                const float* weight_scale, const void* weight_p_q,
                                                const float* weight_p_scale, int64_t w_se, int64_t w_sk,
                                                int64_t w_sn, int64_t ws_se, const void* bias, const void* bias_p,
                                                int64_t bias_se, int E, int K, int N, int epilogue, void* out,
                                                int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(index == nullptr || index_div >= 1, "index_select_jagged_bmm_fp8: index_div must be >= 1");
  FMOE_REQUIRE(jagged_scale && weight_scale, "index_select_jagged_bmm_fp8: scales are required");
  FMOE_REQUIRE((weight_p_q == nullptr) == (weight_p_scale == nullptr),
               "index_select_jagged_bmm_fp8: weight_p_q and weight_p_scale go together");
  FMOE_REQUIRE((epilogue == FMOE_EPI_SWIGLU) == (weight_p_q != nullptr),
               "index_select_jagged_bmm_fp8: SwiGLU epilogue if and only if weight_p_q is given");
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = FMOE_E4M3;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = jagged_q; g.a_rows = L; g.lda = ldj;
  g.index = index; g.index_div = index_div;
  g.b0 = weight_q; g.b1 = weight_p_q;
  int rc = set_weight(g, "index_select_jagged_bmm_fp8", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias1 = bias_p; g.bias_se = bias_se;
  g.a_scale = jagged_scale; g.b0_scale = weight_scale; g.b1_scale = weight_p_scale; g.bscale_se = ws_se;
  g.epilogue = epilogue;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_silu_jagged_bmm(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype,
                                    int64_t ldj, const float* jagged_scale, const void* weight,
                                    const float* weight_scale, int64_t w_se, int64_t w_sk, int64_t w_sn,
                                    int64_t ws_se, const void* bias, int64_t bias_se, int E, int K, int N,
                                    int has_silu, void* act_scratch, const int64_t* jagged_index,
                                    const int64_t* out_row_index, void* out, int out_dtype, int64_t ldo,
                                    void* stream) {
  const bool fp8 = dtype == FMOE_E4M3;
  FMOE_REQUIRE(fp8 || dtype == FMOE_BF16 || dtype == FMOE_F32, "silu_jagged_bmm: bad dtype %d", dtype);
  FMOE_REQUIRE(!fp8 || (jagged_scale && weight_scale), "silu_jagged_bmm: FP8 operands need their scales");
  FMOE_REQUIRE(!(fp8 && has_silu), "silu_jagged_bmm: has_silu is not available on FP8 input (quantise silu(x) instead)");
  FMOE_REQUIRE(!has_silu || act_scratch != nullptr || total_rows == 0, "silu_jagged_bmm: has_silu needs act_scratch");
  FMOE_REQUIRE(!(has_silu && jagged_index), "silu_jagged_bmm: has_silu and jagged_index cannot be combined");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const void* a = jagged;
  int64_t lda = ldj;
  if (has_silu && total_rows > 0) {
    int rc = launch_silu(jagged, dtype, ldj, act_scratch, K, total_rows, K, st);
    if (rc != FMOE_OK) return rc;
    a = act_scratch;
    lda = K;
  }
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = a; g.a_rows = total_rows; g.lda = lda;
  g.index = jagged_index; g.index_div = 1;
  g.out_index = out_row_index;
  g.b0 = weight;
  int rc = set_weight(g, "silu_jagged_bmm", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias_se = bias_se;
  g.a_scale = jagged_scale; g.b0_scale = weight_scale; g.bscale_se = ws_se;
  g.epilogue = FMOE_EPI_NONE;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, st);
}

extern "C" int fmoe_jagged_bmm_two_weights(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype,
                                           int64_t ldj, const void* weight0, const void* weight1, int k_split,
                                           int64_t w_se, int64_t w_sk, int64_t w_sn, int E, int K, int N, void* out,
                                           int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "jagged_bmm_two_weights: dtype must be bf16 or f32");
  FMOE_REQUIRE(weight0 && weight1 && k_split > 0 && k_split < K, "jagged_bmm_two_weights: need two weights and 0 < k_split < K");
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = jagged; g.a_rows = total_rows; g.lda = ldj;
  g.index_div = 1;
  g.b0 = weight0;
  g.b1 = weight1;
  g.b_ksplit = k_split;
  int rc = set_weight(g, "jagged_bmm_two_weights", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.epilogue = FMOE_EPI_NONE;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_silu_jagged_bmm_combine(const int64_t* offsets, int64_t total_rows, const void* jagged,
                                            int dtype, int64_t ldj, const void* weight, int64_t w_se, int64_t w_sk,
                                            int64_t w_sn, const void* bias, int64_t bias_se,
                                            const int64_t* reverse_index, const void* gating_scores, int g_dtype,
                                            const int64_t* gates_index, int64_t L, int k, int E, int K, int N,
                                            int has_silu, void* act_scratch, void* bmm_scratch, void* out,
                                            int out_dtype, int64_t ldo, void* stream) {
  FMOE_REQUIRE(L == 0 || bmm_scratch != nullptr, "silu_jagged_bmm_combine: bmm_scratch is NULL");
  FMOE_REQUIRE(total_rows == L * k, "silu_jagged_bmm_combine: rows %lld != L*k = %lld", (long long)total_rows,
               (long long)(L * k));
  // the GEMM result has the activation type, as F.linear returns it
  const int bmm_dtype = dtype;
  int rc = fmoe_silu_jagged_bmm(offsets, total_rows, jagged, dtype, ldj, nullptr, weight, nullptr, w_se, w_sk, w_sn,
                                0, bias, bias_se, E, K, N, has_silu, act_scratch, nullptr, nullptr, bmm_scratch, bmm_dtype, N,
                                stream);
  if (rc != FMOE_OK) return rc;
  return fmoe_mul_merge_k_add(reverse_index, bmm_scratch, bmm_dtype, N, gating_scores, g_dtype, gates_index, L, k, N,
                              out, out_dtype, ldo, stream);
}

extern "C" int fmoe_silu_jagged_bmm_combine_fused(const int64_t* offsets, int64_t total_rows, const void* jagged,
                                                  int dtype, int64_t ldj, const float* jagged_scale,
                                                  const void* weight, const float* weight_scale, int64_t w_se,
                                                  int64_t w_sk, int64_t w_sn, int64_t ws_se, const void* bias,
                                                  int64_t bias_se, const void* gating_scores, int g_dtype,
                                                  const int64_t* gates_index, int64_t L, int k, int E, int K, int N,
                                                  int has_silu, void* act_scratch, void* out, int out_dtype,
                                                  int64_t ldo, int flags, void* stream) {
  const bool fp8 = dtype == FMOE_E4M3;
  FMOE_REQUIRE(fp8 || dtype == FMOE_BF16 || dtype == FMOE_F32, "silu_jagged_bmm_combine_fused: bad dtype %d", dtype);
  FMOE_REQUIRE((flags & ~(FMOE_COMBINE_ACCUMULATE | FMOE_COMBINE_ROUND_GATE)) == 0,
               "silu_jagged_bmm_combine_fused: unknown flags 0x%x", flags);
  FMOE_REQUIRE(!fp8 || (jagged_scale && weight_scale), "silu_jagged_bmm_combine_fused: FP8 operands need their scales");
  FMOE_REQUIRE(!(fp8 && has_silu), "silu_jagged_bmm_combine_fused: has_silu is not available on FP8 input");
  FMOE_REQUIRE(!has_silu || act_scratch != nullptr || total_rows == 0,
               "silu_jagged_bmm_combine_fused: has_silu needs act_scratch");
  FMOE_REQUIRE(L == 0 || (gating_scores && gates_index),
               "silu_jagged_bmm_combine_fused: gating_scores and gates_index are required");
  FMOE_REQUIRE(g_dtype == FMOE_BF16 || g_dtype == FMOE_F32, "silu_jagged_bmm_combine_fused: gate weights must be bf16 or f32");
  FMOE_REQUIRE(total_rows == L * k, "silu_jagged_bmm_combine_fused: rows %lld != L*k = %lld", (long long)total_rows,
               (long long)(L * k));
  FMOE_REQUIRE((L == 0 || out != nullptr) && ldo >= N, "silu_jagged_bmm_combine_fused: bad output");
  if (L == 0) return FMOE_OK;   // an empty batch is valid input (its tensors have NULL data pointers)
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int os = dtype_size(out_dtype);
  if (L > 0 && !(flags & FMOE_COMBINE_ACCUMULATE)) {
    FMOE_CUDA_OK(cudaMemset2DAsync(out, static_cast<size_t>(ldo) * os, 0, static_cast<size_t>(N) * os, L, st));
  }
  const void* a = jagged;
  int64_t lda = ldj;
  if (has_silu && total_rows > 0) {
    int rc = launch_silu(jagged, dtype, ldj, act_scratch, K, total_rows, K, st);
    if (rc != FMOE_OK) return rc;
    a = act_scratch;
    lda = K;
  }
  GemmDesc g;
  memset(&g, 0, sizeof(g));
  g.dtype = dtype;
  g.E = E; g.N = N; g.K = K;
  g.offsets = offsets;
  g.total_rows = total_rows;
  g.a = a; g.a_rows = total_rows; g.lda = lda;
  g.b0 = weight;
  int rc = set_weight(g, "silu_jagged_bmm_combine_fused", w_se, w_sk, w_sn);
  if (rc != FMOE_OK) return rc;
  g.bias0 = bias; g.bias_se = bias_se;
  g.a_scale = jagged_scale; g.b0_scale = weight_scale; g.bscale_se = ws_se;
  g.epilogue = FMOE_EPI_NONE;
  g.gate = gating_scores; g.gate_dtype = g_dtype; g.gate_index = gates_index; g.gate_div = k; g.combine_rows = L;
  g.gate_round = (flags & FMOE_COMBINE_ROUND_GATE) ? 1 : 0;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, st);
}
