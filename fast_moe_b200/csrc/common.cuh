// Shared declarations of the library's translation units: status codes, the error
// string, the device-side status word and the internal launchers behind the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fmoe_b200.h"

namespace fmoe {

// Records a message for fmoe_last_error() (thread-local) and returns `code`.
int fail(int code, const char* fmt, ...);
// Wraps a CUDA runtime return code.
int cuda_fail(cudaError_t e, const char* what);

#define FMOE_CUDA_OK(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::fmoe::cuda_fail(_e, #expr); \
  } while (0)

#define FMOE_REQUIRE(cond, ...)                                          \
  do {                                                                   \
    if (!(cond)) return ::fmoe::fail(FMOE_ERR_BAD_ARG, __VA_ARGS__);     \
  } while (0)

// Device-side status word of the current device (0 = clean). Kernels record the first
// problem they meet (a wait that ran out, an index out of range) and return; they never
// trap. Defined in api.cu; the address is resolved once per device.
int* device_status_ptr(int* err);
// Ordinal of the current device, checked against the per-device tables (kMaxDevices slots) the
// library keeps for cached symbol addresses and kernel attributes. FMOE_OK or an error status.
constexpr int kMaxDevices = 64;
int current_device_slot(int* dev_out);

// FMOE_PDL=1 (read once): kernels of the layer's chain are launched with programmatic stream
// serialization, so a kernel's set-up overlaps the tail of the kernel before it.
bool programmatic_launch_enabled();

static inline int dtype_size(int dt) {
  switch (dt) {
    case FMOE_F32: return 4;
    case FMOE_BF16: return 2;
    case FMOE_E4M3: return 1;
    default: return 0;
  }
}

// ------------------------------------------------------------------ grouped GEMM
// out[r, :] = epilogue( A[src(r), :] @ B[e(r)] ), r in [offsets[e], offsets[e+1]).
struct GemmDesc {
  int dtype;                 // operand type of A and B: FMOE_BF16, FMOE_F32 (tf32 math), FMOE_E4M3
  int E, N, K;
  const int64_t* offsets;    // device [E+1]
  int64_t total_rows;        // upper bound on offsets[E] (= rows of `out`)
  // A operand
  const void* a;
  int64_t a_rows;            // rows of the A source
  int64_t lda;               // elements
  const int64_t* index;      // device [total_rows] or null; source row = index[r] / index_div
  int index_div;
  // B operands, logical [E, K, N], element (e,k,n) at b + e*b_se + n*b_sn + k*b_sk. Either K is
  // contiguous (b_sk 0 or 1: the weights' storage layout) or N is (b_sn == 1, b_sk = row stride:
  // a plain [E, K, N] tensor, read as an MN-major tensor-core operand; bf16 only, N % 64 == 0)
  const void* b0;
  const void* b1;            // second operand of the gated (SwiGLU) form, else null
  int64_t b_se, b_sn;        // elements
  int64_t b_sk;              // elements; 0 or 1: K contiguous
  // b_ksplit > 0 (plain epilogues only): the reduction runs over two weights, A[:, :b_ksplit] @ b0[e]
  // + A[:, b_ksplit:] @ b1[e], b0 logical [E, b_ksplit, N] and b1 [E, K - b_ksplit, N] with the same
  // strides; b_ksplit a multiple of one K step (128 bytes)
  int b_ksplit;
  // bias [E, N] in the output type (nullable)
  const void* bias0;
  const void* bias1;
  int64_t bias_se;
  // FP8 row scales (the multipliers used at quantisation; the epilogue divides by them)
  const float* a_scale;      // per A-source row, or null
  const float* b0_scale;     // [E, N]
  const float* b1_scale;
  int64_t bscale_se;
  int epilogue;              // FMOE_EPI_*
  const int64_t* out_index;  // device [total_rows] or null: row r is stored at out[out_index[r]]
  // Stores into several output buffers (the expert-parallel return path): when out_peers is
  // non-null it is a DEVICE array of n_peers base addresses (buffers of peer_rows rows each, 16-byte
  // aligned, possibly in another GPU's memory, written with plain stores) and out_index[r] is
  // (peer << 40) | row.
  const int64_t* out_peers;
  int n_peers;
  int64_t peer_rows;
  // out = epilogue(...) * mul_in, elementwise: mul_in [total_rows, N] in the output type, row stride
  // ld_mul elements (the second factor of the two-input gated product); null = none
  const void* mul_in;
  int64_t ld_mul;
  // Reduction over the rows of each group (weight gradients): `a` is [a_rows, K] and b0 [N, K]
  // with K = the padded total row count of all groups, kseg [E+1] (device, elements, multiples
  // of one K step of 128 bytes, every group at least one step) the start of each group's range;
  // offsets must be the uniform [0, a_rows, 2 a_rows, ...] and the result is [E * a_rows, N].
  const int64_t* kseg;
  // total_rows may be a capacity rather than a row count; rows_hint (> 0) then tells the tile-shape
  // heuristic how many rows to expect
  int64_t rows_hint;
  // fused combine (all null/0 when unused): row r is multiplied by gate[gate_index[r]] and added
  // to out[gate_index[r] / gate_div]; out has combine_rows rows and must start at zero
  const void* gate;
  int gate_dtype;
  const int64_t* gate_index;
  int gate_div;
  int gate_round;   // round f32 gate weights to the output type before use
  int64_t combine_rows;
  void* out;
  int out_dtype;             // FMOE_BF16 or FMOE_F32
  int64_t ldo;               // elements
};
int launch_grouped_gemm(const GemmDesc& d, cudaStream_t stream);
int grouped_gemm_launch_count();
int launch_selftest_wait(unsigned long long limit_ns, cudaStream_t stream);

}  // namespace fmoe
