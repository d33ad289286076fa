// Grouped ("jagged") GEMM for sm_100a: every expert e multiplies its own row segment
// [offsets[e], offsets[e+1]) of the activations by its own weight matrix.
//
//   out[r, n] = epilogue( sum_k A[src(r), k] * B[e(r)][k, n] )
//
// Replaces the reference's per-expert loops
//   pytorch_index_select_jagged_bmm          kernels/pytorch/moe.py:40-84
//   pytorch_index_select_jagged_bmm_swiglu   kernels/pytorch/moe.py:87-146
//   pytorch_silu_jagged_bmm                  kernels/pytorch/moe.py:255-275
//   pytorch_index_select_jagged_bmm_fp8      kernels/pytorch/moe_fp8.py:98-139
// and the Triton kernels that sit behind the same operators
// (kernels/triton/triton_moe.py:184-282, :2526-2671, :3167-3347; triton_moe_fp8.py:770-884).
//
// Shape of the kernel: persistent CTAs, one per SM, either alone (128-row tiles) or as CTA pairs
// (clusters of two, tcgen05 cta_group::2, 256-row tiles: each CTA stages its own 128 activation
// rows and its half of the 256 weight rows, which halves the shared-memory traffic per FLOP).
//   warp 0     one thread issues the TMA loads (weights as 3-D tiles of [E, N, K]; activations
//              as 2-D tiles when their rows are contiguous) into a ring of shared-memory stages.
//   warp 1     one thread (of the pair's leader CTA) issues tcgen05.mma, M = 128 or 256, N = 256,
//              fp32 accumulators in tensor memory, double buffered so that the epilogue of tile
//              i overlaps the MMAs of tile i+1.
//   warps 2-9  epilogue: tcgen05.ld the accumulator, rowwise FP8 descale / bias / SiLU / SwiGLU,
//              convert, transpose through shared memory and store whole lines; only rows and
//              columns that exist are written; rows may be scattered (out_index).
//   warps 10-13 (kernels that gather): the rows of a tile are scattered over the token matrix, so
//              these warps fetch them with 16-byte cp.async copies straight into the 128-byte-
//              swizzled K-major layout the tensor core reads (TMA's 4-row gather mode was
//              measured at half the throughput of this for 128-byte row pieces).
//   warp 14    (pairs that gather) forwards "rows have landed" to the leader CTA's barrier.
// Tiles are enumerated on the device from `offsets` (variable rows per expert, empty experts
// contribute nothing), so no host synchronisation is needed and no CTA is launched for work that
// does not exist. Every wait is bounded; a wait that gives up records a status code and the
// kernel drains instead of hanging.
#include <stdarg.h>
#include <stdlib.h>
#include <stdio.h>

#include <atomic>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

// The file compiles either as one object (FMOE_GEMM_PART undefined) or in four parts that build
// in parallel: part 0 holds the host code, parts 1 / 2 / 3 the kernel instantiations for 2-byte,
// 4-byte and 1-byte operands.
#ifndef FMOE_GEMM_PART
#define FMOE_GEMM_PART -1
#endif
#define FMOE_GEMM_HOST (FMOE_GEMM_PART <= 0)
#define FMOE_GEMM_KERNELS (FMOE_GEMM_PART != 0)

namespace fmoe {
namespace gemm_detail {

constexpr int kBM = 128;            // rows per CTA and tile (= TMEM lanes)
constexpr int kMmaN = 256;          // accumulator columns per tile
constexpr int kRowBytes = 128;      // bytes of K per stage row: one swizzle atom
constexpr int kEpilogueWarps = 8;
constexpr int kGatherWarps = 4;
constexpr int kGatherThreads = 32 * kGatherWarps;
constexpr int kBaseThreads = 64 + 32 * kEpilogueWarps;           // TMA warp, MMA warp, epilogue warps
constexpr int kGatherKernelThreads = kBaseThreads + kGatherThreads + 32;   // + gather warps + relay warp
constexpr int kMaxExperts = 1024;
constexpr int kABytes = kBM * kRowBytes;

struct GemmParams {
  const long long* offsets;
  const long long* index;
  const long long* out_index;
  const long long* out_peers;   // device array of output base addresses, or null (see GemmDesc)
  int n_peers;
  int index_div;
  int E, N, K;
  int num_kb;
  int n_tiles;
  const void* a;
  long long lda;
  long long a_rows;
  long long out_rows;
  void* out;
  long long ldo;
  const void* bias0;
  const void* bias1;
  long long bias_se;
  const float* a_scale;
  const float* b0_scale;
  const float* b1_scale;
  long long bscale_se;
  int epilogue;
  // fused combine: row r is scaled by gate[gate_index[r]] and ADDED to out[gate_index[r] / gate_div]
  const void* gate;
  int gate_is_f32;
  int gate_round;
  const long long* gate_index;
  int gate_div;
  int vec_ok;        // output rows are 16-byte aligned: vector stores allowed
  // Reduction over an expert's ROWS instead of over a fixed K (the weight-gradient product
  // dW[e] = A_e^T B_e): both operands are stored transposed, [features, padded rows], and kseg[e]
  // (elements, multiples of one K step) is where expert e's padded row range starts. Every
  // expert then owns the same number of output rows; its tiles differ in the length of the K loop.
  const long long* kseg;
  // elementwise multiplier applied last: out[r, n] = (...)[r, n] * mul_in[r * ld_mul + n] (output type)
  const void* mul_in;
  long long ld_mul;
  int b_ksplit;      // > 0: K steps from here on read the second weight (tmB1) at k - b_ksplit
  int b_mn;          // B tiles are MN-major (N contiguous in memory): 4-D tensor map, MN-major descriptors
  int mul_vec;       // rows of mul_in are 16-byte aligned: 16-byte loads in the store phase
  int* status;
};

template <int CTAS>
struct SmemPlan {
  static constexpr int kBBytes = (kMmaN / CTAS) * kRowBytes;     // weight rows this CTA stages
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (CTAS == 1) ? 4 : 6;
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kStagingBytes = kEpilogueWarps * 2048;    // 32 rows x 64 bytes per epilogue warp
  static constexpr int kBarBytes = 256;
  static constexpr int kPmBytes = 3 * ((kMaxExperts + 1) * 4 + 12);   // tile prefix + row offsets + reduction offsets
  static constexpr int kTotal = 1024 + kTileBytes + kStagingBytes + kBarBytes + kPmBytes;
};

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <typename OutT>
__device__ __forceinline__ float load_as_float(const void* p, long long i) {
  if constexpr (sizeof(OutT) == 4) {
    return reinterpret_cast<const float*>(p)[i];
  } else {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
}

// Stores v[0..31] to dst[0..31] (columns col0..col0+31 of one output row), masking columns
// that lie beyond N.
template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* dst, const float (&v)[32], int ncols, bool vec_ok) {
  if constexpr (sizeof(OutT) == 2) {
    if (vec_ok && ncols == 32) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols) dst[i] = __float2bfloat16_rn(v[i]);
    }
  } else {
    if (vec_ok && ncols == 32) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(dst + 4 * j) =
            make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols) dst[i] = v[i];
    }
  }
}


// Writes one 32-column chunk (v) of 32 rows - one row per lane - to global memory with full-line
// accesses: the chunk is first laid out in the warp's 2 KB staging area (64-byte rows, 16-byte
// pieces XOR-swizzled so that neither phase has bank conflicts), then every group of 4 lanes
// writes one row's 64 contiguous bytes, 8 rows per instruction. Rows that do not exist (tail of
// a segment) are skipped; rows may go anywhere (st_row), which also serves the scattered store.
// For 4-byte outputs the chunk goes out in two halves of 16 columns.
// With `accumulate` the 16-byte pieces are added to memory (one vector red.global.add per
// piece) instead of stored: the fused combine, where several expert rows land on
// one token row.
// `mul_row` (optional, per stored row): a second factor of the same shape as the output, read here
// in the same coalesced pattern (16 bytes per lane, a row's 64 bytes from 4 neighbouring lanes)
// and multiplied into the staged values, which are already rounded to the output type.
template <typename OutT>
__device__ __forceinline__ void stage_and_store(uint32_t stage_w, int lane, const float (&v)[32],
                                                OutT* const (&st_row)[4], const bool (&st_ok)[4], int col0,
                                                bool accumulate, const OutT* const (&mul_row)[4], bool has_mul) {
  constexpr int kHalves = sizeof(OutT) == 2 ? 1 : 2;
  constexpr int kPieceElemsM = 16 / sizeof(OutT);
  const uint32_t my_row = stage_w + lane * 64;
  const int wsw = (lane >> 1) & 3;
#pragma unroll
  for (int h = 0; h < kHalves; ++h) {
    uint4 mv[4];
    if (has_mul) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        mv[i] = make_uint4(0, 0, 0, 0);
        if (st_ok[i])
          mv[i] = *reinterpret_cast<const uint4*>(mul_row[i] + col0 + (kHalves == 2 ? 16 * h : 0) + (lane & 3) * kPieceElemsM);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w0, w1, w2, w3;
      if constexpr (sizeof(OutT) == 2) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * c + 0], v[8 * c + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * c + 2], v[8 * c + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * c + 4], v[8 * c + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * c + 6], v[8 * c + 7]);
        w0 = *reinterpret_cast<uint32_t*>(&h0);
        w1 = *reinterpret_cast<uint32_t*>(&h1);
        w2 = *reinterpret_cast<uint32_t*>(&h2);
        w3 = *reinterpret_cast<uint32_t*>(&h3);
      } else {
        w0 = __float_as_uint(v[16 * h + 4 * c + 0]);
        w1 = __float_as_uint(v[16 * h + 4 * c + 1]);
        w2 = __float_as_uint(v[16 * h + 4 * c + 2]);
        w3 = __float_as_uint(v[16 * h + 4 * c + 3]);
      }
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + ((c ^ wsw) << 4)), "r"(w0), "r"(w1),
                   "r"(w2), "r"(w3)
                   : "memory");
    }
    __syncwarp();
    const int piece = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = (lane >> 2) + 8 * i;
      uint32_t w0, w1, w2, w3;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                   : "r"(stage_w + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4))
                   : "memory");
      if (st_ok[i]) {
        constexpr int kPieceElems = 16 / sizeof(OutT);
        OutT* dst = st_row[i] + col0 + (kHalves == 2 ? 16 * h : 0) + piece * kPieceElems;
        if (has_mul) {
          if constexpr (sizeof(OutT) == 2) {
            const uint32_t m4[4] = {mv[i].x, mv[i].y, mv[i].z, mv[i].w};
            uint32_t* w4[4] = {&w0, &w1, &w2, &w3};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(w4[u]),
                                                  *reinterpret_cast<const __nv_bfloat162*>(&m4[u]));
              *w4[u] = *reinterpret_cast<const uint32_t*>(&prod);
            }
          } else {
            w0 = __float_as_uint(__uint_as_float(w0) * __uint_as_float(mv[i].x));
            w1 = __float_as_uint(__uint_as_float(w1) * __uint_as_float(mv[i].y));
            w2 = __float_as_uint(__uint_as_float(w2) * __uint_as_float(mv[i].z));
            w3 = __float_as_uint(__uint_as_float(w3) * __uint_as_float(mv[i].w));
          }
        }
        if (!accumulate) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(w0, w1, w2, w3);
        } else if constexpr (sizeof(OutT) == 2) {
          // one 16-byte reduction: eight independent bf16 additions
          asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(w0), "r"(w1), "r"(w2),
                       "r"(w3)
                       : "memory");
        } else {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(w0)),
                       "f"(__uint_as_float(w1)), "f"(__uint_as_float(w2)), "f"(__uint_as_float(w3))
                       : "memory");
        }
      }
    }
    __syncwarp();
  }
}

// Walks the tile list. Tiles are ordered expert-major, then column block, then row block, so
// CTAs that run at the same time share the weight tile of one expert through L2.
struct TileWalker {
  const int* pm;   // prefix of row-tile counts per expert, pm[E] = total row tiles
  int n_tiles;
  int E;
  int e;
  __device__ TileWalker(const int* pm_, int n_tiles_, int E_) : pm(pm_), n_tiles(n_tiles_), E(E_), e(0) {}
  // Decodes tile t (monotonically increasing across calls).
  __device__ __forceinline__ void decode(int t, int& expert, int& mb, int& nb) {
    while (e < E - 1 && t >= pm[e + 1] * n_tiles) ++e;
    const int local = t - pm[e] * n_tiles;
    const int mt = pm[e + 1] - pm[e];
    nb = local / mt;
    mb = local - nb * mt;
    expert = e;
  }
};

template <int ESIZE, int CTAS, bool DUAL, bool GATHER, bool COMBINE, typename OutT>
__global__ void __launch_bounds__(GATHER ? kGatherKernelThreads : kBaseThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, const GemmParams p) {
  using Plan = SmemPlan<CTAS>;
  constexpr bool kPair = (CTAS == 2);
  constexpr int kStages = Plan::kStages;
  constexpr int kTileRows = kBM * CTAS;                  // rows per tile (both CTAs of a pair)
  constexpr int kTileN = DUAL ? kMmaN / 2 : kMmaN;       // output columns per tile
  constexpr int kKElems = kRowBytes / ESIZE;             // K elements per stage
  constexpr int kUmmaKBytes = 32;                        // bytes of K per tcgen05.mma
  constexpr int kKind = ESIZE == 2 ? ptx::KIND_F16 : (ESIZE == 4 ? ptx::KIND_TF32 : ptx::KIND_F8);
  constexpr uint32_t kFmt = ESIZE == 2 ? 1u : (ESIZE == 4 ? 2u : 0u);
  constexpr uint32_t kIdesc = ptx::umma_idesc(kFmt, kTileRows, kMmaN);
  constexpr uint32_t kTmemCols = 2 * kMmaN;              // two accumulator buffers
  // Bytes the TMA unit reports per stage to the (leader's) full barrier; gathered activation rows
  // arrive through cp.async and are tracked by thread arrivals instead.
  constexpr uint32_t kStageTx = CTAS * ((GATHER ? 0 : kABytes) + Plan::kBBytes);
  // Arrivals on a full barrier: the leader's TMA thread, plus (gather) either every gather thread
  // of a lone CTA or one relay thread per CTA of a pair.
  constexpr uint32_t kFullArrivals = !GATHER ? 1 : (kPair ? 1 + CTAS : 1 + kGatherThreads);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  const uint32_t staging_addr = tiles_addr + Plan::kTileBytes;
  const uint32_t bar_addr = staging_addr + Plan::kStagingBytes;
  uint8_t* bar_ptr = tiles_ptr + Plan::kTileBytes + Plan::kStagingBytes;
  // barrier map (8 bytes each): full[S], empty[S], afull[S], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_addr + 8u * s; };
  auto empty_bar = [&](int s) { return bar_addr + 8u * (kStages + s); };
  auto afull_bar = [&](int s) { return bar_addr + 8u * (2 * kStages + s); };
  auto tfull_bar = [&](int a) { return bar_addr + 8u * (3 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_addr + 8u * (3 * kStages + 2 + a); };
  static_assert(8 * (3 * kStages + 4) <= 192, "barrier area too small");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 200);
  int* pm = reinterpret_cast<int*>(bar_ptr + Plan::kBarBytes);
  int* soff = pm + kMaxExperts + 2;   // offsets[] as 32-bit rows, read by every role at tile changes
  int* skb = soff + kMaxExperts + 2;  // kseg[] (reduction-over-rows mode): start of each expert's K range
  const bool kseg_mode = p.kseg != nullptr;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? ptx::cluster_ctarank() : 0u;    // 0 = leader of the pair
  const int unit = blockIdx.x / CTAS;                            // persistent work unit (CTA or pair)
  const int num_units = gridDim.x / CTAS;

  // ---- set-up: barriers, tile prefix, tensor memory
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), kFullArrivals);
      ptx::mbar_init(empty_bar(s), 1);
      ptx::mbar_init(afull_bar(s), kGatherThreads);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), kEpilogueWarps * CTAS);
    }
    *abort_flag = 0;
    pm[0] = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB0);
    if (DUAL) ptx::prefetch_tmap(&tmB1);
  }
  // Everything above touched only this CTA's shared memory. From here on the kernel reads what
  // earlier kernels of the stream wrote (offsets, operands): with a programmatic dependent launch
  // this is where it waits for them; the next kernel in the stream may be scheduled from now on.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const long long o0 = p.offsets[e], o1 = p.offsets[e + 1];
    long long len = o1 - o0;
    if (len < 0) len = 0;
    pm[e + 1] = static_cast<int>((len + kTileRows - 1) / kTileRows);
    soff[e] = static_cast<int>(o0);
    if (e == p.E - 1) soff[p.E] = static_cast<int>(o1 < o0 ? o0 : o1);
    if (kseg_mode) {
      skb[e] = static_cast<int>(p.kseg[e]);
      if (e == p.E - 1) skb[p.E] = static_cast<int>(p.kseg[p.E]);
    }
  }
  __syncthreads();
  if (warp == 0) {
    // inclusive scan of pm[1..E], 32 entries at a time
    int carry = 0;
    for (int base = 1; base <= p.E; base += 32) {
      const int i = base + lane;
      int v = (i <= p.E) ? pm[i] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      v += carry;
      if (i <= p.E) pm[i] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTAS>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    ptx::tmem_relinquish<CTAS>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kPair) ptx::cluster_sync_all();   // the peer's barriers exist before anything signals them
  ptx::tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = pm[p.E] * p.n_tiles;
  const int num_kb = p.num_kb;

  if (warp == 0) {
    // =========================================================== TMA producer (one thread)
    // Two versions of the loop, chosen once: the common one (K-contiguous weights, one weight per
    // reduction) carries none of the other modes' address arithmetic.
    if (lane == 0) {
      auto produce = [&](auto alt_tag) {
        constexpr bool ALT = decltype(alt_tag)::value;    // N-contiguous weights and / or a second weight along K
        TileWalker walk(pm, p.n_tiles, p.E);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = unit; t < total_tiles && ok; t += num_units) {
          int e, mb, nb;
          walk.decode(t, e, mb, nb);
          // reduction-over-rows mode: A rows are the expert's output rows (the same for every
          // expert), the K range is the expert's, and B is a single matrix
          const int row0 = (kseg_mode ? 0 : soff[e]) + mb * kTileRows + static_cast<int>(rank) * kBM;
          const int n0 = nb * kTileN;
          const int k_begin = kseg_mode ? skb[e] : 0;
          const int nkb = kseg_mode ? (skb[e + 1] - skb[e]) / kKElems : num_kb;
          if (kseg_mode) e = 0;
          for (int kb = 0; kb < nkb; ++kb) {
            if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                        FMOE_DEV_WAIT_PRODUCER)) {
              ok = false;
              break;
            }
            const uint32_t a_dst = tiles_addr + stage * Plan::kStageBytes;
            const uint32_t b_dst = a_dst + kABytes;
            const int k0 = k_begin + kb * kKElems;
            if constexpr (!ALT) {
              if constexpr (!kPair) {
                const uint32_t bar = full_bar(stage);
                ptx::mbar_arrive_expect_tx(bar, kStageTx);
                if constexpr (!GATHER) ptx::tma_load_2d(a_dst, &tmA, bar, k0, row0);
                ptx::tma_load_3d(b_dst, &tmB0, bar, k0, n0, e);
                if constexpr (DUAL) ptx::tma_load_3d(b_dst + kTileN * kRowBytes, &tmB1, bar, k0, n0, e);
              } else {
                // Both CTAs report their bytes to the leader's barrier; only the leader arms it.
                const uint32_t bar = ptx::mapa(full_bar(stage), 0);
                if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), kStageTx);
                if constexpr (!GATHER) ptx::tma_load_2d_pair(a_dst, &tmA, bar, k0, row0);
                if constexpr (DUAL) {
                  // leader stages the gate weights, its peer the up weights: 128 rows each
                  ptx::tma_load_3d_pair(b_dst, rank == 0 ? &tmB0 : &tmB1, bar, k0, n0, e);
                } else {
                  ptx::tma_load_3d_pair(b_dst, &tmB0, bar, k0, n0 + static_cast<int>(rank) * (kMmaN / 2), e);
                }
              }
            } else {
              // two weights along the reduction (plain tiles only): the second one takes over at b_ksplit
              const bool second = !DUAL && p.b_ksplit > 0 && k0 >= p.b_ksplit;
              const CUtensorMap* tb = second ? &tmB1 : &tmB0;
              const int kw = second ? k0 - p.b_ksplit : k0;
              if constexpr (!kPair) {
                const uint32_t bar = full_bar(stage);
                ptx::mbar_arrive_expect_tx(bar, kStageTx);
                if constexpr (!GATHER) ptx::tma_load_2d(a_dst, &tmA, bar, k0, row0);
                if (p.b_mn) {
                  // N contiguous in memory: box = 64 columns x one K step x (atoms of 64 columns)
                  ptx::tma_load_4d(b_dst, tb, bar, 0, kw, n0 >> 6, e);
                  if constexpr (DUAL) ptx::tma_load_4d(b_dst + kTileN * kRowBytes, &tmB1, bar, 0, k0, n0 >> 6, e);
                } else {
                  ptx::tma_load_3d(b_dst, tb, bar, kw, n0, e);
                  if constexpr (DUAL) ptx::tma_load_3d(b_dst + kTileN * kRowBytes, &tmB1, bar, k0, n0, e);
                }
              } else {
                const uint32_t bar = ptx::mapa(full_bar(stage), 0);
                if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), kStageTx);
                if constexpr (!GATHER) ptx::tma_load_2d_pair(a_dst, &tmA, bar, k0, row0);
                if constexpr (DUAL) {
                  if (p.b_mn) {
                    ptx::tma_load_4d_pair(b_dst, rank == 0 ? &tmB0 : &tmB1, bar, 0, k0, n0 >> 6, e);
                  } else {
                    ptx::tma_load_3d_pair(b_dst, rank == 0 ? &tmB0 : &tmB1, bar, k0, n0, e);
                  }
                } else {
                  const int nh = n0 + static_cast<int>(rank) * (kMmaN / 2);
                  if (p.b_mn) {
                    ptx::tma_load_4d_pair(b_dst, tb, bar, 0, kw, nh >> 6, e);
                  } else {
                    ptx::tma_load_3d_pair(b_dst, tb, bar, kw, nh, e);
                  }
                }
              }
            }
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      };
      if (p.b_mn != 0 || p.b_ksplit > 0) {
        produce(std::true_type{});
      } else {
        produce(std::false_type{});
      }
    }
  } else if (warp == 1) {
    // =========================================================== MMA issuer (one thread, leader CTA)
    if (lane == 0 && rank == 0) {
     auto issue = [&](auto bmn_tag) {
      constexpr bool BMN = decltype(bmn_tag)::value;     // B tiles are MN-major
      TileWalker walk(pm, p.n_tiles, p.E);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += num_units, ++it) {
        int nkb = num_kb;
        if (kseg_mode) {
          int e, mb, nb;
          walk.decode(t, e, mb, nb);
          nkb = (skb[e + 1] - skb[e]) / kKElems;
        }
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, FMOE_DEV_WAIT_MMA)) {
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kMmaN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.status, FMOE_DEV_WAIT_MMA)) {
            ok = false;
            break;
          }
          if constexpr (GATHER) ptx::fence_proxy_async_smem();   // rows written by cp.async (generic proxy)
          ptx::tc_fence_after();
          const uint32_t a_src = tiles_addr + stage * Plan::kStageBytes;
          const uint64_t da = ptx::umma_desc_k_sw128(a_src);
          if constexpr (!BMN) {
            const uint64_t db = ptx::umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
            for (int k = 0; k < kRowBytes / kUmmaKBytes; ++k) {
              ptx::umma_ss<kKind, CTAS>(d_tmem, da + 2u * k, db + 2u * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
            }
          } else {
            // MN-major B: a K step of one MMA is kUmmaKBytes / ESIZE rows of 128 bytes
            constexpr uint32_t kAtomBytes = (kRowBytes / ESIZE) * kRowBytes;          // 64 K rows x 128 B (bf16)
            constexpr uint32_t kStep = (kUmmaKBytes / ESIZE) * kRowBytes;             // bytes per MMA along K
            const uint64_t db = ptx::umma_desc_mn_sw128(a_src + kABytes, kAtomBytes);
#pragma unroll
            for (int k = 0; k < kRowBytes / kUmmaKBytes; ++k) {
              ptx::umma_ss<kKind, CTAS>(d_tmem, da + 2u * k, db + static_cast<uint64_t>((kStep >> 4) * k),
                                        kIdesc | ptx::kUmmaIdescBMnMajor, (kb | k) != 0 ? 1u : 0u);
            }
          }
          ptx::umma_commit<CTAS>(empty_bar(stage));      // stage reusable once these MMAs have read it
          if (kb == nkb - 1) ptx::umma_commit<CTAS>(tfull_bar(acc));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
     };
     if (p.b_mn != 0) {
       issue(std::true_type{});
     } else {
       issue(std::false_type{});
     }
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // =========================================================== epilogue (8 warps)
    // A warp may only read the TMEM lanes of its quarter (warp id mod 4); two warps share a
    // quarter and split the tile's columns. Each round pulls 64 accumulator values per thread
    // into registers; after the last round the buffer is handed back to the MMA thread, and
    // only then come the arithmetic and the stores of that round.
    TileWalker walk(pm, p.n_tiles, p.E);
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = static_cast<int>(rank) * kBM + q * 32 + lane;
    constexpr bool fp8 = (ESIZE == 1);
    constexpr int kChunks = kTileN / 64;              // 32-column chunks per warp: 4 plain, 2 gated
    const bool plain_math = p.bias0 == nullptr && p.bias1 == nullptr && !(fp8 && p.a_scale != nullptr);
    const int c_begin = half * kChunks * 32;
    const uint32_t stage_w = staging_addr + (warp - 2) * 2048;
    int it = 0;
    for (int t = unit; t < total_tiles; t += num_units, ++it) {
      int e, mb, nb;
      walk.decode(t, e, mb, nb);
      const long long row = static_cast<long long>(soff[e]) + mb * kTileRows + row_in_tile;
      const bool row_ok = row < soff[e + 1];
      float scale_a = 1.0f;
      if (fp8 && p.a_scale != nullptr && row_ok) {
        long long src = row;
        if (GATHER && p.index) src = p.index[row] / p.index_div;
        if (src < 0 || src >= p.a_rows) src = 0;
        scale_a = p.a_scale[src];
      }
      long long dst_row = row;
      float gate_scale = 1.0f;
      bool store_ok = row_ok;             // false: the row exists but its destination does not - nothing is written
      constexpr bool combine = COMBINE;   // compiled in only for the plain, contiguous-row kernels
      if (combine && row_ok) {
        const long long gi = p.gate_index[row];
        if (gi < 0 || gi >= p.out_rows * p.gate_div) {
          atomicCAS(p.status, 0, FMOE_DEV_BAD_INDEX);
          store_ok = false;
        } else {
          dst_row = gi / p.gate_div;
          gate_scale = p.gate_is_f32 ? reinterpret_cast<const float*>(p.gate)[gi]
                                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.gate)[gi]);
          if (p.gate_round && sizeof(OutT) == 2) gate_scale = __bfloat162float(__float2bfloat16_rn(gate_scale));
        }
      }
      OutT* out_base = reinterpret_cast<OutT*>(p.out);
      if (p.out_index != nullptr && row_ok && !combine) {
        dst_row = p.out_index[row];
        if (p.out_peers != nullptr) {
          // (peer << 40) | row: the row goes to that peer's buffer (plain stores, possibly over NVLink)
          const long long peer = dst_row >> 40;
          dst_row &= (1ll << 40) - 1;
          if (peer < 0 || peer >= p.n_peers) {
            dst_row = -1;
          } else {
            out_base = reinterpret_cast<OutT*>(p.out_peers[peer]);
          }
        }
        if (dst_row < 0 || dst_row >= p.out_rows) {
          atomicCAS(p.status, 0, FMOE_DEV_BAD_INDEX);
          dst_row = 0;
          store_ok = false;
        }
      }
      OutT* out_row = out_base + dst_row * p.ldo;
      // Coalesced store phase: lane l writes the 16-byte piece (l & 3) of rows (l >> 2) + 8 i.
      // It needs those rows' destinations, which live in the lanes that own them.
      OutT* st_row[4];
      bool st_ok[4];
      const OutT* mul_row[4] = {nullptr, nullptr, nullptr, nullptr};
      // the multiplier of a gated product goes in with the coalesced store phase (not with a combine)
      // (plain tiles only; the in-kernel-gather variants run at their register cap and keep the
      //  multiplier in the math phase)
      constexpr bool kMulStaged = !GATHER && !DUAL;
      const bool mul_staged = kMulStaged && p.mul_in != nullptr && !combine && p.mul_vec != 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int src_lane = (lane >> 2) + 8 * i;
        const unsigned long long ptr_bits =
            __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(out_row), src_lane);
        st_row[i] = reinterpret_cast<OutT*>(ptr_bits);
        st_ok[i] = __shfl_sync(0xffffffffu, store_ok ? 1 : 0, src_lane) != 0;
        if constexpr (kMulStaged) {
          if (mul_staged) {
            const long long mrow = __shfl_sync(0xffffffffu, row, src_lane);
            mul_row[i] = reinterpret_cast<const OutT*>(p.mul_in) + mrow * p.ld_mul;
          }
        }
      }
      const int n0 = nb * kTileN;
      // Column factors of this tile (bias, FP8 column scales): fetched before the wait for the
      // accumulator, lane i holding column i of every 32-column chunk, so that their latency
      // hides behind the MMAs instead of stalling every chunk.
      // (Plain tiles: their epilogue has no slack at small K. The gated tiles keep fetching per chunk:
      //  they run at the register cap and measured slower with the extra live values.)
      constexpr bool kPrefetch = !DUAL;
      float pre_b0[kPrefetch ? kChunks : 1], pre_b1[1], pre_f0[(kPrefetch && fp8) ? kChunks : 1], pre_f1[1];
      pre_b0[0] = 0.f; pre_b1[0] = 0.f; pre_f0[0] = 1.f; pre_f1[0] = 1.f;
#pragma unroll
      for (int j = 0; j < (kPrefetch ? kChunks : 0); ++j) {
        pre_b0[j] = 0.f;
        if constexpr (DUAL) pre_b1[j] = 0.f;
        if constexpr (fp8) pre_f0[j] = 1.f;
        if constexpr (fp8 && DUAL) pre_f1[j] = 1.f;
        const int col = n0 + c_begin + 32 * j + lane;
        if (col < p.N) {
          if (p.bias0 != nullptr) pre_b0[j] = load_as_float<OutT>(p.bias0, static_cast<long long>(e) * p.bias_se + col);
          if constexpr (DUAL) {
            if (p.bias1 != nullptr) pre_b1[j] = load_as_float<OutT>(p.bias1, static_cast<long long>(e) * p.bias_se + col);
          }
          if constexpr (fp8) {
            if (p.a_scale != nullptr) {
              const long long so = static_cast<long long>(e) * p.bscale_se + col;
              pre_f0[j] = 1.0f / p.b0_scale[so];
              if constexpr (DUAL) pre_f1[j] = 1.0f / p.b1_scale[so];
            }
          }
        }
      }
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, p.status, FMOE_DEV_WAIT_EPILOGUE)) {
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kMmaN + c_begin;
      // 64 accumulator registers in flight per round: two 32-column chunks (plain), or one chunk
      // of each of the two accumulators (gated)
      constexpr int kPerRound = DUAL ? 1 : 2;
#pragma unroll
      for (int j0 = 0; j0 < kChunks; j0 += kPerRound) {
        uint32_t r0[kPerRound][32];
        uint32_t r1[kPerRound][32];
#pragma unroll
        for (int j = 0; j < kPerRound; ++j) {
          ptx::tmem_ld_32x32b_x32(t_row + 32 * (j0 + j), r0[j]);
          if constexpr (DUAL) ptx::tmem_ld_32x32b_x32(t_row + kTileN + 32 * (j0 + j), r1[j]);
        }
        ptx::tmem_ld_wait();
        if (j0 + kPerRound >= kChunks) {
          // last read of this accumulator buffer: the next tile's MMAs may overwrite it
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(acc), 0));
            } else {
              ptx::mbar_arrive(tempty_bar(acc));
            }
          }
        }
        // the arithmetic of all chunks of the round first (independent special-function work back
        // to back), then their stores
        float vv[kPerRound][32];
        const bool want_silu = !DUAL && p.epilogue == FMOE_EPI_SILU;
#pragma unroll
        for (int j = 0; j < kPerRound; ++j) {
          const int col0 = n0 + c_begin + 32 * (j0 + j);
          const int ncols = min(32, p.N - col0);
          float (&v)[32] = vv[j];
          if (DUAL && ncols == 32 && plain_math) {
            // gated tile, whole chunk inside N, no bias, no dequantisation: straight-line arithmetic
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = silu_f(__uint_as_float(r0[j][i])) * __uint_as_float(r1[j][i]);
          } else if (!DUAL && !combine && ncols == 32 && plain_math && p.epilogue == FMOE_EPI_NONE) {
            // plain tile, nothing to add or scale: the accumulator values as they are
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[j][i]);
          } else if (ncols == 32) {
            // Whole chunk inside N with scales and / or bias: lane i fetches the factors of column i
            // once and the warp shares them by shuffle. Dividing by s_row * s_col equals
            // multiplying by the two reciprocals whenever the scales are powers of two, which the
            // quantisation rule guarantees.
            const bool scaled = fp8 && p.a_scale != nullptr;
            const bool has_b0 = p.bias0 != nullptr;
            const bool has_b1 = DUAL && p.bias1 != nullptr;
            const float inv_a = 1.0f / scale_a;          // this lane's row
            // column factors: lane i holds column i's
            float f0 = 1.f, f1 = 1.f, bb0 = 0.f, bb1 = 0.f;
            if constexpr (kPrefetch) {                   // fetched at the top of the tile
              f0 = pre_f0[fp8 ? j0 + j : 0];
              bb0 = pre_b0[j0 + j];
            } else {
              if (scaled) {
                const long long so = static_cast<long long>(e) * p.bscale_se + col0 + lane;
                f0 = 1.0f / p.b0_scale[so];
                if constexpr (DUAL) f1 = 1.0f / p.b1_scale[so];
              }
              if (has_b0) bb0 = load_as_float<OutT>(p.bias0, static_cast<long long>(e) * p.bias_se + col0 + lane);
              if (has_b1) bb1 = load_as_float<OutT>(p.bias1, static_cast<long long>(e) * p.bias_se + col0 + lane);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float g = __uint_as_float(r0[j][i]);
              float u = DUAL ? __uint_as_float(r1[j][i]) : 0.f;
              if (scaled) {
                g = __bfloat162float(__float2bfloat16_rn(g)) * (inv_a * __shfl_sync(0xffffffffu, f0, i));
                if constexpr (DUAL) {
                  u = __bfloat162float(__float2bfloat16_rn(u)) * (inv_a * __shfl_sync(0xffffffffu, f1, i));
                }
                // the reference casts the descaled product to the output type BEFORE it adds the
                // bias (kernels/pytorch/moe_fp8.py:126-133)
                if constexpr (sizeof(OutT) == 2) {
                  if (has_b0) g = __bfloat162float(__float2bfloat16_rn(g));
                  if (has_b1) u = __bfloat162float(__float2bfloat16_rn(u));
                }
              }
              if (has_b0) g += __shfl_sync(0xffffffffu, bb0, i);
              if (has_b1) u += __shfl_sync(0xffffffffu, bb1, i);
              if constexpr (DUAL) {
                v[i] = silu_f(g) * u;
              } else {
                v[i] = g;
              }
            }
            if (want_silu) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
            }
          } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + i;
            float g = __uint_as_float(r0[j][i]);
            float u = DUAL ? __uint_as_float(r1[j][i]) : 0.f;
            if (col < p.N) {
              if (fp8 && p.a_scale != nullptr) {
                const long long so = static_cast<long long>(e) * p.bscale_se + col;
                g = __bfloat162float(__float2bfloat16_rn(g)) / (scale_a * p.b0_scale[so]);
                if constexpr (DUAL) u = __bfloat162float(__float2bfloat16_rn(u)) / (scale_a * p.b1_scale[so]);
                if constexpr (sizeof(OutT) == 2) {   // cast, then bias: see the fast path above
                  if (p.bias0) g = __bfloat162float(__float2bfloat16_rn(g));
                  if (DUAL && p.bias1) u = __bfloat162float(__float2bfloat16_rn(u));
                }
              }
              if (p.bias0) g += load_as_float<OutT>(p.bias0, static_cast<long long>(e) * p.bias_se + col);
              if constexpr (DUAL) {
                if (p.bias1) u += load_as_float<OutT>(p.bias1, static_cast<long long>(e) * p.bias_se + col);
              }
            }
            if constexpr (DUAL) {
              v[i] = silu_f(g) * u;
            } else {
              v[i] = (p.epilogue == FMOE_EPI_SILU) ? silu_f(g) : g;
            }
          }
          }
        }
#pragma unroll
        for (int j = 0; j < kPerRound; ++j) {
          const int col0 = n0 + c_begin + 32 * (j0 + j);
          const int ncols = min(32, p.N - col0);
          float (&v)[32] = vv[j];
          const bool staged = ncols == 32 && p.vec_ok;
          if (p.mul_in != nullptr && row_ok && !(staged && mul_staged)) {
            // second factor of a gated product on the paths without the staged store: this row's
            // values of the multiplier tensor, the product of the two rounded operands as there
            const OutT* mrow = reinterpret_cast<const OutT*>(p.mul_in) + row * p.ld_mul + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i < ncols) {
                float y = v[i];
                if constexpr (sizeof(OutT) == 2) y = __bfloat162float(__float2bfloat16_rn(y));
                v[i] = y * load_as_float<OutT>(mrow, i);
              }
            }
          }
          if (combine) {
            // what the reference does in the activation type: round the GEMM row, multiply by the
            // gate weight, round again (Tensor.mul), then accumulate
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float y = v[i];
              if constexpr (sizeof(OutT) == 2) y = __bfloat162float(__float2bfloat16_rn(y));
              v[i] = y * gate_scale;
            }
          }
          if (staged) {
            stage_and_store<OutT>(stage_w, lane, v, st_row, st_ok, col0, combine, mul_row, mul_staged);
          } else if (store_ok && ncols > 0) {
            if (combine) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (i < ncols) {
                  if constexpr (sizeof(OutT) == 2) {
                    atomicAdd(out_row + col0 + i, __float2bfloat16_rn(v[i]));
                  } else {
                    atomicAdd(out_row + col0 + i, v[i]);
                  }
                }
              }
            } else {
              store_chunk<OutT>(out_row + col0, v, ncols, false);
            }
          }
        }
      }
    }
  } else if (warp < 2 + kEpilogueWarps + kGatherWarps) {
    // =========================================================== activation-row gather (4 warps)
    // Thread g copies the 16-byte piece (g & 7) of rows (g >> 3) + 16 i, i = 0..7: eight
    // neighbouring threads read one full 128-byte line of a token row, and write it into the
    // 128-byte-swizzled tile (piece c of row r lands at r * 128 + ((c ^ (r & 7)) << 4)).
    if constexpr (GATHER) {
      TileWalker walk(pm, p.n_tiles, p.E);
      const int g = threadIdx.x - kBaseThreads;
      const int piece = g & 7;
      const int rbase = g >> 3;
      const uint32_t dst_off = rbase * kRowBytes + ((piece ^ (rbase & 7)) << 4);
      const long long k_bytes = static_cast<long long>(p.K) * ESIZE;
      const long long lda_bytes = p.lda * ESIZE;
      const uint8_t* a_base = reinterpret_cast<const uint8_t*>(p.a);
      // Row addresses of a tile: rows past the end of the segment re-read the tile's first row
      // (their results are never stored).
      auto tile_rows = [&](int t, const uint8_t* (&dst)[8]) {
        int e, mb, nb;
        walk.decode(t, e, mb, nb);
        const int seg1 = soff[e + 1];
        const int tile0 = soff[e] + mb * kTileRows;
        const int row0 = tile0 + static_cast<int>(rank) * kBM;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int rr = row0 + rbase + 16 * i;
          if (rr >= seg1) rr = tile0;
          // indices and row counts are below 2^31 (the host checks the counts): 32-bit
          // arithmetic, and no division at all in the common case of one row per index
          const long long raw = p.index[rr];
          unsigned srow = static_cast<unsigned>(raw);
          if (p.index_div != 1) srow /= static_cast<unsigned>(p.index_div);
          if (raw < 0 || raw > 0x7fffffffll || srow >= static_cast<unsigned>(p.a_rows)) {
            atomicCAS(p.status, 0, FMOE_DEV_BAD_INDEX);
            srow = 0;
          }
          dst[i] = a_base + srow * lda_bytes + piece * 16;
        }
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint8_t* src[8];
      const uint8_t* nsrc[8];
      if (unit < total_tiles) tile_rows(unit, src);
      for (int t = unit; t < total_tiles && ok; t += num_units) {
        // the next tile's indices are fetched while this tile's K loop runs
        const int t_next = t + num_units;
        if (t_next < total_tiles) {
          tile_rows(t_next, nsrc);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) nsrc[i] = src[i];
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                      FMOE_DEV_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          const long long koff = static_cast<long long>(kb) * kRowBytes;
          // K is a multiple of 16 bytes: a piece is either whole or entirely past the end (zero-filled)
          const uint32_t nbytes = (koff + piece * 16 < k_bytes) ? 16u : 0u;
          const uint32_t dst = tiles_addr + stage * Plan::kStageBytes + dst_off;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            ptx::cp_async_16(dst + i * 16 * kRowBytes, src[i] + (nbytes ? koff : 0), nbytes);
          }
          // one arrival per thread, delivered by the hardware when this thread's copies have landed
          ptx::cp_async_mbar_arrive_noinc(kPair ? afull_bar(stage) : full_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) src[i] = nsrc[i];
      }
      ptx::cp_async_wait_all();
    }
  } else {
    // =========================================================== relay (pairs that gather)
    // "This CTA's gathered rows of stage s have landed" -> one arrival on the leader's full barrier.
    if constexpr (GATHER && kPair) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = unit; t < total_tiles && ok; t += num_units) {
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!ptx::mbar_wait_bounded(afull_bar(stage), phase, abort_flag, p.status, FMOE_DEV_WAIT_PRODUCER)) {
              ok = false;
              break;
            }
            ptx::fence_proxy_async_smem();   // cp.async wrote through the generic proxy; the MMA reads via the async proxy
            ptx::mbar_arrive_cluster(ptx::mapa(full_bar(stage), 0));
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  }

  // ---- tear-down
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out. Give copies still in flight time to land before shared memory and
    // tensor memory are handed back.
    __nanosleep(2000000);
    __syncthreads();
  }
  // a CTA of a pair must not leave while its peer can still signal its barriers or read its tiles
  if constexpr (kPair) ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CTAS>(tmem_base, kTmemCols);
  }
}

#if FMOE_GEMM_HOST
// One CTA waits on a barrier that nothing will ever signal, with a short limit. Exercises the
// path every wait of the GEMM takes when it gives up: status code recorded, abort flag raised,
// thread returns; nothing traps and the context stays usable.
__global__ void selftest_wait_kernel(unsigned long long limit_ns, int* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, status, FMOE_DEV_WAIT_PRODUCER, limit_ns, 64);
  }
  __syncthreads();
  // a second waiter sees the abort flag and leaves at once
  if (threadIdx.x == 32) {
    ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, status, FMOE_DEV_WAIT_MMA, 5000000000ull, 64);
  }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn(int* err) {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || sym == nullptr) {
    *err = fail(FMOE_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available (%s)",
                e != cudaSuccess ? cudaGetErrorString(e) : "driver query failed");
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

CUtensorMapDataType tmap_dtype(int dt) {
  switch (dt) {
    case FMOE_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case FMOE_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

int make_tmap(CUtensorMap* m, int dt, int rank, const void* base, const cuuint64_t* dims,
              const cuuint64_t* strides_bytes, const cuuint32_t* box, const char* what) {
  int err = 0;
  EncodeTiledFn fn = encode_fn(&err);
  if (!fn) return err;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, tmap_dtype(dt), rank, const_cast<void*>(base), dims, strides_bytes, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(FMOE_ERR_UNSUPPORTED,
                "tensor map for %s rejected (CUresult %d): base %p, dims %llu x %llu, row stride %llu B", what,
                static_cast<int>(r), base, (unsigned long long)dims[0], (unsigned long long)dims[1],
                (unsigned long long)strides_bytes[0]);
  }
  return FMOE_OK;
}

int g_launches = 0;
int g_num_sms = 0;
#else
extern int g_launches;
#endif  // FMOE_GEMM_HOST

template <int ESIZE, typename OutT>
int dispatch_shape(int ctas, bool dual, bool gather, const CUtensorMap& tmA, const CUtensorMap& tmB0,
                   const CUtensorMap& tmB1, const GemmParams& p, int grid, cudaStream_t stream);

#if FMOE_GEMM_KERNELS
template <int ESIZE, int CTAS, bool DUAL, bool GATHER, bool COMBINE, typename OutT>
int launch_t(const CUtensorMap& tmA, const CUtensorMap& tmB0, const CUtensorMap& tmB1, const GemmParams& p,
             int grid, cudaStream_t stream) {
  using Plan = SmemPlan<CTAS>;
  auto kern = grouped_gemm_kernel<ESIZE, CTAS, DUAL, GATHER, COMBINE, OutT>;
  // function attributes belong to a device's context: set once per device
  static std::atomic<bool> attr_set[kMaxDevices];
  int dev = 0;
  int rc = current_device_slot(&dev);
  if (rc != FMOE_OK) return rc;
  if (!attr_set[dev].load(std::memory_order_acquire)) {
    FMOE_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kTotal));
    attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(GATHER ? kGatherKernelThreads : kBaseThreads, 1, 1);
  cfg.dynamicSmemBytes = Plan::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (CTAS > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = CTAS;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (programmatic_launch_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  FMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmA, tmB0, tmB1, p));
  ++g_launches;
  return FMOE_OK;
}

template <int ESIZE, typename OutT>
int dispatch_shape(int ctas, bool dual, bool gather, const CUtensorMap& tmA, const CUtensorMap& tmB0,
                   const CUtensorMap& tmB1, const GemmParams& p, int grid, cudaStream_t stream) {
#define FMOE_GO(C, D, G) return launch_t<ESIZE, C, D, G, false, OutT>(tmA, tmB0, tmB1, p, grid, stream)
  if (p.gate_index != nullptr) {
    // fused combine: plain epilogue on contiguous rows only (checked by the caller)
    if (ctas == 2) return launch_t<ESIZE, 2, false, false, true, OutT>(tmA, tmB0, tmB1, p, grid, stream);
    return launch_t<ESIZE, 1, false, false, true, OutT>(tmA, tmB0, tmB1, p, grid, stream);
  }
  if (ctas == 2) {
    if (dual) { if (gather) FMOE_GO(2, true, true); else FMOE_GO(2, true, false); }
    if (gather) FMOE_GO(2, false, true); else FMOE_GO(2, false, false);
  }
  if (dual) { if (gather) FMOE_GO(1, true, true); else FMOE_GO(1, true, false); }
  if (gather) FMOE_GO(1, false, true); else FMOE_GO(1, false, false);
#undef FMOE_GO
}
#if FMOE_GEMM_PART == 1
template int dispatch_shape<2, __nv_bfloat16>(int, bool, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                              const GemmParams&, int, cudaStream_t);
template int dispatch_shape<2, float>(int, bool, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                      const GemmParams&, int, cudaStream_t);
#elif FMOE_GEMM_PART == 2
template int dispatch_shape<4, float>(int, bool, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                      const GemmParams&, int, cudaStream_t);
#elif FMOE_GEMM_PART == 3
template int dispatch_shape<1, __nv_bfloat16>(int, bool, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                              const GemmParams&, int, cudaStream_t);
template int dispatch_shape<1, float>(int, bool, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                      const GemmParams&, int, cudaStream_t);
#endif
#endif  // FMOE_GEMM_KERNELS

#if FMOE_GEMM_HOST
// 0 = choose by shape, 1 / 2 = force lone CTAs / CTA pairs (environment FMOE_GEMM_CTAS, read once).
int forced_ctas() {
  static int v = -1;
  if (v < 0) {
    const char* s = getenv("FMOE_GEMM_CTAS");
    v = (s && (s[0] == '1' || s[0] == '2') && s[1] == 0) ? s[0] - '0' : 0;
  }
  return v;
}

#endif  // FMOE_GEMM_HOST

}  // namespace gemm_detail

#if FMOE_GEMM_HOST
using namespace gemm_detail;

int grouped_gemm_launch_count() { return g_launches; }

int launch_selftest_wait(unsigned long long limit_ns, cudaStream_t stream) {
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  selftest_wait_kernel<<<1, 64, 0, stream>>>(limit_ns, status);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_launches;
  return FMOE_OK;
}

int launch_grouped_gemm(const GemmDesc& d, cudaStream_t stream) {
  const int esize = dtype_size(d.dtype);
  FMOE_REQUIRE(esize != 0, "grouped_gemm: unknown operand dtype %d", d.dtype);
  FMOE_REQUIRE(d.E >= 1 && d.E <= kMaxExperts, "grouped_gemm: E=%d outside [1, %d]", d.E, kMaxExperts);
  FMOE_REQUIRE(d.N >= 1 && d.K >= 1, "grouped_gemm: N=%d K=%d must be positive", d.N, d.K);
  // No rows: nothing to compute. Checked before the pointers, because an empty tensor's data
  // pointer is NULL and an empty batch (a rank of an expert-parallel job that receives no rows)
  // is valid input.
  if (d.total_rows <= 0) return FMOE_OK;
  FMOE_REQUIRE(d.offsets && d.a && d.b0 && d.out, "grouped_gemm: null pointer argument");
  FMOE_REQUIRE(d.out_dtype == FMOE_BF16 || d.out_dtype == FMOE_F32, "grouped_gemm: output must be bf16 or f32");
  FMOE_REQUIRE(d.dtype != FMOE_F32 || d.out_dtype == FMOE_F32, "grouped_gemm: f32 operands need an f32 output");
  FMOE_REQUIRE(d.epilogue != FMOE_EPI_SWIGLU || d.b1 != nullptr, "grouped_gemm: SwiGLU needs a second weight");
  FMOE_REQUIRE(d.index == nullptr || d.index_div >= 1, "grouped_gemm: index_div must be >= 1");
  const bool b_mn = d.b_sk > 1;
  if (b_mn) {
    FMOE_REQUIRE(esize == 2 && d.b_sn == 1 && d.N % 64 == 0 && d.kseg == nullptr,
                 "grouped_gemm: an N-contiguous weight needs bf16 operands and N a multiple of 64 (N=%d)", d.N);
  }
  const int ksplit = d.b_ksplit;
  if (ksplit > 0) {
    FMOE_REQUIRE(d.b1 != nullptr && d.epilogue != FMOE_EPI_SWIGLU && d.kseg == nullptr && ksplit < d.K &&
                     (static_cast<long long>(ksplit) * esize) % kRowBytes == 0,
                 "grouped_gemm: a reduction over two weights needs a second weight, a plain epilogue and a split at a "
                 "multiple of %d elements inside K (split %d, K %d)", kRowBytes / esize, ksplit, d.K);
  }
  const long long b_row_stride = b_mn ? d.b_sk : d.b_sn;     // stride of the non-contiguous matrix dimension
  if ((d.lda * esize) % 16 != 0 || (b_row_stride * esize) % 16 != 0 || (d.b_se * esize) % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(d.a) & 15) || (reinterpret_cast<uintptr_t>(d.b0) & 15) ||
      (d.b1 && (reinterpret_cast<uintptr_t>(d.b1) & 15))) {
    return fail(FMOE_ERR_UNSUPPORTED,
                "grouped_gemm: TMA needs 16-byte aligned bases and row strides (lda=%lld, b_sn=%lld, b_se=%lld "
                "elements of %d bytes)", (long long)d.lda, (long long)d.b_sn, (long long)d.b_se, esize);
  }
  if (d.index != nullptr && (static_cast<long long>(d.K) * esize) % 16 != 0) {
    return fail(FMOE_ERR_UNSUPPORTED, "grouped_gemm: gathered rows need K to be a multiple of 16 bytes (K=%d x %d B); pad K",
                d.K, esize);
  }
  FMOE_REQUIRE(d.mul_in == nullptr || (d.gate_index == nullptr && d.out_index == nullptr && d.epilogue != FMOE_EPI_SWIGLU),
               "grouped_gemm: the elementwise multiplier goes with the plain and SiLU epilogues only");
  FMOE_REQUIRE(d.kseg == nullptr || (d.index == nullptr && d.gate_index == nullptr && d.out_index == nullptr &&
                                     d.epilogue == FMOE_EPI_NONE && d.a_scale == nullptr),
               "grouped_gemm: the reduction-over-rows mode takes plain contiguous operands only");
  FMOE_REQUIRE(d.out_peers == nullptr || (d.out_index != nullptr && d.gate_index == nullptr && d.n_peers >= 1),
               "grouped_gemm: peer stores need a route table and exclude the fused combine");
  if (d.gate_index != nullptr && (d.index != nullptr || d.epilogue != FMOE_EPI_NONE)) {
    return fail(FMOE_ERR_UNSUPPORTED, "grouped_gemm: the fused combine needs contiguous rows and the plain epilogue");
  }
  FMOE_REQUIRE(d.a_rows >= 1, "grouped_gemm: empty A source with %lld output rows", (long long)d.total_rows);
  FMOE_REQUIRE(d.a_rows < (1ll << 31) && d.total_rows < (1ll << 31), "grouped_gemm: more than 2^31 rows");

  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  if (g_num_sms == 0) {
    int dev = 0;
    FMOE_CUDA_OK(cudaGetDevice(&dev));
    FMOE_CUDA_OK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
  }

  const bool dual = d.epilogue == FMOE_EPI_SWIGLU;
  const bool gather = d.index != nullptr;
  const int tile_n = dual ? 128 : 256;
  // Contiguous rows with a thousand or more rows per expert on average: CTA pairs (256-row tiles,
  // each CTA stages half of the weight tile, a third fewer operand bytes per SM and FLOP): 8-12 %
  // faster than lone CTAs on the down projections measured. With fewer rows per expert the
  // half-empty last tile of every segment costs more than that (512 rows per expert: pairs 5 %
  // slower). Gathered rows stay on lone CTAs: a pair needs a relay hop for the peer's gathered
  // rows and runs at half speed. FMOE_GEMM_CTAS forces either.
  int ctas = forced_ctas();
  const long long expect_rows = d.rows_hint > 0 ? d.rows_hint : d.total_rows;
  if (ctas == 0) ctas = (!gather && expect_rows / d.E >= 1024) ? 2 : 1;
  if (g_num_sms < 2) ctas = 1;
  const int box_n = (ctas == 2 || dual) ? 128 : 256;   // weight rows one TMA load brings in
  const int k_elems = kRowBytes / esize;

  CUtensorMap tmA, tmB0, tmB1;
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(d.K), static_cast<cuuint64_t>(d.a_rows)};
    cuuint64_t str[1] = {static_cast<cuuint64_t>(d.lda) * esize};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(k_elems), static_cast<cuuint32_t>(kBM)};
    int rc = make_tmap(&tmA, d.dtype, 2, d.a, dims, str, box, "activations");
    if (rc != FMOE_OK) return rc;
  }
  if (b_mn) {
    // N contiguous: dimensions (64 columns of an atom, K, atoms, expert); one load brings
    // box_n / 64 atoms of [one K step x 64 columns], each atom laid out as 128-byte rows
    cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(ksplit > 0 ? ksplit : d.K), static_cast<cuuint64_t>(d.N / 64),
                          static_cast<cuuint64_t>(d.E)};
    cuuint64_t str[3] = {static_cast<cuuint64_t>(d.b_sk) * esize, 64ull * esize, static_cast<cuuint64_t>(d.b_se) * esize};
    cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(k_elems), static_cast<cuuint32_t>(box_n / 64), 1u};
    int rc = make_tmap(&tmB0, d.dtype, 4, d.b0, dims, str, box, "weights (N contiguous)");
    if (rc != FMOE_OK) return rc;
    if (dual || ksplit > 0) {
      if (ksplit > 0) dims[1] = static_cast<cuuint64_t>(d.K - ksplit);
      rc = make_tmap(&tmB1, d.dtype, 4, d.b1, dims, str, box, "second weights (N contiguous)");
      if (rc != FMOE_OK) return rc;
    } else {
      tmB1 = tmB0;
    }
  } else {
    // reduction-over-rows mode: one B matrix [N, K] shared by all groups
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(ksplit > 0 ? ksplit : d.K), static_cast<cuuint64_t>(d.N),
                          static_cast<cuuint64_t>(d.kseg ? 1 : d.E)};
    cuuint64_t str[2] = {static_cast<cuuint64_t>(d.b_sn) * esize, static_cast<cuuint64_t>(d.b_se) * esize};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(k_elems), static_cast<cuuint32_t>(box_n), 1u};
    int rc = make_tmap(&tmB0, d.dtype, 3, d.b0, dims, str, box, "weights");
    if (rc != FMOE_OK) return rc;
    if (dual || ksplit > 0) {
      if (ksplit > 0) dims[0] = static_cast<cuuint64_t>(d.K - ksplit);
      rc = make_tmap(&tmB1, d.dtype, 3, d.b1, dims, str, box, "second weights");
      if (rc != FMOE_OK) return rc;
    } else {
      tmB1 = tmB0;
    }
  }

  GemmParams p;
  p.offsets = reinterpret_cast<const long long*>(d.offsets);
  p.index = reinterpret_cast<const long long*>(d.index);
  p.out_index = reinterpret_cast<const long long*>(d.out_index);
  p.out_rows = d.gate_index ? d.combine_rows : (d.out_peers ? d.peer_rows : d.total_rows);
  p.out_peers = reinterpret_cast<const long long*>(d.out_peers);
  p.n_peers = d.n_peers;
  p.index_div = d.index_div > 0 ? d.index_div : 1;
  p.E = d.E;
  p.N = d.N;
  p.K = d.K;
  p.num_kb = (d.K + k_elems - 1) / k_elems;
  p.n_tiles = (d.N + tile_n - 1) / tile_n;
  p.a = d.a;
  p.lda = d.lda;
  p.a_rows = d.a_rows;
  p.out = d.out;
  p.ldo = d.ldo;
  p.bias0 = d.bias0;
  p.bias1 = d.bias1;
  p.bias_se = d.bias_se;
  p.a_scale = d.a_scale;
  p.b0_scale = d.b0_scale;
  p.b1_scale = d.b1_scale;
  p.bscale_se = d.bscale_se;
  p.epilogue = d.epilogue;
  p.gate = d.gate;
  p.gate_is_f32 = d.gate_dtype == FMOE_F32 ? 1 : 0;
  p.gate_round = d.gate_round;
  p.gate_index = reinterpret_cast<const long long*>(d.gate_index);
  p.gate_div = d.gate_div > 0 ? d.gate_div : 1;
  const int osize = dtype_size(d.out_dtype);
  // peer buffers are 16-byte aligned by contract (their addresses live on the device)
  p.kseg = reinterpret_cast<const long long*>(d.kseg);
  p.mul_in = d.mul_in;
  p.ld_mul = d.ld_mul;
  p.b_mn = b_mn ? 1 : 0;
  p.b_ksplit = ksplit;
  p.mul_vec = d.mul_in != nullptr && ((d.ld_mul * osize) % 16 == 0) && (reinterpret_cast<uintptr_t>(d.mul_in) & 15) == 0;
  p.vec_ok = ((d.ldo * osize) % 16 == 0) && (d.out_peers != nullptr || (reinterpret_cast<uintptr_t>(d.out) & 15) == 0);
  p.status = status;

  // Persistent grid: one CTA per SM, never more CTAs than the largest possible tile count.
  const int tile_rows = kBM * ctas;
  const long long max_m_tiles = (d.total_rows + tile_rows - 1) / tile_rows + d.E;
  const long long max_tiles = max_m_tiles * p.n_tiles;
  const int units_avail = g_num_sms / ctas;
  int units = static_cast<int>(max_tiles < units_avail ? max_tiles : units_avail);
  if (units < 1) units = 1;
  const int grid = units * ctas;

  if (d.dtype == FMOE_BF16) {
    if (d.out_dtype == FMOE_BF16) return dispatch_shape<2, __nv_bfloat16>(ctas, dual, gather, tmA, tmB0, tmB1, p, grid, stream);
    return dispatch_shape<2, float>(ctas, dual, gather, tmA, tmB0, tmB1, p, grid, stream);
  } else if (d.dtype == FMOE_F32) {
    return dispatch_shape<4, float>(ctas, dual, gather, tmA, tmB0, tmB1, p, grid, stream);
  } else {
    if (d.out_dtype == FMOE_BF16) return dispatch_shape<1, __nv_bfloat16>(ctas, dual, gather, tmA, tmB0, tmB1, p, grid, stream);
    return dispatch_shape<1, float>(ctas, dual, gather, tmA, tmB0, tmB1, p, grid, stream);
  }
}

#endif  // FMOE_GEMM_HOST

}  // namespace fmoe
