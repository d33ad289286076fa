// Expert-parallel exchange over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The reference advertises an expert-parallel layer (README.md:100-113) but ships none, so these
// kernels mirror no reference code; they implement the exchange steps around the grouped GEMMs:
//
//   counts  every rank knows how many rows every rank routes to every expert (an all-gather of
//           the [E] histogram the routing kernel produced).
//   plan    (ep_plan_kernel) from those counts each rank derives, on the device and without the
//           host, (a) where its own rows for expert e start in the receive buffer of e's owner
//           and (b) the jagged offsets of its local experts over the rows it will receive. The
//           receive buffer is laid out expert-major (expert, source rank, token order), so the
//           expert GEMMs read it as plain contiguous tiles: no permutation pass, no gather.
//   dispatch (ep_dispatch_kernel) one warp per routed row copies the token row straight into the
//           owner's receive buffer with 16-byte stores through the peer mapping, and leaves the
//           row's return address (source rank, position in the source's expert-sorted order) in
//           the owner's route table.
//   return  happens inside the down-projection GEMM: its epilogue stores every result row at its
//           return address in the source rank's buffer (grouped_gemm.cu, out_peers), so the
//           transfer overlaps the tensor-core work tile by tile and no second exchange runs.
// Only plain loads and stores touch peer memory (no TMA, no multicast). Ordering between ranks
// (rows landed before the GEMM reads them, results landed before the combine) is the caller's:
// a collective on the same stream between the steps.
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace fmoe {

extern long long g_misc_launches;

namespace {

constexpr int kPlanThreads = 1024;
constexpr int kRouteShift = 40;       // return address = (source rank << 40) | row in the source's sorted order

// counts [W, E] int64: counts[s, e] = rows rank s routes to global expert e; expert e lives on rank
// e / El. One block; thread e handles expert e.
__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const long long* __restrict__ counts, int W, int E, int El, int rank,
               long long* __restrict__ dst_base, long long* __restrict__ offsets_local,
               long long capacity, int* status) {
  extern __shared__ long long tot[];              // rows every rank together sends to expert e
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    long long t = 0;
    for (int s = 0; s < W; ++s) {
      const long long c = counts[static_cast<long long>(s) * E + e];
      t += c < 0 ? 0 : c;
    }
    tot[e] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int owner = e / El;
    long long base = 0;                           // start of expert e in its owner's receive buffer
    for (int f = owner * El; f < e; ++f) base += tot[f];
    long long before = 0;                         // rows of lower-ranked sources for the same expert
    for (int s = 0; s < rank; ++s) {
      const long long c = counts[static_cast<long long>(s) * E + e];
      before += c < 0 ? 0 : c;
    }
    dst_base[e] = base + before;
    if (owner == rank) {
      offsets_local[e - owner * El] = base;
      if (e == owner * El + El - 1) {
        const long long total = base + tot[e];
        offsets_local[El] = total;
        if (total > capacity) atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);   // more rows than the receive buffer holds
      }
    }
  }
}

// One warp per routed row p (rows are in this rank's expert-sorted order).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint8_t* __restrict__ x, long long x_rows, long long ldx_bytes, int row_bytes,
                   const long long* __restrict__ offsets, const long long* __restrict__ token_index,
                   long long rows, int E, int El, const long long* __restrict__ dst_base,
                   const long long* __restrict__ recv_ptrs, const long long* __restrict__ route_ptrs,
                   long long ld_recv_bytes, long long capacity, int rank, int vec_ok, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  // Rows are sorted by owner and blocks start in index order: every rank begins a different
  // fraction of the way through its rows, so that the ranks do not all write to the same owner
  // at the same time (its NVLink ingress would be the one busy port).
  const long long shift = rows * rank / (E / El);
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < rows; i += warps) {
    const long long p = (i + shift) % rows;
    // expert of row p: the last e with offsets[e] <= p
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= p) lo = mid; else hi = mid;
    }
    const int e = lo;
    const long long q = dst_base[e] + (p - offsets[e]);
    const long long src = token_index[p];
    if (q < 0 || q >= capacity || src < 0 || src >= x_rows || p >= offsets[E]) {
      if (lane == 0) atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      continue;                                   // nothing is written for a row without a valid place
    }
    const int owner = e / El;
    uint8_t* dst = reinterpret_cast<uint8_t*>(recv_ptrs[owner]) + q * ld_recv_bytes;
    const uint8_t* a = x + src * ldx_bytes;
    if (vec_ok) {
      const int vec = row_bytes >> 4;
      const uint4* a4 = reinterpret_cast<const uint4*>(a);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int c0 = lane; c0 < vec; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + 32 * u < vec) v[u] = a4[c0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + 32 * u < vec) d4[c0 + 32 * u] = v[u];
      }
    } else {
      for (int c = lane; c < row_bytes; c += 32) dst[c] = a[c];
    }
    if (lane == 0) {
      reinterpret_cast<long long*>(route_ptrs[owner])[q] = (static_cast<long long>(rank) << kRouteShift) | p;
    }
  }
}

// The same dispatch with one bulk copy per row: the warp stages the token row in shared memory
// (ordinary 16-byte loads) and one lane sends it with a single cp.async.bulk shared -> global
// store to the owner's buffer, so a row crosses NVLink as a few large write bursts instead of 512
// separate 16-byte stores. Two staging buffers per warp: the next row is loaded while the previous
// one is still being read out by the copy engine. Plain bulk store, no multicast, no tensor map.
constexpr int kBulkWarps = 8;

__global__ void __launch_bounds__(kBulkWarps * 32)
ep_dispatch_bulk_kernel(const uint8_t* __restrict__ x, long long x_rows, long long ldx_bytes, int row_bytes,
                        const long long* __restrict__ offsets, const long long* __restrict__ token_index,
                        long long rows, int E, int El, const long long* __restrict__ dst_base,
                        const long long* __restrict__ recv_ptrs, const long long* __restrict__ route_ptrs,
                        long long ld_recv_bytes, long long capacity, int rank, int* status) {
  extern __shared__ __align__(128) uint8_t s_stage[];          // [kBulkWarps][2][row_bytes]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* my_stage = s_stage + static_cast<size_t>(warp) * 2 * row_bytes;
  const long long warps = static_cast<long long>(gridDim.x) * kBulkWarps;
  int buf = 0;
  // Rows are sorted by owner; every rank starts a different fraction of the way through its rows
  // so that the ranks do not all write to the same owner at the same time.
  const long long shift = rows * rank / (E / El);
  for (long long i = static_cast<long long>(blockIdx.x) * kBulkWarps + warp; i < rows; i += warps) {
    const long long p = (i + shift) % rows;
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= p) lo = mid; else hi = mid;
    }
    const int e = lo;
    const long long q = dst_base[e] + (p - offsets[e]);
    const long long src = token_index[p];
    if (q < 0 || q >= capacity || src < 0 || src >= x_rows || p >= offsets[E]) {
      if (lane == 0) atomicCAS(status, 0, FMOE_DEV_BAD_INDEX);
      continue;
    }
    const int owner = e / El;
    uint8_t* stage = my_stage + static_cast<size_t>(buf) * row_bytes;
    // the copy issued two rows ago from this buffer must have finished reading it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
    const uint4* a4 = reinterpret_cast<const uint4*>(x + src * ldx_bytes);
    uint4* s4 = reinterpret_cast<uint4*>(stage);
    const int vec = row_bytes >> 4;
    for (int c0 = lane; c0 < vec; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < vec) v[u] = a4[c0 + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < vec) s4[c0 + 32 * u] = v[u];
    }
    // the staged row was written through the generic proxy; the bulk copy reads through the async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(recv_ptrs[owner]) + q * ld_recv_bytes;
      const uint32_t saddr = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(saddr), "r"(row_bytes)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      reinterpret_cast<long long*>(route_ptrs[owner])[q] = (static_cast<long long>(rank) << kRouteShift) | p;
    }
    buf ^= 1;
  }
  // every copy has left shared memory and is complete before the block exits
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_ep_plan(const int64_t* counts, int world, int E, int rank, int64_t capacity, int64_t* dst_base,
                            int64_t* offsets_local, void* stream) {
  FMOE_REQUIRE(world >= 1 && E >= 1 && E <= 4096 && E % world == 0, "ep_plan: E=%d must be a multiple of world=%d", E,
               world);
  FMOE_REQUIRE(rank >= 0 && rank < world, "ep_plan: rank %d outside [0, %d)", rank, world);
  FMOE_REQUIRE(counts && dst_base && offsets_local, "ep_plan: NULL pointer argument");
  FMOE_REQUIRE(capacity >= 0, "ep_plan: negative capacity");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ep_plan_kernel<<<1, kPlanThreads, static_cast<size_t>(E) * sizeof(long long), st>>>(
      reinterpret_cast<const long long*>(counts), world, E, E / world, rank, reinterpret_cast<long long*>(dst_base),
      reinterpret_cast<long long*>(offsets_local), capacity, status);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_ep_dispatch(const void* x, int dtype, int64_t x_rows, int64_t ldx, int cols,
                                const int64_t* offsets, const int64_t* token_index, int64_t rows, int E, int world,
                                int rank, const int64_t* dst_base, const int64_t* recv_ptrs,
                                const int64_t* route_ptrs, int64_t ld_recv, int64_t capacity, void* stream) {
  const int es = dtype_size(dtype);
  FMOE_REQUIRE(es != 0, "ep_dispatch: unknown dtype %d", dtype);
  FMOE_REQUIRE(world >= 1 && E >= 1 && E % world == 0 && rank >= 0 && rank < world, "ep_dispatch: E=%d world=%d rank=%d",
               E, world, rank);
  FMOE_REQUIRE(rows >= 0 && cols >= 1 && ld_recv >= cols, "ep_dispatch: rows=%lld cols=%d ld_recv=%lld", (long long)rows,
               cols, (long long)ld_recv);
  if (rows == 0) return FMOE_OK;
  FMOE_REQUIRE(x && offsets && token_index && dst_base && recv_ptrs && route_ptrs, "ep_dispatch: NULL pointer argument");
  int err = 0;
  int* status = device_status_ptr(&err);
  if (!status) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int row_bytes = cols * es;
  // 16-byte copies need aligned rows on both sides; peer buffers are allocated 16-byte aligned by
  // contract, their row stride is checked here
  const int vec_ok = (row_bytes % 16 == 0) && ((ldx * es) % 16 == 0) && ((ld_recv * es) % 16 == 0) &&
                     ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  // FMOE_EP_DISPATCH=bulk: rows of 16 KB or less that are 16-byte aligned go out as one bulk copy
  // each instead of 16-byte stores (measured equal at 2 GPUs: 0.155 vs 0.14 ms for 134 MB)
  static int mode = -1;
  if (mode < 0) {
    const char* m = getenv("FMOE_EP_DISPATCH");
    mode = (m && m[0] == 'b') ? 1 : 0;
  }
  if (mode == 1 && vec_ok && row_bytes <= 16 * 1024 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const size_t smem = static_cast<size_t>(kBulkWarps) * 2 * row_bytes;
    static std::atomic<bool> attr_set[kMaxDevices];
    int dev = 0;
    int rc = current_device_slot(&dev);
    if (rc != FMOE_OK) return rc;
    if (smem > 48 * 1024 && !attr_set[dev].load(std::memory_order_acquire)) {
      FMOE_CUDA_OK(cudaFuncSetAttribute(ep_dispatch_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_set[dev].store(true, std::memory_order_release);
    }
    long long nb = (rows + kBulkWarps - 1) / kBulkWarps;
    if (nb > 148) nb = 148;
    ep_dispatch_bulk_kernel<<<static_cast<unsigned>(nb), kBulkWarps * 32, smem, st>>>(
        static_cast<const uint8_t*>(x), x_rows, ldx * es, row_bytes, reinterpret_cast<const long long*>(offsets),
        reinterpret_cast<const long long*>(token_index), rows, E, E / world, reinterpret_cast<const long long*>(dst_base),
        reinterpret_cast<const long long*>(recv_ptrs), reinterpret_cast<const long long*>(route_ptrs), ld_recv * es,
        capacity, rank, status);
    FMOE_CUDA_OK(cudaGetLastError());
    ++g_misc_launches;
    return FMOE_OK;
  }
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ep_dispatch_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const uint8_t*>(x), x_rows, ldx * es, row_bytes, reinterpret_cast<const long long*>(offsets),
      reinterpret_cast<const long long*>(token_index), rows, E, E / world, reinterpret_cast<const long long*>(dst_base),
      reinterpret_cast<const long long*>(recv_ptrs), reinterpret_cast<const long long*>(route_ptrs), ld_recv * es,
      capacity, rank, vec_ok, status);
  FMOE_CUDA_OK(cudaGetLastError());
  ++g_misc_launches;
  return FMOE_OK;
}

extern "C" int fmoe_ep_up_projection(const int64_t* offsets_local, int64_t capacity, int64_t rows_hint,
                                     const void* recv, int dtype, int64_t ld_recv, const void* weight,
                                     const void* weight_p, int64_t w_se, int64_t w_sn, int E_local, int K, int N,
                                     void* out, int64_t ldo, void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "ep_up_projection: dtype must be bf16 or f32");
  FMOE_REQUIRE(weight_p != nullptr, "ep_up_projection: weight_p is NULL");
  GemmDesc g = {};
  g.dtype = dtype;
  g.E = E_local; g.N = N; g.K = K;
  g.offsets = offsets_local;
  g.total_rows = capacity;
  g.rows_hint = rows_hint;
  g.a = recv; g.a_rows = capacity; g.lda = ld_recv;
  g.b0 = weight; g.b1 = weight_p;
  g.b_se = w_se; g.b_sn = w_sn;
  g.epilogue = FMOE_EPI_SWIGLU;
  g.out = out; g.out_dtype = dtype; g.ldo = ldo;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}

extern "C" int fmoe_ep_down_projection(const int64_t* offsets_local, int64_t capacity, int64_t rows_hint,
                                       const void* hidden, int dtype, int64_t ldh, const void* weight, int64_t w_se,
                                       int64_t w_sn, int E_local, int K, int N, const int64_t* route,
                                       const int64_t* back_ptrs, int world, int64_t back_rows, int64_t ld_back,
                                       void* stream) {
  FMOE_REQUIRE(dtype == FMOE_BF16 || dtype == FMOE_F32, "ep_down_projection: dtype must be bf16 or f32");
  FMOE_REQUIRE(world >= 1 && back_rows >= 0, "ep_down_projection: world=%d back_rows=%lld", world, (long long)back_rows);
  FMOE_REQUIRE(capacity == 0 || (route && back_ptrs), "ep_down_projection: NULL route table or peer pointers");
  GemmDesc g = {};
  g.dtype = dtype;
  g.E = E_local; g.N = N; g.K = K;
  g.offsets = offsets_local;
  g.total_rows = capacity;
  g.rows_hint = rows_hint;
  g.a = hidden; g.a_rows = capacity; g.lda = ldh;
  g.b0 = weight;
  g.b_se = w_se; g.b_sn = w_sn;
  g.epilogue = FMOE_EPI_NONE;
  g.out_index = route;
  g.out_peers = back_ptrs;
  g.n_peers = world;
  g.peer_rows = back_rows;
  g.out = const_cast<int64_t*>(back_ptrs);   // never dereferenced as a matrix: rows go to out_peers[peer]
  g.out_dtype = dtype; g.ldo = ld_back;
  return launch_grouped_gemm(g, static_cast<cudaStream_t>(stream));
}
