// Expert-parallel token dispatch / combine over NVLink peer memory (sm_100a).
//
// Every rank of an expert-parallel group owns a symmetric receive buffer laid out by local expert, each expert's
// region padded to a multiple of 128 rows (the layout the grouped GEMM consumes). After a tiny exchange of the routing
// histograms every rank can compute where each of its routed token copies lands on which rank, so dispatch is ONE kernel
// per rank that copies rows straight into the owners' buffers with P2P stores (one warp per row, 16-byte vectors) and
// records, next to every row, where it came from. The expert owner later returns each output row to the recorded
// (rank, slot) the same way. Both kernels end with a flag barrier between the ranks (bounded wait, status code on
// time-out), so no NCCL all-to-all, no host-side split sizes and no staging copies are involved. The NCCL
// `all_to_all_single` path (rl_b200/parallel/expert.py) is the twin.
//
// Reference counterpart: Megatron's alltoall / DeepEP token dispatchers selected by `moe_token_dispatcher_type`
// (nemo_rl/models/megatron/setup.py:888-1023).
#include "common.cuh"

namespace {
using namespace rlb;
constexpr int MAX_EP = 8;

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerBufs {
  unsigned char* rows[MAX_EP];   // destination row buffers
  int2* meta[MAX_EP];            // per destination row: (source rank, source slot); null when not recorded
  unsigned int* flags[MAX_EP];   // [2][MAX_EP] epoch words per rank; word `done` at index 16
};

// Grid barrier (atomic counter in this rank's flag block) followed by a flag barrier between ranks, run at the end of a
// push kernel: all my stores are visible everywhere before any peer proceeds.
__device__ void finish_and_barrier(const PeerBufs& pb, int rank, int world, int stage, unsigned int epoch,
                                   unsigned long long limit_ns, int* status) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  unsigned int* mine = pb.flags[rank];
  const unsigned int arrived = atomicAdd(mine + 16, 1u) + 1;
  if (arrived != gridDim.x) return;
  mine[16] = 0;
  __threadfence_system();
  for (int r = 0; r < world; ++r) st_release_sys(pb.flags[r] + stage * MAX_EP + rank, epoch);
  const unsigned long long t0 = globaltimer_ns();
  for (int r = 0; r < world; ++r) {
    while (static_cast<int>(ld_acquire_sys(mine + stage * MAX_EP + r) - epoch) < 0) {
      if (globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, RLB_ERR_WAIT_PEER);
        return;
      }
    }
  }
}

// One warp per row i: dst = rows[dst_rank[i]] + dst_row[i] * row_bytes, src = src_base + src_row[i] * src_pitch.
// Rows with dst_rank < 0 are skipped (dropped / padding entries).
__global__ void __launch_bounds__(256) push_rows_kernel(const unsigned char* __restrict__ src_base, long long src_pitch,
                                                        const int* __restrict__ src_row, const int* __restrict__ dst_rank,
                                                        const int* __restrict__ dst_row, int n, int row_bytes, PeerBufs pb,
                                                        int rank, int world, int record_meta, int stage, unsigned int epoch,
                                                        unsigned long long limit_ns, int* status, long long dst_capacity) {
  const int warps_per_cta = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = row_bytes / 16;
  for (int i = blockIdx.x * warps_per_cta + warp; i < n; i += gridDim.x * warps_per_cta) {
    const int r = dst_rank[i];
    if (r < 0) continue;
    const long long drow = dst_row[i];
    if (r >= world || drow < 0 || drow >= dst_capacity) {   // a store outside the peer's buffer is recorded and skipped
      if (lane == 0 && status) atomicCAS(status, 0, RLB_ERR_BOUNDS);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src_base + static_cast<long long>(src_row ? src_row[i] : i) * src_pitch);
    uint4* d = reinterpret_cast<uint4*>(pb.rows[r] + drow * row_bytes);
    for (int v0 = lane; v0 < vecs; v0 += 128) {  // four vectors in flight per lane
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) x[u] = s[v0 + u * 32];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) d[v0 + u * 32] = x[u];
    }
    if (record_meta && lane == 0) pb.meta[r][drow] = make_int2(rank, i);
  }
  finish_and_barrier(pb, rank, world, stage, epoch, limit_ns, status);
}

// Expert side: row j of `src` goes back to (meta[j].x, meta[j].y). `valid[j]` tells which rows hold a token of the
// current call (padding rows and rows beyond the received counts keep stale meta entries and are skipped).
__global__ void __launch_bounds__(256) return_rows_kernel(const unsigned char* __restrict__ src_base, long long src_pitch,
                                                          const int2* __restrict__ meta, const int* __restrict__ valid, int n,
                                                          int row_bytes, PeerBufs pb,
                                                          int rank, int world, int stage, unsigned int epoch,
                                                          unsigned long long limit_ns, int* status, long long dst_capacity) {
  const int warps_per_cta = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = row_bytes / 16;
  for (int j = blockIdx.x * warps_per_cta + warp; j < n; j += gridDim.x * warps_per_cta) {
    if (!valid[j]) continue;
    const int2 m = meta[j];
    if (m.x < 0 || m.x >= world || m.y < 0 || m.y >= dst_capacity) {   // a stale or corrupt return address: recorded, skipped
      if (lane == 0 && status) atomicCAS(status, 0, RLB_ERR_BOUNDS);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src_base + static_cast<long long>(j) * src_pitch);
    uint4* d = reinterpret_cast<uint4*>(pb.rows[m.x] + static_cast<long long>(m.y) * row_bytes);
    for (int v0 = lane; v0 < vecs; v0 += 128) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) x[u] = s[v0 + u * 32];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * 32 < vecs) d[v0 + u * 32] = x[u];
    }
  }
  finish_and_barrier(pb, rank, world, stage, epoch, limit_ns, status);
}

int grid_for(int n) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = (n + 7) / 8;
  if (grid > sms) grid = sms;   // one CTA per SM at most: every CTA must be resident for the closing barrier
  return grid < 1 ? 1 : grid;
}

void fill(PeerBufs& pb, void* const* row_ptrs, void* const* meta_ptrs, void* const* flag_ptrs, int world) {
  for (int r = 0; r < MAX_EP; ++r) {
    pb.rows[r] = r < world ? static_cast<unsigned char*>(row_ptrs[r]) : nullptr;
    pb.meta[r] = (r < world && meta_ptrs) ? static_cast<int2*>(meta_ptrs[r]) : nullptr;
    pb.flags[r] = r < world ? static_cast<unsigned int*>(flag_ptrs[r]) : nullptr;
  }
}
}  // namespace

// Copies row src_row[i] (or i when src_row is null) of `src` to row dst_row[i] of rank dst_rank[i]'s buffer, for
// i < n, then waits until every rank of the group has finished its own copies (flag stage `stage`, epoch `epoch`).
// flag_ptrs[r]: 32 zero-initialised uint32 words of symmetric memory per rank. row_bytes must be a multiple of 16.
RLB_API int rlb_moe_push_rows(const void* src, long long src_pitch_bytes, const int* src_row, const int* dst_rank,
                              const int* dst_row, int n, int row_bytes, void* const* row_ptrs, void* const* meta_ptrs,
                              void* const* flag_ptrs, int rank, int world, int stage, unsigned int epoch, double wait_limit_s,
                              int* status, long long dst_capacity_rows, void* stream) {
  if (world < 1 || world > MAX_EP || (row_bytes % 16) || (src_pitch_bytes % 16) || stage < 0 || stage > 1) return -2;
  PeerBufs pb;
  fill(pb, row_ptrs, meta_ptrs, flag_ptrs, world);
  const int grid = grid_for(n);
  void* args[] = {&src, &src_pitch_bytes, &src_row, &dst_rank, &dst_row, &n, &row_bytes, &pb, &rank, &world, nullptr, &stage, &epoch, nullptr, &status,
                  &dst_capacity_rows};
  int record = meta_ptrs != nullptr;
  unsigned long long limit = static_cast<unsigned long long>(wait_limit_s * 1e9);
  args[10] = &record;
  args[13] = &limit;
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(push_rows_kernel), dim3(grid), dim3(256), args, 0,
                                                      static_cast<cudaStream_t>(stream)));
}

// Returns row j of `src` (j < n) to rank meta[j].x, row meta[j].y of that rank's buffer, then barriers like above.
RLB_API int rlb_moe_return_rows(const void* src, long long src_pitch_bytes, const void* meta, const int* valid, int n, int row_bytes,
                                void* const* row_ptrs, void* const* flag_ptrs, int rank, int world, int stage, unsigned int epoch,
                                double wait_limit_s, int* status, long long dst_capacity_rows, void* stream) {
  if (world < 1 || world > MAX_EP || (row_bytes % 16) || (src_pitch_bytes % 16) || stage < 0 || stage > 1) return -2;
  PeerBufs pb;
  fill(pb, row_ptrs, nullptr, flag_ptrs, world);
  const int grid = grid_for(n);
  unsigned long long limit = static_cast<unsigned long long>(wait_limit_s * 1e9);
  void* args[] = {&src, &src_pitch_bytes, &meta, &valid, &n, &row_bytes, &pb, &rank, &world, &stage, &epoch, &limit, &status, &dst_capacity_rows};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(return_rows_kernel), dim3(grid), dim3(256), args, 0,
                                                      static_cast<cudaStream_t>(stream)));
}
