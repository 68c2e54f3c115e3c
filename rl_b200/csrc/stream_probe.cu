// Read-bandwidth probe for the decode GEMMs' weight stream: the same TMA access pattern as gemm_skinny.cu (2-D boxes of
// [rows x 64] bf16 elements of a row-major [N, K] matrix, 128-byte swizzle, mbarrier ring, two CTAs per SM) with a consumer
// that only releases the stages. What this kernel reaches is the ceiling of any kernel that streams W this way; the gap
// between it and a GEMM's time is what the MMA issue, the epilogue and the prologue cost.
#include "common.cuh"

namespace {
using namespace rlb;

struct ProbeParams {
  int N, K, stages, kboxes, rows;
  int* status;
  unsigned long long* sink;
};

__global__ void __launch_bounds__(64, 2) stream_probe_kernel(const __grid_constant__ CUtensorMap tm, ProbeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int box_bytes = p.rows * 128;
  const int stage_bytes = box_bytes * p.kboxes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    abort_flag_s = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  const int tiles = p.N / p.rows;
  const int num_k = p.K / (64 * p.kboxes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    uint32_t stage = 0, phase = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      for (int kb = 0; kb < num_k; ++kb) {
        if (!mbar_wait(smem_u32(&empty[stage]), phase ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) return;
        const uint32_t bar = smem_u32(&full[stage]);
        mbar_arrive_expect_tx(bar, stage_bytes);
        for (int b = 0; b < p.kboxes; ++b)
          tma_load_2d(smem_u32(smem + stage * stage_bytes + b * box_bytes), &tm, bar, (kb * p.kboxes + b) * 64, t * p.rows);
        if (++stage == static_cast<uint32_t>(p.stages)) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    unsigned long long acc = 0;
    uint32_t stage = 0, phase = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      for (int kb = 0; kb < num_k; ++kb) {
        if (!mbar_wait(smem_u32(&full[stage]), phase, abort_flag, p.status, RLB_ERR_WAIT_FULL)) return;
        acc += *reinterpret_cast<volatile unsigned long long*>(smem + stage * stage_bytes);
        mbar_arrive(smem_u32(&empty[stage]));
        if (++stage == static_cast<uint32_t>(p.stages)) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (acc == 0x123456789abcdefull) *p.sink = acc;  // keeps the loads observable
  }
}
}  // namespace

// Streams W [N, K] (bf16, row pitch ldw elements) once. rows: 32, 64 or 128 per box; kboxes adjacent 64-element boxes per
// stage; grid <= 0: one CTA per row tile. Shared memory stages * kboxes * rows * 128 bytes must stay below 110 KB.
RLB_API int rlb_stream_probe(const void* W, long long ldw, int N, int K, int rows, int kboxes, int stages, int grid, void* sink,
                             int* status, void* stream) {
  if (N <= 0 || K <= 0 || N % rows || K % (64 * kboxes) || (rows != 32 && rows != 64 && rows != 128)) return -2;
  const int smem = stages * kboxes * rows * 128 + 1024;
  if (smem > 110 * 1024 || stages < 2) return -3;
  CUtensorMap tm;
  int rc = rlb_make_tmap_2d(&tm, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldw * 2, 64, rows, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  cudaError_t e = cudaFuncSetAttribute(stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int tiles = N / rows;
  if (grid <= 0 || grid > tiles) grid = tiles;
  ProbeParams p{N, K, stages, kboxes, rows, status, static_cast<unsigned long long*>(sink)};
  stream_probe_kernel<<<grid, 64, smem, static_cast<cudaStream_t>(stream)>>>(tm, p);
  return static_cast<int>(cudaGetLastError());
}
