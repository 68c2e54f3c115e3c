// Refit re-shard copy (sm_100a): executes a batch of 2-D strided copies, each from this GPU's memory (a trainer
// parameter shard) to any GPU's memory (an engine rank's weight arena, local or peer-mapped over NVLink), in ONE
// launch. The host splits the copies into work items of at most WORK_VECS 16-byte vectors; CTAs take work items
// grid-stride and every thread keeps four independent vectors in flight, so thousands of small tensors (norms, biases)
// and a few huge ones (embeddings, MLP matrices) are balanced over the whole GPU without per-tensor launches.
// Only plain loads (local) and plain stores (local or peer) are used.
//
// Reference counterparts: the per-bucket CUDA-IPC hand-off and the packed NCCL broadcast of weights
// (nemo_rl/models/policy/utils.py:361-549, nemo_rl/utils/packed_tensor.py) and the nccl_reshard planner's send/recv
// lists (docs/design-docs/nccl-reshard-refit.md).
#include "common.cuh"

namespace {

struct RefitDesc {
  const unsigned char* src;
  unsigned char* dst;
  long long src_pitch;  // bytes
  long long dst_pitch;  // bytes
  int rows;
  int row_bytes;        // multiple of 16 for the vector path
};
struct RefitWork {
  int desc;
  int first_vec;  // index of the first 16-byte vector (row-major over rows x row_bytes/16), or first byte pair
  int num_vec;
  int scalar;     // 1: 2-byte granularity (unaligned tensors)
};

__global__ void __launch_bounds__(256) refit_copy_kernel(const RefitDesc* __restrict__ descs,
                                                         const RefitWork* __restrict__ work, int num_work) {
  for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
    const RefitWork wk = work[w];
    const RefitDesc d = descs[wk.desc];
    if (wk.scalar) {
      const int per_row = d.row_bytes / 2;
      for (int i = threadIdx.x; i < wk.num_vec; i += blockDim.x) {
        const int v = wk.first_vec + i;
        const int r = v / per_row, c = v - r * per_row;
        *reinterpret_cast<unsigned short*>(d.dst + r * d.dst_pitch + c * 2) =
            *reinterpret_cast<const unsigned short*>(d.src + r * d.src_pitch + c * 2);
      }
      continue;
    }
    const int per_row = d.row_bytes / 16;
    for (int i0 = threadIdx.x; i0 < wk.num_vec; i0 += blockDim.x * 4) {
      uint4 x[4];
      long long doff[4];
      bool live[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        live[u] = i < wk.num_vec;
        const int v = wk.first_vec + (live[u] ? i : 0);
        const int r = v / per_row, c = v - r * per_row;
        doff[u] = r * d.dst_pitch + c * 16LL;
        if (live[u]) x[u] = *reinterpret_cast<const uint4*>(d.src + r * d.src_pitch + c * 16LL);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (live[u]) *reinterpret_cast<uint4*>(d.dst + doff[u]) = x[u];
    }
  }
}
}  // namespace

RLB_API int rlb_refit_desc_bytes() { return static_cast<int>(sizeof(RefitDesc)); }
RLB_API int rlb_refit_work_bytes() { return static_cast<int>(sizeof(RefitWork)); }

// descs / work: device arrays prepared by the host (see rl_b200/refit/synchronizer.py).
RLB_API int rlb_refit_copy(const void* descs, const void* work, int num_work, int max_ctas, void* stream) {
  if (num_work <= 0) return 0;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * 4;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid > num_work) grid = num_work;
  refit_copy_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const RefitDesc*>(descs),
                                                                         static_cast<const RefitWork*>(work), num_work);
  return static_cast<int>(cudaGetLastError());
}
