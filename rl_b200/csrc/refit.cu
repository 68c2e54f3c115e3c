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
//
// Quantising form (refit_quant_kernel): the same push, but a work item is a run of 128 x 128 blocks of a linear weight.
// A CTA holds one block in registers between the amax reduction and the conversion and stores e4m3 bytes plus one fp32
// de-scale per block into the destination rank's FP8 arena (half the bytes of a bf16 push cross NVLink), and, for a
// destination on this GPU, the fp8-rounded bf16 values the bf16 GEMMs compute with: one read of the trainer's weights
// instead of copy + quantise + expand. Block-128 format of nemo_rl/models/generation/vllm/quantization/fp8.py:533-620.
#include "common.cuh"

#include <cuda_fp8.h>

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

struct RefitQDesc {
  const __nv_bfloat16* src;   // first element of the piece in the trainer's parameter
  unsigned char* dst_q;       // e4m3 destination of the piece (local or peer)
  float* dst_s;               // de-scale of the piece's first block (local or peer)
  __nv_bfloat16* dst_w;       // optional: fp8-rounded bf16 destination (null: not written)
  long long src_pitch;        // elements
  long long dst_pitch;        // elements (the e4m3 and the bf16 destination share the serving shape)
  int scale_pitch;            // de-scales per block row of the destination parameter
  int block_cols;             // 128-column blocks per block row of this piece
};
struct RefitQWork {
  int desc;
  int first_block;  // row-major over the piece's blocks
  int num_blocks;
  int pad;
};

// 256 threads; thread t owns row (t / 2) and 64 columns of the block. Pieces are whole blocks (checked by the host).
__global__ void __launch_bounds__(256) refit_quant_kernel(const RefitQDesc* __restrict__ descs,
                                                          const RefitQWork* __restrict__ work, int num_work) {
  __shared__ float red[32];
  using namespace rlb;
  const int lr = threadIdx.x >> 1, lc = (threadIdx.x & 1) * 64;
  for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
    const RefitQWork wk = work[w];
    const RefitQDesc d = descs[wk.desc];
    for (int b = wk.first_block; b < wk.first_block + wk.num_blocks; ++b) {
      const int br = b / d.block_cols, bc = b - br * d.block_cols;
      const long long r = br * 128LL + lr, c0 = bc * 128LL + lc;
      const __nv_bfloat16* sp = d.src + r * d.src_pitch + c0;
      float v[64];
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint4 x = *reinterpret_cast<const uint4*>(sp + q * 8);
        const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
        v[q * 8 + 0] = a0.x; v[q * 8 + 1] = a0.y; v[q * 8 + 2] = a1.x; v[q * 8 + 3] = a1.y;
        v[q * 8 + 4] = a2.x; v[q * 8 + 5] = a2.y; v[q * 8 + 6] = a3.x; v[q * 8 + 7] = a3.y;
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[q * 8 + k]));
      }
      amax = block_max(amax, red);
      const float scale = (amax == 0.f || isinf(amax)) ? 1.f : 448.f / amax;
      const float ds = 1.f / scale;
      if (threadIdx.x == 0) d.dst_s[static_cast<long long>(br) * d.scale_pitch + bc] = ds;
      unsigned char* qp = d.dst_q + r * d.dst_pitch + c0;
      __nv_bfloat16* wp = d.dst_w ? d.dst_w + r * d.dst_pitch + c0 : nullptr;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        unsigned char bytes[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float y = fminf(fmaxf(v[q * 16 + k] * scale, -448.f), 448.f);
          bytes[k] = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
        }
        *reinterpret_cast<uint4*>(qp + q * 16) = *reinterpret_cast<const uint4*>(bytes);
        if (wp) {
          __nv_bfloat16 o[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const __half_raw h = __nv_cvt_fp8_to_halfraw(bytes[k], __NV_E4M3);
            o[k] = __float2bfloat16(__half2float(*reinterpret_cast<const __half*>(&h)) * ds);
          }
          reinterpret_cast<uint4*>(wp + q * 16)[0] = reinterpret_cast<const uint4*>(o)[0];
          reinterpret_cast<uint4*>(wp + q * 16)[1] = reinterpret_cast<const uint4*>(o)[1];
        }
      }
    }
  }
}
}  // namespace

RLB_API int rlb_refit_qdesc_bytes() { return static_cast<int>(sizeof(RefitQDesc)); }
RLB_API int rlb_refit_qwork_bytes() { return static_cast<int>(sizeof(RefitQWork)); }

// Quantising push: descs / work prepared by the host (rl_b200/refit/synchronizer.py), every piece made of whole
// 128 x 128 blocks with 16-byte aligned rows on both sides.
RLB_API int rlb_refit_quant(const void* descs, const void* work, int num_work, int max_ctas, void* stream) {
  if (num_work <= 0) return 0;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms * 4;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid > num_work) grid = num_work;
  refit_quant_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const RefitQDesc*>(descs),
                                                                          static_cast<const RefitQWork*>(work), num_work);
  return static_cast<int>(cudaGetLastError());
}

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
