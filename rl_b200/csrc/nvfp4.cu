// NVFP4 quantisation (sm_100a): blocks of 16 E2M1 values with one E4M3 scale per block and one fp32 scale per tensor, the
// 4-bit operand format of the fifth-generation tensor cores (tcgen05.mma kind::mxf4nvf4).
//   * fake_quant: quantise-dequantise in one pass (read 16 values, write 16 values of the same type), the operator that
//     quantisation-aware training puts in front of the linear layers (role of ModelOpt's quantizers behind
//     nemo_rl/modelopt/models/policy/workers/utils.py::quantize_model);
//   * quant: the real thing for export / weight hand-over: two values per byte (element 2i in the low nibble) + the block
//     scales.
// Every operation is written with explicit round-to-nearest intrinsics (the library is built with fast-math) in the order of
// the PyTorch statement in rl_b200/ops/nvfp4.py, so both produce the same bits.
// One thread owns one block of 16 values: 32 or 64 bytes in, the same out; the kernels are plain streaming passes.
#include "common.cuh"

#include <cuda_fp8.h>

namespace {
using namespace rlb;

__device__ __forceinline__ float e4m3_round(float x) {   // nearest representable E4M3 value of 0 <= x <= 448
  const __nv_fp8_storage_t s = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(s, __NV_E4M3)));
}

// index 0..7 of the nearest E2M1 magnitude; a tie goes to the even mantissa (0, 1, 2, 4)
__device__ __forceinline__ int e2m1_index(float m) {
  return (m > 0.25f) + (m > 0.7499999f) + (m > 1.25f) + (m > 1.7499999f) + (m > 2.5f) + (m > 3.4999998f) + (m > 5.0f);
}

__device__ __forceinline__ float e2m1_value(int i) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6
  return i < 4 ? 0.5f * static_cast<float>(i) : (i == 4 ? 2.f : (i == 5 ? 3.f : (i == 6 ? 4.f : 6.f)));
}

template <typename T>
__device__ __forceinline__ void load16(const T* p, float* v);
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    v[2 * i] = x.x, v[2 * i + 1] = x.y, v[8 + 2 * i] = y.x, v[8 + 2 * i + 1] = y.y;
  }
}
template <>
__device__ __forceinline__ void load16<float>(const float* p, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 x = *reinterpret_cast<const float4*>(p + 4 * i);
    v[4 * i] = x.x, v[4 * i + 1] = x.y, v[4 * i + 2] = x.z, v[4 * i + 3] = x.w;
  }
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const float* v);
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
  uint4 a, b;
  __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&a);
  __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    pa[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    pb[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
  }
  *reinterpret_cast<uint4*>(p) = a;
  *reinterpret_cast<uint4*>(p + 8) = b;
}
template <>
__device__ __forceinline__ void store16<float>(float* p, const float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(p + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// codes[i] = magnitude index | 8 for negative values; returns the block's E4M3 scale (as a float) through *sb
__device__ __forceinline__ void block_codes(const float* v, float s2, int* codes, float* sb_out, float* step_out) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float want = __fdiv_rn(__fmul_rn(amax, 0x1.555556p-3f), s2);   // fp32(1 / 6), as in the PyTorch statement
  const float sb = e4m3_round(fminf(want, 448.f));
  const float step = __fmul_rn(sb, s2);
  const float den = fmaxf(step, 1e-30f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float m = step > 0.f ? fminf(__fdiv_rn(fabsf(v[i]), den), 6.f) : 0.f;
    codes[i] = e2m1_index(m) | (v[i] < 0.f ? 8 : 0);
  }
  *sb_out = sb;
  *step_out = step;
}

// amax: one value per group of `rows_per_scale` rows (a tensor of its own, e.g. one expert's matrix)
template <typename T>
__global__ void __launch_bounds__(256) fake_quant_nvfp4_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                               const float* __restrict__ amax, long long rows_per_scale,
                                                               long long R, int blocks_per_row) {
  const long long b = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= R * blocks_per_row) return;
  const long long r = b / blocks_per_row;
  const float s2 = fmaxf(__fmul_rn(amax[r / rows_per_scale], 0x1.861862p-12f), 1e-30f);   // fp32(1 / (6 * 448))
  float v[16], sb, step;
  int codes[16];
  load16<T>(src + b * 16, v);
  block_codes(v, s2, codes, &sb, &step);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float q = e2m1_value(codes[i] & 7);
    v[i] = __fmul_rn((codes[i] & 8) ? -q : q, step);
  }
  store16<T>(dst + b * 16, v);
}

template <typename T>
__global__ void __launch_bounds__(256) quant_nvfp4_kernel(const T* __restrict__ src, unsigned char* __restrict__ packed,
                                                          __nv_fp8_storage_t* __restrict__ scales, const float* __restrict__ amax,
                                                          long long rows_per_scale, long long R, int blocks_per_row) {
  const long long b = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= R * blocks_per_row) return;
  const long long r = b / blocks_per_row;
  const float s2 = fmaxf(__fmul_rn(amax[r / rows_per_scale], 0x1.861862p-12f), 1e-30f);
  float v[16], sb, step;
  int codes[16];
  load16<T>(src + b * 16, v);
  block_codes(v, s2, codes, &sb, &step);
  unsigned long long out = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) out |= static_cast<unsigned long long>(codes[i]) << (4 * i);
  *reinterpret_cast<unsigned long long*>(packed + b * 8) = out;
  scales[b] = __nv_cvt_float_to_fp8(sb, __NV_SATFINITE, __NV_E4M3);
}
}  // namespace

// src / dst: [R, C] contiguous, C a multiple of 16, 16-byte aligned; dtype 0 = bf16, 1 = fp32; amax: ceil(R / rows_per_scale)
// floats on the device (the tensor-level maxima; the caller reduces them, nothing is read on the host).
RLB_API int rlb_fake_quant_nvfp4(const void* src, void* dst, const float* amax, long long rows_per_scale, long long R, int C,
                                 int dtype, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 16) || rows_per_scale <= 0 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -2;
  const long long n = R * (C / 16);
  const unsigned grid = static_cast<unsigned>((n + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    fake_quant_nvfp4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst),
                                                                 amax, rows_per_scale, R, C / 16);
  else
    fake_quant_nvfp4_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), static_cast<float*>(dst), amax, rows_per_scale, R, C / 16);
  return static_cast<int>(cudaGetLastError());
}

// packed: [R, C / 2] bytes; scales: [R, C / 16] E4M3 bytes.
RLB_API int rlb_quant_nvfp4(const void* src, void* packed, void* scales, const float* amax, long long rows_per_scale, long long R,
                            int C, int dtype, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 16) || rows_per_scale <= 0 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(packed)) & 15)) return -2;
  const long long n = R * (C / 16);
  const unsigned grid = static_cast<unsigned>((n + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    quant_nvfp4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), static_cast<unsigned char*>(packed),
                                                            static_cast<__nv_fp8_storage_t*>(scales), amax, rows_per_scale, R, C / 16);
  else
    quant_nvfp4_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), static_cast<unsigned char*>(packed),
                                                    static_cast<__nv_fp8_storage_t*>(scales), amax, rows_per_scale, R, C / 16);
  return static_cast<int>(cudaGetLastError());
}
