// FP8 weight quantisation for refit (sm_100a): bf16 -> e4m3 with
//   * 128x128 block scales (fp32 de-scale per block; optionally rounded up to a power of two), the format of
//     block-FP8 checkpoints and of `cast_tensor_to_fp8_blockwise`
//     (nemo_rl/models/generation/vllm/quantization/fp8.py:533-620), and
//   * MXFP8: 1x32 groups along the row with an E8M0 (power-of-two, biased by 127) scale byte per group
//     (the layout FlashInfer's sm_100 MXFP8 GEMM consumes, fp8.py:798-870).
// Both are one pass over the matrix in HBM: a CTA holds its block in registers between the amax reduction and the
// conversion, so the cost is one bf16 read + one byte write per element. Dequantisation kernels are provided for
// tests and for engines that keep bf16 compute.
#include "common.cuh"

#include <cuda_fp8.h>

namespace {
using namespace rlb;

constexpr float FP8_MAX = 448.f;

__device__ __forceinline__ float pow2_ceil_descale(float descale, unsigned char* e8m0) {
  // exponent = clamp(ceil(log2(descale)), -127, 127) + 127 as a byte; byte 0 stands for scale 1 (all-zero block)
  // ceil(log2(x)) from the float's own exponent: exact, unlike log2f near powers of two
  int ex = 0;
  const float mant = frexpf(descale, &ex);  // descale = mant * 2^ex, mant in [0.5, 1)
  float e = static_cast<float>(mant == 0.5f ? ex - 1 : ex);
  e = fminf(fmaxf(e, -127.f), 127.f) + 127.f;
  if (!(descale > 0.f)) e = 0.f;
  const unsigned char b = static_cast<unsigned char>(e);
  if (e8m0) *e8m0 = b;
  return b == 0 ? 1.f : exp2f(static_cast<float>(b) - 127.f);
}

// One CTA (256 threads) per 128x128 block; thread t handles row (t / 2), columns [(t % 2) * 64, +64).
__global__ void __launch_bounds__(256) quant_block128_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                                             __nv_fp8_storage_t* __restrict__ dst, long long ldd,
                                                             float* __restrict__ descale, int R, int C, int pow2,
                                                             float pad_abs) {
  __shared__ float red[32];
  const int br = blockIdx.y, bc = blockIdx.x;
  const int r = br * 128 + (threadIdx.x >> 1);
  const int c0 = bc * 128 + (threadIdx.x & 1) * 64;
  float v[64];
  float amax = 0.f;
  const bool row_ok = r < R;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int c = c0 + q * 8;
    if (row_ok && c + 8 <= C) {
      const uint4 x = *reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * lds + c);
      const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
      v[q * 8 + 0] = a0.x; v[q * 8 + 1] = a0.y; v[q * 8 + 2] = a1.x; v[q * 8 + 3] = a1.y;
      v[q * 8 + 4] = a2.x; v[q * 8 + 5] = a2.y; v[q * 8 + 6] = a3.x; v[q * 8 + 7] = a3.y;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[q * 8 + k] = (row_ok && c + k < C) ? __bfloat162float(src[static_cast<long long>(r) * lds + c + k]) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[q * 8 + k]));
  }
  // a ragged edge block is padded with the matrix's last element (it takes part in the block's amax)
  if ((br + 1) * 128 > R || (bc + 1) * 128 > C) amax = fmaxf(amax, pad_abs);
  amax = block_max(amax, red);
  float scale, ds;
  if (pow2) {
    ds = pow2_ceil_descale(amax / FP8_MAX, nullptr);
    scale = 1.f / ds;
  } else {
    scale = (amax == 0.f || isinf(amax)) ? 1.f : FP8_MAX / amax;
    ds = 1.f / scale;
  }
  if (threadIdx.x == 0) descale[static_cast<long long>(br) * gridDim.x + bc] = ds;
  if (!row_ok) return;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int c = c0 + q * 16;
    unsigned char b[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float y = fminf(fmaxf(v[q * 16 + k] * scale, -FP8_MAX), FP8_MAX);
      b[k] = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
    }
    if (c + 16 <= C && (ldd % 16) == 0) {
      *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * ldd + c) = *reinterpret_cast<const uint4*>(b);
    } else {
      for (int k = 0; k < 16; ++k)
        if (c + k < C) dst[static_cast<long long>(r) * ldd + c + k] = b[k];
    }
  }
}

// MXFP8: each thread quantises one 32-element group. C must be a multiple of 32.
__global__ void __launch_bounds__(256) quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                                          __nv_fp8_storage_t* __restrict__ dst, long long ldd,
                                                          unsigned char* __restrict__ scales, long long ldsc, int R,
                                                          int groups, int blocked, int R_pad) {
  // blocked: scales go straight into the layout the block-scaled MMA reads (one 512-byte atom per 128 rows x 128 columns,
  // byte (r % 32) * 16 + (r % 128 / 32) * 4 + g % 4); rows R..R_pad of the last atom row get scale byte 0.
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(blocked ? R_pad : R) * groups) return;
  const long long r = gid / groups;
  const int g = static_cast<int>(gid - r * groups);
  unsigned char* sc_out = blocked ? scales + ((r >> 7) * (groups >> 2) + (g >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3)
                                  : scales + r * ldsc + g;
  if (r >= R) {
    *sc_out = 0;
    return;
  }
  const __nv_bfloat16* p = src + r * lds + g * 32;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 x = *reinterpret_cast<const uint4*>(p + q * 8);
    const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
    v[q * 8 + 0] = a0.x; v[q * 8 + 1] = a0.y; v[q * 8 + 2] = a1.x; v[q * 8 + 3] = a1.y;
    v[q * 8 + 4] = a2.x; v[q * 8 + 5] = a2.y; v[q * 8 + 6] = a3.x; v[q * 8 + 7] = a3.y;
  }
#pragma unroll
  for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(v[k]));
  unsigned char e;
  const float ds = pow2_ceil_descale(amax / FP8_MAX, &e);
  const float scale = 1.f / ds;
  *sc_out = e;
  unsigned char b[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) b[k] = __nv_cvt_float_to_fp8(fminf(fmaxf(v[k] * scale, -FP8_MAX), FP8_MAX), __NV_SATFINITE, __NV_E4M3);
  uint4* o = reinterpret_cast<uint4*>(dst + r * ldd + g * 32);
  o[0] = reinterpret_cast<const uint4*>(b)[0];
  o[1] = reinterpret_cast<const uint4*>(b)[1];
}

__device__ __forceinline__ float fp8_to_float(unsigned char b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__global__ void dequant_block128_kernel(const __nv_fp8_storage_t* __restrict__ src, long long lds,
                                        const float* __restrict__ descale, int blocks_c, __nv_bfloat16* __restrict__ dst,
                                        long long ldd, int R, int C) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(R) * C) return;
  const long long r = i / C;
  const int c = static_cast<int>(i - r * C);
  dst[r * ldd + c] = __float2bfloat16(fp8_to_float(src[r * lds + c]) * descale[(r / 128) * blocks_c + c / 128]);
}

__global__ void dequant_mxfp8_kernel(const __nv_fp8_storage_t* __restrict__ src, long long lds,
                                     const unsigned char* __restrict__ scales, long long ldsc,
                                     __nv_bfloat16* __restrict__ dst, long long ldd, int R, int C) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(R) * C) return;
  const long long r = i / C;
  const int c = static_cast<int>(i - r * C);
  const unsigned char e = scales[r * ldsc + c / 32];
  dst[r * ldd + c] = __float2bfloat16(fp8_to_float(src[r * lds + c]) * (e == 0 ? 1.f : exp2f(static_cast<float>(e) - 127.f)));
}
}  // namespace

// descale: [ceil(R/128), ceil(C/128)] fp32. pad_abs = |src[R-1, C-1]| when the matrix has ragged edge blocks (the caller
// reads it once), else 0.
RLB_API int rlb_quant_fp8_block128(const void* src, long long lds, void* dst, long long ldd, float* descale, int R, int C,
                                   int pow2, float pad_abs, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if ((lds % 8) || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  dim3 grid((C + 127) / 128, (R + 127) / 128);
  quant_block128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), lds, static_cast<__nv_fp8_storage_t*>(dst), ldd, descale, R, C, pow2, pad_abs);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_quant_mxfp8(const void* src, long long lds, void* dst, long long ldd, void* scales, long long ldsc, int R,
                            int C, void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 32) || (lds % 8) || (ldd % 16) || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -2;
  const long long n = static_cast<long long>(R) * (C / 32);
  quant_mxfp8_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), lds, static_cast<__nv_fp8_storage_t*>(dst), ldd,
      static_cast<unsigned char*>(scales), ldsc, R, C / 32, 0, R);
  return static_cast<int>(cudaGetLastError());
}

// Same quantisation with the scales written in the blocked layout of the MXFP8 GEMM: `scales` holds
// ceil(R / 128) * (C / 128) atoms of 512 bytes. C must be a multiple of 128.
RLB_API int rlb_quant_mxfp8_blocked(const void* src, long long lds, void* dst, long long ldd, void* scales, int R, int C,
                                    void* stream) {
  if (R <= 0 || C <= 0) return 0;
  if ((C % 128) || (lds % 8) || (ldd % 16) || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -2;
  const int R_pad = (R + 127) / 128 * 128;
  const long long n = static_cast<long long>(R_pad) * (C / 32);
  quant_mxfp8_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), lds, static_cast<__nv_fp8_storage_t*>(dst), ldd,
      static_cast<unsigned char*>(scales), 0, R, C / 32, 1, R_pad);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_dequant_fp8_block128(const void* src, long long lds, const float* descale, void* dst, long long ldd, int R,
                                     int C, void* stream) {
  const long long n = static_cast<long long>(R) * C;
  if (n <= 0) return 0;
  dequant_block128_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_fp8_storage_t*>(src), lds, descale, (C + 127) / 128, static_cast<__nv_bfloat16*>(dst), ldd, R, C);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_dequant_mxfp8(const void* src, long long lds, const void* scales, long long ldsc, void* dst, long long ldd,
                              int R, int C, void* stream) {
  const long long n = static_cast<long long>(R) * C;
  if (n <= 0) return 0;
  dequant_mxfp8_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_fp8_storage_t*>(src), lds, static_cast<const unsigned char*>(scales), ldsc,
      static_cast<__nv_bfloat16*>(dst), ldd, R, C);
  return static_cast<int>(cudaGetLastError());
}
