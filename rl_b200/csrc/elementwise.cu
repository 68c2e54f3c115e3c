// Memory-bound transformer kernels for sm_100a: RMSNorm, RoPE, SwiGLU, embedding, fused AdamW with a
// split fp32 master (bf16 + 16 low bits), gradient-norm partials, and the ClippedPG loss.
// All of them move 16 bytes per thread per access and keep the arithmetic in fp32.
//
// They stand in for the HF-eager / Transformer-Engine fused modules of the reference
// (nemo_rl/models/megatron/setup.py:1103-1110), torch.optim.AdamW
// (examples/configs/grpo_math_1B.yaml:344-350) and the torch-eager ClippedPGLossFn
// (nemo_rl/algorithms/loss/loss_functions.py:374-788).
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

struct alignas(16) BF8 {
  uint32_t w[4];
};
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const BF8 v = *reinterpret_cast<const BF8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(v.w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  BF8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<BF8*>(p) = v;
}

// ------------------------------------------------------------------ RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w ; optional residual: h = x + res is normalised and written back
// to `res_out` (the new residual stream). One CTA per row; d must be a multiple of 8.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out,
                                   int d, long long x_stride, long long y_stride, float eps) {
  pdl_sync();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  const __nv_bfloat16* rr = res ? res + row * static_cast<long long>(d) : nullptr;
  __nv_bfloat16* ro = res_out ? res_out + row * static_cast<long long>(d) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    float f[8];
    load8(xr + i, f);
    if (rr) {
      float g[8];
      load8(rr + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      // the normalised value must be the bf16-rounded residual stream, as a separate add would give
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16(f[j]));
      store8(ro + i, f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
  const __nv_bfloat16* src = rr ? ro : xr;
  __nv_bfloat16* yr = y + row * y_stride;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    float f[8], g[8];
    load8(src + i, f);
    load8(w + i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
    store8(yr + i, f);
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)); dw partial per CTA (rows strided over the grid).
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                                   int d, long long x_stride, long long dy_stride, int add_to_dx) {
  __shared__ float red[32];
  // Each thread owns fixed column groups, so the dw partial lives in registers (d <= 8 * 8 * blockDim).
  constexpr int MAXV = 8;
  float dwacc[MAXV][8];
#pragma unroll
  for (int a = 0; a < MAXV; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[a][j] = 0.f;

  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * x_stride;
    const __nv_bfloat16* dyr = dy + row * dy_stride;
    const float rs = rstd[row];
    float dot = 0.f;
    {
      int a = 0;
      for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8, ++a) {
        float fx[8], fd[8], fw[8];
        load8(xr + i, fx);
        load8(dyr + i, fd);
        load8(w + i, fw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += fd[j] * fw[j] * fx[j];
          if (a < MAXV) dwacc[a][j] += fd[j] * fx[j] * rs;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rs * rs / d;
    __nv_bfloat16* dxr = dx + row * static_cast<long long>(d);
    for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
      float fx[8], fd[8], fw[8], o[8];
      load8(xr + i, fx);
      load8(dyr + i, fd);
      load8(w + i, fw);
      if (add_to_dx) load8(dxr + i, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = rs * (fd[j] * fw[j] - fx[j] * c);
        o[j] = add_to_dx ? o[j] + v : v;
      }
      store8(dxr + i, o);
    }
  }
  int a = 0;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8, ++a) {
    if (a < MAXV) {
      float* p = dw_partial + static_cast<long long>(blockIdx.x) * d + i;
      *reinterpret_cast<float4*>(p) = make_float4(dwacc[a][0], dwacc[a][1], dwacc[a][2], dwacc[a][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dwacc[a][4], dwacc[a][5], dwacc[a][6], dwacc[a][7]);
    }
  }
}

// Column sums of a [parts, d] fp32 matrix, added into (or written to) a gradient buffer.
__global__ void colsum_kernel(const float* __restrict__ partial, int parts, int d, float* __restrict__ out_f32,
                              __nv_bfloat16* __restrict__ out_bf16, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<long long>(p) * d + c];
  if (out_f32) out_f32[c] = accumulate ? out_f32[c] + s : s;
  if (out_bf16) out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + s : s);
}

// ------------------------------------------------------------------ RoPE (HF rotate_half convention)
// In place on `heads` consecutive heads of width D starting at `x` in each row. sign=+1 forward,
// -1 backward (the inverse rotation, which is the transpose). One warp per (row, head).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ inv_freq, long long rows, int heads, int D,
                            long long row_stride, float sign) {
  pdl_sync();
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const long long row = wid / heads;
  const int head = static_cast<int>(wid - row * heads);
  __nv_bfloat16* p = x + row * row_stride + static_cast<long long>(head) * D;
  const float ps = static_cast<float>(pos[row]);
  const int half = D >> 1;
  for (int i = lane * 2; i < half; i += 64) {
    const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i));
    const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i + half));
    float s0, c0, s1, c1;
    sincosf(ps * inv_freq[i], &s0, &c0);
    sincosf(ps * inv_freq[i + 1], &s1, &c1);
    s0 *= sign;
    s1 *= sign;
    *reinterpret_cast<uint32_t*>(p + i) = pack_bf16x2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
    *reinterpret_cast<uint32_t*>(p + i + half) = pack_bf16x2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
  }
}

// Per-head RMSNorm (Qwen3 q_norm / k_norm): rows x heads vectors of width D (<= 256, multiple of 8
// and of 64... one warp per vector, D/32 elements per lane handled as bf16x2 pairs).
__global__ void head_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                        long long rows, int heads, int D, long long x_stride,
                                        long long y_stride, float eps) {
  pdl_sync();
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const long long row = wid / heads;
  const int head = static_cast<int>(wid - row * heads);
  const __nv_bfloat16* p = x + row * x_stride + static_cast<long long>(head) * D;
  __nv_bfloat16* q = y + row * y_stride + static_cast<long long>(head) * D;
  float ss = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i));
    ss += v.x * v.x + v.y * v.y;
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / D + eps);
  if (rstd_out && lane == 0) rstd_out[wid] = rs;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + i));
    *reinterpret_cast<uint32_t*>(q + i) = pack_bf16x2(v.x * rs * g.x, v.y * rs * g.y);
  }
}

__global__ void head_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_accum,
                                        long long rows, int heads, int D, long long x_stride,
                                        long long dy_stride, long long dx_stride) {
  // dw is accumulated with atomics into a [D] fp32 buffer (D is tiny: 128).
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const long long row = wid / heads;
  const int head = static_cast<int>(wid - row * heads);
  const __nv_bfloat16* px = x + row * x_stride + static_cast<long long>(head) * D;
  const __nv_bfloat16* pd = dy + row * dy_stride + static_cast<long long>(head) * D;
  __nv_bfloat16* po = dx + row * dx_stride + static_cast<long long>(head) * D;
  const float rs = rstd[wid];
  float dot = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(px + i));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + i));
    const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + i));
    dot += d.x * g.x * v.x + d.y * g.y * v.y;
    atomicAdd(dw_accum + i, d.x * v.x * rs);
    atomicAdd(dw_accum + i + 1, d.y * v.y * rs);
  }
  dot = warp_sum(dot);
  const float c = dot * rs * rs / D;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(px + i));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + i));
    const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + i));
    *reinterpret_cast<uint32_t*>(po + i) = pack_bf16x2(rs * (d.x * g.x - v.x * c), rs * (d.y * g.y - v.y * c));
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu: [rows, 2F] (gate | up). y[rows, F] = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y,
                                  long long rows, int F) {
  pdl_sync();
  const long long vecs_per_row = F / 8;
  const long long total = rows * vecs_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = v / vecs_per_row;
    const int c = static_cast<int>(v - row * vecs_per_row) * 8;
    float g[8], u[8], o[8];
    load8(gu + row * 2 * F + c, g);
    load8(gu + row * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(y + row * F + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const long long vecs_per_row = F / 8;
  const long long total = rows * vecs_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = v / vecs_per_row;
    const int c = static_cast<int>(v - row * vecs_per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * 2 * F + c, g);
    load8(gu + row * 2 * F + F + c, u);
    load8(dy + row * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
      du[j] = d[j] * silu;
    }
    store8(dgu + row * 2 * F + c, dg);
    store8(dgu + row * 2 * F + F + c, du);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long rows, int d, int vocab) {
  pdl_sync();
  const long long vecs_per_row = d / 8;
  const long long total = rows * vecs_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = v / vecs_per_row;
    const int c = static_cast<int>(v - row * vecs_per_row) * 8;
    int id = ids[row];
    BF8 val;
    if (id < 0 || id >= vocab) {
      val.w[0] = val.w[1] = val.w[2] = val.w[3] = 0u;
    } else {
      val = *reinterpret_cast<const BF8*>(table + static_cast<long long>(id) * d + c);
    }
    *reinterpret_cast<BF8*>(out + row * d + c) = val;
  }
}
// Scatter-add of output gradients into an fp32 embedding gradient.
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dtable, long long rows, int d, int vocab) {
  const long long vecs_per_row = d / 8;
  const long long total = rows * vecs_per_row;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = v / vecs_per_row;
    const int c = static_cast<int>(v - row * vecs_per_row) * 8;
    const int id = ids[row];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    load8(dy + row * d + c, f);
    float* dst = dtable + static_cast<long long>(id) * d + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ------------------------------------------------------------------ AdamW
// The fp32 master weight is stored as the bf16 parameter (the tensor the GEMMs read) plus a signed 16-bit
// remainder: master_bits = (bf16_bits << 16) + lo. The bf16 half is the master rounded to nearest with ties
// away from zero, which keeps the remainder inside [-32768, 32767] for every input, so the pair restores
// the fp32 value exactly at 4 bytes per parameter instead of 6.
__device__ __forceinline__ float master_join(__nv_bfloat16 hi, int16_t lo) {
  const uint32_t bits = (static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16) + static_cast<uint32_t>(static_cast<int32_t>(lo));
  return __uint_as_float(bits);
}
__device__ __forceinline__ void master_split(float v, __nv_bfloat16& hi, int16_t& lo) {
  const uint32_t bits = __float_as_uint(v);
  const uint32_t hb = (bits + 0x8000u) & 0xFFFF0000u;
  hi = __ushort_as_bfloat16(static_cast<unsigned short>(hb >> 16));
  lo = static_cast<int16_t>(static_cast<int32_t>(bits - hb));
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^step
};

template <typename GradT>
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, int16_t* __restrict__ p_lo, float* __restrict__ p32,
                             const GradT* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             long long n, AdamArgs a, const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float w = p32 ? p32[i] : master_join(p[i], p_lo[i]);
    const float grad = static_cast<float>(g[i]) * gs;
    const float mi = a.beta1 * m[i] + (1.f - a.beta1) * grad;
    const float vi = a.beta2 * v[i] + (1.f - a.beta2) * grad * grad;
    m[i] = mi;
    v[i] = vi;
    w *= (1.f - a.lr * a.weight_decay);
    w -= a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
    if (p32) {
      p32[i] = w;
      if (p) p[i] = __float2bfloat16_rn(w);
    } else {
      __nv_bfloat16 hi;
      int16_t lo;
      master_split(w, hi, lo);
      p[i] = hi;
      p_lo[i] = lo;
    }
  }
}

template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = static_cast<float>(x[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// scale = min(1, max_norm / (sqrt(sumsq) + 1e-6)) * extra ; also stores the norm.
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm, float extra,
                                  float* __restrict__ scale_out, float* __restrict__ norm_out) {
  const float norm = sqrtf(*sumsq);
  if (norm_out) *norm_out = norm;
  float s = 1.f;
  if (max_norm > 0.f) s = fminf(1.f, max_norm / (norm + 1e-6f));
  *scale_out = s * extra;
}

// ------------------------------------------------------------------ ClippedPG loss
// One pass over T tokens: per-token loss terms, their analytic gradient w.r.t. the current
// log-probability, and every metric partial sum. Slots of `sums`:
//  0 actor loss numerator (sum of w_is * clip_loss * mask)   1 kl numerator
//  2 sum ratio*mask   3 sum clamped ratio*mask   4 sum exp(|gen-prev|)*mask (token_mult_prob_error)
//  5 sum mask   6 gen_kl_error numerator   7 policy_kl_error numerator   8 sum w_is*mask
//  9 approx entropy numerator (-sum curr*mask... with IS weight)   10 ratio min  11 ratio max
//  12 clamped ratio min   13 clamped ratio max   14 js_divergence numerator  15 tokens whose IS weight left the truncation bounds
struct PGArgs {
  float eps_lo, eps_hi, dual_c;  // dual_c <= 0: no dual clip
  float kl_beta;
  int kl_type;  // 1,2,3
  float kl_in_clamp, kl_out_clamp;
  int use_is;        // importance-sampling correction
  int tis_type;      // 0 none, 1 tis (clamp max), 2 icepop (zero outside [min,max])
  float tis_max, tis_min;
  int force_on_policy;
  int use_cispo;
  int on_policy_kl_approx;
  float inv_norm;    // 1 / (global valid tokens + 1e-8)
};

__global__ void clipped_pg_kernel(const float* __restrict__ curr, const float* __restrict__ prev,
                                  const float* __restrict__ gen, const float* __restrict__ ref,
                                  const float* __restrict__ adv, const float* __restrict__ mask, long long T,
                                  PGArgs a, float* __restrict__ sums, float* __restrict__ dcurr) {
  __shared__ float red[32];
  float acc[10];
#pragma unroll
  for (int i = 0; i < 10; ++i) acc[i] = 0.f;
  float js = 0.f, nclip = 0.f, oob = 0.f;
  float rmin = INFINITY, rmax = -INFINITY, cmin = INFINITY, cmax = -INFINITY;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < T;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float mk = mask[i];
    const float c = curr[i];
    const float pv = a.force_on_policy ? c : prev[i];
    const float gn = gen ? gen[i] : pv;
    const float A = adv[i];
    float grad = 0.f;
    // KL penalty against the reference policy
    float kl = 0.f;
    if (a.kl_beta != 0.f && ref) {
      float logr = ref[i] - c;
      const bool inside = fabsf(logr) <= a.kl_in_clamp;  // same test as `logr == clamp(logr)`
      logr = fminf(fmaxf(logr, -a.kl_in_clamp), a.kl_in_clamp);
      float dkl_dc;  // d kl / d curr through logr (zero where the input clamp is active)
      if (a.kl_type == 1) {
        kl = -logr;
        dkl_dc = 1.f;
      } else if (a.kl_type == 2) {
        kl = 0.5f * logr * logr;
        dkl_dc = -logr;
      } else {
        const float e = __expf(logr);
        kl = e - 1.f - logr;
        dkl_dc = -(e - 1.f);
      }
      if (!inside) dkl_dc = 0.f;
      float wkl = 1.f;  // exp(curr - curr.detach()) = 1 in value, gradient kl * 1
      if (a.on_policy_kl_approx) wkl = __expf(c - gn);
      if (!isfinite(wkl)) wkl = 0.f;  // nan_to_num(nan = 0, +-inf = 0) on the weight
      // product rule; d wkl / d curr = wkl in both cases, except where the input clamp is active: there the weight is
      // detached, so the clamp suppresses the score-function term as well
      const float dw_dc = inside ? wkl : 0.f;
      float klw = kl * wkl;
      float dklw = dkl_dc * wkl + kl * dw_dc;
      if (isnan(klw)) {
        klw = 0.f;
        dklw = 0.f;
      }
      if (fabsf(klw) > a.kl_out_clamp) {
        klw = fminf(fmaxf(klw, -a.kl_out_clamp), a.kl_out_clamp);
        dklw = 0.f;
      }
      kl = klw;
      grad += a.kl_beta * dklw;
    }
    // ratio and clipped surrogate
    const float ratio = __expf(c - pv);
    const float rc = fminf(fmaxf(ratio, 1.f - a.eps_lo), 1.f + a.eps_hi);
    float loss, dloss;
    if (a.use_cispo) {
      loss = -A * rc * c;
      dloss = -A * rc;
    } else {
      const float l1 = -A * ratio, l2 = -A * rc;
      const bool clipped_active = l2 > l1;  // max picks the clamped branch: no gradient
      loss = clipped_active ? l2 : l1;
      dloss = clipped_active ? 0.f : -A * ratio;
      if (clipped_active) nclip += mk;
      if (a.dual_c > 0.f && A < 0.f) {
        const float l3 = -A * a.dual_c;
        if (l3 < loss) {
          loss = l3;
          dloss = 0.f;
        }
      }
    }
    // importance-sampling weight between trainer and generator probabilities (a constant w.r.t. curr)
    float wis = __expf(pv - gn);
    if (isnan(wis)) wis = 0.f;
    float wis_used = 1.f;
    if (a.use_is) {
      wis_used = wis;
      if (a.tis_type != 0 && (wis > a.tis_max || wis < a.tis_min)) oob += mk;
      if (a.tis_type == 1) wis_used = fminf(fmaxf(wis, a.tis_min), a.tis_max);
      else if (a.tis_type == 2) wis_used = (wis >= a.tis_min && wis <= a.tis_max) ? wis : 0.f;
    }
    grad += wis_used * dloss;
    if (dcurr) dcurr[i] = grad * mk * a.inv_norm;

    acc[0] += wis_used * loss * mk;
    acc[1] += kl * mk;
    acc[2] += ratio * mk;
    acc[3] += rc * mk;
    acc[4] += __expf(fabsf(gn - pv)) * mk;
    acc[5] += mk;
    {
      // gen_kl_error: KL(gen || train) estimated with logr = prev - gen; policy_kl_error: the reverse.
      const float d = pv - gn;
      float gk, pk;
      if (a.kl_type == 1) {
        gk = -d;
        pk = d;
      } else if (a.kl_type == 2) {
        gk = 0.5f * d * d;
        pk = gk;
      } else {
        gk = __expf(d) - 1.f - d;
        pk = __expf(-d) - 1.f + d;
      }
      acc[6] += gk * mk;
      acc[7] += pk * mk;
      // Jensen-Shannon: M = (P_train + P_gen) / 2, JSD = (KL(P_train||M) + KL(P_gen||M)) / 2, k3 estimates
      const float lm = __logf(0.5f * __expf(pv) + 0.5f * __expf(gn));
      const float a1 = pv - lm, a2 = gn - lm;
      js += 0.5f * ((__expf(a1) - 1.f - a1) + (__expf(a2) - 1.f - a2)) * mk;
    }
    acc[8] += wis * mk;
    acc[9] += -(__expf(c - gn) * c) * mk;
    if (mk > 0.f) {
      rmin = fminf(rmin, ratio);
      rmax = fmaxf(rmax, ratio);
      cmin = fminf(cmin, rc);
      cmax = fmaxf(cmax, rc);
    }
  }
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const float s = block_sum(acc[i], red);
    if (threadIdx.x == 0) atomicAdd(sums + i, s);
  }
  {
    const float s = block_sum(js, red);
    if (threadIdx.x == 0) atomicAdd(sums + 14, s);
    (void)nclip;
    const float s2 = block_sum(oob, red);
    if (threadIdx.x == 0) atomicAdd(sums + 15, s2);
  }
  // min/max via integer atomics on non-negative floats (ratios are > 0)
  rmin = -block_max(-rmin, red);
  rmax = block_max(rmax, red);
  cmin = -block_max(-cmin, red);
  cmax = block_max(cmax, red);
  if (threadIdx.x == 0) {
    if (isfinite(rmin)) atomicMin(reinterpret_cast<int*>(sums + 10), __float_as_int(rmin));
    if (isfinite(rmax)) atomicMax(reinterpret_cast<int*>(sums + 11), __float_as_int(rmax));
    if (isfinite(cmin)) atomicMin(reinterpret_cast<int*>(sums + 12), __float_as_int(cmin));
    if (isfinite(cmax)) atomicMax(reinterpret_cast<int*>(sums + 13), __float_as_int(cmax));
  }
}

__global__ void pg_init_sums_kernel(float* sums) {
  const int i = threadIdx.x;
  if (i < 16) {
    float v = 0.f;
    if (i == 10 || i == 12) v = 3.0e38f;  // running minima start high
    sums[i] = v;
  }
}

// ------------------------------------------------------------------ misc
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16_rn(x[i]);
}
// y = a + b (bf16), the residual add
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float fa[8], fb[8];
    load8(a + i * 8, fa);
    load8(b + i * 8, fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) fa[j] += fb[j];
    store8(y + i * 8, fa);
  }
}

inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}
inline int rms_threads(int d) {
  int t = d / 8;
  if (t > 512) t = 512;
  t = (t + 31) / 32 * 32;
  if (t < 32) t = 32;
  return t;
}

}  // namespace

#define S(stream) static_cast<cudaStream_t>(stream)
#define BF(p) reinterpret_cast<__nv_bfloat16*>(p)
#define CBF(p) reinterpret_cast<const __nv_bfloat16*>(p)

RLB_API int rlb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                            long long rows, int d, long long x_stride, long long y_stride, float eps,
                            void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 || x_stride % 8 || y_stride % 8) return -2;
  rlb_launch_pdl(rmsnorm_fwd_kernel, dim3(static_cast<unsigned>(rows)), dim3(rms_threads(d)), 0, S(stream), 
      CBF(x), CBF(res), CBF(w), BF(y), BF(res_out), rstd, d, x_stride, y_stride, eps);
  return static_cast<int>(cudaGetLastError());
}

// Number of CTAs (= rows of the dw partial buffer) the backward uses.
RLB_API int rlb_rmsnorm_bwd_parts(long long rows) { return static_cast<int>(rows < 296 ? rows : 296); }

// dw_partial: scratch of rlb_rmsnorm_bwd_parts(rows) * d floats. The column sums are written (or
// added) to dw_f32 / dw_bf16, whichever is non-null.
RLB_API int rlb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                            float* dw_partial, float* dw_f32, void* dw_bf16, int dw_accumulate, long long rows,
                            int d, long long x_stride, long long dy_stride, int add_to_dx, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 || x_stride % 8 || dy_stride % 8) return -2;
  const int threads = rms_threads(d);
  if (d > threads * 8 * 8) return -4;
  const int parts = rlb_rmsnorm_bwd_parts(rows);
  rmsnorm_bwd_kernel<<<parts, threads, 0, S(stream)>>>(CBF(dy), CBF(x), CBF(w), rstd, BF(dx), dw_partial,
                                                       static_cast<int>(rows), d, x_stride, dy_stride, add_to_dx);
  colsum_kernel<<<(d + 255) / 256, 256, 0, S(stream)>>>(dw_partial, parts, d, dw_f32, BF(dw_bf16), dw_accumulate);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_rope(void* x, const int* pos, const float* inv_freq, long long rows, int heads, int D,
                     long long row_stride, int backward, void* stream) {
  if (rows <= 0) return 0;
  if (D % 4) return -2;
  const long long warps = rows * heads;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  rlb_launch_pdl(rope_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, S(stream), BF(x), pos, inv_freq, rows, heads, D,
                                                                         row_stride, backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_head_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int heads,
                                 int D, long long x_stride, long long y_stride, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (D % 2) return -2;
  const long long blocks = (rows * heads * 32 + 255) / 256;
  rlb_launch_pdl(head_rmsnorm_fwd_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, S(stream), CBF(x), CBF(w), BF(y), rstd, rows,
                                                                                 heads, D, x_stride, y_stride, eps);
  return static_cast<int>(cudaGetLastError());
}
RLB_API int rlb_head_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                 float* dw_accum, long long rows, int heads, int D, long long x_stride,
                                 long long dy_stride, long long dx_stride, void* stream) {
  if (rows <= 0) return 0;
  const long long blocks = (rows * heads * 32 + 255) / 256;
  head_rmsnorm_bwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, S(stream)>>>(
      CBF(dy), CBF(x), CBF(w), rstd, BF(dx), dw_accum, rows, heads, D, x_stride, dy_stride, dx_stride);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_swiglu_fwd(const void* gu, void* y, long long rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  rlb_launch_pdl(swiglu_fwd_kernel, dim3(grid_for(rows * (F / 8), 256)), dim3(256), 0, S(stream), CBF(gu), BF(y), rows, F);
  return static_cast<int>(cudaGetLastError());
}
RLB_API int rlb_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  swiglu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, S(stream)>>>(CBF(dy), CBF(gu), BF(dgu), rows, F);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_embedding_fwd(const int* ids, const void* table, void* out, long long rows, int d, int vocab,
                              void* stream) {
  if (rows <= 0) return 0;
  if (d % 8) return -2;
  rlb_launch_pdl(embedding_fwd_kernel, dim3(grid_for(rows * (d / 8), 256)), dim3(256), 0, S(stream), ids, CBF(table), BF(out), rows, d,
                                                                             vocab);
  return static_cast<int>(cudaGetLastError());
}
RLB_API int rlb_embedding_bwd(const int* ids, const void* dy, float* dtable, long long rows, int d, int vocab,
                              void* stream) {
  if (rows <= 0) return 0;
  if (d % 8) return -2;
  embedding_bwd_kernel<<<grid_for(rows * (d / 8), 256), 256, 0, S(stream)>>>(ids, CBF(dy), dtable, rows, d, vocab);
  return static_cast<int>(cudaGetLastError());
}

// AdamW over a flat shard. Master weight either fp32 (`p32`, with an optional bf16 copy `p`) or the
// split form (`p` bf16 + `p_lo` int16, p32 null). grad_is_bf16 selects the gradient type.
// grad_scale: device scalar multiplied into every gradient (clip coefficient / loss scale), or null.
RLB_API int rlb_adamw(void* p, void* p_lo, float* p32, const void* g, int grad_is_bf16, float* m, float* v,
                      long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                      const float* grad_scale, void* stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, static_cast<float>(step)),
             1.f - powf(beta2, static_cast<float>(step))};
  const int grid = grid_for(n, 256, 148 * 8);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(BF(p), reinterpret_cast<int16_t*>(p_lo), p32, CBF(g), m,
                                                              v, n, a, grad_scale);
  else
    adamw_kernel<float><<<grid, 256, 0, S(stream)>>>(BF(p), reinterpret_cast<int16_t*>(p_lo), p32,
                                                      reinterpret_cast<const float*>(g), m, v, n, a, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

// out += sum(x^2). `out` is a device float the caller zeroes.
RLB_API int rlb_sumsq(const void* x, int is_bf16, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 256, 148 * 4);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, S(stream)>>>(CBF(x), n, out);
  else sumsq_kernel<float><<<grid, 256, 0, S(stream)>>>(reinterpret_cast<const float*>(x), n, out);
  return static_cast<int>(cudaGetLastError());
}
RLB_API int rlb_clip_scale(const float* sumsq, float max_norm, float extra, float* scale_out, float* norm_out,
                           void* stream) {
  clip_scale_kernel<<<1, 1, 0, S(stream)>>>(sumsq, max_norm, extra, scale_out, norm_out);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_clipped_pg(const float* curr, const float* prev, const float* gen, const float* ref,
                           const float* adv, const float* mask, long long T, float eps_lo, float eps_hi,
                           float dual_c, float kl_beta, int kl_type, float kl_in_clamp, float kl_out_clamp,
                           int use_is, int tis_type, float tis_max, float tis_min, int force_on_policy,
                           int use_cispo, int on_policy_kl_approx, float inv_norm, float* sums, float* dcurr,
                           void* stream) {
  PGArgs a{eps_lo, eps_hi, dual_c, kl_beta, kl_type, kl_in_clamp, kl_out_clamp, use_is, tis_type, tis_max,
           tis_min, force_on_policy, use_cispo, on_policy_kl_approx, inv_norm};
  pg_init_sums_kernel<<<1, 32, 0, S(stream)>>>(sums);
  if (T > 0)
    clipped_pg_kernel<<<grid_for(T, 256, 148 * 2), 256, 0, S(stream)>>>(curr, prev, gen, ref, adv, mask, T, a, sums,
                                                                        dcurr);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_cast_f32_bf16(const float* x, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, S(stream)>>>(x, BF(y), n);
  return static_cast<int>(cudaGetLastError());
}
RLB_API int rlb_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, S(stream)>>>(CBF(a), CBF(b), BF(y), n / 8);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ RMSNorm backward without device allocation
// See no_alloc.h for who this is for and what it costs. The scratch that rlb_rmsnorm_bwd takes from its caller is a
// fixed array in the library image here. In host code the array's name is only a host-side handle, not a device
// address, so the address the kernels receive is looked up once per device with cudaGetSymbolAddress.
#include "no_alloc.h"

namespace {
static __device__ __align__(256) float g_rmsnorm_static_scratch[RLB_RMSNORM_STATIC_MAX_PARTS * RLB_RMSNORM_STATIC_MAX_D];
constexpr int kMaxDevices = 64;
float* g_rmsnorm_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device, resolved on first use there.
int rmsnorm_static_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return RLB_STATIC_ERR_NO_SYMBOL;
  if (!g_rmsnorm_static_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_static_scratch);
    if (e != cudaSuccess || !p) return e != cudaSuccess ? static_cast<int>(e) : RLB_STATIC_ERR_NO_SYMBOL;
    g_rmsnorm_static_ptr[dev] = p;
  }
  *out = g_rmsnorm_static_ptr[dev];
  return 0;
}
}  // namespace

RLB_API int rlb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                   float* dw_f32, int dw_accumulate, long long rows, int d, long long x_stride,
                                   long long dy_stride, void* stream) {
  if (rows <= 0) return 0;
  if (d <= 0 || d % 8 || x_stride % 8 || dy_stride % 8) return RLB_STATIC_ERR_BAD_SHAPE;
  if (d > RLB_RMSNORM_STATIC_MAX_D) return RLB_STATIC_ERR_TOO_LARGE;
  // The kernels use 16-byte vector loads and stores on every operand and index rows with int: refuse what would
  // otherwise reach the device as a misaligned address or a truncated row count.
  if (x_stride < d || dy_stride < d || rows > 2147483647ll) return RLB_STATIC_ERR_BAD_SHAPE;
  const void* vec_ptrs[4] = {dy, x, w, dx};  // bf16 operands: 16-byte vector access
  for (const void* q : vec_ptrs)
    if (q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15u)) return RLB_STATIC_ERR_BAD_SHAPE;
  if (rstd == nullptr || dw_f32 == nullptr || (reinterpret_cast<uintptr_t>(rstd) & 3u) ||
      (reinterpret_cast<uintptr_t>(dw_f32) & 3u))
    return RLB_STATIC_ERR_BAD_SHAPE;
  float* scratch = nullptr;
  const int rc = rmsnorm_static_scratch(&scratch);
  if (rc) return rc;
  const int threads = rms_threads(d);
  const int parts = static_cast<int>(rows < RLB_RMSNORM_STATIC_MAX_PARTS ? rows : RLB_RMSNORM_STATIC_MAX_PARTS);
  // Every CTA writes its whole row of the partial matrix before the column-sum kernel reads it, so what an earlier
  // call left in the array is never read.
  rmsnorm_bwd_kernel<<<parts, threads, 0, S(stream)>>>(CBF(dy), CBF(x), CBF(w), rstd, BF(dx), scratch,
                                                       static_cast<int>(rows), d, x_stride, dy_stride, 0);
  colsum_kernel<<<(d + 255) / 256, 256, 0, S(stream)>>>(scratch, parts, d, dw_f32, nullptr, dw_accumulate);
  return static_cast<int>(cudaGetLastError());
}

RLB_API const char* rlb_rmsnorm_bwd_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case RLB_STATIC_ERR_BAD_SHAPE: return "d and the strides must be positive multiples of 8 elements (strides >= d, rows < 2^31), dy / x / w / dx non-null and 16-byte aligned, rstd / dw_f32 non-null";
    case RLB_STATIC_ERR_TOO_LARGE: return "d exceeds RLB_RMSNORM_STATIC_MAX_D (8192): use rlb_rmsnorm_bwd with caller scratch";
    case RLB_STATIC_ERR_NO_SYMBOL: return "the static scratch array's device address could not be resolved";
    default: return code > 0 ? "CUDA error (see cudaGetErrorString)" : "unknown code";
  }
}
