// Paged KV cache kernels for the generation engine: cache write and split-KV decode attention (GQA).
//
// Cache layout: k_cache / v_cache are [num_blocks, Hkv, block_size, D] bf16, so that one (block, head)
// is a contiguous [block_size, D] tile. A sequence owns a list of blocks (block table).
//
// Decode attention is memory-bound: the kernel streams each K/V row once for all G = Hq/Hkv query
// heads that share it. Eight lanes cooperate on one token (16 dims each, 32-byte loads), four tokens
// per warp step; softmax is kept online per lane group and merged through shared memory, then across
// KV splits by a second kernel (flash-decoding).
//
// This replaces the attention / KV-cache kernels that the reference reaches through vLLM
// (nemo_rl/models/generation/vllm/vllm_worker.py:570-597) and mcore's DynamicInferenceEngine
// (nemo_rl/models/generation/megatron/megatron_worker.py:174-202).
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

// qkv: [T, (Hq + 2*Hkv) * D] with layout [q | k | v]; slot[t] = block * block_size + offset, <0: skip.
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, const long long* __restrict__ slots,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      long long T, int Hq, int Hkv, int D, int block_size, long long row_stride,
                                      long long num_slots, int* status) {
  pdl_sync();
  const int vec_per_row = Hkv * D / 8;
  const long long total = T * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vec_per_row;
    const int r = static_cast<int>(i - t * vec_per_row) * 8;
    const int h = r / D, d = r - h * D;
    const long long slot = slots[t];
    if (slot < 0) continue;
    if (slot >= num_slots) {  // a slot outside the cache is recorded and skipped, never written
      if (status) atomicCAS(status, 0, RLB_ERR_BAD_ARG);
      continue;
    }
    const long long blk = slot / block_size;
    const int off = static_cast<int>(slot - blk * block_size);
    const long long dst = ((blk * Hkv + h) * block_size + off) * D + d;
    const __nv_bfloat16* src_k = qkv + t * row_stride + static_cast<long long>(Hq) * D + r;
    const __nv_bfloat16* src_v = src_k + static_cast<long long>(Hkv) * D;
    *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(src_k);
    *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(src_v);
  }
}

// Rotary embedding of the q and k heads (in place, HF rotate_half convention) fused with the scatter of the rotated k and of
// v into the paged cache: one warp per (token, head) of the fused [q | k | v] row. slot < 0: rotate only.
__global__ void rope_kv_write_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                     const long long* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                                     __nv_bfloat16* __restrict__ v_cache, long long T, int Hq, int Hkv, int D, int block_size,
                                     long long row_stride, long long num_slots, int* status) {
  pdl_sync();
  const int heads = Hq + 2 * Hkv;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * heads) return;
  const long long t = wid / heads;
  const int h = static_cast<int>(wid - t * heads);
  __nv_bfloat16* p = qkv + t * row_stride + static_cast<long long>(h) * D;
  const long long slot = slots[t];
  __nv_bfloat16* dst = nullptr;
  if (slot >= num_slots && h >= Hq) {  // outside the cache: recorded, rotated in place, not written
    if (status && lane == 0) atomicCAS(status, 0, RLB_ERR_BAD_ARG);
  } else if (h >= Hq && slot >= 0) {
    const long long blk = slot / block_size;
    const int off = static_cast<int>(slot - blk * block_size);
    const int kh = h < Hq + Hkv ? h - Hq : h - Hq - Hkv;
    dst = (h < Hq + Hkv ? k_cache : v_cache) + ((blk * Hkv + kh) * block_size + off) * D;
  }
  if (h >= Hq + Hkv) {  // v: copy
    if (dst)
      for (int i = lane * 2; i < D; i += 64) *reinterpret_cast<uint32_t*>(dst + i) = *reinterpret_cast<const uint32_t*>(p + i);
    return;
  }
  const float ps = static_cast<float>(pos[t]);
  const int half = D >> 1;
  for (int i = lane * 2; i < half; i += 64) {
    const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i));
    const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + i + half));
    float s0, c0, s1, c1;
    sincosf(ps * inv_freq[i], &s0, &c0);
    sincosf(ps * inv_freq[i + 1], &s1, &c1);
    const uint32_t a = pack_bf16x2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
    const uint32_t b = pack_bf16x2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
    *reinterpret_cast<uint32_t*>(p + i) = a;
    *reinterpret_cast<uint32_t*>(p + i + half) = b;
    if (dst) {
      *reinterpret_cast<uint32_t*>(dst + i) = a;
      *reinterpret_cast<uint32_t*>(dst + i + half) = b;
    }
  }
}

constexpr int DEC_THREADS = 128;
constexpr int LANES_PER_TOKEN = 8;
constexpr int TOKENS_PER_WARP = 32 / LANES_PER_TOKEN;  // 4
constexpr int GROUPS_PER_CTA = DEC_THREADS / LANES_PER_TOKEN;  // 16 token groups

// D = 128 only (16 dims per lane). G = query heads per kv head (1..8).
template <int G>
__global__ void __launch_bounds__(DEC_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride,  // q: [B, Hq*D] rows
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_table, int max_blocks_per_seq,
                    const int* __restrict__ seq_lens, int Hkv, int block_size, float scale, int num_splits,
                    float* __restrict__ part_o,   // [B, Hq, splits, D]
                    float* __restrict__ part_ml,  // [B, Hq, splits, 2]
                    __nv_bfloat16* __restrict__ out, long long out_stride) {
  constexpr int D = 128;
  constexpr int DL = D / LANES_PER_TOKEN;  // 16 dims per lane
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int Hq = Hkv * G;
  const int len = seq_lens[seq];
  const int per_split = ((len + num_splits - 1) / num_splits + block_size - 1) / block_size * block_size;
  const int t_begin = split * per_split;
  const int t_end = min(len, t_begin + per_split);

  const int grp = threadIdx.x / LANES_PER_TOKEN;  // which token slot of the CTA step
  const int sub = threadIdx.x % LANES_PER_TOKEN;  // which 16-dim slice

  float qr[G][DL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + seq * q_stride + static_cast<long long>(kvh * G + g) * D + sub * DL;
    const uint4 a = *reinterpret_cast<const uint4*>(qp);
    const uint4 b = *reinterpret_cast<const uint4*>(qp + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      qr[g][2 * j] = f.x * scale;
      qr[g][2 * j + 1] = f.y * scale;
    }
  }
  float o[G][DL];
  float m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DL; ++j) o[g][j] = 0.f;
  }

  const int* bt = block_table + static_cast<long long>(seq) * max_blocks_per_seq;
  // The trip count is uniform over the CTA, so every shuffle below runs with all 32 lanes present;
  // a lane group past the end re-reads the last valid row and contributes with weight zero.
  for (int t0 = t_begin; t0 < t_end; t0 += GROUPS_PER_CTA) {
    const bool valid = t0 + grp < t_end;
    const int t = valid ? t0 + grp : t_end - 1;
    const int blk = bt[t / block_size];
    const int off = t % block_size;
    const long long base = ((static_cast<long long>(blk) * Hkv + kvh) * block_size + off) * D + sub * DL;
    const uint4 ka = *reinterpret_cast<const uint4*>(k_cache + base);
    const uint4 kb = *reinterpret_cast<const uint4*>(k_cache + base + 8);
    const uint4 va = *reinterpret_cast<const uint4*>(v_cache + base);
    const uint4 vb = *reinterpret_cast<const uint4*>(v_cache + base + 8);
    float kf[DL], vf[DL];
    {
      const uint32_t kw[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
      const uint32_t vw[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 a = unpack_bf16x2(kw[j]);
        const float2 b = unpack_bf16x2(vw[j]);
        kf[2 * j] = a.x; kf[2 * j + 1] = a.y;
        vf[2 * j] = b.x; vf[2 * j + 1] = b.y;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < DL; ++j) s += qr[g][j] * kf[j];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        if (s > m[g]) {  // rare after the first tokens: rescale only when the maximum moves
          const float c = __expf(m[g] - s);
          l[g] *= c;
#pragma unroll
          for (int j = 0; j < DL; ++j) o[g][j] *= c;
          m[g] = s;
        }
        const float p = __expf(s - m[g]);
        l[g] += p;
#pragma unroll
        for (int j = 0; j < DL; ++j) o[g][j] += p * vf[j];
      }
    }
  }
  __syncwarp();

  // Merge the four lane groups of each warp with shuffles, then the four warps through shared memory.
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mw = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], 8));
    mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
    const float c = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mw);
    float lw = l[g] * c;
    lw += __shfl_xor_sync(0xffffffffu, lw, 8);
    lw += __shfl_xor_sync(0xffffffffu, lw, 16);
#pragma unroll
    for (int j = 0; j < DL; ++j) {
      float v = o[g][j] * c;
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      o[g][j] = v;
    }
    m[g] = mw;
    l[g] = lw;
  }
  constexpr int NW = DEC_THREADS / 32;
  __shared__ float sm_m[NW][G];
  __shared__ float sm_l[NW][G];
  __shared__ float sm_o[NW][G][D];  // 4 * G * 512 B
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      sm_m[wid][g] = m[g];
      sm_l[wid][g] = l[g];
    }
  }
  if (lane < LANES_PER_TOKEN) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int j = 0; j < DL; ++j) sm_o[wid][g][sub * DL + j] = o[g][j];
  }
  __syncthreads();
  // thread d (0..127) finalises dimension d of every head
  const int d = threadIdx.x;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < NW; ++r) mm = fmaxf(mm, sm_m[r][g]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int r = 0; r < NW; ++r) {
      const float c = (sm_m[r][g] == -INFINITY) ? 0.f : __expf(sm_m[r][g] - mm);
      ll += sm_l[r][g] * c;
      acc += sm_o[r][g][d] * c;
    }
    const int hq = kvh * G + g;
    if (num_splits == 1) {
      const float v = ll > 0.f ? acc / ll : 0.f;
      out[seq * out_stride + static_cast<long long>(hq) * D + d] = __float2bfloat16(v);
    } else {
      const long long pi = (static_cast<long long>(seq) * Hq + hq) * num_splits + split;
      part_o[pi * D + d] = acc;
      if (d == 0) {
        part_ml[pi * 2] = mm;
        part_ml[pi * 2 + 1] = ll;
      }
    }
  }
}

__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      int num_splits, int Hq, __nv_bfloat16* __restrict__ out,
                                      long long out_stride) {
  constexpr int D = 128;
  const int seq = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const long long base = (static_cast<long long>(seq) * Hq + hq) * num_splits;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += part_ml[(base + s) * 2 + 1] * c;
    acc += part_o[(base + s) * D + d] * c;
  }
  out[seq * out_stride + static_cast<long long>(hq) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}

template <int G>
int launch_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                  const int* block_table, int max_blocks_per_seq, const int* seq_lens, int B, int Hkv,
                  int block_size, float scale, int num_splits, float* part_o, float* part_ml, void* out,
                  long long out_stride, cudaStream_t stream) {
  dim3 grid(B, Hkv, num_splits);
  paged_decode_kernel<G><<<grid, DEC_THREADS, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<const __nv_bfloat16*>(k_cache),
      reinterpret_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks_per_seq, seq_lens, Hkv, block_size,
      scale, num_splits, part_o, part_ml, reinterpret_cast<__nv_bfloat16*>(out), out_stride);
  if (num_splits > 1) {
    dim3 g2(B, Hkv * G);
    decode_combine_kernel<<<g2, 128, 0, stream>>>(part_o, part_ml, num_splits, Hkv * G,
                                                  reinterpret_cast<__nv_bfloat16*>(out), out_stride);
  }
  return static_cast<int>(cudaGetLastError());
}

// Copies whole cache blocks src[i] -> dst[i] in both caches.
__global__ void block_copy_kernel(__nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                  const int* __restrict__ src, const int* __restrict__ dst, long long elems) {
  const int pair = blockIdx.y;
  const long long s = static_cast<long long>(src[pair]) * elems, d = static_cast<long long>(dst[pair]) * elems;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < elems;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    *reinterpret_cast<uint4*>(k_cache + d + i) = *reinterpret_cast<const uint4*>(k_cache + s + i);
    *reinterpret_cast<uint4*>(v_cache + d + i) = *reinterpret_cast<const uint4*>(v_cache + s + i);
  }
}

// out[i, :] = x[idx[i], :], bf16 rows of width d (multiple of 8).
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out, long long n, int d, long long x_stride,
                                   long long out_stride) {
  const int vecs = d / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n * vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vecs;
    const int c = static_cast<int>(i - r * vecs) * 8;
    *reinterpret_cast<uint4*>(out + r * out_stride + c) =
        *reinterpret_cast<const uint4*>(x + static_cast<long long>(idx[r]) * x_stride + c);
  }
}

}  // namespace

RLB_API int rlb_block_copy(void* k_cache, void* v_cache, const int* src, const int* dst, int n, long long elems,
                           void* stream) {
  if (n <= 0) return 0;
  if (elems % 8) return -2;
  dim3 grid(static_cast<unsigned>((elems / 8 + 255) / 256), n);
  block_copy_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), src, dst, elems);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_gather_rows(const void* x, const int* idx, void* out, long long n, int d, long long x_stride,
                            long long out_stride, void* stream) {
  if (n <= 0) return 0;
  if (d % 8 || x_stride % 8 || out_stride % 8) return -2;
  long long grid = (n * (d / 8) + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  gather_rows_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), idx, reinterpret_cast<__nv_bfloat16*>(out), n, d, x_stride,
      out_stride);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_kv_cache_write(const void* qkv, const long long* slots, void* k_cache, void* v_cache, long long T,
                               int Hq, int Hkv, int D, int block_size, long long row_stride, long long num_blocks, int* status,
                               void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || row_stride % 8) return -2;
  const long long total = T * (Hkv * D / 8);
  long long grid = (total + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  rlb_launch_pdl(kv_cache_write_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0, static_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(qkv), slots, reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), T, Hq, Hkv, D, block_size, row_stride, num_blocks * block_size, status);
  return static_cast<int>(cudaGetLastError());
}

// Rotates q and k of the fused rows in place and writes the rotated k and v into the paged cache (see rope_kv_write_kernel).
RLB_API int rlb_rope_kv_cache_write(void* qkv, const int* pos, const float* inv_freq, const long long* slots, void* k_cache,
                                    void* v_cache, long long T, int Hq, int Hkv, int D, int block_size, long long row_stride,
                                    long long num_blocks, int* status, void* stream) {
  if (T <= 0) return 0;
  if (D % 4 || row_stride % 2) return -2;
  const long long warps = T * (Hq + 2 * Hkv);
  const long long blocks = (warps * 32 + 255) / 256;
  rlb_launch_pdl(rope_kv_write_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                 reinterpret_cast<__nv_bfloat16*>(qkv), pos, inv_freq, slots, reinterpret_cast<__nv_bfloat16*>(k_cache),
                 reinterpret_cast<__nv_bfloat16*>(v_cache), T, Hq, Hkv, D, block_size, row_stride, num_blocks * block_size, status);
  return static_cast<int>(cudaGetLastError());
}

// Decode attention for B sequences, one query token each. head_dim must be 128, Hq/Hkv in {1,2,4,8}.
// With num_splits > 1 the caller provides scratch: part_o [B*Hq*splits*128] floats and part_ml
// [B*Hq*splits*2] floats.
RLB_API int rlb_paged_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                             const int* block_table, int max_blocks_per_seq, const int* seq_lens, int B, int Hq,
                             int Hkv, int D, int block_size, float scale, int num_splits, float* part_o,
                             float* part_ml, void* out, long long out_stride, void* stream) {
  if (B <= 0) return 0;
  if (D != 128 || Hq % Hkv) return -2;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_ml)) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (Hq / Hkv) {
    case 1: return launch_decode<1>(q, q_stride, k_cache, v_cache, block_table, max_blocks_per_seq, seq_lens, B, Hkv, block_size, scale, num_splits, part_o, part_ml, out, out_stride, s);
    case 2: return launch_decode<2>(q, q_stride, k_cache, v_cache, block_table, max_blocks_per_seq, seq_lens, B, Hkv, block_size, scale, num_splits, part_o, part_ml, out, out_stride, s);
    case 4: return launch_decode<4>(q, q_stride, k_cache, v_cache, block_table, max_blocks_per_seq, seq_lens, B, Hkv, block_size, scale, num_splits, part_o, part_ml, out, out_stride, s);
    case 8: return launch_decode<8>(q, q_stride, k_cache, v_cache, block_table, max_blocks_per_seq, seq_lens, B, Hkv, block_size, scale, num_splits, part_o, part_ml, out, out_stride, s);
    default: return -4;
  }
}
