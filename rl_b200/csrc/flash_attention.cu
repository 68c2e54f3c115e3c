// Causal self-attention over packed (variable-length) sequences on the 5th-generation tensor cores:
// forward and backward, grouped-query heads, head dimension 128, bf16 in / fp32 accumulate.
//
// Inputs are read in place from the fused projection buffer qkv[T, (Hq + 2*Hkv) * 128] ([q | k | v] per token, after
// RoPE) through 2-D TMA tensor maps; `cu_seqlens[B+1]` marks sequence boundaries. The same kernels serve training
// (packed micro-batches) and the prefill of the generation engine.
//
// Forward, one CTA per (128-row query tile, query head), two CTAs per SM so that one CTA's softmax overlaps the
// other's MMAs:
//   warp 0      TMA producer: Q once, then K/V tiles of 64 keys through a 2-stage ring
//   warp 1      tcgen05.mma issuer: S = Q K^T (128x64x128) into TMEM, then O += P V (128x128x64)
//   warps 2..5  softmax: one thread per query row reads its 64 scores from TMEM (no shuffles), keeps the running
//               max / sum in the exp2 domain, writes P in bf16 into 128B-swizzled shared memory as the A operand of
//               the second MMA, and rescales the O accumulator in TMEM only when the row maximum moved by more than
//               2^8 (stale maxima are exact because the final normalisation uses the same reference).
// Output: O[T, Hq*128] bf16 and the per-row log-sum-exp lse[Hq, T] (natural log) for the backward pass.
//
// Backward is two kernels without atomics: one per (64-key tile, kv head) accumulating dK / dV over all query tiles
// and the G query heads of the group, one per (128-row query tile, query head) accumulating dQ over key tiles. Both
// recompute S and P from Q, K and lse.
//
// Replaces flash-attn 2 / cuDNN fused attention in the reference's policy workers
// (nemo_rl/models/automodel/setup.py:321-325, nemo_rl/models/megatron/setup.py:1114-1140).
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 64;   // keys per pipeline stage
#ifndef RLB_HD
#define RLB_HD 128        // head dimension of this translation unit; flash_attention_d64.cu includes this file with 64
#endif
#ifndef RLB_NAME
#define RLB_NAME(x) x     // exported names get a suffix in the other instantiations (rlb_flash_attn_fwd_d64, ...)
#endif
constexpr int HD = RLB_HD;
static_assert(HD == 64 || HD == 128, "head dimension: 64 or 128");
constexpr int ATOMS = HD / 64;            // [rows x 64] swizzle atoms per operand tile along the head dimension
constexpr int KV_STAGES = 2;
constexpr int Q_BYTES = BQ * HD * 2;         // 32 KB at HD 128: two [128 x 64] swizzle atoms
constexpr int Q_ATOM = BQ * 64 * 2;
constexpr int KV_ATOM = BKV * 64 * 2;
constexpr int K_BYTES = BKV * HD * 2;        // 16 KB: two [64 x 64] atoms
constexpr int V_BYTES = BKV * HD * 2;        // 16 KB: two boxes of 64 head-dim columns
constexpr int P_BYTES = BQ * BKV * 2;        // 16 KB: one [128 x 64] atom
constexpr int FWD_SMEM = Q_BYTES + KV_STAGES * (K_BYTES + V_BYTES) + P_BYTES + 256;  // 2 CTAs fit in 227 KB
constexpr int FWD_THREADS = 192;
constexpr int TMEM_COLS_FWD = 256;  // S at column 0 (64 columns), O at column 128 (128 columns)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Finds the (sequence, tile-in-sequence) of a flat tile index; tiles of `rows` rows never straddle sequences.
// Returns false when `tile` is past the last tile. One thread calls it; the result is broadcast through smem.
__device__ bool locate_tile(const int* __restrict__ cu, int num_seqs, int rows, int tile, int& seq, int& start,
                            int& len, int& tile_in_seq) {
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int n = (e - b + rows - 1) / rows;
    if (tile < acc + n) {
      seq = s;
      start = b;
      len = e - b;
      tile_in_seq = tile - acc;
      return true;
    }
    acc += n;
  }
  return false;
}

// Writes 8 bf16 (one 16-byte chunk) of row `r` at logical chunk `c` (0..7) of a 128B-swizzled [rows x 64] atom.
__device__ __forceinline__ void st_swizzled_chunk(uint8_t* atom, int r, int c, uint4 v) {
  *reinterpret_cast<uint4*>(atom + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}

struct FwdParams {
  const int* cu_seqlens;
  int num_seqs;
  int T;
  int Hq, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* out;
  long long out_stride;
  float* lse;  // [Hq, T]
  int* status;
};

__global__ void __launch_bounds__(FWD_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                 FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1024-byte aligned base; report instead of misreading
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, RLB_ERR_BAD_ARG);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + Q_BYTES;
  uint8_t* v_s = k_s + KV_STAGES * K_BYTES;
  uint8_t* p_s = v_s + KV_STAGES * V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* kv_empty = bars + 5;  // [2]
  uint64_t* s_full = bars + 7;
  uint64_t* p_full = bars + 8;
  uint64_t* o_done = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* tile_info = reinterpret_cast<int*>(tmem_slot + 2);  // seq_start, seq_len, tile_in_seq, valid

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);

  if (threadIdx.x == 0) {
    int seq = 0, start = 0, len = 0, tis = 0;
    const bool ok = locate_tile(p.cu_seqlens, p.num_seqs, BQ, blockIdx.x, seq, start, len, tis);
    tile_info[0] = start;
    tile_info[1] = len;
    tile_info[2] = tis;
    tile_info[3] = ok ? 1 : 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(o_done), 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (!tile_info[3]) return;  // uniform: past the last tile (before any TMEM allocation)
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS_FWD);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;

  const int seq_start = tile_info[0], seq_len = tile_info[1];
  const int q0 = tile_info[2] * BQ;                       // first query row, relative to the sequence
  const int q_rows = min(BQ, seq_len - q0);
  const int n_kv = (q0 + q_rows + BKV - 1) / BKV;         // causal: keys up to the tile's last row
  const int q_col = head * HD;
  const int k_col = (p.Hq + kv_head) * HD;
  const int v_col = (p.Hq + p.Hkv + kv_head) * HD;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_kv);
      mbar_arrive_expect_tx(smem_u32(q_full), Q_BYTES);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a)
        tma_load_2d(smem_u32(q_s + a * Q_ATOM), &tmap_q, smem_u32(q_full), q_col + a * 64, seq_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[st]), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) break;
        const int row = seq_start + j * BKV;
        mbar_arrive_expect_tx(smem_u32(&k_full[st]), K_BYTES);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_2d(smem_u32(k_s + st * K_BYTES + a * KV_ATOM), &tmap_kv, smem_u32(&k_full[st]), k_col + a * 64, row);
        mbar_arrive_expect_tx(smem_u32(&v_full[st]), V_BYTES);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_2d(smem_u32(v_s + st * V_BYTES + a * KV_ATOM), &tmap_kv, smem_u32(&v_full[st]), v_col + a * 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, HD, false, true);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, RLB_ERR_WAIT_FULL);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(smem_u32(&k_full[st]), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL)) break;
        tc_fence_after();
        // S = Q K^T over the head dimension: 8 steps of 16, two swizzle atoms of 64
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t qa = smem_u32(q_s) + (kk / 4) * Q_ATOM + (kk % 4) * 32;
          const uint32_t ka = smem_u32(k_s + st * K_BYTES) + (kk / 4) * KV_ATOM + (kk % 4) * 32;
          umma_f16(tmem_s, make_smem_desc_sw128(qa, 16, 1024), make_smem_desc_sw128(ka, 16, 1024), idesc_s,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
        if (!mbar_wait(smem_u32(p_full), j & 1, abort_flag, p.status, RLB_ERR_WAIT_FLAG)) break;
        if (!mbar_wait(smem_u32(&v_full[st]), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL)) break;
        tc_fence_after();
        // O += P V over the 64 keys: 4 steps of 16 key rows
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t pa = smem_u32(p_s) + kk * 32;
          const uint32_t va = smem_u32(v_s + st * V_BYTES) + kk * (16 * 128);
          umma_f16(tmem_o, make_smem_desc_sw128(pa, 16, 1024), make_smem_desc_sw128(va, KV_ATOM, 1024), idesc_o,
                   (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&kv_empty[st]));
        umma_commit(smem_u32(o_done));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: thread = query row
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + r;  // row index inside the sequence
    float m_ref = -INFINITY;  // reference maximum used for the exponentials (log2 domain)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(smem_u32(s_full), j & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32b_x32(tmem_s + lane_addr, s0);
      tmem_ld_32x32b_x32(tmem_s + lane_addr + 32, s1);
      tmem_ld_wait();
      const int k0 = j * BKV;
      const bool diag = k0 + BKV - 1 > q0;  // tile touches the causal boundary of some row
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float a = __uint_as_float(s0[i]) * p.scale_log2;
        float b = __uint_as_float(s1[i]) * p.scale_log2;
        if (diag) {
          if (k0 + i > qi) a = -INFINITY;
          if (k0 + 32 + i > qi) b = -INFINITY;
        }
        s0[i] = __float_as_uint(a);
        s1[i] = __float_as_uint(b);
        mx = fmaxf(mx, fmaxf(a, b));
      }
      // Lazy rescale: move the reference only when the maximum grew by more than the threshold.
      float factor = 1.f;
      bool need = false;
      if (mx > m_ref + RESCALE_THRESHOLD || m_ref == -INFINITY) {
        const float m_new = fmaxf(mx, m_ref);
        if (m_new != -INFINITY) {
          factor = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
          need = m_ref != -INFINITY;  // nothing accumulated yet: no O to rescale
          m_ref = m_new;
        }
      }
      l *= factor;
      float rowsum = 0.f;
      uint32_t pk[32];
      const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float e0 = exp2f(__uint_as_float(s0[2 * i]) - mr), e1 = exp2f(__uint_as_float(s0[2 * i + 1]) - mr);
        const float f0 = exp2f(__uint_as_float(s1[2 * i]) - mr), f1 = exp2f(__uint_as_float(s1[2 * i + 1]) - mr);
        rowsum += (e0 + e1) + (f0 + f1);
        pk[i] = pack_bf16x2(e0, e1);
        pk[16 + i] = pack_bf16x2(f0, f1);
      }
      l += rowsum;
      // P and O may be touched only after the previous P V product has completed.
      if (j > 0) {
        if (!mbar_wait(smem_u32(o_done), (j - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_32x32b_x32(tmem_o + lane_addr + c * 32, o);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        st_swizzled_chunk(p_s, r, c, make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]));
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok && mbar_wait(smem_u32(o_done), (n_kv - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = r < q_rows;
      __nv_bfloat16* dst = p.out + static_cast<long long>(seq_start + qi) * p.out_stride + head * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv_l, __uint_as_float(o[q * 8 + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv_l, __uint_as_float(o[q * 8 + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv_l, __uint_as_float(o[q * 8 + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv_l, __uint_as_float(o[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = v;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[static_cast<long long>(head) * p.T + seq_start + qi] = (m_ref + log2f(l)) * (1.f / LOG2E);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS_FWD);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]  (one warp per (t, h))
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ delta, int T, int Hq, long long do_stride, long long o_stride) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(wid / Hq), h = static_cast<int>(wid % Hq);
  constexpr int PER = HD / 32;   // elements per lane: 4 or 2
  const __nv_bfloat16* a = dout + t * do_stride + h * HD + lane * PER;
  const __nv_bfloat16* b = out + t * o_stride + h * HD + lane * PER;
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < PER / 2; ++q) {
    const float2 x = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a)[q]), y = unpack_bf16x2(reinterpret_cast<const uint32_t*>(b)[q]);
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

int g_fwd_configured = 0;

}  // namespace

// qkv: [T, (Hq+2Hkv)*128] bf16 with row stride `qkv_stride` (elements); out: [T, Hq*128]; lse: [Hq, T] or null.
// cu_seqlens: device int32 [num_seqs + 1]. max_tiles: an upper bound on the number of 128-row query tiles
// (ceil(T / 128) + num_seqs is always enough).
RLB_API int RLB_NAME(rlb_flash_attn_fwd)(const void* qkv, long long qkv_stride, const int* cu_seqlens, int num_seqs, int T,
                               int Hq, int Hkv, int D, float scale, void* out, long long out_stride, float* lse,
                               int max_tiles, int* status, void* stream) {
  if (T <= 0 || num_seqs <= 0) return 0;
  if (D != HD || Hq % Hkv || qkv_stride % 8 || out_stride % 8) return -2;
  CUtensorMap tq, tkv;
  const long long C = static_cast<long long>(Hq + 2 * Hkv) * HD;
  int rc = rlb_make_tmap_2d(&tq, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, T, qkv_stride * 2, 64, BQ,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tkv, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, T, qkv_stride * 2, 64, BKV,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  if (!g_fwd_configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_fwd_configured = 1;
  }
  FwdParams p;
  p.cu_seqlens = cu_seqlens;
  p.num_seqs = num_seqs;
  p.T = T;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale_log2 = scale * LOG2E;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.lse = lse;
  p.status = status;
  dim3 grid(max_tiles, Hq);
  flash_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, static_cast<cudaStream_t>(stream)>>>(tq, tkv, p);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int RLB_NAME(rlb_attn_delta)(const void* dout, const void* out, float* delta, int T, int Hq, long long do_stride,
                           long long o_stride, void* stream) {
  if (T <= 0) return 0;
  const long long warps = static_cast<long long>(T) * Hq;
  const long long blocks = (warps * 32 + 255) / 256;
  attn_delta_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(out), delta, T, Hq,
      do_stride, o_stride);
  return static_cast<int>(cudaGetLastError());
}
