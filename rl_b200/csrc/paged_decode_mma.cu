// Paged decode attention on the tensor cores (sm_100a, tcgen05 + TMEM + TMA): flash-decoding for one query token per
// sequence against its paged KV cache, one CTA per (sequence, KV head, KV split).
//
// Both products of a 128-token tile run as tcgen05 MMAs with the tokens / head dimensions on the M side and the G = Hq / Hkv
// query heads of the group (padded to 16) on the N side:
//     S^T[128 tokens, 16] = K_tile[128, 128 dims] * Q^T           (K tile K-major from TMA, Q staged once in shared memory)
//     O^T[128 dims, 16]   = V_tile^T[128 dims, 128 tokens] * P    (V tile read MN-major from the same TMA layout, P^T written
//                                                                   by the softmax warps as a K-major operand)
// so the only cross-thread work of the softmax is one max and one sum reduction per head and TILE (not per token), and the
// CUDA cores never touch K or V. Warp roles: warp 0 streams K and V tiles with TMA (one buffer each; the next K tile is
// requested as soon as the QK MMAs of the current one have completed, the next V tile after the PV MMAs), warp 1 issues
// the MMAs, warps 2-5 own one token row of S^T / one dim row of O^T each and keep the running max / sum / output in
// registers. Every wait is bounded (status word, no hang).
//
// The CUDA-core kernel in paged_decode_tma.cu (same contract) is kept as the fallback for block sizes / head dims this
// kernel does not cover. Reference counterpart: the FlashInfer / vLLM paged-attention decode kernels behind
// nemo_rl/models/generation/vllm.
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

constexpr int DM_D = 128;        // head dim
constexpr int DM_TOK = 128;      // tokens per tile
constexpr int DM_N = 16;         // query heads of a group, padded
constexpr int DM_THREADS = 192;
constexpr int DM_CHUNK = DM_TOK * 128;        // one 64-dim chunk of a K / V tile: 128 rows x 128 B = 16 KB
constexpr int DM_KV_BYTES = 2 * DM_CHUNK;     // 32 KB
constexpr int DM_QP_BYTES = 2 * DM_N * 128;   // Q or P^T: 2 chunks x 16 rows x 128 B = 4 KB
constexpr int DM_SMEM = 2 * DM_KV_BYTES + 2 * DM_QP_BYTES + 1024 /*reductions + barriers*/ + 1024 /*alignment*/;
constexpr int DM_TMEM_COLS = 32;

struct DmParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const int* block_table;
  int max_blocks_per_seq;
  const int* seq_lens;
  int Hkv, G, block_size;
  float scale;
  int num_splits;
  float* part_o;
  float* part_ml;
  __nv_bfloat16* out;
  long long out_stride;
  int* status;
};

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// byte offset of element (row, col) of a K-major bf16 tile with 128-byte swizzle whose rows hold 64 elements per chunk;
// `chunk_bytes` separates consecutive 64-column chunks
__device__ __forceinline__ uint32_t sw128_off(int row, int col, int chunk_bytes) {
  const int chunk = col >> 6, c = col & 63;
  return chunk * chunk_bytes + (row >> 3) * 1024 + (row & 7) * 128 + ((((c * 2) >> 4) ^ (row & 7)) << 4) + ((c * 2) & 15);
}

__global__ void __launch_bounds__(DM_THREADS, 2)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, DmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_sm = smem;
  uint8_t* v_sm = smem + DM_KV_BYTES;
  uint8_t* q_sm = smem + 2 * DM_KV_BYTES;
  uint8_t* p_sm = q_sm + DM_QP_BYTES;
  float* red = reinterpret_cast<float*>(p_sm + DM_QP_BYTES);   // [2][4][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * 4 * DM_N);
  uint64_t* k_full = bars + 0;
  uint64_t* k_empty = bars + 1;
  uint64_t* v_full = bars + 2;
  uint64_t* v_empty = bars + 3;
  uint64_t* s_full = bars + 4;
  uint64_t* s_empty = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* o_empty = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Set-up that touches no global memory runs before the dependency wait and overlaps the previous kernel's tail.
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(k_full), 1);
    mbar_init(smem_u32(k_empty), 1);
    mbar_init(smem_u32(v_full), 1);
    mbar_init(smem_u32(v_empty), 1);
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_empty), 4);
    mbar_init(smem_u32(p_ready), 1);
    mbar_init(smem_u32(o_full), 1);
    mbar_init(smem_u32(o_empty), 4);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), DM_TMEM_COLS);
    tmem_relinquish();
  }
  pdl_sync();

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.G, Hq = p.Hkv * G;
  const int len = p.seq_lens[seq];
  const int bs = p.block_size;
  const int per_split = ((len + p.num_splits - 1) / p.num_splits + DM_TOK - 1) / DM_TOK * DM_TOK;
  const int t_begin = split * per_split;
  const int t_end = min(len, t_begin + per_split);
  const int n_tiles = t_end > t_begin ? (t_end - t_begin + DM_TOK - 1) / DM_TOK : 0;

  // Q (pre-scaled) and a zeroed P^T, both in the swizzled K-major operand layout: 256 pieces of 16 bytes each
  for (int i = threadIdx.x; i < 2 * DM_QP_BYTES / 16; i += DM_THREADS) {
    uint4 val = make_uint4(0, 0, 0, 0);
    const int which = i / (DM_QP_BYTES / 16);          // 0: Q, 1: P
    const int j = i % (DM_QP_BYTES / 16);              // piece inside the 4 KB operand
    const int g = j / 16, piece = j % 16;              // row (head), 8-dim piece of the 128 dims
    if (which == 0 && g < G) {
      const __nv_bfloat16* qp = p.q + seq * p.q_stride + static_cast<long long>(kvh * G + g) * DM_D + piece * 8;
      const uint4 raw = *reinterpret_cast<const uint4*>(qp);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w[k]);
        o[k] = pack_bf16x2(f.x * p.scale, f.y * p.scale);
      }
      val = make_uint4(o[0], o[1], o[2], o[3]);
    }
    uint8_t* base = which == 0 ? q_sm : p_sm;
    *reinterpret_cast<uint4*>(base + sw128_off(g, piece * 8, DM_N * 128)) = val;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + DM_N;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int* bt = p.block_table + static_cast<long long>(seq) * p.max_blocks_per_seq;
      const int box_rows = bs < DM_TOK ? bs : DM_TOK;
      const int nbox = DM_TOK / box_rows;
      bool ok = true;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const uint32_t ph = i & 1;
        const int t0 = t_begin + i * DM_TOK;
        for (int kv = 0; kv < 2 && ok; ++kv) {
          uint64_t* empty = kv == 0 ? k_empty : v_empty;
          uint64_t* full = kv == 0 ? k_full : v_full;
          if (!mbar_wait(smem_u32(empty), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(full);
          mbar_arrive_expect_tx(bar, DM_KV_BYTES);
          const uint32_t dst = smem_u32(kv == 0 ? k_sm : v_sm);
          for (int b = 0; b < nbox; ++b) {
            const int t = t0 + b * box_rows;
            // tokens past the sequence end read block-table entries that point to valid (if unrelated) cache blocks;
            // their scores are masked before the softmax
            const int blk = bt[min(t / bs, p.max_blocks_per_seq - 1)];
            const int row = (blk * p.Hkv + kvh) * bs + (t % bs);
            for (int c = 0; c < 2; ++c)
              tma_load_2d(dst + c * DM_CHUNK + b * box_rows * 128, kv == 0 ? &tmap_k : &tmap_v, bar, c * 64, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(DM_TOK, DM_N, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(DM_D, DM_N, true, false);
      auto issue_qk = [&](int i) -> bool {
        const uint32_t ph = i & 1;
        if (!mbar_wait(smem_u32(k_full), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL)) return false;
        if (!mbar_wait(smem_u32(s_empty), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DM_D / 16; ++kk) {
          const uint64_t a = make_smem_desc_sw128(smem_u32(k_sm) + (kk >> 2) * DM_CHUNK + (kk & 3) * 32, 16, 1024);
          const uint64_t b = make_smem_desc_sw128(smem_u32(q_sm) + (kk >> 2) * (DM_N * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_s, a, b, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
        umma_commit(smem_u32(k_empty));
        return true;
      };
      bool ok = n_tiles > 0 ? issue_qk(0) : true;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const uint32_t ph = i & 1;
        if (i + 1 < n_tiles) ok = issue_qk(i + 1);   // overlaps the softmax of tile i
        if (!ok) break;
        if (!mbar_wait(smem_u32(p_ready), ph, abort_flag, p.status, RLB_ERR_WAIT_FLAG) ||
            !mbar_wait(smem_u32(v_full), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL) ||
            !mbar_wait(smem_u32(o_empty), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DM_TOK / 16; ++kk) {
          // V^T: M = dims (two 64-dim chunks 16 KB apart), K = tokens: 16 token rows of 128 B per MMA
          const uint64_t a = make_smem_desc_sw128(smem_u32(v_sm) + kk * 2048, DM_CHUNK, 1024);
          const uint64_t b = make_smem_desc_sw128(smem_u32(p_sm) + (kk >> 2) * (DM_N * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_o, a, b, idesc_pv, kk != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(o_full));
        umma_commit(smem_u32(v_empty));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / output warps: row r of S^T (token) and O^T (dim)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_run[8], l_run[8], o_run[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      o_run[g] = 0.f;
    }
    float* red_max = red;                 // [4][16]
    float* red_sum = red + 4 * DM_N;      // [4][16]
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const uint32_t ph = i & 1;
      if (!mbar_wait(smem_u32(s_full), ph, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[16];
      tmem_ld_32x32b_x16(tmem_s + lane_addr, sr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_empty));
      const bool valid = t_begin + i * DM_TOK + r < t_end;
      float s[8], pr[8], c[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        s[g] = (valid && g < G) ? __uint_as_float(sr[g]) : -INFINITY;
        float mx = s[g];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) red_max[quarter * DM_N + g] = mx;
      }
      named_bar_sync(1, 128);
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float mt = fmaxf(fmaxf(red_max[g], red_max[DM_N + g]), fmaxf(red_max[2 * DM_N + g], red_max[3 * DM_N + g]));
        const float mn = fmaxf(m_run[g], mt);
        c[g] = (m_run[g] == -INFINITY) ? 0.f : __expf(m_run[g] - mn);
        pr[g] = (s[g] == -INFINITY) ? 0.f : __expf(s[g] - mn);
        m_run[g] = mn;
        float sm = pr[g];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, off);
        if (lane == 0) red_sum[quarter * DM_N + g] = sm;
        if (g < G) *reinterpret_cast<__nv_bfloat16*>(p_sm + sw128_off(g, r, DM_N * 128)) = __float2bfloat16(pr[g]);
      }
      fence_proxy_async();           // P^T is read by the tensor core (async proxy)
      named_bar_sync(1, 128);        // also publishes red_sum and orders this tile's red_max reads before the next writes
      if (threadIdx.x == 64) mbar_arrive(smem_u32(p_ready));
#pragma unroll
      for (int g = 0; g < 8; ++g)
        l_run[g] = l_run[g] * c[g] + (red_sum[g] + red_sum[DM_N + g]) + (red_sum[2 * DM_N + g] + red_sum[3 * DM_N + g]);
      if (!mbar_wait(smem_u32(o_full), ph, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t orr[16];
      tmem_ld_32x32b_x16(tmem_o + lane_addr, orr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(o_empty));
#pragma unroll
      for (int g = 0; g < 8; ++g) o_run[g] = o_run[g] * c[g] + __uint_as_float(orr[g]);
      named_bar_sync(1, 128);        // red_sum of this tile has been consumed by everyone before the next tile overwrites it
    }
    // results: thread r owns head dimension r of every head of the group
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (g >= G) break;
      const int hq = kvh * G + g;
      if (p.num_splits == 1) {
        p.out[seq * p.out_stride + static_cast<long long>(hq) * DM_D + r] = __float2bfloat16(l_run[g] > 0.f ? o_run[g] / l_run[g] : 0.f);
      } else {
        const long long pi = (static_cast<long long>(seq) * Hq + hq) * p.num_splits + split;
        p.part_o[pi * DM_D + r] = o_run[g];
        if (r == 0) {
          p.part_ml[pi * 2] = m_run[g];
          p.part_ml[pi * 2 + 1] = l_run[g];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, DM_TMEM_COLS);
  }
}

__global__ void dm_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int num_splits, int Hq,
                                  __nv_bfloat16* __restrict__ out, long long out_stride) {
  pdl_sync();
  const int seq = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const long long base = (static_cast<long long>(seq) * Hq + hq) * num_splits;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += part_ml[(base + s) * 2 + 1] * c;
    acc += part_o[(base + s) * DM_D + d] * c;
  }
  out[seq * out_stride + static_cast<long long>(hq) * DM_D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}
}  // namespace

// Same contract as rlb_paged_decode_tma. Supported: head_dim 128, Hq / Hkv <= 8, block_size 16, 32, 64 or a multiple of 128.
RLB_API int rlb_paged_decode_mma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, int num_blocks,
                                 const int* block_table, int max_blocks_per_seq, const int* seq_lens, int B, int Hq, int Hkv, int D,
                                 int block_size, float scale, int num_splits, float* part_o, float* part_ml, void* out,
                                 long long out_stride, int* status, void* stream) {
  if (B <= 0) return 0;
  if (D != DM_D || Hq % Hkv || Hq / Hkv > 8) return -2;
  if (!(block_size == 16 || block_size == 32 || block_size == 64 || block_size % 128 == 0)) return -2;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_ml)) return -3;
  const int box_rows = block_size < DM_TOK ? block_size : DM_TOK;
  const unsigned long long rows = static_cast<unsigned long long>(num_blocks) * Hkv * block_size;
  CUtensorMap tk, tv;
  int rc = rlb_make_tmap_2d(&tk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, DM_D, rows, DM_D * 2, 64, box_rows,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tv, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, DM_D, rows, DM_D * 2, 64, box_rows,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  DmParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.seq_lens = seq_lens;
  p.Hkv = Hkv;
  p.G = Hq / Hkv;
  p.block_size = block_size;
  p.scale = scale;
  p.num_splits = num_splits;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.status = status;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DM_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(B, Hkv, num_splits);
  rlb_launch_pdl(paged_decode_mma_kernel, grid, dim3(DM_THREADS), DM_SMEM, s, tk, tv, p);
  if (num_splits > 1) {
    dim3 g2(B, Hq);
    rlb_launch_pdl(dm_combine_kernel, g2, dim3(DM_D), 0, s, part_o, part_ml, num_splits, Hq, static_cast<__nv_bfloat16*>(out), out_stride);
  }
  return static_cast<int>(cudaGetLastError());
}
