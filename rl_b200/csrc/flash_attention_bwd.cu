// Backward of the packed causal attention (see flash_attention.cu for the forward and the data layout).
//
// Two kernels, no atomics, S and P recomputed from Q, K and the saved log-sum-exp:
//   flash_bwd_dq_kernel   one CTA per (128-row query tile, query head); loops over 64-key tiles:
//                         S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale, dQ += dS K
//   flash_bwd_dkv_kernel  one CTA per (128-key tile, kv head); loops over the G query heads of the group and over
//                         64-row query tiles at or below the diagonal, working on transposed tiles so that the key
//                         index is the TMEM lane: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q
// All five products run on tcgen05 with fp32 accumulators in TMEM. A tile loaded by TMA with the 128-byte swizzle
// ([rows x 64 columns] boxes) serves both as a K-major and as an MN-major operand: the bytes are the same, only the
// shared-memory descriptor differs, so Q, K, V and dO are each loaded once per use.
// delta[h, t] = sum_d dO * O is computed beforehand by rlb_attn_delta.
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

#ifndef RLB_HD
#define RLB_HD 128        // head dimension of this translation unit; flash_attention_bwd_d64.cu includes this file with 64
#endif
#ifndef RLB_NAME
#define RLB_NAME(x) x
#endif
constexpr int HD = RLB_HD;
static_assert(HD == 64 || HD == 128, "head dimension: 64 or 128");
constexpr int ATOMS = HD / 64;   // [rows x 64] swizzle atoms per operand tile along the head dimension
constexpr float LOG2E = 1.4426950408889634f;
constexpr int BWD_THREADS = 192;

__device__ bool locate_tile_b(const int* __restrict__ cu, int num_seqs, int rows, int tile, int& start, int& len,
                              int& tile_in_seq) {
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int n = (e - b + rows - 1) / rows;
    if (tile < acc + n) {
      start = b;
      len = e - b;
      tile_in_seq = tile - acc;
      return true;
    }
    acc += n;
  }
  return false;
}
__device__ __forceinline__ void st_swz(uint8_t* atom, int r, int c, uint4 v) {
  *reinterpret_cast<uint4*>(atom + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct BwdParams {
  const int* cu_seqlens;
  int num_seqs;
  int T;
  int Hq, Hkv;
  float scale;
  float scale_log2;
  const float* lse;    // [Hq, T] natural log
  const float* delta;  // [Hq, T]
  __nv_bfloat16* dqkv;
  long long dqkv_stride;
  int* status;
};

// ------------------------------------------------------------------------------------------------ dQ
constexpr int DQ_BQ = 128, DQ_BKV = 64;
constexpr int DQ_Q_BYTES = DQ_BQ * HD * 2;     // 32 KB
constexpr int DQ_KV_BYTES = DQ_BKV * HD * 2;   // 16 KB
constexpr int DQ_Q_ATOM = DQ_BQ * 128, DQ_KV_ATOM = DQ_BKV * 128;   // bytes of one [rows x 64] bf16 atom
constexpr int DQ_DS_BYTES = DQ_BQ * DQ_BKV * 2;  // 16 KB
constexpr int DQ_SMEM = 2 * DQ_Q_BYTES + 4 * DQ_KV_BYTES + DQ_DS_BYTES + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                    const __grid_constant__ CUtensorMap tmap_do, BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* do_s = q_s + DQ_Q_BYTES;
  uint8_t* k_s = do_s + DQ_Q_BYTES;
  uint8_t* v_s = k_s + 2 * DQ_KV_BYTES;
  uint8_t* ds_s = v_s + 2 * DQ_KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + DQ_DS_BYTES);
  uint64_t* q_full = bars;        // Q and dO
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* dq_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* info = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  if (threadIdx.x == 0) {
    int start = 0, len = 0, tis = 0;
    const bool ok = locate_tile_b(p.cu_seqlens, p.num_seqs, DQ_BQ, blockIdx.x, start, len, tis) &&
                    (smem_u32(smem) & 1023u) == 0;
    info[0] = start; info[1] = len; info[2] = tis; info[3] = ok ? 1 : 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(dq_done), 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (!info[3]) return;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 64, tmem_dq = tmem_base + 128;
  const int seq_start = info[0], seq_len = info[1];
  const int q0 = info[2] * DQ_BQ;
  const int q_rows = min(DQ_BQ, seq_len - q0);
  const int n_kv = (q0 + q_rows + DQ_BKV - 1) / DQ_BKV;
  const int q_col = head * HD, k_col = (p.Hq + kv_head) * HD, v_col = (p.Hq + p.Hkv + kv_head) * HD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(q_full), 2 * DQ_Q_BYTES);
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_2d(smem_u32(q_s + a * DQ_Q_ATOM), &tmap_q, smem_u32(q_full), q_col + a * 64, seq_start + q0);
        tma_load_2d(smem_u32(do_s + a * DQ_Q_ATOM), &tmap_do, smem_u32(q_full), head * HD + a * 64, seq_start + q0);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[st]), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) break;
        const int row = seq_start + j * DQ_BKV;
        mbar_arrive_expect_tx(smem_u32(&kv_full[st]), 2 * DQ_KV_BYTES);
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_2d(smem_u32(k_s + st * DQ_KV_BYTES + a * DQ_KV_ATOM), &tmap_kv, smem_u32(&kv_full[st]), k_col + a * 64, row);
          tma_load_2d(smem_u32(v_s + st * DQ_KV_BYTES + a * DQ_KV_ATOM), &tmap_kv, smem_u32(&kv_full[st]), v_col + a * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(DQ_BQ, DQ_BKV, false, false);
      constexpr uint32_t idesc_dq = make_idesc_bf16(DQ_BQ, HD, false, true);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, RLB_ERR_WAIT_FULL);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&kv_full[st]), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off_a = (kk / 4) * DQ_Q_ATOM + (kk % 4) * 32;
          const uint32_t off_b = (kk / 4) * DQ_KV_ATOM + (kk % 4) * 32;
          umma_f16(tmem_s, make_smem_desc_sw128(smem_u32(q_s) + off_a, 16, 1024),
                   make_smem_desc_sw128(smem_u32(k_s + st * DQ_KV_BYTES) + off_b, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off_a = (kk / 4) * DQ_Q_ATOM + (kk % 4) * 32;
          const uint32_t off_b = (kk / 4) * DQ_KV_ATOM + (kk % 4) * 32;
          umma_f16(tmem_dp, make_smem_desc_sw128(smem_u32(do_s) + off_a, 16, 1024),
                   make_smem_desc_sw128(smem_u32(v_s + st * DQ_KV_BYTES) + off_b, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(s_full));
        if (!mbar_wait(smem_u32(p_full), j & 1, abort_flag, p.status, RLB_ERR_WAIT_FLAG)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DQ_BKV / 16; ++kk) {
          umma_f16(tmem_dq, make_smem_desc_sw128(smem_u32(ds_s) + kk * 32, 16, 1024),
                   make_smem_desc_sw128(smem_u32(k_s + st * DQ_KV_BYTES) + kk * 2048, DQ_KV_ATOM, 1024), idesc_dq,
                   (j | kk) != 0);
        }
        umma_commit(smem_u32(&kv_empty[st]));
        umma_commit(smem_u32(dq_done));
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + r;
    const bool row_ok = r < q_rows;
    const long long stat_idx = static_cast<long long>(head) * p.T + seq_start + qi;
    const float lse2 = row_ok ? p.lse[stat_idx] * LOG2E : 0.f;
    const float dlt = row_ok ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(smem_u32(s_full), j & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int k0 = j * DQ_BKV;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], dpv[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c * 32, s);
        tmem_ld_32x32b_x32(tmem_dp + lane_addr + c * 32, dpv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float d2[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col = c * 32 + 2 * i + h;
            const bool keep = row_ok && (k0 + col <= qi);
            const float pr = keep ? exp2f(__uint_as_float(s[2 * i + h]) * p.scale_log2 - lse2) : 0.f;
            d2[h] = pr * (__uint_as_float(dpv[2 * i + h]) - dlt) * p.scale;
          }
          pk[c * 16 + i] = pack_bf16x2(d2[0], d2[1]);
        }
      }
      if (j > 0) {
        if (!mbar_wait(smem_u32(dq_done), (j - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) st_swz(ds_s, r, c, make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]));
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok && mbar_wait(smem_u32(dq_done), (n_kv - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dqkv + static_cast<long long>(seq_start + qi) * p.dqkv_stride + q_col;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_dq + lane_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]), __uint_as_float(o[q * 8 + 1]));
            v.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]), __uint_as_float(o[q * 8 + 3]));
            v.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]), __uint_as_float(o[q * 8 + 5]));
            v.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]), __uint_as_float(o[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------ dK / dV
constexpr int KV_BKV = 128, KV_BQ = 64;
constexpr int KV_K_BYTES = KV_BKV * HD * 2;      // 32 KB (two [128 x 64] atoms)
constexpr int KV_Q_BYTES = KV_BQ * HD * 2;       // 16 KB (two [64 x 64] atoms)
constexpr int KV_K_ATOM = KV_BKV * 128, KV_Q_ATOM = KV_BQ * 128;
constexpr int KV_P_BYTES = KV_BKV * KV_BQ * 2;   // 16 KB (one [128 x 64] atom)
constexpr int KV_STAT_BYTES = 2 * 2 * KV_BQ * 4; // lse2 / delta of the 64 query rows, double buffered
constexpr int KV_SMEM = 2 * KV_K_BYTES + 4 * KV_Q_BYTES + 2 * KV_P_BYTES + KV_STAT_BYTES + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_kv128, const __grid_constant__ CUtensorMap tmap_q64,
                     const __grid_constant__ CUtensorMap tmap_do64, BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + KV_K_BYTES;
  uint8_t* q_s = v_s + KV_K_BYTES;            // [2 stages]
  uint8_t* do_s = q_s + 2 * KV_Q_BYTES;       // [2 stages]
  uint8_t* pt_s = do_s + 2 * KV_Q_BYTES;      // P^T
  uint8_t* dst_s = pt_s + KV_P_BYTES;         // dS^T
  float* stat_s = reinterpret_cast<float*>(dst_s + KV_P_BYTES);  // [2][2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stat_s) + KV_STAT_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* info = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  if (threadIdx.x == 0) {
    int start = 0, len = 0, tis = 0;
    const bool ok = locate_tile_b(p.cu_seqlens, p.num_seqs, KV_BKV, blockIdx.x, start, len, tis) &&
                    (smem_u32(smem) & 1023u) == 0;
    info[0] = start; info[1] = len; info[2] = tis; info[3] = ok ? 1 : 0;
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&qdo_full[s]), 1);
      mbar_init(smem_u32(&qdo_empty[s]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(acc_done), 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (!info[3]) return;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_st = tmem_base, tmem_dpt = tmem_base + 64, tmem_dv = tmem_base + 128, tmem_dk = tmem_base + 256;
  const int seq_start = info[0], seq_len = info[1];
  const int kv0 = info[2] * KV_BKV;
  const int kv_rows = min(KV_BKV, seq_len - kv0);
  const int qt_first = kv0 / KV_BQ;                           // first 64-row query tile at or below the diagonal
  const int qt_count = (seq_len + KV_BQ - 1) / KV_BQ - qt_first;
  const int n_iter = qt_count * G;                            // (query head of the group, query tile) pairs
  const int k_col = (p.Hq + kv_head) * HD, v_col = (p.Hq + p.Hkv + kv_head) * HD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(kv_full), 2 * KV_K_BYTES);
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_2d(smem_u32(k_s + a * KV_K_ATOM), &tmap_kv128, smem_u32(kv_full), k_col + a * 64, seq_start + kv0);
        tma_load_2d(smem_u32(v_s + a * KV_K_ATOM), &tmap_kv128, smem_u32(kv_full), v_col + a * 64, seq_start + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(smem_u32(&qdo_empty[st]), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) break;
        const int g = it / qt_count, qt = qt_first + it % qt_count;
        const int head = kv_head * G + g;
        const int row = seq_start + qt * KV_BQ;
        mbar_arrive_expect_tx(smem_u32(&qdo_full[st]), 2 * KV_Q_BYTES);
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_2d(smem_u32(q_s + st * KV_Q_BYTES + a * KV_Q_ATOM), &tmap_q64, smem_u32(&qdo_full[st]), head * HD + a * 64, row);
          tma_load_2d(smem_u32(do_s + st * KV_Q_BYTES + a * KV_Q_ATOM), &tmap_do64, smem_u32(&qdo_full[st]), head * HD + a * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(KV_BKV, KV_BQ, false, false);  // [128 keys] x [64 queries]
      constexpr uint32_t idesc_acc = make_idesc_bf16(KV_BKV, HD, false, true);     // += [128 x 64] * [64 x 128]
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, p.status, RLB_ERR_WAIT_FULL);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(smem_u32(&qdo_full[st]), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off_a = (kk / 4) * KV_K_ATOM + (kk % 4) * 32;
          const uint32_t off_b = (kk / 4) * KV_Q_ATOM + (kk % 4) * 32;
          umma_f16(tmem_st, make_smem_desc_sw128(smem_u32(k_s) + off_a, 16, 1024),
                   make_smem_desc_sw128(smem_u32(q_s + st * KV_Q_BYTES) + off_b, 16, 1024), idesc_st, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off_a = (kk / 4) * KV_K_ATOM + (kk % 4) * 32;
          const uint32_t off_b = (kk / 4) * KV_Q_ATOM + (kk % 4) * 32;
          umma_f16(tmem_dpt, make_smem_desc_sw128(smem_u32(v_s) + off_a, 16, 1024),
                   make_smem_desc_sw128(smem_u32(do_s + st * KV_Q_BYTES) + off_b, 16, 1024), idesc_st, kk != 0);
        }
        umma_commit(smem_u32(s_full));
        if (!mbar_wait(smem_u32(p_full), it & 1, abort_flag, p.status, RLB_ERR_WAIT_FLAG)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KV_BQ / 16; ++kk) {
          // the query tile read as an MN-major operand: 16 query rows per step, 64-column groups 8 KB apart
          umma_f16(tmem_dv, make_smem_desc_sw128(smem_u32(pt_s) + kk * 32, 16, 1024),
                   make_smem_desc_sw128(smem_u32(do_s + st * KV_Q_BYTES) + kk * 2048, KV_Q_ATOM, 1024), idesc_acc,
                   (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < KV_BQ / 16; ++kk) {
          umma_f16(tmem_dk, make_smem_desc_sw128(smem_u32(dst_s) + kk * 32, 16, 1024),
                   make_smem_desc_sw128(smem_u32(q_s + st * KV_Q_BYTES) + kk * 2048, KV_Q_ATOM, 1024), idesc_acc,
                   (it | kk) != 0);
        }
        umma_commit(smem_u32(&qdo_empty[st]));
        umma_commit(smem_u32(acc_done));
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;   // key row of this thread
    const int ct = threadIdx.x - 64;     // 0..127 among the consumer threads
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int kj = kv0 + r;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int g = it / qt_count, qt = qt_first + it % qt_count;
      const int head = kv_head * G + g;
      const int qbase = qt * KV_BQ;
      float* st_lse = stat_s + (it & 1) * 2 * KV_BQ;
      float* st_dlt = st_lse + KV_BQ;
      {  // statistics of the 64 query rows (threads 0..63: lse, 64..127: delta)
        const int c = ct & 63;
        const int qi = qbase + c;
        const long long idx = static_cast<long long>(head) * p.T + seq_start + qi;
        const bool in = qi < seq_len;
        if (ct < 64) st_lse[c] = in ? p.lse[idx] * LOG2E : 0.f;
        else st_dlt[c] = in ? p.delta[idx] : 0.f;
      }
      named_bar_sync(1, 128);
      if (!mbar_wait(smem_u32(s_full), it & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t pp[32], dd[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], dpv[32];
        tmem_ld_32x32b_x32(tmem_st + lane_addr + c * 32, s);
        tmem_ld_32x32b_x32(tmem_dpt + lane_addr + c * 32, dpv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float pv[2], dv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int col = c * 32 + 2 * i + h;
            const int qi = qbase + col;
            const bool keep = (qi >= kj) && (qi < seq_len) && (r < kv_rows);
            pv[h] = keep ? exp2f(__uint_as_float(s[2 * i + h]) * p.scale_log2 - st_lse[col]) : 0.f;
            dv[h] = pv[h] * (__uint_as_float(dpv[2 * i + h]) - st_dlt[col]) * p.scale;
          }
          pp[c * 16 + i] = pack_bf16x2(pv[0], pv[1]);
          dd[c * 16 + i] = pack_bf16x2(dv[0], dv[1]);
        }
      }
      if (it > 0) {
        if (!mbar_wait(smem_u32(acc_done), (it - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        st_swz(pt_s, r, c, make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]));
        st_swz(dst_s, r, c, make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]));
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok && n_iter > 0 && mbar_wait(smem_u32(acc_done), (n_iter - 1) & 1, abort_flag, p.status, RLB_ERR_WAIT_TMEM_EMPTY)) {
      tc_fence_after();
      const bool row_ok = r < kv_rows;
      __nv_bfloat16* dk_dst = p.dqkv + static_cast<long long>(seq_start + kj) * p.dqkv_stride + k_col;
      __nv_bfloat16* dv_dst = p.dqkv + static_cast<long long>(seq_start + kj) * p.dqkv_stride + v_col;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tmem_dk : tmem_dv;
        __nv_bfloat16* dst = which == 0 ? dk_dst : dv_dst;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(src + lane_addr + c * 32, o);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]), __uint_as_float(o[q * 8 + 1]));
              v.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]), __uint_as_float(o[q * 8 + 3]));
              v.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]), __uint_as_float(o[q * 8 + 5]));
              v.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]), __uint_as_float(o[q * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = v;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int g_bwd_configured = 0;

}  // namespace

// dqkv[T, (Hq+2Hkv)*128] = gradient of the packed causal attention w.r.t. the fused [q | k | v] buffer.
// lse and delta are [Hq, T] fp32 (lse from the forward pass, delta from rlb_attn_delta).
// max_q_tiles / max_kv_tiles: upper bounds on the number of 128-row tiles (ceil(T/128) + num_seqs is enough for both).
RLB_API int RLB_NAME(rlb_flash_attn_bwd)(const void* qkv, long long qkv_stride, const void* dout, long long do_stride,
                               const float* lse, const float* delta, const int* cu_seqlens, int num_seqs, int T, int Hq,
                               int Hkv, int D, float scale, void* dqkv, long long dqkv_stride, int max_q_tiles,
                               int max_kv_tiles, int* status, void* stream) {
  if (T <= 0 || num_seqs <= 0) return 0;
  if (D != HD || Hq % Hkv || qkv_stride % 8 || do_stride % 8 || dqkv_stride % 8) return -2;
  const long long C = static_cast<long long>(Hq + 2 * Hkv) * HD;
  CUtensorMap tq128, tq64, tkv64, tkv128, tdo128, tdo64;
  int rc = 0;
  rc |= rlb_make_tmap_2d(&tq128, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, T, qkv_stride * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  rc |= rlb_make_tmap_2d(&tq64, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, T, qkv_stride * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  tkv64 = tq64;
  tkv128 = tq128;
  rc |= rlb_make_tmap_2d(&tdo128, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<long long>(Hq) * HD, T, do_stride * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  rc |= rlb_make_tmap_2d(&tdo64, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<long long>(Hq) * HD, T, do_stride * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  if (!g_bwd_configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_bwd_configured = 1;
  }
  BwdParams p;
  p.cu_seqlens = cu_seqlens;
  p.num_seqs = num_seqs;
  p.T = T;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.lse = lse;
  p.delta = delta;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.dqkv_stride = dqkv_stride;
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  flash_bwd_dq_kernel<<<dim3(max_q_tiles, Hq), BWD_THREADS, DQ_SMEM, s>>>(tq128, tkv64, tdo128, p);
  flash_bwd_dkv_kernel<<<dim3(max_kv_tiles, Hkv), BWD_THREADS, KV_SMEM, s>>>(tkv128, tq64, tdo64, p);
  return static_cast<int>(cudaGetLastError());
}
