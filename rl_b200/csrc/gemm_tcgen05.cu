// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands staged
// by TMA into 128B-swizzled shared memory).
//
//   C[M,N] = op(A) * op(B)^T      A: [M,K] (K-major) or stored as [K,M] (MN-major)
//                                  B: [N,K] (K-major) or stored as [K,N] (MN-major)
//
// The three operand layouts cover a linear layer's forward (K,K), input gradient (K,MN) and
// weight gradient (MN,MN) without transposing anything in memory.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + tcgen05.mma issuer (one elected lane)
//   warps 2..5  epilogue: tcgen05.ld -> registers -> global
// A 4-deep shared-memory ring feeds 128x256x16 MMAs; two 256-column TMEM accumulators let the
// epilogue of tile i overlap the main loop of tile i+1.
//
// Epilogues:
//   EPI_STORE    C = acc (+ bias) (+ C), bf16 or fp32
//   EPI_LOGPROB  for a vocab projection: per (row, n-tile) online-softmax partials (max, sum-exp,
//                sum of z*exp) and the target logit; logits are never written. A small second
//                kernel folds the partials into logprob / entropy / logsumexp per row.
//   EPI_DLOGITS  recomputes the logits tile and writes coef[row]*(onehot - softmax)*inv_temp in
//                bf16, the gradient that the dH / dW GEMMs consume.
// Replaces the cuBLAS calls behind nn.Linear and the chunked hidden->logprob path of the reference
// (nemo_rl/distributed/model_utils.py:2137-2316).
#include "common.cuh"

#include <cstdlib>

#include <math.h>
#include <stdio.h>

namespace {

using namespace rlb;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BARRIER_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SMEM_BARRIER_BYTES + 1024;  // +1024: manual alignment
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;  // rasterisation: 16 m-tiles share each sweep over n

enum { EPI_STORE = 0, EPI_LOGPROB = 1, EPI_DLOGITS = 2 };

struct EpiParams {
  void* C;              // output (EPI_STORE, EPI_DLOGITS)
  long long ldc;        // leading dimension of C in elements
  const float* bias;    // [N] or null
  const void* residual; // bf16 [M, ldr] added to the result (the residual stream), or null
  long long ldr;
  int out_fp32;         // EPI_STORE: 1 -> fp32 output
  int accumulate;       // EPI_STORE: 1 -> C += acc
  // vocab-projection epilogues
  const int* targets;   // [M] target column per row (global vocab id - vocab_offset), <0 or >=N: not here
  float inv_temp;
  float* part_max;      // [num_n_tiles, M]
  float* part_sum;      // [num_n_tiles, M]
  float* part_zsum;     // [num_n_tiles, M]
  float* target_logit;  // [M], written only by the tile that owns the target column
  const float* lse;     // [M] log-sum-exp of the scaled logits (EPI_DLOGITS)
  const float* coef;    // [M] upstream gradient of the log-probability (EPI_DLOGITS)
  const float* ent_coef;  // [M] upstream gradient of the entropy, or null (EPI_DLOGITS)
  const float* entropy;   // [M] entropy per row, needed with ent_coef
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 int M, int N, int K, EpiParams ep, int* status) {
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle needs 1024-byte aligned stage buffers.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_k = (K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, num_m, num_n, m_blk, n_blk);
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, status, RLB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(a_dst, &tmap_a, bar, kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(a_dst + j * (BK * 128), &tmap_a, bar, m_blk * BM + j * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmap_b, bar, kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * (BK * 128), &tmap_b, bar, n_blk * BN + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t stage = 0, phase = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, status, RLB_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, status, RLB_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t a_desc = A_MN ? make_smem_desc_sw128(a_addr, BK * 128, 1024)
                                       : make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr, BK * 128, 1024)
                                       : make_smem_desc_sw128(b_addr, 16, 1024);
          // Advance along K inside the stage: 32 B per MMA for a K-major tile (inside the swizzle
          // atom), 16 k-rows of 128 B for an MN-major tile.
          constexpr uint32_t a_step = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
          constexpr uint32_t b_step = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_f16(tmem_d, a_desc + kk * a_step, b_desc + kk * b_step, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // stage reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(smem_u32(&tfull_bar[acc]));  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, status, RLB_ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const int col0 = n_blk * BN;

      if (EPI == EPI_STORE) {
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = col0 + c * 32;
          if (!row_ok || col >= N) continue;
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (ep.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < N) v[i] += ep.bias[col + i];
          }
          if (ep.residual) {
            const __nv_bfloat16* rsd =
                reinterpret_cast<const __nv_bfloat16*>(ep.residual) + static_cast<long long>(row) * ep.ldr + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < N) {
                const uint4 old = *reinterpret_cast<const uint4*>(rsd + q * 8);
                const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
                             o3 = unpack_bf16x2(old.w);
                v[q * 8 + 0] += o0.x; v[q * 8 + 1] += o0.y; v[q * 8 + 2] += o1.x; v[q * 8 + 3] += o1.y;
                v[q * 8 + 4] += o2.x; v[q * 8 + 5] += o2.y; v[q * 8 + 6] += o3.x; v[q * 8 + 7] += o3.y;
              }
            }
          }
          if (ep.out_fp32) {
            float* dst = reinterpret_cast<float*>(ep.C) + static_cast<long long>(row) * ep.ldc + col;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (col + q * 4 < N) {  // N is a multiple of 8
                float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                if (ep.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + q * 4);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + q * 4) = o;
              }
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(ep.C) + static_cast<long long>(row) * ep.ldc + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < N) {
                if (ep.accumulate) {
                  const uint4 old = *reinterpret_cast<const uint4*>(dst + q * 8);
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y),
                               o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
                  v[q * 8 + 0] += o0.x; v[q * 8 + 1] += o0.y; v[q * 8 + 2] += o1.x; v[q * 8 + 3] += o1.y;
                  v[q * 8 + 4] += o2.x; v[q * 8 + 5] += o2.y; v[q * 8 + 6] += o3.x; v[q * 8 + 7] += o3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(dst + q * 8) = o;
              }
            }
          }
        }
      } else if (EPI == EPI_LOGPROB) {
        // Online softmax statistics of this row over the tile's columns.
        float mx = -INFINITY, sum = 0.f, zsum = 0.f;
        const int tgt = row_ok ? ep.targets[row] : -1;
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = col0 + c * 32;
          if (col >= N) continue;
          float cmax = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float z = __uint_as_float(r[i]) * ep.inv_temp;
            r[i] = __float_as_uint(z);
            if (col + i < N) cmax = fmaxf(cmax, z);
          }
          const float nmx = fmaxf(mx, cmax);
          const float scale = __expf(mx - nmx);  // exp(-inf) = 0 on the first chunk
          sum *= scale;
          zsum *= scale;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col + i < N) {
              const float z = __uint_as_float(r[i]);
              const float e = __expf(z - nmx);
              sum += e;
              zsum += z * e;
              if (col + i == tgt) ep.target_logit[row] = z;
            }
          }
          mx = nmx;
        }
        if (row_ok) {
          const long long idx = static_cast<long long>(n_blk) * M + row;
          ep.part_max[idx] = mx;
          ep.part_sum[idx] = sum;
          ep.part_zsum[idx] = zsum;
        }
      } else {  // EPI_DLOGITS
        const int tgt = row_ok ? ep.targets[row] : -1;
        const float lse = row_ok ? ep.lse[row] : 0.f;
        const float g = row_ok ? ep.coef[row] : 0.f;
        const float ge = (row_ok && ep.ent_coef) ? ep.ent_coef[row] : 0.f;
        const float ent = (row_ok && ep.ent_coef) ? ep.entropy[row] : 0.f;
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = col0 + c * 32;
          if (!row_ok || col >= N) continue;
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float z = __uint_as_float(r[i]) * ep.inv_temp;
            const float logp = z - lse;
            const float p = __expf(logp);
            // d logprob_t / dz_j = 1[j=t] - p_j ;  dH/dz_j = -p_j (logp_j + H)
            float d = g * ((col + i == tgt ? 1.f : 0.f) - p);
            d -= ge * p * (logp + ent);
            v[i] = d * ep.inv_temp;
          }
          __nv_bfloat16* dst =
              reinterpret_cast<__nv_bfloat16*>(ep.C) + static_cast<long long>(row) * ep.ldc + col;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col + q * 8 < N) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(dst + q * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Folds the per-n-tile partials of EPI_LOGPROB into per-row results.
__global__ void logprob_combine_kernel(const float* __restrict__ part_max, const float* __restrict__ part_sum,
                                       const float* __restrict__ part_zsum,
                                       const float* __restrict__ target_logit, int M, int num_parts,
                                       float* __restrict__ logprob, float* __restrict__ entropy,
                                       float* __restrict__ lse_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float mx = -INFINITY;
  for (int p = 0; p < num_parts; ++p) mx = fmaxf(mx, part_max[static_cast<long long>(p) * M + row]);
  float sum = 0.f, zsum = 0.f;
  for (int p = 0; p < num_parts; ++p) {
    const long long i = static_cast<long long>(p) * M + row;
    const float s = __expf(part_max[i] - mx);
    sum += part_sum[i] * s;
    zsum += part_zsum[i] * s;
  }
  const float lse = mx + logf(sum);
  if (lse_out) lse_out[row] = lse;
  if (logprob) logprob[row] = target_logit[row] - lse;
  if (entropy) entropy[row] = lse - zsum / sum;  // H = lse - E[z]
}

int g_sm_count = 0;

template <bool A_MN, bool B_MN, int EPI>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, int M, int N, int K, const EpiParams& ep,
                int* status, int max_ctas, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = num_tiles < g_sm_count ? num_tiles : g_sm_count;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, M, N, K, ep, status);
  return static_cast<int>(cudaGetLastError());
}

template <int EPI>
int dispatch_layout(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, int M, int N, int K,
                    const EpiParams& ep, int* status, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm<false, false, EPI>(ta, tb, M, N, K, ep, status, max_ctas, stream);
  if (!a_mn && b_mn) return launch_gemm<false, true, EPI>(ta, tb, M, N, K, ep, status, max_ctas, stream);
  if (a_mn && b_mn) return launch_gemm<true, true, EPI>(ta, tb, M, N, K, ep, status, max_ctas, stream);
  return launch_gemm<true, false, EPI>(ta, tb, M, N, K, ep, status, max_ctas, stream);
}

int make_operand_maps(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                      bool a_mn, bool b_mn, CUtensorMap* ta, CUtensorMap* tb) {
  int rc;
  if (!a_mn)
    rc = rlb_make_tmap_2d(ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, BK, BM,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = rlb_make_tmap_2d(ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, 64, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if (!b_mn)
    rc = rlb_make_tmap_2d(tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, BK, BN,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = rlb_make_tmap_2d(tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, 64, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  return rc;
}

}  // namespace

// ---------------------------------------------------------------- host helpers (shared by all .cu files)
bool rlb_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("RLB_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

RlbEncodeTiledFn rlb_get_encode_tiled() {
  static RlbEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<RlbEncodeTiledFn>(p);
  }
  return fn;
}

int rlb_make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                     uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                     uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  RlbEncodeTiledFn enc = rlb_get_encode_tiled();
  if (!enc) return -1;
  (void)elem_bytes;
  // The driver call needs the primary context current on the calling thread. Threads that have made
  // no runtime call yet (autograd's backward threads) get it bound by a no-op runtime call.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// ---------------------------------------------------------------- C API
// C = op(A) op(B)^T (+bias) (+C). lda/ldb/ldc in elements; all of them, and the base pointers, must
// keep 16-byte alignment (multiples of 8 elements for bf16). Returns 0, a CUDA error, or a negative
// code for bad arguments.
RLB_API int rlb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                          long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_fp32,
                          int accumulate, const float* bias, const void* residual, long long ldr, int* status,
                          int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8)) || (N % 8)) return -2;
  if (residual && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  CUtensorMap ta, tb;
  int rc = make_operand_maps(A, B, M, N, K, lda, ldb, a_mn_major != 0, b_mn_major != 0, &ta, &tb);
  if (rc) return -100 - rc;
  EpiParams ep{};
  ep.C = C;
  ep.ldc = ldc;
  ep.bias = bias;
  ep.residual = residual;
  ep.ldr = ldr;
  ep.out_fp32 = out_fp32;
  ep.accumulate = accumulate;
  return dispatch_layout<EPI_STORE>(a_mn_major != 0, b_mn_major != 0, ta, tb, M, N, K, ep, status, max_ctas,
                                    static_cast<cudaStream_t>(stream));
}

// Number of n-tiles the vocab-projection epilogues split N into (size of the partial buffers).
RLB_API int rlb_gemm_num_n_tiles(int N) { return (N + BN - 1) / BN; }

// Fused vocab projection + log-softmax statistics: H[M,K] x W[N,K]^T, logits never stored.
// part_* are scratch of num_n_tiles*M floats each; target_logit is scratch of M floats.
// Outputs (any may be null): logprob[M], entropy[M], lse[M].
RLB_API int rlb_lm_head_logprob(const void* H, const void* W, int M, int N, int K, long long ldh, long long ldw,
                                const int* targets, float inv_temp, float* part_max, float* part_sum,
                                float* part_zsum, float* target_logit, float* logprob, float* entropy,
                                float* lse, int* status, void* stream) {
  if (M <= 0) return 0;
  if ((ldh % 8) || (ldw % 8)) return -2;
  CUtensorMap ta, tb;
  int rc = make_operand_maps(H, W, M, N, K, ldh, ldw, false, false, &ta, &tb);
  if (rc) return -100 - rc;
  EpiParams ep{};
  ep.targets = targets;
  ep.inv_temp = inv_temp;
  ep.part_max = part_max;
  ep.part_sum = part_sum;
  ep.part_zsum = part_zsum;
  ep.target_logit = target_logit;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rc = launch_gemm<false, false, EPI_LOGPROB>(ta, tb, M, N, K, ep, status, 0, s);
  if (rc) return rc;
  const int parts = (N + BN - 1) / BN;
  logprob_combine_kernel<<<(M + 255) / 256, 256, 0, s>>>(part_max, part_sum, part_zsum, target_logit, M, parts,
                                                          logprob, entropy, lse);
  return static_cast<int>(cudaGetLastError());
}

// Folds partials only (used by the vocab-parallel path after the cross-rank exchange).
RLB_API int rlb_logprob_combine(const float* part_max, const float* part_sum, const float* part_zsum,
                                const float* target_logit, int M, int parts, float* logprob, float* entropy,
                                float* lse, void* stream) {
  if (M <= 0) return 0;
  logprob_combine_kernel<<<(M + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      part_max, part_sum, part_zsum, target_logit, M, parts, logprob, entropy, lse);
  return static_cast<int>(cudaGetLastError());
}

// Statistics pass only: writes the partials and the target logit, no combine. For a vocab-parallel
// lm_head each rank runs this on its shard; the partials are then exchanged and folded.
RLB_API int rlb_lm_head_partials(const void* H, const void* W, int M, int N, int K, long long ldh,
                                 long long ldw, const int* targets, float inv_temp, float* part_max,
                                 float* part_sum, float* part_zsum, float* target_logit, int* status,
                                 void* stream) {
  if (M <= 0) return 0;
  if ((ldh % 8) || (ldw % 8)) return -2;
  CUtensorMap ta, tb;
  int rc = make_operand_maps(H, W, M, N, K, ldh, ldw, false, false, &ta, &tb);
  if (rc) return -100 - rc;
  EpiParams ep{};
  ep.targets = targets;
  ep.inv_temp = inv_temp;
  ep.part_max = part_max;
  ep.part_sum = part_sum;
  ep.part_zsum = part_zsum;
  ep.target_logit = target_logit;
  return launch_gemm<false, false, EPI_LOGPROB>(ta, tb, M, N, K, ep, status, 0, static_cast<cudaStream_t>(stream));
}

// Backward of the fused projection: recomputes logits tile by tile and writes
// dZ[M,N] = (coef*(onehot - p) - ent_coef * p * (logp + H)) * inv_temp in bf16.
RLB_API int rlb_lm_head_dlogits(const void* H, const void* W, void* dZ, int M, int N, int K, long long ldh,
                                long long ldw, long long lddz, const int* targets, float inv_temp,
                                const float* lse, const float* coef, const float* ent_coef,
                                const float* entropy, int* status, void* stream) {
  if (M <= 0) return 0;
  if ((ldh % 8) || (ldw % 8) || (lddz % 8) || (N % 8)) return -2;
  CUtensorMap ta, tb;
  int rc = make_operand_maps(H, W, M, N, K, ldh, ldw, false, false, &ta, &tb);
  if (rc) return -100 - rc;
  EpiParams ep{};
  ep.C = dZ;
  ep.ldc = lddz;
  ep.targets = targets;
  ep.inv_temp = inv_temp;
  ep.lse = lse;
  ep.coef = coef;
  ep.ent_coef = ent_coef;
  ep.entropy = entropy;
  return launch_gemm<false, false, EPI_DLOGITS>(ta, tb, M, N, K, ep, status, 0, static_cast<cudaStream_t>(stream));
}
