// Grouped GEMM for mixture-of-experts layers (sm_100a, tcgen05 + TMEM + TMA, persistent CTAs).
//
// Tokens routed to the experts of this rank sit in one buffer sorted by expert, every expert's segment padded with
// zero rows to a multiple of 128, so that each 128-row m-tile belongs to exactly one expert. Two kernels cover the
// six GEMMs of an expert MLP:
//
//   rows mode       C[Mpad, N] = A[Mpad, K] * op(B[e(m_tile)])        forward (gate_up, down) and the input gradient
//                   B stacked as [E, N, K] (b_mn = 0, C = A B^T) or [E, K, N] (b_mn = 1, C = A B)
//   reduction mode  C[e][M, N] (+)= A[rows of e, M]^T * B[rows of e, N]   weight gradients: the reduction runs over the
//                   expert's (padded) rows, outputs are stacked per expert
//
// The tile -> expert map (`tile_expert`, -1 for unused tail tiles) and the per-expert row ranges live in device memory,
// produced from the router's histogram without a host round trip; the grid is sized for the worst case and CTAs skip
// tiles that are not in use. One launch replaces the per-expert loop of cuBLAS calls (nv-grouped-gemm / TE grouped
// linear in the reference's Megatron path, nemo_rl/models/megatron/setup.py:888-1023).
#include "common.cuh"

namespace {
using namespace rlb;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

struct GroupedArgs {
  int mode;                 // 0 rows, 1 reduction
  int M, N, K;              // rows: M = padded rows (upper bound), N, K per expert; reduction: M, N of one expert's output
  int num_experts;
  const int* tile_expert;   // rows mode: [ceil(M/128)] expert of each m-tile, -1 = unused
  const int* expert_row0;   // reduction mode: [E] first padded row of each expert
  const int* expert_rows;   // reduction mode: [E] padded row count (multiple of 128; 0 = expert unused)
  void* C;
  long long ldc;
  long long c_expert_stride;  // reduction mode: elements between consecutive experts' outputs
  int out_fp32;
  int accumulate;
};

// One unit of work: which tile, which k range, where B / C start.
struct Work {
  int m_blk, n_blk;
  int a_row0;      // rows mode: first row of A tile; reduction: first reduction row
  int num_k;
  int b_row0;      // row offset of this expert inside the stacked B tensor map (rows mode)
  long long c_off; // element offset of the output tile's expert slab
  bool valid;
};

template <bool B_MN>
__device__ __forceinline__ Work get_work(const GroupedArgs& g, int tile, int num_m, int num_n) {
  Work w;
  if (g.mode == 0) {
    w.m_blk = tile % num_m;  // consecutive CTAs take consecutive m-tiles of one n-panel: experts' B panels stay in L2
    w.n_blk = tile / num_m;
    const int e = g.tile_expert[w.m_blk];
    w.valid = e >= 0;
    w.a_row0 = w.m_blk * BM;
    w.num_k = (g.K + BK - 1) / BK;
    w.b_row0 = e * (B_MN ? g.K : g.N);
    w.c_off = 0;
  } else {
    const int per = num_m * num_n;
    const int e = tile / per;
    const int r = tile - e * per;
    w.m_blk = r % num_m;
    w.n_blk = r / num_m;
    const int rows = g.expert_rows[e];
    w.valid = rows > 0;
    w.a_row0 = g.expert_row0[e];
    w.num_k = rows / BK;
    w.b_row0 = 0;
    w.c_off = static_cast<long long>(e) * g.c_expert_stride;
  }
  return w;
}

// rows mode: A K-major [Mpad, K]; B K-major stacked [E*N, K] or MN-major stacked [E*K, N].
// reduction mode: A MN-major [Mpad, M] (loaded as k-rows x m-cols), B MN-major [Mpad, N].
template <bool REDUCE, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GroupedArgs g,
                    int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
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
      mbar_init(smem_u32(&tempty_bar[a]), 4);
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

  const int num_m = (g.M + BM - 1) / BM;
  const int num_n = (g.N + BN - 1) / BN;
  const int num_tiles = (REDUCE ? g.num_experts : 1) * num_m * num_n;
  constexpr bool A_MN = REDUCE;
  constexpr bool BMN = REDUCE ? true : B_MN;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Work w = get_work<B_MN>(g, tile, num_m, num_n);
        if (!w.valid) continue;
        for (int kb = 0; kb < w.num_k; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, status, RLB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(a_dst, &tmap_a, bar, kb * BK, w.a_row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(a_dst + j * (BK * 128), &tmap_a, bar, w.m_blk * BM + j * 64, w.a_row0 + kb * BK);
          }
          if (!BMN) {
            tma_load_2d(b_dst, &tmap_b, bar, kb * BK, w.b_row0 + w.n_blk * BN);
          } else {
            const int krow = REDUCE ? w.a_row0 + kb * BK : w.b_row0 + kb * BK;
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmap_b, bar, w.n_blk * BN + j * 64, krow);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, BMN);
      uint32_t stage = 0, phase = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Work w = get_work<B_MN>(g, tile, num_m, num_n);
        if (!w.valid) continue;
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        ++local_tile;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, status, RLB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < w.num_k; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, status, RLB_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t a_desc = A_MN ? make_smem_desc_sw128(a_addr, BK * 128, 1024) : make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = BMN ? make_smem_desc_sw128(b_addr, BK * 128, 1024) : make_smem_desc_sw128(b_addr, 16, 1024);
          constexpr uint32_t a_step = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
          constexpr uint32_t b_step = (BMN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_f16(tmem_d, a_desc + kk * a_step, b_desc + kk * b_step, idesc, (kb | kk) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(smem_u32(&tfull_bar[acc]));
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const Work w = get_work<B_MN>(g, tile, num_m, num_n);
      if (!w.valid) continue;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, status, RLB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = w.m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < g.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const int col0 = w.n_blk * BN;
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = col0 + c * 32;
        if (!row_ok || col >= g.N) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (g.out_fp32) {
          float* dst = reinterpret_cast<float*>(g.C) + w.c_off + static_cast<long long>(row) * g.ldc + col;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (col + q * 4 < g.N) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (g.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dst + q * 4);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dst + q * 4) = o;
            }
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + w.c_off + static_cast<long long>(row) * g.ldc + col;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col + q * 8 < g.N) {
              if (g.accumulate) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + q * 8);
                const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
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

int g_sms = 0;
int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

template <bool REDUCE, bool B_MN>
int launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, const GroupedArgs& g, int* status, int num_tiles,
                   cudaStream_t stream) {
  auto kern = gemm_grouped_kernel<REDUCE, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, g, status);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

// C[Mpad, N] = A[Mpad, K] * op(B[e]) with e = tile_expert[row / 128]. B: [E, N, K] (b_mn = 0) or [E, K, N] (b_mn = 1),
// contiguous. Rows of tiles marked -1 are left untouched.
RLB_API int rlb_gemm_grouped_rows(const void* A, long long lda, const void* B, int b_mn, void* C, long long ldc, int Mpad, int N,
                                  int K, int num_experts, const int* tile_expert, int out_fp32, int* status, void* stream) {
  if (Mpad <= 0 || N <= 0 || K <= 0) return 0;
  if ((Mpad % 128) || (lda % 8) || (ldc % (out_fp32 ? 4 : 8)) || (N % 8) || (K % 8)) return -2;
  if (b_mn && (K % 64)) return -2;  // a ragged last k-block would read the next expert's rows
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -3;
  CUtensorMap ta, tb;
  int rc = rlb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, Mpad, lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  if (!b_mn)
    rc = rlb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, static_cast<uint64_t>(num_experts) * N,
                          static_cast<uint64_t>(K) * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = rlb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, static_cast<uint64_t>(num_experts) * K,
                          static_cast<uint64_t>(N) * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  GroupedArgs g{};
  g.mode = 0;
  g.M = Mpad;
  g.N = N;
  g.K = K;
  g.num_experts = num_experts;
  g.tile_expert = tile_expert;
  g.C = C;
  g.ldc = ldc;
  g.out_fp32 = out_fp32;
  const int tiles = (Mpad / BM) * ((N + BN - 1) / BN);
  return b_mn ? launch_grouped<false, true>(ta, tb, g, status, tiles, static_cast<cudaStream_t>(stream))
              : launch_grouped<false, false>(ta, tb, g, status, tiles, static_cast<cudaStream_t>(stream));
}

// C[e][M, N] (+)= A[rows_e, M]^T * B[rows_e, N] for every expert e with rows_e = [expert_row0[e], +expert_rows[e]).
// A is [Mpad, M] and B is [Mpad, N] (row-major); C is [E, M, N] contiguous (ldc = N).
RLB_API int rlb_gemm_grouped_reduce(const void* A, long long lda, const void* B, long long ldb, void* C, int Mpad, int M, int N,
                                    int num_experts, const int* expert_row0, const int* expert_rows, int out_fp32,
                                    int accumulate, int* status, void* stream) {
  if (Mpad <= 0 || M <= 0 || N <= 0 || num_experts <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (M % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -3;
  CUtensorMap ta, tb;
  int rc = rlb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, Mpad, lda * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, Mpad, ldb * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  GroupedArgs g{};
  g.mode = 1;
  g.M = M;
  g.N = N;
  g.K = 0;
  g.num_experts = num_experts;
  g.expert_row0 = expert_row0;
  g.expert_rows = expert_rows;
  g.C = C;
  g.ldc = N;
  g.c_expert_stride = static_cast<long long>(M) * N;
  g.out_fp32 = out_fp32;
  g.accumulate = accumulate;
  const int tiles = num_experts * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch_grouped<true, true>(ta, tb, g, status, tiles, static_cast<cudaStream_t>(stream));
}
