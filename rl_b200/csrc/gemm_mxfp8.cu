// MXFP8 GEMM (sm_100a): C[M, N] (bf16) = A[M, K] * B[N, K]^T with e4m3 operands and one UE8M0 scale per 32 consecutive
// K elements of every row of A and B (OCP microscaling), multiplied in by the tensor core itself:
//   tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale, operands from shared memory (TMA, 128-byte swizzle),
//   accumulators and the scale factors in tensor memory (scales copied smem -> TMEM with tcgen05.cp.32x128b.warpx4).
//
// Tile 128 x 128 x 128 (four K = 32 MMAs per stage), 4-stage TMA ring, two TMEM accumulators, persistent CTAs with the
// same warp roles as the bf16 GEMM. Scale factors are expected in the blocked layout the hardware reads: for every
// (128-row block, 128-column K block) one 512-byte atom with byte offset (r % 32) * 16 + (r / 32) * 4 + j for row r of
// the block and 32-wide K group j (rl_b200/ops/quant.py::swizzle_mx_scales produces it), so a stage's scales arrive as
// plain 512-byte bulk copies.
//
// Counterpart in the reference: FlashInfer's CUTLASS sm_100 MXFP8 linear kernel selected for refit-friendly MXFP8
// serving (nemo_rl/models/generation/vllm/quantization/fp8.py:798-870).
#include "common.cuh"

namespace {
using namespace rlb;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;           // bytes == elements for fp8
constexpr int STAGES = 4;
constexpr int UMMA_K = 32;
constexpr int A_BYTES = BM * BK;  // 16 KB
constexpr int B_BYTES = BN * BK;  // 16 KB
constexpr int SF_BYTES = 512;     // one atom: 128 rows x 4 scales
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;  // 33 KB; every part starts 1024-byte aligned or better
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int ACC_COLS = BN;                    // two accumulators: columns [0, 256)
constexpr int SF_COL0 = 2 * BN;                 // scale factors: 8 columns per stage from column 256
constexpr int GROUP_M = 16;

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

// kind::mxf8f6f4 block-scaled instruction descriptor: e4m3 x e4m3, UE8M0 scales, K-major operands.
__device__ __forceinline__ uint32_t idesc_mx(uint32_t sf_id) {
  return (sf_id << 4)                                   // B scale-factor byte
         | (1u << 23)                                   // scale format UE8M0
         | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24)
         | (sf_id << 29);                               // A scale-factor byte
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const unsigned char* __restrict__ sfa, const unsigned char* __restrict__ sfb, int M, int N, int K,
                  __nv_bfloat16* __restrict__ C, long long ldc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_k = K / BK;  // K is a multiple of 128

  if (warp == 0) {
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
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, bar, kb * BK, m_blk * BM);
          tma_load_2d(a_dst + A_BYTES, &tmap_b, bar, kb * BK, n_blk * BN);
          // scale atoms: [row block][k block][512 B]
          bulk_load(a_dst + A_BYTES + B_BYTES, sfa + (static_cast<long long>(m_blk) * num_k + kb) * SF_BYTES, SF_BYTES, bar);
          bulk_load(a_dst + A_BYTES + B_BYTES + SF_BYTES, sfb + (static_cast<long long>(n_blk) * num_k + kb) * SF_BYTES, SF_BYTES, bar);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1, acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, status, RLB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, status, RLB_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint32_t sfa_addr = b_addr + B_BYTES, sfb_addr = sfa_addr + SF_BYTES;
          const uint32_t t_sfa = tmem_base + SF_COL0 + stage * 8, t_sfb = t_sfa + 4;
          // 32 rows x 16 bytes, rows 16 bytes apart: 8-row core matrices 128 bytes apart
          tmem_cp_32x128b_warpx4(t_sfa, make_smem_desc_noswz(sfa_addr, 16, 128));
          tmem_cp_32x128b_warpx4(t_sfb, make_smem_desc_noswz(sfb_addr, 16, 128));
          const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = make_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 32 bytes further along K inside the 128-byte swizzle atom; scale byte kk of the stage's four
            umma_mxf8(tmem_d, a_desc + kk * 2, b_desc + kk * 2, idesc_mx(kk), (kb | kk) != 0 ? 1u : 0u, t_sfa, t_sfb);
          }
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
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const uint32_t acc = local_tile & 1, acc_phase = (local_tile >> 1) & 1;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, status, RLB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * ACC_COLS;
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_blk * BN + c * 32;
        if (row >= M || col >= N) continue;
        __nv_bfloat16* dst = C + static_cast<long long>(row) * ldc + col;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col + q * 8 < N) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + q * 8) = o;
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
}  // namespace

// A [M, K] e4m3 (lda bytes), B [N, K] e4m3 (ldb bytes), scales in the blocked atom layout:
// sfa [ceil(M/128)][K/128][512], sfb [ceil(N/128)][K/128][512]. C [M, N] bf16. K % 128 == 0, N % 8 == 0.
RLB_API int rlb_gemm_mxfp8(const void* A, long long lda, const void* B, long long ldb, const void* sfa, const void* sfb, void* C,
                           long long ldc, int M, int N, int K, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % BK) || (N % 8) || (lda % 16) || (ldb % 16) || (ldc % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb)) & 15)
    return -3;
  CUtensorMap ta, tb;
  int rc = rlb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  gemm_mxfp8_kernel<<<grid, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      ta, tb, static_cast<const unsigned char*>(sfa), static_cast<const unsigned char*>(sfb), M, N, K,
      static_cast<__nv_bfloat16*>(C), ldc, status);
  return static_cast<int>(cudaGetLastError());
}
