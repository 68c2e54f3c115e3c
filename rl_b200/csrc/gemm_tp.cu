// Tensor-parallel GEMMs fused with their collectives over NVLink peer memory (sm_100a).
//
//   gather mode   C[M, N] = allgather_rows(A_local)[M, K] * op(B)      (sequence-parallel all-gather -> column GEMM)
//   scatter mode  out     = reduce_scatter_rows(A[M, K] * op(B)) (+ residual)   (row GEMM -> reduce-scatter), or an
//                 all-reduce when every rank needs all rows (decode)
//
// Both are ONE cooperative kernel per rank built on the same persistent tcgen05 mainloop as the plain GEMM (TMA ->
// 4-stage smem ring -> tcgen05.mma into two TMEM accumulators -> 4 epilogue warps).
//
// gather: a few extra CTAs of the grid ("pushers") copy this rank's row shard into the staging buffer of every rank
// (plain P2P stores, the local copy included) and then raise a flag on each peer. The GEMM CTAs start with the tiles
// whose rows are local (read straight from A_local, no wait) and take a remote rank's rows only once that rank's
// flag has arrived, so the transfer hides behind the local tiles. A remote tile crosses NVLink once and is then read
// from local HBM / L2 by every n-tile that needs it.
//
// scatter: the epilogue converts each accumulator tile to bf16 and stores it directly into the slot that this rank
// owns in the destination rank's staging buffer (P2P stores issued tile by tile, overlapping the mainloop of the
// next tile). After the last tile a flag barrier between the ranks makes the partials visible, and the same kernel
// sums the `world` slots of its own rows in fp32 (fixed rank order: bit-reproducible), adds the residual and writes
// the bf16 result.
//
// Staging buffers may be rewritten by peers only after a start-of-kernel flag barrier (every rank has entered call n,
// hence finished call n-1). Every cross-GPU wait is bounded by %globaltimer and records RLB_ERR_WAIT_PEER /
// RLB_ERR_WAIT_FLAG instead of hanging. Only plain loads/stores touch peer memory: no multimem, no TMA on peer
// addresses. NCCL all-gather / reduce-scatter around the plain GEMM (rl_b200/parallel/tensor.py) is the twin.
//
// Counterpart in the reference: DTensor colwise / rowwise parallel linear layers with sequence parallelism
// (nemo_rl/models/dtensor/parallelize.py:355-470) and Megatron's column / row parallel linears, which issue NCCL
// all-gather / reduce-scatter kernels next to cuBLAS GEMMs.
#include "common.cuh"

#include <cooperative_groups.h>
#include <string.h>

namespace {
using namespace rlb;
namespace cg = cooperative_groups;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_ROW_BYTES = 144;  // 128 B of bf16 per row + 16 B pad (conflict-free 16-byte accesses)
constexpr int EPI_STAGE_BYTES = 4 * 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + EPI_STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;
constexpr int MAX_TP = 8;

enum { MODE_GATHER = 1, MODE_SCATTER = 2 };
// flag words of one rank (uint32, symmetric memory, zero-initialised)
enum { FLAG_START = 0, FLAG_DATA = 8, FLAG_END = 16, FLAG_GO = 32, FLAG_COUNT = 33, FLAG_WORDS = 64 };

// Phase timestamps (%globaltimer, ns) of the last scatter-mode launch, written by thread 0 of CTA 0:
// [0] kernel start, [1] own tiles done, [2] after the first grid sync, [3] after the peer barrier + second grid sync,
// [4] reduce phase done. Read back with rlb_gemm_tp_phase_times (a profiling aid; costs five stores).
__device__ unsigned long long g_tp_phase_ns[8];

struct TpArgs {
  int mode, rank, world;
  unsigned int epoch;
  unsigned int* epoch_ptr;  // scatter mode: when set, the call's epoch is *epoch_ptr + 1 and the kernel stores it back
                            // (a launch recorded in a CUDA graph then advances the epoch on every replay)
  unsigned long long limit_ns;
  unsigned int* flags[MAX_TP];
  unsigned char* stage[MAX_TP];
  int rows_per_rank;
  // gather
  int gemm_ctas;
  const __nv_bfloat16* a_local;
  long long lda_local;
  __nv_bfloat16* C;
  long long ldc;
  const float* bias;
  // scatter
  int all_reduce;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* residual;
  long long ldr;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *p has reached `epoch` (epochs only grow; the signed difference tolerates wrap-around).
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int epoch, unsigned long long limit_ns,
                                          bool sys, int* status, int code) {
  const unsigned long long t0 = globaltimer_ns();
  while (static_cast<int>((sys ? ld_acquire_sys(p) : ld_acquire_gpu(p)) - epoch) < 0) {
    if (globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

// Flag barrier between the ranks run by one full warp: lane r signals rank r and waits for rank r's signal.
__device__ __forceinline__ bool peer_barrier_warp(const TpArgs& t, int word0, int* status) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  if (lane < t.world) {
    st_release_sys(t.flags[lane] + word0 + t.rank, t.epoch);
    ok = wait_flag(t.flags[t.rank] + word0 + lane, t.epoch, t.limit_ns, true, status, RLB_ERR_WAIT_PEER);
  }
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int m_rot, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % rows + m_rot;
  if (m_blk >= num_m) m_blk -= num_m;
  n_blk = in_group / rows;
}

// ------------------------------------------------------------------------------------------ pusher CTAs (gather)
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}

// Copies this rank's [rows_per_rank, K] shard into rows [rank * rows_per_rank, ...) of every rank's staging buffer
// ([world * rows_per_rank, K] bf16, row pitch K) and then raises FLAG_DATA[rank] on every rank.
//
// A contiguous shard (row pitch K) moves as 48 KB bulk copies through the CTA's (otherwise unused) pipeline buffers:
// one thread keeps three loads in flight and forwards every chunk to all ranks with bulk stores, so a handful of CTAs
// saturates NVLink. A strided shard falls back to 16-byte loads / stores by all threads.
__device__ void push_rows(const TpArgs& t, int K, int* status, int* s_flag, uint8_t* smem, uint64_t* full_bar,
                          volatile int* abort_flag) {
  const int npush = gridDim.x - t.gemm_ctas;
  const int pidx = blockIdx.x - t.gemm_ctas;
  unsigned int* my_flags = t.flags[t.rank];
  if (pidx == 0 && (threadIdx.x >> 5) == 0) {
    // every rank has entered this call, so nobody still reads the staging rows of the previous call
    const bool ok = peer_barrier_warp(t, FLAG_START, status);
    if ((threadIdx.x & 31) == 0 && ok) st_release_gpu(my_flags + FLAG_GO, t.epoch);
  }
  if (threadIdx.x == 0)
    *s_flag = wait_flag(my_flags + FLAG_GO, t.epoch, t.limit_ns, false, status, RLB_ERR_WAIT_FLAG) ? 1 : 0;
  __syncthreads();
  const long long shard_bytes = static_cast<long long>(t.rows_per_rank) * K * 2;
  const long long rank_off = static_cast<long long>(t.rank) * shard_bytes;
  if (*s_flag && t.lda_local == K) {
    if (threadIdx.x == 0) {
      const unsigned char* src = reinterpret_cast<const unsigned char*>(t.a_local);
      const long long nchunks = (shard_bytes + STAGE_BYTES - 1) / STAGE_BYTES;
      const long long mine = pidx < nchunks ? (nchunks - pidx + npush - 1) / npush : 0;  // chunks pidx, pidx+npush, ...
      auto issue = [&](long long j) {
        const long long c = pidx + j * npush;
        const long long off = c * STAGE_BYTES;
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(STAGE_BYTES), shard_bytes - off));
        const uint32_t bar = smem_u32(&full_bar[j % STAGES]);
        mbar_arrive_expect_tx(bar, bytes);
        bulk_load(smem_u32(smem + (j % STAGES) * STAGE_BYTES), src + off, bytes, bar);
      };
      for (long long j = 0; j < mine && j < STAGES - 1; ++j) issue(j);
      bool ok = true;
      for (long long j = 0; j < mine && ok; ++j) {
        if (!mbar_wait(smem_u32(&full_bar[j % STAGES]), static_cast<uint32_t>((j / STAGES) & 1), abort_flag, status,
                       RLB_ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        const long long off = (pidx + j * npush) * static_cast<long long>(STAGE_BYTES);
        const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long long>(STAGE_BYTES), shard_bytes - off));
        const uint32_t s_src = smem_u32(smem + (j % STAGES) * STAGE_BYTES);
        for (int p = 0; p < t.world; ++p) {
          int peer = t.rank + p;
          if (peer >= t.world) peer -= t.world;
          bulk_store(t.stage[peer] + rank_off + off, s_src, bytes);
        }
        tma_store_commit();
        // the buffer of chunk j-1 is free once its stores have read it: refill it with chunk j + STAGES - 1
        if (j + STAGES - 1 < mine) {
          tma_store_wait_read<1>();
          issue(j + STAGES - 1);
        }
      }
      tma_store_wait<0>();   // all bulk stores of this CTA are complete
      fence_proxy_async();
      if (!ok) *s_flag = 0;
    }
  } else if (*s_flag) {
    const long long vec_per_row = K / 8;
    const long long total = static_cast<long long>(t.rows_per_rank) * vec_per_row;
    for (long long i = static_cast<long long>(pidx) * NUM_THREADS + threadIdx.x; i < total;
         i += static_cast<long long>(npush) * NUM_THREADS) {
      const long long row = i / vec_per_row, v = i - row * vec_per_row;
      const uint4 x = *reinterpret_cast<const uint4*>(t.a_local + row * t.lda_local + v * 8);
      const long long off = rank_off + (row * K + v * 8) * 2;
      for (int p = 0; p < t.world; ++p) {
        int peer = t.rank + p;
        if (peer >= t.world) peer -= t.world;
        *reinterpret_cast<uint4*>(t.stage[peer] + off) = x;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int old = atomicAdd(my_flags + FLAG_COUNT, 1u);
    if (old == static_cast<unsigned int>(npush - 1)) {
      my_flags[FLAG_COUNT] = 0;
      __threadfence_system();
      if (*s_flag)
        for (int p = 0; p < t.world; ++p) st_release_sys(t.flags[p] + FLAG_DATA + t.rank, t.epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------ the kernel
template <bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a_local,
               const __grid_constant__ CUtensorMap tmap_b, int M, int N, int K, TpArgs t, int* status) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_flag = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // on-chip waits follow the call's limit, so a call with a short limit gives up everywhere within that time
  const unsigned long long bar_limit = t.limit_ns < kWaitLimitNs ? t.limit_ns : kWaitLimitNs;
  if (t.epoch_ptr) t.epoch = *reinterpret_cast<volatile unsigned int*>(t.epoch_ptr) + 1;
  const bool stamp = blockIdx.x == 0 && threadIdx.x == 0 && t.mode == MODE_SCATTER;
  if (stamp) g_tp_phase_ns[0] = globaltimer_ns();
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
    *s_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_a_local);
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
  const bool gather = t.mode == MODE_GATHER;
  const int nctas = gather ? t.gemm_ctas : static_cast<int>(gridDim.x);
  // gather: every rank starts with the m-tiles that hold its own rows
  const int m_rot = gather ? static_cast<int>((static_cast<long long>(t.rank) * t.rows_per_rank) / BM) % num_m : 0;
  unsigned int* my_flags = t.flags[t.rank];

  if (gather && static_cast<int>(blockIdx.x) >= t.gemm_ctas) {
    push_rows(t, K, status, s_flag, smem, full_bar, abort_flag);
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, seen = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas) {
        int m_blk, n_blk;
        tile_coords(tile, num_m, num_n, m_rot, m_blk, n_blk);
        const CUtensorMap* amap = &tmap_a;
        int a_row = m_blk * BM;
        if (gather) {
          const int m0 = m_blk * BM, m1 = min(M, m0 + BM) - 1;
          const int s_lo = m0 / t.rows_per_rank, s_hi = m1 / t.rows_per_rank;
          if (s_lo == t.rank && s_hi == t.rank) {
            amap = &tmap_a_local;
            a_row = m0 - t.rank * t.rows_per_rank;
          } else {
            for (int s = s_lo; s <= s_hi && ok; ++s) {
              if (seen & (1u << s)) continue;
              ok = wait_flag(my_flags + FLAG_DATA + s, t.epoch, t.limit_ns, true, status, RLB_ERR_WAIT_PEER);
              seen |= 1u << s;
            }
            if (!ok) {
              *abort_flag = 1;
              break;
            }
            fence_proxy_async();  // rows written by generic-proxy stores, read by TMA
          }
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, status, RLB_ERR_WAIT_EMPTY, bar_limit)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(a_dst, amap, bar, kb * BK, a_row);
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
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, B_MN);
      uint32_t stage = 0, phase = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, status, RLB_ERR_WAIT_TMEM_EMPTY, bar_limit)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, status, RLB_ERR_WAIT_FULL, bar_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr, BK * 128, 1024) : make_smem_desc_sw128(b_addr, 16, 1024);
          constexpr uint32_t a_step = (UMMA_K * 2) >> 4;
          constexpr uint32_t b_step = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
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
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    bool ok = true;
    if (!gather) {
      // peers' staging slots may be overwritten once every rank has entered this call
      if (blockIdx.x == 0 && warp == 2) {
        const bool b_ok = peer_barrier_warp(t, FLAG_START, status);
        if (lane == 0 && b_ok) st_release_gpu(my_flags + FLAG_GO, t.epoch);
      }
      bool go = true;
      if (lane == 0) go = wait_flag(my_flags + FLAG_GO, t.epoch, t.limit_ns, false, status, RLB_ERR_WAIT_FLAG);
      ok = __shfl_sync(0xffffffffu, go, 0);
      // the producer and MMA roles of this CTA depend on this one: tell them to stop instead of letting each wait out
      // its own limit on a barrier that will never complete
      if (!ok && lane == 0) *abort_flag = 1;
    }
    const int rows_out = t.all_reduce ? M : t.rows_per_rank;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += nctas, ++local_tile) {
      int m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_rot, m_blk, n_blk);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, status, RLB_ERR_WAIT_TMEM_FULL, bar_limit)) break;
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const int col0 = n_blk * BN;
      uint8_t* epi = smem + STAGES * STAGE_BYTES + 256 + (warp - 2) * 32 * EPI_ROW_BYTES;
      const int row_base = m_blk * BM + quarter * 32;
      for (int c = 0; c < BN / 64; ++c) {
        const int col = col0 + c * 64;
        uint4 o[8];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 64 + half * 32, r);
          tmem_ld_wait();
          if (gather && t.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + half * 32 + i < N) r[i] = __float_as_uint(__uint_as_float(r[i]) + t.bias[col + half * 32 + i]);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            o[half * 4 + q].x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            o[half * 4 + q].y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            o[half * 4 + q].z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            o[half * 4 + q].w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
          }
        }
        if (col >= N) continue;  // uniform over the warp
        if (gather) {
          if (row_ok) {
            __nv_bfloat16* dst = t.C + static_cast<long long>(row) * t.ldc + col;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (col + q * 8 < N) *reinterpret_cast<uint4*>(dst + q * 8) = o[q];
          }
        } else {
          // transpose through shared memory so that 8 lanes write one row's 128 contiguous bytes: peer stores leave
          // the GPU as full 128-byte NVLink writes instead of scattered 16-byte ones
#pragma unroll
          for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(epi + lane * EPI_ROW_BYTES + q * 16) = o[q];
          __syncwarp();
          const int piece = lane & 7;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const int grow = row_base + rr;
            if (grow < M && col + piece * 8 < N) {
              const uint4 v = *reinterpret_cast<const uint4*>(epi + rr * EPI_ROW_BYTES + piece * 16);
              if (t.all_reduce) {
                const long long off = ((static_cast<long long>(t.rank) * rows_out + grow) * N + col + piece * 8) * 2;
                for (int p = 0; p < t.world; ++p) {
                  int peer = t.rank + p;
                  if (peer >= t.world) peer -= t.world;
                  *reinterpret_cast<uint4*>(t.stage[peer] + off) = v;
                }
              } else {
                const int dest = grow / t.rows_per_rank;
                const long long srow = static_cast<long long>(t.rank) * rows_out + (grow - dest * t.rows_per_rank);
                *reinterpret_cast<uint4*>(t.stage[dest] + (srow * N + col + piece * 8) * 2) = v;
              }
            }
          }
          __syncwarp();
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
  if (gather) return;

  // ------------------------------------------------------------ scatter: partials visible everywhere, then reduce
  if (stamp) g_tp_phase_ns[1] = globaltimer_ns();
  __threadfence_system();
  grid.sync();
  if (stamp) g_tp_phase_ns[2] = globaltimer_ns();
  if (stamp && t.epoch_ptr) *t.epoch_ptr = t.epoch;  // every CTA has read the old value before the grid sync
  if (blockIdx.x == 0) {
    if (warp == 0) {
      const bool b_ok = peer_barrier_warp(t, FLAG_END, status);
      if (lane == 0) *s_flag = b_ok ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(my_flags + FLAG_GO + 2, *s_flag ? t.epoch : t.epoch - 1);
  }
  grid.sync();
  if (stamp) g_tp_phase_ns[3] = globaltimer_ns();
  if (ld_acquire_gpu(my_flags + FLAG_GO + 2) != t.epoch) return;  // a peer did not arrive: leave `out` untouched
  const int rows_out = t.all_reduce ? M : t.rows_per_rank;
  const long long vec_per_row = N / 8;
  const long long total = static_cast<long long>(rows_out) * vec_per_row;
  const unsigned char* mine = t.stage[t.rank];
  // four independent vectors per thread and iteration keep enough loads in flight to run at memory bandwidth
  constexpr int U = 4;
  const long long stride = static_cast<long long>(gridDim.x) * NUM_THREADS;
  for (long long i0 = static_cast<long long>(blockIdx.x) * NUM_THREADS + threadIdx.x; i0 < total; i0 += stride * U) {
    float acc[U][8];
    long long row[U], c[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      live[u] = i < total;
      row[u] = live[u] ? i / vec_per_row : 0;
      c[u] = live[u] ? (i - row[u] * vec_per_row) * 8 : 0;
    }
    if (t.residual) {
      uint4 rv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) rv[u] = live[u] ? *reinterpret_cast<const uint4*>(t.residual + row[u] * t.ldr + c[u]) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float2 a0 = unpack_bf16x2(rv[u].x), a1 = unpack_bf16x2(rv[u].y), a2 = unpack_bf16x2(rv[u].z), a3 = unpack_bf16x2(rv[u].w);
        acc[u][0] = a0.x; acc[u][1] = a0.y; acc[u][2] = a1.x; acc[u][3] = a1.y;
        acc[u][4] = a2.x; acc[u][5] = a2.y; acc[u][6] = a3.x; acc[u][7] = a3.y;
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
    }
    // all slots of all U vectors are requested before the first one is consumed (up to 32 loads in flight per thread)
    uint4 pv[MAX_TP][U];
#pragma unroll
    for (int s = 0; s < MAX_TP; ++s) {
      if (s < t.world) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          pv[s][u] = live[u] ? __ldcg(reinterpret_cast<const uint4*>(mine + ((static_cast<long long>(s) * rows_out + row[u]) * N + c[u]) * 2))
                             : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int s = 0; s < MAX_TP; ++s) {
      if (s < t.world) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float2 a0 = unpack_bf16x2(pv[s][u].x), a1 = unpack_bf16x2(pv[s][u].y), a2 = unpack_bf16x2(pv[s][u].z),
                       a3 = unpack_bf16x2(pv[s][u].w);
          acc[u][0] += a0.x; acc[u][1] += a0.y; acc[u][2] += a1.x; acc[u][3] += a1.y;
          acc[u][4] += a2.x; acc[u][5] += a2.y; acc[u][6] += a3.x; acc[u][7] += a3.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      uint4 o;
      o.x = pack_bf16x2(acc[u][0], acc[u][1]);
      o.y = pack_bf16x2(acc[u][2], acc[u][3]);
      o.z = pack_bf16x2(acc[u][4], acc[u][5]);
      o.w = pack_bf16x2(acc[u][6], acc[u][7]);
      *reinterpret_cast<uint4*>(t.out + row[u] * t.ldo + c[u]) = o;
    }
  }
  if (stamp) g_tp_phase_ns[4] = globaltimer_ns();
}

int g_sms = 0;

template <bool B_MN>
int launch_tp(const CUtensorMap& ta, const CUtensorMap& tal, const CUtensorMap& tb, int M, int N, int K, TpArgs& t,
              int* status, int grid, cudaStream_t stream) {
  auto kern = gemm_tp_kernel<B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  void* args[] = {const_cast<CUtensorMap*>(&ta), const_cast<CUtensorMap*>(&tal), const_cast<CUtensorMap*>(&tb),
                  &M, &N, &K, &t, &status};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(grid), dim3(NUM_THREADS),
                                                      args, SMEM_BYTES, stream));
}

int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sms;
}

int make_b_map(CUtensorMap* tb, const void* B, int N, int K, long long ldb, bool b_mn) {
  if (!b_mn)
    return rlb_make_tmap_2d(tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  return rlb_make_tmap_2d(tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
}

void fill_common(TpArgs& t, void* const* stage_ptrs, void* const* flag_ptrs, int rank, int world, unsigned int epoch,
                 double wait_limit_s, int rows_per_rank) {
  memset(&t, 0, sizeof(t));
  t.rank = rank;
  t.world = world;
  t.epoch = epoch;
  t.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  t.rows_per_rank = rows_per_rank;
  for (int r = 0; r < world; ++r) {
    t.stage[r] = static_cast<unsigned char*>(stage_ptrs[r]);
    t.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  }
}

}  // namespace

// Copies the five phase timestamps of the last scatter-mode launch to `out_ns` (host memory). Synchronises the device.
RLB_API int rlb_gemm_tp_phase_times(unsigned long long* out_ns) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemcpyFromSymbol(out_ns, g_tp_phase_ns, 5 * sizeof(unsigned long long)));
}

// Bytes of flag memory each rank must provide (zero-initialised, symmetric).
RLB_API int rlb_gemm_tp_flag_bytes() { return FLAG_WORDS * 4; }

// C[world*rows_per_rank, N] = allgather_rows(A_local[rows_per_rank, K]) * op(B) (+ bias).
// B is [N, K] row-major (b_mn = 0: C = A B^T) or [K, N] row-major (b_mn = 1: C = A B). stage_ptrs[r] is rank r's
// staging buffer of world*rows_per_rank*K bf16; after the call this rank's staging buffer holds the gathered A.
// `pushers` CTAs of the grid do the copies (0: default).
RLB_API int rlb_gemm_tp_gather(const void* a_local, long long lda_local, const void* B, long long ldb, int b_mn, void* C,
                               long long ldc, const float* bias, int rows_per_rank, int N, int K, void* const* stage_ptrs,
                               void* const* flag_ptrs, int rank, int world, unsigned int epoch, int pushers,
                               double wait_limit_s, int* status, void* stream) {
  if (world < 2 || world > MAX_TP || rows_per_rank <= 0 || N <= 0 || K <= 0) return -2;
  if ((lda_local % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || (K % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(a_local) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -3;
  const int M = world * rows_per_rank;
  TpArgs t;
  fill_common(t, stage_ptrs, flag_ptrs, rank, world, epoch, wait_limit_s, rows_per_rank);
  t.mode = MODE_GATHER;
  t.a_local = static_cast<const __nv_bfloat16*>(a_local);
  t.lda_local = lda_local;
  t.C = static_cast<__nv_bfloat16*>(C);
  t.ldc = ldc;
  t.bias = bias;
  CUtensorMap ta, tal, tb;
  int rc = rlb_make_tmap_2d(&ta, stage_ptrs[rank], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, static_cast<uint64_t>(K) * 2, BK,
                            BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tal, a_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, rows_per_rank, lda_local * 2, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = make_b_map(&tb, B, N, K, ldb, b_mn != 0);
  if (rc) return -100 - rc;
  const int sms = sm_count();
  if (pushers <= 0) pushers = 12;
  if (pushers > sms / 2) pushers = sms / 2;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  t.gemm_ctas = tiles < sms - pushers ? tiles : sms - pushers;
  const int grid = t.gemm_ctas + pushers;
  return b_mn ? launch_tp<true>(ta, tal, tb, M, N, K, t, status, grid, static_cast<cudaStream_t>(stream))
              : launch_tp<false>(ta, tal, tb, M, N, K, t, status, grid, static_cast<cudaStream_t>(stream));
}

// out = reduce over ranks of (A[M, K] * op(B)) (+ residual), rows scattered: rank j receives rows
// [j*rows_per_rank, (j+1)*rows_per_rank) (all_reduce = 0, M = world*rows_per_rank, out is [rows_per_rank, N]), or every
// rank receives all M rows (all_reduce = 1, out is [M, N]). stage_ptrs[r]: rank r's staging buffer of
// world * rows_out * N bf16 (one slot per source rank). `epoch_ptr` (device, may be null): see TpArgs.
RLB_API int rlb_gemm_tp_scatter(const void* A, long long lda, const void* B, long long ldb, int b_mn, int M, int N, int K,
                                int rows_per_rank, int all_reduce, void* out, long long ldo, const void* residual,
                                long long ldr, void* const* stage_ptrs, void* const* flag_ptrs, int rank, int world,
                                unsigned int epoch, void* epoch_ptr, double wait_limit_s, int* status, void* stream) {
  if (world < 2 || world > MAX_TP || M <= 0 || N <= 0 || K <= 0) return -2;
  if (!all_reduce && M != world * rows_per_rank) return -2;
  if ((lda % 8) || (ldb % 8) || (ldo % 8) || (N % 8) || (residual && (ldr % 8))) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(residual)) & 15)
    return -3;
  TpArgs t;
  fill_common(t, stage_ptrs, flag_ptrs, rank, world, epoch, wait_limit_s, all_reduce ? M : rows_per_rank);
  t.mode = MODE_SCATTER;
  t.epoch_ptr = static_cast<unsigned int*>(epoch_ptr);
  t.all_reduce = all_reduce;
  t.out = static_cast<__nv_bfloat16*>(out);
  t.ldo = ldo;
  t.residual = static_cast<const __nv_bfloat16*>(residual);
  t.ldr = ldr;
  CUtensorMap ta, tb;
  int rc = rlb_make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = make_b_map(&tb, B, N, K, ldb, b_mn != 0);
  if (rc) return -100 - rc;
  const int sms = sm_count();
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  // the reduce phase wants many CTAs even when there are few tiles
  const int grid = all_reduce ? sms : (tiles < sms ? (tiles > sms / 2 ? tiles : sms / 2) : sms);
  t.gemm_ctas = grid;
  return b_mn ? launch_tp<true>(ta, ta, tb, M, N, K, t, status, grid, static_cast<cudaStream_t>(stream))
              : launch_tp<false>(ta, ta, tb, M, N, K, t, status, grid, static_cast<cudaStream_t>(stream));
}
