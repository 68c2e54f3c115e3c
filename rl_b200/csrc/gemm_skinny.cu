// Small-batch ("skinny") bf16 GEMM for decode: Y[M, N] = X[M, K] W[N, K]^T with M <= 256 tokens.
//
// At decode time a projection is a weight stream: every byte of W is read once and the arithmetic is nearly free, so
// the kernel is organised around memory parallelism rather than tile reuse.
//   * Operands are swapped: 128 rows of W form the M side of the tcgen05 MMA, the tokens form the N side
//     (UMMA 128 x NT x 16 with NT = 32 / 64 / 128 / 256), so no tensor-core lanes idle on padding rows of X.
//   * The reduction dimension is split over the CTAs of a thread-block cluster (1..8). Each CTA streams its K range
//     through a deep TMA ring, parks its fp32 partial tile in its own shared memory, and after a cluster barrier every
//     CTA of the cluster sums one slice of the tokens over all partials through distributed shared memory and writes
//     the bf16 result: no atomics, no workspace, no second kernel, bit-reproducible.
//   * Two CTAs fit per SM, and cluster size x number of 128-row tiles is chosen near the SM count, so that all SMs pull
//     on HBM for the projections of one layer (N = 4096 would otherwise occupy 16 of the 148 SMs).
// The epilogue adds an optional bias and residual (the transformer's skip connection) and can emit fp32 (logits).
//
// Counterpart in the reference: the cuBLAS / vLLM GEMMs behind every decode-step nn.Linear
// (nemo_rl/models/generation/vllm/vllm_worker.py:570-597).
#include "common.cuh"

#include <cooperative_groups.h>

namespace {
using namespace rlb;
namespace cg = cooperative_groups;

constexpr int SK_BM = 128;     // rows of W per tile
constexpr int SK_BK = 64;
constexpr int SK_THREADS = 192;

template <int NT>
struct SkinnyCfg {
  static constexpr int A_BYTES = SK_BM * SK_BK * 2;  // 16 KB
  static constexpr int B_BYTES = NT * SK_BK * 2;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  // ring depth so that one CTA uses <= ~110 KB (two CTAs per SM)
  static constexpr int STAGES = (NT <= 64) ? 4 : (NT == 128 ? 3 : 2);
  static constexpr int RING = STAGES * STAGE;
  static constexpr int PARTIAL = NT * SK_BM * 4;  // fp32 [NT][128]
  static constexpr int MAIN = RING > PARTIAL ? RING : PARTIAL;
  static constexpr int SMEM = MAIN + 256;
  static constexpr int TMEM = NT < 32 ? 32 : NT;
};

struct SkinnyParams {
  void* Y;
  long long ldy;
  const float* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int M, N, K;
  int out_fp32;
  int w_static;  // W is not written by the kernel that precedes this one on the stream: its stream may start early
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

template <int NT>
__global__ void __launch_bounds__(SK_THREADS, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   SkinnyParams p) {
  using Cfg = SkinnyCfg<NT>;
  extern __shared__ __align__(1024) uint8_t smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t split = cluster.num_blocks();
  const uint32_t krank = cluster_ctarank();
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::MAIN);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::STAGES;
  uint64_t* acc_bar = bars + 2 * Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blk = blockIdx.x / split;  // tile of 128 W rows
  const int num_k = (p.K + SK_BK - 1) / SK_BK;
  const int k_per = (num_k + split - 1) / split;
  const int kb_begin = krank * k_per;
  const int kb_end = min(num_k, kb_begin + k_per);
  const bool aligned = (smem_u32(smem) & 1023u) == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(acc_bar), 1);
    *abort_flag = aligned ? 0 : 1;
    if (!aligned && p.status) atomicCAS(p.status, 0, RLB_ERR_BAD_ARG);
    mbar_fence_init();
    fence_proxy_async();
  }
  const bool have_work = kb_end > kb_begin && aligned;
  // Weights that the preceding kernel cannot have written are requested before the dependency wait: the first ring
  // stages fill while that kernel drains. The activations of the same stages follow after the wait.
  int early = 0;
  if (threadIdx.x == 0 && have_work) {
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_x);
    if (p.w_static) {
      for (; early < Cfg::STAGES && kb_begin + early < kb_end; ++early) {
        const uint32_t bar = smem_u32(&full_bar[early]);
        mbar_arrive_expect_tx(bar, Cfg::STAGE);
        tma_load_2d(smem_u32(smem + early * Cfg::STAGE), &tmap_w, bar, (kb_begin + early) * SK_BK, n_blk * SK_BM);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  pdl_sync();  // everything above overlaps the tail of the previous kernel on the stream

  if (warp == 0) {
    if (lane == 0 && have_work) {
      for (int e = 0; e < early; ++e)
        tma_load_2d(smem_u32(smem + e * Cfg::STAGE) + Cfg::A_BYTES, &tmap_x, smem_u32(&full_bar[e]), (kb_begin + e) * SK_BK, 0);
      uint32_t stage = early == Cfg::STAGES ? 0 : early, phase = early == Cfg::STAGES ? 1 : 0;
      for (int kb = kb_begin + early; kb < kb_end; ++kb) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) break;
        const uint32_t bar = smem_u32(&full_bar[stage]);
        const uint32_t a_dst = smem_u32(smem + stage * Cfg::STAGE);
        mbar_arrive_expect_tx(bar, Cfg::STAGE);
        tma_load_2d(a_dst, &tmap_w, bar, kb * SK_BK, n_blk * SK_BM);
        tma_load_2d(a_dst + Cfg::A_BYTES, &tmap_x, bar, kb * SK_BK, 0);
        if (++stage == Cfg::STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && have_work) {
      constexpr uint32_t idesc = make_idesc_bf16(SK_BM, NT, false, false);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, RLB_ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE);
        const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
        const uint64_t b_desc = make_smem_desc_sw128(a_addr + Cfg::A_BYTES, 16, 1024);
#pragma unroll
        for (int kk = 0; kk < SK_BK / 16; ++kk)
          umma_f16(tmem_acc, a_desc + kk * 2, b_desc + kk * 2, idesc, (kb > kb_begin || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&empty_bar[stage]));
        if (++stage == Cfg::STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(smem_u32(acc_bar));
    }
  } else {
    // Epilogue part 1: park the fp32 partial tile in shared memory as [token][w_row] (the ring is drained by then:
    // the accumulator barrier fires only after every MMA, hence every TMA load, of this CTA has completed).
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // W row inside the tile
    float* part = reinterpret_cast<float*>(smem);
    bool ok = have_work && mbar_wait(smem_u32(acc_bar), 0, abort_flag, p.status, RLB_ERR_WAIT_TMEM_FULL);
    if (ok) tc_fence_after();
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < NT / 32; ++c) {
      uint32_t r[32];
      if (ok) {
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;  // a CTA without a K range contributes zeros
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) part[(c * 32 + i) * SK_BM + row] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, Cfg::TMEM);
  }
  // Epilogue part 2: every CTA of the cluster reduces a slice of the tokens over all partial tiles.
  cluster.sync();
  {
    const int tok_per = (NT + split - 1) / split;
    const int m_begin = krank * tok_per;
    const int m_end = min(min(NT, p.M), m_begin + tok_per);
    const uint32_t part_addr = smem_u32(smem);
    const int n0 = n_blk * SK_BM;
    // work items: (token m, group of 4 consecutive W rows)
    const int items = (m_end - m_begin) * (SK_BM / 4);
    for (int it = threadIdx.x; it < items; it += SK_THREADS) {
      const int m = m_begin + it / (SK_BM / 4);
      const int n4 = (it % (SK_BM / 4)) * 4;
      const uint32_t off = static_cast<uint32_t>((m * SK_BM + n4) * 4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (uint32_t r = 0; r < split; ++r) {
        const float4 v = ld_dsmem_f4(mapa_shared(part_addr + off, r));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const int n = n0 + n4;
      if (n >= p.N) continue;  // N is a multiple of 8, so a group of 4 is all in or all out
      if (p.bias) {
        acc.x += p.bias[n]; acc.y += p.bias[n + 1]; acc.z += p.bias[n + 2]; acc.w += p.bias[n + 3];
      }
      if (p.residual) {
        const uint2 rv = *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(m) * p.ldr + n);
        const float2 r0 = unpack_bf16x2(rv.x), r1 = unpack_bf16x2(rv.y);
        acc.x += r0.x; acc.y += r0.y; acc.z += r1.x; acc.w += r1.y;
      }
      if (p.out_fp32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.Y) + static_cast<long long>(m) * p.ldy + n) = acc;
      } else {
        uint2 o;
        o.x = pack_bf16x2(acc.x, acc.y);
        o.y = pack_bf16x2(acc.z, acc.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.Y) + static_cast<long long>(m) * p.ldy + n) = o;
      }
    }
  }
  cluster.sync();  // peers may still be reading this CTA's partial tile
}

int g_sk_sms = 0;
int g_sk_static_w = 0;

template <int NT>
int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, int split, cudaStream_t stream) {
  using Cfg = SkinnyCfg<NT>;
  auto kern = gemm_skinny_kernel<NT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int tiles = (p.N + SK_BM - 1) / SK_BM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * split, 1, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = rlb_pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
  return static_cast<int>(e);
}

}  // namespace

// Picks the cluster size (K split) for a projection: enough CTAs to cover the SMs twice over at most, never more than
// 8 (the portable cluster limit), never more than one CTA per 4 k-blocks.
RLB_API int rlb_gemm_skinny_split(int N, int K) {
  if (g_sk_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sk_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sk_sms <= 0) g_sk_sms = 148;
  }
  const int tiles = (N + SK_BM - 1) / SK_BM;
  const int num_k = (K + SK_BK - 1) / SK_BK;
  int best = 1;
  for (int s = 1; s <= 8; s *= 2) {
    if (tiles * s > 2 * g_sk_sms) break;
    if (num_k / s < 4) break;
    best = s;
  }
  return best;
}

// While set, callers promise that the W operand of every skinny GEMM was not written by the kernel launched just before
// it on the same stream (true for model weights during generation); the kernel then starts streaming W while that
// kernel is still draining. Returns the previous value.
RLB_API int rlb_gemm_skinny_static_weights(int on) {
  const int prev = g_sk_static_w;
  g_sk_static_w = on ? 1 : 0;
  return prev;
}

// Y[M, N] = X[M, K] W[N, K]^T (+ bias) (+ residual); M <= 256. ldx / ldw / ldy / ldr in elements (multiples of 8;
// fp32 output: ldy multiple of 4). `split` = 0 lets the library choose. Returns 0, a CUDA error or a negative code.
RLB_API int rlb_gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, long long ldx, long long ldw,
                            long long ldy, int out_fp32, const float* bias, const void* residual, long long ldr,
                            int split, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256) return -7;
  if ((ldx % 8) || (ldw % 8) || (N % 8) || (ldy % (out_fp32 ? 4 : 8)) || (residual && (ldr % 4))) return -2;
  const int NT = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
  CUtensorMap tw, tx;
  int rc = rlb_make_tmap_2d(&tw, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldw * 2, SK_BK, SK_BM,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tx, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, SK_BK, NT,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  if (split <= 0) split = rlb_gemm_skinny_split(N, K);
  if (split > 8) split = 8;
  SkinnyParams p;
  p.Y = Y;
  p.ldy = ldy;
  p.bias = bias;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.M = M;
  p.N = N;
  p.K = K;
  p.out_fp32 = out_fp32;
  p.w_static = g_sk_static_w;
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (NT) {
    case 32: return launch_skinny<32>(tw, tx, p, split, s);
    case 64: return launch_skinny<64>(tw, tx, p, split, s);
    case 128: return launch_skinny<128>(tw, tx, p, split, s);
    default: return launch_skinny<256>(tw, tx, p, split, s);
  }
}
