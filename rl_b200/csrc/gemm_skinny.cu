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
// Three optional epilogue fusions remove the small kernels that would otherwise sit between the projections of a decoder
// layer (each costs more in launch and dependency latency than in work at 64 tokens):
//   * RMSNorm on the INPUT, split in two. The kernel that produces the residual stream h (o_proj / down_proj with the
//     residual add) also writes hw = h * w_norm (the per-channel weight of the NEXT norm) and, per 128-column tile, the
//     partial sum of squares of h for every token. The consuming projection multiplies hw and scales each output row by
//     rstd = rsqrt(sum of the partials / d + eps) in its epilogue: the row scale commutes with the product.
//   * SwiGLU: for the [gate | up] weight, a tile is 64 gate rows stacked on the 64 matching up rows (two TMA boxes into
//     one 128-row operand, no re-layout of the weight), and the epilogue writes silu(gate) * up.
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
  static constexpr int SMEM = MAIN + 256 + 1024;  // ring / partial tile, barriers, per-token rstd (256 floats)
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
  // fused RMSNorm of the input: partial sums of squares [ssq_in_tiles][ssq_in_stride] written by the producer of X
  const float* ssq_in;
  int ssq_in_tiles;
  long long ssq_in_stride;
  float eps;
  // hand-off to the next norm: Y2 = bf16(Y) * norm_w, ssq_out[tile][m] = sum over the tile's columns of bf16(Y)^2
  float* ssq_out;
  long long ssq_out_stride;
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* Y2;
  long long ldy2;
  int swiglu;  // W is [2F, K] = [gate | up]; the output is silu(gate) * up of width F = N
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
  float* s_rstd = reinterpret_cast<float*>(smem + Cfg::MAIN + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blk = blockIdx.x / split;  // tile of 128 W rows (SwiGLU: 64 gate rows + the 64 matching up rows)
  // W rows of the tile: one 128-row box, or two 64-row boxes (gate rows, then up rows F further down)
  const int w_row0 = p.swiglu ? n_blk * 64 : n_blk * SK_BM;
  const int w_row1 = p.N + n_blk * 64;
  auto load_w = [&](uint32_t dst, uint32_t bar, int kb) {
    if (p.swiglu) {
      tma_load_2d(dst, &tmap_w, bar, kb * SK_BK, w_row0);
      tma_load_2d(dst + Cfg::A_BYTES / 2, &tmap_w, bar, kb * SK_BK, w_row1);
    } else {
      tma_load_2d(dst, &tmap_w, bar, kb * SK_BK, w_row0);
    }
  };
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
        load_w(smem_u32(smem + early * Cfg::STAGE), bar, kb_begin + early);
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
        load_w(a_dst, bar, kb);
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
    if (p.ssq_in) {
      // per-token reciprocal RMS of the input from the producer's per-tile partial sums (this runs under the mainloop)
      for (int m = threadIdx.x - 64; m < NT; m += 128) {
        float ss = 0.f;
        if (m < p.M)
          for (int t = 0; t < p.ssq_in_tiles; ++t) ss += p.ssq_in[t * p.ssq_in_stride + m];
        s_rstd[m] = m < p.M ? rsqrtf(ss / static_cast<float>(p.K) + p.eps) : 0.f;
      }
    }
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
    const int out_cols = p.swiglu ? 64 : SK_BM;      // output columns of this tile
    const int groups = out_cols / 4;                 // work item: (token m, 4 consecutive output columns)
    const int n0 = n_blk * out_cols;
    // a warp always works on one token (groups is 16 or 32, the stride a multiple of 32), so the per-token sum of
    // squares for the next norm is one warp reduction
    const int items = max(m_end - m_begin, 0) * groups;
    const int items_pad = (items + 31) & ~31;
    for (int it = threadIdx.x; it < items_pad; it += SK_THREADS) {
      const bool live = it < items;
      const int m = m_begin + (live ? it / groups : 0);
      const int n4 = (live ? it % groups : 0) * 4;
      const int n = n0 + n4;
      const bool valid = live && n < p.N;  // N is a multiple of 8, so a group of 4 is all in or all out
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), acc_u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) {
        const uint32_t off = static_cast<uint32_t>((m * SK_BM + n4) * 4);
        for (uint32_t r = 0; r < split; ++r) {
          const float4 v = ld_dsmem_f4(mapa_shared(part_addr + off, r));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          if (p.swiglu) {
            const float4 u = ld_dsmem_f4(mapa_shared(part_addr + off + 64 * 4, r));
            acc_u.x += u.x; acc_u.y += u.y; acc_u.z += u.z; acc_u.w += u.w;
          }
        }
        if (p.ssq_in) {
          const float rs = s_rstd[m];
          acc.x *= rs; acc.y *= rs; acc.z *= rs; acc.w *= rs;
          acc_u.x *= rs; acc_u.y *= rs; acc_u.z *= rs; acc_u.w *= rs;
        }
        if (p.swiglu) {
          acc.x = acc.x / (1.f + __expf(-acc.x)) * acc_u.x;
          acc.y = acc.y / (1.f + __expf(-acc.y)) * acc_u.y;
          acc.z = acc.z / (1.f + __expf(-acc.z)) * acc_u.z;
          acc.w = acc.w / (1.f + __expf(-acc.w)) * acc_u.w;
        }
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
          if (p.ssq_out) {
            // what the next norm sees is the bf16 value that was just stored
            const float2 h0 = unpack_bf16x2(o.x), h1 = unpack_bf16x2(o.y);
            acc = make_float4(h0.x, h0.y, h1.x, h1.y);
            const uint2 wv = *reinterpret_cast<const uint2*>(p.norm_w + n);
            const float2 w0 = unpack_bf16x2(wv.x), w1 = unpack_bf16x2(wv.y);
            uint2 o2;
            o2.x = pack_bf16x2(acc.x * w0.x, acc.y * w0.y);
            o2.y = pack_bf16x2(acc.z * w1.x, acc.w * w1.y);
            *reinterpret_cast<uint2*>(p.Y2 + static_cast<long long>(m) * p.ldy2 + n) = o2;
          }
        }
      }
      if (p.ssq_out) {
        float sq = valid ? acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w : 0.f;
        sq = warp_sum(sq);
        if (live && (threadIdx.x & 31) == 0) p.ssq_out[n_blk * p.ssq_out_stride + m] = sq;
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
  const int tiles = p.swiglu ? (p.N + 63) / 64 : (p.N + SK_BM - 1) / SK_BM;
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
//
// Optional fusions (see the head of this file), each switched on by a non-null pointer / non-zero flag:
//   ssq_in [ssq_in_tiles, ssq_in_stride] fp32: the output rows are scaled by rsqrt(sum_t ssq_in[t][m] / K + eps), i.e. X is
//       h * w_norm of an RMSNorm whose row statistic the producer of X left in ssq_in;
//   ssq_out [ceil(N / 128), ssq_out_stride] fp32 + norm_w [N] bf16 + Y2 [M, N] bf16 (bf16 output only): besides Y the kernel
//       writes Y2 = Y * norm_w and the per-tile partial sums of squares of Y for the next norm;
//   swiglu: W is [2N, K] = [gate | up] and Y[M, N] = silu(X gate^T) * (X up^T); N must be a multiple of 64.
RLB_API int rlb_gemm_skinny_fused(const void* X, const void* W, void* Y, int M, int N, int K, long long ldx, long long ldw,
                                  long long ldy, int out_fp32, const float* bias, const void* residual, long long ldr,
                                  int split, const float* ssq_in, int ssq_in_tiles, long long ssq_in_stride, float eps,
                                  float* ssq_out, long long ssq_out_stride, const void* norm_w, void* Y2, long long ldy2,
                                  int swiglu, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256) return -7;
  if ((ldx % 8) || (ldw % 8) || (N % 8) || (ldy % (out_fp32 ? 4 : 8)) || (residual && (ldr % 4))) return -2;
  if (swiglu && ((N % 64) || bias || residual || ssq_out)) return -2;
  if (ssq_out && (out_fp32 || !norm_w || !Y2 || (ldy2 % 4) || ssq_out_stride < M)) return -2;
  if (ssq_in && (ssq_in_tiles <= 0 || ssq_in_stride < M)) return -2;
  const int NT = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
  CUtensorMap tw, tx;
  const int w_rows = swiglu ? 2 * N : N;
  int rc = rlb_make_tmap_2d(&tw, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, w_rows, ldw * 2, SK_BK, swiglu ? 64 : SK_BM,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tx, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, SK_BK, NT,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return -100 - rc;
  if (split <= 0) split = rlb_gemm_skinny_split(w_rows, K);
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
  p.ssq_in = ssq_in;
  p.ssq_in_tiles = ssq_in_tiles;
  p.ssq_in_stride = ssq_in_stride;
  p.eps = eps;
  p.ssq_out = ssq_out;
  p.ssq_out_stride = ssq_out_stride;
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.Y2 = reinterpret_cast<__nv_bfloat16*>(Y2);
  p.ldy2 = ldy2;
  p.swiglu = swiglu ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (NT) {
    case 32: return launch_skinny<32>(tw, tx, p, split, s);
    case 64: return launch_skinny<64>(tw, tx, p, split, s);
    case 128: return launch_skinny<128>(tw, tx, p, split, s);
    default: return launch_skinny<256>(tw, tx, p, split, s);
  }
}

RLB_API int rlb_gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, long long ldx, long long ldw,
                            long long ldy, int out_fp32, const float* bias, const void* residual, long long ldr,
                            int split, int* status, void* stream) {
  return rlb_gemm_skinny_fused(X, W, Y, M, N, K, ldx, ldw, ldy, out_fp32, bias, residual, ldr, split, nullptr, 0, 0, 0.f,
                               nullptr, 0, nullptr, nullptr, 0, 0, status, stream);
}
