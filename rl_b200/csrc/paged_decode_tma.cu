// Paged decode attention, TMA-pipelined: the bandwidth-critical kernel of generation.
//
// One CTA per (sequence, kv head, KV split). A producer warp walks the sequence's block table and streams K and V
// tiles of 64 tokens ([64 x 128] bf16, 16 KB each) from the paged cache into a 3-stage shared-memory ring with
// cp.async.bulk.tensor (plain row-major boxes, no swizzle: the consumers are CUDA cores). Four consumer warps read
// the tiles from shared memory: eight lanes share one token (16 head dimensions each), all G = Hq / Hkv query heads
// of the group reuse every K/V row, softmax is online per lane group. With ~100 KB of loads in flight per CTA and two
// CTAs per SM the kernel is limited by HBM, not by load latency (the plain-load variant in paged_attention.cu keeps
// only a few hundred bytes per thread in flight and reaches about a quarter of the bandwidth).
// Partial results of different KV splits are merged by a second kernel (flash-decoding).
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

constexpr int PD_D = 128;
constexpr int PD_TOK = 64;                       // tokens per stage
constexpr int PD_STAGES = 3;
constexpr int PD_TILE = PD_TOK * PD_D * 2;       // 16 KB
constexpr int PD_STAGE_BYTES = 2 * PD_TILE;      // K + V
constexpr int PD_GS = 4;                         // query heads per consumer thread: groups of 8 heads use two warp sets (no register spills); 2 was measured slower for groups of 4
constexpr int PD_LANES = 8;                      // lanes per token
constexpr int PD_GROUPS = 128 / PD_LANES;        // 16 tokens per consumer step
constexpr int PD_DL = PD_D / PD_LANES;           // 16 dims per lane

template <int G>
struct PdSmem {
  static constexpr int GS = G < PD_GS ? G : PD_GS;      // heads per thread
  static constexpr int SETS = G / GS;                   // warp sets: each set of 4 warps covers GS heads for all tokens
  static constexpr int THREADS = 32 + 128 * SETS;       // warp 0 producer, then 4 consumer warps per set
  static constexpr int MERGE = 4 * G * (PD_D + 2) * 4;
  static constexpr int BYTES = PD_STAGES * PD_STAGE_BYTES + MERGE + 128;
};

struct PdParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const int* block_table;
  int max_blocks_per_seq;
  const int* seq_lens;
  int Hkv, block_size;
  float scale;
  int num_splits;
  float* part_o;
  float* part_ml;
  __nv_bfloat16* out;
  long long out_stride;
  int* status;
};

template <int G>
__global__ void __launch_bounds__(PdSmem<G>::THREADS, (G <= 4 ? 2 : 1))
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        PdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  float* merge = reinterpret_cast<float*>(smem + PD_STAGES * PD_STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PD_STAGES * PD_STAGE_BYTES + PdSmem<G>::MERGE);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + PD_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * PD_STAGES);

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int Hq = p.Hkv * G;
  const int len = p.seq_lens[seq];
  const int bs = p.block_size;
  const int box_rows = bs < PD_TOK ? bs : PD_TOK;
  // split boundaries are multiples of the stage size
  const int per_split = ((len + p.num_splits - 1) / p.num_splits + PD_TOK - 1) / PD_TOK * PD_TOK;
  const int t_begin = split * per_split;
  const int t_end = min(len, t_begin + per_split);
  const int n_stage = t_end > t_begin ? (t_end - t_begin + PD_TOK - 1) / PD_TOK : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PD_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 4 * PdSmem<G>::SETS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      const int* bt = p.block_table + static_cast<long long>(seq) * p.max_blocks_per_seq;
      for (int i = 0; i < n_stage; ++i) {
        const int st = i % PD_STAGES;
        const uint32_t ph = (i / PD_STAGES) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[st]), ph ^ 1, abort_flag, p.status, RLB_ERR_WAIT_EMPTY)) break;
        const int t0 = t_begin + i * PD_TOK;
        // boxes of this stage: one per cache block (block_size < 64) or one slice of a block (block_size >= 64)
        int nbox = 0;
        for (int off = 0; off < PD_TOK && t0 + off < t_end; off += box_rows) ++nbox;
        const uint32_t bar = smem_u32(&full_bar[st]);
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nbox) * box_rows * PD_D * 2 * 2);
        const uint32_t k_dst = smem_u32(ring + st * PD_STAGE_BYTES);
        const uint32_t v_dst = k_dst + PD_TILE;
        for (int b = 0; b < nbox; ++b) {
          const int t = t0 + b * box_rows;
          const int blk = bt[t / bs];
          const int row = (blk * p.Hkv + kvh) * bs + (t % bs);
          tma_load_2d(k_dst + b * box_rows * PD_D * 2, &tmap_k, bar, 0, row);
          tma_load_2d(v_dst + b * box_rows * PD_D * 2, &tmap_v, bar, 0, row);
        }
      }
    }
  } else {
    constexpr int GS = PdSmem<G>::GS;
    const int cw = warp - 1;                   // consumer warp
    const int hset = cw >> 2;                  // which GS heads of the group this warp set serves
    const int ct = (cw & 3) * 32 + lane;       // 0..127 inside the set
    const int grp = ct / PD_LANES;             // token slot within a step
    const int sub = ct % PD_LANES;             // 16-dim slice
    float qr[GS][PD_DL];
#pragma unroll
    for (int g = 0; g < GS; ++g) {
      const __nv_bfloat16* qp = p.q + seq * p.q_stride + static_cast<long long>(kvh * G + hset * GS + g) * PD_D + sub * PD_DL;
      const uint4 a = *reinterpret_cast<const uint4*>(qp);
      const uint4 b = *reinterpret_cast<const uint4*>(qp + 8);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        qr[g][2 * j] = f.x * p.scale;
        qr[g][2 * j + 1] = f.y * p.scale;
      }
    }
    float o[GS][PD_DL], m[GS], l[GS];
#pragma unroll
    for (int g = 0; g < GS; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int j = 0; j < PD_DL; ++j) o[g][j] = 0.f;
    }
    for (int i = 0; i < n_stage; ++i) {
      const int st = i % PD_STAGES;
      const uint32_t ph = (i / PD_STAGES) & 1;
      // the verdict is made warp-uniform so that the shuffles below always see all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[st]), ph, abort_flag, p.status, RLB_ERR_WAIT_FULL))) break;
      const uint8_t* k_t = ring + st * PD_STAGE_BYTES;
      const uint8_t* v_t = k_t + PD_TILE;
      const int t0 = t_begin + i * PD_TOK;
#pragma unroll
      for (int step = 0; step < PD_TOK / PD_GROUPS; ++step) {
        const int tl = step * PD_GROUPS + grp;  // token inside the stage
        const bool valid = t0 + tl < t_end;
        const uint4 ka = *reinterpret_cast<const uint4*>(k_t + tl * (PD_D * 2) + sub * 32);
        const uint4 kb = *reinterpret_cast<const uint4*>(k_t + tl * (PD_D * 2) + sub * 32 + 16);
        const uint4 va = *reinterpret_cast<const uint4*>(v_t + tl * (PD_D * 2) + sub * 32);
        const uint4 vb = *reinterpret_cast<const uint4*>(v_t + tl * (PD_D * 2) + sub * 32 + 16);
        float kf[PD_DL], vf[PD_DL];
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
        for (int g = 0; g < GS; ++g) {
          // four independent partial sums: the 16-term dot product is not one serial FMA chain
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int j = 0; j < PD_DL; j += 4) {
            s0 += qr[g][j] * kf[j];
            s1 += qr[g][j + 1] * kf[j + 1];
            s2 += qr[g][j + 2] * kf[j + 2];
            s3 += qr[g][j + 3] * kf[j + 3];
          }
          float s = (s0 + s1) + (s2 + s3);
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          if (valid) {
            if (s > m[g]) {
              const float c = __expf(m[g] - s);
              l[g] *= c;
#pragma unroll
              for (int j = 0; j < PD_DL; ++j) o[g][j] *= c;
              m[g] = s;
            }
            const float pr = __expf(s - m[g]);
            l[g] += pr;
#pragma unroll
            for (int j = 0; j < PD_DL; ++j) o[g][j] += pr * vf[j];
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[st]));
    }
    __syncwarp();
    // merge the four lane groups of the warp with shuffles
#pragma unroll
    for (int g = 0; g < GS; ++g) {
      float mw = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], 8));
      mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
      const float c = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mw);
      float lw = l[g] * c;
      lw += __shfl_xor_sync(0xffffffffu, lw, 8);
      lw += __shfl_xor_sync(0xffffffffu, lw, 16);
#pragma unroll
      for (int j = 0; j < PD_DL; ++j) {
        float v = o[g][j] * c;
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        o[g][j] = v;
      }
      m[g] = mw;
      l[g] = lw;
    }
    // per-warp results to shared memory: [token warp 0..3][head of the group][D + 2]
    float* mine = merge + (static_cast<size_t>(cw & 3) * G + hset * GS) * (PD_D + 2);
    if (lane < PD_LANES) {
#pragma unroll
      for (int g = 0; g < GS; ++g) {
#pragma unroll
        for (int j = 0; j < PD_DL; ++j) mine[g * (PD_D + 2) + sub * PD_DL + j] = o[g][j];
        if (lane == 0) {
          mine[g * (PD_D + 2) + PD_D] = m[g];
          mine[g * (PD_D + 2) + PD_D + 1] = l[g];
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < PD_D) {
    const int d = threadIdx.x;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * G + g) * (PD_D + 2) + PD_D]);
      float ll = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = merge[(w * G + g) * (PD_D + 2) + PD_D];
        const float c = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
        ll += merge[(w * G + g) * (PD_D + 2) + PD_D + 1] * c;
        acc += merge[(w * G + g) * (PD_D + 2) + d] * c;
      }
      const int hq = kvh * G + g;
      if (p.num_splits == 1) {
        p.out[seq * p.out_stride + static_cast<long long>(hq) * PD_D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
      } else {
        const long long pi = (static_cast<long long>(seq) * Hq + hq) * p.num_splits + split;
        p.part_o[pi * PD_D + d] = acc;
        if (d == 0) {
          p.part_ml[pi * 2] = mm;
          p.part_ml[pi * 2 + 1] = ll;
        }
      }
    }
  }
}

__global__ void pd_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int num_splits,
                                  int Hq, __nv_bfloat16* __restrict__ out, long long out_stride) {
  const int seq = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const long long base = (static_cast<long long>(seq) * Hq + hq) * num_splits;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += part_ml[(base + s) * 2 + 1] * c;
    acc += part_o[(base + s) * PD_D + d] * c;
  }
  out[seq * out_stride + static_cast<long long>(hq) * PD_D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}

template <int G>
int launch_pd(const CUtensorMap& tk, const CUtensorMap& tv, const PdParams& p, int B, cudaStream_t stream) {
  auto kern = paged_decode_tma_kernel<G>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PdSmem<G>::BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(B, p.Hkv, p.num_splits);
  kern<<<grid, PdSmem<G>::THREADS, PdSmem<G>::BYTES, stream>>>(tk, tv, p);
  if (p.num_splits > 1) {
    dim3 g2(B, p.Hkv * G);
    pd_combine_kernel<<<g2, PD_D, 0, stream>>>(p.part_o, p.part_ml, p.num_splits, p.Hkv * G, p.out, p.out_stride);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Same contract as rlb_paged_decode, plus the total number of cache blocks (for the tensor maps) and a status word.
// block_size must be 16, 32, 64 or a multiple of 64; head_dim 128.
RLB_API int rlb_paged_decode_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                 int num_blocks, const int* block_table, int max_blocks_per_seq, const int* seq_lens,
                                 int B, int Hq, int Hkv, int D, int block_size, float scale, int num_splits,
                                 float* part_o, float* part_ml, void* out, long long out_stride, int* status,
                                 void* stream) {
  if (B <= 0) return 0;
  if (D != PD_D || Hq % Hkv) return -2;
  if (!(block_size == 16 || block_size == 32 || block_size % 64 == 0)) return -2;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_ml)) return -3;
  const int box_rows = block_size < PD_TOK ? block_size : PD_TOK;
  const unsigned long long rows = static_cast<unsigned long long>(num_blocks) * Hkv * block_size;
  CUtensorMap tk, tv;
  int rc = rlb_make_tmap_2d(&tk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PD_D, rows, PD_D * 2, PD_D, box_rows,
                            CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return -100 - rc;
  rc = rlb_make_tmap_2d(&tv, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PD_D, rows, PD_D * 2, PD_D, box_rows,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return -100 - rc;
  PdParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.seq_lens = seq_lens;
  p.Hkv = Hkv;
  p.block_size = block_size;
  p.scale = scale;
  p.num_splits = num_splits;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (Hq / Hkv) {
    case 1: return launch_pd<1>(tk, tv, p, B, s);
    case 2: return launch_pd<2>(tk, tv, p, B, s);
    case 4: return launch_pd<4>(tk, tv, p, B, s);
    case 8: return launch_pd<8>(tk, tv, p, B, s);
    default: return -4;
  }
}
