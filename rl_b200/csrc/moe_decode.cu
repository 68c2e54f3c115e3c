// Mixture-of-experts layer for small token counts (decode steps, short prefills) on sm_100a: the whole routing /
// layout / combine chain as five small kernels around the two grouped GEMMs, with fixed shapes and no host visit, so a
// decode step of an MoE model can be captured in a CUDA graph.
//
//   route_topk     one warp per token: soft-max over the router logits, top-k (lowest index wins ties), optional
//                  renormalisation of the k weights.
//   decode_plan    one CTA: stable counting sort of the token copies whose expert lives on this rank into the
//                  padded-by-expert row layout of the grouped GEMM (each expert's rows padded to a multiple of 128);
//                  writes, per padded row, the token it holds, per copy its row (or -1: expert of another rank), and
//                  the tile -> expert table.
//   gather_rows    padded rows <- token rows (zeros in padding rows of live tiles).
//   combine        out[t] = residual[t] + sum_j w[t, j] * y[row(t, j)] over this rank's copies, in copy order.
//   combine_reduce the expert-parallel form: every rank has ALL ranks' tokens (gathered before the router, which every
//                  rank evaluates identically), computes the contribution of its own experts to every token, writes
//                  these fp32 partial sums to its symmetric stage, meets the other ranks at a flag barrier and sums its own
//                  tokens' rows from all ranks' stages over NVLink (plain peer loads), adding the residual. Stages are
//                  double-buffered by the parity of a device-resident epoch, so consecutive layers need one barrier
//                  each and the kernel can be replayed from a graph. Waits are bounded; a rank that gives up sets the
//                  status word and leaves its output untouched.
//
// With few tokens per rank this replaces the dispatch / combine all-to-all of the training path: the bytes that cross
// NVLink per layer are tokens x hidden (in) and tokens x hidden x 4 (out) per peer, far below the expert weights
// every rank streams from its own HBM anyway.
// Reference counterpart: the token dispatchers of the Megatron MoE layer (nemo_rl/models/megatron/setup.py:888-1023)
// and vLLM's fused MoE decode path used by the reference's generation backend.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {
using namespace rlb;
constexpr int MAX_EP = 8;
constexpr int MAX_K = 16;
constexpr int PLAN_MAX_COPIES = 16384;
constexpr int PLAN_MAX_EXPERTS = 256;

__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------------------ routing
// logits bf16 [T, E] (row stride ld). One warp per token; the row is staged in shared memory as fp32.
__global__ void __launch_bounds__(256) route_topk_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int T, int E, int k,
                                                         int renorm, float* __restrict__ out_w, int* __restrict__ out_idx) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* p = smem + warp * E;
  const __nv_bfloat16* row = logits + static_cast<long long>(t) * ld;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float v = __bfloat162float(row[e]);
    p[e] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = __expf(p[e] - mx);
    p[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = 1.f / sum;
  float wsel = 0.f, wtot = 0.f;   // lane j keeps the j-th winner
  int isel = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = p[e];
      if (v > best) { best = v; bi = e; }   // ascending e per lane: the lowest index of equal values is kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == j) { wsel = best * inv; isel = bi; }
    wtot += best * inv;
    if (lane == 0) p[bi] = -2.f;
    __syncwarp();
  }
  if (lane < k) {
    out_w[static_cast<long long>(t) * k + lane] = renorm ? wsel / wtot : wsel;
    out_idx[static_cast<long long>(t) * k + lane] = isel;
  }
}

// ------------------------------------------------------------------------------------------------ layout plan
// idx [n_copies] global expert of every token copy (copy c belongs to token c / k). Experts [e_lo, e_lo + El) are local.
__global__ void __launch_bounds__(1024) decode_plan_kernel(const int* __restrict__ idx, int n_copies, int k, int e_lo, int El, int mpad,
                                                           int* __restrict__ src_tok, int* __restrict__ copy_row,
                                                           int* __restrict__ tile_expert, int* __restrict__ row0_out,
                                                           int* __restrict__ rows_out, int* status) {
  __shared__ short s_idx[PLAN_MAX_COPIES];   // local expert of every copy (-1: another rank's)
  __shared__ int s_cnt[PLAN_MAX_EXPERTS];
  __shared__ int s_row0[PLAN_MAX_EXPERTS + 1];
  const int tid = threadIdx.x, nthr = blockDim.x;
  for (int e = tid; e < El; e += nthr) s_cnt[e] = 0;
  __syncthreads();
  for (int c = tid; c < n_copies; c += nthr) {
    const int e = idx[c] - e_lo;
    const bool local = e >= 0 && e < El;
    s_idx[c] = local ? static_cast<short>(e) : static_cast<short>(-1);
    copy_row[c] = -1;
    if (local) atomicAdd(&s_cnt[e], 1);
  }
  for (int r = tid; r < mpad; r += nthr) src_tok[r] = -1;
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < El; ++e) {
      s_row0[e] = at;
      at += (s_cnt[e] + 127) / 128 * 128;
    }
    s_row0[El] = at;
    if (at > mpad && status) atomicCAS(status, 0, RLB_ERR_BOUNDS);   // cannot happen when mpad >= n_copies + El * 127
  }
  __syncthreads();
  const int total = min(s_row0[El], mpad);
  for (int e = tid; e < El; e += nthr) {
    row0_out[e] = s_row0[e];
    rows_out[e] = s_row0[e + 1] - s_row0[e];
  }
  for (int tile = tid; tile < mpad / 128; tile += nthr) {
    const int start = tile * 128;
    int te = -1;
    if (start < total) {
      int lo = 0, hi = El - 1;   // last expert whose first row is <= start
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_row0[mid] <= start) lo = mid; else hi = mid - 1;
      }
      te = lo;
    }
    tile_expert[tile] = te;
  }
  // stable ranks: one warp per expert walks the copies in order
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthr >> 5;
  for (int e = warp; e < El; e += nwarps) {
    if (s_cnt[e] == 0) continue;
    int at = s_row0[e];
    for (int c0 = 0; c0 < n_copies; c0 += 32) {
      const int c = c0 + lane;
      const bool hit = c < n_copies && s_idx[c] == e;
      const unsigned int m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int row = at + __popc(m & ((1u << lane) - 1u));
        if (row < mpad) {
          copy_row[c] = row;
          src_tok[row] = c / k;
        }
      }
      at += __popc(m);
    }
  }
}

// One warp per padded row of a live tile: x_pad[row] = x[src_tok[row]] (zeros when the row is padding).
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x, long long x_stride_vecs, const int* __restrict__ src_tok,
                                                          const int* __restrict__ tile_expert, uint4* __restrict__ out, int mpad, int vecs) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * (blockDim.x >> 5) + warp; row < mpad; row += gridDim.x * (blockDim.x >> 5)) {
    if (tile_expert[row >> 7] < 0) continue;
    const int t = src_tok[row];
    uint4* d = out + static_cast<long long>(row) * vecs;
    if (t < 0) {
      for (int v = lane; v < vecs; v += 32) d[v] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* s = x + static_cast<long long>(t) * x_stride_vecs;
      for (int v = lane; v < vecs; v += 32) d[v] = s[v];
    }
  }
}

// acc[8] += w * y_row[8 bf16 at vector v]
__device__ __forceinline__ void fma_row(float (&acc)[8], const uint4 v, float w) {
  const float2 a0 = unpack_bf16x2(v.x), a1 = unpack_bf16x2(v.y), a2 = unpack_bf16x2(v.z), a3 = unpack_bf16x2(v.w);
  acc[0] += w * a0.x; acc[1] += w * a0.y; acc[2] += w * a1.x; acc[3] += w * a1.y;
  acc[4] += w * a2.x; acc[5] += w * a2.y; acc[6] += w * a3.x; acc[7] += w * a3.y;
}

// Weighted sum of a token's local copies, 8 columns per thread. y rows are rounded to bf16 after the weight is applied,
// as the unfused path does (ys * w in the model dtype).
__device__ __forceinline__ void token_partial(float (&acc)[8], const uint4* __restrict__ y, int vecs, int v, const int* rows, const float* w, int k) {
#pragma unroll
  for (int q = 0; q < 8; ++q) acc[q] = 0.f;
  for (int j = 0; j < k; ++j) {
    const int r = rows[j];
    if (r < 0) continue;
    float one[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    fma_row(one, y[static_cast<long long>(r) * vecs + v], __bfloat162float(__float2bfloat16(w[j])));
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] += __bfloat162float(__float2bfloat16(one[q]));
  }
}

__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 o;
  o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]); o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
  return o;
}

__global__ void __launch_bounds__(256) combine_kernel(const uint4* __restrict__ y, const int* __restrict__ copy_row, const float* __restrict__ w,
                                                      const uint4* __restrict__ residual, uint4* __restrict__ out, int T, int k, int vecs) {
  const long long n = static_cast<long long>(T) * vecs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vecs), v = static_cast<int>(i - static_cast<long long>(t) * vecs);
    float acc[8];
    token_partial(acc, y, vecs, v, copy_row + static_cast<long long>(t) * k, w + static_cast<long long>(t) * k, k);
    if (residual) {
      const uint4 r = residual[i];
      const float2 a0 = unpack_bf16x2(r.x), a1 = unpack_bf16x2(r.y), a2 = unpack_bf16x2(r.z), a3 = unpack_bf16x2(r.w);
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    out[i] = pack8(acc);
  }
}

struct CombineReduceArgs {
  const uint4* y;            // [mpad, d] bf16 expert outputs in the padded layout
  const int* copy_row;       // [world * T, k]
  const float* w;            // [world * T, k]
  const uint4* residual;     // [T, d] bf16 or null
  uint4* out;                // [T, d] bf16
  float4* stage[MAX_EP];     // per rank: 2 halves of world * T * d floats
  unsigned int* flags[MAX_EP];
  unsigned int* epoch_ptr;
  int* abort_word;
  int* status;
  unsigned long long limit_ns;
  long long half_f4;
  int T, k, vecs, rank, world;
};

__global__ void __launch_bounds__(512, 1) combine_reduce_kernel(CombineReduceArgs a) {
  cg::grid_group grid = cg::this_grid();
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(a.epoch_ptr) + 1;
  const long long per_rank = static_cast<long long>(a.T) * a.vecs;          // 8-column groups of one rank's tokens
  const long long all = per_rank * a.world;
  const long long half = (epoch & 1u) ? a.half_f4 : 0;                      // fixed offset of the second half (float4 units)
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* mine = a.stage[a.rank] + half;
  for (long long i = tid; i < all; i += nthreads) {
    const int t = static_cast<int>(i / a.vecs), v = static_cast<int>(i - static_cast<long long>(t) * a.vecs);
    float acc[8];
    token_partial(acc, a.y, a.vecs, v, a.copy_row + static_cast<long long>(t) * a.k, a.w + static_cast<long long>(t) * a.k, a.k);
    mine[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    mine[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < a.world) {
      st_release_sys_u32(a.flags[threadIdx.x] + a.rank, epoch);
      const unsigned int* slot = a.flags[a.rank] + threadIdx.x;
      const unsigned long long t0 = globaltimer_ns();
      while (static_cast<int>(ld_acquire_sys_u32(slot) - epoch) < 0) {
        if (globaltimer_ns() - t0 > a.limit_ns) {
          if (a.status) atomicCAS(a.status, 0, RLB_ERR_WAIT_PEER);
          s_ok = 0;
          break;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *a.abort_word = s_ok ? 0 : 1;
      *a.epoch_ptr = epoch;   // every CTA read the old value before the grid barrier above
    }
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(a.abort_word)) return;
  for (long long i = tid; i < per_rank; i += nthreads) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < a.world; ++r) {   // fixed rank order: the sum does not depend on who arrives first
      const float4* src = a.stage[r] + half + 2 * (static_cast<long long>(a.rank) * per_rank + i);
      const float4 lo = src[0], hi = src[1];
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
    if (a.residual) {
      const uint4 rr = a.residual[i];
      const float2 a0 = unpack_bf16x2(rr.x), a1 = unpack_bf16x2(rr.y), a2 = unpack_bf16x2(rr.z), a3 = unpack_bf16x2(rr.w);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = __bfloat162float(__float2bfloat16(acc[q]));   // the experts' sum in the model dtype first
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    a.out[i] = pack8(acc);
  }
}
}  // namespace

RLB_API int rlb_moe_route_topk(const void* logits, long long ld, int T, int E, int k, int renorm, float* out_w, int* out_idx,
                               void* stream) {
  if (T <= 0) return 0;
  if (k < 1 || k > MAX_K || k > 32 || E < k || E > 4096) return -2;
  const int warps = 8;
  const size_t smem = static_cast<size_t>(warps) * E * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(route_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  route_topk_kernel<<<(T + warps - 1) / warps, warps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, T, E, k, renorm, out_w, out_idx);
  return static_cast<int>(cudaGetLastError());
}

// mpad: rows of the padded layout, a multiple of 128 and >= n_copies + El * 127 rounded up (worst case: all copies local).
RLB_API int rlb_moe_decode_plan(const int* idx, int n_copies, int k, int e_lo, int El, int mpad, int* src_tok, int* copy_row,
                                int* tile_expert, int* row0, int* rows, int* status, void* stream) {
  if (n_copies <= 0 || n_copies > PLAN_MAX_COPIES || El < 1 || El > PLAN_MAX_EXPERTS || k < 1 || (mpad % 128) ||
      mpad < n_copies + El * 127)
    return -2;
  decode_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(idx, n_copies, k, e_lo, El, mpad, src_tok, copy_row, tile_expert,
                                                                         row0, rows, status);
  return static_cast<int>(cudaGetLastError());
}

RLB_API int rlb_moe_gather_rows(const void* x, long long x_stride_bytes, const int* src_tok, const int* tile_expert, void* out, int mpad,
                                int row_bytes, void* stream) {
  if (mpad <= 0) return 0;
  if ((row_bytes % 16) || (x_stride_bytes % 16) || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15)) return -2;
  int grid = (mpad + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(x), x_stride_bytes / 16, src_tok,
                                                                           tile_expert, static_cast<uint4*>(out), mpad, row_bytes / 16);
  return static_cast<int>(cudaGetLastError());
}

// out[T, d] = residual + sum of this rank's weighted expert rows (single-rank form). d a multiple of 8, bf16.
RLB_API int rlb_moe_combine(const void* y, const int* copy_row, const float* w, const void* residual, void* out, int T, int k, int d,
                            void* stream) {
  if (T <= 0) return 0;
  if ((d % 8) || k < 1 || k > MAX_K) return -2;
  const long long n = static_cast<long long>(T) * (d / 8);
  int grid = static_cast<int>((n + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(y), copy_row, w,
                                                                       static_cast<const uint4*>(residual), static_cast<uint4*>(out), T, k, d / 8);
  return static_cast<int>(cudaGetLastError());
}

// Expert-parallel form. copy_row / w cover world * T tokens (rank-major); out / residual this rank's T tokens.
// stage_ptrs[r]: rank r's symmetric stage of 2 * half_bytes bytes (half_bytes >= world * T * d * 4, fixed per stage); flag_ptrs[r]: 8 zero-initialised uint32 words;
// epoch_ptr: device uint32 (starts at 0, advanced by the kernel); scratch: one device int.
RLB_API int rlb_moe_combine_reduce(const void* y, const int* copy_row, const float* w, const void* residual, void* out, int T, int k,
                                   int d, void* const* stage_ptrs, void* const* flag_ptrs, int rank, int world, void* epoch_ptr,
                                   double wait_limit_s, int* scratch, int* status, long long half_bytes, void* stream) {
  if (T <= 0 || world < 1 || world > MAX_EP || (d % 8) || k < 1 || k > MAX_K) return -2;
  if ((half_bytes % 16) || half_bytes < static_cast<long long>(world) * T * d * 4) return -2;
  CombineReduceArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.stage[r] = static_cast<float4*>(stage_ptrs[r]);
    a.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  }
  a.y = static_cast<const uint4*>(y);
  a.copy_row = copy_row;
  a.w = w;
  a.residual = static_cast<const uint4*>(residual);
  a.out = static_cast<uint4*>(out);
  a.epoch_ptr = static_cast<unsigned int*>(epoch_ptr);
  a.abort_word = scratch;
  a.status = status;
  a.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  a.half_f4 = half_bytes / 16;
  a.T = T; a.k = k; a.vecs = d / 8; a.rank = rank; a.world = world;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  void* args[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(combine_reduce_kernel), dim3(sms), dim3(512), args, 0,
                                                      static_cast<cudaStream_t>(stream)));
}
