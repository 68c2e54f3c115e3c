// Peer-memory communication over NVLink / NVSwitch: symmetric buffers shared between the ranks of one node through
// CUDA IPC, flag barriers with bounded waits, and the fused optimizer step
//
//     reduce-scatter(fp32 grads) -> global grad-norm + clip -> AdamW on the local shard -> all-gather(bf16 params)
//
// as ONE cooperative kernel. Every rank pulls its shard of the gradient from all peers with plain P2P loads (fixed
// rank order, so the sum is bit-reproducible), keeps the reduced shard in its own gradient buffer, exchanges one
// float per rank for the global norm, applies AdamW to the split fp32 master (bf16 + 16 low bits), and pushes the new
// bf16 parameters straight into every peer's parameter buffer with P2P stores. No NCCL call, no staging copy, no
// separate cast / scale / norm kernels; the NCCL form in rl_b200/policy/optimizer.py is its twin.
//
// Cross-GPU waits spin on flag words that peers write with st.release.sys; every wait is bounded by %globaltimer and
// records a status code instead of hanging. No multimem / multicast object is used, so a rank that dies cannot fault
// its peers' GPUs through a shared multicast binding.
//
// Counterpart in the reference: FSDP2 reduce-scatter + torch.optim.AdamW + parameter all-gather
// (nemo_rl/models/automodel/setup.py:481-493, nemo_rl/models/dtensor/parallelize.py:780-882).
#include "common.cuh"

#include <cooperative_groups.h>
#include <string.h>

namespace {
using namespace rlb;
namespace cg = cooperative_groups;

constexpr int MAX_RANKS = 8;
constexpr int FLAG_STAGES = 4;

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerTable {
  float* grad[MAX_RANKS];            // full fp32 gradient buffers
  __nv_bfloat16* param[MAX_RANKS];   // full bf16 parameter buffers
  unsigned int* flags[MAX_RANKS];    // [FLAG_STAGES][MAX_RANKS] epoch words
  float* slots[MAX_RANKS];           // [MAX_RANKS] per-rank partial sums of squares
};

// Flag barrier run by the first `world` threads of one CTA. Returns false when a peer did not arrive in time.
__device__ bool peer_barrier(const PeerTable& t, int rank, int world, int stage, unsigned int epoch,
                             unsigned long long limit_ns, int* status) {
  bool ok = true;
  if (threadIdx.x < world) {
    st_release_sys(t.flags[threadIdx.x] + stage * MAX_RANKS + rank, epoch);
    const unsigned int* mine = t.flags[rank] + stage * MAX_RANKS + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    // epochs only grow; the signed difference tolerates wrap-around
    while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
      if (globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, RLB_ERR_WAIT_PEER);
        ok = false;
        break;
      }
    }
  }
  return __syncthreads_and(ok);
}

struct FusedOptimArgs {
  PeerTable peers;
  int rank, world;
  long long shard_n;      // elements per rank (multiple of 8)
  int16_t* p_lo;          // [shard_n] low 16 bits of the fp32 master
  float* m;
  float* v;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  float max_grad_norm;    // <= 0: no clipping
  float grad_div;         // the summed gradient is divided by this
  unsigned int epoch;     // grows by one per call
  unsigned long long limit_ns;
  float* sumsq_local;     // [1] scratch, zeroed by the kernel
  int* abort_word;        // [1] scratch: set when a peer barrier ran out, read by the whole grid after the next grid.sync
  float* norm_out;        // [1] global gradient norm
  int* status;
};

__device__ __forceinline__ void split16(float w, __nv_bfloat16& hi, int16_t& lo) {
  const uint32_t bits = __float_as_uint(w);
  const uint32_t hb = (bits + 0x8000u) & 0xFFFF0000u;
  hi = __ushort_as_bfloat16(static_cast<unsigned short>(hb >> 16));
  lo = static_cast<int16_t>(static_cast<int32_t>(bits - hb));
}
__device__ __forceinline__ float join16(__nv_bfloat16 hi, int16_t lo) {
  return __uint_as_float((static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16) + static_cast<uint32_t>(static_cast<int32_t>(lo)));
}

__global__ void __launch_bounds__(512, 1) fused_optim_kernel(FusedOptimArgs a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float red[32];
  __shared__ float s_scale;
  const long long lo = static_cast<long long>(a.rank) * a.shard_n;
  const long long n4 = a.shard_n / 4;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;

  // A peer barrier that runs out aborts the whole grid at the next grid-wide synchronisation: the status word holds
  // RLB_ERR_WAIT_PEER, and parameters, moments and every peer's buffers are left exactly as they were (a failure after
  // pass 1 leaves the locally reduced gradient shard behind, nothing else).
  // stage 0: every rank's gradients are complete
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) *a.sumsq_local = 0.f;
    const bool ok = peer_barrier(a.peers, a.rank, a.world, 0, a.epoch, a.limit_ns, a.status);
    if (threadIdx.x == 0) *a.abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(a.abort_word)) return;

  // pass 1: pull-reduce my shard from all peers (fixed order), keep it locally, accumulate the sum of squares
  float ss = 0.f;
  float* mine = a.peers.grad[a.rank] + lo;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < a.world) {
        const float4 g = reinterpret_cast<const float4*>(a.peers.grad[r] + lo)[i];
        acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
      }
    }
    reinterpret_cast<float4*>(mine)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) atomicAdd(a.sumsq_local, ss);
  grid.sync();

  // stage 1: exchange the partial sums, derive the clip coefficient
  if (blockIdx.x == 0) {
    if (threadIdx.x < a.world) a.peers.slots[threadIdx.x][a.rank] = *a.sumsq_local;
    __threadfence_system();
    __syncthreads();
    const bool ok = peer_barrier(a.peers, a.rank, a.world, 1, a.epoch, a.limit_ns, a.status);
    if (threadIdx.x == 0 && !ok) *a.abort_word = 1;
    if (threadIdx.x == 0 && ok) {
      float total = 0.f;
      for (int r = 0; r < a.world; ++r) total += reinterpret_cast<volatile float*>(a.peers.slots[a.rank])[r];
      const float norm = sqrtf(total) / a.grad_div;
      float scale = 1.f / a.grad_div;
      if (a.max_grad_norm > 0.f) scale *= fminf(1.f, a.max_grad_norm / (norm + 1e-6f));
      *a.norm_out = norm;
      *a.sumsq_local = scale;  // broadcast to the grid through global memory
    }
  }
  __threadfence();
  grid.sync();
  if (*reinterpret_cast<volatile int*>(a.abort_word)) return;
  if (threadIdx.x == 0) s_scale = *reinterpret_cast<volatile float*>(a.sumsq_local);
  __syncthreads();
  const float gs = s_scale;

  // pass 2: AdamW on the shard, new bf16 parameters written into every rank's parameter buffer
  const __nv_bfloat16* p_mine = a.peers.param[a.rank] + lo;
  for (long long i = tid; i < n4; i += nthreads) {
    const float4 g4 = reinterpret_cast<const float4*>(mine)[i];
    float4 m4 = reinterpret_cast<float4*>(a.m)[i];
    float4 v4 = reinterpret_cast<float4*>(a.v)[i];
    const uint2 pw = reinterpret_cast<const uint2*>(p_mine)[i];
    const uint2 lw = reinterpret_cast<const uint2*>(a.p_lo)[i];
    const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(&pw);
    const int16_t* pl = reinterpret_cast<const int16_t*>(&lw);
    float g[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
    __nv_bfloat16 nh[4];
    int16_t nl[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w = join16(ph[j], pl[j]);
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * g[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * g[j] * g[j];
      w *= (1.f - a.lr * a.weight_decay);
      w -= a.lr * (mm[j] / a.bc1) / (sqrtf(vv[j] / a.bc2) + a.eps);
      split16(w, nh[j], nl[j]);
    }
    reinterpret_cast<float4*>(a.m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(a.v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<uint2*>(a.p_lo)[i] = *reinterpret_cast<const uint2*>(nl);
    const uint2 out = *reinterpret_cast<const uint2*>(nh);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < a.world) reinterpret_cast<uint2*>(a.peers.param[r] + lo)[i] = out;
  }
  __threadfence_system();
  grid.sync();
  // stage 2: every rank has written its shard into my parameter buffer
  if (blockIdx.x == 0) peer_barrier(a.peers, a.rank, a.world, 2, a.epoch, a.limit_ns, a.status);
}

// out[r * n .. (r+1) * n) = peer r's `src` for every r (pull all-gather); flags as in the optimizer.
struct GatherArgs {
  const uint4* src[MAX_RANKS];
  uint4* dst;
  unsigned int* flags[MAX_RANKS];
  int rank, world;
  long long n16;  // 16-byte words per rank
  unsigned int epoch;
  unsigned long long limit_ns;
  int* status;
};
__global__ void __launch_bounds__(512, 1) p2p_allgather_kernel(GatherArgs a) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0) {
    PeerTable t;
    for (int r = 0; r < MAX_RANKS; ++r) t.flags[r] = a.flags[r];
    peer_barrier(t, a.rank, a.world, 3, a.epoch, a.limit_ns, a.status);
  }
  grid.sync();
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int r = 0; r < a.world; ++r) {
    const int src_rank = (a.rank + r) % a.world;  // start with the local copy, stagger the peers
    for (long long i = tid; i < a.n16; i += nthreads) a.dst[src_rank * a.n16 + i] = a.src[src_rank][i];
  }
}

// Column all-gather for tensor-parallel logits: every rank holds a [rows, cols_local] slice and needs the full
// [rows, world * cols_local] matrix. One cooperative kernel per rank, safe to record in a CUDA graph:
//   1. the local slice is copied into this rank's symmetric staging buffer, half (epoch & 1);
//   2. flag barrier: every rank has published its slice of this call (and so has finished reading the previous call's);
//   3. every rank pulls all slices (its own included) into its output with plain peer loads.
// The call's epoch lives in device memory (*epoch_ptr + 1, stored back), so replays of a captured launch stay in step;
// the two staging halves make the closing barrier unnecessary: a fast rank can only overwrite the half that every
// rank finished reading before it passed the barrier of the call in between.
struct GatherColsArgs {
  const uint4* local;            // [rows, row_vecs] 16-byte vectors of this rank's slice (dense)
  uint4* stage[MAX_RANKS];       // per rank: 2 halves of rows * row_vecs vectors
  unsigned int* flags[MAX_RANKS];
  uint4* out;                    // [rows, out_stride_vecs]
  long long out_stride_vecs;
  int rows, row_vecs;
  int rank, world;
  unsigned int* epoch_ptr;
  unsigned long long limit_ns;
  int* abort_word;
  int* status;
  long long half_vecs;           // offset of the second half of every stage
};
__global__ void __launch_bounds__(512, 1) p2p_gather_cols_kernel(GatherColsArgs a) {
  cg::grid_group grid = cg::this_grid();
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(a.epoch_ptr) + 1;
  const long long n = static_cast<long long>(a.rows) * a.row_vecs;
  // the two halves sit at fixed offsets, whatever this call's size: consecutive calls of different sizes never overlap
  const long long half = (epoch & 1u) ? a.half_vecs : 0;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* mine = a.stage[a.rank] + half;
  for (long long i = tid; i < n; i += nthreads) mine[i] = a.local[i];
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    PeerTable t;
    for (int r = 0; r < MAX_RANKS; ++r) t.flags[r] = a.flags[r];
    const bool ok = peer_barrier(t, a.rank, a.world, 0, epoch, a.limit_ns, a.status);
    if (threadIdx.x == 0) {
      *a.abort_word = ok ? 0 : 1;
      *a.epoch_ptr = epoch;   // every CTA read the old value before the grid barrier above
    }
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(a.abort_word)) return;   // a peer did not arrive: the output is left alone
  for (int p = 0; p < a.world; ++p) {
    const int r = (a.rank + p) % a.world;  // start with the local slice, stagger the peers
    const uint4* src = a.stage[r] + half;
    for (long long i = tid; i < n; i += nthreads) {
      const long long row = i / a.row_vecs, c = i - row * a.row_vecs;
      a.out[row * a.out_stride_vecs + static_cast<long long>(r) * a.row_vecs + c] = src[i];
    }
  }
}

// One-shot all-reduce of decode-sized partial sums over peer memory, with the epilogue of a row-parallel projection:
//   out[M, N]  = bf16( sum over ranks of partial_r[M, N] (fp32, fixed rank order) + residual )
//   out2[M, N] = out * rsqrt(mean(out^2) + eps) * norm_w          (optional: the RMSNorm that follows in the layer)
// One CTA per row and no grid-wide step: CTA r copies row r of this rank's partial sums into its symmetric stage, tells
// every peer "row r of epoch e is there" (one release store per peer), waits for the same word from every peer, then
// reduces row r from all stages with plain peer loads. The CTAs of one GPU never wait for each other, only for the same
// row's CTA on the other GPUs, which starts whether or not this GPU is ahead, so an ordinary (non-cooperative) launch
// is enough and the latency is one NVLink round trip instead of two grid barriers and a cross-GPU barrier.
// Stage and flag slots are double-buffered by the parity of a device-resident epoch: a peer signals epoch e + 1 only
// after its epoch-e kernel has finished reading, so the slots of epoch e are free again at e + 2. The last CTA to finish
// advances the epoch (every CTA read it on entry), so the launch replays from a CUDA graph. Waits are bounded; a CTA that
// gives up sets the status word and leaves its row's outputs untouched.
constexpr int AR_MAX_ROWS = 256;
struct AllReduceRowsArgs {
  const float4* partial;          // [M, N] fp32, this rank's partial sums
  const uint4* residual;          // [M, N] bf16 or null
  uint4* out;                     // [M, N] bf16
  const uint4* norm_w;            // [N] bf16 or null
  uint4* out2;                    // [M, N] bf16 (with norm_w)
  float4* stage[MAX_RANKS];       // per rank: two halves of half_f4 float4, rows at a pitch of N floats
  unsigned int* flags[MAX_RANKS]; // per rank: [2][AR_MAX_ROWS][MAX_RANKS] epoch words
  unsigned int* epoch_ptr;
  unsigned int* done_counter;     // device word, zero between launches
  unsigned long long limit_ns;
  int* status;
  long long half_f4;
  float eps;
  int M, N, rank, world;
};
__global__ void __launch_bounds__(256) p2p_allreduce_rows_kernel(AllReduceRowsArgs a) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const int row = blockIdx.x;
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(a.epoch_ptr) + 1;
  const unsigned int parity = epoch & 1u;
  const long long half = parity ? a.half_f4 : 0;
  const int f4_per_row = a.N / 4;
  float4* mine = a.stage[a.rank] + half + static_cast<long long>(row) * f4_per_row;
  const float4* src_row = a.partial + static_cast<long long>(row) * f4_per_row;
  for (int i = threadIdx.x; i < f4_per_row; i += blockDim.x) mine[i] = src_row[i];
  if (threadIdx.x == 0) s_ok = 1;
  __threadfence_system();
  __syncthreads();
  const long long slot = (static_cast<long long>(parity) * AR_MAX_ROWS + row) * MAX_RANKS;
  if (threadIdx.x < a.world) {
    st_release_sys(a.flags[threadIdx.x] + slot + a.rank, epoch);
    const unsigned int* wait_on = a.flags[a.rank] + slot + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    while (static_cast<int>(ld_acquire_sys(wait_on) - epoch) < 0) {
      if (globaltimer_ns() - t0 > a.limit_ns) {
        if (a.status) atomicCAS(a.status, 0, RLB_ERR_WAIT_PEER);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    const int vecs = a.N / 8;   // 8 columns per thread step
    float ssq = 0.f;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      const long long i = static_cast<long long>(row) * vecs + v;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < a.world; ++r) {
        const float4* src = a.stage[r] + half + 2 * i;
        const float4 lo = src[0], hi = src[1];
        acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
        acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
      }
      if (a.residual) {
        const uint4 rr = a.residual[i];
        const float2 r0 = rlb::unpack_bf16x2(rr.x), r1 = rlb::unpack_bf16x2(rr.y), r2 = rlb::unpack_bf16x2(rr.z), r3 = rlb::unpack_bf16x2(rr.w);
        acc[0] += r0.x; acc[1] += r0.y; acc[2] += r1.x; acc[3] += r1.y; acc[4] += r2.x; acc[5] += r2.y; acc[6] += r3.x; acc[7] += r3.y;
      }
      uint4 o;
      o.x = rlb::pack_bf16x2(acc[0], acc[1]); o.y = rlb::pack_bf16x2(acc[2], acc[3]);
      o.z = rlb::pack_bf16x2(acc[4], acc[5]); o.w = rlb::pack_bf16x2(acc[6], acc[7]);
      a.out[i] = o;
      if (a.norm_w) {   // the norm sees the bf16 residual stream, as the unfused RMSNorm kernel does
        const float2 q0 = rlb::unpack_bf16x2(o.x), q1 = rlb::unpack_bf16x2(o.y), q2 = rlb::unpack_bf16x2(o.z), q3 = rlb::unpack_bf16x2(o.w);
        ssq += q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y + q2.x * q2.x + q2.y * q2.y + q3.x * q3.x + q3.y * q3.y;
      }
    }
    if (a.norm_w) {
      const float tot = rlb::block_sum(ssq, red);
      const float rstd = rsqrtf(tot / static_cast<float>(a.N) + a.eps);
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
        const long long i = static_cast<long long>(row) * vecs + v;
        const uint4 o = a.out[i];   // written by this thread just above
        const uint4 w = a.norm_w[v];
        const float2 q0 = rlb::unpack_bf16x2(o.x), q1 = rlb::unpack_bf16x2(o.y), q2 = rlb::unpack_bf16x2(o.z), q3 = rlb::unpack_bf16x2(o.w);
        const float2 w0 = rlb::unpack_bf16x2(w.x), w1 = rlb::unpack_bf16x2(w.y), w2 = rlb::unpack_bf16x2(w.z), w3 = rlb::unpack_bf16x2(w.w);
        uint4 y;
        y.x = rlb::pack_bf16x2(q0.x * rstd * w0.x, q0.y * rstd * w0.y); y.y = rlb::pack_bf16x2(q1.x * rstd * w1.x, q1.y * rstd * w1.y);
        y.z = rlb::pack_bf16x2(q2.x * rstd * w2.x, q2.y * rstd * w2.y); y.w = rlb::pack_bf16x2(q3.x * rstd * w3.x, q3.y * rstd * w3.y);
        a.out2[i] = y;
      }
    }
  }
  // the last CTA to finish publishes the new epoch: every CTA of this launch read the old one on entry
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.done_counter, 1u) + 1u == gridDim.x) {
      *a.done_counter = 0;
      *a.epoch_ptr = epoch;
      __threadfence();
    }
  }
}

// Pull gather for fully sharded parameters: dst[r * n .. (r + 1) * n) = peer r's shard[off .. off + n) for every rank r.
// An ordinary (non-cooperative) launch of a few CTAs, meant for a side stream: the peers' shards do not change while a
// forward / backward pass runs, so no flag is needed, and the copy shares the GPU with the GEMMs of the previous unit
// instead of waiting for all SMs like the cooperative kernels above. Plain peer loads, four vectors in flight per thread.
__global__ void __launch_bounds__(512) p2p_pull_kernel(PeerTable t, long long src_off16, uint4* __restrict__ dst, long long n16,
                                                       int rank, int world) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int p = 0; p < world; ++p) {
    const int r = (rank + p) % world;   // the local slice first, then the peers, staggered by rank
    const uint4* src = reinterpret_cast<const uint4*>(t.param[r]) + src_off16;
    uint4* out = dst + static_cast<long long>(r) * n16;
    for (long long i0 = tid; i0 < n16; i0 += 4 * nthreads) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * nthreads < n16) v[u] = src[i0 + u * nthreads];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * nthreads < n16) out[i0 + u * nthreads] = v[u];
    }
  }
}

int coop_grid(const void* kernel, int threads) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0);
  if (per_sm < 1) per_sm = 1;
  return sms;  // one CTA per SM leaves the copy engines and other streams room
}

}  // namespace

// ---------------------------------------------------------------- symmetric buffers (CUDA IPC)
// Allocates `bytes` of device memory and returns its 64-byte IPC handle. Peers of the same node map it with
// rlb_symm_open. The memory comes from cudaMalloc (not the framework's caching allocator) so that it can be exported.
RLB_API int rlb_symm_alloc(unsigned long long bytes, void** ptr, char* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
RLB_API int rlb_symm_open(const char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
RLB_API int rlb_symm_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
RLB_API int rlb_symm_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }

// One fused optimizer step. Pointer tables have `world` entries, entry `rank` being this rank's own buffer.
// flags: uint32 [4][8] per rank (zero-initialised symmetric memory); slots: float [8] per rank; sumsq_scratch: 2 floats.
RLB_API int rlb_fused_optim_step(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs,
                                 void* const* slot_ptrs, int rank, int world, long long shard_n, void* p_lo, float* m,
                                 float* v, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                                 float max_grad_norm, float grad_div, unsigned int epoch, double wait_limit_s,
                                 float* sumsq_scratch, float* norm_out, int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || shard_n % 8) return -2;
  FusedOptimArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.peers.grad[r] = static_cast<float*>(grad_ptrs[r]);
    a.peers.param[r] = static_cast<__nv_bfloat16*>(param_ptrs[r]);
    a.peers.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
    a.peers.slots[r] = static_cast<float*>(slot_ptrs[r]);
  }
  a.rank = rank;
  a.world = world;
  a.shard_n = shard_n;
  a.p_lo = static_cast<int16_t*>(p_lo);
  a.m = m;
  a.v = v;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bc2 = 1.f - powf(beta2, static_cast<float>(step));
  a.max_grad_norm = max_grad_norm;
  a.grad_div = grad_div;
  a.epoch = epoch;
  a.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  a.sumsq_local = sumsq_scratch;
  a.abort_word = reinterpret_cast<int*>(sumsq_scratch + 1);
  a.norm_out = norm_out;
  a.status = status;
  const int grid = coop_grid(reinterpret_cast<const void*>(fused_optim_kernel), 512);
  void* args[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(fused_optim_kernel), dim3(grid), dim3(512),
                                                      args, 0, static_cast<cudaStream_t>(stream)));
}

// dst[r * bytes_per_rank ...] = peer r's src (pull all-gather over peer memory). bytes_per_rank multiple of 16.
RLB_API int rlb_p2p_allgather(void* const* src_ptrs, void* dst, void* const* flag_ptrs, int rank, int world,
                              long long bytes_per_rank, unsigned int epoch, double wait_limit_s, int* status,
                              void* stream) {
  if (world < 1 || world > MAX_RANKS || bytes_per_rank % 16) return -2;
  GatherArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.src[r] = static_cast<const uint4*>(src_ptrs[r]);
    a.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  }
  a.dst = static_cast<uint4*>(dst);
  a.rank = rank;
  a.world = world;
  a.n16 = bytes_per_rank / 16;
  a.epoch = epoch;
  a.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  a.status = status;
  const int grid = coop_grid(reinterpret_cast<const void*>(p2p_allgather_kernel), 512);
  void* args[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(p2p_allgather_kernel), dim3(grid),
                                                      dim3(512), args, 0, static_cast<cudaStream_t>(stream)));
}

// out[rows, world * cols] = concatenation over ranks of their `local` [rows, cols] slices (see p2p_gather_cols_kernel).
// row_bytes = cols * element size, a multiple of 16; stage_ptrs[r]: rank r's staging of 2 * half_bytes bytes, with
// half_bytes >= rows * row_bytes the same on every rank and in every call that shares the stage;
// flag_ptrs[r]: 8 zero-initialised uint32 words of symmetric memory; epoch_ptr: device uint32 (starts at 0);
// scratch: one device int.
RLB_API int rlb_p2p_gather_cols(const void* local, void* const* stage_ptrs, void* const* flag_ptrs, void* out,
                                long long out_stride_bytes, int rows, int row_bytes, int rank, int world, void* epoch_ptr,
                                double wait_limit_s, int* scratch, int* status, long long half_bytes, void* stream) {
  if (world < 1 || world > MAX_RANKS || rows <= 0 || row_bytes <= 0 || (row_bytes % 16) || (out_stride_bytes % 16)) return -2;
  if ((half_bytes % 16) || half_bytes < static_cast<long long>(rows) * row_bytes) return -2;
  if ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(out)) & 15) return -3;
  GatherColsArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.stage[r] = static_cast<uint4*>(stage_ptrs[r]);
    a.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  }
  a.local = static_cast<const uint4*>(local);
  a.out = static_cast<uint4*>(out);
  a.out_stride_vecs = out_stride_bytes / 16;
  a.rows = rows;
  a.row_vecs = row_bytes / 16;
  a.rank = rank;
  a.world = world;
  a.epoch_ptr = static_cast<unsigned int*>(epoch_ptr);
  a.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  a.abort_word = scratch;
  a.status = status;
  a.half_vecs = half_bytes / 16;
  const int grid = coop_grid(reinterpret_cast<const void*>(p2p_gather_cols_kernel), 512);
  void* args[] = {&a};
  return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(p2p_gather_cols_kernel), dim3(grid),
                                                      dim3(512), args, 0, static_cast<cudaStream_t>(stream)));
}

// One-shot all-reduce of fp32 partial sums [M, N] with residual add and optional fused RMSNorm (see
// p2p_allreduce_rows_kernel). M <= 256, N a multiple of 8; stage_ptrs[r]: rank r's stage of 2 * half_bytes bytes with
// half_bytes >= M * N * 4 (fixed per stage); flag_ptrs[r]: rlb_p2p_allreduce_flag_bytes() zero-initialised bytes of
// symmetric memory; epoch_ptr: device uint32 (starts at 0); scratch: one zero-initialised device word.
RLB_API int rlb_p2p_allreduce_flag_bytes() { return 2 * AR_MAX_ROWS * MAX_RANKS * static_cast<int>(sizeof(unsigned int)); }
RLB_API int rlb_p2p_allreduce_rows(const void* partial, const void* residual, void* out, const void* norm_w, void* out2, float eps,
                                   int M, int N, void* const* stage_ptrs, void* const* flag_ptrs, int rank, int world,
                                   void* epoch_ptr, double wait_limit_s, int* scratch, int* status, long long half_bytes,
                                   void* stream) {
  if (world < 1 || world > MAX_RANKS || M <= 0 || M > AR_MAX_ROWS || N <= 0 || (N % 8) || (half_bytes % 16) ||
      half_bytes < static_cast<long long>(M) * N * 4)
    return -2;
  if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual) |
       reinterpret_cast<uintptr_t>(norm_w) | reinterpret_cast<uintptr_t>(out2)) & 15)
    return -3;
  if (norm_w && !out2) return -2;
  AllReduceRowsArgs a;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < world; ++r) {
    a.stage[r] = static_cast<float4*>(stage_ptrs[r]);
    a.flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  }
  a.partial = static_cast<const float4*>(partial);
  a.residual = static_cast<const uint4*>(residual);
  a.out = static_cast<uint4*>(out);
  a.norm_w = static_cast<const uint4*>(norm_w);
  a.out2 = static_cast<uint4*>(out2);
  a.epoch_ptr = static_cast<unsigned int*>(epoch_ptr);
  a.done_counter = reinterpret_cast<unsigned int*>(scratch);
  a.limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
  a.status = status;
  a.half_f4 = half_bytes / 16;
  a.eps = eps;
  a.M = M; a.N = N; a.rank = rank; a.world = world;
  p2p_allreduce_rows_kernel<<<M, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// dst[r * bytes_per_rank ...] = (shard_ptrs[r] + src_offset_bytes)[0 .. bytes_per_rank) for r < world, with `ctas` CTAs
// (0: 24). Offsets and sizes are multiples of 16 bytes. No synchronisation between ranks: the caller guarantees that the
// peers' shards are stable for the duration of the call (see p2p_pull_kernel).
RLB_API int rlb_p2p_pull(void* const* shard_ptrs, long long src_offset_bytes, void* dst, long long bytes_per_rank, int rank,
                         int world, int ctas, void* stream) {
  if (world < 1 || world > MAX_RANKS || (src_offset_bytes % 16) || (bytes_per_rank % 16) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return -2;
  if (bytes_per_rank == 0) return 0;
  PeerTable t;
  memset(&t, 0, sizeof(t));
  for (int r = 0; r < world; ++r) t.param[r] = static_cast<__nv_bfloat16*>(shard_ptrs[r]);
  if (ctas <= 0) ctas = 24;
  p2p_pull_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(t, src_offset_bytes / 16, static_cast<uint4*>(dst),
                                                                      bytes_per_rank / 16, rank, world);
  return static_cast<int>(cudaGetLastError());
}
