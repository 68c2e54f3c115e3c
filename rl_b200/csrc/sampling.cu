// Token sampling for the generation engine: temperature, top-k, top-p, multinomial draw and the
// log-probability of the drawn token under the *processed* distribution, one CTA per sequence.
//
// The draw uses the Gumbel-max construction: argmax_i (z_i / T + g_i) with g_i ~ Gumbel(0,1) is a
// sample of softmax(z / T). That needs no normalisation and no prefix sums, so the unfiltered case
// is a single pass over the logits. top-k / top-p turn into a threshold on the logit value, found by
// bisection over the ordered bit pattern of fp32 (exact, 32 passes over an L2-resident row).
// Random numbers come from Philox4x32-10 keyed by (seed, step), counter (row, column / 4).
//
// Stands in for the vLLM sampler and FlashInfer sampling kernels the reference calls
// (nemo_rl/models/generation/vllm/vllm_worker.py:641-668) and mirrors the train-side filter
// semantics of nemo_rl/algorithms/logits_sampling_utils.py:112-210.
#include "common.cuh"

#include <math.h>

namespace {
using namespace rlb;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                           uint32_t k1, uint32_t (&out)[4]) {
  uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  // u in (0,1): 24 random bits, centred
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(-__logf(u));
}
// order-preserving map float -> uint
__device__ __forceinline__ uint32_t f2ord(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o;
  return __uint_as_float(u);
}

template <typename T>
__device__ __forceinline__ float ldz(const T* p, int i) {
  return static_cast<float>(p[i]);
}

struct ArgBest {
  float key;
  int idx;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.key > a.key || (b.key == a.key && b.idx < a.idx)) return b;
  return a;
}
__device__ __forceinline__ ArgBest block_argmax(ArgBest v, ArgBest* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest t;
    t.key = __shfl_xor_sync(0xffffffffu, v.key, o);
    t.idx = __shfl_xor_sync(0xffffffffu, v.idx, o);
    v = better(v, t);
  }
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  ArgBest r = (lane < nw) ? red[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest t;
    t.key = __shfl_xor_sync(0xffffffffu, r.key, o);
    t.idx = __shfl_xor_sync(0xffffffffu, r.idx, o);
    r = better(r, t);
  }
  return r;
}

// Per-row parameters may be null (then the scalar defaults apply).
template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, long long row_stride, int V, const float* __restrict__ temps,
              const int* __restrict__ top_ks, const float* __restrict__ top_ps, float def_temp, int def_top_k,
              float def_top_p, int greedy, unsigned long long seed, unsigned long long step,
              const unsigned long long* __restrict__ step_ptr, const long long* __restrict__ row_keys,
              int* __restrict__ out_tok, float* __restrict__ out_logprob) {
  if (step_ptr) step = *step_ptr;  // a counter in device memory lets a captured graph draw fresh numbers
  // With row_keys the random stream of a row depends only on (seed, key), e.g. key = request id and token position:
  // the draw is then independent of which other rows share the batch or which rank serves the request.
  const unsigned long long rk = row_keys ? static_cast<unsigned long long>(row_keys[blockIdx.x]) : 0ull;
  __shared__ float red[32];
  __shared__ ArgBest redb[32];
  const int row = blockIdx.x;
  const T* z = logits + static_cast<long long>(row) * row_stride;
  float temp = temps ? temps[row] : def_temp;
  const int top_k = top_ks ? top_ks[row] : def_top_k;
  const float top_p = top_ps ? top_ps[row] : def_top_p;
  const bool is_greedy = greedy || temp <= 0.f;
  if (temp <= 0.f) temp = 1.f;
  const float inv_t = 1.f / temp;

  const bool filtered = (top_k > 0 && top_k < V) || top_p < 1.f;
  // pass 1: maximum (only the filters need it up front; the unfiltered draw below finds it on the way)
  float mx = -INFINITY;
  if (filtered) {
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, ldz(z, i));
    mx = block_max(mx, red);
  }

  // Threshold from top-k / top-p (on raw logits; scaling by 1/T > 0 keeps the order). The filters compose the way the
  // train-side filter and vLLM apply them: top-k first, then the nucleus inside the renormalised top-k set. Both are a
  // bisection on the ordered-uint image of fp32; invariant: `lo` satisfies the predicate.
  float thr = -INFINITY;
  const bool need_k = top_k > 0 && top_k < V;
  const bool need_p = top_p < 1.f;
  if (need_k) {
    // x_k = largest x with count(z >= x) >= k, i.e. the k-th largest logit (ties at x_k are all kept)
    uint32_t lo = 0u, hi = f2ord(mx);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo + 1u) >> 1);
      const float x = ord2f(mid);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += (ldz(z, i) >= x) ? 1.f : 0.f;
      cnt = block_sum(cnt, red);
      if (cnt >= static_cast<float>(top_k)) lo = mid;
      else hi = mid - 1u;
    }
    thr = ord2f(lo);
  }
  if (need_p) {
    // mass of the set that survived top-k, then x_p = largest x >= x_k with mass(z >= x) >= top_p * that mass
    float total = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = ldz(z, i);
      if (v >= thr) total += __expf((v - mx) * inv_t);
    }
    total = block_sum(total, red);
    uint32_t lo = need_k ? f2ord(thr) : 0u, hi = f2ord(mx);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo + 1u) >> 1);
      const float x = ord2f(mid);
      float mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = ldz(z, i);
        if (v >= x) mass += __expf((v - mx) * inv_t);
      }
      mass = block_sum(mass, red);
      if (mass >= top_p * total) lo = mid;
      else hi = mid - 1u;
    }
    thr = ord2f(lo);
  }

  // final pass: normaliser over the kept set, and the draw. Without filters this is the only pass over the row: every
  // thread keeps a running maximum with a rescaled running sum (online softmax), and the Gumbel key needs no maximum.
  float sum = 0.f;
  float m_t = -INFINITY;
  ArgBest best{-INFINITY, 0x7fffffff};
  const uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  // fp32 rows that start on a 16-byte boundary are read four logits at a time
  const bool vec4 = sizeof(T) == 4 && (reinterpret_cast<uintptr_t>(z) & 15u) == 0;
  for (int i4 = threadIdx.x * 4; i4 < V; i4 += blockDim.x * 4) {
    uint32_t rnd[4] = {0, 0, 0, 0};
    if (!is_greedy)
      philox4x32(static_cast<uint32_t>(i4 >> 2), row_keys ? static_cast<uint32_t>(rk) : static_cast<uint32_t>(row),
                 row_keys ? static_cast<uint32_t>(rk >> 32) : static_cast<uint32_t>(step),
                 row_keys ? 0x5eedu : static_cast<uint32_t>(step >> 32), k0, k1, rnd);
    float vals[4];
    if (vec4 && i4 + 3 < V) {
      const float4 q = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(z) + i4);
      vals[0] = q.x; vals[1] = q.y; vals[2] = q.z; vals[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) vals[j] = i4 + j < V ? ldz(z, i4 + j) : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i4 + j;
      if (i < V) {
        const float v = vals[j];
        if (filtered) {
          if (v >= thr) {
            const float s = (v - mx) * inv_t;
            sum += __expf(s);
            const float key = is_greedy ? v : s + gumbel_from_bits(rnd[j]);
            best = better(best, ArgBest{key, i});
          }
        } else if (v > -INFINITY) {
          if (v > m_t) {
            sum = sum * __expf((m_t - v) * inv_t) + 1.f;
            m_t = v;
          } else {
            sum += __expf((v - m_t) * inv_t);
          }
          const float key = is_greedy ? v : v * inv_t + gumbel_from_bits(rnd[j]);
          best = better(best, ArgBest{key, i});
        }
      }
    }
  }
  if (!filtered) {
    mx = block_max(m_t, red);
    sum = m_t > -INFINITY ? sum * __expf((m_t - mx) * inv_t) : 0.f;
  }
  sum = block_sum(sum, red);
  best = block_argmax(best, redb);
  if (threadIdx.x == 0) {
    out_tok[row] = best.idx;
    if (out_logprob) {
      const float zt = ldz(z, best.idx);
      out_logprob[row] = (zt - mx) * inv_t - __logf(sum);
    }
  }
}

}  // namespace

// logits: [B, V] with row stride; dtype 0 = fp32, 1 = bf16. temps / top_ks / top_ps: per-row device arrays
// or null. Writes the sampled token and (optionally) its log-probability after temperature and filtering.
RLB_API int rlb_sample(const void* logits, int dtype, long long row_stride, int B, int V, const float* temps,
                       const int* top_ks, const float* top_ps, float def_temp, int def_top_k, float def_top_p,
                       int greedy, unsigned long long seed, unsigned long long step,
                       const unsigned long long* step_ptr, const long long* row_keys, int* out_tok,
                       float* out_logprob, void* stream) {
  if (B <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    sample_kernel<float><<<B, 1024, 0, s>>>(reinterpret_cast<const float*>(logits), row_stride, V, temps, top_ks,
                                           top_ps, def_temp, def_top_k, def_top_p, greedy, seed, step, step_ptr,
                                           row_keys, out_tok, out_logprob);
  else
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(logits), row_stride, V,
                                                    temps, top_ks, top_ps, def_temp, def_top_k, def_top_p, greedy,
                                                    seed, step, step_ptr, row_keys, out_tok, out_logprob);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------- device-resident decode state
// After a decode step has sampled one token per row, this kernel advances the engine's step inputs in place so that
// the next step can run without the host: the sampled token becomes the next input id, position / context length /
// random-stream key grow by one, the KV slot of the next token is looked up in the (pre-extended) block table, stop
// tokens and the per-row length limit retire a row (no further cache writes, empty context), and the token and its
// log-probability are appended to the window's output arrays. The host reads the outputs once per window of steps.
namespace {
struct AdvanceArgs {
  const int* tok;            // [B] sampled this step
  const float* lp;           // [B]
  int* ids;                  // [B] next step's input ids
  int* positions;            // [B]
  int* seq_lens;             // [B]
  long long* slots;          // [B] KV slot of the next step's token, -1: no write
  long long* keys;           // [B] random-stream keys
  const int* block_table;    // [B, bt_stride]
  int bt_stride;
  int* active;               // [B] 1 while the row still generates
  int* remaining;            // [B] tokens the row may still generate
  int* produced;             // [B] tokens appended to the outputs in this window
  const int* stop_ids;       // [n_stop]
  int n_stop;
  int* out_tok;              // [window, out_stride]
  float* out_lp;             // [window, out_stride]
  int out_stride;
  int max_window;
  int* win_step;             // [1] index of this step inside the window; incremented here
  int B, block_size;
};

__global__ void __launch_bounds__(1024) decode_advance_kernel(AdvanceArgs a) {
  pdl_wait();
  const int j = *a.win_step;
  for (int b = threadIdx.x; b < a.B; b += blockDim.x) {
    if (!a.active[b] || j >= a.max_window) {
      if (j == 0) a.produced[b] = 0;   // a row that is inactive from the start of the window produced nothing
      a.slots[b] = -1;
      continue;
    }
    const int t = a.tok[b];
    a.out_tok[static_cast<long long>(j) * a.out_stride + b] = t;
    a.out_lp[static_cast<long long>(j) * a.out_stride + b] = a.lp[b];
    a.produced[b] = j + 1;
    const int rem = a.remaining[b] - 1;
    a.remaining[b] = rem;
    bool stop = rem <= 0;
    for (int s = 0; s < a.n_stop; ++s) stop |= (a.stop_ids[s] == t);
    if (stop) {
      a.active[b] = 0;
      a.slots[b] = -1;
      a.seq_lens[b] = 0;
      a.ids[b] = 0;
      a.positions[b] = 0;
    } else {
      const int pos = a.positions[b] + 1;
      a.ids[b] = t;
      a.positions[b] = pos;
      a.seq_lens[b] = pos + 1;
      a.keys[b] += 1;
      const int blk = pos / a.block_size;
      a.slots[b] = blk < a.bt_stride
                       ? static_cast<long long>(a.block_table[static_cast<long long>(b) * a.bt_stride + blk]) * a.block_size + pos % a.block_size
                       : -1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *a.win_step = j + 1;
}
}  // namespace

// Advances the decode-step inputs of B rows after sampling (see above). All pointers are device memory; `win_step`
// must be zeroed by the host at the start of every window of at most `max_window` steps.
RLB_API int rlb_decode_advance(const int* tok, const float* lp, int* ids, int* positions, int* seq_lens, long long* slots,
                               long long* keys, const int* block_table, int bt_stride, int* active, int* remaining,
                               int* produced, const int* stop_ids, int n_stop, int* out_tok, float* out_lp, int out_stride,
                               int max_window, int* win_step, int B, int block_size, void* stream) {
  if (B <= 0) return 0;
  if (block_size <= 0 || bt_stride <= 0 || out_stride < B || max_window <= 0) return -2;
  AdvanceArgs a{tok, lp, ids, positions, seq_lens, slots, keys, block_table, bt_stride, active, remaining, produced,
                stop_ids, n_stop, out_tok, out_lp, out_stride, max_window, win_step, B, block_size};
  const int threads = B >= 1024 ? 1024 : ((B + 31) / 32) * 32;
  return static_cast<int>(rlb_launch_pdl(decode_advance_kernel, dim3(1), dim3(threads), 0, static_cast<cudaStream_t>(stream), a));
}
