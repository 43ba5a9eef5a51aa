// Next-token choice from float32 logits [R, V]: greedy argmax, or temperature sampling by the
// Gumbel-max rule  argmax_i(logit_i / T + g_i),  g_i = -log(-log(u_i)),  which draws from
// softmax(logits / T) without a pass to normalise.  The uniforms come from Philox4x32-10 keyed
// by the row's stream key (made on the host from the sampling seed and the request) with the
// counter (vocabulary index / 4, position of the sampled token): the draw does not depend on
// the row's place in the batch or on what else is in it.
// Also: the chosen token's log-probability under softmax(logits / T) (T = 1 for greedy rows),
// the scatter of the chosen ids into the per-slot last-token table, and top-k log-probabilities.
#include "common.cuh"
#include <float.h>

using namespace tkb;

namespace {

struct Philox {
  static constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  __device__ static uint4 run(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
      const uint32_t hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
      const uint32_t hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
      c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
      k.x += W0;
      k.y += W1;
    }
    return c;
  }
};

__device__ __forceinline__ float uniform_open(uint32_t x) {
  // Inside (0, 1) and exact in float32: 23 random bits plus one half need 24 bits of significand, so the
  // largest value is 8388607.5 / 8388608 < 1 and the smallest 0.5 / 8388608 > 0.  (With 24 random bits the
  // sum 16777215.5 would round to 16777216, u = 1 and the Gumbel value to +inf.)
  return ((float)(x >> 9) + 0.5f) * (1.0f / 8388608.0f);
}
__device__ __forceinline__ float gumbel_of(uint32_t x) { return -logf(-logf(uniform_open(x))); }

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // larger value wins; equal values: smaller index wins (the first maximum)
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ Best warp_best(Best a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  return a;
}

constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ stream_key, const int* __restrict__ sample_pos,
              const int* __restrict__ row_slot, int* __restrict__ out_ids, float* __restrict__ out_logprob,
              int* __restrict__ last_token, int V) {
  __shared__ float s_v[SAMPLE_THREADS / 32];
  __shared__ int s_i[SAMPLE_THREADS / 32];
  __shared__ float s_m[SAMPLE_THREADS / 32];
  __shared__ float s_l[SAMPLE_THREADS / 32];
  __shared__ int s_choice;
  __shared__ float s_lse;
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const float* lg = logits + (size_t)r * V;
  const float T = temperature ? temperature[r] : 0.f;
  const bool greedy = !(T > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / T;
  const unsigned long long key = stream_key ? stream_key[r] : 0ull;
  const uint2 k2 = make_uint2((uint32_t)key, (uint32_t)(key >> 32));
  const uint32_t pos = sample_pos ? (uint32_t)sample_pos[r] : 0u;

  Best best = {-FLT_MAX, 0x7fffffff};
  float m = -FLT_MAX, l = 0.f;  // running max and sum of exp of logits * inv_t
  const int ngroups = (V + 3) >> 2;
  for (int g = threadIdx.x; g < ngroups; g += SAMPLE_THREADS) {
    uint4 rnd = make_uint4(0, 0, 0, 0);
    if (!greedy) rnd = Philox::run(make_uint4((uint32_t)g, pos, 0u, 0u), k2);
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int i = g * 4 + u;
      if (i >= V) break;
      const float z = lg[i] * inv_t;
      if (!(z == z)) continue;  // NaN never wins
      if (z > m) {
        l = l * expf(m - z) + 1.f;
        m = z;
      } else {
        l += expf(z - m);
      }
      float score = z;
      if (!greedy) score = z + gumbel_of(rr[u]);
      Best c = {score, i};
      best = better(best, c);
    }
  }
  // block reductions
  best = warp_best(best);
  float wm = warp_max(m);
  float wl = warp_sum(l * expf(m - wm));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_v[warp] = best.v;
    s_i[warp] = best.i;
    s_m[warp] = wm;
    s_l[warp] = wl;
  }
  __syncthreads();
  if (warp == 0) {
    Best b = {-FLT_MAX, 0x7fffffff};
    float mm = -FLT_MAX, ll = 0.f;
    if (lane < SAMPLE_THREADS / 32) {
      b.v = s_v[lane];
      b.i = s_i[lane];
      mm = s_m[lane];
      ll = s_l[lane];
    }
    b = warp_best(b);
    const float gm = warp_max(mm);
    const float gl = warp_sum(ll * expf(mm - gm));
    if (lane == 0) {
      s_choice = b.i < V ? b.i : 0;
      s_lse = gm + logf(gl);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int c = s_choice;
    out_ids[r] = c;
    if (out_logprob) out_logprob[r] = lg[c] * inv_t - s_lse;
    if (last_token && row_slot && row_slot[r] >= 0) last_token[row_slot[r]] = c;
  }
}

// Top-k log-probabilities under softmax(logits / T): k rounds of "largest entry that comes after
// the previous pick in (value descending, index ascending) order".
__global__ void __launch_bounds__(SAMPLE_THREADS)
topk_logprobs_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                     int* __restrict__ out_idx, float* __restrict__ out_lp, int V, int k) {
  __shared__ float s_v[SAMPLE_THREADS / 32];
  __shared__ int s_i[SAMPLE_THREADS / 32];
  __shared__ float s_m[SAMPLE_THREADS / 32];
  __shared__ float s_l[SAMPLE_THREADS / 32];
  __shared__ Best s_prev;
  __shared__ float s_lse;
  const int r = blockIdx.x;
  const float* lg = logits + (size_t)r * V;
  const float T = temperature ? temperature[r] : 0.f;
  const float inv_t = T > 0.f ? 1.f / T : 1.f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // log-sum-exp
  float m = -FLT_MAX, l = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float z = lg[i] * inv_t;
    if (!(z == z)) continue;
    if (z > m) {
      l = l * expf(m - z) + 1.f;
      m = z;
    } else {
      l += expf(z - m);
    }
  }
  float wm = warp_max(m);
  float wl = warp_sum(l * expf(m - wm));
  if (lane == 0) {
    s_m[warp] = wm;
    s_l[warp] = wl;
  }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < SAMPLE_THREADS / 32 ? s_m[lane] : -FLT_MAX;
    float ll = lane < SAMPLE_THREADS / 32 ? s_l[lane] : 0.f;
    const float gm = warp_max(mm);
    const float gl = warp_sum(ll * expf(mm - gm));
    if (lane == 0) {
      s_lse = gm + logf(gl);
      s_prev.v = FLT_MAX;
      s_prev.i = -1;
    }
  }
  __syncthreads();
  for (int round = 0; round < k; round++) {
    const Best prev = s_prev;
    Best best = {-FLT_MAX, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
      const float z = lg[i] * inv_t;
      if (!(z == z)) continue;
      const bool after = z < prev.v || (z == prev.v && i > prev.i);
      if (after) {
        Best c = {z, i};
        best = better(best, c);
      }
    }
    best = warp_best(best);
    __syncthreads();
    if (lane == 0) {
      s_v[warp] = best.v;
      s_i[warp] = best.i;
    }
    __syncthreads();
    if (warp == 0) {
      Best b = {-FLT_MAX, 0x7fffffff};
      if (lane < SAMPLE_THREADS / 32) {
        b.v = s_v[lane];
        b.i = s_i[lane];
      }
      b = warp_best(b);
      if (lane == 0) {
        const bool found = b.i < V;
        out_idx[(size_t)r * k + round] = found ? b.i : -1;
        out_lp[(size_t)r * k + round] = found ? b.v - s_lse : -INFINITY;
        s_prev = b;
      }
    }
    __syncthreads();
  }
}


// Two-stage form for large vocabularies: the vocabulary of each row is cut into `nch` chunks, one block
// each, so that a handful of rows still fills the GPU.  part[r][c] = {best score, best index (bits),
// running max, running sum}.  The second stage folds the chunks in chunk order.
constexpr int CH_THREADS = 256;

__global__ void __launch_bounds__(CH_THREADS)
sample_chunk_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                    const unsigned long long* __restrict__ stream_key, const int* __restrict__ sample_pos,
                    float4* __restrict__ part, int V, int nch, int groups_per_chunk) {
  __shared__ float s_v[CH_THREADS / 32];
  __shared__ int s_i[CH_THREADS / 32];
  __shared__ float s_m[CH_THREADS / 32];
  __shared__ float s_l[CH_THREADS / 32];
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.y, ch = blockIdx.x;
  const float* lg = logits + (size_t)r * V;
  const float T = temperature ? temperature[r] : 0.f;
  const bool greedy = !(T > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / T;
  const unsigned long long key = stream_key ? stream_key[r] : 0ull;
  const uint2 k2 = make_uint2((uint32_t)key, (uint32_t)(key >> 32));
  const uint32_t pos = sample_pos ? (uint32_t)sample_pos[r] : 0u;
  const int ngroups = (V + 3) >> 2;
  const int g_begin = ch * groups_per_chunk;
  const int g_end = min(ngroups, g_begin + groups_per_chunk);
  Best best = {-FLT_MAX, 0x7fffffff};
  float m = -FLT_MAX, l = 0.f;
  const bool vec = (((uintptr_t)lg) & 15) == 0;
  // Sixteen values a thread and pass: their loads are in flight together, and the running maximum and sum, on
  // which every value of a one-by-one update waits, move once a pass (values that are not numbers count as -inf).
  constexpr int PASS = 4;
  for (int g0 = g_begin + threadIdx.x; g0 < g_end; g0 += PASS * CH_THREADS) {
    float z[PASS][4];
#pragma unroll
    for (int u = 0; u < PASS; u++) {
      const int g = g0 + u * CH_THREADS;
      if (g < g_end && g * 4 + 3 < V && vec) {
        const float4 v = *reinterpret_cast<const float4*>(lg + g * 4);
        z[u][0] = v.x; z[u][1] = v.y; z[u][2] = v.z; z[u][3] = v.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; e++) z[u][e] = (g < g_end && g * 4 + e < V) ? lg[g * 4 + e] : -INFINITY;
      }
    }
    float top = -INFINITY;
#pragma unroll
    for (int u = 0; u < PASS; u++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float x = z[u][e] * inv_t;
        x = (x == x) ? x : -INFINITY;
        z[u][e] = x;
        top = fmaxf(top, x);
      }
    if (top > m) {
      l *= expf(m - top);
      m = top;
    }
    float add = 0.f;
#pragma unroll
    for (int u = 0; u < PASS; u++) {
      const int g = g0 + u * CH_THREADS;
      uint4 rnd = make_uint4(0, 0, 0, 0);
      if (!greedy && g < g_end) rnd = Philox::run(make_uint4((uint32_t)g, pos, 0u, 0u), k2);
      const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float x = z[u][e];
        add += expf(x - m);
        if (x > -INFINITY) {
          Best c = {greedy ? x : x + gumbel_of(rr[e]), g * 4 + e};
          best = better(best, c);
        }
      }
    }
    l += add;
  }
  best = warp_best(best);
  const float wm = warp_max(m);
  const float wl = warp_sum(l * expf(m - wm));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_v[warp] = best.v;
    s_i[warp] = best.i;
    s_m[warp] = wm;
    s_l[warp] = wl;
  }
  __syncthreads();
  if (warp == 0) {
    Best b = {-FLT_MAX, 0x7fffffff};
    float mm = -FLT_MAX, ll = 0.f;
    if (lane < CH_THREADS / 32) {
      b.v = s_v[lane];
      b.i = s_i[lane];
      mm = s_m[lane];
      ll = s_l[lane];
    }
    b = warp_best(b);
    const float gm = warp_max(mm);
    const float gl = warp_sum(ll * expf(mm - gm));
    if (lane == 0) part[(size_t)r * nch + ch] = make_float4(b.v, __int_as_float(b.i), gm, gl);
  }
}

__global__ void sample_finish_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                     const float4* __restrict__ part, const int* __restrict__ row_slot,
                                     int* __restrict__ out_ids, float* __restrict__ out_logprob,
                                     int* __restrict__ last_token, int V, int nch) {
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int lane = threadIdx.x;
  Best b = {-FLT_MAX, 0x7fffffff};
  float mm = -FLT_MAX, ll = 0.f;
  for (int c = lane; c < nch; c += 32) {
    const float4 p = part[(size_t)r * nch + c];
    Best o = {p.x, __float_as_int(p.y)};
    b = better(b, o);
    if (p.z > mm) {
      ll = ll * expf(mm - p.z) + p.w;
      mm = p.z;
    } else {
      ll += p.w * expf(p.z - mm);
    }
  }
  b = warp_best(b);
  const float gm = warp_max(mm);
  const float gl = warp_sum(ll * expf(mm - gm));
  if (lane == 0) {
    const int c = b.i < V ? b.i : 0;
    const float T = temperature ? temperature[r] : 0.f;
    const float inv_t = T > 0.f ? 1.f / T : 1.f;
    out_ids[r] = c;
    if (out_logprob) out_logprob[r] = logits[(size_t)r * V + c] * inv_t - (gm + logf(gl));
    if (last_token && row_slot && row_slot[r] >= 0) last_token[row_slot[r]] = c;
  }
}

}  // namespace

TKB_EXPORT int tkb_sample(const float* logits, const float* temperature, const unsigned long long* stream_key,
                          const int* sample_pos, const int* row_slot, int* out_ids, float* out_logprob,
                          int* last_token, int R, int V, void* st) {
  if (R <= 0) return 0;
  if (V <= 0) return -2;
  return launch_pdl(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, (cudaStream_t)st, logits, temperature, stream_key,
                    sample_pos, row_slot, out_ids, out_logprob, last_token, V);
}

// The same result as tkb_sample through two kernels and `part` (R * nch float4 of scratch), for rows that
// are too few to fill the GPU with one block each.  nch = tkb_sample_chunks(R, V).
TKB_EXPORT int tkb_sample_chunks(int R, int V) {
  if (R <= 0 || V < 32768) return 1;
  int nch = (6 * sm_count() + R - 1) / R;  // six blocks of 256 threads an SM
  if (nch > 64) nch = 64;
  const int ngroups = (V + 3) / 4;
  if (nch > ngroups / 256) nch = ngroups / 256;
  return nch < 1 ? 1 : nch;
}

TKB_EXPORT int tkb_sample_two_stage(const float* logits, const float* temperature, const unsigned long long* stream_key,
                                    const int* sample_pos, const int* row_slot, int* out_ids, float* out_logprob,
                                    int* last_token, void* part, int nch, int R, int V, void* st) {
  if (R <= 0) return 0;
  if (V <= 0 || nch < 1 || R > 65535) return -2;
  const int ngroups = (V + 3) / 4;
  const int gpc = (ngroups + nch - 1) / nch;
  int rc = launch_pdl(sample_chunk_kernel, dim3(nch, R), dim3(CH_THREADS), 0, (cudaStream_t)st, logits, temperature,
                      stream_key, sample_pos, (float4*)part, V, nch, gpc);
  if (rc) return rc;
  return launch_pdl(sample_finish_kernel, dim3(R), dim3(32), 0, (cudaStream_t)st, logits, temperature,
                    (const float4*)part, row_slot, out_ids, out_logprob, last_token, V, nch);
}

namespace {
__global__ void noise_of_bits_kernel(const uint32_t* __restrict__ bits, float* __restrict__ uniform,
                                     float* __restrict__ gumbel, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    uniform[i] = uniform_open(bits[i]);
    gumbel[i] = gumbel_of(bits[i]);
  }
}

}  // namespace

// The uniform number and the Gumbel value that the sampling kernels make of 32 random bits, for tests of the
// extremes (all bits set, no bit set), which a Philox draw reaches once in 2^32.
TKB_EXPORT int tkb_noise_of_bits(const uint32_t* bits, float* uniform, float* gumbel, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  noise_of_bits_kernel<<<(n + 255) / 256, 256, 0, st>>>(bits, uniform, gumbel, n);
  return launch_status();
}

TKB_EXPORT int tkb_topk_logprobs(const float* logits, const float* temperature, int* out_idx, float* out_lp, int R,
                                 int V, int k, void* st) {
  if (R <= 0 || k <= 0) return 0;
  if (V <= 0) return -2;
  topk_logprobs_kernel<<<R, SAMPLE_THREADS, 0, (cudaStream_t)st>>>(logits, temperature, out_idx, out_lp, V, k);
  return launch_status();
}
