// Memory-bound kernels of the forward pass: embedding gather, fused residual add + RMS norm,
// rotary encoding fused with the write of keys and values into cache pages, SiLU-gated product,
// row gather.  Each is written for both activation types (float and bfloat16); arithmetic is float.
#include "common.cuh"

using namespace tkb;

// ------------------------------------------------------------------------------------------------
// Embedding gather into the float32 residual stream.
// A token id < 0 means "the token this request sampled last": it is read from last_token[slot].
// Rows whose token_seq is < 0 are padding and become zero.
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                    const int* __restrict__ last_token, float* __restrict__ x, int H, int V,
                                    int* __restrict__ status) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  int id = ids[t];
  bool valid = s >= 0;
  if (valid && id < 0) id = last_token[seq_slot[s]];
  if (valid && (id < 0 || id >= V)) {
    if (threadIdx.x == 0) atomicOr(status, TKB_STATUS_BAD_TOKEN_ID);
    valid = false;
  }
  float* xr = x + (size_t)t * H;
  if (!valid) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] = to_float(row[i]);
}

template <typename T>
static int embed_gather_launch(const void* table, const int* ids, const int* token_seq, const int* seq_slot,
                               const int* last_token, float* x, int n_tokens, int H, int V, int* status,
                               cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  return launch_pdl(embed_gather_kernel<T>, dim3(n_tokens), dim3(threads), 0, st, (const T*)table, ids, token_seq, seq_slot,
                    last_token, x, H, V, status);
}
TKB_EXPORT int tkb_embed_gather_f32(const void* table, const int* ids, const int* token_seq, const int* seq_slot,
                                    const int* last_token, float* x, int n_tokens, int H, int V, int* status,
                                    void* st) {
  return embed_gather_launch<float>(table, ids, token_seq, seq_slot, last_token, x, n_tokens, H, V, status,
                                    (cudaStream_t)st);
}
TKB_EXPORT int tkb_embed_gather_bf16(const void* table, const int* ids, const int* token_seq, const int* seq_slot,
                                     const int* last_token, float* x, int n_tokens, int H, int V, int* status,
                                     void* st) {
  return embed_gather_launch<__nv_bfloat16>(table, ids, token_seq, seq_slot, last_token, x, n_tokens, H, V, status,
                                            (cudaStream_t)st);
}

// ------------------------------------------------------------------------------------------------
// x += delta (if delta is given; x is float32 and is written back), then
// out = (x * rsqrt(mean(x^2) + eps)) * w, rounded once to the activation type.
// One block per row.
// 4 consecutive elements of the activation type
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// MODE: 0 no update, 1 update in the activation type, 2 update as float32 slices.  One instantiation a mode,
// and only two steps' worth of values kept in registers: with many rows (a prompt) what matters is how many
// rows an SM holds at once, and that is set by the registers a thread takes.
template <typename T, int MODE, int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT <= 256 ? 6 : 2)
add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ partials,
                   int n_partials, long long partial_stride, const float* __restrict__ w, T* __restrict__ out,
                   float eps, int H) {
  trigger_dependents();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * H;
  float* xr = x + base;
  T* orow = out + base;
  float ss = 0.f;
  if ((H & 3) == 0) {
    // four elements a thread and step; the first two steps' sums stay in registers for the second pass
    constexpr int KEEP = 2;
    const int n4 = H >> 2;
    float4 kept[KEEP], gain[KEEP];
    // the norm's weight is written by no kernel: it is fetched while the kernel ahead still runs
#pragma unroll
    for (int k = 0; k < KEEP; k++) {
      const int i4 = threadIdx.x + k * blockDim.x;
      if (i4 < n4) gain[k] = load4(w + 4 * i4);
    }
    grid_dependency_wait();
    // x + update of four elements at 4 * i4, stored back
    auto updated = [&](int i4) {
      float4 v = load4(xr + 4 * i4);
      if (MODE == 2) {
        // float32 slices of a split matrix product: four loads in flight together, added in slice order
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = partials + base + 4 * i4;
        for (int p0 = 0; p0 < n_partials; p0 += 4) {
          float4 q[4];
#pragma unroll
          for (int j = 0; j < 4; j++)
            q[j] = p0 + j < n_partials ? load4(src + (size_t)(p0 + j) * partial_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            if (p0 + j < n_partials) {
              d.x += q[j].x; d.y += q[j].y; d.z += q[j].z; d.w += q[j].w;
            }
          }
        }
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        store4(xr + 4 * i4, v);
      } else if (MODE == 1) {
        const float4 d = load4(delta + base + 4 * i4);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        store4(xr + 4 * i4, v);
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      return v;
    };
#pragma unroll
    for (int k = 0; k < KEEP; k++) {
      const int i4 = threadIdx.x + k * blockDim.x;
      if (i4 < n4) kept[k] = updated(i4);
    }
    for (int i4 = threadIdx.x + KEEP * blockDim.x; i4 < n4; i4 += blockDim.x) updated(i4);
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)H + eps);
#pragma unroll
    for (int k = 0; k < KEEP; k++) {
      const int i4 = threadIdx.x + k * blockDim.x;
      if (i4 < n4) {
        const float4 v = kept[k], g = gain[k];
        store4(orow + 4 * i4, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z, v.w * rstd * g.w));
      }
    }
    for (int i4 = threadIdx.x + KEEP * blockDim.x; i4 < n4; i4 += blockDim.x) {
      const float4 v = load4(xr + 4 * i4), g = load4(w + 4 * i4);
      store4(orow + 4 * i4, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z, v.w * rstd * g.w));
    }
    return;
  }
  grid_dependency_wait();
  if (MODE == 2) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float d = 0.f;
      for (int p = 0; p < n_partials; p++) d += partials[(size_t)p * partial_stride + base + i];
      float v = xr[i] + d;
      xr[i] = v;
      ss += v * v;
    }
  } else if (MODE == 1) {
    const T* dr = delta + base;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i] + to_float(dr[i]);
      xr[i] = v;
      ss += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_float<T>(xr[i] * rstd * w[i]);
}

// The same for few rows whose update arrives as slices: the row of x and the rows of the slices come into shared
// memory by bulk copies (the copy engine keeps all of them in flight at once; 512 threads with nine 16-byte loads
// each do not: the load phase of 8 slices of 2,048 took 2.5 us that way, twice that of 4 slices).  One thread
// issues the copies and everybody waits on their mbarrier, with a limit; if the limit runs out the block reads
// from global memory instead, so the result does not depend on the wait.
__device__ __forceinline__ uint32_t ew_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <typename T>
__global__ void add_rmsnorm_bulk_kernel(float* __restrict__ x, const float* __restrict__ partials, int n_partials,
                                        long long partial_stride, const float* __restrict__ w, T* __restrict__ out,
                                        float eps, int H) {
  extern __shared__ __align__(128) unsigned char ew_smem[];
  float* rows = reinterpret_cast<float*>(ew_smem);  // [1 + n_partials][H]
  __shared__ __align__(8) unsigned long long bar;
  __shared__ float scratch[33];
  trigger_dependents();
  const size_t base = (size_t)blockIdx.x * H;
  float* xr = x + base;
  T* orow = out + base;
  constexpr int KEEP = 4;
  const int n4 = H >> 2;
  float4 kept[KEEP], gain[KEEP];
#pragma unroll
  for (int k = 0; k < KEEP; k++) {
    const int i4 = threadIdx.x + k * blockDim.x;
    if (i4 < n4) gain[k] = load4(w + 4 * i4);
  }
  const uint32_t bar_a = ew_smem_u32(&bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dependency_wait();
  const uint32_t row_bytes = (uint32_t)H * 4u;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(row_bytes * (uint32_t)(n_partials + 1)) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ew_smem_u32(rows)), "l"(xr), "r"(row_bytes), "r"(bar_a) : "memory");
    for (int p = 0; p < n_partials; p++)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(ew_smem_u32(rows + (size_t)(p + 1) * H)), "l"(partials + (size_t)p * partial_stride + base),
                     "r"(row_bytes), "r"(bar_a) : "memory");
  }
  bool arrived = false;
  for (uint32_t i = 0; i < (1u << 20) && !arrived; i++) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar_a) : "memory");
    arrived = done != 0;
  }
  float ss = 0.f;
  auto updated = [&](int i4) {
    float4 v, d = make_float4(0.f, 0.f, 0.f, 0.f);
    if (arrived) {
      v = load4(rows + 4 * i4);
      for (int p = 0; p < n_partials; p++) {
        const float4 q = load4(rows + (size_t)(p + 1) * H + 4 * i4);
        d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
      }
    } else {
      v = load4(xr + 4 * i4);
      for (int p = 0; p < n_partials; p++) {
        const float4 q = load4(partials + (size_t)p * partial_stride + base + 4 * i4);
        d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
      }
    }
    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    store4(xr + 4 * i4, v);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    return v;
  };
#pragma unroll
  for (int k = 0; k < KEEP; k++) {
    const int i4 = threadIdx.x + k * blockDim.x;
    if (i4 < n4) kept[k] = updated(i4);
  }
  for (int i4 = threadIdx.x + KEEP * blockDim.x; i4 < n4; i4 += blockDim.x) updated(i4);
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
#pragma unroll
  for (int k = 0; k < KEEP; k++) {
    const int i4 = threadIdx.x + k * blockDim.x;
    if (i4 < n4) {
      const float4 v = kept[k], g = gain[k];
      store4(orow + 4 * i4, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z, v.w * rstd * g.w));
    }
  }
  for (int i4 = threadIdx.x + KEEP * blockDim.x; i4 < n4; i4 += blockDim.x) {
    const float4 v = load4(xr + 4 * i4), g = load4(w + 4 * i4);
    store4(orow + 4 * i4, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z, v.w * rstd * g.w));
  }
}

template <typename T>
static int add_rmsnorm_launch(float* x, const void* delta, const float* partials, int n_partials,
                              long long partial_stride, const float* w, void* out, float eps, int rows, int H,
                              cudaStream_t st) {
  if (rows <= 0) return 0;
  // few rows with slices: bulk copies into shared memory (rows of 16-byte multiples, everything 16-byte aligned)
  const size_t bulk_bytes = (size_t)(n_partials + 1) * H * 4;
  if (partials != nullptr && rows <= 64 && (H & 3) == 0 && bulk_bytes <= 200 * 1024 && ((uintptr_t)x & 15) == 0 &&
      ((uintptr_t)partials & 15) == 0 && (partial_stride & 3) == 0) {
    static bool attr_done[2] = {false, false};
    constexpr int which = sizeof(T) == 4 ? 0 : 1;
    if (!attr_done[which]) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_bulk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return (int)e;
      attr_done[which] = true;
    }
    return launch_pdl(add_rmsnorm_bulk_kernel<T>, dim3(rows), dim3(H >= 2048 ? 512 : 256), bulk_bytes, st, x, partials,
                      n_partials, partial_stride, w, (T*)out, eps, H);
  }
  // few rows: many threads a row, they hide the latency; many rows: several rows an SM in flight do
  int threads = H >= 8192 || (H >= 2048 && rows < 592) ? 512 : (H >= 512 ? 256 : 128);
#define TKB_NORM(MODE, MAXT)                                                                                        \
  return launch_pdl(add_rmsnorm_kernel<T, MODE, MAXT>, dim3(rows), dim3(threads), 0, st, x, (const T*)delta, partials, \
                    n_partials, partial_stride, w, (T*)out, eps, H)
  const int mode = partials != nullptr ? 2 : (delta != nullptr ? 1 : 0);
  if (threads <= 256) {  // up to 256 threads a row: six rows an SM (40 registers a thread)
    if (mode == 2) TKB_NORM(2, 256);
    if (mode == 1) TKB_NORM(1, 256);
    TKB_NORM(0, 256);
  }
  if (mode == 2) TKB_NORM(2, 512);
  if (mode == 1) TKB_NORM(1, 512);
  TKB_NORM(0, 512);
#undef TKB_NORM
}
// delta: update in the activation type [rows, H], or null.  partials: the update as float32 slices
// [n_partials][rows, H] spaced partial_stride floats apart, or null.  At most one of the two.
TKB_EXPORT int tkb_add_rmsnorm_f32(float* x, const void* delta, const float* partials, int n_partials,
                                   long long partial_stride, const float* w, void* out, float eps, int rows, int H,
                                   void* st) {
  return add_rmsnorm_launch<float>(x, delta, partials, n_partials, partial_stride, w, out, eps, rows, H,
                                   (cudaStream_t)st);
}
TKB_EXPORT int tkb_add_rmsnorm_bf16(float* x, const void* delta, const float* partials, int n_partials,
                                    long long partial_stride, const float* w, void* out, float eps, int rows, int H,
                                    void* st) {
  return add_rmsnorm_launch<__nv_bfloat16>(x, delta, partials, n_partials, partial_stride, w, out, eps, rows, H,
                                           (cudaStream_t)st);
}

// ------------------------------------------------------------------------------------------------
// From a step's q|k|v rows to rotated q and to the cache: rotary position encoding of q and k (half-split
// pairing: element j pairs with j + rot/2), the rotated q written out (in place or to a tensor of its own), the
// rotated k and v written into the cache pages of the token's request.  q|k|v row layout: [nh*hd | nkv*hd |
// nkv*hd], as rows of the activation type or as float32 slices of a K-split product, [n_partials][tokens, C],
// which are added in order and rounded to the activation type first.  Cache layout per layer: [page, kv head,
// slot in page, hd].  The angle is the float32 product position * inv_freq[j]; cos and sin use the accurate
// float routines (full range reduction), once per token and pair, shared by heads.  rot == 0: no position
// encoding.  Tokens with token_seq < 0 are padding and are skipped.
//
// Between "q|k|v ready" and "rotate" sits an element-wise stage that a mixer may ask for:
//   bias       float32 [C] or null: added to the row (and the sum rounded to the activation type);
//   qk_norm_w  float32 [2][hd] or null: every q head and every k head is RMS-normalised over its hd elements
//              (statistics in float32, eps = norm_eps) and scaled by the first (q) or second (k) weight row.
//
// A block takes tokens t = blockIdx.x, blockIdx.x + gridDim.x, ...; the token's row is staged in shared memory
// as float32 with 16-byte loads, everything after reads it from there and leaves in 16-byte stores.  What the
// host wrote for the step (positions, request rows, block tables) is there before any kernel of the step runs:
// the first token's page and angles are worked out before the wait for the kernel that makes q|k|v.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// element `d` of a head after the rotation; `x` points at the head's first element in shared memory
__device__ __forceinline__ float rotated(const float* x, const float* cs, int d, int half, int rot) {
  if (d < half) return x[d] * cs[d] - x[d + half] * cs[half + d];
  if (d < rot) return x[d] * cs[d - half] + x[d - half] * cs[d];
  return x[d];
}
// elements d .. d+3 of a head after the rotation (d and rot/2 multiples of 4: the four lie on one side of the
// rotation), read from shared memory as 16-byte vectors: a thread that read them one by one would meet the
// other threads of its warp in the same banks
__device__ __forceinline__ void rotated4(float* out, const float* x, const float* cs, int d, int half, int rot) {
  const float4 a = *reinterpret_cast<const float4*>(x + d);
  if (d >= rot) {
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    return;
  }
  const bool low = d < half;
  const int j = low ? d : d - half;
  const float4 b = *reinterpret_cast<const float4*>(x + (low ? d + half : j));
  const float4 c = *reinterpret_cast<const float4*>(cs + j), sn = *reinterpret_cast<const float4*>(cs + half + j);
  if (low) {
    out[0] = a.x * c.x - b.x * sn.x; out[1] = a.y * c.y - b.y * sn.y;
    out[2] = a.z * c.z - b.z * sn.z; out[3] = a.w * c.w - b.w * sn.w;
  } else {
    out[0] = a.x * c.x + b.x * sn.x; out[1] = a.y * c.y + b.y * sn.y;
    out[2] = a.z * c.z + b.z * sn.z; out[3] = a.w * c.w + b.w * sn.w;
  }
}
// N (4 or 8) elements from d0 on
template <int N>
__device__ __forceinline__ void rotated_n(float (&v)[N], const float* x, const float* cs, int d0, int half, int rot) {
  if ((half & 3) == 0) {
#pragma unroll
    for (int e = 0; e < N; e += 4) rotated4(v + e, x, cs, d0 + e, half, rot);
  } else {
#pragma unroll
    for (int e = 0; e < N; e++) v[e] = rotated(x, cs, d0 + e, half, rot);
  }
}

constexpr int ROPE_THREADS = 128;

template <typename T, bool PARTS>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_write_kernel(const T* __restrict__ rows, const float* __restrict__ partials, int n_partials,
                     long long partial_stride, T* __restrict__ q_out, long long q_out_stride,
                     const int* __restrict__ positions, const int* __restrict__ token_seq,
                     const int* __restrict__ page_indptr, const int* __restrict__ page_ids,
                     const float* __restrict__ inv_freq, T* __restrict__ kcache, T* __restrict__ vcache, int n_tokens,
                     int nh, int nkv, int hd, int rot, int page_size, int num_pages, int write_cache,
                     int* __restrict__ status, const float* __restrict__ bias, const float* __restrict__ qk_norm_w,
                     float norm_eps) {
  trigger_dependents();
  extern __shared__ __align__(16) float sm[];  // row[C], cos[rot/2], sin[rot/2]
  constexpr int N = Vec16<T>::N;
  const int C = (nh + 2 * nkv) * hd;
  float* row = sm;
  float* cs = sm + C;
  const int half = rot >> 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  bool waited = false;
  // A token's request row, position and page: three loads that depend on one another.  Those of the block's next
  // token are sent for before the current token is worked on, so that only the first token waits for them.
  auto lookup = [&](int t, int& s, int& pos, int& page) {
    s = -1;
    pos = page = 0;
    if (t < n_tokens) {
      s = token_seq[t];
      if (s >= 0) {
        pos = positions[t];
        page = write_cache ? page_ids[page_indptr[s] + pos / page_size] : 0;
      }
    }
  };
  int s, pos, page;
  lookup(blockIdx.x, s, pos, page);
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    const int s_now = s, pos_now = pos, page_now = page;
    lookup(t + gridDim.x, s, pos, page);
    if (s_now < 0) continue;  // padding (the same for every thread of the block)
    const int pos = pos_now, page = page_now;
    for (int j = tid; j < half; j += blockDim.x) {
      float sn, c;
      sincosf((float)pos * inv_freq[j], &sn, &c);
      cs[j] = c;
      cs[half + j] = sn;
    }
    if (!waited) {
      grid_dependency_wait();
      waited = true;
    }
    // the row, as float32 values that the activation type can hold
    if (PARTS) {
      for (int i = tid * 4; i < C; i += blockDim.x * 4) {
        const float* src = partials + (size_t)t * C + i;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < n_partials; p++) {
          const float4 e = *reinterpret_cast<const float4*>(src + (size_t)p * partial_stride);
          v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
        }
        if (bias != nullptr) {
          const float4 b = *reinterpret_cast<const float4*>(bias + i);
          v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        *reinterpret_cast<float4*>(row + i) = make_float4(to_float(from_float<T>(v.x)), to_float(from_float<T>(v.y)),
                                                          to_float(from_float<T>(v.z)), to_float(from_float<T>(v.w)));
      }
    } else {
      const T* src = rows + (size_t)t * C;
      for (int i = tid * N; i < C; i += blockDim.x * N) {
        float v[N];
        Vec16<T>::load(src + i, v);
        if (bias != nullptr) {
#pragma unroll
          for (int e = 0; e < N; e++) v[e] = to_float(from_float<T>(v[e] + bias[i + e]));
        }
#pragma unroll
        for (int e = 0; e < N; e += 4) *reinterpret_cast<float4*>(row + i + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
      }
    }
    __syncthreads();
    if (qk_norm_w != nullptr) {
      // RMS norm of every q head and every k head over its hd elements; one warp a head
      for (int h = warp; h < nh + nkv; h += nwarps) {
        float* x = row + (size_t)h * hd;
        const float* w = qk_norm_w + (h < nh ? 0 : hd);
        float ss = 0.f;
        for (int d = lane; d < hd; d += 32) ss += x[d] * x[d];
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / (float)hd + norm_eps);
        for (int d = lane; d < hd; d += 32) x[d] = to_float(from_float<T>(x[d] * scale * w[d]));
      }
      __syncthreads();
    }
    // q: rotate and write out
    T* qo = q_out + (size_t)t * q_out_stride;
    for (int i = tid * N; i < nh * hd; i += blockDim.x * N) {
      const int h = i / hd, d0 = i - h * hd;
      float v[N];
      rotated_n<N>(v, row + h * hd, cs, d0, half, rot);
      Vec16<T>::store(qo + i, v);
    }
    if (write_cache) {  // a layer call that reads another call's cache writes none of its own
      if (page < 0 || page >= num_pages) {
        if (tid == 0) atomicOr(status, TKB_STATUS_BAD_PAGE);
      } else {
        const int slot = pos % page_size;
        const float* krow = row + nh * hd;
        const float* vrow = krow + nkv * hd;
        for (int i = tid * N; i < nkv * hd; i += blockDim.x * N) {
          const int h = i / hd, d0 = i - h * hd;
          const size_t dst = (((size_t)page * nkv + h) * page_size + slot) * hd + d0;
          float kv[N], vv[N];
          rotated_n<N>(kv, krow + h * hd, cs, d0, half, rot);
#pragma unroll
          for (int e = 0; e < N; e += 4) {
            const float4 x = *reinterpret_cast<const float4*>(vrow + i + e);
            vv[e] = x.x; vv[e + 1] = x.y; vv[e + 2] = x.z; vv[e + 3] = x.w;
          }
          Vec16<T>::store(kcache + dst, kv);
          Vec16<T>::store(vcache + dst, vv);
        }
      }
    }
    __syncthreads();  // the row and the angles are reused by the block's next token
  }
}

// The plain case (rows of the activation type, no element-wise stage): one block a token, every thread rotates
// the element pairs it loads and stores them straight back, nothing passes through shared memory but the angles.
// Measured at 2,048 tokens of 32 + 8 heads of 64 with the rows in the L2 cache: 8 us against 19 us staged.
template <typename T>
__global__ void rope_kv_write_direct_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ page_indptr,
                                     const int* __restrict__ page_ids, const float* __restrict__ inv_freq,
                                     T* __restrict__ kcache, T* __restrict__ vcache, int nh, int nkv, int hd, int rot,
                                     int page_size, int num_pages, int write_cache, int* __restrict__ status) {
  trigger_dependents();
  // What the host wrote for the step (positions, request rows, block tables) is there before any kernel of the
  // step runs: the token's page and its angles are worked out before the wait for the kernel that makes q|k|v.
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int pos = positions[t];
  const int page = write_cache ? page_ids[page_indptr[s] + pos / page_size] : 0;  // on its way during the sin/cos
  const int half = rot >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float ang = (float)pos * inv_freq[j];
    float sn, c;
    sincosf(ang, &sn, &c);
    cs[j] = c;
    cs[half + j] = sn;
  }
  __syncthreads();
  grid_dependency_wait();

  T* row = qkv + (size_t)t * (size_t)(nh + 2 * nkv) * hd;
  const bool vec = (half & 3) == 0 && (hd & 3) == 0;  // four elements a thread and step
  // q heads: rotate in place.
  if (vec) {
    const int h4 = half >> 2;
    for (int idx = threadIdx.x; idx < nh * h4; idx += blockDim.x) {
      const int h = idx / h4, j = (idx - h * h4) * 4;
      T* p = row + h * hd;
      const float4 x1 = load4(p + j), x2 = load4(p + j + half);
      const float4 c = *reinterpret_cast<const float4*>(cs + j), sn = *reinterpret_cast<const float4*>(cs + half + j);
      store4(p + j, make_float4(x1.x * c.x - x2.x * sn.x, x1.y * c.y - x2.y * sn.y, x1.z * c.z - x2.z * sn.z,
                                x1.w * c.w - x2.w * sn.w));
      store4(p + j + half, make_float4(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y, x2.z * c.z + x1.z * sn.z,
                                       x2.w * c.w + x1.w * sn.w));
    }
  } else {
    for (int idx = threadIdx.x; idx < nh * half; idx += blockDim.x) {
      const int h = idx / half, j = idx - h * half;
      T* p = row + h * hd;
      const float x1 = to_float(p[j]), x2 = to_float(p[j + half]);
      const float c = cs[j], sn = cs[half + j];
      p[j] = from_float<T>(x1 * c - x2 * sn);
      p[j + half] = from_float<T>(x2 * c + x1 * sn);
    }
  }
  if (!write_cache) return;  // a layer call that reads another call's cache writes none of its own
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, TKB_STATUS_BAD_PAGE);
    return;
  }
  const int slot = pos % page_size;
  const T* krow = row + nh * hd;
  const T* vrow = krow + nkv * hd;
  if (vec) {
    const int d4n = hd >> 2;
    for (int idx = threadIdx.x; idx < nkv * d4n; idx += blockDim.x) {
      const int h = idx / d4n, d = (idx - h * d4n) * 4;
      const size_t dst = (((size_t)page * nkv + h) * page_size + slot) * hd + d;
      const T* kh = krow + h * hd;
      float4 kv = load4(kh + d);
      if (d < half) {
        const float4 y = load4(kh + d + half);
        const float4 c = *reinterpret_cast<const float4*>(cs + d), sn = *reinterpret_cast<const float4*>(cs + half + d);
        kv = make_float4(kv.x * c.x - y.x * sn.x, kv.y * c.y - y.y * sn.y, kv.z * c.z - y.z * sn.z, kv.w * c.w - y.w * sn.w);
      } else if (d < rot) {
        const int j = d - half;
        const float4 y = load4(kh + j);
        const float4 c = *reinterpret_cast<const float4*>(cs + j), sn = *reinterpret_cast<const float4*>(cs + half + j);
        kv = make_float4(kv.x * c.x + y.x * sn.x, kv.y * c.y + y.y * sn.y, kv.z * c.z + y.z * sn.z, kv.w * c.w + y.w * sn.w);
      }
      store4(kcache + dst, kv);
      store4(vcache + dst, load4(vrow + h * hd + d));
    }
    return;
  }
  for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
    const int h = idx / hd, d = idx - h * hd;
    const size_t dst = (((size_t)page * nkv + h) * page_size + slot) * hd + d;
    float kv;
    if (d < half) {
      kv = to_float(krow[idx]) * cs[d] - to_float(krow[idx + half]) * cs[half + d];
    } else if (d < rot) {
      const int j = d - half;
      kv = to_float(krow[idx]) * cs[j] + to_float(krow[idx - half]) * cs[half + j];
    } else {
      kv = to_float(krow[idx]);
    }
    kcache[dst] = from_float<T>(kv);
    vcache[dst] = vrow[idx];
  }
}

template <typename T, bool PARTS>
static int rope_kv_write_launch(const void* rows, const float* partials, int n_partials, long long partial_stride,
                                void* q_out, long long q_out_stride, const int* positions, const int* token_seq,
                                const int* page_indptr, const int* page_ids, const float* inv_freq, void* kcache,
                                void* vcache, int n_tokens, int nh, int nkv, int hd, int rot, int page_size,
                                int num_pages, int write_cache, int* status, const float* bias,
                                const float* qk_norm_w, float norm_eps, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1) || (hd & 15) || nh <= 0 || nkv <= 0 || (PARTS && n_partials < 1)) return -2;
  const size_t smem = ((size_t)(nh + 2 * nkv) * hd + (rot > 0 ? rot : 2)) * sizeof(float);
  if (smem > 160 * 1024) return -2;  // a row wider than an SM's shared memory holds
  if (!PARTS && bias == nullptr && qk_norm_w == nullptr && (const void*)rows == (const void*)q_out) {
    int work = nh * (rot / 2) > nkv * hd ? nh * (rot / 2) : nkv * hd;
    int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
    return launch_pdl(rope_kv_write_direct_kernel<T>, dim3(n_tokens), dim3(threads), (size_t)(rot > 0 ? rot : 2) * sizeof(float),
                      st, (T*)q_out, positions, token_seq, page_indptr, page_ids, inv_freq, (T*)kcache, (T*)vcache, nh, nkv,
                      hd, rot, page_size, num_pages, write_cache, status);
  }
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(rope_kv_write_kernel<T, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         160 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  // as many blocks as the GPU holds at once; each walks over its share of the tokens
  static int per_sm_cached = 0;
  static size_t per_sm_smem = 0;
  if (per_sm_cached == 0 || per_sm_smem != smem) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, rope_kv_write_kernel<T, PARTS>, ROPE_THREADS, smem) !=
            cudaSuccess || n < 1)
      n = 1;
    per_sm_cached = n;
    per_sm_smem = smem;
  }
  int blocks = sm_count() * per_sm_cached;
  if (blocks > n_tokens) blocks = n_tokens;
  return launch_pdl(rope_kv_write_kernel<T, PARTS>, dim3(blocks), dim3(ROPE_THREADS), smem, st, (const T*)rows, partials,
                    n_partials, partial_stride, (T*)q_out, q_out_stride, positions, token_seq, page_indptr, page_ids,
                    inv_freq, (T*)kcache, (T*)vcache, n_tokens, nh, nkv, hd, rot, page_size, num_pages, write_cache,
                    status, bias, qk_norm_w, norm_eps);
}

// qkv: rows [n_tokens, C] of float32 / bfloat16; q is rotated in place.  bias, qk_norm_w: see above (null: none).
TKB_EXPORT int tkb_rope_kv_write_f32(void* qkv, const int* positions, const int* token_seq, const int* page_indptr,
                                     const int* page_ids, const float* inv_freq, void* kcache, void* vcache,
                                     int n_tokens, int nh, int nkv, int hd, int rot, int page_size, int num_pages,
                                     int write_cache, int* status, const float* bias, const float* qk_norm_w,
                                     float norm_eps, void* st) {
  return rope_kv_write_launch<float, false>(qkv, nullptr, 0, 0, qkv, (long long)(nh + 2 * nkv) * hd, positions,
                                            token_seq, page_indptr, page_ids, inv_freq, kcache, vcache, n_tokens, nh,
                                            nkv, hd, rot, page_size, num_pages, write_cache, status, bias, qk_norm_w,
                                            norm_eps, (cudaStream_t)st);
}
TKB_EXPORT int tkb_rope_kv_write_bf16(void* qkv, const int* positions, const int* token_seq, const int* page_indptr,
                                      const int* page_ids, const float* inv_freq, void* kcache, void* vcache,
                                      int n_tokens, int nh, int nkv, int hd, int rot, int page_size, int num_pages,
                                      int write_cache, int* status, const float* bias, const float* qk_norm_w,
                                      float norm_eps, void* st) {
  return rope_kv_write_launch<__nv_bfloat16, false>(qkv, nullptr, 0, 0, qkv, (long long)(nh + 2 * nkv) * hd, positions,
                                                    token_seq, page_indptr, page_ids, inv_freq, kcache, vcache,
                                                    n_tokens, nh, nkv, hd, rot, page_size, num_pages, write_cache,
                                                    status, bias, qk_norm_w, norm_eps, (cudaStream_t)st);
}

// The same for q|k|v that arrive as float32 slices of a split matrix product, [n_partials][tokens, C]; the rotated
// q goes to q_out [tokens, nh*hd] in bfloat16.
TKB_EXPORT int tkb_rope_kv_write_partials_bf16(const float* partials, int n_partials, long long partial_stride,
                                               void* q_out, const int* positions, const int* token_seq,
                                               const int* page_indptr, const int* page_ids, const float* inv_freq,
                                               void* kcache, void* vcache, int n_tokens, int nh, int nkv, int hd,
                                               int rot, int page_size, int num_pages, int write_cache, int* status,
                                               const float* bias, const float* qk_norm_w, float norm_eps, void* st) {
  return rope_kv_write_launch<__nv_bfloat16, true>(nullptr, partials, n_partials, partial_stride, q_out,
                                                   (long long)nh * hd, positions, token_seq, page_indptr, page_ids,
                                                   inv_freq, kcache, vcache, n_tokens, nh, nkv, hd, rot, page_size,
                                                   num_pages, write_cache, status, bias, qk_norm_w, norm_eps,
                                                   (cudaStream_t)st);
}

// ------------------------------------------------------------------------------------------------
// interleave == 0: gate columns first, then up columns.  interleave == 8: columns come in groups of 16, the
// 8 gate columns of features 8j..8j+7 followed by their 8 up columns (the layout the small-batch
// matrix product wants for its fused epilogue).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int I,
                                int interleave) {
  trigger_dependents();
  grid_dependency_wait();
  if ((I & 7) == 0) {
    // eight features a thread: two 4-element loads of gate, two of up
    const long long total8 = total >> 3;
    const int I8 = I >> 3;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
         idx += (long long)gridDim.x * blockDim.x) {
      const long long t = idx / I8;
      const int i = (int)(idx - t * I8) * 8;
      const int gc = interleave ? ((i >> 3) << 4) : i;
      const int uc = interleave ? gc + 8 : I + i;
      const T* row = gu + t * 2 * I;
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const float4 g = load4(row + gc + 4 * h), u = load4(row + uc + 4 * h);
        float4 r;
        r.x = g.x / (1.f + expf(-g.x)) * u.x;
        r.y = g.y / (1.f + expf(-g.y)) * u.y;
        r.z = g.z / (1.f + expf(-g.z)) * u.z;
        r.w = g.w / (1.f + expf(-g.w)) * u.w;
        store4(out + t * I + i + 4 * h, r);
      }
    }
    return;
  }
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const int gc = interleave ? ((i >> 3) << 4) + (i & 7) : i;
    const int uc = interleave ? gc + 8 : I + i;
    const float g = to_float(gu[t * 2 * I + gc]);
    const float u = to_float(gu[t * 2 * I + uc]);
    const float sg = g / (1.f + expf(-g));
    out[idx] = from_float<T>(sg * u);
  }
}
template <typename T>
static int silu_mul_launch(const void* gu, void* out, int rows, int I, int interleave, cudaStream_t st) {
  if (interleave != 0 && (interleave != 8 || (I & 7))) return -2;
  long long total = (long long)rows * I;
  if (total <= 0) return 0;
  long long blocks = (((I & 7) == 0 ? total / 8 : total) + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (blocks < 1) blocks = 1;
  return launch_pdl(silu_mul_kernel<T>, dim3((int)blocks), dim3(256), 0, st, (const T*)gu, (T*)out, total, I, interleave);
}
TKB_EXPORT int tkb_silu_mul_f32(const void* gu, void* out, int rows, int I, int interleave, void* st) {
  return silu_mul_launch<float>(gu, out, rows, I, interleave, (cudaStream_t)st);
}
TKB_EXPORT int tkb_silu_mul_bf16(const void* gu, void* out, int rows, int I, int interleave, void* st) {
  return silu_mul_launch<__nv_bfloat16>(gu, out, rows, I, interleave, (cudaStream_t)st);
}

// ------------------------------------------------------------------------------------------------
// dst[r, :] = src[rows[r], :], rows of row_bytes bytes (a multiple of 2).
__global__ void gather_rows_kernel(const unsigned short* __restrict__ src, unsigned short* __restrict__ dst,
                                   const int* __restrict__ rows, int row_halfwords) {
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const unsigned short* s = src + (size_t)rows[r] * row_halfwords;
  unsigned short* d = dst + (size_t)r * row_halfwords;
  if ((row_halfwords & 7) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    const uint4* s4 = (const uint4*)s;
    uint4* d4 = (uint4*)d;
    for (int i = threadIdx.x; i < (row_halfwords >> 3); i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < row_halfwords; i += blockDim.x) d[i] = s[i];
  }
}
TKB_EXPORT int tkb_gather_rows(const void* src, void* dst, const int* rows, int n_rows, int row_bytes, void* st) {
  if (n_rows <= 0) return 0;
  if (row_bytes & 1) return -2;
  return launch_pdl(gather_rows_kernel, dim3(n_rows), dim3(128), 0, (cudaStream_t)st, (const unsigned short*)src,
                    (unsigned short*)dst, rows, row_bytes / 2);
}
