// Causal grouped-query attention over the paged cache, for any mix of prompt portions and single
// decoded tokens, on the FP32 pipes.  It is the attention of the true 32-bit path and the
// reference-grade kernel for bfloat16 (the tensor-core kernels live in other files).
//
// Compile with -DTKB_HD=<head size> (a multiple of 16, at most 256).
//
// One warp owns one (token, query head).  A token at position p sees the keys at positions
// max(0, p - window + 1) .. p of its own request (window <= 0: all of them); the keys of the
// step's own tokens are already in the cache when this runs.  Scores, softmax and the weighted sum
// of values are float32; exp2 with log2(e)/sqrt(hd) folded into the score scale.
// Lane j of a warp scores key base + j (a dot product over the head size with the query in shared
// memory); after the warp-wide running max and sum are updated, lane d accumulates output
// elements d, d + 32, ...: the probability of key jj is broadcast by shuffle.
#include "common.cuh"
#include <float.h>

#ifndef TKB_HD
#error "compile with -DTKB_HD=<head size>"
#endif
static_assert(TKB_HD % 16 == 0 && TKB_HD >= 16 && TKB_HD <= 256, "head size must be a multiple of 16 up to 256");

using namespace tkb;

namespace {

constexpr int HD = TKB_HD;
constexpr int WARPS = 4;
constexpr int DPL = (HD + 31) / 32;  // output elements per lane

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ k, const float* __restrict__ q) {
  float acc = 0.f;
  const float4* k4 = reinterpret_cast<const float4*>(k);
#pragma unroll
  for (int i = 0; i < HD / 4; i++) {
    const float4 v = k4[i];
    acc = fmaf(v.x, q[4 * i + 0], acc);
    acc = fmaf(v.y, q[4 * i + 1], acc);
    acc = fmaf(v.z, q[4 * i + 2], acc);
    acc = fmaf(v.w, q[4 * i + 3], acc);
  }
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k,
                                                        const float* __restrict__ q) {
  float acc = 0.f;
  const uint4* k8 = reinterpret_cast<const uint4*>(k);
#pragma unroll
  for (int i = 0; i < HD / 8; i++) {
    const uint4 v = k8[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const float2 f = __bfloat1622float2(h[u]);
      acc = fmaf(f.x, q[8 * i + 2 * u + 0], acc);
      acc = fmaf(f.y, q[8 * i + 2 * u + 1], acc);
    }
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_paged_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                       const T* __restrict__ kcache, const T* __restrict__ vcache,
                       const int* __restrict__ token_seq, const int* __restrict__ positions,
                       const int* __restrict__ page_indptr, const int* __restrict__ page_ids,
                       const int* __restrict__ rows, int nh, int nkv, int page_size, float scale_log2, int window,
                       int num_pages, int* __restrict__ status) {
  __shared__ float qs[WARPS][HD];
  trigger_dependents();
  grid_dependency_wait();
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const int kvh = blockIdx.y;
  const int s = token_seq[t];
  if (s < 0) return;
  const int p = positions[t];
  const int group = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* table = page_ids + page_indptr[s];
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;

  for (int gq = warp; gq < group; gq += WARPS) {
    const int h = kvh * group + gq;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * HD;
    for (int d = lane; d < HD; d += 32) qs[warp][d] = to_float(qrow[d]) * scale_log2;
    __syncwarp();

    float m = -FLT_MAX, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    for (int base = lo; base <= p; base += 32) {
      const int j = base + lane;
      const bool live = j <= p;
      long long rowoff = 0;
      float sc = -FLT_MAX;
      if (live) {
        const int page = checked_page(table[j / page_size], num_pages, status);
        if (page >= 0) {  // else: an id beyond the pool (the status flag is set); the key counts for nothing
          rowoff = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * HD;
          sc = dot_row<T>(kcache + rowoff, qs[warp]);
        }
      }
      const float bm = warp_max(sc);
      const float m_new = fmaxf(m, bm);
      const float alpha = exp2f(m - m_new);
      const float pj = live ? exp2f(sc - m_new) : 0.f;
      l = l * alpha + warp_sum(pj);
      m = m_new;
#pragma unroll
      for (int i = 0; i < DPL; i++) acc[i] *= alpha;
      const int nlive = (p - base + 1) < 32 ? (p - base + 1) : 32;
      for (int jj = 0; jj < nlive; jj++) {
        const float pv = __shfl_sync(0xffffffffu, pj, jj);
        const long long ro = __shfl_sync(0xffffffffu, rowoff, jj);
        const T* vrow = vcache + ro;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
          const int d = lane + 32 * i;
          if (d < HD) acc[i] = fmaf(pv, to_float(vrow[d]), acc[i]);
        }
      }
    }
    const float inv_l = 1.f / l;
    T* orow = out + (size_t)blockIdx.x * out_stride + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      if (d < HD) orow[d] = from_float<T>(acc[i] * inv_l);
    }
    __syncwarp();
  }
}

template <typename T>
int attn_launch(const void* q, int q_stride, void* out, int out_stride, const void* kcache, const void* vcache,
                const int* token_seq, const int* positions, const int* page_indptr, const int* page_ids,
                const int* rows, int n_rows, int nh, int nkv, int page_size, float scale, int window, int num_pages,
                int* status, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0) return -2;
  if (nkv > 65535) return -3;
  dim3 grid(n_rows, nkv);
  const float scale_log2 = scale * 1.4426950408889634f;
  return launch_pdl(attn_paged_simt_kernel<T>, grid, dim3(WARPS * 32), 0, st, (const T*)q, q_stride, (T*)out, out_stride,
                    (const T*)kcache, (const T*)vcache, token_seq, positions, page_indptr, page_ids, rows, nh, nkv,
                    page_size, scale_log2, window, num_pages, status);
}

}  // namespace

// q: [tokens, q_stride] with head h at column h*HD; out: [n_rows, out_stride].  `rows` (nullable)
// names the tokens whose output is wanted; row r of `out` belongs to token rows[r].  num_pages, status: a page id
// beyond the pool sets the status flag and its keys count for nothing (num_pages <= 0: not checked).
TKB_EXPORT int tkb_attn_paged_simt_f32(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                       const void* vcache, const int* token_seq, const int* positions,
                                       const int* page_indptr, const int* page_ids, const int* rows, int n_rows,
                                       int nh, int nkv, int page_size, float scale, int window, int num_pages,
                                       int* status, void* st) {
  return attn_launch<float>(q, q_stride, out, out_stride, kcache, vcache, token_seq, positions, page_indptr, page_ids,
                            rows, n_rows, nh, nkv, page_size, scale, window, num_pages, status, (cudaStream_t)st);
}
TKB_EXPORT int tkb_attn_paged_simt_bf16(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                        const void* vcache, const int* token_seq, const int* positions,
                                        const int* page_indptr, const int* page_ids, const int* rows, int n_rows,
                                        int nh, int nkv, int page_size, float scale, int window, int num_pages,
                                        int* status, void* st) {
  return attn_launch<__nv_bfloat16>(q, q_stride, out, out_stride, kcache, vcache, token_seq, positions, page_indptr,
                                    page_ids, rows, n_rows, nh, nkv, page_size, scale, window, num_pages, status,
                                    (cudaStream_t)st);
}
TKB_EXPORT int tkb_attn_head_dim() { return HD; }
