// Matrix products for steps with few tokens (decode): out[M, N] = A[M, K] . W[N, K]^T in bfloat16
// with float32 accumulation, M <= 64.  Such a product is a read of W and nothing else, so the
// kernel is built to stream W at memory speed:
//   * the weight rows are the 16-row side of mma.sync m16n8k16 and the tokens the 8-column side,
//     so a token count of 1..8 wastes nothing of W's traffic;
//   * a block owns 64 output features and one slice of K; 64x64 weight tiles arrive through a
//     multi-stage cp.async pipeline; the grid is (feature tiles, K slices), sized by the host so that
//     every SM holds several blocks;
//   * K slices do not meet inside this kernel: each writes its float32 partial [slice, M, N] and the
//     consumer (the fused add + norm kernel, or the rotary/cache-write kernel) adds the slices in a
//     fixed order, so results do not depend on timing.
// Variant "gated": W holds gate and up rows interleaved in groups of 8 (8 gate rows, then the 8 up
// rows of the same features); the epilogue writes silu(gate) * up as bfloat16 [M, N/2].
#include "common.cuh"

using namespace tkb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BN = 64;               // output features per block of four warps (16 a warp)
constexpr int BK = 128;              // k per stage
constexpr int ROWB = BK * 2 + 16;    // padded row bytes (conflict-free ldmatrix)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// WARPS warps a block, 16 output features a warp.  Four warps and two blocks an SM is the general shape; a wide
// product whose feature tiles do not divide evenly over the SMs that way (gate/up of 16,384 rows: 256 blocks
// on a B200's 148 SMs, so most SMs stream twice what the others do, and an SM streams at a fixed rate) runs as one
// block of up to eight warps an SM instead.
template <int NT, int WARPS = 4> struct Tile {
  static constexpr int A_ROWS = NT * 8;                      // token rows kept in shared memory (8 rows: ldmatrix.x2)
  static constexpr int ROWS = WARPS * 16;                    // weight rows (output features) per block
  static constexpr int STAGE_B = (ROWS + A_ROWS) * ROWB;
  // deep for few tokens: the weight tiles in flight are what is prefetched; one block an SM takes what fits
#ifndef TKB_WIDE_STAGES_KIB
#define TKB_WIDE_STAGES_KIB 200
#endif
#ifndef TKB_FEW_ROWS_STAGES
#define TKB_FEW_ROWS_STAGES 5
#endif
  static constexpr int STAGES = WARPS > 4 ? (TKB_WIDE_STAGES_KIB * 1024) / STAGE_B : (NT <= 2 ? TKB_FEW_ROWS_STAGES : 4);
  static constexpr int SMEM_B = STAGES * STAGE_B;
};

template <int WARPS>
__device__ __forceinline__ void load_w(unsigned char* stage, const bf16* __restrict__ W, int ldw, int N, int n0,
                                       int k0, int k_end, int tid) {
  const uint32_t sw = smem_u32(stage);
  constexpr int CPR = BK / 8;  // 16-byte chunks per row
#pragma unroll
  for (int i = 0; i < (16 * CPR) / 32; i++) {
    const int idx = tid + i * (WARPS * 32);
    const int r = idx / CPR, c = idx % CPR;
    const int n = n0 + r, k = k0 + c * 8;
    const bool valid = n < N && k < k_end;
    cp_async16(sw + r * ROWB + c * 16, W + (valid ? (size_t)n * ldw + k : 0), valid);
  }
}

template <int NT, int WARPS>
__device__ __forceinline__ void load_a(unsigned char* stage, const bf16* __restrict__ A, int lda, int M, int k0,
                                       int k_end, int tid) {
  const uint32_t sa = smem_u32(stage) + Tile<NT, WARPS>::ROWS * ROWB;
  constexpr int CPR = BK / 8;
  constexpr int A_CHUNKS = Tile<NT, WARPS>::A_ROWS * CPR;
  constexpr int THREADS = WARPS * 32;
#pragma unroll
  for (int i = 0; i < (A_CHUNKS + THREADS - 1) / THREADS; i++) {
    const int idx = tid + i * THREADS;
    if (idx < A_CHUNKS) {
      const int r = idx / CPR, c = idx % CPR;
      const int k = k0 + c * 8;
      const bool valid = r < M && k < k_end;
      cp_async16(sa + r * ROWB + c * 16, A + (valid ? (size_t)r * lda + k : 0), valid);
    }
  }
}

template <int NT, bool GATED, int WARPS = 4>
__global__ void __launch_bounds__(WARPS * 32)
linear_smallm_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw, void* __restrict__ out,
                     int M, int N, int K, int kblocks_per_slice) {
  extern __shared__ __align__(128) unsigned char smem[];
  using T = Tile<NT, WARPS>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * T::ROWS;
  const int slice = blockIdx.y;
  const int k_begin = slice * kblocks_per_slice * BK;
  const int k_end = min(K, k_begin + kblocks_per_slice * BK);
  const int nkb = (k_end - k_begin + BK - 1) / BK;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[j][i] = 0.f;

  constexpr int STAGES = T::STAGES;
  // Weights are written by no kernel: their first tiles are fetched while the kernel before this one
  // may still be running.  The activations are read only after the wait.
  trigger_dependents();
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++)
    if (s < nkb) load_w<WARPS>(smem + s * T::STAGE_B, W, ldw, N, n0, k_begin + s * BK, k_end, tid);
  grid_dependency_wait();
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if (s < nkb) load_a<NT, WARPS>(smem + s * T::STAGE_B, A, lda, M, k_begin + s * BK, k_end, tid);
    cp_async_commit();
  }
  const int w_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int w_chunk = lane >> 4;
  // eight token rows (NT == 1) are read with ldmatrix.x2, whose addresses come from lanes 0..15; the other lanes
  // repeat them, so that every address stays inside the eight rows
  const int a_row = (lane & 7) + (NT > 1 ? (lane >> 4) * 8 : 0);
  const int a_chunk = (lane >> 3) & 1;
  for (int kb = 0; kb < nkb; kb++) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    // refill the stage that was consumed in the previous iteration
    {
      const int nxt = kb + STAGES - 1;
      if (nxt < nkb) {
        unsigned char* st = smem + (nxt % STAGES) * T::STAGE_B;
        load_w<WARPS>(st, W, ldw, N, n0, k_begin + nxt * BK, k_end, tid);
        load_a<NT, WARPS>(st, A, lda, M, k_begin + nxt * BK, k_end, tid);
      }
      cp_async_commit();
    }
    const uint32_t sw = smem_u32(smem + (kb % STAGES) * T::STAGE_B), sa = sw + T::ROWS * ROWB;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ks++) {
      uint32_t wf[4];
      ldmatrix_x4(wf[0], wf[1], wf[2], wf[3], sw + w_row * ROWB + (ks * 2 + w_chunk) * 16);
      if constexpr (NT == 1) {
        uint32_t b0, b1;
        ldmatrix_x2(b0, b1, sa + a_row * ROWB + (ks * 2 + a_chunk) * 16);
        mma_bf16(acc[0], wf, b0, b1);
      } else {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, sa + (j * 8 + a_row) * ROWB + (ks * 2 + a_chunk) * 16);
          mma_bf16(acc[j], wf, b0, b1);
          if (j + 1 < NT) mma_bf16(acc[j + 1], wf, b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();

  const int r = lane >> 2, cq = (lane & 3) * 2;
  const int f0 = n0 + warp * 16 + r;  // weight row of acc[][0..1]; acc[][2..3] belong to row f0 + 8
  if (!GATED) {
    float* o = reinterpret_cast<float*>(out) + (size_t)slice * M * N;
#pragma unroll
    for (int j = 0; j < NT; j++) {
      const int b = j * 8 + cq;
      if (b < M) {
        if (f0 < N) o[(size_t)b * N + f0] = acc[j][0];
        if (f0 + 8 < N) o[(size_t)b * N + f0 + 8] = acc[j][2];
      }
      if (b + 1 < M) {
        if (f0 < N) o[(size_t)(b + 1) * N + f0] = acc[j][1];
        if (f0 + 8 < N) o[(size_t)(b + 1) * N + f0 + 8] = acc[j][3];
      }
    }
  } else {
    // rows f0 (gate) and f0 + 8 (up) belong to feature (f0 / 16) * 8 + f0 % 16
    bf16* o = reinterpret_cast<bf16*>(out);
    const int I = N >> 1;
    const int g = ((n0 + warp * 16) >> 1) + r;
    if (f0 + 8 < N) {
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int b = j * 8 + cq;
        const float g0 = acc[j][0], g1 = acc[j][1];
        if (b < M) o[(size_t)b * I + g] = __float2bfloat16_rn(g0 / (1.f + expf(-g0)) * acc[j][2]);
        if (b + 1 < M) o[(size_t)(b + 1) * I + g] = __float2bfloat16_rn(g1 / (1.f + expf(-g1)) * acc[j][3]);
      }
    }
  }
}

template <int NT, bool GATED, int WARPS>
int launch(const void* A, int lda, const void* W, int ldw, void* out, int M, int N, int K, int slices,
           int kblocks_per_slice, cudaStream_t st) {
  using T = Tile<NT, WARPS>;
  static bool attr_done = false;
  if (!attr_done && T::SMEM_B > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(linear_smallm_kernel<NT, GATED, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_B);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid((N + T::ROWS - 1) / T::ROWS, slices);
  // A slice of fewer k-blocks than the ring has stages never touches the stages beyond them: ask only for the
  // shared memory that is used, so that blocks of the kernels before and after this one fit on the SM beside
  // these (they fetch their weights or keys while this kernel runs).
  const int stages_used = kblocks_per_slice < T::STAGES ? (kblocks_per_slice < 1 ? 1 : kblocks_per_slice) : T::STAGES;
  return launch_pdl(linear_smallm_kernel<NT, GATED, WARPS>, grid, dim3(WARPS * 32), (size_t)stages_used * T::STAGE_B, st,
                    (const bf16*)A, lda, (const bf16*)W, ldw, out, M, N, K, kblocks_per_slice);
}

template <bool GATED>
int dispatch(const void* A, int lda, const void* W, int ldw, void* out, int M, int N, int K, int slices,
             int kblocks_per_slice, cudaStream_t st) {
  if (GATED && M <= 8 && slices == 1) {
    // one block an SM when that gives every SM the same share of the weights (see Tile)
    const int sms = sm_count();
    const int per_sm = ((N + 15) / 16 + sms - 1) / sms;  // 16-row tiles an SM
    if (per_sm == 5) return launch<1, GATED, 5>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
    if (per_sm == 6) return launch<1, GATED, 6>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
    if (per_sm == 7) return launch<1, GATED, 7>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
    if (per_sm == 8) return launch<1, GATED, 8>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
  }
  if (M <= 8) return launch<1, GATED, 4>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
  if (M <= 16) return launch<2, GATED, 4>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
  if (M <= 32) return launch<4, GATED, 4>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
  return launch<8, GATED, 4>(A, lda, W, ldw, out, M, N, K, slices, kblocks_per_slice, st);
}

}  // namespace

// How the host should slice K: returns the number of slices for a grid that fills the GPU; the
// k-blocks per slice follow as ceil(ceil(K / 64) / slices).
TKB_EXPORT int tkb_linear_smallm_slices(int N, int K, int max_slices) {
  const int tiles = (N + BN - 1) / BN;
  const int kblocks = (K + BK - 1) / BK;
  const int sms = sm_count();
  int s = (2 * sms + tiles - 1) / tiles;
  if (s > max_slices) s = max_slices;
  if (s > kblocks / 2) s = kblocks / 2;  // at least two k-blocks (256 k) a slice
  if (s < 1) s = 1;
  // Fewer slices where that costs nothing: if a slice's k-blocks all fit the stages that are fetched before the
  // wait for the kernel ahead (so the whole matrix is in shared memory by then) and the grid still covers the SMs,
  // the consumer has fewer slices to add (the output product of Llama-3.2-1B: 4 slices instead of 8 took 13 us
  // off a decode step of 795 us, all of it in the norm kernel that adds them).
  const int prefetched = TKB_FEW_ROWS_STAGES - 1;
  const int s_few = (kblocks + prefetched - 1) / prefetched;
  if (s_few >= 1 && s_few < s && (long long)tiles * s_few * 100 >= 85LL * sms) s = s_few;
  const int per = (kblocks + s - 1) / s;
  return (kblocks + per - 1) / per;
}

// out: float32 [slices, M, N].  M <= 64, K a multiple of 8, row strides multiples of 8.
TKB_EXPORT int tkb_linear_smallm_bf16(const void* A, int lda, const void* W, int ldw, float* out, int M, int N, int K,
                                      int slices, void* st) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || slices < 1 || slices > 65535) return -2;
  const int kblocks = (K + BK - 1) / BK;
  const int per = (kblocks + slices - 1) / slices;
  if ((long long)(slices - 1) * per >= kblocks) return -2;  // an empty slice would leave its partial unwritten
  return dispatch<false>(A, lda, W, ldw, out, M, N, K, slices, per, (cudaStream_t)st);
}

// W: [N, K] with N = 2 * I rows interleaved in groups of 8 (8 gate rows, then their 8 up rows);
// out: bfloat16 [M, I] = silu(gate) * up.  I a multiple of 8.
TKB_EXPORT int tkb_linear_smallm_gated_bf16(const void* A, int lda, const void* W, int ldw, void* out, int M, int N,
                                            int K, void* st) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || (N & 15)) return -2;
  const int kblocks = (K + BK - 1) / BK;
  return dispatch<true>(A, lda, W, ldw, out, M, N, K, 1, kblocks, (cudaStream_t)st);
}
