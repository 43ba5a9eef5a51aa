// Fused matrix products for steps with at most 16 tokens (decode).
//
//   out[M, N] = prologue(A)[M, K] . W[N, K]^T,   bfloat16 operands, float32 accumulation
//
// A block owns 16 output features (one mma.sync m16n8k16 row tile of W) and ALL of K, so its result is
// complete and needs no second kernel: the epilogue can add it to the residual stream, apply the
// SiLU gate, or store it.  Eight warps share K: every 1,024-wide chunk of K is cut into eight
// 128-wide parts, one per warp, each with its own cp.async ring of three stages (no block-wide
// barrier in the loop); the warps' partial sums meet once, in shared memory, in a fixed order.
//
// Prologues: A in bfloat16; or A = the float32 residual stream with an RMS norm folded in.  The norm's
// 1/rms factor is the same for a whole row, so it is applied to the finished sums; the loop
// multiplies by the norm weight only and gathers the row's sum of squares on the way.
//
// The tokens sit on the 8-column side of the MMA and are read straight from global memory into
// fragments (they are few and come from L2).  With programmatic dependent launch the weight tiles of
// the first three chunks are in flight before the kernel that produces A has finished.
#include "common.cuh"

using namespace tkb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int WARPS = 8;
constexpr int KW = 128;                  // k per warp per chunk
constexpr int CHUNK_K = WARPS * KW;      // 1024
constexpr int ROWB = KW * 2 + 16;        // padded bytes per weight row part
constexpr int PART_B = 16 * ROWB;        // one warp's part of one stage
constexpr int STAGES = 3;
constexpr int STAGE_B = WARPS * PART_B;
constexpr int RING_B = STAGES * STAGE_B;  // 104,448 bytes

enum { PRO_BF16 = 0, PRO_NORM = 1 };
enum { EPI_BF16 = 0, EPI_ADD = 1, EPI_GATED = 2, EPI_F32 = 3 };

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
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// This warp's 16 x 128 part of W for chunk c: rows n0 .. n0+15, k = c*1024 + warp*128 ...
__device__ __forceinline__ void load_w_part(unsigned char* part, const bf16* __restrict__ W, int ldw, int N, int K,
                                            int n0, int k0, int lane) {
  const uint32_t s = smem_u32(part);
#pragma unroll
  for (int i = 0; i < (16 * 16) / 32; i++) {  // 16 rows x 16 chunks of 16 bytes
    const int idx = lane + i * 32;
    const int r = idx >> 4, c = idx & 15;
    const int n = n0 + r, k = k0 + c * 8;
    const bool valid = n < N && k < K;
    cp_async16(s + r * ROWB + c * 16, W + (valid ? (size_t)n * ldw + k : 0), valid);
  }
}

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
linear_decode_kernel(const void* __restrict__ A_, int lda, const float* __restrict__ norm_w, float eps,
                     const bf16* __restrict__ W, int ldw, void* __restrict__ out_, int ldo, int M, int N, int K) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * 16;
  const int n_chunks = (K + CHUNK_K - 1) / CHUNK_K;
  unsigned char* my_ring = smem + warp * PART_B;  // + stage * STAGE_B

  trigger_dependents();
  // weights first: nothing writes them, so this may overlap the kernel that is still producing A
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if (s < n_chunks) load_w_part(my_ring + s * STAGE_B, W, ldw, N, K, n0, s * CHUNK_K + warp * KW, lane);
    cp_async_commit();
  }
  grid_dependency_wait();

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[j][i] = 0.f;
  float ssq[NT] = {};  // PRO_NORM: this thread's share of sum(x^2) of token row j*8 + lane/4

  const int bn = lane >> 2;          // token row within an 8-token tile
  const int kq = (lane & 3) * 2;     // k offset of this thread's fragment elements
  const int w_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int w_chunk = lane >> 4;

  for (int c = 0; c < n_chunks; c++) {
    {
      const int nxt = c + STAGES - 1;
      if (nxt < n_chunks)
        load_w_part(my_ring + (nxt % STAGES) * STAGE_B, W, ldw, N, K, n0, nxt * CHUNK_K + warp * KW, lane);
      cp_async_commit();
    }
    const int kbase = c * CHUNK_K + warp * KW;
    // token fragments for this warp's 8 k-steps, straight from global memory
    uint32_t bfrag[KW / 16][NT][2];
#pragma unroll
    for (int ks = 0; ks < KW / 16; ks++) {
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int row = j * 8 + bn;
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int k = kbase + ks * 16 + kq + h * 8;
          uint32_t v = 0u;
          if (row < M && k < K) {
            if (PRO == PRO_BF16) {
              v = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const bf16*>(A_) + (size_t)row * lda + k);
            } else {
              const float2 x = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(A_) + (size_t)row * lda + k);
              const float2 w = *reinterpret_cast<const float2*>(norm_w + k);
              ssq[j] += x.x * x.x + x.y * x.y;
              v = pack_bf16(x.x * w.x, x.y * w.y);
            }
          }
          bfrag[ks][j][h] = v;
        }
      }
    }
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const uint32_t sw = smem_u32(my_ring + (c % STAGES) * STAGE_B);
#pragma unroll
    for (int ks = 0; ks < KW / 16; ks++) {
      uint32_t wf[4];
      ldmatrix_x4(wf[0], wf[1], wf[2], wf[3], sw + w_row * ROWB + (ks * 2 + w_chunk) * 16);
#pragma unroll
      for (int j = 0; j < NT; j++) mma_bf16(acc[j], wf, bfrag[ks][j][0], bfrag[ks][j][1]);
    }
    __syncwarp();  // the stage is refilled two iterations from now by this same warp
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: reuse the memory for the reduction

  // red[warp][feature 0..15][token 0..NT*8-1], ssum[warp][token]
  float* red = reinterpret_cast<float*>(smem);
  float* ssum = red + WARPS * 16 * NT * 8;
  {
    const int r = lane >> 2;
#pragma unroll
    for (int j = 0; j < NT; j++) {
      float* b = red + ((warp * 16 + r) * NT * 8) + j * 8 + kq;
      b[0] = acc[j][0];
      b[1] = acc[j][1];
      b[8 * NT * 8] = acc[j][2];
      b[8 * NT * 8 + 1] = acc[j][3];
    }
    if (PRO == PRO_NORM) {
#pragma unroll
      for (int j = 0; j < NT; j++) {
        float v = ssq[j];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if ((lane & 3) == 0) ssum[warp * NT * 8 + j * 8 + bn] = v;
      }
    }
  }
  __syncthreads();
  constexpr int TOK = NT * 8;
  constexpr int OUTS = (EPI == EPI_GATED ? 8 : 16) * TOK;
  for (int o = tid; o < OUTS; o += WARPS * 32) {
    const int f = o / TOK, b = o - f * TOK;
    if (b >= M) continue;
    float v = 0.f, v2 = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
      v += red[(w * 16 + f) * TOK + b];
      if (EPI == EPI_GATED) v2 += red[(w * 16 + f + 8) * TOK + b];
    }
    if (PRO == PRO_NORM) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; w++) s += ssum[w * TOK + b];
      const float rstd = rsqrtf(s / (float)K + eps);
      v *= rstd;
      v2 *= rstd;
    }
    if (EPI == EPI_GATED) {
      // weight rows n0..n0+7 are gate rows of features (n0/2)..(n0/2)+7, rows n0+8.. their up rows
      const int g = (n0 >> 1) + f;
      if (n0 + f + 8 < N)
        reinterpret_cast<bf16*>(out_)[(size_t)b * ldo + g] = __float2bfloat16_rn(v / (1.f + expf(-v)) * v2);
    } else {
      const int n = n0 + f;
      if (n >= N) continue;
      if (EPI == EPI_BF16) reinterpret_cast<bf16*>(out_)[(size_t)b * ldo + n] = __float2bfloat16_rn(v);
      else if (EPI == EPI_F32) reinterpret_cast<float*>(out_)[(size_t)b * ldo + n] = v;
      else reinterpret_cast<float*>(out_)[(size_t)b * ldo + n] += v;  // this block alone owns the element
    }
  }
}

template <int NT, int PRO, int EPI>
int launch(const void* A, int lda, const float* norm_w, float eps, const void* W, int ldw, void* out, int ldo, int M,
           int N, int K, cudaStream_t st) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(linear_decode_kernel<NT, PRO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         RING_B);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid((N + 15) / 16);
  return launch_pdl(linear_decode_kernel<NT, PRO, EPI>, grid, dim3(WARPS * 32), (size_t)RING_B, st, A, lda, norm_w, eps,
                    (const bf16*)W, ldw, out, ldo, M, N, K);
}

template <int PRO, int EPI>
int dispatch(const void* A, int lda, const float* norm_w, float eps, const void* W, int ldw, void* out, int ldo, int M,
             int N, int K, cudaStream_t st) {
  if (M <= 8) return launch<1, PRO, EPI>(A, lda, norm_w, eps, W, ldw, out, ldo, M, N, K, st);
  return launch<2, PRO, EPI>(A, lda, norm_w, eps, W, ldw, out, ldo, M, N, K, st);
}

}  // namespace

// prologue: 0 = A is bfloat16 [M, K]; 1 = A is the float32 stream [M, K] and an RMS norm with weight
// norm_w [K] and eps is folded in.  epilogue: 0 = store bfloat16 [M, N]; 1 = add into float32 out [M, N];
// 2 = W interleaves gate/up rows in groups of 8, store silu(gate)*up as bfloat16 [M, N/2]; 3 = store float32.
// M <= 16; K and the row strides multiples of 8; N a multiple of 16 for the gated epilogue.
TKB_EXPORT int tkb_linear_decode_bf16(const void* A, int lda, const float* norm_w, float eps, const void* W, int ldw,
                                      void* out, int ldo, int M, int N, int K, int prologue, int epilogue, void* st_) {
  cudaStream_t st = (cudaStream_t)st_;
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7)) return -2;
  if (epilogue == EPI_GATED && (N & 15)) return -2;
  if (prologue == PRO_NORM && norm_w == nullptr) return -2;
#define TKB_CASE(P, E) \
  if (prologue == P && epilogue == E) return dispatch<P, E>(A, lda, norm_w, eps, W, ldw, out, ldo, M, N, K, st);
  TKB_CASE(PRO_BF16, EPI_BF16)
  TKB_CASE(PRO_BF16, EPI_ADD)
  TKB_CASE(PRO_BF16, EPI_F32)
  TKB_CASE(PRO_NORM, EPI_BF16)
  TKB_CASE(PRO_NORM, EPI_GATED)
  TKB_CASE(PRO_NORM, EPI_F32)
#undef TKB_CASE
  return -2;
}
