// Matrix products for steps with few tokens (decode) on the fifth-generation tensor cores, built to stream the
// weights at memory speed:
//
//   out[M, N] = A[M, K] . W[N, K]^T,   M <= 64,   bfloat16 operands, float32 accumulation in tensor memory
//
// The WEIGHT rows are the 128-row side of tcgen05.mma and the tokens its 16-, 32- or 64-column side, so the instruction's
// shape wastes nothing of the weight traffic.  A block owns 128 output features and one slice of K:
//   warp 0   one lane issues TMA loads (128 x 64 weight box, 16 x 64 token box, 128-byte swizzle) into a
//            ten-stage ring: 160 KiB of weights in flight per SM, issued by a handful of instructions;
//   warp 1   allocates tensor memory; one lane issues the MMAs (128 x 16 x 16) and frees stages with
//            tcgen05.commit;
//   warps 2-5  read the 128 x 16 accumulator with tcgen05.ld (one feature per thread) and store it.
// K slices leave float32 partial results [slice, M, N] that the consumer adds in slice order, as with the
// mma.sync kernel of linear_smallm.cu.  The gated form (one slice) pairs gate and up features (interleaved in
// groups of 8 rows) with a shuffle and stores silu(gate) * up as bfloat16 [M, N/2].
// With programmatic dependent launch the weight boxes of all ten stages are requested before the kernel that
// produces A has finished; the token boxes follow after griddepcontrol.wait.
// No load uses cluster multicast; every mbarrier wait is bounded (TKB_STATUS_WAIT_TIMEOUT).
#include "tcgen05.cuh"

using namespace tkb5;

namespace {

constexpr int BMW = 128;   // weight rows (features) per block
constexpr int THREADS = 192;
constexpr int W_BYTES = BMW * BK * 2;  // 16 KiB

// NTOK: token columns of the MMA (16, 32 or 64)
template <int NTOK> struct DCfg {
  static constexpr int T_BYTES = NTOK * BK * 2;           // 2, 4 or 8 KiB
  static constexpr int STAGE_BYTES = W_BYTES + T_BYTES;   // both parts start on 1,024-byte boundaries
  static constexpr int STAGES = NTOK == 16 ? 10 : (NTOK == 32 ? 9 : 8);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr int TMEM_COLS = NTOK < 32 ? 32 : NTOK;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int NTOK, bool GATED>
__global__ void __launch_bounds__(THREADS, 1)
linear_tcgen05_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                             void* __restrict__ out_, int M, int N, int K, int kblocks_per_slice,
                             int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int STAGES = DCfg<NTOK>::STAGES, STAGE_BYTES = DCfg<NTOK>::STAGE_BYTES, TMEM_COLS = DCfg<NTOK>::TMEM_COLS;
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BMW;
  const int slice = blockIdx.y;
  const int kb_begin = slice * kblocks_per_slice;
  const int kb_total = (K + BK - 1) / BK;
  const int nkb = min(kblocks_per_slice, kb_total - kb_begin);

  trigger_dependents();
  const int first = nkb < STAGES ? nkb : STAGES;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // Weights first: no kernel writes them, so their boxes may be on their way while the kernel before this
    // one still runs.
    for (int kb = 0; kb < first; kb++) {
      mbar_expect_tx(&full_bar[kb], STAGE_BYTES);
      tma_load_2d(ring + kb * STAGE_BYTES, &map_w, &full_bar[kb], (kb_begin + kb) * BK, n0);
    }
  }
  if (warp == 1) {
    // Tensor memory is taken only after the kernel ahead has finished: a block of that kernel that still
    // waits for columns on this SM could otherwise wait for this block, which waits for that kernel.
    grid_dependency_wait();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer: the tokens only after the kernel ahead has finished
      grid_dependency_wait();
      for (int kb = 0; kb < first; kb++)
        tma_load_2d(ring + kb * STAGE_BYTES + W_BYTES, &map_a, &full_bar[kb], (kb_begin + kb) * BK, 0);
      for (int kb = STAGES; kb < nkb; kb++) {
        const int s = kb % STAGES;
        if (!mbar_wait(&empty_bar[s], ((kb / STAGES) - 1) & 1)) { failed = 1; break; }
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(ring + s * STAGE_BYTES, &map_w, &full_bar[s], (kb_begin + kb) * BK, n0);
        tma_load_2d(ring + s * STAGE_BYTES + W_BYTES, &map_a, &full_bar[s], (kb_begin + kb) * BK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = make_idesc(BMW, NTOK);
      for (int kb = 0; kb < nkb; kb++) {
        const int s = kb % STAGES;
        if (!mbar_wait(&full_bar[s], (kb / STAGES) & 1)) { failed = 1; break; }
        tcgen05_fence_after();
        const uint32_t w_addr = smem_u32(ring + s * STAGE_BYTES);
        const uint32_t t_addr = w_addr + W_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; k++)
          umma(tmem_acc, make_desc(w_addr + k * UMMA_K * 2), make_desc(t_addr + k * UMMA_K * 2), idesc,
               (kb > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(&empty_bar[s]);
      }
      tcgen05_commit(&acc_bar);
    }
  } else {
    // ---------------- epilogue: thread = one feature (a lane of tensor memory), 16 token columns
    const int q = warp & 3;
    grid_dependency_wait();  // nothing is stored before the kernel ahead of this one has finished
    const bool ok = mbar_wait(&acc_bar, 0);
    tcgen05_fence_after();
    if (!ok) failed = 1;
    if (ok) {
      const int f = n0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < NTOK; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        if (!GATED) {
          float* o = reinterpret_cast<float*>(out_) + (size_t)slice * M * N;
          if (f < N) {
#pragma unroll
            for (int t = 0; t < 16; t++)
              if (c0 + t < M) o[(size_t)(c0 + t) * N + f] = __uint_as_float(r[t]);
          }
        } else {
          // weight rows come in groups of 16: 8 gate rows, then the 8 up rows of the same features
          bf16* o = reinterpret_cast<bf16*>(out_);
          const int I = N >> 1;
          const bool is_gate = (lane & 8) == 0;
          const int g = ((n0 + q * 32 + (lane & 16)) >> 1) + (lane & 7);
#pragma unroll
          for (int t = 0; t < 16; t++) {
            const float mine = __uint_as_float(r[t]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
            if (is_gate && c0 + t < M && f + 8 < N)
              o[(size_t)(c0 + t) * I + g] = __float2bfloat16_rn(silu_mul_fast(mine, other));
          }
        }
      }
    }
    tcgen05_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && failed) atomicOr(status, TKB_STATUS_WAIT_TIMEOUT);
}

template <int NTOK, bool GATED>
int launch(const void* A, int lda, const void* W, int ldw, void* out, int M, int N, int K, int slices, int per,
           int* status, cudaStream_t st) {
  static bool attr_done = false;
  constexpr int SMEM_BYTES = DCfg<NTOK>::SMEM_BYTES;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(linear_tcgen05_decode_kernel<NTOK, GATED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  CUtensorMap map_w, map_a;
  int rc = make_map(&map_w, W, N, K, ldw, BMW);
  if (rc) return rc;
  rc = make_map(&map_a, A, M, K, lda, NTOK);
  if (rc) return rc;
  dim3 grid((N + BMW - 1) / BMW, slices);
  return launch_pdl(linear_tcgen05_decode_kernel<NTOK, GATED>, grid, dim3(THREADS), (size_t)SMEM_BYTES, st, map_w, map_a,
                    out, M, N, K, per, status);
}

}  // namespace

// Number of K slices for a grid of about one block per SM; k-blocks per slice follow as
// ceil(ceil(K / 64) / slices).
TKB_EXPORT int tkb_linear_tcgen05_decode_slices(int N, int K, int max_slices) {
  const int tiles = (N + BMW - 1) / BMW;
  const int kblocks = (K + BK - 1) / BK;
  int s = tkb::sm_count() / tiles;
  if (s > max_slices) s = max_slices;
  if (s > kblocks / 2) s = kblocks / 2;
  if (s < 1) s = 1;
  const int per = (kblocks + s - 1) / s;
  return (kblocks + per - 1) / per;
}

// out: float32 [slices, M, N] (gated == 0) or bfloat16 [M, N/2] = silu(gate) * up (gated != 0, slices == 1,
// W interleaved in groups of 8 rows, N a multiple of 16).  M <= 64; K and the row strides multiples of 8; base
// addresses 16-byte aligned.
TKB_EXPORT int tkb_linear_tcgen05_decode_bf16(const void* A, int lda, const void* W, int ldw, void* out, int M, int N,
                                              int K, int slices, int gated, int* status, void* st_) {
  cudaStream_t st = (cudaStream_t)st_;
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15) ||
      slices < 1 || slices > 65535)
    return -2;
  if (gated && ((N & 15) || slices != 1)) return -2;
  int rc = get_encode();
  if (rc) return rc;
  const int kblocks = (K + BK - 1) / BK;
  const int per = (kblocks + slices - 1) / slices;
  if ((long long)(slices - 1) * per >= kblocks) return -2;  // an empty slice would leave its partial unwritten
#define TKB_GO(NT) \
  return gated ? launch<NT, true>(A, lda, W, ldw, out, M, N, K, slices, per, status, st) \
               : launch<NT, false>(A, lda, W, ldw, out, M, N, K, slices, per, status, st);
  if (M <= 16) { TKB_GO(16) }
  if (M <= 32) { TKB_GO(32) }
  TKB_GO(64)
#undef TKB_GO
}
