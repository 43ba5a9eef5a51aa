// Matrix products for many tokens (prefill) on the fifth-generation tensor cores:
//
//   out[M, N] = A[M, K] . W[N, K]^T      bfloat16 operands, float32 accumulation in tensor memory
//
// A block computes 128 x BN tiles, one after the other (persistent).  Roles inside the block:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the A and W tiles of
//            each 64-wide k-block into a ring of shared-memory stages and arms the stage's mbarrier;
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (128 x BN x 16 per instruction, four
//            per k-block) on the stages as they fill and lets tcgen05.commit free them;
//   warps 2-5  wait for a tile's accumulator, read it with tcgen05.ld (each warp its 32 lanes of tensor
//            memory, i.e. 32 rows of the tile) and store the epilogue's result, while the MMAs of the next
//            tile fill the second accumulator buffer.
// Epilogues: bfloat16 store; or, for a weight that interleaves gate and up rows in groups of 8,
// silu(gate) * up as bfloat16 [M, N/2] (the activation pass over memory disappears).
//
// No load uses cluster multicast.  Every wait on an mbarrier is bounded: after the limit the block sets
// TKB_STATUS_WAIT_TIMEOUT in the status word, stops waiting, frees its tensor memory and returns.
#include "tcgen05.cuh"

using namespace tkb5;

namespace {

constexpr int BM = 128;
constexpr int THREADS = 192;  // 6 warps

template <int BN> struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN >= 256 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack to align the ring to 1024 bytes
  static constexpr int TMEM_COLS = 2 * BN;                       // two accumulators; a power of two >= 32
};

// Persistent: a block walks the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...; consecutive tiles share
// their W columns (tile t covers row block t % m_tiles of column block t / m_tiles), so W tiles stay in L2.
// The accumulator is double buffered in tensor memory: the epilogue of one tile runs while the next tile's
// MMAs fill the other buffer.
template <int BN, bool GATED>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ out, int ldo, int M, int N, int K, int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int STAGES = Cfg<BN>::STAGES;
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kblocks = (K + BK - 1) / BK;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b2 = 0; b2 < 2; b2++) {
      mbar_init(&acc_full[b2], 1);
      mbar_init(&acc_empty[b2], 4);  // one arrival from each epilogue warp
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)Cfg<BN>::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      uint32_t it = 0;  // k-blocks issued so far, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < n_kblocks; kb++, it++) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) { failed = 1; ok = false; break; }
          unsigned char* a_dst = ring + s * Cfg<BN>::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg<BN>::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * BK, m0);
          tma_load_2d(a_dst + Cfg<BN>::A_BYTES, &map_w, &full_bar[s], kb * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = make_idesc(BM, BN);
      uint32_t it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, j++) {
        const uint32_t buf = j & 1;
        if (j >= 2 && !mbar_wait(&acc_empty[buf], ((j >> 1) - 1) & 1)) { failed = 1; ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_acc + buf * BN;
        for (int kb = 0; kb < n_kblocks; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) { failed = 1; ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * Cfg<BN>::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg<BN>::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            // 16 k-elements further = 32 bytes further inside the swizzled row
            umma(d_tmem, make_desc(a_addr + k * UMMA_K * 2), make_desc(b_addr + k * UMMA_K * 2), idesc,
                 (kb > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
        }
        tcgen05_commit(&acc_full[buf]);  // this tile's accumulator is complete when the MMAs above are
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5; a warp may touch only its own quarter of tensor memory
    const int q = warp & 3;
    uint32_t j = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, j++) {
      const uint32_t buf = j & 1;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      if (!mbar_wait(&acc_full[buf], (j >> 1) & 1)) { failed = 1; ok = false; break; }
      tcgen05_fence_after();
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        if (row < M) {
          if (!GATED) {
            const int n = n0 + c0;
            bf16* dst = out + (size_t)row * ldo + n;
            if (n + 32 <= N && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; v++) {
                uint4 u;
                u.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                u.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                u.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                u.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                reinterpret_cast<uint4*>(dst)[v] = u;
              }
            } else {
              for (int jj = 0; jj < 32; jj++)
                if (n + jj < N) dst[jj] = __float2bfloat16_rn(__uint_as_float(r[jj]));
            }
          } else {
            // columns come in groups of 16: 8 gate columns, then the 8 up columns of the same features
#pragma unroll
            for (int g = 0; g < 2; g++) {
              const int n = n0 + c0 + 16 * g;
              if (n + 16 <= N) {
                float y[8];
#pragma unroll
                for (int jj = 0; jj < 8; jj++)
                  y[jj] = silu_mul_fast(__uint_as_float(r[16 * g + jj]), __uint_as_float(r[16 * g + 8 + jj]));
                uint4 u;
                u.x = pack_bf16(y[0], y[1]);
                u.y = pack_bf16(y[2], y[3]);
                u.z = pack_bf16(y[4], y[5]);
                u.w = pack_bf16(y[6], y[7]);
                bf16* dst = out + (size_t)row * ldo + (n >> 1);
                if ((((uintptr_t)dst) & 15) == 0) {
                  *reinterpret_cast<uint4*>(dst) = u;
                } else {
                  for (int jj = 0; jj < 8; jj++) dst[jj] = __float2bfloat16_rn(y[jj]);
                }
              }
            }
          }
        }
      }
      // this warp has read its part of the buffer: let the MMA issuer have it again
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    tcgen05_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)Cfg<BN>::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && failed) atomicOr(status, TKB_STATUS_WAIT_TIMEOUT);
}

template <int BN, bool GATED>
int launch(const void* A, int lda, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int* status,
           cudaStream_t st) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, A, M, K, lda, BM);
  if (rc) return rc;
  rc = make_map(&map_w, W, N, K, ldw, BN);
  if (rc) return rc;
  const int n_sms = tkb::sm_count();
  const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  dim3 grid(tiles < n_sms ? tiles : n_sms);
  gemm_tcgen05_kernel<BN, GATED><<<grid, THREADS, Cfg<BN>::SMEM_BYTES, st>>>(map_a, map_w, (bf16*)out, ldo, M, N, K, status);
  return launch_status();
}

}  // namespace

// out[M, N] (bfloat16, row stride ldo) = A[M, K] . W[N, K]^T.  gated != 0: W interleaves gate/up rows in groups of
// 8 and out is [M, N/2] = silu(gate) * up.  K and the row strides must be multiples of 8 elements and the base
// addresses 16-byte aligned (what a TMA descriptor asks for); N a multiple of 16 for the gated form.
TKB_EXPORT int tkb_gemm_tcgen05_bf16(const void* A, int lda, const void* W, int ldw, void* out, int ldo, int M, int N,
                                     int K, int gated, int* status, void* st_) {
  cudaStream_t st = (cudaStream_t)st_;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return -2;
  if (gated && (N & 15)) return -2;
  int rc = get_encode();
  if (rc) return rc;
  if (N >= 256) {
    return gated ? launch<256, true>(A, lda, W, ldw, out, ldo, M, N, K, status, st)
                 : launch<256, false>(A, lda, W, ldw, out, ldo, M, N, K, status, st);
  }
  return gated ? launch<128, true>(A, lda, W, ldw, out, ldo, M, N, K, status, st)
               : launch<128, false>(A, lda, W, ldw, out, ldo, M, N, K, status, st);
}
