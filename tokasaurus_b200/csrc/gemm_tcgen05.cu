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
#include "common.cuh"
#include <cuda.h>

using namespace tkb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;  // 6 warps
constexpr uint32_t WAIT_LIMIT = 1u << 22;

template <int BN> struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN >= 256 ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack to align the ring to 1024 bytes
  static constexpr int TMEM_COLS = 2 * BN;                       // two accumulators; a power of two >= 32
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle, groups of 8 rows
// 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)0 << 16;                        // leading byte offset: not used for this layout
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
  return d;
}
// Instruction descriptor: D = float32, A = B = bfloat16, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// silu(g) * u with the special-function unit: g * u / (1 + 2^(-g * log2 e))
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-g * 1.4426950408889634f));
  return __fdividef(g * u, 1.f + e);
}

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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode() {
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return (int)e;
  if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return -5;
  g_encode = (EncodeTiledFn)fn;
  return 0;
}

// A [rows, K] bfloat16 matrix with row stride `ld` elements; boxes of 64 x box_rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
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
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0) n_sms = 148;
  }
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
