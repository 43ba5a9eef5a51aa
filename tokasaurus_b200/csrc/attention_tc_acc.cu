// Causal attention for prompt portions on the fifth-generation tensor cores with the output accumulated in tensor
// memory (head sizes 64 and 128, bfloat16; compile with -DTKB_HD).
//
// A block owns 128 consecutive query tokens of TWO query heads that share a kv head (one head where the group
// size is odd and no partner is left) and walks the keys they may see in tiles of 64.  For each head:
//     S = Q . K^T      tcgen05.mma 128 x 64 x 16, HD / 16 per tile, two S tiles in tensor memory (the product of
//                      tile j+2 starts as soon as the softmax threads are through with S_j)
//     softmax          a warpgroup per head, one thread per query row (a lane of tensor memory): row maximum, then
//                      exp2 and row sum, each a pass of tcgen05.ld over S; P (bfloat16) goes to shared memory
//                      in the 128-byte-swizzled K-major layout (two buffers)
//     O += P . V       tcgen05.mma 128 x HD x 16, four per tile, accumulating in tensor memory over ALL tiles; V
//                      stays as the cache holds it ([key][head size]), an MN-major operand
// The exponentials of a row use a reference that stays put while the row's scores stay below reference + 16
// (probabilities up to 2^16 are no problem for bfloat16 or for float32 sums).  When a row tops that, its warp
// waits for the P . V products issued so far, reads its 32 lanes of O, scales the rows concerned and writes them
// back (tcgen05.st): rare after the first tiles, so the loop has no pass over O at all and a thread needs no
// registers for it.  The row sum l follows the same reference; O / l at the end does not depend on it.
// Roles: warps 0-3 and 4-7 softmax and output of the two heads; warp 8 brings K tiles and warp 9 V tiles into
// rings (TMA boxes of whole pages where the page size is a power of two from 8 up and the tile's keys all exist,
// else cp.async gathers that zero-fill keys beyond the request); warps 10 and 11 issue the MMAs of one head each
// (one lane); warp 10 allocates all 512 columns of tensor memory, after the kernel ahead has finished.
// Every wait on an mbarrier is bounded; after the limit the block sets TKB_STATUS_WAIT_TIMEOUT and leaves.
#include "tcgen05.cuh"

#ifndef TKB_HD
#error "compile with -DTKB_HD=64 or 128"
#endif
static_assert(TKB_HD == 64 || TKB_HD == 128, "head size 64 or 128");

using namespace tkb5;

namespace {

constexpr int HD = TKB_HD;
constexpr int ATOMS = HD / 64;           // 64-column (128-byte) blocks of a row of head size
constexpr int BQ = 128;                  // queries per block
constexpr int BKV = 64;                  // keys per tile
constexpr int KV_STAGES = 3;
constexpr int THREADS = 384;
constexpr int Q_BYTES = BQ * HD * 2;     // per head: ATOMS blocks of [128 rows x 128 B]
constexpr int KV_BYTES = BKV * HD * 2;   // per tile: ATOMS blocks of [64 rows x 128 B]
constexpr int P_BYTES = BQ * BKV * 2;    // [128 rows x 128 B]
constexpr int SMEM_BYTES = 2 * Q_BYTES + 2 * KV_STAGES * KV_BYTES + 4 * P_BYTES + 1024;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_S = 0, TMEM_O = 256;  // S: head * 128 + buffer * 64; O: head * 128
constexpr float NEG_BIG = -1.0e30f;
constexpr float REF_SLACK = 16.f;        // a row's reference moves when a score tops it by more than this (log2)

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand (V as [key][head size]): rows of 128 bytes, 8-key groups 1,024 bytes apart, the 64-column
// blocks of a wider head KV_BYTES / ATOMS bytes apart
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((BKV * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// One tile (64 keys) of K or V of one kv head into ATOMS swizzled [64 x 64] blocks; keys outside [key_lo, key_hi)
// are zero.  A warp's lane takes rows lane and lane + 32: their page lookups go out together.
__device__ __forceinline__ void gather_tile(uint32_t dst, const bf16* __restrict__ cache, const int* __restrict__ table,
                                            int kvh, int nkv, int ps, int ps_shift, int key_base, int key_lo, int key_hi,
                                            int lane, int num_pages, bool& bad_page) {
  size_t off[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int key = key_base + lane + 32 * i;
    valid[i] = key >= key_lo && key < key_hi;
    off[i] = 0;
    if (valid[i]) {
      const int pi = ps_shift >= 0 ? key >> ps_shift : key / ps;
      const int slot = ps_shift >= 0 ? key & (ps - 1) : key - pi * ps;
      const int page = checked_page(__ldg(table + pi), num_pages, bad_page);
      valid[i] = page >= 0;  // a page given back behind a window, or an id beyond the pool: zeros
      off[i] = valid[i] ? (((size_t)page * nkv + kvh) * ps + slot) * HD : 0;
    }
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int r = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < HD / 8; c++)
      cp_async16(dst + (c >> 3) * (BKV * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4), cache + off[i] + c * 8, valid[i]);
  }
}

// Row maximum of one thread's 64 scores in tensor memory (loops stay rolled: this code runs once per key tile and
// must stay in the instruction cache).
template <bool MASKED>
__device__ __forceinline__ float row_max(uint32_t s_addr, int lo, uint32_t span) {
  uint32_t a[32], b[32];
  tmem_ld32_issue(s_addr, a);
  tmem_ld32_issue(s_addr + 32, b);
  tmem_wait();
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float x0 = __uint_as_float(a[i]), x1 = __uint_as_float(a[i + 1]);
    float y0 = __uint_as_float(b[i]), y1 = __uint_as_float(b[i + 1]);
    if (MASKED) {
      const int c = i - lo;
      if ((uint32_t)c > span) x0 = -INFINITY;
      if ((uint32_t)(c + 1) > span) x1 = -INFINITY;
      if ((uint32_t)(c + 32) > span) y0 = -INFINITY;
      if ((uint32_t)(c + 33) > span) y1 = -INFINITY;
    }
    m0 = fmaxf(m0, x0);
    m1 = fmaxf(m1, x1);
    m2 = fmaxf(m2, y0);
    m3 = fmaxf(m3, y1);
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// p = 2^(s * scale - ref) of one row: bfloat16 into the row's place of the swizzled P tile; returns the row sum.
template <bool MASKED>
__device__ __forceinline__ float row_exp(uint32_t s_addr, unsigned char* prow, int r, int lo, uint32_t span, float scale,
                                         float neg_ref) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll 1
  for (int c0 = 0; c0 < BKV; c0 += 32) {
    uint32_t v[32];
    tmem_ld32_issue(s_addr + c0, v);
    tmem_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
      if (MASKED) {
        const int c = c0 + i - lo;
        if ((uint32_t)c > span) x0 = -INFINITY;
        if ((uint32_t)(c + 1) > span) x1 = -INFINITY;
      }
      const float p0 = fast_exp2(fmaf(x0, scale, neg_ref)), p1 = fast_exp2(fmaf(x1, scale, neg_ref));
      s0 += p0;
      s1 += p1;
      pk[i >> 1] = pack_bf16(p0, p1);
    }
    const int cbase = c0 >> 3;  // 32 keys = four 16-byte chunks of this row
#pragma unroll
    for (int cc = 0; cc < 4; cc++)
      *reinterpret_cast<uint4*>(prow + (((cbase + cc) ^ (r & 7)) << 4)) =
          make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
  }
  return s0 + s1;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_acc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int tma_rows,
                        const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                        const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                        const int* __restrict__ page_ids, const int* __restrict__ tiles,
                        const int* __restrict__ n_tiles_ptr, int nh, int nkv, int ps, float scale_log2, int window,
                        int* __restrict__ status, int num_pages, int single) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES],
      s_full[2][2], p_full[2], pv_done[2][2];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  trigger_dependents();
  grid_dependency_wait();
  if ((int)blockIdx.y >= *n_tiles_ptr) return;
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = base;                         // two heads
  unsigned char* sK = sQ + 2 * Q_BYTES;             // ring
  unsigned char* sV = sK + KV_STAGES * KV_BYTES;    // ring
  unsigned char* sP = sV + KV_STAGES * KV_BYTES;    // two heads x two buffers
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int s = tiles[2 * blockIdx.y], qt0 = tiles[2 * blockIdx.y + 1];
  const int group = nh / nkv;
  // `single`: one head a block (the host asks for it when pairs would leave SMs without a block)
  const int pairs = single ? group : (group + 1) >> 1;
  const int kvh = blockIdx.x / pairs;
  const int pair = blockIdx.x - kvh * pairs;
  const int head0 = kvh * group + (single ? pair : 2 * pair);
  const int n_heads_here = (!single && 2 * pair + 1 < group) ? 2 : 1;
  const int q_len = seq_q_len[s], kv_len = seq_kv_len[s];
  const int rows_live = min(BQ, q_len - qt0);
  const int pos0 = kv_len - q_len + qt0;
  int k_begin = 0;  // a multiple of the tile, so that whole tiles are whole pages
  if (window > 0 && pos0 - window + 1 > 0) k_begin = (pos0 - window + 1) & ~(BKV - 1);
  const int k_end = pos0 + rows_live;  // one past the last key any row of the tile sees
  const int n_kv_tiles = (k_end - k_begin + BKV - 1) / BKV;
  const int* table = page_ids + page_indptr[s];
  const int t0 = seq_q_start[s] + qt0;

  if (tid == 0) {
    for (int i = 0; i < KV_STAGES; i++) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], n_heads_here);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], n_heads_here);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&p_full[i], 128);
      for (int b = 0; b < 2; b++) {
        mbar_init(&s_full[i][b], 1);
        mbar_init(&pv_done[i][b], 1);
      }
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 10) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp < 8) {
    // Q tiles: thread = (head, row); rows past the portion and the missing partner head are zero
    const int hh = warp >> 2, r = tid & 127;
    const bool live = r < rows_live && hh < n_heads_here;
    const bf16* src = q + (size_t)(t0 + (live ? r : 0)) * q_stride + (size_t)(head0 + (live ? hh : 0)) * HD;
    const uint32_t dst = smem_u32(sQ + hh * Q_BYTES) + r * 128;
#pragma unroll
    for (int c = 0; c < HD / 8; c++) cp_async16(dst + (c >> 3) * (BQ * 128) + (((c & 7) ^ (r & 7)) << 4), src + c * 8, live);
    cp_async_wait_all();
    fence_proxy_async();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = tmem_slot;
  const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;

  if (warp == 8 || warp == 9) {
    // ---------------- loaders: warp 8 K tiles, warp 9 V tiles
    const bool is_v = warp == 9;
    const bf16* cache = is_v ? vcache : kcache;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    unsigned char* ring = is_v ? sV : sK;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    bool ok = true, bad_page = false;
    for (int j = 0; j < n_kv_tiles; j++) {
      const int b = j % KV_STAGES;
      const int key_base = k_begin + j * BKV;
      if (j >= KV_STAGES && !mbar_wait_idle(&empty[b], ((j / KV_STAGES) - 1) & 1)) { ok = false; break; }
      if (tma_rows > 0 && key_base + BKV <= kv_len) {
        // every key of the tile exists: per 64-column block one box per page (or per 64 slots of a larger page)
        if (lane == 0) mbar_expect_tx(&full[b], KV_BYTES);
        __syncwarp();
        const int boxes = BKV / tma_rows;
        if (lane < boxes * ATOMS) {
          const int atom = lane / boxes, bx = lane - atom * boxes;
          const int key = key_base + bx * tma_rows;
          // an id beyond the pool becomes -1: a negative row is outside the tensor map and reads as zeros
          const int row = (checked_page(__ldg(table + (key >> ps_shift)), num_pages, bad_page) * nkv + kvh) * ps + (key & (ps - 1));
          tma_load_2d(ring + b * KV_BYTES + atom * (BKV * 128) + bx * tma_rows * 128, map, &full[b], atom * 64, row);
        }
      } else {
        gather_tile(smem_u32(ring + b * KV_BYTES), cache, table, kvh, nkv, ps, ps_shift, key_base, 0, kv_len, lane, num_pages, bad_page);
        cp_async_wait_all();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[b]);
      }
    }
    if (!ok) failed = 1;
    report_bad_page(bad_page, status);
  } else if (warp >= 10) {
    const int hh = warp - 10;
    if (lane == 0 && hh < n_heads_here) {
      // ---------------- MMA issuer of head hh: S_0 and S_1; then for every tile: (wait P_j, which also frees its S
      // tile) Q . K_{j+2}^T, O += P_j . V_j
      const uint32_t idesc_qk = make_idesc(BQ, BKV);
      const uint32_t idesc_pv = make_idesc(BQ, HD) | (1u << 16);  // B operand MN-major
      const uint64_t desc_q = make_desc(smem_u32(sQ + hh * Q_BYTES));
      const uint64_t desc_k0 = make_desc(smem_u32(sK)), desc_v0 = make_desc_mn(smem_u32(sV));
      const uint64_t desc_p0 = make_desc(smem_u32(sP + (hh * 2) * P_BYTES));
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int kb = j % KV_STAGES;
        if (!mbar_wait(&k_full[kb], (j / KV_STAGES) & 1)) return false;
        tcgen05_fence_after();
        const uint64_t dk = desc_k0 + (uint64_t)(kb * (KV_BYTES / 16));
#pragma unroll
        for (int k = 0; k < HD / UMMA_K; k++)  // 16 dims a step: 32 bytes further in the 64-column block k / 4
          umma(tmem + TMEM_S + hh * 128 + (j & 1) * BKV, desc_q + (uint64_t)((k >> 2) * (BQ * 128 / 16) + (k & 3) * 2),
               dk + (uint64_t)((k >> 2) * (BKV * 128 / 16) + (k & 3) * 2), idesc_qk, k > 0 ? 1u : 0u);
        tcgen05_commit(&k_empty[kb]);
        tcgen05_commit(&s_full[hh][j & 1]);
        return true;
      };
      ok = issue_qk(0);
      if (ok && n_kv_tiles > 1) ok = issue_qk(1);
      for (int j = 0; j < n_kv_tiles && ok; j++) {
        const int vb = j % KV_STAGES, pb = j & 1;
        if (!mbar_wait(&p_full[hh], j & 1)) { ok = false; break; }
        if (j + 2 < n_kv_tiles && !issue_qk(j + 2)) { ok = false; break; }
        if (!mbar_wait(&v_full[vb], (j / KV_STAGES) & 1)) { ok = false; break; }
        tcgen05_fence_after();
        const uint64_t dp = desc_p0 + (uint64_t)(pb * (P_BYTES / 16)), dv = desc_v0 + (uint64_t)(vb * (KV_BYTES / 16));
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; k++)  // 16 keys a step: 32 bytes of a P row, two 8-key groups of V
          umma(tmem + TMEM_O + hh * 128, dp + (uint64_t)(k * 2), dv + (uint64_t)(k * (2048 / 16)), idesc_pv,
               (j > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(&v_empty[vb]);
        tcgen05_commit(&pv_done[hh][pb]);
      }
      if (!ok) failed = 1;
    }
  } else if ((warp >> 2) < n_heads_here) {
    // ---------------- softmax and output: thread = query row = lane of tensor memory
    const int hh = warp >> 2;
    const int r = tid & 127;
    const int pos = pos0 + r;
    const int lim_hi = pos < k_end - 1 ? pos : k_end - 1;
    const int lim_lo = window > 0 ? max(pos - window + 1, 0) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + TMEM_S + hh * 128, o_addr = lane_addr + TMEM_O + hh * 128;
    float ref = NEG_BIG, l = 0.f;  // reference of the exponentials (and so of O and l); row sum
    bool ok = true;
    for (int j = 0; j < n_kv_tiles; j++) {
      const int key0 = k_begin + j * BKV;
      if (!mbar_wait(&s_full[hh][j & 1], (j >> 1) & 1)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t sj = s_addr + (j & 1) * BKV;
      // a tile every row of the block sees whole needs no mask; else columns [lo, lo + span] of this tile are visible
      const bool whole = key0 + BKV - 1 <= pos0 && key0 + BKV <= k_end && (window <= 0 || key0 >= pos0 + BQ - window);
      const int lo = lim_hi >= lim_lo ? lim_lo - key0 : (1 << 30);
      const uint32_t span = lim_hi >= lim_lo ? (uint32_t)(lim_hi - lim_lo) : 0u;
      const float tile_max = (whole ? row_max<false>(sj, lo, span) : row_max<true>(sj, lo, span)) * scale_log2;
      const bool moves = tile_max - ref > REF_SLACK;  // also the row's first visible key (ref is hugely negative)
      if (j == 0) {
        if (moves) ref = tile_max;
      } else if (__any_sync(0xffffffffu, moves)) {
        // rows of this warp move their reference: O and l of those rows are scaled to the new one.  Every P . V
        // product issued so far must be over (the next one waits for this thread's P).
        if (!mbar_wait(&pv_done[hh][(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
        tcgen05_fence_after();
        const float new_ref = moves ? fmaxf(ref, tile_max) : ref;
        const float alpha = fast_exp2(ref - new_ref);
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          tmem_ld32_issue(o_addr + c0, v);
          tmem_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st32(o_addr + c0, v);
        }
        tmem_wait_st();
        l *= alpha;
        ref = new_ref;
      }
      // the P buffer of this tile was read by the P . V product of two tiles ago
      if (j >= 2 && !mbar_wait(&pv_done[hh][j & 1], ((j - 2) >> 1) & 1)) { ok = false; break; }
      unsigned char* prow = sP + (hh * 2 + (j & 1)) * P_BYTES + r * 128;
      l += whole ? row_exp<false>(sj, prow, r, lo, span, scale_log2, -ref) : row_exp<true>(sj, prow, r, lo, span, scale_log2, -ref);
      tcgen05_fence_before();
      fence_proxy_async();
      mbar_arrive(&p_full[hh]);
    }
    if (ok) ok = mbar_wait(&pv_done[hh][(n_kv_tiles - 1) & 1], ((n_kv_tiles - 1) >> 1) & 1);
    if (!ok) failed = 1;
    if (ok) {
      tcgen05_fence_after();
      const float inv = 1.f / l;
      bf16* dst = out + (size_t)(t0 + r) * out_stride + (size_t)(head0 + hh) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t v[32];
        tmem_ld32_issue(o_addr + c0, v);
        tmem_wait();
        if (r < rows_live) {
#pragma unroll
          for (int c = 0; c < 4; c++)
            *reinterpret_cast<uint4*>(dst + c0 + c * 8) = make_uint4(
                pack_bf16(__uint_as_float(v[8 * c]) * inv, __uint_as_float(v[8 * c + 1]) * inv),
                pack_bf16(__uint_as_float(v[8 * c + 2]) * inv, __uint_as_float(v[8 * c + 3]) * inv),
                pack_bf16(__uint_as_float(v[8 * c + 4]) * inv, __uint_as_float(v[8 * c + 5]) * inv),
                pack_bf16(__uint_as_float(v[8 * c + 6]) * inv, __uint_as_float(v[8 * c + 7]) * inv));
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 10) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
  if (tid == 0 && failed) atomicOr(status, TKB_STATUS_WAIT_TIMEOUT);
}

}  // namespace

// tiles: int32 [tiles_cap * 2] (request row, first query of a 128-query tile within the portion), the tiles that
// see the most keys first; n_tiles_ptr: live count on the device.  q/out rows are token rows; head h occupies
// columns h*HD .. h*HD+HD-1.  q and out row strides multiples of 8 elements.  kcache/vcache: [n_pages, nkv, ps, HD].
TKB_EXPORT int tkb_attn_prefill_acc_bf16(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                         const void* vcache, int n_pages, const int* seq_q_start, const int* seq_q_len,
                                         const int* seq_kv_len, const int* page_indptr, const int* page_ids,
                                         const int* tiles, const int* n_tiles_ptr, int tiles_cap, int nh, int nkv, int ps,
                                         float scale, int window, int single, int* status, void* st) {
  if (tiles_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0 || (q_stride & 7) || (out_stride & 7)) return -2;
  if (tiles_cap > 65535) return -3;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_acc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  // TMA boxes of whole pages where the page size allows; else every tile is gathered
  CUtensorMap map_k, map_v;
  memset(&map_k, 0, sizeof(map_k));
  memset(&map_v, 0, sizeof(map_v));
  int tma_rows = 0;
  const long long rows = (long long)n_pages * nkv * ps;
  if ((ps & (ps - 1)) == 0 && ps >= 8 && rows < (1ll << 31) && ((uintptr_t)kcache & 15) == 0 && ((uintptr_t)vcache & 15) == 0) {
    tma_rows = ps < BKV ? ps : BKV;
    int rc = get_encode();
    if (rc == 0) rc = make_map(&map_k, kcache, (int)rows, HD, HD, tma_rows);
    if (rc == 0) rc = make_map(&map_v, vcache, (int)rows, HD, HD, tma_rows);
    if (rc != 0) return rc;
  }
  const int pairs = single ? nh / nkv : (nh / nkv + 1) / 2;
  dim3 grid(nkv * pairs, tiles_cap);  // the head pairs of one query tile are neighbours: long tiles start first
  return launch_pdl(attn_prefill_acc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)st, map_k, map_v,
                    tma_rows, (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache,
                    seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles_ptr, nh, nkv, ps,
                    scale * 1.4426950408889634f, window, status, n_pages, single ? 1 : 0);
}

TKB_EXPORT int tkb_attn_prefill_acc_head_dim() { return HD; }
