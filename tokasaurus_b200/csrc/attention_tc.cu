// Causal attention for prompt portions on the fifth-generation tensor cores (head size 64, bfloat16).
//
// A block owns 128 consecutive query tokens of TWO query heads that share a kv head (one head where the group
// size is odd and no partner is left) and walks the keys they may see in tiles of 128.  The K and V tiles are
// gathered once for both heads.  For each head:
//     S = Q . K^T      tcgen05.mma 128 x 128 x 16, four per tile, Q and K tiles K-major in shared memory,
//                      S (float32) in tensor memory
//     softmax          a warpgroup per head, one thread per query row (a lane of tensor memory): two passes of
//                      tcgen05.ld over S (row maximum, then exp2 and row sum), no shuffles; P (bfloat16) goes to
//                      shared memory in the 128-byte-swizzled K-major layout
//     O += P . V       tcgen05.mma 128 x 64 x 16, eight per tile, accumulating in tensor memory over ALL tiles; V
//                      stays as the cache holds it ([key][head size]), described to the tensor core as an
//                      MN-major operand
// The exponentials of a row use a reference that stays put while the row's scores stay below reference + 16
// (probabilities up to 2^16 are no problem for bfloat16 or for float32 sums).  When a row tops that, its warp
// waits for the P . V products issued so far, reads its 32 lanes of O, scales the rows concerned and writes
// them back (tcgen05.st): rare after the first tiles, so the loop has no pass over O and a thread keeps no
// output in registers (104 registers a thread; folding an O tile into registers every key tile took 158 and
// measured 2 % slower).  The row sum l follows the same reference; O / l at the end does not depend on it.
// Roles: warps 0-3 and 4-7 softmax and output of the two heads; warp 8 brings K tiles and warp 9 V tiles, two
// buffers each: a tile whose 128 keys all exist comes by TMA, one box per page through the block table (page
// sizes that are powers of two from 8 up); the request's last, partial tile and other page sizes are gathered
// with cp.async, zero-filling keys beyond the request.  Warps 10 and 11 issue the MMAs, one lane each, one
// warp per head: the tensor core is fed by single threads, and two instruction streams feed it twice as fast.
// Warp 10 also allocates tensor memory.  The second head starts half a tile behind the first, so that one
// head's exponentials run while the other scans for its row maxima.  P is double buffered: after a thread has
// handed P_j over it never waits for P_j . V; the tensor core computes Q . K_{j+1}^T first, then P_j . V, while
// the thread starts on S_{j+1}.  The softmax warps (one a scheduler and head) are the bound: trading ex2 for a
// polynomial on the FMA pipe, or pairs of float32 operations for the packed f32x2 forms, measured no faster.
// One block per SM (225 KiB of shared memory, 384 columns of tensor memory in use).  Tensor memory is taken only
// after the kernel ahead in the stream has finished.  Every wait on an mbarrier is bounded; after the limit
// the block sets TKB_STATUS_WAIT_TIMEOUT and leaves.
#include "tcgen05.cuh"

using namespace tkb5;

namespace {

constexpr int HD = 64;
constexpr int BQ = 128;   // queries per block
constexpr int BKV = 128;  // keys per tile
constexpr int THREADS = 384;
constexpr int Q_BYTES = BQ * HD * 2;    // 16 KiB
constexpr int KV_BYTES = BKV * HD * 2;  // 16 KiB
constexpr int P_BYTES = BQ * BKV * 2;   // 32 KiB: two [128 x 64] atoms
constexpr int SMEM_BYTES = 2 * Q_BYTES + 2 * KV_BYTES + 2 * KV_BYTES + 4 * P_BYTES + 1024;
constexpr uint32_t TMEM_COLS = 512;     // S of head 0, S of head 1 (128 columns each), O of each head (64 of 128)
constexpr uint32_t TMEM_S = 0, TMEM_O = 256;
constexpr float NEG_BIG = -1.0e30f;

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
// tcgen05.ld of 32 columns without the wait: several may be in flight before tmem_wait()
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

constexpr float REF_SLACK = 16.f;  // a row's reference moves when a score tops it by more than this (log2)

// MN-major operand (V as [key][64]): rows of 128 bytes, 8-key groups 1,024 bytes apart
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// One 128-key tile of K or V of one kv head into a swizzled [128 x 64] tile; keys outside [key_lo, key_hi) are
// zero.  A warp's lane takes rows lane, lane+32, lane+64, lane+96: the four page lookups go out together.
__device__ __forceinline__ void gather_tile(uint32_t dst, const bf16* __restrict__ cache, const int* __restrict__ table,
                                            int kvh, int nkv, int ps, int ps_shift, int key_base, int key_lo, int key_hi,
                                            int lane, int num_pages, bool& bad_page) {
  size_t off[4];
  bool valid[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
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
  for (int i = 0; i < 4; i++) {
    const int r = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < 8; c++) cp_async16(dst + r * 128 + ((c ^ (r & 7)) << 4), cache + off[i] + c * 8, valid[i]);
  }
}

// Row maximum of one thread's 128 scores in tensor memory.  The loops over column blocks stay rolled on purpose:
// the softmax warps run this code once per key tile, and unrolled it no longer fits the instruction cache.
template <bool MASKED>
__device__ __forceinline__ float row_max(uint32_t s_addr, int lo, uint32_t span) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll 1
  for (int c0 = 0; c0 < BKV; c0 += 64) {
    uint32_t a[32], b[32];
    tmem_ld32_issue(s_addr + c0, a);
    tmem_ld32_issue(s_addr + c0 + 32, b);
    tmem_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0 = __uint_as_float(a[i]), x1 = __uint_as_float(a[i + 1]);
      float y0 = __uint_as_float(b[i]), y1 = __uint_as_float(b[i + 1]);
      if (MASKED) {
        const int c = c0 + i - lo;
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
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// 32 columns of one row: p = 2^(s * scale - m) as bfloat16 into the row's place of the swizzled P tile; returns
// the sum of the even columns and adds that of the odd ones to `odd`.
template <bool MASKED>
__device__ __forceinline__ float exp_32_columns(const uint32_t (&v)[32], unsigned char* prow, int r, int c0, int lo,
                                                uint32_t span, float scale, float neg_m, float& odd) {
  float s0 = 0.f, s1 = 0.f;
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float x0 = __uint_as_float(v[i]), x1 = __uint_as_float(v[i + 1]);
    if (MASKED) {
      const int c = c0 + i - lo;
      if ((uint32_t)c > span) x0 = -INFINITY;
      if ((uint32_t)(c + 1) > span) x1 = -INFINITY;
    }
    const float p0 = fast_exp2(fmaf(x0, scale, neg_m)), p1 = fast_exp2(fmaf(x1, scale, neg_m));
    s0 += p0;
    s1 += p1;
    pk[i >> 1] = pack_bf16(p0, p1);
  }
  // 32 keys = four 16-byte chunks of this row in atom c0 / 64
  unsigned char* dst = prow + (c0 >> 6) * (BQ * 128);
  const int cbase = (c0 & 63) >> 3;
#pragma unroll
  for (int cc = 0; cc < 4; cc++)
    *reinterpret_cast<uint4*>(dst + (((cbase + cc) ^ (r & 7)) << 4)) =
        make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
  odd += s1;
  return s0;
}

// p = 2^(s * scale - m) of one row: bfloat16 into the row's place of the swizzled P tile; returns the row sum.
template <bool MASKED>
__device__ __forceinline__ float row_exp(uint32_t s_addr, unsigned char* prow, int r, int lo, uint32_t span, float scale,
                                         float neg_m) {
  float s0 = 0.f, s1 = 0.f;
  // 32 columns at a time; the load of the next 32 is on its way while these are worked on
  uint32_t v[32], w[32];
  tmem_ld32_issue(s_addr, v);
#pragma unroll 1
  for (int c0 = 0; c0 < BKV; c0 += 64) {
    tmem_wait();
    tmem_ld32_issue(s_addr + c0 + 32, w);
    s0 += exp_32_columns<MASKED>(v, prow, r, c0, lo, span, scale, neg_m, s1);
    tmem_wait();
    if (c0 + 64 < BKV) tmem_ld32_issue(s_addr + c0 + 64, v);
    s0 += exp_32_columns<MASKED>(w, prow, r, c0 + 32, lo, span, scale, neg_m, s1);
  }
  return s0 + s1;
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int tma_rows,
                       const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                       const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                       const int* __restrict__ page_ids, const int* __restrict__ tiles,
                       const int* __restrict__ n_tiles_ptr, int nh, int nkv, int ps, float scale_log2, int window,
                       int* __restrict__ status, int num_pages, int single) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2][2], skew;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  trigger_dependents();
  grid_dependency_wait();
  if ((int)blockIdx.y >= *n_tiles_ptr) return;
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = base;                 // two heads
  unsigned char* sK = sQ + 2 * Q_BYTES;     // two buffers
  unsigned char* sV = sK + 2 * KV_BYTES;    // two buffers
  unsigned char* sP = sV + 2 * KV_BYTES;    // two heads x two buffers
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
  // the first tile starts on a multiple of 128 keys, so that whole tiles are whole pages
  int k_begin = 0;
  if (window > 0 && pos0 - window + 1 > 0) k_begin = (pos0 - window + 1) & ~(BKV - 1);
  const int k_end = pos0 + rows_live;  // one past the last key any row of the tile sees
  const int n_kv_tiles = (k_end - k_begin + BKV - 1) / BKV;
  const int* table = page_ids + page_indptr[s];
  const int t0 = seq_q_start[s] + qt0;

  if (tid == 0) {
    for (int i = 0; i < 2; i++) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], n_heads_here);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], n_heads_here);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i][0], 1);
      mbar_init(&pv_done[i][1], 1);
    }
    mbar_init(&skew, 128);
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
#pragma unroll
    for (int c = 0; c < 8; c++) cp_async16(smem_u32(sQ + hh * Q_BYTES) + r * 128 + ((c ^ (r & 7)) << 4), src + c * 8, live);
    cp_async_wait_all();
    fence_proxy_async();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = tmem_slot;
  const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;

  if (warp == 8 || warp == 9) {
    // ---------------- loaders: warp 8 K tiles, warp 9 V tiles, two buffers each
    const bool is_v = warp == 9;
    const bf16* cache = is_v ? vcache : kcache;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    unsigned char* ring = is_v ? sV : sK;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    bool ok = true, bad_page = false;
    for (int j = 0; j < n_kv_tiles; j++) {
      const int b = j & 1;
      const int key_base = k_begin + j * BKV;
      if (j >= 2 && !mbar_wait_idle(&empty[b], ((j >> 1) - 1) & 1)) { ok = false; break; }
      if (tma_rows > 0 && key_base + BKV <= kv_len) {
        // every key of the tile exists: one box per page (or per 128 slots of a larger page)
        if (lane == 0) mbar_expect_tx(&full[b], KV_BYTES);
        __syncwarp();
        if (lane * tma_rows < BKV) {
          const int key = key_base + lane * tma_rows;
          // an id beyond the pool becomes -1: a negative row is outside the tensor map and reads as zeros
          const int row = (checked_page(__ldg(table + (key >> ps_shift)), num_pages, bad_page) * nkv + kvh) * ps + (key & (ps - 1));
          tma_load_2d(ring + b * KV_BYTES + lane * tma_rows * 128, map, &full[b], 0, row);
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
      // ---------------- MMA issuer of head hh: QK_0; then for every tile: (wait P_j) QK_{j+1}, P_j . V
      // All operand descriptors are made once; a k step adds its byte offset (in 16-byte units) to the address field.
      const uint32_t idesc_qk = make_idesc(BQ, BKV);
      const uint32_t idesc_pv = make_idesc(BQ, HD) | (1u << 16);  // B operand MN-major
      const uint64_t desc_q = make_desc(smem_u32(sQ + hh * Q_BYTES));
      const uint64_t desc_k0 = make_desc(smem_u32(sK)), desc_v0 = make_desc_mn(smem_u32(sV));
      const uint64_t desc_p0 = make_desc(smem_u32(sP + (hh * 2) * P_BYTES));
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int kb = j & 1;
        if (!mbar_wait_idle(&k_full[kb], (j >> 1) & 1)) return false;
        tcgen05_fence_after();
        const uint64_t dk = desc_k0 + (uint64_t)(kb * (KV_BYTES / 16));
#pragma unroll
        for (int k = 0; k < HD / UMMA_K; k++)
          umma(tmem + TMEM_S + hh * 128, desc_q + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, k > 0 ? 1u : 0u);
        tcgen05_commit(&k_empty[kb]);
        tcgen05_commit(&s_full[hh]);
        return true;
      };
      ok = issue_qk(0);
      for (int j = 0; j < n_kv_tiles && ok; j++) {
        const int vb = j & 1;
        if (!mbar_wait_idle(&p_full[hh], j & 1)) { ok = false; break; }
        if (j + 1 < n_kv_tiles && !issue_qk(j + 1)) { ok = false; break; }
        if (!mbar_wait_idle(&v_full[vb], (j >> 1) & 1)) { ok = false; break; }
        tcgen05_fence_after();
        const uint64_t dp = desc_p0 + (uint64_t)(vb * (P_BYTES / 16)), dv = desc_v0 + (uint64_t)(vb * (KV_BYTES / 16));
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; k++)
          umma(tmem + TMEM_O + hh * 128, dp + (uint64_t)((k >> 2) * (BQ * 128 / 16) + (k & 3) * 2),
                  dv + (uint64_t)(k * (2048 / 16)), idesc_pv, (k > 0 || j > 0) ? 1u : 0u);
        tcgen05_commit(&v_empty[vb]);
        tcgen05_commit(&pv_done[hh][vb]);
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
    float m = NEG_BIG, l = 0.f;  // reference of the row's exponentials (and so of O and l); row sum
    bool ok = true;
    // the second head starts when the first has handed over its first P
    if (hh == 1 && !mbar_wait(&skew, 0)) ok = false;
    for (int j = 0; j < n_kv_tiles && ok; j++) {
      const int key0 = k_begin + j * BKV;
      if (!mbar_wait(&s_full[hh], j & 1)) { ok = false; break; }
      tcgen05_fence_after();
      const bool whole = key0 + BKV - 1 <= pos0 && key0 + BKV <= k_end && (window <= 0 || key0 >= pos0 + BQ - window);
      const int lo = lim_hi >= lim_lo ? lim_lo - key0 : (1 << 30);
      const uint32_t span = lim_hi >= lim_lo ? (uint32_t)(lim_hi - lim_lo) : 0u;
      const float tile_max = (whole ? row_max<false>(s_addr, lo, span) : row_max<true>(s_addr, lo, span)) * scale_log2;
      const bool moves = tile_max - m > REF_SLACK;
      if (j == 0) {
        if (moves) m = tile_max;
      } else if (__any_sync(0xffffffffu, moves)) {
        if (!mbar_wait(&pv_done[hh][(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
        tcgen05_fence_after();
        const float m_new = moves ? fmaxf(m, tile_max) : m;
        const float alpha = fast_exp2(m - m_new);
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
        m = m_new;
      }
      if (j >= 2 && !mbar_wait(&pv_done[hh][j & 1], ((j - 2) >> 1) & 1)) { ok = false; break; }
      unsigned char* prow = sP + (hh * 2 + (j & 1)) * P_BYTES + r * 128;
      l += whole ? row_exp<false>(s_addr, prow, r, lo, span, scale_log2, -m) : row_exp<true>(s_addr, prow, r, lo, span, scale_log2, -m);
      tcgen05_fence_before();
      fence_proxy_async();
      mbar_arrive(&p_full[hh]);
      if (j == 0 && hh == 0) mbar_arrive(&skew);
    }
    if (ok) ok = mbar_wait(&pv_done[hh][(n_kv_tiles - 1) & 1], ((n_kv_tiles - 1) >> 1) & 1);
    if (!ok) failed = 1;
    if (ok) {
      tcgen05_fence_after();
      uint32_t a[32], b[32];
      tmem_ld32_issue(o_addr, a);
      tmem_ld32_issue(o_addr + 32, b);
      tmem_wait();
      if (r < rows_live) {
        const float inv = 1.f / l;
        bf16* dst = out + (size_t)(t0 + r) * out_stride + (size_t)(head0 + hh) * HD;
        auto two = [&](const uint32_t (&v)[32], int i) {
          return pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
        };
#pragma unroll
        for (int c = 0; c < 4; c++) {
          *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(two(a, 8 * c), two(a, 8 * c + 2), two(a, 8 * c + 4), two(a, 8 * c + 6));
          *reinterpret_cast<uint4*>(dst + 32 + c * 8) = make_uint4(two(b, 8 * c), two(b, 8 * c + 2), two(b, 8 * c + 4), two(b, 8 * c + 6));
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
// columns h*64 .. h*64+63.  Head size 64 only; q and out row strides multiples of 8 elements (16-byte rows).
// kcache/vcache: [n_pages, nkv, ps, 64].
TKB_EXPORT int tkb_attn_prefill_tc_bf16(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                        const void* vcache, int n_pages, const int* seq_q_start, const int* seq_q_len,
                                        const int* seq_kv_len, const int* page_indptr, const int* page_ids,
                                        const int* tiles, const int* n_tiles_ptr, int tiles_cap, int nh, int nkv, int ps,
                                        float scale, int window, int single, int* status, void* st) {
  if (tiles_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0 || (q_stride & 7) || (out_stride & 7)) return -2;
  if (tiles_cap > 65535) return -3;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
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
  return launch_pdl(attn_prefill_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)st, map_k, map_v,
                    tma_rows, (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache,
                    seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, tiles, n_tiles_ptr, nh, nkv, ps,
                    scale * 1.4426950408889634f, window, status, n_pages, single ? 1 : 0);
}
