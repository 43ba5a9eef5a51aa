// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32
// accumulation; scores, softmax and the running rescale are float32).
//
//   attn_decode_mma:  one query token per request, keys split into chunks (work items (request, first key,
//                     keys) built on the host); the last block of a request to finish merges the partial
//                     results (an arrival counter; nobody waits), or attn_decode_merge does for callers
//                     without counters.  The 16 rows of the MMA tile are the query heads that share one
//                     key/value head, so every key and value is read once for the whole group.
//   attn_prefill_mma: portions of prompts; a block owns 64 consecutive query tokens of one head
//                     (16 per warp) and walks the keys they may see.
//
// Compile with -DTKB_HD=<head size> (multiple of 16, at most 256).
//
// Keys and values reach shared memory page by page through the request's block table, two or three stages
// deep.  In the split-key kernel a tile whose 64 keys all exist comes by TMA (head sizes that are multiples
// of 64, page sizes that are powers of two from 8 up, items that start on a tile boundary and are longer than
// the pipeline): one warp asks for one box a page and 64-column block and an mbarrier counts the bytes, so
// no thread works out addresses or issues copies of its own.  That was what bounded the loop: with two or
// three blocks of four warps an SM, the 16 cp.async a thread and tile and their address arithmetic were a
// third of a warp's instructions (measured at head size 128, 64 requests at context 8,192: 505 us gathered,
// 367 us by TMA, 0.88 of the HBM roofline).  Everything else (the request's last, partial tile, other head and
// page sizes, the kernel for portions) is gathered with 16-byte cp.async copies; rows outside the request's
// keys are zero-filled, so nothing that an earlier owner of a page left behind can reach a sum.  Tiles of
// head sizes that are multiples of 64 lie in shared memory as the TMA leaves them (128-byte swizzle); rows of
// other head sizes are padded by 16 bytes; both keep ldmatrix free of bank conflicts.
#include "tcgen05.cuh"
#include <float.h>

#ifndef TKB_HD
#error "compile with -DTKB_HD=<head size>"
#endif
static_assert(TKB_HD % 16 == 0 && TKB_HD >= 16 && TKB_HD <= 256, "head size must be a multiple of 16 up to 256");

using namespace tkb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int HD = TKB_HD;
constexpr int KT = 64;                // keys per shared-memory tile
// Layout of a K or V tile in shared memory.  Head sizes that are multiples of 64: blocks of 64 columns, each
// [KT rows x 128 bytes] with the 128-byte swizzle (16-byte chunk c of row r lies at chunk c ^ (r & 7)), which is
// what a TMA box leaves and keeps ldmatrix free of bank conflicts.  Other head sizes: rows padded by 16 bytes.
constexpr bool SWZ = HD % 64 == 0;
constexpr int ROWB = SWZ ? 128 : HD * 2 + 16;  // bytes from one row to the next
constexpr int CPR = HD / 8;                    // 16-byte chunks per row
constexpr int ATOM_B = KT * 128;               // one 64-column block (swizzled layout)
constexpr int TILE_B = SWZ ? KT * HD * 2 : KT * ROWB;  // bytes of one K or V tile
constexpr int STAGE_B = 2 * TILE_B;   // K tile then V tile
constexpr int SMEM_ALIGN = SWZ ? 1024 : 128;   // the swizzle pattern repeats every 1,024 bytes
constexpr int SMEM_B = 2 * STAGE_B + SMEM_ALIGN;  // two stages (tiled kernel for portions)
// The split-key kernel: three stages where they leave room for two or three blocks an SM (three at head sizes
// to 80, two to 128), else two.  Four stages at head size 64 were measured slower, with padded rows (the
// blocks of a step then no longer fit the SMs all at once) and again with the swizzled layout, where three
// blocks of 65 KiB should fit an SM (batch 64: 38 k -> 30 k tok/s; batch 8 unchanged).
#ifdef TKB_DSTAGES
constexpr int DSTAGES = TKB_DSTAGES;  // a deeper ring for one block an SM (see the planner's "deep" steps)
#else
constexpr int DSTAGES = 3 * STAGE_B <= 110 * 1024 ? 3 : 2;
#endif
static_assert(DSTAGES >= 2 && DSTAGES * STAGE_B <= 200 * 1024, "the ring must fit an SM's shared memory");
constexpr int DEC_SMEM_B = DSTAGES * STAGE_B + SMEM_ALIGN;
static_assert(4 * 16 * (HD + 8 + 2) * 4 <= DSTAGES * STAGE_B, "the warps' partial results are combined in the ring's memory");
// byte offset of 16-byte chunk `chunk` of row `row` within a tile
__device__ __forceinline__ int tile_off(int row, int chunk) {
  return SWZ ? (chunk >> 3) * ATOM_B + row * 128 + (((chunk & 7) ^ (row & 7)) << 4) : row * ROWB + chunk * 16;
}
__device__ __forceinline__ unsigned char* align_smem(unsigned char* p) {
  return reinterpret_cast<unsigned char*>(((uintptr_t)p + (SMEM_ALIGN - 1)) & ~(uintptr_t)(SMEM_ALIGN - 1));
}
constexpr int KSTEPS = HD / 16;       // k-steps of Q.K^T
constexpr int DTILES = HD / 8;        // n-tiles of P.V
constexpr float NEG_BIG = -1.0e30f;   // finite stand-in for -inf in running maxima

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit, one instruction (denormal results flush to zero, which is what a
// softmax weight that small is worth)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy keys [key_base, key_base + KT) of one kv head into a stage; keys outside [key_lo, key_hi) become zero.
// In two halves, so that a caller may look the pages up an iteration before it issues the copies (a lookup is a
// load that the copies' addresses depend on: done together, its latency is paid in every iteration).
template <int NTHREADS>
struct KvTileLoad {
  static constexpr int ITERS = (KT * CPR + NTHREADS - 1) / NTHREADS;
  int page[ITERS];  // page of each row this thread copies; -1: the row is outside the keys wanted

  __device__ __forceinline__ void lookup(const int* __restrict__ table, int ps, int key_base, int key_lo, int key_hi,
                                         int tid) {
    const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;  // page sizes that are powers of two: shifts
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
      const int idx = tid + i * NTHREADS;
      const int key = key_base + idx / CPR;
      page[i] = -1;
      // (checked against the pool in issue(), when the value is needed: a check here would wait for the load)
      if (idx < KT * CPR && key >= key_lo && key < key_hi) page[i] = table[ps_shift >= 0 ? key >> ps_shift : key / ps];
    }
  }
  __device__ __forceinline__ void issue(unsigned char* stage, const bf16* __restrict__ kcache,
                                        const bf16* __restrict__ vcache, int kvh, int nkv, int ps, int key_base,
                                        int tid, int num_pages, bool& bad_page) const {
    const uint32_t sk = smem_u32(stage), sv = sk + TILE_B;
    const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
      const int idx = tid + i * NTHREADS;
      if (idx < KT * CPR) {
        const int r = idx / CPR, c = idx - r * CPR;
        const int key = key_base + r;
        const int slot = ps_shift >= 0 ? key & (ps - 1) : key % ps;
        const int pg = checked_page(page[i], num_pages, bad_page);
        const bool valid = pg >= 0;
        const size_t off = valid ? (((size_t)pg * nkv + kvh) * ps + slot) * HD + c * 8 : 0;
        const uint32_t d = tile_off(r, c);
        cp_async16(sk + d, kcache + off, valid);
        cp_async16(sv + d, vcache + off, valid);
      }
    }
  }
};

template <int NTHREADS>
__device__ __forceinline__ void load_kv_tile(unsigned char* stage, const bf16* __restrict__ kcache,
                                             const bf16* __restrict__ vcache, const int* __restrict__ table, int kvh,
                                             int nkv, int ps, int key_base, int key_lo, int key_hi, int tid,
                                             int num_pages, bool& bad_page) {
  KvTileLoad<NTHREADS> t;
  t.lookup(table, ps, key_base, key_lo, key_hi, tid);
  t.issue(stage, kcache, vcache, kvh, nkv, ps, key_base, tid, num_pages, bad_page);
}

// S[16 x 16 keys] = Q . K^T for the 16 key rows starting at key_row of the K tile.  s[nt][4], nt = 0, 1.
__device__ __forceinline__ void qk_16keys(float (&s)[2][4], const uint32_t (&qf)[KSTEPS][4], uint32_t k_tile,
                                          int key_row, int lane) {
#pragma unroll
  for (int nt = 0; nt < 2; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) s[nt][i] = 0.f;
  const int row = key_row + (lane & 7) + ((lane >> 4) << 3);
  const int chunk_sel = (lane >> 3) & 1;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ks++) {
    uint32_t b0, b1, b2, b3;
    ldmatrix_x4(b0, b1, b2, b3, k_tile + tile_off(row, ks * 2 + chunk_sel));
    mma_bf16(s[0], qf[ks], b0, b1);
    mma_bf16(s[1], qf[ks], b2, b3);
  }
}

// O[16 x HD] += P[16 x 16 keys] . V for the 16 key rows starting at key_row of the V tile.
__device__ __forceinline__ void pv_16keys(float (&o)[DTILES][4], const uint32_t (&pf)[4], uint32_t v_tile, int key_row,
                                          int lane) {
  const int row = key_row + (lane & 7) + (((lane >> 3) & 1) << 3);
  const int chunk_sel = lane >> 4;
#pragma unroll
  for (int dt = 0; dt < DTILES; dt += 2) {
    uint32_t b0, b1, b2, b3;
    ldmatrix_x4_trans(b0, b1, b2, b3, v_tile + tile_off(row, dt + chunk_sel));
    mma_bf16(o[dt], pf, b0, b1);
    mma_bf16(o[dt + 1], pf, b2, b3);
  }
}

// Online softmax over a 16-row x 16-key block held as s[2][4] (rows lane/4 and lane/4 + 8).
// lim_lo/lim_hi: per-row inclusive key limits; key0: key index of the block's first column.
__device__ __forceinline__ void softmax_16keys(float (&s)[2][4], float (&m)[2], float (&l)[2], float (&alpha)[2],
                                               uint32_t (&pf)[4], const int (&lim_lo)[2], const int (&lim_hi)[2],
                                               int key0, float scale_log2, int lane) {
  const int c0 = key0 + (lane & 3) * 2;
#pragma unroll
  for (int h = 0; h < 2; h++) {  // h: row half (rows r and r + 8)
    float mx = NEG_BIG;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int key = c0 + nt * 8 + e;
        float v = s[nt][h * 2 + e] * scale_log2;
        if (key < lim_lo[h] || key > lim_hi[h]) v = -INFINITY;
        s[nt][h * 2 + e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    alpha[h] = fast_exp2(m[h] - m_new);
    m[h] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const float p = fast_exp2(s[nt][h * 2 + e] - m_new);
        s[nt][h * 2 + e] = p;
        sum += p;
      }
    l[h] = l[h] * alpha[h] + sum;  // per-thread partial; the four threads of a row are summed at the end
  }
  pf[0] = pack_bf16(s[0][0], s[0][1]);
  pf[1] = pack_bf16(s[0][2], s[0][3]);
  pf[2] = pack_bf16(s[1][0], s[1][1]);
  pf[3] = pack_bf16(s[1][2], s[1][3]);
}

// ------------------------------------------------------------------------------------------------
// Two neighbouring output elements (d, d + 1) of the merge of splits i0 .. i1-1 of one head.  All loads of up
// to eight splits are in flight together (one trip to the L2 for the usual case); the sums run in split order,
// so every caller gets the same bits.
__device__ __forceinline__ float2 merge_splits(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               int i0, int i1, int nh, int head, int d) {
  const float* ml = part_ml + ((size_t)i0 * nh + head) * 2;
  const float* po = part_o + ((size_t)i0 * nh + head) * HD + d;
  const size_t ml_step = (size_t)nh * 2, po_step = (size_t)nh * HD;
  const int n = i1 - i0;
  float2 mlv[8], ov[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const bool live = k < n;
    mlv[k] = live ? __ldcg(reinterpret_cast<const float2*>(ml + (size_t)k * ml_step)) : make_float2(NEG_BIG, 0.f);
    ov[k] = live ? __ldcg(reinterpret_cast<const float2*>(po + (size_t)k * po_step)) : make_float2(0.f, 0.f);
  }
  float mm = NEG_BIG;
#pragma unroll
  for (int k = 0; k < 8; k++) mm = fmaxf(mm, mlv[k].x);
  for (int k = 8; k < n; k++) mm = fmaxf(mm, __ldcg(ml + (size_t)k * ml_step));
  float ax = 0.f, ay = 0.f, ll = 0.f;
#pragma unroll
  for (int k = 0; k < 8; k++) {
    if (k < n) {
      const float f = exp2f(mlv[k].x - mm);
      ll += f * mlv[k].y;
      ax += f * ov[k].x;
      ay += f * ov[k].y;
    }
  }
  for (int k = 8; k < n; k++) {
    const float2 e = __ldcg(reinterpret_cast<const float2*>(ml + (size_t)k * ml_step));
    const float2 o = __ldcg(reinterpret_cast<const float2*>(po + (size_t)k * po_step));
    const float f = exp2f(e.x - mm);
    ll += f * e.y;
    ax += f * o.x;
    ay += f * o.y;
  }
  return make_float2(ax / ll, ay / ll);
}

// ------------------------------------------------------------------------------------------------
// Decode: blockIdx.x = work item (request row, split), blockIdx.y = kv head * head_tiles + head tile.
// FUSED: q points at the un-rotated q|k|v rows of the step [tokens, (nh + 2 nkv) * HD]; the kernel rotates
// q on the fly, and the block that owns the split holding the token's own position rotates this kv
// head's k, writes it and v into the cache page, and only then reads its tiles.
// The TMA descriptors of the K and V cache as a kernel parameter: two of them for the instantiation that uses
// them, nothing for the other (256 bytes of parameters less to hand to every launch).
template <bool TMA>
struct KvMapsParam {
  CUtensorMap k, v;
};
template <>
struct KvMapsParam<false> {};

template <bool FUSED, bool TMA>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(const __grid_constant__ KvMapsParam<TMA> maps, int tma_rows,
                       const bf16* __restrict__ q, int q_stride, bf16* __restrict__ kcache,
                       bf16* __restrict__ vcache, const int* __restrict__ seq_q_start,
                       const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                       const int* __restrict__ page_ids, const int* __restrict__ items,
                       const int* __restrict__ n_items_ptr, float* __restrict__ part_o, float* __restrict__ part_ml,
                       int nh, int nkv, int ps, float scale_log2, int window, int head_tiles,
                       const float* __restrict__ inv_freq, int rot, int write_cache, int num_pages,
                       int* __restrict__ status, const float* __restrict__ qkv_parts, int n_parts,
                       long long part_stride, int* __restrict__ counters, const int* __restrict__ item_entry,
                       const int* __restrict__ dec_item_start, const int* __restrict__ out_row_of,
                       bf16* __restrict__ out, int out_stride, const float* __restrict__ qkv_bias,
                       const float* __restrict__ qk_norm_w, float norm_eps) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = align_smem(smem_raw);
  trigger_dependents();
  // What the host wrote for this step (work items, lengths, block tables) is there before any kernel of the
  // step starts, so the block works out its geometry while the kernel ahead (the q|k|v product) still runs.
  const int item = blockIdx.x;
  if (item >= *n_items_ptr) return;
  const int s = items[3 * item];  // work item: request row, first key (counted from the first visible key), keys
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y - kvh * head_tiles;
  const int group = nh / nkv;
  const int g0 = ht * 16;
  const int gn = min(16, group - g0);  // live rows of the MMA tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kv_len = seq_kv_len[s];
  const int p = kv_len - 1;
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  const int k_begin = lo + items[3 * item + 1];
  const int k_end = min(kv_len, k_begin + items[3 * item + 2]);
  const int* table = page_ids + page_indptr[s];
  const int t = seq_q_start[s];
  const bf16* qrow = q + (size_t)t * q_stride + (size_t)(kvh * group + g0) * HD;
  const int n_tiles = (k_end - k_begin + KT - 1) / KT;

  // The first tiles of keys and values go on their way before anything else.  With the rotary encoding fused
  // the only key of this step is the token's own (position p), which is patched into the last tile in shared
  // memory; all older keys were written by earlier steps, so tiles that end before p may be read even before
  // the kernel ahead has finished.  Otherwise (keys of this step come from a kernel ahead) the wait comes first.
  const bool early = FUSED && (k_end < kv_len || n_tiles > DSTAGES - 1);
  // Tiles whose keys all exist come by TMA where the page size allows it (tma_rows > 0: a power of two from 8
  // up) and the item starts on a tile boundary: warp 0 asks for one box a page and 64-column block, nobody
  // computes an address or issues a copy of its own; the tile's arrival is counted by an mbarrier.  The
  // request's last, partial tile and everything else is gathered with cp.async, zero-filling what lies outside.
  __shared__ __align__(8) uint64_t kv_full[DSTAGES];
  const bool use_tma = TMA && SWZ && tma_rows > 0 && (k_begin & (KT - 1)) == 0 && n_tiles > DSTAGES;  // short items gain nothing
  const int ps_shift = 31 - __clz(ps);  // used with TMA only (page sizes that are powers of two)
  bool bad_page = false;  // a page id beyond the pool was met (its keys read as zeros); reported once, at the end
  auto by_tma = [&](int tile) { return use_tma && k_begin + (tile + 1) * KT <= kv_len; };
  // warp 0: the page of the box that this lane asks for (lanes beyond the tile's boxes ask for nothing)
  const int tma_boxes = use_tma ? KT / tma_rows : 1;
  const int tma_atom = lane / tma_boxes, tma_box = lane - tma_atom * tma_boxes;
  const bool tma_lane = use_tma && warp == 0 && tma_atom < HD / 64;
  auto tma_lookup = [&](int tile) {
    return tma_lane ? table[(k_begin + tile * KT + tma_box * tma_rows) >> ps_shift] : 0;
  };
  auto tma_issue = [&](int tile, int page) {  // warp 0, all lanes
    unsigned char* stage = smem + (tile % DSTAGES) * STAGE_B;
    uint64_t* bar = &kv_full[tile % DSTAGES];
    if (lane == 0) tkb5::mbar_expect_tx(bar, STAGE_B);
    __syncwarp();
    if (tma_lane) {
      const int key = k_begin + tile * KT + tma_box * tma_rows;
      // an id beyond the pool becomes -1: a negative row lies outside the tensor map and reads as zeros
      const int row = (checked_page(page, num_pages, bad_page) * nkv + kvh) * ps + (key & (ps - 1));
      unsigned char* dst = stage + tma_atom * ATOM_B + tma_box * tma_rows * 128;
      if constexpr (TMA) {
        tkb5::tma_load_2d(dst, &maps.k, bar, tma_atom * 64, row);
        tkb5::tma_load_2d(dst + TILE_B, &maps.v, bar, tma_atom * 64, row);
      }
    }
  };
  if (use_tma) {
    if (tid == 0) {
#pragma unroll
      for (int i = 0; i < DSTAGES; i++) tkb5::mbar_init(&kv_full[i], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }
  if (!early) grid_dependency_wait();
#pragma unroll
  for (int st = 0; st < DSTAGES - 1; st++) {
    if (st < n_tiles) {
      if (by_tma(st)) {
        if (warp == 0) tma_issue(st, tma_lookup(st));
      } else {
        load_kv_tile<128>(smem + st * STAGE_B, kcache, vcache, table, kvh, nkv, ps, k_begin + st * KT, k_begin, k_end, tid,
                          num_pages, bad_page);
      }
    }
    cp_async_commit();
  }
  // Q fragments: row r of the tile is query head g0 + r; rows >= gn are zero.
  uint32_t qf[KSTEPS][4];
  // What the fused form needs only until the key loop starts lives in the ring's LAST stage, which no tile enters
  // before the loop's first iteration: the token's q rows of this head tile, then its k and v row (float32,
  // srow[18][HD]); the rotated q as bfloat16 pairs (sq, rows 4 words longer than the head); cos and sin of the
  // token's position (cs).  As static shared memory these 7 KiB cost the fourth block an SM, and with it a quarter
  // of the speed of steps whose work items outnumber three blocks an SM (batch 64: 38 k -> 30 k tok/s).
  constexpr int SQ_STRIDE = HD / 2 + 4;  // words (two bfloat16 each) from one row of sq to the next
  static_assert(!FUSED || (18 * HD + 16 * SQ_STRIDE + HD) * 4 <= STAGE_B, "the fused prologue's scratch must fit one stage");
  unsigned char* pro = smem + (DSTAGES - 1) * STAGE_B;
  float* srow = reinterpret_cast<float*>(pro);
  uint32_t* sq = reinterpret_cast<uint32_t*>(pro + 18 * HD * 4);
  float* cs = reinterpret_cast<float*>(pro + 18 * HD * 4 + 16 * SQ_STRIDE * 4);
  __shared__ bf16 knew[FUSED ? HD : 2], vnew[FUSED ? HD : 2];  // the token's own rotated key and its value
  // this split holds position p, and this layer call keeps its own keys (a call that reads another call's cache
  // finds the key at p already there)
  const bool owns_new = FUSED && write_cache && k_end == kv_len;
  // the page of the token's own position: looked up here, before the wait, so that the write below waits for nothing
  const int own_page = owns_new ? table[p / ps] : 0;
  if (FUSED) {
    const int half = rot >> 1;
    for (int j = tid; j < half; j += 128) {
      float sn, c;
      sincosf((float)p * inv_freq[j], &sn, &c);
      cs[j] = c;
      cs[half + j] = sn;
    }
  }
  if (early) grid_dependency_wait();
  if (FUSED) {
    const int half = rot >> 1;
    // gather q (gn heads), k and v of this kv head as the activation type would hold them
    const int C = (nh + 2 * nkv) * HD;
    if (n_parts > 0) {
      // float32 slices of a K-split product: four columns a thread, the loads of up to eight slices in flight
      // together, added in slice order
      for (int idx = tid; idx < (gn + 2) * (HD / 4); idx += 128) {
        const int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
        const int col = r < gn ? (kvh * group + g0 + r) * HD + d : (r == gn ? (nh + kvh) * HD + d : (nh + nkv + kvh) * HD + d);
        const float* src = qkv_parts + (size_t)t * C + col;
        float4 pv[8];
#pragma unroll
        for (int pi = 0; pi < 8; pi++)
          pv[pi] = pi < n_parts ? *reinterpret_cast<const float4*>(src + (size_t)pi * part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int pi = 0; pi < 8; pi++) {
          v.x += pv[pi].x;
          v.y += pv[pi].y;
          v.z += pv[pi].z;
          v.w += pv[pi].w;
        }
        for (int pi = 8; pi < n_parts; pi++) {
          const float4 e = *reinterpret_cast<const float4*>(src + (size_t)pi * part_stride);
          v.x += e.x;
          v.y += e.y;
          v.z += e.z;
          v.w += e.w;
        }
        if (qkv_bias != nullptr) {
          const float4 b = *reinterpret_cast<const float4*>(qkv_bias + col);
          v.x += b.x;
          v.y += b.y;
          v.z += b.z;
          v.w += b.w;
        }
        v.x = __bfloat162float(__float2bfloat16_rn(v.x));
        v.y = __bfloat162float(__float2bfloat16_rn(v.y));
        v.z = __bfloat162float(__float2bfloat16_rn(v.z));
        v.w = __bfloat162float(__float2bfloat16_rn(v.w));
        *reinterpret_cast<float4*>(srow + (r < gn ? r : 16 + (r - gn)) * HD + d) = v;
      }
    } else {
      for (int idx = tid; idx < (gn + 2) * HD; idx += 128) {
        const int r = idx / HD, d = idx - r * HD;
        const int col = r < gn ? (kvh * group + g0 + r) * HD + d : (r == gn ? (nh + kvh) * HD + d : (nh + nkv + kvh) * HD + d);
        float v = __bfloat162float(q[(size_t)t * q_stride + col]);
        if (qkv_bias != nullptr) v = __bfloat162float(__float2bfloat16_rn(v + qkv_bias[col]));
        srow[(r < gn ? r : 16 + (r - gn)) * HD + d] = v;
      }
    }
    __syncthreads();
    if (qk_norm_w != nullptr) {
      // the element-wise stage a mixer may ask for: every q head and the k head RMS-normalised over the head size
      for (int r = warp; r < gn + 1; r += 4) {
        float* x = srow + (r < gn ? r : 16) * HD;
        const float* w = qk_norm_w + (r < gn ? 0 : HD);
        float ss = 0.f;
        for (int d = lane; d < HD; d += 32) ss += x[d] * x[d];
        ss = warp_sum(ss);
        const float sc = rsqrtf(ss / (float)HD + norm_eps);
        for (int d = lane; d < HD; d += 32) x[d] = __bfloat162float(__float2bfloat16_rn(x[d] * sc * w[d]));
      }
      __syncthreads();
    }
    if (owns_new) {
      // this block's split holds position p: rotate the token's own key, keep it and the value for the patch
      // of the tile, and store them in the cache page for later steps (blocks of other head tiles of the
      // same kv head store the same bytes)
      const float* krow = srow + 16 * HD;
      const float* vrow = srow + 17 * HD;
      const int page = own_page;
      const bool page_ok = page >= 0 && page < num_pages;
      if (!page_ok && tid == 0) atomicOr(status, TKB_STATUS_BAD_PAGE);
      const size_t dst = (((size_t)(page_ok ? page : 0) * nkv + kvh) * ps + (p % ps)) * HD;
      for (int d = tid; d < HD; d += 128) {
        float kv = krow[d];
        if (d < half) kv = kv * cs[d] - krow[d + half] * cs[half + d];
        else if (d < rot) kv = kv * cs[d - half] + krow[d - half] * cs[d];
        const bf16 kb = __float2bfloat16_rn(kv), vb = __float2bfloat16_rn(vrow[d]);
        knew[d] = kb;
        vnew[d] = vb;
        if (page_ok) {
          kcache[dst + d] = kb;
          vcache[dst + d] = vb;
        }
      }
    }
  }
  // Fused: the q rows are rotated ONCE, by all threads together, into a bfloat16 tile in shared memory whose rows
  // are 4 words longer than the head, so that the fragment loads below (eight rows a warp instruction) fall into
  // 32 different banks.  (Each thread rotating the fragments it needs straight from the float32 rows cost 1.5 us
  // of a 17 us kernel: sixteen times the arithmetic, and every load an eight-way bank conflict.)
  if (FUSED) {
    const int half = rot >> 1;
    for (int idx = tid; idx < gn * (HD / 2); idx += 128) {
      const int row = idx / (HD / 2), col = (idx - row * (HD / 2)) * 2;
      const float* src = srow + row * HD;
      float2 x = *reinterpret_cast<const float2*>(src + col);
      if (col < rot) {
        const bool low = col < half;
        const int pc = low ? col + half : col - half;   // partner column
        const int j = low ? col : col - half;           // angle index
        const float2 y = *reinterpret_cast<const float2*>(src + pc);
        const float2 c = *reinterpret_cast<const float2*>(cs + j), sn = *reinterpret_cast<const float2*>(cs + half + j);
        x = low ? make_float2(x.x * c.x - y.x * sn.x, x.y * c.y - y.y * sn.y)
                : make_float2(x.x * c.x + y.x * sn.x, x.y * c.y + y.y * sn.y);
      }
      sq[row * SQ_STRIDE + (col >> 1)] = pack_bf16(x.x, x.y);
    }
    __syncthreads();
  }
  {
    const int r = lane >> 2, cq = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int row = r + (i & 1) * 8, col = ks * 16 + cq + (i >> 1) * 8;
        uint32_t v = 0u;
        if (row < gn)
          v = FUSED ? sq[row * SQ_STRIDE + (col >> 1)] : *reinterpret_cast<const uint32_t*>(qrow + (size_t)row * HD + col);
        qf[ks][i] = v;
      }
    }
  }
  float o[DTILES][4];
#pragma unroll
  for (int dt = 0; dt < DTILES; dt++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[dt][i] = 0.f;
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  const int lim_lo[2] = {k_begin, k_begin}, lim_hi[2] = {k_end - 1, k_end - 1};

  // the pages of the tile that the loop's first iteration sends for; from then on each iteration looks up the
  // pages of the tile that the next one sends for, so that no iteration waits for a lookup
  KvTileLoad<128> ahead;
  int ahead_page = 0;
  auto look_ahead = [&](int tile) {
    if (tile >= n_tiles) return;
    if (by_tma(tile)) ahead_page = tma_lookup(tile);
    else ahead.lookup(table, ps, k_begin + tile * KT, k_begin, k_end, tid);
  };
  look_ahead(DSTAGES - 1);
  bool timed_out = false;
  for (int it = 0; it < n_tiles; it++) {
    unsigned char* cur = smem + (it % DSTAGES) * STAGE_B;
    cp_async_wait<DSTAGES - 2>();
    if (by_tma(it) && !tkb5::mbar_wait(&kv_full[it % DSTAGES], (it / DSTAGES) & 1)) timed_out = true;
    __syncthreads();  // tile `it` is there for every warp, and every warp is through with tile it - 1
    {
      const int nxt = it + DSTAGES - 1;  // into the stage that tile it - 1 has just left
      if (nxt < n_tiles) {
        if (by_tma(nxt)) {
          if (warp == 0) tma_issue(nxt, ahead_page);
        } else {
          ahead.issue(smem + (nxt % DSTAGES) * STAGE_B, kcache, vcache, kvh, nkv, ps, k_begin + nxt * KT, tid, num_pages,
                      bad_page);
        }
      }
      cp_async_commit();
      look_ahead(nxt + 1);
    }
    if (owns_new && it == n_tiles - 1) {
      // the tile came from the cache as it was before this step: put the token's own key and value in
      const int row = p - (k_begin + it * KT);
      for (int d = tid; d < HD; d += 128) {
        const int at = tile_off(row, d >> 3) + (d & 7) * 2;
        *reinterpret_cast<bf16*>(cur + at) = knew[d];
        *reinterpret_cast<bf16*>(cur + TILE_B + at) = vnew[d];
      }
      __syncthreads();
    }
    const int key0 = k_begin + it * KT + warp * 16;
    if (key0 < k_end) {  // warp-uniform: this warp's 16 keys hold at least one live key
      float sc[2][4], alpha[2];
      uint32_t pf[4];
      qk_16keys(sc, qf, smem_u32(cur), warp * 16, lane);
      softmax_16keys(sc, m, l, alpha, pf, lim_lo, lim_hi, key0, scale_log2, lane);
#pragma unroll
      for (int dt = 0; dt < DTILES; dt++) {
        o[dt][0] *= alpha[0];
        o[dt][1] *= alpha[0];
        o[dt][2] *= alpha[1];
        o[dt][3] *= alpha[1];
      }
      pv_16keys(o, pf, smem_u32(cur) + TILE_B, warp * 16, lane);
    }
  }
  cp_async_wait<0>();
  if (timed_out && status != nullptr) atomicOr(status, TKB_STATUS_WAIT_TIMEOUT);
  report_bad_page(bad_page, status);
  __syncthreads();
  // row sums over the four threads of a row
#pragma unroll
  for (int h = 0; h < 2; h++) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  // combine the four warps through shared memory: so[warp][row][HD + 8], sml[warp][row][2]; the rows are 8 words
  // longer than the head so that the 8-byte stores of a half-warp (four rows, four column pairs) hit 32 banks
  constexpr int SO = HD + 8;
  float* so = reinterpret_cast<float*>(smem);
  float* sml = so + 4 * 16 * SO;
  {
    const int r = lane >> 2, cq = (lane & 3) * 2;
#pragma unroll
    for (int dt = 0; dt < DTILES; dt++) {
      float* b = so + ((warp * 16 + r) * SO) + dt * 8 + cq;
      *reinterpret_cast<float2*>(b) = make_float2(o[dt][0], o[dt][1]);
      *reinterpret_cast<float2*>(b + 8 * SO) = make_float2(o[dt][2], o[dt][3]);
    }
    if ((lane & 3) == 0) {
      sml[(warp * 16 + r) * 2] = m[0];
      sml[(warp * 16 + r) * 2 + 1] = l[0];
      sml[(warp * 16 + r + 8) * 2] = m[1];
      sml[(warp * 16 + r + 8) * 2 + 1] = l[1];
    }
  }
  __syncthreads();
  // With `counters` the merge of the splits happens here too: the block that finishes last for its
  // (request, kv head, head tile) adds up all splits in split order; a request with one split is finished
  // by its only block.  Without `counters` the partial results are left for attn_decode_merge_kernel.
  int e = 0, i0 = 0, i1 = 0;
  if (counters != nullptr) {
    e = item_entry[item];
    i0 = dec_item_start[e];
    i1 = dec_item_start[e + 1];
  }
  const bool single = counters != nullptr && i1 - i0 == 1;
  for (int idx = tid; idx < gn * HD; idx += 128) {
    const int r = idx / HD, d = idx - r * HD;
    float mm = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; w++) mm = fmaxf(mm, sml[(w * 16 + r) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float f = exp2f(sml[(w * 16 + r) * 2] - mm);
      acc += f * so[(w * 16 + r) * SO + d];
      ll += f * sml[(w * 16 + r) * 2 + 1];
    }
    const int head = kvh * group + g0 + r;
    if (single) {
      out[(size_t)out_row_of[s] * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc / ll);
      continue;
    }
    part_o[((size_t)item * nh + head) * HD + d] = acc;
    if (d == 0) {
      part_ml[((size_t)item * nh + head) * 2] = mm;
      part_ml[((size_t)item * nh + head) * 2 + 1] = ll;
    }
  }
  if (counters == nullptr || single) return;
  __shared__ int s_last;
  __threadfence();  // this block's partial results are visible before its arrival is counted
  __syncthreads();
  if (tid == 0) {
    int* c = counters + (size_t)e * gridDim.y + blockIdx.y;
    const int prev = atomicAdd(c, 1);
    s_last = prev == i1 - i0 - 1;
    if (s_last) *c = 0;  // every block of this group has arrived: leave the counter ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const size_t orow = (size_t)out_row_of[s] * out_stride;
  for (int idx = tid; idx < gn * (HD / 2); idx += 128) {
    const int r = idx / (HD / 2), d = (idx - r * (HD / 2)) * 2;
    const int head = kvh * group + g0 + r;
    const float2 v = merge_splits(part_o, part_ml, i0, i1, nh, head, d);
    *reinterpret_cast<uint32_t*>(out + orow + (size_t)head * HD + d) = pack_bf16(v.x, v.y);
  }
}

// Merge the splits of each decode request: grid (request entry, head), HD threads (rounded up to 32).
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ dec_seqs, const int* __restrict__ dec_item_start,
                                         const int* __restrict__ n_dec_ptr, const int* __restrict__ seq_q_start,
                                         bf16* __restrict__ out, int out_stride, int nh) {
  trigger_dependents();
  grid_dependency_wait();
  const int e = blockIdx.x;
  if (e >= *n_dec_ptr) return;
  const int head = blockIdx.y;
  const int s = dec_seqs[e];
  const int i0 = dec_item_start[e], i1 = dec_item_start[e + 1];
  const int t = seq_q_start[s];
  for (int d = 2 * threadIdx.x; d < HD; d += 2 * blockDim.x) {
    const float2 v = merge_splits(part_o, part_ml, i0, i1, nh, head, d);
    *reinterpret_cast<uint32_t*>(out + (size_t)t * out_stride + (size_t)head * HD + d) = pack_bf16(v.x, v.y);
  }
}

// ------------------------------------------------------------------------------------------------
// Prefill: blockIdx.x = tile (request row, first query of the tile within the portion), blockIdx.y = head.
__global__ void __launch_bounds__(128)
attn_prefill_mma_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                        const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                        const int* __restrict__ page_ids, const int* __restrict__ tiles,
                        const int* __restrict__ n_tiles_ptr, int nh, int nkv, int ps, float scale_log2, int window,
                        int num_pages, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = align_smem(smem_raw);
  trigger_dependents();
  grid_dependency_wait();
  if ((int)blockIdx.x >= *n_tiles_ptr) return;
  const int s = tiles[2 * blockIdx.x], qt0 = tiles[2 * blockIdx.x + 1];
  const int head = blockIdx.y;
  const int kvh = head / (nh / nkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q_len = seq_q_len[s], kv_len = seq_kv_len[s];
  const int rows_live = min(64, q_len - qt0);
  const int pos0 = kv_len - q_len + qt0;  // position of the tile's first query
  const int pos_last = pos0 + rows_live - 1;
  int k_begin = 0;
  if (window > 0 && pos0 - window + 1 > 0) k_begin = pos0 - window + 1;
  const int k_end = pos_last + 1;
  const int* table = page_ids + page_indptr[s];
  const int t0 = seq_q_start[s] + qt0;

  // this warp's rows: r and r + 8 of its 16
  const int r = lane >> 2, cq = (lane & 3) * 2;
  const int row_a = warp * 16 + r, row_b = row_a + 8;
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int row = (i & 1) ? row_b : row_a, col = ks * 16 + cq + (i >> 1) * 8;
      qf[ks][i] = row < rows_live
                      ? *reinterpret_cast<const uint32_t*>(q + (size_t)(t0 + row) * q_stride + (size_t)head * HD + col)
                      : 0u;
    }
  }
  float o[DTILES][4];
#pragma unroll
  for (int dt = 0; dt < DTILES; dt++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[dt][i] = 0.f;
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  int lim_lo[2], lim_hi[2];
  lim_hi[0] = pos0 + row_a;
  lim_hi[1] = pos0 + row_b;
  lim_lo[0] = window > 0 ? lim_hi[0] - window + 1 : 0;
  lim_lo[1] = window > 0 ? lim_hi[1] - window + 1 : 0;
  // what this warp's 16 rows can see at all
  const int warp_hi = pos0 + warp * 16 + 15;
  const int warp_lo = window > 0 ? pos0 + warp * 16 - window + 1 : 0;

  const int n_tiles = (k_end - k_begin + KT - 1) / KT;
  bool bad_page = false;
  load_kv_tile<128>(smem, kcache, vcache, table, kvh, nkv, ps, k_begin, k_begin, k_end, tid, num_pages, bad_page);
  cp_async_commit();
  for (int it = 0; it < n_tiles; it++) {
    unsigned char* cur = smem + (it & 1) * STAGE_B;
    if (it + 1 < n_tiles)
      load_kv_tile<128>(smem + ((it + 1) & 1) * STAGE_B, kcache, vcache, table, kvh, nkv, ps, k_begin + (it + 1) * KT,
                        k_begin, k_end, tid, num_pages, bad_page);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int tile_key0 = k_begin + it * KT;
    if (warp * 16 < rows_live && tile_key0 <= warp_hi && tile_key0 + KT - 1 >= warp_lo) {
      // scores of the whole 64-key tile, one softmax update per row and tile
      float sc[KT / 8][4];
#pragma unroll
      for (int kb = 0; kb < KT / 16; kb++) {
        float s2[2][4];
        qk_16keys(s2, qf, smem_u32(cur), kb * 16, lane);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          sc[2 * kb][i] = s2[0][i];
          sc[2 * kb + 1][i] = s2[1][i];
        }
      }
      // a tile that every row of this warp sees whole needs no mask
      const bool whole = tile_key0 + KT - 1 <= pos0 + warp * 16 && tile_key0 + KT <= k_end &&
                         (window <= 0 || tile_key0 >= pos0 + warp * 16 + 15 - window + 1);
      const int c0 = tile_key0 + cq;
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        // running maximum in units of the raw score (the scale is positive); one FMA and one ex2 an element
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            float v = sc[nt][h * 2 + e];
            if (!whole) {
              const int key = c0 + nt * 8 + e;
              if (key < lim_lo[h] || key > lim_hi[h]) v = -INFINITY;
              sc[nt][h * 2 + e] = v;
            }
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx * scale_log2);  // m[] is kept in scaled units; NEG_BIG until a key is seen
        alpha[h] = fast_exp2(m[h] - m_new);
        m[h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const float pr = fast_exp2(fmaf(sc[nt][h * 2 + e], scale_log2, -m_new));
            sc[nt][h * 2 + e] = pr;
            sum += pr;
          }
        l[h] = l[h] * alpha[h] + sum;
      }
#pragma unroll
      for (int dt = 0; dt < DTILES; dt++) {
        o[dt][0] *= alpha[0];
        o[dt][1] *= alpha[0];
        o[dt][2] *= alpha[1];
        o[dt][3] *= alpha[1];
      }
#pragma unroll
      for (int kb = 0; kb < KT / 16; kb++) {
        uint32_t pf[4];
        pf[0] = pack_bf16(sc[2 * kb][0], sc[2 * kb][1]);
        pf[1] = pack_bf16(sc[2 * kb][2], sc[2 * kb][3]);
        pf[2] = pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
        pf[3] = pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
        pv_16keys(o, pf, smem_u32(cur) + TILE_B, kb * 16, lane);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; h++) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  const float inv_a = 1.f / l[0], inv_b = 1.f / l[1];
#pragma unroll
  for (int dt = 0; dt < DTILES; dt++) {
    const int col = dt * 8 + cq;
    if (row_a < rows_live)
      *reinterpret_cast<uint32_t*>(out + (size_t)(t0 + row_a) * out_stride + (size_t)head * HD + col) =
          pack_bf16(o[dt][0] * inv_a, o[dt][1] * inv_a);
    if (row_b < rows_live)
      *reinterpret_cast<uint32_t*>(out + (size_t)(t0 + row_b) * out_stride + (size_t)head * HD + col) =
          pack_bf16(o[dt][2] * inv_b, o[dt][3] * inv_b);
  }
  report_bad_page(bad_page, status);
}

static bool g_attr_set = false;
static int ensure_smem_attr() {
  if (g_attr_set) return 0;
  cudaError_t e = cudaSuccess;
  if (SMEM_B > 48 * 1024) {
    e = cudaFuncSetAttribute(attn_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_B);
  }
  if (e == cudaSuccess && DEC_SMEM_B > 48 * 1024) {
    e = cudaFuncSetAttribute(attn_decode_mma_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_B);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_mma_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_B);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_mma_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_B);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_decode_mma_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_B);
  }
  if (e != cudaSuccess) return (int)e;
  g_attr_set = true;
  return 0;
}

// TMA descriptors of the K and V cache of one layer, seen as [pages * kv heads * page size, HD] matrices, with
// boxes of 64 columns x min(page size, 64) rows.  rows == 0: no TMA (the head size is no multiple of 64, the page
// size no power of two from 8 up, or the caller did not say how many pages there are).  The last descriptors made
// are kept: a model asks for the same few (one pair a layer) at every step.
struct KvMaps {
  CUtensorMap k, v;
  int rows;
};
struct KvMapsKey {
  const void *k, *v;
  long long pages;
  int nkv, ps;
};
static int kv_maps(KvMaps& m, const void* kcache, const void* vcache, long long num_pages, int nkv, int ps) {
  memset(&m, 0, sizeof(m));
  const long long rows = num_pages * nkv * ps;
  if (!SWZ || num_pages <= 0 || ps < 8 || (ps & (ps - 1)) != 0 || rows >= (1ll << 31) || ((uintptr_t)kcache & 15) ||
      ((uintptr_t)vcache & 15))
    return 0;
  constexpr int SLOTS = 128;
  static KvMapsKey keys[SLOTS];
  static KvMaps maps[SLOTS];
  static int used = 0, next = 0;
  for (int i = 0; i < used; i++) {
    if (keys[i].k == kcache && keys[i].v == vcache && keys[i].pages == num_pages && keys[i].nkv == nkv && keys[i].ps == ps) {
      m = maps[i];
      return 0;
    }
  }
  int rc = tkb5::get_encode();
  const int box = ps < KT ? ps : KT;
  if (rc == 0) rc = tkb5::make_map(&m.k, kcache, (int)rows, HD, HD, box);
  if (rc == 0) rc = tkb5::make_map(&m.v, vcache, (int)rows, HD, HD, box);
  if (rc != 0) return rc;
  m.rows = box;
  keys[next] = KvMapsKey{kcache, vcache, num_pages, nkv, ps};
  maps[next] = m;
  next = (next + 1) % SLOTS;
  if (used < SLOTS) used++;
  return 0;
}

// Launch of the split-key kernel: the instantiation with TMA tiles if `tma` and there are descriptors
template <bool FUSED, bool TMA, typename... Rest>
static int launch_decode_as(dim3 grid, cudaStream_t st, const KvMaps& maps, Rest... rest) {
  KvMapsParam<TMA> param;
  if constexpr (TMA) {
    param.k = maps.k;
    param.v = maps.v;
  }
  return launch_pdl(attn_decode_mma_kernel<FUSED, TMA>, grid, dim3(128), (size_t)DEC_SMEM_B, st, param, maps.rows, rest...);
}
template <bool FUSED, typename... Rest>
static int launch_decode(bool tma, dim3 grid, void* st, const KvMaps& maps, Rest... rest) {
  if (tma && maps.rows > 0) return launch_decode_as<FUSED, true>(grid, (cudaStream_t)st, maps, rest...);
  return launch_decode_as<FUSED, false>(grid, (cudaStream_t)st, maps, rest...);
}

}  // namespace

// Scratch a decode launch needs for `items_cap` work items: floats of part_o and of part_ml.
TKB_EXPORT long long tkb_attn_decode_scratch_floats(int items_cap, int nh) {
  return (long long)items_cap * nh * (HD + 2);
}

// num_pages, status: page ids of the block tables are checked against the pool's size; an id beyond it sets the
// status flag and reads as zeros (num_pages <= 0: unknown, nothing is checked; status may be null).
// items: int32 [n_items_cap * 3] (request row, first key counted from the first visible one, number of keys); n_items_ptr: device int32 with the live count.
// The grid is sized by items_cap, so a captured graph serves any count up to it.
TKB_EXPORT int tkb_attn_decode_mma_bf16(const void* q, int q_stride, const void* kcache, const void* vcache,
                                        const int* seq_q_start, const int* seq_kv_len, const int* page_indptr,
                                        const int* page_ids, const int* items, const int* n_items_ptr, int items_cap,
                                        float* part_o, float* part_ml, int nh, int nkv, int ps, float scale, int window,
                                        int num_pages, int* status, void* st) {
  if (items_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0) return -2;
  int rc = ensure_smem_attr();
  if (rc) return rc;
  const int group = nh / nkv;
  const int head_tiles = (group + 15) / 16;
  if ((long long)nkv * head_tiles > 65535) return -3;
  dim3 grid(items_cap, nkv * head_tiles);
  KvMaps maps;
  memset(&maps, 0, sizeof(maps));  // every tile is gathered (num_pages <= 0: the caller does not know the pool's size)
  return launch_decode<false>(false, grid, st, maps, (const bf16*)q, q_stride, (bf16*)kcache, (bf16*)vcache, seq_q_start,
                              seq_kv_len, page_indptr, page_ids, items, n_items_ptr, part_o, part_ml, nh, nkv, ps,
                              scale * 1.4426950408889634f, window, head_tiles, (const float*)nullptr, 0, 0, num_pages,
                              status, (const float*)nullptr, 0, 0LL, (int*)nullptr, (const int*)nullptr,
                              (const int*)nullptr, (const int*)nullptr, (bf16*)nullptr, 0, (const float*)nullptr,
                              (const float*)nullptr, 0.f);
}

// The same with rotary encoding and the cache write folded in: qkv holds the step's un-rotated q|k|v rows
// [tokens, (nh + 2 nkv) * HD] in bfloat16, or (n_parts > 0) qkv_parts holds them as float32 slices of a
// K-split product, [n_parts][tokens, C] spaced part_stride floats apart, which are added in order and
// rounded to bfloat16 first.  rot is the rotary width (0: none); the pages of the requests must
// already cover the tokens' positions.
// tma: the step has work items of more than three tiles, so the instantiation that fetches whole tiles by TMA
// is worth its registers and code; steps of short items (a request or two at short contexts) take the one
// without, which measured 3 % faster a step there.
TKB_EXPORT int tkb_attn_decode_rope_mma_bf16(const void* qkv, int q_stride, const float* qkv_parts, int n_parts,
                                             long long part_stride, void* kcache, void* vcache,
                                             const int* seq_q_start, const int* seq_kv_len, const int* page_indptr,
                                             const int* page_ids, const int* items, const int* n_items_ptr,
                                             int items_cap, float* part_o, float* part_ml, int nh, int nkv, int ps,
                                             float scale, int window, const float* inv_freq, int rot,
                                             int write_cache, int num_pages, int tma, int* status,
                                             const float* qkv_bias, const float* qk_norm_w, float norm_eps, void* st) {
  if (items_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0 || rot < 0 || rot > HD || (rot & 3)) return -2;
  int rc = ensure_smem_attr();
  if (rc) return rc;
  const int group = nh / nkv;
  const int head_tiles = (group + 15) / 16;
  if ((long long)nkv * head_tiles > 65535) return -3;
  dim3 grid(items_cap, nkv * head_tiles);
  KvMaps maps;
  rc = kv_maps(maps, kcache, vcache, num_pages, nkv, ps);
  if (rc) return rc;
  return launch_decode<true>(tma != 0, grid, st, maps, (const bf16*)qkv, q_stride, (bf16*)kcache, (bf16*)vcache, seq_q_start,
                             seq_kv_len, page_indptr, page_ids, items, n_items_ptr, part_o, part_ml, nh, nkv, ps,
                             scale * 1.4426950408889634f, window, head_tiles, inv_freq, rot, write_cache, num_pages,
                             status, qkv_parts, n_parts, part_stride, (int*)nullptr, (const int*)nullptr,
                             (const int*)nullptr, (const int*)nullptr, (bf16*)nullptr, 0, qkv_bias, qk_norm_w, norm_eps);
}

// Split-key attention with the merge of the splits inside the same kernel (the last block to finish a request's
// group of heads adds the splits up).  qkv/q_stride as in tkb_attn_decode_mma_bf16 when fused == 0 (rotated q),
// as in tkb_attn_decode_rope_mma_bf16 when fused != 0.  counters: int32 [dec_cap * grid.y] that are zero
// before the first launch and are left zero by every launch; item_entry[i]: index of item i's request in the
// decode list; dec_item_start: CSR over that list; out_row_of[request row]: row of `out` to write.
TKB_EXPORT int tkb_attn_decode_merged_bf16(const void* qkv, int q_stride, const float* qkv_parts, int n_parts,
                                           long long part_stride, void* kcache, void* vcache, const int* seq_q_start,
                                           const int* seq_kv_len, const int* page_indptr, const int* page_ids,
                                           const int* items, const int* n_items_ptr, int items_cap, float* part_o,
                                           float* part_ml, int nh, int nkv, int ps, float scale, int window,
                                           int fused, const float* inv_freq, int rot, int write_cache,
                                           int num_pages, int tma, int* status, int* counters, const int* item_entry,
                                           const int* dec_item_start, const int* out_row_of, void* out, int out_stride,
                                           const float* qkv_bias, const float* qk_norm_w, float norm_eps, void* st) {
  if (items_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0 || counters == nullptr) return -2;
  if (fused && (rot < 0 || rot > HD || (rot & 3))) return -2;
  int rc = ensure_smem_attr();
  if (rc) return rc;
  const int group = nh / nkv;
  const int head_tiles = (group + 15) / 16;
  if ((long long)nkv * head_tiles > 65535) return -3;
  dim3 grid(items_cap, nkv * head_tiles);
  const float sl2 = scale * 1.4426950408889634f;
  KvMaps maps;
  rc = kv_maps(maps, kcache, vcache, num_pages, nkv, ps);
  if (rc) return rc;
  if (fused)
    return launch_decode<true>(tma != 0, grid, st, maps, (const bf16*)qkv, q_stride, (bf16*)kcache, (bf16*)vcache,
                               seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items_ptr, part_o, part_ml, nh, nkv,
                               ps, sl2, window, head_tiles, inv_freq, rot, write_cache, num_pages, status, qkv_parts,
                               n_parts, part_stride, counters, item_entry, dec_item_start, out_row_of, (bf16*)out,
                               out_stride, qkv_bias, qk_norm_w, norm_eps);
  return launch_decode<false>(tma != 0, grid, st, maps, (const bf16*)qkv, q_stride, (bf16*)kcache, (bf16*)vcache,
                              seq_q_start, seq_kv_len, page_indptr, page_ids, items, n_items_ptr, part_o, part_ml, nh, nkv,
                              ps, sl2, window, head_tiles, (const float*)nullptr, 0, 0, num_pages, status,
                              (const float*)nullptr, 0, 0LL, counters, item_entry, dec_item_start, out_row_of, (bf16*)out,
                              out_stride, (const float*)nullptr, (const float*)nullptr, 0.f);
}

TKB_EXPORT int tkb_attn_decode_merge_bf16(const float* part_o, const float* part_ml, const int* dec_seqs,
                                          const int* dec_item_start, const int* n_dec_ptr, int dec_cap,
                                          const int* seq_q_start, void* out, int out_stride, int nh, void* st) {
  if (dec_cap <= 0) return 0;
  if (nh > 65535) return -3;
  dim3 grid(dec_cap, nh);
  const int threads = HD >= 128 ? 128 : (HD >= 64 ? 64 : 32);
  return launch_pdl(attn_decode_merge_kernel, grid, dim3(threads), 0, (cudaStream_t)st, part_o, part_ml, dec_seqs,
                    dec_item_start, n_dec_ptr, seq_q_start, (bf16*)out, out_stride, nh);
}

TKB_EXPORT int tkb_attn_prefill_mma_bf16(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                         const void* vcache, const int* seq_q_start, const int* seq_q_len,
                                         const int* seq_kv_len, const int* page_indptr, const int* page_ids,
                                         const int* tiles, const int* n_tiles_ptr, int tiles_cap, int nh, int nkv, int ps,
                                         float scale, int window, int num_pages, int* status, void* st) {
  if (tiles_cap <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || ps <= 0) return -2;
  if (nh > 65535) return -3;
  int rc = ensure_smem_attr();
  if (rc) return rc;
  dim3 grid(tiles_cap, nh);
  return launch_pdl(attn_prefill_mma_kernel, grid, dim3(128), (size_t)SMEM_B, (cudaStream_t)st, (const bf16*)q, q_stride,
                    (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, seq_q_start, seq_q_len, seq_kv_len,
                    page_indptr, page_ids, tiles, n_tiles_ptr, nh, nkv, ps, scale * 1.4426950408889634f, window, num_pages,
                    status);
}
TKB_EXPORT int tkb_attn_mma_head_dim() { return HD; }
