// The allocation-free variant of split-key decode attention: same kernels as attention_mma.cu,
// with the partial results kept in a fixed __device__ array instead of caller-provided scratch.
// See attention_decode_static.h for who needs this, the size limit and the rules of use.
//
// Compile with -DTKB_HD=<head size>.
#include "attention_mma.cu"
#include "attention_decode_static.h"

// The scratch itself.  In host code this name is only a handle for the runtime's symbol lookup, not
// a device address: the address a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[TKB_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return -2;
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return (int)cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

TKB_EXPORT int tkb_attn_decode_static_scratch_bf16(const void* q, int q_stride, const void* kcache, const void* vcache,
                                                   const int* seq_q_start, const int* seq_kv_len,
                                                   const int* page_indptr, const int* page_ids, const int* items,
                                                   const int* n_items_ptr, int items_cap, const int* dec_seqs,
                                                   const int* dec_item_start, const int* n_dec_ptr, int dec_cap,
                                                   void* out, int out_stride, int nh, int nkv, int ps, float scale,
                                                   int window, int num_pages, int* status, void* stream) {
  if (items_cap <= 0 || dec_cap <= 0) return 0;
  if (nh <= 0) return -2;
  const long long need = tkb_attn_decode_scratch_floats(items_cap, nh);
  if (need > (long long)TKB_STATIC_SCRATCH_FLOATS) return -4;
  float* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  float* part_o = scratch;                                   // [items_cap, nh, HD]
  float* part_ml = scratch + (size_t)items_cap * nh * HD;    // [items_cap, nh, 2]
  rc = tkb_attn_decode_mma_bf16(q, q_stride, kcache, vcache, seq_q_start, seq_kv_len, page_indptr, page_ids, items,
                                n_items_ptr, items_cap, part_o, part_ml, nh, nkv, ps, scale, window, num_pages, status,
                                stream);
  if (rc) return rc;
  return tkb_attn_decode_merge_bf16(part_o, part_ml, dec_seqs, dec_item_start, n_dec_ptr, dec_cap, seq_q_start, out,
                                    out_stride, nh, stream);
}

TKB_EXPORT long long tkb_attn_decode_static_scratch_capacity() { return (long long)TKB_STATIC_SCRATCH_FLOATS; }
