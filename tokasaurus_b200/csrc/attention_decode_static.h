// Split-key decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference (whose attention library sizes and owns a
// workspace that the caller allocates with torch).  It exists for callers that hold device
// pointers but may not allocate device memory themselves:
//   * a host program that has already handed all free device memory to its own pool (a server that
//     reserved the whole GPU for its key/value pages) and has no allocator left to ask;
//   * a plug-in or callback that runs inside someone else's runtime where cudaMalloc and cudaFree
//     are off limits, because they synchronise the whole device and would stall the host's other
//     streams, or because the host forbids allocation in its hot path;
//   * a caller without torch, which is what the engine's own wrappers use to get scratch memory.
// Such callers still pass every input and the output; only the scratch between the split-key
// kernel and the merge kernel comes from this library, from a fixed array in device memory.
//
// The scratch array is a file-scope __device__ array of TKB_STATIC_SCRATCH_FLOATS floats (8 MiB).
// Every GPU whose context loads this library holds that array until the process exits.
//
// Limits and rules
//   * items_cap * n_heads * (head_dim + 2) must not exceed TKB_STATIC_SCRATCH_FLOATS; a larger call
//     is refused with return code -4 and nothing is launched.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and keeps it; make that first call outside any stream capture.
//   * All calls share the one array, which keeps whatever the last call left in it.  Nothing in it
//     has to start at zero: every partial result that the merge kernel reads was written by the
//     split-key kernel of the same call.  Two calls that overlap on the GPU (different streams, or
//     different host threads without ordering between them) race on the array; order them.
//   * No cudaMalloc, cudaFree or other allocating routine is called, on the first call or later.
//
// Arguments are those of tkb_attn_decode_mma_bf16 followed by those of tkb_attn_decode_merge_bf16
// (see attention_mma.cu), without the two scratch pointers.  num_pages is the number of pages of the caller's
// cache and status a device int (or null): a page id of the block tables beyond the pool sets bit 2 of *status and
// reads as zeros instead of reaching memory outside the cache (num_pages <= 0 switches the check off).  Returns 0, a CUDA error code (> 0),
// or a refusal (< 0: -2 sizes not supported, -3 grid too large, -4 beyond the built-in scratch).
#pragma once

#define TKB_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int tkb_attn_decode_static_scratch_bf16(const void* q, int q_stride, const void* kcache, const void* vcache,
                                        const int* seq_q_start, const int* seq_kv_len, const int* page_indptr,
                                        const int* page_ids, const int* items, const int* n_items_ptr, int items_cap,
                                        const int* dec_seqs, const int* dec_item_start, const int* n_dec_ptr,
                                        int dec_cap, void* out, int out_stride, int nh, int nkv, int ps, float scale,
                                        int window, int num_pages, int* status, void* stream);

#ifdef __cplusplus
}
#endif
