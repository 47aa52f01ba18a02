// Attention over the paged cache with split key ranges, for callers that must not allocate.
//
// This entry point has no counterpart in the reference project (which has no kernels of its own
// and lets its tensor library allocate whatever it needs); it exists for the users of this
// library described below.
//
// Who needs it: code that calls into this library from a place where device memory cannot be
// obtained - a host that handed all of the GPU's memory to its own pools at start-up and forbids
// further cudaMalloc calls, a plug-in running inside another runtime's allocator discipline, or a
// latency-critical loop in which an allocation (which may synchronise the device) is not
// acceptable.  The ordinary entry points (de_attn_simt + de_attn_combine) leave the scratch memory
// for the partial results to the caller, who normally takes it from an allocator.  Here the
// scratch lives inside the library instead: a file-scope __device__ array of
// DE_ATTN_STATIC_SCRATCH_FLOATS floats (4 MiB), which every GPU that loads the library holds until
// the process exits.  The caller still passes all inputs and the output.
//
// What it computes: exactly de_attn_simt followed by de_attn_combine (float32 arithmetic on the
// CUDA cores, float32 or bfloat16 storage): every work item writes its unnormalised partial result
// into the scratch array and the combine items merge them into `out`.
//
// Limits and rules:
//   * num_partials * kv_heads * 8 * (head_dim + 2) must not exceed DE_ATTN_STATIC_SCRATCH_FLOATS.
//     A larger request is refused: the function returns DE_ATTN_STATIC_TOO_LARGE, launches
//     nothing, and de_attn_static_scratch_error() gives the sizes in words.
//   * `num_partials` is the number of partial slots the work items use; it is what the size check
//     is made with, so the kernels are told it too: a work item or combine item that names a
//     slot at or beyond num_partials is skipped (it writes nothing into the array or beyond it,
//     and the rows it would have produced are left as they were in `out`).
//   * It calls no cudaMalloc, cudaFree or other allocating routine, on any call.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
//     outside any stream capture.  Later calls on the device only launch kernels.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing a call
//     reads from it depends on earlier contents: each call writes every partial it later merges.
//     Two calls whose kernels overlap on the GPU (different streams, or the same stream from two
//     threads without ordering) race on the array; keep calls that use it ordered on one stream.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define DE_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)
#define DE_ATTN_STATIC_TOO_LARGE (-10)

// dtype: 0 float32, 1 bfloat16.  Arguments as for de_attn_simt and de_attn_combine; `items` are
// num_items work items of 8 ints, `combine_items` num_combine items of 4 ints.  Returns 0, a
// negative code for refused sizes, or a CUDA error code.
int de_attn_simt_static_scratch(int dtype, const void* q, int q_stride, void* out, int out_stride,
                                const void* k_pages, const void* v_pages, const int* block_table,
                                int table_stride, int num_pages, const int* seq_slot,
                                const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                                const int* items, int num_items, const int* combine_items,
                                int num_combine, int num_partials, int heads, int kv_heads,
                                int head_dim, int page, float scale, int window, void* stream);

// The reason of the calling thread's last refusal, in words (empty if there was none).
const char* de_attn_static_scratch_error(void);

#ifdef __cplusplus
}
#endif
