// tvb_attention_rows_static: the split mode of the row attention kernel for callers that
// must not allocate device memory.
//
// This entry point has no counterpart in RicardoMin/tiny-vLLM; it exists for users of this
// library only.
//
// Who needs it.  tvb_attention_rows in split mode wants a scratch buffer in global memory for
// the partial (max, sum, output) of every chunk of keys, and its caller has to allocate that
// buffer.  Some callers cannot: a host program that handed the whole GPU to a memory pool of
// its own at start-up and forbids any later cudaMalloc (a serving process with a fixed memory
// budget, a plug-in that is not allowed to allocate behind its host's back), or code on a path
// where an allocation could block or fail at a bad moment.  For them the scratch lives inside
// the library: a file-scope `static __device__` array of TVB_STATIC_SCRATCH_FLOATS floats
// (16 MiB).  Every GPU on which the library is loaded holds that array until the process
// exits, whether or not this function is ever called.
//
// What it does.  Same arguments and same result as tvb_attention_rows with max_chunks > 0,
// minus the scratch pointer.  The call allocates nothing: no cudaMalloc, no cudaFree, no
// allocating library routine.  A batch whose partials do not fit
// (tokens * num_q * max_chunks * (head_dim + 2) > TVB_STATIC_SCRATCH_FLOATS) is refused with
// TVB_STATIC_SCRATCH_TOO_SMALL before anything is launched; max_chunks == 0 (no scratch needed)
// is refused with TVB_BAD_ARGUMENT, use tvb_attention_rows for that.
//
// What the caller must get right.  max_chunks has to be at least
// ceil((largest position in `positions` + 1) / 256): the partials of a row are stored
// max_chunks to a row.  The positions live on the device, so the call cannot check this; a row
// whose position needs more chunks than max_chunks comes out as NaN (nothing outside the
// array is touched).  max_chunks and num_q up to 65,535 and head_dim up to 256 are accepted.
//
// First call on a device.  The first call made while a device is current looks up the device
// address of the array (cudaGetSymbolAddress) and keeps it for that device; later calls reuse
// it.  Make that first call before any stream capture begins.
//
// Sharing.  All calls on a device use the same array, and it keeps whatever the previous call
// left in it.  Nothing in it has to start at zero: the kernels write every partial they later
// read.  Two calls whose kernels overlap on the GPU (different streams, or one stream per
// thread) race on the array and give wrong results; serialise them.
#pragma once

#define TVB_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define TVB_STATIC_SCRATCH_TOO_SMALL (-2)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a cudaError_t (> 0), TVB_BAD_ARGUMENT (-1) or TVB_STATIC_SCRATCH_TOO_SMALL (-2).
int tvb_attention_rows_static(const void* q, long long q_token_stride, const void* key_cache,
                              const void* value_cache, const int* block_tables, int table_stride,
                              const int* token_row, const int* positions, void* out, int max_chunks,
                              int tokens, int num_q, int num_kv, int head_dim, int page_size,
                              int window, float scale, int dtype, void* stream);

// Floats the built-in scratch holds.
long long tvb_attention_rows_static_capacity(void);

// One line of text for a code returned by tvb_attention_rows_static.
const char* tvb_attention_rows_static_error(int code);

#ifdef __cplusplus
}
#endif
