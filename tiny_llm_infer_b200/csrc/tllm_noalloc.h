/* Entry point of libtllm_kernels.so for callers that must not allocate device memory.
 *
 * It has no counterpart in xu797/tiny-llm-infer: the reference allocates scratch for its
 * attention scores through its caching allocator on every step.
 *
 * Who needs it.  Some programs that embed these kernels cannot call cudaMalloc (or any
 * routine that may call it, such as a framework's tensor allocator) at the point where they
 * launch work: a real-time loop whose memory was fixed at start-up, a plug-in that runs
 * inside a host process which owns all device memory and hands out none, code that runs
 * while another thread holds the driver's allocation lock, or a process working under a
 * hard memory limit where an allocation late in its life may fail.  The ordinary decode
 * attention entry point, tllm_paged_attention_decode, needs the caller to bring scratch
 * memory for the partial results of its key splits; this variant brings its own.
 *
 * How.  The scratch is one array in the library's device image,
 *   static __device__ __align__(256) float[TLLM_NOALLOC_SCRATCH_FLOATS]   (16 MiB),
 * which every GPU that loads the library holds until the process exits.  A call needs
 *   n_rows * q_heads * splits * (head_dim + 2)
 * floats of it (splits > 1; with splits == 1 none) and is refused with an error text, and
 * nothing launched, if that exceeds the array.  The function calls no cudaMalloc, cudaFree
 * or other allocating routine; inputs and outputs are still the caller's.
 *
 * First call on a device.  The array's device address is looked up with
 * cudaGetSymbolAddress once per device, by the first call made while that device is
 * current, and remembered.  Make that first call before any stream capture begins.
 *
 * Sharing.  All calls on a device use the same array, and it keeps what the last call
 * left in it.  Nothing in it has to start at zero: every partial result that the combining
 * step of a call reads was written earlier in that same call.  Two calls whose work
 * overlaps on the GPU (different streams, or threads launching at once) write the same
 * memory and race: run them one after the other on one stream, or order them with events.
 *
 * Arguments, result and the computed values are those of tllm_paged_attention_decode
 * without the two scratch pointers: 0 on success, -1 for a refused argument, a cudaError_t
 * otherwise; the text of the last error is returned by tllm_last_error().
 */
#ifndef TLLM_NOALLOC_H_
#define TLLM_NOALLOC_H_

#include <cuda_runtime_api.h>

#define TLLM_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int tllm_paged_attention_decode_noalloc(
    const void* q,            /* [tokens, q_heads * head_dim] bfloat16 */
    const void* cache,        /* [pages, 2, kv_heads, page_size, head_dim] bfloat16 */
    const int* positions,     /* [tokens] position of each row in its request */
    const int* token_slot,    /* [tokens] row of the block table, negative: skip the row */
    const int* rows,          /* [n_rows] rows to compute, or NULL for rows 0 .. n_rows-1 */
    int n_rows,
    const int* block_table,   /* [slots, max_pages] page ids */
    int max_pages, int page_size, int q_heads, int kv_heads, int head_dim,
    int window,               /* 0: every key; w: the last w keys */
    float scale, int splits,
    void* out,                /* [tokens, q_heads * head_dim] bfloat16 */
    cudaStream_t stream);

/* Floats of the built-in scratch a call with these sizes would use. */
long long tllm_noalloc_scratch_needed(int n_rows, int q_heads, int head_dim, int splits);

#ifdef __cplusplus
}
#endif

#endif /* TLLM_NOALLOC_H_ */
