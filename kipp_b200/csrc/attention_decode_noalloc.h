/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference: it is an addition of
 * this library.
 *
 * Who it is for.  The ordinary entry point, kipp_attn_decode_mma, wants a
 * scratch buffer from its caller (partial outputs and (max, sum) pairs of
 * every key split).  Some callers have nowhere to get one: code that runs
 * inside another framework's stream callback or plugin hook where cudaMalloc
 * is forbidden, a host whose memory pool is fixed at start-up and fully given
 * out, or a caller that must not disturb an allocator it does not own.  For
 * them the scratch lives inside the library, in a file-scope device array of
 * fixed size.
 *
 * What it costs.  KIPP_NOALLOC_SCRATCH_BYTES (16 MiB) of device memory on
 * every GPU on which the library is loaded, from load to process exit, whether
 * the entry point is called or not.
 *
 * Limits and rules.
 *   - The scratch need of a call is
 *         n * n_q * max_splits * (head_dim + 2) * 4 bytes
 *     (n decoded tokens).  A call that needs more than
 *     KIPP_NOALLOC_SCRATCH_BYTES is refused with KIPP_ERR_SCRATCH (-4) and
 *     launches nothing; kipp_attn_decode_noalloc_scratch_bytes tells the need
 *     beforehand.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and keeps it for later
 *     calls.  Make that first call before any stream capture begins on the
 *     device; the look-up is not a stream operation.
 *   - It calls no cudaMalloc, cudaFree or any allocating library routine.
 *   - All calls on a device share the one array.  Nothing in it has to be
 *     cleared between calls: every value the merge step reads was written by
 *     the split kernel of the same call.  But two calls whose kernels overlap
 *     on the GPU (different streams, or graphs replayed side by side) write
 *     the same memory and race: keep calls on one stream, or order them.
 *   - The looked-up address is kept in a plain per-device table without a lock.
 *     Two host threads that make their first call on a device at the same moment
 *     both look the address up and store the same value, which is harmless; the
 *     library adds no other synchronisation between host threads.
 *   - split_keys points at ONE value on the device: the keys per split of the step.
 *   - Inputs, outputs and every other rule are those of kipp_attn_decode_mma.
 */
#ifndef KIPP_ATTENTION_DECODE_NOALLOC_H
#define KIPP_ATTENTION_DECODE_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define KIPP_NOALLOC_SCRATCH_BYTES (16ll << 20)
#define KIPP_ERR_SCRATCH (-4)

/* Bytes of library scratch a call with these sizes needs. */
long long kipp_attn_decode_noalloc_scratch_bytes(int n, int n_q, int head_dim, int max_splits);

/* Same arguments as kipp_attn_decode_mma without the scratch pointer.
 * Returns 0, a negative argument error (KIPP_ERR_SCRATCH when the sizes need
 * more than the built-in scratch) or a positive cudaError_t. */
int kipp_attn_decode_mma_noalloc(void* out, const void* q, const void* k_pages, const void* v_pages,
                                 const int* q_start, const int* context_len, const int* block_table,
                                 int table_width, int page_size, const int* rows, int n, int n_q,
                                 int n_kv, int head_dim, float scale, int window, int max_splits,
                                 const int* split_keys, void* stream);

#ifdef __cplusplus
}
#endif
#endif
