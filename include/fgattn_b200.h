/* C ABI of libfgattn_b200: fine-grained threshold block-sparse attention forward path for B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the given CUDA stream
 * and returns an fgattn_status (0 = ok) without synchronising.  Nothing here allocates or frees
 * device memory except a 4-byte per-device error word on first use; scratch memory is passed in by
 * the caller.  Citations name the interface of sankeerth95/fgattn_tk_cuda that each entry point
 * replaces (paths inside that project).
 *
 * Conventions (python/extension.cpp:52-73, python/spattn/sparseattn_functionals.py:10-26):
 *   q, k, v, o : bf16, [B, H, S, D] contiguous, 16-byte aligned, D in {64, 128}
 *   max_q, denom : fp32 [B, H, 1, S_pad], S_pad = ceil(S/128)*128; tail max = 0, tail denom = -inf
 *   seq        : query rows S; o, max_q, denom follow it
 *   kv_rows    : rows per head of the k / v tensors ([B, H, kv_rows, D]); equal to seq in the reference,
 *                free here (shorter or longer key / value sequences)
 *   kv_seq_len : number of leading key/value rows that take part (1..kv_rows); the reference hard-codes
 *                this per shape (python/cuda_attn.cu:28-31), here it is a run-time argument
 *   scale      : softmax scale; pass 0 for 1/sqrt(D) (the reference hard-codes 1/sqrt(128),
 *                include/fullattn_tma.cuh:182-183)
 *   stream     : a cudaStream_t (may be NULL for the default stream)
 */
#ifndef FGATTN_B200_H_
#define FGATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FGATTN_OK = 0,
  FGATTN_INVALID_ARGUMENT = 1,   /* null pointer, non-positive size, kv_seq_len out of range ... */
  FGATTN_UNSUPPORTED = 2,        /* head dimension other than 64 / 128, list too long ...          */
  FGATTN_MISALIGNED = 3,         /* a tensor base address is not 16-byte aligned                    */
  FGATTN_CUDA_ERROR = 4,         /* a CUDA runtime / launch error; see fgattn_last_cuda_error       */
  FGATTN_NO_DRIVER = 5,          /* the tensor-map encoder of the CUDA driver could not be found    */
  FGATTN_DEVICE_TIMEOUT = 6,     /* a bounded in-kernel wait ran out (reported by fgattn_check)     */
  FGATTN_SCRATCH_TOO_SMALL = 7
} fgattn_status;

const char* fgattn_status_string(int status);
/* cudaError_t of the most recent FGATTN_CUDA_ERROR on this thread. */
int fgattn_last_cuda_error(void);
/* Scheduling knobs, for tuning runs and tests; results never depend on them.  (No counterpart in the
 * reference.)  "group_heads": (batch, head) units per group of the longest-first thread-block orders
 * (0 = built-in choice, negative = back to the environment variable FGATTN_GROUP_HEADS, which is read
 * once per process); "dense_persist": 1 / 0 forces the persistent / one-item form of the dense family,
 * -1 = chosen by key length, below -1 = back to FGATTN_DENSE_PERSIST; "dense_halves": 0 keeps the dense family from cutting the items of a
 * less-than-half-full last wave of thread blocks into their two query tiles (1 = default, negative = back
 * to FGATTN_DENSE_HALVES); "token_block_route": 1 allows the
 * block route of fgattn_sp_attn (given the large workspace), 0 keeps it on the row gather (default),
 * negative = back to FGATTN_TOKEN_BLOCK_ROUTE; "maxq_wide": 0 runs the max / denominator pass and the token mask
 * over all key tiles on the dense family's own modes instead of the two-threads-per-row kernel (1 / -1 = default, below -1 = back to
 * FGATTN_MAXQ_WIDE). */
int fgattn_set_tuning(const char* name, int value);
/* Synchronise `stream` and report whether any kernel launched through this library on the current
 * device gave up on a bounded wait.  Returns FGATTN_OK or FGATTN_DEVICE_TIMEOUT; *code (optional)
 * receives the id of the wait that ran out.  Clears the error word. */
int fgattn_check(void* stream, int* code);

/* Dense attention o = softmax(q k^T * scale) v.
 * Replaces attn_fwd_wg_impl (python/extension.cpp:4-7, python/cuda_attn.cu:9-38), i.e. the
 * full_attn operator (python/extension.cpp:52-73). */
int fgattn_full_attn(void* o, const void* q, const void* k, const void* v, int batch, int heads, int seq, int D,
                     int kv_rows, int kv_seq_len, float scale, void* stream);

/* Dense attention that also emits the per-row raw maximum and softmax denominator.
 * Replaces attn_maxq_denom_impl (python/extension.cpp:22-27, python/cuda_attn.cu:97-139), the
 * fullattn_maxq_denom operator (python/extension.cpp:178-204). */
int fgattn_fullattn_maxq_denom(void* o, float* max_q, float* denom, const void* q, const void* k, const void* v,
                               int batch, int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale,
                               void* stream);

/* Per-row raw maximum m_i = max_j q_i.k_j and denominator l_i = sum_j exp((q_i.k_j - m_i)*scale).
 * Replaces maxq_denom_impl (python/extension.cpp:29-33, python/cuda_attn.cu:142-180), the
 * maxq_denom operator (python/extension.cpp:226-248). */
int fgattn_maxq_denom(float* max_q, float* denom, const void* q, const void* k, int batch, int heads, int seq, int D,
                      int kv_rows, int kv_seq_len, float scale, void* stream);

/* Threshold mask at the reference granularity: booleanmask[b,h,qblk,j] (int32,
 * [B,H,ceil(S/128),mask_stride]) becomes 1 where some row of the 128-row query block has softmax
 * probability > threshold for key token j; other entries are set to 0 (the whole tensor is
 * cleared first, so pre-zeroing by the caller is harmless but not needed).
 * Replaces booleanmask_128_impl (python/extension.cpp:36-41, python/cuda_attn.cu:183-266), the
 * booleanmask_128 operator (python/extension.cpp:271-297). */
int fgattn_booleanmask_128(int* booleanmask, float threshold, int mask_stride, const float* max_q, const float* denom,
                           const void* q, const void* k, int batch, int heads, int seq, int D, int kv_rows,
                           int kv_seq_len, float scale, void* stream);

/* Same token mask, computed only inside the 64x64 blocks that fgattn_block_index_lists kept for the
 * same q, k and threshold (kb_indices / kb_counts / list_stride as that call wrote them, max_q / denom
 * from the same call).  A token can only pass the threshold inside a kept block, so the result is the
 * mask of fgattn_booleanmask_128 (up to scores within rounding of the threshold) while the second
 * Q K^T pass of include/mask_utils.cuh:131-243 shrinks to the key tiles that some kept block touches.
 * `workspace` (fgattn_sp_attn_workspace_bytes, scratch) is optional: with it the thread blocks take the
 * query blocks with the longest lists first; null = storage order.  Same mask either way. */
int fgattn_booleanmask_128_listed(int* booleanmask, float threshold, int mask_stride, const float* max_q,
                                  const float* denom, const void* q, const void* k, const int* kb_indices,
                                  const int* kb_counts, int list_stride, int batch, int heads, int seq, int D,
                                  int kv_rows, int kv_seq_len, float scale, void* workspace, size_t workspace_bytes,
                                  void* stream);

/* Mask rows -> ascending index lists: for every (b,h,seqblock) row of booleanmask
 * ([B,H,seqblocks,mask_stride] int32, > 0 = keep) write the kept columns < seq in ascending order
 * to kv_indices, fill the remaining slots with mask_stride and write the count.
 * Replaces booleanmask_to_indexmask_impl (python/extension.cpp:44-49, python/cuda_attn.cu:269-303;
 * kernel include/mask_utils.cuh:273-302, whose list order was nondeterministic). */
int fgattn_booleanmask_to_indexmask(int* kv_indices, int* kv_num_indices, const int* booleanmask, int batch, int heads,
                                    int seq, int seqblocks, int mask_stride, void* stream);

/* Identity lists: kv_indices[b,h,sb,s] = s for all s < index_stride, kv_num_indices = seq.
 * Replaces allindex_mask_impl (python/extension.cpp:16-19, python/cuda_attn.cu:78-94). */
int fgattn_all_index_mask(int* kv_indices, int* kv_num_indices, int batch, int heads, int seqblocks, int seq,
                          int index_stride, void* stream);

/* Sparse attention over key-TOKEN lists at the reference granularity: for each 128-row query
 * block, softmax restricted to the listed key tokens (renormalised), times the listed v rows.
 * kv_indices int32 [B,H,ceil(S/128),mask_stride], kv_num_indices int32 [B,H,ceil(S/128)].
 * Replaces attn_sparse_fwd_wg_impl (python/extension.cpp:10-14, python/cuda_attn.cu:41-75), the
 * sp_attn operator (python/extension.cpp:125-154).  `workspace` (scratch) is optional and comes in two
 * sizes.  With fgattn_sp_attn_workspace_bytes the thread blocks take the query blocks longest list first,
 * which shortens the end of the launch when list lengths differ; null = storage order.  With
 * fgattn_sp_attn_token_workspace_bytes AND the "token_block_route" knob of fgattn_set_tuning switched on,
 * the call additionally converts every list into the 64-key blocks it touches plus a column mask per
 * block, and query blocks whose listed tokens fill at least three quarters of the touched blocks load
 * those blocks whole by TMA instead of gathering rows (include/asyncloadutils.cuh:73-153) -- the unlisted
 * columns are switched off in the softmax; lists that are scattered or name a token twice stay on the
 * row gather.  It pays for lists made of (nearly) whole key blocks (1.24x at C3 with every token of the
 * kept blocks listed); threshold-mask lists fill 55-60 % of the blocks they touch and are faster on the
 * row gather, which is why the knob is off by default.  Same result within rounding in every case. */
int fgattn_sp_attn(void* o, const void* q, const void* k, const void* v, const int* kv_indices,
                   const int* kv_num_indices, int mask_stride, int batch, int heads, int seq, int D, int kv_rows,
                   float scale, void* workspace, size_t workspace_bytes, void* stream);

/* ---- 64x64 block granularity --------------------------------------------------------------- */

/* Bytes of scratch that fgattn_block_index_lists wants in order to process all batch*heads units
 * in one pass (it works with less, down to one unit's worth, by looping over head chunks). */
size_t fgattn_block_scratch_bytes(int batch, int heads, int seq, int kv_seq_len);

/* One pass over all keys that produces max_q / denom (and, when o and v are non-null, the dense
 * attention output) and from them the per-query-block key-BLOCK lists: block (qb, kb) of 64x64 is
 * kept iff its largest softmax probability exceeds threshold (strict).  kb_indices int32
 * [B,H,nqb,list_stride] receives ascending block indices, unused slots = nkb; kb_counts int32
 * [B,H,nqb].  nqb = ceil(S/64), nkb = ceil(kv_seq_len/64), list_stride >= nkb.
 * Fuses what the reference does as maxq_denom / fullattn_maxq_denom + booleanmask_128 +
 * booleanmask_to_indexmask (python/spattn/mask_utils.py:306-334, :358-382) for the block
 * granularity, without the second Q K^T pass of include/mask_utils.cuh:131-243. */
int fgattn_block_index_lists(int* kb_indices, int* kb_counts, int list_stride, float* max_q, float* denom, void* o,
                             const void* q, const void* k, const void* v, float threshold, int batch, int heads,
                             int seq, int D, int kv_rows, int kv_seq_len, float scale, void* scratch,
                             size_t scratch_bytes, void* stream);

/* The threshold step of fgattn_block_index_lists alone, on block maxima that an earlier call left behind:
 * when that call was given scratch for all batch*heads units (fgattn_block_scratch_bytes), the scratch holds,
 * as fp32 [B*H][nkb][ceil(seq/128)*128], the raw maximum of Q K^T per query row and 64-key block, and together
 * with the max_q / denom of the same call this entry point builds the lists for ANOTHER threshold without a
 * new pass over the keys (what the reference can only do by re-running booleanmask_128,
 * python/spattn/mask_utils.py:306-334).  HBM-bound: reads the maxima once, writes lists and counts.
 * Same list layout and rules as fgattn_block_index_lists; scale and D only set the softmax scale. */
int fgattn_block_lists_from_maxima(int* kb_indices, int* kb_counts, int list_stride, const float* block_maxima,
                                   const float* max_q, const float* denom, float threshold, int batch, int heads,
                                   int seq, int D, int kv_seq_len, float scale, void* stream);

/* Largest scratch the library itself can lend: see fgattn_block_index_lists_noalloc. */
#define FGATTN_NOALLOC_SCRATCH_BYTES (64u << 20)

/* fgattn_block_index_lists for callers that are not allowed to touch the CUDA allocator at all.
 * (No counterpart in the reference: every reference entry point leaves allocation to PyTorch.)
 * Who needs this: code that runs inside a region where cudaMalloc is off limits -- the enqueue hook of
 * an inference-engine plugin, a latency-critical serving loop whose device memory was carved up once
 * at start-up, a host framework that forbids (or would serialise the whole device on) an allocation.
 * Such a caller still owns q, k, v, the lists and max_q / denom, but has nowhere to get the
 * block-maxima scratch from, so here the scratch is a 64 MiB array that lives inside the library
 * image (FGATTN_NOALLOC_SCRATCH_BYTES; every GPU that loads the library holds it until the process
 * exits).  One (batch, head) unit needs ceil(kv_seq_len/64) * ceil(seq/128)*128 * 4 bytes of it, so a
 * unit up to seq = kv_seq_len = 32768 fits; units are processed in as many head chunks as needed, and
 * a unit that does not fit returns FGATTN_SCRATCH_TOO_SMALL without launching anything.
 * Same arguments and results as fgattn_block_index_lists, minus the scratch pointer and with
 * kv_rows = seq (k / v as long as q: the k / v tensors MUST have exactly seq rows per head).  It calls no
 * cudaMalloc / cudaFree and no allocating library routine; bounded-wait time-outs go to the error
 * word that other entry points created if one exists, else to a word inside the library; fgattn_check
 * reads both (and allocates nothing itself), so it reports a time-out of this entry point even when
 * it is the only one ever called.
 * The first call on a device looks up the device address of the built-in array (once per device,
 * with that device current); make that first call outside any stream capture.
 * All calls share the one array and it keeps whatever the last call left in it (nothing in it needs
 * clearing: each call overwrites what it reads); two calls that overlap on the GPU -- different
 * streams, or different host threads -- race on it and must be serialised by the caller. */
int fgattn_block_index_lists_noalloc(int* kb_indices, int* kb_counts, int list_stride, float* max_q, float* denom,
                                     void* o, const void* q, const void* k, const void* v, float threshold,
                                     int batch, int heads, int seq, int D, int kv_seq_len, float scale, void* stream);

/* Block-sparse attention with the precomputed (max_q, denom) of the softmax over ALL keys: rows
 * of query block qb attend to the listed key blocks only, probabilities are not renormalised
 * (the masked attention of python/test_mask.py:37-54).  The gather of K/V tiles by index replaces
 * include/sparseattn_asyncgatherload_padded.cuh:130-256 and include/asyncloadutils.cuh:73-153.
 * `workspace` (device memory, >= fgattn_sp_attn_workspace_bytes, 16-byte aligned) holds the work queue
 * of the persistent kernel. */
int fgattn_sp_attn_blocks_ml(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                             const int* kb_counts, int list_stride, const float* max_q, const float* denom, int batch,
                             int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                             size_t workspace_bytes, void* stream);

/* Bytes of device workspace fgattn_sp_attn_blocks_ml / fgattn_sp_attn_blocks_hint need and
 * fgattn_sp_attn_blocks / fgattn_sp_attn / fgattn_booleanmask_128_listed can use (work-queue counter,
 * processing order of the query-block pairs, re-run flags).  The workspace is scratch: contents need not
 * survive the call, but two calls that may overlap on the device must not share it. */
size_t fgattn_sp_attn_workspace_bytes(int batch, int heads, int seq);

/* Bytes of the large workspace that lets fgattn_sp_attn take the block route (see there): the two queue
 * regions plus, per 128-row query block, the touched key blocks of its token list with their column
 * masks (12 bytes per query block and key block), a route flag and a per-row exponent hint. */
size_t fgattn_sp_attn_token_workspace_bytes(int batch, int heads, int seq, int kv_rows);

/* fgattn_sp_attn_blocks (renormalising softmax over the kept key blocks, the sp_attn semantics of
 * include/sparseattn_asyncgatherload_padded.cuh:198-249) at the speed of fgattn_sp_attn_blocks_ml, for
 * the case the reference replays most: lists cached from an earlier diffusion step meet new q, k
 * (python/spattn/sparseattn_functionals.py:110-113).  max_q_hint (fp32 [B,H,1,S_pad], the max_q layout)
 * is a per-row ESTIMATE of max_j q_i.k_j over the listed keys -- typically the max_q that
 * fgattn_block_index_lists wrote when the lists were built.  It only positions the exponent range
 * (the result does not depend on it): an estimate within about +-60/(scale*log2 e) of the true row
 * maximum is good; rows for which it is not (their probability sum overflows or underflows) are
 * detected and their query blocks are recomputed by the running-maximum kernel of
 * fgattn_sp_attn_blocks inside the same call, so the result is always that of fgattn_sp_attn_blocks
 * within rounding.  `workspace` as for fgattn_sp_attn_blocks_ml (required). */
int fgattn_sp_attn_blocks_hint(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                               const int* kb_counts, int list_stride, const float* max_q_hint, int batch, int heads,
                               int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Block-sparse attention with the renormalising softmax of the sp_attn operator (softmax over the kept
 * keys only, include/sparseattn_asyncgatherload_padded.cuh:198-249) on key-block lists.  `workspace`
 * (fgattn_sp_attn_workspace_bytes, scratch) is optional: with it the thread blocks take the groups of
 * query blocks longest list first, which shortens the end of the launch when list lengths differ; with
 * a null workspace they run in storage order.  The result is the same either way. */
int fgattn_sp_attn_blocks(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                          const int* kb_counts, int list_stride, int batch, int heads, int seq, int D, int kv_rows,
                          int kv_seq_len, float scale, void* workspace, size_t workspace_bytes, void* stream);

/* ---- one-bit-per-entry masks (mask caches) ---------------------------------------------------
 * Entry e of a row lives in byte e / 8, bit e % 8 (least significant bit first): the format of pack /
 * unpack in python/spattn/mask_utils.py:421-440, which CompressedBitMaskCache (:87-98) stores.  A
 * "row" is one (batch, head, query block); `width` entries per row, width % 8 == 0.  The same four
 * calls serve token masks (width = mask_stride) and 64x64 block maps (width >= number of key blocks). */

/* mask [rows, width] with elem_size 1 (bool / uint8) or 4 (int32), kept iff > 0 -> packed
 * [rows, width / 8].  Replaces pack (python/spattn/mask_utils.py:421-430). */
int fgattn_pack_mask(unsigned char* packed, const void* mask, int elem_size, long long rows, int width, void* stream);

/* packed -> mask of 0 / 1 entries (elem_size 1 or 4).  Replaces unpack
 * (python/spattn/mask_utils.py:433-440). */
int fgattn_unpack_mask(void* mask, int elem_size, const unsigned char* packed, long long rows, int width, void* stream);

/* packed mask rows -> ascending index lists [rows, list_stride] + counts [rows]: set bits at
 * positions < n_valid, in ascending order; unused slots = sentinel.  Does in one kernel what
 * CompressedBitMaskCache.get_mask_from_cache does as unpack + int conversion +
 * booleanmask_to_indexmask (python/spattn/mask_utils.py:89-93), without materialising the int32 mask. */
int fgattn_packedmask_to_indexmask(int* indices, int* num_indices, const unsigned char* packed, long long rows,
                                   int width, int list_stride, int n_valid, int sentinel, void* stream);

/* index lists -> packed mask rows: bit e is set iff e occurs among the first num_indices[r] entries
 * of row r and e < width.  (The reference caches packed masks only from the int mask; this is the
 * direct route from lists.) */
int fgattn_indexmask_to_packedmask(unsigned char* packed, const int* indices, const int* num_indices, long long rows,
                                   int list_stride, int width, void* stream);

/* ---- top-k selector ------------------------------------------------------------------------- */

/* Bytes of scratch fgattn_topk_indices needs (block means as two bf16 tensors + the fp32 score rows). */
size_t fgattn_topk_scratch_bytes(int batch, int heads, int seq, int D, int blocksz, int kv_seq_len);

/* Alternative list producer: for every block of `blocksz` query rows (the last block may be shorter)
 * score(key) = mean of the block's query rows . key * scale, and the select_k keys < kv_seq_len with the
 * largest score are listed in kv_indices int32 [B,H,ceil(S/blocksz),list_stride] in descending score
 * order (equal scores: smaller key index first); unused slots = list_stride; kv_num_indices = select_k.
 * The lists feed fgattn_sp_attn.  Scores are computed in fp32 from the bf16 inputs (the reference
 * rounds block means and scores to bf16, which makes its order among near-equal scores arbitrary).
 * select_k <= 8192.  Replaces qk_topkmask_indices (python/spattn/mask_utils.py:389-417). */
int fgattn_topk_indices(int* kv_indices, int* kv_num_indices, int list_stride, const void* q, const void* k,
                        int select_k, int batch, int heads, int seq, int D, int blocksz, int kv_rows, int kv_seq_len,
                        float scale, void* scratch, size_t scratch_bytes, void* stream);

/* ---- self-test ------------------------------------------------------------------------------- */

/* Launches one warp that waits, with a budget of budget_cycles clock cycles (1 .. 1e8), on an mbarrier
 * nobody arrives at.  The wait gives up, the kernel returns normally and the next fgattn_check on the
 * stream reports FGATTN_DEVICE_TIMEOUT with code 9001: the path every kernel of this library takes when
 * one of its bounded waits runs out, exercised without disturbing the GPU.  (The reference's kernels
 * wait without bound -- include/fullattn_tma.cuh:152-158 -- so it has nothing of the kind.) */
int fgattn_selftest_bounded_wait(long long budget_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FGATTN_B200_H_ */
