/*
 * msa_b200 -- C ABI of the B200 (sm_100a) kernels for MSA's Memory-Parallel routing and
 * sparse-attention hot path.
 *
 * Conventions
 *   - Every pointer is a raw address.  "device" pointers are CUDA device addresses
 *     (tensor.data_ptr() of a CUDA tensor); "host-mapped" pointers are device-visible
 *     addresses of pinned host memory.  The caller owns every buffer; the library borrows
 *     it for the lifetime of the enqueued work and never allocates on the hot path.
 *   - `stream` is a cudaStream_t passed as void*.  All work is enqueued asynchronously.
 *   - Strides are in ELEMENTS of the tensor's dtype unless the name says bytes.
 *   - Return value: MSA_OK, or a negative MSA_ERR_* after which msa_last_error() holds a
 *     message for the calling thread.  Argument errors are detected before any launch.
 *   - Kernels that wait on hardware barriers bound every wait; a wait that runs out sets
 *     a non-zero word in the caller's `status` buffer instead of hanging.
 *   - `status` buffers are device int32[4]: word 0 = code of a barrier wait that ran out (0 = none),
 *     word 1 = used by msa_selftest_bounded_wait, word 2 = number of indices a kernel found outside
 *     their table and skipped (chunk -> document ids in routing, winners in msa_gather_plan),
 *     word 3 = reserved.  Nothing is read or written through an index that failed its check.
 *
 * Reference interfaces are cited by path inside the EverMind-AI/MSA repository.
 */
#ifndef MSA_B200_H
#define MSA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSA_ABI_VERSION 2

enum msa_status {
  MSA_OK = 0,
  MSA_ERR_ARG = -1,         /* bad pointer / size / stride / alignment */
  MSA_ERR_UNSUPPORTED = -2, /* a mode the reference has but this build rejects */
  MSA_ERR_CUDA = -3,        /* a CUDA runtime or driver call failed */
  MSA_ERR_NO_DEVICE = -4    /* no sm_100 device is current */
};

enum msa_dtype { MSA_F32 = 0, MSA_BF16 = 1 };

/* query_reduce_method of the reference (src/msa_service.py:749-780) */
enum msa_query_reduce { MSA_QREDUCE_MAX = 0, MSA_QREDUCE_MEAN = 1, MSA_QREDUCE_LAST = 2 };

/* head_reduce_method / chunk_reduce_method of the reference (src/msa_service.py:740-745, 787-812) */
enum msa_head_reduce { MSA_HREDUCE_MEAN = 0, MSA_HREDUCE_MAX = 1 };
enum msa_chunk_reduce { MSA_CREDUCE_MAX = 0, MSA_CREDUCE_MEAN = 1 };

/* flags of msa_route_scores */
#define MSA_ROUTE_FORCE_SIMT 1u /* use the CUDA-core kernel even for bf16 (cross-checks) */
#define MSA_ROUTE_KEYS_BLOCKED 4u /* rk is in the tile-blocked layout of msa_router_keys_block (bf16 only) */
#define MSA_ROUTE_NO_INIT 2u    /* do not reset the score table first: it was reset by
                                   msa_route_table_reset or holds the scores of other chunk ranges.
                                   Every call must then cover whole documents. */

int msa_abi_version(void);
const char* msa_last_error(void);

/* ---------------------------------------------------------------------------------------
 * Stage 1: chunk bookkeeping.
 * Replaces the inline tensor code of src/msa/memory_sparse_attention.py:138-163
 * (doc-token mask, rank inside the document, chunk id, owning doc per chunk).
 *
 * doc_ids, attention_mask: device int64 [n_rows * row_len]; attention_mask may be NULL
 * (all ones).  A document is a run of equal doc_ids > 0 inside one row.
 * Outputs (device): token_index[i] = flat position of the i-th document token;
 * chunk_offsets[c] .. chunk_offsets[c+1] = range of chunk c in that token stream;
 * pooled_doc_ids[c] = doc id owning chunk c; counts[0] = #document tokens,
 * counts[1] = #chunks, counts[2] = 1 if max_chunks was too small (outputs truncated).
 * token_index needs n_rows*row_len entries, chunk_offsets max_chunks+1, pooled_doc_ids
 * max_chunks.  workspace: device, 8-byte aligned, msa_bookkeeping_workspace_bytes() bytes
 * (per-tile summaries of the multi-CTA scan).
 */
int64_t msa_bookkeeping_workspace_bytes(int32_t n_rows, int32_t row_len);

int msa_chunk_bookkeeping(const int64_t* doc_ids, const int64_t* attention_mask, int32_t n_rows,
                          int32_t row_len, int32_t pooling_kernel_size, int32_t* token_index,
                          int32_t* chunk_offsets, int64_t* pooled_doc_ids, int32_t max_chunks,
                          int32_t* counts, void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage 1: chunk-mean pooling (+ optional L2 normalisation of the pooled rows).
 * Replaces MemorySparseAttention.sequence_pooling_kv
 * (src/msa/memory_sparse_attention.py:467-486), the inline K_r pooling (:177-190) and
 * F.normalize of the pooled router keys (:192-194).
 *
 * states: device, element (row r, head h, d) at states[r*token_stride + h*head_stride + d].
 * Row of the i-th document token is token_index[i] (or i when token_index is NULL).
 * out: element (chunk c, head h, d) at out[c*out_chunk_stride + h*out_head_stride + d].
 * Mean over the tokens actually in the chunk, fp32 accumulation, result in `dtype`.
 * n_chunks_dev (nullable): device int32 holding the live chunk count (<= n_chunks).
 * Requires n_heads*head_dim*sizeof(dtype)/16 to divide 256 and head_dim*sizeof/16 <= 32.
 */
int msa_pool_chunks(const void* states, int32_t dtype, int64_t token_stride, int64_t head_stride,
                    const int32_t* token_index, const int32_t* chunk_offsets,
                    const int32_t* n_chunks_dev, int32_t n_chunks, int32_t n_heads,
                    int32_t head_dim, void* out, int64_t out_chunk_stride, int64_t out_head_stride,
                    int32_t l2_normalize, void* stream);

/* ---------------------------------------------------------------------------------------
 * Routing, step 1: fold the query heads.
 * Replaces the view/scale/pad part of MSAService._gather_querys
 * (src/msa_service.py:1095-1100), F.normalize of the routing query
 * (src/msa/memory_sparse_attention.py:264-265) and, because the head reduction is a mean,
 * the 4x redundant per-group matmul of Memory.prefill_stage2 (src/msa_service.py:730-745):
 * folded[b, s, h, :] = sum_g q[b, h*G + g, s, :], so one 1024-wide dot product per
 * (token, chunk) gives the head-mean score after scaling by alpha = scale/(Hkv*G).
 *
 * q: device [B, Hq, S, D] addressed by strides (D contiguous).  query_mask: device uint8
 * [B, S] (row stride mask_stride_b), non-zero = routing-query token.
 * query_reduce MAX keeps S rows per sequence (padded to s_pad rows; pad and masked rows get
 * row_bias = -inf).  MEAN / LAST reduce the tokens here (mean of valid tokens / last valid
 * token) and need s_pad == 1.
 * q_folded: device [B*s_pad, Hkv*D] in `dtype`; row_bias: device float [B*s_pad].
 */
int msa_fold_queries(const void* q, int32_t dtype, int64_t stride_b, int64_t stride_h,
                     int64_t stride_s, const uint8_t* query_mask, int64_t mask_stride_b,
                     int32_t n_seq, int32_t n_q_heads, int32_t n_groups, int32_t seq_len,
                     int32_t head_dim, int32_t l2_normalize, int32_t query_reduce, int32_t s_pad,
                     void* q_folded, float* row_bias, void* stream);

/* ---------------------------------------------------------------------------------------
 * Tile-blocked router keys.  (Layout of this library; the reference keeps K_r as [1, Hkv, C, D],
 * src/msa_service.py:481-492.)  The routing kernels fetch 128 chunks x one 128-byte K block per copy.  In the
 * row-major [C, kdim] layout that is 128 pieces 2 KiB apart; in the blocked layout
 * [ceil(C/128) tiles][kdim/64 K blocks][128 chunks][64 elements] it is 16 contiguous KiB, which the bandwidth-bound
 * (decode-time) routing reads about 19 % faster from HBM (5.7 -> 6.8 TB/s measured on B200).  The results are
 * bit-identical to the row-major layout.
 * msa_router_keys_blocked_bytes: size of the blocked storage (whole tiles; zero it once so that padding rows are
 * finite); -1 for a kdim that is not a multiple of 64.
 * msa_router_keys_block: writes rows first_chunk .. first_chunk + n_rows - 1 (given row-major at rk_rows, row r of
 * the call = chunk first_chunk + r) into the blocked storage.  bf16 only.  Pass the blocked storage to
 * msa_route_scores with MSA_ROUTE_KEYS_BLOCKED (n_chunks = the real chunk count, rk_chunk_stride ignored).
 */
int64_t msa_router_keys_blocked_bytes(int32_t n_chunks, int32_t kdim);
int msa_router_keys_block(const void* rk_rows, int64_t rk_chunk_stride, int32_t first_chunk, int32_t n_rows,
                          int32_t kdim, void* rk_blocked, void* stream);

/* Rows per sequence msa_route_scores wants for a query of seq_len tokens (>= seq_len). */
int32_t msa_route_s_pad(int32_t seq_len, int32_t query_reduce);

/* ---------------------------------------------------------------------------------------
 * Routing, step 2: score + reduce.
 * Replaces the slice loop of Memory.prefill_stage2 (src/msa_service.py:716-821): matmul,
 * masked_fill, head mean, token max, chunk->doc amax, for head_reduce "mean",
 * chunk_reduce "max".  Per-(token, chunk) scores stay on chip.
 *
 * q_folded / row_bias: output of msa_fold_queries (n_seq sequences of s_pad rows).
 * rk: device pooled router keys, chunk c at rk + c*rk_chunk_stride, kdim contiguous elements.
 * chunk_doc: device int32 [n_chunks], 1-based local doc id of each chunk (the reference's
 * BlockDesc.pool_ids, src/msa_service.py:196-198), non-decreasing.  An id outside 1..n_docs is never
 * used as a column: the chunk is skipped and counted in status[2].
 * score_keys: device uint32 [n_seq, table_stride]; column d (0..n_docs) receives the
 * order-preserving key of max(min_val, alpha * max_tokens max_chunks dot).  Column 0 is the
 * reference's dummy document (src/msa_service.py:716-717).  Decode with msa_topk_select.
 * bf16 runs on the tcgen05 tensor-core kernel (needs kdim % 64 == 0, 16-byte aligned rows,
 * s_pad == 1 or s_pad % 16 == 0); fp32 runs on the CUDA-core kernel.
 * status: device int32 [4], zero on success; word 0 != 0 reports a barrier wait that ran out.
 */
int msa_route_scores(const void* q_folded, const float* row_bias, int32_t dtype, int32_t n_seq,
                     int32_t s_pad, const void* rk, int64_t rk_chunk_stride, int32_t n_chunks,
                     int32_t kdim, const int32_t* chunk_doc, float alpha, uint32_t* score_keys,
                     int64_t table_stride, int32_t n_docs, float min_val, uint32_t flags,
                     int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Routing in the other reduce modes of Memory.prefill_stage2 (src/msa_service.py:740-745 head_reduce
 * "max", :794-812 chunk_reduce "mean").  Both go through a per-(sequence, chunk) table of keys,
 * chunk_keys uint32 [n_seq, chunk_table_stride] with chunk c in column c + 1 (column 0 unused):
 *
 *   - head "mean": fill it with msa_route_scores, passing chunk_doc[c] = c + 1 and n_docs = n_chunks
 *     (every chunk its own document), i.e. on the tensor-core kernel for bf16;
 *   - head "max": msa_route_chunk_scores computes, per (sequence, chunk), the query_reduce over the valid
 *     tokens of the max (or mean) over all n_q_heads of q[b, head, s, :] . rk[chunk, head / n_groups, :], times
 *     `scale`, on CUDA cores.  q is the UNFOLDED query [B, Hq, S, D] by strides; rk chunk major as in
 *     msa_route_scores.  Writes max(min_val, score) as keys, every (sequence, chunk) exactly once;
 *   - msa_route_reduce_chunks then reduces the chunks of every document (runs of equal ids in chunk_doc) with
 *     max or mean into score_keys [n_seq, table_stride] (atomicMax: reset it first with
 *     msa_route_table_reset).  With "mean" a document must lie wholly inside one call.  Ids outside 1..n_docs
 *     are skipped and counted in status[2] (status may be NULL).
 */
int msa_route_chunk_scores(const void* q, int32_t dtype, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                           const uint8_t* query_mask, int64_t mask_stride_b, int32_t n_seq, int32_t n_q_heads,
                           int32_t n_groups, int32_t seq_len, int32_t head_dim, int32_t head_reduce,
                           int32_t query_reduce, const void* rk, int64_t rk_chunk_stride, int32_t n_chunks,
                           float scale, float min_val, uint32_t* chunk_keys, int64_t chunk_table_stride,
                           void* stream);

int msa_route_reduce_chunks(const uint32_t* chunk_keys, int64_t chunk_table_stride, int32_t n_seq,
                            int32_t n_chunks, const int32_t* chunk_doc, int32_t n_docs, int32_t chunk_reduce,
                            float min_val, uint32_t* score_keys, int64_t table_stride, int32_t* status,
                            void* stream);

/* Failure-path self-test: launches one CTA that waits, with the routing kernel's bounded-wait
 * routine and the given limit (<= 1 s), on a barrier that nothing completes.  After the stream
 * drains, status[0] == 9 and status[1] == 1: the wait gave up and the kernel returned; the
 * context stays usable.  (No counterpart in the reference, whose waits are unbounded:
 * src/msa_service.py:1427-1442, 1904.) */
int msa_selftest_bounded_wait(int64_t limit_ns, int32_t* status, void* stream);

/* Resets a score table to min_val (and `status`, when given, to zero).  msa_route_scores does
 * this itself unless MSA_ROUTE_NO_INIT is set; the separate entry point exists so that a bank
 * scored in several calls (or a caller timing the scoring kernel alone) resets once.
 * Counterpart of torch.full((bsz, total_docs), min_val) at src/msa_service.py:716-717. */
int msa_route_table_reset(uint32_t* score_keys, int64_t table_stride, int32_t n_docs, int32_t n_seq,
                          float min_val, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Routing, step 3: exact per-shard top-k in two levels: every CTA keeps the best k of one
 * 2048-column slice of a row, a second launch reduces the survivors.  k <= 32: threshold at the
 * k-th largest lane maximum, compaction, ranks by counting; k <= 64: rounds of a warp arg-max;
 * larger k: a shared-memory bitonic sort.
 * Replaces torch.topk + create_global_doc_ids (src/msa_service.py:826-828).
 * Selects k_eff = min(k, n_cols) columns per row, sorted by descending score; equal scores
 * are ordered by ascending column.  out_* are [n_seq, k_eff].  doc_ids_table (nullable) is the
 * local->global table (BlockDesc.doc_ids, src/msa_service.py:199-201, 218-219).
 * workspace: device, msa_topk_workspace_bytes(n_seq, n_cols, k) bytes (0 for rows up to 2048).
 * Limits: k <= 1024, n_seq <= 65535, n_cols * k <= 2^26.
 */
int64_t msa_topk_workspace_bytes(int32_t n_seq, int32_t n_cols, int32_t k);

int msa_topk_select(const uint32_t* score_keys, int64_t table_stride, int32_t n_seq,
                    int32_t n_cols, int32_t k, const int64_t* doc_ids_table, float* out_scores,
                    int64_t* out_local_ids, int64_t* out_global_ids, void* workspace,
                    int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * Routing, steps 2 + 3 in one call for decode-time routing (one query row per sequence).
 * Same result as msa_route_scores followed by msa_topk_select (src/msa_service.py:716-828 with one token per
 * query), without the [n_seq, n_docs + 1] score table: every CTA scores the documents that start in its share of
 * the 128-chunk tiles, keeps their scores in shared memory, selects its best k per sequence there, and a
 * second small launch reduces the per-CTA candidates.  The scoring is bound by HBM (the
 * shard's router keys are read once).
 *
 * q_folded / row_bias: output of msa_fold_queries with s_pad == 1 (n_seq rows).  rk, chunk_doc, alpha, n_docs,
 * min_val, doc_ids_table, out_*: as in msa_route_scores / msa_topk_select; out_* are [n_seq, min(k, n_docs + 1)].
 * workspace: device, msa_route_score_select_workspace_bytes(n_seq, k) bytes (per-CTA candidates; -1 = no device).
 * flags: 0, or MSA_ROUTE_KEYS_BLOCKED when rk is the tile-blocked copy made by msa_router_keys_block
 * (rk_chunk_stride is then ignored).
 * status: device int32[4], written only on error (zero it once): word 0 = a barrier wait ran out, word 2 =
 * chunk -> document ids outside 1..n_docs (or not non-decreasing) were skipped.
 * Takes bf16, n_seq <= 128, k <= 32, kdim % 64 == 0; other shapes return MSA_ERR_UNSUPPORTED before any launch
 * (use the two-call path).
 */
int64_t msa_route_score_select_workspace_bytes(int32_t n_seq, int32_t k);

int msa_route_score_select(const void* q_folded, const float* row_bias, int32_t dtype, int32_t n_seq,
                           const void* rk, int64_t rk_chunk_stride, int32_t n_chunks, int32_t kdim,
                           const int32_t* chunk_doc, float alpha, int32_t n_docs, float min_val, int32_t k,
                           const int64_t* doc_ids_table, float* out_scores, int64_t* out_local_ids,
                           int64_t* out_global_ids, void* workspace, int64_t workspace_bytes,
                           uint32_t flags, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Cross-rank merge of the per-shard candidates.
 * Replaces steps 4-5 of MSAService.doc_query (src/msa_service.py:1174-1196): top-k over
 * the W*kc candidates of each query, owner rank of each winner, invalidation of winners
 * whose score is <= invalid_below (-1e9 in the reference, :1190).
 * cand_*: device, candidate (w, b, j) at element index w*stride_w + b*kc + j of cand_scores and at
 * w*stride_w_ids + b*kc + j of cand_local / cand_global (two strides, so that the three arrays can be
 * planes of one all-gathered buffer: float scores and 64-bit ids have different element sizes).
 * Outputs [n_seq, k]: scores, local ids (-1 where invalid), global ids, owner ranks.
 * Ties: lower rank, then lower position first.  Requires W*kc <= 4096.
 */
int msa_topk_merge(const float* cand_scores, const int64_t* cand_local, const int64_t* cand_global,
                   int64_t stride_w, int64_t stride_w_ids, int32_t world, int32_t n_seq, int32_t kc, int32_t k,
                   float invalid_below, float* out_scores, int64_t* out_local, int64_t* out_global,
                   int32_t* out_rank, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fetch of the selected documents' pooled K/V from pinned host memory.
 * Replaces steps 5-8 of MSAService.doc_query (src/msa_service.py:1193-1312): request
 * exchange, CPU index build, index_select on the pinned bank, H2D, all-to-all-v, regroup.
 *
 * Bank layout (this library's): per shard one host-mapped array [chunks, 2, Hkv, D]
 * (K then V per chunk), so a document is one contiguous run.  The directory lives on the
 * device: shard_doc_base[w] = first row of shard w in doc_chunk_offset / doc_chunk_len
 * (indexed by shard_doc_base[w] + local id, slot 0 = dummy of length 0);
 * shard_kv_base[w] = host-mapped address of shard w's array.
 *
 * msa_gather_plan: orders each sample's valid winners by (owner rank, local id), as the
 * reference's exchange does, and computes where their chunks go.  plan is device int64
 * [n_seq*k, 4] = (source address, chunks, destination entry, sample); n_sel device int64
 * [n_seq]; total device int64 [1] (also written to *total_host_mapped when non-NULL).
 * n_dir_rows = number of rows of doc_chunk_offset / doc_chunk_len; shard w owns rows
 * shard_doc_base[w] .. shard_doc_base[w+1]-1 (the last shard up to n_dir_rows-1).  A winner whose
 * owner rank is not in 0..world-1 or whose local id is not a row of its shard is dropped and counted
 * in status[2] (status may be NULL); local ids <= 0 (dummy document, invalidated winner) select nothing.
 * sample_stride == 0: samples are packed one after another (destination entry counts from the start of
 * the output).  sample_stride > 0: destination entries count from the start of the SAMPLE and a sample
 * takes at most sample_stride entries (documents beyond that are cut); pass the same layout to
 * msa_gather_run through out_sample_stride.
 * msa_gather_run: copies every planned document into out_k / out_v.  Packed (out_sample_stride == 0):
 * device [Hkv, out_entries, D] (entry stride = D, head stride = out_head_stride elements).  Per sample
 * (out_sample_stride > 0, in elements): entry e of sample b, head h goes to
 * out + b*out_sample_stride + h*out_head_stride + e*D and out_entries is the room of ONE sample, so the
 * gather can write straight into the retrieved segment of a [B, Hkv, L, D] cache.  Entries that have no
 * room are not read.
 * max_ctas: 0 = one CTA per document (fastest next to compute-bound kernels: 35 GB/s under the
 * prefill routing kernel); a small cap (24 measured best) when the fetch runs beside kernels that
 * saturate HBM, as in a decode step: the link is full from about a dozen CTAs, and reads queued
 * beyond that inside the GPU only delay the neighbours' memory traffic.
 */
/* Pins and maps [host_ptr, host_ptr+bytes) (memory the caller allocated, e.g. a shared-memory
 * file opened by every rank of the node; the reference pins its bank with pin_memory=True,
 * src/msa_service.py:490-491) and returns the address the device uses for it. */
int msa_bank_register_host(void* host_ptr, int64_t bytes, uint64_t* device_address);
int msa_bank_unregister_host(void* host_ptr);

int msa_gather_plan(const int64_t* sel_local, const int32_t* sel_rank, int32_t n_seq, int32_t k,
                    int32_t world, const int64_t* shard_doc_base, int64_t n_dir_rows,
                    const int64_t* doc_chunk_offset, const int32_t* doc_chunk_len,
                    const uint64_t* shard_kv_base, int64_t chunk_bytes, int64_t sample_stride,
                    int64_t* plan, int64_t* n_sel, int64_t* total, int64_t* total_host_mapped,
                    int32_t* status, void* stream);

/* msa_gather_plan_resident: msa_gather_plan for a decode loop that refreshes the same per-sample segment every step
 * (what a per-step doc_query, src/msa_service.py:1193-1283, would fetch again and again).  A sample's room is k
 * slots of slot_len entries; resident [n_seq, k] int64 (filled with -1 by the caller before the first call, then
 * owned by this function) records which document (owner rank << 40 | local id) each slot holds.  For a sample whose
 * k winners are all valid and hold exactly slot_len entries each, the winners that already sit in a slot are left
 * there and only the others are planned, into the slots of the documents that dropped out (attention is indifferent
 * to the order of the entries); n_sel[b] is then k * slot_len.  Any other sample is planned in full, as by
 * msa_gather_plan with sample_stride = k * slot_len, and its row of the table is cleared.
 */
int msa_gather_plan_resident(const int64_t* sel_local, const int32_t* sel_rank, int32_t n_seq, int32_t k,
                             int32_t world, const int64_t* shard_doc_base, int64_t n_dir_rows,
                             const int64_t* doc_chunk_offset, const int32_t* doc_chunk_len,
                             const uint64_t* shard_kv_base, int64_t chunk_bytes, int32_t slot_len,
                             int64_t* resident, int64_t* plan, int64_t* n_sel, int64_t* total, int32_t* status,
                             void* stream);

int msa_gather_run(const int64_t* plan, int32_t n_items, int32_t dtype, int32_t n_kv_heads,
                   int32_t head_dim, void* out_k, void* out_v, int64_t out_head_stride,
                   int64_t out_entries, int64_t out_sample_stride, int32_t max_ctas, void* stream);

/* ---------------------------------------------------------------------------------------
 * Decode attention over the sparse context (split-KV flash-decode, GQA).
 * Replaces the decode branch of MemorySparseAttention
 * (src/msa/memory_sparse_attention.py:371-399): torch.cat of the cache, repeat_kv,
 * boolean-mask SDPA with q_len == 1.
 *
 * q: device [B, Hq, D].  k_cache / v_cache: device, element (b, h, pos, d) at
 * b*stride_b + h*stride_h + pos*D + d with capacity >= kv_start[b] + kv_len[b] + 1.
 * Sequence b's valid entries are positions kv_start[b] .. kv_start[b]+kv_len[b]-1
 * (kv_start NULL = 0; a left-padded cache of the reference has kv_start = maxL - kv_len).
 * new_k / new_v: device [B, Hkv, D] (nullable together): this step's key/value; they take
 * part in the attention and are appended in place at position kv_start[b] + kv_len[b].
 * out: device [B, Hq*D].  scale: softmax scale (D^-0.5 in the reference).
 * workspace: device, msa_decode_workspace_bytes(...) bytes (needed when n_splits > 1).
 */
int64_t msa_decode_workspace_bytes(int32_t n_seq, int32_t n_q_heads, int32_t head_dim,
                                   int32_t n_splits);

int msa_sparse_decode_attn(const void* q, int32_t dtype, void* k_cache, void* v_cache,
                           int64_t stride_b, int64_t stride_h, const int32_t* kv_start,
                           const int32_t* kv_len, const void* new_k, const void* new_v,
                           int32_t n_seq, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                           float scale, void* out, void* workspace, int64_t workspace_bytes,
                           int32_t n_splits, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage-2 sparse prefill: context assembly and causal attention.
 * Replace the packing, flash_attn_varlen_func call and left-padded re-pack of
 * src/msa/memory_sparse_attention.py:282-357.
 *
 * msa_assemble_context writes, for sequence b, the entries [template | its n_sel[b] retrieved
 * entries | its valid query tokens] into k_store / v_store (element (b, h, pos, d) at
 * b*store_stride_b + h*store_stride_h + pos*D + d) at positions max_kv-len_b .. max_kv-1, i.e.
 * left padded like the reference's compact cache but inside storage of store_len >= max_kv
 * positions, so decode can append in place; every other position of the storage is zero-filled
 * (the storage may be handed over uninitialised).  template_*: [Hkv, t, D] contiguous; sel_*: [Hkv, sum(n_sel), D]
 * with head stride sel_head_stride (msa_gather_run's output); q_k / q_v: this step's key/value
 * states [B, Hkv, S, D] by strides; valid: uint8 [B, S].  Outputs: kv_start[B], kv_len[B],
 * num_q[B] (valid query tokens), q_tok[B, S] (token index of the r-th valid token for r < num_q[b],
 * then the other tokens in order), error_flag
 * (1 if some len_b exceeds max_kv: that sequence's storage is zero-filled and its kv_start is negative).
 *
 * msa_sparse_prefill_attn: out[b, tok, hq*D + d] for every valid query token.  causal != 0: the token attends
 * to the template, all retrieved entries and the query tokens up to itself (bottom-right aligned causal
 * mask, stage 2).  causal == 0: every valid token attends to all kv_len[b] entries (the multi-token
 * segments of the reference's qa_mode, src/msa/memory_sparse_attention.py:375-380, after
 * msa_append_segment has put the segment's own tokens into the store).  q: [B, Hq, S, D] by strides; out:
 * [B, S, Hq*D] contiguous; the rows of invalid tokens are zero-filled.  bf16 with head_dim 128 runs on the
 * tensor-core kernel; fp32 and other head sizes (<= 256) on a general CUDA-core kernel.
 *
 * msa_append_segment: appends the valid tokens (valid: uint8 [B, S]) of seg_k / seg_v [B, Hkv, S, D] (by
 * strides) to every sequence's store at positions kv_start[b] + kv_len[b] .., in order, adds their number to
 * kv_len[b], and writes q_tok[B, S] (valid tokens first) and num_q[B] as msa_assemble_context does.  Tokens
 * whose mask is 0 are not stored: they are never attended to, so leaving them out keeps a sequence's valid
 * entries contiguous (the reference stores them and carries a mask instead).  error_flag is set to 1 when a
 * sequence's store (store_len positions) has no room; that sequence is left unchanged with num_q = 0.
 */
int msa_assemble_context(const void* template_k, const void* template_v, int32_t template_len,
                         const void* sel_k, const void* sel_v, int64_t sel_head_stride,
                         const int64_t* n_sel, const void* q_k, const void* q_v, int64_t q_stride_b,
                         int64_t q_stride_h, int64_t q_stride_s, const uint8_t* valid, int32_t n_seq,
                         int32_t seq_len, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                         int32_t max_kv, int32_t store_len, void* k_store, void* v_store, int64_t store_stride_b,
                         int64_t store_stride_h, int32_t* kv_start, int32_t* kv_len, int32_t* q_tok,
                         int32_t* num_q, int32_t* error_flag, void* stream);

int msa_sparse_prefill_attn(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                            const void* k_store, const void* v_store, int64_t store_stride_b,
                            int64_t store_stride_h, const int32_t* kv_start, const int32_t* kv_len,
                            const int32_t* q_tok, const int32_t* num_q, int32_t n_seq, int32_t seq_len,
                            int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                            int32_t causal, float scale, void* out, void* stream);

int msa_append_segment(const void* seg_k, const void* seg_v, int64_t seg_stride_b, int64_t seg_stride_h,
                       int64_t seg_stride_s, const uint8_t* valid, int32_t n_seq, int32_t seq_len,
                       int32_t n_kv_heads, int32_t head_dim, int32_t dtype, void* k_store, void* v_store,
                       int64_t store_stride_b, int64_t store_stride_h, int32_t store_len,
                       const int32_t* kv_start, int32_t* kv_len, int32_t* q_tok, int32_t* num_q,
                       int32_t* error_flag, void* stream);

/* ---------------------------------------------------------------------------------------
 * Stage-1 attention inside every document, with the chunk means of K and V as a by-product.
 * Replaces flash_attn_varlen_func over the document tokens and the K / V pooling of
 * src/msa/memory_sparse_attention.py:216-241 and :166-176.  bf16 with head_dim 128 runs on tensor cores; fp32
 * and other head sizes (<= 256) on a general CUDA-core kernel, without the pooling by-product (chunk_offsets
 * must then be NULL).
 *
 * token_index[Td]: flat positions b*seq_len + s of the tokens that take part, document after
 * document (msa_chunk_bookkeeping's order); seg_offsets[n_segments + 1]: where each document starts
 * in token_index.  q: [B, Hq, S, D], k / v: [B, Hkv, S, D] by strides.  out: [B, S, Hq*D]
 * contiguous; only the rows of listed tokens are written.  A token attends to the tokens of its own
 * segment up to itself.  With chunk_offsets != NULL (msa_chunk_bookkeeping's table, n_chunks + 1
 * entries, every document starting a chunk), pooled_k / pooled_v receive the mean K and V of every
 * chunk (element (c, h, d) at c*pool_chunk_stride + h*pool_head_stride + d), accumulated in fp32 and
 * rounded once; pool_size must be a multiple of 32.  K_r is not read by attention and is pooled by
 * msa_pool_chunks.  At most 65535 segments per call.
 */
int msa_doc_attention_pool(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                           const void* k, const void* v, int64_t k_stride_b, int64_t k_stride_h,
                           int64_t k_stride_s, const int32_t* token_index, const int32_t* seg_offsets,
                           int32_t n_segments, int32_t max_segment_len, int32_t seq_len, int32_t n_q_heads,
                           int32_t n_kv_heads, int32_t head_dim, int32_t dtype, float scale, void* out,
                           const int32_t* chunk_offsets, int32_t n_chunks, int32_t pool_size, void* pooled_k,
                           void* pooled_v, int64_t pool_chunk_stride, int64_t pool_head_stride, void* stream);

/* msa_doc_attention_tc: the same attention as msa_doc_attention_pool (without the pooling by-product) on
 * tcgen05 tensor cores, for segments that are runs of CONSECUTIVE tokens of one row (token_index of a
 * segment ascending by one; the caller checks this, e.g. documents without masked tokens).  q, k, v must
 * be token-major ([B, S, H, D] storage viewed as [B, H, S, D]; the row stride may exceed H*D) or contiguous
 * head-major tensors; anything else is rejected with MSA_ERR_ARG and belongs to msa_doc_attention_pool.
 * The tiles TMA brings in reach up to 127 positions past a document's end (the next document's rows, padding
 * positions, or zero fill past the tensor): their scores are masked, but V rows there are multiplied by zero
 * probabilities, so they must hold finite numbers (projections of any token do).
 * status: int32[4], zeroed by the caller; status[0] != 0 after completion means a bounded barrier wait ran
 * out inside the kernel (output invalid).
 */
int msa_doc_attention_tc(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, const void* k,
                         const void* v, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                         const int32_t* token_index, const int32_t* seg_offsets, int32_t n_segments,
                         int32_t max_segment_len, int32_t n_seq, int32_t seq_len, int32_t n_q_heads,
                         int32_t n_kv_heads, int32_t head_dim, int32_t dtype, float scale, void* out,
                         int32_t* status, void* stream);

/* msa_doc_attention_tc_masked: msa_doc_attention_tc for documents with tokens inside them that do not take part
 * (attention mask 0: src/msa/memory_sparse_attention.py:216-241 indexes them away before the attention call).  A
 * segment is the SPAN of memory from a document's first to its last participating token: span_index lists every
 * position of the span (ascending by one), span_offsets the spans, and valid_bits (bit p of the bitmap = flat token
 * position p takes part; n_bit_words 32-bit words, covering every token plus 256 positions, plus one more word)
 * says which of them are tokens of the document.  The others are never attended to and their rows of out are left
 * as they are; causality follows the position in the span, which orders the participating tokens as the
 * reference's compacted list does.  Spans of different documents must not overlap (documents that are packed one
 * after the other, as the reference's blocks are, never do).
 */
int msa_doc_attention_tc_masked(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, const void* k,
                                const void* v, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                const int32_t* span_index, const int32_t* span_offsets, int32_t n_segments,
                                int32_t max_span_len, int32_t n_seq, int32_t seq_len, int32_t n_q_heads,
                                int32_t n_kv_heads, int32_t head_dim, int32_t dtype, float scale, void* out,
                                const uint32_t* valid_bits, int64_t n_bit_words, int32_t* status, void* stream);

/* msa_sparse_prefill_attn_tc: msa_sparse_prefill_attn (same arguments, same result, rows of tokens that are not
 * queries zero-filled) on the tcgen05 kernel of msa_doc_attention_tc, for the case that the valid tokens of every
 * sequence are ONE run of consecutive tokens (q_tok[b, r] = q_tok[b, 0] + r for r < num_q[b]; the caller checks
 * this: left- or right-padded segments are, tokens masked in the middle are not).  bf16, head_dim 128; q
 * token-major or contiguous head-major; the stores contiguous [B, Hkv, store_len, D] whose positions outside a
 * sequence's entries hold finite numbers (msa_assemble_context zero-fills them).  Replaces the attention call of
 * src/msa/memory_sparse_attention.py:334-339 (stage 2, causal != 0) and :375-380 (causal == 0).
 * status: int32[4], zeroed by the caller; status[0] != 0 after completion means a bounded barrier wait ran
 * out inside the kernel (output invalid).
 */
int msa_sparse_prefill_attn_tc(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                               const void* k_store, const void* v_store, int64_t store_stride_b,
                               int64_t store_stride_h, int32_t store_len, const int32_t* kv_start,
                               const int32_t* kv_len, const int32_t* q_tok, const int32_t* num_q, int32_t n_seq,
                               int32_t seq_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                               int32_t dtype, int32_t causal, float scale, void* out, int32_t* status,
                               void* stream);

/* ---------------------------------------------------------------------------------------
 * Dense glue of a decode step (bf16).  No single reference function: they replace the chains of
 * elementwise torch kernels that transformers' Qwen3 modules issue between the GEMMs of a layer as
 * driven by src/msa/model.py:67-135 (Qwen3RMSNorm on q / k heads + apply_rotary_pos_emb; residual add
 * + Qwen3RMSNorm; SiLU(gate) * up).  Each computes in fp32 and rounds once per module boundary.
 *
 * msa_qk_norm_rope: qkv row b = [n_q_heads*128 | n_kv_heads*128 | ...] (row_stride elements apart);
 *   q_out[b, h, :] = rope(rmsnorm(q head) * q_weight), k_out likewise; cos_table / sin_table: [n_seq, 128]
 *   (rotate-half convention, the sequence's position already applied).  head_dim must be 128.
 * msa_add_rmsnorm: x_out = x + y (y, x_out may be NULL: no add), h_out = rmsnorm(x_out) * weight; rows of
 *   `hidden` contiguous elements.
 * msa_silu_mul: out[r, j] = silu(gate_up[r, j]) * gate_up[r, ffn + j], out rows contiguous.
 */
int msa_qk_norm_rope(const void* qkv, int64_t row_stride, int32_t n_seq, int32_t n_q_heads, int32_t n_kv_heads,
                     int32_t head_dim, const void* q_weight, const void* k_weight, float eps,
                     const void* cos_table, const void* sin_table, void* q_out, void* k_out, void* stream);
int msa_add_rmsnorm(const void* x, const void* y, const void* weight, float eps, int32_t n_rows, int32_t hidden,
                    void* x_out, void* h_out, void* stream);
int msa_silu_mul(const void* gate_up, int64_t row_stride, int32_t n_rows, int32_t ffn, void* out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Decode attention without any allocation.  (No counterpart in the reference: this entry
 * point exists for hosts of this library that cannot allocate device memory when a decode
 * step runs -- a serving loop whose pool already owns the whole GPU, a plugin that is handed
 * only its inputs and outputs, a policy that forbids allocation after start-up.)
 *
 * Same computation and arguments as msa_sparse_decode_attn, but the split-KV partials go to
 * an 8 MiB array built into the library (msa_decode_static_scratch_bytes()); every GPU that
 * loads the library holds that array until the process exits.  A call whose
 * msa_decode_workspace_bytes(n_seq, n_q_heads, head_dim, n_splits) exceeds it is rejected
 * with MSA_ERR_ARG before anything is launched.  The call itself performs no cudaMalloc,
 * cudaFree or other allocating call.
 *
 * The first call on each device resolves the array's device address (with that device
 * current) and caches it; make that first call outside of any stream capture.
 * All calls on a device share the one array.  Nothing in it has to start at zero -- every
 * launch rewrites every partial it later reads -- but two calls whose kernels overlap on the
 * GPU (different streams, no ordering between them) race on it: order them.
 */
int64_t msa_decode_static_scratch_bytes(void);

int msa_sparse_decode_attn_static(const void* q, int32_t dtype, void* k_cache, void* v_cache,
                                  int64_t stride_b, int64_t stride_h, const int32_t* kv_start,
                                  const int32_t* kv_len, const void* new_k, const void* new_v,
                                  int32_t n_seq, int32_t n_q_heads, int32_t n_kv_heads,
                                  int32_t head_dim, float scale, void* out, int32_t n_splits,
                                  void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MSA_B200_H */
