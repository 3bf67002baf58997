// Exact top-k over the document score table (block radix select) and the cross-rank merge.
//
// Scores live in the table as order-preserving uint32 keys, so selection is four 8-bit radix
// passes over one row per CTA: each pass histograms the next byte of the keys that still
// match the prefix found so far and narrows the prefix to the bucket holding the k-th
// largest key.  The winners are then gathered and sorted in shared memory.  HBM/L2 bound:
// 5 reads of the row, nothing written but the k results.
#include "common.cuh"

namespace msa {

constexpr int kSelThreads = 256;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kMaxK = 1024;

__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const uint32_t* __restrict__ keys, long long table_stride, int n_cols, int k,
                   const int64_t* __restrict__ doc_ids_table, float* __restrict__ out_scores,
                   int64_t* __restrict__ out_local, int64_t* __restrict__ out_global) {
  __shared__ unsigned int s_hist[kSelWarps][256];
  __shared__ unsigned int s_prefix, s_krem, s_count_gt, s_count_eq;
  __shared__ unsigned int s_warp_eq[kSelWarps];
  __shared__ unsigned long long s_win[kMaxK];
  const uint32_t* row = keys + (long long)blockIdx.x * table_stride;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int k_eff = min(k, n_cols);

  uint32_t prefix = 0, mask = 0;
  unsigned int k_rem = k_eff;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < kSelWarps * 256; i += kSelThreads) (&s_hist[0][0])[i] = 0;
    __syncthreads();
    for (int i = tid; i < n_cols; i += kSelThreads) {
      const uint32_t key = row[i];
      if ((key & mask) == prefix) atomicAdd(&s_hist[warp][(key >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    // thread b owns bucket b: suffix counts via a shared-memory scan from the top bucket down
    unsigned int mine = 0;
    for (int w = 0; w < kSelWarps; ++w) mine += s_hist[w][tid];
    __syncthreads();
    s_hist[0][tid] = mine;
    __syncthreads();
    for (int d = 1; d < 256; d <<= 1) {  // inclusive suffix sum
      unsigned int other = (tid + d < 256) ? s_hist[0][tid + d] : 0u;
      __syncthreads();
      s_hist[0][tid] += other;
      __syncthreads();
    }
    const unsigned int ge = s_hist[0][tid], gt = ge - mine;
    if (gt < k_rem && k_rem <= ge) {  // exactly one bucket satisfies this
      s_prefix = prefix | ((uint32_t)tid << shift);
      s_krem = k_rem - gt;
    }
    __syncthreads();
    prefix = s_prefix;
    k_rem = s_krem;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  // prefix is now the k-th largest key; take everything above it and the first k_rem equal to it
  if (tid == 0) { s_count_gt = 0; s_count_eq = 0; }
  __syncthreads();
  const unsigned int n_gt = k_eff - k_rem;
  for (int base = 0; base < n_cols; base += kSelThreads) {
    const int i = base + tid;
    const uint32_t key = i < n_cols ? row[i] : 0u;
    const bool gt = i < n_cols && key > prefix;
    const bool eq = i < n_cols && key == prefix;
    if (gt) {
      const unsigned int slot = atomicAdd(&s_count_gt, 1u);
      s_win[slot] = ((unsigned long long)key << 32) | (0xffffffffu - (uint32_t)i);
    }
    const unsigned int bal = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) s_warp_eq[warp] = __popc(bal);
    __syncthreads();
    unsigned int before = s_count_eq;
    for (int w = 0; w < warp; ++w) before += s_warp_eq[w];
    const unsigned int ord = before + __popc(bal & ((1u << lane) - 1u));
    if (eq && ord < k_rem) s_win[n_gt + ord] = ((unsigned long long)key << 32) | (0xffffffffu - (uint32_t)i);
    __syncthreads();
    if (tid == 0) {
      unsigned int tot = 0;
      for (int w = 0; w < kSelWarps; ++w) tot += s_warp_eq[w];
      s_count_eq += tot;
    }
    __syncthreads();
  }
  // bitonic sort, descending, of the winners (key high, inverted column low => ties by column asc)
  int n2 = 1;
  while (n2 < k_eff) n2 <<= 1;
  for (int i = k_eff + tid; i < n2; i += kSelThreads) s_win[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < n2; i += kSelThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const unsigned long long a = s_win[i], b = s_win[j];
          if (desc ? a < b : a > b) { s_win[i] = b; s_win[j] = a; }
        }
      }
      __syncthreads();
    }
  for (int i = tid; i < k_eff; i += kSelThreads) {
    const unsigned long long w = s_win[i];
    const long long col = 0xffffffffu - (uint32_t)(w & 0xffffffffull);
    const long long o = (long long)blockIdx.x * k_eff + i;
    out_scores[o] = key_to_float((uint32_t)(w >> 32));
    out_local[o] = col;
    if (out_global) out_global[o] = doc_ids_table ? doc_ids_table[col] : col;
  }
}

// One CTA per query: rank every candidate by counting the candidates that beat it.
constexpr int kMergeThreads = 128;
constexpr int kMergeMax = 4096;

__global__ void __launch_bounds__(kMergeThreads)
topk_merge_kernel(const float* __restrict__ cand_scores, const int64_t* __restrict__ cand_local,
                  const int64_t* __restrict__ cand_global, long long stride_w, int world, int kc, int k,
                  float invalid_below, float* __restrict__ out_scores, int64_t* __restrict__ out_local,
                  int64_t* __restrict__ out_global, int32_t* __restrict__ out_rank) {
  __shared__ unsigned long long s_key[kMergeMax];
  const int b = blockIdx.x, n = world * kc;
  for (int p = threadIdx.x; p < n; p += kMergeThreads) {
    const int w = p / kc, j = p % kc;
    const float s = cand_scores[(long long)w * stride_w + (long long)b * kc + j];
    s_key[p] = ((unsigned long long)float_to_key(s) << 32) | (0xffffffffu - (uint32_t)p);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n; p += kMergeThreads) {
    const unsigned long long mine = s_key[p];
    int rank = 0;
    for (int o = 0; o < n; ++o) rank += s_key[o] > mine ? 1 : 0;
    if (rank < k) {
      const int w = p / kc, j = p % kc;
      const long long src = (long long)w * stride_w + (long long)b * kc + j;
      const float s = cand_scores[src];
      const long long o = (long long)b * k + rank;
      out_scores[o] = s;
      out_local[o] = s > invalid_below ? cand_local[src] : -1;
      out_global[o] = cand_global[src];
      out_rank[o] = w;
    }
  }
}

}  // namespace msa

using namespace msa;

extern "C" int msa_topk_select(const uint32_t* score_keys, int64_t table_stride, int32_t n_seq, int32_t n_cols,
                               int32_t k, const int64_t* doc_ids_table, float* out_scores, int64_t* out_local_ids,
                               int64_t* out_global_ids, void* stream) {
  MSA_REQUIRE(score_keys && out_scores && out_local_ids, "topk_select: null pointer");
  MSA_REQUIRE(n_seq >= 0 && n_cols >= 1 && k >= 1, "topk_select: bad sizes (n_cols=%d k=%d)", n_cols, k);
  MSA_REQUIRE(k <= kMaxK, "topk_select: k=%d exceeds the supported maximum %d", k, kMaxK);
  MSA_REQUIRE(table_stride >= n_cols, "topk_select: table_stride < n_cols");
  if (n_seq == 0) return MSA_OK;
  topk_select_kernel<<<n_seq, kSelThreads, 0, (cudaStream_t)stream>>>(
      score_keys, table_stride, n_cols, k, doc_ids_table, out_scores, out_local_ids, out_global_ids);
  MSA_LAUNCH_OK("topk_select_kernel");
  return MSA_OK;
}

extern "C" int msa_topk_merge(const float* cand_scores, const int64_t* cand_local, const int64_t* cand_global,
                              int64_t stride_w, int32_t world, int32_t n_seq, int32_t kc, int32_t k,
                              float invalid_below, float* out_scores, int64_t* out_local, int64_t* out_global,
                              int32_t* out_rank, void* stream) {
  MSA_REQUIRE(cand_scores && cand_local && cand_global && out_scores && out_local && out_global && out_rank,
              "topk_merge: null pointer");
  MSA_REQUIRE(world >= 1 && n_seq >= 0 && kc >= 1 && k >= 1, "topk_merge: bad sizes");
  MSA_REQUIRE((int64_t)world * kc <= kMergeMax, "topk_merge: world*kc=%lld exceeds %d", (long long)world * kc,
              kMergeMax);
  MSA_REQUIRE(k <= world * kc, "topk_merge: k=%d exceeds the %d candidates per query", k, world * kc);
  if (n_seq == 0) return MSA_OK;
  topk_merge_kernel<<<n_seq, kMergeThreads, 0, (cudaStream_t)stream>>>(
      cand_scores, cand_local, cand_global, stride_w, world, kc, k, invalid_below, out_scores, out_local,
      out_global, out_rank);
  MSA_LAUNCH_OK("topk_merge_kernel");
  return MSA_OK;
}
