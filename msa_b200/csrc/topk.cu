// Exact top-k over the document score table, and the cross-rank merge.
//
// Scores live in the table as order-preserving uint32 keys; items are 64-bit composites (key high, inverted
// column low), so equal scores order by ascending column and items are unique.  Selection has two levels: every
// CTA of level 1 takes one slice of a row and keeps its best k, a second launch reduces the survivors of all
// slices of a row and writes the result; rows are cut into slices so that even a handful of queries (decode-time
// routing) spreads over the whole GPU.  One read of the table, k results written.
//   k <= 64 (select_topk_kernel): no sort.  Level 1: per warp, threshold = k-th largest lane maximum, compaction of
//   the survivors, ranks by counting (k <= 32) or k rounds of a warp arg-max; final level (one CTA per row, where
//   latency counts): threshold = k-th largest of the CTA's 256 per-thread maxima, compaction, ranks by counting.
//   larger k (sort_topk_kernel): a bitonic network over the slice in shared memory.
// The final level also serves the fused decode-time routing kernel, whose CTAs write k candidates per sequence.
#include "common.cuh"
#include "topk_warp.cuh"

namespace msa {

constexpr int kSortThreads = 256;
constexpr int kMaxK = 1024;
constexpr int kMinSlice = 2048;   // items per CTA at level 1 (power of two)
constexpr int kMaxSlice = 8192;   // 64 KiB of shared memory
constexpr int kSurvivorCap = 1024;   // items that may pass the threshold of the final level's selection

__device__ __forceinline__ void bitonic_sort_desc(unsigned long long* s, int n2) {
  for (int size = 2; size <= n2; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n2; i += kSortThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const unsigned long long a = s[i], b = s[j];
          if (desc ? a < b : a > b) { s[i] = b; s[j] = a; }
        }
      }
      __syncthreads();
    }
}

// grid (n_slices, n_rows).  FROM_KEYS: items come from a slice of the key table; otherwise from
// `cand` (n_in composite items per row).  The best `keep` items go to `cand_out` (level 1) or,
// when cand_out is null, to the result arrays (final level).
template <bool FROM_KEYS>
__global__ void __launch_bounds__(kSortThreads)
sort_topk_kernel(const uint32_t* __restrict__ keys, long long table_stride, int n_cols, int slice,
                 const unsigned long long* __restrict__ cand, int n_in, int n2, int keep,
                 unsigned long long* __restrict__ cand_out, const int64_t* __restrict__ doc_ids_table,
                 float* __restrict__ out_scores, int64_t* __restrict__ out_local, int64_t* __restrict__ out_global) {
  extern __shared__ unsigned long long s_items[];
  const int row = blockIdx.y, sl = blockIdx.x;
  if (FROM_KEYS) {
    const int c0 = sl * slice;
    const uint32_t* src = keys + (long long)row * table_stride;
    for (int i = threadIdx.x; i < n2; i += kSortThreads) {
      const int c = c0 + i;
      s_items[i] = (i < slice && c < n_cols) ? (((unsigned long long)src[c] << 32) | (0xffffffffu - (uint32_t)c)) : 0ull;
    }
  } else {
    const unsigned long long* src = cand + (long long)row * n_in;
    for (int i = threadIdx.x; i < n2; i += kSortThreads) s_items[i] = i < n_in ? src[i] : 0ull;
  }
  __syncthreads();
  bitonic_sort_desc(s_items, n2);
  if (cand_out) {
    unsigned long long* dst = cand_out + ((long long)row * gridDim.x + sl) * keep;
    for (int i = threadIdx.x; i < keep; i += kSortThreads) dst[i] = s_items[i];
  } else {
    for (int i = threadIdx.x; i < keep; i += kSortThreads) {
      const unsigned long long w = s_items[i];
      const long long col = 0xffffffffu - (uint32_t)(w & 0xffffffffull);
      const long long o = (long long)row * keep + i;
      out_scores[o] = key_to_float((uint32_t)(w >> 32));
      out_local[o] = col;
      if (out_global) out_global[o] = doc_ids_table ? doc_ids_table[col] : col;
    }
  }
}

template <bool FROM_KEYS>
__global__ void __launch_bounds__(kSortThreads)
select_topk_kernel(const uint32_t* __restrict__ keys, long long table_stride, int n_cols, int slice,
                   const unsigned long long* __restrict__ cand, int n_in, int n2, int keep,
                   unsigned long long* __restrict__ cand_out, const int64_t* __restrict__ doc_ids_table, float* __restrict__ out_scores,
                   int64_t* __restrict__ out_local, int64_t* __restrict__ out_global) {
  extern __shared__ unsigned long long s_items[];
  __shared__ unsigned long long s_win[(kSortThreads / 32) * kSelectMaxK];
  __shared__ unsigned long long s_final[kSelectMaxK];
  __shared__ unsigned long long s_scratch[kSortThreads / 32][32];
  __shared__ unsigned long long s_best[kSortThreads];
  __shared__ unsigned long long s_surv[kSurvivorCap];
  __shared__ unsigned long long s_threshold;
  __shared__ int s_count;
  const int row = blockIdx.y, sl = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = kSortThreads / 32;
  grid_dependency_wait();      // launched as a programmatic dependent, this kernel may be resident before its input is complete
  if (FROM_KEYS) {
    const int c0 = sl * slice;
    const uint32_t* src = keys + (long long)row * table_stride;
    for (int i = threadIdx.x; i < n2; i += kSortThreads) {
      const int c = c0 + i;
      const unsigned long long v = (i < slice && c < n_cols) ? (((unsigned long long)src[c] << 32) | (0xffffffffu - (uint32_t)c)) : 0ull;
      s_items[i] = v;
    }
  } else {
    const unsigned long long* src = cand + (long long)row * n_in;
    for (int i = threadIdx.x; i < n2; i += kSortThreads) {
      const unsigned long long v = i < n_in ? src[i] : 0ull;
      s_items[i] = v;
    }
  }
  __syncthreads();
  auto cta_select = [&](int n_items) {   // best `keep` of s_items[0..n_items) -> s_final, in order
    const int seg = (n_items + n_warps - 1) / n_warps;
    const int lo = min(n_items, warp * seg), hi = min(n_items, lo + seg);
    if (keep <= 32) warp_filter_topk(s_items + lo, hi - lo, keep, s_win + warp * keep, s_scratch[warp]);
    else warp_extract_topk(s_items + lo, hi - lo, keep, s_win + warp * keep);
    __syncthreads();
    if (warp == 0) {
      if (keep <= 32) warp_filter_topk(s_win, n_warps * keep, keep, s_final, s_scratch[0]);
      else warp_extract_topk(s_win, n_warps * keep, keep, s_final);
    }
    __syncthreads();
  };
  // Final level (one CTA per row, so latency counts, not instructions): the keep-th largest of the 256 per-thread
  // maxima is a lower bound T of the keep-th largest item (keep items are >= T), so only items >= T can win.
  // Typically a few dozen survive; they are ranked by counting.  (Level 1 runs hundreds of CTAs and keeps the
  // warp-level selection, which executes far fewer instructions.)
  bool done = false;
  if (!FROM_KEYS && keep <= kSortThreads / 2) {
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < n2; i += kSortThreads) best = s_items[i] > best ? s_items[i] : best;
    s_best[threadIdx.x] = best;
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    int rank = 0;
#pragma unroll 8
    for (int j = 0; j < kSortThreads; ++j) {
      const unsigned long long o = s_best[j];
      rank += (o > best || (o == best && j < (int)threadIdx.x)) ? 1 : 0;
    }
    if (rank == keep - 1) s_threshold = best;      // exactly one thread; 0 when fewer than keep threads hold an item
    __syncthreads();
    const unsigned long long threshold = s_threshold;
    for (int i0 = 0; i0 < n2; i0 += kSortThreads) {
      const int i = i0 + threadIdx.x;
      const unsigned long long v = i < n2 ? s_items[i] : 0ull;
      const bool take = v != 0ull && v >= threshold;
      const uint32_t bal = __ballot_sync(0xffffffffu, take);
      int base = 0;
      if (lane == 0 && bal) base = atomicAdd(&s_count, __popc(bal));
      base = __shfl_sync(0xffffffffu, base, 0);
      const int pos = base + __popc(bal & ((1u << lane) - 1u));
      if (take && pos < kSurvivorCap) s_surv[pos] = v;
    }
    __syncthreads();
    const int n_c = s_count;
    if (n_c <= kSurvivorCap) {      // (more survivors than the buffer holds: the general path below)
      for (int c = threadIdx.x; c < n_c; c += kSortThreads) {
        const unsigned long long mine = s_surv[c];
        int r = 0;
        for (int j = 0; j < n_c; ++j) r += s_surv[j] > mine ? 1 : 0;   // composite items are unique
        if (r < keep) s_final[r] = mine;
      }
      for (int r = n_c + threadIdx.x; r < keep; r += kSortThreads) s_final[r] = 0ull;
      __syncthreads();
      done = true;
    }
  }
  if (!done) cta_select(n2);
  if (cand_out) {
    unsigned long long* dst = cand_out + ((long long)row * gridDim.x + sl) * keep;
    for (int i = threadIdx.x; i < keep; i += kSortThreads) dst[i] = s_final[i];
    return;
  }
  for (int i = threadIdx.x; i < keep; i += kSortThreads) {
    const unsigned long long w = s_final[i];
    const long long o = (long long)row * keep + i;
    if (w == 0ull) {   // fewer than `keep` real items (producers that dropped entries): an empty slot, not a column
      out_scores[o] = -INFINITY;
      out_local[o] = 0;
      if (out_global) out_global[o] = doc_ids_table ? doc_ids_table[0] : 0;
      continue;
    }
    const long long col = 0xffffffffu - (uint32_t)(w & 0xffffffffull);
    out_scores[o] = key_to_float((uint32_t)(w >> 32));
    out_local[o] = col;
    if (out_global) out_global[o] = doc_ids_table ? doc_ids_table[col] : col;
  }
}

static inline int pow2_ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }

// Slice length and slice count for a row of n_cols with k winners: slices are at least
// kMinSlice (and 2k) long, and few enough that all survivors fit one final sort.
static void topk_plan(int n_cols, int k, int* slice, int* n_slices) {
  const int k_eff = k < n_cols ? k : n_cols;
  int sl = pow2_ceil(2 * k_eff) > kMinSlice ? pow2_ceil(2 * k_eff) : kMinSlice;
  while ((long long)((n_cols + sl - 1) / sl) * k_eff > kMaxSlice && sl < kMaxSlice) sl <<= 1;
  *slice = sl;
  *n_slices = (n_cols + sl - 1) / sl;
}

// One CTA per query: rank every candidate by counting the candidates that beat it.
constexpr int kMergeThreads = 128;
constexpr int kMergeMax = 4096;

__global__ void __launch_bounds__(kMergeThreads)
topk_merge_kernel(const float* __restrict__ cand_scores, const int64_t* __restrict__ cand_local,
                  const int64_t* __restrict__ cand_global, long long stride_w, long long stride_w_ids, int world, int kc, int k,
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
      const float s = cand_scores[(long long)w * stride_w + (long long)b * kc + j];
      const long long src = (long long)w * stride_w_ids + (long long)b * kc + j;
      const long long o = (long long)b * k + rank;
      out_scores[o] = s;
      out_local[o] = s > invalid_below ? cand_local[src] : -1;
      out_global[o] = cand_global[src];
      out_rank[o] = w;
    }
  }
}

// Final level on its own: every row of `cand` holds n_in composite items (score key high, inverted column low,
// 0 = empty) gathered from several producers; writes the best k_eff per row.  Used by the fused decode-time
// routing kernel, whose CTAs are the producers.
int launch_topk_from_candidates(const unsigned long long* cand, int n_in, int n_seq, int k_eff, const int64_t* doc_ids_table,
                                float* out_scores, int64_t* out_local, int64_t* out_global, cudaStream_t stream, bool pdl) {
  MSA_REQUIRE(n_in >= 1 && n_in <= kMaxSlice && k_eff >= 1 && k_eff <= kSelectMaxK && n_seq >= 1 && n_seq <= 65535,
              "topk (candidates): bad sizes");
  const int n2 = pow2_ceil(n_in);
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(select_topk_kernel<false>, kMaxSlice * 8, configured));
  MSA_CUDA_OK(launch_kernel_pdl(select_topk_kernel<false>, dim3(1, n_seq), dim3(kSortThreads), (size_t)n2 * 8, stream, pdl,
                                (const uint32_t*)nullptr, 0ll, 0, 0, cand, n_in, n2, k_eff, (unsigned long long*)nullptr,
                                doc_ids_table, out_scores, out_local, out_global));
  return MSA_OK;
}

}  // namespace msa

using namespace msa;

extern "C" int64_t msa_topk_workspace_bytes(int32_t n_seq, int32_t n_cols, int32_t k) {
  if (n_seq <= 0 || n_cols <= 0 || k <= 0) return 0;
  int slice, n_slices;
  topk_plan(n_cols, k, &slice, &n_slices);
  if (n_slices <= 1) return 0;
  return (int64_t)n_seq * n_slices * (k < n_cols ? k : n_cols) * (int64_t)sizeof(unsigned long long);
}

extern "C" int msa_topk_select(const uint32_t* score_keys, int64_t table_stride, int32_t n_seq, int32_t n_cols,
                               int32_t k, const int64_t* doc_ids_table, float* out_scores, int64_t* out_local_ids,
                               int64_t* out_global_ids, void* workspace, int64_t workspace_bytes, void* stream) {
  MSA_REQUIRE(score_keys && out_scores && out_local_ids, "topk_select: null pointer");
  MSA_REQUIRE(n_seq >= 0 && n_cols >= 1 && k >= 1, "topk_select: bad sizes (n_cols=%d k=%d)", n_cols, k);
  MSA_REQUIRE(k <= kMaxK, "topk_select: k=%d exceeds the supported maximum %d", k, kMaxK);
  MSA_REQUIRE(table_stride >= n_cols, "topk_select: table_stride < n_cols");
  MSA_REQUIRE(n_seq <= 65535, "topk_select: at most 65535 rows per call");
  if (n_seq == 0) return MSA_OK;
  const int k_eff = k < n_cols ? k : n_cols;
  int slice, n_slices;
  topk_plan(n_cols, k, &slice, &n_slices);
  MSA_REQUIRE((long long)n_slices * k_eff <= kMaxSlice, "topk_select: n_cols=%d with k=%d is too large for two levels",
              n_cols, k);
  cudaStream_t st = (cudaStream_t)stream;
  static DeviceSmem configured[4] = {};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(sort_topk_kernel<true>, kMaxSlice * 8, configured[0]));
  MSA_OK_OR_RETURN(ensure_dynamic_smem(sort_topk_kernel<false>, kMaxSlice * 8, configured[1]));
  MSA_OK_OR_RETURN(ensure_dynamic_smem(select_topk_kernel<true>, kMaxSlice * 8, configured[2]));
  MSA_OK_OR_RETURN(ensure_dynamic_smem(select_topk_kernel<false>, kMaxSlice * 8, configured[3]));
  const bool small_k = k_eff <= kSelectMaxK;
  if (n_slices == 1) {
    const int n2 = pow2_ceil(n_cols);
    if (small_k)
      select_topk_kernel<true><<<dim3(1, n_seq), kSortThreads, (size_t)n2 * 8, st>>>(
          score_keys, table_stride, n_cols, n2, nullptr, 0, n2, k_eff, nullptr, doc_ids_table, out_scores,
          out_local_ids, out_global_ids);
    else
      sort_topk_kernel<true><<<dim3(1, n_seq), kSortThreads, (size_t)n2 * 8, st>>>(
          score_keys, table_stride, n_cols, n2, nullptr, 0, n2, k_eff, nullptr, doc_ids_table, out_scores,
          out_local_ids, out_global_ids);
    MSA_LAUNCH_OK("topk kernel");
    return MSA_OK;
  }
  MSA_REQUIRE(workspace && workspace_bytes >= msa_topk_workspace_bytes(n_seq, n_cols, k),
              "topk_select: workspace of %lld bytes needed", (long long)msa_topk_workspace_bytes(n_seq, n_cols, k));
  unsigned long long* cand = (unsigned long long*)workspace;
  const int n_in = n_slices * k_eff, n2 = pow2_ceil(n_in);
  if (small_k) {
    select_topk_kernel<true><<<dim3(n_slices, n_seq), kSortThreads, (size_t)slice * 8, st>>>(
        score_keys, table_stride, n_cols, slice, nullptr, 0, slice, k_eff, cand, nullptr, nullptr, nullptr, nullptr);
    MSA_LAUNCH_OK("select_topk_kernel (slices)");
    select_topk_kernel<false><<<dim3(1, n_seq), kSortThreads, (size_t)n2 * 8, st>>>(
        nullptr, 0, 0, 0, cand, n_in, n2, k_eff, nullptr, doc_ids_table, out_scores, out_local_ids,
        out_global_ids);
  } else {
    sort_topk_kernel<true><<<dim3(n_slices, n_seq), kSortThreads, (size_t)slice * 8, st>>>(
        score_keys, table_stride, n_cols, slice, nullptr, 0, slice, k_eff, cand, nullptr, nullptr, nullptr, nullptr);
    MSA_LAUNCH_OK("sort_topk_kernel (slices)");
    sort_topk_kernel<false><<<dim3(1, n_seq), kSortThreads, (size_t)n2 * 8, st>>>(
        nullptr, 0, 0, 0, cand, n_in, n2, k_eff, nullptr, doc_ids_table, out_scores, out_local_ids, out_global_ids);
  }
  MSA_LAUNCH_OK("sort_topk_kernel (final)");
  return MSA_OK;
}

extern "C" int msa_topk_merge(const float* cand_scores, const int64_t* cand_local, const int64_t* cand_global,
                              int64_t stride_w, int64_t stride_w_ids, int32_t world, int32_t n_seq, int32_t kc, int32_t k,
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
      cand_scores, cand_local, cand_global, stride_w, stride_w_ids, world, kc, k, invalid_below, out_scores, out_local,
      out_global, out_rank);
  MSA_LAUNCH_OK("topk_merge_kernel");
  return MSA_OK;
}
