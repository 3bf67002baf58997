// Stage-1 chunk bookkeeping on many CTAs.
//
// The token stream of a block is cut into tiles of 2048 tokens, one CTA each:
//   summarise (all tiles in parallel) : per tile, how many document tokens, the first and last
//                                       document seen, the length of the leading and trailing
//                                       runs, and the chunk starts that belong to documents
//                                       beginning inside the tile;
//   carry     (one thread)            : walks the tile summaries in order and hands every tile its
//                                       starting state (token base, chunk base, the document the
//                                       tile opens in and the rank of its first token there);
//   emit      (all tiles in parallel) : replays the tile with that state and writes token_index,
//                                       chunk_offsets and pooled_doc_ids.
// Tokens are staged through shared memory with coalesced loads; each thread then owns eight
// consecutive tokens, and a tile needs three block scans.  Bound by latency, not bandwidth
// (8 bytes per token are read twice).
#include "common.cuh"

namespace msa {

constexpr int kBkThreads = 256;
constexpr int kBkSeg = 8;                       // consecutive tokens per thread
constexpr int kBkTile = kBkThreads * kBkSeg;    // 2048 tokens per CTA
constexpr long long kNoDoc = -1;

struct TileSummary {   // written by summarise, read by carry
  long long first_gid, last_gid;
  int cnt, lead_len, tail_len, chunks_after_lead;
};
struct TileCarry {     // written by carry, read by emit
  long long prev_gid;  // last document token before the tile (kNoDoc: none)
  long long ds;        // compact index at which the tile's opening document started
  int ci_base, ch_base;
};

template <typename T, typename Op>
__device__ inline T bk_exclusive_scan(T v, T identity, Op op, T* smem, T* total) {
  const int t = threadIdx.x;
  smem[t] = v;
  __syncthreads();
  for (int d = 1; d < kBkThreads; d <<= 1) {
    T other = (t >= d) ? smem[t - d] : identity;
    __syncthreads();
    smem[t] = op(other, smem[t]);
    __syncthreads();
  }
  T incl_prev = (t > 0) ? smem[t - 1] : identity;
  if (total) *total = smem[kBkThreads - 1];
  __syncthreads();
  return incl_prev;
}

// Document id of every token of the tile (kNoDoc for non-document tokens), row folded in so that
// equal ids in different rows differ.  Padded by one slot per segment against bank conflicts.
__device__ inline void bk_stage_tile(const int64_t* __restrict__ doc_ids, const int64_t* __restrict__ attn,
                                     long long lo, long long n, int row_len, long long* s_gid) {
  for (int i = threadIdx.x; i < kBkTile; i += kBkThreads) {
    const long long t = lo + i;
    long long g = kNoDoc;
    if (t < n) {
      const long long id = doc_ids[t];
      if (id > 0 && (attn == nullptr || attn[t] == 1)) g = (t / row_len) * (1ll << 40) + id;
    }
    s_gid[i + i / kBkSeg] = g;
  }
  __syncthreads();
}

struct BkShared {
  long long gid[kBkTile + kBkTile / kBkSeg];
  long long scan_ll[kBkThreads];
  int scan_int[kBkThreads];
};

// The three scan phases over one staged tile.  `prev0` / `ds0` are the state before the tile's
// first token.  Calls `visit(i, ci, ds, ch, g, chunk_start, total)` for every document token (i = slot
// in the tile, total = document tokens in the tile), with ci / ds / ch counted from the given bases.
template <typename Visit>
__device__ inline void bk_walk_tile(BkShared& sh, long long carry_prev, long long carry_ds, int ci_base, int ch_base,
                                    int* cnt_out, Visit visit, int P) {
  const long long* seg = sh.gid + threadIdx.x * (kBkSeg + 1);
  // phase 1: compact index and the last document token before each segment
  int cnt = 0;
  long long last = kNoDoc;
#pragma unroll
  for (int e = 0; e < kBkSeg; ++e)
    if (seg[e] != kNoDoc) { ++cnt; last = seg[e]; }
  int total;
  const int ci0 = ci_base + bk_exclusive_scan<int>(cnt, 0, [](int a, int b) { return a + b; }, sh.scan_int, &total);
  long long prev0 = bk_exclusive_scan<long long>(
      last, kNoDoc, [](long long a, long long b) { return b != kNoDoc ? b : a; }, sh.scan_ll, nullptr);
  if (prev0 == kNoDoc) prev0 = carry_prev;
  // phase 2: where the document open at each segment's start began
  long long ds_local = -(1ll << 60);
  {
    int ci = ci0;
    long long prev = prev0;
#pragma unroll
    for (int e = 0; e < kBkSeg; ++e)
      if (seg[e] != kNoDoc) {
        if (prev != seg[e]) ds_local = ci;
        prev = seg[e];
        ++ci;
      }
  }
  long long ds0 = bk_exclusive_scan<long long>(
      ds_local, -(1ll << 60), [](long long a, long long b) { return a > b ? a : b; }, sh.scan_ll, nullptr);
  if (ds0 == -(1ll << 60)) ds0 = carry_ds;
  // phase 3: chunk starts
  int nch = 0;
  {
    int ci = ci0;
    long long prev = prev0, ds = ds0;
#pragma unroll
    for (int e = 0; e < kBkSeg; ++e)
      if (seg[e] != kNoDoc) {
        if (prev != seg[e]) ds = ci;
        prev = seg[e];
        if ((ci - ds) % P == 0) ++nch;
        ++ci;
      }
  }
  const int ch0 = ch_base + bk_exclusive_scan<int>(nch, 0, [](int a, int b) { return a + b; }, sh.scan_int, nullptr);
  {
    int ci = ci0, ch = ch0;
    long long prev = prev0, ds = ds0;
#pragma unroll
    for (int e = 0; e < kBkSeg; ++e)
      if (seg[e] != kNoDoc) {
        if (prev != seg[e]) ds = ci;
        prev = seg[e];
        const bool start = (ci - ds) % P == 0;
        visit(threadIdx.x * kBkSeg + e, ci, ds, ch, seg[e], start, total);
        if (start) ++ch;
        ++ci;
      }
  }
  if (cnt_out) *cnt_out = total;
}

__global__ void __launch_bounds__(kBkThreads)
bk_summarise_kernel(const int64_t* __restrict__ doc_ids, const int64_t* __restrict__ attn, long long n, int row_len,
                    int P, TileSummary* __restrict__ summaries) {
  __shared__ BkShared sh;
  __shared__ int s_lead, s_tail_start, s_chunks;
  __shared__ long long s_first, s_last;
  const long long lo = (long long)blockIdx.x * kBkTile;
  bk_stage_tile(doc_ids, attn, lo, n, row_len, sh.gid);
  if (threadIdx.x == 0) { s_lead = 1 << 30; s_tail_start = 0; s_chunks = 0; s_first = kNoDoc; s_last = kNoDoc; }
  __syncthreads();
  int cnt;
  // walked as if no document were open before the tile: ranks inside the leading run are then
  // relative to the tile, which is why only chunk starts AFTER the leading run are counted here
  bk_walk_tile(sh, kNoDoc, 0, 0, 0, &cnt,
               [&](int, int ci, long long ds, int, long long g, bool start, int total) {
                 if (ci == 0) s_first = g;
                 if (ci == total - 1) s_last = g;
                 if (ds > 0 && ds == ci) atomicMin(&s_lead, ci);        // first change of document
                 if (ds == ci) atomicMax(&s_tail_start, ci);            // start of the last run
                 if (start && ds > 0) atomicAdd(&s_chunks, 1);          // documents that begin inside the tile
               }, P);
  __syncthreads();
  if (threadIdx.x == 0) {
    TileSummary s;
    s.cnt = cnt;
    s.first_gid = s_first;
    s.last_gid = s_last;
    s.lead_len = cnt == 0 ? 0 : (s_lead == (1 << 30) ? cnt : s_lead);
    s.tail_len = cnt - s_tail_start;
    s.chunks_after_lead = s_chunks;
    summaries[blockIdx.x] = s;
  }
}

// Multiples of P in [r0, r0 + len): the chunk starts of a run whose first token has rank r0.
__device__ __forceinline__ int chunk_starts_in_run(long long r0, int len, int P) {
  if (len <= 0) return 0;
  const long long hi = (r0 + len - 1) / P, lo = r0 == 0 ? -1 : (r0 - 1) / P;
  return (int)(hi - lo);
}

__global__ void bk_carry_kernel(const TileSummary* __restrict__ summaries, int n_tiles, int P, int max_chunks,
                                TileCarry* __restrict__ carries, int32_t* __restrict__ chunk_offsets,
                                int32_t* __restrict__ counts) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  long long prev_gid = kNoDoc, rank_out = 0;
  int ci = 0, ch = 0;
  for (int t = 0; t < n_tiles; ++t) {
    const TileSummary s = summaries[t];
    TileCarry c;
    c.prev_gid = prev_gid;
    c.ci_base = ci;
    c.ch_base = ch;
    c.ds = ci;
    if (s.cnt > 0) {
      const bool cont = prev_gid != kNoDoc && prev_gid == s.first_gid;
      const long long r0 = cont ? rank_out : 0;
      c.ds = ci - r0;
      ch += chunk_starts_in_run(r0, s.lead_len, P) + s.chunks_after_lead;
      rank_out = s.lead_len == s.cnt ? r0 + s.cnt : s.tail_len;
      prev_gid = s.last_gid;
      ci += s.cnt;
    }
    carries[t] = c;
  }
  const bool overflow = ch > max_chunks;
  chunk_offsets[overflow ? max_chunks : ch] = ci;
  counts[0] = ci;
  counts[1] = overflow ? max_chunks : ch;
  counts[2] = overflow ? 1 : 0;
}

__global__ void __launch_bounds__(kBkThreads)
bk_emit_kernel(const int64_t* __restrict__ doc_ids, const int64_t* __restrict__ attn, long long n, int row_len, int P,
               const TileCarry* __restrict__ carries, int32_t* __restrict__ token_index,
               int32_t* __restrict__ chunk_offsets, int64_t* __restrict__ pooled_doc_ids, int max_chunks) {
  __shared__ BkShared sh;
  const long long lo = (long long)blockIdx.x * kBkTile;
  bk_stage_tile(doc_ids, attn, lo, n, row_len, sh.gid);
  const TileCarry c = carries[blockIdx.x];
  bk_walk_tile(sh, c.prev_gid, c.ds, c.ci_base, c.ch_base, nullptr,
               [&](int i, int ci, long long, int ch, long long g, bool start, int) {
                 token_index[ci] = (int32_t)(lo + i);
                 if (start && ch < max_chunks) {
                   chunk_offsets[ch] = ci;
                   pooled_doc_ids[ch] = g & ((1ll << 40) - 1);
                 }
               }, P);
}

}  // namespace msa

using namespace msa;

extern "C" int64_t msa_bookkeeping_workspace_bytes(int32_t n_rows, int32_t row_len) {
  const long long n = (long long)n_rows * row_len;
  const long long tiles = (n + kBkTile - 1) / kBkTile;
  return tiles * (long long)(sizeof(TileSummary) + sizeof(TileCarry)) + 64;
}

extern "C" int msa_chunk_bookkeeping(const int64_t* doc_ids, const int64_t* attention_mask, int32_t n_rows,
                                     int32_t row_len, int32_t pooling_kernel_size, int32_t* token_index,
                                     int32_t* chunk_offsets, int64_t* pooled_doc_ids, int32_t max_chunks,
                                     int32_t* counts, void* workspace, int64_t workspace_bytes, void* stream) {
  MSA_REQUIRE(doc_ids && token_index && chunk_offsets && pooled_doc_ids && counts, "bookkeeping: null pointer");
  MSA_REQUIRE(n_rows >= 0 && row_len >= 0 && (int64_t)n_rows * row_len < (1ll << 31), "bookkeeping: bad sizes");
  MSA_REQUIRE(pooling_kernel_size > 0 && max_chunks >= 0, "bookkeeping: pooling_kernel_size must be > 0");
  const long long n = (long long)n_rows * row_len;
  const int tiles = (int)((n + kBkTile - 1) / kBkTile);
  MSA_REQUIRE(workspace && workspace_bytes >= msa_bookkeeping_workspace_bytes(n_rows, row_len) &&
                  ((uintptr_t)workspace & 7u) == 0,
              "bookkeeping: workspace of %lld bytes (8-byte aligned) needed",
              (long long)msa_bookkeeping_workspace_bytes(n_rows, row_len));
  cudaStream_t st = (cudaStream_t)stream;
  TileSummary* summaries = (TileSummary*)workspace;
  TileCarry* carries = (TileCarry*)(summaries + tiles);
  if (tiles > 0) {
    bk_summarise_kernel<<<tiles, kBkThreads, 0, st>>>(doc_ids, attention_mask, n, row_len > 0 ? row_len : 1,
                                                      pooling_kernel_size, summaries);
    MSA_LAUNCH_OK("bk_summarise_kernel");
  }
  bk_carry_kernel<<<1, 32, 0, st>>>(summaries, tiles, pooling_kernel_size, max_chunks, carries, chunk_offsets, counts);
  MSA_LAUNCH_OK("bk_carry_kernel");
  if (tiles > 0) {
    bk_emit_kernel<<<tiles, kBkThreads, 0, st>>>(doc_ids, attention_mask, n, row_len > 0 ? row_len : 1,
                                                 pooling_kernel_size, carries, token_index, chunk_offsets,
                                                 pooled_doc_ids, max_chunks);
    MSA_LAUNCH_OK("bk_emit_kernel");
  }
  return MSA_OK;
}
