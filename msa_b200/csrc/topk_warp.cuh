// Warp-level exact top-k over 64-bit items in shared memory (item = score key in the high word, inverted
// column in the low word: larger item = better score, ties to the smaller column; 0 = empty slot).
// Shared by the stand-alone selection kernels and by the fused decode-time routing kernel.
#pragma once
#include "common.cuh"

namespace msa {

// Small k (<= kSelectMaxK): no sort.  Each warp extracts the k largest items of its eighth of the
// slice by k rounds of a warp arg-max (shuffles only, no CTA barrier); warp 0 then extracts the
// final k from the 8*k survivors.  Output order is descending by construction.
constexpr int kSelectMaxK = 64;

// k rounds over items[0..n) (shared memory, owned by this warp): writes the k largest, in order.
// Every lane keeps the best of its own (strided) items in registers; a round is one redux on the
// 32-bit score keys, a ballot (plus a second redux only when scores tie), and a rescan by the one
// lane that lost its item.
__device__ __forceinline__ void warp_extract_topk(unsigned long long* items, int n, int k, unsigned long long* out) {
  const int lane = threadIdx.x & 31;
  unsigned long long best = 0ull;
  int best_i = -1;
  auto rescan = [&]() {
    best = 0ull;
    best_i = -1;
    for (int i = lane; i < n; i += 32) {
      const unsigned long long v = items[i];
      if (v > best) { best = v; best_i = i; }
    }
  };
  rescan();
  for (int r = 0; r < k; ++r) {
    const uint32_t hi = (uint32_t)(best >> 32), lo = (uint32_t)best;
    const uint32_t kmax = __reduce_max_sync(0xffffffffu, hi);
    uint32_t tie = __ballot_sync(0xffffffffu, best != 0ull && hi == kmax);
    if (__popc(tie) > 1) {  // equal scores: the smaller column (larger inverted column) goes first
      const bool in_tie = (tie >> lane) & 1u;
      const uint32_t lmax = __reduce_max_sync(0xffffffffu, in_tie ? lo : 0u);
      tie = __ballot_sync(0xffffffffu, in_tie && lo == lmax);
    }
    unsigned long long top = 0ull;
    if (tie != 0u) {
      const int winner = __ffs(tie) - 1;
      top = __shfl_sync(0xffffffffu, best, winner);
      if (lane == winner) {
        items[best_i] = 0ull;
        rescan();
      }
    }
    if (lane == 0) out[r] = top;
    __syncwarp();
  }
}

// k <= 32 without serial rounds.  The k-th largest of the 32 per-lane maxima is a lower bound T of the
// k-th largest item (k items are >= T), so only items >= T can win: they are compacted in place
// (typically a few more than k survive) and ordered by counting.  `scratch` holds 32 items.
__device__ __forceinline__ void warp_filter_topk(unsigned long long* items, int n, int k, unsigned long long* out,
                                                 unsigned long long* scratch) {
  const int lane = threadIdx.x & 31;
  const uint32_t lt_mask = (1u << lane) - 1u;
  unsigned long long best = 0ull;
  for (int i = lane; i < n; i += 32) best = items[i] > best ? items[i] : best;
  scratch[lane] = best;
  __syncwarp();
  int rank = 0;
#pragma unroll 8
  for (int j = 0; j < 32; ++j) rank += (scratch[j] > best || (scratch[j] == best && j < lane)) ? 1 : 0;
  const uint32_t kth = __ballot_sync(0xffffffffu, rank == k - 1);
  const unsigned long long threshold = __shfl_sync(0xffffffffu, best, __ffs(kth) - 1);   // may be 0: keep everything
  int n_c = 0;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    const unsigned long long v = i < n ? items[i] : 0ull;
    const bool keep = v != 0ull && v >= threshold;
    const uint32_t bal = __ballot_sync(0xffffffffu, keep);
    __syncwarp();                                   // this row is in registers: its slots may be overwritten
    if (keep) items[n_c + __popc(bal & lt_mask)] = v;
    n_c += __popc(bal);
  }
  __syncwarp();
  for (int c = lane; c < n_c; c += 32) {
    const unsigned long long mine = items[c];
    int r = 0;
    for (int j = 0; j < n_c; ++j) r += items[j] > mine ? 1 : 0;   // composite items are unique
    if (r < k) out[r] = mine;
  }
  for (int r = n_c + lane; r < k; r += 32) out[r] = 0ull;
  __syncwarp();
}

}  // namespace msa
