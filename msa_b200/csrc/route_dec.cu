// Decode-time routing in one launch: score every chunk of the shard against a handful of query rows (one row per
// sequence) on the tensor cores AND select, per CTA, the best k documents of every sequence.
//
// With one query token per sequence the scoring is bound by HBM (the shard's router keys are read once; the
// contraction is a sliver of the tensor pipe), and the [sequences x documents] score table that the general
// kernel fills is pure overhead: a reset launch, 4-byte scattered stores, and a selection kernel that reads it
// back.  Here the table never leaves the SM:
//
//   * every CTA owns ONE contiguous range of chunks whose ends are moved to document boundaries, so a document is
//     scored by exactly one CTA; ranges are equal (no partial last wave), tiles step through a range 128 chunks at
//     a time from wherever the range starts (TMA has no alignment rule for the row coordinate), and the last tile
//     of a range is fetched in 32-row boxes so that rows of the neighbour's range are not read twice;
//   * the epilogue reduces chunk scores to document scores into a SHARED-MEMORY table [document][sequence] of
//     order-preserving keys (atomicMax on shared memory; documents are addressed relative to the first document of
//     the current segment);
//   * when the table is full, and at the end of the range, the epilogue warps select every sequence's best k among
//     (table column + the sequence's running list) with the warp routines of topk_warp.cuh; a document that is
//     still open at a flush (its chunks continue in the next tile) is carried over, not selected;
//   * the CTA writes k candidates per sequence; one small launch (the second level of the stand-alone selection)
//     reduces the n_ctas * k candidates of a sequence to the result.
//
// Layer-step launches: fold, this kernel, final selection (5 before: fold, table reset, scoring, two selection
// levels).  Exactness: the candidates are exact per CTA and every document belongs to one CTA, so the result
// equals the selection over the full table, ties included (column 0, the reference's dummy document with
// finfo.min, is seeded by CTA 0).
//
// Roles as in route_tc.cu: warps 0-3 epilogue (TMEM lane quarter = warp), warp 4 TMA producer, warp 5 MMA issuer
// and TMEM owner.  Every mbarrier wait is bounded; a wait that runs out raises status[0] and the CTA drains and
// returns (its candidates are then incomplete, which status reports).
#include <cuda.h>

#include "common.cuh"
#include "route.cuh"
#include "tc_common.cuh"
#include "topk_warp.cuh"

namespace msa {

constexpr int kDecBM = 128;         // chunks per tile (UMMA M)
constexpr int kDecBK = 64;          // bf16 elements per K block (one 128-byte swizzle row)
constexpr int kDecUmmaK = 16;
constexpr int kDecThreads = 192;
constexpr int kDecEpiThreads = 128;
constexpr int kDecMaxBN = 128;      // sequences (query rows) per launch
constexpr int kDecMaxKeep = 32;     // candidates per CTA and sequence
constexpr int kDecTmemCols = 256;   // two accumulators of up to 128 columns
constexpr int kDecTailBox = 32;     // rows per TMA box of a range's last tile
constexpr int kDecMaxStages = 8;

struct RouteDecParams {
  int n_seq, bn, bn_pad, n_chunks, n_docs, k_blocks, stages, cap, keep, per_cta;
  uint32_t min_key;
  float alpha;
  const float* row_bias;
  const int32_t* chunk_doc;
  unsigned long long* cand;   // [n_seq][gridDim.x * keep]
  int32_t* status;
};

struct DecSeg { int start, len, doc; };
struct DecEpiScratch {
  float xpose[16][33];
  DecSeg seg[32];
};

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// First chunk at or after p that starts a document (p itself when it does; n_chunks at the end).
__device__ __forceinline__ int snap_to_document(const int32_t* chunk_doc, int p, int n_chunks) {
  if (p <= 0) return 0;
  if (p >= n_chunks) return n_chunks;
  const int d = chunk_doc[p - 1];
  while (p < n_chunks && chunk_doc[p] == d) ++p;
  return p;
}

__global__ void __launch_bounds__(kDecThreads, 1)
route_dec_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_k_tail,
                 const __grid_constant__ CUtensorMap tmap_q, const RouteDecParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint64_t s_full[kDecMaxStages], s_empty[kDecMaxStages], s_acc_full[2], s_acc_empty[2], s_drain;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_lo, s_hi;
  __shared__ float s_bias[kDecMaxBN];
  __shared__ DecEpiScratch s_epi[kDecEpiThreads / 32];
  __shared__ unsigned long long s_scr32[kDecEpiThreads / 32][32];

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = kDecBM * kDecBK * 2, b_bytes = (uint32_t)p.bn * kDecBK * 2, stage_bytes = a_bytes + b_bytes;
  uint32_t* tbl = reinterpret_cast<uint32_t*>(tiles + (size_t)p.stages * stage_bytes);            // [cap][bn_pad]
  unsigned long long* run = reinterpret_cast<unsigned long long*>(tbl + (size_t)p.cap * p.bn_pad + (((size_t)p.cap * p.bn_pad) & 1));
  unsigned long long* scratch = run + (size_t)p.bn * p.keep;                                       // [4][cap + keep]
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_acc_full[b], 1); mbar_init(&s_acc_empty[b], kDecEpiThreads / 32); }
    mbar_init(&s_drain, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // this CTA's range: equal shares of the chunk axis, both ends moved forward to the next document start
    const long long a = (long long)blockIdx.x * p.per_cta, b = a + p.per_cta;
    s_lo = snap_to_document(p.chunk_doc, (int)(a < p.n_chunks ? a : p.n_chunks), p.n_chunks);
    s_hi = snap_to_document(p.chunk_doc, (int)(b < p.n_chunks ? b : p.n_chunks), p.n_chunks);
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kDecTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int lo = s_lo, hi = s_hi;
  const int n_tiles = (hi - lo + kDecBM - 1) / kDecBM;

  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int row0 = lo + t * kDecBM, rows = min(kDecBM, hi - row0);
        const int tail_boxes = rows < kDecBM ? (rows + kDecTailBox - 1) / kDecTailBox : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_empty[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          if (tail_boxes == 0) {
            mbar_expect_tx(&s_full[stage], stage_bytes);
            tma_load_2d(sa, &tmap_k, kb * kDecBK, row0, &s_full[stage]);
          } else {   // 32-row boxes land where the rows of a 128-row box would (8-row swizzle groups of 1 KiB)
            mbar_expect_tx(&s_full[stage], (uint32_t)tail_boxes * kDecTailBox * kDecBK * 2 + b_bytes);
            for (int j = 0; j < tail_boxes; ++j)
              tma_load_2d(sa + (size_t)j * kDecTailBox * kDecBK * 2, &tmap_k_tail, kb * kDecBK, row0 + j * kDecTailBox,
                          &s_full[stage]);
          }
          tma_load_2d(sa + a_bytes, &tmap_q, kb * kDecBK, 0, &s_full[stage]);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {  // gave up: let the copies already issued land before the CTA's smem is released
        for (int s = 0; s < p.stages; ++s)
          if (armed & (1u << s)) {
            const unsigned long long t0 = global_ns();
            while (!mbar_try_wait(&s_full[s], (armed_parity >> s) & 1u) && global_ns() - t0 < kWaitLimitNs) {}
          }
      }
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer ----------------------------------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) |
                             ((uint32_t)(kDecBM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int buf = t & 1;
        const uint32_t acc_phase = (uint32_t)((t >> 1) & 1);
        if (!(ok = mbar_wait(&s_acc_empty[buf], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kDecMaxBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_full[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint64_t a_desc = make_smem_desc(sa), b_desc = make_smem_desc(sa + a_bytes);
#pragma unroll
          for (int k = 0; k < kDecBK / kDecUmmaK; ++k)
            tc_mma_bf16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&s_empty[stage]);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&s_acc_full[buf]);
      }
      tc_commit(&s_drain);
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&s_drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
  } else {
    // ------------------------------- epilogue + selection (warps 0-3) ------------------
    const int tid = threadIdx.x;   // 0..127
    DecEpiScratch& scr = s_epi[warp];
    unsigned long long* my_scratch = scratch + (size_t)warp * (p.cap + p.keep);
    for (int i = tid; i < p.cap * p.bn_pad; i += kDecEpiThreads) tbl[i] = p.min_key;
    for (int i = tid; i < p.bn * p.keep; i += kDecEpiThreads) run[i] = 0ull;
    if (tid < p.bn) s_bias[tid] = tid < p.n_seq ? p.row_bias[tid] : -INFINITY;
    epi_barrier();
    if (blockIdx.x == 0 && tid < p.n_seq)   // column 0: the dummy document, scored finfo.min like every untouched column
      run[(size_t)tid * p.keep] = ((unsigned long long)p.min_key << 32) | 0xffffffffull;
    int seg_base = lo < hi ? p.chunk_doc[lo] : 0;   // document id of table row 0
    int rows_used = 0;

    // Select every sequence's best `keep` among the table rows in use (except an open document) and its running
    // list; then clear the table, keeping the open document's partial maxima as row 0.
    auto flush = [&](int open_doc) {
      epi_barrier();                                   // every warp's table updates are in
      const int open_row = open_doc >= 0 ? open_doc - seg_base : -1;
      for (int seq = warp; seq < p.n_seq; seq += kDecEpiThreads / 32) {
        for (int r = lane; r < rows_used; r += 32)
          my_scratch[r] = r == open_row ? 0ull
                                        : (((unsigned long long)tbl[(size_t)r * p.bn_pad + seq] << 32) |
                                           (unsigned long long)(0xffffffffu - (uint32_t)(seg_base + r)));
        for (int j = lane; j < p.keep; j += 32) my_scratch[rows_used + j] = run[(size_t)seq * p.keep + j];
        __syncwarp();
        warp_filter_topk(my_scratch, rows_used + p.keep, p.keep, run + (size_t)seq * p.keep, s_scr32[warp]);
        __syncwarp();
      }
      epi_barrier();                                   // selections have read the table
      if (tid < p.bn) {
        const uint32_t keep_val = open_row >= 0 && open_row < rows_used ? tbl[(size_t)open_row * p.bn_pad + tid] : p.min_key;
        for (int r = 0; r < rows_used; ++r) tbl[(size_t)r * p.bn_pad + tid] = p.min_key;
        if (open_row >= 0) tbl[tid] = keep_val;
      }
      epi_barrier();
    };

    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int row0 = lo + t * kDecBM;
      const int chunk = row0 + tid;
      const int last_chunk = min(row0 + kDecBM, hi) - 1;
      const int first_doc = p.chunk_doc[row0], last_doc = p.chunk_doc[last_chunk];
      if (last_doc - seg_base >= p.cap && rows_used > 0) {      // the tile's documents do not fit: flush first
        const int open_doc = (row0 > lo && p.chunk_doc[row0 - 1] == first_doc) ? first_doc : -1;
        flush(open_doc);
        seg_base = first_doc;
        rows_used = open_doc >= 0 ? 1 : 0;
      }
      // runs of lanes that hold chunks of one document
      int doc = chunk < hi ? p.chunk_doc[chunk] : -1 - lane;
      if (chunk < hi && (doc < 1 || doc > p.n_docs || (unsigned)(doc - seg_base) >= (unsigned)p.cap)) {
        atomicAdd(p.status + 2, 1);                     // an id outside the table: counted, never used as a row
        doc = -1 - lane;
      }
      const int doc_up = __shfl_up_sync(0xffffffffu, doc, 1);
      const bool head = lane == 0 || doc_up != doc;
      const uint32_t heads = __ballot_sync(0xffffffffu, head);
      const int n_seg = __popc(heads);
      if (head) {
        const uint32_t later = lane == 31 ? 0u : (heads >> (lane + 1));
        scr.seg[__popc(heads & ((1u << lane) - 1u))] = DecSeg{lane, later ? __ffs(later) : 32 - lane, doc};
      }
      __syncwarp();
      const int buf = t & 1;
      const uint32_t acc_phase = (uint32_t)((t >> 1) & 1);
      ok = mbar_wait(&s_acc_full[buf], acc_phase, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * kDecMaxBN;
      const int n_items = n_seg * 16;
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) scr.xpose[j][lane] = __uint_as_float(r[j]) + s_bias[c0 + j];
        __syncwarp();
        // (document, column) pairs dealt over the lanes: max over the document's chunks, one shared-memory atomic
        for (int item = lane; item < n_items; item += 32) {
          const DecSeg e = scr.seg[item >> 4];
          const int j = item & 15, seq = c0 + j;
          if (e.doc > 0 && seq < p.n_seq) {
            float m = scr.xpose[j][e.start];
            for (int u = 1; u < e.len; ++u) m = fmaxf(m, scr.xpose[j][e.start + u]);
            atomicMax(tbl + (size_t)(e.doc - seg_base) * p.bn_pad + seq, float_to_key(m * p.alpha));
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_acc_empty[buf]);
      rows_used = max(rows_used, min(min(last_doc, p.n_docs) - seg_base + 1, p.cap));   // rows never stand for ids > n_docs
    }
    if (ok) {
      flush(-1);
      const long long n_in = (long long)gridDim.x * p.keep;
      for (int i = tid; i < p.n_seq * p.keep; i += kDecEpiThreads)
        p.cand[(long long)(i / p.keep) * n_in + (long long)blockIdx.x * p.keep + (i % p.keep)] = run[i];
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 5)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDecTmemCols) : "memory");
}

// Shared-memory plan for bn query rows and `keep` candidates; returns false when it does not fit.
static bool route_dec_plan(int bn, int keep, RouteDecParams* p, size_t* smem) {
  const size_t stage_bytes = (size_t)kDecBM * kDecBK * 2 + (size_t)bn * kDecBK * 2;
  const int bn_pad = bn + 1;
  const size_t budget = 212 * 1024;   // dynamic part; the kernel's static arrays take another 12 KB of the 227 KB
  // table rows: at least one tile's worth of single-chunk documents plus a carried one; more when there is room
  for (int stages = kDecMaxStages; stages >= 4; --stages) {
    for (int cap = 256; cap >= kDecBM + 2; cap -= 2) {
      const size_t tbl = ((size_t)cap * bn_pad * 4 + 7) & ~(size_t)7;
      const size_t total = 1024 + stages * stage_bytes + tbl + (size_t)bn * keep * 8 + 4ull * (cap + keep) * 8;
      if (total <= budget) {
        p->stages = stages; p->cap = cap; p->bn = bn; p->bn_pad = bn_pad; p->keep = keep;
        *smem = total;
        return true;
      }
    }
  }
  return false;
}

}  // namespace msa

using namespace msa;

namespace msa {
int launch_topk_from_candidates(const unsigned long long* cand, int n_in, int n_seq, int k_eff, const int64_t* doc_ids_table,
                                float* out_scores, int64_t* out_local, int64_t* out_global, cudaStream_t stream);
}

extern "C" int64_t msa_route_score_select_workspace_bytes(int32_t n_seq, int32_t k) {
  if (n_seq <= 0 || k <= 0) return 0;
  int n_sm = 0;
  if (device_sm_count(&n_sm) != MSA_OK) return -1;
  return (int64_t)n_seq * n_sm * (k < kDecMaxKeep ? k : kDecMaxKeep) * (int64_t)sizeof(unsigned long long);
}

extern "C" int msa_route_score_select(const void* q_folded, const float* row_bias, int32_t dtype, int32_t n_seq,
                                      const void* rk, int64_t rk_chunk_stride, int32_t n_chunks, int32_t kdim,
                                      const int32_t* chunk_doc, float alpha, int32_t n_docs, float min_val, int32_t k,
                                      const int64_t* doc_ids_table, float* out_scores, int64_t* out_local_ids,
                                      int64_t* out_global_ids, void* workspace, int64_t workspace_bytes,
                                      int32_t* status, void* stream) {
  MSA_REQUIRE(q_folded && row_bias && rk && chunk_doc && out_scores && out_local_ids && status && workspace,
              "route_score_select: null pointer");
  MSA_REQUIRE(n_seq >= 1 && n_chunks >= 1 && kdim > 0 && n_docs >= 1 && k >= 1, "route_score_select: bad sizes");
  MSA_REQUIRE(alpha > 0.f, "route_score_select: alpha must be positive (it is applied after the max)");
  if (dtype != MSA_BF16 || n_seq > kDecMaxBN || k > kDecMaxKeep || kdim % kDecBK != 0) {
    set_error("route_score_select takes bf16 keys, at most %d sequences of one row, k <= %d and kdim %% %d == 0; "
              "use msa_route_scores + msa_topk_select for other shapes", kDecMaxBN, kDecMaxKeep, kDecBK);
    return MSA_ERR_UNSUPPORTED;
  }
  MSA_REQUIRE(aligned16(q_folded) && aligned16(rk) && rk_chunk_stride % 8 == 0 && rk_chunk_stride >= kdim,
              "route_score_select: rows must be 16-byte aligned");
  const int k_eff = k < n_docs + 1 ? k : n_docs + 1;
  RouteDecParams p{};
  size_t smem = 0;
  const int bn = (n_seq + 15) / 16 * 16;
  if (!route_dec_plan(bn, k_eff, &p, &smem)) {
    set_error("route_score_select: %d sequences with k=%d do not fit shared memory", n_seq, k_eff);
    return MSA_ERR_UNSUPPORTED;
  }
  int n_sm = 0;
  MSA_OK_OR_RETURN(device_sm_count(&n_sm));
  const int n_tiles = (n_chunks + kDecBM - 1) / kDecBM;
  const int grid = n_tiles < n_sm ? n_tiles : n_sm;
  MSA_REQUIRE(workspace_bytes >= (int64_t)n_seq * grid * k_eff * 8, "route_score_select: workspace of %lld bytes needed",
              (long long)n_seq * grid * k_eff * 8);
  MSA_REQUIRE((long long)grid * k_eff <= 8192, "route_score_select: too many candidates per sequence");
  p.n_seq = n_seq; p.n_chunks = n_chunks; p.n_docs = n_docs; p.k_blocks = kdim / kDecBK;
  p.per_cta = (n_chunks + grid - 1) / grid;
  p.min_key = float_to_key(min_val); p.alpha = alpha; p.row_bias = row_bias; p.chunk_doc = chunk_doc;
  p.cand = (unsigned long long*)workspace; p.status = status;

  CUtensorMap map_k, map_k_tail, map_q;
  MSA_OK_OR_RETURN(make_map(&map_k, rk, (uint64_t)n_chunks, (uint64_t)kdim, (uint64_t)rk_chunk_stride, kDecBK, kDecBM));
  MSA_OK_OR_RETURN(make_map(&map_k_tail, rk, (uint64_t)n_chunks, (uint64_t)kdim, (uint64_t)rk_chunk_stride, kDecBK, kDecTailBox));
  MSA_OK_OR_RETURN(make_map(&map_q, q_folded, (uint64_t)n_seq, (uint64_t)kdim, (uint64_t)kdim, kDecBK, (uint32_t)bn));
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(route_dec_kernel, smem, configured));
  cudaStream_t st = (cudaStream_t)stream;
  route_dec_kernel<<<grid, kDecThreads, smem, st>>>(map_k, map_k_tail, map_q, p);
  MSA_LAUNCH_OK("route_dec_kernel");
  return launch_topk_from_candidates(p.cand, grid * k_eff, n_seq, k_eff, doc_ids_table, out_scores, out_local_ids,
                                     out_global_ids, st);
}
