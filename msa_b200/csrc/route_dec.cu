// Decode-time routing in one launch: score every chunk of the shard against a handful of query rows (one row per
// sequence) on the tensor cores AND select, per CTA, the best k documents of every sequence.
//
// With one query token per sequence the scoring is bound by HBM (the shard's router keys are read once; the
// contraction is a sliver of the tensor pipe), and the [sequences x documents] score table that the general
// kernel fills is pure overhead: a reset launch, 4-byte scattered stores, and a selection kernel that reads it
// back.  Here the table never leaves the SM:
//
//   * the keys are cut into fixed tiles of 128 chunks (the rows of one UMMA); every CTA takes an equal share of
//     whole tiles and owns the documents that START in its share: both ends of the share are moved forward to the
//     next document start, so a document is scored by exactly one CTA.  The first tile's rows before that start
//     are masked; the tile after the share is read, in 32-row boxes, only as far as the CTA's last document
//     reaches.  Tiles being whole and aligned, the same loop reads row-major keys (2-D tensor map) or the
//     tile-blocked copy (4-D map; every box is one contiguous 16 KiB run, which HBM serves measurably faster);
//   * the epilogue reduces a tile's chunk scores to document scores into a SHARED-MEMORY table [document][sequence]
//     of order-preserving keys (atomicMax on shared memory; rows are documents relative to the first document of
//     the tile);
//   * after every tile, epilogue thread s (one per sequence) walks the tile's finished documents in its own table
//     column and feeds them to a sorted list of its best k that lives in REGISTERS (a branch-free chain of k
//     compare-and-swaps per document, skipped when no lane of the warp has a candidate above its k-th best); a
//     document whose chunks continue in the next tile is carried over in row 0, not consumed.  This runs while
//     the next tile streams in, so nothing but the last tile's walk is left after the stream ends;
//   * the CTA writes k candidates per sequence; one small launch (the second level of the stand-alone selection)
//     reduces the n_ctas * k candidates of a sequence to the result.
//
// Layer-step launches: fold, this kernel, final selection (5 before: fold, table reset, scoring, two selection
// levels).  Exactness: the candidates are exact per CTA and every document belongs to one CTA, so the result
// equals the selection over the full table, ties included (column 0, the reference's dummy document with
// finfo.min, is seeded by CTA 0).
//
// Roles: warps 0-7 epilogue (TMEM lane quarter = warp % 4; the two warps of a quarter split a tile's columns),
// warp 8 TMA producer, warp 9 MMA issuer and TMEM owner.  Every mbarrier wait is bounded; a wait that runs out raises status[0] and the CTA drains and
// returns (its candidates are then incomplete, which status reports).
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "route.cuh"
#include "tc_common.cuh"

namespace msa {

constexpr int kDecBM = 128;         // chunks per tile (UMMA M)
constexpr int kDecBK = 64;          // bf16 elements per K block (one 128-byte swizzle row)
constexpr int kDecUmmaK = 16;
constexpr int kDecEpiWarps = 8;     // two per TMEM lane quarter: they split a tile's columns
constexpr int kDecEpiThreads = kDecEpiWarps * 32;
constexpr int kDecThreads = kDecEpiThreads + 64;
constexpr int kDecProducerWarp = kDecEpiWarps, kDecMmaWarp = kDecEpiWarps + 1;
constexpr int kDecMaxBN = 128;      // sequences (query rows) per launch
constexpr int kDecMaxKeep = 32;     // candidates per CTA and sequence
constexpr int kDecTmemCols = 256;   // two accumulators of up to 128 columns
constexpr int kDecTailBox = 32;     // rows per TMA box of a partly needed tile
constexpr int kDecMaxStages = 12;
constexpr int kDecRows = kDecBM + 2;  // table rows: a tile's documents (at most one per chunk) and a carried one

struct RouteDecParams {
  int n_seq, bn, bn_pad, n_chunks, n_docs, k_blocks, stages, cap, keep, lists, tiles_q, tiles_rem, blocked;
  uint32_t min_key;
  float alpha;
  const float* row_bias;
  const int32_t* chunk_doc;
  unsigned long long* cand;   // [n_seq][gridDim.x * keep]
  int32_t* status;
};

#ifdef MSA_ROUTE_DEC_TRACE
__device__ unsigned long long g_dec_trace[160][12];
#define TRACE(i) g_dec_trace[blockIdx.x][i] = global_ns()
#define TRACE_ADD(i, v) g_dec_trace[blockIdx.x][i] += (v)
#else
#define TRACE(i)
#define TRACE_ADD(i, v)
#endif
struct DecSeg { int start, len, doc; };
struct alignas(16) DecEpiScratch {
  float xpose[16][33];
  DecSeg seg[32];
};

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kDecEpiThreads) : "memory"); }

// First chunk at or after p that starts a document (p itself when it does; n_chunks at the end).  One warp: the
// lanes look at 32 chunks at a time, so a boundary costs one round of global loads, not one per chunk.
__device__ __forceinline__ int snap_to_document(const int32_t* chunk_doc, int p, int n_chunks, int lane) {
  if (p <= 0) return 0;
  if (p >= n_chunks) return n_chunks;
  const int d = chunk_doc[p - 1];
  for (;;) {
    const int c = p + lane;
    const bool other = c >= n_chunks || chunk_doc[c] != d;      // the end of the shard ends the document too
    const uint32_t bal = __ballot_sync(0xffffffffu, other);
    if (bal) return min(p + __ffs(bal) - 1, n_chunks);
    p += 32;
  }
}

// One step of a sorted insertion without branches: (key, doc) falls through the descending list, swapping
// with every entry it beats.  Strict comparison: of two equal scores the earlier document (documents arrive in
// ascending order) stays ahead, which is the tie order of the table path.
template <int KMAX>
__device__ __forceinline__ void list_insert(uint32_t (&lk)[KMAX], int (&ld)[KMAX], uint32_t key, int doc) {
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const bool up = key > lk[i];
    const uint32_t tk = lk[i];
    const int td = ld[i];
    lk[i] = up ? key : tk;
    ld[i] = up ? doc : td;
    key = up ? tk : key;
    doc = up ? td : doc;
  }
}

// (key, doc) a is better than b: the higher score, and of equal scores the earlier document (empty slots, key 0, last).
__device__ __forceinline__ bool list_better(uint32_t ka, int da, uint32_t kb, int db) {
  return ka > kb || (ka == kb && da < db);
}
__device__ __forceinline__ void list_take_better(uint32_t& k, int& d, uint32_t ko, int d_o) {
  const bool other = list_better(ko, d_o, k, d);
  k = other ? ko : k;
  d = other ? d_o : d;
}
// compare-exchange: the better entry ends up in (k0, d0)
__device__ __forceinline__ void list_order_pair(uint32_t& k0, int& d0, uint32_t& k1, int& d1) {
  const bool swap = list_better(k1, d1, k0, d0);
  const uint32_t tk = k0;
  const int td = d0;
  k0 = swap ? k1 : k0;
  d0 = swap ? d1 : d0;
  k1 = swap ? tk : k1;
  d1 = swap ? td : d1;
}

// tmap_k / tmap_k_tail: 128-row and 32-row boxes over the keys, 2-D (row-major keys) or 4-D (tile-blocked keys).
template <int KMAX>
__global__ void __launch_bounds__(kDecThreads, 1)
route_dec_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_k_tail,
                 const __grid_constant__ CUtensorMap tmap_q, const RouteDecParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint64_t s_full[kDecMaxStages], s_empty[kDecMaxStages], s_acc_full[2], s_acc_empty[2], s_drain;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort, s_lo, s_hi;
  __shared__ float s_bias[kDecMaxBN];
  __shared__ DecEpiScratch s_epi[kDecEpiWarps];

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = kDecBM * kDecBK * 2, b_bytes = (uint32_t)p.bn * kDecBK * 2, stage_bytes = a_bytes + b_bytes;
  uint32_t* tbl = reinterpret_cast<uint32_t*>(tiles + (size_t)p.stages * stage_bytes);            // [cap][bn_pad]
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    TRACE(0);
#ifdef MSA_ROUTE_DEC_TRACE
    g_dec_trace[blockIdx.x][9] = 0; g_dec_trace[blockIdx.x][10] = 0;
#endif
    for (int s = 0; s < p.stages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_acc_full[b], 1); mbar_init(&s_acc_empty[b], kDecEpiWarps); }
    mbar_init(&s_drain, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();                                   // the barriers exist
  // This CTA's share of the (whole, aligned) tiles; it owns the documents that START there: both ends of the share
  // are moved forward to the next document start, so its last document may reach into the next CTA's first tile,
  // whose leading rows that CTA masks.
  const int first_tile = (int)blockIdx.x * p.tiles_q + min((int)blockIdx.x, p.tiles_rem);
  const int prologue = min(p.stages, p.k_blocks);    // K blocks of the first tile that are requested before the ends are known
  if (warp == kDecProducerWarp && lane == 0) {
    for (int kb = 0; kb < prologue; ++kb) {          // the ring is empty: no waits; the first tile is read whole
      unsigned char* sa = tiles + (size_t)kb * stage_bytes;
      mbar_expect_tx(&s_full[kb], stage_bytes);
      if (p.blocked) tma_load_4d(sa, &tmap_k, 0, 0, kb, first_tile, &s_full[kb]);
      else tma_load_2d(sa, &tmap_k, kb * kDecBK, first_tile * kDecBM, &s_full[kb]);
    }
    TRACE(2);
    // Everything up to here reads only the bank.  The folded queries and their bias come from the kernel before this
    // one in the stream; as a programmatic dependent this kernel may have started beside it.
    grid_dependency_wait();
    for (int kb = 0; kb < prologue; ++kb)
      tma_load_2d(tiles + (size_t)kb * stage_bytes + a_bytes, &tmap_q, kb * kDecBK, 0, &s_full[kb]);
  }
  if (warp < 2) {                                    // two dependent rounds of global loads, beside the first requests
    const int c = (int)blockIdx.x + warp;            // warp 0: start of this share, warp 1: start of the next
    const long long a = ((long long)c * p.tiles_q + min(c, p.tiles_rem)) * kDecBM;
    const int v = snap_to_document(p.chunk_doc, (int)(a < p.n_chunks ? a : p.n_chunks), p.n_chunks, lane);
    if (lane == 0) *(warp == 0 ? &s_lo : &s_hi) = v;
  }
  if (!(warp == kDecProducerWarp && lane == 0)) grid_dependency_wait();   // (the producer thread has waited above)
  if (warp == kDecMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kDecTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int lo = s_lo, hi = s_hi;
  if (threadIdx.x == 0) TRACE(1);
  const bool owns = lo < hi;                         // false: one document covers the whole share (the first tile is still drained)
  const int n_tiles = owns ? (hi + kDecBM - 1) / kDecBM - first_tile : 1;

  if (warp == kDecProducerWarp) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      for (int s = 0; s < prologue; ++s) { armed |= 1u << s; }
      stage = prologue == p.stages ? 0 : prologue;
      phase = prologue == p.stages ? 1u : 0u;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int tile = first_tile + t, row0 = tile * kDecBM, rows = min(kDecBM, hi - row0);
        // a tile of which only the first rows are wanted (the end of the CTA's last document) comes in 32-row boxes
        const int tail_boxes = (t > 0 && rows <= kDecBM - kDecTailBox) ? (rows + kDecTailBox - 1) / kDecTailBox : 0;
        for (int kb = (t == 0 ? prologue : 0); kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_empty[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          if (tail_boxes == 0) {
            mbar_expect_tx(&s_full[stage], stage_bytes);
            if (p.blocked) tma_load_4d(sa, &tmap_k, 0, 0, kb, tile, &s_full[stage]);
            else tma_load_2d(sa, &tmap_k, kb * kDecBK, row0, &s_full[stage]);
          } else {   // 32-row boxes land where the rows of a 128-row box would (8-row swizzle groups of 1 KiB)
            mbar_expect_tx(&s_full[stage], (uint32_t)tail_boxes * kDecTailBox * kDecBK * 2 + b_bytes);
            for (int j = 0; j < tail_boxes; ++j) {
              unsigned char* dst = sa + (size_t)j * kDecTailBox * kDecBK * 2;
              if (p.blocked) tma_load_4d(dst, &tmap_k_tail, 0, j * kDecTailBox, kb, tile, &s_full[stage]);
              else tma_load_2d(dst, &tmap_k_tail, kb * kDecBK, row0 + j * kDecTailBox, &s_full[stage]);
            }
          }
          tma_load_2d(sa + a_bytes, &tmap_q, kb * kDecBK, 0, &s_full[stage]);
          TRACE(3);
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
  } else if (warp == kDecMmaWarp) {
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
        TRACE(4);
      }
      tc_commit(&s_drain);
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&s_drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
  } else {
    // ------------------------------- epilogue + selection (warps 0-7) ------------------
    const int tid = threadIdx.x;                       // 0..255
    const int quarter = warp & 3, part = warp >> 2;    // TMEM lane quarter; share of the tile's columns
    DecEpiScratch& scr = s_epi[warp];
    for (int i = tid; i < p.cap * p.bn_pad; i += kDecEpiThreads) tbl[i] = p.min_key;
    if (tid < p.bn) s_bias[tid] = tid < p.n_seq ? p.row_bias[tid] : -INFINITY;
    // Selection: every table column (sequence) is walked by p.lists threads, thread (seq, phase) taking the rows
    // phase, phase + lists, ...; each keeps the best `keep` documents it has seen, sorted, in registers
    // (key 0 = empty slot).  With few sequences this spreads the insertion chains over all epilogue warps.
    const int seq = tid % p.bn, phase = tid / p.bn;
    const bool walker = phase < p.lists;
    const bool owns_seq = walker && seq < p.n_seq;
    uint32_t lk[KMAX];
    int ld[KMAX];
#pragma unroll
    for (int i = 0; i < KMAX; ++i) { lk[i] = 0u; ld[i] = 0; }
    if (blockIdx.x == 0 && owns_seq && phase == 0) lk[0] = p.min_key;   // column 0: the dummy document, scored finfo.min like every untouched column
    epi_barrier();
    const int doc_lo = owns ? p.chunk_doc[lo] : 0;         // the first document of this CTA
    int seg_base = doc_lo;                                 // document id of table row 0
    bool carried = false;                                  // row 0 holds the partial maxima of a document that continues

    // chunk -> document ids of a tile, requested one tile ahead (the loads have a tile's time to arrive)
    struct TileIds { int doc, last_doc, next_doc; bool mine, any_mine; };
    auto load_ids = [&](int t) {
      TileIds r;
      const int row0 = (first_tile + t) * kDecBM;
      const int chunk = row0 + quarter * 32 + lane;
      r.mine = owns && t < n_tiles && chunk >= lo && chunk < hi;   // rows before lo belong to the previous CTA's last document
      const int last_chunk = min(row0 + kDecBM, hi) - 1;
      r.any_mine = owns && t < n_tiles && last_chunk >= lo;        // false: the whole tile belongs to the previous CTA
      r.last_doc = r.any_mine ? p.chunk_doc[last_chunk] : 0;
      r.next_doc = r.any_mine && last_chunk + 1 < hi ? p.chunk_doc[last_chunk + 1] : -1;   // first document of the next tile
      r.doc = r.mine ? p.chunk_doc[chunk] : -1 - lane;
      return r;
    };
    TileIds nxt = load_ids(0);
    const uint32_t walkers = __ballot_sync(0xffffffffu, walker);   // lanes of this warp that walk a column

    bool alive = true;       // false once a wait ran out: the remaining tiles only keep the barriers in step
    for (int t = 0; t < n_tiles; ++t) {
      const TileIds cur = nxt;
      nxt = load_ids(t + 1);
      const int last_doc = cur.last_doc, next_doc = cur.next_doc;
      const bool any_mine = cur.any_mine;
      // runs of lanes that hold chunks of one document
      int doc = cur.doc;
      if (cur.mine && (doc < 1 || doc > p.n_docs || (unsigned)(doc - seg_base) >= (unsigned)p.cap)) {
        if (part == 0) atomicAdd(p.status + 2, 1);      // an id outside the table: counted, never used as a row
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
#ifdef MSA_ROUTE_DEC_TRACE
      const unsigned long long tw0 = global_ns();
#endif
      if (alive) alive = mbar_wait(&s_acc_full[buf], acc_phase, abort_flag, p.status, 4);
#ifdef MSA_ROUTE_DEC_TRACE
      if (tid == 0) { TRACE_ADD(9, global_ns() - tw0); if (t == 0) TRACE(5); TRACE(6); }
#endif
      alive = __all_sync(0xffffffffu, alive);
      if (alive) {
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kDecMaxBN;
        const int n_items = n_seg * 16;
        for (int c0 = part * 16; c0 < p.bn; c0 += 16 * (kDecEpiWarps / 4)) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) scr.xpose[j][lane] = __uint_as_float(r[j]) + s_bias[c0 + j];
          __syncwarp();
          // (document, column) pairs dealt over the lanes: max over the document's chunks, one shared-memory atomic
          for (int item = lane; item < n_items; item += 32) {
            const DecSeg e = scr.seg[item >> 4];
            const int j = item & 15, col = c0 + j;
            if (e.doc > 0 && col < p.n_seq) {
              float m = scr.xpose[j][e.start];
#pragma unroll 8
              for (int u = 1; u < e.len; ++u) m = fmaxf(m, scr.xpose[j][e.start + u]);   // independent loads
              atomicMax(tbl + (size_t)(e.doc - seg_base) * p.bn_pad + col, float_to_key(m * p.alpha));
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_acc_empty[buf]);
      }

      // ---- walk the tile's finished documents
      epi_barrier();                                     // every warp's table updates of this tile are in
      const int n_rows = any_mine ? max(carried ? 1 : 0, min(min(last_doc, p.n_docs) - seg_base + 1, p.cap)) : 0;
      const bool open = n_rows >= 1 && next_doc == last_doc && last_doc - seg_base == n_rows - 1;   // the last row's document continues
      const int n_done = open ? n_rows - 1 : n_rows;
      if (walker) {
        for (int r0 = 0; r0 < n_done; r0 += p.lists) {   // the same trip count for every walker of the warp
          const int r = r0 + phase;
          uint32_t key = 0u;                             // 0 never enters a list
          if (r < n_done) {
            key = tbl[(size_t)r * p.bn_pad + seq];
            tbl[(size_t)r * p.bn_pad + seq] = p.min_key;
          }
          // the whole warp takes the insertion chain or skips it together
          if (__any_sync(walkers, owns_seq && key > lk[KMAX - 1])) list_insert<KMAX>(lk, ld, key, seg_base + r);
        }
        if (phase == 0) {
          uint32_t keep_val = p.min_key;
          if (open) {                                    // carry the open document's partial maxima to row 0
            keep_val = tbl[(size_t)n_done * p.bn_pad + seq];
            tbl[(size_t)n_done * p.bn_pad + seq] = p.min_key;
          }
          tbl[seq] = keep_val;
        }
      }
      seg_base = max(doc_lo, open ? last_doc : (next_doc > 0 ? next_doc : seg_base));
      carried = open;
      epi_barrier();                                     // the table is clean before the next tile is reduced into it
      if (tid == 0) TRACE(7);
    }

    if (tid == 0) grid_launch_dependents();      // the final selection may start launching; it waits for this grid to end
    // ---- merge the lists of a sequence, pairwise: in round r the thread of phase p (p % 2^(r+1) == 0) takes the sorted
    // list of phase p + 2^r from shared memory; the element-wise better of (mine[i], theirs[KMAX-1-i]) are the best
    // KMAX of both as a bitonic sequence, which a merge network sorts in registers.  The operand ring is free now (the
    // last accumulator was complete, so every copy has landed and every MMA has read its operands) and holds the lists,
    // element i of thread t at [i][t].
    unsigned long long* xchg = reinterpret_cast<unsigned long long*>(tiles);
    for (int stride = 1; stride < p.lists; stride *= 2) {
      const bool sender = walker && (phase & (2 * stride - 1)) == stride;
      const bool receiver = walker && (phase & (2 * stride - 1)) == 0;
      if (sender) {
#pragma unroll
        for (int i = 0; i < KMAX; ++i) xchg[i * kDecEpiThreads + tid] = ((unsigned long long)lk[i] << 32) | (uint32_t)ld[i];
      }
      epi_barrier();
      if (receiver) {
        const int partner = tid + stride * p.bn;
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
          const unsigned long long o = xchg[(KMAX - 1 - i) * kDecEpiThreads + partner];
          list_take_better(lk[i], ld[i], (uint32_t)(o >> 32), (int)(uint32_t)o);
        }
#pragma unroll
        for (int span = KMAX / 2; span >= 1; span /= 2)
#pragma unroll
          for (int i = 0; i < KMAX; ++i)
            if ((i & span) == 0) list_order_pair(lk[i], ld[i], lk[i + span], ld[i + span]);
      }
    }
    if (alive && owns_seq && phase == 0) {
      unsigned long long* dst = p.cand + ((long long)seq * gridDim.x + blockIdx.x) * p.keep;
#pragma unroll
      for (int i = 0; i < KMAX; ++i)
        if (i < p.keep)
          dst[i] = lk[i] ? (((unsigned long long)lk[i] << 32) | (unsigned long long)(0xffffffffu - (uint32_t)ld[i])) : 0ull;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TRACE(8);
  tc_fence_after();
  if (warp == kDecMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDecTmemCols) : "memory");
}

// Shared-memory plan for bn query rows: as many operand stages as fit beside the document table.
static bool route_dec_plan(int bn, int keep, RouteDecParams* p, size_t* smem) {
  const size_t stage_bytes = (size_t)kDecBM * kDecBK * 2 + (size_t)bn * kDecBK * 2;
  const int bn_pad = bn + 1;
  const size_t budget = 202 * 1024;   // dynamic part; the kernel's static arrays (epilogue scratch) take 23 KB more of the 227 KB
  const size_t tbl = ((size_t)kDecRows * bn_pad * 4 + 15) & ~(size_t)15;
  int lists = 1;                                                           // walker threads per sequence: a power of two
  int max_lists = 2;                                                       // every doubling costs a merge round at the end
  if (const char* e = getenv("MSA_B200_DEC_LISTS")) max_lists = atoi(e);    // tuning knob
  while (lists * 2 <= kDecEpiThreads / bn && lists * 2 <= max_lists) lists *= 2;
  const size_t merge_bytes = (size_t)kDecEpiThreads * (keep <= 16 ? 16 : 32) * 8;   // the exchanged lists, in the freed ring
  for (int stages = kDecMaxStages; stages >= 3; --stages) {
    const size_t total = 1024 + stages * stage_bytes + tbl;
    if (total <= budget && stages * stage_bytes >= merge_bytes) {
      p->stages = stages; p->cap = kDecRows; p->bn = bn; p->bn_pad = bn_pad; p->keep = keep; p->lists = lists;
      *smem = total;
      return true;
    }
  }
  return false;
}

}  // namespace msa

using namespace msa;

namespace msa {
int launch_topk_from_candidates(const unsigned long long* cand, int n_in, int n_seq, int k_eff, const int64_t* doc_ids_table,
                                float* out_scores, int64_t* out_local, int64_t* out_global, cudaStream_t stream,
                                bool pdl = false);
}

#ifdef MSA_ROUTE_DEC_TRACE
extern "C" int msa_route_dec_trace(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_dec_trace, sizeof(g_dec_trace)) == cudaSuccess ? 0 : 1;
}
#endif
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
                                      uint32_t flags, int32_t* status, void* stream) {
  MSA_REQUIRE(q_folded && row_bias && rk && chunk_doc && out_scores && out_local_ids && status && workspace,
              "route_score_select: null pointer");
  MSA_REQUIRE(n_seq >= 1 && n_chunks >= 1 && kdim > 0 && n_docs >= 1 && k >= 1, "route_score_select: bad sizes");
  MSA_REQUIRE(alpha > 0.f, "route_score_select: alpha must be positive (it is applied after the max)");
  if (dtype != MSA_BF16 || n_seq > kDecMaxBN || k > kDecMaxKeep || kdim % kDecBK != 0) {
    set_error("route_score_select takes bf16 keys, at most %d sequences of one row, k <= %d and kdim %% %d == 0; "
              "use msa_route_scores + msa_topk_select for other shapes", kDecMaxBN, kDecMaxKeep, kDecBK);
    return MSA_ERR_UNSUPPORTED;
  }
  const bool blocked = (flags & MSA_ROUTE_KEYS_BLOCKED) != 0;
  MSA_REQUIRE(aligned16(q_folded) && aligned16(rk) && (blocked || (rk_chunk_stride % 8 == 0 && rk_chunk_stride >= kdim)),
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
  p.tiles_q = n_tiles / grid; p.tiles_rem = n_tiles % grid; p.blocked = blocked ? 1 : 0;
  p.min_key = float_to_key(min_val); p.alpha = alpha; p.row_bias = row_bias; p.chunk_doc = chunk_doc;
  p.cand = (unsigned long long*)workspace; p.status = status;

  CUtensorMap map_k, map_k_tail, map_q;
  if (blocked) {
    MSA_OK_OR_RETURN(make_map_blocked(&map_k, rk, (uint64_t)n_tiles, (uint64_t)p.k_blocks));
    MSA_OK_OR_RETURN(make_map_blocked(&map_k_tail, rk, (uint64_t)n_tiles, (uint64_t)p.k_blocks, kDecTailBox));
  } else {
    MSA_OK_OR_RETURN(make_map(&map_k, rk, (uint64_t)n_chunks, (uint64_t)kdim, (uint64_t)rk_chunk_stride, kDecBK, kDecBM));
    MSA_OK_OR_RETURN(make_map(&map_k_tail, rk, (uint64_t)n_chunks, (uint64_t)kdim, (uint64_t)rk_chunk_stride, kDecBK, kDecTailBox));
  }
  MSA_OK_OR_RETURN(make_map(&map_q, q_folded, (uint64_t)n_seq, (uint64_t)kdim, (uint64_t)kdim, kDecBK, (uint32_t)bn));
  static DeviceSmem configured[2] = {};
  cudaStream_t st = (cudaStream_t)stream;
  // programmatic dependent launches: this kernel sets itself up and requests its first key tile while the fold
  // kernel before it still runs, and the final selection is resident when this kernel ends
  static const bool pdl = getenv("MSA_B200_NO_PDL") == nullptr;   // measured: 84.6 -> 81.5 us per layer-step at 32 sequences
  if (k_eff <= 16) {
    MSA_OK_OR_RETURN(ensure_dynamic_smem(route_dec_kernel<16>, smem, configured[0]));
    MSA_CUDA_OK(launch_kernel_pdl(route_dec_kernel<16>, dim3(grid), dim3(kDecThreads), smem, st, pdl, map_k, map_k_tail, map_q, p));
  } else {
    MSA_OK_OR_RETURN(ensure_dynamic_smem(route_dec_kernel<32>, smem, configured[1]));
    MSA_CUDA_OK(launch_kernel_pdl(route_dec_kernel<32>, dim3(grid), dim3(kDecThreads), smem, st, pdl, map_k, map_k_tail, map_q, p));
  }
  MSA_LAUNCH_OK("route_dec_kernel");
  return launch_topk_from_candidates(p.cand, grid * k_eff, n_seq, k_eff, doc_ids_table, out_scores, out_local_ids,
                                     out_global_ids, st, pdl);
}
