// Routing on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16.
//
// The head-mean score of every (query token, chunk) pair is one 1024-wide dot product of
// the folded query row with the chunk's pooled router key, so a layer's scoring is the
// contraction  S[c, r] = sum_k Kr[c, k] * Qf[r, k]  followed by reductions.  The kernel
// puts CHUNKS on the UMMA M axis (128 TMEM lanes = 128 chunks) and QUERY ROWS on the N
// axis (TMEM columns): after tcgen05.ld each epilogue thread owns one chunk and sees all
// query rows of the tile in its registers, so
//     max over a sequence's tokens   = an in-thread max over columns  (no shuffles),
//     max over a document's chunks   = a shuffle scan over the lanes that hold that document (batched
//                                      over 16 columns; with one row per sequence: a shared-memory
//                                      transpose that deals (document, column) pairs over the lanes),
//     table update                   = a plain store for documents no other warp touches, else one
//                                      atomicMax on an order-preserving key per (sequence, document, warp).
// Per-(token, chunk) scores therefore never leave the SM.
//
// Persistent, warp specialised: warps 0-3 epilogue (TMEM lane quarter = warp id), warp 4
// TMA producer, warp 5 MMA issuer + TMEM owner.  Operands are streamed in 64-element
// (128-byte, SWIZZLE_128B) K blocks through a ring of shared-memory stages; two TMEM
// accumulators let the epilogue of tile i overlap the MMAs of tile i+1.  Loads are plain
// per-CTA TMA (no cluster qualifiers).  Every mbarrier wait is bounded by a wall-clock
// limit; on expiry the CTA raises status[0], drains what it has in flight, frees TMEM and
// returns.
//
// Bounds: flops = 2*rows*chunks*kdim on the tensor pipe; bytes = chunks*kdim*2 (router keys,
// once) + rows*kdim*2 (queries) from HBM.  Tensor bound when rows >~ 220, HBM bound below.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "route.cuh"
#include "tc_common.cuh"

namespace msa {

constexpr int kBM = 128;        // chunks per tile (UMMA M)
constexpr int kBK = 64;         // bf16 elements per K block = one 128-byte swizzle row
constexpr int kUmmaK = 16;      // K of one tcgen05.mma (bf16)
constexpr int kTcThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kMaxStages = 12;
constexpr int kTmemCols = 512;

struct RouteTcParams {
  int n_rows, n_seq, s_pad, bn, n_chunks, n_docs, n_ctiles, n_qtiles, qgroup, k_blocks, stages, blocked;
  uint32_t min_key;
  float alpha;
  const float* row_bias;
  const int32_t* chunk_doc;
  uint32_t* keys;
  long long table_stride;
  int32_t* status;
};

struct TileCoord { int ct, qt; };
__device__ __forceinline__ TileCoord tile_coord(const RouteTcParams& p, long long t) {
  // query tiles are walked in groups small enough to stay in L2 while every chunk tile passes
  const long long per_group = (long long)p.n_ctiles * p.qgroup;
  const int grp = (int)(t / per_group);
  const long long r = t - grp * per_group;
  const int gq = min(p.qgroup, p.n_qtiles - grp * p.qgroup);
  return TileCoord{(int)(r / gq), grp * p.qgroup + (int)(r % gq)};
}

// ---- epilogue pieces shared by the 1-CTA and the 2-CTA kernel ---------------------------
// Segments = runs of lanes holding chunks of one document.  `dist` is the distance to the
// segment's first lane; the last lane of a segment publishes the document's score.  A document
// that lies wholly inside this warp's 32 chunks (and whose sequence is not cut over several
// column tiles) has no other writer: a plain store replaces the atomic.
struct SegInfo { int doc, dist, max_len, n_seg; bool publish, exclusive; };
struct SegEntry { int start, len, doc, exclusive; };   // one document's lanes inside a warp
struct EpiScratch {                                      // per epilogue warp
  float xpose[16][33];                                   // 16 columns x 32 lanes (+1 pad)
  SegEntry seg[32];
};

__device__ __forceinline__ SegInfo seg_info(const RouteTcParams& p, int chunk, int lane, EpiScratch& scr) {
  int doc = chunk < p.n_chunks ? p.chunk_doc[chunk] : -1 - lane;  // out-of-range lanes stay alone
  if (chunk < p.n_chunks && (doc < 1 || doc > p.n_docs)) {  // an id outside the table: counted, never used as a column
    atomicAdd(p.status + 2, 1);
    doc = -1 - lane;
  }
  const int doc_up = __shfl_up_sync(0xffffffffu, doc, 1), doc_dn = __shfl_down_sync(0xffffffffu, doc, 1);
  const bool head = lane == 0 || doc_up != doc, tail = lane == 31 || doc_dn != doc;
  const uint32_t heads = __ballot_sync(0xffffffffu, head);
  const int head_lane = 31 - __clz(heads & (0xffffffffu >> (31 - lane)));
  const int dist = lane - head_lane;
  int max_len = dist + 1;  // longest segment in this warp
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_len = max(max_len, __shfl_xor_sync(0xffffffffu, max_len, o));
  bool starts_here = true, ends_here = true;  // does the document cross the warp's edges?
  if (lane == 0 && chunk > 0 && chunk < p.n_chunks) starts_here = p.chunk_doc[chunk - 1] != doc;
  if (lane == 31 && chunk + 1 < p.n_chunks) ends_here = p.chunk_doc[chunk + 1] != doc;
  const bool open_lo = !__shfl_sync(0xffffffffu, starts_here, 0), open_hi = !__shfl_sync(0xffffffffu, ends_here, 31);
  const bool crosses = (open_lo && head_lane == 0) || (open_hi && (heads >> lane) <= 1u);
  const bool exclusive = !crosses && p.s_pad <= p.bn;
  // segment table: entry i describes the i-th run of lanes (documents and out-of-range lanes alike)
  const int seg_idx = __popc(heads & ((1u << lane) - 1u));
  if (head) {
    const uint32_t later = lane == 31 ? 0u : (heads >> (lane + 1));
    const int len = later ? __ffs(later) : 32 - lane;
    scr.seg[seg_idx] = SegEntry{lane, len, doc, exclusive ? 1 : 0};
  }
  __syncwarp();
  return SegInfo{doc, dist, max_len, __popc(heads), tail && doc > 0, exclusive};
}

// Reads this warp's 32 accumulator rows (one chunk per lane, p.bn columns) and publishes the
// per-(sequence, document) maxima.
// `part` of `n_parts`: the warps that share a TMEM lane quarter split the tile's columns among themselves.
__device__ __forceinline__ void epilogue_compute(const RouteTcParams& p, const SegInfo& si, const float* bias,
                                                 uint32_t taddr, int q0, EpiScratch& scr, int lane, int part = 0,
                                                 int n_parts = 1) {
  const int seg = min(p.s_pad, p.bn);  // columns of one sequence inside a tile
  auto publish_score = [&](float v, int seq) {
    if (seq < p.n_seq) {
      const uint32_t key = float_to_key(v * p.alpha);
      uint32_t* dst = p.keys + (long long)seq * p.table_stride + si.doc;
      if (si.exclusive) *dst = max(key, p.min_key);
      else atomicMax(dst, key);
    }
  };
  auto load16 = [&](int c0, float (&v)[16]) {
    uint32_t r[16];
    tmem_ld16(taddr + c0, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) + bias[c0 + j];
  };
  // Segmented max over the lanes of a document: log2(longest segment) shuffle steps, done for a
  // whole batch of independent values at a time so that the shuffles pipeline.
  if (p.s_pad == 1) {  // every column is its own sequence
    // 16 columns at a time go through shared memory: lane = chunk writes its 16 values, then the
    // (document, column) pairs are dealt out over the lanes, so every lane reduces and publishes
    // distinct pairs instead of all lanes shuffling every column.
    const int n_items = si.n_seg * 16;
    for (int c0 = part * 16; c0 < p.bn; c0 += 16 * n_parts) {
      float v[16];
      load16(c0, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) scr.xpose[j][lane] = v[j];
      __syncwarp();
      for (int item = lane; item < n_items; item += 32) {
        const SegEntry e = scr.seg[item >> 4];
        const int j = item & 15;
        if (e.doc > 0) {
          float m = scr.xpose[j][e.start];
          for (int t = 1; t < e.len; ++t) m = fmaxf(m, scr.xpose[j][e.start + t]);
          const int seq = q0 + c0 + j;
          if (seq < p.n_seq) {
            const uint32_t key = float_to_key(m * p.alpha);
            uint32_t* dst = p.keys + (long long)seq * p.table_stride + e.doc;
            if (e.exclusive) *dst = max(key, p.min_key);
            else atomicMax(dst, key);
          }
        }
      }
      __syncwarp();
    }
  } else {             // `seg` consecutive columns belong to one sequence: in-thread max first
    for (int s0 = part * seg; s0 < p.bn; s0 += seg * n_parts) {
      float run = -INFINITY;
      for (int c0 = s0; c0 < s0 + seg; c0 += 16) {
        float v[16];
        load16(c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) run = fmaxf(run, v[j]);
      }
      for (int d = 1; d < si.max_len; d <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, run, d);
        if (si.dist >= d) run = fmaxf(run, o);
      }
      if (si.publish) publish_score(run, (q0 + s0) / p.s_pad);
    }
  }
}

// kEpiWarps = 4: one epilogue warp per TMEM lane quarter.  kEpiWarps = 8 (bandwidth-bound shapes, one row per
// sequence): two warps per quarter split the tile's columns; there the epilogue, not the stream, was what set the
// pace (a tile's 16 K blocks arrive in ~5 us, its reduction took longer), and the CTA's other warps are idle anyway.
template <int kEpiWarps>
__global__ void __launch_bounds__((kEpiWarps + 2) * 32, 1)
route_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
                const RouteTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint64_t s_full[kMaxStages], s_empty[kMaxStages], s_acc_full[2], s_acc_empty[2], s_drain;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  // kEpiWarps == 4: one private bias copy per epilogue warp, refilled per tile (query tiles change).  More warps
  // only run with a single query tile: one copy, which every warp fills with the same values before it reads it.
  __shared__ float s_bias[kEpiWarps == 4 ? 4 : 1][kRouteMaxN];
  __shared__ EpiScratch s_epi[kEpiWarps];
  constexpr int kProducerWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = kBM * kBK * 2, b_bytes = (uint32_t)p.bn * kBK * 2, stage_bytes = a_bytes + b_bytes;
  volatile int* abort_flag = &s_abort;
  const long long n_tiles = (long long)p.n_ctiles * p.n_qtiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_acc_full[b], 1); mbar_init(&s_acc_empty[b], kEpiWarps); }
    mbar_init(&s_drain, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(p, t);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_empty[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          mbar_expect_tx(&s_full[stage], stage_bytes);
          if (p.blocked) tma_load_4d(sa, &tmap_k, 0, 0, kb, tc.ct, &s_full[stage]);   // one contiguous 16 KiB
          else tma_load_2d(sa, &tmap_k, kb * kBK, tc.ct * kBM, &s_full[stage]);
          tma_load_2d(sa + a_bytes, &tmap_q, kb * kBK, tc.qt * p.bn, &s_full[stage]);
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
  } else if (warp == kMmaWarp) {
    // ------------------------------- MMA issuer ----------------------------------------
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, both K-major, N=bn, M=128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.bn >> 3) << 17) |
                             ((uint32_t)(kBM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      long long it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++it) {
        const int buf = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!(ok = mbar_wait(&s_acc_empty[buf], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kRouteMaxN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_full[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint64_t a_desc = make_smem_desc(sa), b_desc = make_smem_desc(sa + a_bytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)  // +32 bytes of K per step = +2 in the address field
            tc_mma_bf16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&s_empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(&s_acc_full[buf]);
      }
      // drain: everything issued so far must retire before TMEM is freed
      tc_commit(&s_drain);
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&s_drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
  } else {
    // ------------------------------- epilogue (warps 0 .. kEpiWarps-1) -----------------
    const int quarter = warp & 3, part = warp >> 2;   // TMEM lane quarter; share of the columns
    long long it = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++it) {
      const TileCoord tc = tile_coord(p, t);
      const int buf = (int)(it & 1);
      const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
      const int q0 = tc.qt * p.bn;
      float* bias = s_bias[kEpiWarps == 4 ? warp : 0];
      __syncwarp();  // the previous tile's reads of this warp's bias copy are done
      if (kEpiWarps == 4 || it == 0)
        for (int j = lane; j < p.bn; j += 32) bias[j] = (q0 + j < p.n_rows) ? p.row_bias[q0 + j] : -INFINITY;
      const SegInfo si = seg_info(p, tc.ct * kBM + quarter * 32 + lane, lane, s_epi[warp]);
      __syncwarp();
      // every lane waits; the warp then agrees on the outcome so that it never diverges
      ok = mbar_wait(&s_acc_full[buf], acc_phase, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kRouteMaxN;

      epilogue_compute(p, si, bias, taddr, q0, s_epi[warp], lane, part, kEpiWarps / 4);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_acc_empty[buf]);
    }
  }

  // teardown: all roles meet, then the allocating warp returns TMEM
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// =========================================================================================
// 2-CTA variant (cta_group::2) for full 256-row query tiles.
//
// A cluster of two CTAs on neighbouring SMs computes a 256-chunk x 256-row tile with one
// tcgen05.mma.cta_group::2 stream issued by the leader (cluster rank 0).  Each CTA stages only
// ITS 128 chunks and ITS 128 query rows per K block (32 KB instead of 48 KB), and the pair's
// MMA reads both halves from both shared memories: a third less L2 -> SM operand traffic per
// flop, which is what limits the 1-CTA kernel (64 % of crossbar peak at 86 % tensor activity).
// Each CTA's TMEM holds the 128 accumulator rows of its own chunks, so the epilogue is the same.
//
// Cross-CTA signalling, all with plain single-destination forms:
//   * both CTAs' TMA loads complete on the LEADER's `full` barrier (cta_group::2 load, barrier
//     address mapped into the leader's shared memory);
//   * the leader's tcgen05.commit is issued twice, once per CTA, for `empty` and `acc_full`;
//   * every epilogue warp of both CTAs arrives on the leader's `acc_empty`.
// =========================================================================================
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

constexpr int kPairBN = 256;  // query rows per cluster tile
constexpr int kPairBM = 256;  // chunks per cluster tile (128 per CTA)

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads, 1)
route_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_q,
                     const RouteTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint64_t s_full[kMaxStages], s_empty[kMaxStages], s_acc_full[2], s_acc_empty[2], s_drain;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_bias[kEpiThreads / 32][kRouteMaxN];
  __shared__ EpiScratch s_epi[kEpiThreads / 32];

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t half_bytes = kBM * kBK * 2, stage_bytes = 2 * half_bytes;  // 128 chunks + 128 query rows
  volatile int* abort_flag = &s_abort;
  const long long n_tiles = (long long)p.n_ctiles * p.n_qtiles;  // counted in cluster tiles
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_acc_full[b], 1); mbar_init(&s_acc_empty[b], 2 * (kEpiThreads / 32)); }
    mbar_init(&s_drain, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {  // both CTAs of the pair allocate, with the same destination offset
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 4) {
    // ------------------------------- TMA producer (each CTA loads its halves) ----------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long t = cluster_id; t < n_tiles && ok; t += n_clusters) {
        const TileCoord tc = tile_coord(p, t);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_empty[stage], phase ^ 1u, abort_flag, p.status, 1))) break;
          unsigned char* sa = tiles + (size_t)stage * stage_bytes;
          if (leader) mbar_expect_tx(&s_full[stage], 2 * stage_bytes);  // both CTAs' bytes land on this barrier
          const uint32_t bar = map_to_cta(smem_u32(&s_full[stage]), 0);
          tma_load_2d_pair(sa, &tmap_k, kb * kBK, tc.ct * kPairBM + (int)rank * kBM, bar);
          tma_load_2d_pair(sa + half_bytes, &tmap_q, kb * kBK, tc.qt * kPairBN + (int)rank * (kPairBN / 2), bar);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      // on give-up the copies in flight are drained by the cluster-wide teardown wait below
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer (leader CTA only) ----------------------
    if (lane == 0 && leader) {
      // instruction descriptor: D=f32, A=B=bf16, both K-major, N=256, M=256 (128 rows per CTA)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPairBN >> 3) << 17) |
                             ((uint32_t)(kPairBM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      long long it = 0;
      bool ok = true;
      for (long long t = cluster_id; t < n_tiles && ok; t += n_clusters, ++it) {
        const int buf = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!(ok = mbar_wait(&s_acc_empty[buf], acc_phase ^ 1u, abort_flag, p.status, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * kRouteMaxN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!(ok = mbar_wait(&s_full[stage], phase, abort_flag, p.status, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint64_t a_desc = make_smem_desc(sa), b_desc = make_smem_desc(sa + half_bytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            tc_mma_bf16_pair(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(smem_u32(&s_empty[stage]));                  // this CTA's stage
          tc_commit_pair(map_to_cta(smem_u32(&s_empty[stage]), 1));   // the partner's stage
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          tc_commit_pair(smem_u32(&s_acc_full[buf]));
          tc_commit_pair(map_to_cta(smem_u32(&s_acc_full[buf]), 1));
        }
      }
      tc_commit_pair(smem_u32(&s_drain));
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&s_drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
  } else {
    // ------------------------------- epilogue (warps 0-3 of both CTAs) -----------------
    long long it = 0;
    bool ok = true;
    for (long long t = cluster_id; t < n_tiles && ok; t += n_clusters, ++it) {
      const TileCoord tc = tile_coord(p, t);
      const int buf = (int)(it & 1);
      const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
      const int q0 = tc.qt * kPairBN;
      float* bias = s_bias[warp];
      __syncwarp();
      for (int j = lane; j < kPairBN; j += 32) bias[j] = (q0 + j < p.n_rows) ? p.row_bias[q0 + j] : -INFINITY;
      const SegInfo si = seg_info(p, tc.ct * kPairBM + (int)rank * kBM + (int)threadIdx.x, lane, s_epi[warp]);
      __syncwarp();
      ok = mbar_wait(&s_acc_full[buf], acc_phase, abort_flag, p.status, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)buf * kRouteMaxN;
      epilogue_compute(p, si, bias, taddr, q0, s_epi[warp], lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s_acc_empty[buf]), 0));
    }
  }

  // teardown: the pair meets (the leader has drained its MMAs), then both CTAs return TMEM
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 5)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// The bounded wait on its own: one CTA waits on a barrier that nothing ever completes, with the
// caller's limit, and reports through `status` exactly as the routing kernel would.
__global__ void wait_selftest_kernel(unsigned long long limit_ns, int32_t* status) {
  __shared__ uint64_t s_bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    mbar_init(&s_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool ok = mbar_wait(&s_bar, 0, &s_abort, status, 9, limit_ns);
  if (!ok && threadIdx.x == 0) atomicExch(status + 1, 1);
}

// ---- host side ------------------------------------------------------------------------
int launch_route_tc(const void* qf, const float* row_bias, int n_seq, int s_pad, const void* rk, int64_t rk_stride,
                    int n_chunks, int kdim, const int32_t* chunk_doc, int n_docs, float alpha, float min_val,
                    uint32_t* keys, int64_t table_stride, int32_t* status, bool blocked, cudaStream_t stream) {
  MSA_REQUIRE(kdim % kBK == 0, "route (tensor-core path): kdim=%d must be a multiple of %d", kdim, kBK);
  MSA_REQUIRE(aligned16(qf) && aligned16(rk) && rk_stride % 8 == 0 && rk_stride >= kdim,
              "route (tensor-core path): rows must be 16-byte aligned");
  RouteTcParams p{};
  p.n_seq = n_seq; p.s_pad = s_pad; p.n_rows = n_seq * s_pad; p.n_chunks = n_chunks; p.n_docs = n_docs;
  if (s_pad == 1) {
    p.bn = n_seq >= kRouteMaxN ? kRouteMaxN : (n_seq + 15) / 16 * 16;
  } else {
    MSA_REQUIRE(s_pad % 16 == 0, "route: s_pad=%d must be 1 or a multiple of 16 (see msa_route_s_pad)", s_pad);
    if (s_pad <= kRouteMaxN) {
      int per_tile = kRouteMaxN / s_pad;
      if (per_tile > n_seq) per_tile = n_seq;
      p.bn = s_pad * per_tile;
    } else {
      const int nt = (s_pad + kRouteMaxN - 1) / kRouteMaxN;
      MSA_REQUIRE(s_pad % nt == 0 && (s_pad / nt) % 16 == 0,
                  "route: s_pad=%d cannot be cut into equal 16-row-aligned tiles (see msa_route_s_pad)", s_pad);
      p.bn = s_pad / nt;
    }
  }
  p.n_ctiles = (n_chunks + kBM - 1) / kBM;
  p.n_qtiles = (p.n_rows + p.bn - 1) / p.bn;
  p.k_blocks = kdim / kBK;
  const size_t stage_bytes = (size_t)kBM * kBK * 2 + (size_t)p.bn * kBK * 2;
  // bandwidth-bound shapes (one row per sequence, a single query tile): 8 or 16 epilogue warps and their scratch
  const int epi_warps = (s_pad == 1 && n_seq <= kRouteMaxN) ? (p.bn > 64 ? 16 : 8) : 4;
  p.stages = (int)(((epi_warps == 16 ? 180 : epi_warps == 8 ? 196 : 204) * 1024) / stage_bytes);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (const char* e = getenv("MSA_B200_ROUTE_STAGES")) {   // tuning knob: fewer operand stages than fit
    const int v = atoi(e);
    if (v >= 2 && v < p.stages) p.stages = v;
  }
  MSA_REQUIRE(p.stages >= 2, "route: tile does not fit shared memory");
  const size_t qtile_bytes = (size_t)p.bn * kdim * 2;
  p.qgroup = (int)((32u << 20) / qtile_bytes);
  if (p.qgroup < 1) p.qgroup = 1;
  if (p.qgroup > p.n_qtiles) p.qgroup = p.n_qtiles;
  p.alpha = alpha; p.row_bias = row_bias; p.chunk_doc = chunk_doc; p.keys = keys; p.table_stride = table_stride;
  p.status = status;
  p.min_key = float_to_key(min_val);

  p.blocked = blocked ? 1 : 0;
  CUtensorMap map_k, map_q;
  int rc = blocked ? make_map_blocked(&map_k, rk, (uint64_t)p.n_ctiles, (uint64_t)p.k_blocks)
                   : make_map(&map_k, rk, (uint64_t)n_chunks, (uint64_t)kdim, (uint64_t)rk_stride, kBK, kBM);
  if (rc != MSA_OK) return rc;
  rc = make_map(&map_q, qf, (uint64_t)p.n_rows, (uint64_t)kdim, (uint64_t)kdim, kBK, (uint32_t)p.bn);
  if (rc != MSA_OK) return rc;

  int n_sm = 0;
  MSA_OK_OR_RETURN(device_sm_count(&n_sm));
  static DeviceSmem smem_set{}, smem_set_8{}, smem_set_16{}, pair_set{};
  const size_t smem = (size_t)p.stages * stage_bytes + 1024;
  if (epi_warps == 16) MSA_OK_OR_RETURN(ensure_dynamic_smem(route_tc_kernel<16>, smem, smem_set_16));
  else if (epi_warps == 8) MSA_OK_OR_RETURN(ensure_dynamic_smem(route_tc_kernel<8>, smem, smem_set_8));
  else MSA_OK_OR_RETURN(ensure_dynamic_smem(route_tc_kernel<4>, smem, smem_set));
  const long long n_tiles = (long long)p.n_ctiles * p.n_qtiles;
  // Tensor-bound shapes (full 256-row query tiles, enough chunk tiles to fill the GPU) run on CTA pairs.
  static const bool pair_off = getenv("MSA_B200_ROUTE_NO_PAIR") != nullptr;
  if (!pair_off && !blocked && p.bn == kPairBN && p.n_rows % kPairBN == 0 && n_tiles >= 2ll * n_sm) {
    RouteTcParams p2 = p;
    p2.n_ctiles = (n_chunks + kPairBM - 1) / kPairBM;
    p2.stages = 6;  // 6 x 32 KB
    CUtensorMap map_q2;
    rc = make_map(&map_q2, qf, (uint64_t)p.n_rows, (uint64_t)kdim, (uint64_t)kdim, kBK, (uint32_t)(kPairBN / 2));
    if (rc != MSA_OK) return rc;
    const size_t smem2 = (size_t)p2.stages * 2 * kBM * kBK * 2 + 1024;
    MSA_OK_OR_RETURN(ensure_dynamic_smem(route_tc_pair_kernel, smem2, pair_set));
    const long long tiles2 = (long long)p2.n_ctiles * p2.n_qtiles;
    long long clusters = n_sm / 2;
    if (clusters > tiles2) clusters = tiles2;
    route_tc_pair_kernel<<<(int)(2 * clusters), kTcThreads, smem2, stream>>>(map_k, map_q2, p2);
    MSA_LAUNCH_OK("route_tc_pair_kernel");
    return MSA_OK;
  }
  const int grid = (int)(n_tiles < n_sm ? n_tiles : n_sm);
  if (epi_warps == 16) route_tc_kernel<16><<<grid, 18 * 32, smem, stream>>>(map_k, map_q, p);
  else if (epi_warps == 8) route_tc_kernel<8><<<grid, 10 * 32, smem, stream>>>(map_k, map_q, p);
  else route_tc_kernel<4><<<grid, kTcThreads, smem, stream>>>(map_k, map_q, p);
  MSA_LAUNCH_OK("route_tc_kernel");
  return MSA_OK;
}

}  // namespace msa

extern "C" int msa_selftest_bounded_wait(int64_t limit_ns, int32_t* status, void* stream) {
  MSA_REQUIRE(status && limit_ns > 0 && limit_ns <= 1000000000ll, "selftest: limit must be in (0, 1e9] ns");
  MSA_CUDA_OK(cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), (cudaStream_t)stream));
  msa::wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, status);
  MSA_LAUNCH_OK("wait_selftest_kernel");
  return MSA_OK;
}
