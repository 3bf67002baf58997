// Stage-1 attention inside every document on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16,
// head_dim 128, for documents that are runs of consecutive tokens of one row.
//
// Work item = 128 query tokens of one head of one document.  Persistent CTAs (two per SM: 97 KB of shared
// memory and 256 TMEM columns each) walk the items with a fixed stride; 192 threads: warps 0-3 softmax (thread
// = query row = TMEM lane), warp 4 TMA producer, warp 5 MMA issuer + TMEM owner.  Per 64-key tile:
//     S = Q K^T        tcgen05.mma, A = Q and B = K both K-major in shared memory, fp32 into one of two 64-column
//                      TMEM buffers: S of tile t+1 (and t+2's keys) are ready before the softmax of tile t ends;
//     softmax          each thread loads its 64 scores once with tcgen05.ld, takes the maximum, and writes P as
//                      packed bf16 over the columns it has consumed (tcgen05.st); it then goes straight on to the
//                      next tile's S without waiting for the tensor pipe;
//     O += P V         tcgen05.mma with A = P read from TMEM and B = V as an MN-major shared-memory operand (V's
//                      rows are keys, the reduction axis, so the tile TMA delivers IS the MN-major image); O
//                      stays in TMEM columns 128..255 for the whole row block.  MMAs of one thread run in order,
//                      so S of tile t+2 overwrites the buffer of P(t) only after PV(t) has read it.
// The running maximum a row's exponentials refer to is only advanced when the true maximum has moved by more
// than 2^8 (then the warp waits for the PV in flight and rescales its rows of O in TMEM and its sums); the final
// division uses the same reference, so the result is exact while almost every tile skips the rescale.
// Causality: a 32-key chunk is fully visible, cut by the diagonal, or hidden for a whole warp (32 rows), decided
// from the chunk's offset to the warp's rows; keys past the document's end are rows of the next document (or TMA's
// zero fill) and sit above the diagonal of every valid row.  K and V are double buffered.  The next item's queries
// are loaded once the current item's last S has been issued.  Every mbarrier wait is bounded; on expiry the CTA
// raises status[0], drains and frees TMEM.
//
// Three uses of one kernel (template flags): documents (segments listed by token index, consecutive tokens);
// documents with tokens inside them that do not take part (MASKED: a segment is the span of memory from the first to
// the last participating token, a bitmap says which positions count; a 32-key chunk with a hole gets -inf scores
// there and then runs the code of a full chunk; rows of the other tokens are not written); and context mode (CTX:
// segment = sequence, queries = its run of valid tokens, keys = its entries in the compact K / V store, key j visible
// to query row i iff j <= i + kv_len - n_q and j < kv_len, or every key when not causal; the item of the last row
// block zero-fills the rows of the tokens that are not queries).
//
// Bounds per 64-key tile and CTA, measured with a kernel that only issues the instructions: an S MMA (128x64x16, both
// operands in shared memory) takes 48 cycles, not the 32 of its math, because it reads 6 KB of operands at 128 B per
// clock; the same with N = 128 takes 64 and with N = 256 128 cycles (the only shape at the nominal rate); a PV MMA
// (128x128x16, P from TMEM, V MN-major) takes 64; one tile as issued here (8 S + 4 PV) takes 619 cycles, whatever the
// number of issuing warps.  The pipe is shared, in order, by the two CTAs of the SM.  The exponentials take 512
// cycles of the SFU per warp and tile (1,024 with two CTAs).  Per-tile timestamps show 2,040 cycles per tile and CTA
// inside long items: the MMA-issuing thread is blocked in its 12 instructions behind the other CTA's for 1,440 of
// them and waits for P for 600; an item boundary costs about 5,000 cycles from the last P to the next item's first
// S.  Over a whole launch on 512-token documents the pipe is busy 38 % of the time.  Measured and dropped: S for pairs
// of key tiles with N = 128 (fewer pipe cycles, but both S buffers must be free at once and the softmax then waits
// after every second tile), reading an item's output out under the next item's first softmax, an L2 prefetch of the
// next item's queries.  Wider tiles with two query tiles per CTA in ping-pong need all 512 TMEM columns (one CTA per SM).
#include <cuda.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace msa {

constexpr int kAtRows = 128, kAtKeys = 64, kAtD = 128;
constexpr int kAtThreads = 192;
constexpr int kAtBlk = kAtRows * 64 * 2;                 // one 64-column block of the 128-row query tile: 16 KB
constexpr int kAtTile = 2 * kAtBlk;                      // the [128 x 128] bf16 query tile
constexpr int kAtKvBlk = kAtKeys * 64 * 2;               // one 64-column block of a 64-key K or V tile: 8 KB
constexpr int kAtKvTile = 2 * kAtKvBlk;                  // a [64 x 128] bf16 K or V tile
constexpr int kAtOutStage = 32 * 64;                     // per softmax warp: 32 rows x 32 bf16 columns of output on their way out
constexpr int kAtSmem = kAtTile + 4 * kAtKvTile + 4 * kAtOutStage + 1024;  // Q, 2 x (K, V), output staging
constexpr uint32_t kColS = 0, kColO = 128, kAtTmemCols = 256;   // TMEM columns: S0 0..63, S1 64..127 (P over them), O 128..255
constexpr float kRescaleStep = 8.f;                      // log2 units the row maximum may run ahead of its reference

struct DocAttnTcParams {
  const int32_t* token_index;   // flat position of every listed token; a segment's tokens are consecutive
  const int32_t* seg_off;
  // context mode (q_tok != nullptr): segment = sequence b; its queries are the run of num_q[b] tokens that starts at
  // token q_tok[b * S], its keys the kv_len[b] positions from kv_start[b] on of (b, head) in the K / V stores
  const int32_t* q_tok;
  const int32_t* num_q;
  const int32_t* kv_start;
  const int32_t* kv_len;
  int causal;                   // context mode: bottom-right aligned causal mask, or every key visible
  // masked documents: bit (flat token position) = the token belongs to its document; a segment then lists EVERY
  // position from its first to its last such token, and the others are neither attended to nor written
  const uint32_t* valid_bits;
  int S, n_q_heads, n_kv_heads;
  int q_yb, q_yh, q_xh;         // q tile coordinates: y = b*q_yb + h*q_yh + s, x = h*q_xh + 64*block
  int k_yb, k_yh, k_xh;
  uint32_t div_mul, div_shift;  // tok / S
  float scale_log2e;
  int max_mb;                   // row blocks of the longest segment
  long long n_sh;               // n_segments * n_q_heads
  long long n_items;            // n_sh * max_mb
  __nv_bfloat16* out;
  int32_t* status;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tcgen05.mma with the A operand in tensor memory.
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// MN-major operand tile in shared memory, SWIZZLE_128B: rows are indices of the reduction axis (keys), each
// row holds 64 consecutive MN elements (128 bytes); 8 rows form a 1024-byte swizzle atom (stride byte offset
// = distance between 8-row groups); the next 64 MN elements are a separate block (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Packed and three-input arithmetic of sm_100: the softmax threads are bound by the number of instructions they issue
// (one thread per row, one or two warps per scheduler), so two elements per FFMA / FADD and two per maximum count.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ unsigned long long f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f32x2_split(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One work item = (document, head, row block).  Items are numbered w = x * (n_segments * n_q_heads) + seg *
// n_q_heads + hq with x counting a document's row blocks from its last (longest) one: the fixed-stride walk
// of the persistent CTAs then hands every CTA the same mix of long and short items, and the heads of a kv
// group run side by side and share K / V through L2.  Item w of a document with fewer row blocks is skipped.
// A query row i of the segment sees key j iff j <= i + shift and j < n_keys.  Documents: shift 0, and keys past the
// document's end sit above the diagonal of every valid row, so n_keys is left unbounded there.
struct AtItem { int len, r0, n_kt, hq, hk, tok0, b, s0, k_s0, shift, n_keys, x; bool valid; };
constexpr int kAtUnbounded = 1 << 29;
template <bool CTX>
__device__ __forceinline__ AtItem at_item(const DocAttnTcParams& p, long long w) {
  AtItem it;
  it.x = (int)(w / p.n_sh);
  const long long sh = w % p.n_sh;
  it.hq = (int)(sh % p.n_q_heads);
  const int seg = (int)(sh / p.n_q_heads);
  it.hk = it.hq / (p.n_q_heads / p.n_kv_heads);
  if constexpr (CTX) {
    it.len = p.num_q[seg];
    const int n_mb = (it.len + kAtRows - 1) / kAtRows;
    it.valid = it.x < n_mb;
    const int mb = n_mb - 1 - it.x;
    it.r0 = mb * kAtRows;
    it.b = seg;
    it.s0 = it.len > 0 ? p.q_tok[(long long)seg * p.S] : 0;
    it.tok0 = seg * p.S + it.s0;
    it.k_s0 = p.kv_start[seg];
    it.n_keys = p.kv_len[seg];
    it.shift = p.causal ? it.n_keys - it.len : kAtUnbounded;
    const long long reach = (long long)it.r0 + kAtRows + it.shift;
    it.n_kt = (int)(((reach < it.n_keys ? reach : (long long)it.n_keys) + kAtKeys - 1) / kAtKeys);
    it.valid = it.valid && it.n_keys > 0 && it.k_s0 >= 0 && it.shift >= 0;
    return it;
  }
  const int t0 = p.seg_off[seg];
  it.len = p.seg_off[seg + 1] - t0;
  const int n_mb = (it.len + kAtRows - 1) / kAtRows;
  it.valid = it.x < n_mb;
  const int mb = n_mb - 1 - it.x;
  it.r0 = mb * kAtRows;
  it.n_kt = 2 * (mb + 1);              // 64-key tiles up to the end of the row block
  it.tok0 = it.valid ? p.token_index[t0] : 0;
  it.b = (int)((__umulhi((uint32_t)it.tok0, p.div_mul) + (uint32_t)it.tok0) >> p.div_shift);
  it.s0 = it.tok0 - it.b * p.S;
  it.k_s0 = it.s0;
  it.shift = 0;
  it.n_keys = kAtUnbounded;
  return it;
}

// Context mode: the rows [lo, hi) of sequence b get zeros in head hq's columns (tokens that are not queries).
__device__ __forceinline__ void at_zero_rows(const DocAttnTcParams& p, int b, int hq, int lo, int hi, int tid) {
  const long long row_stride = (long long)p.n_q_heads * kAtD;
  __nv_bfloat16* base = p.out + (long long)b * p.S * row_stride + (long long)hq * kAtD;
  for (int idx = tid; idx < (hi - lo) * 16; idx += 128)
    *reinterpret_cast<uint4*>(base + (long long)(lo + (idx >> 4)) * row_stride + 8 * (idx & 15)) = make_uint4(0u, 0u, 0u, 0u);
}

// 32 bits of a bitmap from bit position pos on (the bitmap is padded so that the word after the last one exists).
__device__ __forceinline__ uint32_t at_bits(const uint32_t* __restrict__ words, long long pos) {
  const long long w = pos >> 5;
  return __funnelshift_r(__ldg(words + w), __ldg(words + w + 1), (uint32_t)(pos & 31));
}
// The keys 0..lim of a 32-key chunk as a bit mask.
__device__ __forceinline__ uint32_t at_upto(int lim) {
  return lim >= 31 ? 0xffffffffu : (lim < 0 ? 0u : ((2u << lim) - 1u));
}

// CTX = false: documents (segments listed by token_index / seg_off); true: context mode.  MASKED (documents only):
// segments are spans of memory with tokens that do not take part (valid_bits).
template <bool CTX, bool MASKED>
__global__ void __launch_bounds__(kAtThreads, 2)
doc_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const DocAttnTcParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ uint64_t s_q_full, s_q_empty, s_k_full[2], s_k_empty[2], s_v_full[2], s_v_empty[2], s_s_full[2], s_p_full[2],
      s_o_full[2], s_drain;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = tiles;
  unsigned char* kv_smem = tiles + kAtTile;      // stage s: K at s * 2 * kAtKvTile, V right after it
  unsigned char* out_stage = kv_smem + 4 * kAtKvTile;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    mbar_init(&s_q_full, 1); mbar_init(&s_q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_k_full[i], 1); mbar_init(&s_k_empty[i], 1);
      mbar_init(&s_v_full[i], 1); mbar_init(&s_v_empty[i], 1);
      mbar_init(&s_s_full[i], 1);
      mbar_init(&s_p_full[i], 4);
      mbar_init(&s_o_full[i], 1);
    }
    mbar_init(&s_drain, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(kAtTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  // Every role walks the same items in the same order.  n_it counts the valid items and n_t the key tiles this
  // CTA has gone through; tile n_t uses stage / S buffer / barrier set n_t & 1 for the (n_t >> 1)-th time, and
  // every barrier's phase follows from those counters.  The softmax may be up to two tiles ahead of the PVs, which
  // is why P-ready and O-ready also come in pairs: within one barrier a waiter is never more than one phase behind.
  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------------
    if (lane == 0) {
      uint32_t n_it = 0, n_t = 0;
      bool ok = true;
      for (long long w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
        const AtItem it = at_item<CTX>(p, w);
        if (!it.valid) continue;
        const int qy = it.b * p.q_yb + it.hq * p.q_yh + it.s0 + it.r0, qx = it.hq * p.q_xh;
        const int ky = it.b * p.k_yb + it.hk * p.k_yh + it.k_s0, kx = it.hk * p.k_xh;
        // the query buffer is free once the previous item's last S has completed
        if (!(ok = mbar_wait(&s_q_empty, (n_it & 1u) ^ 1u, abort_flag, p.status, 1))) break;
        mbar_expect_tx(&s_q_full, kAtTile);
        tma_load_2d(q_smem, &tmap_q, qx, qy, &s_q_full);
        tma_load_2d(q_smem + kAtBlk, &tmap_q, qx + 64, qy, &s_q_full);
        for (int t = 0; t < it.n_kt; ++t, ++n_t) {
          const uint32_t st = n_t & 1u, ph = (n_t >> 1) & 1u;
          unsigned char* ks = kv_smem + (size_t)st * 2 * kAtKvTile;
          if (!(ok = mbar_wait(&s_k_empty[st], ph ^ 1u, abort_flag, p.status, 1))) break;
          mbar_expect_tx(&s_k_full[st], kAtKvTile);
          tma_load_2d(ks, &tmap_k, kx, ky + t * kAtKeys, &s_k_full[st]);
          tma_load_2d(ks + kAtKvBlk, &tmap_k, kx + 64, ky + t * kAtKeys, &s_k_full[st]);
          if (!(ok = mbar_wait(&s_v_empty[st], ph ^ 1u, abort_flag, p.status, 1))) break;
          mbar_expect_tx(&s_v_full[st], kAtKvTile);
          tma_load_2d(ks + kAtKvTile, &tmap_v, kx, ky + t * kAtKeys, &s_v_full[st]);
          tma_load_2d(ks + kAtKvTile + kAtKvBlk, &tmap_v, kx + 64, ky + t * kAtKeys, &s_v_full[st]);
        }
        ++n_it;
      }
      if (!ok) {   // gave up: give the copies already issued time to land before shared memory is released
        const unsigned long long w0 = global_ns();
        while (global_ns() - w0 < 1000000ull) {}   // 1 ms, far above any copy's latency
      }
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer ----------------------------------------
    if (lane == 0) {
      // D = f32, A = B = bf16, M = 128; S: N = 64 keys, both operands K-major; PV: N = 128, B (= V) MN-major
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kAtKeys >> 3) << 17) |
                               ((uint32_t)(kAtRows >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kAtD >> 3) << 17) |
                                ((uint32_t)(kAtRows >> 4) << 24);
      const uint32_t qa = smem_u32(q_smem), kva = smem_u32(kv_smem);
      uint32_t n_it = 0, n_t = 0;     // n_t: tiles whose PV has been issued
      bool ok = true;
      // S of tile g (global count) of the current item; `last` = the item's last tile
      auto issue_s = [&](uint32_t g, bool last) -> bool {
        const uint32_t st = g & 1u, ph = (g >> 1) & 1u;
        if (!mbar_wait(&s_k_full[st], ph, abort_flag, p.status, 3)) return false;
        tc_fence_after();
        const uint32_t ka = kva + st * 2 * kAtKvTile;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t a_desc = make_smem_desc(qa + kb * kAtBlk), b_desc = make_smem_desc(ka + kb * kAtKvBlk);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_bf16(tmem_base + kColS + st * kAtKeys, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc_s,
                        (kb > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&s_s_full[st]);
        tc_commit(&s_k_empty[st]);
        if (last) tc_commit(&s_q_empty);   // the next item's queries may land under this item's tail
        return true;
      };
      for (long long w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
        const AtItem it = at_item<CTX>(p, w);
        if (!it.valid) continue;
        if (!(ok = mbar_wait(&s_q_full, n_it & 1u, abort_flag, p.status, 2))) break;
        // two S tiles run ahead of the softmax (n_kt is even: a row block spans whole pairs of key tiles)
        if (!(ok = issue_s(n_t, it.n_kt == 1))) break;
        if (it.n_kt > 1 && !(ok = issue_s(n_t + 1, it.n_kt == 2))) break;
        for (int t = 0; t < it.n_kt; ++t, ++n_t) {
          const uint32_t st = n_t & 1u, ph = (n_t >> 1) & 1u;
          if (!(ok = mbar_wait(&s_v_full[st], ph, abort_flag, p.status, 3))) break;
          if (!(ok = mbar_wait(&s_p_full[st], ph, abort_flag, p.status, 4))) break;
          tc_fence_after();
          const uint32_t va = kva + st * 2 * kAtKvTile + kAtKvTile;
#pragma unroll
          for (int j = 0; j < kAtKeys / 16; ++j)   // 16 keys per step: 8 TMEM columns of P, two 8-key groups of V
            tc_mma_bf16_ts(tmem_base + kColO, tmem_base + kColS + st * kAtKeys + (uint32_t)(8 * j),
                           make_smem_desc_mn(va + j * 2048, kAtKvBlk), idesc_pv, (t > 0 || j > 0) ? 1u : 0u);
          tc_commit(&s_o_full[st]);
          tc_commit(&s_v_empty[st]);
          // S of tile t+2 reuses this tile's buffer: in order after the PV that read P from it
          if (t + 2 < it.n_kt && !(ok = issue_s(n_t + 2, t + 3 == it.n_kt))) break;
        }
        ++n_it;
      }
      tc_commit(&s_drain);   // everything issued so far must retire before TMEM is freed
      const unsigned long long w0 = global_ns();
      while (!mbar_try_wait(&s_drain, 0) && global_ns() - w0 < kWaitLimitNs) {}
    }
  } else {
    // ------------------------------- softmax / output (warps 0-3) ----------------------
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    uint32_t n_t = 0;
    bool ok = true;
    for (long long w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
      const AtItem it = at_item<CTX>(p, w);
      if (!it.valid) {
        if (CTX && it.x == 0) at_zero_rows(p, it.b, it.hq, 0, p.S, threadIdx.x);   // no query at all
        continue;
      }
      float m_ref = -INFINITY, l_run = 0.f;                // m_ref: the maximum the exponentials refer to
      for (int t = 0; t < it.n_kt; ++t, ++n_t) {
        const uint32_t st = n_t & 1u;
        uint32_t km0 = 0xffffffffu, km1 = 0xffffffffu;       // MASKED: which keys of the tile's two chunks take part
        if constexpr (MASKED) {                               // fetched while the tile's S is still on its way
          const long long kpos = (long long)it.tok0 + (long long)t * kAtKeys;
          km0 = at_bits(p.valid_bits, kpos);
          km1 = at_bits(p.valid_bits, kpos + 32);
        }
        ok = mbar_wait(&s_s_full[st], (n_t >> 1) & 1u, abort_flag, p.status, 5);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = lane_base + kColS + st * kAtKeys;
        // Visibility of the two 32-key chunks for this warp's 32 rows.  Key i of a chunk is visible to a lane iff
        // i <= lim = min(lane + d, ke), d = (first row of the warp) + shift - (first key of the chunk), ke = (last
        // key of the segment) - (first key of the chunk).  A chunk is fully visible (class 2: d >= 31 and ke >= 31),
        // hidden from the whole warp (class 0: d <= -32 or ke < 0) or cut (class 1).  For documents d is a multiple of
        // 32 and ke unbounded: the classes are d >= 32, d == 0 (lim = lane) and d < 0.
        int cls0, cls1, lim0, lim1;
        if constexpr (CTX) {
          const int d0 = it.r0 + warp * 32 + it.shift - t * kAtKeys, d1 = d0 - 32;
          const int ke0 = it.n_keys - 1 - t * kAtKeys, ke1 = ke0 - 32;
          cls0 = (d0 >= 31 && ke0 >= 31) ? 2 : ((d0 <= -32 || ke0 < 0) ? 0 : 1);
          cls1 = (d1 >= 31 && ke1 >= 31) ? 2 : ((d1 <= -32 || ke1 < 0) ? 0 : 1);
          lim0 = min(lane + d0, ke0);
          lim1 = min(lane + d1, ke1);
        } else {
          const int d0 = it.r0 + warp * 32 - t * kAtKeys, d1 = d0 - 32;
          cls0 = d0 >= 32 ? 2 : (d0 == 0 ? 1 : 0);
          cls1 = d1 >= 32 ? 2 : (d1 == 0 ? 1 : 0);
          lim0 = lim1 = lane;
        }
        uint32_t vis0 = 0xffffffffu, vis1 = 0xffffffffu;      // MASKED: the keys this lane's row sees, chunk by chunk
        if constexpr (MASKED) {
          vis0 = km0 & (cls0 == 2 ? 0xffffffffu : (cls0 == 1 ? at_upto(lim0) : 0u));
          vis1 = km1 & (cls1 == 2 ? 0xffffffffu : (cls1 == 1 ? at_upto(lim1) : 0u));
          // a chunk with a hole is handled like a cut one; a chunk without a visible key for the whole warp is hidden
          if (cls0 == 2 && km0 != 0xffffffffu) cls0 = 1;
          if (cls1 == 2 && km1 != 0xffffffffu) cls1 = 1;
          if (km0 == 0u) cls0 = 0;
          if (km1 == 0u) cls1 = 0;
        }
        uint32_t va[32], vb[32];
        tmem_ld32(s_addr, va);
        tmem_ld32(s_addr + 32, vb);
        tmem_ld_wait();
        if constexpr (MASKED) {
          // a chunk with hidden keys: their scores become -inf once (their exponentials are then zero by themselves)
          // and the chunk goes through the code of a fully visible one
          if (cls0 == 1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (!((vis0 >> i) & 1u)) va[i] = 0xff800000u;
            cls0 = 2;
          }
          if (cls1 == 1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (!((vis1 >> i) & 1u)) vb[i] = 0xff800000u;
            cls1 = 2;
          }
        }
        // row maximum: two elements per instruction, two independent chains per chunk
        float mx = -INFINITY, mx2 = -INFINITY;
        if (cls0 == 2) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx = max3(mx, __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
            mx2 = max3(mx2, __uint_as_float(va[i + 2]), __uint_as_float(va[i + 3]));
          }
        } else if (cls0 == 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            mx = fmaxf(mx, (MASKED ? (vis0 >> i) & 1u : (uint32_t)(i <= lim0)) ? __uint_as_float(va[i]) : -INFINITY);
            mx2 = fmaxf(mx2, (MASKED ? (vis0 >> (i + 1)) & 1u : (uint32_t)(i + 1 <= lim0)) ? __uint_as_float(va[i + 1]) : -INFINITY);
          }
        }
        if (cls1 == 2) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx = max3(mx, __uint_as_float(vb[i]), __uint_as_float(vb[i + 1]));
            mx2 = max3(mx2, __uint_as_float(vb[i + 2]), __uint_as_float(vb[i + 3]));
          }
        } else if (cls1 == 1) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            mx = fmaxf(mx, (MASKED ? (vis1 >> i) & 1u : (uint32_t)(i <= lim1)) ? __uint_as_float(vb[i]) : -INFINITY);
            mx2 = fmaxf(mx2, (MASKED ? (vis1 >> (i + 1)) & 1u : (uint32_t)(i + 1 <= lim1)) ? __uint_as_float(vb[i + 1]) : -INFINITY);
          }
        }
        mx = fmaxf(mx, mx2);
        // advance the reference only when the maximum ran ahead by more than the step (always on the first tile;
        // never on a tile this warp does not see at all, where mx is -inf)
        const bool move = (mx - m_ref) * p.scale_log2e > kRescaleStep;
        if (__any_sync(0xffffffffu, move)) {
          if (t > 0) {   // wait for the PV in flight, then rescale this warp's rows of O in place
            ok = mbar_wait(&s_o_full[(n_t - 1u) & 1u], ((n_t - 1u) >> 1) & 1u, abort_flag, p.status, 6);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const float f = move ? exp2f((m_ref - mx) * p.scale_log2e) : 1.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint32_t v[16];
              tmem_ld16(lane_base + kColO + 16 * c, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
              tmem_st16(lane_base + kColO + 16 * c, v);
            }
            l_run *= f;
          }
          if (move) m_ref = mx;
        }
        const float neg_m = -m_ref * p.scale_log2e;
        // exponentials, row sum, P as packed bf16 over the consumed columns of this buffer
        unsigned long long sum_a = 0ull, sum_b = 0ull;       // two packed accumulators = four partial row sums
        const unsigned long long scale2 = f32x2(p.scale_log2e, p.scale_log2e), neg_m2 = f32x2(neg_m, neg_m);
        uint32_t pk[16];
        auto exps = [&](const uint32_t (&v)[32], int cls, int lim, uint32_t vis) {
          if (cls == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = 0u;
            return;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float x0, x1, x2, x3;
            f32x2_split(fma_f32x2(f32x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), scale2, neg_m2), x0, x1);
            f32x2_split(fma_f32x2(f32x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), scale2, neg_m2), x2, x3);
            float e0 = ex2_approx(x0), e1 = ex2_approx(x1), e2 = ex2_approx(x2), e3 = ex2_approx(x3);
            if (cls == 1) {                                    // a cut chunk: key i is visible iff i <= lim
              if constexpr (MASKED) {                          // ... and the token takes part
                if (!((vis >> i) & 1u)) e0 = 0.f;
                if (!((vis >> (i + 1)) & 1u)) e1 = 0.f;
                if (!((vis >> (i + 2)) & 1u)) e2 = 0.f;
                if (!((vis >> (i + 3)) & 1u)) e3 = 0.f;
              } else {
                if (i > lim) e0 = 0.f;
                if (i + 1 > lim) e1 = 0.f;
                if (i + 2 > lim) e2 = 0.f;
                if (i + 3 > lim) e3 = 0.f;
              }
            }
            sum_a = add_f32x2(sum_a, f32x2(e0, e1));
            sum_b = add_f32x2(sum_b, f32x2(e2, e3));
            pk[i >> 1] = pack2_bf16(e0, e1);
            pk[(i >> 1) + 1] = pack2_bf16(e2, e3);
          }
        };
        exps(va, cls0, lim0, vis0);
        tmem_st16(s_addr, pk);
        exps(vb, cls1, lim1, vis1);
        tmem_st16(s_addr + 16, pk);
        {
          float s0, s1, s2, s3;
          f32x2_split(sum_a, s0, s1);
          f32x2_split(sum_b, s2, s3);
          l_run += (s0 + s1) + (s2 + s3);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_p_full[st]);
      }
      if (!ok) break;
      // the item's output: O is complete after the last PV
      ok = mbar_wait(&s_o_full[(n_t - 1u) & 1u], ((n_t - 1u) >> 1) & 1u, abort_flag, p.status, 6);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float inv = 1.f / l_run;
      // A thread holds one row, and rows are 8 KB apart in the output: stored straight from the registers, every
      // store instruction touched 32 lines (measured: 5,600 cycles per item).  The warp's 32 x 32 block of a
      // column group goes through shared memory instead (16-byte pieces, XOR-swizzled so that both sides are free of
      // bank conflicts) and leaves with four lanes per row: 8 rows x 64 contiguous bytes per instruction.
      unsigned char* stg = out_stage + warp * kAtOutStage;
      const long long row_stride = (long long)p.n_q_heads * kAtD;
      __nv_bfloat16* dst0 = p.out + ((long long)it.tok0 + it.r0 + warp * 32) * row_stride + (long long)it.hq * kAtD;
      uint32_t row_bits = 0xffffffffu;    // MASKED: which of the warp's 32 rows are tokens of the document
      if constexpr (MASKED) row_bits = at_bits(p.valid_bits, (long long)it.tok0 + it.r0 + warp * 32);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + kColO + 32 * c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o;
          o.x = pack2_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
          o.y = pack2_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
          o.z = pack2_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
          o.w = pack2_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
          *reinterpret_cast<uint4*>(stg + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4)) = o;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = (lane >> 2) + 8 * i, piece = lane & 3;
          const uint4 o = *reinterpret_cast<const uint4*>(stg + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4));
          if (it.r0 + warp * 32 + r < it.len && ((row_bits >> r) & 1u))
            *reinterpret_cast<uint4*>(dst0 + (long long)r * row_stride + 32 * c + 8 * piece) = o;
        }
        __syncwarp();   // the staging block is rewritten by the next column group
      }
      if (CTX && it.x == 0) {   // the item of the last row block also clears the rows around the run
        at_zero_rows(p, it.b, it.hq, 0, it.s0, threadIdx.x);
        at_zero_rows(p, it.b, it.hq, it.s0 + it.len, p.S, threadIdx.x);
      }
      tc_fence_before();   // the next item's first PV (gated by this warp's next arrival) overwrites O
    }
  }

  // teardown: all roles meet, then the allocating warp returns TMEM
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 5)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAtTmemCols) : "memory");
}

}  // namespace msa

using namespace msa;

namespace {
// A [B, H, S, D] tensor given by strides as a 2-D tensor map with one row per token.
// Token major (projection output, heads side by side in a row): rows B*S, columns H*D.
// Head major (contiguous [B, H, S, D]): rows B*H*S, columns D.
struct View2D { uint64_t rows, cols, row_stride; int yb, yh, xh; bool ok; };
View2D view_2d(int64_t sb, int64_t sh, int64_t ss, int B, int H, int S, int D) {
  View2D v{};
  if (sh == D && ss >= (int64_t)H * D && (B == 1 || sb == (int64_t)S * ss)) {
    v = View2D{(uint64_t)B * S, (uint64_t)H * D, (uint64_t)ss, S, 0, D, true};
  } else if (ss >= D && sh == (int64_t)S * ss && (B == 1 || sb == (int64_t)H * sh)) {
    v = View2D{(uint64_t)B * H * S, (uint64_t)D, (uint64_t)ss, H * S, S, 0, true};
  }
  return v;
}
}  // namespace

namespace {
template <bool CTX, bool MASKED>
int launch_doc_attn_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, DocAttnTcParams& p,
                       int n_segments, int max_rows, cudaStream_t stream) {
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(doc_attn_tc_kernel<CTX, MASKED>, kAtSmem, configured));
  p.max_mb = (max_rows + kAtRows - 1) / kAtRows;
  p.n_sh = (long long)n_segments * p.n_q_heads;
  p.n_items = p.n_sh * p.max_mb;
  int n_sm = 0;
  MSA_OK_OR_RETURN(device_sm_count(&n_sm));
  const long long grid = p.n_items < 2ll * n_sm ? p.n_items : 2ll * n_sm;   // persistent: two CTAs per SM
  doc_attn_tc_kernel<CTX, MASKED><<<(unsigned)grid, kAtThreads, kAtSmem, stream>>>(map_q, map_k, map_v, p);
  MSA_LAUNCH_OK("doc_attn_tc_kernel");
  return MSA_OK;
}
void set_token_division(DocAttnTcParams& p, int seq_len) {
  uint32_t shift = 0;
  while ((1ull << shift) < (uint64_t)seq_len) ++shift;
  p.div_shift = shift;
  p.div_mul = (uint32_t)((((1ull << shift) - (uint64_t)seq_len) << 32) / (uint64_t)seq_len + 1);
}
}  // namespace

namespace {
int doc_attention_tc_impl(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, const void* k,
                          const void* v, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                          const int32_t* token_index, const int32_t* seg_offsets, int32_t n_segments,
                          int32_t max_segment_len, int32_t n_seq, int32_t seq_len, int32_t n_q_heads, int32_t n_kv_heads,
                          int32_t head_dim, int32_t dtype, float scale, void* out, const uint32_t* valid_bits,
                          int32_t* status, void* stream) {
  MSA_REQUIRE(q && k && v && token_index && seg_offsets && out && status, "doc_attention_tc: null pointer");
  MSA_REQUIRE(dtype == MSA_BF16 && head_dim == kAtD, "doc_attention_tc: bf16 with head_dim 128 only");
  MSA_REQUIRE(n_segments >= 0 && max_segment_len >= 0 && n_seq > 0 && seq_len > 0 && n_q_heads > 0 &&
                  n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "doc_attention_tc: bad sizes");
  MSA_REQUIRE((long long)n_seq * seq_len * n_q_heads < (1ll << 31), "doc_attention_tc: more than 2^31 token rows");
  MSA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && q_stride_s % 8 == 0 &&
                  k_stride_s % 8 == 0, "doc_attention_tc: rows must be 16-byte aligned");
  const View2D vq = view_2d(q_stride_b, q_stride_h, q_stride_s, n_seq, n_q_heads, seq_len, head_dim);
  const View2D vk = view_2d(k_stride_b, k_stride_h, k_stride_s, n_seq, n_kv_heads, seq_len, head_dim);
  MSA_REQUIRE(vq.ok && vk.ok, "doc_attention_tc: q / k / v must be token-major or contiguous head-major tensors");
  if (n_segments == 0 || max_segment_len == 0) return MSA_OK;

  CUtensorMap map_q, map_k, map_v;
  int rc = make_map(&map_q, q, vq.rows, vq.cols, vq.row_stride, 64, kAtRows);
  if (rc != MSA_OK) return rc;
  rc = make_map(&map_k, k, vk.rows, vk.cols, vk.row_stride, 64, kAtKeys);
  if (rc != MSA_OK) return rc;
  rc = make_map(&map_v, v, vk.rows, vk.cols, vk.row_stride, 64, kAtKeys);
  if (rc != MSA_OK) return rc;

  DocAttnTcParams p{};
  p.token_index = token_index; p.seg_off = seg_offsets; p.S = seq_len; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.q_yb = vq.yb; p.q_yh = vq.yh; p.q_xh = vq.xh; p.k_yb = vk.yb; p.k_yh = vk.yh; p.k_xh = vk.xh;
  set_token_division(p, seq_len);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  p.valid_bits = valid_bits;
  if (valid_bits != nullptr)
    return launch_doc_attn_tc<false, true>(map_q, map_k, map_v, p, n_segments, max_segment_len, (cudaStream_t)stream);
  return launch_doc_attn_tc<false, false>(map_q, map_k, map_v, p, n_segments, max_segment_len, (cudaStream_t)stream);
}
}  // namespace

extern "C" int msa_doc_attention_tc(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                    const void* k, const void* v, int64_t k_stride_b, int64_t k_stride_h,
                                    int64_t k_stride_s, const int32_t* token_index, const int32_t* seg_offsets,
                                    int32_t n_segments, int32_t max_segment_len, int32_t n_seq, int32_t seq_len,
                                    int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype, float scale,
                                    void* out, int32_t* status, void* stream) {
  return doc_attention_tc_impl(q, q_stride_b, q_stride_h, q_stride_s, k, v, k_stride_b, k_stride_h, k_stride_s, token_index,
                               seg_offsets, n_segments, max_segment_len, n_seq, seq_len, n_q_heads, n_kv_heads, head_dim,
                               dtype, scale, out, nullptr, status, stream);
}

extern "C" int msa_doc_attention_tc_masked(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                           const void* k, const void* v, int64_t k_stride_b, int64_t k_stride_h,
                                           int64_t k_stride_s, const int32_t* span_index, const int32_t* span_offsets,
                                           int32_t n_segments, int32_t max_span_len, int32_t n_seq, int32_t seq_len,
                                           int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                                           float scale, void* out, const uint32_t* valid_bits, int64_t n_bit_words,
                                           int32_t* status, void* stream) {
  MSA_REQUIRE(valid_bits != nullptr, "doc_attention_tc_masked: null pointer");
  // the kernel reads bits up to 256 positions past the last token and the word after the one that holds a position
  MSA_REQUIRE(n_seq > 0 && seq_len > 0 && n_bit_words >= ((int64_t)n_seq * seq_len + 256 + 31) / 32 + 1,
              "doc_attention_tc_masked: the bitmap must cover every token plus 256 positions and one more word");
  return doc_attention_tc_impl(q, q_stride_b, q_stride_h, q_stride_s, k, v, k_stride_b, k_stride_h, k_stride_s, span_index,
                               span_offsets, n_segments, max_span_len, n_seq, seq_len, n_q_heads, n_kv_heads, head_dim,
                               dtype, scale, out, valid_bits, status, stream);
}

extern "C" int msa_sparse_prefill_attn_tc(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                          const void* k_store, const void* v_store, int64_t store_stride_b,
                                          int64_t store_stride_h, int32_t store_len, const int32_t* kv_start,
                                          const int32_t* kv_len, const int32_t* q_tok, const int32_t* num_q, int32_t n_seq,
                                          int32_t seq_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                          int32_t dtype, int32_t causal, float scale, void* out, int32_t* status,
                                          void* stream) {
  MSA_REQUIRE(q && k_store && v_store && kv_start && kv_len && q_tok && num_q && out && status,
              "sparse_prefill_attn_tc: null pointer");
  MSA_REQUIRE(dtype == MSA_BF16 && head_dim == kAtD, "sparse_prefill_attn_tc: bf16 with head_dim 128 only");
  MSA_REQUIRE(n_seq > 0 && seq_len > 0 && store_len > 0 && n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
              "sparse_prefill_attn_tc: bad sizes");
  MSA_REQUIRE((long long)n_seq * seq_len * n_q_heads < (1ll << 31) && (long long)n_seq * store_len * n_kv_heads < (1ll << 31),
              "sparse_prefill_attn_tc: more than 2^31 token rows");
  MSA_REQUIRE(aligned16(q) && aligned16(k_store) && aligned16(v_store) && aligned16(out) && q_stride_s % 8 == 0,
              "sparse_prefill_attn_tc: rows must be 16-byte aligned");
  const View2D vq = view_2d(q_stride_b, q_stride_h, q_stride_s, n_seq, n_q_heads, seq_len, head_dim);
  const View2D vk = view_2d(store_stride_b, store_stride_h, head_dim, n_seq, n_kv_heads, store_len, head_dim);
  MSA_REQUIRE(vq.ok, "sparse_prefill_attn_tc: q must be a token-major or contiguous head-major tensor");
  MSA_REQUIRE(vk.ok, "sparse_prefill_attn_tc: the stores must be contiguous [B, Hkv, store_len, D] tensors");

  CUtensorMap map_q, map_k, map_v;
  int rc = make_map(&map_q, q, vq.rows, vq.cols, vq.row_stride, 64, kAtRows);
  if (rc != MSA_OK) return rc;
  rc = make_map(&map_k, k_store, vk.rows, vk.cols, vk.row_stride, 64, kAtKeys);
  if (rc != MSA_OK) return rc;
  rc = make_map(&map_v, v_store, vk.rows, vk.cols, vk.row_stride, 64, kAtKeys);
  if (rc != MSA_OK) return rc;

  DocAttnTcParams p{};
  p.q_tok = q_tok; p.num_q = num_q; p.kv_start = kv_start; p.kv_len = kv_len; p.causal = causal != 0;
  p.S = seq_len; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.q_yb = vq.yb; p.q_yh = vq.yh; p.q_xh = vq.xh; p.k_yb = vk.yb; p.k_yh = vk.yh; p.k_xh = vk.xh;
  set_token_division(p, seq_len);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  return launch_doc_attn_tc<true, false>(map_q, map_k, map_v, p, n_seq, seq_len, (cudaStream_t)stream);
}
