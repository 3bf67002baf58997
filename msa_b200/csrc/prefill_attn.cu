// Stage-2 sparse prefill: context assembly and causal attention over [template | retrieved | query].
//
// assemble_kernel builds, per sequence, the left-padded compact cache the reference assembles with
// a dozen index_put / boolean-mask copies (src/msa/memory_sparse_attention.py:299-351), directly in
// storage that has room to append decode tokens, and the rank -> token map of the valid query tokens.
// prefill_attn_kernel is a flash-attention forward over that cache (bf16, head_dim 128): CTA = 64
// query tokens of one head, 4 warps x 16 rows, K/V tiles of 32 keys double-buffered with cp.async,
// mma.sync.m16n8k16, online softmax on the fragments, bottom-right aligned causal mask (a query token
// sees the template, every retrieved entry and the query tokens up to itself).  The contexts are a few
// hundred keys long, so the kernel is latency bound: small tiles and query fragments re-read from
// shared memory keep it at 128 registers and 51 KB, i.e. four CTAs per SM (two at 64-key tiles with
// the query in registers measured 20 % slower).  The point is one launch instead of the gather /
// scatter / re-pack sequence around a library call.
#include <cstdlib>

#include "common.cuh"
#include "mma_helpers.cuh"

namespace msa {

// attn_generic.cu: the same attentions for fp32 and for head sizes other than 128
int launch_attention_rows_by_index(int32_t dtype, const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* k,
                                   const void* v, int64_t k_sb, int64_t k_sh, int64_t k_ss, const int32_t* token_index,
                                   const int32_t* seg_off, int n_segments, long long n_rows, int S, int n_q_heads,
                                   int n_kv_heads, int D, float scale, void* out, cudaStream_t stream);
int launch_attention_rows_in_store(int32_t dtype, const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                                   const void* k_store, const void* v_store, int64_t st_b, int64_t st_h,
                                   const int32_t* kv_start, const int32_t* kv_len, const int32_t* q_tok, const int32_t* num_q,
                                   int n_seq, int S, int n_q_heads, int n_kv_heads, int D, int causal, float scale, void* out,
                                   cudaStream_t stream);

constexpr int kAsmThreads = 256;
constexpr int kAsmSlices = 16;   // CTAs per sequence: the copy loop is dealt over them

// Grid (kAsmSlices, B).  Every CTA of a sequence recomputes the (cheap) token compaction so that no CTA
// waits for another; slice 0 publishes the lengths and the rank -> token map.  Positions outside
// [start, max_kv) of the [0, cap) storage rows are zero-filled here, so the caller hands over
// uninitialised storage.
template <typename T>
__global__ void __launch_bounds__(kAsmThreads)
assemble_kernel(const T* __restrict__ tmpl_k, const T* __restrict__ tmpl_v, int t_len, const T* __restrict__ sel_k,
                const T* __restrict__ sel_v, long long sel_head_stride, const int64_t* __restrict__ n_sel,
                const T* __restrict__ q_k, const T* __restrict__ q_v, long long qs_b, long long qs_h, long long qs_s,
                const uint8_t* __restrict__ valid, int S, int n_kv, int D, int max_kv, int cap, T* __restrict__ k_store,
                T* __restrict__ v_store, long long st_b, long long st_h, int32_t* __restrict__ kv_start,
                int32_t* __restrict__ kv_len, int32_t* __restrict__ q_tok, int32_t* __restrict__ num_q_out,
                int32_t* __restrict__ error_flag) {
  constexpr int V = Elem<T>::kVec;
  extern __shared__ int32_t s_tok[];   // [S] rank -> token: the valid tokens in order, then the others in order
  int32_t* s_pref = s_tok + S;         // [S] valid tokens before token s
  __shared__ int s_warp[kAsmThreads / 32];
  __shared__ int s_base;
  __shared__ long long s_sel_off;
  const int b = blockIdx.y, slice = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_base = 0;
    long long off = 0;
    for (int i = 0; i < b; ++i) off += n_sel[i];
    s_sel_off = off;
  }
  __syncthreads();
  // rank -> token map of the valid query tokens (ordered compaction, 256 tokens per round)
  for (int s0 = 0; s0 < S; s0 += kAsmThreads) {
    const int s = s0 + tid;
    const bool keep = s < S && valid[(long long)b * S + s] != 0;
    const uint32_t bal = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = s_base;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    const int mine = before + __popc(bal & ((1u << lane) - 1u));
    if (keep) s_tok[mine] = s;
    if (s < S) s_pref[s] = keep ? -1 : mine;
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < kAsmThreads / 32; ++w) tot += s_warp[w];
      s_base += tot;
    }
    __syncthreads();
  }
  const int num_q = s_base, ns = (int)n_sel[b];
  for (int t = tid; t < S; t += kAsmThreads)
    if (s_pref[t] >= 0) s_tok[num_q + t - s_pref[t]] = t;
  __syncthreads();
  const int len = t_len + ns + num_q;
  const int start = max_kv - len;
  if (slice == 0) {
    if (tid == 0) {
      kv_len[b] = len;
      kv_start[b] = start;
      num_q_out[b] = num_q;
      if (start < 0) atomicExch(error_flag, 1);
    }
    for (int r = tid; r < S; r += kAsmThreads) q_tok[(long long)b * S + r] = s_tok[r];
  }
  const int vec_row = D / V;
  const long long total = (long long)n_kv * cap * vec_row;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = (long long)slice * kAsmThreads + tid; i < total; i += (long long)kAsmSlices * kAsmThreads) {
    const int dv = (int)(i % vec_row) * V;
    const int pos = (int)((i / vec_row) % cap);
    const int h = (int)(i / ((long long)vec_row * cap));
    const long long d = (long long)b * st_b + (long long)h * st_h + (long long)pos * D + dv;
    const int e = pos - start;
    if (start < 0 || e < 0 || pos >= max_kv) {   // padding, reserve, or a sequence that does not fit
      *reinterpret_cast<uint4*>(k_store + d) = zero;
      *reinterpret_cast<uint4*>(v_store + d) = zero;
      continue;
    }
    const T *sk, *sv;
    if (e < t_len) {
      sk = tmpl_k + ((long long)h * t_len + e) * D + dv;
      sv = tmpl_v + ((long long)h * t_len + e) * D + dv;
    } else if (e < t_len + ns) {
      const long long o = (long long)h * sel_head_stride + (s_sel_off + e - t_len) * D + dv;
      sk = sel_k + o;
      sv = sel_v + o;
    } else {
      const long long o = (long long)b * qs_b + (long long)h * qs_h + (long long)s_tok[e - t_len - ns] * qs_s + dv;
      sk = q_k + o;
      sv = q_v + o;
    }
    *reinterpret_cast<uint4*>(k_store + d) = *reinterpret_cast<const uint4*>(sk);
    *reinterpret_cast<uint4*>(v_store + d) = *reinterpret_cast<const uint4*>(sv);
  }
}

// ---------------------------------------------------------------------------------------
constexpr int kPfRows = 64;    // query tokens per CTA (16 per warp)
constexpr int kPfKeys = 32;    // keys per tile
constexpr int kPfTile = kPfKeys * kMmaRow;                 // one staged K (or V) tile
constexpr int kPfSmem = kPfRows * kMmaRow + 4 * kPfTile;   // Q + 2 x (K, V)

__device__ __forceinline__ void mma_bf16_full(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Running state of one warp's 16 query rows (this thread: rows g and g + 8, columns of its quad).
struct AttnState {
  float o[kMmaD / 8][4];
  float m_run[2], l_run[2];   // l_run: this thread's share of the row sum (reduced over the quad at the end)
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < kMmaD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    m_run[0] = m_run[1] = -INFINITY;
    l_run[0] = l_run[1] = 0.f;
  }
};

// One tile of kPfKeys keys against the warp's 16 rows: S = Q K^T, causal limit per row, online softmax,
// O += P V.  q_frag / kbuf / vbuf are shared-memory addresses; key0 is the tile's first key; limit[rr]
// is the last key row rr may see (kMasked = false: the caller knows every key of the tile is visible to
// every row of the warp).  m_run is kept in raw score units; the softmax scale (times log2 e) enters
// through one fused multiply-add per element.  Key 0 is visible to every row, so the running maximum is
// finite from the first tile on.
template <bool kMasked>
__device__ __forceinline__ void attn_tile(AttnState& st, uint32_t q_frag, uint32_t kbuf, uint32_t vbuf, int key0,
                                          const int (&limit)[2], float scale_log2e, int lane) {
  const int quad = lane & 3, mi = lane >> 3, r = lane & 7;
  float s[kPfKeys / 8][4];
#pragma unroll
  for (int nb = 0; nb < kPfKeys / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
  {
    const uint32_t a = kbuf + ((mi >> 1) * 8 + r) * kMmaRow + (mi & 1) * 16;
#pragma unroll
    for (int j = 0; j < kMmaD / 16; ++j) {   // independent accumulator chains per k-step
      uint32_t qa[4];
      ldmatrix_x4(q_frag + j * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
      for (int nb = 0; nb < kPfKeys / 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(a + nb * 8 * kMmaRow + j * 32, b0, b1, b2, b3);
        mma_bf16_full(s[nb], qa, b0, b1);
        mma_bf16_full(s[nb + 1], qa, b2, b3);
      }
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < kPfKeys / 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (kMasked) {
        const int key = key0 + nb * 8 + 2 * quad + (e & 1);
        if (key > limit[e >> 1]) s[nb][e] = -INFINITY;
      }
      mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
    }
  float f[2], neg_m[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
    mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
    const float m_new = fmaxf(st.m_run[rr], mx[rr]);
    f[rr] = exp2f((st.m_run[rr] - m_new) * scale_log2e);
    st.m_run[rr] = m_new;
    neg_m[rr] = -m_new * scale_log2e;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nb = 0; nb < kPfKeys / 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s[nb][e] = exp2f(fmaf(s[nb][e], scale_log2e, neg_m[e >> 1]));
      sum[e >> 1] += s[nb][e];
    }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) st.l_run[rr] = st.l_run[rr] * f[rr] + sum[rr];
  if (!__all_sync(0xffffffffu, f[0] == 1.f && f[1] == 1.f)) {   // some row's maximum moved: rescale the outputs
#pragma unroll
    for (int nb = 0; nb < kMmaD / 8; ++nb) {
      st.o[nb][0] *= f[0]; st.o[nb][1] *= f[0]; st.o[nb][2] *= f[1]; st.o[nb][3] *= f[1];
    }
  }
#pragma unroll
  for (int kk = 0; kk < kPfKeys / 16; ++kk) {
    uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                      pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
    const uint32_t a = vbuf + (kk * 16 + (mi & 1) * 8 + r) * kMmaRow + (mi >> 1) * 16;
#pragma unroll
    for (int nb = 0; nb < kMmaD / 8; nb += 2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(a + nb * 16, b0, b1, b2, b3);
      mma_bf16_full(st.o[nb], pa, b0, b1);
      mma_bf16_full(st.o[nb + 1], pa, b2, b3);
    }
  }
}

// Dispatch on whether the tile crosses the diagonal of any row of the warp (first_limit: the smallest
// limit among the warp's rows).
__device__ __forceinline__ void attn_tile_auto(AttnState& st, uint32_t q_frag, uint32_t kbuf, uint32_t vbuf, int key0,
                                               const int (&limit)[2], int first_limit, float scale_log2e, int lane) {
  if (key0 + kPfKeys - 1 <= first_limit) attn_tile<false>(st, q_frag, kbuf, vbuf, key0, limit, scale_log2e, lane);
  else attn_tile<true>(st, q_frag, kbuf, vbuf, key0, limit, scale_log2e, lane);
}

// Normalise the warp's rows and write row rr of this thread to dst[rr] (nullptr: the row does not exist).
__device__ __forceinline__ void attn_store(const AttnState& st, __nv_bfloat16* const (&dst)[2], int lane) {
  const int quad = lane & 3;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    float l = st.l_run[rr];   // whole warp: the quad holds the four shares of a row's sum
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (dst[rr] == nullptr) continue;
    const float inv = 1.f / l;
#pragma unroll
    for (int nb = 0; nb < kMmaD / 8; ++nb)
      *reinterpret_cast<uint32_t*>(dst[rr] + nb * 8 + 2 * quad) =
          pack_bf16(st.o[nb][2 * rr] * inv, st.o[nb][2 * rr + 1] * inv);
  }
}

__global__ void __launch_bounds__(128, 4)
prefill_attn_kernel(const __nv_bfloat16* __restrict__ q, long long q_sb, long long q_sh, long long q_ss,
                    const __nv_bfloat16* __restrict__ k_store, const __nv_bfloat16* __restrict__ v_store, long long st_b,
                    long long st_h, const int32_t* __restrict__ kv_start, const int32_t* __restrict__ kv_len,
                    const int32_t* __restrict__ q_tok, const int32_t* __restrict__ num_q_arr, int S, int n_q_heads,
                    int n_kv_heads, int causal, float scale_log2e, __nv_bfloat16* __restrict__ out) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int b = blockIdx.z, hq = blockIdx.y, r0 = blockIdx.x * kPfRows;
  const int num_q = num_q_arr[b];
  // ranks >= num_q are the tokens that take no part: their output rows are zero
  for (int i = threadIdx.x; i < kPfRows * 16; i += 128) {
    const int r = r0 + (i >> 4), ch = i & 15;
    if (r >= num_q && r < S)
      *reinterpret_cast<uint4*>(out + ((long long)b * S + q_tok[(long long)b * S + r]) * n_q_heads * kMmaD +
                                (long long)hq * kMmaD + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (r0 >= num_q) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  // keys every query token sees; without the causal mask (multi-token decode segments) that is the whole context
  const int len = kv_len[b], base_keys = causal ? len - num_q : len - 1;
  const int hk = hq / (n_q_heads / n_kv_heads);
  const long long kv_base = (long long)b * st_b + (long long)hk * st_h + (long long)kv_start[b] * kMmaD;
  const int last_row = causal ? min(r0 + kPfRows, num_q) - 1 : 0;
  const int n_keys = base_keys + last_row + 1;
  const int n_tiles = (n_keys + kPfKeys - 1) / kPfKeys;

  const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t s_kv = s_q + kPfRows * kMmaRow;
  // stage Q (rows beyond num_q are zero-filled)
  for (int i = threadIdx.x; i < kPfRows * 16; i += 128) {
    const int r = i >> 4, ch = i & 15;
    const bool ok = r0 + r < num_q;
    const int tok = ok ? q_tok[(long long)b * S + r0 + r] : 0;
    cp_async16(s_q + r * kMmaRow + ch * 16, q + (long long)b * q_sb + (long long)hq * q_sh + (long long)tok * q_ss + ch * 8,
               ok ? 16u : 0u);
  }
  auto issue = [&](int tile, int buf) {
    const uint32_t kd = s_kv + buf * 2 * kPfTile, vd = kd + kPfTile;
    for (int i = threadIdx.x; i < kPfKeys * 16; i += 128) {
      const int r = i >> 4, ch = i & 15;
      const int key = tile * kPfKeys + r;
      const bool ok = key < n_keys;
      const long long o = kv_base + (long long)(ok ? key : 0) * kMmaD + ch * 8;
      cp_async16(kd + r * kMmaRow + ch * 16, k_store + o, ok ? 16u : 0u);
      cp_async16(vd + r * kMmaRow + ch * 16, v_store + o, ok ? 16u : 0u);
    }
  };
  issue(0, 0);
  cp_async_commit();

  AttnState st;
  st.init();
  const int row_rank[2] = {causal ? min(r0 + warp * 16 + g, num_q - 1) : 0, causal ? min(r0 + warp * 16 + g + 8, num_q - 1) : 0};
  const int limit[2] = {base_keys + row_rank[0], base_keys + row_rank[1]};   // last visible key of each row
  const int warp_limit = base_keys + (causal ? min(r0 + warp * 16 + 15, num_q - 1) : 0);
  const uint32_t q_frag = s_q + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kMmaRow + (lane >> 4) * 16;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) issue(t + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (t * kPfKeys <= warp_limit) {   // later tiles are wholly masked for every row of this warp
      const uint32_t kbuf = s_kv + buf * 2 * kPfTile;
      attn_tile_auto(st, q_frag, kbuf, kbuf + kPfTile, t * kPfKeys, limit,
                     base_keys + (causal ? min(r0 + warp * 16, num_q - 1) : 0), scale_log2e, lane);
    }
    __syncthreads();   // the tile's buffers may be refilled
  }
  cp_async_wait<0>();
  __nv_bfloat16* dst[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int rank = r0 + warp * 16 + g + rr * 8;
    dst[rr] = rank < num_q ? out + ((long long)b * S + q_tok[(long long)b * S + rank]) * n_q_heads * kMmaD +
                                 (long long)hq * kMmaD
                           : nullptr;
  }
  attn_store(st, dst, lane);
}

// ---------------------------------------------------------------------------------------
// Stage 1: causal attention inside every document, with the chunk means of K and V taken from the
// tiles the kernel has staged anyway (src/msa/memory_sparse_attention.py:216-241 and :166-176).
//
// A segment is a run seg_off[i] .. seg_off[i+1] of token_index (flat positions b*S + s of the tokens
// of one document, in order).  CTA = 64 query tokens of one head of one segment; K/V rows are fetched
// through the index, so masked tokens inside a document simply do not appear.  The CTA of a segment's
// last row block walks over every key of the document: for the first head of each kv group it also
// sums the staged rows per chunk (pool_size keys, a multiple of the tile) in fp32 and writes the
// chunk's mean, rounded once, to the bank's pooled K and V.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 4)
doc_attn_pool_kernel(const __nv_bfloat16* __restrict__ q, long long q_sb, long long q_sh, long long q_ss,
                     const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long k_sb,
                     long long k_sh, long long k_ss, const int32_t* __restrict__ token_index,
                     const int32_t* __restrict__ seg_off, int S, uint32_t div_mul, uint32_t div_shift, int n_q_heads,
                     int n_kv_heads, float scale_log2e,
                     __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ chunk_offsets, int n_chunks,
                     int pool_size, __nv_bfloat16* __restrict__ pooled_k, __nv_bfloat16* __restrict__ pooled_v,
                     long long pool_chunk_stride, long long pool_head_stride) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int seg = blockIdx.z, hq = blockIdx.y, r0 = blockIdx.x * kPfRows;
  const int t0 = seg_off[seg], len = seg_off[seg + 1] - t0;
  if (r0 >= len) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  const int grp = n_q_heads / n_kv_heads, hk = hq / grp;
  const int last_row = min(r0 + kPfRows, len) - 1;
  const int n_keys = last_row + 1;
  const int n_tiles = (n_keys + kPfKeys - 1) / kPfKeys;
  const bool pools = chunk_offsets != nullptr && last_row == len - 1 && hq % grp == 0;
  const int32_t* tix = token_index + t0;
  // flat token position -> element offset inside a [B, H, S, D] tensor; tok / S by multiply-high and shift
  auto offset = [&](int tok, long long sb, long long ss) {
    const uint32_t bi = (__umulhi((uint32_t)tok, div_mul) + (uint32_t)tok) >> div_shift;
    return (long long)bi * sb + (long long)(tok - (int)bi * S) * ss;
  };

  const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t s_kv = s_q + kPfRows * kMmaRow;
  for (int i = threadIdx.x; i < kPfRows * 16; i += 128) {
    const int r = i >> 4, ch = i & 15;
    const bool ok = r0 + r < len;
    const int tok = ok ? tix[r0 + r] : 0;
    cp_async16(s_q + r * kMmaRow + ch * 16, q + offset(tok, q_sb, q_ss) + (long long)hq * q_sh + ch * 8, ok ? 16u : 0u);
  }
  // A document without masked tokens is a run of consecutive positions of one row: its keys are
  // addressed without the index (token_index is ascending, so first/last decide it).
  const int tok0 = tix[0];
  const bool run = tix[len - 1] - tok0 == len - 1 &&
                   ((__umulhi((uint32_t)tok0, div_mul) + (uint32_t)tok0) >> div_shift) ==
                       ((__umulhi((uint32_t)(tok0 + len - 1), div_mul) + (uint32_t)(tok0 + len - 1)) >> div_shift);
  const long long run_base = offset(tok0, k_sb, k_ss) + (long long)hk * k_sh;
  auto issue = [&](int tile, int buf) {
    const uint32_t kd = s_kv + buf * 2 * kPfTile, vd = kd + kPfTile;
    for (int i = threadIdx.x; i < kPfKeys * 16; i += 128) {
      const int r = i >> 4, ch = i & 15;
      const int key = tile * kPfKeys + r;
      const bool ok = key < n_keys;
      long long o;
      if (run) o = run_base + (long long)(ok ? key : 0) * k_ss + ch * 8;
      else o = offset(ok ? tix[key] : 0, k_sb, k_ss) + (long long)hk * k_sh + ch * 8;
      cp_async16(kd + r * kMmaRow + ch * 16, k + o, ok ? 16u : 0u);
      cp_async16(vd + r * kMmaRow + ch * 16, v + o, ok ? 16u : 0u);
    }
  };
  issue(0, 0);
  cp_async_commit();

  // first chunk of this document: the chunk whose first token is the segment's first token
  int chunk0 = 0;
  if (pools) {
    int lo = 0, hi = n_chunks;   // chunk_offsets is ascending; find the entry equal to t0
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (chunk_offsets[mid] < t0) lo = mid + 1; else hi = mid;
    }
    chunk0 = lo;
  }
  float pk = 0.f, pv = 0.f;   // thread d: running sums of column d over the current chunk

  AttnState st;
  st.init();
  const int limit[2] = {min(r0 + warp * 16 + g, len - 1), min(r0 + warp * 16 + g + 8, len - 1)};
  const int warp_limit = min(r0 + warp * 16 + 15, len - 1);
  const uint32_t q_frag = s_q + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kMmaRow + (lane >> 4) * 16;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) issue(t + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kbuf = s_kv + buf * 2 * kPfTile;
    if (t * kPfKeys <= warp_limit)
      attn_tile_auto(st, q_frag, kbuf, kbuf + kPfTile, t * kPfKeys, limit, min(r0 + warp * 16, len - 1), scale_log2e, lane);
    if (pools) {   // CTA-uniform; rows past the document's end are zero in shared memory
      const unsigned char* kb = smem + kPfRows * kMmaRow + buf * 2 * kPfTile + threadIdx.x * 2;
#pragma unroll 8
      for (int r = 0; r < kPfKeys; ++r) {
        pk += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(kb + r * kMmaRow));
        pv += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(kb + kPfTile + r * kMmaRow));
      }
      const int key_end = min((t + 1) * kPfKeys, len);
      if (key_end % pool_size == 0 || key_end == len) {   // the chunk is complete
        const int c = (key_end - 1) / pool_size;
        const float inv = 1.f / (float)(key_end - c * pool_size);
        const long long o = (long long)(chunk0 + c) * pool_chunk_stride + (long long)hk * pool_head_stride + threadIdx.x;
        pooled_k[o] = __float2bfloat16_rn(pk * inv);
        pooled_v[o] = __float2bfloat16_rn(pv * inv);
        pk = pv = 0.f;
      }
    }
    __syncthreads();   // the tile's buffers may be refilled
  }
  cp_async_wait<0>();
  __nv_bfloat16* dst[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int rank = r0 + warp * 16 + g + rr * 8;
    dst[rr] = rank < len ? out + (long long)tix[rank] * n_q_heads * kMmaD + (long long)hq * kMmaD : nullptr;
  }
  attn_store(st, dst, lane);
}

}  // namespace msa

using namespace msa;

extern "C" int msa_assemble_context(const void* template_k, const void* template_v, int32_t template_len,
                                    const void* sel_k, const void* sel_v, int64_t sel_head_stride, const int64_t* n_sel,
                                    const void* q_k, const void* q_v, int64_t q_stride_b, int64_t q_stride_h,
                                    int64_t q_stride_s, const uint8_t* valid, int32_t n_seq, int32_t seq_len,
                                    int32_t n_kv_heads, int32_t head_dim, int32_t dtype, int32_t max_kv,
                                    int32_t store_len, void* k_store, void* v_store, int64_t store_stride_b, int64_t store_stride_h, int32_t* kv_start,
                                    int32_t* kv_len, int32_t* q_tok, int32_t* num_q, int32_t* error_flag, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "assemble: unknown dtype %d", dtype);
  MSA_REQUIRE(n_sel && q_k && q_v && valid && k_store && v_store && kv_start && kv_len && q_tok && num_q && error_flag,
              "assemble: null pointer");
  MSA_REQUIRE(template_len == 0 || (template_k && template_v), "assemble: template pointers missing");
  MSA_REQUIRE(n_seq >= 0 && seq_len >= 0 && n_kv_heads > 0 && head_dim > 0 && max_kv >= 0 && template_len >= 0 &&
                  store_len >= max_kv && n_seq <= 65535, "assemble: bad sizes");
  MSA_REQUIRE((size_t)seq_len * 2 * sizeof(int32_t) <= 40 * 1024, "assemble: seq_len %d above 5120 tokens", seq_len);
  const int vec = 16 / (int)dtype_size(dtype);
  MSA_REQUIRE(head_dim % vec == 0 && q_stride_b % vec == 0 && q_stride_h % vec == 0 && q_stride_s % vec == 0 &&
                  sel_head_stride % vec == 0 && store_stride_b % vec == 0 && store_stride_h % vec == 0,
              "assemble: rows must keep 16-byte alignment");
  MSA_REQUIRE(aligned16(q_k) && aligned16(q_v) && aligned16(k_store) && aligned16(v_store) &&
                  (!sel_k || (aligned16(sel_k) && aligned16(sel_v))) &&
                  (!template_k || (aligned16(template_k) && aligned16(template_v))),
              "assemble: pointers must be 16-byte aligned");
  if (n_seq == 0) return MSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  MSA_CUDA_OK(cudaMemsetAsync(error_flag, 0, sizeof(int32_t), st));
  if (dtype == MSA_BF16)
    assemble_kernel<__nv_bfloat16><<<dim3(kAsmSlices, n_seq), kAsmThreads, 2 * seq_len * sizeof(int32_t), st>>>(
        (const __nv_bfloat16*)template_k, (const __nv_bfloat16*)template_v, template_len, (const __nv_bfloat16*)sel_k,
        (const __nv_bfloat16*)sel_v, sel_head_stride, n_sel, (const __nv_bfloat16*)q_k, (const __nv_bfloat16*)q_v,
        q_stride_b, q_stride_h, q_stride_s, valid, seq_len, n_kv_heads, head_dim, max_kv, store_len,
        (__nv_bfloat16*)k_store,
        (__nv_bfloat16*)v_store, store_stride_b, store_stride_h, kv_start, kv_len, q_tok, num_q, error_flag);
  else
    assemble_kernel<float><<<dim3(kAsmSlices, n_seq), kAsmThreads, 2 * seq_len * sizeof(int32_t), st>>>(
        (const float*)template_k, (const float*)template_v, template_len, (const float*)sel_k, (const float*)sel_v,
        sel_head_stride, n_sel, (const float*)q_k, (const float*)q_v, q_stride_b, q_stride_h, q_stride_s, valid, seq_len,
        n_kv_heads, head_dim, max_kv, store_len, (float*)k_store, (float*)v_store, store_stride_b, store_stride_h, kv_start,
        kv_len, q_tok, num_q, error_flag);
  MSA_LAUNCH_OK("assemble_kernel");
  return MSA_OK;
}

extern "C" int msa_sparse_prefill_attn(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                       const void* k_store, const void* v_store, int64_t store_stride_b,
                                       int64_t store_stride_h, const int32_t* kv_start, const int32_t* kv_len,
                                       const int32_t* q_tok, const int32_t* num_q, int32_t n_seq, int32_t seq_len,
                                       int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t dtype,
                                       int32_t causal, float scale, void* out, void* stream) {
  MSA_REQUIRE(q && k_store && v_store && kv_start && kv_len && q_tok && num_q && out, "prefill: null pointer");
  MSA_REQUIRE(dtype_ok(dtype) && head_dim > 0, "prefill: unknown dtype %d or bad head_dim", dtype);
  MSA_REQUIRE(n_seq >= 0 && seq_len >= 0 && n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0 &&
                  n_q_heads <= 65535 && n_seq <= 65535, "prefill: bad sizes");
  if (dtype != MSA_BF16 || head_dim != kMmaD) {   // fp32 / other head sizes: the general kernel
    if (n_seq == 0 || seq_len == 0) return MSA_OK;
    return launch_attention_rows_in_store(dtype, q, q_stride_b, q_stride_h, q_stride_s, k_store, v_store, store_stride_b,
                                          store_stride_h, kv_start, kv_len, q_tok, num_q, n_seq, seq_len, n_q_heads,
                                          n_kv_heads, head_dim, causal != 0, scale, out, (cudaStream_t)stream);
  }
  MSA_REQUIRE(q_stride_b % 8 == 0 && q_stride_h % 8 == 0 && q_stride_s % 8 == 0 && store_stride_b % 8 == 0 &&
                  store_stride_h % 8 == 0 && aligned16(q) && aligned16(k_store) && aligned16(v_store) && aligned16(out),
              "prefill: rows must be 16-byte aligned");
  if (n_seq == 0 || seq_len == 0) return MSA_OK;
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(prefill_attn_kernel, kPfSmem, configured));
  dim3 grid((seq_len + kPfRows - 1) / kPfRows, n_q_heads, n_seq);
  prefill_attn_kernel<<<grid, 128, kPfSmem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q, q_stride_b, q_stride_h, q_stride_s, (const __nv_bfloat16*)k_store,
      (const __nv_bfloat16*)v_store, store_stride_b, store_stride_h, kv_start, kv_len, q_tok, num_q, seq_len, n_q_heads,
      n_kv_heads, causal != 0, scale * 1.4426950408889634f, (__nv_bfloat16*)out);
  MSA_LAUNCH_OK("prefill_attn_kernel");
  return MSA_OK;
}

extern "C" int msa_doc_attention_pool(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                      const void* k, const void* v, int64_t k_stride_b, int64_t k_stride_h,
                                      int64_t k_stride_s, const int32_t* token_index, const int32_t* seg_offsets,
                                      int32_t n_segments, int32_t max_segment_len, int32_t seq_len, int32_t n_q_heads,
                                      int32_t n_kv_heads, int32_t head_dim, int32_t dtype, float scale, void* out,
                                      const int32_t* chunk_offsets, int32_t n_chunks, int32_t pool_size, void* pooled_k,
                                      void* pooled_v, int64_t pool_chunk_stride, int64_t pool_head_stride, void* stream) {
  MSA_REQUIRE(q && k && v && token_index && seg_offsets && out, "doc_attention: null pointer");
  MSA_REQUIRE(dtype_ok(dtype) && head_dim > 0, "doc_attention: unknown dtype %d or bad head_dim", dtype);
  if (dtype != MSA_BF16 || head_dim != kMmaD) {   // fp32 / other head sizes: the general kernel, pooling separately
    MSA_REQUIRE(chunk_offsets == nullptr, "doc_attention: the K / V pooling by-product needs bf16 with head_dim 128 "
                                          "(pool with msa_pool_chunks instead)");
    MSA_REQUIRE(n_segments >= 0 && max_segment_len >= 0 && seq_len > 0 && n_q_heads > 0 && n_kv_heads > 0 &&
                    n_q_heads % n_kv_heads == 0, "doc_attention: bad sizes");
    if (n_segments == 0 || max_segment_len == 0) return MSA_OK;
    return launch_attention_rows_by_index(dtype, q, q_stride_b, q_stride_h, q_stride_s, k, v, k_stride_b, k_stride_h,
                                          k_stride_s, token_index, seg_offsets, n_segments,
                                          (long long)n_segments * max_segment_len, seq_len, n_q_heads, n_kv_heads, head_dim,
                                          scale, out, (cudaStream_t)stream);
  }
  MSA_REQUIRE(n_segments >= 0 && max_segment_len >= 0 && seq_len > 0 && n_q_heads > 0 && n_kv_heads > 0 &&
                  n_q_heads % n_kv_heads == 0 && n_q_heads <= 65535 && n_segments <= 65535,
              "doc_attention: bad sizes (at most 65535 segments per call)");
  MSA_REQUIRE(q_stride_b % 8 == 0 && q_stride_h % 8 == 0 && q_stride_s % 8 == 0 && k_stride_b % 8 == 0 &&
                  k_stride_h % 8 == 0 && k_stride_s % 8 == 0 && aligned16(q) && aligned16(k) && aligned16(v) &&
                  aligned16(out), "doc_attention: rows must be 16-byte aligned");
  if (chunk_offsets) {
    MSA_REQUIRE(pooled_k && pooled_v && n_chunks >= 0, "doc_attention: pooled outputs missing");
    MSA_REQUIRE(pool_size > 0 && pool_size % kPfKeys == 0,
                "doc_attention: pooling_kernel_size %d is not a multiple of %d (pool with msa_pool_chunks instead)",
                pool_size, kPfKeys);
  }
  if (n_segments == 0 || max_segment_len == 0) return MSA_OK;
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(doc_attn_pool_kernel, kPfSmem, configured));
  // tok / seq_len for tok < 2^31: (mulhi(tok, mul) + tok) >> shift with shift = ceil(log2 seq_len)
  uint32_t div_shift = 0;
  while ((1ull << div_shift) < (uint64_t)seq_len) ++div_shift;
  const uint32_t div_mul = (uint32_t)((((1ull << div_shift) - (uint64_t)seq_len) << 32) / (uint64_t)seq_len + 1);
  dim3 grid((max_segment_len + kPfRows - 1) / kPfRows, n_q_heads, n_segments);
  doc_attn_pool_kernel<<<grid, 128, kPfSmem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q, q_stride_b, q_stride_h, q_stride_s, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
      k_stride_b, k_stride_h, k_stride_s, token_index, seg_offsets, seq_len, div_mul, div_shift, n_q_heads, n_kv_heads,
      scale * 1.4426950408889634f, (__nv_bfloat16*)out, chunk_offsets, n_chunks, pool_size, (__nv_bfloat16*)pooled_k,
      (__nv_bfloat16*)pooled_v, pool_chunk_stride, pool_head_stride);
  MSA_LAUNCH_OK("doc_attn_pool_kernel");
  return MSA_OK;
}
