// Attention for the shapes the tensor-core kernels do not take (fp32, or a head size other than 128), and the
// append of a multi-token segment to the compact cache.
//
// The bf16 / head_dim 128 kernels (prefill_attn.cu, doc_attn_tc.cu) are the fast path.  Everything else -- the
// reference's CPU-runnable fp32 configuration above all -- used to fall to a library call; these kernels close that
// gap so that every attention of the path runs on this package's code.  They are written for exactness, not speed:
// one warp per (query row, head); keys are walked 32 at a time (one per lane: a dot product of D), an online
// softmax in the log2 domain keeps a running maximum and sum, and the value rows are accumulated with every lane
// owning the dims d = lane, lane + 32, ...; accumulation in fp32, one rounding at the end.
//
// Two ways of naming rows and keys:
//   rows_by_index  (stage 1, src/msa/memory_sparse_attention.py:216-241): segment i = rows seg_off[i] .. seg_off[i+1]
//                  of token_index (flat positions b*S + s); row j of a segment sees rows 0..j of the same segment;
//   rows_in_store  (stage 2 and multi-token decode segments, :282-357 and :375-380): sequence b's r-th valid token
//                  (q_tok) sees positions kv_start[b] .. of the [B, Hkv, L, D] store: all kv_len[b] of them, or, with
//                  the bottom-right aligned causal mask, the first kv_len[b] - num_q[b] + r + 1.
#include "common.cuh"

namespace msa {

constexpr int kGaWarps = 4;
constexpr int kGaMaxD = 256;

// q_row: this row's query [D]; key(j) / val(j): pointers to key / value row j (D contiguous elements).
template <typename T, typename KeyFn, typename ValFn>
__device__ __forceinline__ void warp_attend(const T* __restrict__ q_row, int D, int n_keys, float scale_log2e, KeyFn key,
                                            ValFn val, float* s_q, T* __restrict__ out_row) {
  const int lane = threadIdx.x & 31;
  for (int d = lane; d < D; d += 32) s_q[d] = (float)q_row[d] * scale_log2e;
  __syncwarp();
  float m = -INFINITY, l = 0.f;
  float acc[kGaMaxD / 32];
#pragma unroll
  for (int i = 0; i < kGaMaxD / 32; ++i) acc[i] = 0.f;
  for (int j0 = 0; j0 < n_keys; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < n_keys) {
      const T* kr = key(j);
      s = 0.f;
      for (int d = 0; d < D; ++d) s = fmaf(s_q[d], (float)kr[d], s);
    }
    float mx = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float m_new = fmaxf(m, mx);                 // finite: the tile holds at least one key
    const float f = exp2f(m - m_new);                 // 0 on the first tile
    const float pr = j < n_keys ? exp2f(s - m_new) : 0.f;
    float sum = pr;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    l = l * f + sum;
    m = m_new;
#pragma unroll
    for (int i = 0; i < kGaMaxD / 32; ++i) acc[i] *= f;
    const int n_here = min(32, n_keys - j0);
    for (int jj = 0; jj < n_here; ++jj) {
      const float w = __shfl_sync(0xffffffffu, pr, jj);
      const T* vr = val(j0 + jj);
#pragma unroll
      for (int i = 0; i < kGaMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(w, (float)vr[d], acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kGaMaxD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out_row[d] = (T)(acc[i] * inv);
  }
  __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(kGaWarps * 32)
attn_rows_by_index_kernel(const T* __restrict__ q, long long q_sb, long long q_sh, long long q_ss, const T* __restrict__ k,
                          const T* __restrict__ v, long long k_sb, long long k_sh, long long k_ss,
                          const int32_t* __restrict__ token_index, const int32_t* __restrict__ seg_off, int n_segments,
                          int S, int n_q_heads, int n_kv_heads, int D, float scale_log2e, T* __restrict__ out) {
  __shared__ float s_q[kGaWarps][kGaMaxD];
  const int warp = threadIdx.x >> 5;
  const long long n_rows = seg_off[n_segments] - seg_off[0];
  const long long item = (long long)blockIdx.x * kGaWarps + warp;     // (row, head)
  if (item >= n_rows * n_q_heads) return;
  const int hq = (int)(item % n_q_heads);
  const long long row = seg_off[0] + item / n_q_heads;
  int lo = 0, hi = n_segments;                                        // the segment that holds this row
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (seg_off[mid] <= row) lo = mid; else hi = mid;
  }
  const int first = seg_off[lo], n_keys = (int)(row - first) + 1;
  const int tok = token_index[row];
  const int b = tok / S, s = tok % S, hk = hq / (n_q_heads / n_kv_heads);
  auto addr = [&](const T* base, int j) {
    const int t = token_index[first + j];
    return base + (long long)(t / S) * k_sb + (long long)hk * k_sh + (long long)(t % S) * k_ss;
  };
  warp_attend<T>(q + (long long)b * q_sb + (long long)hq * q_sh + (long long)s * q_ss, D, n_keys, scale_log2e,
                 [&](int j) { return addr(k, j); }, [&](int j) { return addr(v, j); }, s_q[warp],
                 out + ((long long)b * S + s) * n_q_heads * D + (long long)hq * D);
}

template <typename T>
__global__ void __launch_bounds__(kGaWarps * 32)
attn_rows_in_store_kernel(const T* __restrict__ q, long long q_sb, long long q_sh, long long q_ss,
                          const T* __restrict__ k_store, const T* __restrict__ v_store, long long st_b, long long st_h,
                          const int32_t* __restrict__ kv_start, const int32_t* __restrict__ kv_len,
                          const int32_t* __restrict__ q_tok, const int32_t* __restrict__ num_q, int n_seq, int S,
                          int n_q_heads, int n_kv_heads, int D, int causal, float scale_log2e, T* __restrict__ out) {
  __shared__ float s_q[kGaWarps][kGaMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kGaWarps + warp;     // (sequence, rank, head)
  if (item >= (long long)n_seq * S * n_q_heads) return;
  const int hq = (int)(item % n_q_heads);
  const int r = (int)((item / n_q_heads) % S), b = (int)(item / ((long long)n_q_heads * S));
  const int tok = q_tok[(long long)b * S + r];
  T* out_row = out + ((long long)b * S + tok) * n_q_heads * D + (long long)hq * D;
  const int nq = num_q[b];
  if (r >= nq) {                                                      // a token that takes no part: zero row
    for (int d = lane; d < D; d += 32) out_row[d] = (T)0.f;
    return;
  }
  const int len = kv_len[b], n_keys = causal ? len - nq + r + 1 : len;
  const int hk = hq / (n_q_heads / n_kv_heads);
  const long long base = (long long)b * st_b + (long long)hk * st_h + (long long)kv_start[b] * D;
  warp_attend<T>(q + (long long)b * q_sb + (long long)hq * q_sh + (long long)tok * q_ss, D, n_keys, scale_log2e,
                 [&](int j) { return k_store + base + (long long)j * D; },
                 [&](int j) { return v_store + base + (long long)j * D; }, s_q[warp], out_row);
}

// Appends the valid tokens of a segment [B, Hkv, S, D] to every sequence's cache, in order, at positions
// kv_start[b] + kv_len[b] ..; writes the rank -> token map (valid tokens first, as msa_assemble_context does) and
// the number of valid tokens, and adds that number to kv_len[b].  One CTA per sequence.
template <typename T>
__global__ void __launch_bounds__(256)
append_segment_kernel(const T* __restrict__ seg_k, const T* __restrict__ seg_v, long long s_sb, long long s_sh,
                      long long s_ss, const uint8_t* __restrict__ valid, int S, int n_kv, int D, T* __restrict__ k_store,
                      T* __restrict__ v_store, long long st_b, long long st_h, int store_len,
                      const int32_t* __restrict__ kv_start, int32_t* __restrict__ kv_len, int32_t* __restrict__ q_tok,
                      int32_t* __restrict__ num_q, int32_t* __restrict__ error_flag) {
  extern __shared__ int32_t s_rank[];      // [S]: destination rank of a valid token, -1 otherwise
  __shared__ int s_n;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {                  // segments are short (tens to hundreds of tokens): a serial scan is enough
    int n = 0;
    for (int s = 0; s < S; ++s) s_rank[s] = valid[(long long)b * S + s] ? n++ : -1;
    int other = n;
    for (int s = 0; s < S; ++s) q_tok[(long long)b * S + (s_rank[s] >= 0 ? s_rank[s] : other++)] = s;
    s_n = n;
  }
  __syncthreads();
  const int n = s_n, start = kv_start ? kv_start[b] : 0, old = kv_len[b];
  const bool fits = start + old + n <= store_len;
  if (fits) {
    for (long long i = threadIdx.x; i < (long long)S * n_kv * D; i += blockDim.x) {
      const int d = (int)(i % D), h = (int)((i / D) % n_kv), s = (int)(i / ((long long)D * n_kv));
      if (s_rank[s] < 0) continue;
      const long long src = (long long)b * s_sb + (long long)h * s_sh + (long long)s * s_ss + d;
      const long long dst = (long long)b * st_b + (long long)h * st_h + (long long)(start + old + s_rank[s]) * D + d;
      k_store[dst] = seg_k[src];
      v_store[dst] = seg_v[src];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    num_q[b] = fits ? n : 0;
    if (fits) kv_len[b] = old + n;
    else atomicExch(error_flag, 1);
  }
}

template <typename T>
int launch_rows_by_index(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* k, const void* v,
                         int64_t k_sb, int64_t k_sh, int64_t k_ss, const int32_t* token_index, const int32_t* seg_off,
                         int n_segments, long long n_rows, int S, int n_q_heads, int n_kv_heads, int D, float scale, void* out,
                         cudaStream_t stream) {
  const long long items = n_rows * n_q_heads;
  if (items == 0) return MSA_OK;
  attn_rows_by_index_kernel<T><<<(unsigned)((items + kGaWarps - 1) / kGaWarps), kGaWarps * 32, 0, stream>>>(
      (const T*)q, q_sb, q_sh, q_ss, (const T*)k, (const T*)v, k_sb, k_sh, k_ss, token_index, seg_off, n_segments, S,
      n_q_heads, n_kv_heads, D, scale * 1.4426950408889634f, (T*)out);
  MSA_LAUNCH_OK("attn_rows_by_index_kernel");
  return MSA_OK;
}

int launch_attention_rows_by_index(int32_t dtype, const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* k,
                                   const void* v, int64_t k_sb, int64_t k_sh, int64_t k_ss, const int32_t* token_index,
                                   const int32_t* seg_off, int n_segments, long long n_rows, int S, int n_q_heads,
                                   int n_kv_heads, int D, float scale, void* out, cudaStream_t stream) {
  MSA_REQUIRE(D >= 1 && D <= kGaMaxD, "attention (general kernel): head_dim %d exceeds %d", D, kGaMaxD);
  return dtype == MSA_BF16
             ? launch_rows_by_index<__nv_bfloat16>(q, q_sb, q_sh, q_ss, k, v, k_sb, k_sh, k_ss, token_index, seg_off,
                                                   n_segments, n_rows, S, n_q_heads, n_kv_heads, D, scale, out, stream)
             : launch_rows_by_index<float>(q, q_sb, q_sh, q_ss, k, v, k_sb, k_sh, k_ss, token_index, seg_off, n_segments,
                                           n_rows, S, n_q_heads, n_kv_heads, D, scale, out, stream);
}

template <typename T>
int launch_rows_in_store(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* k_store, const void* v_store,
                         int64_t st_b, int64_t st_h, const int32_t* kv_start, const int32_t* kv_len, const int32_t* q_tok,
                         const int32_t* num_q, int n_seq, int S, int n_q_heads, int n_kv_heads, int D, int causal, float scale,
                         void* out, cudaStream_t stream) {
  const long long items = (long long)n_seq * S * n_q_heads;
  if (items == 0) return MSA_OK;
  attn_rows_in_store_kernel<T><<<(unsigned)((items + kGaWarps - 1) / kGaWarps), kGaWarps * 32, 0, stream>>>(
      (const T*)q, q_sb, q_sh, q_ss, (const T*)k_store, (const T*)v_store, st_b, st_h, kv_start, kv_len, q_tok, num_q, n_seq,
      S, n_q_heads, n_kv_heads, D, causal, scale * 1.4426950408889634f, (T*)out);
  MSA_LAUNCH_OK("attn_rows_in_store_kernel");
  return MSA_OK;
}

int launch_attention_rows_in_store(int32_t dtype, const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                                   const void* k_store, const void* v_store, int64_t st_b, int64_t st_h,
                                   const int32_t* kv_start, const int32_t* kv_len, const int32_t* q_tok, const int32_t* num_q,
                                   int n_seq, int S, int n_q_heads, int n_kv_heads, int D, int causal, float scale, void* out,
                                   cudaStream_t stream) {
  MSA_REQUIRE(D >= 1 && D <= kGaMaxD, "attention (general kernel): head_dim %d exceeds %d", D, kGaMaxD);
  return dtype == MSA_BF16
             ? launch_rows_in_store<__nv_bfloat16>(q, q_sb, q_sh, q_ss, k_store, v_store, st_b, st_h, kv_start, kv_len, q_tok,
                                                   num_q, n_seq, S, n_q_heads, n_kv_heads, D, causal, scale, out, stream)
             : launch_rows_in_store<float>(q, q_sb, q_sh, q_ss, k_store, v_store, st_b, st_h, kv_start, kv_len, q_tok, num_q,
                                           n_seq, S, n_q_heads, n_kv_heads, D, causal, scale, out, stream);
}

}  // namespace msa

using namespace msa;

extern "C" int msa_append_segment(const void* seg_k, const void* seg_v, int64_t seg_stride_b, int64_t seg_stride_h,
                                  int64_t seg_stride_s, const uint8_t* valid, int32_t n_seq, int32_t seq_len,
                                  int32_t n_kv_heads, int32_t head_dim, int32_t dtype, void* k_store, void* v_store,
                                  int64_t store_stride_b, int64_t store_stride_h, int32_t store_len,
                                  const int32_t* kv_start, int32_t* kv_len, int32_t* q_tok, int32_t* num_q,
                                  int32_t* error_flag, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "append_segment: unknown dtype %d", dtype);
  MSA_REQUIRE(seg_k && seg_v && valid && k_store && v_store && kv_len && q_tok && num_q && error_flag,
              "append_segment: null pointer");
  MSA_REQUIRE(n_seq >= 0 && seq_len >= 1 && seq_len <= 8192 && n_kv_heads > 0 && head_dim > 0 && store_len > 0,
              "append_segment: bad sizes (a segment holds at most 8192 tokens)");
  if (n_seq == 0) return MSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)seq_len * sizeof(int32_t);
  if (dtype == MSA_BF16)
    append_segment_kernel<__nv_bfloat16><<<n_seq, 256, smem, st>>>(
        (const __nv_bfloat16*)seg_k, (const __nv_bfloat16*)seg_v, seg_stride_b, seg_stride_h, seg_stride_s, valid, seq_len,
        n_kv_heads, head_dim, (__nv_bfloat16*)k_store, (__nv_bfloat16*)v_store, store_stride_b, store_stride_h, store_len,
        kv_start, kv_len, q_tok, num_q, error_flag);
  else
    append_segment_kernel<float><<<n_seq, 256, smem, st>>>(
        (const float*)seg_k, (const float*)seg_v, seg_stride_b, seg_stride_h, seg_stride_s, valid, seq_len, n_kv_heads,
        head_dim, (float*)k_store, (float*)v_store, store_stride_b, store_stride_h, store_len, kv_start, kv_len, q_tok,
        num_q, error_flag);
  MSA_LAUNCH_OK("append_segment_kernel");
  return MSA_OK;
}
