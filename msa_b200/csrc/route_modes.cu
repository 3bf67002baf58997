// Routing in the reduce modes the fused kernels do not cover: head_reduce "max" (any query reduce) and
// chunk_reduce "mean".
//
// The fused kernels (route_tc.cu, route_simt.cu) rest on two facts of the shipped configuration: a MEAN over
// heads is linear, so the 32 per-head dot products fold into one 1024-wide one, and a MAX over chunks can be
// taken with atomicMax on keys.  Neither holds here, so these modes go through a per-(sequence, chunk) score
// table [n_seq, n_chunks + 1] of order-preserving keys (column c + 1 = chunk c, the layout the fused kernels
// produce when every chunk is given its own document id) and a second, small kernel that reduces chunks to
// documents:
//   head "max"   : chunk_scores_kernel below - per-head dot products on CUDA cores, head reduce across lanes,
//                  query reduce in registers;
//   head "mean"  : the fused kernel with identity document ids fills the chunk table (no new scoring code);
//   chunk "mean" / "max": reduce_chunks_kernel, one thread per (sequence, first chunk of a document).
#include "common.cuh"

namespace msa {

constexpr int kCsChunks = 16;    // chunks per CTA
constexpr int kCsThreads = 256;  // 16 chunks x 16 lanes; a chunk's 16 lanes split the query heads
constexpr int kCsPad = 4;        // floats of padding per head row: spreads the kv heads over the banks

// grid (chunk tiles, sequences).  K tile in shared memory as fp32 [16][Hkv][D + pad].
template <typename T>
__global__ void __launch_bounds__(kCsThreads)
chunk_scores_kernel(const T* __restrict__ q, long long stride_b, long long stride_h, long long stride_s,
                    const uint8_t* __restrict__ mask, long long mask_stride_b, int n_q_heads, int n_groups, int seq_len,
                    int head_dim, int head_reduce, int query_reduce, const T* __restrict__ rk, long long rk_stride,
                    int n_chunks, float scale, uint32_t min_key, uint32_t* __restrict__ chunk_keys,
                    long long table_stride) {
  extern __shared__ float s_k[];
  const int n_kv = n_q_heads / n_groups, row = head_dim + kCsPad;
  const int c0 = blockIdx.x * kCsChunks, b = blockIdx.y;
  for (int i = threadIdx.x; i < kCsChunks * n_kv * head_dim; i += kCsThreads) {
    const int c = i / (n_kv * head_dim), r = i % (n_kv * head_dim);
    const int h = r / head_dim, d = r % head_dim;
    s_k[(c * n_kv + h) * row + d] = c0 + c < n_chunks ? (float)rk[(long long)(c0 + c) * rk_stride + r] : 0.f;
  }
  __syncthreads();
  const int c = threadIdx.x / 16, j = threadIdx.x % 16;   // a chunk's 16 lanes are half a warp
  const uint8_t* m = mask + (long long)b * mask_stride_b;
  int count = 0;
  for (int t = 0; t < seq_len; ++t) count += m[t] ? 1 : 0;
  const int last = max(count - 1, 0);
  float acc = query_reduce == MSA_QREDUCE_MEAN ? 0.f : -INFINITY;
  for (int s = 0; s < seq_len; ++s) {
    if (query_reduce == MSA_QREDUCE_LAST ? s != last : !m[s]) continue;   // uniform over the CTA
    // this lane's share of the heads, reduced locally, then across the chunk's 16 lanes
    float part = head_reduce == MSA_HREDUCE_MAX ? -INFINITY : 0.f;
    for (int hq = j; hq < n_q_heads; hq += 16) {
      const T* qr = q + (long long)b * stride_b + (long long)hq * stride_h + (long long)s * stride_s;
      const float* kr = s_k + (c * n_kv + hq / n_groups) * row;
      float dot = 0.f;
      for (int d = 0; d < head_dim; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kr + d);
        dot = fmaf((float)qr[d], kv.x, dot);
        dot = fmaf((float)qr[d + 1], kv.y, dot);
        dot = fmaf((float)qr[d + 2], kv.z, dot);
        dot = fmaf((float)qr[d + 3], kv.w, dot);
      }
      part = head_reduce == MSA_HREDUCE_MAX ? fmaxf(part, dot) : part + dot;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, part, o);
      part = head_reduce == MSA_HREDUCE_MAX ? fmaxf(part, other) : part + other;
    }
    if (head_reduce == MSA_HREDUCE_MEAN) part /= (float)n_q_heads;
    // a token that is selected but masked scores min_val in the reference (query_reduce "last" with no valid token)
    if (!m[s]) part = -INFINITY;
    acc = query_reduce == MSA_QREDUCE_MEAN ? acc + part : fmaxf(acc, part);
  }
  if (query_reduce == MSA_QREDUCE_MEAN) acc /= (float)max(count, 1);
  if (j == 0 && c0 + c < n_chunks) {
    const uint32_t key = float_to_key(acc * scale);
    chunk_keys[(long long)b * table_stride + 1 + c0 + c] = max(key, min_key);
  }
}

// One thread per (sequence, chunk); the thread that holds the first chunk of a document walks the
// document's run.  Documents are runs of equal ids in chunk_doc; ids outside 1..n_docs are skipped and counted.
__global__ void reduce_chunks_kernel(const uint32_t* __restrict__ chunk_keys, long long chunk_stride, int n_seq,
                                     int n_chunks, const int32_t* __restrict__ chunk_doc, int n_docs, int mode,
                                     uint32_t min_key, uint32_t* __restrict__ doc_keys, long long table_stride,
                                     int32_t* __restrict__ status) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)n_seq * n_chunks) return;
  const int b = (int)(i / n_chunks), c = (int)(i % n_chunks);
  const int doc = chunk_doc[c];
  if (c > 0 && chunk_doc[c - 1] == doc) return;
  if (doc < 1 || doc > n_docs) {
    if (b == 0 && status) atomicAdd(status + 2, 1);
    return;
  }
  const uint32_t* src = chunk_keys + (long long)b * chunk_stride + 1;
  float sum = 0.f, mx = -INFINITY;
  int n = 0;
  for (int t = c; t < n_chunks && chunk_doc[t] == doc; ++t, ++n) {
    const float v = key_to_float(src[t]);
    sum += v;
    mx = fmaxf(mx, v);
  }
  const float r = mode == MSA_CREDUCE_MEAN ? sum / (float)n : mx;
  const uint32_t key = float_to_key(r);
  // a document cut over several calls (only legal for "max") keeps the larger value
  atomicMax(doc_keys + (long long)b * table_stride + doc, max(key, min_key));
}

}  // namespace msa

using namespace msa;

extern "C" int msa_route_chunk_scores(const void* q, int32_t dtype, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                                      const uint8_t* query_mask, int64_t mask_stride_b, int32_t n_seq, int32_t n_q_heads,
                                      int32_t n_groups, int32_t seq_len, int32_t head_dim, int32_t head_reduce,
                                      int32_t query_reduce, const void* rk, int64_t rk_chunk_stride, int32_t n_chunks,
                                      float scale, float min_val, uint32_t* chunk_keys, int64_t table_stride,
                                      void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "route_chunk_scores: unknown dtype %d", dtype);
  MSA_REQUIRE(n_seq >= 0 && n_q_heads > 0 && n_groups > 0 && n_q_heads % n_groups == 0 && seq_len >= 0 &&
                  head_dim > 0 && head_dim % 4 == 0 && n_chunks >= 0, "route_chunk_scores: bad sizes");
  MSA_REQUIRE(head_reduce == MSA_HREDUCE_MEAN || head_reduce == MSA_HREDUCE_MAX, "route_chunk_scores: unknown head_reduce %d",
              head_reduce);
  MSA_REQUIRE(query_reduce >= MSA_QREDUCE_MAX && query_reduce <= MSA_QREDUCE_LAST,
              "route_chunk_scores: unknown query_reduce %d", query_reduce);
  MSA_REQUIRE(scale > 0.f, "route_chunk_scores: scale must be positive");
  MSA_REQUIRE(table_stride >= (int64_t)n_chunks + 1, "route_chunk_scores: table_stride %lld < n_chunks+1",
              (long long)table_stride);
  MSA_REQUIRE(n_seq <= 65535, "route_chunk_scores: at most 65535 sequences per call");
  if (n_seq == 0 || n_chunks == 0) return MSA_OK;
  MSA_REQUIRE(q && query_mask && rk && chunk_keys, "route_chunk_scores: null pointer");
  const int n_kv = n_q_heads / n_groups;
  MSA_REQUIRE(rk_chunk_stride >= (int64_t)n_kv * head_dim, "route_chunk_scores: rk_chunk_stride is smaller than a key row");
  const size_t smem = (size_t)kCsChunks * n_kv * (head_dim + kCsPad) * sizeof(float);
  MSA_REQUIRE(smem <= 200 * 1024, "route_chunk_scores: %d kv heads x %d need %zu bytes of shared memory", n_kv, head_dim,
              smem);
  const dim3 grid((n_chunks + kCsChunks - 1) / kCsChunks, n_seq);
  const uint32_t min_key = float_to_key(min_val);
  cudaStream_t st = (cudaStream_t)stream;
  static DeviceSmem configured[2] = {};
  if (dtype == MSA_BF16) {
    if (smem > 48 * 1024) MSA_OK_OR_RETURN(ensure_dynamic_smem(chunk_scores_kernel<__nv_bfloat16>, smem, configured[0]));
    chunk_scores_kernel<__nv_bfloat16><<<grid, kCsThreads, smem, st>>>(
        (const __nv_bfloat16*)q, stride_b, stride_h, stride_s, query_mask, mask_stride_b, n_q_heads, n_groups, seq_len,
        head_dim, head_reduce, query_reduce, (const __nv_bfloat16*)rk, rk_chunk_stride, n_chunks, scale, min_key,
        chunk_keys, table_stride);
  } else {
    if (smem > 48 * 1024) MSA_OK_OR_RETURN(ensure_dynamic_smem(chunk_scores_kernel<float>, smem, configured[1]));
    chunk_scores_kernel<float><<<grid, kCsThreads, smem, st>>>(
        (const float*)q, stride_b, stride_h, stride_s, query_mask, mask_stride_b, n_q_heads, n_groups, seq_len, head_dim,
        head_reduce, query_reduce, (const float*)rk, rk_chunk_stride, n_chunks, scale, min_key, chunk_keys,
        table_stride);
  }
  MSA_LAUNCH_OK("chunk_scores_kernel");
  return MSA_OK;
}

extern "C" int msa_route_reduce_chunks(const uint32_t* chunk_keys, int64_t chunk_table_stride, int32_t n_seq,
                                       int32_t n_chunks, const int32_t* chunk_doc, int32_t n_docs, int32_t chunk_reduce,
                                       float min_val, uint32_t* score_keys, int64_t table_stride, int32_t* status,
                                       void* stream) {
  MSA_REQUIRE(chunk_reduce == MSA_CREDUCE_MAX || chunk_reduce == MSA_CREDUCE_MEAN,
              "route_reduce_chunks: unknown chunk_reduce %d", chunk_reduce);
  MSA_REQUIRE(n_seq >= 0 && n_chunks >= 0 && n_docs >= 0, "route_reduce_chunks: bad sizes");
  MSA_REQUIRE(chunk_table_stride >= (int64_t)n_chunks + 1 && table_stride >= (int64_t)n_docs + 1,
              "route_reduce_chunks: table strides are smaller than the tables");
  if (n_seq == 0 || n_chunks == 0) return MSA_OK;
  MSA_REQUIRE(chunk_keys && chunk_doc && score_keys, "route_reduce_chunks: null pointer");
  const long long total = (long long)n_seq * n_chunks;
  reduce_chunks_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      chunk_keys, chunk_table_stride, n_seq, n_chunks, chunk_doc, n_docs, chunk_reduce, float_to_key(min_val), score_keys,
      table_stride, status);
  MSA_LAUNCH_OK("reduce_chunks_kernel");
  return MSA_OK;
}
