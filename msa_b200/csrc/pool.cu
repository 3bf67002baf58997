// Stage-1 chunk bookkeeping and chunk-mean pooling.
//
// Pooling is a pure streaming reduction: every document token's [Hkv*D] row is read once
// with 16-byte loads and a chunk's mean is written once, so the kernel is bound by HBM
// bandwidth (algorithmic bytes = T*Hkv*D*e read + C*Hkv*D*e written per tensor).
#include "common.cuh"

namespace msa {

// ---------------------------------------------------------------------------------------
// Bookkeeping: one CTA walks the doc_ids of a block in three scan phases.
// ---------------------------------------------------------------------------------------
constexpr int kBkThreads = 1024;

template <typename T, typename Op>
__device__ inline T block_exclusive_scan(T v, T identity, Op op, T* smem, T* total) {
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

struct LastGid {  // right-biased "last document token seen"
  long long gid;
  int has;
};

__global__ void __launch_bounds__(kBkThreads)
bookkeeping_kernel(const int64_t* __restrict__ doc_ids, const int64_t* __restrict__ attn, int n_rows,
                   int row_len, int P, int32_t* __restrict__ token_index,
                   int32_t* __restrict__ chunk_offsets, int64_t* __restrict__ pooled_doc_ids,
                   int max_chunks, int32_t* __restrict__ counts) {
  __shared__ long long s_ll[kBkThreads];
  __shared__ int s_int[kBkThreads];
  __shared__ LastGid s_gid[kBkThreads];
  const long long n = (long long)n_rows * row_len;
  const long long seg = (n + kBkThreads - 1) / kBkThreads;
  const long long lo = min(n, seg * threadIdx.x), hi = min(n, lo + seg);
  auto is_doc = [&](long long i) { return doc_ids[i] > 0 && (attn == nullptr || attn[i] == 1); };
  auto gid_of = [&](long long i) { return (long long)(i / row_len) * (1ll << 40) + doc_ids[i]; };

  // phase 1: compact index of every document token, and the last document token before it
  int cnt = 0;
  LastGid last{0, 0};
  for (long long i = lo; i < hi; ++i)
    if (is_doc(i)) { ++cnt; last = LastGid{gid_of(i), 1}; }
  int total_tokens;
  int ci0 = block_exclusive_scan<int>(cnt, 0, [](int a, int b) { return a + b; }, s_int, &total_tokens);
  LastGid prev0 = block_exclusive_scan<LastGid>(
      last, LastGid{0, 0}, [](LastGid a, LastGid b) { return b.has ? b : a; }, s_gid, nullptr);

  // phase 2: compact index at which the current document started
  long long ds_local = -1;
  {
    int ci = ci0;
    LastGid prev = prev0;
    for (long long i = lo; i < hi; ++i)
      if (is_doc(i)) {
        long long g = gid_of(i);
        if (!prev.has || prev.gid != g) ds_local = ci;
        prev = LastGid{g, 1};
        ++ci;
      }
  }
  long long ds0 = block_exclusive_scan<long long>(
      ds_local, -1ll, [](long long a, long long b) { return a > b ? a : b; }, s_ll, nullptr);

  // phase 3: chunk starts
  int nchunk_local = 0;
  {
    int ci = ci0;
    LastGid prev = prev0;
    long long ds = ds0;
    for (long long i = lo; i < hi; ++i)
      if (is_doc(i)) {
        long long g = gid_of(i);
        if (!prev.has || prev.gid != g) ds = ci;
        prev = LastGid{g, 1};
        if ((ci - ds) % P == 0) ++nchunk_local;
        ++ci;
      }
  }
  int total_chunks;
  int ch0 = block_exclusive_scan<int>(nchunk_local, 0, [](int a, int b) { return a + b; }, s_int,
                                      &total_chunks);
  {
    int ci = ci0, ch = ch0;
    LastGid prev = prev0;
    long long ds = ds0;
    for (long long i = lo; i < hi; ++i)
      if (is_doc(i)) {
        long long g = gid_of(i);
        if (!prev.has || prev.gid != g) ds = ci;
        prev = LastGid{g, 1};
        token_index[ci] = (int32_t)i;
        if ((ci - ds) % P == 0) {
          if (ch < max_chunks) {
            chunk_offsets[ch] = ci;
            pooled_doc_ids[ch] = doc_ids[i];
          }
          ++ch;
        }
        ++ci;
      }
  }
  if (threadIdx.x == 0) {
    const bool overflow = total_chunks > max_chunks;
    chunk_offsets[overflow ? max_chunks : total_chunks] = total_tokens;
    counts[0] = total_tokens;
    counts[1] = overflow ? max_chunks : total_chunks;
    counts[2] = overflow ? 1 : 0;
  }
}

// ---------------------------------------------------------------------------------------
// Pooling: one CTA per chunk, 256 threads, each thread owns one 16-byte column of the row.
// ---------------------------------------------------------------------------------------
constexpr int kPoolThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kPoolThreads)
pool_kernel(const T* __restrict__ states, long long token_stride, long long head_stride,
            const int32_t* __restrict__ token_index, const int32_t* __restrict__ chunk_offsets,
            const int32_t* __restrict__ n_chunks_dev, int n_chunks, int head_dim, int vpr,
            T* __restrict__ out, long long out_chunk_stride, long long out_head_stride,
            int normalize) {
  constexpr int V = Elem<T>::kVec;
  __shared__ float s_part[kPoolThreads][V];
  const int live = n_chunks_dev ? min(n_chunks, *n_chunks_dev) : n_chunks;
  const int rows_par = kPoolThreads / vpr;
  const int col = threadIdx.x % vpr, sub = threadIdx.x / vpr;
  const int h = (col * V) / head_dim, d = (col * V) % head_dim;
  const long long col_off = (long long)h * head_stride + d;
  const int lanes_per_head = head_dim / V;

  for (int c = blockIdx.x; c < live; c += gridDim.x) {
    const int t0 = chunk_offsets[c], t1 = chunk_offsets[c + 1];
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    int i = t0 + sub;
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * rows_par < t1; i += 4 * rows_par) {
      float v[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long row = token_index ? token_index[i + u * rows_par] : (i + u * rows_par);
        Elem<T>::load(states + row * token_stride + col_off, v[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += v[u][j];
    }
    for (; i < t1; i += rows_par) {
      float v[V];
      const long long row = token_index ? token_index[i] : i;
      Elem<T>::load(states + row * token_stride + col_off, v);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += v[j];
    }
    if (rows_par > 1) {
#pragma unroll
      for (int j = 0; j < V; ++j) s_part[threadIdx.x][j] = acc[j];
      __syncthreads();
      if (sub == 0)
        for (int s = 1; s < rows_par; ++s)
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += s_part[s * vpr + col][j];
    }
    const float inv_n = 1.f / (float)max(t1 - t0, 1);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      acc[j] = Elem<T>::round(acc[j] * inv_n);
      ss += acc[j] * acc[j];
    }
    if (normalize) {  // executed by whole warps; a head's lanes are an aligned power-of-two group
      for (int o = lanes_per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] *= inv;
    }
    if (sub == 0) Elem<T>::store(out + (long long)c * out_chunk_stride + (long long)h * out_head_stride + d, acc);
    if (rows_par > 1) __syncthreads();
  }
}

}  // namespace msa

using namespace msa;

extern "C" int msa_chunk_bookkeeping(const int64_t* doc_ids, const int64_t* attention_mask, int32_t n_rows,
                                     int32_t row_len, int32_t pooling_kernel_size, int32_t* token_index,
                                     int32_t* chunk_offsets, int64_t* pooled_doc_ids, int32_t max_chunks,
                                     int32_t* counts, void* stream) {
  MSA_REQUIRE(doc_ids && token_index && chunk_offsets && pooled_doc_ids && counts, "bookkeeping: null pointer");
  MSA_REQUIRE(n_rows >= 0 && row_len >= 0 && (int64_t)n_rows * row_len < (1ll << 31), "bookkeeping: bad sizes");
  MSA_REQUIRE(pooling_kernel_size > 0 && max_chunks >= 0, "bookkeeping: pooling_kernel_size must be > 0");
  bookkeeping_kernel<<<1, kBkThreads, 0, (cudaStream_t)stream>>>(doc_ids, attention_mask, n_rows, row_len,
                                                                 pooling_kernel_size, token_index, chunk_offsets,
                                                                 pooled_doc_ids, max_chunks, counts);
  MSA_LAUNCH_OK("bookkeeping_kernel");
  return MSA_OK;
}

extern "C" int msa_pool_chunks(const void* states, int32_t dtype, int64_t token_stride, int64_t head_stride,
                               const int32_t* token_index, const int32_t* chunk_offsets,
                               const int32_t* n_chunks_dev, int32_t n_chunks, int32_t n_heads, int32_t head_dim,
                               void* out, int64_t out_chunk_stride, int64_t out_head_stride,
                               int32_t l2_normalize, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "pool: unknown dtype %d", dtype);
  MSA_REQUIRE(states && chunk_offsets && out, "pool: null pointer");
  MSA_REQUIRE(n_chunks >= 0 && n_heads > 0 && head_dim > 0, "pool: bad sizes");
  const int vec = 16 / (int)dtype_size(dtype);
  MSA_REQUIRE(head_dim % vec == 0, "pool: head_dim*sizeof must be a multiple of 16 bytes");
  const int vpr = n_heads * head_dim / vec, lph = head_dim / vec;
  MSA_REQUIRE(vpr <= kPoolThreads && kPoolThreads % vpr == 0,
              "pool: n_heads*head_dim*sizeof/16 = %d must divide %d", vpr, kPoolThreads);
  MSA_REQUIRE(lph <= 32 && (lph & (lph - 1)) == 0, "pool: head_dim*sizeof/16 must be a power of two <= 32");
  MSA_REQUIRE(aligned16(states) && aligned16(out), "pool: pointers must be 16-byte aligned");
  MSA_REQUIRE(token_stride % vec == 0 && head_stride % vec == 0 && out_chunk_stride % vec == 0 &&
                  out_head_stride % vec == 0, "pool: strides must keep 16-byte alignment");
  if (n_chunks == 0) return MSA_OK;
  const int grid = n_chunks < 148 * 64 ? n_chunks : 148 * 64;
  if (dtype == MSA_BF16)
    pool_kernel<__nv_bfloat16><<<grid, kPoolThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)states, token_stride, head_stride, token_index, chunk_offsets, n_chunks_dev,
        n_chunks, head_dim, vpr, (__nv_bfloat16*)out, out_chunk_stride, out_head_stride, l2_normalize);
  else
    pool_kernel<float><<<grid, kPoolThreads, 0, (cudaStream_t)stream>>>(
        (const float*)states, token_stride, head_stride, token_index, chunk_offsets, n_chunks_dev, n_chunks,
        head_dim, vpr, (float*)out, out_chunk_stride, out_head_stride, l2_normalize);
  MSA_LAUNCH_OK("pool_kernel");
  return MSA_OK;
}
