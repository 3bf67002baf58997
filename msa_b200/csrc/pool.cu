// Stage-1 chunk-mean pooling (the chunk tables it reads come from bookkeeping.cu).
//
// Pooling is a pure streaming reduction: every document token's [Hkv*D] row is read once
// with 16-byte loads and a chunk's mean is written once, so the kernel is bound by HBM
// bandwidth (algorithmic bytes = T*Hkv*D*e read + C*Hkv*D*e written per tensor).
#include "common.cuh"

namespace msa {

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
