// Routing on CUDA cores: query-head folding, score-table reset, and the fp32 scoring kernel.
//
// The fp32 kernel is the product path for fp32 banks (the reference's CPU-runnable
// configuration) and a cross-check for the tensor-core kernel; bf16 banks are scored by
// route_tc.cu.
#include "common.cuh"
#include "route.cuh"

namespace msa {

// ---------------------------------------------------------------------------------------
// fold: folded[b, s, h, :] = sum_g q[b, h*G+g, s, :]   (optionally L2-normalised per head)
// One CTA per output row; thread = (kv head, 16-byte column of D).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void fold_kernel(const T* __restrict__ q, long long stride_b, long long stride_h, long long stride_s,
                            const uint8_t* __restrict__ mask, long long mask_stride_b, int n_groups, int seq_len,
                            int head_dim, int n_kv, int normalize, int query_reduce, int s_pad, T* __restrict__ folded,
                            float* __restrict__ row_bias) {
  constexpr int V = Elem<T>::kVec;
  grid_launch_dependents();      // a routing kernel launched as a programmatic dependent may set itself up beside this one
  const int lph = head_dim / V;  // lanes per head (power of two <= 32)
  // the CTA is padded to whole warps; surplus threads shadow head 0 and store nothing
  const bool live = (int)threadIdx.x < n_kv * lph;
  const int h = live ? threadIdx.x / lph : 0, d = (threadIdx.x % lph) * V;
  const int row = blockIdx.x;
  const int b = row / s_pad, s = row % s_pad;
  const uint8_t* m = mask + (long long)b * mask_stride_b;
  T* dst = folded + (long long)row * n_kv * head_dim + h * head_dim + d;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;

  auto add_token = [&](int tok) {
    for (int g = 0; g < n_groups; ++g) {
      float v[V];
      Elem<T>::load(q + (long long)b * stride_b + (long long)(h * n_groups + g) * stride_h +
                        (long long)tok * stride_s + d, v);
      if (normalize) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) ss += v[j] * v[j];
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = Elem<T>::round(v[j] * inv);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += v[j];
    }
  };

  float bias = 0.f;
  if (query_reduce == MSA_QREDUCE_MAX) {
    if (s < seq_len) {
      add_token(s);
      if (!m[s]) bias = -INFINITY;
    } else {
      bias = -INFINITY;
    }
  } else {
    int count = 0;
    for (int t = 0; t < seq_len; ++t) count += m[t] ? 1 : 0;
    if (query_reduce == MSA_QREDUCE_MEAN) {
      for (int t = 0; t < seq_len; ++t)
        if (m[t]) add_token(t);  // uniform branch: every thread of the CTA sees the same mask
      const float inv = 1.f / (float)max(count, 1);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] *= inv;
    } else {  // LAST: the reference indexes token (count - 1), clamped at 0
      const int t = max(count - 1, 0);
      if (seq_len > 0) {
        add_token(t);
        if (!m[t]) bias = -INFINITY;
      } else {
        bias = -INFINITY;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = Elem<T>::round(acc[j]);
  if (live) Elem<T>::store(dst, acc);
  if (threadIdx.x == 0) row_bias[row] = bias;
}

__global__ void fill_keys_kernel(uint32_t* __restrict__ keys, long long table_stride, int n_cols, int n_seq,
                                 uint32_t value) {
  const long long total = (long long)n_seq * n_cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    keys[(i / n_cols) * table_stride + (i % n_cols)] = value;
}

int reset_score_table(uint32_t* keys, int64_t table_stride, int32_t n_cols, int32_t n_seq, float min_val,
                      cudaStream_t stream) {
  const long long total = (long long)n_seq * n_cols;
  if (total == 0) return MSA_OK;
  const int grid = (int)((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
  fill_keys_kernel<<<grid, 256, 0, stream>>>(keys, table_stride, n_cols, n_seq, float_to_key(min_val));
  MSA_LAUNCH_OK("fill_keys_kernel");
  return MSA_OK;
}

// ---------------------------------------------------------------------------------------
// CUDA-core scoring: 64 chunks x 64 query rows per CTA, 4x4 per thread, fp32 FMA.
// ---------------------------------------------------------------------------------------
constexpr int kTile = 64, kStepK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
route_simt_kernel(const T* __restrict__ qf, const float* __restrict__ row_bias, int n_rows, int s_pad,
                  const T* __restrict__ rk, long long rk_stride, int n_chunks, int kdim,
                  const int32_t* __restrict__ chunk_doc, int n_docs, float alpha, uint32_t* __restrict__ keys,
                  long long table_stride, int32_t* __restrict__ status) {
  __shared__ float s_a[kStepK][kTile + 4];  // chunks
  __shared__ float s_b[kStepK][kTile + 4];  // query rows
  __shared__ float s_c[kTile][kTile + 1];   // [row][chunk]
  const int c0 = blockIdx.x * kTile, r0 = blockIdx.y * kTile;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;  // loader: 64 rows x 16 k, 4 elements each
  for (int k0 = 0; k0 < kdim; k0 += kStepK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + lk + e;
      float a = 0.f, b = 0.f;
      if (kk < kdim) {
        if (c0 + lr < n_chunks) a = (float)rk[(long long)(c0 + lr) * rk_stride + kk];
        if (r0 + lr < n_rows) b = (float)qf[(long long)(r0 + lr) * kdim + kk];
      }
      s_a[lk + e][lr] = a;
      s_b[lk + e][lr] = b;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kStepK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = s_a[k][tx * 4 + i]; b[i] = s_b[k][ty * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = r0 + ty * 4 + j;
    const float bias = r < n_rows ? row_bias[r] : -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) s_c[ty * 4 + j][tx * 4 + i] = acc[i][j] + bias;
  }
  __syncthreads();
  // (chunk, sequence) pairs of this tile: max over the sequence's rows, then chunk -> doc max
  const int rows_here = min(kTile, n_rows - r0);
  const int seq_first = r0 / s_pad, seq_last = (r0 + rows_here - 1) / s_pad;
  const int n_seq_tile = seq_last - seq_first + 1;
  for (int item = threadIdx.x; item < kTile * n_seq_tile; item += blockDim.x) {
    const int cc = item % kTile, sq = seq_first + item / kTile;
    if (c0 + cc >= n_chunks) continue;
    const int ra = max(sq * s_pad, r0) - r0, rb = min((sq + 1) * s_pad, r0 + rows_here) - r0;
    float m = -INFINITY;
    for (int r = ra; r < rb; ++r) m = fmaxf(m, s_c[r][cc]);
    const int doc = chunk_doc[c0 + cc];
    if (doc < 1 || doc > n_docs) {   // an id outside the table: counted, never used as a column
      atomicAdd(status + 2, 1);
      continue;
    }
    atomicMax(keys + (long long)sq * table_stride + doc, float_to_key(m * alpha));
  }
}

template <typename T>
int launch_route_simt_t(const void* qf, const float* row_bias, int n_seq, int s_pad, const void* rk,
                        int64_t rk_stride, int n_chunks, int kdim, const int32_t* chunk_doc, int n_docs, float alpha,
                        uint32_t* keys, int64_t table_stride, int32_t* status, cudaStream_t stream) {
  const int n_rows = n_seq * s_pad;
  if (n_rows == 0 || n_chunks == 0) return MSA_OK;
  dim3 grid((n_chunks + kTile - 1) / kTile, (n_rows + kTile - 1) / kTile);
  MSA_REQUIRE(grid.y <= 65535, "route (CUDA-core path): too many query rows (%d)", n_rows);
  route_simt_kernel<T><<<grid, 256, 0, stream>>>((const T*)qf, row_bias, n_rows, s_pad, (const T*)rk, rk_stride,
                                                 n_chunks, kdim, chunk_doc, n_docs, alpha, keys, table_stride, status);
  MSA_LAUNCH_OK("route_simt_kernel");
  return MSA_OK;
}

int launch_route_simt(int32_t dtype, const void* qf, const float* row_bias, int n_seq, int s_pad, const void* rk,
                      int64_t rk_stride, int n_chunks, int kdim, const int32_t* chunk_doc, int n_docs, float alpha,
                      uint32_t* keys, int64_t table_stride, int32_t* status, cudaStream_t stream) {
  return dtype == MSA_BF16
             ? launch_route_simt_t<__nv_bfloat16>(qf, row_bias, n_seq, s_pad, rk, rk_stride, n_chunks, kdim,
                                                  chunk_doc, n_docs, alpha, keys, table_stride, status, stream)
             : launch_route_simt_t<float>(qf, row_bias, n_seq, s_pad, rk, rk_stride, n_chunks, kdim, chunk_doc,
                                          n_docs, alpha, keys, table_stride, status, stream);
}

}  // namespace msa

using namespace msa;

// Row-major router keys -> the tile-blocked layout (see tc_common.cuh): one 16-byte vector per thread.
__global__ void block_keys_kernel(const uint4* __restrict__ rows, long long row_stride_vec, long long first_chunk,
                                  long long n_rows, int kdim, uint4* __restrict__ blocked) {
  const int vec_row = kdim / 8, k_blocks = kdim / 64;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n_rows * vec_row) return;
  const long long r = i / vec_row, c = first_chunk + r;
  const int v = (int)(i % vec_row), kb = v / 8, in_kb = v % 8;
  const long long dst = (((c / 128) * k_blocks + kb) * 128 + (c % 128)) * 8 + in_kb;
  blocked[dst] = rows[r * row_stride_vec + v];
}

extern "C" int64_t msa_router_keys_blocked_bytes(int32_t n_chunks, int32_t kdim) {
  if (n_chunks < 0 || kdim <= 0 || kdim % 64 != 0) return -1;
  return (int64_t)((n_chunks + 127) / 128) * 128 * kdim * 2;
}

extern "C" int msa_router_keys_block(const void* rk_rows, int64_t rk_chunk_stride, int32_t first_chunk, int32_t n_rows,
                                     int32_t kdim, void* rk_blocked, void* stream) {
  MSA_REQUIRE(first_chunk >= 0 && n_rows >= 0 && kdim > 0 && kdim % 64 == 0, "router_keys_block: bad sizes (kdim %% 64 == 0)");
  if (n_rows == 0) return MSA_OK;
  MSA_REQUIRE(rk_rows && rk_blocked && aligned16(rk_rows) && aligned16(rk_blocked) && rk_chunk_stride % 8 == 0 &&
                  rk_chunk_stride >= kdim, "router_keys_block: rows must be 16-byte aligned");
  const long long total = (long long)n_rows * (kdim / 8);
  block_keys_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)rk_rows, rk_chunk_stride / 8, first_chunk, n_rows, kdim, (uint4*)rk_blocked);
  MSA_LAUNCH_OK("block_keys_kernel");
  return MSA_OK;
}

extern "C" int32_t msa_route_s_pad(int32_t seq_len, int32_t query_reduce) {
  if (query_reduce != MSA_QREDUCE_MAX || seq_len <= 1) return 1;
  const int s16 = (seq_len + 15) / 16 * 16;
  if (s16 <= kRouteMaxN) return s16;
  // longer queries are cut into equal column tiles of at most kRouteMaxN rows
  const int nt = (seq_len + kRouteMaxN - 1) / kRouteMaxN;
  const int per = ((seq_len + nt - 1) / nt + 15) / 16 * 16;
  return per * nt;
}

extern "C" int msa_fold_queries(const void* q, int32_t dtype, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                                const uint8_t* query_mask, int64_t mask_stride_b, int32_t n_seq, int32_t n_q_heads,
                                int32_t n_groups, int32_t seq_len, int32_t head_dim, int32_t l2_normalize,
                                int32_t query_reduce, int32_t s_pad, void* q_folded, float* row_bias,
                                void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "fold: unknown dtype %d", dtype);
  MSA_REQUIRE(q && query_mask && q_folded && row_bias, "fold: null pointer");
  MSA_REQUIRE(n_seq >= 0 && n_q_heads > 0 && n_groups > 0 && n_q_heads % n_groups == 0 && seq_len >= 0 &&
                  head_dim > 0, "fold: bad sizes");
  MSA_REQUIRE(query_reduce >= MSA_QREDUCE_MAX && query_reduce <= MSA_QREDUCE_LAST, "fold: unknown query_reduce %d",
              query_reduce);
  MSA_REQUIRE(query_reduce == MSA_QREDUCE_MAX ? s_pad >= seq_len && s_pad >= 1 : s_pad == 1,
              "fold: s_pad=%d does not fit seq_len=%d for this query_reduce", s_pad, seq_len);
  const int vec = 16 / (int)dtype_size(dtype);
  const int lph = head_dim / vec, n_kv = n_q_heads / n_groups;
  MSA_REQUIRE(head_dim % vec == 0 && lph <= 32 && (lph & (lph - 1)) == 0,
              "fold: head_dim*sizeof/16 must be a power of two <= 32");
  MSA_REQUIRE(n_kv * lph <= 1024, "fold: too many kv heads");
  MSA_REQUIRE(aligned16(q) && aligned16(q_folded) && stride_b % vec == 0 && stride_h % vec == 0 &&
                  stride_s % vec == 0, "fold: q rows must be 16-byte aligned");
  if (n_seq == 0) return MSA_OK;
  const int rows = n_seq * s_pad;
  const int threads = (n_kv * lph + 31) / 32 * 32;
  if (dtype == MSA_BF16)
    fold_kernel<__nv_bfloat16><<<rows, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, stride_b, stride_h, stride_s, query_mask, mask_stride_b, n_groups, seq_len,
        head_dim, n_kv, l2_normalize, query_reduce, s_pad, (__nv_bfloat16*)q_folded, row_bias);
  else
    fold_kernel<float><<<rows, threads, 0, (cudaStream_t)stream>>>(
        (const float*)q, stride_b, stride_h, stride_s, query_mask, mask_stride_b, n_groups, seq_len, head_dim,
        n_kv, l2_normalize, query_reduce, s_pad, (float*)q_folded, row_bias);
  MSA_LAUNCH_OK("fold_kernel");
  return MSA_OK;
}

extern "C" int msa_route_table_reset(uint32_t* score_keys, int64_t table_stride, int32_t n_docs, int32_t n_seq,
                                     float min_val, int32_t* status, void* stream) {
  MSA_REQUIRE(score_keys && n_docs >= 0 && n_seq >= 0 && table_stride >= (int64_t)n_docs + 1,
              "route_table_reset: bad arguments");
  int rc = reset_score_table(score_keys, table_stride, n_docs + 1, n_seq, min_val, (cudaStream_t)stream);
  if (rc != MSA_OK) return rc;
  if (status) MSA_CUDA_OK(cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), (cudaStream_t)stream));
  return MSA_OK;
}

extern "C" int msa_route_scores(const void* q_folded, const float* row_bias, int32_t dtype, int32_t n_seq,
                                int32_t s_pad, const void* rk, int64_t rk_chunk_stride, int32_t n_chunks,
                                int32_t kdim, const int32_t* chunk_doc, float alpha, uint32_t* score_keys,
                                int64_t table_stride, int32_t n_docs, float min_val, uint32_t flags,
                                int32_t* status, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "route: unknown dtype %d", dtype);
  MSA_REQUIRE(score_keys && status, "route: null pointer");
  MSA_REQUIRE(n_seq >= 0 && s_pad >= 1 && n_chunks >= 0 && kdim > 0 && n_docs >= 0, "route: bad sizes");
  MSA_REQUIRE(table_stride >= (int64_t)n_docs + 1, "route: table_stride %lld < n_docs+1", (long long)table_stride);
  MSA_REQUIRE(alpha > 0.f, "route: alpha must be positive (it is applied after the max)");
  MSA_REQUIRE(n_seq == 0 || n_chunks == 0 || (q_folded && row_bias && rk && chunk_doc), "route: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (!(flags & MSA_ROUTE_NO_INIT)) {
    int rc = reset_score_table(score_keys, table_stride, n_docs + 1, n_seq, min_val, st);
    if (rc != MSA_OK) return rc;
    MSA_CUDA_OK(cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), st));
  }
  if (n_seq == 0 || n_chunks == 0) return MSA_OK;
  const bool blocked = (flags & MSA_ROUTE_KEYS_BLOCKED) != 0;
  MSA_REQUIRE(!blocked || (dtype == MSA_BF16 && !(flags & MSA_ROUTE_FORCE_SIMT) && kdim % 64 == 0),
              "route: tile-blocked router keys are read by the tensor-core kernel only (bf16, kdim %% 64 == 0)");
  if (dtype == MSA_BF16 && !(flags & MSA_ROUTE_FORCE_SIMT))
    return launch_route_tc(q_folded, row_bias, n_seq, s_pad, rk, rk_chunk_stride, n_chunks, kdim, chunk_doc, n_docs,
                           alpha, min_val, score_keys, table_stride, status, blocked, st);
  return launch_route_simt(dtype, q_folded, row_bias, n_seq, s_pad, rk, rk_chunk_stride, n_chunks, kdim, chunk_doc,
                           n_docs, alpha, score_keys, table_stride, status, st);
}
