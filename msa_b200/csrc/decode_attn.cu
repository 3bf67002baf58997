// Decode attention over the sparse context: split-KV flash-decode with GQA.
//
// One CTA = one (sequence, kv head, KV split).  The G query heads of the group share every
// K/V tile that is staged in shared memory, so K and V are read from HBM exactly once per
// step: 2*L*Hkv*D*e bytes per sequence, the algorithmic minimum.  Each split keeps an
// online softmax (running max / sum) and writes an unnormalised partial; a second kernel
// merges the splits.  The new token's K/V takes part straight from its own buffer and is
// appended to the cache in place, which replaces the reference's per-step torch.cat.
#include "common.cuh"
#include "decode_mma.cuh"

namespace msa {

constexpr int kDecThreads = 128;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kMaxAcc = 4;  // float4 accumulators per thread: G*D <= 2048

template <typename T> struct DecTile { static constexpr int kKeys = 64; };
template <> struct DecTile<float> { static constexpr int kKeys = 32; };

template <typename T>
__global__ void append_kv_kernel(T* __restrict__ k_cache, T* __restrict__ v_cache, long long stride_b,
                                 long long stride_h, const int32_t* __restrict__ kv_start,
                                 const int32_t* __restrict__ kv_len, const T* __restrict__ new_k,
                                 const T* __restrict__ new_v, int n_kv_heads, int head_dim) {
  const int b = blockIdx.y, h = blockIdx.x;
  const long long pos = (kv_start ? kv_start[b] : 0) + (long long)kv_len[b];
  const long long dst = (long long)b * stride_b + (long long)h * stride_h + pos * head_dim;
  const long long src = ((long long)b * n_kv_heads + h) * head_dim;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    k_cache[dst + d] = new_k[src + d];
    v_cache[dst + d] = new_v[src + d];
  }
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads)
decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                    long long stride_b, long long stride_h, const int32_t* __restrict__ kv_start,
                    const int32_t* __restrict__ kv_len, const T* __restrict__ new_k, const T* __restrict__ new_v,
                    int n_q_heads, int n_kv_heads, int head_dim, float scale_log2e, T* __restrict__ out,
                    float* __restrict__ ws, int n_splits) {
  constexpr int V = Elem<T>::kVec;
  constexpr int KT = DecTile<T>::kKeys;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int G = n_q_heads / n_kv_heads, D = head_dim;
  const int kstride = D + V;  // one 16-byte pad per K row keeps 16-byte smem reads conflict free
  T* s_k = reinterpret_cast<T*>(smem_raw);
  T* s_v = s_k + KT * kstride;
  float* s_q = reinterpret_cast<float*>(s_v + KT * D);  // [G][D], pre-scaled by scale*log2(e)
  float* s_p = s_q + G * D;                             // [G][KT]
  float* s_m = s_p + G * KT;                            // [G] running max
  float* s_l = s_m + G;                                 // [G] running sum
  float* s_f = s_l + G;                                 // [G] rescale factor of this tile

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int cached = kv_len[b];
  const int total = cached + (new_k ? 1 : 0);
  int per = (total + n_splits - 1) / n_splits;
  per = (per + KT - 1) / KT * KT;
  const int p_lo = split * per, p_hi = min(total, p_lo + per);
  const long long base = (long long)b * stride_b + (long long)h * stride_h +
                         (long long)(kv_start ? kv_start[b] : 0) * D;
  const long long new_off = ((long long)b * n_kv_heads + h) * D;

  for (int i = tid; i < G * D; i += kDecThreads)
    s_q[i] = (float)q[((long long)b * n_q_heads + (long long)h * G) * D + i] * scale_log2e;
  for (int g = tid; g < G; g += kDecThreads) { s_m[g] = -INFINITY; s_l[g] = 0.f; }
  float4 acc[kMaxAcc];
#pragma unroll
  for (int a = 0; a < kMaxAcc; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int dvecs = D / 4, n_pairs = G * dvecs;
  __syncthreads();

  for (int p0 = p_lo; p0 < p_hi; p0 += KT) {
    // stage the K and V tile
    const int vec_row = D / V;
    for (int i = tid; i < KT * vec_row; i += kDecThreads) {
      const int key = i / vec_row, dv = (i % vec_row) * V;
      const int p = p0 + key;
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (p < p_hi) {
        if (p < cached) {
          kv = *reinterpret_cast<const uint4*>(k_cache + base + (long long)p * D + dv);
          vv = *reinterpret_cast<const uint4*>(v_cache + base + (long long)p * D + dv);
        } else {
          kv = *reinterpret_cast<const uint4*>(new_k + new_off + dv);
          vv = *reinterpret_cast<const uint4*>(new_v + new_off + dv);
        }
      }
      *reinterpret_cast<uint4*>(s_k + key * kstride + dv) = kv;
      *reinterpret_cast<uint4*>(s_v + key * D + dv) = vv;
    }
    __syncthreads();
    // scores (log2 domain): one (key, head) pair at a time per thread
    for (int pr = tid; pr < KT * G; pr += kDecThreads) {
      const int key = pr % KT, g = pr / KT;
      float s = 0.f;
      const T* kr = s_k + key * kstride;
      const float* qr = s_q + g * D;
      for (int d = 0; d < D; d += V) {
        float kf[V];
        Elem<T>::load(kr + d, kf);
#pragma unroll
        for (int j = 0; j < V; ++j) s = fmaf(kf[j], qr[d + j], s);
      }
      s_p[g * KT + key] = (p0 + key < p_hi) ? s : -INFINITY;
    }
    __syncthreads();
    // online softmax: warp w owns heads w, w+4, ...
    for (int g = warp; g < G; g += kDecWarps) {
      float mx = -INFINITY;
      for (int key = lane; key < KT; key += 32) mx = fmaxf(mx, s_p[g * KT + key]);
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = s_m[g], m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int key = lane; key < KT; key += 32) {
        const float e = exp2f(s_p[g * KT + key] - m_new);  // tile is never empty, m_new is finite
        s_p[g * KT + key] = e;
        sum += e;
      }
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        const float f = exp2f(m_old - m_new);  // 0 on the first tile (m_old = -inf)
        s_f[g] = f;
        s_m[g] = m_new;
        s_l[g] = s_l[g] * f + sum;
      }
    }
    __syncthreads();
    // P.V: thread owns (head, 4 dims)
#pragma unroll
    for (int a = 0; a < kMaxAcc; ++a) {
      const int pr = tid + a * kDecThreads;
      if (pr < n_pairs) {
        const int g = pr / dvecs, d = (pr % dvecs) * 4;
        const float f = s_f[g];
        float4 r = acc[a];
        r.x *= f; r.y *= f; r.z *= f; r.w *= f;
        const float* pp = s_p + g * KT;
        for (int key = 0; key < KT; ++key) {
          const float w = pp[key];
          const T* vr = s_v + key * D + d;
          r.x = fmaf(w, (float)vr[0], r.x);
          r.y = fmaf(w, (float)vr[1], r.y);
          r.z = fmaf(w, (float)vr[2], r.z);
          r.w = fmaf(w, (float)vr[3], r.w);
        }
        acc[a] = r;
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int a = 0; a < kMaxAcc; ++a) {
    const int pr = tid + a * kDecThreads;
    if (pr < n_pairs) {
      const int g = pr / dvecs, d = (pr % dvecs) * 4;
      const int hq = h * G + g;
      if (n_splits == 1) {
        const float inv = s_l[g] > 0.f ? 1.f / s_l[g] : 0.f;
        T* o = out + ((long long)b * n_q_heads + hq) * D + d;
        o[0] = (T)(acc[a].x * inv); o[1] = (T)(acc[a].y * inv);
        o[2] = (T)(acc[a].z * inv); o[3] = (T)(acc[a].w * inv);
      } else {
        float* w = ws + (((long long)b * n_q_heads + hq) * n_splits + split) * (D + 2);
        w[d] = acc[a].x; w[d + 1] = acc[a].y; w[d + 2] = acc[a].z; w[d + 3] = acc[a].w;
        if (d == 0) { w[D] = s_m[g]; w[D + 1] = s_l[g]; }
      }
    }
  }
}

template <typename T>
__global__ void decode_combine_kernel(const float* __restrict__ ws, int head_dim, int n_splits,
                                      T* __restrict__ out) {
  const long long bh = blockIdx.x;
  const float* w = ws + bh * n_splits * (head_dim + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, w[s * (head_dim + 2) + head_dim]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = w[s * (head_dim + 2) + head_dim];
    if (ms > -INFINITY) l += w[s * (head_dim + 2) + head_dim + 1] * exp2f(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = w[s * (head_dim + 2) + head_dim];
      if (ms > -INFINITY) a += w[s * (head_dim + 2) + d] * exp2f(ms - m);
    }
    out[bh * head_dim + d] = (T)(a * inv);
  }
}

template <typename T>
int launch_decode(const void* q, void* k_cache, void* v_cache, int64_t stride_b, int64_t stride_h,
                  const int32_t* kv_start, const int32_t* kv_len, const void* new_k, const void* new_v, int n_seq,
                  int n_q_heads, int n_kv_heads, int head_dim, float scale, void* out, void* workspace,
                  int n_splits, cudaStream_t stream) {
  constexpr int KT = DecTile<T>::kKeys;
  constexpr int V = Elem<T>::kVec;
  const int G = n_q_heads / n_kv_heads;
  if (new_k) {
    append_kv_kernel<T><<<dim3(n_kv_heads, n_seq), 128, 0, stream>>>(
        (T*)k_cache, (T*)v_cache, stride_b, stride_h, kv_start, kv_len, (const T*)new_k, (const T*)new_v,
        n_kv_heads, head_dim);
    MSA_LAUNCH_OK("append_kv_kernel");
  }
  const size_t smem = (size_t)KT * (head_dim + V) * sizeof(T) + (size_t)KT * head_dim * sizeof(T) +
                      ((size_t)G * head_dim + (size_t)G * KT + 3 * G) * sizeof(float);
  MSA_REQUIRE(smem <= 200 * 1024, "decode: head_dim/group size need %zu bytes of shared memory", smem);
  static DeviceSmem configured{};
  if (smem > 48 * 1024) MSA_OK_OR_RETURN(ensure_dynamic_smem(decode_split_kernel<T>, smem, configured));
  const float scale_log2e = scale * 1.4426950408889634f;
  decode_split_kernel<T><<<dim3(n_splits, n_kv_heads, n_seq), kDecThreads, smem, stream>>>(
      (const T*)q, (const T*)k_cache, (const T*)v_cache, stride_b, stride_h, kv_start, kv_len, (const T*)new_k,
      (const T*)new_v, n_q_heads, n_kv_heads, head_dim, scale_log2e, (T*)out, (float*)workspace, n_splits);
  MSA_LAUNCH_OK("decode_split_kernel");
  if (n_splits > 1) {
    decode_combine_kernel<T><<<n_seq * n_q_heads, 128, 0, stream>>>((const float*)workspace, head_dim, n_splits,
                                                                    (T*)out);
    MSA_LAUNCH_OK("decode_combine_kernel");
  }
  return MSA_OK;
}

// bf16, head_dim 128, group size <= 8: the tensor-core fragment kernel of decode_mma.cuh.
int launch_decode_mma(const void* q, void* k_cache, void* v_cache, int64_t stride_b, int64_t stride_h,
                      const int32_t* kv_start, const int32_t* kv_len, const void* new_k, const void* new_v, int n_seq,
                      int n_q_heads, int n_kv_heads, float scale, void* out, void* workspace, int n_splits,
                      cudaStream_t stream) {
  using T = __nv_bfloat16;
  if (new_k) {
    append_kv_kernel<T><<<dim3(n_kv_heads, n_seq), 128, 0, stream>>>(
        (T*)k_cache, (T*)v_cache, stride_b, stride_h, kv_start, kv_len, (const T*)new_k, (const T*)new_v,
        n_kv_heads, kMmaD);
    MSA_LAUNCH_OK("append_kv_kernel");
  }
  static DeviceSmem configured{};
  MSA_OK_OR_RETURN(ensure_dynamic_smem(decode_mma_kernel, kMmaSmemBytes, configured));
  decode_mma_kernel<<<dim3(n_splits, n_kv_heads, n_seq), kMmaWarps * 32, kMmaSmemBytes, stream>>>(
      (const T*)q, (const T*)k_cache, (const T*)v_cache, stride_b, stride_h, kv_start, kv_len, (const T*)new_k,
      (const T*)new_v, n_q_heads, n_kv_heads, scale * 1.4426950408889634f, (T*)out, (float*)workspace, n_splits);
  MSA_LAUNCH_OK("decode_mma_kernel");
  if (n_splits > 1) {
    decode_combine_kernel<T><<<n_seq * n_q_heads, 128, 0, stream>>>((const float*)workspace, kMmaD, n_splits, (T*)out);
    MSA_LAUNCH_OK("decode_combine_kernel");
  }
  return MSA_OK;
}

}  // namespace msa

using namespace msa;

extern "C" int64_t msa_decode_workspace_bytes(int32_t n_seq, int32_t n_q_heads, int32_t head_dim,
                                              int32_t n_splits) {
  if (n_splits <= 1) return 0;
  return (int64_t)n_seq * n_q_heads * n_splits * (head_dim + 2) * (int64_t)sizeof(float);
}

extern "C" int msa_sparse_decode_attn(const void* q, int32_t dtype, void* k_cache, void* v_cache, int64_t stride_b,
                                      int64_t stride_h, const int32_t* kv_start, const int32_t* kv_len,
                                      const void* new_k, const void* new_v, int32_t n_seq, int32_t n_q_heads,
                                      int32_t n_kv_heads, int32_t head_dim, float scale, void* out, void* workspace,
                                      int64_t workspace_bytes, int32_t n_splits, void* stream) {
  MSA_REQUIRE(dtype_ok(dtype), "decode: unknown dtype %d", dtype);
  MSA_REQUIRE(q && k_cache && v_cache && kv_len && out, "decode: null pointer");
  MSA_REQUIRE((new_k == nullptr) == (new_v == nullptr), "decode: new_k and new_v must be given together");
  MSA_REQUIRE(n_seq >= 0 && n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0 && head_dim > 0,
              "decode: bad sizes");
  const int vec = 16 / (int)dtype_size(dtype);
  MSA_REQUIRE(head_dim % vec == 0 && head_dim % 4 == 0, "decode: head_dim*sizeof must be a multiple of 16 bytes");
  MSA_REQUIRE((int64_t)(n_q_heads / n_kv_heads) * head_dim <= (int64_t)kMaxAcc * kDecThreads * 4,
              "decode: group_size*head_dim must be <= %d", kMaxAcc * kDecThreads * 4);
  MSA_REQUIRE(stride_b % vec == 0 && stride_h % vec == 0 && aligned16(q) && aligned16(k_cache) &&
                  aligned16(v_cache) && aligned16(out) && (!new_k || (aligned16(new_k) && aligned16(new_v))),
              "decode: pointers and strides must keep 16-byte alignment");
  MSA_REQUIRE(n_splits >= 1 && n_splits <= 65535, "decode: n_splits out of range");
  MSA_REQUIRE(n_splits == 1 || (workspace && workspace_bytes >= msa_decode_workspace_bytes(n_seq, n_q_heads,
                                                                                         head_dim, n_splits)),
              "decode: workspace too small for %d splits", n_splits);
  if (n_seq == 0) return MSA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MSA_BF16 && head_dim == kMmaD && n_q_heads / n_kv_heads <= 8)
    return launch_decode_mma(q, k_cache, v_cache, stride_b, stride_h, kv_start, kv_len, new_k, new_v, n_seq, n_q_heads,
                             n_kv_heads, scale, out, workspace, n_splits, st);
  return dtype == MSA_BF16
             ? launch_decode<__nv_bfloat16>(q, k_cache, v_cache, stride_b, stride_h, kv_start, kv_len, new_k, new_v,
                                            n_seq, n_q_heads, n_kv_heads, head_dim, scale, out, workspace, n_splits, st)
             : launch_decode<float>(q, k_cache, v_cache, stride_b, stride_h, kv_start, kv_len, new_k, new_v, n_seq,
                                    n_q_heads, n_kv_heads, head_dim, scale, out, workspace, n_splits, st);
}

// ---------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where a decode step runs:
// a serving loop whose memory pool has already claimed the whole GPU, a plugin that is only
// handed input and output buffers by its framework, or code running under a policy that
// forbids allocation after start-up.  For them the split-KV partials live in the fixed array
// below instead of a caller-provided workspace.  The array is part of the library image, so
// every GPU that loads the library holds kStaticScratchFloats*4 bytes (8 MiB) until exit.
// ---------------------------------------------------------------------------------------
namespace msa {
constexpr long long kStaticScratchFloats = 2ll * 1024 * 1024;  // 8 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];
static float* g_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace msa

extern "C" int64_t msa_decode_static_scratch_bytes(void) { return msa::kStaticScratchFloats * (int64_t)sizeof(float); }

extern "C" int msa_sparse_decode_attn_static(const void* q, int32_t dtype, void* k_cache, void* v_cache,
                                             int64_t stride_b, int64_t stride_h, const int32_t* kv_start,
                                             const int32_t* kv_len, const void* new_k, const void* new_v,
                                             int32_t n_seq, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                                             float scale, void* out, int32_t n_splits, void* stream) {
  MSA_REQUIRE(n_seq >= 0 && n_q_heads > 0 && head_dim > 0 && n_splits >= 1, "decode (static scratch): bad sizes");
  const int64_t need = msa_decode_workspace_bytes(n_seq, n_q_heads, head_dim, n_splits);
  MSA_REQUIRE(need <= msa_decode_static_scratch_bytes(),
              "decode (static scratch): n_seq*n_q_heads*n_splits*(head_dim+2)*4 = %lld bytes exceeds the built-in "
              "%lld-byte scratch; use fewer splits or msa_sparse_decode_attn with your own workspace",
              (long long)need, (long long)msa_decode_static_scratch_bytes());
  int dev = -1;
  MSA_OK_OR_RETURN(current_device(&dev));
  if (g_scratch_addr[dev] == nullptr) {
    // First call on this device: resolve the array's address on the CURRENT device.  The symbol
    // name is only a host-side handle; the kernel must be given the address obtained here.
    float* p = nullptr;
    MSA_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_decode_scratch));
    MSA_REQUIRE(p != nullptr, "decode (static scratch): could not resolve the scratch array");
    g_scratch_addr[dev] = p;
  }
  return msa_sparse_decode_attn(q, dtype, k_cache, v_cache, stride_b, stride_h, kv_start, kv_len, new_k, new_v, n_seq,
                                n_q_heads, n_kv_heads, head_dim, scale, out, g_scratch_addr[dev], need, n_splits,
                                stream);
}
