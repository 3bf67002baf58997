// Small fused kernels for the dense algebra between the GEMMs of a decode step (bf16).
//
// A decode step is launch bound between its weight-streaming GEMMs: per layer the reference's modules
// (Qwen3RMSNorm, apply_rotary_pos_emb, residual adds, SiLU * up; transformers' modeling_qwen3 as used by
// src/msa/model.py:67-135) issue some twenty elementwise kernels over a few KB each.  These three kernels
// replace them; each computes in fp32 and rounds once.
#include "common.cuh"

namespace msa {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per (sequence, head) of the fused projection output row [q heads | k heads | v heads | ...]:
// RMS-normalise the head (weight w), rotate by the sequence's cos / sin (rotate-half convention),
// write to q_out / k_out.  head_dim = 128: lane l holds dims 4l .. 4l+3, its rotation partner is lane l ^ 16.
__global__ void __launch_bounds__(128)
qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride, int n_seq, int n_q_heads,
                    int n_kv_heads, const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
                    float eps, const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int heads = n_q_heads + n_kv_heads;
  if (warp >= n_seq * heads) return;
  const int b = warp / heads, h = warp % heads;
  const bool is_q = h < n_q_heads;
  const __nv_bfloat16* src = qkv + (long long)b * row_stride + (long long)h * 128 + lane * 4;
  const __nv_bfloat16* w = (is_q ? q_w : k_w) + lane * 4;
  float x[4], wv[4], c[4], s[4];
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const uint2 wr = *reinterpret_cast<const uint2*>(w);
    const uint2 cr = *reinterpret_cast<const uint2*>(cos_t + (long long)b * 128 + lane * 4);
    const uint2 sr = *reinterpret_cast<const uint2*>(sin_t + (long long)b * 128 + lane * 4);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wr);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&cr);
    const __nv_bfloat162* ps = reinterpret_cast<const __nv_bfloat162*>(&sr);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float2 f = __bfloat1622float2(p[i]);  x[2 * i] = f.x;  x[2 * i + 1] = f.y;
      f = __bfloat1622float2(pw[i]);        wv[2 * i] = f.x; wv[2 * i + 1] = f.y;
      f = __bfloat1622float2(pc[i]);        c[2 * i] = f.x;  c[2 * i + 1] = f.y;
      f = __bfloat1622float2(ps[i]);        s[2 * i] = f.x;  s[2 * i + 1] = f.y;
    }
  }
  const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
  const float inv = rsqrtf(ss * (1.f / 128.f) + eps);
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) y[i] = Elem<__nv_bfloat16>::round(Elem<__nv_bfloat16>::round(x[i] * inv) * wv[i]);
  float out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, y[i], 16);   // dim +- 64
    const float rot = lane < 16 ? -other : other;
    out[i] = y[i] * c[i] + rot * s[i];
  }
  __nv_bfloat16* dst = (is_q ? q_out + ((long long)b * n_q_heads + h) * 128
                             : k_out + ((long long)b * n_kv_heads + (h - n_q_heads)) * 128) + lane * 4;
  uint2 o;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
  po[0] = __floats2bfloat162_rn(out[0], out[1]);
  po[1] = __floats2bfloat162_rn(out[2], out[3]);
  *reinterpret_cast<uint2*>(dst) = o;
}

// x_out = x + y (y may be null); h_out = rmsnorm(x_out) * w.  One CTA of 256 threads per row.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                   const __nv_bfloat16* __restrict__ w, float eps, int hidden, __nv_bfloat16* __restrict__ x_out,
                   __nv_bfloat16* __restrict__ h_out) {
  extern __shared__ float s_row[];   // [hidden]
  __shared__ float s_part[8];
  const long long base = (long long)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x * 2; i < hidden; i += 512) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + base + i));
    if (y) {
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y + base + i));
      a.x = Elem<__nv_bfloat16>::round(a.x + b.x);
      a.y = Elem<__nv_bfloat16>::round(a.y + b.y);
      if (x_out) *reinterpret_cast<__nv_bfloat162*>(x_out + base + i) = __floats2bfloat162_rn(a.x, a.y);
    }
    s_row[i] = a.x;
    s_row[i + 1] = a.y;
    ss += a.x * a.x + a.y * a.y;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_part[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  for (int i = threadIdx.x * 2; i < hidden; i += 512) {
    const float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + i));
    *reinterpret_cast<__nv_bfloat162*>(h_out + base + i) =
        __floats2bfloat162_rn(Elem<__nv_bfloat16>::round(s_row[i] * inv) * wv.x,
                              Elem<__nv_bfloat16>::round(s_row[i + 1] * inv) * wv.y);
  }
}

// out[r, j] = silu(gu[r, j]) * gu[r, ffn + j]
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, long long row_stride, int ffn, int n_rows,
                __nv_bfloat16* __restrict__ out) {
  const long long total = (long long)n_rows * (ffn / 2);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / (ffn / 2)), j = (int)(i % (ffn / 2)) * 2;
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (long long)r * row_stride + j));
    const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + (long long)r * row_stride + ffn + j));
    const float a = Elem<__nv_bfloat16>::round(g.x / (1.f + __expf(-g.x))) * u.x;
    const float b = Elem<__nv_bfloat16>::round(g.y / (1.f + __expf(-g.y))) * u.y;
    *reinterpret_cast<__nv_bfloat162*>(out + (long long)r * ffn + j) = __floats2bfloat162_rn(a, b);
  }
}

}  // namespace msa

using namespace msa;

extern "C" int msa_qk_norm_rope(const void* qkv, int64_t row_stride, int32_t n_seq, int32_t n_q_heads,
                                int32_t n_kv_heads, int32_t head_dim, const void* q_weight, const void* k_weight,
                                float eps, const void* cos_table, const void* sin_table, void* q_out, void* k_out,
                                void* stream) {
  MSA_REQUIRE(qkv && q_weight && k_weight && cos_table && sin_table && q_out && k_out, "qk_norm_rope: null pointer");
  MSA_REQUIRE(head_dim == 128, "qk_norm_rope: head_dim must be 128");
  MSA_REQUIRE(n_seq >= 0 && n_q_heads > 0 && n_kv_heads > 0 && row_stride % 4 == 0, "qk_norm_rope: bad sizes");
  MSA_REQUIRE((reinterpret_cast<uintptr_t>(qkv) & 7u) == 0 && (reinterpret_cast<uintptr_t>(q_out) & 7u) == 0 &&
                  (reinterpret_cast<uintptr_t>(k_out) & 7u) == 0 && (reinterpret_cast<uintptr_t>(cos_table) & 7u) == 0 &&
                  (reinterpret_cast<uintptr_t>(sin_table) & 7u) == 0, "qk_norm_rope: pointers must be 8-byte aligned");
  if (n_seq == 0) return MSA_OK;
  const long long warps = (long long)n_seq * (n_q_heads + n_kv_heads);
  qk_norm_rope_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, row_stride, n_seq, n_q_heads, n_kv_heads, (const __nv_bfloat16*)q_weight,
      (const __nv_bfloat16*)k_weight, eps, (const __nv_bfloat16*)cos_table, (const __nv_bfloat16*)sin_table,
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out);
  MSA_LAUNCH_OK("qk_norm_rope_kernel");
  return MSA_OK;
}

extern "C" int msa_add_rmsnorm(const void* x, const void* y, const void* weight, float eps, int32_t n_rows,
                               int32_t hidden, void* x_out, void* h_out, void* stream) {
  MSA_REQUIRE(x && weight && h_out, "add_rmsnorm: null pointer");
  MSA_REQUIRE(n_rows >= 0 && hidden > 0 && hidden % 2 == 0 && hidden <= 12288, "add_rmsnorm: hidden must be even and <= 12288");
  if (n_rows == 0) return MSA_OK;
  add_rmsnorm_kernel<<<n_rows, 256, hidden * sizeof(float), (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)weight, eps, hidden,
      (__nv_bfloat16*)x_out, (__nv_bfloat16*)h_out);
  MSA_LAUNCH_OK("add_rmsnorm_kernel");
  return MSA_OK;
}

extern "C" int msa_silu_mul(const void* gate_up, int64_t row_stride, int32_t n_rows, int32_t ffn, void* out,
                            void* stream) {
  MSA_REQUIRE(gate_up && out, "silu_mul: null pointer");
  MSA_REQUIRE(n_rows >= 0 && ffn > 0 && ffn % 2 == 0 && row_stride % 2 == 0, "silu_mul: ffn and the row stride must be even");
  if (n_rows == 0) return MSA_OK;
  const long long total = (long long)n_rows * (ffn / 2);
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  silu_mul_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gate_up, row_stride, ffn, n_rows,
                                                          (__nv_bfloat16*)out);
  MSA_LAUNCH_OK("silu_mul_kernel");
  return MSA_OK;
}
