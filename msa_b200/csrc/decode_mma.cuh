// bf16, head_dim 128 decode attention on mma.sync tensor-core fragments.
//
// Decode attention is bound by HBM (every K/V byte is used once), so the job of the kernel
// is to keep enough loads in flight and spend as few issue slots per key as possible.  The
// G <= 8 query heads of a kv group are rows 0..G-1 of a 16-row mma tile (the other rows are
// zero and cost nothing that matters), which turns the per-key work from ~50 CUDA-core
// warp instructions into ~6.  Each warp owns its own stream of 16-key blocks: cp.async
// (16-byte, L1-bypassing) into a private 3-stage ring, ldmatrix, mma.m16n8k16, online
// softmax on the accumulator fragments, no CTA-wide barrier inside the loop.  The four warps'
// partial (max, sum, output) are merged through shared memory at the end.
#pragma once
#include "common.cuh"
#include "mma_helpers.cuh"

namespace msa {

__global__ void __launch_bounds__(kMmaWarps * 32, 2)
decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                  const __nv_bfloat16* __restrict__ v_cache, long long stride_b, long long stride_h,
                  const int32_t* __restrict__ kv_start, const int32_t* __restrict__ kv_len,
                  const __nv_bfloat16* __restrict__ new_k, const __nv_bfloat16* __restrict__ new_v, int n_q_heads,
                  int n_kv_heads, float scale_log2e, __nv_bfloat16* __restrict__ out, float* __restrict__ ws,
                  int n_splits) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int G = n_q_heads / n_kv_heads;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = lane >> 2, quad = lane & 3;  // accumulator row (= query head of the group), column pair

  const int cached = kv_len[b];
  const int total = cached + (new_k ? 1 : 0);
  int per = (total + n_splits - 1) / n_splits;
  per = (per + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
  const int p_lo = split * per, p_hi = min(total, p_lo + per);
  const int n_blocks = p_hi > p_lo ? (p_hi - p_lo + kMmaKeys - 1) / kMmaKeys : 0;
  const long long base = (long long)b * stride_b + (long long)h * stride_h +
                         (long long)(kv_start ? kv_start[b] : 0) * kMmaD;
  const long long new_off = ((long long)b * n_kv_heads + h) * kMmaD;

  // query fragments: a0 = cols [16j + 2*quad, +1], a2 = cols +8, of row `row` (zero beyond the group)
  uint32_t qa[kMmaD / 16][2];
  {
    const __nv_bfloat16* qr = q + ((long long)b * n_q_heads + (long long)h * G + (row < G ? row : 0)) * kMmaD;
#pragma unroll
    for (int j = 0; j < kMmaD / 16; ++j) {
      qa[j][0] = row < G ? *reinterpret_cast<const uint32_t*>(qr + 16 * j + 2 * quad) : 0u;
      qa[j][1] = row < G ? *reinterpret_cast<const uint32_t*>(qr + 16 * j + 8 + 2 * quad) : 0u;
    }
  }

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * kMmaWarpBytes;
  auto issue = [&](int blk, int stage) {  // blk counts this split's 16-key blocks
    const uint32_t kdst = ring + stage * 2 * kMmaTileBytes, vdst = kdst + kMmaTileBytes;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int idx = lane + 32 * c, r = idx >> 4, ch = idx & 15;
      const int p = p_lo + blk * kMmaKeys + r;
      const __nv_bfloat16 *ks = k_cache, *vs = v_cache;
      uint32_t bytes = 0;
      if (p < p_hi) {
        bytes = 16;
        if (p < cached) {
          ks = k_cache + base + (long long)p * kMmaD + ch * 8;
          vs = v_cache + base + (long long)p * kMmaD + ch * 8;
        } else {
          ks = new_k + new_off + ch * 8;
          vs = new_v + new_off + ch * 8;
        }
      }
      cp_async16(kdst + r * kMmaRow + ch * 16, ks, bytes);  // bytes == 0 zero-fills the row
      cp_async16(vdst + r * kMmaRow + ch * 16, vs, bytes);
    }
  };

  float o[kMmaD / 8][4];
#pragma unroll
  for (int i = 0; i < kMmaD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;

  // this warp's blocks: warp, warp + 4, ...
  const int my_n = n_blocks > warp ? (n_blocks - warp + kMmaWarps - 1) / kMmaWarps : 0;
#pragma unroll
  for (int s = 0; s < kMmaStages - 1; ++s) {
    if (s < my_n) issue(warp + s * kMmaWarps, s);
    cp_async_commit();
  }
  for (int it = 0; it < my_n; ++it) {
    cp_async_wait<kMmaStages - 2>();
    __syncwarp();
    const int blk = warp + it * kMmaWarps, stage = it % kMmaStages;
    {  // refill the stage that was consumed in the previous iteration
      const int nxt = it + kMmaStages - 1;
      if (nxt < my_n) issue(warp + nxt * kMmaWarps, nxt % kMmaStages);
      cp_async_commit();
    }
    const uint32_t kbuf = ring + stage * 2 * kMmaTileBytes, vbuf = kbuf + kMmaTileBytes;

    // S = Q K^T for 16 keys: two n-blocks of 8 keys
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a = kbuf + ((mi >> 1) * 8 + r) * kMmaRow + (mi & 1) * 16;
#pragma unroll
      for (int j = 0; j < kMmaD / 16; ++j) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(a + j * 32, b0, b1, b2, b3);
        mma_bf16_top(s0, qa[j][0], qa[j][1], b0, b1);
        mma_bf16_top(s1, qa[j][0], qa[j][1], b2, b3);
      }
    }
    // scale, mask the tail, online softmax over the quad that shares a row
    const int key0 = p_lo + blk * kMmaKeys + 2 * quad;
    float v00 = key0 < p_hi ? s0[0] * scale_log2e : -INFINITY;
    float v01 = key0 + 1 < p_hi ? s0[1] * scale_log2e : -INFINITY;
    float v10 = key0 + 8 < p_hi ? s1[0] * scale_log2e : -INFINITY;
    float v11 = key0 + 9 < p_hi ? s1[1] * scale_log2e : -INFINITY;
    float mx = fmaxf(fmaxf(v00, v01), fmaxf(v10, v11));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);           // finite: every issued block has a valid key
    const float f = exp2f(m_run - m_new);
    v00 = exp2f(v00 - m_new); v01 = exp2f(v01 - m_new); v10 = exp2f(v10 - m_new); v11 = exp2f(v11 - m_new);
    float sum = (v00 + v01) + (v10 + v11);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l_run = l_run * f + sum;
    m_run = m_new;
    const uint32_t pa0 = pack_bf16(v00, v01), pa2 = pack_bf16(v10, v11);
    // O = O*f + P V
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t a = vbuf + ((mi & 1) * 8 + r) * kMmaRow + (mi >> 1) * 16;
#pragma unroll
      for (int nb = 0; nb < kMmaD / 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(a + nb * 16, b0, b1, b2, b3);
        o[nb][0] *= f; o[nb][1] *= f; o[nb + 1][0] *= f; o[nb + 1][1] *= f;
        mma_bf16_top(o[nb], pa0, pa2, b0, b1);
        mma_bf16_top(o[nb + 1], pa0, pa2, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // every ring is idle: reuse shared memory for the cross-warp merge

  float* s_o = reinterpret_cast<float*>(smem);                 // [warp][8 rows][128]
  float* s_m = s_o + kMmaWarps * 8 * kMmaD;                    // [warp][8]
  float* s_l = s_m + kMmaWarps * 8;
  if (row < G) {
#pragma unroll
    for (int nb = 0; nb < kMmaD / 8; ++nb) {
      s_o[(warp * 8 + row) * kMmaD + nb * 8 + 2 * quad] = o[nb][0];
      s_o[(warp * 8 + row) * kMmaD + nb * 8 + 2 * quad + 1] = o[nb][1];
    }
    if (quad == 0) { s_m[warp * 8 + row] = m_run; s_l[warp * 8 + row] = l_run; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * kMmaD; i += kMmaWarps * 32) {
    const int g = i / kMmaD, d = i % kMmaD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) m = fmaxf(m, s_m[w * 8 + g]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float mw = s_m[w * 8 + g];
      if (mw > -INFINITY) {
        const float e = exp2f(mw - m);
        l += s_l[w * 8 + g] * e;
        acc += s_o[(w * 8 + g) * kMmaD + d] * e;
      }
    }
    const int hq = h * G + g;
    if (n_splits == 1) {
      out[((long long)b * n_q_heads + hq) * kMmaD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      float* w = ws + (((long long)b * n_q_heads + hq) * n_splits + split) * (kMmaD + 2);
      w[d] = acc;
      if (d == 0) { w[kMmaD] = m; w[kMmaD + 1] = l; }
    }
  }
}

}  // namespace msa
