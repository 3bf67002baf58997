// Tensor-core fragment helpers shared by the decode and prefill attention kernels
// (bf16, head_dim 128): cp.async staging, ldmatrix, mma.sync.m16n8k16 wrappers.
#pragma once
#include "common.cuh"

namespace msa {

constexpr int kMmaD = 128;       // head_dim
constexpr int kMmaKeys = 16;     // keys per block
constexpr int kMmaStages = 3;
constexpr int kMmaRow = 272;     // bytes per staged row: 256 + 16 pad -> conflict-free ldmatrix
constexpr int kMmaWarps = 4;
constexpr int kMmaTileBytes = kMmaKeys * kMmaRow;                       // one K (or V) block
constexpr int kMmaWarpBytes = kMmaStages * 2 * kMmaTileBytes;           // K+V ring of one warp
constexpr int kMmaSmemBytes = kMmaWarps * kMmaWarpBytes;                // 104,448 bytes -> 2 CTAs per SM

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8 f32) += A (16x16 bf16, rows 8..15 zero) * B (16x8 bf16)
__device__ __forceinline__ void mma_bf16_top(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace msa
