// Shared host/device helpers of the msa_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/msa_b200.h"

namespace msa {

// Thread-local message behind msa_last_error().
void set_error(const char* fmt, ...);

#define MSA_REQUIRE(cond, ...)        \
  do {                                \
    if (!(cond)) {                    \
      ::msa::set_error(__VA_ARGS__);  \
      return MSA_ERR_ARG;             \
    }                                 \
  } while (0)

#define MSA_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess) {                                                          \
      (void)cudaGetLastError(); /* reported here: do not leave it for the next launch check */ \
      ::msa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return MSA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

#define MSA_LAUNCH_OK(name)                                                            \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess) {                                                          \
      ::msa::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));      \
      return MSA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

// Per-device launch state.  The opt-in dynamic shared-memory size of a kernel and the SM count are
// properties of a (kernel, device) pair, not of the calling thread: a host thread that drives a second
// GPU has to set them there too.  Every launcher keeps one DeviceSmem per kernel, indexed by the
// current device's ordinal.
constexpr int kMaxDevices = 64;
struct DeviceSmem { size_t enabled[kMaxDevices]; };

int current_device(int* dev);   // cudaGetDevice + range check (ordinal < kMaxDevices)
int device_sm_count(int* n_sm); // SM count of the current device (cached per device)

template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kernel, size_t bytes, DeviceSmem& state) {
  int dev = 0;
  const int rc = current_device(&dev);
  if (rc != MSA_OK) return rc;
  if (bytes > state.enabled[dev]) {
    MSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    state.enabled[dev] = bytes;
  }
  return MSA_OK;
}
#define MSA_OK_OR_RETURN(expr)        \
  do {                                \
    const int rc__ = (expr);          \
    if (rc__ != MSA_OK) return rc__;  \
  } while (0)

inline size_t dtype_size(int32_t dtype) { return dtype == MSA_BF16 ? 2 : 4; }
inline bool dtype_ok(int32_t dtype) { return dtype == MSA_F32 || dtype == MSA_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Order-preserving map float -> uint32 (larger float <=> larger key), and back.
__host__ __device__ inline uint32_t float_to_key(float f) {
#ifdef __CUDA_ARCH__
  uint32_t b = __float_as_uint(f);
#else
  union { float f; uint32_t u; } c; c.f = f; uint32_t b = c.u;
#endif
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ inline float key_to_float(uint32_t k) {
  uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
#ifdef __CUDA_ARCH__
  return __uint_as_float(b);
#else
  union { float f; uint32_t u; } c; c.u = b; return c.f;
#endif
}

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  __device__ static inline void load(const float* p, float (&o)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
  __device__ static inline void store(float* p, const float (&o)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  }
  __device__ static inline float round(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static inline void load(const __nv_bfloat16* p, float (&o)[8]) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
  __device__ static inline void store(__nv_bfloat16* p, const float (&o)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
  __device__ static inline float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};


// Programmatic dependent launch (sm_90+): a kernel launched with `pdl` may start while the kernel before it in the
// stream is still running; it must execute grid_dependency_wait() before it touches anything that kernel writes.
// The earlier kernel lets dependents start early with grid_launch_dependents(); without that call they start when
// it completes.  Both are no-ops in a kernel that was launched normally.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace msa
