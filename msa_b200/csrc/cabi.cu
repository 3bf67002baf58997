// Error reporting and version of the C ABI.
#include "common.cuh"

namespace msa {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int current_device(int* dev) {
  MSA_CUDA_OK(cudaGetDevice(dev));
  MSA_REQUIRE(*dev >= 0 && *dev < kMaxDevices, "device ordinal %d is outside the supported range 0..%d", *dev,
              kMaxDevices - 1);
  return MSA_OK;
}

int device_sm_count(int* n_sm) {
  static int cached[kMaxDevices] = {0};
  int dev = 0;
  MSA_OK_OR_RETURN(current_device(&dev));
  if (cached[dev] == 0) MSA_CUDA_OK(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
  *n_sm = cached[dev];
  return MSA_OK;
}

}  // namespace msa

extern "C" const char* msa_last_error(void) { return msa::g_error; }
extern "C" int msa_abi_version(void) { return MSA_ABI_VERSION; }

// Pin and map a host range that was allocated elsewhere (for example a shared-memory file
// that every rank of a node opens), so that msa_gather_run can read it from the device.
extern "C" int msa_bank_register_host(void* host_ptr, int64_t bytes, uint64_t* device_address) {
  MSA_REQUIRE(host_ptr && bytes > 0 && device_address, "bank_register_host: bad arguments");
  MSA_CUDA_OK(cudaHostRegister(host_ptr, (size_t)bytes, cudaHostRegisterPortable | cudaHostRegisterMapped));
  void* dev = nullptr;
  const cudaError_t e = cudaHostGetDevicePointer(&dev, host_ptr, 0);
  if (e != cudaSuccess) {   // do not leave the range pinned when it cannot be used
    (void)cudaGetLastError();
    (void)cudaHostUnregister(host_ptr);
    ::msa::set_error("cudaHostGetDevicePointer failed: %s", cudaGetErrorString(e));
    return MSA_ERR_CUDA;
  }
  *device_address = (uint64_t)(uintptr_t)dev;
  return MSA_OK;
}

extern "C" int msa_bank_unregister_host(void* host_ptr) {
  MSA_REQUIRE(host_ptr, "bank_unregister_host: null pointer");
  MSA_CUDA_OK(cudaHostUnregister(host_ptr));
  return MSA_OK;
}
