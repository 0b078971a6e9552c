// Entry points that need no kernel: version, error text, size queries, runtime switches.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pnv {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

// PAIRED_NVFP4_PDL=0 turns programmatic dependent launch off for every kernel of the library;
// read once per process.
bool pdl_enabled() {
  static int value = -1;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* env = std::getenv("PAIRED_NVFP4_PDL");
    value = (env != nullptr && std::strcmp(env, "0") == 0) ? 0 : 1;
  });
  return value != 0;
}

}  // namespace pnv

using namespace pnv;

extern "C" int pnv_abi_version(void) { return PNV_ABI_VERSION; }

extern "C" const char* pnv_last_error(void) { return last_error_buffer(); }

// Buffers other processes' GPUs store into (the direct expert-parallel exchange).  Plain cudaMalloc memory, so
// that the interprocess handle names exactly this allocation; set-up time only, never on the forward path.
extern "C" int pnv_peer_buffer_alloc(int64_t bytes, void** ptr_out, void* handle_out) {
  PNV_REQUIRE(bytes > 0 && ptr_out && handle_out, "bad peer buffer request");
  void* p = nullptr;
  PNV_CUDA(cudaMalloc(&p, (size_t)bytes));
  cudaIpcMemHandle_t h;
  cudaError_t err = cudaIpcGetMemHandle(&h, p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return fail(PNV_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(err));
  }
  static_assert(sizeof(h) == PNV_PEER_HANDLE_BYTES, "interprocess handle size");
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return PNV_OK;
}

extern "C" int pnv_peer_buffer_open(const void* handle, void** ptr_out) {
  PNV_REQUIRE(handle && ptr_out, "null pointer argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  // maps the other process's allocation into the CURRENT device's address space and enables peer access to
  // the device it lives on, so kernels launched on the current device can store into it
  PNV_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = p;
  return PNV_OK;
}

extern "C" int pnv_peer_buffer_close(void* ptr) {
  if (ptr != nullptr) PNV_CUDA(cudaIpcCloseMemHandle(ptr));
  return PNV_OK;
}

extern "C" int pnv_peer_buffer_free(void* ptr) {
  if (ptr != nullptr) PNV_CUDA(cudaFree(ptr));
  return PNV_OK;
}

extern "C" int pnv_physical_dims(int features, int k, int* m_aligned_ac, int* k_aligned_ac,
                                 int* m_aligned_e, int* k_aligned_e) {
  PNV_REQUIRE(features >= 1 && k >= 1, "features and k must be positive");
  PNV_REQUIRE(m_aligned_ac && k_aligned_ac && m_aligned_e && k_aligned_e, "null pointer argument");
  WeightDims wd = weight_dims(features, k);
  *m_aligned_ac = wd.m_ac;
  *k_aligned_ac = wd.k_ac;
  *m_aligned_e = wd.m_e;
  *k_aligned_e = wd.k_e;
  return PNV_OK;
}

extern "C" int64_t pnv_sf_numel(int rows, int k, int groups) {
  if (rows < 1 || k < 1 || groups < 1) return 0;
  return sf_numel(rows, k, groups);
}
