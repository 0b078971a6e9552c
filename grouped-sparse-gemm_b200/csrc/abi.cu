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
