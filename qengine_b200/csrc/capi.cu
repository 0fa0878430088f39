// Library-wide state behind the C ABI: version, device queries, run-time switches and the L2
// persistence controls (reference csrc/ops.h:31-36, csrc/basic.cu:384-398).
#include <atomic>

#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace qb {

bool& pdl_launch_enabled() {
  static bool on = true;
  return on;
}
static std::atomic<int> g_trigger{1};
int pdl_trigger_enabled() { return g_trigger.load(std::memory_order_relaxed); }

}  // namespace qb

extern "C" int qe_abi_version(void) { return 3; }

extern "C" int qe_sm_count(void) {
  static int per_dev[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!per_dev[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;  // B200
    per_dev[dev] = n;
  }
  return per_dev[dev];
}

// Programmatic dependent launch needs both halves: the consumer launched with the attribute and
// the producer signalling early. Either switch off gives plain stream order.
extern "C" void qe_set_pdl_launch(int on) { qb::pdl_launch_enabled() = on != 0; }
extern "C" void qe_set_pdl_trigger(int on) { qb::g_trigger.store(on != 0); }

extern "C" int qe_l2_persist_limit(size_t bytes) {
  cudaError_t e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaCtxResetPersistingL2Cache();
}

extern "C" int qe_stream_access_window(uintptr_t base, size_t bytes, float hit_ratio, void* stream) {
  cudaStreamAttrValue v = {};
  v.accessPolicyWindow.base_ptr = reinterpret_cast<void*>(base);
  v.accessPolicyWindow.num_bytes = bytes;
  v.accessPolicyWindow.hitRatio = bytes ? hit_ratio : 0.f;
  v.accessPolicyWindow.hitProp = bytes ? cudaAccessPropertyPersisting : cudaAccessPropertyNormal;
  v.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  return (int)cudaStreamSetAttribute((cudaStream_t)stream, cudaStreamAttributeAccessPolicyWindow, &v);
}
