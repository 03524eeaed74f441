// gdn2_prefill_static: the whole-chunk prefill (chunk-local stage + fused scan) for callers that
// must not allocate device memory. The scratch the two kernels exchange lives in a fixed array
// compiled into the library instead of a caller-provided workspace.
//
// Who needs this: code that runs after a serving engine has handed every free byte of HBM to its
// own pool (a cudaMalloc there fails or fragments the pool), code inside a latency-critical loop
// where the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable, and
// plugins whose host only lends them pre-registered input and output buffers.
#include <mutex>

#include "common.cuh"

namespace gdn2 {
namespace {

// Scratch shared by every call on a device. It is part of the library image: each GPU that loads
// the library holds these bytes until the process exits, so the size is deliberately modest.
static __device__ __align__(256) unsigned char g_static_scratch[GDN2_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

// The array's name is only a host-side handle in host code; the kernels need its device address.
// Resolved once per device, with that device current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  GDN2_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GDN2_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    GDN2_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    if (ptr == nullptr) return GDN2_ERR_CUDA;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return GDN2_OK;
}

}  // namespace
}  // namespace gdn2

using namespace gdn2;

extern "C" int gdn2_prefill_static(const void* q, const void* k, const void* v, const float* g, const void* b,
                                   const void* w, const float* initial_state, void* o, float* final_state,
                                   int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV,
                                   int64_t in_batch_stride, int64_t o_batch_stride, float scale, int dtype,
                                   void* stream) {
  if (!q || !k || !v || !g || !b || !w || !o) return GDN2_ERR_NULL_POINTER;
  const size_t need = gdn2_prefill_workspace_bytes(B, S, H, H, DK, DV, dtype, GDN2_PATH_AUTO);
  if (need == 0) {
    // Not a size problem: let the regular entry point's validation name the reason (bad shape,
    // bad dtype, unsupported head dims). With a zero-byte workspace it cannot launch anything.
    const int why = gdn2_chunk_prep(q, k, v, g, b, w, const_cast<void*>(q), 0, B, S, H, H, DK, DV, in_batch_stride,
                                    scale, dtype, GDN2_PATH_AUTO, stream);
    return (why == GDN2_OK || why == GDN2_ERR_WORKSPACE) ? GDN2_ERR_UNSUPPORTED : why;
  }
  if (need > (size_t)GDN2_STATIC_SCRATCH_BYTES) return GDN2_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != GDN2_OK) return rc;
  // Every record of the scratch that the scan reads is rewritten by the chunk-local stage of the
  // same call, so nothing has to be cleared between calls.
  rc = gdn2_chunk_prep(q, k, v, g, b, w, scratch, GDN2_STATIC_SCRATCH_BYTES, B, S, H, H, DK, DV, in_batch_stride,
                       scale, dtype, GDN2_PATH_AUTO, stream);
  if (rc != GDN2_OK) return rc;
  return gdn2_prefill_scan(scratch, GDN2_STATIC_SCRATCH_BYTES, initial_state, o, final_state, nullptr, B, S, H, H,
                           DK, DV, o_batch_stride, dtype, GDN2_PATH_AUTO, stream);
}
