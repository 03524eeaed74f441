// extern "C" entry points declared in include/gdn2_b200.h: argument validation, kernel-family
// dispatch and error reporting. Nothing here allocates device memory.
#include <cstdio>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace gdn2 {

namespace {
thread_local int g_last_cuda_error = 0;
__device__ uint32_t g_device_status;   // one word per device image of this library
}  // namespace

int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return GDN2_ERR_CUDA;
}

uint32_t* device_status_word() {
  static void* cached[64] = {};                   // per device ordinal: the address is looked up once
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev >= 0 && dev < 64 && cached[dev]) return static_cast<uint32_t*>(cached[dev]);
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
  if (dev >= 0 && dev < 64) cached[dev] = p;
  return static_cast<uint32_t*>(p);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) sticks to a (kernel, device) pair: made once, not on every launch
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::unordered_map<unsigned long long, size_t> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long key = reinterpret_cast<unsigned long long>(kernel) ^ (static_cast<unsigned long long>(dev) << 56);
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = done.find(key);
    if (it != done.end() && it->second >= bytes) return cudaSuccess;
  }
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) {
    std::lock_guard<std::mutex> lk(mu);
    done[key] = bytes;
  }
  return e;
}

int device_sm_count() {
  static int cached[64] = {};                     // per device ordinal; 0 = not asked yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool valid_dtype(int dtype) { return dtype == GDN2_F32 || dtype == GDN2_BF16 || dtype == GDN2_F16; }

// Resolve AUTO and check that the chosen family supports the shape. Returns a gdn2_status; *resolved is
// GDN2_PATH_SIMT or GDN2_PATH_TCGEN05, *segments whether the scan may cut the sequence.
int resolve_path(int64_t DK, int64_t DV, int dtype, int path, int* resolved, bool* segments) {
  const bool tc_ok = (DK == 128 && DV == 128 && dtype == GDN2_BF16);
  const bool simt_ok = (DK >= 8 && DK <= 128 && DK % 8 == 0 && DV >= 4 && DV % 4 == 0);
  if (path == GDN2_PATH_AUTO) path = tc_ok ? GDN2_PATH_TCGEN05 : GDN2_PATH_SIMT;
  *segments = path == GDN2_PATH_TCGEN05;
  if (path == GDN2_PATH_TCGEN05_SERIAL) path = GDN2_PATH_TCGEN05;
  if (path == GDN2_PATH_TCGEN05 && !tc_ok) return GDN2_ERR_UNSUPPORTED;
  if (path == GDN2_PATH_SIMT && !simt_ok) return GDN2_ERR_UNSUPPORTED;
  if (path != GDN2_PATH_SIMT && path != GDN2_PATH_TCGEN05) return GDN2_ERR_UNSUPPORTED;
  *resolved = path;
  return GDN2_OK;
}

// The workspace layout of a validated problem.
WsLayout layout_for(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int family, bool segments) {
  return make_ws_layout(B, S, H, HK, (int)DK, (int)DV, family == GDN2_PATH_TCGEN05 ? 2 : 4, segments);
}

int check_prefill_shape(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int dtype) {
  if (!valid_dtype(dtype)) return GDN2_ERR_BAD_DTYPE;
  if (B <= 0 || S <= 0 || H <= 0 || DK <= 0 || DV <= 0 || S % kChunk != 0) return GDN2_ERR_BAD_SHAPE;
  if (HK <= 0 || H % HK != 0) return GDN2_ERR_BAD_SHAPE;            // value heads share key heads in equal groups
  // the chunk-local kernels put (batch, head) on gridDim.y
  if (B * H > 65535 || S > (1LL << 30)) return GDN2_ERR_BAD_SHAPE;
  return GDN2_OK;
}

}  // namespace
}  // namespace gdn2

using namespace gdn2;

extern "C" {

int gdn2_abi_version(void) { return GDN2_B200_ABI_VERSION; }

const char* gdn2_status_string(int status) {
  switch (status) {
    case GDN2_OK: return "ok";
    case GDN2_ERR_NULL_POINTER: return "a required pointer is NULL";
    case GDN2_ERR_BAD_SHAPE: return "bad shape (sizes must be positive, S a multiple of 64, B*H <= 65535 for the chunkwise calls)";
    case GDN2_ERR_BAD_DTYPE: return "unknown element type";
    case GDN2_ERR_MISALIGNED: return "a pointer is not 16-byte aligned";
    case GDN2_ERR_WORKSPACE: return "workspace too small";
    case GDN2_ERR_CUDA: return "a CUDA call failed (see gdn2_last_cuda_error)";
    case GDN2_ERR_DEVICE_WAIT: return "a kernel gave up on a bounded wait";
    case GDN2_ERR_UNSUPPORTED: return "no kernel is built for this shape / dtype / path";
    case GDN2_ERR_STATIC_LIMIT:
      return "the problem needs more scratch than the built-in static buffer (GDN2_STATIC_SCRATCH_BYTES) holds";
    default: return "unknown status";
  }
}

int gdn2_last_cuda_error(void) { return g_last_cuda_error; }

int gdn2_decode(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                float* state, void* o, int64_t B, int64_t n, int64_t H, int64_t HK, int64_t DK, int64_t DV,
                int64_t in_batch_stride, int64_t o_batch_stride, float scale, int dtype, void* stream) {
  if (!q || !k || !v || !g || !b || !w || !state || !o) return GDN2_ERR_NULL_POINTER;
  if (!valid_dtype(dtype)) return GDN2_ERR_BAD_DTYPE;
  if (B <= 0 || n <= 0 || H <= 0 || DK <= 0 || DV <= 0 || DK > 256) return GDN2_ERR_BAD_SHAPE;
  if (HK <= 0 || H % HK != 0) return GDN2_ERR_BAD_SHAPE;
  if (B * H > 2147483647LL / 4 || n > (1 << 24)) return GDN2_ERR_BAD_SHAPE;
  if (in_batch_stride < n || o_batch_stride < n) return GDN2_ERR_BAD_SHAPE;
  if (DK == 128 && DV == 128 && (!aligned16(state) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(g) ||
                                 !aligned16(b) || !aligned16(w) || !aligned16(o)))
    return GDN2_ERR_MISALIGNED;                            // bulk copies and 16-byte loads on this path
  return launch_decode(q, k, v, g, b, w, state, o, (int)B, (int)n, (int)H, (int)HK, (int)DK, (int)DV, in_batch_stride,
                       o_batch_stride, scale, dtype, static_cast<cudaStream_t>(stream));
}

size_t gdn2_prefill_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int dtype,
                                    int path) {
  if (check_prefill_shape(B, S, H, HK, DK, DV, dtype) != GDN2_OK) return 0;
  int p;
  bool seg;
  if (resolve_path(DK, DV, dtype, path, &p, &seg) != GDN2_OK) return 0;
  return layout_for(B, S, H, HK, DK, DV, p, seg).total;
}

int gdn2_prefill_workspace_layout(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int dtype,
                                  int path, int64_t* out8) {
  if (!out8) return GDN2_ERR_NULL_POINTER;
  int rc = check_prefill_shape(B, S, H, HK, DK, DV, dtype);
  if (rc != GDN2_OK) return rc;
  int p;
  bool seg;
  rc = resolve_path(DK, DV, dtype, path, &p, &seg);
  if (rc != GDN2_OK) return rc;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  const size_t v[8] = {L.off_wq, L.off_aqk, L.off_kgt, L.off_ut, L.off_gl, L.off_flags, L.off_seg, L.total};
  for (int i = 0; i < 8; ++i) out8[i] = (int64_t)v[i];
  return GDN2_OK;
}

int gdn2_prefill_scan_segments(int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV, int dtype, int path) {
  const int64_t HK = H;                                    // the cut depends on the (batch, value head) pairs only
  if (check_prefill_shape(B, S, H, HK, DK, DV, dtype) != GDN2_OK) return 0;
  int p;
  bool seg;
  if (resolve_path(DK, DV, dtype, path, &p, &seg) != GDN2_OK) return 0;
  return layout_for(B, S, H, HK, DK, DV, p, seg).nseg;
}

int gdn2_prefill_scan_launches(int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV, int dtype, int path) {
  const int64_t HK = H;
  if (check_prefill_shape(B, S, H, HK, DK, DV, dtype) != GDN2_OK) return 0;
  int p;
  bool seg;
  if (resolve_path(DK, DV, dtype, path, &p, &seg) != GDN2_OK) return 0;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  return L.nseg <= 1 ? 1 : L.nseg_guarded ? 4 : 3;
}

int gdn2_chunk_prep(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                    void* workspace, size_t workspace_bytes, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                    int64_t DV, int64_t in_batch_stride, float scale, int dtype, int path, void* stream) {
  if (!q || !k || !v || !g || !b || !w || !workspace) return GDN2_ERR_NULL_POINTER;
  int rc = check_prefill_shape(B, S, H, HK, DK, DV, dtype);
  if (rc != GDN2_OK) return rc;
  if (in_batch_stride < S) return GDN2_ERR_BAD_SHAPE;
  int p;
  bool seg;
  rc = resolve_path(DK, DV, dtype, path, &p, &seg);
  if (rc != GDN2_OK) return rc;
  if (!aligned16(workspace) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(g) ||
      !aligned16(b) || !aligned16(w))
    return GDN2_ERR_MISALIGNED;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  if (workspace_bytes < L.total) return GDN2_ERR_WORKSPACE;
  const WsPtrs P = ws_pointers(workspace, L);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p == GDN2_PATH_TCGEN05) {
    rc = launch_prep_tc(q, k, v, g, b, w, L, P, (int)B, (int)S, (int)H, (int)HK, in_batch_stride, scale, st);
    if (rc != GDN2_OK) return rc;
    // chunks whose decay is too fast for the factorised diagonal blocks are redone exactly
    return launch_prep_simt(q, k, v, g, b, w, L, P, (int)B, (int)S, (int)H, (int)HK, in_batch_stride, scale, dtype, true, st);
  }
  return launch_prep_simt(q, k, v, g, b, w, L, P, (int)B, (int)S, (int)H, (int)HK, in_batch_stride, scale, dtype, false, st);
}

namespace {
int prefill_scan_impl(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                      float* final_state, float* chunk_states, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                      int64_t DV, int64_t o_batch_stride, int dtype, int path, int part, void* stream);
}

int gdn2_prefill_scan(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                      float* final_state, float* chunk_states, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                      int64_t DV, int64_t o_batch_stride, int dtype, int path, void* stream) {
  return prefill_scan_impl(workspace, workspace_bytes, initial_state, o, final_state, chunk_states, B, S, H, HK, DK, DV,
                           o_batch_stride, dtype, path, 0, stream);
}

int gdn2_prefill_scan_part(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                           float* final_state, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV,
                           int64_t o_batch_stride, int dtype, int path, int part, void* stream) {
  if (part != 1 && part != 2) return GDN2_ERR_BAD_SHAPE;
  return prefill_scan_impl(workspace, workspace_bytes, initial_state, o, final_state, nullptr, B, S, H, HK, DK, DV,
                           o_batch_stride, dtype, path, part, stream);
}

namespace {
int prefill_scan_impl(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                      float* final_state, float* chunk_states, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                      int64_t DV, int64_t o_batch_stride, int dtype, int path, int part, void* stream) {
  if (!workspace || !o) return GDN2_ERR_NULL_POINTER;
  int rc = check_prefill_shape(B, S, H, HK, DK, DV, dtype);
  if (rc != GDN2_OK) return rc;
  if (o_batch_stride < S) return GDN2_ERR_BAD_SHAPE;
  int p;
  bool seg;
  rc = resolve_path(DK, DV, dtype, path, &p, &seg);
  if (rc != GDN2_OK) return rc;
  if (!aligned16(workspace)) return GDN2_ERR_MISALIGNED;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  if (workspace_bytes < L.total) return GDN2_ERR_WORKSPACE;
  const WsPtrs P = ws_pointers(const_cast<void*>(workspace), L);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p == GDN2_PATH_TCGEN05)
    return launch_scan_tc(L, P, initial_state, o, final_state, chunk_states, (int)B, (int)S, (int)H,
                          o_batch_stride, nullptr, part, st);
  if (part == 2) return GDN2_OK;                           // the exact family's scan is one launch
  return launch_scan_simt(L, P, initial_state, o, final_state, chunk_states, (int)B, (int)S, (int)H,
                          o_batch_stride, dtype, st);
}
}  // namespace

int gdn2_prefill_ragged(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                        const float* initial_state, void* o, float* final_state, void* workspace, size_t workspace_bytes,
                        int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int64_t in_batch_stride,
                        int64_t o_batch_stride, float scale, int dtype, int path, void* side_stream, void* stream) {
  if (!q || !k || !v || !g || !b || !w || !o || !final_state) return GDN2_ERR_NULL_POINTER;
  if (!valid_dtype(dtype)) return GDN2_ERR_BAD_DTYPE;
  if (B <= 0 || S <= 0 || H <= 0 || HK <= 0 || H % HK != 0 || DK <= 0 || DV <= 0) return GDN2_ERR_BAD_SHAPE;
  if (in_batch_stride < S || o_batch_stride < S) return GDN2_ERR_BAD_SHAPE;
  const int64_t n_full = S / kChunk * kChunk, n_tail = S - n_full;
  const size_t esz = dtype == GDN2_F32 ? 4 : 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream), side = static_cast<cudaStream_t>(side_stream);
  int rc = GDN2_OK;
  if (n_full) {
    if (!workspace) return GDN2_ERR_NULL_POINTER;
    rc = gdn2_chunk_prep(q, k, v, g, b, w, workspace, workspace_bytes, B, n_full, H, HK, DK, DV, in_batch_stride, scale,
                         dtype, path, stream);
    if (rc != GDN2_OK) return rc;
    rc = gdn2_prefill_scan_part(workspace, workspace_bytes, initial_state, o, final_state, B, n_full, H, HK, DK, DV,
                                o_batch_stride, dtype, path, 1, stream);
    if (rc != GDN2_OK) return rc;
  } else {
    const size_t sbytes = (size_t)B * H * DK * DV * sizeof(float);
    if (!initial_state) GDN2_CUDA_TRY(cudaMemsetAsync(final_state, 0, sbytes, st));
    else if (initial_state != final_state)
      GDN2_CUDA_TRY(cudaMemcpyAsync(final_state, initial_state, sbytes, cudaMemcpyDeviceToDevice, st));
  }
  auto scan_rest = [&]() -> int {
    return n_full ? gdn2_prefill_scan_part(workspace, workspace_bytes, initial_state, o, final_state, B, n_full, H, HK, DK,
                                           DV, o_batch_stride, dtype, path, 2, stream)
                  : GDN2_OK;
  };
  if (!n_tail) return scan_rest();
  // the ragged tail: the same tensors from token n_full on, the state in place
  auto at = [&](const void* p, int64_t heads, int64_t d, size_t es) {
    return static_cast<const void*>(static_cast<const char*>(p) + (size_t)n_full * heads * d * es);
  };
  auto decode_tail = [&](void* on) -> int {
    return gdn2_decode(at(q, HK, DK, esz), at(k, HK, DK, esz), at(v, H, DV, esz),
                       static_cast<const float*>(at(g, HK, DK, sizeof(float))), at(b, HK, DK, esz), at(w, H, DV, esz),
                       final_state, const_cast<void*>(at(o, H, DV, esz)), B, n_tail, H, HK, DK, DV, in_batch_stride,
                       o_batch_stride, scale, dtype, on);
  };
  const bool beside = n_full && side && side != st &&
                      gdn2_prefill_scan_launches(B, n_full, H, DK, DV, dtype, path) > 1;
  if (!beside) {
    rc = scan_rest();
    return rc != GDN2_OK ? rc : decode_tail(stream);
  }
  // the tail needs the final state only: it runs on the side stream beside the cut scan's correction pass
  cudaEvent_t ready = nullptr, done = nullptr;
  GDN2_CUDA_TRY(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming));
  cudaError_t ce = cudaEventCreateWithFlags(&done, cudaEventDisableTiming);
  if (ce != cudaSuccess) { cudaEventDestroy(ready); return record_cuda_error(ce); }
  auto finish = [&](int code) { cudaEventDestroy(ready); cudaEventDestroy(done); return code; };
  if ((ce = cudaEventRecord(ready, st)) != cudaSuccess || (ce = cudaStreamWaitEvent(side, ready, 0)) != cudaSuccess)
    return finish(record_cuda_error(ce));
  rc = decode_tail(side_stream);
  // whatever happened on the side stream, the caller's stream is ordered after it
  if ((ce = cudaEventRecord(done, side)) != cudaSuccess) return finish(record_cuda_error(ce));
  const int rc2 = scan_rest();
  if ((ce = cudaStreamWaitEvent(st, done, 0)) != cudaSuccess) return finish(record_cuda_error(ce));
  return finish(rc != GDN2_OK ? rc : rc2);
}

int gdn2_prefill_scan_gated_norm(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                                 float* final_state, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                                 int64_t DV, int64_t o_batch_stride, int dtype, int path, const gdn2_gated_norm* norm,
                                 void* stream) {
  if (!norm)
    return gdn2_prefill_scan(workspace, workspace_bytes, initial_state, o, final_state, nullptr, B, S, H, HK, DK, DV,
                             o_batch_stride, dtype, path, stream);
  if (!workspace || !o || !norm->gate || !norm->weight) return GDN2_ERR_NULL_POINTER;
  int rc = check_prefill_shape(B, S, H, HK, DK, DV, dtype);
  if (rc != GDN2_OK) return rc;
  if (o_batch_stride < S || norm->gate_batch_stride < S || norm->gate_row_stride < H * DV || norm->gate_row_stride % 8 != 0)
    return GDN2_ERR_BAD_SHAPE;
  int p;
  bool seg;
  rc = resolve_path(DK, DV, dtype, path, &p, &seg);
  if (rc != GDN2_OK) return rc;
  if (p != GDN2_PATH_TCGEN05) return GDN2_ERR_UNSUPPORTED;
  if (!aligned16(workspace) || !aligned16(norm->gate) || !aligned16(norm->weight)) return GDN2_ERR_MISALIGNED;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  if (workspace_bytes < L.total) return GDN2_ERR_WORKSPACE;
  const WsPtrs P = ws_pointers(const_cast<void*>(workspace), L);
  return launch_scan_tc(L, P, initial_state, o, final_state, nullptr, (int)B, (int)S, (int)H, o_batch_stride, norm, 0,
                        static_cast<cudaStream_t>(stream));
}

int gdn2_chunk_output(const void* workspace, size_t workspace_bytes, const float* chunk_states, void* o,
                      int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int64_t o_batch_stride,
                      int dtype, int path, void* stream) {
  if (!workspace || !o || !chunk_states) return GDN2_ERR_NULL_POINTER;
  int rc = check_prefill_shape(B, S, H, HK, DK, DV, dtype);
  if (rc != GDN2_OK) return rc;
  if (o_batch_stride < S) return GDN2_ERR_BAD_SHAPE;
  int p;
  bool seg;
  rc = resolve_path(DK, DV, dtype, path, &p, &seg);
  if (rc != GDN2_OK) return rc;
  if (!aligned16(workspace)) return GDN2_ERR_MISALIGNED;
  const WsLayout L = layout_for(B, S, H, HK, DK, DV, p, seg);
  if (workspace_bytes < L.total) return GDN2_ERR_WORKSPACE;
  const WsPtrs P = ws_pointers(const_cast<void*>(workspace), L);
  if (p == GDN2_PATH_TCGEN05)
    return launch_output_tc(L, P, chunk_states, o, (int)B, (int)S, (int)H, o_batch_stride,
                            static_cast<cudaStream_t>(stream));
  return launch_output_simt(L, P, chunk_states, o, (int)B, (int)S, (int)H, o_batch_stride, dtype,
                            static_cast<cudaStream_t>(stream));
}

int gdn2_check_device_status(void* stream, uint32_t* detail) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* dw = device_status_word();
  if (!dw) return record_cuda_error(cudaGetLastError());
  uint32_t host = 0;
  GDN2_CUDA_TRY(cudaMemcpyAsync(&host, dw, sizeof(host), cudaMemcpyDeviceToHost, st));
  GDN2_CUDA_TRY(cudaStreamSynchronize(st));
  if (host != 0) GDN2_CUDA_TRY(cudaMemsetAsync(dw, 0, sizeof(host), st));
  if (detail) *detail = host;
  return host == 0 ? GDN2_OK : GDN2_ERR_DEVICE_WAIT;
}

size_t gdn2_oproj_reduce_buffer_bytes(int64_t world, int64_t hidden, size_t* flags_offset) {
  if (world < 1 || world > 64 || hidden < 32 || hidden % 32 != 0 || hidden > (1 << 20)) return 0;
  const size_t slots = align_up((size_t)2 * world * 8 * hidden * sizeof(float), 256);
  if (flags_offset) *flags_offset = slots;
  return slots + align_up((size_t)2 * world * (hidden / 32) * sizeof(uint32_t), 256);
}

int gdn2_oproj_reduce(const gdn2_oproj_reduce_args* a, int dtype, void* stream) {
  if (!a || !a->x || !a->weight || !a->out || !a->epochs) return GDN2_ERR_NULL_POINTER;
  if (!valid_dtype(dtype)) return GDN2_ERR_BAD_DTYPE;
  const int64_t e16 = dtype == GDN2_F32 ? 4 : 8, esz = dtype == GDN2_F32 ? 4 : 2;
  if (a->rows < 1 || a->rows > 8 || a->K < e16 || a->K % e16 != 0 || a->hidden < 32 || a->hidden % 32 != 0 ||
      a->hidden > (1 << 20) || a->rows * a->K * esz > 64 * 1024)
    return GDN2_ERR_BAD_SHAPE;
  if (a->world < 1 || a->world > 64 || a->rank < 0 || a->rank >= a->world) return GDN2_ERR_BAD_SHAPE;
  if (a->world > 1 && (!a->peer_slots || !a->peer_flags)) return GDN2_ERR_NULL_POINTER;
  if (a->wait_cycles < 0 || a->wait_cycles > 2000000000LL) return GDN2_ERR_BAD_SHAPE;
  if (!aligned16(a->x) || !aligned16(a->weight) || !aligned16(a->out)) return GDN2_ERR_MISALIGNED;
  return launch_oproj_reduce(*a, dtype, static_cast<cudaStream_t>(stream));
}

int gdn2_selftest_wait(int64_t limit_cycles, int* gave_up, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL) return GDN2_ERR_BAD_SHAPE;   // about a second at most
  return launch_selftest_wait(limit_cycles, gave_up, static_cast<cudaStream_t>(stream));
}

int gdn2_selftest_mma(const float* a, const float* bt, float* out, void* stream) {
  if (!a || !bt || !out) return GDN2_ERR_NULL_POINTER;
  if (!aligned16(a) || !aligned16(bt) || !aligned16(out)) return GDN2_ERR_MISALIGNED;
  return launch_selftest_mma(a, bt, out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
