// Shared definitions for the GDN-2 sm_100a kernels: element conversion, the workspace layout
// that the chunk-local stage writes and the scan reads, and launch-error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gdn2_b200.h"

namespace gdn2 {

constexpr int kChunk = 64;                       // tokens per chunk (BS)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kValScale = 256.f;               // tensor-core family: KGT = 256*KG, UT = U/256 (fp16)

// ---------------------------------------------------------------- element conversion

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Round to the nearest tf32 (10-bit mantissa). tcgen05.mma kind::tf32 reads fp32 words and ignores
// the low 13 mantissa bits, i.e. truncates; rounding operands first removes that bias, which
// otherwise shows up as a systematic ~1e-3 shrink of products of two tf32 operands.
__device__ __forceinline__ float tf32_rn(float x) {
  // round to nearest, ties away from zero, on the bit pattern: add half a tf32 unit, drop the low 13 bits
  // (a carry into the exponent is the correct rounding; infinities and NaNs do not occur on these paths)
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// ---------------------------------------------------------------- workspace layout
//
// One record set per chunk-head. The records that depend on q, k, b, g only (WQ, AQK, KGT, GL) exist once per
// KEY head, index (b*HK + hk)*NC + n; UT exists per VALUE head, index (b*H + h)*NC + n, and value head h reads the
// records of key head h / (H/HK) (grouped-query heads share them; with HK = H the two indices coincide). All matrices are stored as
// "K-chunked" operand images: a matrix with R rows and a reduction axis of K elements is an
// array [K/E][R][E] where E elements fill 16 bytes (E = 8 for bf16, 4 for fp32). This is the
// no-swizzle, K-major shared-memory layout tcgen05.mma reads (8 rows x 16 bytes core matrices,
// 128 bytes between 8-row groups, R*16 bytes between adjacent K chunks), so the scan can bring a
// record on chip with one bulk copy and hand it to the tensor core unchanged.
//
//   WQ   rows 0..63 = W (per token), rows 64..127 = Qg = scale*q*gamma (per token); K = DK; type TW
//   AQK  rows = query token r, K = key token s; lower triangular incl. diagonal;      type TW
//   KGT  rows = key channel, K = token: k * gamma_C / gamma_t;                         type TV
//   UT   rows = value channel, K = token: U;                                           type TV
//   GL   gamma at the chunk's last token, [DK];                                        fp32
//
// SIMT family: TW = TV = fp32. Tensor-core family: TW = bf16 and TV = fp16 with a fixed power-of-two
// scale (KGT holds 256 * KG, UT holds U / 256): fp16 carries the same 11 significant bits as the tf32
// the value path needs (bf16's 8 are not enough), the scale keeps |U| up to 1.6e7 finite while
// everything above 0.016 stays a normal number, and the product (Un/256) * (256 KG) is exact.

struct WsLayout {
  int64_t nch;        // number of key chunk-heads, B * HK * S/64: records WQ, AQK, KG^T, gamma_last, flags
  int64_t nch_v;      // number of value chunk-heads, B * H * S/64: records U^T
  int64_t BH;         // (batch, value head) pairs
  int rep;            // value heads per key head, H / HK (grouped-query heads; 1 = every head has its own q, k, b, g)
  int DK, DV;
  int esz;            // bytes per TW element (2 or 4); TV has the same size
  int nseg;           // sequence segments of the tensor-core scan (1 = one block per head walks the whole sequence)
  int nseg_guarded;   // 1 = that cut launches more blocks than SMs and is taken back on the device when the decay is slow
  size_t wq_bytes, aqk_bytes, kgt_bytes, ut_bytes, gl_bytes;   // per chunk-head
  size_t off_wq, off_aqk, off_kgt, off_ut, off_gl, off_flags, off_seg, total;
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Segments the tensor-core scan cuts a sequence of NC chunks into when a GPU holds BH (batch, head) pairs.
// The first pass runs nseg "local" blocks and nseg - 1 "transition" blocks per pair, one per SM; the correction
// pass may have to redo whole segments (slow decay), so the cut costs up to two chains of NC / nseg chunks.
//   * While all 2 nseg - 1 blocks per pair fit on 144 SMs at once and nseg >= 3, the cut can only shorten the
//     chain: it is made unconditionally.
//   * Otherwise (two segments, or local blocks that fit while the transition blocks on top of them do not) the
//     cut pays only when the transition blocks end after a few chunks, which they do when the decay makes the
//     carried state vanish quickly. That cut is "guarded": a decay check on the device takes it back for slowly
//     decaying inputs. Its segments are at least 24 chunks, twice what the check looks at.
// A segment is at least 8 chunks; 1 = no cut.
__host__ __device__ inline int scan_segments(int64_t BH, int64_t NC, int* guarded) {
  int64_t fit = (144 / BH + 1) / 2, over = 144 / BH, cap = NC / 8 < 16 ? NC / 8 : 16;
  if (fit > cap) fit = cap;
  if (over > cap) over = cap;
  *guarded = 0;
  if (fit >= 3) return (int)fit;
  for (int64_t n = over > fit ? over : fit; n >= 2; --n)
    if (NC / n >= 24) {
      *guarded = 1;
      return (int)n;
    }
  return 1;
}

__host__ inline WsLayout make_ws_layout(int64_t B, int64_t S, int64_t H, int64_t HK, int DK, int DV, int esz,
                                        bool allow_segments = false) {
  WsLayout L;
  L.nch = B * HK * (S / kChunk);
  L.nch_v = B * H * (S / kChunk);
  L.BH = B * H;
  L.rep = (int)(H / HK);
  L.DK = DK; L.DV = DV; L.esz = esz;
  L.nseg_guarded = 0;
  L.nseg = (allow_segments && esz == 2) ? scan_segments(B * H, S / kChunk, &L.nseg_guarded) : 1;
  L.wq_bytes = (size_t)2 * kChunk * DK * esz;
  L.aqk_bytes = (size_t)kChunk * kChunk * esz;
  L.kgt_bytes = (size_t)DK * kChunk * esz;
  L.ut_bytes = (size_t)DV * kChunk * esz;
  L.gl_bytes = (size_t)DK * 4;
  size_t off = 0;
  L.off_wq = off;   off = align_up(off + L.wq_bytes * L.nch, 1024);
  L.off_aqk = off;  off = align_up(off + L.aqk_bytes * L.nch, 1024);
  L.off_kgt = off;  off = align_up(off + L.kgt_bytes * L.nch, 1024);
  L.off_ut = off;   off = align_up(off + L.ut_bytes * L.nch_v, 1024);
  L.off_gl = off;   off = align_up(off + L.gl_bytes * L.nch, 1024);
  L.off_flags = off; off = align_up(off + sizeof(int) * (2 * L.nch + 4), 1024);   // flags, compacted list, count
  // per (batch, head) and segment: transition T_j, local final state C_j, true entering state (fp32 [DK, DV]
  // each), then one int per (batch, head, segment): the chunks the correction pass has to redo; one mode word
  L.off_seg = off;
  if (L.nseg > 1)
    off = align_up(off + (size_t)B * H * L.nseg * ((size_t)3 * DK * DV * 4 + sizeof(int)) + sizeof(int), 1024);
  L.total = off;
  return L;
}

// element offset of (row, kk) inside a K-chunked image with R rows and E elements per 16 bytes
template <int E> __host__ __device__ __forceinline__ int kc_index(int row, int kk, int R) {
  return ((kk / E) * R + row) * E + (kk % E);
}

struct WsPtrs {
  char* wq; char* aqk; char* kgt; char* ut; float* gl; int* flags;
  float* seg_t; float* seg_c; float* seg_in; int* seg_stop; int* seg_mode;   // segment records of the cut scan (nseg > 1)
};

__host__ inline WsPtrs ws_pointers(void* base, const WsLayout& L) {
  char* p = static_cast<char*>(base);
  WsPtrs P{p + L.off_wq, p + L.off_aqk, p + L.off_kgt, p + L.off_ut, reinterpret_cast<float*>(p + L.off_gl),
           reinterpret_cast<int*>(p + L.off_flags), nullptr, nullptr, nullptr, nullptr, nullptr};
  if (L.nseg > 1) {
    const size_t mats = (size_t)L.BH * L.nseg * L.DK * L.DV;      // floats per record kind
    P.seg_t = reinterpret_cast<float*>(p + L.off_seg);
    P.seg_c = P.seg_t + mats;
    P.seg_in = P.seg_c + mats;
    P.seg_stop = reinterpret_cast<int*>(P.seg_in + mats);
    P.seg_mode = P.seg_stop + (size_t)L.BH * L.nseg;
  }
  return P;
}

// Per-family element types of the workspace: TW for WQ, TV (+ scales) for AQK/KGT/UT
// (AQK and KGT hold 256 * value, UT holds value / 256 in the 16-bit family).
template <typename TW> struct WsTraits;
template <> struct WsTraits<float> {
  using TV = float;
  static constexpr int E = 4;                       // elements per 16 bytes (both TW and TV)
  static __device__ __forceinline__ float kg_store(float x) { return x; }
  static __device__ __forceinline__ float u_store(float x) { return x; }
  static __device__ __forceinline__ float kg_load(float x) { return x; }
  static __device__ __forceinline__ float u_load(float x) { return x; }
};
template <> struct WsTraits<__nv_bfloat16> {
  using TV = __half;
  static constexpr int E = 8;
  static __device__ __forceinline__ __half kg_store(float x) { return __float2half_rn(x * kValScale); }
  static __device__ __forceinline__ __half u_store(float x) { return __float2half_rn(x * (1.f / kValScale)); }
  static __device__ __forceinline__ float kg_load(__half x) { return __half2float(x) * (1.f / kValScale); }
  static __device__ __forceinline__ float u_load(__half x) { return __half2float(x) * kValScale; }
};

// ---------------------------------------------------------------- host-side error plumbing

int record_cuda_error(cudaError_t e);   // stores e for gdn2_last_cuda_error(), returns GDN2_ERR_CUDA

#define GDN2_CUDA_TRY(expr)                                     \
  do {                                                          \
    cudaError_t e__ = (expr);                                   \
    if (e__ != cudaSuccess) return gdn2::record_cuda_error(e__); \
  } while (0)

// Device status word: kernels OR a code into it when a bounded wait runs out.
uint32_t* device_status_word();   // device pointer for the current device (lazily initialised)
int device_sm_count();            // streaming multiprocessors of the current device
// raises the dynamic shared-memory limit of `kernel` to `bytes` on the current device, once per (kernel, device)
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);

// ---------------------------------------------------------------- launchers (one per .cu file)

// H = value heads, HK = key heads (H % HK == 0): q, k, b, g are [.., HK, DK], v, w, o [.., H, DV]
int launch_decode(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                  float* state, void* o, int B, int n, int H, int HK, int DK, int DV, int64_t in_bs, int64_t o_bs,
                  float scale, int dtype, cudaStream_t st);
int launch_prep_simt(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                     const WsLayout& L, const WsPtrs& P, int B, int S, int H, int HK, int64_t in_bs, float scale,
                     int dtype, bool only_flagged, cudaStream_t st);
int launch_scan_simt(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                     int B, int S, int H, int64_t o_bs, int dtype, cudaStream_t st);
int launch_output_simt(const WsLayout& L, const WsPtrs& P, const float* hs, void* o, int B, int S, int H,
                       int64_t o_bs, int dtype, cudaStream_t st);
int launch_prep_tc(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                   const WsLayout& L, const WsPtrs& P, int B, int S, int H, int HK, int64_t in_bs, float scale,
                   cudaStream_t st);
int launch_scan_tc(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                   int B, int S, int H, int64_t o_bs, const gdn2_gated_norm* norm, int part, cudaStream_t st);
int launch_output_tc(const WsLayout& L, const WsPtrs& P, const float* hs, void* o, int B, int S, int H, int64_t o_bs,
                     cudaStream_t st);
int launch_oproj_reduce(const gdn2_oproj_reduce_args& a, int dtype, cudaStream_t st);
int launch_selftest_wait(long long limit_cycles, int* gave_up, cudaStream_t st);
int launch_selftest_mma(const float* a, const float* bt, float* out, cudaStream_t st);

}  // namespace gdn2
