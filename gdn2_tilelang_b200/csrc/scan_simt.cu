// Sequential state scan fused with the output, SIMT (CUDA-core) family, and the chunk-parallel
// output from stored chunk states. fp32 arithmetic; any DK <= 128, any DV.
//
// Scan: one 256-thread block per (32-column value tile, batch*head), sequential over chunks, the
// [DK x 32] state tile resident in shared memory. Per chunk (prefill_scan_kernel,
// gdn2/inference.py:446-475 of the reference project):
//     Un = U - W S ;  o = Qg S + tril(Aqk) Un ;  S <- diag(gamma_C) S + KG^T Un
// Optionally the state entering each chunk is stored (state_kernel, gdn2/forward.py:617-620).
//
// Output: one block per (value tile, chunk, batch*head) doing the first two lines from a stored
// chunk state (output_kernel, gdn2/forward.py:710-725).
#include "common.cuh"

namespace gdn2 {

namespace {

constexpr int NV = 32;   // value columns per block


struct ScanSmem {
  float *Ws, *Qs, *As, *Ks, *Us, *Un, *St, *gl;
  __device__ ScanSmem(float* base, int DK) {
    Ws = base;                    // [64][DK]
    Qs = Ws + kChunk * DK;        // [64][DK]
    Ks = Qs + kChunk * DK;        // [64][DK]   KG[t][k]
    As = Ks + kChunk * DK;        // [64][64]
    Us = As + kChunk * kChunk;    // [64][NV]
    Un = Us + kChunk * NV;        // [64][NV]
    St = Un + kChunk * NV;        // [DK][NV]
    gl = St + DK * NV;            // [DK]
  }
  static size_t bytes(int DK) {
    return ((size_t)3 * kChunk * DK + kChunk * kChunk + 2 * kChunk * NV + (size_t)DK * NV + DK) * sizeof(float);
  }
};

template <typename TW>
__device__ __forceinline__ void load_chunk_operands(const WsLayout& L, const WsPtrs& P, int64_t ch, int64_t chv, int lo,
                                                    ScanSmem& s, bool want_kg) {
  using WT = WsTraits<TW>;
  using TV = typename WT::TV;
  constexpr int E = WT::E;
  const int DK = L.DK, DV = L.DV, tid = threadIdx.x;
  const TW* wq = reinterpret_cast<const TW*>(P.wq + (size_t)ch * L.wq_bytes);
  const TV* aqk = reinterpret_cast<const TV*>(P.aqk + (size_t)ch * L.aqk_bytes);
  const TV* kgt = reinterpret_cast<const TV*>(P.kgt + (size_t)ch * L.kgt_bytes);
  const TV* ut = reinterpret_cast<const TV*>(P.ut + (size_t)chv * L.ut_bytes);   // per value head; the rest per key head
  for (int idx = tid; idx < kChunk * DK; idx += 256) {
    const int t = idx / DK, c = idx % DK;
    s.Ws[idx] = to_f32(wq[kc_index<E>(t, c, 2 * kChunk)]);
    s.Qs[idx] = to_f32(wq[kc_index<E>(kChunk + t, c, 2 * kChunk)]);
    if (want_kg) s.Ks[idx] = WT::kg_load(kgt[kc_index<E>(c, t, DK)]);
  }
  for (int idx = tid; idx < kChunk * kChunk; idx += 256)
    s.As[idx] = WT::kg_load(aqk[kc_index<E>(idx / kChunk, idx % kChunk, kChunk)]);
  for (int idx = tid; idx < kChunk * NV; idx += 256) {
    const int t = idx / NV, c = lo + idx % NV;
    s.Us[idx] = c < DV ? WT::u_load(ut[kc_index<E>(c, t, DV)]) : 0.f;
  }
  if (want_kg && tid < DK) s.gl[tid] = P.gl[(size_t)ch * DK + tid];
}

// Un = U - W S and o = Qg S + tril(Aqk) Un for the 8 tokens [wid*8, wid*8+8) and column `lane`.
template <typename TOut>
__device__ __forceinline__ void un_and_output(ScanSmem& s, int DK, int DV, int lo, TOut* __restrict__ o_rows,
                                              size_t o_row_stride) {
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int c = 0; c < DK; ++c) {
    const float sv = s.St[c * NV + lane];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(s.Ws[(wid * 8 + i) * DK + c], sv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) s.Un[(wid * 8 + i) * NV + lane] = s.Us[(wid * 8 + i) * NV + lane] - acc[i];
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int c = 0; c < DK; ++c) {
    const float sv = s.St[c * NV + lane];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(s.Qs[(wid * 8 + i) * DK + c], sv, acc[i]);
  }
  for (int t = 0; t < wid * 8 + 8; ++t) {
    const float un = s.Un[t * NV + lane];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (t <= wid * 8 + i) acc[i] = fmaf(s.As[(wid * 8 + i) * kChunk + t], un, acc[i]);
  }
  if (lo + lane < DV) {
#pragma unroll
    for (int i = 0; i < 8; ++i) o_rows[(size_t)(wid * 8 + i) * o_row_stride + lo + lane] = from_f32<TOut>(acc[i]);
  }
}

template <typename TOut, typename TW>
__global__ void __launch_bounds__(256)
scan_simt_kernel(WsLayout L, WsPtrs P, const float* __restrict__ s0, TOut* __restrict__ o,
                 float* __restrict__ sT, float* __restrict__ hs, int S, int H, int64_t o_bs) {
  const int DK = L.DK, DV = L.DV, NC = S / kChunk;
  const int bh = blockIdx.y, ib = bh / H, ih = bh % H;
  const int lo = blockIdx.x * NV;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  extern __shared__ float sm[];
  ScanSmem s(sm, DK);
  const bool col_ok = lo + lane < DV;

  for (int idx = tid; idx < DK * NV; idx += 256) {
    const int c = idx / NV, d = lo + idx % NV;
    s.St[idx] = (s0 != nullptr && d < DV) ? s0[((size_t)bh * DK + c) * DV + d] : 0.f;
  }
  const int64_t bk = (int64_t)ib * (H / L.rep) + ih / L.rep;       // (batch, key head) whose records this value head reads
  for (int n = 0; n < NC; ++n) {
    const int64_t ch = bk * NC + n;
    __syncthreads();
    load_chunk_operands<TW>(L, P, ch, (int64_t)bh * NC + n, lo, s, true);
    if (hs != nullptr) {
      float* hp = hs + (((size_t)ib * NC + n) * H + ih) * DK * DV;
      for (int idx = tid; idx < DK * NV; idx += 256) {
        const int c = idx / NV, d = lo + idx % NV;
        if (d < DV) hp[(size_t)c * DV + d] = s.St[idx];
      }
    }
    __syncthreads();
    TOut* o_rows = o + (((size_t)ib * o_bs + (size_t)n * kChunk) * H + ih) * DV;
    un_and_output<TOut>(s, DK, DV, lo, o_rows, (size_t)H * DV);
    __syncthreads();
    // state update: warp `wid` owns key rows wid, wid+8, ...
    for (int c = wid; c < DK; c += 8) {
      float acc = s.gl[c] * s.St[c * NV + lane];
      for (int t = 0; t < kChunk; ++t) acc = fmaf(s.Ks[t * DK + c], s.Un[t * NV + lane], acc);
      s.St[c * NV + lane] = acc;
    }
  }
  __syncthreads();
  if (sT != nullptr) {
    for (int idx = tid; idx < DK * NV; idx += 256) {
      const int c = idx / NV, d = lo + idx % NV;
      if (d < DV) sT[((size_t)bh * DK + c) * DV + d] = s.St[idx];
    }
  }
  (void)col_ok;
}

template <typename TOut, typename TW>
__global__ void __launch_bounds__(256)
output_simt_kernel(WsLayout L, WsPtrs P, const float* __restrict__ hs, TOut* __restrict__ o, int S, int H, int64_t o_bs) {
  const int DK = L.DK, DV = L.DV, NC = S / kChunk;
  const int n = blockIdx.y, bh = blockIdx.z, ib = bh / H, ih = bh % H;
  const int lo = blockIdx.x * NV;
  const int tid = threadIdx.x;
  extern __shared__ float sm[];
  ScanSmem s(sm, DK);
  const int64_t ch = ((int64_t)ib * (H / L.rep) + ih / L.rep) * NC + n;
  const float* hp = hs + (((size_t)ib * NC + n) * H + ih) * DK * DV;
  for (int idx = tid; idx < DK * NV; idx += 256) {
    const int c = idx / NV, d = lo + idx % NV;
    s.St[idx] = d < DV ? hp[(size_t)c * DV + d] : 0.f;
  }
  load_chunk_operands<TW>(L, P, ch, (int64_t)bh * NC + n, lo, s, false);
  __syncthreads();
  TOut* o_rows = o + (((size_t)ib * o_bs + (size_t)n * kChunk) * H + ih) * DV;
  un_and_output<TOut>(s, DK, DV, lo, o_rows, (size_t)H * DV);
}

template <typename TOut, typename TW>
int launch_scan_typed(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                      int B, int S, int H, int64_t o_bs, cudaStream_t st) {
  const size_t smem = ScanSmem::bytes(L.DK);
  auto kern = scan_simt_kernel<TOut, TW>;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  dim3 grid((L.DV + NV - 1) / NV, B * H);
  kern<<<grid, 256, smem, st>>>(L, P, s0, static_cast<TOut*>(o), sT, hs, S, H, o_bs);
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

template <typename TOut, typename TW>
int launch_output_typed(const WsLayout& L, const WsPtrs& P, const float* hs, void* o, int B, int S, int H,
                        int64_t o_bs, cudaStream_t st) {
  const size_t smem = ScanSmem::bytes(L.DK);
  auto kern = output_simt_kernel<TOut, TW>;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  dim3 grid((L.DV + NV - 1) / NV, S / kChunk, B * H);
  kern<<<grid, 256, smem, st>>>(L, P, hs, static_cast<TOut*>(o), S, H, o_bs);
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace

int launch_scan_simt(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                     int B, int S, int H, int64_t o_bs, int dtype, cudaStream_t st) {
  if (L.esz != 4) return GDN2_ERR_UNSUPPORTED;   // 16-bit records belong to the tensor-core family's kernels
  switch (dtype) {
    case GDN2_F32: return launch_scan_typed<float, float>(L, P, s0, o, sT, hs, B, S, H, o_bs, st);
    case GDN2_BF16: return launch_scan_typed<__nv_bfloat16, float>(L, P, s0, o, sT, hs, B, S, H, o_bs, st);
    case GDN2_F16: return launch_scan_typed<__half, float>(L, P, s0, o, sT, hs, B, S, H, o_bs, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

int launch_output_simt(const WsLayout& L, const WsPtrs& P, const float* hs, void* o, int B, int S, int H,
                       int64_t o_bs, int dtype, cudaStream_t st) {
  if (L.esz != 4) return GDN2_ERR_UNSUPPORTED;
  switch (dtype) {
    case GDN2_F32: return launch_output_typed<float, float>(L, P, hs, o, B, S, H, o_bs, st);
    case GDN2_BF16: return launch_output_typed<__nv_bfloat16, float>(L, P, hs, o, B, S, H, o_bs, st);
    case GDN2_F16: return launch_output_typed<__half, float>(L, P, hs, o, B, S, H, o_bs, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

}  // namespace gdn2
