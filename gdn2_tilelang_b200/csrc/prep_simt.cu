// Chunk-local stage of the chunkwise forward, SIMT (CUDA-core) family: any DK <= 128 (multiple
// of 8), any DV (multiple of 4), fp32 arithmetic throughout. One 256-thread block per
// (chunk, batch*head).
//
// Every entry of the two intra-chunk matrices is evaluated with the exact pairwise decay
//     sum_c x_r[c] * k_s[c] * exp2(G_r[c] - G_s[c]),   r >= s   (exponent <= 0 by construction)
// which is the form the reference uses only for its diagonal sub-blocks (intra_diag_kernel,
// gdn2/forward.py:220-235 of the reference project); using it everywhere makes this family safe
// for arbitrarily fast decay without any reference-row factorisation. The inverse (I + Tm)^-1 is
// built column by column with forward substitution (solve_kernel, gdn2/forward.py:424-434), then
// W = Ai E, U = Ai (w*v), KG and Qg follow wy_kernel (gdn2/forward.py:512-533) and the query
// scaling of prefill_scan_kernel (gdn2/inference.py:461).
//
// This family also serves as the exact path for chunks the tensor-core family flags as decaying
// too fast for its factorised diagonal blocks (`only_flagged`).
#include "common.cuh"

namespace gdn2 {

namespace {


// The whole chunk-local stage for chunk n of (batch, KEY head) bk, by one 256-thread block: everything that depends
// on q, k, b, g once, then U = Ai (w*v) for each of the H / HK value heads that share the key head.
template <typename TIn, typename TW>
__device__ __forceinline__ void prep_simt_chunk(const TIn* __restrict__ q, const TIn* __restrict__ k,
                                                const TIn* __restrict__ v, const float* __restrict__ g,
                                                const TIn* __restrict__ b, const TIn* __restrict__ w,
                                                const WsLayout& L, const WsPtrs& P, int S, int H, int HK, int64_t in_bs,
                                                float scale, int n, int bk) {
  constexpr int BS = kChunk;
  using WT = WsTraits<TW>;
  using TV = typename WT::TV;
  constexpr int E = WT::E;
  const int DK = L.DK, DV = L.DV;
  const int NC = S / BS;
  const int ib = bk / HK, ihk = bk % HK;
  const int64_t ch = (int64_t)bk * NC + n;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;

  extern __shared__ float sm[];
  float* Gs = sm;                    // [BS][DK] cumulative log2 decay
  float* ks = Gs + BS * DK;          // [BS][DK] k
  float* es = ks + BS * DK;          // [BS][DK] b*k, later E = b*k*gamma
  float* qs = es + BS * DK;          // [BS][DK] q, later the w*v tiles
  float* Tm = qs + BS * DK;          // [BS][BS] strictly lower
  float* Aq = Tm + BS * BS;          // [BS][BS] lower incl. diagonal (scaled)
  float* Ai = Aq + BS * BS;          // [BS][BS] (I + Tm)^-1

  const size_t tok0 = ((size_t)ib * in_bs + (size_t)n * BS) * HK + ihk;   // token index of row 0 (stride HK per row)
  for (int idx = tid; idx < BS * DK; idx += 256) {
    const int t = idx / DK, c = idx % DK;
    const size_t gi = (tok0 + (size_t)t * HK) * DK + c;
    const float kk = to_f32(k[gi]);
    ks[idx] = kk;
    qs[idx] = to_f32(q[gi]);
    es[idx] = to_f32(b[gi]) * kk;
    Gs[idx] = g[gi];
  }
  for (int idx = tid; idx < BS * BS; idx += 256) { Tm[idx] = 0.f; Aq[idx] = 0.f; Ai[idx] = 0.f; }
  __syncthreads();
  if (tid < DK) {
    float run = 0.f;
    for (int t = 0; t < BS; ++t) { run += Gs[t * DK + tid]; Gs[t * DK + tid] = run * kLog2e; }
  }
  __syncthreads();

  // pairwise matrices: warp `wid` takes rows {wid+8j, 63-(wid+8j)}, 65 pairs per row pair
  for (int j = 0; j < 4; ++j) {
    for (int half = 0; half < 2; ++half) {
      const int r = half ? (BS - 1 - (wid + 8 * j)) : (wid + 8 * j);
      for (int s = 0; s <= r; ++s) {
        float aq = 0.f, ae = 0.f;
        for (int c = lane; c < DK; c += 32) {
          const float kd = ks[s * DK + c] * exp2f(Gs[r * DK + c] - Gs[s * DK + c]);
          aq = fmaf(qs[r * DK + c], kd, aq);
          ae = fmaf(es[r * DK + c], kd, ae);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) {
          aq += __shfl_xor_sync(0xffffffffu, aq, off);
          ae += __shfl_xor_sync(0xffffffffu, ae, off);
        }
        if (lane == 0) {
          Aq[r * BS + s] = aq * scale;
          if (s < r) Tm[r * BS + s] = ae;
        }
      }
    }
  }
  __syncthreads();

  // inverse by columns: thread j solves (I + Tm) x = e_j
  if (tid < BS) {
    const int j = tid;
    Ai[j * BS + j] = 1.f;
    for (int r = j + 1; r < BS; ++r) {
      float acc = 0.f;
      for (int s = j; s < r; ++s) acc = fmaf(Tm[r * BS + s], Ai[s * BS + j], acc);
      Ai[r * BS + j] = -acc;
    }
  }
  // outputs that need only G, q, k: Aqk image, Qg rows, KG^T image, gamma_last; E in place
  TW* wq = reinterpret_cast<TW*>(P.wq + (size_t)ch * L.wq_bytes);
  TV* aqk = reinterpret_cast<TV*>(P.aqk + (size_t)ch * L.aqk_bytes);
  TV* kgt = reinterpret_cast<TV*>(P.kgt + (size_t)ch * L.kgt_bytes);
  float* gl = P.gl + (size_t)ch * DK;
  for (int idx = tid; idx < BS * BS; idx += 256) {
    const int r = idx / BS, s = idx % BS;
    aqk[kc_index<E>(r, s, BS)] = WT::kg_store(Aq[idx]);
  }
  for (int idx = tid; idx < BS * DK; idx += 256) {
    const int t = idx / DK, c = idx % DK;
    const float G = Gs[idx];
    const float gam = exp2f(G);
    wq[kc_index<E>(BS + t, c, 2 * BS)] = from_f32<TW>(scale * qs[idx] * gam);
    kgt[kc_index<E>(c, t, DK)] = WT::kg_store(ks[idx] * exp2f(Gs[(BS - 1) * DK + c] - G));
    es[idx] *= gam;
  }
  if (tid < DK) gl[tid] = exp2f(Gs[(BS - 1) * DK + tid]);
  __syncthreads();

  // W = Ai E
  for (int idx = tid; idx < BS * DK; idx += 256) {
    const int r = idx / DK, c = idx % DK;
    float acc = 0.f;
    for (int s = 0; s <= r; ++s) acc = fmaf(Ai[r * BS + s], es[s * DK + c], acc);
    wq[kc_index<E>(r, c, 2 * BS)] = from_f32<TW>(acc);
  }
  // U = Ai (w*v) for every value head of this key head, value columns in tiles of DK
  const int rep = H / HK;
  for (int hr = 0; hr < rep; ++hr) {
    const int ih = ihk * rep + hr;
    const size_t tok0v = ((size_t)ib * in_bs + (size_t)n * BS) * H + ih;
    TV* ut = reinterpret_cast<TV*>(P.ut + (size_t)(((int64_t)ib * H + ih) * NC + n) * L.ut_bytes);
    for (int c0 = 0; c0 < DV; c0 += DK) {
      const int cw = min(DK, DV - c0);
      __syncthreads();
      for (int idx = tid; idx < BS * cw; idx += 256) {
        const int t = idx / cw, c = idx % cw;
        const size_t gi = (tok0v + (size_t)t * H) * DV + c0 + c;
        qs[t * DK + c] = to_f32(w[gi]) * to_f32(v[gi]);
      }
      __syncthreads();
      for (int idx = tid; idx < BS * cw; idx += 256) {
        const int r = idx / cw, c = idx % cw;
        float acc = 0.f;
        for (int s = 0; s <= r; ++s) acc = fmaf(Ai[r * BS + s], qs[s * DK + c], acc);
        ut[kc_index<E>(c0 + c, r, DV)] = WT::u_store(acc);
      }
    }
  }
}

template <typename TIn, typename TW>
__global__ void __launch_bounds__(256)
prep_simt_kernel(const TIn* __restrict__ q, const TIn* __restrict__ k, const TIn* __restrict__ v,
                 const float* __restrict__ g, const TIn* __restrict__ b, const TIn* __restrict__ w,
                 WsLayout L, WsPtrs P, int S, int H, int HK, int64_t in_bs, float scale) {
  prep_simt_chunk<TIn, TW>(q, k, v, g, b, w, L, P, S, H, HK, in_bs, scale, blockIdx.x, blockIdx.y);
}

// Exact redo of the chunks the tensor-core kernel flagged: a fixed small grid walks the compacted list
// (workspace ints: flags[nch], list[nch], count), so a call with nothing flagged costs two tiny launches.
template <typename TIn, typename TW>
__global__ void __launch_bounds__(256)
prep_simt_flagged_kernel(const TIn* __restrict__ q, const TIn* __restrict__ k, const TIn* __restrict__ v,
                         const float* __restrict__ g, const TIn* __restrict__ b, const TIn* __restrict__ w,
                         WsLayout L, WsPtrs P, int S, int H, int HK, int64_t in_bs, float scale) {
  const int NC = S / kChunk;
  const int* list = P.flags + L.nch;
  const int count = P.flags[2 * L.nch];
  for (int li = blockIdx.x; li < count; li += gridDim.x) {
    const int ch = list[li];
    prep_simt_chunk<TIn, TW>(q, k, v, g, b, w, L, P, S, H, HK, in_bs, scale, ch % NC, ch / NC);
    __syncthreads();                                   // shared memory is reused by the next chunk
  }
}

template <typename TIn, typename TW>
int launch_typed(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                 const WsLayout& L, const WsPtrs& P, int B, int S, int H, int HK, int64_t in_bs, float scale,
                 bool only_flagged, cudaStream_t st) {
  const size_t smem = ((size_t)4 * kChunk * L.DK + 3 * kChunk * kChunk) * sizeof(float);
  const TIn* tq = static_cast<const TIn*>(q); const TIn* tk = static_cast<const TIn*>(k);
  const TIn* tv = static_cast<const TIn*>(v); const TIn* tb = static_cast<const TIn*>(b);
  const TIn* tw = static_cast<const TIn*>(w);
  if (only_flagged) {
    auto kern = prep_simt_flagged_kernel<TIn, TW>;
    GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
    // the tensor-core kernel has appended the flagged chunks to the list behind the flags
    const int nch = (int)L.nch;
    kern<<<nch < 296 ? nch : 296, 256, smem, st>>>(tq, tk, tv, g, tb, tw, L, P, S, H, HK, in_bs, scale);
  } else {
    auto kern = prep_simt_kernel<TIn, TW>;
    GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
    dim3 grid(S / kChunk, B * HK);
    kern<<<grid, 256, smem, st>>>(tq, tk, tv, g, tb, tw, L, P, S, H, HK, in_bs, scale);
  }
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace

int launch_prep_simt(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                     const WsLayout& L, const WsPtrs& P, int B, int S, int H, int HK, int64_t in_bs, float scale,
                     int dtype, bool only_flagged, cudaStream_t st) {
  if (L.esz == 4) {
    switch (dtype) {
      case GDN2_F32: return launch_typed<float, float>(q, k, v, g, b, w, L, P, B, S, H, HK, in_bs, scale, only_flagged, st);
      case GDN2_BF16: return launch_typed<__nv_bfloat16, float>(q, k, v, g, b, w, L, P, B, S, H, HK, in_bs, scale, only_flagged, st);
      case GDN2_F16: return launch_typed<__half, float>(q, k, v, g, b, w, L, P, B, S, H, HK, in_bs, scale, only_flagged, st);
      default: return GDN2_ERR_BAD_DTYPE;
    }
  }
  if (dtype != GDN2_BF16) return GDN2_ERR_UNSUPPORTED;
  return launch_typed<__nv_bfloat16, __nv_bfloat16>(q, k, v, g, b, w, L, P, B, S, H, HK, in_bs, scale, only_flagged, st);
}

}  // namespace gdn2
