// Recurrent decode: n tokens per launch, the fp32 state streamed from HBM once and back once.
//
// Per token (reference arithmetic, gdn2/inference.py:136-151 and :279-299 of the reference project):
//     S <- diag(exp g) S ;  u = w*v - S^T (b*k) ;  S <- S + k u^T ;  o = scale * S^T q
// evaluated here as three fused multiply-adds per state element:
//     read += S * (a * b*k)         (a = exp g, so this is the read of the decayed state)
//     S     = a * S + k * u
//     out  += S * (scale * q)
//
// Fast kernel (DK = DV = 128): one 128-thread block per (batch, head). Warp w owns key rows
// [32w, 32w+32); lane l owns value columns [4l, 4l+4), so every state access is a 128-bit load
// or store and a warp covers a full 512-byte row. The state tile lives in registers (128 per
// thread) for all n tokens; the reductions over key rows are in-thread sums followed by one
// 4-way cross-warp sum through shared memory.
//
// Generic kernel: any DK <= 256 and any DV, one block per (32-column value tile, batch, head).
#include "common.cuh"

namespace gdn2 {

namespace {

constexpr int kTokBatch = 8;   // token vectors staged in shared memory per barrier round

template <typename T>
__global__ void __launch_bounds__(128, 3)
decode_d128_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const float* __restrict__ g, const T* __restrict__ b, const T* __restrict__ w,
                   float* __restrict__ state, T* __restrict__ o, int n, int H, int64_t in_bs, int64_t o_bs, float scale) {
  constexpr int D = 128;
  const int bh = blockIdx.x;
  const int ib = bh / H, ih = bh % H;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;

  __shared__ float s_abk[kTokBatch][D];   // exp(g) * b * k
  __shared__ float s_a[kTokBatch][D];     // exp(g)
  __shared__ float s_k[kTokBatch][D];
  __shared__ float s_q[kTokBatch][D];     // scale * q
  __shared__ float s_wv[kTokBatch][D];    // w * v
  __shared__ float4 s_red[2][4][32];      // cross-warp partial sums, double buffered

  float4 S[32];
  float4* gS = reinterpret_cast<float4*>(state + ((size_t)bh * D + wid * 32) * D) + lane;
#pragma unroll
  for (int i = 0; i < 32; ++i) S[i] = __ldcs(gS + i * (D / 4));

  for (int t0 = 0; t0 < n; t0 += kTokBatch) {
    const int nt = min(kTokBatch, n - t0);
    __syncthreads();   // previous round's vectors are no longer read
    for (int j = 0; j < nt; ++j) {
      const size_t tok = ((size_t)ib * in_bs + (t0 + j)) * H + ih;
      const float a = exp2f(g[tok * D + tid] * kLog2e);
      const float kk = to_f32(k[tok * D + tid]);
      s_a[j][tid] = a;
      s_abk[j][tid] = a * to_f32(b[tok * D + tid]) * kk;
      s_k[j][tid] = kk;
      s_q[j][tid] = to_f32(q[tok * D + tid]) * scale;
      s_wv[j][tid] = to_f32(w[tok * D + tid]) * to_f32(v[tok * D + tid]);
    }
    __syncthreads();

    for (int j = 0; j < nt; ++j) {
      // read of the decayed state with the erase row
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float c = s_abk[j][wid * 32 + i];
        acc.x = fmaf(S[i].x, c, acc.x); acc.y = fmaf(S[i].y, c, acc.y);
        acc.z = fmaf(S[i].z, c, acc.z); acc.w = fmaf(S[i].w, c, acc.w);
      }
      s_red[0][wid][lane] = acc;
      __syncthreads();
      float4 u = reinterpret_cast<const float4*>(s_wv[j])[lane];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float4 p = s_red[0][x][lane];
        u.x -= p.x; u.y -= p.y; u.z -= p.z; u.w -= p.w;
      }
      // decay + rank-1 write, then the output read
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float a = s_a[j][wid * 32 + i], kk = s_k[j][wid * 32 + i], qq = s_q[j][wid * 32 + i];
        S[i].x = fmaf(a, S[i].x, kk * u.x); S[i].y = fmaf(a, S[i].y, kk * u.y);
        S[i].z = fmaf(a, S[i].z, kk * u.z); S[i].w = fmaf(a, S[i].w, kk * u.w);
        acc.x = fmaf(S[i].x, qq, acc.x); acc.y = fmaf(S[i].y, qq, acc.y);
        acc.z = fmaf(S[i].z, qq, acc.z); acc.w = fmaf(S[i].w, qq, acc.w);
      }
      s_red[1][wid][lane] = acc;
      __syncthreads();
      if (wid == 0) {
        float4 r = s_red[1][0][lane];
#pragma unroll
        for (int x = 1; x < 4; ++x) {
          const float4 p = s_red[1][x][lane];
          r.x += p.x; r.y += p.y; r.z += p.z; r.w += p.w;
        }
        T* po = o + (((size_t)ib * o_bs + (t0 + j)) * H + ih) * D + lane * 4;
        po[0] = from_f32<T>(r.x); po[1] = from_f32<T>(r.y); po[2] = from_f32<T>(r.z); po[3] = from_f32<T>(r.w);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) __stcs(gS + i * (D / 4), S[i]);
}

// Any DK <= 4*MAXR, any DV. Block = 128 threads = 4 warps; lane = value column inside a 32-wide
// tile, warp w owns key rows [w*rpw, (w+1)*rpw) with rpw = ceil(DK/4).
template <typename T, int MAXR>
__global__ void __launch_bounds__(128)
decode_generic_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      const float* __restrict__ g, const T* __restrict__ b, const T* __restrict__ w,
                      float* __restrict__ state, T* __restrict__ o, int n, int H, int DK, int DV, int64_t in_bs,
                      int64_t o_bs, float scale) {
  const int bh = blockIdx.y;
  const int ib = bh / H, ih = bh % H;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int dv = blockIdx.x * 32 + lane;
  const bool col_ok = dv < DV;
  const int rpw = (DK + 3) / 4;
  const int r0 = wid * rpw;

  extern __shared__ float smem[];
  float* s_abk = smem;            // [DK]
  float* s_a = s_abk + DK;
  float* s_k = s_a + DK;
  float* s_q = s_k + DK;
  __shared__ float s_red[2][4][32];

  float S[MAXR];
#pragma unroll
  for (int i = 0; i < MAXR; ++i) {
    const int r = r0 + i;
    S[i] = (i < rpw && r < DK && col_ok) ? state[((size_t)bh * DK + r) * DV + dv] : 0.f;
  }
  for (int t = 0; t < n; ++t) {
    const size_t tok = ((size_t)ib * in_bs + t) * H + ih;
    const size_t otok = ((size_t)ib * o_bs + t) * H + ih;
    __syncthreads();
    for (int c = tid; c < DK; c += 128) {
      const float a = exp2f(g[tok * DK + c] * kLog2e);
      const float kk = to_f32(k[tok * DK + c]);
      s_a[c] = a; s_k[c] = kk;
      s_abk[c] = a * to_f32(b[tok * DK + c]) * kk;
      s_q[c] = to_f32(q[tok * DK + c]) * scale;
    }
    const float wv = col_ok ? to_f32(w[tok * DV + dv]) * to_f32(v[tok * DV + dv]) : 0.f;
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < MAXR; ++i) {
      const int r = r0 + i;
      if (i < rpw && r < DK) acc = fmaf(S[i], s_abk[r], acc);
    }
    s_red[0][wid][lane] = acc;
    __syncthreads();
    const float u = wv - (s_red[0][0][lane] + s_red[0][1][lane] + s_red[0][2][lane] + s_red[0][3][lane]);
    acc = 0.f;
#pragma unroll
    for (int i = 0; i < MAXR; ++i) {
      const int r = r0 + i;
      if (i < rpw && r < DK) {
        S[i] = fmaf(s_a[r], S[i], s_k[r] * u);
        acc = fmaf(S[i], s_q[r], acc);
      }
    }
    s_red[1][wid][lane] = acc;
    __syncthreads();
    if (wid == 0 && col_ok)
      o[otok * DV + dv] = from_f32<T>(s_red[1][0][lane] + s_red[1][1][lane] + s_red[1][2][lane] + s_red[1][3][lane]);
  }
#pragma unroll
  for (int i = 0; i < MAXR; ++i) {
    const int r = r0 + i;
    if (i < rpw && r < DK && col_ok) state[((size_t)bh * DK + r) * DV + dv] = S[i];
  }
}

template <typename T>
int launch_typed(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                 float* state, void* o, int B, int n, int H, int DK, int DV, int64_t in_bs, int64_t o_bs, float scale,
                 cudaStream_t st) {
  const T* tq = static_cast<const T*>(q); const T* tk = static_cast<const T*>(k);
  const T* tv = static_cast<const T*>(v); const T* tb = static_cast<const T*>(b);
  const T* tw = static_cast<const T*>(w); T* to = static_cast<T*>(o);
  if (DK == 128 && DV == 128) {
    decode_d128_kernel<T><<<B * H, 128, 0, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, in_bs, o_bs, scale);
  } else {
    dim3 grid((DV + 31) / 32, B * H);
    const size_t sm = (size_t)4 * DK * sizeof(float);
    if (DK <= 64)
      decode_generic_kernel<T, 16><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, DK, DV, in_bs, o_bs, scale);
    else if (DK <= 128)
      decode_generic_kernel<T, 32><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, DK, DV, in_bs, o_bs, scale);
    else
      decode_generic_kernel<T, 64><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, DK, DV, in_bs, o_bs, scale);
  }
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace

int launch_decode(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                  float* state, void* o, int B, int n, int H, int DK, int DV, int64_t in_bs, int64_t o_bs,
                  float scale, int dtype, cudaStream_t st) {
  switch (dtype) {
    case GDN2_F32: return launch_typed<float>(q, k, v, g, b, w, state, o, B, n, H, DK, DV, in_bs, o_bs, scale, st);
    case GDN2_BF16: return launch_typed<__nv_bfloat16>(q, k, v, g, b, w, state, o, B, n, H, DK, DV, in_bs, o_bs, scale, st);
    case GDN2_F16: return launch_typed<__half>(q, k, v, g, b, w, state, o, B, n, H, DK, DV, in_bs, o_bs, scale, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

}  // namespace gdn2
