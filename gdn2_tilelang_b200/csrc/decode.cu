// Recurrent decode: n tokens per launch, the fp32 state streamed from HBM once and back once.
//
// Per token (reference arithmetic, gdn2/inference.py:136-151 and :279-299 of the reference project):
//     S <- diag(exp g) S ;  u = w*v - S^T (b*k) ;  S <- S + k u^T ;  o = scale * S^T q
// evaluated here as three fused multiply-adds per state element:
//     read += S * (a * b*k)         (a = exp g, so this is the read of the decayed state)
//     S     = a * S + k * u
//     out  += S * (scale * q)
//
// Fast kernel (DK = DV = 128): one 128-thread block per (batch, head). Warp w owns value columns
// [32w, 32w+32); inside the warp, 8 lanes x 4 columns cover those and the 4 lane groups split the key
// rows into 32-row slabs, so every state access is a 128-bit load/store on full 128-byte lines and
// the tile (128 registers per thread) stays in registers for all n tokens. Reductions over key rows
// are in-thread sums plus two shuffle steps: no shared-memory reduction, no block barrier per token.
// The output is formed from the OLD state in the same sweep as the read,
//     o = scale*q^T (a*S + k u^T) = sum_r (scale*q_r*a_r) S_r + (scale*q.k) u,
// and all sweeps use packed f32x2 arithmetic with per-row coefficients fetched as 128-bit broadcasts.
//
// Generic kernel: any DK <= 256 and any DV, one block per (32-column value tile, batch, head).
#include "common.cuh"

namespace gdn2 {

// decode_blocked.cu: blocks of up to 8 tokens without a per-token dependent sweep (DK = DV = 128)
template <typename T>
int launch_decode_blocked(const T* q, const T* k, const T* v, const float* g, const T* b, const T* w, float* state,
                          T* o, int B, int n, int H, int HK, int64_t in_bs, int64_t o_bs, float scale, cudaStream_t st);

namespace {

constexpr int kBlockedMinTokens = 4;   // from here on the blocked form wins over the token-by-token sweeps
constexpr int kTokBatch = 8;   // token vectors staged in shared memory per barrier round

// packed fp32 pairs (Blackwell): two FMAs / multiplies per instruction on 64-bit register pairs
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return d;
}

constexpr int kRowPad = 132;   // 128 rows + one 16-byte slot per 32-row group: the 4 row groups hit distinct banks
__device__ __forceinline__ int prow(int r) { return r + (r >> 5); }

template <typename T>
__global__ void __launch_bounds__(128, 3)
decode_d128_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const float* __restrict__ g, const T* __restrict__ b, const T* __restrict__ w,
                   float* __restrict__ state, T* __restrict__ o, int n, int H, int HK, int64_t in_bs, int64_t o_bs,
                   float scale) {
  constexpr int D = 128;
  const int bh = blockIdx.x;
  const int ib = bh / H, ih = bh % H;
  const int ihk = ih / (H / HK);                         // the key head this value head reads q, k, b, g from
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int rg = lane >> 3, cq = lane & 7;               // 32-row group, 4-column group inside the warp's 32 columns
  const int col0 = 32 * wid + 4 * cq;

  // per token and key row: (a*b*k, a*b*k, scale*q*a, scale*q*a) and (k, k, a, a), duplicated for the packed math
  __shared__ float4 s_p1[kTokBatch][kRowPad];
  __shared__ float4 s_p2[kTokBatch][kRowPad];
  __shared__ float s_wv[kTokBatch][D];                   // w * v
  __shared__ float s_qk[kTokBatch][4];                   // per-warp partial sums of scale * q . k

  float4 S[32];
  float4* gS = reinterpret_cast<float4*>(state + ((size_t)bh * D + 32 * rg) * D + col0);
#pragma unroll
  for (int i = 0; i < 32; ++i) S[i] = __ldcs(gS + i * (D / 4));

  for (int t0 = 0; t0 < n; t0 += kTokBatch) {
    const int nt = min(kTokBatch, n - t0);
    __syncthreads();                                     // the previous batch's vectors are no longer read
    for (int j = 0; j < nt; ++j) {
      const size_t tok = ((size_t)ib * in_bs + (t0 + j)) * H + ih;
      const size_t tokk = ((size_t)ib * in_bs + (t0 + j)) * HK + ihk;
      const float a = exp2f(g[tokk * D + tid] * kLog2e);
      const float kk = to_f32(k[tokk * D + tid]);
      const float abk = a * to_f32(b[tokk * D + tid]) * kk;
      const float qs = to_f32(q[tokk * D + tid]) * scale;
      s_p1[j][prow(tid)] = make_float4(abk, abk, qs * a, qs * a);
      s_p2[j][prow(tid)] = make_float4(kk, kk, a, a);
      s_wv[j][tid] = to_f32(w[tok * D + tid]) * to_f32(v[tok * D + tid]);
      float qk = qs * kk;
#pragma unroll
      for (int off = 16; off; off >>= 1) qk += __shfl_xor_sync(0xffffffffu, qk, off);
      if (lane == 0) s_qk[j][wid] = qk;
    }
    __syncthreads();

    for (int j = 0; j < nt; ++j) {
      // pass 1 over the old state: read with the erase row, and the part of the output that does not depend on u
      float2 rd0 = make_float2(0.f, 0.f), rd1 = rd0, oa0 = rd0, oa1 = rd0;
      const float4* p1 = &s_p1[j][33 * rg];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float4 P = p1[i];
        const float2 c_rd = make_float2(P.x, P.y), c_oa = make_float2(P.z, P.w);
        rd0 = ffma2(make_float2(S[i].x, S[i].y), c_rd, rd0);
        rd1 = ffma2(make_float2(S[i].z, S[i].w), c_rd, rd1);
        oa0 = ffma2(make_float2(S[i].x, S[i].y), c_oa, oa0);
        oa1 = ffma2(make_float2(S[i].z, S[i].w), c_oa, oa1);
      }
      float r8[8] = {rd0.x, rd0.y, rd1.x, rd1.y, oa0.x, oa0.y, oa1.x, oa1.y};
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        r8[x] += __shfl_xor_sync(0xffffffffu, r8[x], 8);
        r8[x] += __shfl_xor_sync(0xffffffffu, r8[x], 16);
      }
      const float4 wv = *reinterpret_cast<const float4*>(&s_wv[j][col0]);
      const float u0 = wv.x - r8[0], u1 = wv.y - r8[1], u2 = wv.z - r8[2], u3 = wv.w - r8[3];
      if (rg == 0) {
        const float qk = s_qk[j][0] + s_qk[j][1] + s_qk[j][2] + s_qk[j][3];
        T* po = o + (((size_t)ib * o_bs + (t0 + j)) * H + ih) * D + col0;
        po[0] = from_f32<T>(fmaf(qk, u0, r8[4])); po[1] = from_f32<T>(fmaf(qk, u1, r8[5]));
        po[2] = from_f32<T>(fmaf(qk, u2, r8[6])); po[3] = from_f32<T>(fmaf(qk, u3, r8[7]));
      }
      // pass 2: decay and rank-1 write
      const float2 uu0 = make_float2(u0, u1), uu1 = make_float2(u2, u3);
      const float4* p2 = &s_p2[j][33 * rg];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float4 Q = p2[i];
        const float2 kk2 = make_float2(Q.x, Q.y), a2 = make_float2(Q.z, Q.w);
        const float2 n0 = ffma2(a2, make_float2(S[i].x, S[i].y), fmul2(kk2, uu0));
        const float2 n1 = ffma2(a2, make_float2(S[i].z, S[i].w), fmul2(kk2, uu1));
        S[i] = make_float4(n0.x, n0.y, n1.x, n1.y);
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
                      float* __restrict__ state, T* __restrict__ o, int n, int H, int HK, int DK, int DV, int64_t in_bs,
                      int64_t o_bs, float scale) {
  const int bh = blockIdx.x;                 // (batch, head) on x: no 65535 limit
  const int ib = bh / H, ih = bh % H;
  const int ihk = ih / (H / HK);             // the key head this value head reads q, k, b, g from
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int dv = blockIdx.y * 32 + lane;
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
    const size_t tokk = ((size_t)ib * in_bs + t) * HK + ihk;
    const size_t otok = ((size_t)ib * o_bs + t) * H + ih;
    __syncthreads();
    for (int c = tid; c < DK; c += 128) {
      const float a = exp2f(g[tokk * DK + c] * kLog2e);
      const float kk = to_f32(k[tokk * DK + c]);
      s_a[c] = a; s_k[c] = kk;
      s_abk[c] = a * to_f32(b[tokk * DK + c]) * kk;
      s_q[c] = to_f32(q[tokk * DK + c]) * scale;
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
                 float* state, void* o, int B, int n, int H, int HK, int DK, int DV, int64_t in_bs, int64_t o_bs, float scale,
                 cudaStream_t st) {
  const T* tq = static_cast<const T*>(q); const T* tk = static_cast<const T*>(k);
  const T* tv = static_cast<const T*>(v); const T* tb = static_cast<const T*>(b);
  const T* tw = static_cast<const T*>(w); T* to = static_cast<T*>(o);
  if (DK == 128 && DV == 128 && n >= kBlockedMinTokens) {
    return launch_decode_blocked<T>(tq, tk, tv, g, tb, tw, state, to, B, n, H, HK, in_bs, o_bs, scale, st);
  } else if (DK == 128 && DV == 128) {
    decode_d128_kernel<T><<<B * H, 128, 0, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, HK, in_bs, o_bs, scale);
  } else {
    dim3 grid(B * H, (DV + 31) / 32);
    const size_t sm = (size_t)4 * DK * sizeof(float);
    if (DK <= 64)
      decode_generic_kernel<T, 16><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, HK, DK, DV, in_bs, o_bs, scale);
    else if (DK <= 128)
      decode_generic_kernel<T, 32><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, HK, DK, DV, in_bs, o_bs, scale);
    else
      decode_generic_kernel<T, 64><<<grid, 128, sm, st>>>(tq, tk, tv, g, tb, tw, state, to, n, H, HK, DK, DV, in_bs, o_bs, scale);
  }
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace

int launch_decode(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                  float* state, void* o, int B, int n, int H, int HK, int DK, int DV, int64_t in_bs, int64_t o_bs,
                  float scale, int dtype, cudaStream_t st) {
  switch (dtype) {
    case GDN2_F32: return launch_typed<float>(q, k, v, g, b, w, state, o, B, n, H, HK, DK, DV, in_bs, o_bs, scale, st);
    case GDN2_BF16: return launch_typed<__nv_bfloat16>(q, k, v, g, b, w, state, o, B, n, H, HK, DK, DV, in_bs, o_bs, scale, st);
    case GDN2_F16: return launch_typed<__half>(q, k, v, g, b, w, state, o, B, n, H, HK, DK, DV, in_bs, o_bs, scale, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

}  // namespace gdn2
