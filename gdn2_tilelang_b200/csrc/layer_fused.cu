// Element-wise stages of the GatedDeltaNet2 layer around the attention kernels, fused:
//
//   front: from ONE projection buffer P = x W_cat^T (columns q | k | v | b | w | f | o_gate) to the six
//          kernel inputs -- causal depthwise convolution + SiLU on q, k, v (with the cached last
//          conv_size-1 columns when decoding), L2 normalisation of q and k per head, the decay
//          g = -exp(A_log) * softplus(f + dt_bias), the gates b = erase_scale * sigmoid(.), w = sigmoid(.),
//          -- q, k, b, g once per key head: the attention kernels index key heads, no repeated copies;
//   tail:  the new convolution cache (the last conv_size-1 pre-convolution columns of q | k | v);
//   back:  per-head RMSNorm of the attention output times SiLU(o_gate).
//
// These replace the torch operator chains of _ShortConv, F.normalize, the gate expressions and
// _GatedRMSNorm (gdn2/attention.py:186-229, 290-297, 323-340 of the reference project): about 25 launches
// and as many round trips through HBM per call become three. All arithmetic is fp32 with one rounding to
// the storage type at the end. One warp per (token, kv head) in front, per (token, value head) in back.
#include "common.cuh"

namespace gdn2 {

namespace {

constexpr int kWarps = 4;

// Hardware exponential, reciprocal, logarithm and reciprocal square root, one instruction each (flush-to-zero
// forms: no denormal fix-up code). A few ulp each, far inside the 16-bit storage rounding and the 2e-5 the
// float32 form is tested to; the precise division and log1pf were most of these kernels' instructions.
__device__ __forceinline__ float ex2_(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float lg2_(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rsq_(float x) { float y; asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
__device__ __forceinline__ float silu(float x) { return x * rcp_(1.f + ex2_(-kLog2e * x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_(1.f + ex2_(-kLog2e * x)); }
__device__ __forceinline__ float softplusf_(float x) {
  const float e = ex2_(-kLog2e * fabsf(x));                // softplus(x) = max(x, 0) + log1p(exp(-|x|))
  const float l = e < 0x1p-12f ? e * (1.f - 0.5f * e) : kLn2 * lg2_(1.f + e);
  return fmaxf(x, 0.f) + l;
}
// 1 / max(sqrt(ss), 1e-12): the scale of F.normalize
__device__ __forceinline__ float inv_norm(float ss) { return rsq_(fmaxf(ss, 1e-24f)); }
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// value at time tt (may be negative: the cached columns, or zero) of projection column `col`, whose
// position among the convolved channels q | k | v is `cch`
template <typename T>
__device__ __forceinline__ float tap(const T* P, const T* conv_state, int64_t b, int tt, int S, int NP, int col, int cch,
                                     int CC, int K) {
  if (tt >= 0) return to_f32(P[((size_t)b * S + tt) * NP + col]);
  if (conv_state == nullptr) return 0.f;
  return to_f32(conv_state[((size_t)b * CC + cch) * (K - 1) + (K - 1 + tt)]);
}

template <typename T>
__global__ void __launch_bounds__(32 * kWarps)
layer_front_kernel(gdn2_layer_front_args a) {
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (item >= a.B * a.S * a.HK) return;
  const int hk = (int)(item % a.HK);
  const int64_t bt = item / a.HK;
  const int t = (int)(bt % a.S);
  const int64_t b = bt / a.S;
  const int S = (int)a.S, NP = (int)a.NP, K = (int)a.K, DK = (int)a.DK, DV = (int)a.DV, H = (int)a.H, HK = (int)a.HK;
  const int rep = H / HK;
  const int Cqk = HK * DK, Cv = H * DV, CC = 2 * Cqk + Cv;
  const T* P = static_cast<const T*>(a.proj);
  const T* cs = static_cast<const T*>(a.conv_state);
  const T* cw = static_cast<const T*>(a.conv_weight);   // [CC, K], channels q | k | v
  const T* cb = static_cast<const T*>(a.conv_bias);     // [CC] or null
  const size_t prow = ((size_t)b * S + t) * NP;

  // ---- q and k: convolution + SiLU, then L2 normalisation over the head
  for (int which = 0; which < 2; ++which) {
    const int col0 = (which == 0 ? (int)a.off_q : (int)a.off_k) + hk * DK;
    const int cch0 = which * Cqk + hk * DK;
    float ss = 0.f;
    float vals[8];                                       // DK <= 256: up to 8 channels per lane
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      float y = 0.f;
      if (c < DK) {
        if (K > 0) {
          y = cb ? to_f32(cb[cch0 + c]) : 0.f;
          for (int j = 0; j < K; ++j)
            y = fmaf(to_f32(cw[(size_t)(cch0 + c) * K + j]), tap(P, cs, b, t - (K - 1) + j, S, NP, col0 + c, cch0 + c, CC, K), y);
          y = silu(y);
        } else {
          y = to_f32(P[prow + col0 + c]);
        }
        ss = fmaf(y, y, ss);
      }
      vals[i] = y;
    }
    ss = warp_sum(ss);
    const float inv = inv_norm(ss);
    T* dst = static_cast<T*>(which == 0 ? a.q : a.k);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      if (c < DK) {
        dst[(((size_t)b * S + t) * HK + hk) * DK + c] = from_f32<T>(vals[i] * inv);
      }
    }
  }
  // ---- erase gate b and decay g of the key head
  {
    const T* A_log = static_cast<const T*>(a.A_log);
    const T* dtb = static_cast<const T*>(a.dt_bias);
    const float nega = -__expf(to_f32(A_log[hk]));
    T* bd = static_cast<T*>(a.b);
    for (int c = lane; c < DK; c += 32) {
      const T bo = from_f32<T>(to_f32(from_f32<T>(sigmoidf_(to_f32(P[prow + a.off_b + hk * DK + c])))) * a.erase_scale);
      const float go = nega * softplusf_(to_f32(P[prow + a.off_f + hk * DK + c]) + to_f32(dtb[hk * DK + c]));
      const size_t o = (((size_t)b * S + t) * HK + hk) * DK + c;
      bd[o] = bo;
      a.g[o] = go;
    }
  }
  // ---- v (convolution + SiLU) and the write gate w for the value heads of this kv head
  {
    T* vd = static_cast<T*>(a.v);
    T* wd = static_cast<T*>(a.w);
    for (int r = 0; r < rep; ++r) {
      const int h = hk * rep + r;
      for (int c = lane; c < DV; c += 32) {
        const int col = (int)a.off_v + h * DV + c;
        const int cch = 2 * Cqk + h * DV + c;
        float y;
        if (K > 0) {
          y = cb ? to_f32(cb[cch]) : 0.f;
          for (int j = 0; j < K; ++j)
            y = fmaf(to_f32(cw[(size_t)cch * K + j]), tap(P, cs, b, t - (K - 1) + j, S, NP, col, cch, CC, K), y);
          y = silu(y);
        } else {
          y = to_f32(P[prow + col]);
        }
        const size_t o = (((size_t)b * S + t) * H + h) * DV + c;
        vd[o] = from_f32<T>(y);
        wd[o] = from_f32<T>(sigmoidf_(to_f32(P[prow + a.off_w + h * DV + c])));
      }
    }
  }
}

// The common shape (DK = DV = 128, four taps, 16-bit storage): lane owns channels 4 lane .. 4 lane + 3 of a
// head, so every access to the projection buffer, the weights and the outputs is one 8- or 16-byte access
// and a warp covers a head's 256 bytes in one instruction.
template <typename T>
struct alignas(4 * sizeof(T)) Vec4 { T x[4]; };

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&o)[4]) {
  const Vec4<T> v = *reinterpret_cast<const Vec4<T>*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = to_f32(v.x[i]);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&o)[4]) {
  Vec4<T> v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.x[i] = from_f32<T>(o[i]);
  *reinterpret_cast<Vec4<T>*>(p) = v;
}

// convolution + SiLU of 4 adjacent channels: projection columns col.., convolved-channel index cch..
// `tail` (or null): where the new convolution cache of these channels goes, [4 channels][K - 1]; the last three taps
// of the LAST token are exactly its contents.
template <typename T>
__device__ __forceinline__ void conv4(const T* P, const T* cs, const T* cw, const T* cb, int64_t b, int t, int S, int NP,
                                      int col, int cch, int CC, float (&y)[4], T* tail) {
  constexpr int K = 4;
  float wt[4][4];                                        // [channel][tap]
#pragma unroll
  for (int i = 0; i < 4; ++i) load4(cw + (size_t)(cch + i) * K, wt[i]);
  if (cb) load4(cb + cch, y);
  else { y[0] = y[1] = y[2] = y[3] = 0.f; }
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int tt = t - (K - 1) + j;
    float x[4];
    if (tt >= 0) {
      load4(P + ((size_t)b * S + tt) * NP + col, x);
    } else if (cs) {
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = to_f32(cs[((size_t)b * CC + cch + i) * (K - 1) + (K - 1 + tt)]);
    } else {
      x[0] = x[1] = x[2] = x[3] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = fmaf(wt[i][j], x[i], y[i]);
    if (tail && j >= 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) tail[i * (K - 1) + (j - 1)] = from_f32<T>(x[i]);   // x came from a T: exact
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) y[i] = silu(y[i]);
}

template <typename T>
__global__ void __launch_bounds__(32 * kWarps)
layer_front_d128_kernel(gdn2_layer_front_args a) {
  constexpr int DK = 128, DV = 128;
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (item >= a.B * a.S * a.HK) return;
  const int hk = (int)(item % a.HK);
  const int64_t bt = item / a.HK;
  const int t = (int)(bt % a.S);
  const int64_t b = bt / a.S;
  const int S = (int)a.S, NP = (int)a.NP, H = (int)a.H, HK = (int)a.HK;
  const int rep = H / HK;
  const int Cqk = HK * DK, CC = 2 * Cqk + H * DV;
  const T* P = static_cast<const T*>(a.proj);
  const T* cs = static_cast<const T*>(a.conv_state);
  const T* cw = static_cast<const T*>(a.conv_weight);
  const T* cb = static_cast<const T*>(a.conv_bias);
  const size_t prow = ((size_t)b * S + t) * NP;
  const int c = 4 * lane;
  const size_t tokh = ((size_t)b * S + t) * H;          // first value head of this token
  const size_t tokk = ((size_t)b * S + t) * HK + hk;    // this key head: q, k, b, g are written once per key head

  // the warp of the last token also writes the new convolution cache of its channels (no separate launch)
  T* tails = (t == S - 1 && a.new_conv_state) ? static_cast<T*>(a.new_conv_state) + (size_t)b * CC * 3 : nullptr;
  for (int which = 0; which < 2; ++which) {
    float y[4];
    const int cchq = which * Cqk + hk * DK + c;
    conv4(P, cs, cw, cb, b, t, S, NP, (which == 0 ? (int)a.off_q : (int)a.off_k) + hk * DK + c, cchq, CC, y,
          tails ? tails + (size_t)cchq * 3 : nullptr);
    const float ss = warp_sum(y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3]);
    const float inv = inv_norm(ss);
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] *= inv;
    T* dst = static_cast<T*>(which == 0 ? a.q : a.k);
    store4(dst + tokk * DK + c, y);
  }
  {
    float pb[4], pf[4], db[4], bo[4], go[4];
    load4(P + prow + a.off_b + hk * DK + c, pb);
    load4(P + prow + a.off_f + hk * DK + c, pf);
    load4(static_cast<const T*>(a.dt_bias) + hk * DK + c, db);
    const float nega = -__expf(to_f32(static_cast<const T*>(a.A_log)[hk]));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      bo[i] = to_f32(from_f32<T>(sigmoidf_(pb[i]))) * a.erase_scale;
      go[i] = nega * softplusf_(pf[i] + db[i]);
    }
    store4(static_cast<T*>(a.b) + tokk * DK + c, bo);
    *reinterpret_cast<float4*>(a.g + tokk * DK + c) = make_float4(go[0], go[1], go[2], go[3]);
  }
  for (int r = 0; r < rep; ++r) {
    const int h = hk * rep + r;
    float y[4], pw[4];
    conv4(P, cs, cw, cb, b, t, S, NP, (int)a.off_v + h * DV + c, 2 * Cqk + h * DV + c, CC, y,
          tails ? tails + (size_t)(2 * Cqk + h * DV + c) * 3 : nullptr);
    load4(P + prow + a.off_w + h * DV + c, pw);
#pragma unroll
    for (int i = 0; i < 4; ++i) pw[i] = sigmoidf_(pw[i]);
    store4(static_cast<T*>(a.v) + (tokh + h) * DV + c, y);
    store4(static_cast<T*>(a.w) + (tokh + h) * DV + c, pw);
  }
}

// The same for prompts, cut finer: one warp per (head-wide slot, FOUR consecutive tokens). A token's slots are its
// HK q heads, HK k heads, H v heads (convolution kinds), HK erase-gate heads, HK decay heads and H write-gate heads
// (element-wise kinds); the slot index runs fastest, so the warps in flight sweep whole projection rows. A
// convolution slot reads the 7 projection rows its four outputs need once (the one-token form reads 16), every
// warp has all of its loads in flight before the first use and holds few enough registers for 32 warps per SM.
// Arithmetic and summation order are those of the one-token form, so the two agree bit for bit.
template <typename T>
__global__ void __launch_bounds__(32 * kWarps, 6)
layer_front_d128x4_kernel(gdn2_layer_front_args a) {
  constexpr int D = 128, K = 4, TT = 4;
  const int lane = threadIdx.x & 31;
  const int S = (int)a.S, NP = (int)a.NP, H = (int)a.H, HK = (int)a.HK;
  const int groups = (S + TT - 1) / TT;
  const int nslots = 4 * HK + 2 * H;
  const unsigned item = blockIdx.x * kWarps + (threadIdx.x >> 5);      // the launcher keeps the count below 2^31
  if (item >= (unsigned)a.B * groups * nslots) return;
  const int slot = (int)(item % (unsigned)nslots);
  const unsigned bg = item / (unsigned)nslots;
  const int t0 = (int)(bg % (unsigned)groups) * TT;
  const int64_t b = bg / (unsigned)groups;
  const int Cqk = HK * D, CC = 2 * Cqk + H * D;
  const T* P = static_cast<const T*>(a.proj);
  const int c = 4 * lane;
  const int nt = S - t0 < TT ? S - t0 : TT;               // tokens of this group that exist
  const size_t tok0 = (size_t)b * S + t0;
  {
    // Pull the rows of the same slot some 4096 warps ahead (about what the GPU holds at once, a whole number of
    // token groups of this batch row) towards L2: 4 rows x 256 B = 8 lines, one per lane 0..7.
    const int ahead = ((4096 + nslots - 1) / nslots) * TT;
    const int scol = slot < HK ? (int)a.off_q + slot * D
                   : slot < 2 * HK ? (int)a.off_k + (slot - HK) * D
                   : slot < 2 * HK + H ? (int)a.off_v + (slot - 2 * HK) * D
                   : slot < 3 * HK + H ? (int)a.off_b + (slot - 2 * HK - H) * D
                   : slot < 4 * HK + H ? (int)a.off_f + (slot - 3 * HK - H) * D
                   : (int)a.off_w + (slot - 4 * HK - H) * D;
    const int tp = t0 + ahead + (lane >> 1);
    if (lane < 2 * TT && tp < S)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(P + ((size_t)b * S + tp) * NP + scol) + (lane & 1) * 128));
  }

  if (slot < 2 * HK + H) {
    // ---- convolution + SiLU of 4 adjacent channels for the group's tokens; q and k then L2-normalised
    const bool is_v = slot >= 2 * HK;
    const int head = is_v ? slot - 2 * HK : slot < HK ? slot : slot - HK;
    const int col = (int)(is_v ? a.off_v : slot < HK ? a.off_q : a.off_k) + head * D + c;
    const int cch = (is_v ? 2 * Cqk : slot < HK ? 0 : Cqk) + head * D + c;
    const T* cs = static_cast<const T*>(a.conv_state);
    const T* cw = static_cast<const T*>(a.conv_weight);
    const T* cb = static_cast<const T*>(a.conv_bias);
    float wt[4][4], bias[4], x[TT + K - 1][4];
#pragma unroll
    for (int r = 0; r < TT + K - 1; ++r) {
      const int tt = t0 - (K - 1) + r;
      if (tt >= 0 && tt < S) {
        load4(P + ((size_t)b * S + tt) * NP + col, x[r]);
      } else if (tt < 0 && cs) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[r][i] = to_f32(cs[((size_t)b * CC + cch + i) * (K - 1) + (K - 1 + tt)]);
      } else {
        x[r][0] = x[r][1] = x[r][2] = x[r][3] = 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) load4(cw + (size_t)(cch + i) * K, wt[i]);
    if (cb) load4(cb + cch, bias);
    else { bias[0] = bias[1] = bias[2] = bias[3] = 0.f; }
    T* dst = static_cast<T*>(is_v ? a.v : slot < HK ? a.q : a.k);
    const int heads = is_v ? H : HK;
#pragma unroll
    for (int u = 0; u < TT; ++u) {
      float y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float acc = bias[i];
#pragma unroll
        for (int j = 0; j < K; ++j) acc = fmaf(wt[i][j], x[u + j][i], acc);
        y[i] = silu(acc);
      }
      if (!is_v) {
        const float ss = warp_sum(y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3]);
        const float inv = inv_norm(ss);
#pragma unroll
        for (int i = 0; i < 4; ++i) y[i] *= inv;
      }
      if (u < nt) store4(dst + ((tok0 + u) * heads + head) * D + c, y);
    }
    return;
  }
  // ---- element-wise slots: erase gate b, decay g (key heads), write gate w (value heads)
  const int e = slot - (2 * HK + H);
  const int kind = e < HK ? 0 : e < 2 * HK ? 1 : 2;
  const int head = kind == 0 ? e : kind == 1 ? e - HK : e - 2 * HK;
  const int col = (int)(kind == 0 ? a.off_b : kind == 1 ? a.off_f : a.off_w) + head * D + c;
  float p[TT][4];
#pragma unroll
  for (int u = 0; u < TT; ++u)
    if (u < nt) load4(P + (tok0 + u) * NP + col, p[u]);
  if (kind == 1) {
    float db[4];
    load4(static_cast<const T*>(a.dt_bias) + head * D + c, db);
    const float nega = -__expf(to_f32(static_cast<const T*>(a.A_log)[head]));
#pragma unroll
    for (int u = 0; u < TT; ++u)
      if (u < nt)
        *reinterpret_cast<float4*>(a.g + ((tok0 + u) * HK + head) * D + c) =
            make_float4(nega * softplusf_(p[u][0] + db[0]), nega * softplusf_(p[u][1] + db[1]),
                        nega * softplusf_(p[u][2] + db[2]), nega * softplusf_(p[u][3] + db[3]));
  } else {
    T* dst = static_cast<T*>(kind == 0 ? a.b : a.w);
    const int heads = kind == 0 ? HK : H;
#pragma unroll
    for (int u = 0; u < TT; ++u)
      if (u < nt) {
        float y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          y[i] = sigmoidf_(p[u][i]);
          if (kind == 0) y[i] = to_f32(from_f32<T>(y[i])) * a.erase_scale;
        }
        store4(dst + ((tok0 + u) * heads + head) * D + c, y);
      }
  }
}

// new_conv[b, cch, s] = pre-convolution value at time S - (K-1) + s (from P, the old cache, or zero)
template <typename T>
__global__ void layer_conv_tail_kernel(gdn2_layer_front_args a) {
  const int K = (int)a.K, S = (int)a.S, NP = (int)a.NP;
  const int Cqk = (int)(a.HK * a.DK), Cv = (int)(a.H * a.DV), CC = 2 * Cqk + Cv;
  const int64_t total = a.B * CC * (K - 1);
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int sidx = (int)(idx % (K - 1));
  const int cch = (int)((idx / (K - 1)) % CC);
  const int64_t b = idx / ((int64_t)(K - 1) * CC);
  const int col = cch < Cqk ? (int)a.off_q + cch : cch < 2 * Cqk ? (int)a.off_k + (cch - Cqk) : (int)a.off_v + (cch - 2 * Cqk);
  const int tt = S - (K - 1) + sidx;
  static_cast<T*>(a.new_conv_state)[idx] =
      from_f32<T>(tap(static_cast<const T*>(a.proj), static_cast<const T*>(a.conv_state), b, tt, S, NP, col, cch, CC, K));
}

template <typename T>
__global__ void __launch_bounds__(32 * kWarps)
layer_back_kernel(const T* __restrict__ o, const T* __restrict__ proj, const T* __restrict__ weight, T* __restrict__ out,
                  int64_t BS, int H, int DV, int NP, int off_gate, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (item >= BS * H) return;
  const int h = (int)(item % H);
  const int64_t bt = item / H;
  const T* orow = o + (size_t)item * DV;
  const T* grow = proj + (size_t)bt * NP + off_gate + h * DV;
  float x[8], ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    x[i] = c < DV ? to_f32(orow[c]) : 0.f;
    ss = fmaf(x[i], x[i], ss);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)DV + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < DV) out[(size_t)item * DV + c] = from_f32<T>(x[i] * r * to_f32(weight[c]) * silu(to_f32(grow[c])));
  }
}

template <typename T>
int launch_front_typed(const gdn2_layer_front_args& a, cudaStream_t st) {
  const int64_t items = a.B * a.S * a.HK;
  const bool aligned = a.NP % 4 == 0 && a.off_q % 4 == 0 && a.off_k % 4 == 0 && a.off_v % 4 == 0 && a.off_b % 4 == 0 &&
                       a.off_w % 4 == 0 && a.off_f % 4 == 0 &&
                       ((reinterpret_cast<uintptr_t>(a.proj) | reinterpret_cast<uintptr_t>(a.conv_weight) |
                         reinterpret_cast<uintptr_t>(a.conv_bias) | reinterpret_cast<uintptr_t>(a.dt_bias) |
                         reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
                         reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.w)) & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.g) & 15) == 0;
  if (sizeof(T) == 2 && a.DK == 128 && a.DV == 128 && a.K == 4 && aligned && a.S >= 8 &&
      a.B * ((a.S + 3) / 4) * (4 * a.HK + 2 * a.H) < (int64_t)1 << 31) {
    const int64_t items4 = a.B * ((a.S + 3) / 4) * (4 * a.HK + 2 * a.H);   // prompts: a slot of four tokens per warp
    layer_front_d128x4_kernel<T><<<(unsigned)((items4 + kWarps - 1) / kWarps), 32 * kWarps, 0, st>>>(a);
  } else if (sizeof(T) == 2 && a.DK == 128 && a.DV == 128 && a.K == 4 && aligned) {
    layer_front_d128_kernel<T><<<(unsigned)((items + kWarps - 1) / kWarps), 32 * kWarps, 0, st>>>(a);
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;                                          // this form writes the new convolution cache itself
  } else
    layer_front_kernel<T><<<(unsigned)((items + kWarps - 1) / kWarps), 32 * kWarps, 0, st>>>(a);
  GDN2_CUDA_TRY(cudaGetLastError());
  if (a.K > 1 && a.new_conv_state) {
    const int64_t total = a.B * (2 * a.HK * a.DK + a.H * a.DV) * (a.K - 1);
    layer_conv_tail_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a);
    GDN2_CUDA_TRY(cudaGetLastError());
  }
  return GDN2_OK;
}

// DV = 128, 16-bit storage: lane owns channels 4 lane .. 4 lane + 3, a warp takes FOUR consecutive (token, head)
// rows with all eight row loads in flight before the first use.
template <typename T>
__global__ void __launch_bounds__(32 * kWarps)
layer_back_d128_kernel(const T* __restrict__ o, const T* __restrict__ proj, const T* __restrict__ weight, T* __restrict__ out,
                       int64_t items, int H, int NP, int off_gate, float eps) {
  constexpr int DV = 128, R = 4;
  const int lane = threadIdx.x & 31;
  const int c = 4 * lane;
  const int64_t item0 = ((int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5)) * R;
  if (item0 >= items) return;
  float x[R][4], g[R][4], wv[4];
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const int64_t item = item0 + u;
    if (item < items) {
      load4(o + (size_t)item * DV + c, x[u]);
      const uint32_t tok = (uint32_t)item / (uint32_t)H;  // the launcher keeps the row count below 2^32
      load4(proj + (size_t)tok * NP + off_gate + (int)((uint32_t)item - tok * (uint32_t)H) * DV + c, g[u]);
    }
  }
  load4(weight + c, wv);
#pragma unroll
  for (int u = 0; u < R; ++u) {
    const int64_t item = item0 + u;
    if (item < items) {                                  // uniform over the warp
      const float ss = warp_sum(x[u][0] * x[u][0] + x[u][1] * x[u][1] + x[u][2] * x[u][2] + x[u][3] * x[u][3]);
      const float r = rsqrtf(ss / (float)DV + eps);
      float y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] = x[u][i] * r * wv[i] * silu(g[u][i]);
      store4(out + (size_t)item * DV + c, y);
    }
  }
}

template <typename T>
int launch_back_typed(const void* o, const void* proj, const void* weight, void* out, int64_t BS, int H, int DV, int NP,
                      int off_gate, float eps, cudaStream_t st) {
  const int64_t items = BS * H;
  const bool aligned = NP % 4 == 0 && off_gate % 4 == 0 &&
                       ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(weight) |
                         reinterpret_cast<uintptr_t>(out)) & 7) == 0;
  if (sizeof(T) == 2 && DV == 128 && aligned && items < (int64_t)1 << 32) {
    const int64_t warps = (items + 3) / 4;
    layer_back_d128_kernel<T><<<(unsigned)((warps + kWarps - 1) / kWarps), 32 * kWarps, 0, st>>>(
        static_cast<const T*>(o), static_cast<const T*>(proj), static_cast<const T*>(weight), static_cast<T*>(out), items, H,
        NP, off_gate, eps);
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  }
  layer_back_kernel<T><<<(unsigned)((items + kWarps - 1) / kWarps), 32 * kWarps, 0, st>>>(
      static_cast<const T*>(o), static_cast<const T*>(proj), static_cast<const T*>(weight), static_cast<T*>(out), BS, H,
      DV, NP, off_gate, eps);
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace

}  // namespace gdn2

extern "C" {

int gdn2_layer_front(const gdn2_layer_front_args* args, int dtype, void* stream) {
  using namespace gdn2;
  if (!args) return GDN2_ERR_NULL_POINTER;
  const gdn2_layer_front_args& a = *args;
  if (!a.proj || !a.q || !a.k || !a.v || !a.g || !a.b || !a.w || !a.A_log || !a.dt_bias) return GDN2_ERR_NULL_POINTER;
  if (a.B <= 0 || a.S <= 0 || a.H <= 0 || a.HK <= 0 || a.H % a.HK != 0 || a.DK <= 0 || a.DV <= 0 || a.DK > 256 ||
      a.DV > 256 || a.K < 0 || a.K > 16 || a.NP <= 0)
    return GDN2_ERR_BAD_SHAPE;
  if (a.K > 0 && !a.conv_weight) return GDN2_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case GDN2_F32: return launch_front_typed<float>(a, st);
    case GDN2_BF16: return launch_front_typed<__nv_bfloat16>(a, st);
    case GDN2_F16: return launch_front_typed<__half>(a, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

int gdn2_layer_back(const void* o, const void* proj, const void* norm_weight, void* out, int64_t BS, int64_t H,
                    int64_t DV, int64_t NP, int64_t off_gate, float eps, int dtype, void* stream) {
  using namespace gdn2;
  if (!o || !proj || !norm_weight || !out) return GDN2_ERR_NULL_POINTER;
  if (BS <= 0 || H <= 0 || DV <= 0 || DV > 256 || NP <= 0 || off_gate < 0) return GDN2_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case GDN2_F32: return launch_back_typed<float>(o, proj, norm_weight, out, BS, (int)H, (int)DV, (int)NP, (int)off_gate, eps, st);
    case GDN2_BF16: return launch_back_typed<__nv_bfloat16>(o, proj, norm_weight, out, BS, (int)H, (int)DV, (int)NP, (int)off_gate, eps, st);
    case GDN2_F16: return launch_back_typed<__half>(o, proj, norm_weight, out, BS, (int)H, (int)DV, (int)NP, (int)off_gate, eps, st);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

}  // extern "C"
