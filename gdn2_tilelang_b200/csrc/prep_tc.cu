// Chunk-local stage of the chunkwise forward, tensor-core (tcgen05 / TMEM) family, for
// DK = DV = 128 and bf16 inputs. One 256-thread block per (chunk, batch*head), two blocks per SM.
// Two thread mappings are used:
//   * gating (steps 1, value side): thread = (channel pair cp, 16-token sub-block sbk). Two adjacent
//     channels per thread turn every 16-bit load, convert and shared-memory store into a packed 32-bit one,
//     and the cumulative decay of a channel is a private running sum plus one prefix per sub-block
//     exchanged through shared memory. A warp holds one sub-block, so its constants are warp-uniform.
//   * everything that reads MMA results (steps 2b, 5): thread = (TMEM lane = row or channel, half of the
//     columns or tokens), because a warp can only address its own 32 lanes of tensor memory.
// What a gating thread produces for later steps (Qg, w*v) waits in spare TMEM columns of whatever lane the
// thread owns: the stash is private scratch, read back by the same thread.
//
// What the reference spreads over five kernels (cumsum, intra_diag, inter_blocks, solve, wy:
// gdn2/forward.py:65-535 of the reference project) is one kernel here, and the intermediates it
// round-trips through HBM (G, Akk, Ai) never leave the SM:
//
//  1. G = log2(e) * cumsum(g) as a running sum. The overflow-safe factorisation of the reference
//     (gdn2/forward.py:266-270): rows of sub-block i (16 tokens) are scaled by 2^(G_r - ref_i) and paired
//     with key rows scaled by 2^(ref_i - G_s). Here ref_i is G at the MIDDLE row of the sub-block. Against
//     keys of earlier sub-blocks the key exponent is <= 0 and the row factor is bounded by the decay of half
//     a sub-block; ON the diagonal sub-block both factors are bounded by half its span. The reference
//     evaluates the diagonal blocks pairwise on CUDA cores (intra_diag_kernel) -- here they ride the same
//     tensor-core product as long as each half of every sub-block decays by less than 2^96 (every product
//     2^(G_r - G_s), r >= s, is then formed from two factors inside bf16 range). A chunk that decays faster
//     is flagged in the workspace and redone exactly by the SIMT family's kernel.
//  2. MMA1 (bf16, M = 128: rows 0..63 = b*k rows, 64..127 = q rows, all scaled by their own ref):
//     four products A * B_i^T, B_i = key rows s < 16(i+1) scaled to ref_i, N = 16(i+1).
//     Row block i of product i gives Tm (strictly lower) and Aqk (lower incl. diagonal, * scale).
//  3. (I + Tm)^-1 by 16x16 blocks: the four diagonal blocks by forward substitution in registers,
//     the off-diagonal blocks from 16 small products on warp-level register fragments.
//  4. MMA2 (tf32, transposed so channels are M): W^T = E^T * Ai^T, U^T = (w*v)^T * Ai^T.
//  5. Outputs in the scan's operand layout (common.cuh): WQ via shared staging + coalesced stores, AQK,
//     KG^T and U^T (scaled fp16), gamma_last with 128-bit coalesced global stores.
//
// Shared memory is two regions reused over the block's life so that two blocks fit on an SM:
//   X (72.5 KiB): MMA1 operands, then Tm + Ai + (w*v)^T;   Y (32.25 KiB): E^T, then the WQ staging.
// Qg = scale*q*gamma is produced in step 1 but only needed in step 5; it waits in 32 spare TMEM
// columns (packed bf16 pairs: the two channels of one token per word).
#include "common.cuh"
#include "tc_utils.cuh"

namespace gdn2 {

namespace {

constexpr int D = 128;
constexpr int BS = kChunk;
constexpr int kThreads = 256;
constexpr int A_PAD = 129;        // rows per K chunk of a 128-row bf16 image, +1 pad row: kills bank conflicts
constexpr int B_PAD = 161;        // 160 key rows (16 + 32 + 48 + 64) + 1 pad row
constexpr int TM_STRIDE = 68;     // floats per Tm row (row-major, padded against bank conflicts)
constexpr float kMaxSpanLog2 = 96.f;     // 2^96 keeps every scaled operand inside bf16 and fp32 range (|k|, |q| << 2^30)
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kZCol = 192;   // TMEM columns [192,256): w*v of the thread's value channel (fp32)
constexpr uint32_t kQgCol = 160;  // TMEM columns [160,192): packed Qg of the thread's channel

struct PrepTcSmem {
  union {
    struct {
      __nv_bfloat16 a_own[16 * A_PAD * 8];   // A of MMA1: [dk/8][129][8]
      __nv_bfloat16 bfam[16 * B_PAD * 8];    // B of MMA1: [dk/8][161][8], rows: B_0 0..15, B_1 16..47, B_2 48..95, B_3 96..159
    } ops;
    struct {
      float tm[BS * TM_STRIDE];              // strictly lower Tm, row-major; N_ik = D_i T_ik overwrites its blocks
      float ai[16 * BS * 4];                 // B of MMA2: (I+Tm)^-1 as [s/4][64 r][4]
      float zt[16 * D * 4];                  // A of MMA2: (w*v)^T [tok/4][128 dv][4]
    } sol;
  } x;
  union {
    float et[16 * D * 4];                    // A of MMA2: E^T  [tok/4][128 dk][4]
    __nv_bfloat16 wq[16 * A_PAD * 8];        // staging of the WQ record: [dk/8][129][8]
  } y;
  float pre[4][2][D];                        // per sub-block and channel: G at its reference row (row 8) and its total, both relative to its start
  uint64_t bar_m1, bar_m2, bar_m2v;
  uint32_t tmem_base;
  int abort_flag;
};

// 2^x by the hardware approximation alone (about 2 ulp; arguments here are differences of log2 decays,
// results that underflow flush to zero, which is the right answer for a vanished decay)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Raw values of one channel pair for 4 consecutive tokens, converted only when consumed: k, q, b as the two bf16
// bit patterns in one 32-bit word (low half = even channel). The decay values are read once for the whole
// sub-block in step 1a and stay in registers.
struct Raw4 {
  uint32_t k[4], q[4], b[4];
};
__device__ __forceinline__ void load_raw4(Raw4& r, const uint32_t* kp, const uint32_t* qp, const uint32_t* bp, size_t pstride) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const size_t off = u * pstride;
    r.k[u] = __ldg(kp + off); r.q[u] = __ldg(qp + off); r.b[u] = __ldg(bp + off);
  }
}
// the two bf16 values of a packed word as fp32 (a bf16 is the top half of an fp32)
__device__ __forceinline__ float2 bf16x2_bits_to_f32(uint32_t x) {
  return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack_f16x2_rn(float lo, float hi) {
  __half2 t = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 ex2(float2 x) { return make_float2(ex2(x.x), ex2(x.y)); }
__device__ __forceinline__ float2 operator-(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ float2 operator+(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 operator*(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ float2 pick4(int j, float2 a0, float2 a1, float2 a2, float2 a3) {
  return j == 0 ? a0 : j == 1 ? a1 : j == 2 ? a2 : a3;
}

// One block per (chunk, batch, KEY head). Everything that depends on q, k, b, g is computed once; U^T = (w*v)^T Ai^T
// is then formed for each of the `rep` value heads that share the key head (grouped-query heads; rep = 1 when every
// head has its own q, k, b, g).
// HT > 0: the number of key heads is a compile-time constant (and RT > 0 the value heads per key head), so every
// token offset of the strided channel loads folds into the load instruction's immediate; 0 takes them from the
// arguments.
template <int HT, int RT>
__global__ void __launch_bounds__(kThreads, 2)
prep_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
               const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
               const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ w, WsPtrs P, int S, int H,
               int HK_arg, int64_t in_bs, float scale, int a_sm_count, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PrepTcSmem& s = *reinterpret_cast<PrepTcSmem*>(smem_raw);
  const int NC = S / BS;
  const int HK = HT > 0 ? HT : HK_arg;                                  // key heads
  const int rep = RT > 0 ? RT : H / HK;                                 // value heads per key head
  const int n = blockIdx.x, bh = blockIdx.y;                            // bh: (batch, key head)
  const int ib = bh / HK, ih = bh % HK;
  const int64_t ch = (int64_t)bh * NC + n;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int c = tid & (D - 1);                                          // lane-true mapping: channel / row = TMEM lane
  const int hf = tid >> 7;                                              // ... and half of the tokens or columns
  const int lq = wid & 3;                                               // TMEM lane quarter of this warp
  // gating mapping: thread = (channel pair cp, 16-token sub-block sbk); a warp has one sub-block
  const int cp = tid & 63;                                              // channels 2 cp, 2 cp + 1
  const int sbk = tid >> 6;
  const int c0 = 2 * cp;
  const size_t row0 = ((size_t)ib * in_bs + (size_t)n * BS) * HK + ih;  // q, k, b, g: token row of t = 0
  const size_t rstride = (size_t)HK * D;                                // ... and elements between tokens
  const size_t pstride = rstride / 2;                                   // channel pairs between tokens
  const size_t soff = (size_t)(16 * sbk) * rstride;                     // first token of this thread's sub-block
  // v, w: the same for the first value head of this key head (the others follow at +D elements each)
  const size_t vrow0 = ((size_t)ib * in_bs + (size_t)n * BS) * HK * rep + (size_t)ih * rep;
  const size_t vstride = rstride * rep, vpstride = vstride / 2;
  const size_t vsoff = (size_t)(16 * sbk) * vstride;
  const float2* gp = reinterpret_cast<const float2*>(g + row0 * D + soff) + cp;

  // Pull the whole input tile of this chunk-head towards L2 before anything depends on it: 64 rows x
  // (5 x 256 B + 512 B) = 896 128-byte lines, 3.5 per thread (v and w of the first value head; the other value
  // heads' lines are adjacent in memory and are fetched when their turn comes).
  {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int line = tid + kThreads * i;                // 0..895: g takes lines [0,256), then 128 per bf16 tensor
      if (line < 896) {
        const int ten = line < 256 ? 0 : 1 + ((line - 256) >> 7);
        const int rem = line < 256 ? line : (line - 256) & 127;
        const int per_row = ten == 0 ? 4 : 2;
        const int rowi = rem / per_row, seg = rem % per_row;
        const void* tb = ten == 0 ? (const void*)g : ten == 1 ? (const void*)k : ten == 2 ? (const void*)q
                       : ten == 3 ? (const void*)b : ten == 4 ? (const void*)v : (const void*)w;
        const size_t es = ten == 0 ? 4 : 2;
        const size_t r0 = ten >= 4 ? vrow0 : row0, rs = ten >= 4 ? vstride : rstride;
        const char* ptr = static_cast<const char*>(tb) + (r0 * D + (size_t)rowi * rs) * es + seg * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
      }
    }
  }

  // ---- 1a. G at the first row of every sub-block and at the last token; decay-span check.
  //          Each thread sums its own sub-block (two channels); the four meet through shared memory.
  float2 ref0, ref1, ref2, ref3, g_last, run0;
  bool bad = false;
  float2 gv[16];                                         // this thread's 16 decay values: read once, used again in step 1b
  const uint32_t* qp = reinterpret_cast<const uint32_t*>(q + row0 * D + soff) + cp;
  const uint32_t* kp = reinterpret_cast<const uint32_t*>(k + row0 * D + soff) + cp;
  const uint32_t* bp = reinterpret_cast<const uint32_t*>(b + row0 * D + soff) + cp;
  Raw4 ra;                                               // first group of step 1b: its loads fly across the barrier below
  {
#pragma unroll
    for (int t = 0; t < 16; ++t) gv[t] = __ldg(gp + t * pstride);                 // 16 independent loads in flight
    load_raw4(ra, kp, qp, bp, pstride);
    float2 run = make_float2(0.f, 0.f);
    float2 mid = make_float2(0.f, 0.f);                  // G at row 8 of the sub-block: its reference row
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      run.x = fmaf(gv[u].x, kLog2e, run.x); run.y = fmaf(gv[u].y, kLog2e, run.y);
      if (u == 8) mid = run;
    }
    // The reference sits in the middle of the sub-block, so both the row factors 2^(G_r - ref) and the key
    // factors 2^(ref - G_s) of its diagonal block stay within 2^(half span): the two half spans are checked.
    const float2 first = make_float2(gv[0].x * kLog2e, gv[0].y * kLog2e);
    bad = !((first.x - mid.x) <= kMaxSpanLog2) || !((first.y - mid.y) <= kMaxSpanLog2) ||
          !((mid.x - run.x) <= kMaxSpanLog2) || !((mid.y - run.y) <= kMaxSpanLog2);
    *reinterpret_cast<float2*>(&s.pre[sbk][0][c0]) = mid;
    *reinterpret_cast<float2*>(&s.pre[sbk][1][c0]) = run;
  }
  if (tid == 0) {
    tc::mbar_init(&s.bar_m1, 4);     // one commit per issuing warp
    tc::mbar_init(&s.bar_m2, 2);
    tc::mbar_init(&s.bar_m2v, 1);    // U^T of the further value heads: one product, one commit each
    s.abort_flag = 0;
    tc::mbar_init_fence();
  }
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (tid == 0) {
    P.flags[ch] = any_bad ? 1 : 0;
    if (any_bad) {                    // append to the compacted list the exact kernel walks (count zeroed by the launcher)
      const int64_t nch_all = (int64_t)gridDim.x * gridDim.y;
      P.flags[nch_all + atomicAdd(&P.flags[2 * nch_all], 1)] = (int)ch;
    }
  }
  if (any_bad) return;              // the exact kernel redoes this chunk; nothing allocated yet
  {
    const float2 f0 = *reinterpret_cast<const float2*>(&s.pre[0][0][c0]), t0_ = *reinterpret_cast<const float2*>(&s.pre[0][1][c0]);
    const float2 f1 = *reinterpret_cast<const float2*>(&s.pre[1][0][c0]), t1_ = *reinterpret_cast<const float2*>(&s.pre[1][1][c0]);
    const float2 f2 = *reinterpret_cast<const float2*>(&s.pre[2][0][c0]), t2_ = *reinterpret_cast<const float2*>(&s.pre[2][1][c0]);
    const float2 f3 = *reinterpret_cast<const float2*>(&s.pre[3][0][c0]), t3_ = *reinterpret_cast<const float2*>(&s.pre[3][1][c0]);
    const float2 p1 = t0_, p2 = t0_ + t1_, p3 = p2 + t2_;
    ref0 = f0; ref1 = p1 + f1; ref2 = p2 + f2; ref3 = p3 + f3;
    g_last = p3 + t3_;
    run0 = pick4(sbk, make_float2(0.f, 0.f), p1, p2, p3);
  }
  if (wid == 0) tc::tmem_alloc(&s.tmem_base, kTmemCols);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = s.tmem_base;

  // ---- 1b. gated operands of the channel pair for this thread's 16 tokens, in four groups of 4 (written out,
  //          so that the decay values of step 1a are addressed statically and stay in registers); the next
  //          group's 12 loads are issued (raw, unconverted) before the current one is processed. Two
  //          channels per thread: every 16-bit operand leaves as a packed pair (one convert, one store).
  {
    uint32_t* a_own32 = reinterpret_cast<uint32_t*>(s.x.ops.a_own) + (cp >> 2) * A_PAD * 4 + (cp & 3);
    uint32_t* bfam32 = reinterpret_cast<uint32_t*>(s.x.ops.bfam) + (cp >> 2) * B_PAD * 4 + (cp & 3);
    char* kgt_g = P.kgt + (size_t)ch * (D * BS * 2) + c0 * 16;   // fp16 image [tok/8][128 dk][8]
    const int j = sbk;                                          // warp-uniform
    const int off_j = 8 * j * (j + 1);                          // first row of B_j: 0, 16, 48, 96
    const int off_j1 = 8 * (j + 1) * (j + 2), off_j2 = 8 * (j + 2) * (j + 3);
    const float2 zero2 = make_float2(0.f, 0.f);
    const float2 ref = pick4(j, ref0, ref1, ref2, ref3);
    const float2 refn = pick4(j, ref1, ref2, ref3, zero2);      // ref of the next sub-block (unused for j = 3)
    const float2 gam_ref = ex2(ref);
    const float2 nx_ref = (j < 3) ? refn : g_last;             // keys of this sub-block, seen from the next one
    const float2 kg_c = (j < 3) ? ex2(g_last - refn) : make_float2(1.f, 1.f);
    const float2 cc_a = ex2(pick4(j, ref2, ref3, zero2, zero2) - refn);   // B_{j+2} relative to B_{j+1}
    const float2 cc_b = ex2(ref3 - refn);                      // B_{j+3} relative to B_{j+1} (j = 0 only)
    float2 run = run0;
    uint32_t kgx[4], kgy[4];                                    // fp16 pairs of KG for 8 tokens of each channel

    // one group: tokens t0 .. t0 + 3 of the chunk (t0 a multiple of 4); hi = second group of an 8-token pair
    auto gate4 = [&](const Raw4& r, const float2* gq, int t0, int hi) {
      float e4x[4], e4y[4], kx[4], ky[4];
      uint32_t qgp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t = t0 + u;
        run.x = fmaf(gq[u].x, kLog2e, run.x); run.y = fmaf(gq[u].y, kLog2e, run.y);
        const float2 kf = bf16x2_bits_to_f32(r.k[u]), qf = bf16x2_bits_to_f32(r.q[u]);
        const float2 a = ex2(run - ref);                      // both bounded by the half-span check
        const float2 co = ex2(ref - run);
        // 2^(refn - run) (2^(g_last - run) for j = 3), <= 1. Formed from its own exponent: the step from this
        // sub-block's reference to the next one's is not covered by the span check, so a product of
        // 2^(refn - ref) (which may flush to zero) and 2^(ref - run) (up to 2^96) would lose keys whose true
        // factor is still a normal number.
        const float2 nx = ex2(nx_ref - run);
        const float2 e = bf16x2_bits_to_f32(r.b[u]) * kf;
        a_own32[t * 4] = pack_bf16x2_rn(e.x * a.x, e.y * a.y);
        a_own32[(BS + t) * 4] = pack_bf16x2_rn(qf.x * a.x, qf.y * a.y);
        bfam32[(off_j + t) * 4] = pack_bf16x2_rn(kf.x * co.x, kf.y * co.y);
        const float2 kn = kf * nx;
        if (j < 3) bfam32[(off_j1 + t) * 4] = pack_bf16x2_rn(kn.x, kn.y);
        if (j < 2) bfam32[(off_j2 + t) * 4] = pack_bf16x2_rn(kn.x * cc_a.x, kn.y * cc_a.y);
        if (j < 1) bfam32[(96 + t) * 4] = pack_bf16x2_rn(kn.x * cc_b.x, kn.y * cc_b.y);
        const float2 gam = a * gam_ref;
        e4x[u] = tf32_rn(e.x * gam.x); e4y[u] = tf32_rn(e.y * gam.y);
        qgp[u] = pack_bf16x2_rn(scale * qf.x * gam.x, scale * qf.y * gam.y);
        kx[u] = kn.x * kg_c.x * kValScale; ky[u] = kn.y * kg_c.y * kValScale;
      }
      const int tq = t0 >> 2;                                   // token quad index
      *reinterpret_cast<float4*>(&s.y.et[(tq * D + c0) * 4]) = make_float4(e4x[0], e4x[1], e4x[2], e4x[3]);
      *reinterpret_cast<float4*>(&s.y.et[(tq * D + c0 + 1) * 4]) = make_float4(e4y[0], e4y[1], e4y[2], e4y[3]);
      tc::tmem_st4(tc::tmem_addr(tm, lq * 32, kQgCol + 16 * (sbk >> 1) + (t0 & 15)), qgp);
      kgx[2 * hi] = pack_f16x2_rn(kx[0], kx[1]); kgx[2 * hi + 1] = pack_f16x2_rn(kx[2], kx[3]);
      kgy[2 * hi] = pack_f16x2_rn(ky[0], ky[1]); kgy[2 * hi + 1] = pack_f16x2_rn(ky[2], ky[3]);
      if (hi) {
        char* dst = kgt_g + (size_t)(t0 >> 3) * D * 16;
        *reinterpret_cast<uint4*>(dst) = make_uint4(kgx[0], kgx[1], kgx[2], kgx[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(kgy[0], kgy[1], kgy[2], kgy[3]);
      }
    };

    Raw4 rb;
    {
      const int t0 = 16 * sbk;
      load_raw4(rb, kp + 4 * pstride, qp + 4 * pstride, bp + 4 * pstride, pstride);
      gate4(ra, gv, t0, 0);
      load_raw4(ra, kp + 8 * pstride, qp + 8 * pstride, bp + 8 * pstride, pstride);
      gate4(rb, gv + 4, t0 + 4, 1);
      load_raw4(rb, kp + 12 * pstride, qp + 12 * pstride, bp + 12 * pstride, pstride);
      gate4(ra, gv + 8, t0 + 8, 0);
      gate4(rb, gv + 12, t0 + 12, 1);
    }
    tc::tmem_st_wait();
    if (sbk == 3) *reinterpret_cast<float2*>(&P.gl[(size_t)ch * D + c0]) = ex2(g_last);
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  // ---- 2. MMA1: D_i[128 x 16(i+1)] at TMEM columns 0, 16, 48, 96
  //         The four products are independent: warps 0..3 issue one each (converged, one elected
  //         lane) and commit it, so no warp falls far behind the others before the value-side loads.
  if (wid < 4) {
    tc::tc_fence_after_sync();
    const int i = wid;
    const int off = 8 * i * (i + 1);
    tc::mma_bf16_ktile_warp(tc::tmem_addr(tm, 0, off), tc::smem_u32(s.x.ops.a_own), A_PAD,
                            tc::smem_u32(s.x.ops.bfam) + off * 16, B_PAD, D, tc::instr_desc(1, 128, 16 * (i + 1)));
    tc::mma_commit_warp(&s.bar_m1);
  }
  // The block that will most likely run next in this slot (two resident blocks per SM, dispatched in
  // linear order) starts with a cold read of its g tile: pull those 256 lines towards L2 now.
  {
    const int64_t nxt = (int64_t)blockIdx.y * gridDim.x + blockIdx.x + 2 * (int64_t)a_sm_count;
    if (nxt < (int64_t)gridDim.x * gridDim.y) {
      const int nb_ = (int)(nxt / gridDim.x), nn_ = (int)(nxt % gridDim.x);
      const size_t r0n = ((size_t)(nb_ / HK) * in_bs + (size_t)nn_ * BS) * HK + (nb_ % HK);
      const char* ptr = reinterpret_cast<const char*>(g + r0n * D + (size_t)(tid >> 2) * rstride) + (tid & 3) * 128;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
    }
  }
  // value side: raw loads issued while the tensor core works
  // z = w*v of this thread's two value channels waits in TMEM columns [192,256) of its own lane until the
  // MMA1 operands are dead and (w*v)^T can take their place in shared memory
  {
    const uint32_t* vp = reinterpret_cast<const uint32_t*>(v + vrow0 * D + vsoff) + cp;
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(w + vrow0 * D + vsoff) + cp;
    uint32_t vr[16], wr[16];                              // raw bf16 pairs: all 32 loads in flight, then converted
#pragma unroll
    for (int u = 0; u < 16; ++u) { vr[u] = __ldg(vp + u * vpstride); wr[u] = __ldg(wp + u * vpstride); }
    float zx[16], zy[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const float2 vf = bf16x2_bits_to_f32(vr[u]), wf = bf16x2_bits_to_f32(wr[u]);
      zx[u] = tf32_rn(vf.x * wf.x); zy[u] = tf32_rn(vf.y * wf.y);
    }
    tc::tmem_st16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * (sbk >> 1)), zx);
    tc::tmem_st16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * (sbk >> 1) + 16), zy);
    tc::tmem_st_wait();
  }
  // one warp polls the MMA barrier; the rest sleep at the block barrier instead of spending issue slots
  if (wid == 0) tc::mbar_wait(&s.bar_m1, 0, &s.abort_flag, status, 0x1000u);
  __syncthreads();
  tc::tc_fence_after_sync();

  // ---- 2b. read back: lane = row (0..63 Tm, 64..127 Aqk); a warp spans sub-blocks i0 and i0+1, and
  //          the two threads of a row split the four 16-column groups.
  //          The MMA1 operands are dead now: Tm, Ai and (w*v)^T take their place.
  {
    const int r = c & 63;
    const bool is_q = c >= 64;
    const int i0 = 2 * (lq & 1);
    const bool hi = lane >= 16;
    const uint32_t t_lo = tc::tmem_addr(tm, lq * 32, 8 * i0 * (i0 + 1));
    const uint32_t t_hi = tc::tmem_addr(tm, lq * 32, 8 * (i0 + 1) * (i0 + 2));
    float* tr = s.x.sol.tm + r * TM_STRIDE;
    __half* ag = reinterpret_cast<__half*>(P.aqk + (size_t)ch * (BS * BS * 2));   // fp16, 256 * Aqk
#pragma unroll 1
    for (int cg = 2 * hf; cg < 2 * hf + 2; ++cg) {
      float lo16[16], hi16[16], row[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) { lo16[x] = 0.f; hi16[x] = 0.f; }
      if (cg <= i0) tc::tmem_ld16(t_lo + 16 * cg, lo16);          // warp-uniform conditions
      if (cg <= i0 + 1) tc::tmem_ld16(t_hi + 16 * cg, hi16);
      tc::tmem_ld_wait();
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        const int sc = 16 * cg + x;
        const float val = hi ? hi16[x] : lo16[x];
        const bool keep = is_q ? (sc <= r) : (sc < r);
        row[x] = keep ? (is_q ? val * scale : val) : 0.f;
      }
      if (!is_q) {
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4)
          *reinterpret_cast<float4*>(tr + 16 * cg + 4 * m4) =
              make_float4(row[4 * m4], row[4 * m4 + 1], row[4 * m4 + 2], row[4 * m4 + 3]);
      } else {
        *reinterpret_cast<uint4*>(ag + ((2 * cg) * BS + r) * 8) = tc::pack8_f16(&row[0], kValScale);
        *reinterpret_cast<uint4*>(ag + ((2 * cg + 1) * BS + r) * 8) = tc::pack8_f16(&row[8], kValScale);
      }
    }
    // (w*v)^T image from the TMEM stash: each thread moves the 16 tokens x 2 channels it produced
    {
      float zx[16], zy[16];
      tc::tmem_ld16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * (sbk >> 1)), zx);
      tc::tmem_ld16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * (sbk >> 1) + 16), zy);
      tc::tmem_ld_wait();
#pragma unroll
      for (int t4 = 0; t4 < 4; ++t4) {
        const int tq = 4 * sbk + t4;
        *reinterpret_cast<float4*>(&s.x.sol.zt[(tq * D + c0) * 4]) =
            make_float4(zx[4 * t4], zx[4 * t4 + 1], zx[4 * t4 + 2], zx[4 * t4 + 3]);
        *reinterpret_cast<float4*>(&s.x.sol.zt[(tq * D + c0 + 1) * 4]) =
            make_float4(zy[4 * t4], zy[4 * t4 + 1], zy[4 * t4 + 2], zy[4 * t4 + 3]);
      }
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();

  // ---- 3. (I + Tm)^-1 by 16x16 blocks. With D_i = (I + T_ii)^-1 and N_ik = D_i T_ik (i > k):
  //          X_ii = D_i,   X_ij = - sum_{k=j}^{i-1} N_ik X_kj   (i > j),   zero above the diagonal.
  //      The diagonal blocks are substituted column by column in registers (one thread per column);
  //      the 16 block products run as warp-level m16n8k8 tf32 MMAs on register fragments.
  {
    float* tmm = s.x.sol.tm;
    float* aim = s.x.sol.ai;
    auto AI = [](int r, int c) { return ((c >> 2) * BS + r) * 4 + (c & 3); };   // (row r, source token c) in the B image
    if (tid < BS) {
      const int i = tid >> 4, j = tid & 15;
      const float* tb = tmm + (16 * i) * TM_STRIDE + 16 * i;
      float x[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int sc = 0; sc < r; ++sc) {
          if (sc & 1) a1 = fmaf(tb[r * TM_STRIDE + sc], x[sc], a1);
          else a0 = fmaf(tb[r * TM_STRIDE + sc], x[sc], a0);
        }
        x[r] = (r == j ? 1.f : 0.f) - (a0 + a1);            // rows above j stay 0, row j is 1
        aim[AI(16 * i + r, 16 * i + j)] = tf32_rn(x[r]);
      }
    } else if (tid >= 128) {
      // zero the blocks above the diagonal: 6 blocks x 256 entries over 128 threads
      const int z = tid - 128;
#pragma unroll
      for (int e = 0; e < 12; ++e) {
        const int idx = z + 128 * e;                        // 0..1535
        const int blk = idx >> 8, rr = (idx >> 4) & 15, cc = idx & 15;
        const int bi = blk < 3 ? 0 : blk < 5 ? 1 : 2;       // (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
        const int bj = blk < 3 ? blk + 1 : blk < 5 ? blk - 1 : 3;
        aim[AI(16 * bi + rr, 16 * bj + cc)] = 0.f;
      }
    }
    __syncthreads();
    const int g8 = lane >> 2, t4 = lane & 3;
    auto T_at = [&](int bi, int bk, int r, int cidx) { return tmm[(16 * bi + r) * TM_STRIDE + 16 * bk + cidx]; };
    auto X_at = [&](int bi, int bk, int r, int cidx) { return aim[AI(16 * bi + r, 16 * bk + cidx)]; };
    // acc[nt][..] += A(16x16) * B(16x16); A and B are read through (row, col) accessors
    auto block_mma = [&](float (&acc)[2][4], auto a_at, auto b_at) {
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        const uint32_t a[4] = {__float_as_uint(tf32_rn(a_at(g8, 8 * kt + t4))), __float_as_uint(tf32_rn(a_at(g8 + 8, 8 * kt + t4))),
                               __float_as_uint(tf32_rn(a_at(g8, 8 * kt + t4 + 4))),
                               __float_as_uint(tf32_rn(a_at(g8 + 8, 8 * kt + t4 + 4)))};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const uint32_t b0 = __float_as_uint(tf32_rn(b_at(8 * kt + t4, 8 * nt + g8)));
          const uint32_t b1 = __float_as_uint(tf32_rn(b_at(8 * kt + t4 + 4, 8 * nt + g8)));
          asm volatile(
              "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(acc[nt][0]), "+f"(acc[nt][1]), "+f"(acc[nt][2]), "+f"(acc[nt][3])
              : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        }
      }
    };
    // N_ik = D_i T_ik, in place over T_ik: warp w < 6 takes pair w of (1,0) (2,0) (2,1) (3,0) (3,1) (3,2)
    if (wid < 6) {
      const int pidx = wid;
      const int bi = pidx < 1 ? 1 : pidx < 3 ? 2 : 3;
      const int bk = pidx < 1 ? 0 : pidx < 3 ? pidx - 1 : pidx - 3;
      float acc[2][4] = {};
      block_mma(acc, [&](int r, int cidx) { return X_at(bi, bi, r, cidx); }, [&](int r, int cidx) { return T_at(bi, bk, r, cidx); });
      __syncwarp();
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float* d0 = tmm + (16 * bi + g8) * TM_STRIDE + 16 * bk + 8 * nt + 2 * t4;
        d0[0] = acc[nt][0]; d0[1] = acc[nt][1];
        d0[8 * TM_STRIDE] = acc[nt][2]; d0[8 * TM_STRIDE + 1] = acc[nt][3];
      }
    }
    __syncthreads();
    // X_ij, distance d = i - j = 1, 2, 3. Block column j belongs to warps 2j and 2j + 1, eight columns each: a
    // warp reads only N (finished above), the diagonal inverse and what it wrote itself in earlier rounds, so the
    // rounds need a warp barrier only; every product is half as wide as a 16 x 16 block product.
    {
      const int bj = wid >> 1, nh = wid & 1;
      auto half_mma = [&](float (&acc)[4], auto a_at, auto b_at) {
#pragma unroll
        for (int kt = 0; kt < 2; ++kt) {
          const uint32_t a[4] = {__float_as_uint(tf32_rn(a_at(g8, 8 * kt + t4))), __float_as_uint(tf32_rn(a_at(g8 + 8, 8 * kt + t4))),
                                 __float_as_uint(tf32_rn(a_at(g8, 8 * kt + t4 + 4))),
                                 __float_as_uint(tf32_rn(a_at(g8 + 8, 8 * kt + t4 + 4)))};
          const uint32_t b0 = __float_as_uint(tf32_rn(b_at(8 * kt + t4, 8 * nh + g8)));
          const uint32_t b1 = __float_as_uint(tf32_rn(b_at(8 * kt + t4 + 4, 8 * nh + g8)));
          asm volatile(
              "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
              : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        }
      };
#pragma unroll 1
      for (int bi = bj + 1; bi < 4; ++bi) {
        float acc[4] = {};
#pragma unroll 1
        for (int bk = bj; bk < bi; ++bk)
          half_mma(acc, [&](int r, int cidx) { return T_at(bi, bk, r, cidx); }, [&](int r, int cidx) { return X_at(bk, bj, r, cidx); });
        const int col = 16 * bj + 8 * nh + 2 * t4;
        aim[AI(16 * bi + g8, col)] = tf32_rn(-acc[0]);
        aim[AI(16 * bi + g8, col + 1)] = tf32_rn(-acc[1]);
        aim[AI(16 * bi + g8 + 8, col)] = tf32_rn(-acc[2]);
        aim[AI(16 * bi + g8 + 8, col + 1)] = tf32_rn(-acc[3]);
        __syncwarp();
      }
    }
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  // ---- 4. MMA2 (tf32): W^T at TMEM columns 0..63, U^T at 64..127
  if (wid < 2 && !s.abort_flag) {  // warp 0: W^T, warp 1: U^T
    tc::tc_fence_after_sync();
    constexpr uint32_t idesc = tc::instr_desc(2, 128, BS);
    tc::mma_tf32_ktile_warp(tc::tmem_addr(tm, 0, 64 * wid), tc::smem_u32(wid == 0 ? s.y.et : s.x.sol.zt), D,
                            tc::smem_u32(s.x.sol.ai), BS, BS, idesc);
    tc::mma_commit_warp(&s.bar_m2);
  }
  if (wid == 0) tc::mbar_wait(&s.bar_m2, 0, &s.abort_flag, status, 0x2000u);
  __syncthreads();
  tc::tc_fence_after_sync();

  // ---- 5. W and Qg rows into the WQ staging image (E^T is dead now), U^T straight to global; each
  //         thread handles the 32 tokens of its half
  {
    const int ca = (c >> 3) * A_PAD * 8 + (c & 7);
    // U^T of the first value head: fp16 image [tok/8][128 dv][8] of value chunk-head (b, ih * rep, n)
    char* ut_g = P.ut + (size_t)(((int64_t)ib * HK * rep + (int64_t)ih * rep) * NC + n) * (D * BS * 2) + c * 16;
    float val[32];
    tc::tmem_ld32(tc::tmem_addr(tm, lq * 32, 32 * hf), val);
    tc::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) s.y.wq[ca + (32 * hf + i) * 8] = __float2bfloat16_rn(val[i]);
    {   // Qg rows from this thread's gating stash: word t = the two channels 2 cp, 2 cp + 1 of token 16 sbk + t
      float qv[16];
      tc::tmem_ld16(tc::tmem_addr(tm, lq * 32, kQgCol + 16 * (sbk >> 1)), qv);
      tc::tmem_ld_wait();
      uint32_t* wq32 = reinterpret_cast<uint32_t*>(s.y.wq) + (cp >> 2) * A_PAD * 4 + (cp & 3);
#pragma unroll
      for (int i = 0; i < 16; ++i) wq32[(BS + 16 * sbk + i) * 4] = __float_as_uint(qv[i]);
    }
    tc::tmem_ld32(tc::tmem_addr(tm, lq * 32, 64 + 32 * hf), val);
    tc::tmem_ld_wait();
#pragma unroll
    for (int i8 = 0; i8 < 4; ++i8) {
      uint32_t pk[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        __half2 h = __floats2half2_rn(val[8 * i8 + 2 * x] * (1.f / kValScale),
                                      val[8 * i8 + 2 * x + 1] * (1.f / kValScale));
        pk[x] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(ut_g + (size_t)(hf * 4 + i8) * D * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  // WQ record: 16 K chunks x 128 rows x 16 bytes; every thread copies 8 pieces with 128-bit accesses
  // (16 consecutive threads cover 256 contiguous bytes) and nothing waits on them
  if (!s.abort_flag) {
    char* g_wq = P.wq + (size_t)ch * (2 * BS * D * 2);
    const char* stage = reinterpret_cast<const char*>(s.y.wq);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const int piece = tid + kThreads * x;                 // 0..2047
      const int kc = piece >> 7, row = piece & 127;
      *reinterpret_cast<uint4*>(g_wq + (size_t)piece * 16) =
          *reinterpret_cast<const uint4*>(stage + (kc * A_PAD + row) * 16);
    }
  }

  // ---- 6. the further value heads of this key head: (w*v)^T straight into its shared-memory image (the previous
  //         head's product has completed, so the image and the U^T columns of tensor memory are free), one tf32
  //         product against the same Ai^T, U^T out. Ai^T, the only other operand, stays where it is.
#pragma unroll 1
  for (int hr = 1; hr < rep; ++hr) {
    {
      const uint32_t* vp = reinterpret_cast<const uint32_t*>(v + (vrow0 + hr) * D + vsoff) + cp;
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(w + (vrow0 + hr) * D + vsoff) + cp;
      uint32_t vr[16], wr[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) { vr[u] = __ldg(vp + u * vpstride); wr[u] = __ldg(wp + u * vpstride); }
#pragma unroll
      for (int t4 = 0; t4 < 4; ++t4) {
        float zx[4], zy[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 vf = bf16x2_bits_to_f32(vr[4 * t4 + u]), wf = bf16x2_bits_to_f32(wr[4 * t4 + u]);
          zx[u] = tf32_rn(vf.x * wf.x); zy[u] = tf32_rn(vf.y * wf.y);
        }
        const int tq = 4 * sbk + t4;
        *reinterpret_cast<float4*>(&s.x.sol.zt[(tq * D + c0) * 4]) = make_float4(zx[0], zx[1], zx[2], zx[3]);
        *reinterpret_cast<float4*>(&s.x.sol.zt[(tq * D + c0 + 1) * 4]) = make_float4(zy[0], zy[1], zy[2], zy[3]);
      }
    }
    tc::fence_async_smem();
    tc::tc_fence_before_sync();
    __syncthreads();
    if (wid == 1 && !s.abort_flag) {
      tc::tc_fence_after_sync();
      constexpr uint32_t idesc = tc::instr_desc(2, 128, BS);
      tc::mma_tf32_ktile_warp(tc::tmem_addr(tm, 0, 64), tc::smem_u32(s.x.sol.zt), D, tc::smem_u32(s.x.sol.ai), BS, BS, idesc);
      tc::mma_commit_warp(&s.bar_m2v);
    }
    if (wid == 0) tc::mbar_wait(&s.bar_m2v, (hr - 1) & 1, &s.abort_flag, status, 0x2000u);
    __syncthreads();
    tc::tc_fence_after_sync();
    {
      char* ut_g = P.ut + (size_t)(((int64_t)ib * HK * rep + (int64_t)ih * rep + hr) * NC + n) * (D * BS * 2) + c * 16;
      float val[32];
      tc::tmem_ld32(tc::tmem_addr(tm, lq * 32, 64 + 32 * hf), val);
      tc::tmem_ld_wait();
#pragma unroll
      for (int i8 = 0; i8 < 4; ++i8) {
        uint32_t pk[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          __half2 h = __floats2half2_rn(val[8 * i8 + 2 * x] * (1.f / kValScale),
                                        val[8 * i8 + 2 * x + 1] * (1.f / kValScale));
          pk[x] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(ut_g + (size_t)(hf * 4 + i8) * D * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
  }
  if (wid == 0) tc::tmem_dealloc(tm, kTmemCols);
}

}  // namespace

int launch_prep_tc(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                   const WsLayout& L, const WsPtrs& P, int B, int S, int H, int HK, int64_t in_bs, float scale,
                   cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  const size_t smem = sizeof(PrepTcSmem) + 128;
  dim3 grid(S / BS, B * HK);
  using bf16 = __nv_bfloat16;
  GDN2_CUDA_TRY(cudaMemsetAsync(P.flags + 2 * (size_t)L.nch, 0, sizeof(int), st));   // length of the flagged list
  auto launch = [&](auto kern) -> int {
    GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
    kern<<<grid, kThreads, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(k),
                                       static_cast<const bf16*>(v), g, static_cast<const bf16*>(b),
                                       static_cast<const bf16*>(w), P, S, H, HK, in_bs, scale, device_sm_count(),
                                       device_status_word());
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  };
  const int rep = H / HK;
  if (rep == 1) {
    switch (HK) {                               // common head counts, whole and sharded
      case 16: return launch(prep_tc_kernel<16, 1>);
      case 8: return launch(prep_tc_kernel<8, 1>);
      case 4: return launch(prep_tc_kernel<4, 1>);
      case 2: return launch(prep_tc_kernel<2, 1>);
      default: return launch(prep_tc_kernel<0, 1>);
    }
  }
  if (rep == 2) {                               // two value heads per key head, whole and sharded
    switch (HK) {
      case 8: return launch(prep_tc_kernel<8, 2>);
      case 4: return launch(prep_tc_kernel<4, 2>);
      case 2: return launch(prep_tc_kernel<2, 2>);
      case 1: return launch(prep_tc_kernel<1, 2>);
      default: break;
    }
  }
  return launch(prep_tc_kernel<0, 0>);
}

}  // namespace gdn2
