// Chunk-local stage of the chunkwise forward, tensor-core (tcgen05 / TMEM) family, for
// DK = DV = 128 and bf16 inputs. One 256-thread block per (chunk, batch*head), two blocks per SM.
// Thread (c, hf) owns key channel c and value channel c for the tokens of half hf of the chunk
// (32 tokens = two 16-token sub-blocks), so the cumulative decay is a private running sum plus one
// prefix exchanged through shared memory. Two threads per channel, rather than one, double the warps
// an SM has to hide latency with at the same shared-memory footprint.
//
// What the reference spreads over five kernels (cumsum, intra_diag, inter_blocks, solve, wy:
// gdn2/forward.py:65-535 of the reference project) is one kernel here, and the intermediates it
// round-trips through HBM (G, Akk, Ai) never leave the SM:
//
//  1. G = log2(e) * cumsum(g) as a running sum. The overflow-safe factorisation of the reference
//     (gdn2/forward.py:266-270): rows of sub-block i (16 tokens) are scaled by 2^(G_r - ref_i),
//     ref_i = G at the sub-block's first row, and paired with key rows scaled by 2^(ref_i - G_s).
//     Left of the diagonal both exponents are <= 0. ON the diagonal sub-block the key factor is
//     >= 1 but bounded by the decay span of 16 tokens; the reference evaluates those blocks
//     pairwise on CUDA cores (intra_diag_kernel) -- here they ride the same tensor-core product
//     as long as every sub-block's span stays below 2^64. A chunk that decays faster is flagged in
//     the workspace and redone exactly by the SIMT family's kernel.
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
// columns of the thread's own lane (packed bf16 pairs).
#include <cstdlib>

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
constexpr float kMaxSpanLog2 = 64.f;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kZCol = 192;   // TMEM columns [192,256): w*v of the thread's value channel (fp32)
constexpr uint32_t kQgCol = 160;  // TMEM columns [160,192): packed Qg of the thread's channel

#ifdef GDN2_SCAN_TIMING
__device__ unsigned long long g_prep_timing[16];
#define PTICK(i) do { if (blockIdx.x == 100 && blockIdx.y == 32 && tid == 0) { long long now_ = clock64(); g_prep_timing[i] = now_ - tprev; tprev = now_; } } while (0)
#else
#define PTICK(i) do {} while (0)
#endif

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
  float pre[2][3][D];                        // per half and channel: first-row G of its two sub-blocks, its total (relative)
  uint64_t bar_m1, bar_m2;
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
__device__ __forceinline__ float pick4(int j, float a0, float a1, float a2, float a3) {
  return j == 0 ? a0 : j == 1 ? a1 : j == 2 ? a2 : a3;
}

// Raw values of one channel for 8 consecutive tokens, converted only when consumed.
struct Raw8 {
  float g[8];
  uint32_t k[8], q[8], b[8];              // bf16 bit patterns, zero-extended: one register each, no packing
};
// 16-bit load into a full register, and its value as fp32 (a bf16 is the top half of an fp32)
__device__ __forceinline__ uint32_t ldg_u16(const __nv_bfloat16* p) {
  return static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p)));
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ void load_raw8(Raw8& r, const float* gp, const __nv_bfloat16* kp, const __nv_bfloat16* qp,
                                          const __nv_bfloat16* bp, size_t rstride) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const size_t off = u * rstride;
    r.g[u] = __ldg(gp + off); r.k[u] = ldg_u16(kp + off); r.q[u] = ldg_u16(qp + off); r.b[u] = ldg_u16(bp + off);
  }
}

// Per-sub-block constants of the gating step.
struct SubConst {
  float ref, refn, gam_ref, kg_c, cc_a, cc_b, nx_c;
  int j, off_j;
};

// HT > 0: the number of heads is a compile-time constant, so every token offset of the strided channel
// loads folds into the load instruction's immediate; HT = 0 takes it from the argument.
template <int HT>
__global__ void __launch_bounds__(kThreads, 2)
prep_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
               const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
               const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ w, WsPtrs P, int S, int H,
               int64_t in_bs, float scale, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PrepTcSmem& s = *reinterpret_cast<PrepTcSmem*>(smem_raw);
  const int NC = S / BS;
  const int n = blockIdx.x, bh = blockIdx.y;
  const int ib = bh / H, ih = bh % H;
  const int64_t ch = (int64_t)bh * NC + n;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int c = tid & (D - 1);                                          // channel = TMEM lane
  const int hf = tid >> 7;                                              // token half: tokens [32 hf, 32 hf + 32)
  const int lq = wid & 3;                                               // TMEM lane quarter of this warp
  const size_t row0 = ((size_t)ib * in_bs + (size_t)n * BS) * H + ih;   // token row of t = 0
  const size_t rstride = HT > 0 ? (size_t)HT * D : (size_t)H * D;       // elements between tokens
  const size_t hoff = (size_t)(32 * hf) * rstride;                      // first token of this thread's half
  const float* gp = g + row0 * D + c + hoff;
#ifdef GDN2_SCAN_TIMING
  long long tprev = clock64();
#endif

  // Pull the whole input tile of this chunk-head towards L2 before anything depends on it: 64 rows x
  // (5 x 256 B + 512 B) = 896 128-byte lines, 3.5 per thread.
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
        const char* ptr = static_cast<const char*>(tb) + (row0 * D + (size_t)rowi * rstride) * es + seg * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
      }
    }
  }

  // ---- 1a. G at the first row of every sub-block and at the last token; decay-span check.
  //          Each thread sums its own half; the halves meet through shared memory.
  float ref0, ref1, ref2, ref3, g_last, run0;
  bool bad = false;
  {
    float gv[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) gv[t] = __ldg(gp + t * rstride) * kLog2e;     // 32 independent loads in flight
    float run = 0.f, first[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      first[j] = run + gv[16 * j];
#pragma unroll
      for (int u = 0; u < 16; ++u) run += gv[16 * j + u];
      bad |= !((first[j] - run) <= kMaxSpanLog2);
    }
    s.pre[hf][0][c] = first[0]; s.pre[hf][1][c] = first[1]; s.pre[hf][2][c] = run;
  }
  if (tid == 0) {
    tc::mbar_init(&s.bar_m1, 4);     // one commit per issuing warp
    tc::mbar_init(&s.bar_m2, 2);
    s.abort_flag = 0;
    tc::mbar_init_fence();
  }
  PTICK(0);
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (tid == 0) P.flags[ch] = any_bad ? 1 : 0;
  if (any_bad) return;              // the exact kernel redoes this chunk; nothing allocated yet
  {
    const float tot0 = s.pre[0][2][c];
    ref0 = s.pre[0][0][c]; ref1 = s.pre[0][1][c];
    ref2 = tot0 + s.pre[1][0][c]; ref3 = tot0 + s.pre[1][1][c];
    g_last = tot0 + s.pre[1][2][c];
    run0 = hf ? tot0 : 0.f;
  }
  if (wid == 0) tc::tmem_alloc(&s.tmem_base, kTmemCols);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = s.tmem_base;

  PTICK(1);
  // ---- 1b. gated operands of channel c for this thread's 32 tokens, in four groups of 8; the next
  //          group's 32 loads are issued (raw, unconverted) before the current one is processed
  {
    const __nv_bfloat16* qp = q + row0 * D + c + hoff;
    const __nv_bfloat16* kp = k + row0 * D + c + hoff;
    const __nv_bfloat16* bp = b + row0 * D + c + hoff;
    const int ca = (c >> 3) * A_PAD * 8 + (c & 7);
    const int cb = (c >> 3) * B_PAD * 8 + (c & 7);
    char* kgt_g = P.kgt + (size_t)ch * (D * BS * 2) + c * 16;   // fp16 image [tok/8][128 dk][8]
    float run = run0;
    SubConst sc;

    auto sub_consts = [&](int j) {
      sc.j = j;
      sc.off_j = 8 * j * (j + 1);                               // first row of B_j: 0, 16, 48, 96
      sc.ref = pick4(j, ref0, ref1, ref2, ref3);
      sc.refn = pick4(j, ref1, ref2, ref3, 0.f);                // ref of the next sub-block (unused for j = 3)
      sc.gam_ref = ex2(sc.ref);
      sc.nx_c = ex2(((j < 3) ? sc.refn : g_last) - sc.ref);    // 2^(refn - run) = nx_c * 2^(ref - run)
      sc.kg_c = (j < 3) ? ex2(g_last - sc.refn) : 1.f;
      sc.cc_a = ex2(pick4(j, ref2, ref3, 0.f, 0.f) - sc.refn);  // B_{j+2} relative to B_{j+1}
      sc.cc_b = ex2(ref3 - sc.refn);                            // B_{j+3} relative to B_{j+1} (j = 0 only)
    };
    // one group: tokens t0 .. t0 + 7 (t0 a multiple of 8)
    auto gate8 = [&](const Raw8& r, int t0) {
      const int j = sc.j;
      uint32_t qgp[4], kgp[4];
#pragma unroll
      for (int t4 = 0; t4 < 2; ++t4) {
        float e4[4], kg4[4], qg4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int uu = 4 * t4 + u;
          const int t = t0 + uu;
          run += r.g[uu] * kLog2e;
          const float kf = bf16_bits_to_f32(r.k[uu]), qf = bf16_bits_to_f32(r.q[uu]);
          const float a = ex2(run - sc.ref);                  // <= 1
          const float co = ex2(sc.ref - run);                 // >= 1, bounded by the span check
          const float nx = sc.nx_c * co;                      // 2^(refn - run) (2^(g_last - run) for j = 3), <= 1
          const float e = bf16_bits_to_f32(r.b[uu]) * kf;
          s.x.ops.a_own[ca + t * 8] = __float2bfloat16_rn(e * a);
          s.x.ops.a_own[ca + (BS + t) * 8] = __float2bfloat16_rn(qf * a);
          s.x.ops.bfam[cb + (sc.off_j + t) * 8] = __float2bfloat16_rn(kf * co);
          const float kn = kf * nx;
          if (j < 3) s.x.ops.bfam[cb + (8 * (j + 1) * (j + 2) + t) * 8] = __float2bfloat16_rn(kn);
          if (j < 2) s.x.ops.bfam[cb + (8 * (j + 2) * (j + 3) + t) * 8] = __float2bfloat16_rn(kn * sc.cc_a);
          if (j < 1) s.x.ops.bfam[cb + (96 + t) * 8] = __float2bfloat16_rn(kn * sc.cc_b);
          const float gam = a * sc.gam_ref;
          e4[u] = tf32_rn(e * gam);
          qg4[u] = scale * qf * gam;
          kg4[u] = kn * sc.kg_c * kValScale;
        }
        const int tq = (t0 >> 2) + t4;                          // token quad index
        *reinterpret_cast<float4*>(&s.y.et[(tq * D + c) * 4]) = make_float4(e4[0], e4[1], e4[2], e4[3]);
        __half2 h01 = __floats2half2_rn(kg4[0], kg4[1]), h23 = __floats2half2_rn(kg4[2], kg4[3]);
        kgp[2 * t4] = *reinterpret_cast<uint32_t*>(&h01);
        kgp[2 * t4 + 1] = *reinterpret_cast<uint32_t*>(&h23);
        __nv_bfloat162 p01 = __floats2bfloat162_rn(qg4[0], qg4[1]), p23 = __floats2bfloat162_rn(qg4[2], qg4[3]);
        qgp[2 * t4] = *reinterpret_cast<uint32_t*>(&p01);
        qgp[2 * t4 + 1] = *reinterpret_cast<uint32_t*>(&p23);
      }
      tc::tmem_st4(tc::tmem_addr(tm, lq * 32, kQgCol + (t0 >> 1)), qgp);
      *reinterpret_cast<uint4*>(kgt_g + (size_t)(t0 >> 3) * D * 16) = make_uint4(kgp[0], kgp[1], kgp[2], kgp[3]);
    };

    Raw8 ra, rb;
    load_raw8(ra, gp, kp, qp, bp, rstride);
#pragma unroll 1
    for (int sb = 0; sb < 2; ++sb) {                            // this thread's two sub-blocks
      const int t0 = 32 * hf + 16 * sb;
      const size_t o8 = (size_t)(16 * sb + 8) * rstride;
      load_raw8(rb, gp + o8, kp + o8, qp + o8, bp + o8, rstride);
      sub_consts(2 * hf + sb);
      gate8(ra, t0);
      if (sb == 0) {
        const size_t o16 = (size_t)16 * rstride;
        load_raw8(ra, gp + o16, kp + o16, qp + o16, bp + o16, rstride);
      }
      gate8(rb, t0 + 8);
    }
    tc::tmem_st_wait();
    if (hf == 1) P.gl[(size_t)ch * D + c] = ex2(g_last);
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  PTICK(2);
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
  PTICK(3);
  // value side: raw loads issued while the tensor core works
  // z = w*v of this thread's value channel waits in TMEM columns [192,256) of its own lane until the
  // MMA1 operands are dead and (w*v)^T can take their place in shared memory
  {
    const __nv_bfloat16* vp = v + row0 * D + c + hoff;
    const __nv_bfloat16* wp = w + row0 * D + c + hoff;
    uint32_t vr[16], wr[16], vn[16], wn[16];              // raw bf16 bits: converted one group behind the loads
#pragma unroll
    for (int u = 0; u < 16; ++u) { vr[u] = ldg_u16(vp + u * rstride); wr[u] = ldg_u16(wp + u * rstride); }
#pragma unroll
    for (int u = 0; u < 16; ++u) { vn[u] = ldg_u16(vp + (16 + u) * rstride); wn[u] = ldg_u16(wp + (16 + u) * rstride); }
    float z[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) z[u] = tf32_rn(bf16_bits_to_f32(vr[u]) * bf16_bits_to_f32(wr[u]));
    tc::tmem_st16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * hf), z);
#pragma unroll
    for (int u = 0; u < 16; ++u) z[u] = tf32_rn(bf16_bits_to_f32(vn[u]) * bf16_bits_to_f32(wn[u]));
    tc::tmem_st16(tc::tmem_addr(tm, lq * 32, kZCol + 32 * hf + 16), z);
    tc::tmem_st_wait();
  }
  PTICK(4);
  // one warp polls the MMA barrier; the rest sleep at the block barrier instead of spending issue slots
  if (wid == 0) tc::mbar_wait(&s.bar_m1, 0, &s.abort_flag, status, 0x1000u);
  __syncthreads();
  tc::tc_fence_after_sync();
  PTICK(5);

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
    // (w*v)^T image from the TMEM stash: each thread moves the 32 tokens it produced
#pragma unroll 1
    for (int jj = 2 * hf; jj < 2 * hf + 2; ++jj) {
      float z[16];
      tc::tmem_ld16(tc::tmem_addr(tm, lq * 32, kZCol + 16 * jj), z);
      tc::tmem_ld_wait();
#pragma unroll
      for (int t4 = 0; t4 < 4; ++t4)
        *reinterpret_cast<float4*>(&s.x.sol.zt[((4 * jj + t4) * D + c) * 4]) =
            make_float4(z[4 * t4], z[4 * t4 + 1], z[4 * t4 + 2], z[4 * t4 + 3]);
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();

  PTICK(6);
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
    // X_ij, distance d = i - j = 1, 2, 3; warp w < 4 - d takes block (w + d, w)
#pragma unroll 1
    for (int d = 1; d < 4; ++d) {
      if (wid + d < 4) {
        const int bj = wid, bi = wid + d;
        float acc[2][4] = {};
#pragma unroll 1
        for (int bk = bj; bk < bi; ++bk)
          block_mma(acc, [&](int r, int cidx) { return T_at(bi, bk, r, cidx); }, [&](int r, int cidx) { return X_at(bk, bj, r, cidx); });
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          aim[AI(16 * bi + g8, 16 * bj + 8 * nt + 2 * t4)] = tf32_rn(-acc[nt][0]);
          aim[AI(16 * bi + g8, 16 * bj + 8 * nt + 2 * t4 + 1)] = tf32_rn(-acc[nt][1]);
          aim[AI(16 * bi + g8 + 8, 16 * bj + 8 * nt + 2 * t4)] = tf32_rn(-acc[nt][2]);
          aim[AI(16 * bi + g8 + 8, 16 * bj + 8 * nt + 2 * t4 + 1)] = tf32_rn(-acc[nt][3]);
        }
      }
      __syncthreads();
    }
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  PTICK(7);
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
  PTICK(8);

  // ---- 5. W and Qg rows into the WQ staging image (E^T is dead now), U^T straight to global; each
  //         thread handles the 32 tokens of its half
  {
    const int ca = (c >> 3) * A_PAD * 8 + (c & 7);
    char* ut_g = P.ut + (size_t)ch * (D * BS * 2) + c * 16;       // fp16 image [tok/8][128 dv][8]
    float val[32];
    tc::tmem_ld32(tc::tmem_addr(tm, lq * 32, 32 * hf), val);
    tc::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) s.y.wq[ca + (32 * hf + i) * 8] = __float2bfloat16_rn(val[i]);
    {
      float qv[16];
      tc::tmem_ld16(tc::tmem_addr(tm, lq * 32, kQgCol + 16 * hf), qv);
      tc::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t pk = __float_as_uint(qv[i]);
        reinterpret_cast<uint16_t*>(s.y.wq)[ca + (BS + 32 * hf + 2 * i) * 8] = static_cast<uint16_t>(pk & 0xFFFFu);
        reinterpret_cast<uint16_t*>(s.y.wq)[ca + (BS + 32 * hf + 2 * i + 1) * 8] = static_cast<uint16_t>(pk >> 16);
      }
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
  PTICK(9);
  if (wid == 0) tc::tmem_dealloc(tm, kTmemCols);
  // WQ record: 16 K chunks x 128 rows x 16 bytes; every thread copies 8 pieces with 128-bit accesses
  // (16 consecutive threads cover 256 contiguous bytes) and the block ends without waiting on them
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
  PTICK(10);
}

}  // namespace

int launch_prep_tc(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                   const WsLayout& L, const WsPtrs& P, int B, int S, int H, int64_t in_bs, float scale,
                   cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  size_t smem = sizeof(PrepTcSmem) + 128;
#ifdef GDN2_SCAN_TIMING
  if (getenv("GDN2_EXP_ONE_BLOCK")) smem = 120 * 1024;    // experiment: one resident block per SM
#endif
  dim3 grid(S / BS, B * H);
  using bf16 = __nv_bfloat16;
  auto launch = [&](auto kern) -> int {
    GDN2_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(k),
                                       static_cast<const bf16*>(v), g, static_cast<const bf16*>(b),
                                       static_cast<const bf16*>(w), P, S, H, in_bs, scale, device_status_word());
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  };
  switch (H) {                                  // common head counts, whole and sharded
    case 16: return launch(prep_tc_kernel<16>);
    case 8: return launch(prep_tc_kernel<8>);
    case 4: return launch(prep_tc_kernel<4>);
    case 2: return launch(prep_tc_kernel<2>);
    default: return launch(prep_tc_kernel<0>);
  }
}

#ifdef GDN2_SCAN_TIMING
extern "C" int gdn2_debug_prep_timing(unsigned long long* out16) {
  return cudaMemcpyFromSymbol(out16, g_prep_timing, sizeof(unsigned long long) * 16) == cudaSuccess ? 0 : -6;
}
#endif

}  // namespace gdn2
