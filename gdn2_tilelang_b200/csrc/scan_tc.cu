// Sequential state scan fused with the output, tensor-core (tcgen05 / TMEM / TMA) family, for
// DK = DV = 128, bf16 outputs, fp32 state. One block walks a run of consecutive chunks of one
// (batch, head); the state never leaves the SM between chunks.
//
// The algebra of the reference's prefill_scan_kernel (gdn2/inference.py:446-475 of the reference
// project) is evaluated TRANSPOSED so that every product has the 128 value channels as the MMA M
// dimension (= TMEM lane = thread), tokens or key channels as N:
//
//   MMA1   [WS | O][dv, tok] = S^T[dv,dk] * [W ; Qg][tok,dk]^T  (W S)^T and (Qg S)^T, one N = 128 product, bf16
//   regs   Un^T[dv,tok] = U^T - WS
//   MMA3   P [dv,dk]    = Un^T[dv,tok] * KG^T[dk,tok]^T       (KG^T Un)^T      fp16 (scaled, see common.cuh)
//   MMA2   O [dv, r]   += Un^T[dv,s] * Aqk[r,s]^T             (tril(Aqk) Un)^T fp16 (same scaled Un^T image)
//   regs   S^T         <- gamma_C[dk] * S^T + P   (the fp32 state lives in registers, 64 values per thread)
//
// Only MMA1, the Un pass, MMA3 and the state pass are on the recurrence's critical path; the
// kernel is organised around that:
//   * warp 8 issues every MMA (converged, one elected lane), MMA3 before MMA2 so the state update never
//     queues behind the output product; one thread of warp 9 issues every bulk copy.
//   * warps 10-13 read each finished O accumulator into registers, release it, and write the rows
//     out through a shared staging tile with 128-bit coalesced stores, off the critical path.
//   * warps 0-7 (256 threads; two warps share each 32-lane quarter of TMEM and split its columns)
//     do the register passes and hand each result over the moment the next product can use it.
//   * operands arrive as whole workspace records with one bulk copy each; WQ, KG^T and U^T are
//     double buffered so that a copy is always issued a full chunk ahead of its use.
//   * hand-offs are mbarriers (arrive / wait), every wait is bounded (tc_utils.cuh); there is no
//     block-level barrier inside the chunk loop.
//   * the A operands (S^T in bf16, Un^T in fp16) never touch shared memory: the register
//     passes store them as packed 16-bit pairs into tensor memory and the MMAs read them from there.
//
// TMEM columns: [0,128) the update product P; [128,192) WS; [192,256) the O accumulator;
// [320,384) S^T bf16 pairs; [384,416) Un^T/256 fp16 pairs.
//
// Sequence-parallel form. One block per (batch, head) leaves most of the GPU idle when a GPU holds few
// (batch, head) pairs (a head-sharded layer), and its chunk-to-chunk chain then sets the time. The
// recurrence is affine in the state, S_out = T S_in + C per run of chunks, with T a [DK, DK] matrix that
// does not depend on the values: running the very same chunk loop from S = I with U = 0 yields T. So the
// sequence is cut into `nseg` segments and evaluated in three launches:
//   pass 1  one "local" block per segment (from the true initial state for segment 0, from zero for the
//           others: outputs, C_j) and one "transition" block per segment j >= 1 (from the identity, no U,
//           no outputs: T_j); the transition block also records after how many chunks every entry of its
//           running T fell below 2^-27 for good (`stop_j`): from there on the local outputs are already
//           the true ones;
//   pass 2  scan_combine_kernel chains S_in(j+1) = T_j S_in(j) + C_j in fp32 (T_j is skipped where it
//           vanished) and writes every segment's true entering state and the final state;
//   pass 3  one block per segment j >= 1 redoes chunks [0, stop_j) from the true entering state and
//           overwrites their outputs.
// Nothing waits on another block inside a launch. With slowly decaying gates stop_j is the segment
// length and the cost is two chains of NC / nseg chunks; with the usual gates it is one such chain plus
// a few chunks.
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc_utils.cuh"

namespace gdn2 {

namespace {

constexpr int D = 128;
constexpr int BS = kChunk;
constexpr int kComputeThreads = 256;
constexpr int kOutputThreads = 128;
constexpr int kThreads = kComputeThreads + 64 + kOutputThreads;   // + issuer warp + producer warp + output warps

constexpr uint32_t kWqBytes = 2 * BS * D * 2;    // 32 KiB
constexpr uint32_t kAqkBytes = BS * BS * 2;      //  8 KiB
constexpr uint32_t kKgtBytes = D * BS * 2;       // 16 KiB (fp16)
constexpr uint32_t kUtBytes = D * BS * 2;        // 16 KiB (fp16)
constexpr uint32_t kColWs = 128, kColO = 192;
constexpr uint32_t kColSb = 320, kColUn16 = 384;   // packed 16-bit A operands in TMEM

struct ScanTcSmem {
  __nv_bfloat16 wq[2][2 * BS * D];   // B of MMA1w/q: [dk/8][128 rows: W tok 0..63, Qg tok 0..63][8]
  __half aqk[BS * BS];               // B of MMA2: [s/8][64 r][8], 256 * Aqk
  __half kgt[2][D * BS];             // B of MMA3: [tok/8][128 dk][8], 256 * KG
  __half ut[2][D * BS];              // U^T / 256: [tok/8][128 dv][8]
  __nv_bfloat16 ostage[BS * D];      // output rows [tok][dv] on their way to global memory
  float gl[4][D];                    // gamma at the last token of chunk n (slot n & 3), copied with KG^T
  uint64_t bar_wq[2], bar_kgt[2], bar_ut[2], bar_aqk;   // bulk-copy arrival
  uint64_t bar_m1, bar_m3, bar_m2;                      // MMA completion
  uint64_t bar_sb, bar_un;                              // compute threads -> issuer (256 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  int last_big[kComputeThreads / 32];                   // transition blocks: last chunk after which an entry was still >= kVanish
  int nc_limit;                                         // chunks this block walks; a transition block lowers it once its matrix vanished
};

// A transition matrix entry below this is treated as vanished: 128 of them times the entering state stay
// below 1e-6 of that state, three orders under the fp32-state tolerance and far under bf16 output resolution.
constexpr float kVanish = 7.450580596923828e-09f;   // 2^-27

// What a block of the cut scan does (ScanPlan::pass). kWhole: one block per (batch, head) over the whole
// sequence. kFirst: blockIdx = slot * BH + bh; slots [0, nseg - 1) are transition blocks of segment slot + 1
// (first, because they are short once their matrix has vanished and free their SMs for the rest), slots
// [nseg - 1, 2 nseg - 1) local blocks of segment slot - nseg + 1. kRedo: blockIdx = (seg - 1) * BH + bh.
// `guarded`: the launch holds more blocks than SMs and only pays off when the transition blocks end early, so
// the blocks first look at the mode word the decay check left in the workspace: if it says "slow", the local
// block of segment 0 walks the whole sequence alone, exactly as kWhole, and every other block returns at once.
// kOutput: the chunk-parallel output from stored chunk states (no recurrence): blockIdx = seg * BH + bh, every
// block walks the chunks of its segment and takes the state entering each chunk from `hs` instead of carrying it.
enum ScanPass : int { kWhole = 0, kFirst = 1, kRedo = 3, kOutput = 4 };
struct ScanPlan {
  int pass, nseg, guarded;
};

// Optional epilogue of the output rows: the layer's gated RMSNorm (gdn2/attention.py:218-229 of the reference
// project), o <- o * rsqrt(mean(o^2) + eps) * weight * silu(gate) per (token, head), applied to the bf16-rounded
// rows on their way from the staging tile to global memory. gate == nullptr: plain outputs.
struct ScanNorm {
  const __nv_bfloat16* gate;     // gate of o[b, t, h, c] at gate[(b * batch_stride + t) * row_stride + h * 128 + c]
  const __nv_bfloat16* weight;   // [128]
  int64_t row_stride, batch_stride;
  float eps;
};

enum : uint32_t {
  kWaitWq = 0x10, kWaitUt = 0x20, kWaitAqk = 0x40, kWaitKgt = 0x80, kWaitM1 = 0x100, kWaitM2 = 0x200,
  kWaitM3 = 0x400, kWaitSb = 0x800, kWaitUn = 0x4000
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
}
// one arrival per warp: every lane has fenced its tensor-memory traffic, the warp converges, lane 0 arrives
// (256 single-thread arrivals on one shared-memory word cost the hand-off several hundred cycles)
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
// barrier among the 128 output threads only (hardware barrier 2)
__device__ __forceinline__ void output_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
// barrier among the 256 compute threads (hardware barrier 3) fused with an AND over one predicate per thread
__device__ __forceinline__ bool compute_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "barrier.cta.red.and.pred q, 3, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ float pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return __uint_as_float(*reinterpret_cast<uint32_t*>(&t));
}
__device__ __forceinline__ float pack_f16x2(float lo, float hi) {
  __half2 t = __floats2half2_rn(lo, hi);
  return __uint_as_float(*reinterpret_cast<uint32_t*>(&t));
}
__device__ __forceinline__ void unpack8_f16(const uint4& p, float* x) {
  float2 f;
  f = __half22float2(*reinterpret_cast<const __half2*>(&p.x)); x[0] = f.x; x[1] = f.y;
  f = __half22float2(*reinterpret_cast<const __half2*>(&p.y)); x[2] = f.x; x[3] = f.y;
  f = __half22float2(*reinterpret_cast<const __half2*>(&p.z)); x[4] = f.x; x[5] = f.y;
  f = __half22float2(*reinterpret_cast<const __half2*>(&p.w)); x[6] = f.x; x[7] = f.y;
}

// The output rows of one chunk from the staging tile to global memory through the gated RMSNorm. 128 output
// threads; the 16 threads that share a row (half a warp) hold its 128 values, 8 each. Kept out of line so that its
// registers do not add to those of the chunk loop.
__device__ __noinline__ void store_rows_normed(const __nv_bfloat16* ostage, __nv_bfloat16* obase, const __nv_bfloat16* gbase,
                                               int64_t gate_row_stride, const __nv_bfloat16* weight, float eps, int otid,
                                               int H) {
  float nw[8];                                         // norm weights of this thread's 8 columns
  {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight + (otid & 15) * 8));
    const uint32_t u[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { nw[2 * i] = __uint_as_float(u[i] << 16); nw[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  uint4 gv[8];
#pragma unroll
  for (int x = 0; x < 8; ++x)                          // all eight gate loads in flight before the first use
    gv[x] = __ldg(reinterpret_cast<const uint4*>(gbase + (size_t)((otid >> 4) + 8 * x) * gate_row_stride));
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int piece = otid + x * kOutputThreads;
    const int row = piece >> 4, col = (piece & 15) * 8;
    const uint4 ovv = *reinterpret_cast<const uint4*>(&ostage[row * D + col]);
    const uint32_t ou[4] = {ovv.x, ovv.y, ovv.z, ovv.w}, gu[4] = {gv[x].x, gv[x].y, gv[x].z, gv[x].w};
    float xv[8], gt[8], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xv[2 * i] = __uint_as_float(ou[i] << 16); xv[2 * i + 1] = __uint_as_float(ou[i] & 0xffff0000u);
      gt[2 * i] = __uint_as_float(gu[i] << 16); gt[2 * i + 1] = __uint_as_float(gu[i] & 0xffff0000u);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(xv[i], xv[i], ss);
#pragma unroll
    for (int off = 8; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = rsqrtf(ss * (1.f / D) + eps);
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // silu(g) = g * sigmoid(g) = g * (0.5 + 0.5 tanh(g / 2)): one special-function instruction per element (the
      // output warps have one special-function pipe each and 64 elements per thread and chunk to get through)
      float th;
      asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * gt[i]));
      y[i] = xv[i] * r * nw[i] * gt[i] * fmaf(0.5f, th, 0.5f);
    }
    *reinterpret_cast<uint4*>(obase + (size_t)row * H * D + col) = tc::pack8_bf16(y);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
scan_tc_kernel(WsLayout L, WsPtrs P, ScanPlan plan, ScanNorm norm, const float* __restrict__ s0,
               __nv_bfloat16* __restrict__ o, float* __restrict__ sT, float* __restrict__ hs, int S, int H, int64_t o_bs,
               uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  ScanTcSmem& s = *reinterpret_cast<ScanTcSmem*>(smem_raw);
  const int NC_all = S / BS;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;

  // ---- this block's job: which (batch, head), which run of chunks, where the state comes from and goes to
  const int BH = (int)L.BH;
  int bh = blockIdx.x, seg = 0;
  bool transition = false;                  // identity start, no U, no outputs: yields the segment's transition matrix
  if (plan.pass != kWhole) {
    const int slot = blockIdx.x / BH;
    bh = blockIdx.x % BH;
    if (plan.pass == kFirst) {
      transition = slot < plan.nseg - 1;
      seg = transition ? slot + 1 : slot - (plan.nseg - 1);
    } else if (plan.pass == kRedo) {
      seg = slot + 1;
    } else {
      seg = slot;
    }
  }
  const bool output_only = plan.pass == kOutput;
  if (plan.guarded && *P.seg_mode != 0) {                  // slow decay: no cut after all (uniform over the launch)
    if (plan.pass != kFirst || transition || seg != 0) return;
    plan.pass = kWhole;
  }
  const int ib = bh / H, ih = bh % H;
  const int c_first = plan.pass == kWhole ? 0 : (int)((int64_t)NC_all * seg / plan.nseg);
  const int c_end = plan.pass == kWhole ? NC_all : (int)((int64_t)NC_all * (seg + 1) / plan.nseg);
  int NC = c_end - c_first;                 // chunks this block walks
  if (plan.pass == kRedo) {
    const int redo = P.seg_stop[bh * plan.nseg + seg];
    NC = redo < NC ? redo : NC;
  }
  if (plan.pass == kFirst || plan.pass == kRedo) hs = nullptr;
  // where the state comes from (nullptr = zero, or the identity for a transition block) and where it goes;
  // evaluated where they are used so that they do not occupy registers across the chunk loop
  auto state_source = [&]() -> const float* {
    const size_t seg_rec = ((size_t)bh * plan.nseg + seg) * D * D;
    if (plan.pass == kRedo) return P.seg_in + seg_rec;
    if (plan.pass == kFirst && seg != 0) return nullptr;
    if (output_only) return hs + (((size_t)ib * NC_all + c_first) * H + ih) * D * D;
    return s0 ? s0 + (size_t)bh * D * D : nullptr;
  };
  auto state_sink = [&]() -> float* {
    const size_t seg_rec = ((size_t)bh * plan.nseg + seg) * D * D;
    if (plan.pass == kRedo || output_only) return nullptr;
    if (plan.pass == kFirst) return (transition ? P.seg_t : P.seg_c) + seg_rec;
    return sT ? sT + (size_t)bh * D * D : nullptr;
  };
  const bool write_o = !transition;
  // records that depend on q, k, b, g only exist once per KEY head; U^T per value head
  const int64_t ch0 = ((int64_t)ib * (H / L.rep) + ih / L.rep) * NC_all + c_first;
  const int64_t chv0 = (int64_t)bh * NC_all + c_first;

  const char* g_wq = P.wq + (size_t)ch0 * kWqBytes;
  const char* g_aqk = P.aqk + (size_t)ch0 * kAqkBytes;
  const char* g_kgt = P.kgt + (size_t)ch0 * kKgtBytes;
  const char* g_ut = P.ut + (size_t)chv0 * kUtBytes;
  const float* g_gl = P.gl + (size_t)ch0 * D;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s.bar_wq[i], 1); tc::mbar_init(&s.bar_kgt[i], 1); tc::mbar_init(&s.bar_ut[i], 1);
    }
    tc::mbar_init(&s.bar_aqk, 1); tc::mbar_init(&s.bar_m1, 1); tc::mbar_init(&s.bar_m3, 1); tc::mbar_init(&s.bar_m2, 1);
    // one arrival per warp; a transition block has no outputs, its output warps take no part
    tc::mbar_init(&s.bar_sb, (kComputeThreads + (transition ? 0 : kOutputThreads)) / 32);
    tc::mbar_init(&s.bar_un, kComputeThreads / 32);
    s.abort_flag = 0;
    s.nc_limit = NC;
    tc::mbar_init_fence();
  }
  if (wid == 0) tc::tmem_alloc(&s.tmem_base, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = s.tmem_base;

  if (wid == 9) {
    // =============================== producer: bulk copies of the workspace records ==============
    if (lane == 0) {
      auto load_wq = [&](int n) {
        tc::mbar_expect_tx(&s.bar_wq[n & 1], kWqBytes);
        tc::bulk_g2s(s.wq[n & 1], g_wq + (size_t)n * kWqBytes, kWqBytes, &s.bar_wq[n & 1]);
      };
      auto load_kgt = [&](int n) {
        if (output_only) return;                           // no state update: KG^T and gamma are not needed
        tc::mbar_expect_tx(&s.bar_kgt[n & 1], kKgtBytes + D * 4);
        tc::bulk_g2s(s.kgt[n & 1], g_kgt + (size_t)n * kKgtBytes, kKgtBytes, &s.bar_kgt[n & 1]);
        tc::bulk_g2s(s.gl[n & 3], g_gl + (size_t)n * D, D * 4, &s.bar_kgt[n & 1]);
      };
      auto load_ut = [&](int n) {
        if (transition) return;                            // U = 0: nothing to bring in, nobody waits for it
        tc::mbar_expect_tx(&s.bar_ut[n & 1], kUtBytes);
        tc::bulk_g2s(s.ut[n & 1], g_ut + (size_t)n * kUtBytes, kUtBytes, &s.bar_ut[n & 1]);
      };
      auto load_aqk = [&](int n) {
        tc::mbar_expect_tx(&s.bar_aqk, kAqkBytes);
        tc::bulk_g2s(s.aqk, g_aqk + (size_t)n * kAqkBytes, kAqkBytes, &s.bar_aqk);
      };
      const volatile int* limit = &s.nc_limit;
      int ahead = 0, ut_ahead = 0, aqk_ahead = 0;            // highest chunk whose WQ + KG^T, U^T and Aqk copies were issued
      load_wq(0); load_ut(0); load_kgt(0); load_aqk(0);
      if (NC > 1) { load_wq(1); load_ut(1); load_kgt(1); ahead = ut_ahead = 1; }
      int n = 0;
      for (; n < NC; ++n) {
        if (n >= *limit) break;                              // a transition block whose matrix has vanished stops early
        const uint32_t ph = n & 1;
        // the Un pass of chunk n has consumed its U^T buffer
        bool ok = tc::mbar_wait(&s.bar_un, ph, &s.abort_flag, status, kWaitUn);
        if (ok && n + 2 < *limit) { load_ut(n + 2); ut_ahead = n + 2; }
        // every product of chunk n has completed: refill the operand buffers it read
        ok = ok && tc::mbar_wait(&s.bar_m2, ph, &s.abort_flag, status, kWaitM2);
        if (ok) {
          if (n + 1 < *limit) { load_aqk(n + 1); aqk_ahead = n + 1; }
          if (n + 2 < *limit) { load_wq(n + 2); load_kgt(n + 2); ahead = n + 2; }
        }
      }
      // Copies issued for chunks that no one will consume any more (the limit dropped after they were issued)
      // must land before the block gives its shared memory back.
      if (!s.abort_flag) {
        for (int c = n; c <= ahead; ++c) {
          tc::mbar_wait(&s.bar_wq[c & 1], (c >> 1) & 1, &s.abort_flag, status, kWaitWq);
          if (!output_only) tc::mbar_wait(&s.bar_kgt[c & 1], (c >> 1) & 1, &s.abort_flag, status, kWaitKgt);
        }
        if (!transition)
          for (int c = n; c <= ut_ahead; ++c) tc::mbar_wait(&s.bar_ut[c & 1], (c >> 1) & 1, &s.abort_flag, status, kWaitUt);
        if (aqk_ahead >= n && n < NC) tc::mbar_wait(&s.bar_aqk, aqk_ahead & 1, &s.abort_flag, status, kWaitAqk);
      }
    }
  } else if (wid == 8) {
    // =============================== issuer: every MMA, in critical-path order ==================
    // The whole warp runs this loop converged (identical waits and operands on every lane); one
    // elected lane issues each instruction.
    {
      constexpr uint32_t idesc_n128 = tc::instr_desc(1, 128, 128);   // bf16 operands, N = 128
      constexpr uint32_t idesc_f16 = tc::instr_desc(0, 128, 128);    // fp16 operands, N = 128
      constexpr uint32_t idesc_f16_n64 = tc::instr_desc(0, 128, 64); // fp16 operands, N = 64
      const uint32_t a_sb = tc::tmem_addr(tm, 0, kColSb), a_un16 = tc::tmem_addr(tm, 0, kColUn16);
      const uint32_t a_aqk = tc::smem_u32(s.aqk);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t code) {
        return __all_sync(0xffffffffu, tc::mbar_wait(bar, parity, &s.abort_flag, status, code)) != 0;
      };
      for (int n = 0; n < NC; ++n) {
        if (n >= *(volatile int*)&s.nc_limit) break;         // uniform: every lane reads the same word
        const int b = n & 1;
        const uint32_t ph = n & 1, ph2 = (n >> 1) & 1;
        // S^T (bf16) of chunk n is in place and the O accumulator has been read out
        bool ok = wait_all(&s.bar_wq[b], ph2, kWaitWq);
        ok = ok && wait_all(&s.bar_sb, ph, kWaitSb);
        if (ok) {
          tc::tc_fence_after_sync();
          // one N = 128 product: columns [128,192) = (W S)^T, [192,256) = (Qg S)^T
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, kColWs), a_sb, tc::smem_u32(s.wq[b]), 2 * BS, D, idesc_n128, false);
          tc::mma_commit_warp(&s.bar_m1);
        }
        ok = output_only || wait_all(&s.bar_kgt[b], ph2, kWaitKgt);
        ok = ok && wait_all(&s.bar_un, ph, kWaitUn);
        if (ok && !output_only) {
          tc::tc_fence_after_sync();
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, 0), a_un16, tc::smem_u32(s.kgt[b]), D, BS, idesc_f16, false);
          tc::mma_commit_warp(&s.bar_m3);
        }
        ok = ok && wait_all(&s.bar_aqk, ph, kWaitAqk);
        if (ok) {
          tc::tc_fence_after_sync();
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, kColO), a_un16, a_aqk, BS, BS, idesc_f16_n64, true);
          tc::mma_commit_warp(&s.bar_m2);
        }
      }
    }
  } else if (wid >= 10) {
    // =============================== output warps: O^T -> bf16 rows in global memory =============
    const int lq = wid & 3;
    const int dv = lq * 32 + lane;
    const int otid = tid - (kComputeThreads + 64);
    const uint32_t t_o = tc::tmem_addr(tm, lq * 32, kColO);
    if (!transition) warp_arrive(&s.bar_sb, lane);         // nothing to read out before chunk 0
    for (int n = 0; n < (transition ? 0 : NC); ++n) {
      float ov[64];
      if (norm.gate) {                                     // this chunk's gate rows towards L2 while its products run
        const __nv_bfloat16* gp_ = norm.gate + ((size_t)ib * norm.batch_stride + (size_t)(c_first + n) * BS + (otid >> 4)) * norm.row_stride +
                                   (size_t)ih * D + (otid & 15) * 8;
#pragma unroll
        for (int x = 0; x < 8; ++x) asm volatile("prefetch.global.L2 [%0];" ::"l"(gp_ + (size_t)(8 * x) * norm.row_stride));
      }
      tc::mbar_wait(&s.bar_m2, n & 1, &s.abort_flag, status, kWaitM2);
      tc::tc_fence_after_sync();
      tc::tmem_ld32(t_o, *reinterpret_cast<float(*)[32]>(&ov[0]));
      tc::tmem_ld32(t_o + 32, *reinterpret_cast<float(*)[32]>(&ov[32]));
      tc::tmem_ld_wait();
      tc::tc_fence_before_sync();
      if (n + 1 < NC) warp_arrive(&s.bar_sb, lane);        // the accumulator may be overwritten by the next MMA1
      output_sync();                                       // the previous chunk's rows have left the staging buffer
#pragma unroll
      for (int i = 0; i < 64; ++i) s.ostage[i * D + dv] = __float2bfloat16_rn(ov[i]);
      output_sync();
      if (write_o && !s.abort_flag) {
        // 64 rows x 256 bytes = 1024 16-byte pieces, 8 per thread, 128-bit coalesced stores
        __nv_bfloat16* obase = o + (((size_t)ib * o_bs + (size_t)(c_first + n) * BS) * H + ih) * D;
        if (norm.gate == nullptr) {
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const int piece = otid + x * kOutputThreads;
            const int row = piece >> 4, col = (piece & 15) * 8;
            *reinterpret_cast<uint4*>(obase + (size_t)row * H * D + col) =
                *reinterpret_cast<const uint4*>(&s.ostage[row * D + col]);
          }
        } else {
          const __nv_bfloat16* gbase = norm.gate + ((size_t)ib * norm.batch_stride + (size_t)(c_first + n) * BS) * norm.row_stride +
                                       (size_t)ih * D + (otid & 15) * 8;
          store_rows_normed(s.ostage, obase, gbase, norm.row_stride, norm.weight, norm.eps, otid, H);
        }
      }
    }
  } else {
    // =============================== compute threads ============================================
    const int lq = wid & 3, part = wid >> 2;              // TMEM lane quarter, column share
    const int dv = lq * 32 + lane;                        // this thread's value channel = TMEM lane
    const uint32_t t_lane = tc::tmem_addr(tm, lq * 32, 0);
    const int tokp = part * 32;                           // first of this thread's 32 tokens
    const int dkp = part * 64;                            // first of this thread's 64 key channels

    // The fp32 state: S[i] = S^T[dv][dkp + i]. It never leaves these registers between chunks.
    float S[64];
    int last_big = -1;                                     // transition blocks: see ScanTcSmem::last_big
    {
      float* h0 = (hs && !output_only) ? hs + (((size_t)ib * NC_all + c_first) * H + ih) * D * D : nullptr;
      const float* init = state_source();
#pragma unroll
      for (int i = 0; i < 64; ++i)
        S[i] = init ? init[(size_t)(dkp + i) * D + dv] : (transition && dkp + i == dv) ? 1.f : 0.f;
      if (h0) {
#pragma unroll
        for (int i = 0; i < 64; ++i) h0[(size_t)(dkp + i) * D + dv] = S[i];
      }
      float pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) pk[i] = pack_bf16x2(S[2 * i], S[2 * i + 1]);
      tc::tmem_st32(t_lane + kColSb + dkp / 2, pk);
      tc::tmem_st_wait();
    }
    tc::tc_fence_before_sync();
    warp_arrive(&s.bar_sb, lane);
    for (int n = 0; n < NC; ++n) {
      if (n >= *(volatile int*)&s.nc_limit) break;
      const int b = n & 1;
      const uint32_t ph = n & 1, ph2 = (n >> 1) & 1;
      const bool more = n + 1 < NC;

      if (output_only && more) {
        // the state entering the next chunk comes from memory; its bf16 copy of this chunk is already in tensor
        // memory, so the registers are free and the loads fly while this chunk's products run
        const float* hn = hs + (((size_t)ib * NC_all + (c_first + n + 1)) * H + ih) * D * D;
#pragma unroll
        for (int i = 0; i < 64; ++i) S[i] = __ldg(hn + (size_t)(dkp + i) * D + dv);
      }

      // ---- Un^T / 256 = U^T / 256 - (W S)^T / 256 for this thread's 32 tokens, as the fp16 operand of
      // both the state update and the output product
      uint4 uraw[4];
      if (!transition) {
        tc::mbar_wait(&s.bar_ut[b], ph2, &s.abort_flag, status, kWaitUt);
#pragma unroll
        for (int j = 0; j < 4; ++j) uraw[j] = *reinterpret_cast<const uint4*>(&s.ut[b][((tokp / 8 + j) * D + dv) * 8]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) uraw[j] = make_uint4(0u, 0u, 0u, 0u);
      }
      tc::mbar_wait(&s.bar_m1, ph, &s.abort_flag, status, kWaitM1);
      tc::tc_fence_after_sync();
      {
        float ws[32];
        tc::tmem_ld32(t_lane + kColWs + tokp, ws);
        tc::tmem_ld_wait();
        float p16[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float u[8];
          unpack8_f16(uraw[j], u);
#pragma unroll
          for (int i = 0; i < 8; ++i) ws[j * 8 + i] = fmaf(ws[j * 8 + i], -1.f / kValScale, u[i]);   // Un / 256
#pragma unroll
          for (int i = 0; i < 4; ++i) p16[j * 4 + i] = pack_f16x2(ws[j * 8 + 2 * i], ws[j * 8 + 2 * i + 1]);
        }
        tc::tmem_st16(t_lane + kColUn16 + tokp / 2, p16);
        tc::tmem_st_wait();
        tc::tc_fence_before_sync();
        warp_arrive(&s.bar_un, lane);
      }

      if (output_only) {
        // MMA1 of this chunk has completed (waited above): its S^T operand may be replaced
        if (more) {
          float pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = pack_bf16x2(S[2 * i], S[2 * i + 1]);
          tc::tmem_st32(t_lane + kColSb + dkp / 2, pk);
          tc::tmem_st_wait();
          tc::tc_fence_before_sync();
          warp_arrive(&s.bar_sb, lane);
        }
        if (s.abort_flag) break;
        continue;
      }

      // ---- new state S <- gamma_C * S + P, its bf16 operand copy for the next chunk, optional snapshot
      tc::mbar_wait(&s.bar_kgt[b], ph2, &s.abort_flag, status, kWaitKgt);   // gamma arrived with KG^T
      tc::mbar_wait(&s.bar_m3, ph, &s.abort_flag, status, kWaitM3);
      tc::tc_fence_after_sync();
      {
        const float* gln = s.gl[n & 3];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          float pr[32];
          tc::tmem_ld32(t_lane + dkp + 32 * hf, pr);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 g4 = *reinterpret_cast<const float4*>(&gln[dkp + 32 * hf + 4 * i]);
            S[32 * hf + 4 * i] = fmaf(g4.x, S[32 * hf + 4 * i], pr[4 * i]);
            S[32 * hf + 4 * i + 1] = fmaf(g4.y, S[32 * hf + 4 * i + 1], pr[4 * i + 1]);
            S[32 * hf + 4 * i + 2] = fmaf(g4.z, S[32 * hf + 4 * i + 2], pr[4 * i + 2]);
            S[32 * hf + 4 * i + 3] = fmaf(g4.w, S[32 * hf + 4 * i + 3], pr[4 * i + 3]);
          }
          if (more) {
            float pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(S[32 * hf + 2 * i], S[32 * hf + 2 * i + 1]);
            tc::tmem_st16(t_lane + kColSb + (dkp + 32 * hf) / 2, pk);
          }
        }
        if (more) {
          tc::tmem_st_wait();
          tc::tc_fence_before_sync();
          warp_arrive(&s.bar_sb, lane);
        }
        float* hn = (hs && more) ? hs + (((size_t)ib * NC_all + (c_first + n + 1)) * H + ih) * D * D : nullptr;
        if (hn) {
#pragma unroll
          for (int i = 0; i < 64; ++i) hn[(size_t)(dkp + i) * D + dv] = S[i];
        }
        if (!more) {
          float* fin = state_sink();
          if (fin) {
#pragma unroll
            for (int i = 0; i < 64; ++i) fin[(size_t)(dkp + i) * D + dv] = S[i];
          }
        }
        if (transition) {
          // Has the running transition matrix vanished? All 256 compute threads agree through one barrier with
          // an AND reduction. If it has, chunks n + 1 and n + 2 are still walked (other warps of the block are
          // already working on them) and every role stops before chunk n + 3: they all pass a hand-off of chunk
          // n + 2 that is ordered after this store before they look at the limit again.
          float m = 0.f;
#pragma unroll
          for (int i = 0; i < 64; ++i) m = fmaxf(m, fabsf(S[i]));
          if (!compute_all(m < kVanish)) last_big = n;
          else if (tid == 0 && n + 3 < s.nc_limit) s.nc_limit = n + 3;
        }
      }
      if (s.abort_flag) break;                             // per thread: no block-level barrier in this loop
    }
    if (lane == 0) s.last_big[wid] = last_big;
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (wid == 0) tc::tmem_dealloc(tm, 512);
  if (transition && tid == 0) {
    // Chunks the correction pass must redo: through the last chunk whose ENTERING state still carried a
    // visible share of the segment's entering state, i.e. one past the last chunk after which the transition
    // matrix was still visible; chunk 0 always (it starts from the true state).
    int last = -1;
    for (int i = 0; i < kComputeThreads / 32; ++i) last = s.last_big[i] > last ? s.last_big[i] : last;
    const int redo = last + 2;                               // < NC whenever the block stopped early: then no matrix was stored
    P.seg_stop[bh * plan.nseg + seg] = redo < NC ? redo : NC;
  }
}

// Decay check before a guarded launch (more blocks than SMs, see ScanPlan): one warp per (batch, head, segment
// j >= 1) multiplies gamma_last of the segment's first kCheckChunks chunks per channel. If the slowest channel
// has not decayed below kVanish by then, the carried state will not vanish quickly either, the transition
// blocks would walk most of their segments, and the launch is better off not cutting: the mode word is set.
// A heuristic for speed only: whatever it says, the results are those of the recurrence.
constexpr int kCheckChunks = 12;
__global__ void __launch_bounds__(256)
scan_mode_kernel(WsPtrs P, int BK, int nseg, int NC_all) {
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= BK * (nseg - 1)) return;
  const int bh = item / (nseg - 1), seg = 1 + item % (nseg - 1);   // (batch, KEY head): gamma is a key-side record
  const int c0 = (int)((int64_t)NC_all * seg / nseg), c1 = (int)((int64_t)NC_all * (seg + 1) / nseg);
  const int n = c1 - c0 < kCheckChunks ? c1 - c0 : kCheckChunks;
  float4 prod = make_float4(1.f, 1.f, 1.f, 1.f);
  for (int c = 0; c < n; ++c) {
    const float4 gv = *reinterpret_cast<const float4*>(P.gl + ((size_t)bh * NC_all + c0 + c) * D + 4 * lane);
    prod.x *= gv.x; prod.y *= gv.y; prod.z *= gv.z; prod.w *= gv.w;
  }
  float m = fmaxf(fmaxf(prod.x, prod.y), fmaxf(prod.z, prod.w));
  m = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
  if (lane == 0 && (m >= kVanish || n < kCheckChunks)) atomicOr(P.seg_mode, 1);
}

// Pass 2 of the cut scan: chains the segments' affine maps in fp32. Block (bh, column slice of 16 value
// channels): S = C_0 (segment 0 ran from the true initial state); for j = 1 .. nseg-1: the state entering
// segment j is S; S <- T_j S + C_j (T_j skipped where the transition block saw it vanish). The value
// columns evolve independently, so the slices need no exchange.
constexpr int kCombineCols = 16;
constexpr int kTPad = D + 1;
__global__ void __launch_bounds__(256)
scan_combine_kernel(WsPtrs P, int nseg, int NC_all, int guarded, float* __restrict__ sT) {
  extern __shared__ __align__(16) float csm[];
  if (guarded && *P.seg_mode != 0) return;                 // the first pass walked the whole sequences itself
  float* Ts = csm;                         // [128][129] transition matrix of the current segment
  float* Ss = csm + D * kTPad;             // [128][16] current state slice
  const int bh = blockIdx.x, col0 = blockIdx.y * kCombineCols;
  const int tid = threadIdx.x, r = tid & (D - 1), cg = tid >> 7;      // row, 8-column group
  const size_t rec0 = (size_t)bh * nseg * D * D;
  float acc[8];
  {
    const float* c0p = P.seg_c + rec0 + (size_t)r * D + col0 + 8 * cg;
    const float4 a = *reinterpret_cast<const float4*>(c0p), b = *reinterpret_cast<const float4*>(c0p + 4);
    acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w; acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
  }
  for (int j = 1; j < nseg; ++j) {
    const size_t rec = rec0 + (size_t)j * D * D;
    float* inp = P.seg_in + rec + (size_t)r * D + col0 + 8 * cg;
    *reinterpret_cast<float4*>(inp) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(inp + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    const int len = (int)((int64_t)NC_all * (j + 1) / nseg) - (int)((int64_t)NC_all * j / nseg);
    const bool vanished = P.seg_stop[bh * nseg + j] < len;             // uniform over the block
    const float* cp = P.seg_c + rec + (size_t)r * D + col0 + 8 * cg;
    const float4 ca = *reinterpret_cast<const float4*>(cp), cb = *reinterpret_cast<const float4*>(cp + 4);
    if (vanished) {
      acc[0] = ca.x; acc[1] = ca.y; acc[2] = ca.z; acc[3] = ca.w; acc[4] = cb.x; acc[5] = cb.y; acc[6] = cb.z; acc[7] = cb.w;
      continue;
    }
    __syncthreads();                       // the previous segment's Ts / Ss have been read
#pragma unroll
    for (int i = 0; i < 8; ++i) Ss[r * kCombineCols + 8 * cg + i] = acc[i];
    const float* tp = P.seg_t + rec;
    for (int idx = tid; idx < D * D / 4; idx += 256) {                 // coalesced 128-bit reads, padded rows
      const float4 t4 = *reinterpret_cast<const float4*>(tp + (size_t)idx * 4);
      float* d = Ts + (idx >> 5) * kTPad + (idx & 31) * 4;
      d[0] = t4.x; d[1] = t4.y; d[2] = t4.z; d[3] = t4.w;
    }
    __syncthreads();
    acc[0] = ca.x; acc[1] = ca.y; acc[2] = ca.z; acc[3] = ca.w; acc[4] = cb.x; acc[5] = cb.y; acc[6] = cb.z; acc[7] = cb.w;
#pragma unroll 4
    for (int kk = 0; kk < D; ++kk) {
      const float t = Ts[r * kTPad + kk];
      const float4 sa = *reinterpret_cast<const float4*>(&Ss[kk * kCombineCols + 8 * cg]);
      const float4 sb = *reinterpret_cast<const float4*>(&Ss[kk * kCombineCols + 8 * cg + 4]);
      acc[0] = fmaf(t, sa.x, acc[0]); acc[1] = fmaf(t, sa.y, acc[1]); acc[2] = fmaf(t, sa.z, acc[2]); acc[3] = fmaf(t, sa.w, acc[3]);
      acc[4] = fmaf(t, sb.x, acc[4]); acc[5] = fmaf(t, sb.y, acc[5]); acc[6] = fmaf(t, sb.z, acc[6]); acc[7] = fmaf(t, sb.w, acc[7]);
    }
  }
  if (sT) {
    float* fp = sT + ((size_t)bh * D + r) * D + col0 + 8 * cg;
    *reinterpret_cast<float4*>(fp) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(fp + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

}  // namespace

// part: 0 = the whole scan; 1 = everything up to the final state (for a cut scan: decay check, first pass, chaining
// of the segments; otherwise the whole scan); 2 = what is left (the correction pass of a cut scan, else nothing).
int launch_scan_tc(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                   int B, int S, int H, int64_t o_bs, const gdn2_gated_norm* gn, int part, cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  const size_t smem = sizeof(ScanTcSmem) + 128;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(scan_tc_kernel), smem));
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(o);
  uint32_t* status = device_status_word();
  const int BH = B * H, NC = S / BS;
  ScanNorm norm{nullptr, nullptr, 0, 0, 0.f};
  if (gn) norm = ScanNorm{static_cast<const __nv_bfloat16*>(gn->gate), static_cast<const __nv_bfloat16*>(gn->weight),
                          gn->gate_row_stride, gn->gate_batch_stride, gn->eps};
  // chunk states are a by-product of the one-block-per-head walk only
  const int nseg = hs ? 1 : L.nseg;
  if (nseg <= 1) {
    if (part == 2) return GDN2_OK;
    scan_tc_kernel<<<BH, kThreads, smem, st>>>(L, P, ScanPlan{kWhole, 1, 0}, norm, s0, ob, sT, hs, S, H, o_bs, status);
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  }
  const int guarded = L.nseg_guarded ? 1 : 0;
  if (part == 2) {
    scan_tc_kernel<<<BH * (nseg - 1), kThreads, smem, st>>>(L, P, ScanPlan{kRedo, nseg, guarded}, norm, nullptr, ob, nullptr, nullptr,
                                                           S, H, o_bs, status);
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  }
  if (guarded) {
    GDN2_CUDA_TRY(cudaMemsetAsync(P.seg_mode, 0, sizeof(int), st));
    const int BK = BH / L.rep;
    scan_mode_kernel<<<(BK * (nseg - 1) + 7) / 8, 256, 0, st>>>(P, BK, nseg, NC);
    GDN2_CUDA_TRY(cudaGetLastError());
  }
  scan_tc_kernel<<<BH * (2 * nseg - 1), kThreads, smem, st>>>(L, P, ScanPlan{kFirst, nseg, guarded}, norm, s0, ob, sT, nullptr,
                                                             S, H, o_bs, status);
  GDN2_CUDA_TRY(cudaGetLastError());
  const size_t csmem = (size_t)(D * kTPad + D * kCombineCols) * sizeof(float);
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(scan_combine_kernel), csmem));
  scan_combine_kernel<<<dim3(BH, D / kCombineCols), 256, csmem, st>>>(P, nseg, NC, guarded, sT);
  GDN2_CUDA_TRY(cudaGetLastError());
  if (part == 1) return GDN2_OK;
  scan_tc_kernel<<<BH * (nseg - 1), kThreads, smem, st>>>(L, P, ScanPlan{kRedo, nseg, guarded}, norm, nullptr, ob, nullptr, nullptr,
                                                         S, H, o_bs, status);
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

// Chunk-parallel output from stored chunk states on the tensor-core family: the scan kernel's chunk body without
// the state update, every block walking a run of chunks of one (batch, head) with the records prefetched a chunk ahead.
int launch_output_tc(const WsLayout& L, const WsPtrs& P, const float* hs, void* o, int B, int S, int H, int64_t o_bs,
                     cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  const size_t smem = sizeof(ScanTcSmem) + 128;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(scan_tc_kernel), smem));
  const int BH = B * H, NC = S / BS;
  // enough runs to give every SM a few blocks, none shorter than 4 chunks
  int runs = (4 * device_sm_count() + BH - 1) / BH;
  if (runs > NC / 4) runs = NC / 4;
  if (runs < 1) runs = 1;
  scan_tc_kernel<<<BH * runs, kThreads, smem, st>>>(L, P, ScanPlan{kOutput, runs, 0}, ScanNorm{nullptr, nullptr, 0, 0, 0.f}, nullptr,
                                                   static_cast<__nv_bfloat16*>(o),
                                                   nullptr, const_cast<float*>(hs), S, H, o_bs, device_status_word());
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace gdn2
