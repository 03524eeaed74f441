// Sequential state scan fused with the output, tensor-core (tcgen05 / TMEM / TMA) family, for
// DK = DV = 128, bf16 outputs, fp32 state. One block per (batch, head), sequential over chunks; the
// state never leaves the SM between chunks.
//
// The algebra of the reference's prefill_scan_kernel (gdn2/inference.py:446-475 of the reference
// project) is evaluated TRANSPOSED so that every product has the 128 value channels as the MMA M
// dimension (= TMEM lane = thread), tokens or key channels as N:
//
//   MMA1w  WS[dv, tok]  = S^T[dv,dk] * W[tok,dk]^T            (W S)^T          bf16
//   MMA1q  O [dv, tok]  = S^T[dv,dk] * Qg[tok,dk]^T           (Qg S)^T         bf16
//   regs   Un^T[dv,tok] = U^T - WS
//   MMA3   P [dv,dk]    = Un^T[dv,tok] * KG^T[dk,tok]^T       (KG^T Un)^T      fp16 (scaled, see common.cuh)
//   MMA2   O [dv, r]   += Un^T[dv,s] * Aqk[r,s]^T             (tril(Aqk) Un)^T fp16 (same scaled Un^T image)
//   regs   S^T         <- gamma_C[dk] * S^T + P   (the fp32 state lives in registers, 64 values per thread)
//
// Only MMA1w, the Un pass, MMA3 and the state pass are on the recurrence's critical path; the
// kernel is organised around that:
//   * warp 8 (one thread) issues every MMA, MMA3 before MMA2 so the state update never queues behind
//     the output product; warp 9 (one thread) issues every bulk copy.
//   * warps 10-13 read each finished O accumulator into registers, release it, and write the rows
//     out through a shared staging tile with 128-bit coalesced stores, off the critical path.
//   * warps 0-7 (256 threads; two warps share each 32-lane quarter of TMEM and split its columns)
//     do the register passes. The output pass of chunk n (TMEM -> bf16 -> shared staging ->
//     128-bit coalesced global stores) runs after the state hand-off, while MMA1w of chunk n+1
//     executes; the O accumulator is double buffered in TMEM for that.
//   * operands arrive as whole workspace records with one bulk copy each; WQ, KG^T and U^T are
//     double buffered so that a copy is always issued a full chunk ahead of its use.
//   * hand-offs are mbarriers (arrive / wait), every wait is bounded (tc_utils.cuh).
//
//   * the A operands (S^T in bf16, Un^T in fp16) never touch shared memory: the register
//     passes store them as packed 16-bit pairs into tensor memory and the MMAs read them from there,
//     which halves the shared-memory traffic the tensor core competes for.
//
// TMEM columns: [0,128) the update product P; [128,192) WS; [192,256) and [256,320) the two O accumulators;
// [320,384) S^T bf16 pairs; [384,416) Un^T/256 fp16 pairs.
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
};

#ifdef GDN2_SCAN_TIMING
__device__ unsigned long long g_scan_timing[32];
#define TICK(i) do { if (blockIdx.x == 0) { long long now_ = clock64(); tacc[i] += now_ - tprev; tprev = now_; } } while (0)
#define TDECL long long tacc[16] = {0}; long long tprev = clock64()
#define TFLUSH(off) do { if (blockIdx.x == 0) for (int i_ = 0; i_ < 16; ++i_) g_scan_timing[off + i_] = tacc[i_]; } while (0)
#else
#define TICK(i) do {} while (0)
#define TDECL do {} while (0)
#define TFLUSH(off) do {} while (0)
#endif

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

__global__ void __launch_bounds__(kThreads, 1)
scan_tc_kernel(WsLayout L, WsPtrs P, const float* __restrict__ s0, __nv_bfloat16* __restrict__ o,
               float* __restrict__ sT, float* __restrict__ hs, int S, int H, int64_t o_bs, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  ScanTcSmem& s = *reinterpret_cast<ScanTcSmem*>(smem_raw);
  const int NC = S / BS;
  const int bh = blockIdx.x, ib = bh / H, ih = bh % H;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int64_t ch0 = (int64_t)bh * NC;

  const char* g_wq = P.wq + (size_t)ch0 * kWqBytes;
  const char* g_aqk = P.aqk + (size_t)ch0 * kAqkBytes;
  const char* g_kgt = P.kgt + (size_t)ch0 * kKgtBytes;
  const char* g_ut = P.ut + (size_t)ch0 * kUtBytes;
  const float* g_gl = P.gl + (size_t)ch0 * D;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s.bar_wq[i], 1); tc::mbar_init(&s.bar_kgt[i], 1); tc::mbar_init(&s.bar_ut[i], 1);
    }
    tc::mbar_init(&s.bar_aqk, 1); tc::mbar_init(&s.bar_m1, 1); tc::mbar_init(&s.bar_m3, 1); tc::mbar_init(&s.bar_m2, 1);
    tc::mbar_init(&s.bar_sb, (kComputeThreads + kOutputThreads) / 32); tc::mbar_init(&s.bar_un, kComputeThreads / 32);   // one arrival per warp
    s.abort_flag = 0;
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
        tc::mbar_expect_tx(&s.bar_kgt[n & 1], kKgtBytes + D * 4);
        tc::bulk_g2s(s.kgt[n & 1], g_kgt + (size_t)n * kKgtBytes, kKgtBytes, &s.bar_kgt[n & 1]);
        tc::bulk_g2s(s.gl[n & 3], g_gl + (size_t)n * D, D * 4, &s.bar_kgt[n & 1]);
      };
      auto load_ut = [&](int n) {
        tc::mbar_expect_tx(&s.bar_ut[n & 1], kUtBytes);
        tc::bulk_g2s(s.ut[n & 1], g_ut + (size_t)n * kUtBytes, kUtBytes, &s.bar_ut[n & 1]);
      };
      auto load_aqk = [&](int n) {
        tc::mbar_expect_tx(&s.bar_aqk, kAqkBytes);
        tc::bulk_g2s(s.aqk, g_aqk + (size_t)n * kAqkBytes, kAqkBytes, &s.bar_aqk);
      };
      load_wq(0); load_ut(0); load_kgt(0); load_aqk(0);
      if (NC > 1) { load_wq(1); load_ut(1); load_kgt(1); }
      for (int n = 0; n < NC; ++n) {
        const uint32_t ph = n & 1;
        // the Un pass of chunk n has consumed its U^T buffer
        bool ok = tc::mbar_wait(&s.bar_un, ph, &s.abort_flag, status, kWaitUn);
        if (ok && n + 2 < NC) load_ut(n + 2);
        // every product of chunk n has completed: refill the operand buffers it read
        ok = ok && tc::mbar_wait(&s.bar_m2, ph, &s.abort_flag, status, kWaitM2);
        if (ok) {
          if (n + 1 < NC) load_aqk(n + 1);
          if (n + 2 < NC) { load_wq(n + 2); load_kgt(n + 2); }
        }
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
      TDECL;
      for (int n = 0; n < NC; ++n) {
        const int b = n & 1;
        const uint32_t ph = n & 1, ph2 = (n >> 1) & 1;
        TICK(0);
        // S^T (bf16) of chunk n is in place and the O accumulator has been read out
        bool ok = wait_all(&s.bar_wq[b], ph2, kWaitWq);
        TICK(1);
        ok = ok && wait_all(&s.bar_sb, ph, kWaitSb);
        TICK(2);
        if (ok) {
          tc::tc_fence_after_sync();
          // one N = 128 product: columns [128,192) = (W S)^T, [192,256) = (Qg S)^T
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, kColWs), a_sb, tc::smem_u32(s.wq[b]), 2 * BS, D, idesc_n128, false);
          tc::mma_commit_warp(&s.bar_m1);
        }
        TICK(3);
#ifdef GDN2_SCAN_TIMING
        wait_all(&s.bar_m1, ph, kWaitM1);
        TICK(9);
#endif
        ok = wait_all(&s.bar_kgt[b], ph2, kWaitKgt);
        TICK(4);
        ok = ok && wait_all(&s.bar_un, ph, kWaitUn);
        TICK(5);
        if (ok) {
          tc::tc_fence_after_sync();
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, 0), a_un16, tc::smem_u32(s.kgt[b]), D, BS, idesc_f16, false);
          tc::mma_commit_warp(&s.bar_m3);
        }
        TICK(6);
        ok = ok && wait_all(&s.bar_aqk, ph, kWaitAqk);
        TICK(7);
        if (ok) {
          tc::mma_f16_ts_ktile_warp(tc::tmem_addr(tm, 0, kColO), a_un16, a_aqk, BS, BS, idesc_f16_n64, true);
          tc::mma_commit_warp(&s.bar_m2);
        }
        TICK(8);
      }
      if (lane == 0) TFLUSH(0);
    }
  } else if (wid >= 10) {
    // =============================== output warps: O^T -> bf16 rows in global memory =============
    const int lq = wid & 3;
    const int dv = lq * 32 + lane;
    const int otid = tid - (kComputeThreads + 64);
    const uint32_t t_o = tc::tmem_addr(tm, lq * 32, kColO);
    warp_arrive(&s.bar_sb, lane);                          // nothing to read out before chunk 0
    for (int n = 0; n < NC; ++n) {
      float ov[64];
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
      if (!s.abort_flag) {
        // 64 rows x 256 bytes = 1024 16-byte pieces, 8 per thread, 128-bit coalesced stores
        __nv_bfloat16* obase = o + (((size_t)ib * o_bs + (size_t)n * BS) * H + ih) * D;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const int piece = otid + x * kOutputThreads;
          const int row = piece >> 4, col = (piece & 15) * 8;
          *reinterpret_cast<uint4*>(obase + (size_t)row * H * D + col) =
              *reinterpret_cast<const uint4*>(&s.ostage[row * D + col]);
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
    {
      float* h0 = hs ? hs + (((size_t)ib * NC + 0) * H + ih) * D * D : nullptr;
#pragma unroll
      for (int i = 0; i < 64; ++i) S[i] = s0 ? s0[((size_t)bh * D + dkp + i) * D + dv] : 0.f;
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

    TDECL;
    for (int n = 0; n < NC; ++n) {
      TICK(0);
      const int b = n & 1;
      const uint32_t ph = n & 1, ph2 = (n >> 1) & 1;
      const bool more = n + 1 < NC;

      // ---- Un^T / 256 = U^T / 256 - (W S)^T / 256 for this thread's 32 tokens, as the fp16 operand of
      // both the state update and the output product
      tc::mbar_wait(&s.bar_ut[b], ph2, &s.abort_flag, status, kWaitUt);
      TICK(2);
      uint4 uraw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) uraw[j] = *reinterpret_cast<const uint4*>(&s.ut[b][((tokp / 8 + j) * D + dv) * 8]);
      tc::mbar_wait(&s.bar_m1, ph, &s.abort_flag, status, kWaitM1);
      tc::tc_fence_after_sync();
      TICK(3);
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
        TICK(4);
      }

      // ---- new state S <- gamma_C * S + P, its bf16 operand copy for the next chunk, optional snapshot
      tc::mbar_wait(&s.bar_kgt[b], ph2, &s.abort_flag, status, kWaitKgt);   // gamma arrived with KG^T
      TICK(5);
      tc::mbar_wait(&s.bar_m3, ph, &s.abort_flag, status, kWaitM3);
      tc::tc_fence_after_sync();
      TICK(7);
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
        TICK(8);
        float* hn = (hs && more) ? hs + (((size_t)ib * NC + (n + 1)) * H + ih) * D * D : nullptr;
        float* fin = (!more && sT) ? sT + (size_t)bh * D * D : nullptr;
        if (hn) {
#pragma unroll
          for (int i = 0; i < 64; ++i) hn[(size_t)(dkp + i) * D + dv] = S[i];
        }
        if (fin) {
#pragma unroll
          for (int i = 0; i < 64; ++i) fin[(size_t)(dkp + i) * D + dv] = S[i];
        }
      }
      TICK(9);
      if (s.abort_flag) break;                             // per thread: no block-level barrier in this loop
    }
    if (tid == 0) TFLUSH(16);
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (wid == 0) tc::tmem_dealloc(tm, 512);
}

}  // namespace

int launch_scan_tc(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                   int B, int S, int H, int64_t o_bs, cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  const size_t smem = sizeof(ScanTcSmem) + 128;
  GDN2_CUDA_TRY(cudaFuncSetAttribute(scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  scan_tc_kernel<<<B * H, kThreads, smem, st>>>(L, P, s0, static_cast<__nv_bfloat16*>(o), sT, hs, S, H, o_bs,
                                                device_status_word());
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

#ifdef GDN2_SCAN_TIMING
extern "C" int gdn2_debug_scan_timing(unsigned long long* out32) {
  return cudaMemcpyFromSymbol(out32, g_scan_timing, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -6;
}
#endif

}  // namespace gdn2
