// Sequential state scan fused with the output, tensor-core (tcgen05 / TMEM / TMA) family, for
// DK = DV = 128, bf16 outputs, fp32 state. One 128-thread block per (batch, head), sequential
// over chunks; the state never leaves the SM between chunks.
//
// The algebra of the reference's prefill_scan_kernel (gdn2/inference.py:446-475 of the reference
// project) is evaluated TRANSPOSED so that every product has the 128 value channels as the MMA M
// dimension (= TMEM lane = thread), tokens or key channels as N:
//
//   MMA1  D1[dv, 0:64]   = S^T[dv,dk] * W[tok,dk]^T          (W S)^T        bf16 operands
//         D1[dv, 64:128] = S^T[dv,dk] * Qg[tok,dk]^T         (Qg S)^T       (one N = 128 product)
//   regs  Un^T[dv,tok]   = U^T - D1[:, 0:64]
//   MMA2  D1[dv, 64:128] += Un^T[dv,s] * Aqk[r,s]^T          (tril(Aqk) Un)^T   bf16 operands
//   MMA3  ST[dv,dk]      += Un^T[dv,tok] * KG^T[dk,tok]^T    (KG^T Un)^T    tf32 operands
//   regs  ST             <- gamma_C(next chunk)[dk] * ST after the bf16 copy of S^T is taken
//
// The value path (U, Un, KG) stays in fp32 storage / tf32 operands because rounding any of them to
// bf16 alone costs about 1.7e-3 relative error in the final state; the erase path (W, S as an
// operand, Aqk, Qg) is bf16. TMEM: columns [0,128) hold the fp32 state S^T, [128,256) hold D1.
//
// Operands arrive as whole records of the workspace (see common.cuh) with one bulk copy each into
// a single shared-memory buffer per operand; a buffer is refilled for the next chunk as soon as
// the MMA that reads it has completed, so the copies overlap the rest of the chunk's chain.
#include <cstdlib>

#include "common.cuh"
#include "tc_utils.cuh"

namespace gdn2 {

namespace {

constexpr int D = 128;
constexpr int BS = kChunk;
#ifndef GDN2_SCAN_NSPLIT
#define GDN2_SCAN_NSPLIT 2      // warps per TMEM lane quarter: 128 * NSPLIT threads per block
#endif

constexpr uint32_t kWqBytes = 2 * BS * D * 2;    // 32 KiB
constexpr uint32_t kAqkBytes = BS * BS * 2;      //  8 KiB
constexpr uint32_t kKgtBytes = D * BS * 4;       // 32 KiB
constexpr uint32_t kUtBytes = D * BS * 4;        // 32 KiB

struct ScanTcSmem {
  __nv_bfloat16 wq[2 * BS * D];      // B of MMA1: [dk/8][128 rows: W tok 0..63, Qg tok 0..63][8]
  __nv_bfloat16 aqk[BS * BS];        // B of MMA2: [s/8][64 r][8]
  float kgt[D * BS];                 // B of MMA3: [tok/4][128 dk][4]
  float un32[D * BS];                // U^T on arrival, Un^T in place: A of MMA3: [tok/4][128 dv][4]
  __nv_bfloat16 sb[D * D];           // A of MMA1: S^T in bf16: [dk/8][128 dv][8]
  __nv_bfloat16 unb[D * BS];         // A of MMA2: Un^T in bf16: [tok/8][128 dv][8]
  float gl[2][D];                    // gamma at the last token of chunk n (slot n & 1)
  uint64_t bar_wq, bar_aqk, bar_kgt, bar_ut, bar_m1, bar_m2, bar_m3;
  uint32_t tmem_base;
  int abort_flag;
};

#ifdef GDN2_SCAN_TIMING
__device__ unsigned long long g_scan_timing[16];
#define TICK(i) do { if (tid == 0 && blockIdx.x == 0) { long long now_ = clock64(); tacc[i] += now_ - tprev; tprev = now_; } } while (0)
#else
#define TICK(i) do {} while (0)
#endif

enum : uint32_t {
  kWaitWq = 0x10, kWaitUt = 0x20, kWaitAqk = 0x40, kWaitKgt = 0x80, kWaitM1 = 0x100, kWaitM2 = 0x200,
  kWaitM3 = 0x400
};

// NSPLIT warps share each 32-lane quarter of TMEM and split its columns (tokens / key channels)
// between them, so the per-chunk register work is spread over 128 * NSPLIT threads.
template <int NSPLIT>
__global__ void __launch_bounds__(128 * NSPLIT, 1)
scan_tc_kernel(WsLayout L, WsPtrs P, const float* __restrict__ s0, __nv_bfloat16* __restrict__ o,
               float* __restrict__ sT, float* __restrict__ hs, int S, int H, int64_t o_bs, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  ScanTcSmem& s = *reinterpret_cast<ScanTcSmem*>(smem_raw);
  constexpr int TOK = BS / NSPLIT;                      // tokens per thread in the Un / output passes
  constexpr int KCH = D / NSPLIT;                       // key channels per thread in the state pass
  const int NC = S / BS;
  const int bh = blockIdx.x, ib = bh / H, ih = bh % H;
  const int tid = threadIdx.x, wid = tid >> 5;
  const int lq = wid & 3, part = wid >> 2;              // TMEM lane quarter, column share
  const int dv = lq * 32 + (tid & 31);                  // this thread's value channel = TMEM lane
  const int64_t ch0 = (int64_t)bh * NC;

  const char* g_wq = P.wq + (size_t)ch0 * kWqBytes;
  const char* g_aqk = P.aqk + (size_t)ch0 * kAqkBytes;
  const char* g_kgt = reinterpret_cast<const char*>(P.kgt) + (size_t)ch0 * kKgtBytes;
  const char* g_ut = reinterpret_cast<const char*>(P.ut) + (size_t)ch0 * kUtBytes;
  const float* g_gl = P.gl + (size_t)ch0 * D;

  if (tid == 0) {
    tc::mbar_init(&s.bar_wq, 1); tc::mbar_init(&s.bar_aqk, 1); tc::mbar_init(&s.bar_kgt, 1);
    tc::mbar_init(&s.bar_ut, 1); tc::mbar_init(&s.bar_m1, 1); tc::mbar_init(&s.bar_m2, 1);
    tc::mbar_init(&s.bar_m3, 1);
    s.abort_flag = 0;
    tc::mbar_init_fence();
  }
  if (wid == 0) tc::tmem_alloc(&s.tmem_base, 256);
  if (tid < D) s.gl[0][tid] = g_gl[tid];
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = s.tmem_base;
  const uint32_t t_state = tc::tmem_addr(tm, lq * 32, part * KCH);          // this thread's share of the state row
  const uint32_t t_ws = tc::tmem_addr(tm, lq * 32, 128 + part * TOK);       // (W S)^T columns of its tokens
  const uint32_t t_o = tc::tmem_addr(tm, lq * 32, 192 + part * TOK);        // O^T columns of its tokens

  if (tid == 0) {   // operands of chunk 0
    tc::mbar_expect_tx(&s.bar_wq, kWqBytes);   tc::bulk_g2s(s.wq, g_wq, kWqBytes, &s.bar_wq);
    tc::mbar_expect_tx(&s.bar_ut, kUtBytes);   tc::bulk_g2s(s.un32, g_ut, kUtBytes, &s.bar_ut);
    tc::mbar_expect_tx(&s.bar_aqk, kAqkBytes); tc::bulk_g2s(s.aqk, g_aqk, kAqkBytes, &s.bar_aqk);
    tc::mbar_expect_tx(&s.bar_kgt, kKgtBytes); tc::bulk_g2s(s.kgt, g_kgt, kKgtBytes, &s.bar_kgt);
  }

  // initial state: this thread's share of its S^T row -> bf16 image, chunk_states[0], gamma_0-scaled TMEM copy
  {
    float* h0 = hs ? hs + (((size_t)ib * NC + 0) * H + ih) * D * D : nullptr;
    float x[16];
#pragma unroll 1
    for (int c0 = part * KCH; c0 < (part + 1) * KCH; c0 += 16) {
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = s0 ? s0[((size_t)bh * D + c0 + i) * D + dv] : 0.f;
      if (h0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) h0[(size_t)(c0 + i) * D + dv] = x[i];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint4*>(&s.sb[((c0 / 8 + j) * D + dv) * 8]) = tc::pack8_bf16(&x[j * 8]);
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] *= s.gl[0][c0 + i];
      tc::tmem_st16(tc::tmem_addr(tm, lq * 32, c0), x);
    }
    tc::tmem_st_wait();
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  constexpr uint32_t idesc_m1 = tc::instr_desc(1, 128, 128);
  constexpr uint32_t idesc_m2 = tc::instr_desc(1, 128, 64);
  constexpr uint32_t idesc_m3 = tc::instr_desc(2, 128, 128);

#ifdef GDN2_SCAN_TIMING
  long long tacc[16] = {0}; long long tprev = clock64();
#endif
  for (int n = 0; n < NC; ++n) {
    if (s.abort_flag) break;
    const uint32_t ph = n & 1;
    TICK(0);
    const bool more = n + 1 < NC;
    float gl_next = (more && tid < D) ? g_gl[(size_t)(n + 1) * D + tid] : 1.f;   // early, independent global load

    // ---- MMA1: D1 = S^T * [W ; Qg]^T
    if (tid == 0) {
      if (tc::mbar_wait(&s.bar_wq, ph, &s.abort_flag, status, kWaitWq)) {
        tc::tc_fence_after_sync();
        tc::mma_bf16_ktile(tc::tmem_addr(tm, 0, 128), tc::smem_u32(s.sb), D, tc::smem_u32(s.wq), 2 * BS, D,
                           idesc_m1, false);
        tc::mma_commit(&s.bar_m1);
      }
    }
    TICK(1);
    tc::mbar_wait(&s.bar_m1, ph, &s.abort_flag, status, kWaitM1);
    tc::tc_fence_after_sync();
    TICK(2);
    if (tid == 0 && more && !s.abort_flag) {
      tc::mbar_expect_tx(&s.bar_wq, kWqBytes);
      tc::bulk_g2s(s.wq, g_wq + (size_t)(n + 1) * kWqBytes, kWqBytes, &s.bar_wq);
    }

    // ---- Un^T = U^T - (W S)^T, written as tf32 (in place) and bf16 operand images
    tc::mbar_wait(&s.bar_ut, ph, &s.abort_flag, status, kWaitUt);
    TICK(3);
#pragma unroll
    for (int t0 = 0; t0 < TOK; t0 += 16) {
      float ws[16];
      tc::tmem_ld16(t_ws + t0, ws);
      tc::tmem_ld_wait();
      const int tok0 = part * TOK + t0;                   // first of 16 tokens
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4* pu = reinterpret_cast<float4*>(&s.un32[((tok0 / 4 + j) * D + dv) * 4]);
        float4 u = *pu;
        u.x -= ws[j * 4 + 0]; u.y -= ws[j * 4 + 1]; u.z -= ws[j * 4 + 2]; u.w -= ws[j * 4 + 3];
        *pu = make_float4(tf32_rn(u.x), tf32_rn(u.y), tf32_rn(u.z), tf32_rn(u.w));
        ws[j * 4 + 0] = u.x; ws[j * 4 + 1] = u.y; ws[j * 4 + 2] = u.z; ws[j * 4 + 3] = u.w;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint4*>(&s.unb[((tok0 / 8 + j) * D + dv) * 8]) = tc::pack8_bf16(&ws[j * 8]);
    }
    if (tid < D) s.gl[(n + 1) & 1][tid] = gl_next;
    TICK(4);
    tc::fence_async_smem();
    tc::tc_fence_before_sync();
    __syncthreads();
    TICK(5);

    // ---- MMA2: D1[:, 64:128] += Un^T * Aqk^T ; MMA3: ST += Un^T * KG
    if (tid == 0 && !s.abort_flag) {
      tc::tc_fence_after_sync();
      if (tc::mbar_wait(&s.bar_aqk, ph, &s.abort_flag, status, kWaitAqk)) {
        tc::mma_bf16_ktile(tc::tmem_addr(tm, 0, 192), tc::smem_u32(s.unb), D, tc::smem_u32(s.aqk), BS, BS,
                           idesc_m2, true);
        tc::mma_commit(&s.bar_m2);
      }
      if (tc::mbar_wait(&s.bar_kgt, ph, &s.abort_flag, status, kWaitKgt)) {
        tc::mma_tf32_ktile(tc::tmem_addr(tm, 0, 0), tc::smem_u32(s.un32), D, tc::smem_u32(s.kgt), D, BS,
                           idesc_m3, true);
        tc::mma_commit(&s.bar_m3);
      }
    }

    // ---- output rows of this chunk
    TICK(6);
    tc::mbar_wait(&s.bar_m2, ph, &s.abort_flag, status, kWaitM2);
    tc::tc_fence_after_sync();
    TICK(7);
    if (tid == 0 && more && !s.abort_flag) {
      tc::mbar_expect_tx(&s.bar_aqk, kAqkBytes);
      tc::bulk_g2s(s.aqk, g_aqk + (size_t)(n + 1) * kAqkBytes, kAqkBytes, &s.bar_aqk);
    }
    {
      __nv_bfloat16* orow = o + (((size_t)ib * o_bs + (size_t)n * BS + part * TOK) * H + ih) * D + dv;
#pragma unroll
      for (int t0 = 0; t0 < TOK; t0 += 16) {
        float ov[16];
        tc::tmem_ld16(t_o + t0, ov);
        tc::tmem_ld_wait();
        if (!s.abort_flag) {
#pragma unroll
          for (int i = 0; i < 16; ++i) orow[(size_t)(t0 + i) * H * D] = __float2bfloat16_rn(ov[i]);
        }
      }
    }

    // ---- new state: bf16 operand copy, optional snapshot, pre-scale for the next chunk
    TICK(8);
    tc::mbar_wait(&s.bar_m3, ph, &s.abort_flag, status, kWaitM3);
    tc::tc_fence_after_sync();
    TICK(9);
    if (tid == 0 && more && !s.abort_flag) {
      tc::mbar_expect_tx(&s.bar_kgt, kKgtBytes);
      tc::bulk_g2s(s.kgt, g_kgt + (size_t)(n + 1) * kKgtBytes, kKgtBytes, &s.bar_kgt);
      tc::mbar_expect_tx(&s.bar_ut, kUtBytes);
      tc::bulk_g2s(s.un32, g_ut + (size_t)(n + 1) * kUtBytes, kUtBytes, &s.bar_ut);
    }
    {
      float* hn = (hs && more) ? hs + (((size_t)ib * NC + (n + 1)) * H + ih) * D * D : nullptr;
      float* fin = (!more && sT) ? sT + (size_t)bh * D * D : nullptr;
      const float* gln = s.gl[(n + 1) & 1];
#pragma unroll
      for (int k0 = 0; k0 < KCH; k0 += 16) {
        const int c0 = part * KCH + k0;
        float x[16];
        tc::tmem_ld16(t_state + k0, x);
        tc::tmem_ld_wait();
        if (hn) {
#pragma unroll
          for (int i = 0; i < 16; ++i) hn[(size_t)(c0 + i) * D + dv] = x[i];
        }
        if (fin) {
#pragma unroll
          for (int i = 0; i < 16; ++i) fin[(size_t)(c0 + i) * D + dv] = x[i];
        }
        if (more) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            *reinterpret_cast<uint4*>(&s.sb[((c0 / 8 + j) * D + dv) * 8]) = tc::pack8_bf16(&x[j * 8]);
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] *= gln[c0 + i];
          tc::tmem_st16(t_state + k0, x);
        }
      }
      tc::tmem_st_wait();
    }
    TICK(10);
    tc::fence_async_smem();
    tc::tc_fence_before_sync();
    __syncthreads();
    TICK(11);
  }
#ifdef GDN2_SCAN_TIMING
  if (tid == 0 && blockIdx.x == 0) for (int i = 0; i < 16; ++i) g_scan_timing[i] = tacc[i];
#endif

  tc::tc_fence_before_sync();
  __syncthreads();
  if (wid == 0) tc::tmem_dealloc(tm, 256);
}

}  // namespace

int launch_scan_tc(const WsLayout& L, const WsPtrs& P, const float* s0, void* o, float* sT, float* hs,
                   int B, int S, int H, int64_t o_bs, cudaStream_t st) {
  if (L.DK != D || L.DV != D || L.esz != 2) return GDN2_ERR_UNSUPPORTED;
  const size_t smem = sizeof(ScanTcSmem) + 128;
  // Tuning knob: warps per TMEM lane quarter (1, 2 or 4 -> 128, 256 or 512 threads per block).
  static const int nsplit = [] {
    const char* e = getenv("GDN2_B200_SCAN_NSPLIT");
    const int v = e ? atoi(e) : GDN2_SCAN_NSPLIT;
    return (v == 1 || v == 2 || v == 4) ? v : GDN2_SCAN_NSPLIT;
  }();
  auto launch = [&](auto kern, int threads) -> int {
    GDN2_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<B * H, threads, smem, st>>>(L, P, s0, static_cast<__nv_bfloat16*>(o), sT, hs, S, H, o_bs,
                                       device_status_word());
    return GDN2_OK;
  };
  int rc = nsplit == 1 ? launch(scan_tc_kernel<1>, 128) : nsplit == 2 ? launch(scan_tc_kernel<2>, 256)
                                                                       : launch(scan_tc_kernel<4>, 512);
  if (rc != GDN2_OK) return rc;
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

#ifdef GDN2_SCAN_TIMING
extern "C" int gdn2_debug_scan_timing(unsigned long long* out16) {
  return cudaMemcpyFromSymbol(out16, g_scan_timing, sizeof(unsigned long long) * 16) == cudaSuccess ? 0 : -6;
}
#endif

}  // namespace gdn2
