// Recurrent decode of several tokens at once, DK = DV = 128: the n-token recurrence of
// decode_multi_kernel (gdn2/inference.py:199-303 of the reference project) evaluated in blocks of up
// to 8 tokens without a per-token dependent sweep over the state.
//
// With A_t = exp(g_1 + .. + g_t) per key channel (A_t / A_s <= 1 for s <= t, so nothing can overflow):
//     u_t = w_t*v_t - (b_t*k_t*A_t)^T S_0 - sum_{s<t} Akk[t,s] u_s      Akk[t,s] = sum_c b_t k_t k_s A_t/A_s
//     o_t = (scale*q_t*A_t)^T S_0 + sum_{s<=t} Aqk[t,s] u_s              Aqk[t,s] = scale * sum_c q_t k_s A_t/A_s
//     S_8 = diag(A_8) S_0 + sum_s (k_s * A_8/A_s) u_s^T
// which is the token-by-token recurrence S <- diag(exp g) S; u = w*v - S^T(b*k); S <- S + k u^T;
// o = scale S^T q with the sums regrouped: two sweeps over the state tile with 64 and 36 independent
// accumulation chains per thread instead of 2 n sweeps that each wait for a cross-thread reduction.
//
// Persistent blocks, one per SM, walk over the (batch, head) tiles with four kinds of warps:
//   * one copy thread brings a tile's 64 KiB of fp32 state into shared memory by bulk copies (TMA) two
//     tiles ahead and sends the updated tile back the same way: HBM traffic is the state once in, once
//     out, and no compute thread ever waits on a global load of it;
//   * one output thread sends each step's output rows, staged in shared memory by the sweep warps, as one
//     bulk copy per token row;
//   * four table warps (thread = channel) fetch the token vectors a step ahead as 16-byte pieces, pass them
//     through a staging buffer to read their own channel, and build the step's coefficient tables and the
//     8 x 8 pair matrices while the current step is swept;
//   * eight sweep warps do the two sweeps in place: warp w owns value columns 16w .. 16w+15, lane
//     (rgl = lane >> 2, cq = lane & 3) columns 16w + 4cq .. +3 of key rows 16 rgl .. 16 rgl + 15.
// Hand-offs are mbarriers with bounded waits.
// Per-row coefficients sit in shared memory once; the packed f32x2 FMAs pair them over products (sweep 1)
// or tokens (sweep 2), so no duplicated copies are stored or fetched.
#include "common.cuh"
#include "tc_utils.cuh"

namespace gdn2 {

namespace {

constexpr int D = 128;
constexpr int NB = 8;                       // tokens per block step
constexpr int kGroupFloats = 16 * D + 16;   // 16 state rows + 64 bytes: adjacent row groups land 64 B apart mod 128
constexpr int kTileFloats = 8 * kGroupFloats;
constexpr uint32_t kGroupBytes = 16 * D * 4;
constexpr int kCoefRows = 136;              // 128 rows + one slot per 16-row group
__device__ __forceinline__ int crow(int r) { return r + (r >> 4); }

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
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Tables {
  // per key row: chunks 0, 1 = b*k*A_t for t < 8, chunks 2, 3 = scale*q*A_t (four consecutive products per chunk)
  float4 c1[4][kCoefRows];
  // per key row: k * A_8/A_s for s = 0..3 (chunk 0) and s = 4..7 (chunk 1); A_8 itself
  float4 c2[2][kCoefRows];
  float gam[kCoefRows];
  float wv[NB][D];                    // w * v
  float akk[NB][NB];                  // strictly lower
  float aqk[NB][NB];                  // lower incl. diagonal, scale folded in
};

struct alignas(128) BlockedSmem {
  float tile[2][kTileFloats];         // the state of two (batch, head) tiles
  Tables tab[2];                      // coefficient tables of two consecutive steps
  float part[4][64];                  // per 32-channel group: partial sums of the 64 pair entries
  // one step's token vectors as they lie in memory: q, k, b, v, w rows of D elements (up to 4 bytes each), then g
  alignas(16) unsigned char stage[6 * NB * D * 4];
  uint64_t tile_full[2], tile_done[2];   // copy thread -> sweep warps (bytes landed); sweep warps -> copy thread
  uint64_t tab_full[2], tab_empty[2];    // table warps -> sweep warps; sweep warps -> table warps
  uint64_t o_full[2];                    // sweep warps -> output thread (a step's rows are staged)
  int abort_flag;
  alignas(16) unsigned char ostage[2][NB * D * 4];   // a step's output rows [token][value channel] on their way out
};

constexpr int kSweepThreads = 256;    // warps 0..7
constexpr int kTableThreads = 128;    // warps 8..11
constexpr int kAllThreads = kSweepThreads + kTableThreads + 64;   // + warp 12: one thread drives the state copies; warp 13: one thread sends the outputs

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
}
// one arrival per warp: the lanes' writes are ordered before lane 0's arrival by the warp barrier
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void table_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// the same barrier fused with an OR over one predicate per thread: every table thread gets the same answer
__device__ __forceinline__ bool table_sync_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// Bounded wait for hand-offs that have thousands of cycles of slack: the polling thread sleeps between probes
// instead of competing with the sweep warps for issue slots.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t* status_word, uint32_t code) {
  if (tc::mbar_try_wait(bar, parity)) return true;
  const long long t_begin = clock64();
  while (true) {
    __nanosleep(128);
    if (tc::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t_begin > tc::kWaitCycles) {
      *abort_flag = 1;
      atomicOr(status_word, code);
      return false;
    }
  }
}

enum : uint32_t { kWaitTile = 0x10000u, kWaitTab = 0x20000u, kWaitEmpty = 0x40000u, kWaitDone = 0x80000u, kWaitOut = 0x100000u };

template <typename T>
__global__ void __launch_bounds__(kAllThreads, 1)
decode_blocked_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      const float* __restrict__ g, const T* __restrict__ b, const T* __restrict__ w,
                      float* __restrict__ state, T* __restrict__ o, int ntiles, int n, int H, int HK, int64_t in_bs,
                      int64_t o_bs, float scale, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  BlockedSmem& s = *reinterpret_cast<BlockedSmem*>(smem_raw);
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s.tile_full[i], 1);
      tc::mbar_init(&s.tile_done[i], kSweepThreads / 32);     // one arrival per warp
      tc::mbar_init(&s.tab_full[i], kTableThreads / 32);
      // a table buffer is free when the eight sweep warps have finished its step AND the output thread has sent
      // the step's rows: the tables of step k + 2 are then built after the staging rows of step k were read, and
      // the sweep warps (which wait for those tables) may overwrite the rows without a hand-off of their own
      tc::mbar_init(&s.tab_empty[i], kSweepThreads / 32 + 1);
      tc::mbar_init(&s.o_full[i], kSweepThreads / 32);
    }
    s.abort_flag = 0;
    tc::mbar_init_fence();
  }
  __syncthreads();

  if (wid == 13) {
    // =============================== output thread: a step's rows leave as bulk copies ==========
    // (256-byte rows for 16-bit outputs: eight scattered 2-byte stores per lane of the sweep warps otherwise)
    if (lane == 0) {
      const int spt = (n + NB - 1) / NB;
      const int my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const int total_steps = my_tiles * spt;
      for (int step = 0; step < total_steps; ++step) {
        const int tile = blockIdx.x + (step / spt) * gridDim.x, t0 = (step % spt) * NB;
        const int ib = tile / H, ih = tile % H;
        const int nb = min(NB, n - t0);
        if (!mbar_wait_relaxed(&s.o_full[step & 1], (step >> 1) & 1, &s.abort_flag, status, kWaitOut)) break;
        const T* src = reinterpret_cast<const T*>(s.ostage[step & 1]);
        for (int t = 0; t < nb; ++t)
          tc::bulk_s2g(o + (((size_t)ib * o_bs + (t0 + t)) * H + ih) * D, src + t * D, D * sizeof(T));
        tc::bulk_commit();
        tc::bulk_wait_read_all();                        // the staging rows may be overwritten
        mbar_arrive(&s.tab_empty[step & 1]);
      }
      tc::bulk_wait_all();
    }
  } else if (wid == 12) {
    // =============================== copy thread: tiles in, tiles out ==========================
    if (lane == 0) {
      auto load_tile = [&](int tile, int buf) {          // 8 bulk copies of 16 rows each
        tc::mbar_expect_tx(&s.tile_full[buf], 8 * kGroupBytes);
        const float* src = state + (size_t)tile * D * D;
#pragma unroll
        for (int gidx = 0; gidx < 8; ++gidx)
          tc::bulk_g2s(&s.tile[buf][gidx * kGroupFloats], src + gidx * 16 * D, kGroupBytes, &s.tile_full[buf]);
      };
      const int first = blockIdx.x, stride = gridDim.x;
      if (first < ntiles) load_tile(first, 0);
      if (first + stride < ntiles) load_tile(first + stride, 1);
      int it = 0;
      for (int tile = first; tile < ntiles; tile += stride, ++it) {
        const int buf = it & 1;
        if (!mbar_wait_relaxed(&s.tile_done[buf], (it >> 1) & 1, &s.abort_flag, status, kWaitDone)) break;
        float* dst = state + (size_t)tile * D * D;
#pragma unroll
        for (int gidx = 0; gidx < 8; ++gidx)
          tc::bulk_s2g(dst + gidx * 16 * D, &s.tile[buf][gidx * kGroupFloats], kGroupBytes);
        tc::bulk_commit();
        if (tile + 2 * stride < ntiles) {
          tc::bulk_wait_read_all();                      // the buffer may be overwritten once the store has read it
          load_tile(tile + 2 * stride, buf);
        }
      }
      tc::bulk_wait_all();
    }
  } else if (wid >= 8) {
    // =============================== table warps: thread = key / value channel =================
    const int c = tid - kSweepThreads;
    const int pw_ = wid - 8;                             // 32-channel group
    const int spt = (n + NB - 1) / NB;                   // steps per tile
    const int my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total_steps = my_tiles * spt;
    // A step's token vectors are 8 rows of D elements per tensor, contiguous per row: the 128 threads fetch them
    // as 16-byte pieces (CH pieces per thread and tensor, two for g), ONE STEP AHEAD, into registers; at the
    // top of a step the pieces go to the staging buffer and every thread reads its own channel from there.
    constexpr int CH = sizeof(T) / 2;                    // 16-byte pieces per thread: 8 rows x D x sizeof(T) / 16 / 128
    constexpr int kRowPieces = D * (int)sizeof(T) / 16;  // pieces per row
    uint4 ldT[5][CH], ldG[2];
    auto issue_loads = [&](int pstep) {
      const int ptile = blockIdx.x + (pstep / spt) * gridDim.x, pt0 = (pstep % spt) * NB;
      const int pib = ptile / H, pih = ptile % H, pihk = pih / (H / HK);
      const int pnb = min(NB, n - pt0);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int e = c + kTableThreads * j, tokr = e / kRowPieces, within = e % kRowPieces;
        const int tt = pt0 + (tokr < pnb ? tokr : pnb - 1);                 // padding tokens re-read the last real one
        const size_t rowk = (((size_t)pib * in_bs + tt) * HK + pihk) * D, rowv = (((size_t)pib * in_bs + tt) * H + pih) * D;
        ldT[0][j] = __ldg(reinterpret_cast<const uint4*>(q + rowk) + within);
        ldT[1][j] = __ldg(reinterpret_cast<const uint4*>(k + rowk) + within);
        ldT[2][j] = __ldg(reinterpret_cast<const uint4*>(b + rowk) + within);
        ldT[3][j] = __ldg(reinterpret_cast<const uint4*>(v + rowv) + within);
        ldT[4][j] = __ldg(reinterpret_cast<const uint4*>(w + rowv) + within);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int e = c + kTableThreads * j, tokr = e / (D / 4), within = e % (D / 4);
        const int tt = pt0 + (tokr < pnb ? tokr : pnb - 1);
        ldG[j] = __ldg(reinterpret_cast<const uint4*>(g + (((size_t)pib * in_bs + tt) * HK + pihk) * D) + within);
      }
    };
    T* stT = reinterpret_cast<T*>(s.stage);                                // [5][NB][D]
    float* stG = reinterpret_cast<float*>(s.stage + 5 * NB * D * sizeof(T));   // [NB][D]
    if (total_steps > 0) issue_loads(0);
    for (int step = 0; step < total_steps; ++step) {
      {
        const int t0 = (step % spt) * NB;
        const int nb = min(NB, n - t0);
        Tables& tb = s.tab[step & 1];
        // every thread has read the previous step's staging buffer (two table barriers lie in between)
#pragma unroll
        for (int j = 0; j < CH; ++j) {
#pragma unroll
          for (int x = 0; x < 5; ++x)
            reinterpret_cast<uint4*>(stT + (size_t)x * NB * D)[c + kTableThreads * j] = ldT[x][j];
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) reinterpret_cast<uint4*>(stG)[c + kTableThreads * j] = ldG[j];
        if (step + 1 < total_steps) issue_loads(step + 1);
        table_sync();
        float graw[NB];
        T kraw[NB], braw[NB], qraw[NB], wraw[NB], vraw[NB];
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          graw[t] = stG[t * D + c];
          qraw[t] = stT[(0 * NB + t) * D + c]; kraw[t] = stT[(1 * NB + t) * D + c]; braw[t] = stT[(2 * NB + t) * D + c];
          vraw[t] = stT[(3 * NB + t) * D + c]; wraw[t] = stT[(4 * NB + t) * D + c];
        }
        float G[NB], kk[NB], bk[NB], qs[NB], wvv[NB];
        float run = 0.f;
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          const bool real = t < nb;                      // padding token: no decay, no write, no read
          run += real ? graw[t] * kLog2e : 0.f;
          kk[t] = real ? to_f32(kraw[t]) : 0.f;
          bk[t] = real ? to_f32(braw[t]) * kk[t] : 0.f;
          qs[t] = real ? to_f32(qraw[t]) * scale : 0.f;
          wvv[t] = real ? to_f32(wraw[t]) * to_f32(vraw[t]) : 0.f;
          G[t] = run;                                    // log2 of A_t
        }
        // the sweep warps have finished with this table buffer (two steps ago)
        // (one warp polls, with pauses; the other three sleep at the barrier below)
        bool okw = true;
        if (wid == 8) okw = mbar_wait_relaxed(&s.tab_empty[step & 1], ((step >> 1) & 1) ^ 1, &s.abort_flag, status, kWaitEmpty);
        // uniform over the table warps; it also orders this step after the reads of the previous step's partial sums
        if (table_sync_or(!okw)) break;
        {
          const int pr = crow(c);
          float c1v[16], c2v[8];
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            const float At = ex2(G[t]);
            c1v[t] = bk[t] * At;
            c1v[8 + t] = qs[t] * At;
            c2v[t] = kk[t] * ex2(G[NB - 1] - G[t]);
            tb.wv[t][c] = wvv[t];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) tb.c1[j][pr] = make_float4(c1v[4 * j], c1v[4 * j + 1], c1v[4 * j + 2], c1v[4 * j + 3]);
#pragma unroll
          for (int j = 0; j < 2; ++j) tb.c2[j][pr] = make_float4(c2v[4 * j], c2v[4 * j + 1], c2v[4 * j + 2], c2v[4 * j + 3]);
          const float An = ex2(G[NB - 1]);
          tb.gam[pr] = An;
        }
        // Slot (t, sx) holds the Akk[t, sx] term for sx < t and the Aqk[sx, t] term for sx >= t (the upper
        // triangle is free). Summing over the warp's 32 channels: each step halves what a lane keeps.
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          float term[32];
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const int t = 4 * hb + tt;
#pragma unroll
            for (int sx = 0; sx < NB; ++sx) {
              float val;
              if (sx < t) val = bk[t] * kk[sx] * ex2(G[t] - G[sx]);          // Akk[t, sx], A_t / A_s <= 1
              else if (sx == t) val = qs[t] * kk[t];                          // Aqk[t, t]
              else val = qs[sx] * kk[t] * ex2(G[sx] - G[t]);                  // Aqk[sx, t]
              term[tt * 8 + sx] = val;
            }
          }
#pragma unroll
          for (int m = 0; m < 5; ++m) {
            const int half = 16 >> m;                    // values kept after this step
            const int bit = 16 >> m;
            const bool up = (lane & bit) != 0;
#pragma unroll
            for (int x = 0; x < half; ++x) {
              const float send = up ? term[x] : term[x + half];
              const float keep = up ? term[x + half] : term[x];
              term[x] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
            }
          }
          int idx = 0;                                   // the lane bit tested at step m chose the upper half of 16 >> m entries
#pragma unroll
          for (int m = 0; m < 5; ++m) idx += ((lane >> (4 - m)) & 1) * (16 >> m);
          s.part[pw_][32 * hb + idx] = term[0];
        }
        table_sync();
        if (c < 64) {
          const float sum = s.part[0][c] + s.part[1][c] + s.part[2][c] + s.part[3][c];
          const int t = c >> 3, sx = c & 7;
          if (sx < t) tb.akk[t][sx] = sum;               // Akk[t, sx]
          else tb.aqk[sx][t] = sum;                      // slot (t, sx) with sx >= t holds Aqk[sx, t]
        }
        warp_arrive(&s.tab_full[step & 1], lane);
      }
      if (s.abort_flag) break;
    }
  } else {
    // =============================== sweep warps ================================================
    const int rgl = lane >> 2, cq = lane & 3;
    const int col0 = 16 * wid + 4 * cq;
    int it = 0, step = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      float* S = s.tile[buf];
      bool ok = true;
      for (int t0 = 0; t0 < n; t0 += NB, ++step) {
        const int nb = min(NB, n - t0);
        const Tables& tb = s.tab[step & 1];
        ok = tc::mbar_wait(&s.tab_full[step & 1], (step >> 1) & 1, &s.abort_flag, status, kWaitTab);
        if (ok && t0 == 0) ok = tc::mbar_wait(&s.tile_full[buf], (it >> 1) & 1, &s.abort_flag, status, kWaitTile);
        ok = __all_sync(0xffffffffu, ok);                // the warp leaves together: what follows uses full-warp shuffles
        if (!ok) break;

        // ---- sweep 1: the 16 products (8 erase rows, 8 query rows) of S_0 for this thread's rows and columns
        //      packed over PAIRS OF PRODUCTS: acc[pp][col] = (product 2pp, product 2pp+1) of column col, so the
        //      coefficients are used as stored (no duplicated copies in shared memory) and the state value is
        //      the operand that is duplicated, in registers
        float2 acc[8][4];
#pragma unroll
        for (int p = 0; p < 8; ++p) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) acc[p][cc] = make_float2(0.f, 0.f);
        }
        const float* Srow = S + rgl * kGroupFloats + col0;
        const int cr0 = 17 * rgl;
#pragma unroll                             // all 16 rows: the loads of later rows are scheduled under the FMAs of earlier ones
        for (int i = 0; i < 16; ++i) {
          const float4 sv = *reinterpret_cast<const float4*>(Srow + i * D);
          const float2 sd[4] = {make_float2(sv.x, sv.x), make_float2(sv.y, sv.y), make_float2(sv.z, sv.z),
                                make_float2(sv.w, sv.w)};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 cf = tb.c1[j][cr0 + i];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              acc[2 * j][cc] = ffma2(sd[cc], make_float2(cf.x, cf.y), acc[2 * j][cc]);
              acc[2 * j + 1][cc] = ffma2(sd[cc], make_float2(cf.z, cf.w), acc[2 * j + 1][cc]);
            }
          }
        }
        // reduce over the 8 row groups. Index = half*32 + column*8 + t (half 0: erase products, 1: query
        // products); lane (rgl) ends with the 8 values of half rgl >> 2, column rgl & 3.
        float pv[8];
        {
          float val[64];
#pragma unroll
          for (int pp = 0; pp < 8; ++pp) {
            const int base = (pp >> 2) * 32 + 2 * (pp & 3);       // products 2pp, 2pp + 1
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) { val[base + cc * 8] = acc[pp][cc].x; val[base + cc * 8 + 1] = acc[pp][cc].y; }
          }
#pragma unroll
          for (int m = 0; m < 3; ++m) {
            const int half = 32 >> m;
            const int bit = 16 >> m;                     // lane bits 4, 3, 2 = rgl bits 2, 1, 0
            const bool up = (lane & bit) != 0;
#pragma unroll
            for (int x = 0; x < half; ++x) {
              const float send = up ? val[x] : val[x + half];
              const float keep = up ? val[x + half] : val[x];
              val[x] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
            }
          }
#pragma unroll
          for (int t = 0; t < 8; ++t) pv[t] = val[t];
        }
        // ---- forward substitution for u on the lanes that hold the erase products; the lanes that hold
        //      the query products of the same column take u from them and form the outputs
        const bool has_q = (rgl & 4) != 0;
        const int mycol = col0 + (rgl & 3);
        float u[8];
        {
          float4 ak[NB][2];                              // rows of Akk, fetched ahead of the dependent chain
#pragma unroll
          for (int t = 1; t < NB; ++t) {
            ak[t][0] = *reinterpret_cast<const float4*>(&tb.akk[t][0]);
            if (t > 4) ak[t][1] = *reinterpret_cast<const float4*>(&tb.akk[t][4]);
          }
          float wvt[NB];
#pragma unroll
          for (int t = 0; t < NB; ++t) wvt[t] = tb.wv[t][mycol];
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            float x = wvt[t] - pv[t];
            const float arow[8] = {ak[t][0].x, ak[t][0].y, ak[t][0].z, ak[t][0].w, ak[t][1].x, ak[t][1].y, ak[t][1].z, ak[t][1].w};
#pragma unroll
            for (int sx = 0; sx < t; ++sx) x = fmaf(-arow[sx], u[sx], x);
            u[t] = x;                                    // meaningful on the erase lanes only
          }
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            const float other = __shfl_xor_sync(0xffffffffu, u[t], 16);
            if (has_q) u[t] = other;
          }
        }
        if (has_q) {
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            const float4 a0 = *reinterpret_cast<const float4*>(&tb.aqk[t][0]);
            const float4 a1 = *reinterpret_cast<const float4*>(&tb.aqk[t][4]);
            const float arow[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float ov = pv[t];
#pragma unroll
            for (int sx = 0; sx <= t; ++sx) ov = fmaf(arow[sx], u[sx], ov);
            reinterpret_cast<T*>(s.ostage[step & 1])[t * D + mycol] = from_f32<T>(ov);
          }
        }
        tc::fence_async_smem();                          // the staged rows are read by the bulk store
        warp_arrive(&s.o_full[step & 1], lane);
        // gather u of the thread's four columns from the lanes that share cq (rgl bits 0 and 1 = lane bits 2, 3)
        //      and pair them over tokens: up[tp][c] = (u_{2tp}, u_{2tp+1}) of column col0 + c
        float2 up[4][4];
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          const float o4 = __shfl_xor_sync(0xffffffffu, u[t], 4);      // column (rgl & 3) ^ 1
          const float e = (rgl & 1) ? o4 : u[t];                       // even column of my pair
          const float od = (rgl & 1) ? u[t] : o4;                      // odd column of my pair
          const float e2 = __shfl_xor_sync(0xffffffffu, e, 8);         // the other pair
          const float od2 = __shfl_xor_sync(0xffffffffu, od, 8);
          const float uc[4] = {(rgl & 2) ? e2 : e, (rgl & 2) ? od2 : od, (rgl & 2) ? e : e2, (rgl & 2) ? od : od2};
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            if (t & 1) up[t >> 1][cc].y = uc[cc];
            else up[t >> 1][cc].x = uc[cc];
          }
        }
        // ---- sweep 2: S <- A_8 * S + sum_s (k_s A_8/A_s) u_s^T, in place
        {
          float* Sw = S + rgl * kGroupFloats + col0;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            // per column a dot product over the 8 tokens, packed over token pairs (coefficients as stored)
            const float4 sv = *reinterpret_cast<const float4*>(Sw + i * D);
            const float4 ka = tb.c2[0][cr0 + i], kb = tb.c2[1][cr0 + i];
            const float ga = tb.gam[cr0 + i];
            const float2 k01 = make_float2(ka.x, ka.y), k23 = make_float2(ka.z, ka.w);
            const float2 k45 = make_float2(kb.x, kb.y), k67 = make_float2(kb.z, kb.w);
            const float svv[4] = {sv.x, sv.y, sv.z, sv.w};
            float nn[4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const float2 d = ffma2(k01, up[0][cc], ffma2(k23, up[1][cc], ffma2(k45, up[2][cc], fmul2(k67, up[3][cc]))));
              nn[cc] = fmaf(ga, svv[cc], d.x + d.y);
            }
            *reinterpret_cast<float4*>(Sw + i * D) = make_float4(nn[0], nn[1], nn[2], nn[3]);
          }
        }
        warp_arrive(&s.tab_empty[step & 1], lane);       // this step's tables may be overwritten
      }
      if (!ok) break;
      tc::fence_async_smem();                            // the tile's new values are visible to the bulk store
      warp_arrive(&s.tile_done[buf], lane);
    }
  }
}

}  // namespace

template <typename T>
int launch_decode_blocked(const T* q, const T* k, const T* v, const float* g, const T* b, const T* w, float* state,
                          T* o, int B, int n, int H, int HK, int64_t in_bs, int64_t o_bs, float scale, cudaStream_t st) {
  const size_t smem = sizeof(BlockedSmem) + 128;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(decode_blocked_kernel<T>), smem));
  const int ntiles = B * H;
  const int sms = device_sm_count();
  const int grid = ntiles < sms ? ntiles : sms;
  decode_blocked_kernel<T><<<grid, kAllThreads, smem, st>>>(q, k, v, g, b, w, state, o, ntiles, n, H, HK, in_bs, o_bs, scale,
                                                         device_status_word());
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

template int launch_decode_blocked<float>(const float*, const float*, const float*, const float*, const float*,
                                          const float*, float*, float*, int, int, int, int, int64_t, int64_t, float,
                                          cudaStream_t);
template int launch_decode_blocked<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*,
                                                  const float*, const __nv_bfloat16*, const __nv_bfloat16*, float*,
                                                  __nv_bfloat16*, int, int, int, int, int64_t, int64_t, float, cudaStream_t);
template int launch_decode_blocked<__half>(const __half*, const __half*, const __half*, const float*, const __half*,
                                           const __half*, float*, __half*, int, int, int, int, int64_t, int64_t, float,
                                           cudaStream_t);

}  // namespace gdn2
