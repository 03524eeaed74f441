// The output projection of the head-parallel layer fused with its all-reduce, for decode-sized inputs
// (at most 8 token rows): out = sum over ranks of x_r W_r^T, every rank receiving the full sum.
//
// The reference layer ends with o_proj (gdn2/attention.py:354-356 of the reference project); split over heads,
// every rank holds a column slice W_r [hidden, K] of the weight and its own x_r [rows, K], and the partial
// products have to be added across ranks. For the one-token step that sum is 8 KiB: a library all-reduce costs
// several launches and a rendezvous for it. Here ONE kernel per rank does the product and the exchange:
//
//   * block c owns 32 output columns. It computes its [rows, 32] partial in fp32 (a skinny product bound by
//     reading W_r once), writes it into slot (parity, my rank) of EVERY rank's exchange buffer with plain stores
//     through peer-mapped pointers (NVLink), makes them visible (system fence) and release-stores the launch's
//     epoch into flag (parity, my rank, c) on every rank;
//   * it then waits, with a bound, until the flags (parity, r, c) in its OWN buffer carry this epoch for every r,
//     adds the partials of all ranks in rank order (so every rank gets bit-identical sums) and writes out.
//
// Only equal-numbered blocks of different ranks talk to each other, and a block writes before it waits, so
// nothing requires all blocks of a launch to be resident at once. The slots are double buffered by the parity
// of the epoch: a rank can run at most one launch ahead of the slowest (to finish launch e+1 it needs every
// rank's flags of e+1, which a rank sends only after it has read its slots of launch e).
// A wait that runs out sets the device status word and the block finishes with what it has; nothing hangs.
// No multicast, no bulk or TMA copy touches another GPU's memory here: plain ld / st only.
#include "common.cuh"

namespace gdn2 {

namespace {

constexpr int kCols = 32;          // output columns per block
constexpr int kMaxRows = 8;
constexpr int kThreads = 128;      // 4 warps x 8 columns
constexpr uint32_t kWaitPeer = 0x40000000u;
constexpr long long kDefaultWait = 200LL * 1000 * 1000;   // about 0.1 s

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int E = 8;
  static __device__ __forceinline__ void unpack(const uint4& p, float* x) {
    const uint32_t u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(u[i] << 16); x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
};
template <> struct Vec16<__half> {
  static constexpr int E = 8;
  static __device__ __forceinline__ void unpack(const uint4& p, float* x) {
    const __half2* h = reinterpret_cast<const __half2*>(&p);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
  }
};
template <> struct Vec16<float> {
  static constexpr int E = 4;
  static __device__ __forceinline__ void unpack(const uint4& p, float* x) {
    x[0] = __uint_as_float(p.x); x[1] = __uint_as_float(p.y); x[2] = __uint_as_float(p.z); x[3] = __uint_as_float(p.w);
  }
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
oproj_reduce_kernel(gdn2_oproj_reduce_args a, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char osm[];
  T* xs = reinterpret_cast<T*>(osm);                                   // [rows][K]
  __shared__ float part[kMaxRows][kCols];
  __shared__ int timed_out;
  constexpr int E = Vec16<T>::E;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;
  const int rows = (int)a.rows, K = (int)a.K, hidden = (int)a.hidden, world = a.world, rank = a.rank;
  const uint32_t epoch = a.epochs[cta] + 1u;                           // this block's launch number, from 1
  const int parity = (int)(epoch & 1u);
  if (tid == 0) timed_out = 0;

  // ---- x rows into shared memory (16-byte pieces)
  {
    const uint4* src = static_cast<const uint4*>(a.x);
    uint4* dst = reinterpret_cast<uint4*>(xs);
    const int n16 = rows * K / E;
    for (int i = tid; i < n16; i += kThreads) dst[i] = src[i];
  }
  __syncthreads();

  // ---- partial product: warp w, columns 32 cta + 8 w .. + 7; the lanes split K in 16-byte pieces
  {
    float acc[8][kMaxRows];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) acc[c][r] = 0.f;
    const T* wbase = static_cast<const T*>(a.weight) + (size_t)(kCols * cta + 8 * wid) * K;
    for (int kk = lane * E; kk < K; kk += 32 * E) {
      uint4 wv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) wv[c] = __ldg(reinterpret_cast<const uint4*>(wbase + (size_t)c * K + kk));
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        if (r < rows) {
          float xf[E];
          Vec16<T>::unpack(*reinterpret_cast<const uint4*>(xs + (size_t)r * K + kk), xf);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float wf[E];
            Vec16<T>::unpack(wv[c], wf);
#pragma unroll
            for (int e = 0; e < E; ++e) acc[c][r] = fmaf(xf[e], wf[e], acc[c][r]);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        float v = acc[c][r];
#pragma unroll
        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) part[r][8 * wid + c] = v;
      }
  }
  __syncthreads();

  T* out = static_cast<T*>(a.out);
  if (world == 1) {
    for (int i = tid; i < rows * kCols; i += kThreads)
      out[(size_t)(i / kCols) * hidden + kCols * cta + (i % kCols)] = from_f32<T>(part[i / kCols][i % kCols]);
    if (tid == 0) a.epochs[cta] = epoch;
    return;
  }

  // ---- my partial into slot (parity, rank) of every rank's buffer: 128-byte rows, coalesced peer stores
  const size_t slot_mine = ((size_t)(parity * world + rank) * kMaxRows) * hidden + (size_t)kCols * cta;
  for (int r = 0; r < world; ++r) {
    float* dst = static_cast<float*>(a.peer_slots[r]) + slot_mine;
    for (int i = tid; i < rows * kCols; i += kThreads) dst[(size_t)(i / kCols) * hidden + (i % kCols)] = part[i / kCols][i % kCols];
  }
  __threadfence_system();
  __syncthreads();
  const size_t flag_base = (size_t)parity * world * ncta;
  if (tid < world) st_release_sys(a.peer_flags[tid] + flag_base + (size_t)rank * ncta + cta, epoch);

  // ---- wait for every rank's partial of this launch (bounded)
  if (tid < world) {
    const uint32_t* f = a.peer_flags[rank] + flag_base + (size_t)tid * ncta + cta;
    const long long limit = a.wait_cycles > 0 ? a.wait_cycles : kDefaultWait;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
      if (clock64() - t0 > limit) {
        atomicOr(status, kWaitPeer);
        timed_out = 1;
        break;
      }
    }
  }
  __syncthreads();

  // ---- sum in rank order (the same order on every rank), reading past L1: the lines were written by peers
  const float* mine = static_cast<const float*>(a.peer_slots[rank]) + ((size_t)parity * world * kMaxRows) * hidden + (size_t)kCols * cta;
  for (int i = tid; i < rows * kCols; i += kThreads) {
    const int r = i / kCols, c = i % kCols;
    float sum = 0.f;
    for (int src = 0; src < world; ++src) sum += __ldcg(mine + ((size_t)src * kMaxRows + r) * hidden + c);
    out[(size_t)r * hidden + kCols * cta + c] = from_f32<T>(sum);
  }
  if (tid == 0) a.epochs[cta] = epoch;
  (void)timed_out;
}

}  // namespace

int launch_oproj_reduce(const gdn2_oproj_reduce_args& a, int dtype, cudaStream_t st) {
  const int esz = dtype == GDN2_F32 ? 4 : 2;
  const size_t smem = (size_t)a.rows * a.K * esz;
  const int grid = (int)(a.hidden / kCols);
  auto launch = [&](auto kern) -> int {
    GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
    kern<<<grid, kThreads, smem, st>>>(a, device_status_word());
    GDN2_CUDA_TRY(cudaGetLastError());
    return GDN2_OK;
  };
  switch (dtype) {
    case GDN2_BF16: return launch(oproj_reduce_kernel<__nv_bfloat16>);
    case GDN2_F16: return launch(oproj_reduce_kernel<__half>);
    case GDN2_F32: return launch(oproj_reduce_kernel<float>);
    default: return GDN2_ERR_BAD_DTYPE;
  }
}

}  // namespace gdn2
