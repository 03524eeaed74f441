// Self-test of the tensor-core building blocks on one thread block: a bulk copy into shared
// memory, K-chunked operand images, tcgen05.mma in bf16 (N = 128) and tf32 (two N = 64 halves
// addressed by a row offset inside the B image), tcgen05.ld, and a tcgen05.st/ld round trip.
//   out[0] = A * B^T with bf16 operands        [128 x 128]
//   out[1] = A * B^T with tf32 operands        [128 x 128]
//   out[2] = 2 * out[1] + 1 after a TMEM store/load round trip
//   out[3] = A * B^T with bf16 operands, A read from tensor memory (packed pairs), B from shared memory
#include "common.cuh"
#include "tc_utils.cuh"

namespace gdn2 {

namespace {

constexpr int M = 128, N = 128, K = 64;

struct alignas(1024) SelfSmem {
  float raw_a[M * K];                 // bulk-copied row-major A
  float a32[M * K];                   // [K/4][M][4]
  float b32[N * K];                   // [K/4][N][4]
  __nv_bfloat16 a16[M * K];           // [K/8][M][8]
  __nv_bfloat16 b16[N * K];           // [K/8][N][8]
  uint64_t bar_copy, bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(128)
selftest_kernel(const float* __restrict__ a, const float* __restrict__ bt, float* __restrict__ out,
                uint32_t* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  SelfSmem& s = *reinterpret_cast<SelfSmem*>(smem_raw);
  const int tid = threadIdx.x, wid = tid >> 5;

  if (tid == 0) {
    tc::mbar_init(&s.bar_copy, 1);
    tc::mbar_init(&s.bar_mma, 1);
    s.abort_flag = 0;
    tc::mbar_init_fence();
  }
  if (wid == 0) tc::tmem_alloc(&s.tmem_base, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = s.tmem_base;

  if (tid == 0) {
    tc::mbar_expect_tx(&s.bar_copy, M * K * 4);
    tc::bulk_g2s(s.raw_a, a, M * K * 4, &s.bar_copy);
  }
  tc::mbar_wait(&s.bar_copy, 0, &s.abort_flag, status, 0x1u);

  // build the operand images: thread = row
  {
    const int r = tid;
    for (int c = 0; c < K / 4; ++c) {
      const float4 va = *reinterpret_cast<const float4*>(&s.raw_a[r * K + c * 4]);
      const float4 vb = *reinterpret_cast<const float4*>(&bt[r * K + c * 4]);
      *reinterpret_cast<float4*>(&s.a32[(c * M + r) * 4]) = va;
      *reinterpret_cast<float4*>(&s.b32[(c * N + r) * 4]) = vb;
    }
    for (int c = 0; c < K / 8; ++c) {
      float xa[8], xb[8];
      for (int i = 0; i < 8; ++i) { xa[i] = s.raw_a[r * K + c * 8 + i]; xb[i] = bt[r * K + c * 8 + i]; }
      *reinterpret_cast<uint4*>(&s.a16[(c * M + r) * 8]) = tc::pack8_bf16(xa);
      *reinterpret_cast<uint4*>(&s.b16[(c * N + r) * 8]) = tc::pack8_bf16(xb);
    }
  }
  {   // A row of this thread as packed bf16 pairs in TMEM columns [320, 352)
    float pk[32];
    for (int c = 0; c < 32; ++c) {
      __nv_bfloat162 h = __floats2bfloat162_rn(s.raw_a[tid * K + 2 * c], s.raw_a[tid * K + 2 * c + 1]);
      pk[c] = __uint_as_float(*reinterpret_cast<uint32_t*>(&h));
    }
    tc::tmem_st32(tc::tmem_addr(tm, (wid & 3) * 32, 320), pk);
    tc::tmem_st_wait();
  }
  tc::fence_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();

  if (tid == 0 && !s.abort_flag) {
    tc::tc_fence_after_sync();
    tc::mma_f16_ts_ktile(tc::tmem_addr(tm, 0, 384), tc::tmem_addr(tm, 0, 320), tc::smem_u32(s.b16), N, K,
                         tc::instr_desc(1, M, N), false);
    tc::mma_bf16_ktile(tc::tmem_addr(tm, 0, 0), tc::smem_u32(s.a16), M, tc::smem_u32(s.b16), N, K,
                       tc::instr_desc(1, M, N), false);
    // tf32: columns [128,192) from B rows 0..63, columns [192,256) from B rows 64..127
    tc::mma_tf32_ktile(tc::tmem_addr(tm, 0, 128), tc::smem_u32(s.a32), M, tc::smem_u32(s.b32), N, K,
                       tc::instr_desc(2, M, 64), false);
    tc::mma_tf32_ktile(tc::tmem_addr(tm, 0, 192), tc::smem_u32(s.a32), M, tc::smem_u32(s.b32) + 64 * 16, N, K,
                       tc::instr_desc(2, M, 64), false);
    tc::mma_commit(&s.bar_mma);
  }
  tc::mbar_wait(&s.bar_mma, 0, &s.abort_flag, status, 0x2u);
  tc::tc_fence_after_sync();

  const uint32_t lane_base = (wid & 3) * 32;
  float vals[32];
  for (int p = 0; p < 2; ++p) {
    for (int c0 = 0; c0 < N; c0 += 32) {
      tc::tmem_ld32(tc::tmem_addr(tm, lane_base, p * 128 + c0), vals);
      tc::tmem_ld_wait();
      for (int i = 0; i < 32; ++i) out[(size_t)p * M * N + tid * N + c0 + i] = vals[i];
      if (p == 1) {
        for (int i = 0; i < 32; ++i) vals[i] = 2.f * vals[i] + 1.f;
        tc::tmem_st32(tc::tmem_addr(tm, lane_base, 256 + c0), vals);
        tc::tmem_st_wait();
      }
    }
  }
  for (int c0 = 0; c0 < N; c0 += 32) {
    tc::tmem_ld32(tc::tmem_addr(tm, lane_base, 256 + c0), vals);
    tc::tmem_ld_wait();
    for (int i = 0; i < 32; ++i) out[(size_t)2 * M * N + tid * N + c0 + i] = vals[i];
  }
  for (int c0 = 0; c0 < N; c0 += 32) {
    tc::tmem_ld32(tc::tmem_addr(tm, lane_base, 384 + c0), vals);
    tc::tmem_ld_wait();
    for (int i = 0; i < 32; ++i) out[(size_t)3 * M * N + tid * N + c0 + i] = vals[i];
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (wid == 0) tc::tmem_dealloc(tm, 512);
}

// A wait that nothing satisfies: the barrier expects one arrival and nobody arrives. The bounded wait gives up
// after `limit_cycles`, records `kWaitSelftest` in the status word, and the block returns normally.
constexpr uint32_t kWaitSelftest = 0x80000000u;
__global__ void __launch_bounds__(64)
selftest_wait_kernel(long long limit_cycles, uint32_t* status, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::mbar_init_fence();
  }
  __syncthreads();
  const bool ok = tc::mbar_wait_limit(&bar, 0, &abort_flag, status, kWaitSelftest, limit_cycles);
  if (!ok && gave_up) atomicAdd(gave_up, 1);
}

}  // namespace

int launch_selftest_wait(long long limit_cycles, int* gave_up, cudaStream_t st) {
  selftest_wait_kernel<<<1, 64, 0, st>>>(limit_cycles, device_status_word(), gave_up);
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

int launch_selftest_mma(const float* a, const float* bt, float* out, cudaStream_t st) {
  const size_t smem = sizeof(SelfSmem) + 1024;
  GDN2_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(selftest_kernel), smem));
  selftest_kernel<<<1, 128, smem, st>>>(a, bt, out, device_status_word());
  GDN2_CUDA_TRY(cudaGetLastError());
  return GDN2_OK;
}

}  // namespace gdn2
