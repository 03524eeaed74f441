// Thin inline-PTX wrappers for the Blackwell (sm_100a) asynchronous machinery the tensor-core
// kernels use: mbarriers with bounded waits, bulk (TMA) copies, tensor memory (TMEM) allocation
// and access, shared-memory matrix descriptors and tcgen05.mma issue.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gdn2 {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Cycles a wait may take before the kernel gives up (about 0.2 s at 2 GHz). Normal waits here
// are microseconds; running out means a producer never arrived.
constexpr long long kWaitCycles = 400LL * 1000 * 1000;

// Bounded wait. `abort_flag` is a shared-memory word shared by the whole block: once any wait has
// run out every later wait returns false at once, so a broken pipeline drains in bounded time.
// On the first failure `code` is OR-ed into the device status word.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                uint32_t* status_word, uint32_t code, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;   // the common case costs one probe and no shared-memory load
  if (*abort_flag) return false;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit_cycles) {
      *abort_flag = 1;
      atomicOr(status_word, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* status_word, uint32_t code) {
  return mbar_wait_limit(bar, parity, abort_flag, status_word, code, kWaitCycles);
}

// ------------------------------------------------------------------ proxy / tcgen05 fences

__device__ __forceinline__ void fence_async_smem() {   // generic-proxy smem writes -> async proxy readers
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ bulk copies (TMA, untiled)

// global -> shared, completion counted in bytes on `bar`. Addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// shared -> global, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ tensor memory

// One full warp allocates `cols` (power of two, 32..512) TMEM columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// 32 lanes x 32 columns: thread i of the warp receives columns [col, col+32) of TMEM lane
// (lane field of taddr) + i. A warp may only touch lanes [32*(warp%4), 32*(warp%4)+32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
        "r"(taddr)
      : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}
// 32 lanes x 2 columns.
__device__ __forceinline__ void tmem_st2(uint32_t taddr, const uint32_t (&r)[2]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%2], {%0, %1};" ::"r"(r[0]), "r"(r[1]), "r"(taddr) : "memory");
}
// 32 lanes x 4 columns.
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%4], {%0, %1, %2, %3};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(taddr)
               : "memory");
}
// 32 lanes x 8 columns.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address of (lane, column) relative to an allocation base.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ------------------------------------------------------------------ descriptors and MMA issue

// Shared-memory matrix descriptor for a K-chunked, no-swizzle, K-major operand image
// [K/E][R][16 bytes] (see common.cuh): 8-row x 16-byte core matrices, 128 bytes between 8-row
// groups (stride byte offset), R*16 bytes between the two 16-byte K chunks one MMA consumes
// (leading byte offset). `addr` is the shared-memory byte address of (row0, first K chunk).
__device__ __forceinline__ uint64_t kchunk_desc(uint32_t addr, uint32_t rows_in_image) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((rows_in_image * 16u) >> 4 & 0x3FFFu) << 16;   // leading byte offset
  d |= static_cast<uint64_t>(128u >> 4) << 32;                               // stride byte offset
  d |= 1ull << 46;                                                           // descriptor version (sm_100)
  return d;                                                                  // layout type 0: no swizzle
}

// Instruction descriptor: fp32 accumulate, both operands K-major. `fmt`: 1 = bf16 (kind::f16), 2 = tf32.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t M, uint32_t N) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// A operand from tensor memory (16-bit elements packed two per 32-bit column, K along columns, row m in
// lane m), B from shared memory. `a_tmem` addresses the first of the K/2 columns this MMA consumes.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[128 x N] (+)= A[128 x K] * B[N x K]^T, A in TMEM (8 columns per 16-element K step), B a K-chunked image.
__device__ __forceinline__ void mma_f16_ts_ktile(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t b_rows,
                                                 int K, uint32_t idesc, bool accumulate_first) {
  uint64_t bd = kchunk_desc(b_addr, b_rows);
  const uint64_t bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int ks = 0; ks < K / 16; ++ks) {
    mma_f16_ts(d_tmem, a_tmem + ks * 8, bd, idesc, (ks > 0 || accumulate_first) ? 1u : 0u);
    bd += bstep;
  }
}

// Warp-collective forms: all 32 lanes of a converged warp execute the call with identical arguments
// and one elected lane issues the instruction. Keeping the issuing warp converged lets the operand
// descriptors live in uniform registers instead of being moved there before every MMA.
__device__ __forceinline__ void mma_f16_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four consecutive K steps in one statement: one election, descriptors stepped in place.
__device__ __forceinline__ void mma_f16_ts_k4_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint64_t b_step,
                                                   uint32_t idesc, uint32_t accumulate_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, t, e;\n\t"
      ".reg .b64 b1, b2, b3;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, %5, %5;\n\t"
      "add.u64 b1, %2, %3;\n\t"
      "add.u64 b2, b1, %3;\n\t"
      "add.u64 b3, b2, %3;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "add.u32 a2, %1, 16;\n\t"
      "add.u32 a3, %1, 24;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %4, p;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %4, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %4, t;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %4, t;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "l"(b_step), "r"(idesc), "r"(accumulate_first)
      : "memory");
}
// D[128 x N] (+)= A[128 x K] * B[N x K]^T, A in TMEM, B a K-chunked image; K a multiple of 64.
__device__ __forceinline__ void mma_f16_ts_ktile_warp(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr,
                                                      uint32_t b_rows, int K, uint32_t idesc, bool accumulate_first) {
  const uint64_t bd = kchunk_desc(b_addr, b_rows);
  const uint64_t bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int k4 = 0; k4 < K / 64; ++k4)
    mma_f16_ts_k4_warp(d_tmem, a_tmem + k4 * 32, bd + 4 * k4 * bstep, bstep, idesc,
                       (k4 > 0 || accumulate_first) ? 1u : 0u);
}
__device__ __forceinline__ void mma_commit_warp(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(smem_u32(bar))
      : "memory");
}

// Both operands from shared memory, four consecutive K steps, warp-collective (one election).
#define GDN2_DEFINE_MMA_SS_K4_WARP(NAME, KIND)                                                              \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t a_desc, uint64_t a_step, uint64_t b_desc,  \
                                       uint64_t b_step, uint32_t idesc, uint32_t accumulate_first) {        \
    asm volatile(                                                                                           \
        "{\n\t"                                                                                             \
        ".reg .pred p, t, e;\n\t"                                                                           \
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"                                                             \
        "setp.ne.b32 p, %6, 0;\n\t"                                                                         \
        "setp.eq.b32 t, %6, %6;\n\t"                                                                        \
        "add.u64 a1, %1, %2;\n\t"                                                                           \
        "add.u64 a2, a1, %2;\n\t"                                                                           \
        "add.u64 a3, a2, %2;\n\t"                                                                           \
        "add.u64 b1, %3, %4;\n\t"                                                                           \
        "add.u64 b2, b1, %4;\n\t"                                                                           \
        "add.u64 b3, b2, %4;\n\t"                                                                           \
        "elect.sync _|e, 0xffffffff;\n\t"                                                                   \
        "@e tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %3, %5, p;\n\t"                               \
        "@e tcgen05.mma.cta_group::1.kind::" KIND " [%0], a1, b1, %5, t;\n\t"                               \
        "@e tcgen05.mma.cta_group::1.kind::" KIND " [%0], a2, b2, %5, t;\n\t"                               \
        "@e tcgen05.mma.cta_group::1.kind::" KIND " [%0], a3, b3, %5, t;\n\t"                               \
        "}" ::"r"(d_tmem), "l"(a_desc), "l"(a_step), "l"(b_desc), "l"(b_step), "r"(idesc),                   \
        "r"(accumulate_first)                                                                               \
        : "memory");                                                                                        \
  }
GDN2_DEFINE_MMA_SS_K4_WARP(mma_bf16_k4_warp, "f16")
GDN2_DEFINE_MMA_SS_K4_WARP(mma_tf32_k4_warp, "tf32")
#undef GDN2_DEFINE_MMA_SS_K4_WARP

// D[128 x N] = A[128 x K] * B[N x K]^T over K-chunked images, warp-collective. KSTEP = elements per MMA
// (16 for 16-bit operands, 8 for tf32); K a multiple of 4 * KSTEP.
__device__ __forceinline__ void mma_bf16_ktile_warp(uint32_t d_tmem, uint32_t a_addr, uint32_t a_rows, uint32_t b_addr,
                                                    uint32_t b_rows, int K, uint32_t idesc) {
  const uint64_t ad = kchunk_desc(a_addr, a_rows), bd = kchunk_desc(b_addr, b_rows);
  const uint64_t astep = (2u * a_rows * 16u) >> 4, bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int k4 = 0; k4 < K / 64; ++k4)
    mma_bf16_k4_warp(d_tmem, ad + 4 * k4 * astep, astep, bd + 4 * k4 * bstep, bstep, idesc, k4 > 0 ? 1u : 0u);
}
__device__ __forceinline__ void mma_tf32_ktile_warp(uint32_t d_tmem, uint32_t a_addr, uint32_t a_rows, uint32_t b_addr,
                                                    uint32_t b_rows, int K, uint32_t idesc) {
  const uint64_t ad = kchunk_desc(a_addr, a_rows), bd = kchunk_desc(b_addr, b_rows);
  const uint64_t astep = (2u * a_rows * 16u) >> 4, bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int k4 = 0; k4 < K / 32; ++k4)
    mma_tf32_k4_warp(d_tmem, ad + 4 * k4 * astep, astep, bd + 4 * k4 * bstep, bstep, idesc, k4 > 0 ? 1u : 0u);
}

// mbarrier arrives once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[128 x N] (+)= A[128 x K] * B[N x K]^T over a K-chunked bf16 image pair; K elements, 16 per MMA.
// The descriptors are built once; each K step only bumps their 14-bit start-address fields.
__device__ __forceinline__ void mma_bf16_ktile(uint32_t d_tmem, uint32_t a_addr, uint32_t a_rows, uint32_t b_addr,
                                               uint32_t b_rows, int K, uint32_t idesc, bool accumulate_first) {
  uint64_t ad = kchunk_desc(a_addr, a_rows), bd = kchunk_desc(b_addr, b_rows);
  const uint64_t astep = (2u * a_rows * 16u) >> 4, bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int ks = 0; ks < K / 16; ++ks) {
    mma_bf16(d_tmem, ad, bd, idesc, (ks > 0 || accumulate_first) ? 1u : 0u);
    ad += astep; bd += bstep;
  }
}
// Same for fp32 images read as tf32; 8 K elements per MMA.
__device__ __forceinline__ void mma_tf32_ktile(uint32_t d_tmem, uint32_t a_addr, uint32_t a_rows, uint32_t b_addr,
                                               uint32_t b_rows, int K, uint32_t idesc, bool accumulate_first) {
  uint64_t ad = kchunk_desc(a_addr, a_rows), bd = kchunk_desc(b_addr, b_rows);
  const uint64_t astep = (2u * a_rows * 16u) >> 4, bstep = (2u * b_rows * 16u) >> 4;
#pragma unroll
  for (int ks = 0; ks < K / 8; ++ks) {
    mma_tf32(d_tmem, ad, bd, idesc, (ks > 0 || accumulate_first) ? 1u : 0u);
    ad += astep; bd += bstep;
  }
}

// pack 8 fp32, each times `mul`, into 8 fp16 (16 bytes)
__device__ __forceinline__ uint4 pack8_f16(const float* x, float mul) {
  uint4 r;
  __half2 t;
  t = __floats2half2_rn(x[0] * mul, x[1] * mul); r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(x[2] * mul, x[3] * mul); r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(x[4] * mul, x[5] * mul); r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(x[6] * mul, x[7] * mul); r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}

// pack 8 fp32 into 8 bf16 (16 bytes)
__device__ __forceinline__ uint4 pack8_bf16(const float* x) {
  uint4 r;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(x[0], x[1]); r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(x[2], x[3]); r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(x[4], x[5]); r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(x[6], x[7]); r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}

}  // namespace tc
}  // namespace gdn2
