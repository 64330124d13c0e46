// sm_100a primitives used by the tcgen05 kernels: mbarriers with bounded waits, tensor-memory
// allocation and access, UMMA shared-memory / instruction descriptors and MMA issue.
//
// Operand tiles live in shared memory in the canonical 128-byte-swizzle layout: a tile of R rows
// by 128 16-bit elements is stored as two halves of R rows x 128 bytes (elements 0..63 and
// 64..127); inside a half, 16-byte chunk c of row r sits at r*128 + ((c ^ (r & 7)) << 4).  Such a
// half-tile pair serves both as a K-major operand (rows = M or N index, the 128 elements = K) and
// as an MN-major operand (rows = K index, the 128 elements = N index).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace va {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// One poll: the thread is suspended by the hardware until the phase completes or `kSuspendNs`
// nanoseconds pass, so waiting warps do not compete for issue slots with working warps.
constexpr uint32_t kSuspendNs = 4000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity), "r"(kSuspendNs)
      : "memory");
  return ok != 0;
}
// Every wait in these kernels is bounded: after `kWaitLimit` failed polls (about a second) the
// caller records an error and leaves its loop, so a protocol bug ends the kernel instead of
// hanging the GPU.
constexpr int kWaitLimit = 1 << 18;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = kWaitLimit) {
#pragma unroll 1  // unrolled, every wait site would carry dozens of copies of the poll
  for (int i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// the barrier receives one arrival (already counted in its expected count) when all cp.async
// copies issued so far by this thread have landed
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// ---- TMA (tensor-map copies global -> shared memory, completion counted in bytes on an mbarrier) ----
// one arrival plus the announcement that `bytes` bytes of asynchronous copies will complete on the barrier
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// One box of a 4-d tensor map (coordinates innermost first) into shared memory.  The innermost
// coordinate times the element size must be a multiple of 16 bytes; parts of the box outside the
// tensor are filled with zeros.  This GPU's own memory only.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_addr(bar))
      : "memory");
}

// generic-proxy writes to shared memory -> visible to the async proxy (UMMA operand reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tensor memory ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

// ---- UMMA ------------------------------------------------------------------------------------
// shared-memory matrix descriptor, 128-byte swizzle.  K-major operand: sbo = distance between
// 8-row groups (1024), lbo unused.  MN-major operand: lbo = distance between 64-element blocks
// along MN (the half stride), sbo = distance between 8-row groups along K (1024).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return d;
}
// instruction descriptor, kind::f16, fp32 accumulate.  in16 = 0 for fp16 inputs, 1 for bf16.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int in16, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(in16) << 7) | (static_cast<uint32_t>(in16) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(
          d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] = A[smem] * B[smem] over K = 128 as eight K16 steps, for operand tiles of 128 rows in the half-tile
// pair layout (both K-major): step ks reads 32 bytes further along the rows, steps 4..7 read the second half.
// a0 / b0 are the descriptors of step 0; only their address field (16-byte units) moves.  One instruction
// sequence without per-step descriptor arithmetic in C++: the issuing thread shares its scheduler with busy
// warps, so every instruction it does not execute shortens the time between tiles.
__device__ __forceinline__ void umma_k128_rows128(uint32_t d_tmem, uint64_t a0, uint64_t b0, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "setp.eq.b32 p, %3, %3;\n\t"
      "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 1024;\n\tadd.u64 b, %2, 1024;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 1026;\n\tadd.u64 b, %2, 1026;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 1028;\n\tadd.u64 b, %2, 1028;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t"
      "add.u64 a, %1, 1030;\n\tadd.u64 b, %2, 1030;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a0), "l"(b0), "r"(idesc)
      : "memory");
}
// the mbarrier receives one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

// byte offset of 16-byte chunk c16 (0..15) of row r in a half-tile pair of `rows` rows
__device__ __forceinline__ uint32_t tile_off(int rows, int r, int c16) {
  return static_cast<uint32_t>(c16 >> 3) * static_cast<uint32_t>(rows) * 128u + static_cast<uint32_t>(r) * 128u +
         (static_cast<uint32_t>((c16 & 7) ^ (r & 7)) << 4);
}

}  // namespace sm100
}  // namespace va
