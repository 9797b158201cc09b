// Thin inline-PTX layer for the Blackwell (sm_100a) features the tensor-core kernels
// use: mbarriers with bounded waits, TMA tile loads, tensor-memory allocation and
// access, and tcgen05 MMA issue/commit.  No multicast forms are used anywhere.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"

namespace tb200 {
namespace sm100 {

// ---- error reporting ---------------------------------------------------------
// Every wait in the kernels is bounded.  When a wait gives up, the kernel records
// where in a device status word, raises a CTA-wide abort flag in shared memory, and
// all roles drain to the common teardown (which frees tensor memory) and return.
enum : int {
  kStatusOk = 0,
  kStatusTimeoutTma = 1,       // tile never landed
  kStatusTimeoutOperand = 2,   // operand stage never produced
  kStatusTimeoutMma = 3,       // MMA completion never signalled
  kStatusTimeoutStageFree = 4, // stage never released
  kStatusTimeoutSelfTest = 5,  // the wait of tb200_selftest_wait_timeout (never satisfied)
  kStatusTimeoutPeer = 6       // a peer's loss sum never arrived (tb200_loss_sum_exchange)
};

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false (after raising *abortFlag and recording `code`) if the
// barrier did not flip within `limitNs` or another role already aborted.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity,
                                                volatile int* abortFlag, int* status, int code,
                                                unsigned long long limitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abortFlag) return false;
      if (global_timer_ns() - t0 > limitNs) {
        *abortFlag = 1;
        if (status) atomicCAS(status, kStatusOk, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abortFlag, int* status, int code) {
  return mbar_wait_limit(bar, parity, abortFlag, status, code, kWaitLimitNs);
}

// ---- TMA ------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// Contiguous copy global -> shared (both 16-byte aligned, size a multiple of 16 bytes),
// completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// 3-D tile load global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y),
      "r"(z)
      : "memory");
}

// 3-D tile store shared -> global (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* src, int x, int y,
                                             int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// The same tile ADDED to global memory (fp32 add done by the copy engine).
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* src, int x,
                                                  int y, int z) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until the stores committed by this thread have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Makes this thread's earlier generic-proxy writes to shared memory visible to the async
// proxy (TMA stores, MMA operand fetches).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor memory ----------------------------------------------------------------
// Warp-wide.  Writes the base address of `ncols` columns (power of two >= 32) to *dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* dstSmem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dstSmem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Each lane of the warp stores 16 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
      "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
      "r"(v[15])
      : "memory");
}

// Each lane loads 16 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// 8-column variants.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                 "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

// ---- MMA ----------------------------------------------------------------------------
// Shared-memory operand descriptor for a tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box with a 128-byte inner extent produces), 8-row
// groups 1024 bytes apart.  `sboBytes`/`lboBytes` are the two group strides; for a
// K-major operand only the stride between 8-row groups matters.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smemAddr, uint32_t lboBytes,
                                                    uint32_t sboBytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smemAddr & 0x3ffff) >> 4);
  d |= (uint64_t)((lboBytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sboBytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// The same for the 128-byte swizzle with 32-byte atoms (rows of 128 bytes, 32-byte chunks
// XORed with row % 4; what a TMA box written with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B holds):
// the only layout an MN-major TF32 operand may use.  Atoms are 32 MN-elements x 4 K-rows;
// lboBytes = distance between atoms along MN, sboBytes = distance between 4-row groups.
__device__ __forceinline__ uint64_t smem_desc_sw128_base32(uint32_t smemAddr, uint32_t lboBytes,
                                                           uint32_t sboBytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smemAddr & 0x3ffff) >> 4);
  d |= (uint64_t)((lboBytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sboBytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;  // SWIZZLE_128B_BASE32B
  return d;
}

// Instruction descriptor, kind::tf32, fp32 accumulate, M x N tile.
// aMajorMN / bMajorMN: 0 = K-major operand, 1 = MN-major operand.
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N, int aMajorMN, int bMajorMN) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)aMajorMN << 15) |
         ((uint32_t)bMajorMN << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[tmem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_tf32_ts(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_tf32_ss(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on `bar` when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// 2^x on the special-function unit (relative error ~2^-22, denormal results flushed).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

#endif  // __CUDACC__

// ---- host: tensor maps ------------------------------------------------------------
// fp32 tensor [d2][d1][d0] (d0 innermost, contiguous), box [1][box1][32] with the
// 128-byte swizzle; out-of-range elements read as zero.
// atom32 selects the 128-byte swizzle with 32-byte atoms instead of the plain one.
CUtensorMap make_tmap_f32_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box1,
                             bool atom32 = false);

// bf16 tensor [d2][d1][d0], box [1][box1][box0] with box0 = 32 or 64 elements (rows of 64 or
// 128 bytes) and the swizzle of that width.
CUtensorMap make_tmap_bf16_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box0,
                              uint32_t box1);

// fp32 tensor [d2][d1][d0], box [1][1][box0] without swizzle (rows of scalars).
CUtensorMap make_tmap_f32_rows(const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1Bytes, uint64_t stride2Bytes, uint32_t box0);

}  // namespace sm100
}  // namespace tb200
