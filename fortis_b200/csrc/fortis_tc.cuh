// Thin wrappers over the sm_100a PTX used by the tensor-core kernels: mbarriers with bounded waits, TMA tile loads,
// tcgen05 MMA / commit / tensor-memory load and store.  Asynchronous instructions are issued warp-uniformly: the whole
// warp runs the loop and `elect.sync` predicates the instruction onto one lane (issuing from a divergent
// `if (lane == 0)` region costs ~100 cycles per tcgen05.mma because operands are moved to uniform registers one by one).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace fortis {
namespace tc {

constexpr uint32_t kWaitLimit = 1u << 24;   // polls of try_wait before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait: returns false (and raises the abort flag, records `code`) when the limit is reached
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code, uint32_t limit) {
  for (uint32_t i = 0; i < limit; i++) {
    if (*abort_flag) return false;
    if (mbar_try_wait(bar, parity)) return true;
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          uint32_t limit = kWaitLimit) {
  if (mbar_try_wait(bar, parity)) return true;          // the common case costs one instruction
  return mbar_wait_slow(bar, parity, abort_flag, status, code, limit);
}

// The same wait without a function call, for kernels whose warpgroups run with different register budgets (setmaxnreg):
// a call there stops the compiler from allocating per budget.  The polling loop is one PTX block, so the surrounding
// code stays as compact as with the call.  The abort flag is read once, after the first failed poll; a thread that is
// already polling when another one gives up runs to its own limit.
__device__ __forceinline__ bool mbar_wait_inline(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .u32 i;\n\tmov.u32 i, 0;\n"
      "WAIT_LOOP_%=:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra WAIT_DONE_%=;\n\t"
      "add.u32 i, i, 1;\n\t"
      "setp.lt.u32 q, i, %3;\n\t"
      "@q bra WAIT_LOOP_%=;\n"
      "WAIT_DONE_%=:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "n"(kWaitLimit) : "memory");
  if (ok) return true;
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n\t}"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n\t}"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}

// linear bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// asks for `bytes` (a multiple of 16) at `src` (16-byte aligned) to be brought into L2; one elected lane issues
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.prefetch.L2.global [%0], %1;\n\t}" ::"l"(src), "r"(bytes) : "memory");
}

// the calling thread's own arrive + expected bytes, and its own linear bulk copy (no election: every calling thread issues)
__device__ __forceinline__ void mbar_arrive_expect_tx_thread(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load_thread(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// the calling thread's own linear bulk copy shared -> global (both 16-byte aligned, size a multiple of 16), in the
// thread's current bulk group
__device__ __forceinline__ void bulk_store_thread(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The MMA and TMA warps run their loops with all 32 lanes (warp-uniform control flow) and let ONE elected lane issue
// each asynchronous instruction.  Issuing from a divergent `if (lane == 0)` region instead costs ~100 cycles per
// tcgen05.mma (operands have to be moved into uniform registers one by one), 3x the 32 cycles a 128x64x16 MMA takes.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] . B[smem]^T, bf16 x bf16 -> fp32, M = 128, N = 64, K = 16
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc) {       // D += A.B
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "n"(IDESC) : "memory");
}
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ts_first(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, q;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "n"(IDESC), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st16p(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);     // .x = lo -> low 16 bits = lower k index
  return *reinterpret_cast<const uint32_t*>(&v);
}


// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 B apart, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);            // start address
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset (leading byte offset unused here)
  d |= (uint64_t)1 << 46;                            // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// D[tmem] (+)= A[smem] . B[smem]^T (both K-major), one elected lane issues
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, q;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "n"(IDESC), "r"(accumulate) : "memory");
}

// ---- two-CTA (cta_group::2) forms: a cluster of two CTAs whose leader (cluster rank 0) issues MMAs over both CTAs'
// rows; each CTA stages its own operand tiles and the leader's barriers collect both CTAs' copies.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of `saddr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier given by its shared::cluster address (possibly in the partner CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// the same without release semantics: for hand-offs that publish no generic-memory writes (an accumulator in tensor
// memory has been read, tcgen05.wait::ld + tcgen05.fence::before_thread_sync done).  A cluster-scope release makes the
// thread wait for its outstanding global stores first, measured at ~1700 cycles per tile in the conv epilogue.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// plain (no multicast) tile load into THIS CTA's shared memory whose completion is counted on `cluster_bar`, a barrier
// given by its shared::cluster address
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3}], [%4];\n\t}"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t cluster_bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3, %4}], [%5];\n\t}"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(cluster_bar) : "memory");
}
// arrives on the barrier at the same shared-memory offset in BOTH CTAs once the pair's earlier MMAs are complete
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}" ::"r"(bar) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem, 128 rows per CTA] . B[smem, half of the N rows per CTA]^T, issued by the leader
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, q;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "n"(IDESC), "r"(accumulate) : "memory");
}

// the same with A in tensor memory: each CTA's 128 rows of A sit at the same columns of its own tensor memory
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ts_acc_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\t"
      "@p tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, 1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "n"(IDESC) : "memory");
}
template <uint32_t IDESC>
__device__ __forceinline__ void tc_mma_ts_first_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\telect.sync _|p, 0xffffffff;\n\tsetp.ne.b32 q, %4, 0;\n\t"
      "@p tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, q;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "n"(IDESC), "r"(accumulate) : "memory");
}

// instruction descriptor: D = f32, A = B = bf16, both K-major
constexpr uint32_t idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

}  // namespace tc
}  // namespace fortis
