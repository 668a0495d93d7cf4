// Thin inline-PTX wrappers for the sm_100a features the NVFP4 kernels use:
// mbarriers with bounded waits, TMA tiled loads, cp.async, tcgen05 (TMEM
// allocation, MMA issue, commit, TMEM loads) and the UMMA descriptors.
//
// Every wait is bounded.  A wait that runs out returns false; callers record
// an error code in the device status word and leave through their normal
// teardown path, so a protocol bug can never spin a GPU forever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nml_sm100 {

// ---- device status word -------------------------------------------------
// One word per device, written by kernels when a bounded wait gives up or an
// internal check fails.  Zero means healthy.
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusBarrierTimeout = 1,
  kStatusTmemAllocFailed = 2,
};

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
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
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait: a second or so at worst, far beyond any legitimate
// pipeline latency.  Returns false when it gives up.
constexpr uint32_t kWaitPolls = 1u << 20;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// ---- async-proxy fences ----------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA --------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// x is the innermost coordinate (elements); x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
        "r"(y)
      : "memory");
}

// 3-D tiled load; x is the innermost coordinate.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
        "r"(y), "r"(z)
      : "memory");
}

// ---- cp.async (LDGSTS) -------------------------------------------------------
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src)
               : "memory");
}

// 16-byte copy that writes zeros when `valid` is false (src-size 0).
__device__ __forceinline__ void cp_async_16_zfill(void* dst, const void* src, bool valid) {
  const uint32_t size = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
               "r"(size)
               : "memory");
}

// The barrier receives one arrival once all earlier cp.async of this thread
// have landed.  .noinc: the arrival is part of the barrier's expected count.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- tcgen05 ------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot_in_smem)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- thread-block clusters ---------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// Every thread of every CTA of the cluster; orders earlier writes before later reads.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of `local` (a shared-memory address of this CTA) in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}

__device__ __forceinline__ void cluster_store_f32x4(uint32_t remote, float a, float b, float c,
                                                    float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// Arrival on an mbarrier of another CTA of the cluster; releases this thread's earlier
// (remote) stores at cluster scope.
__device__ __forceinline__ void cluster_mbar_arrive(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar)
               : "memory");
}

// try_wait that acquires at cluster scope (pairs with cluster_mbar_arrive).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// ---- warp-uniform issue -------------------------------------------------------
// The forms below are executed by every lane of a converged warp; one elected lane issues
// the instruction.  Code that reaches a tcgen05.mma under `if (lane == 0)` is divergent to
// the compiler, which then moves every descriptor from vector to uniform registers again
// for each instruction: about 80 cycles of the issuing thread per MMA beside busy warps,
// against about 25 when the surrounding loop is uniform.
__device__ __forceinline__ void umma_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .pred pe;\n"
      "elect.sync _|pe, 0xffffffff;\n"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n"
      :
      : "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void umma_f16_elect(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred pe, pa;\n"
      "elect.sync _|pe, 0xffffffff;\n"
      "setp.ne.b32 pa, %4, 0;\n"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pa;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// A operand in tensor memory (lane = row of A, 32-bit column c = elements 2c and 2c + 1 of
// the K = 16 slice), B operand in shared memory.
__device__ __forceinline__ void umma_f16_tmem_a_elect(uint32_t tmem_d, uint32_t tmem_a,
                                                      uint64_t b_desc, uint32_t idesc,
                                                      uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred pe, pa;\n"
      "elect.sync _|pe, 0xffffffff;\n"
      "setp.ne.b32 pa, %4, 0;\n"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pa;\n"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Bounded wait with no result, so that the caller's control flow stays uniform.  When the
// polls run out it raises the CTA's abort flag and the BARRIER_TIMEOUT status bit; once the
// abort flag is up, by this or any other role, every later call returns at once, so the
// caller runs out its (bounded) loops on whatever data is there and the host sees the status.
__device__ __forceinline__ void mbar_wait_or_abort(uint64_t* bar, uint32_t parity,
                                                   volatile int* abort_flag, int* status,
                                                   int site) {
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .u32 n, f;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n"
      "@p bra WAIT_DONE;\n"
      "mov.u32 n, 0;\n"
      "WAIT_LOOP:\n"
      "ld.volatile.shared.u32 f, [%2];\n"
      "setp.ne.u32 q, f, 0;\n"
      "@q bra WAIT_DONE;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n"
      "@p bra WAIT_DONE;\n"
      "add.u32 n, n, 1;\n"
      "setp.lt.u32 q, n, %4;\n"
      "@q bra WAIT_LOOP;\n"
      "st.volatile.shared.u32 [%2], 1;\n"
      "red.global.or.b32 [%3], %5;\n"
      "WAIT_DONE:\n"
      "}\n"
      :
      : "r"(smem_u32(bar)), "r"(parity),
        "r"(smem_u32(const_cast<int*>(abort_flag))), "l"(status), "r"(kWaitPolls),
        "r"(1 | (0x100 << site))
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread L of the warp receives
// columns [c, c+32) of TMEM lane (lane_base + L).
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(address)
      : "memory");
}

__device__ __forceinline__ void tmem_load_32x16(uint32_t address, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(address)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Each thread writes 8 consecutive 32-bit columns of its own TMEM lane (the warp's lanes are
// 32 * (warp % 4) + lane; the address carries the warp's first lane).
__device__ __forceinline__ void tmem_store_32x8(uint32_t address, const uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      :
      : "r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
        "r"(v[6]), "r"(v[7])
      : "memory");
}

__device__ __forceinline__ void tmem_store_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// The same descriptor split in halves: only the low word (start address, leading offset)
// changes between operand tiles, so an issue loop keeps the high word constant.
constexpr uint32_t kUmmaDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);

__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_address) {
  return ((smem_address & 0x3ffffu) >> 4) | (1u << 16);
}

// Untiled bulk copy global -> shared; both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

enum UmmaFormat : uint32_t { kUmmaF16 = 0, kUmmaBF16 = 1 };

// Instruction descriptor for kind::f16: f32 accumulator, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t a_format, uint32_t b_format,
                                                      uint32_t m, uint32_t n) {
  return (1u << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace nml_sm100
