// tc_ptx.cuh — inline-PTX wrappers for the sm_100a features the attention kernels use: mbarriers
// with bounded waits, TMA tile loads, tensor-memory allocation / load / store, tcgen05.mma issue
// and commit, and the shared-memory and instruction descriptors of the 5th-generation tensor cores.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hc {
namespace {

constexpr int kTcThreads = 512;          // 16 warps: four warpgroups
constexpr int kRows = 128;               // query rows per CTA (MMA M)
constexpr unsigned long long kWaitCycles = 3000000000ull;   // ~1.5 s at 1.9 GHz

// ---- PTX wrappers ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// The same with a suspend-time hint: the hardware may park the warp for up to `ns` nanoseconds
// instead of returning at once, so a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return done != 0;
}
// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out of time).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
        if (mbar_try_wait_parked(bar, parity, 2000)) return true;
        __nanosleep(64);      // a waiting warp that polls flat out takes issue slots from the working ones
        if (*abort_flag != 0) return false;
        if (static_cast<unsigned long long>(clock64() - start) > kWaitCycles) {
            *abort_flag = 1;
            atomicCAS(status_word, 0, 0x100 + where);
            return false;
        }
    }
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 16 bytes global -> shared without passing through registers; `bytes` = 16 copies, 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(chosen));
    return chosen != 0;
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Register reallocation between warpgroups (all four warps of a warpgroup execute it together).
template <int N>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
// Named barrier over `threads` threads (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t v;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr) : "memory");
    return v;
}

#define HC_TMEM_LD32(taddr, v)                                                                              \
    asm volatile(                                                                                           \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                           \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                          \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"          \
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),  \
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),         \
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),       \
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),       \
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])                                                             \
        : "r"(taddr) : "memory")

// 16 lanes x 256 bits, eight times along the columns: 16 rows x 64 columns.  Thread i of the warp
// gets, for n = 0..7, v[4n], v[4n+1] = row i/4, columns 8n + 2(i%4) + {0, 1} and v[4n+2], v[4n+3] =
// row i/4 + 8, the same columns (the layout of an m16n8 accumulator fragment).
#define HC_TMEM_LD_16x256b_x8(taddr, v)                                                                     \
    asm volatile(                                                                                           \
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "                                                           \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                          \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"          \
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),  \
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),         \
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),       \
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),       \
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])                                                             \
        : "r"(taddr) : "memory")

// 16 lanes x 128 bits, eight times along the columns: 16 rows x 32 columns.  Thread i holds, for
// n = 0..7, v[2n] = row i/4, column 4n + i%4 and v[2n+1] = row i/4 + 8, the same column: the packed
// bf16 pair of the two fp32 columns the 16x256b load gave that thread.
#define HC_TMEM_ST_16x128b_x8(taddr, v)                                                                     \
    asm volatile(                                                                                           \
        "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "                                                     \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                          \
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),         \
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),     \
          "r"(v[15]) : "memory")

#define HC_TMEM_ST16(taddr, v)                                                                              \
    asm volatile(                                                                                           \
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                     \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                          \
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),         \
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),     \
          "r"(v[15]) : "memory")

// ---- descriptors ----------------------------------------------------------------------------------

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).  Addresses and offsets in
// units of 16 bytes.  K-major operands: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO).
// MN-major operands (V): the same rows, and 64-element column blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t desc = 0;
    desc |= uint64_t((addr & 0x3FFFF) >> 4);
    desc |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
    desc |= uint64_t((1024 >> 4) & 0x3FFF) << 32;
    desc |= uint64_t(1) << 46;             // descriptor version
    desc |= uint64_t(2) << 61;             // SWIZZLE_128B
    return desc;
}
// Instruction descriptor: bf16 x bf16 -> f32, M = 128, N = n; B MN-major when b_mn is set.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) |
           (uint32_t(kRows >> 4) << 24);
}

}  // namespace
}  // namespace hc
