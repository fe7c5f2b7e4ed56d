// What the attention kernels on the 5th-generation tensor cores share: instruction and shared-memory descriptors, the
// tcgen05 product / commit / tensor-memory load and store wrappers, the exact int8 -> f16 conversion of cache bytes,
// the 128-byte swizzle of a K-major tile, and bounded waits that sleep instead of polling.
#pragma once
#include "attn_common.cuh"

namespace qb {
namespace tc {

// kind::f16 with f32 accumulation, A and B K-major f16, M = 128 rows, N = n columns
constexpr uint32_t idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate)
        : "memory");
}
// the same product with A read from tensor memory (lane = row, f16 pairs along the columns)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(id), "r"(accumulate)
        : "memory");
}
// Four such products in one statement, over four consecutive 16-wide steps of the inner dimension: A columns a, a + 8,
// a + 16, a + 24 and B 32 bytes further along its 128-byte rows each time; the first overwrites the accumulator where
// `accumulate` is 0. The issuing thread spends two additions per product instead of rebuilding a descriptor and a
// predicate: with a thread-side cost of some 100 cycles per product the tensor core waits for the issue, not for data
// (measured: 112 cycles per product issued one by one from a loop, 52 in blocks like this; the products themselves
// take 47 (N <= 64) to 64 cycles (N 128)).
__device__ __forceinline__ void umma_ts4(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, t;\n"
        ".reg .b32 a1;\n"
        ".reg .b64 b1;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.eq.b32 t, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "add.u32 a1, %1, 8;\n"
        "add.u64 b1, %2, 2;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n"
        "add.u32 a1, %1, 16;\n"
        "add.u64 b1, %2, 4;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n"
        "add.u32 a1, %1, 24;\n"
        "add.u64 b1, %2, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(id), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
        "%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void async_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// two code bytes of a cache word -> two halves of their signed values, exactly: 1024 + (q + 128) by prmt, minus 1152
__device__ __forceinline__ uint32_t exact2(uint32_t w, uint32_t sel) {
    const uint32_t off = 0x64806480u;
    uint32_t v = __byte_perm(w, 0x64646464u, sel);
    __half2 r = __hsub2(*(__half2*)&v, *(const __half2*)&off);
    return *(uint32_t*)&r;
}

// byte offset of (row, 16-byte chunk) in a K-major tile with the 128-byte swizzle: 8-row groups of 1 KB
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// try_wait with a suspend-time hint: the waiting thread sleeps until the phase completes or the hint (ns) runs out,
// instead of spending issue slots on polls
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_sleepy(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (WAIT_LIMIT >> 4); i++)
        if (mbar_try_wait_hint(bar, parity, 2000)) return true;
    return false;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// A bounded wait that remembers failure: once a wait ran out the role stops waiting and walks on
struct Waiter {
    int* err;
    int code;
    bool dead = false;
    __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, int lane) {
        if (dead) return;
        bool ok = true;
        if (lane == 0) ok = mbar_wait_sleepy(bar, parity);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
            dead = true;
            if (lane == 0) atomicExch(err, code);
        }
    }
};

}  // namespace tc
}  // namespace qb
