// Device helpers shared by the sm_100a kernels: mbarrier + bulk-copy (TMA) wrappers, mma.sync, warp reductions,
// the order-preserving float key of the argmax epilogue, programmatic-dependent-launch controls.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace qb {

// ---------------------------------------------------------------- model constants (the 27B build of the reference:
// kernels/qwen.cu:8-35 with QWEN_27B, kernels/qwen_deltanet.cuh:21-34)
constexpr int H = 5120;
constexpr int NH = 24, NKV = 4, HD = 256, GROUP = NH / NKV, ROT = 64;
constexpr int QG_ROWS = 2 * NH * HD;               // q_proj rows: per head [q; gate]
constexpr int ATTN_IN = QG_ROWS + 2 * NKV * HD;    // 14336
constexpr int LK_HEADS = 16, LV_HEADS = 48, LKD = 128, LVD = 128;
constexpr int LQKV = 2 * LK_HEADS * LKD + LV_HEADS * LVD;  // 10240 conv channels
constexpr int DELTA_IN = LQKV + LV_HEADS * LVD;             // 16384
constexpr int CONV_K = 4;
constexpr int MIX = NH * HD;  // 6144 (== LV_HEADS * LVD)
constexpr int FF = 17408;
constexpr float EPS = 1e-6f;
// DeltaNet slot memory (kernels/qwen_deltanet.cuh:21-34)
constexpr int CR = 32, KEEP = 16, META = 4;
constexpr int REP = LK_HEADS * LKD + LV_HEADS * LVD + 2 * LV_HEADS;  // 8288
constexpr int SLOT_STATE = LV_HEADS * LVD * LKD;
constexpr int SLOT_BANK = KEEP * REP;
constexpr int SLOT_RING = 2 * SLOT_STATE + 2 * SLOT_BANK;
constexpr int CVW = LQKV + 2 * LV_HEADS;  // 10336

// Every bounded wait gives up after this many polls (each poll may itself suspend for a hardware-chosen time), sets
// the error word and lets the kernel drain: nothing here can spin forever.
constexpr uint32_t WAIT_LIMIT = 1u << 22;

// ---------------------------------------------------------------- small math
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result. sh: one float per warp (32 at most).
__device__ __forceinline__ float block_sum(float v, float* sh) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    v = warp_sum(v);
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = lane < (int)(blockDim.x >> 5) ? sh[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

// Order-preserving map float -> u32, and the argmax key (value, ~index): a 64-bit max picks the largest logit and,
// among equal ones, the lowest index (kernels/common.cuh:60-63, kernels/gemm.cuh:71-74 of the reference).
__device__ __forceinline__ unsigned ordered(float v) {
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    return ((unsigned long long)ordered(v) << 32) | (0xffffffffu - (uint32_t)i);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *(uint32_t*)&h;
}

// ---------------------------------------------------------------- tensor cores (legacy warp-level path; the
// skinny products have 1..16 token rows, far below a tcgen05 tile, and are HBM bound)
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// d = a . b (no accumulator input: the zeros are immediates, not registers to clear)
__device__ __forceinline__ void mma16816_zero(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ldmatrix: four 8x8 b16 matrices; lane i gives the shared address of row i % 8 of matrix i / 8
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// ---------------------------------------------------------------- mbarriers, bulk copies

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out (the caller records it and drains).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
// 1-D bulk async copy global -> shared (the TMA engine without a tensor map): both addresses 16-byte aligned, size
// a multiple of 16; completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
            "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}

// ---------------------------------------------------------------- per-thread asynchronous copies (Ampere-style)
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// ---------------------------------------------------------------- programmatic dependent launch
// wait: blocks until the grids this launch depends on have completed and their writes are visible (a no-op for a
// launch without the attribute). launch_dependents: lets the next kernel in the stream start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All non-exited threads of the cluster arrive and wait (release / acquire: shared-memory writes before it are
// visible to the cluster's other blocks after it).
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The two halves separately: arrive as soon as this block is done with the others' memory, wait where their answer is
// needed (work in between overlaps the barrier)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// The address of this block's shared location `p` in block `rank` of the cluster, and a 128-bit load from there
__device__ __forceinline__ uint32_t cluster_map(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 cluster_ld4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------- global loads that bypass L1 (data another CTA
// wrote during this kernel)
__device__ __forceinline__ float4 ld_cg4(const float4* p) { return __ldcg(p); }

}  // namespace qb
