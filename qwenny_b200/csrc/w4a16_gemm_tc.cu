// W4A16 product for prompt-sized steps (more than 16 token rows) on the 5th-generation tensor cores: Y = X . W^T with
// W int4 in the reference's Marlin layout. Replaces marlin::mul<{1..4},16,4,*> (kernels/marlin.cuh:171-582,
// launched by Gemm::marlin, src/cuda/core.rs:569-612, for n > 16).
//
// A block owns a 256-output x 256-token tile and walks k in blocks of 64:
//   warp 0      copies: the block's Marlin words (4 bulk copies of 2 KB), its group scales, and the X tile as one
//               tensor-map TMA load (box 64 k x 256 tokens, 128-byte swizzle) per stage; full/empty mbarriers
//   warps 1-8   dequantise: each lane's Marlin word holds outputs {g, g+8} x columns {2t, 2t+1, 2t+8, 2t+9} of a
//               16 x 16 block; lop3 / hsub2 to q - 8, hmul2 by the f16 group scale (the reference's rounding:
//               w = f16((q - 8) s), kernels/marlin.cuh:100-124), and four 4-byte stores per word put it where
//               tcgen05 expects a K-major operand with the 128-byte swizzle (8-row groups of 1 KB, 16-byte chunk c of
//               row r at chunk c ^ (r % 8)); a warp's 32 stores of one instruction fall on 32 distinct banks
//   warp 9      one elected lane issues tcgen05.mma kind::f16, M = 128 (two halves of the 256 outputs), N = 256
//               tokens, K = 16 per instruction, accumulating f32 in tensor memory (2 x 256 columns), and
//               tcgen05.commit hands each stage back to the copy warp when its MMAs have read it
//   epilogue    warps 1-8 read the accumulators with tcgen05.ld (32 lanes x 32 columns per instruction) and write
//               Y [token][output] f32, or silu(gate) * up as f16 for the interleaved SwiGLU matrices
// Weights are the A operand, so one dequantised tile serves 256 tokens; a 2048-token chunk re-dequantises each weight
// 8 times (once per token tile), which the 8 dequant warps hide behind the MMAs.
#include <cuda.h>
#include "common.cuh"
#include "launch.h"

namespace qb {

namespace tc {

enum { EPI_PLAIN_TC = 0, EPI_SILU_TC = 1 };
constexpr int BO = 256;             // outputs per block (two M = 128 accumulators)
constexpr int BT = 256;             // tokens per block (the MMA's N)
constexpr int BK = 64;              // k per stage: one 128-byte swizzle row of f16
constexpr int NSTAGE = 3;
constexpr int X_BYTES = BT * BK * 2;        // 32 KB
constexpr int A_BYTES = 128 * BK * 2;       // 16 KB per accumulator half
constexpr int W_BYTES = BO * BK / 2;        // 8 KB of Marlin words
constexpr int S_BYTES = 1024;               // 256 f16 scales, padded
constexpr int STAGE_BYTES = X_BYTES + 2 * A_BYTES + W_BYTES + S_BYTES;  // 73 KB
constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + 1024 /* barriers, tmem address */ + 1024 /* alignment slack */;
constexpr int DQ_WARPS = 8;
constexpr int THREADS = (1 + DQ_WARPS + 1) * 32;
constexpr int TMEM_COLS = 512;

// instruction descriptor of tcgen05.mma kind::f16: D f32 (bits 4-5 = 1), A and B f16 (0), both K-major (0),
// N >> 3 at bits 17-22, M >> 4 at bits 24-28
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

// shared-memory matrix descriptor of a K-major operand with the 128-byte swizzle: start address >> 4, leading byte
// offset 1 (unused with a swizzle), stride byte offset 1024 >> 4 (between 8-row groups), descriptor version 1
// (bit 46), layout type 2 = SWIZZLE_128B (bits 61-63)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
            "r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
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

struct Args {
    const uint32_t* B;   // Marlin words [K/16][2N]
    const __half* S;     // scales [K/128][N]
    void* Y;             // plain: f32 [.][N]; silu: f16 [.][N/2]; rows row0 ..
    int m, N, K, row0;
    int* err;
};

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1) w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1 KB
    uint8_t* ctl = smem + NSTAGE * STAGE_BYTES;
    uint64_t* full = (uint64_t*)ctl;            // copies landed
    uint64_t* aready = full + NSTAGE;           // the dequantised A halves are written
    uint64_t* empty = aready + NSTAGE;          // the stage's MMAs are done
    uint64_t* done = empty + NSTAGE;            // all MMAs are done
    uint32_t* tmem_slot = (uint32_t*)(done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BO, tok0 = blockIdx.y * BT, nkb = a.K / BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&aready[i], DQ_WARPS);
            mbar_init(&empty[i], 1);
        }
        mbar_init(done, 1);
        mbar_fence_init();
    }
    if (warp == DQ_WARPS + 1) {  // the MMA warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- copies
        const uint64_t pol = policy_evict_first();
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % NSTAGE;
            if (kb >= NSTAGE) {
                if (lane == 0) ok = mbar_wait(&empty[s], ((kb / NSTAGE) - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            uint8_t* st = smem + s * STAGE_BYTES;
            if (lane == 0) {
                mbar_expect_tx(&full[s], X_BYTES + W_BYTES + BO * 2);
                tma_load_2d(st, &xmap, kb * BK, tok0, &full[s]);
            }
            __syncwarp();
            if (lane < 4) {  // k16 step `lane` of the k block: 256 outputs = 2 KB of words
                const uint8_t* src = (const uint8_t*)a.B + ((size_t)(kb * 4 + lane) * 2 * a.N + (size_t)(n0 / 64) * 128) * 4;
                bulk_g2s(st + X_BYTES + 2 * A_BYTES + lane * 2048, src, 2048, &full[s], pol);
            } else if (lane == 4) {
                bulk_g2s(st + X_BYTES + 2 * A_BYTES + W_BYTES, a.S + (size_t)(kb / 2) * a.N + n0, BO * 2, &full[s], pol);
            }
        }
        if (!ok && lane == 0) atomicExch(a.err, 5);
    } else if (warp <= DQ_WARPS) {
        // ---------------------------------------------------------------- dequantise into the swizzled A halves
        const int dw = warp - 1, ks = dw & 3, cpair = dw >> 2, g = lane >> 2, t = lane & 3;
        bool dead = false;
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % NSTAGE;
            if (!dead) {
                dead = !mbar_wait(&full[s], (kb / NSTAGE) & 1);
                if (dead && lane == 0) atomicExch(a.err, 6);
            }
            uint8_t* st = smem + s * STAGE_BYTES;
            const uint4* wsm = (const uint4*)(st + X_BYTES + 2 * A_BYTES);  // [ks 4][c64 4][lane 32] x 4 words
            const __half* ssm = (const __half*)(st + X_BYTES + 2 * A_BYTES + W_BYTES);
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const int c64 = cpair * 2 + cc;
                uint4 w4 = wsm[(ks * 4 + c64) * 32 + lane];
                uint4 s4 = *(const uint4*)(ssm + c64 * 64 + 8 * g);  // scales of outputs 16 b + g + 8 h at 2 b + h
                const uint32_t wq[4] = {w4.x, w4.y, w4.z, w4.w};
                const __half* sh = (const __half*)&s4;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    uint32_t q = wq[b], lo0, hi0, lo1, hi1;
                    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;\n" : "=r"(lo0) : "r"(q));
                    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;\n" : "=r"(hi0) : "r"(q));
                    uint32_t q8 = q >> 8;
                    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;\n" : "=r"(lo1) : "r"(q8));
                    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;\n" : "=r"(hi1) : "r"(q8));
                    const uint32_t SUB_LO = 0x64086408u, SUB_HI = 0x54805480u;
                    const __half2 s0 = __half2half2(sh[2 * b]), s1 = __half2half2(sh[2 * b + 1]);
                    __half2 r0 = __hmul2(__hsub2(*(__half2*)&lo0, *(const __half2*)&SUB_LO), s0);  // row g,   k 2t
                    __half2 r1 = __hmul2(__hsub2(*(__half2*)&lo1, *(const __half2*)&SUB_LO), s1);  // row g+8, k 2t
                    __half2 r2 = __hmul2(__hsub2(*(__half2*)&hi0, *(const __half2*)&SUB_HI), s0);  // row g,   k 2t+8
                    __half2 r3 = __hmul2(__hsub2(*(__half2*)&hi1, *(const __half2*)&SUB_HI), s1);  // row g+8, k 2t+8
                    // output row in the block: 64 c64 + 16 b + g (+ 8); A half row / 128, row inside it % 128
                    const int row = c64 * 64 + b * 16 + g, half_i = row >> 7, r = row & 127;
                    uint8_t* abase = st + X_BYTES + half_i * A_BYTES + (r >> 3) * 1024;
                    // rows r and r + 8 share r % 8 = g; 16-byte chunk (k / 8) of a row sits at chunk ^ (r % 8)
                    const int c0 = (2 * ks) ^ g, c1 = (2 * ks + 1) ^ g;
                    *(__half2*)(abase + g * 128 + c0 * 16 + 4 * t) = r0;
                    *(__half2*)(abase + 1024 + g * 128 + c0 * 16 + 4 * t) = r1;
                    *(__half2*)(abase + g * 128 + c1 * 16 + 4 * t) = r2;
                    *(__half2*)(abase + 1024 + g * 128 + c1 * 16 + 4 * t) = r3;
                }
            }
            // generic-proxy stores -> visible to the tensor core's async proxy, then tell the MMA warp
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&aready[s]);
        }
    } else {
        // ---------------------------------------------------------------- MMA issue (one elected lane)
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % NSTAGE;
            if (lane == 0) ok = mbar_wait(&aready[s], (kb / NSTAGE) & 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                const uint32_t xb = smem_u32(smem + s * STAGE_BYTES), ab = xb + X_BYTES;
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; k16++) {
                    const uint64_t bd = smem_desc(xb + k16 * 32);
                    const uint32_t acc = (kb > 0 || k16 > 0) ? 1u : 0u;
                    umma(tmem, smem_desc(ab + k16 * 32), bd, acc);
                    umma(tmem + BT, smem_desc(ab + A_BYTES + k16 * 32), bd, acc);
                }
                umma_commit(&empty[s]);  // arrives when the MMAs issued so far have read their operands
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (ok) umma_commit(done);
            else atomicExch(a.err, 7);
        }
        __syncwarp();
    }

    // -------------------------------------------------------------------- epilogue: warps 1-8 read the accumulators
    if (warp >= 1 && warp <= DQ_WARPS) {
        bool ok = mbar_wait(done, 0);
        if (!ok && lane == 0) atomicExch(a.err, 8);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (ok) {
            // a warp may only read the 32 tensor-memory lanes of its quarter (warp id % 4)
            const int q = warp & 3, half_i = (warp - 1) >> 2, orow = n0 + half_i * 128 + q * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BT; c += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + half_i * BT + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (EPI == EPI_SILU_TC) {
                    // packed rows 16 p + i are gate rows, 16 p + 8 + i their up rows: the up value sits 8 lanes on
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float gate = __uint_as_float(v[j]);
                        float up = __shfl_down_sync(0xffffffffu, gate, 8);
                        int tok = tok0 + c + j;
                        if ((lane & 8) == 0 && tok < a.m)
                            ((__half*)a.Y)[(size_t)(a.row0 + tok) * (a.N / 2) + (orow >> 4) * 8 + (orow & 7)] =
                                __float2half_rn(silu(gate) * up);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        int tok = tok0 + c + j;
                        if (tok < a.m) ((float*)a.Y)[(size_t)(a.row0 + tok) * a.N + orow] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == DQ_WARPS + 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

}  // namespace tc

}  // namespace qb

using namespace qb;

namespace {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

}  // namespace

// Y = X . W^T for m > 16 rows: plain (f32 [m][n]) or SwiGLU (f16 [m][n/2]). X f16 [.][k], rows row0 .. row0 + m - 1.
int qb_gemm_tc_launch(qb_ctx* ctx, cudaStream_t st, const void* X, const void* B, void* Y, const void* S, int m, int n,
                      int k, int row0, int epi) {
    if (n % tc::BO || k % 128 || m < 1) return QB_ERR_ARG;
    EncodeTiled enc = encode_tiled();
    if (!enc) return QB_ERR_UNSUPPORTED;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {tc::BK, tc::BT};
    const cuuint32_t estr[2] = {1, 1};
    void* base = (void*)((const __half*)X + (size_t)row0 * k);
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return QB_ERR_ARG;
    tc::Args a;
    a.B = (const uint32_t*)B; a.S = (const __half*)S; a.Y = Y; a.m = m; a.N = n; a.K = k; a.row0 = row0; a.err = ctx->err;
    dim3 grid(n / tc::BO, (m + tc::BT - 1) / tc::BT);
    if (epi == QB_EPI_SILU)
        return launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_SILU_TC>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a);
    return launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_PLAIN_TC>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a);
}
