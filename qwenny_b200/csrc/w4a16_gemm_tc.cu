// W4A16 product for prompt-sized steps (more than 16 token rows) on the 5th-generation tensor cores: Y = X . W^T with
// W int4 in the reference's Marlin layout. Replaces marlin::mul<{1..4},16,4,*> (kernels/marlin.cuh:171-582,
// launched by Gemm::marlin, src/cuda/core.rs:569-612, for n > 16).
//
// The work is the list of (256-output x 256-token tile, k block of 64) pairs, tile after tile. Where whole tiles would
// leave the last wave mostly empty (160 tiles of the 5120-output matrices on 148 SMs are two waves), a persistent grid
// of one block per SM deals the list out in equal contiguous shares (stream-K): a block that ends or starts inside a
// tile writes that tile's partial accumulators to scratch and takes a ticket; the tile's last arriver adds the parts
// in block order and runs the epilogue, nobody waits. Otherwise a block is a tile. Per (tile, k block):
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
//               Y [token][output] f32, or silu(gate) * up as f16 for the interleaved SwiGLU matrices (or the partial
//               tile, see above); the copy warp fills the ring for the block's next tile meanwhile
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
constexpr int S_BYTES = 1024;               // 256 f16 scales, then (zero-point matrices) their 256 offsets (8 - z) * scale
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
    float* part;         // [grid][2][BT][BO] partial tiles: [.][0] a share's first tile begun by an earlier block, [.][1] its last, unfinished one
    int* tickets;        // one per tile, zero between launches
    long long iters;     // tiles x k blocks
    int zp;              // S holds a second table [K/128][N] after the scales: the offsets (8 - z) * scale of zero-point matrices
    int whole, tiles;    // whole = 1: block b takes the whole tiles b, b + grid, ... (grid = tiles: one each); 0: equal contiguous shares of the list
};

// the share of block b of a grid of g blocks: iterations [share_start(b), share_start(b + 1))
__device__ __forceinline__ long long share_start(long long iters, int g, int b) { return iters * b / g; }
__device__ __forceinline__ int share_of(long long iters, int g, long long it) {
    int b = (int)(it * g / iters);
    while (b + 1 < g && share_start(iters, g, b + 1) <= it) b++;
    while (b > 0 && share_start(iters, g, b) > it) b--;
    return b;
}

// A block's work as a list of segments (tile, k blocks [kb0, kb1)); every role of the block walks the same list.
// SHARES: equal contiguous shares of the (tile, k block) list; otherwise block b takes the whole tiles b, b + grid, ...
template <bool SHARES>
struct Walk {
    const Args& a;
    int nkb, G, b, j = 0;
    long long it, it1;
    __device__ Walk(const Args& a_, int nkb_, int G_, int b_) : a(a_), nkb(nkb_), G(G_), b(b_) {
        it = SHARES ? share_start(a.iters, G, b) : 0;
        it1 = SHARES ? share_start(a.iters, G, b + 1) : 0;
    }
    __device__ bool next(int& tile, int& kb0, int& kb1) {
        if (!SHARES) {
            tile = j * G + b; kb0 = 0; kb1 = nkb; j++;
            return tile < a.tiles;
        }
        if (it >= it1) return false;
        tile = (int)(it / nkb); kb0 = (int)(it % nkb); kb1 = (int)min((long long)nkb, kb0 + (it1 - it));
        it += kb1 - kb0;
        return true;
    }
    // the blocks that hold the parts of a tile cut by this walk: the first one and how many
    __device__ void parts_of(int tile, int& first, int& parts) const {
        first = share_of(a.iters, G, (long long)tile * nkb);
        parts = share_of(a.iters, G, (long long)(tile + 1) * nkb - 1) - first + 1;
    }
};

template <int EPI, bool SHARES>
__global__ void __launch_bounds__(THREADS, 1) w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles want 1 KB
    uint8_t* ctl = smem + NSTAGE * STAGE_BYTES;
    uint64_t* full = (uint64_t*)ctl;            // copies landed
    uint64_t* aready = full + NSTAGE;           // the dequantised A halves are written
    uint64_t* empty = aready + NSTAGE;          // the stage's MMAs are done
    uint64_t* done = empty + NSTAGE;            // all MMAs of a segment are done
    uint64_t* accfree = done + 1;               // the epilogue warps have read the segment's accumulators
    uint32_t* tmem_slot = (uint32_t*)(accfree + 1);
    int* flag = (int*)(tmem_slot + 1);          // this block finishes the tile (the ticket's answer, for warps 1-8)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = a.K / BK, ntn = a.N / BO, G = gridDim.x;
    Walk<SHARES> walk(a, nkb, G, blockIdx.x);
    int tile, kb0, kb1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&aready[i], DQ_WARPS);
            mbar_init(&empty[i], 1);
        }
        mbar_init(done, 1);
        mbar_init(accfree, DQ_WARPS);
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

    // Every role walks the block's share as the same list of segments (tile, k blocks [kb0, kb1)); `ring` counts the
    // stages of the whole share, so the ring's slots and phases run on from one segment to the next.
    if (warp == 0) {
        // ---------------------------------------------------------------- copies
        const uint64_t pol = policy_evict_first();
        bool ok = true;
        uint32_t ring = 0;  // (a block's share is far below 2^32 stages)
        while (ok && walk.next(tile, kb0, kb1)) {
            const int n0 = (tile % ntn) * BO, tok0 = (tile / ntn) * BT;
            for (int kb = kb0; kb < kb1 && ok; kb++, ring++) {
                const int s = (int)(ring % NSTAGE);
                if (ring >= NSTAGE) {
                    if (lane == 0) ok = mbar_wait(&empty[s], ((ring / NSTAGE) - 1) & 1);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                uint8_t* st = smem + s * STAGE_BYTES;
                if (lane == 0) {
                    mbar_expect_tx(&full[s], X_BYTES + W_BYTES + BO * 2 * (1 + a.zp));
                    tma_load_2d(st, &xmap, kb * BK, tok0, &full[s]);
                }
                __syncwarp();
                if (lane < 4) {  // k16 step `lane` of the k block: 256 outputs = 2 KB of words
                    const uint8_t* src = (const uint8_t*)a.B + ((size_t)(kb * 4 + lane) * 2 * a.N + (size_t)(n0 / 64) * 128) * 4;
                    bulk_g2s(st + X_BYTES + 2 * A_BYTES + lane * 2048, src, 2048, &full[s], pol);
                } else if (lane == 4) {
                    bulk_g2s(st + X_BYTES + 2 * A_BYTES + W_BYTES, a.S + (size_t)(kb / 2) * a.N + n0, BO * 2, &full[s], pol);
                } else if (lane == 5 && a.zp) {
                    bulk_g2s(st + X_BYTES + 2 * A_BYTES + W_BYTES + BO * 2, a.S + (size_t)(a.K / 128 + kb / 2) * a.N + n0, BO * 2,
                             &full[s], pol);
                }
            }
        }
        if (!ok && lane == 0) atomicExch(a.err, 5);
    } else if (warp <= DQ_WARPS) {
        // ---------------------------------------------------------------- dequantise into the swizzled A halves
        const int dw = warp - 1, ks = dw & 3, cpair = dw >> 2, g = lane >> 2, t = lane & 3;
        bool dead = false;
        uint32_t ring = 0;  // (a block's share is far below 2^32 stages)
        int seg = 0;
        for (; walk.next(tile, kb0, kb1); seg++) {
            const int n0 = (tile % ntn) * BO, tok0 = (tile / ntn) * BT;
            for (int kb = kb0; kb < kb1; kb++, ring++) {
                const int s = (int)(ring % NSTAGE);
                if (!dead) {
                    dead = !mbar_wait(&full[s], (ring / NSTAGE) & 1);
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
                    uint4 z4 = make_uint4(0u, 0u, 0u, 0u);               // their offsets (0: the symmetric form)
                    if (a.zp) z4 = *(const uint4*)(ssm + BO + c64 * 64 + 8 * g);
                    const uint32_t wq[4] = {w4.x, w4.y, w4.z, w4.w};
                    const __half* sh = (const __half*)&s4;
                    const __half* zh = (const __half*)&z4;
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
                        const __half2 z0 = __half2half2(zh[2 * b]), z1 = __half2half2(zh[2 * b + 1]);
                        // (q - 8) * scale + offset, rounded once (scale_z, kernels/marlin.cuh:126-133); with offset 0 the
                        // symmetric form's product
                        __half2 r0 = __hfma2(__hsub2(*(__half2*)&lo0, *(const __half2*)&SUB_LO), s0, z0);  // row g,   k 2t
                        __half2 r1 = __hfma2(__hsub2(*(__half2*)&lo1, *(const __half2*)&SUB_LO), s1, z1);  // row g+8, k 2t
                        __half2 r2 = __hfma2(__hsub2(*(__half2*)&hi0, *(const __half2*)&SUB_HI), s0, z0);  // row g,   k 2t+8
                        __half2 r3 = __hfma2(__hsub2(*(__half2*)&hi1, *(const __half2*)&SUB_HI), s1, z1);  // row g+8, k 2t+8
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

            // ------------------------------------------------------------ the segment's accumulators
            if (!dead) {
                dead = !mbar_wait(done, (uint32_t)seg & 1);
                if (dead && lane == 0) atomicExch(a.err, 8);
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // a warp may only read the 32 tensor-memory lanes of its quarter (warp id % 4)
            const int q = warp & 3, half_i = (warp - 1) >> 2, lrow = half_i * 128 + q * 32 + lane, orow = n0 + lrow;
            const uint32_t tbase = tmem + ((uint32_t)(q * 32) << 16) + half_i * BT;
            int parts = 1, first = 0;
            bool finish = !dead;
            if (SHARES && (kb0 > 0 || kb1 < nkb)) {
                // a part of the tile: store it, take the tile's ticket; the last arriver finishes the tile
                walk.parts_of(tile, first, parts);
                float* slot = a.part + ((size_t)blockIdx.x * 2 + (kb0 == 0 ? 1 : 0)) * (BT * BO);
                if (!dead) {
#pragma unroll 1
                    for (int c = 0; c < BT; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(tbase + c, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; j++) slot[(size_t)(c + j) * BO + lrow] = __uint_as_float(v[j]);
                    }
                }
                __threadfence();
                named_bar_sync(1, DQ_WARPS * 32);
                if (threadIdx.x == 32) {
                    const int tk = atomicAdd(&a.tickets[tile], 1);
                    *flag = tk == parts - 1;
                    if (tk == parts - 1) a.tickets[tile] = 0;
                }
                named_bar_sync(1, DQ_WARPS * 32);
                finish = *flag != 0 && !dead;
                named_bar_sync(1, DQ_WARPS * 32);  // (the flag may be rewritten by the next segment)
                if (finish) __threadfence();
            }
            if (finish) {
                const int mine = blockIdx.x - first;
#pragma unroll 1
                for (int c = 0; c < BT; c += 32) {
                    uint32_t v[32];
                    if (!SHARES || parts <= 2) {
                        tmem_ld32(tbase + c, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                        if (SHARES && parts == 2) {  // own + other = other + own: no order to keep
                            const float* o = a.part + ((size_t)(first + 1 - mine) * 2 + (mine == 1 ? 1 : 0)) * (BT * BO);
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(o + (size_t)(c + j) * BO + lrow));
                        }
                    } else {  // more parts: all of them from scratch, in block order
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = 0;
                        for (int p = 0; p < parts; p++) {
                            const float* o = a.part + ((size_t)(first + p) * 2 + (p == 0 ? 1 : 0)) * (BT * BO);
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(o + (size_t)(c + j) * BO + lrow));
                        }
                    }
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
            // the accumulator columns may be overwritten by the next segment's first MMA
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accfree);
        }
    } else {
        // ---------------------------------------------------------------- MMA issue (one elected lane)
        bool ok = true;
        uint32_t ring = 0;  // (a block's share is far below 2^32 stages)
        int seg = 0;
        for (; ok && walk.next(tile, kb0, kb1); seg++) {
            if (seg > 0) {  // the epilogue warps have read the previous segment's accumulators
                if (lane == 0) ok = mbar_wait(accfree, (uint32_t)(seg - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            for (int kb = kb0; kb < kb1 && ok; kb++, ring++) {
                const int s = (int)(ring % NSTAGE);
                if (lane == 0) ok = mbar_wait(&aready[s], (ring / NSTAGE) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const uint32_t xb = smem_u32(smem + s * STAGE_BYTES), ab = xb + X_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; k16++) {
                        const uint64_t bd = smem_desc(xb + k16 * 32);
                        const uint32_t acc = (kb > kb0 || k16 > 0) ? 1u : 0u;
                        umma(tmem, smem_desc(ab + k16 * 32), bd, acc);
                        umma(tmem + BT, smem_desc(ab + A_BYTES + k16 * 32), bd, acc);
                    }
                    umma_commit(&empty[s]);  // arrives when the MMAs issued so far have read their operands
                }
                __syncwarp();
            }
            if (lane == 0 && ok) umma_commit(done);
            __syncwarp();
        }
        if (!ok && lane == 0) atomicExch(a.err, 7);
        __syncwarp();
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


// Y = X . W^T for m > 16 rows: plain (f32 [m][n]) or SwiGLU (f16 [m][n/2]). X f16 [.][k], rows row0 .. row0 + m - 1.
int qb_gemm_tc_launch(qb_ctx* ctx, cudaStream_t st, const void* X, const void* B, void* Y, const void* S, int m, int n,
                      int k, int row0, int epi, int zp) {
    if (n % tc::BO || k % 128 || m < 1) return QB_ERR_ARG;
    qb::EncodeTiled enc = qb::encode_tiled();
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
    const long long tiles = (long long)(n / tc::BO) * ((m + tc::BT - 1) / tc::BT);
    if (tiles > QB_TC_TICKETS) return QB_ERR_ARG;
    if (!ctx->tc_part) {
        // partial tiles of the stream-K shares (two per block) and the tiles' tickets, taken with the first product
        QB_CUDA(cudaMalloc(&ctx->tc_part, (size_t)ctx->sms * 2 * tc::BT * tc::BO * sizeof(float)));
        QB_CUDA(cudaMalloc(&ctx->tc_tickets, QB_TC_TICKETS * sizeof(int)));
        QB_CUDA(cudaMemset(ctx->tc_tickets, 0, QB_TC_TICKETS * sizeof(int)));
    }
    tc::Args a;
    a.B = (const uint32_t*)B; a.S = (const __half*)S; a.Y = Y; a.m = m; a.N = n; a.K = k; a.row0 = row0; a.err = ctx->err;
    a.zp = zp ? 1 : 0; a.part = ctx->tc_part; a.tickets = ctx->tc_tickets; a.iters = tiles * (k / tc::BK);
    // One block per tile (the hardware hands a freed SM the next tile) when the partly filled last wave wastes
    // less than a fifth of the time; otherwise one block per SM and equal shares of the whole list, where a tile has
    // two parts, seldom three. Measured at 2048 rows: 16384 x 5120 (3.46 waves) 298 us as tiles, 312 us as shares;
    // 5120 x 17408 (160 tiles, 1.08 waves) 445 us as tiles, 310 us as shares; 14336 x 5120 (3.03 waves) 273 us as shares.
    const double waves = (double)tiles / ctx->sms;
    a.tiles = (int)tiles;
    a.whole = ((long long)(waves + 0.999999) < 1.2 * waves) ? 1 : 0;
    if (ctx->tune_ctas == 1000) a.whole = 0;  // measurement: shares whatever the shape
    if (ctx->tune_ctas == 1001) a.whole = 1;  //              tiles whatever the shape
    const int G = a.whole ? (int)tiles : (int)(a.iters < ctx->sms ? a.iters : ctx->sms);
    dim3 grid((unsigned)G);
    if (epi == QB_EPI_SILU)
        return a.whole ? launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_SILU_TC, false>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a)
                       : launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_SILU_TC, true>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a);
    return a.whole ? launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_PLAIN_TC, false>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a)
                   : launch(ctx, tc::w4a16_gemm_tc_kernel<tc::EPI_PLAIN_TC, true>, grid, dim3(tc::THREADS), tc::SMEM_BYTES, st, map, a);
}
