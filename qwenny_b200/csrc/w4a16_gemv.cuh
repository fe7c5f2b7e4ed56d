// W4A16 skinny matrix product for decode / verify steps (1..16 token rows): Y = X . W^T with W int4 (symmetric,
// groups of 128 columns, f16 scales) in the reference's Marlin layout, X f16, f32 accumulation.
//
// Replaces marlin::mul<1,8,8,*> (kernels/marlin.cuh:171-582 of the reference) for steps of up to 16 tokens. It is a
// bandwidth-bound GEMV, organised around the HBM stream rather than around the tensor pipe:
//  * a producer warp streams the weights with three tensor-map loads per stage (cp.async.bulk.tensor.2d: words,
//    scales, X rows; plain bulk copies where a box does not fit: 512-output tiles, gathered rows)
//    into a ring of shared-memory stages; a stage is TN = 64 CG outputs x TK = 128 KG columns of packed int4
//    (4 KB per consumer warp), its group scales and the matching slice of X; full/empty mbarriers, no __syncthreads
//    in the stream;
//  * consumer warp (cg, kg) owns 64 outputs x one scale group of the stage. The Marlin word of lane (g, t) holds
//    outputs {g, g + 8} x columns {2t, 2t+1, 2t+8, 2t+9} of a 16-output block: exactly the A fragment of
//    mma.m16n8k16 when the WEIGHTS are the A operand and the tokens the n = 8 side, so the nibbles go from one
//    128-bit shared load through one shift and four ands straight into the tensor core as f16 subnormals
//    (n * 2^-24), no shuffles, no re-layout, no subtraction: the offset of 8 leaves through one extra mma per k16
//    step. The group scale (times 2^24) is applied in f32 to the group's partial sum (exact, and 8x fewer
//    multiplies than scaling every weight);
//  * two ways to deal the work. Matrices whose column blocks x k splits fit one wave of blocks run CLUSTERED: one
//    thread-block cluster per column block, rank r takes the r-th equal share of its k stages, and the ranks' f32
//    partials meet in rank 0 through distributed shared memory (no global traffic, no fences), added in rank order.
//    (With 64 x 1024 tiles and as many block slots as column blocks the cluster is one block: its eight warps' k
//    groups add up in shared memory and nothing crosses blocks.) Larger matrices run STREAM-K:
//  * the stages of the whole matrix, numbered column block by column block, are cut into one equal contiguous
//    range per block of a persistent grid (stream-K), so every SM streams the same number of bytes whatever the
//    shape and the copy pipeline never drains between column blocks. The KG warps of a column group add up in
//    shared memory in a fixed order; a column block that several blocks share gets their f32 partials in an
//    L2-resident scratch, and the LAST block to arrive (an atomic ticket, no waiting) adds them in k order and runs
//    the epilogue. Every sum has a fixed order that depends on the shape and the grid alone, never on the number of
//    rows or on timing: a row's result is bit-identical alone or next to drafts.
// Epilogues as the reference's: plain f32 [m][n]; SwiGLU of interleaved gate/up blocks -> f16 [m][n/2]
// (kernels/marlin.cuh:472-498); plain + argmax keys over the first n_valid outputs (:499-517).
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace qb {

enum { EPI_PLAIN = 0, EPI_SILU = 1, EPI_ARGMAX = 2 };

// tensor maps of the weights ([K/16] rows of N 8-byte elements) and of the scale table(s) ([K/128 (x 2)] rows of N halves)
// and of the step's X rows when they are contiguous ([m] rows of K/4 8-byte elements; the box is XROW halves wide, so
// the rows land in shared memory with the pad the ldmatrix reads want; the last k tile's pad reads past the row: zeros)
struct GemvMaps {
    CUtensorMap w, s, x;
};

__device__ __forceinline__ void tma_tile_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n" ::
            "r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}

// the copy engine reads a tensor map's 128 bytes before its first copy through it: asking for them at the kernel's very
// start takes that round trip off the first stage
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

struct GemvArgs {
    const __half* X;      // [rows][K] f16
    const int* xrows;     // X row of token t (null: row0 + t)
    const uint32_t* B;    // Marlin words [K/16][2N]
    const __half* S;      // scales [K/128][N], permuted per 64 outputs
    void* Y;              // plain/argmax: f32 [.][N]; silu: f16 [.][N/2]; rows row0 .. row0 + m - 1
    int m, N, K, row0;
    int nstages;          // ring depth
    int cluster_s;        // > 0: clustered split K, cluster_s ranks per column block (grid (cluster_s, N / TN))
    int maxc;             // most blocks that share a column block (scratch stride)
    float4* scratch;      // partials of shared column blocks: [N/64][maxc][NT][4][32] float4
    int* counters;        // [N/64] tickets, zero between launches
    unsigned long long* keys;
    int n_valid;
    int xmap;             // the X rows arrive by the tensor map (contiguous rows, a padded row fits a box)
    int early;            // stages of weights requested before the wait for the previous kernel
    int zp;               // zero points: S holds a second table [K/128][N] of (8 - z) * scale after the scales
    int* err;             // set non-zero when a bounded wait ran out
    int probe;            // measurement only: 1 = consumers release every stage unread (the copy pipeline alone);
                          // 2 (tests) = the copy warp leaves out its second stage, so the consumers' wait for it runs out
    uint32_t wait_limit;  // polls the consumers give a stage (WAIT_LIMIT; short under probe 2)
    long long* trace;     // measurement only (may be null): per block {start, first stage landed, last stage
                          // consumed, end} in ns of the global timer
};

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr int GEMV_MAX_STAGES = 8;

template <int CG, int KG, int NT>
struct GemvCfg {
    static constexpr int NW = CG * KG;               // consumer warps
    static constexpr int THREADS = (NW + 1) * 32;    // + the producer warp
    static constexpr int TN = CG * 64, TK = KG * 128;
    static constexpr int W_BYTES = NW * 4096;        // TK/16 k16-steps x CG x 512 B
    static constexpr int XROW = TK + 8;              // halves; the pad spreads the 8 token rows over the banks
    static constexpr int S_BYTES = KG * TN * 2;
    static constexpr int RED_BYTES = (KG > 1 ? KG - 1 : 1) * CG * NT * 2048;  // lives in a consumed stage's weights
    static constexpr int BAR_BYTES = 128;
    static constexpr int ZROW_BYTES = (XROW * 2 + 127) / 128 * 128;
    // tiles of up to 256 outputs: a stage's weights and its scales arrive as ONE tensor-map TMA load each (a box of
    // TK / 16 rows of CG x 512 bytes; KG rows of TN scales) instead of TK / 16 + KG bulk copies: the copy warp has 7
    // operations to issue per stage, not 23, which is worth 7-11 % of a large product's time
    static constexpr bool TENSOR = CG <= 4;
    static constexpr bool XTENSOR = XROW / 4 <= 256;  // a padded X row fits one box (8-byte elements, at most 256)
    // a stage holds the weights, the group scales and the m live rows of X; one zero row serves the other token rows
    // (zp: the zero-point offsets of the stage's groups follow its scales); stages start on 128-byte boundaries
    static constexpr int stage_bytes(int m, int zp = 0) { return (W_BYTES + (1 + zp) * S_BYTES + m * XROW * 2 + 127) / 128 * 128; }
    static constexpr int smem(int nstages, int m, int zp = 0) { return BAR_BYTES + ZROW_BYTES + nstages * stage_bytes(m, zp); }
    static_assert(RED_BYTES <= W_BYTES, "the reduction buffer fits a stage's weights");
};

// One Marlin word (8 nibbles q + 8) -> the four A-fragment registers of signed values q - 8, exactly:
// 0x6400 | n is the half 1024 + n (nibbles 0, 4), 0x5400 | (n << 4) the half 64 + n (nibbles 1, 5).
__device__ __forceinline__ void dequant_word(uint32_t q, uint32_t* a) {
    uint32_t lo0, hi0, lo1, hi1;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;\n" : "=r"(lo0) : "r"(q));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;\n" : "=r"(hi0) : "r"(q));
    uint32_t q8 = q >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;\n" : "=r"(lo1) : "r"(q8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;\n" : "=r"(hi1) : "r"(q8));
    const uint32_t SUB_LO = 0x64086408u, SUB_HI = 0x54805480u;  // 1032, 72
    __half2 r0 = __hsub2(*(__half2*)&lo0, *(const __half2*)&SUB_LO);  // outputs g,     columns 2t, 2t+1
    __half2 r1 = __hsub2(*(__half2*)&lo1, *(const __half2*)&SUB_LO);  // outputs g + 8, columns 2t, 2t+1
    __half2 r2 = __hsub2(*(__half2*)&hi0, *(const __half2*)&SUB_HI);  // outputs g,     columns 2t+8, 2t+9
    __half2 r3 = __hsub2(*(__half2*)&hi1, *(const __half2*)&SUB_HI);  // outputs g + 8, columns 2t+8, 2t+9
    a[0] = *(uint32_t*)&r0; a[1] = *(uint32_t*)&r1; a[2] = *(uint32_t*)&r2; a[3] = *(uint32_t*)&r3;
}

// The epilogue of 64 finished outputs x 8 NT tokens held in the accumulator layout of the mma (acc[j][b][2h+e]:
// output col + 16 b + g + 8 h, token 8 j + 2 t + e).
template <int NT, int EPI>
__device__ __forceinline__ void gemv_epilogue(const GemvArgs& a, float (&acc)[NT][4][4], const int col, const int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            int tok = 8 * j + 2 * t + e;
            if (tok >= a.m) continue;
            if (EPI == EPI_SILU) {
                __half* y = (__half*)a.Y + (size_t)(a.row0 + tok) * (a.N / 2) + col / 2 + g;
#pragma unroll
                for (int b = 0; b < 4; b++) y[8 * b] = __float2half_rn(silu(acc[j][b][e]) * acc[j][b][2 + e]);
            } else {
                float* y = (float*)a.Y + (size_t)(a.row0 + tok) * a.N + col + g;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    y[16 * b] = acc[j][b][e];
                    y[16 * b + 8] = acc[j][b][2 + e];
                }
            }
        }
    if (EPI == EPI_ARGMAX) {
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                unsigned long long k = 0;
#pragma unroll
                for (int b = 0; b < 4; b++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        int o = col + 16 * b + g + 8 * h;
                        if (o < a.n_valid) {
                            unsigned long long kk = argmax_key(acc[j][b][2 * h + e], o);
                            k = kk > k ? kk : k;
                        }
                    }
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    unsigned long long kk = __shfl_xor_sync(0xffffffffu, k, o);
                    k = kk > k ? kk : k;
                }
                int tok = 8 * j + 2 * t + e;
                if (g == 0 && tok < a.m && k) atomicMax(a.keys + a.row0 + tok, k);
            }
    }
}

// ZP: the zero-point variant (a.zp set): compiled apart so that the symmetric product carries none of it
template <int CG, int KG, int NT, int EPI, int ZP = 0>
__global__ void __launch_bounds__(GemvCfg<CG, KG, NT>::THREADS) w4a16_gemv_kernel(const __grid_constant__ GemvMaps maps, const GemvArgs a) {
    using C = GemvCfg<CG, KG, NT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + GEMV_MAX_STAGES;
    uint8_t* zrow = smem + C::BAR_BYTES;              // XROW halves of zeros: the token rows m .. 8 NT - 1
    uint8_t* stages = zrow + C::ZROW_BYTES;
    const int STAGE_BYTES = C::stage_bytes(a.m, ZP);  // weights | scales (| offsets) | m rows of X
    const int X_OFF = C::W_BYTES + (1 + ZP) * C::S_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == C::NW * 32) {
        if (C::TENSOR) { prefetch_tensormap(&maps.w); prefetch_tensormap(&maps.s); }
        if (a.xmap) prefetch_tensormap(&maps.x);
    }
    const int nstages = a.nstages;
    // stream-K: stage x of the matrix is (column block x / kst, k stage x % kst); block i owns [b(i), b(i+1))
    const int kst = a.K / C::TK;
    const bool clustered = a.cluster_s > 0;
    // (32-bit arithmetic: the host refuses a product with (stages + 1) x (blocks + 1) beyond 2^31; a 64-bit division
    // is a subroutine of a hundred instructions, twice on the way to the first copy and twice in the tail)
    const uint32_t total = (uint32_t)(a.N / C::TN) * (uint32_t)kst, G = gridDim.x;
    int beg, end;
    if (clustered) {  // rank blockIdx.x of the cluster of column block blockIdx.y
        beg = blockIdx.y * kst + (int)blockIdx.x * kst / a.cluster_s;
        end = blockIdx.y * kst + ((int)blockIdx.x + 1) * kst / a.cluster_s;
    } else {
        beg = (int)(blockIdx.x * total / G);
        end = (int)((blockIdx.x + 1) * total / G);
    }
    // the block that owns stage x: the largest i with b(i) <= x
    auto owner = [&](uint32_t x) { return (int)(((x + 1) * G + total - 1) / total - 1); };

    const int bid = blockIdx.y * gridDim.x + blockIdx.x;
    if (a.trace && threadIdx.x == 0) a.trace[bid * 4] = global_ns();
    // The copy warp's first lane sets up the ring's barriers itself and requests the block's first stage of weights
    // before the block meets: the weights do not depend on the previous kernel, and every launch is as long as its
    // first stage takes to arrive plus the streaming.
    if (threadIdx.x == C::NW * 32) {
        for (int i = 0; i < nstages; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], C::NW);
        }
        mbar_fence_init();
    }
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    const uint32_t mine = (uint32_t)(end - beg);
    const uint32_t tx = C::W_BYTES + (1 + ZP) * C::S_BYTES + a.m * (a.xmap ? C::XROW : C::TK) * 2;
    if (warp == C::NW) {
        // ------------------------------------------------------------ producer
        // what stage `it` of this block copies: 0 = weights and scales, 1 = X, 2 = both
        auto issue = [&](int cb, int st, int slot, int what) {
            int n0 = cb * C::TN, k0 = st * C::TK;
            uint8_t* base = stages + (size_t)slot * STAGE_BYTES;
            if (what != 1) {
                if (lane == 0) mbar_expect_tx(&full[slot], tx);
                __syncwarp();
                if (C::TENSOR) {
                    if (lane == 0) {
                        tma_tile_2d(base, &maps.w, n0, k0 / 16, &full[slot], pol_w);
                        tma_tile_2d(base + C::W_BYTES, &maps.s, n0, k0 / 128, &full[slot], pol_w);
                        if (ZP) tma_tile_2d(base + C::W_BYTES + C::S_BYTES, &maps.s, n0, a.K / 128 + k0 / 128, &full[slot], pol_w);
                    }
                } else {
                    const uint8_t* wsrc = (const uint8_t*)a.B + ((size_t)(k0 / 16) * 2 * a.N + (size_t)(n0 / 64) * 128) * 4;
                    for (int c = lane; c < C::TK / 16; c += 32)
                        bulk_g2s(base + c * (CG * 512), wsrc + (size_t)c * 8 * a.N, CG * 512, &full[slot], pol_w);
                    if (lane < KG)
                        bulk_g2s(base + C::W_BYTES + lane * (C::TN * 2),
                                 a.S + (size_t)(k0 / 128 + lane) * a.N + n0, C::TN * 2, &full[slot], pol_w);
                    if (ZP && lane >= 8 && lane < 8 + KG)
                        bulk_g2s(base + C::W_BYTES + C::S_BYTES + (lane - 8) * (C::TN * 2),
                                 a.S + (size_t)(a.K / 128 + k0 / 128 + lane - 8) * a.N + n0, C::TN * 2, &full[slot], pol_w);
                }
            }
            if (what != 0 && a.xmap) {
                if (lane == 0) tma_tile_2d(base + X_OFF, &maps.x, k0 / 4, 0, &full[slot], pol_x);
            } else if (what != 0) {
                if (lane < a.m) {
                    int row = a.xrows ? a.xrows[lane] : a.row0 + lane;
                    bulk_g2s(base + X_OFF + lane * (C::XROW * 2), a.X + (size_t)row * a.K + k0, C::TK * 2,
                             &full[slot], pol_x);
                }
            }
        };
        // the weights do not depend on the previous kernel: start them, then wait for it (its activations are this
        // kernel's X)
        uint32_t pre = mine < (uint32_t)nstages ? mine : (uint32_t)nstages;
        const int cb0 = beg / kst, st0 = beg - cb0 * kst;
        int cb = cb0, st = st0;
        auto next = [&]() { if (++st == kst) { st = 0; cb++; } };
        // (only the first stage's: with the whole ring requested at once by every block, the first stages land behind
        // the later ones' traffic; the rest follow right after the wait, while the consumers are busy with stage 0)
        const uint32_t early = min(pre, (uint32_t)a.early);
        __syncwarp();
        for (uint32_t it = 0; it < early; it++, next()) issue(cb, st, (int)it, 0);
        for (int i = lane; i < C::XROW * 2 / 16; i += 32) ((uint4*)zrow)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        pdl_launch_dependents();
        pdl_wait();
        cb = cb0; st = st0;
        for (uint32_t it = 0; it < pre; it++, next())
            if (!(a.probe == 2 && it == 1)) issue(cb, st, (int)it, it < early ? 1 : 2);
        bool ok = true;
        int slot = 0;
        uint32_t par = 0;  // parity of the consumers' release this slot is waiting for
        for (uint32_t it = pre; it < mine && ok; it++, next()) {
            if (lane == 0) ok = mbar_wait(&empty[slot], par);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            issue(cb, st, slot, 2);
            if (++slot == nstages) { slot = 0; par ^= 1; }
        }
        if (!ok && lane == 0) atomicExch(a.err, 1);
        return;
    }

    // ---------------------------------------------------------------- consumers
    __syncthreads();  // the ring's barriers are set up and the zero row is written (by the copy warp)
    pdl_launch_dependents();
    pdl_wait();
    const int cg = warp % CG, kg = warp / CG, g = lane >> 2, t = lane & 3;
    float acc[NT][4][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[j][b][i] = 0.f;

    // A wait that runs out marks the warp dead: it records the error, then walks the rest of its schedule with
    // short waits only (so that copies already in flight still land in a live block) and keeps meeting the block's
    // barriers, and the kernel ends instead of hanging.
    bool dead = false;
    int cb = beg / kst, st = beg - cb * kst, slot = 0;
    uint32_t par = 0;
    for (int x = beg; x < end; x++) {
        {
            if (!dead) {
                dead = !mbar_wait(&full[slot], par, a.wait_limit);
                if (dead && lane == 0) atomicExch(a.err, 2);
            } else {
                for (int i = 0; i < 1024 && !mbar_try_wait(&full[slot], par); i++) {}
            }
            if (a.trace && threadIdx.x == 0 && x == beg) a.trace[bid * 4 + 1] = global_ns();
            const uint8_t* base = stages + (size_t)slot * STAGE_BYTES;
            const uint4* wp = (const uint4*)(base + (size_t)(kg * 8 * CG + cg) * 512) + lane;
            // ldmatrix row addresses of this lane: token row lane % 8 (+ 8 j) of X, or the zero row past the m live
            // rows; columns 8 (lane / 8) of each pair of k16 steps
            uint32_t xs[NT];
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const int row = 8 * j + (lane & 7);
                xs[j] = (row < a.m ? smem_u32(base + X_OFF) + row * C::XROW * 2 : smem_u32(zrow)) +
                        (kg * 128 + 8 * (lane >> 3)) * 2;
            }
            uint4 sc4 = *(const uint4*)(base + C::W_BYTES + (kg * C::TN + cg * 64 + 8 * g) * 2);
            uint4 zs4 = make_uint4(0, 0, 0, 0);
            if (ZP) zs4 = *(const uint4*)(base + C::W_BYTES + C::S_BYTES + (kg * C::TN + cg * 64 + 8 * g) * 2);
            if (a.probe == 1) goto stage_done;
            // The nibbles go to the tensor core as f16 SUBNORMALS, with no subtraction at all: a low nibble n of a
            // 16-bit half is, as it stands, the half n * 2^-24 (q & 0x000f000f), a high one 16 n * 2^-24
            // (q & 0x00f000f0), both exact. The columns the high nibbles meet (b1 of the X fragment) are scaled by
            // 1/16 once per fragment, and the offset of 8 leaves through ONE extra mma per k16 step against a constant
            // A fragment (-8 * 2^-24 and -128 * 2^-24): corr = -8 * 2^-24 * sum_k x_k, the same for the 64 outputs.
            // Per Marlin word that is 1 shift + 4 and (+ the mma) instead of 4 lop3 + 1 shift + 4 hsub2; the products
            // are exact either way, the sums stay in f32, and 2^24 is folded into the group scale.
            float tmp[NT][4][4], corr[NT][4];
            uint32_t bx[NT][2][2];  // [token tile][k16 step of the pair][b0, b1 / 16]
            const uint32_t nbias[4] = {0x80088008u, 0x80088008u, 0x80808080u, 0x80808080u};
            const uint32_t sixteenth = 0x2c002c00u;  // half2(0.0625, 0.0625)
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                // (a volatile load: in program order with the ldmatrix loads. Left to itself the compiler sometimes
                // requests the stage's eight words together at the top, at the 96-register limit of two blocks per SM,
                // and the products are 4 % slower for it; which of the two it does changed with unrelated edits)
                uint4 w;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(smem_u32(wp + ks * CG * 32)));
                if ((ks & 1) == 0) {
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        ldsm_x4(bx[j][0][0], bx[j][0][1], bx[j][1][0], bx[j][1][1], xs[j] + ks * 32);
                        __half2 h0 = __hmul2(*(__half2*)&bx[j][0][1], *(const __half2*)&sixteenth);
                        __half2 h1 = __hmul2(*(__half2*)&bx[j][1][1], *(const __half2*)&sixteenth);
                        bx[j][0][1] = *(uint32_t*)&h0;
                        bx[j][1][1] = *(uint32_t*)&h1;
                    }
                }
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    if (ks == 0) mma16816_zero(corr[j], nbias, bx[j][0][0], bx[j][0][1]);
                    else mma16816(corr[j], nbias, bx[j][ks & 1][0], bx[j][ks & 1][1]);
                }
                uint32_t wq[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const uint32_t q = wq[b], q8 = q >> 8;
                    uint32_t af[4] = {q & 0x000f000fu, q8 & 0x000f000fu, q & 0x00f000f0u, q8 & 0x00f000f0u};
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        if (ks == 0) mma16816_zero(tmp[j][b], af, bx[j][0][0], bx[j][0][1]);
                        else mma16816(tmp[j][b], af, bx[j][ks & 1][0], bx[j][ks & 1][1]);
                    }
                }
            }
            // the group's scales (times 2^24): half 2 b + h of the lane's 16 bytes is output 16 b + g + 8 h
            const __half* sh = (const __half*)&sc4;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                float s0 = __half2float(sh[2 * b]) * 16777216.f, s1 = __half2float(sh[2 * b + 1]) * 16777216.f;
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    acc[j][b][0] += s0 * (tmp[j][b][0] + corr[j][0]); acc[j][b][1] += s0 * (tmp[j][b][1] + corr[j][1]);
                    acc[j][b][2] += s1 * (tmp[j][b][2] + corr[j][2]); acc[j][b][3] += s1 * (tmp[j][b][3] + corr[j][3]);
                }
            }
            if (ZP) {
                // zero points: w = (q - 8) * scale + (8 - z) * scale; the second term times the group's sum of x, which
                // the offset mma already holds: corr = -2^-21 * sum_k x_k
                const __half* zh = (const __half*)&zs4;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    float z0 = __half2float(zh[2 * b]) * -2097152.f, z1 = __half2float(zh[2 * b + 1]) * -2097152.f;
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        acc[j][b][0] += z0 * corr[j][0]; acc[j][b][1] += z0 * corr[j][1];
                        acc[j][b][2] += z1 * corr[j][2]; acc[j][b][3] += z1 * corr[j][3];
                    }
                }
            }
        }
    stage_done:
        if (a.trace && threadIdx.x == 0 && x + 1 == end) a.trace[bid * 4 + 2] = global_ns();
        // the piece (this block's stages of column block cb) goes on: release the stage and take the next
        const int pcb = cb, pslot = slot;
        if (++st == kst) { st = 0; cb++; }
        if (++slot == nstages) { slot = 0; par ^= 1; }
        if (x + 1 < end && st != 0) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[pslot]);
            continue;
        }
        // The piece ends. Its last stage is not released yet: once every consumer warp is past it (the barrier below)
        // its weight area is this block's reduction buffer, and the copy warp gets the slot back afterwards.
        float4* red = (float4*)(stages + (size_t)pslot * STAGE_BYTES);

        // ---- the KG warps of a column group: kg > 0 hand their sums to kg = 0, which adds them in kg order
        if (KG > 1) {
            named_bar_sync(1, C::NW * 32);  // every warp has finished reading the stage that becomes the buffer
            if (kg > 0) {
                float4* r = red + (size_t)((kg - 1) * CG + cg) * NT * 4 * 32;
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int b = 0; b < 4; b++)
                        r[(j * 4 + b) * 32 + lane] = make_float4(acc[j][b][0], acc[j][b][1], acc[j][b][2], acc[j][b][3]);
            }
            named_bar_sync(2, C::NW * 32);
            if (kg == 0) {
#pragma unroll
                for (int kk = 1; kk < KG; kk++) {
                    const float4* r = red + (size_t)((kk - 1) * CG + cg) * NT * 4 * 32;
#pragma unroll
                    for (int j = 0; j < NT; j++)
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            float4 v = r[(j * 4 + b) * 32 + lane];
                            acc[j][b][0] += v.x; acc[j][b][1] += v.y; acc[j][b][2] += v.z; acc[j][b][3] += v.w;
                        }
                }
            }
            named_bar_sync(1, C::NW * 32);
        }

        if (clustered) {
            // ---- the ranks of the cluster meet in rank 0. Every block's kg = 0 warps park their sums in their own
            // shared memory, the cluster synchronises, rank 0 reads the
            // others' through distributed shared memory and adds them in rank order, and a second barrier keeps the
            // others' shared memory alive until it has.
            if (kg != 0) return;  // exited threads do not count in the cluster barrier
            // the block is done streaming (one piece per block here): every slot is free, and slot 0 is at the same
            // shared-memory offset in every rank
            float4* mine = (float4*)stages + (size_t)cg * NT * 4 * 32;
            if (blockIdx.x != 0) {
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int b = 0; b < 4; b++)
                        mine[(j * 4 + b) * 32 + lane] = make_float4(acc[j][b][0], acc[j][b][1], acc[j][b][2], acc[j][b][3]);
            }
            cluster_sync();
            if (blockIdx.x == 0) {
                for (int r = 1; r < a.cluster_s; r++) {
                    const uint32_t rem = cluster_map(mine, r);
#pragma unroll
                    for (int j = 0; j < NT; j++)
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            float4 v = cluster_ld4(rem + ((j * 4 + b) * 32 + lane) * 16);
                            acc[j][b][0] += v.x; acc[j][b][1] += v.y; acc[j][b][2] += v.z; acc[j][b][3] += v.w;
                        }
                }
                gemv_epilogue<NT, EPI>(a, acc, (pcb * CG + cg) * 64, lane);
            }
            cluster_sync();
            return;
        }
        __syncwarp();
        // the reduction buffer is read: the slot goes back to the copy warp (the kg = 0 warps keep it a little longer:
        // a finishing block stages the other blocks' partial sums in it; with one k group per tile no barrier has
        // been met yet, and every warp must be done with the stage's words before one of them writes there)
        if (KG == 1) named_bar_sync(1, C::NW * 32);
        if (lane == 0 && kg != 0) mbar_arrive(&empty[pslot]);
        if (kg == 0) {
            const int colgrp = pcb * CG + cg;  // 64 outputs
            bool finish = true;
            // the blocks that share column block cb, in k order: first .. last
            const int first = owner((uint32_t)(pcb * kst)), nshare = owner((uint32_t)(pcb * kst + kst - 1)) - first + 1;
            if (nshare > 1) {
                float4* mine = a.scratch + ((size_t)colgrp * a.maxc + (blockIdx.x - first)) * (NT * 4 * 32);
#pragma unroll
                for (int j = 0; j < NT; j++)
#pragma unroll
                    for (int b = 0; b < 4; b++)
                        __stcg(mine + (j * 4 + b) * 32 + lane,
                               make_float4(acc[j][b][0], acc[j][b][1], acc[j][b][2], acc[j][b][3]));
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(a.counters + colgrp, 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                finish = ticket == nshare - 1;
                if (finish) {
                    __threadfence();
                    const float4* p0 = a.scratch + (size_t)colgrp * a.maxc * (NT * 4 * 32);
#pragma unroll
                    for (int j = 0; j < NT; j++)
#pragma unroll
                        for (int b = 0; b < 4; b++)
#pragma unroll
                            for (int i = 0; i < 4; i++) acc[j][b][i] = 0.f;
                    // The partial sums of UCH sharers at a time come into the warp's part of the slot by cp.async (L2
                    // only), all in flight together, and are added from there in block order: a column block of a
                    // long-k matrix has some 15 sharers, and one L2 round trip each was 5 us of tail.
                    constexpr int UCH = (2 * KG / NT) < 1 ? 1 : ((2 * KG / NT) > 4 ? 4 : (2 * KG / NT));
                    float4* stg = red + (size_t)cg * UCH * (NT * 4 * 32);
                    for (int s0 = 0; s0 < nshare; s0 += UCH) {
#pragma unroll
                        for (int u = 0; u < UCH; u++)
                            if (s0 + u < nshare) {
#pragma unroll
                                for (int q = 0; q < NT * 4; q++)
                                    cp_async16(stg + (u * NT * 4 + q) * 32 + lane,
                                               p0 + (size_t)(s0 + u) * (NT * 4 * 32) + q * 32 + lane);
                            }
                        cp_async_commit();
                        cp_async_wait_all();
                        __syncwarp();
#pragma unroll
                        for (int u = 0; u < UCH; u++)
                            if (s0 + u < nshare) {
#pragma unroll
                                for (int j = 0; j < NT; j++)
#pragma unroll
                                    for (int b = 0; b < 4; b++) {
                                        float4 v = stg[(u * NT * 4 + j * 4 + b) * 32 + lane];
                                        acc[j][b][0] += v.x; acc[j][b][1] += v.y; acc[j][b][2] += v.z; acc[j][b][3] += v.w;
                                    }
                            }
                        __syncwarp();
                    }
                    if (lane == 0) a.counters[colgrp] = 0;  // left zero for the next product
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[pslot]);
            if (finish) gemv_epilogue<NT, EPI>(a, acc, colgrp * 64, lane);
        }
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int b = 0; b < 4; b++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[j][b][i] = 0.f;
    }
    if (a.trace && threadIdx.x == 0) a.trace[bid * 4 + 3] = global_ns();
}

}  // namespace qb
