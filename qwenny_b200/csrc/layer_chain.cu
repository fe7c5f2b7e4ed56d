// One persistent launch for the part of a decode / verify layer that is nothing but weight streaming:
//     out_proj -> (h += ., RMSNorm) -> gate_up (SwiGLU) -> down -> (h += ., RMSNorm) -> the next layer's in-projection
// which the reference runs as four Marlin launches and two add_rmsnorm launches (Stack::mlp and the mixers' out / in
// projections, src/cuda/qwen/mod.rs:744-766; kernels/marlin.cuh, kernels/dense.cuh:12-26). Between separate launches
// the copy pipeline drains and refills (several microseconds each, against 3-20 us of streaming per product); here
// one block per SM stays resident, its copy warp streams the weights of product after product through one ring of
// shared-memory stages and never stops at a product boundary, and the blocks meet at grid barriers (the launch is
// cooperative) where a product needs the whole result of the one before.
//  * 16 consumer warps as 4 column groups x 4 k groups: a stage is 256 outputs x 512 columns of int4 (64 KB), its
//    group scales, and, for products whose input another phase wrote to global memory, the matching slice of X.
//    The arithmetic is the 16-row product's (w4a16_gemv.cuh): Marlin word = mma A fragment, lop3/hsub2 dequant,
//    f32 group scale on the group's partial sum; the stages of a product are dealt stream-K (equal contiguous
//    ranges), shared column blocks meet through an L2 scratch and an atomic ticket, every sum in a fixed order.
//  * the two residual + RMSNorm steps run redundantly in every block: after the barrier each block adds the finished
//    product to the residual stream, normalises, and keeps the f16 result in its own shared memory as the resident X
//    of the next product (no X copies for it at all); block r writes row r of the new residual stream (and of the
//    normalised rows, for the kernels after this one) back to global memory.
//  * every wait is bounded: a poll limit on the mbarriers and on the grid barriers, after which the error word is
//    set and the block carries on (wrong numbers, no hang).
#include "launch.h"
#include "w4a16_gemv.cuh"

namespace qb {

constexpr int CH_CG = 4, CH_KG = 4, CH_NW = CH_CG * CH_KG;
constexpr int CH_THREADS = (CH_NW + 1) * 32;
constexpr int CH_TN = CH_CG * 64, CH_TK = CH_KG * 128;
constexpr int CH_W_BYTES = CH_NW * 4096, CH_S_BYTES = CH_KG * CH_TN * 2;
constexpr int CH_XROW = CH_TK + 8;      // halves: row stride of a stage's X slice
constexpr int CH_RES_ROW = H + 8;       // halves: row stride of the resident X
constexpr int CH_MAXPH = 4, CH_MAXM = 7, CH_MAXSTG = 4;
constexpr int CH_FIXED = 128 /* mbarriers */ + 256 /* row sums */ + CH_XROW * 2 + 112 /* pad to 128 */;
static_assert(CH_FIXED % 128 == 0 && (CH_RES_ROW * 2) % 16 == 0 && (CH_XROW * 2) % 16 == 0, "16-byte copies, 128-byte stages");
constexpr int CH_BAR_EXIT = 7;          // gbar[0..6]: the phases' barriers; gbar[7]: blocks that have left
constexpr uint32_t GRID_WAIT_LIMIT = 1u << 21;

// X of a phase
enum { CH_X_GLOBAL = 0,   // f16 rows in global memory, complete before this launch
       CH_X_NORM = 1,     // rmsnorm(h_in + add) * norm_w, computed by every block after the previous phase's barrier
       CH_X_PHASE = 2 };  // f16 rows in global memory written by the previous phase (copied after its barrier)

struct ChainPhase {
    const uint32_t* B;    // Marlin words (null: no product, the phase is its norm alone)
    const __half* S;
    const __half* X;      // CH_X_GLOBAL / CH_X_PHASE: [m][K]
    void* Y;              // EPI_PLAIN: f32 [m][N]; EPI_SILU: f16 [m][N/2]
    const float* h_in;    // CH_X_NORM: residual stream in, the finished product to add, residual stream out
    const float* add;
    float* h_out;
    const float* norm_w;
    __half* xn_out;       // optional global copy of the normalised rows
    int N, K, epi, xmode;
};

struct ChainArgs {
    ChainPhase ph[CH_MAXPH];
    int nph, m, nstages, maxc;
    float4* scratch;
    int* counters;
    unsigned* gbar;
    int* err;
    float eps;
    int probe;          // measurement only: 1 = consumers release every stage unread, 2 = no residual / norm prologue
    long long* trace;   // measurement only (may be null): per block 17 timestamps (ns): per phase {begin, X ready,
                        // first stage landed, share written}, then the end
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// One thread: wait until all `G` blocks have arrived at barrier `b` (bounded)
__device__ __forceinline__ bool grid_wait(const ChainArgs& a, int b, unsigned G) {
    for (uint32_t i = 0; i < GRID_WAIT_LIMIT; i++) {
        if (ld_acquire(a.gbar + b) >= G) return true;
        __nanosleep(40);
    }
    atomicExch(a.err, 3);
    return false;
}

// A block's walk over its stages, product after product (the copy warp keeps two of these: weights ahead, X behind)
struct ChainCur {
    int p, x, end, cb, st, kst, slot, wrap;
};
__device__ __forceinline__ void cur_range(const ChainArgs& a, int p, int& beg, int& end, int& kst) {
    const ChainPhase& P = a.ph[p];
    kst = P.K / CH_TK;
    const long long total = (long long)(P.N / CH_TN) * kst, G = gridDim.x;
    beg = (int)((long long)blockIdx.x * total / G);
    end = (int)((long long)(blockIdx.x + 1) * total / G);
}
// moves to the first stage at or after phase p; false past the last phase
__device__ __forceinline__ bool cur_seek(const ChainArgs& a, ChainCur& c, int p) {
    for (; p < a.nph; p++) {
        if (!a.ph[p].B) continue;
        int beg, end, kst;
        cur_range(a, p, beg, end, kst);
        if (beg >= end) continue;
        c.p = p; c.x = beg; c.end = end; c.kst = kst; c.cb = beg / kst; c.st = beg - c.cb * kst;
        return true;
    }
    c.p = a.nph;
    return false;
}
__device__ __forceinline__ bool cur_next(const ChainArgs& a, ChainCur& c) {
    if (++c.slot == a.nstages) { c.slot = 0; c.wrap++; }
    if (++c.x < c.end) {
        if (++c.st == c.kst) { c.st = 0; c.cb++; }
        return true;
    }
    return cur_seek(a, c, c.p + 1);
}

__global__ void __launch_bounds__(CH_THREADS, 1) layer_chain_kernel(const __grid_constant__ ChainArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + 8;
    float* rowsum = (float*)(smem + 128);                 // [2][16] warp partials of a row's sum of squares
    uint8_t* zrow = smem + 128 + 256;                     // CH_XROW halves of zeros: the token rows m .. 7
    __half* xres = (__half*)(smem + CH_FIXED);            // resident X: m rows of CH_RES_ROW halves
    const int RES_BYTES = (a.m * CH_RES_ROW * 2 + 127) / 128 * 128;
    uint8_t* stages = smem + CH_FIXED + RES_BYTES;
    const int STAGE_BYTES = (CH_W_BYTES + CH_S_BYTES + a.m * CH_XROW * 2 + 127) / 128 * 128;
    const int X_OFF = CH_W_BYTES + CH_S_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const unsigned G = gridDim.x;

    if (tid == 0) {
        for (int i = 0; i < a.nstages; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], CH_NW);
        }
        mbar_fence_init();
    }
    for (int i = tid; i < CH_XROW * 2 / 16; i += CH_THREADS) ((uint4*)zrow)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    pdl_launch_dependents();

    if (warp == CH_NW) {
        // ------------------------------------------------------------------------------------ the copy warp
        // Two cursors over the same sequence of stages: `w` issues weights and scales as soon as a slot is free
        // (they depend on nothing), `x` follows and issues the stage's X slice once its source is complete (the
        // kernels before this launch; the previous phase's barrier). A stage's full barrier expects all its bytes
        // from the moment its weights are issued.
        const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
        ChainCur w = {}, x = {};
        bool more_w = cur_seek(a, w, 0), more_x = cur_seek(a, x, 0), ok = true;
        int passed = -2;   // -2: nothing waited for yet; -1: the kernels before this launch; p >= 0: grid barrier p
        int inflight = 0;  // stages whose weights are issued and whose X is not
        while (more_x && ok) {
            // weights ahead; a full ring blocks this warp only when no X copy is owed
            while (more_w && inflight < a.nstages) {
                if (w.wrap > 0) {
                    bool freed = false;
                    if (lane == 0)
                        freed = inflight > 0 ? mbar_try_wait(&empty[w.slot], (w.wrap - 1) & 1)
                                             : mbar_wait(&empty[w.slot], (w.wrap - 1) & 1);
                    freed = __shfl_sync(0xffffffffu, freed, 0);
                    if (!freed) {
                        if (inflight == 0) ok = false;
                        break;
                    }
                }
                const ChainPhase& P = a.ph[w.p];
                const int n0 = w.cb * CH_TN, k0 = w.st * CH_TK;
                uint8_t* base = stages + (size_t)w.slot * STAGE_BYTES;
                const uint32_t tx = CH_W_BYTES + CH_S_BYTES + (P.xmode == CH_X_NORM ? 0 : a.m * CH_TK * 2);
                if (lane == 0) mbar_expect_tx(&full[w.slot], tx);
                __syncwarp();
                const uint8_t* wsrc = (const uint8_t*)P.B + ((size_t)(k0 / 16) * 2 * P.N + (size_t)(n0 / 64) * 128) * 4;
                bulk_g2s(base + lane * (CH_CG * 512), wsrc + (size_t)lane * 8 * P.N, CH_CG * 512, &full[w.slot], pol_w);
                if (lane < CH_KG)
                    bulk_g2s(base + CH_W_BYTES + lane * (CH_TN * 2), P.S + (size_t)(k0 / 128 + lane) * P.N + n0,
                             CH_TN * 2, &full[w.slot], pol_w);
                inflight++;
                more_w = cur_next(a, w);
            }
            if (!ok) break;
            // the X slice of the oldest stage in flight
            const ChainPhase& P = a.ph[x.p];
            if (P.xmode != CH_X_NORM) {
                const int need = P.xmode == CH_X_PHASE ? x.p - 1 : -1;
                if (passed == -2) {
                    pdl_wait();
                    passed = -1;
                }
                if (need > passed) {
                    if (lane == 0) grid_wait(a, need, G);
                    __syncwarp();
                    asm volatile("fence.proxy.async;\n" ::: "memory");
                    passed = need;
                }
                if (lane < a.m) {
                    uint8_t* base = stages + (size_t)x.slot * STAGE_BYTES;
                    bulk_g2s(base + X_OFF + lane * (CH_XROW * 2), P.X + (size_t)lane * P.K + x.st * CH_TK, CH_TK * 2,
                             &full[x.slot], pol_x);
                }
            }
            inflight--;
            more_x = cur_next(a, x);
        }
        if (!ok && lane == 0) atomicExch(a.err, 1);
        return;
    }

    // ------------------------------------------------------------------------------------------ consumers
    pdl_wait();
    const int cg = warp % CH_CG, kg = warp / CH_CG, g = lane >> 2, t = lane & 3;
    const int NCT = CH_NW * 32;  // consumer threads
    float acc[4][4];
#pragma unroll
    for (int b = 0; b < 4; b++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[b][i] = 0.f;
    bool dead = false;
    int slot = 0, wrap = 0;

    long long* tr = a.trace ? a.trace + (size_t)blockIdx.x * 17 : nullptr;
    for (int p = 0; p < a.nph; p++) {
        const ChainPhase& P = a.ph[p];
        if (tr && tid == 0) tr[4 * p] = global_ns();
        if (P.xmode == CH_X_NORM && a.probe != 2) {
            // ---- every block: h_out = h_in + add, resident X = norm_w * h_out / rms(h_out), after the barrier of the
            // phase that produced `add`
            if (p > 0) {
                if (tid == 0) grid_wait(a, p - 1, G);
                named_bar_sync(3, NCT);
            }
            float4 v[2][3];
            auto fetch = [&](int r, float4 (&d)[3]) {
#pragma unroll
                for (int i = 0; i < 3; i++) {
                    int idx = tid + NCT * i;
                    if (idx < H / 4) {
                        float4 hv = __ldcg((const float4*)(P.h_in + (size_t)r * H) + idx);
                        float4 av = __ldcg((const float4*)(P.add + (size_t)r * H) + idx);
                        d[i] = make_float4(hv.x + av.x, hv.y + av.y, hv.z + av.z, hv.w + av.w);
                    }
                }
            };
            fetch(0, v[0]);
#pragma unroll
            for (int r = 0; r < CH_MAXM; r++) {
                if (r < a.m) {
                    if (r + 1 < a.m) fetch(r + 1, v[(r + 1) & 1]);
                    float4(&d)[3] = v[r & 1];
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < 3; i++)
                        if (tid + NCT * i < H / 4) ss += d[i].x * d[i].x + d[i].y * d[i].y + d[i].z * d[i].z + d[i].w * d[i].w;
                    ss = warp_sum(ss);
                    float* rs = rowsum + (r & 1) * 16;
                    if (lane == 0) rs[warp] = ss;
                    named_bar_sync(3, NCT);
                    float tot = 0.f;
#pragma unroll
                    for (int i = 0; i < CH_NW; i++) tot += rs[i];
                    const float rinv = rsqrtf(tot / H + a.eps);
                    const bool owner_blk = (int)blockIdx.x == r % (int)G;
#pragma unroll
                    for (int i = 0; i < 3; i++) {
                        int idx = tid + NCT * i;
                        if (idx < H / 4) {
                            float4 wv = ((const float4*)P.norm_w)[idx];
                            uint2 o = make_uint2(pack_half2(wv.x * (d[i].x * rinv), wv.y * (d[i].y * rinv)),
                                                 pack_half2(wv.z * (d[i].z * rinv), wv.w * (d[i].w * rinv)));
                            *(uint2*)(xres + (size_t)r * CH_RES_ROW + 4 * idx) = o;
                            if (owner_blk) {
                                ((float4*)(P.h_out + (size_t)r * H))[idx] = d[i];
                                if (P.xn_out) *(uint2*)(P.xn_out + (size_t)r * H + 4 * idx) = o;
                            }
                        }
                    }
                }
            }
            named_bar_sync(3, NCT);  // the resident X is complete
        }
        if (tr && tid == 0) tr[4 * p + 1] = global_ns();
        if (!P.B) continue;

        int beg, end, kst;
        cur_range(a, p, beg, end, kst);
        const long long total = (long long)(P.N / CH_TN) * kst;
        auto owner = [&](long long x) { return (int)(((x + 1) * (long long)G + total - 1) / total - 1); };
        int cb = beg < end ? beg / kst : 0, st = beg - cb * kst;
        for (int x = beg; x < end; x++) {
            const uint32_t par = wrap & 1;
            if (!dead) {
                dead = !mbar_wait(&full[slot], par);
                if (dead && lane == 0) atomicExch(a.err, 2);
            } else {
                for (int i = 0; i < 1024 && !mbar_try_wait(&full[slot], par); i++) {}
            }
            if (tr && tid == 0 && x == beg) tr[4 * p + 2] = global_ns();
            const uint8_t* base = stages + (size_t)slot * STAGE_BYTES;
            if (a.probe != 1) {
                const uint4* wp = (const uint4*)(base + (size_t)(kg * 8 * CH_CG + cg) * 512) + lane;
                // ldmatrix row address of this lane: token row lane % 8 of the stage's X slice or of the resident X, or
                // the zero row past the m live rows; columns 8 (lane / 8) of each pair of k16 steps
                const int row = lane & 7;
                uint32_t xs;
                if (row >= a.m) xs = smem_u32(zrow) + (kg * 128 + 8 * (lane >> 3)) * 2;
                else if (P.xmode == CH_X_NORM)
                    xs = smem_u32(xres) + (row * CH_RES_ROW + st * CH_TK + kg * 128 + 8 * (lane >> 3)) * 2;
                else
                    xs = smem_u32(base + X_OFF) + (row * CH_XROW + kg * 128 + 8 * (lane >> 3)) * 2;
                uint4 sc4 = *(const uint4*)(base + CH_W_BYTES + (kg * CH_TN + cg * 64 + 8 * g) * 2);
                float tmp[4][4];
                uint32_t bx[2][2];
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    uint4 w = wp[ks * CH_CG * 32];
                    if ((ks & 1) == 0) ldsm_x4(bx[0][0], bx[0][1], bx[1][0], bx[1][1], xs + ks * 32);
                    uint32_t wq[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        uint32_t af[4];
                        dequant_word(wq[b], af);
                        if (ks == 0) mma16816_zero(tmp[b], af, bx[0][0], bx[0][1]);
                        else mma16816(tmp[b], af, bx[ks & 1][0], bx[ks & 1][1]);
                    }
                }
                const __half* sh = (const __half*)&sc4;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    float s0 = __half2float(sh[2 * b]), s1 = __half2float(sh[2 * b + 1]);
                    acc[b][0] += s0 * tmp[b][0]; acc[b][1] += s0 * tmp[b][1];
                    acc[b][2] += s1 * tmp[b][2]; acc[b][3] += s1 * tmp[b][3];
                }
            }
            const int pcb = cb, pslot = slot;
            if (++st == kst) { st = 0; cb++; }
            if (++slot == a.nstages) { slot = 0; wrap++; }
            if (x + 1 < end && st != 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[pslot]);
                continue;
            }
            // ---- the piece (this block's stages of column block pcb) ends. Its last stage is released only after its
            // weight area has served as the reduction buffer of the k groups.
            float4* red = (float4*)(stages + (size_t)pslot * STAGE_BYTES);
            named_bar_sync(1, NCT);
            if (kg > 0) {
                float4* r = red + (size_t)((kg - 1) * CH_CG + cg) * 4 * 32;
#pragma unroll
                for (int b = 0; b < 4; b++) r[b * 32 + lane] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
            }
            named_bar_sync(2, NCT);
            if (kg == 0) {
#pragma unroll
                for (int kk = 1; kk < CH_KG; kk++) {
                    const float4* r = red + (size_t)((kk - 1) * CH_CG + cg) * 4 * 32;
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        float4 v = r[b * 32 + lane];
                        acc[b][0] += v.x; acc[b][1] += v.y; acc[b][2] += v.z; acc[b][3] += v.w;
                    }
                }
            }
            named_bar_sync(1, NCT);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[pslot]);
            if (kg == 0) {
                const int colgrp = pcb * CH_CG + cg;
                bool finish = true;
                const int first = owner((long long)pcb * kst), nshare = owner((long long)pcb * kst + kst - 1) - first + 1;
                if (nshare > 1) {
                    float4* mine = a.scratch + ((size_t)colgrp * a.maxc + ((int)blockIdx.x - first)) * (4 * 32);
#pragma unroll
                    for (int b = 0; b < 4; b++)
                        __stcg(mine + b * 32 + lane, make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]));
                    __threadfence();
                    __syncwarp();
                    int ticket = 0;
                    if (lane == 0) ticket = atomicAdd(a.counters + colgrp, 1);
                    ticket = __shfl_sync(0xffffffffu, ticket, 0);
                    finish = ticket == nshare - 1;
                    if (finish) {
                        __threadfence();
                        const float4* p0 = a.scratch + (size_t)colgrp * a.maxc * (4 * 32);
#pragma unroll
                        for (int b = 0; b < 4; b++)
#pragma unroll
                            for (int i = 0; i < 4; i++) acc[b][i] = 0.f;
                        for (int s = 0; s < nshare; s++) {
#pragma unroll
                            for (int b = 0; b < 4; b++) {
                                float4 v = __ldcg(p0 + (size_t)s * (4 * 32) + b * 32 + lane);
                                acc[b][0] += v.x; acc[b][1] += v.y; acc[b][2] += v.z; acc[b][3] += v.w;
                            }
                        }
                        if (lane == 0) a.counters[colgrp] = 0;  // left zero for the next product
                    }
                }
                if (finish) {
                    // acc[b][2h+e]: output col + 16 b + g + 8 h, token 2 t + e
                    const int col = colgrp * 64;
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int tok = 2 * t + e;
                        if (tok >= a.m) continue;
                        if (P.epi == EPI_SILU) {
                            __half* y = (__half*)P.Y + (size_t)tok * (P.N / 2) + col / 2 + g;
#pragma unroll
                            for (int b = 0; b < 4; b++) y[8 * b] = __float2half_rn(silu(acc[b][e]) * acc[b][2 + e]);
                        } else {
                            float* y = (float*)P.Y + (size_t)tok * P.N + col + g;
#pragma unroll
                            for (int b = 0; b < 4; b++) {
                                y[16 * b] = acc[b][e];
                                y[16 * b + 8] = acc[b][2 + e];
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < 4; b++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[b][i] = 0.f;
        }
        if (tr && tid == 0) tr[4 * p + 3] = global_ns();
        // ---- the block's share of the product is written: arrive at the phase's barrier
        if (p + 1 < a.nph) {
            __threadfence();
            named_bar_sync(3, NCT);
            if (tid == 0) {
                __threadfence();
                atomicAdd(a.gbar + p, 1u);
            }
        }
    }
    // ---- the last block to leave clears the barriers for the next launch
    named_bar_sync(3, NCT);
    if (tr && tid == 0) tr[16] = global_ns();
    if (tid == 0) {
        __threadfence();
        unsigned old = atomicAdd(a.gbar + CH_BAR_EXIT, 1u);
        if (old == G - 1) {
            for (int i = 0; i <= CH_BAR_EXIT; i++) a.gbar[i] = 0;
            __threadfence();
        }
    }
}

}  // namespace qb

using namespace qb;

extern "C" {

int qb_layer_chain_max_rows(void) { return CH_MAXM; }

int qb_layer_chain(qb_ctx* ctx, void* stream, const qb_chain* c) {
    if (!ctx || !c || c->m < 1 || !c->mix || !c->out_w || !c->out_s || !c->gate_up_w || !c->gate_up_s || !c->down_w ||
        !c->down_s || !c->post_norm || !c->next_norm || !c->h || !c->h_tmp || !c->part_h || !c->mid || !c->xn)
        return QB_ERR_ARG;
    if (c->m > CH_MAXM) return QB_ERR_UNSUPPORTED;
    if (c->next_w && (!c->next_s || !c->part || c->next_n <= 0 || c->next_n % CH_TN)) return QB_ERR_ARG;
    static_assert(H % CH_TK == 0 && MIX % CH_TK == 0 && FF % CH_TK == 0 && H % CH_TN == 0 && (2 * FF) % CH_TN == 0,
                  "the 27B widths are whole stages");
    ChainArgs a = {};
    a.m = c->m;
    a.eps = c->eps;
    ChainPhase* P = a.ph;
    P[0].B = (const uint32_t*)c->out_w; P[0].S = (const __half*)c->out_s; P[0].X = (const __half*)c->mix;
    P[0].Y = c->part_h; P[0].N = H; P[0].K = MIX; P[0].epi = EPI_PLAIN; P[0].xmode = CH_X_GLOBAL;
    P[1].B = (const uint32_t*)c->gate_up_w; P[1].S = (const __half*)c->gate_up_s; P[1].Y = c->mid;
    P[1].N = 2 * FF; P[1].K = H; P[1].epi = EPI_SILU; P[1].xmode = CH_X_NORM;
    P[1].h_in = c->h; P[1].add = c->part_h; P[1].h_out = c->h_tmp; P[1].norm_w = c->post_norm; P[1].xn_out = nullptr;
    P[2].B = (const uint32_t*)c->down_w; P[2].S = (const __half*)c->down_s; P[2].X = (const __half*)c->mid;
    P[2].Y = c->part_h; P[2].N = H; P[2].K = FF; P[2].epi = EPI_PLAIN; P[2].xmode = CH_X_PHASE;
    P[3].B = (const uint32_t*)c->next_w; P[3].S = (const __half*)c->next_s; P[3].Y = c->part;
    P[3].N = c->next_w ? c->next_n : 0; P[3].K = H; P[3].epi = EPI_PLAIN; P[3].xmode = CH_X_NORM;
    P[3].h_in = c->h_tmp; P[3].add = c->part_h; P[3].h_out = c->h; P[3].norm_w = c->next_norm;
    P[3].xn_out = (__half*)c->xn;
    a.nph = 4;
    a.scratch = (float4*)ctx->scratch;
    a.counters = ctx->counters;
    a.gbar = ctx->gbar;
    a.err = ctx->err;
    a.probe = ctx->probe;
    a.trace = ctx->trace;
    if (ctx->trace) ctx->trace += 4 * 1024;  // the next launch's slots

    const int grid = ctx->sms;
    // the most blocks that share a column block: a block's range is at least floor(total / grid) stages
    int maxc = 1, maxn = 0;
    for (int p = 0; p < a.nph; p++) {
        if (!P[p].B) continue;
        const long long kst = P[p].K / CH_TK, total = (long long)(P[p].N / CH_TN) * kst;
        const long long per = total / grid > 0 ? total / grid : 1;
        const int share = (int)((kst + per - 1) / per) + 1;
        maxc = share > maxc ? share : maxc;
        maxn = P[p].N > maxn ? P[p].N : maxn;
    }
    a.maxc = maxc;
    if ((size_t)(maxn / 64) * maxc * 4 * 32 * sizeof(float4) > ctx->scratch_bytes || (size_t)(maxn / 64) > ctx->ncounters)
        return QB_ERR_TOO_LARGE;

    const int res = (a.m * CH_RES_ROW * 2 + 127) / 128 * 128;
    const int stage = (CH_W_BYTES + CH_S_BYTES + a.m * CH_XROW * 2 + 127) / 128 * 128;
    int nst = (232448 - CH_FIXED - res) / stage;
    nst = nst > CH_MAXSTG ? CH_MAXSTG : nst;
    if (nst < 2) return QB_ERR_UNSUPPORTED;
    a.nstages = nst;
    const size_t smem = (size_t)CH_FIXED + res + (size_t)nst * stage;

    static bool opted = false;
    if (!opted) {
        QB_CUDA(cudaFuncSetAttribute(layer_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        QB_CUDA(cudaFuncSetAttribute(layer_chain_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
        opted = true;
    }
    // cooperative: the blocks wait for one another at the grid barriers, so all of them must be resident
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(CH_THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = ctx->pdl && ctx->chain_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, layer_chain_kernel, a);
    if (e != cudaSuccess && lc.numAttrs == 2) {
        // a driver that does not take the two attributes together: cooperative alone from now on
        cudaGetLastError();
        ctx->chain_pdl = false;
        lc.numAttrs = 1;
        e = cudaLaunchKernelEx(&lc, layer_chain_kernel, a);
    }
    return e == cudaSuccess ? QB_OK : (int)e;
}

}  // extern "C"
