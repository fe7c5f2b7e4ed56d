// Prompt attention over the int8 KV cache on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
// Replaces attn_prefill (kernels/attn.cuh:351-553 of the reference) for steps with many prompt tiles.
//
// A block is (a pair of prompt tiles = 2 x 64 (token, head) rows, kv head) and walks the keys its rows may see in
// stages of 64. Tensor memory (512 columns x 128 lanes, lane = row) holds everything that belongs to a row:
//   columns   0-255  O, the f32 accumulator of the 256 output dims
//   columns 256-383  two score buffers S (64 f32 each); P of a stage overwrites the first 32 columns of its S as f16
//   columns 384-511  Q, 256 dims as f16 pairs: the A operand of S = Q K^T for the whole block
// so the only things in shared memory are the f16 keys and values, in a ring of three stages:
//   warps 8-15  read a stage's int8 keys and values from the cache (128-bit loads, one stage ahead in registers) and
//               write them as f16 where the tensor core wants them: K as four [64 keys][64 dims] K-major tiles, V
//               transposed as one [256 dims][64 keys] tile, both with the 128-byte swizzle; the codes are converted
//               EXACTLY (1024 + byte via prmt, minus 1152), so no offset has to be folded out afterwards
//   warp 16     one elected lane issues S = Q K^T (M 128 rows, N 64 keys, K 256 dims: 16 tcgen05.mma, A from tensor
//               memory) and O += P V (M 128, N 256 dims, K 64 keys: 4 tcgen05.mma, A = P from tensor memory);
//               tcgen05.commit tells the others when a product is complete. S of stage i + 1 is issued before P V of
//               stage i, so the tensor core has work while the softmax of stage i runs
//   warps 0-7   softmax: tensor memory hands a THREAD its row of S (tcgen05.ld); two threads (warps w, w + 4) share a
//               row, 32 keys each, and exchange their maxima through shared memory. Scores are scaled by the keys'
//               scales, masked causally where the stage reaches the diagonal, and P = 2^(s - m) times the values'
//               scales goes back as f16 (tcgen05.st), m the row's running maximum: the same rounding points as the
//               reference's kernel. A stage in which some row's maximum grows rescales that warp's accumulator rows
//               (tcgen05.ld / st, half of the dims per thread); a lazier rule (rescale only past a threshold) was
//               measured 1 % faster and decorrelates the f16 rounding of P from the reference's, so it is not used
// At the end the softmax threads read their rows of O, divide by the row sum, multiply by the gate and write f32
// (+ f16). Every wait is bounded: a wait that runs out sets the context's error word and the block drains.
#include "attn_tc.cuh"
#include "launch.h"

namespace qb {
namespace pft {

constexpr int TROWS = 64;                    // rows of one prompt tile; a block has two
constexpr int SK = 64;                       // keys per stage
constexpr int NST = 3;                       // stages of the key / value ring
constexpr int K_BYTES = SK * HD * 2;         // 32 KB: four [64][64] tiles
constexpr int V_BYTES = HD * SK * 2;         // 32 KB: [256][64]
constexpr int SC_BYTES = 2 * SK * 4;         // key scales, value scales
constexpr int CTL_BYTES = 1024;
constexpr int ROWS = 128;
constexpr int X_BYTES = 2 * 2 * ROWS * 4;    // the row maxima of the two halves, two stages deep
constexpr int SMEM_BYTES = NST * (K_BYTES + V_BYTES + SC_BYTES) + X_BYTES + CTL_BYTES + 1024;
constexpr int SM_WARPS = 8, CVT_WARP0 = 8, CVT_WARPS = 8, MMA_WARP = 16;
constexpr int THREADS = 32 * (MMA_WARP + 1);
constexpr int TMEM_COLS = 512, O_COL = 0, S_COL = 256, Q_COL = 384;

using namespace tc;

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const float* q, const uint8_t* kc, const uint8_t* vc, const float* ks, const float* vs,
                       const int* ptile, int ntile, const int* tok_slot, const int* tok_pos, int cap, float* out,
                       __half* mix, int* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* kf = smem;                    // [NST][K_BYTES]
    uint8_t* vf = kf + NST * K_BYTES;      // [NST][V_BYTES]
    float* scl = (float*)(vf + NST * V_BYTES);  // [NST][ksc 64 | vsc 64]
    float* xm = scl + NST * 2 * SK;        // [2 stages][2 halves][ROWS]
    uint8_t* ctl = (uint8_t*)(xm + 2 * 2 * ROWS);
    uint64_t* kv_ready = (uint64_t*)ctl;   // [NST] a stage's f16 tiles and scales are written (8 convert warps)
    uint64_t* kv_free = kv_ready + NST;    // [NST] both products of the stage in that ring slot are complete
    uint64_t* s_ready = kv_free + NST;     // [2] S of a stage is complete in tensor memory
    uint64_t* p_ready = s_ready + 2;       // [2] P of a stage is written over its S (8 warps)
    uint64_t* o_done = p_ready + 2;        // [2] O += P V of a stage is complete
    uint32_t* tmem_slot = (uint32_t*)(o_done + 2);

    const int g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < NST; i++) {
            mbar_init(&kv_ready[i], CVT_WARPS);
            mbar_init(&kv_free[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_ready[i], 1);
            mbar_init(&p_ready[i], SM_WARPS);
            mbar_init(&o_done[i], 1);
        }
        mbar_fence_init();
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    // the block's tiles: 2 pair, 2 pair + 1 (the last pairs, with the longest contexts, first)
    const int pair = gridDim.x - 1 - blockIdx.x, ta = 2 * pair, tb = ta + 1;
    const int firstA = ptile[2 * ta], ntA = ptile[2 * ta + 1];
    int firstB = 0, ntB = 0;
    bool paired = false;
    if (tb < ntile) {
        firstB = ptile[2 * tb]; ntB = ptile[2 * tb + 1];
        paired = firstB == firstA + ntA && tok_slot[firstB] == tok_slot[firstA] && tok_pos[firstB] == tok_pos[firstA] + ntA;
    }
    const int npass = tb < ntile && !paired ? 2 : 1;
    int jbase = 0;  // stages of earlier passes: ring slots and barrier phases run on
    Waiter w_mma{err, 11}, w_sm{err, 12}, w_cv{err, 13};

    for (int pass = 0; pass < npass; pass++) {
        // rows 0..63: tile 0 of the pass; rows 64..127: its partner (present only in a pair of consecutive tiles)
        const int first0 = pass == 0 ? firstA : firstB, nt0 = pass == 0 ? ntA : ntB;
        const int first1 = firstB, nt1 = paired ? ntB : 0;
        const int tlast = nt1 ? first1 + nt1 - 1 : first0 + nt0 - 1;
        const int keys = tok_pos[tlast] + 1, slot = tok_slot[tlast], nstg = (keys + SK - 1) / SK;
        const uint8_t* kh = kc + cache_head(slot, g, cap);
        const uint8_t* vh = vc + cache_head(slot, g, cap);
        const float* ksh = ks + scale_head(slot, g, cap);
        const float* vsh = vs + scale_head(slot, g, cap);
        // the softmax threads' rows (row = 64 group + token * GROUP + head) and halves
        const int qd = warp & 3, half = (warp >> 2) & 1, row = qd * 32 + lane, grp = row / TROWS, lr = row % TROWS;
        const int tok = lr / GROUP, head = g * GROUP + lr % GROUP;
        const int tokn = tok < (grp ? nt1 : nt0) ? (grp ? first1 : first0) + tok : -1;
        const uint32_t trow = tmem + ((uint32_t)(qd * 32) << 16);

        // ---- Q of the 128 rows into tensor memory: every softmax thread converts and stores half of its row
        if (warp < SM_WARPS) {
            const float* qp = q + ((size_t)max(tokn, 0) * NH + head) * HD;
#pragma unroll 1
            for (int c = 128 * half; c < 128 * half + 128; c += 64) {
                uint32_t qv[32];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (tokn >= 0) v = *(const float4*)(qp + c + 4 * j);
                    qv[2 * j] = pack_half2(v.x, v.y);
                    qv[2 * j + 1] = pack_half2(v.z, v.w);
                }
                tmem_st32(trow + Q_COL + (c >> 1), qv);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();

        if (warp == MMA_WARP) {
            // ------------------------------------------------------------ tensor-core issue
            auto issue_s = [&](int i) {
                const int J = jbase + i, b2 = J & 1, rs = J % NST;
                w_mma.wait(&kv_ready[rs], (J / NST) & 1, lane);
                // (the S buffer is free: P V of stage J - 2, which read P out of it, was issued before this)
                tc_fence_after();
                if (lane == 0 && !w_mma.dead) {
                    const uint64_t kd = smem_desc(smem_u32(kf + rs * K_BYTES));
#pragma unroll
                    for (int b = 0; b < 4; b++)   // (a [64 keys][64 dims] tile is 8 KB: 512 descriptor units)
                        umma_ts4(tmem + S_COL + b2 * SK, tmem + Q_COL + b * 32, kd + b * (SK * 128 / 16), idesc(SK), b ? 1u : 0u);
                    umma_commit(&s_ready[b2]);
                }
                __syncwarp();
            };
            issue_s(0);
            for (int i = 0; i < nstg; i++) {
                const int J = jbase + i, b2 = J & 1, rs = J % NST;
                if (i + 1 < nstg) issue_s(i + 1);
                w_mma.wait(&p_ready[b2], (J >> 1) & 1, lane);
                tc_fence_after();
                if (lane == 0 && !w_mma.dead) {
                    umma_ts4(tmem + O_COL, tmem + S_COL + b2 * SK, smem_desc(smem_u32(vf + rs * V_BYTES)), idesc(HD), i ? 1u : 0u);
                    umma_commit(&kv_free[rs]);
                    umma_commit(&o_done[b2]);
                }
                __syncwarp();
            }
        } else if (warp < SM_WARPS) {
            // ------------------------------------------------------------ softmax: two threads per row, 32 keys each
            const int lim = tokn >= 0 ? tok_pos[tokn] + 1 : 1 << 30;  // (rows without a token: Q = 0, nothing masked)
            float m = -INFINITY, l = 0.f;
            for (int i = 0; i < nstg; i++) {
                const int J = jbase + i, b2 = J & 1, rs = J % NST, kb0 = i * SK + 32 * half;
                w_sm.wait(&s_ready[b2], (J >> 1) & 1, lane);
                tc_fence_after();
                uint32_t sv[32];
                tmem_ld32(trow + S_COL + b2 * SK + 32 * half, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                const float4* ksc4 = (const float4*)(scl + rs * 2 * SK + 32 * half);
                const float4* vsc4 = ksc4 + SK / 4;
                // scores times the keys' scales; the causal mask only where the stage reaches past a row's last key
                // (a masked score is a large negative number: 2^(that - m) is 0)
                const bool edge = __any_sync(0xffffffffu, kb0 + 32 > lim);
                float sc[32];
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 k4 = ksc4[j >> 2];
                    sc[j] = __uint_as_float(sv[j]) * k4.x; sc[j + 1] = __uint_as_float(sv[j + 1]) * k4.y;
                    sc[j + 2] = __uint_as_float(sv[j + 2]) * k4.z; sc[j + 3] = __uint_as_float(sv[j + 3]) * k4.w;
                }
                if (edge) {
#pragma unroll
                    for (int j = 0; j < 32; j++) sc[j] = kb0 + j < lim ? sc[j] : -1e30f;
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 32; j++) mx[j & 3] = fmaxf(mx[j & 3], sc[j]);
                const float mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                // the row's maximum over both halves (the partner has read its S by the time it passes the barrier,
                // so P may overwrite those columns afterwards)
                float* xs = xm + (J & 1) * 2 * ROWS;
                xs[half * ROWS + row] = mine;
                named_bar_sync(1 + qd, 64);
                const float both = fmaxf(mine, xs[(1 - half) * ROWS + row]);
                const float mold = m;
                if (both > -1e29f) m = fmaxf(m, both);
                const bool move = m > mold;
                const float factor = mold == -INFINITY ? 0.f : ex2(mold - m);  // 1 where the maximum stays
                const float nref = m == -INFINITY ? 0.f : -m;
                float sum = 0.f;
                uint32_t ph[16];
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 v4 = vsc4[j >> 2];
                    const float p0 = ex2(sc[j] + nref), p1 = ex2(sc[j + 1] + nref), p2 = ex2(sc[j + 2] + nref), p3 = ex2(sc[j + 3] + nref);
                    sum += (p0 + p1) + (p2 + p3);
                    ph[j >> 1] = pack_half2(p0 * v4.x, p1 * v4.y);
                    ph[(j >> 1) + 1] = pack_half2(p2 * v4.z, p3 * v4.w);
                }
                l = l * factor + sum;
                tmem_st16(trow + S_COL + b2 * SK + 16 * half, ph);
                if (i > 0 && __any_sync(0xffffffffu, move)) {
                    // rescale this thread's half of its accumulator row (rows whose maximum stayed multiply by 1) once
                    // the previous stage's product has landed in it
                    w_sm.wait(&o_done[(J - 1) & 1], ((J - 1) >> 1) & 1, lane);
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 128 * half; c < 128 * half + 128; c += 32) {
                        uint32_t ov[32];
                        tmem_ld32(trow + O_COL + c, ov);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; j++) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * factor);
                        tmem_st32(trow + O_COL + c, ov);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[b2]);
            }
            // ---- the rows' results: O / (the two halves' sums) times the gate, half of the dims per thread
            const int Jl = jbase + nstg - 1;
            float* xs = xm + ((Jl + 1) & 1) * 2 * ROWS;
            xs[half * ROWS + row] = l;
            named_bar_sync(1 + qd, 64);
            l += xs[(1 - half) * ROWS + row];
            w_sm.wait(&o_done[Jl & 1], (Jl >> 1) & 1, lane);
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
            for (int c = 128 * half; c < 128 * half + 128; c += 32) {
                uint32_t ov[32];
                tmem_ld32(trow + O_COL + c, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (tokn >= 0 && !w_sm.dead) {
                    float* op = out + (size_t)tokn * MIX + head * HD + c;
                    __half* mp = mix ? mix + (size_t)tokn * MIX + head * HD + c : nullptr;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 gt = *(const float4*)(op + j);
                        const float4 res = make_float4(gt.x * __uint_as_float(ov[j]) * inv, gt.y * __uint_as_float(ov[j + 1]) * inv,
                                                       gt.z * __uint_as_float(ov[j + 2]) * inv, gt.w * __uint_as_float(ov[j + 3]) * inv);
                        *(float4*)(op + j) = res;
                        if (mp) *(uint2*)(mp + j) = make_uint2(pack_half2(res.x, res.y), pack_half2(res.z, res.w));
                    }
                }
            }
            tc_fence_before();
        } else if (warp >= CVT_WARP0) {
            // ------------------------------------------------------------ int8 -> f16 tiles, one stage ahead in registers
            const int cw = warp - CVT_WARP0, ct = threadIdx.x - CVT_WARP0 * 32;
            uint4 kraw[4], vraw[4];
            float sraw = 0.f;
            auto fetch = [&](int i) {
                const int kb0 = i * SK;
                // keys 8 cw + lane / 4, 16-byte group (b = it, t4 = lane % 4) of their rows
                const uint8_t* kp = kh + (size_t)(kb0 + 8 * cw + (lane >> 2)) * HD + (lane & 3) * 16;
#pragma unroll
                for (int it = 0; it < 4; it++) kraw[it] = *(const uint4*)(kp + 64 * it);
                // dims 32 cw + lane, 16-key block `it` of the stage
                const uint8_t* vp = vh + ((size_t)(kb0 >> 4) * HD + 32 * cw + lane) * 16;
#pragma unroll
                for (int it = 0; it < 4; it++) vraw[it] = *(const uint4*)(vp + (size_t)it * HD * 16);
                // (scales of positions past the last key are not read: such cache entries may hold anything)
                if (ct < 2 * SK) sraw = kb0 + (ct & (SK - 1)) < keys ? (ct < SK ? ksh : vsh)[kb0 + (ct & (SK - 1))] : 0.f;
            };
            fetch(0);
            for (int i = 0; i < nstg; i++) {
                const int J = jbase + i, rs = J % NST;
                if (J >= NST) w_cv.wait(&kv_free[rs], (J / NST - 1) & 1, lane);  // the slot's earlier stage is consumed
                uint8_t* kt = kf + rs * K_BYTES;
                uint8_t* vt = vf + rs * V_BYTES;
                {
                    const int key = 8 * cw + (lane >> 2), t4 = lane & 3;
#pragma unroll
                    for (int it = 0; it < 4; it++) {
                        const uint32_t wq[4] = {kraw[it].x, kraw[it].y, kraw[it].z, kraw[it].w};
                        uint8_t* tile = kt + it * (SK * 128);
#pragma unroll
                        for (int s = 0; s < 4; s++) {
                            // word s: dims 16 s + 2 t4 + {0, 1} (bytes 0, 1) and 16 s + 8 + 2 t4 + {0, 1} (bytes 2, 3)
                            *(uint32_t*)(tile + sw128(key, 2 * s) + 4 * t4) = exact2(wq[s], 0x4140);
                            *(uint32_t*)(tile + sw128(key, 2 * s + 1) + 4 * t4) = exact2(wq[s], 0x4342);
                        }
                    }
                }
                {
                    const int d = 32 * cw + lane;
#pragma unroll
                    for (int it = 0; it < 4; it++) {
                        // word t of a 16-byte group: keys 2 t, 2 t + 1 (bytes 0, 1) and 2 t + 8, 2 t + 9 (bytes 2, 3)
                        const uint32_t wq[4] = {vraw[it].x, vraw[it].y, vraw[it].z, vraw[it].w};
                        *(uint4*)(vt + sw128(d, 2 * it)) = make_uint4(exact2(wq[0], 0x4140), exact2(wq[1], 0x4140),
                                                                     exact2(wq[2], 0x4140), exact2(wq[3], 0x4140));
                        *(uint4*)(vt + sw128(d, 2 * it + 1)) = make_uint4(exact2(wq[0], 0x4342), exact2(wq[1], 0x4342),
                                                                         exact2(wq[2], 0x4342), exact2(wq[3], 0x4342));
                    }
                }
                if (ct < 2 * SK) scl[rs * 2 * SK + ct] = sraw;
                if (i + 1 < nstg) fetch(i + 1);
                async_proxy_fence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&kv_ready[rs]);
            }
        }
        jbase += nstg;
        tc_fence_before();
        __syncthreads();  // the pass is complete: Q may be rewritten
        tc_fence_after();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

}  // namespace pft
}  // namespace qb

// the many-tile form of qb_attn_prefill (one key split): see attn.cu
int qb_attn_prefill_tc_launch(qb_ctx* ctx, cudaStream_t st, const float* q, const void* kc, const void* vc, const float* ks,
                              const float* vs, const int* ptile, int ntile, const int* tok_slot, const int* tok_pos,
                              int cap, float* out, void* mix_f16) {
    using namespace qb;
    return launch(ctx, pft::attn_prefill_tc_kernel, dim3((ntile + 1) / 2, NKV), dim3(pft::THREADS), pft::SMEM_BYTES, st, q,
                  (const uint8_t*)kc, (const uint8_t*)vc, ks, vs, ptile, ntile, tok_slot, tok_pos, cap, out,
                  (__half*)mix_f16, ctx->err);
}
