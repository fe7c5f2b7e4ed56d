// Gated DeltaNet of a decode / verify step in ONE launch (qb_delta_mixer): the conv, the gated delta rule with the
// two-buffer rollback plan and the gated RMSNorm, which the reference runs as three kernels (kernels/qwen_deltanet.cuh:
// delta_conv :84-131, delta_rule :172-288, delta_norm :295-315). Steps with longer segments take the three entry points
// of delta_prompt.cu. Slot memory layout, the plan and the metadata are the reference's (delta_common.cuh).
#include "delta_common.cuh"
#include "launch.h"

namespace qb {
constexpr int TCH = 8;                    // tokens per round
constexpr int LPC = 4, RPT = LKD / LPC;   // lanes per value column, state rows per thread
}  // namespace qb

// delta_conv + delta_rule + delta_norm of a decode / verify step in ONE launch: a cluster of two blocks per (value
// head h, segment), each with half of the head's 128 value columns (256 threads: column tid / 4, rows
// 4 (tid % 4 + 4 j) + i: the operation order of dot_rows, so the token form of the prompt path gives the same bits). A
// block's slice of the f32 state lives in its registers; it recomputes the conv of the 320 channels it needs (its key
// head's q and k, its own v columns) from the in-projection rows or the ring, runs the recurrence, and the two blocks
// finish the gated RMSNorm over the head's 128 columns together: they exchange their per-lane partial sums of
// squares through distributed shared memory and add them in the order one warp over the whole row would. Every
// phase's global loads are issued together (one round trip per phase). The conv ring is written by the blocks in
// shares; the slot metadata by the LAST block of the launch to finish (an atomic ticket), because every block reads
// the old metadata when it starts.
namespace qb {

constexpr int FNT = 256;             // threads of a block
constexpr int FCOLS = LVD / 2;       // value columns of a block
constexpr int FCH = 2 * LKD + FCOLS; // q, k, v channels of a block
constexpr int FLD = 8;               // loads in flight per thread in the staging loops

struct FusedRound {
    float x[TCH + CONV_K - 1][FCH];  // conv inputs of the round's tokens and the 3 positions before them
    float c[TCH][FCH];               // conv outputs: q [0,128), k [128,256), v [256,320)
    float z[TCH][FCOLS];             // the gate input of the norm
    float o[TCH][FCOLS];             // raw outputs of the round
    float w[FCH][CONV_K];            // conv taps of the block's channels
    float lp[TCH][32];               // per token: the 32 lane partials of the row's sum of squares (16 per block)
    float e[TCH], b[TCH], kq[TCH], rn[TCH];
};

__global__ void __launch_bounds__(FNT)
delta_fused_kernel(const float* p, int splits, int n, const float* ba, int ba_splits, const float* cw,
                   const float* a_log, const float* dt_bias, const float* nw, float* mem, long long sst, int* meta,
                   float* out, __half* y, const int* seg_start, const int* seg_len, const int* seg_slot,
                   const int* seg_pos0, int segs, int* ticket, long long* trace) {
    extern __shared__ __align__(16) uint8_t fsm[];
    FusedRound& R = *(FusedRound*)fsm;
    pdl_launch_dependents();
    // measurement only: thread 0 stamps the phases of the (first) round into trace[block][10]
    long long* tr = trace && threadIdx.x == 0 ? trace + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 10 : nullptr;
    auto stamp = [&](int i) {
        if (tr) { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); tr[i] = t; }
    };
    stamp(0);
    const int h = blockIdx.x >> 1, hf = blockIdx.x & 1, sg = blockIdx.y, kh = h / (LV_HEADS / LK_HEADS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, rg = tid % LPC, lc = tid / LPC;
    const int col = hf * FCOLS + lc;  // the thread's value column of the head
    const int t0 = seg_start[sg], len = seg_len[sg], slot = seg_slot[sg], p0 = seg_pos0[sg];
    // global conv channel of the block's channel ch
    auto gchan = [&](int ch) {
        return ch < LKD ? kh * LKD + ch : ch < 2 * LKD ? LK_HEADS * LKD + kh * LKD + (ch - LKD)
                                                       : 2 * LK_HEADS * LKD + h * LVD + hf * FCOLS + (ch - 2 * LKD);
    };
    // ---- everything that does not depend on this step's earlier kernels: the taps, the norm weight, the state
    for (int c = tid; c < FCH; c += FNT) *(float4*)R.w[c] = ld4(cw + gchan(c) * CONV_K);
    const float nwv = nw[hf * FCOLS + tid % FCOLS], alog = a_log[h], dtb = dt_bias[h];
    const Plan pl = make_plan(meta, slot, p0, len);
    float* sm0 = mem + slot * sst;
    auto sbuf = [&](int b) { return sm0 + (size_t)b * SLOT_STATE + ((size_t)h * LVD + col) * LKD; };
    auto entry = [&](int b, int pos) { return sm0 + 2 * SLOT_STATE + (size_t)b * SLOT_BANK + (size_t)(pos % KEEP) * REP; };
    float S[RPT];
    if (pl.zero) {
#pragma unroll
        for (int i = 0; i < RPT; i++) S[i] = 0.f;
    } else {
        ld_rows<4>(S, sbuf(pl.in), rg);
    }
    for (int i = 0; i < pl.r; i++) {
        const float* e = entry(pl.in, pl.from + i);
        float k[RPT];
        ld_rows<4>(k, e + kh * LKD, rg);
        float dk = dot_rows<4>(S, k);
        float ex = e[LK_HEADS * LKD + LV_HEADS * LVD + h], be = e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h];
        float delta = (e[LK_HEADS * LKD + h * LVD + col] - ex * dk) * be;
#pragma unroll
        for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
    }
    pdl_wait();
    stamp(1);

    // the block's share of the conv ring: channels cb .. cb + ch of the segment's last CR tokens
    constexpr int NB = 2 * LV_HEADS, CH = (LQKV + NB - 1) / NB;  // channels per block (the last block has fewer)
    const int cb = blockIdx.x * CH, mm = min(len, CR);
    static_assert(TCH * ((LQKV + 2 * LV_HEADS - 1) / (2 * LV_HEADS)) <= 4 * FNT, "a round's ring share fits 4 values per thread");

    bool lp_pending = false;  // a cluster barrier phase this block has arrived at and not yet waited for
    for (int c0 = 0; c0 < len; c0 += TCH) {
        const int m = min(TCH, len - c0);
        // ---- ONE round trip of independent loads: conv inputs (step rows or ring), z, gates, the ring share.
        // With one split of the in-projection (the usual case) the conv inputs and z go straight to shared memory as
        // 16-byte asynchronous copies from a short loop (L2 only: another kernel wrote them): a handful of
        // instructions per thread. Unrolled into some thirty register loads with their own address arithmetic the
        // same staging took 2 us just to ISSUE: the kernel runs once per launch, so every instruction of it is also
        // an instruction fetched cold.
        constexpr int NROW = TCH + CONV_K - 1, NZV = (TCH * FCOLS + FNT - 1) / FNT;
        float ringv[4], gate = 0.f;
        const bool direct = splits == 1;
        if (direct) {
            const int nrow = m + CONV_K - 1;
            for (int e = tid; e < nrow * (FCH / 4); e += FNT) {
                const int row = e / (FCH / 4), c = (e - row * (FCH / 4)) * 4;
                const int si = c0 + row - (CONV_K - 1), qp = p0 + si;
                float* dst = &R.x[row][c];
                if (qp < 0) {
                    *(float4*)dst = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    cp_async16(dst, si >= 0 ? p + (size_t)(t0 + si) * DELTA_IN + gchan(c)
                                            : sm0 + SLOT_RING + (size_t)(qp & (CR - 1)) * LQKV + gchan(c));
                }
            }
            for (int e = tid; e < m * (FCOLS / 4); e += FNT) {
                const int tk = e / (FCOLS / 4), c = (e - tk * (FCOLS / 4)) * 4;
                cp_async16(&R.z[tk][c], p + (size_t)(t0 + c0 + tk) * DELTA_IN + LQKV + h * LVD + hf * FCOLS + c);
            }
            cp_async_commit();
        }
        // several splits: thread tid takes channel tid of every row, and threads below FCH - FNT also channel FNT + tid
        float xv[NROW][2], zv[NZV];
        const int gc0 = gchan(tid), gc1 = gchan(min(FNT + tid, FCH - 1));
        const bool two = FNT + tid < FCH;
        if (!direct) {
#pragma unroll
            for (int row = 0; row < NROW; row++) {
                xv[row][0] = xv[row][1] = 0.f;
                const int si = c0 + row - (CONV_K - 1), qp = p0 + si;
                if (row < m + CONV_K - 1 && qp >= 0) {
                    if (si >= 0) {
                        // (the first split's value is a plain load, so that every row's first loads are in flight
                        // together: a warp issues in order, and a sum inside a loop waits for each load before the next)
                        const float* pr = p + (size_t)(t0 + si) * DELTA_IN;
                        xv[row][0] = __ldcg(pr + gc0);
                        if (two) xv[row][1] = __ldcg(pr + gc1);
                        for (int s = 1; s < splits; s++) {
                            pr += (size_t)n * DELTA_IN;
                            xv[row][0] += __ldcg(pr + gc0);
                            if (two) xv[row][1] += __ldcg(pr + gc1);
                        }
                    } else {
                        const float* rr = sm0 + SLOT_RING + (size_t)(qp & (CR - 1)) * LQKV;
                        xv[row][0] = __ldcg(rr + gc0);
                        if (two) xv[row][1] = __ldcg(rr + gc1);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < NZV; u++) {
                const int x = u * FNT + tid;
                zv[u] = 0.f;
                if (x < m * FCOLS) {
                    int tk = x / FCOLS, c = x - tk * FCOLS;
                    const float* pz = p + (size_t)(t0 + c0 + tk) * DELTA_IN + LQKV + h * LVD + hf * FCOLS + c;
                    zv[u] = __ldcg(pz);
                    for (int s = 1; s < splits; s++) zv[u] += __ldcg(pz + (size_t)s * n * DELTA_IN);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = u * FNT + tid, tk = c0 + i / CH, c = cb + i % CH;
            ringv[u] = 0.f;
            if (i < m * CH && c < LQKV && tk >= len - mm) {
                const float* pq = p + (size_t)(t0 + tk) * DELTA_IN + c;
                ringv[u] = __ldcg(pq);
                for (int s = 1; s < splits; s++) ringv[u] += __ldcg(pq + (size_t)s * n * DELTA_IN);
            }
        }
        if (tid < 2 * m) {  // the gates of head h
            int tk = tid >> 1, which = tid & 1, t = t0 + c0 + tk;
            const float* pb = ba + (size_t)t * (2 * LV_HEADS) + (which ? h : LV_HEADS + h);
            float gs[8];  // up to 8 splits in flight together, added in split order
#pragma unroll
            for (int s = 0; s < 8; s++) gs[s] = s < ba_splits ? __ldcg(pb + (size_t)s * n * (2 * LV_HEADS)) : 0.f;
#pragma unroll
            for (int s = 0; s < 8; s++) gate += gs[s];
            for (int s = 8; s < ba_splits; s++) gate += __ldcg(pb + (size_t)s * n * (2 * LV_HEADS));
        }
        if (!direct) {
#pragma unroll
            for (int row = 0; row < NROW; row++) {
                if (row < m + CONV_K - 1) {
                    R.x[row][tid] = xv[row][0];
                    if (two) R.x[row][FNT + tid] = xv[row][1];
                }
            }
#pragma unroll
            for (int u = 0; u < NZV; u++) {
                const int x = u * FNT + tid;
                if (x < m * FCOLS) R.z[x / FCOLS][x % FCOLS] = zv[u];
            }
        }
        if (tid < 2 * m) {
            int tk = tid >> 1, which = tid & 1;
            if (which) {
                R.b[tk] = 1.f / (1.f + expf(-gate));
            } else {
                float a = gate + dtb;
                float sp = a > 20.f ? a : log1pf(expf(a));
                R.e[tk] = expf(-expf(alog) * sp);
            }
        }
        if (direct) cp_async_wait_all();
        __syncthreads();
        stamp(2);
        // ---- conv + SiLU
        for (int x = tid; x < m * FCH; x += FNT) {
            int tk = x / FCH, c = x - tk * FCH;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < CONV_K; j++) acc += R.w[c][j] * R.x[tk + j][c];
            R.c[tk][c] = silu(acc);
        }
        __syncthreads();
        stamp(3);
        // ---- L2 norm of q and k (a warp per (token, q | k), 4 channels per lane), q also / sqrt(128)
        for (int task = warp; task < 2 * m; task += FNT / 32) {
            int tk = task >> 1, which = task & 1;
            float4* v4 = (float4*)&R.c[tk][which * LKD + lane * 4];
            float4 v = *v4;
            float sc = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) + 1e-6f);
            if (!which) sc *= rsqrtf((float)LKD);
            *v4 = make_float4(v.x * sc, v.y * sc, v.z * sc, v.w * sc);
        }
        __syncthreads();
        stamp(4);
        for (int tk = warp; tk < m; tk += FNT / 32) {  // k . q
            float4 a = ld4(&R.c[tk][lane * 4]), b = ld4(&R.c[tk][LKD + lane * 4]);
            float x = warp_sum(a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w);
            if (lane == 0) R.kq[tk] = x;
        }
        // ---- the delta rule inputs from the new checkpoint on, for a later restart (k by the first block of the key
        // head's first value head, v by each block for its columns, the gates by the head's first block)
        for (int tk = max(0, pl.ck - (p0 + c0)); tk < m; tk++) {
            float* e = entry(pl.cbuf, p0 + c0 + tk);
            if (hf == 0 && h % (LV_HEADS / LK_HEADS) == 0 && tid < LKD) e[kh * LKD + tid] = R.c[tk][LKD + tid];
            if (tid >= LKD && tid < LKD + FCOLS)
                e[LK_HEADS * LKD + h * LVD + hf * FCOLS + tid - LKD] = R.c[tk][2 * LKD + tid - LKD];
            if (hf == 0 && tid == LKD + FCOLS) {
                e[LK_HEADS * LKD + LV_HEADS * LVD + h] = R.e[tk];
                e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h] = R.b[tk];
            }
        }
        __syncthreads();
        stamp(5);
        // ---- the recurrence
        for (int tk = 0; tk < m; tk++) {
            if (pl.wck && p0 + c0 + tk == pl.ck) st_rows<4>(sbuf(pl.cbuf), S, rg);
            float k[RPT], q[RPT];
            ld_rows<4>(k, &R.c[tk][LKD], rg);
            ld_rows<4>(q, &R.c[tk][0], rg);
            float dk = dot_rows<4>(S, k), dq = dot_rows<4>(S, q);
            float ex = R.e[tk], delta = (R.c[tk][2 * LKD + lc] - ex * dk) * R.b[tk];
            if (rg == 0) R.o[tk][lc] = ex * dq + delta * R.kq[tk];
#pragma unroll
            for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
        }
        __syncthreads();
        stamp(6);
        // ---- gated RMSNorm over the head's 128 value columns. One warp over the whole row would give lane L the
        // columns 4 L .. 4 L + 3 and add the 32 lane partials as a butterfly; this block has the columns of lanes
        // 16 hf .. 16 hf + 15: it computes those partials, hands them to its partner through distributed shared
        // memory, and both run the same butterfly over the 32.
        if (lp_pending) { cluster_wait(); lp_pending = false; }  // the partner is done with the last round's partials
        for (int x = tid; x < m * 16; x += FNT) {
            int tk = x >> 4, l16 = x & 15;
            float4 v = ld4(&R.o[tk][l16 * 4]);
            float part = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            R.lp[tk][hf * 16 + l16] = part;
        }
        cluster_sync();
        {
            const uint32_t rem = cluster_map(&R.lp[0][0], hf ^ 1);
            for (int x = tid; x < m * 16; x += FNT) {
                int tk = x >> 4, l16 = x & 15, idx = tk * 32 + (hf ^ 1) * 16 + l16;
                float v;
                asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(rem + idx * 4));
                R.lp[tk][(hf ^ 1) * 16 + l16] = v;
            }
        }
        cluster_arrive();  // this block has read its partner's partials (the matching wait: before they are rewritten)
        __syncthreads();   // this block's copy of them is complete
        lp_pending = true;
        for (int tk = warp; tk < m; tk += FNT / 32) {
            float ss = warp_sum(R.lp[tk][lane]);
            if (lane == 0) R.rn[tk] = rsqrtf(ss / LVD + EPS);
        }
        __syncthreads();
        for (int x = tid; x < m * FCOLS; x += FNT) {
            int tk = x / FCOLS, c = x - tk * FCOLS, t = t0 + c0 + tk;
            float o = R.o[tk][c];
            if (out) out[(size_t)t * MIX + h * LVD + hf * FCOLS + c] = o;
            y[(size_t)t * MIX + h * LVD + hf * FCOLS + c] = __float2half_rn(nwv * (o * R.rn[tk]) * silu(R.z[tk][c]));
        }
        // ---- this round's rows of the conv ring (the block's channel share), loaded with the round's inputs
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = u * FNT + tid, tk = c0 + i / CH, c = cb + i % CH;
            if (i < m * CH && c < LQKV && tk >= len - mm) sm0[SLOT_RING + (size_t)((p0 + tk) & (CR - 1)) * LQKV + c] = ringv[u];
        }
        __syncthreads();
        stamp(7);
    }
    st_rows<4>(sbuf(pl.ebuf), S, rg);
    stamp(8);
    if (lp_pending) cluster_wait();  // the partner may read this block's shared memory until here
    // ---- the last block of the launch records the segments' steps in the slot metadata
    __shared__ int last;
    if (tid == 0) {
        __threadfence();
        int tkt = atomicAdd(ticket, 1);
        last = tkt == (int)(gridDim.x * gridDim.y) - 1;
    }
    __syncthreads();
    if (last) {
        for (int s = tid; s < segs; s += FNT) {
            int sl = seg_slot[s], q0 = seg_pos0[s], ln = seg_len[s];
            Plan q = make_plan(meta, sl, q0, ln);
            meta[sl * META] = q0 + ln;
            meta[sl * META + 1] = q.ck;
            meta[sl * META + 2] = q.ebuf;
        }
        if (tid == 0) *ticket = 0;
    }
}

}  // namespace qb

// conv + rule + norm in one launch (same arguments as the three together); `out` (the raw output before the gated
// norm, f32 [n][MIX]) may be NULL
extern "C" int qb_delta_mixer(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* ba,
                              int ba_splits, const float* cw, const float* a_log, const float* dt_bias,
                              const float* nw, float* mem, long long sst, int* meta, float* out, void* y,
                              const int* seg_start, const int* seg_len, const int* seg_slot, const int* seg_pos0,
                              int segs) {
    if (!ctx || !p || !ba || !cw || !a_log || !dt_bias || !nw || !mem || !meta || !y || !seg_start || !seg_len ||
        !seg_slot || !seg_pos0 || n <= 0 || segs <= 0 || splits < 1 || ba_splits < 1)
        return QB_ERR_ARG;
    // Blocks read the conv ring's last 3 positions and write the step's own; with a segment of 30 tokens or more the
    // two would touch the same ring rows from different blocks. Such steps take the three-kernel path.
    if (n > qb::CR - qb::CONV_K + 1) return QB_ERR_UNSUPPORTED;
    // the launch's ticket: the last int of the context's ticket array (the products use the first n / 64)
    int* ticket = ctx->counters + ctx->ncounters - 1;
    if (int rc = qb::prepare_kernel(ctx->device, (const void*)qb::delta_fused_kernel, (int)sizeof(qb::FusedRound))) return rc;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(2 * qb::LV_HEADS, segs);
    lc.blockDim = dim3(qb::FNT);
    lc.dynamicSmemBytes = sizeof(qb::FusedRound);
    lc.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = ctx->pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, qb::delta_fused_kernel, p, splits, n, ba, ba_splits, cw, a_log, dt_bias, nw, mem,
                                       sst, meta, out, (__half*)y, seg_start, seg_len, seg_slot, seg_pos0, segs, ticket,
                                       ctx->trace);
    return e == cudaSuccess ? QB_OK : (int)e;
}
