// Gated DeltaNet of a decode / verify step, three entry points with the reference's own split
// (kernels/qwen_deltanet.cuh):
//  delta_conv  sum of the in-projection parts; causal depthwise conv (4 taps) over the step's tokens or the slot's
//              ring; SiLU; L2 norm of the q and k heads (q also / sqrt(128)); exp(g) and beta per value head
//              -> cv [n][CVW]                                                              (:84-131)
//  delta_rule  the gated delta rule with the two-buffer rollback plan: the f32 state slice of a block (32 value
//              columns x 128 keys of one head) lives in registers while the block walks the segment's tokens; replay
//              of accepted drafts from the bank with the same operation order as the step's own tokens; logs the
//              bank, writes the checkpoint / end state and the conv ring                     (:172-288)
//  delta_norm  per value head RMSNorm(w) * SiLU(z) -> f16 mix; then the slots' metadata      (:295-315)
// Slot memory layout, plan() and the metadata are the reference's (they are what its host saves, loads and rolls
// back): state [2][48][128 v][128 k] f32, banks [2][16][REP], ring [32][LQKV]; meta {end, ck, ebuf, _}.
#include "common.cuh"
#include "launch.h"

namespace qb {

struct Plan {
    int in, r, from, ck, cbuf, ebuf;
    bool zero, wck;
};

// What a segment's step does with the slot's state (the same in delta_rule and delta_norm)
__device__ __forceinline__ Plan make_plan(const int* meta, int slot, int p0, int len) {
    int end = meta[slot * META], ck = meta[slot * META + 1], eb = meta[slot * META + 2];
    Plan p;
    p.ck = max(p0, p0 + len - KEEP);
    p.r = 0;
    p.from = 0;
    p.zero = p0 == 0 || end < 0;
    if (p.zero) p.in = 0;
    else if (p0 == end) p.in = eb;
    else { p.in = 1 - eb; p.from = ck; p.r = min(max(p0 - ck, 0), KEEP); }
    p.wck = p.zero || p.r > 0 || p.ck > p0;
    p.cbuf = p.wck ? 1 - p.in : p.in;
    p.ebuf = 1 - p.cbuf;
    return p;
}

__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }

__device__ __forceinline__ float4 part_sum4(const float* p, int splits, int n, int t, int c) {
    float4 v = ld4(p + (size_t)t * DELTA_IN + c);
    for (int s = 1; s < splits; s++) {
        float4 x = ld4(p + ((size_t)s * n + t) * DELTA_IN + c);
        v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
    }
    return v;
}

// ------------------------------------------------------------------------------------------------ delta_conv
// grid (LQKV / 128, ceil(n / 4)), block 128: warp w handles token 4 blockIdx.y + w, channels 128 blockIdx.x ..,
// four per lane (one q, k or v head per block column)
__global__ void __launch_bounds__(128)
delta_conv_kernel(const float* p, int splits, int n, const float* ba, int ba_splits, const float* cw,
                  const float* a_log, const float* dt_bias, const float* mem, long long sst, float* cv,
                  const int* tok_slot, const int* tok_pos) {
    pdl_launch_dependents();
    const int grp = blockIdx.x, lane = threadIdx.x & 31, t = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int c = grp * 128 + lane * 4;
    float w[4][CONV_K];  // [channel][tap]
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 v = ld4(cw + (c + i) * CONV_K);
        w[i][0] = v.x; w[i][1] = v.y; w[i][2] = v.z; w[i][3] = v.w;
    }
    pdl_wait();
    if (t >= n) return;
    const int slot = tok_slot[t], pos = tok_pos[t];
    float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < CONV_K; j++) {
        int qp = pos - (CONV_K - 1) + j, tt = t - (CONV_K - 1) + j;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qp >= 0) {
            if (tt >= 0 && tok_slot[tt] == slot) x = part_sum4(p, splits, n, tt, c);
            else x = ld4(mem + slot * sst + SLOT_RING + (size_t)(qp & (CR - 1)) * LQKV + c);
        }
        y[0] += w[0][j] * x.x; y[1] += w[1][j] * x.y; y[2] += w[2][j] * x.z; y[3] += w[3][j] * x.w;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) { y[i] = silu(y[i]); ss += y[i] * y[i]; }
    if (grp < 2 * LK_HEADS) {
        float sc = rsqrtf(warp_sum(ss) + 1e-6f);
        if (grp < LK_HEADS) sc *= rsqrtf((float)LKD);
#pragma unroll
        for (int i = 0; i < 4; i++) y[i] *= sc;
    }
    *(float4*)(cv + (size_t)t * CVW + c) = make_float4(y[0], y[1], y[2], y[3]);
    if (grp == 0) {
        for (int v = lane; v < LV_HEADS; v += 32) {
            float b = 0.f, a = 0.f;
            for (int s = 0; s < ba_splits; s++) {
                const float* r = ba + ((size_t)s * n + t) * (2 * LV_HEADS);
                b += r[v];
                a += r[LV_HEADS + v];
            }
            a += dt_bias[v];
            float sp = a > 20.f ? a : log1pf(expf(a));
            cv[(size_t)t * CVW + LQKV + v] = expf(-expf(a_log[v]) * sp);
            cv[(size_t)t * CVW + LQKV + LV_HEADS + v] = 1.f / (1.f + expf(-b));
        }
    }
}

// ------------------------------------------------------------------------------------------------ delta_rule
// Geometry: 128 threads per block, LPC lanes per value column, 128 / LPC columns per block. LPC = 4 (32 key rows per
// thread, the reference's split) for decode steps; LPC = 8 (16 rows per thread, twice the blocks and warps) for
// prompt segments, where the per-token dependency chain, not the state traffic, sets the pace. Both add a column's
// products in the same order, so a state is bit for bit the same whichever ran.
constexpr int RCOLS = 32;               // value columns per block at most (LPC = 4)
constexpr int RNT = 128;                // threads
constexpr int TCH = 8;                  // tokens staged per round (two rounds of shared memory: one computing, one landing)

struct Round {
    float q[TCH][LKD], k[TCH][LKD], v[TCH][RCOLS], e[TCH], b[TCH], kq[TCH];
};

// The rows of a thread. LPC = 4, sub = rg: rows 4 (rg + 4 j) + i as x[4 j + i], j < 8, i < 4.
// LPC = 8, sub = 4 ih + rg: rows 4 (rg + 4 j) + 2 ih + e as x[2 j + e], j < 8, e < 2 (the same rows, split by i / 2).
template <int LPC>
__device__ __forceinline__ void ld_rows(float* x, const float* src, int sub) {
    if (LPC == 4) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float4 v = ld4(src + 4 * (sub + 4 * j));
            x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float2 v = *(const float2*)(src + 4 * ((sub & 3) + 4 * j) + 2 * (sub >> 2));
            x[2 * j] = v.x; x[2 * j + 1] = v.y;
        }
    }
}
template <int LPC>
__device__ __forceinline__ void st_rows(float* dst, const float* x, int sub) {
    if (LPC == 4) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            *(float4*)(dst + 4 * (sub + 4 * j)) = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++)
            *(float2*)(dst + 4 * ((sub & 3) + 4 * j) + 2 * (sub >> 2)) = make_float2(x[2 * j], x[2 * j + 1]);
    }
}
__device__ __forceinline__ float col_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
// S^T x for the thread's rows: the partial sum of the rows with the same i (row % 4) runs over j in order; then
// (d0 + d1) + (d2 + d3) (inside the thread for LPC = 4, across the ih lanes for LPC = 8), then the column's 4 rg lanes.
// Replayed and fresh tokens share this function, so a replayed state is bit for bit the state one token per step
// reaches.
template <int LPC>
__device__ __forceinline__ float dot_rows(const float* S, const float* x) {
    if (LPC == 4) {
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 32; j++) d4[j & 3] += S[j] * x[j];
        return col_sum((d4[0] + d4[1]) + (d4[2] + d4[3]));
    } else {
        float d2[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 16; j++) d2[j & 1] += S[j] * x[j];
        float s = d2[0] + d2[1];
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        return col_sum(s);
    }
}

template <int LPC>
__global__ void __launch_bounds__(RNT)
delta_rule_kernel(const float* p, int splits, int n, const float* cv, float* mem, long long sst, const int* meta,
                  float* out, const int* seg_start, const int* seg_len, const int* seg_slot, const int* seg_pos0) {
    constexpr int COLS = RNT / LPC, RPT = LKD / LPC, SLICES = LVD / COLS;
    __shared__ __align__(16) Round Rb[2];  // the round being computed and the one in flight (cp.async)
    pdl_launch_dependents();
    const int slice = blockIdx.x, h = blockIdx.y, sg = blockIdx.z, kh = h / (LV_HEADS / LK_HEADS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, rg = lane % LPC;  // rg: the lane's place in its column
    const int lc = warp * (32 / LPC) + lane / LPC, col = slice * COLS + lc;
    // the segment arrays and the slot metadata were written before this step's first kernel
    const int t0 = seg_start[sg], len = seg_len[sg], slot = seg_slot[sg], p0 = seg_pos0[sg];
    const Plan pl = make_plan(meta, slot, p0, len);
    float* sm0 = mem + slot * sst;
    auto sbuf = [&](int b) { return sm0 + (size_t)b * SLOT_STATE + ((size_t)h * LVD + col) * LKD; };
    auto entry = [&](int b, int pos) { return sm0 + 2 * SLOT_STATE + (size_t)b * SLOT_BANK + (size_t)(pos % KEEP) * REP; };

    // the state does not depend on this step's earlier kernels: in flight before the wait
    float S[RPT];
    if (pl.zero) {
#pragma unroll
        for (int i = 0; i < RPT; i++) S[i] = 0.f;
    } else {
        ld_rows<LPC>(S, sbuf(pl.in), rg);
    }
    // replay the accepted tokens between the checkpoint and the restart position, from the bank
    for (int i = 0; i < pl.r; i++) {
        const float* e = entry(pl.in, pl.from + i);
        float k[RPT];
        ld_rows<LPC>(k, e + kh * LKD, rg);
        float dk = dot_rows<LPC>(S, k);
        float ex = e[LK_HEADS * LKD + LV_HEADS * LVD + h], be = e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h];
        float delta = (e[LK_HEADS * LKD + h * LVD + col] - ex * dk) * be;
#pragma unroll
        for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
    }
    pdl_wait();

    // stage a round with asynchronous copies: q and k of the key head, the block's v columns, the gates of head h
    auto stage = [&](Round& R, int c0) {
        const int m = min(TCH, len - c0);
        for (int x = tid; x < m * (LKD / 4); x += RNT) {
            int tk = x / (LKD / 4), d = (x % (LKD / 4)) * 4;
            const float* row = cv + (size_t)(t0 + c0 + tk) * CVW + kh * LKD + d;
            cp_async16(&R.q[tk][d], row);
            cp_async16(&R.k[tk][d], row + LK_HEADS * LKD);
        }
        for (int x = tid; x < m * (COLS / 4); x += RNT) {
            int tk = x / (COLS / 4), d = (x % (COLS / 4)) * 4;
            cp_async16(&R.v[tk][d], cv + (size_t)(t0 + c0 + tk) * CVW + 2 * LK_HEADS * LKD + h * LVD + slice * COLS + d);
        }
        if (tid < 2 * m) {
            int tk = tid >> 1, which = tid & 1;
            cp_async4(&(which ? R.b : R.e)[tk], cv + (size_t)(t0 + c0 + tk) * CVW + LQKV + which * LV_HEADS + h);
        }
        cp_async_commit();
    };
    stage(Rb[0], 0);
    for (int c0 = 0, rb = 0; c0 < len; c0 += TCH, rb ^= 1) {
        const int m = min(TCH, len - c0);
        Round& R = Rb[rb];
        cp_async_wait_all();
        __syncthreads();  // the round has landed, and every thread is past the previous round (its buffer is free)
        if (c0 + TCH < len) stage(Rb[rb ^ 1], c0 + TCH);
        // k . q per token: warp w takes tokens w, w + 4
        for (int tk = warp; tk < m; tk += RNT / 32) {
            float4 a = ld4(&R.q[tk][lane * 4]), b = ld4(&R.k[tk][lane * 4]);
            float x = warp_sum(a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w);
            if (lane == 0) R.kq[tk] = x;
        }
        // the delta rule inputs of the tokens from the new checkpoint on, for a later restart
        for (int tk = max(0, pl.ck - (p0 + c0)); tk < m; tk++) {
            float* e = entry(pl.cbuf, p0 + c0 + tk);
            if (slice == 0 && h % (LV_HEADS / LK_HEADS) == 0 && tid < LKD / 4)
                *(float4*)(e + kh * LKD + tid * 4) = ld4(&R.k[tk][tid * 4]);
            if (tid < COLS) e[LK_HEADS * LKD + h * LVD + slice * COLS + tid] = R.v[tk][tid];
            if (slice == 0 && tid == 0) {
                e[LK_HEADS * LKD + LV_HEADS * LVD + h] = R.e[tk];
                e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h] = R.b[tk];
            }
        }
        __syncthreads();
        for (int tk = 0; tk < m; tk++) {
            if (pl.wck && p0 + c0 + tk == pl.ck) st_rows<LPC>(sbuf(pl.cbuf), S, rg);
            float k[RPT], q[RPT];
            ld_rows<LPC>(k, R.k[tk], rg);
            ld_rows<LPC>(q, R.q[tk], rg);
            float dk = dot_rows<LPC>(S, k), dq = dot_rows<LPC>(S, q);
            float ex = R.e[tk], delta = (R.v[tk][lc] - ex * dk) * R.b[tk];
            if (rg == 0) out[(size_t)(t0 + c0 + tk) * MIX + h * LVD + col] = ex * dq + delta * R.kq[tk];
#pragma unroll
            for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
        }
    }
    st_rows<LPC>(sbuf(pl.ebuf), S, rg);
    // conv ring: the conv inputs of the segment's last CR tokens, this block's share of the channels
    const int NB = SLICES * LV_HEADS, CH = (LQKV + NB - 1) / NB;
    const int cb = (h * SLICES + slice) * CH, ch = max(0, min(CH, LQKV - cb)), mm = min(len, CR);
    for (int i = tid; i < mm * ch; i += RNT) {
        int tk = len - mm + i / ch, c = cb + i % ch;
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += p[((size_t)s * n + t0 + tk) * DELTA_IN + c];
        sm0[SLOT_RING + (size_t)((p0 + tk) & (CR - 1)) * LQKV + c] = v;
    }
}

constexpr int LPC = 4, RPT = LKD / LPC;  // the decode geometry, shared with the one-launch mixer below

// ------------------------------------------------------------------------------------------------ delta_norm
constexpr int NORM_HEADS = 16;
__global__ void __launch_bounds__(NORM_HEADS * 32)
delta_norm_kernel(const float* p, int splits, int n, const float* nw, const float* out, __half* y, int* meta,
                  const int* seg_len, const int* seg_slot, const int* seg_pos0, int segs) {
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y * NORM_HEADS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    float4 w = ld4(nw + lane * 4);
    pdl_wait();
    size_t o = (size_t)t * MIX + h * LVD + lane * 4;
    float4 v = ld4(out + o), z = part_sum4(p, splits, n, t, LQKV + h * LVD + lane * 4);
    float r = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) / LVD + EPS);
    *(uint2*)(y + o) = make_uint2(pack_half2(w.x * (v.x * r) * silu(z.x), w.y * (v.y * r) * silu(z.y)),
                                  pack_half2(w.z * (v.z * r) * silu(z.z), w.w * (v.w * r) * silu(z.w)));
    if (t == 0 && blockIdx.y == 0) {
        for (int s = threadIdx.x; s < segs; s += blockDim.x) {
            int slot = seg_slot[s], p0 = seg_pos0[s], len = seg_len[s];
            Plan pl = make_plan(meta, slot, p0, len);
            meta[slot * META] = p0 + len;
            meta[slot * META + 1] = pl.ck;
            meta[slot * META + 2] = pl.ebuf;
        }
    }
}

}  // namespace qb

using namespace qb;

extern "C" {

int qb_delta_conv(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* ba, int ba_splits,
                  const float* cw, const float* a_log, const float* dt_bias, const float* mem, long long sst,
                  float* cv, const int* tok_slot, const int* tok_pos) {
    if (!ctx || !p || !ba || !cw || !a_log || !dt_bias || !mem || !cv || !tok_slot || !tok_pos || n <= 0 ||
        splits < 1 || ba_splits < 1)
        return QB_ERR_ARG;
    return launch(ctx, delta_conv_kernel, dim3(LQKV / 128, (n + 3) / 4), dim3(128), 0, (cudaStream_t)stream, p, splits,
                  n, ba, ba_splits, cw, a_log, dt_bias, mem, sst, cv, tok_slot, tok_pos);
}

int qb_delta_rule(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* cv, float* mem,
                  long long sst, const int* meta, float* out, const int* seg_start, const int* seg_len,
                  const int* seg_slot, const int* seg_pos0, int segs) {
    if (!ctx || !p || !cv || !mem || !meta || !out || !seg_start || !seg_len || !seg_slot || !seg_pos0 || n <= 0 ||
        segs <= 0 || splits < 1)
        return QB_ERR_ARG;
    // steps with prompt segments take the finer geometry (same bits, more blocks and warps)
    if (n >= 64)
        return launch(ctx, delta_rule_kernel<8>, dim3(LVD / (RNT / 8), LV_HEADS, segs), dim3(RNT), 0, (cudaStream_t)stream,
                      p, splits, n, cv, mem, sst, meta, out, seg_start, seg_len, seg_slot, seg_pos0);
    return launch(ctx, delta_rule_kernel<4>, dim3(LVD / (RNT / 4), LV_HEADS, segs), dim3(RNT), 0, (cudaStream_t)stream, p,
                  splits, n, cv, mem, sst, meta, out, seg_start, seg_len, seg_slot, seg_pos0);
}

int qb_delta_norm(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* nw, const float* out,
                  void* y, int* meta, const int* seg_len, const int* seg_slot, const int* seg_pos0, int segs) {
    if (!ctx || !p || !nw || !out || !y || !meta || !seg_len || !seg_slot || !seg_pos0 || n <= 0 || segs <= 0 ||
        splits < 1)
        return QB_ERR_ARG;
    return launch(ctx, delta_norm_kernel, dim3(n, LV_HEADS / NORM_HEADS), dim3(NORM_HEADS * 32), 0,
                  (cudaStream_t)stream, p, splits, n, nw, out, (__half*)y, meta, seg_len, seg_slot, seg_pos0, segs);
}

}  // extern "C"

// =================================================================================================== fused mixer
// delta_conv + delta_rule + delta_norm of a decode / verify step in ONE launch: a cluster of two blocks per (value
// head h, segment), each with half of the head's 128 value columns (256 threads: column tid / 4, rows
// 4 (tid % 4 + 4 j) + i, the same layout and operation order as delta_rule_kernel<4>, so both give the same bits). A
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
        // ---- ONE round trip of independent loads: conv inputs (step rows or ring), z, gates, the ring share; all of
        // them into registers first, the shared-memory stores after
        constexpr int NROW = TCH + CONV_K - 1, NZV = (TCH * FCOLS + FNT - 1) / FNT;
        // conv inputs: thread tid takes channel tid of every row, and threads below FCH - FNT also channel FNT + tid
        float xv[NROW][2], zv[NZV], ringv[4], gate = 0.f;
        const int gc0 = gchan(tid), gc1 = gchan(min(FNT + tid, FCH - 1));
        const bool two = FNT + tid < FCH;
#pragma unroll
        for (int row = 0; row < NROW; row++) {
            xv[row][0] = xv[row][1] = 0.f;
            const int si = c0 + row - (CONV_K - 1), qp = p0 + si;
            if (row < m + CONV_K - 1 && qp >= 0) {
                if (si >= 0) {
                    // (one split is the common case: a plain load, so that every row's loads are in flight together;
                    // a warp issues in order, and a sum inside a loop would wait for each load before the next)
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
