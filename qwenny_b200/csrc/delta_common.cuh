// Gated DeltaNet pieces shared by the one-launch decode mixer (deltanet.cu) and the prompt path (delta_prompt.cu): the
// rollback plan of a segment's step, and the token form of the delta rule on a thread's slice of the f32 state.
// Slot memory, plan and metadata are the reference's (kernels/qwen_deltanet.cuh:12-82; they are what its host saves,
// loads and rolls back): state [2][48][128 v][128 k] f32, banks [2][16][REP], ring [32][LQKV]; meta {end, ck, ebuf, _}.
#pragma once
#include "common.cuh"

namespace qb {

struct Plan {
    int in, r, from, ck, cbuf, ebuf;
    bool zero, wck;
};

// What a segment's step does with the slot's state: start from zeros or from buffer `in`, replay `r` accepted tokens
// from position `from` out of that buffer's bank, write the checkpoint at position ck into buffer cbuf (when wck) and
// the end state into ebuf.
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

// The state rows of a thread, LPC lanes per value column. LPC = 4, sub = rg: rows 4 (rg + 4 j) + i as x[4 j + i],
// j < 8, i < 4. LPC = 8, sub = 4 ih + rg: rows 4 (rg + 4 j) + 2 ih + e as x[2 j + e], j < 8, e < 2 (the same rows,
// split by i / 2).
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
// Replayed and fresh tokens share this function, and both lane counts add in the same order, so a replayed state is
// bit for bit the state one token per step reaches, whichever kernel ran the tokens.
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

}  // namespace qb
