// The small per-token kernels of a step: embedding lookup, RMSNorm, residual + split sum + RMSNorm, f32 -> f16 cast,
// split sum, the seen-token bitsets, row gather. One entry point per kernel of the reference
// (kernels/dense.cuh, kernels/qwen.cu:57-80,136-143, kernels/sampling.cuh:14-26, kernels/marlin.cuh:605-608).
// They move kilobytes; what matters is latency, so each token row is spread over a whole block with 128-bit
// accesses and every kernel can be launched ahead of its predecessor (pdl_wait guards the first dependent read).
#include "common.cuh"
#include "launch.h"

namespace qb {

constexpr int ROW_THREADS = 640;         // H / 8: one 8-element vector per thread
static_assert(H % 8 == 0 && H / 8 == ROW_THREADS, "a row of H is one vector of 8 per thread");

// out[t] = E[ids[t]] (bf16 -> f32); the first nkeys blocks clear the step's argmax keys
__global__ void __launch_bounds__(ROW_THREADS) embed_kernel(const __nv_bfloat16* E, const int* ids, float* out,
                                                            unsigned long long* keys, int nkeys) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    if (threadIdx.x == 0 && t < nkeys) keys[t] = 0;
    const uint4* row = (const uint4*)(E + (size_t)ids[t] * H);
    uint4 v = row[threadIdx.x];
    const __nv_bfloat162* b = (const __nv_bfloat162*)&v;
    float4* o = (float4*)(out + (size_t)t * H) + 2 * threadIdx.x;
    float2 a0 = __bfloat1622float2(b[0]), a1 = __bfloat1622float2(b[1]), a2 = __bfloat1622float2(b[2]),
           a3 = __bfloat1622float2(b[3]);
    o[0] = make_float4(a0.x, a0.y, a1.x, a1.y);
    o[1] = make_float4(a2.x, a2.y, a3.x, a3.y);
}

// out[t] = row ids[t] of an int8 embedding table as stored: (E - 128) * its scale per 128 columns (S [rows][H / 128]).
// A thread takes 8 codes (one 64-bit load; the table may sit in mapped host memory, so the row is fetched in as few,
// as wide requests as the block has threads) and writes two float4; the first nkeys blocks clear the argmax keys.
__global__ void __launch_bounds__(ROW_THREADS) embed_q8_kernel(const uint8_t* E, const float* S, const int* ids, float* out,
                                                               unsigned long long* keys, int nkeys) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (threadIdx.x == 0 && t < nkeys) keys[t] = 0;
    const size_t row = (size_t)ids[t];
    const uint2 v = ((const uint2*)(E + row * H))[threadIdx.x];
    const float sc = S[row * (H / 128) + threadIdx.x / 16];
    float4* o = (float4*)(out + (size_t)t * H) + 2 * threadIdx.x;
    auto code = [](uint32_t w, int b) { return (float)((int)((w >> (8 * b)) & 255u) - 128); };
    o[0] = make_float4(code(v.x, 0) * sc, code(v.x, 1) * sc, code(v.x, 2) * sc, code(v.x, 3) * sc);
    o[1] = make_float4(code(v.y, 0) * sc, code(v.y, 1) * sc, code(v.y, 2) * sc, code(v.y, 3) * sc);
}

// One learned 16-row block into a Marlin matrix of n rows: thread (k16, lane) of the block's words [k16][32] writes the
// word of lane `lane` and block `blk` of the 64-row group c64 (per k16 step 2 n words, at 128 c64 + 4 lane + blk);
// threads (k16 < tables * groups, lane < 16) also write row lane's scale of group k16 to its permuted place.
__global__ void __launch_bounds__(256) put_block_kernel(uint32_t* B, __half* S, const uint32_t* words, const __half* sc,
                                                        int n, int c64, int blk, int groups, int tables, int k16s) {
    pdl_launch_dependents();
    pdl_wait();
    const int k16 = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (k16 >= k16s) return;
    B[(size_t)k16 * 2 * n + (size_t)(c64 * 32 + lane) * 4 + blk] = words[k16 * 32 + lane];
    if (k16 < groups * tables && lane < 16) {
        const int c = blk * 16 + lane;
        S[(size_t)k16 * n + c64 * 64 + 8 * (c % 8) + c / 8] = sc[k16 * 16 + lane];
    }
}

__device__ __forceinline__ void store_norm8(__half* y, const float* v, const float* w, float r) {
    uint4 o;
    o.x = pack_half2(w[0] * (v[0] * r), w[1] * (v[1] * r));
    o.y = pack_half2(w[2] * (v[2] * r), w[3] * (v[3] * r));
    o.z = pack_half2(w[4] * (v[4] * r), w[5] * (v[5] * r));
    o.w = pack_half2(w[6] * (v[6] * r), w[7] * (v[7] * r));
    *(uint4*)y = o;
}

// y = w * x / rms(x) -> f16, one block per token
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_kernel(const float* x, const float* w, __half* y, float eps) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    float wv[8];
    *(float4*)&wv[0] = ((const float4*)w)[2 * threadIdx.x];
    *(float4*)&wv[4] = ((const float4*)w)[2 * threadIdx.x + 1];
    pdl_wait();
    const float4* xr = (const float4*)(x + (size_t)blockIdx.x * H) + 2 * threadIdx.x;
    float v[8];
    *(float4*)&v[0] = xr[0];
    *(float4*)&v[4] = xr[1];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss += v[i] * v[i];
    float r = rsqrtf(block_sum(ss, sh) / H + eps);
    store_norm8(y + (size_t)blockIdx.x * H + 8 * threadIdx.x, v, wv, r);
}

// h += sum over splits of x [split][n][H]; y = w_next * h / rms(h) -> f16
__global__ void __launch_bounds__(ROW_THREADS) add_rmsnorm_kernel(float* h, const float* x, int splits, int n,
                                                                  const float* w_next, __half* y, float eps) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    float wv[8];
    *(float4*)&wv[0] = ((const float4*)w_next)[2 * threadIdx.x];
    *(float4*)&wv[4] = ((const float4*)w_next)[2 * threadIdx.x + 1];
    pdl_wait();
    size_t base = (size_t)blockIdx.x * H + 8 * threadIdx.x;
    float v[8];
    *(float4*)&v[0] = *(const float4*)(h + base);
    *(float4*)&v[4] = *(const float4*)(h + base + 4);
    for (int s = 0; s < splits; s++) {
        const float* p = x + (size_t)s * n * H + base;
        float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
    }
    *(float4*)(h + base) = *(float4*)&v[0];
    *(float4*)(h + base + 4) = *(float4*)&v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss += v[i] * v[i];
    float r = rsqrtf(block_sum(ss, sh) / H + eps);
    store_norm8(y + base, v, wv, r);
}

__global__ void __launch_bounds__(256) to_xin_kernel(const float* x, __half* y, int len) {
    pdl_launch_dependents();
    pdl_wait();
    int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    for (; i + 3 < len; i += gridDim.x * blockDim.x * 4) {
        float4 v = *(const float4*)(x + i);
        *(uint2*)(y + i) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    }
    if (blockIdx.x == 0 && threadIdx.x < (len & 3)) y[(len & ~3) + threadIdx.x] = __float2half_rn(x[(len & ~3) + threadIdx.x]);
}

__global__ void __launch_bounds__(256) sum_parts_kernel(const float* x, int splits, int n, int ld, float* y) {
    pdl_launch_dependents();
    pdl_wait();
    for (int c = threadIdx.x; c < ld; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += x[((size_t)s * n + blockIdx.x) * ld + c];
        y[(size_t)blockIdx.x * ld + c] = v;
    }
}

// One block per segment: a segment at position 0 clears its slot's set, then its marked tokens are set
__global__ void __launch_bounds__(256) mark_seen_kernel(unsigned* seen, const int* mark, const int* mark_at,
                                                        const int* seg_slot, const int* seg_pos0, int seen_words) {
    pdl_launch_dependents();
    pdl_wait();
    int sg = blockIdx.x;
    unsigned* sb = seen + (size_t)seg_slot[sg] * seen_words;
    if (seg_pos0[sg] == 0) {
        for (int i = threadIdx.x; i < seen_words; i += blockDim.x) sb[i] = 0;
        __syncthreads();
    }
    for (int i = mark_at[sg] + threadIdx.x; i < mark_at[sg + 1]; i += blockDim.x) {
        int id = mark[i];
        atomicOr(sb + (id >> 5), 1u << (id & 31));
    }
}

__global__ void __launch_bounds__(128) gather_rows_kernel(const uint4* x, const int* rows, uint4* out, int k8) {
    pdl_launch_dependents();
    pdl_wait();
    const uint4* row = x + (size_t)rows[blockIdx.x] * k8;
    for (int c = threadIdx.x; c < k8; c += blockDim.x) out[(size_t)blockIdx.x * k8 + c] = row[c];
}

// MTP input (the draft layer of speculative decoding), one block per token t:
// y[t] = [pre_e * e / rms(e); pre_h * g / rms(g)] as f16 [2 H], e = the token's embedding (emb [n][H], from embed),
// g = fw * h[rows[t]] / rms(h[rows[t]]): h is the residual stream before a final norm fw (the target's and its final
// norm, or the MTP layer's own of the step before and its norm). Replaces mtp_in, kernels/qwen.cu:100-133.
__global__ void __launch_bounds__(ROW_THREADS) mtp_in_kernel(const float* emb, const float* h, const int* rows,
                                                             const float* fw, const float* pre_e, const float* pre_h,
                                                             __half* y, float eps) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    float wf[8], we[8], wh[8];
    const int c = 8 * threadIdx.x;
    *(float4*)&wf[0] = *(const float4*)(fw + c); *(float4*)&wf[4] = *(const float4*)(fw + c + 4);
    *(float4*)&we[0] = *(const float4*)(pre_e + c); *(float4*)&we[4] = *(const float4*)(pre_e + c + 4);
    *(float4*)&wh[0] = *(const float4*)(pre_h + c); *(float4*)&wh[4] = *(const float4*)(pre_h + c + 4);
    pdl_wait();
    const float* er = emb + (size_t)blockIdx.x * H + c;
    const float* hr = h + (size_t)rows[blockIdx.x] * H + c;
    float e[8], g[8];
    *(float4*)&e[0] = *(const float4*)er; *(float4*)&e[4] = *(const float4*)(er + 4);
    *(float4*)&g[0] = *(const float4*)hr; *(float4*)&g[4] = *(const float4*)(hr + 4);
    float se = 0.f, sg = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) { se += e[i] * e[i]; sg += g[i] * g[i]; }
    const float re = rsqrtf(block_sum(se, sh) / H + eps), rg = rsqrtf(block_sum(sg, sh) / H + eps);
    float sg2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) { g[i] = wf[i] * (g[i] * rg); sg2 += g[i] * g[i]; }
    const float rg2 = rsqrtf(block_sum(sg2, sh) / H + eps);
    __half* yr = y + (size_t)blockIdx.x * 2 * H + c;
    store_norm8(yr, e, we, re);
    store_norm8(yr + H, g, wh, rg2);
}

// The greedy case of the reference's draft sampler (draft_sample with top_k 1, kernels/sampling.cuh:298; the row of
// argmax_draft_row, src/sample.rs:58-62): draft i of a chain is the argmax of its logit row, which the argmax epilogue
// of the head product left in keys[i] (largest logit, lowest index among equals); a draft head's columns map to tokens
// through head_ids. Writes the draft as the next MTP step's token id and at chain[i][t].
__global__ void __launch_bounds__(64) draft_pick_kernel(const unsigned long long* keys, const int* head_ids, int n_out,
                                                        int* next_ids, int* chain, int chain_ld, int t) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_out) return;
    const int idx = (int)(0xffffffffu - (uint32_t)(keys[i] & 0xffffffffu));
    const int tok = head_ids ? head_ids[idx] : idx;
    next_ids[i] = tok;
    chain[(size_t)i * chain_ld + t] = tok;
}

}  // namespace qb

using namespace qb;

extern "C" {

int qb_mtp_in(qb_ctx* ctx, void* stream, const float* emb, const float* h, const int* rows, const float* fw,
              const float* pre_e, const float* pre_h, void* y, float eps, int n) {
    if (!ctx || !emb || !h || !rows || !fw || !pre_e || !pre_h || !y || n <= 0) return QB_ERR_ARG;
    return launch(ctx, mtp_in_kernel, dim3(n), dim3(ROW_THREADS), 0, (cudaStream_t)stream, emb, h, rows, fw, pre_e, pre_h,
                  (__half*)y, eps);
}

int qb_draft_pick(qb_ctx* ctx, void* stream, const unsigned long long* keys, const int* head_ids, int n_out,
                  int* next_ids, int* chain, int chain_ld, int t) {
    if (!ctx || !keys || !next_ids || !chain || n_out <= 0 || t < 0 || t >= chain_ld) return QB_ERR_ARG;
    return launch(ctx, draft_pick_kernel, dim3((n_out + 63) / 64), dim3(64), 0, (cudaStream_t)stream, keys, head_ids, n_out,
                  next_ids, chain, chain_ld, t);
}

int qb_embed(qb_ctx* ctx, void* stream, const void* E, const int* ids, float* out, unsigned long long* keys,
             int nkeys, int n) {
    if (!ctx || !E || !ids || !out || n <= 0 || nkeys > n || (nkeys > 0 && !keys)) return QB_ERR_ARG;
    return launch(ctx, embed_kernel, dim3(n), dim3(ROW_THREADS), 0, (cudaStream_t)stream, (const __nv_bfloat16*)E, ids,
                  out, keys, nkeys);
}

int qb_embed_q8(qb_ctx* ctx, void* stream, const void* E, const float* S, const int* ids, float* out,
                unsigned long long* keys, int nkeys, int n) {
    if (!ctx || !E || !S || !ids || !out || n <= 0 || nkeys > n || (nkeys > 0 && !keys)) return QB_ERR_ARG;
    return launch(ctx, embed_q8_kernel, dim3(n), dim3(ROW_THREADS), 0, (cudaStream_t)stream, (const uint8_t*)E, S, ids,
                  out, keys, nkeys);
}

int qb_marlin_put_block(qb_ctx* ctx, void* stream, void* B, void* S, const void* words, const void* sc, int n, int c64,
                        int blk, int groups, int tables, int k16s) {
    if (!ctx || !B || !S || !words || !sc || n <= 0 || n % 64 || c64 < 0 || (c64 + 1) * 64 > n || blk < 0 || blk > 3 ||
        groups <= 0 || tables < 1 || tables > 2 || k16s < groups * tables)
        return QB_ERR_ARG;
    return launch(ctx, put_block_kernel, dim3((k16s + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (uint32_t*)B, (__half*)S,
                  (const uint32_t*)words, (const __half*)sc, n, c64, blk, groups, tables, k16s);
}

int qb_rmsnorm(qb_ctx* ctx, void* stream, const float* x, const float* w, void* y, float eps, int n) {
    if (!ctx || !x || !w || !y || n <= 0) return QB_ERR_ARG;
    return launch(ctx, rmsnorm_kernel, dim3(n), dim3(ROW_THREADS), 0, (cudaStream_t)stream, x, w, (__half*)y, eps);
}

int qb_add_rmsnorm(qb_ctx* ctx, void* stream, float* h, const float* x, int splits, int n, const float* w_next,
                   void* y, float eps) {
    if (!ctx || !h || !x || !w_next || !y || n <= 0 || splits < 1) return QB_ERR_ARG;
    return launch(ctx, add_rmsnorm_kernel, dim3(n), dim3(ROW_THREADS), 0, (cudaStream_t)stream, h, x, splits, n,
                  w_next, (__half*)y, eps);
}

int qb_to_xin(qb_ctx* ctx, void* stream, const float* x, void* y, int len) {
    if (!ctx || !x || !y || len <= 0) return QB_ERR_ARG;
    int blocks = (len + 1023) / 1024;
    if (blocks > 1024) blocks = 1024;
    return launch(ctx, to_xin_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (__half*)y, len);
}

int qb_sum_parts(qb_ctx* ctx, void* stream, const float* x, int splits, int n, int ld, float* y) {
    if (!ctx || !x || !y || n <= 0 || ld <= 0 || splits < 1) return QB_ERR_ARG;
    return launch(ctx, sum_parts_kernel, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, splits, n, ld, y);
}

int qb_mark_seen(qb_ctx* ctx, void* stream, unsigned* seen, const int* mark, const int* mark_at, const int* seg_slot,
                 const int* seg_pos0, int segs, int vocab) {
    if (!ctx || !seen || !mark || !mark_at || !seg_slot || !seg_pos0 || segs <= 0 || vocab % 32) return QB_ERR_ARG;
    return launch(ctx, mark_seen_kernel, dim3(segs), dim3(256), 0, (cudaStream_t)stream, seen, mark, mark_at, seg_slot,
                  seg_pos0, vocab / 32);
}

int qb_marlin_gather(qb_ctx* ctx, void* stream, const void* x, const int* rows, void* out, int k8, int n) {
    if (!ctx || !x || !rows || !out || n <= 0 || k8 <= 0) return QB_ERR_ARG;
    return launch(ctx, gather_rows_kernel, dim3(n), dim3(128), 0, (cudaStream_t)stream, (const uint4*)x, rows,
                  (uint4*)out, k8);
}

}  // extern "C"
