// Gated GQA attention of a decode / verify step over the int8 KV cache.
//  attn_prep    per token: sum of the in-projection parts, q/k RMSNorm(1+w), partial RoPE, q scaled to base-2 scores,
//               sigmoid gate -> out, k and v quantised into the cache in the reference's byte order
//               (replaces attn_prep + kv_store, kernels/qwen.cu:156-202, kernels/attn.cuh:50-64)
//  attn_decode  split-K flash-decode: block (segment, kv head, key split) streams its run of keys and values with
//               bulk async copies into a shared-memory ring (keys are [pos][256] and values [pos/16][256][16] bytes
//               per head, both contiguous per run) while RT x 4 warps compute S = Q K^T and O += P V on tensor cores
//               with a warp-level base-2 online softmax, straight from the int8 bytes (prmt to 1152 + q halves, the
//               offset folded out through the row sums as the reference does, kernels/attn.cuh:38-40,198-234)
//               (replaces attn_mq_tc<RT>, kernels/attn.cuh:77-261)
//  attn_combine merges the splits of a (token, head) in split order, multiplies into the gated output and can write
//               the f16 copy the out-projection reads (replaces attn_combine + to_xin, kernels/attn.cuh:271-325,
//               kernels/qwen.cu:136-138)
// The size of a key split is a function of the key count alone (dec_chunk), so a token's sums are the same whether
// it runs alone or with drafts.
#include "attn_common.cuh"
#include "launch.h"

namespace qb {

// ------------------------------------------------------------------------------------------------ attn_prep
// grid (n tokens, 2): block (t, 0) makes the 24 query heads and their gates (a warp per head), block (t, 1) the 4 key
// and 4 value heads and stores them in the cache. A warp's lane owns dims lane + 32 j of its head: the RoPE pair
// (d, d + 32) of the 64 rotated dims is then elements 0 and 1 of one lane, and the sum of squares adds the lane's eight
// values in dim order, then the lanes as a butterfly: the order that makes the int8 codes the reference's, bit for bit.
constexpr int HEAD_VALS = HD / 32;

struct HeadRow {
    float v[HEAD_VALS];
};

// the head row at `col` of token t's in-projection, summed over the split-K parts
__device__ __forceinline__ HeadRow head_row(const float* part, int splits, int n, int t, int col, int lane) {
    HeadRow r;
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) r.v[j] = 0.f;
    for (int sp = 0; sp < splits; sp++) {
        const float* p = part + ((size_t)sp * n + t) * ATTN_IN + col + lane;
#pragma unroll
        for (int j = 0; j < HEAD_VALS; j++) r.v[j] += p[32 * j];
    }
    return r;
}

// RMSNorm with the head's weight (pre-biased 1 + w), then the rotation of the first 64 dims by pos * inv_freq
__device__ __forceinline__ void norm_and_rotate(HeadRow& r, const float* w_lane, float angle) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) ss += r.v[j] * r.v[j];
    const float rms = rsqrtf(warp_sum(ss) / HD + EPS);
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) r.v[j] = w_lane[j] * (r.v[j] * rms);
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float a = r.v[0], b = r.v[1];
    r.v[0] = a * cs - b * sn;
    r.v[1] = b * cs + a * sn;
}

// One head row into the int8 cache: a scale per (position, head) = max |v| / 127, code = round(v * 127 / max) + 128.
// KEY: the row's place is [pos][256] in kslot order; else the 16-position block [pos / 16][256][16] in vslot order.
template <bool KEY>
__device__ __forceinline__ void store_quantised(const HeadRow& r, uint8_t* head_cache, float* head_scales, int pos, int lane) {
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) mx = fmaxf(mx, fabsf(r.v[j]));
    mx = warp_max(mx);
    const float inv = mx > 0.f ? 127.f / mx : 0.f;
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) {
        const int d = lane + 32 * j;
        const uint8_t code = (uint8_t)(__float2int_rn(r.v[j] * inv) + 128);
        head_cache[KEY ? (size_t)pos * HD + kslot(d) : vslot(pos, d)] = code;
    }
    if (lane == 0) head_scales[pos] = mx / 127.f;
}

__global__ void __launch_bounds__(32 * NH)
attn_prep_kernel(const float* part, int splits, int n, const float* q_norm, const float* k_norm, const float* inv_freq,
                 float qscale, float* q, float* out, uint8_t* kc, uint8_t* vc, float* ks, float* vs,
                 const int* tok_slot, const int* tok_pos, int cap) {
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool cache_block = blockIdx.y == 1;
    if (cache_block && warp >= 2 * NKV) return;
    // the norm weight of the lane's dims and its rotation frequency do not depend on earlier kernels
    const bool normed = !cache_block || warp < NKV;
    float w_lane[HEAD_VALS];
#pragma unroll
    for (int j = 0; j < HEAD_VALS; j++) w_lane[j] = normed ? (cache_block ? k_norm : q_norm)[lane + 32 * j] : 0.f;
    const float freq = inv_freq[lane];
    pdl_wait();
    const int pos = tok_pos[t];
    if (!cache_block) {
        // query head `warp`: rows [q; gate] of the head are adjacent in the in-projection
        HeadRow qr = head_row(part, splits, n, t, warp * 2 * HD, lane);
        const HeadRow gate = head_row(part, splits, n, t, warp * 2 * HD + HD, lane);
        norm_and_rotate(qr, w_lane, (float)pos * freq);
        float* qo = q + ((size_t)t * NH + warp) * HD + lane;
        float* go = out + (size_t)t * MIX + warp * HD + lane;
#pragma unroll
        for (int j = 0; j < HEAD_VALS; j++) {
            qo[32 * j] = qr.v[j] * qscale;
            go[32 * j] = 1.f / (1.f + expf(-gate.v[j]));
        }
        return;
    }
    const int slot = tok_slot[t], g = warp % NKV;
    if (warp < NKV) {
        HeadRow kr = head_row(part, splits, n, t, QG_ROWS + g * HD, lane);
        norm_and_rotate(kr, w_lane, (float)pos * freq);
        store_quantised<true>(kr, kc + cache_head(slot, g, cap), ks + scale_head(slot, g, cap), pos, lane);
    } else {
        const HeadRow vr = head_row(part, splits, n, t, QG_ROWS + NKV * HD + g * HD, lane);
        store_quantised<false>(vr, vc + cache_head(slot, g, cap), vs + scale_head(slot, g, cap), pos, lane);
    }
}

// ------------------------------------------------------------------------------------------------ attn_decode
__device__ __forceinline__ uint32_t kv_half2(uint32_t w, uint32_t sel) { return __byte_perm(w, 0x64646464u, sel); }

// Prompt tiles: z key splits of a whole number of 64-key blocks (z from tile_splits on the host: one value per step).
__host__ __device__ __forceinline__ int tile_chunk(int keys, int z) { return max(64, ((keys + z - 1) / z + 63) / 64 * 64); }
__host__ inline int tile_splits(int ntile, int max_keys) {
    int z = 1;  // fill about two blocks per SM, no split shorter than 256 keys
    while (z < TSPLITS && ntile * NKV * z * 2 <= 2 * 148 && max_keys / (z * 2) >= 256) z *= 2;
    return z;
}

// RT row tiles of 16 (token, head) rows; KW warps per row tile, one 16-key block of a stage each; NS ring stages
template <int RT, int KW, int NS>
struct DecCfg {
    static constexpr int KWARPS = KW, NSTG = NS;
    static constexpr int SK = 16 * KW;                // keys per ring stage
    static constexpr int STG_BYTES = SK * HD * 2 + SK * 4 * 2;  // keys, values, key scales, value scales
    static constexpr int CW = RT * KW;                // warps (warp 0 also issues the copies)
    static constexpr int THREADS = CW * 32;
    static constexpr int Q_BYTES = RT * 16 * SROW * 2;
    static constexpr int BAR_BYTES = 128;
    static constexpr int SMEM = BAR_BYTES + Q_BYTES + NS * STG_BYTES;
    static constexpr int MERGE_FLOATS = 32 * (HD / 8 * 4 + 6);  // one warp's o, m, l, ps
    static_assert(RT * (KW / 2) * MERGE_FLOATS * 4 <= NS * STG_BYTES, "the merge buffers reuse the ring");
};

// TILES = false: block (short segment, kv head, key split) of the decode attention (dseg / dtok name the tokens).
// TILES = true: block (prompt tile, kv head): `dseg` is the host's ptile array (first token, count) of tiles of
// consecutive tokens, each block takes all the keys of its tile (one split) and finishes its rows.
template <int RT, int KW, int NS, bool TILES>
__global__ void __launch_bounds__(DecCfg<RT, KW, NS>::THREADS, 1)
attn_decode_kernel(const float* q, const uint8_t* kc, const uint8_t* vc, const float* ks, const float* vs,
                   const int* dseg, const int* dtok, const int* tok_slot, const int* tok_pos, int cap, int z,
                   float* part_ml, float* part_acc, float* out, __half* mix, int* err) {
    using C = DecCfg<RT, KW, NS>;
    constexpr int KWARPS = C::KWARPS, NSTG = C::NSTG, SK = C::SK, STG_BYTES = C::STG_BYTES;
    constexpr int NTD = HD / 8;  // n8 dim tiles of the output
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + NSTG;
    __half* qsh = (__half*)(smem + C::BAR_BYTES);
    uint8_t* ring = smem + C::BAR_BYTES + C::Q_BYTES;

    const int seg = TILES ? gridDim.x - 1 - blockIdx.x : blockIdx.x;  // prompt tiles: the longest contexts first
    const int g = blockIdx.y, s = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTG; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], C::CW); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();  // the step's own keys and values are written by attn_prep just before

    const int first = dseg[2 * seg], nt = dseg[2 * seg + 1];
    auto token = [&](int i) { return TILES ? first + i : dtok[first + i]; };
    const int tlast = token(nt - 1), keys = tok_pos[tlast] + 1;
    const int chunk = TILES ? tile_chunk(keys, z) : dec_chunk(keys, DSPLITS), ns = (keys + chunk - 1) / chunk;
    if (s >= ns) return;
    const int kbeg = s * chunk, ke = min(keys, kbeg + chunk), nstg = (ke - kbeg + SK - 1) / SK;
    const int slot = tok_slot[tlast];

    // ---- the copies: warp 0 issues stage j two stages ahead of its own consumption (three stages in flight, four
    // slots: the slot it refills was released two iterations ago by everyone who keeps pace), one lane per region
    const uint64_t pol = policy_evict_first();
    const uint8_t* kh = kc + cache_head(slot, g, cap);
    const uint8_t* vh = vc + cache_head(slot, g, cap);
    const float* ksh = ks + scale_head(slot, g, cap);
    const float* vsh = vs + scale_head(slot, g, cap);
    bool copy_ok = true;
    auto issue = [&](int j) {
        const int sl = j % NSTG;
        if (j >= NSTG) {
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&empty[sl], ((j / NSTG) - 1) & 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0 && copy_ok) atomicExch(err, 3);
                copy_ok = false;
                return;
            }
        }
        uint8_t* base = ring + sl * STG_BYTES;
        const int kb = kbeg + j * SK;
        if (lane == 0) mbar_expect_tx(&full[sl], STG_BYTES);
        __syncwarp();
        if (lane == 0) bulk_g2s(base, kh + (size_t)kb * HD, SK * HD, &full[sl], pol);
        if (lane == 1) bulk_g2s(base + SK * HD, vh + (size_t)kb * HD, SK * HD, &full[sl], pol);
        if (lane == 2) bulk_g2s(base + 2 * SK * HD, ksh + kb, SK * 4, &full[sl], pol);
        if (lane == 3) bulk_g2s(base + 2 * SK * HD + SK * 4, vsh + kb, SK * 4, &full[sl], pol);
    };
    if (warp == 0) {
        issue(0);
        if (nstg > 1) issue(1);
    }

    // ---------------------------------------------------------------- compute warps
    const int wt = warp / KWARPS, kw = warp % KWARPS, r = lane >> 2, t4 = lane & 3;
    // Q of the segment's rows (row = token * GROUP + head) as f16
    for (int x = threadIdx.x; x < RT * 16 * HD / 4; x += C::CW * 32) {
        int row = x / (HD / 4), d = (x % (HD / 4)) * 4, tok = row / GROUP;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tok < nt) v = *(const float4*)(q + ((size_t)token(tok) * NH + g * GROUP + row % GROUP) * HD + d);
        *(uint2*)&qsh[row * SROW + d] = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    }
    named_bar_sync(1, C::CW * 32);
    // this lane's rows wt * 16 + r and + 8: the keys they may see end at lim; KV_OFF times the sums of their Q
    int lim[2];
    float qoff[2];
    {
        float qs = 0.f;
        const __half* qr = qsh + (wt * 16 + (lane & 15)) * SROW + (lane >> 4) * (HD / 2);
        for (int d = 0; d < HD / 2; d += 2) {
            float2 f = __half22float2(*(const __half2*)(qr + d));
            qs += f.x + f.y;
        }
        qs += __shfl_xor_sync(0xffffffffu, qs, 16);
        qoff[0] = KV_OFF * __shfl_sync(0xffffffffu, qs, r);
        qoff[1] = KV_OFF * __shfl_sync(0xffffffffu, qs, r + 8);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
        int tok = (wt * 16 + r + 8 * h2) / GROUP;
        lim[h2] = tok < nt ? min(ke, tok_pos[token(tok)] + 1) : 0;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, ps[2] = {0.f, 0.f}, o[NTD][4];
#pragma unroll
    for (int j = 0; j < NTD; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const uint32_t qa = smem_u32(qsh + (wt * 16 + (lane & 15)) * SROW + (lane >> 4) * 8);

    int sl = 0;
    uint32_t par = 0;
    bool dead = false;
    for (int i = 0; i < nstg; i++) {
        if (warp == 0 && i + 2 < nstg && copy_ok) issue(i + 2);
        if (!dead) {
            dead = !mbar_wait(&full[sl], par);
            if (dead && lane == 0) atomicExch(err, 4);
        } else {
            for (int k = 0; k < 1024 && !mbar_try_wait(&full[sl], par); k++) {}
        }
        const uint8_t* base = ring + sl * STG_BYTES;
        const int kb = kbeg + i * SK + 16 * kw;  // this warp's 16 keys of the stage
        if (kb < ke) {
            const uint8_t* kp = base + (16 * kw + r) * HD + 16 * t4;
            const uint8_t* vp = base + SK * HD + kw * 16 * HD + r * 16 + t4 * 4;
            const float* ksc_s = (const float*)(base + 2 * SK * HD) + 16 * kw;
            const float* vsc_s = ksc_s + SK;
            float ksc[2][2], vsc[2][2];
#pragma unroll
            for (int nn = 0; nn < 2; nn++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    int kk = 8 * nn + 2 * t4 + e;
                    bool in = kb + kk < ke;
                    ksc[nn][e] = in ? ksc_s[kk] : 0.f;
                    vsc[nn][e] = in ? vsc_s[kk] : 0.f;
                }
            // S = Q K^T
            float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int b = 0; b < HD / 64; b++) {
                uint4 kf0 = *(const uint4*)(kp + 64 * b), kf1 = *(const uint4*)(kp + 8 * HD + 64 * b);
                uint32_t w0[4] = {kf0.x, kf0.y, kf0.z, kf0.w}, w1[4] = {kf1.x, kf1.y, kf1.z, kf1.w};
#pragma unroll
                for (int st = 0; st < 4; st++) {
                    uint32_t a[4];
                    ldsm_x4(a[0], a[1], a[2], a[3], qa + (b * 64 + st * 16) * 2);
                    mma16816(sacc[0], a, kv_half2(w0[st], 0x4140), kv_half2(w0[st], 0x4342));
                    mma16816(sacc[1], a, kv_half2(w1[st], 0x4140), kv_half2(w1[st], 0x4342));
                }
            }
            // scale, mask, online softmax per row; P times the value scales as the A fragments of P V
            float pv[2][4];
            bool grew = false;
            float corr[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                float v[2][2], mx = -INFINITY;
#pragma unroll
                for (int nn = 0; nn < 2; nn++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        int k = kb + 8 * nn + 2 * t4 + e;
                        v[nn][e] = k < lim[h2] ? (sacc[nn][2 * h2 + e] - qoff[h2]) * ksc[nn][e] : -INFINITY;
                        mx = fmaxf(mx, v[nn][e]);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                float mn = fmaxf(m[h2], mx);
                corr[h2] = mn == -INFINITY ? 1.f : exp2f(m[h2] - mn);
                m[h2] = mn;
                float sum = 0.f;
#pragma unroll
                for (int nn = 0; nn < 2; nn++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        float p = v[nn][e] == -INFINITY ? 0.f : exp2f(v[nn][e] - mn);
                        sum += p;
                        pv[nn][2 * h2 + e] = p * vsc[nn][e];
                    }
                l[h2] = l[h2] * corr[h2] + sum;
                ps[h2] *= corr[h2];
                grew |= corr[h2] != 1.f;
            }
            if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
                for (int j = 0; j < NTD; j++) {
                    o[j][0] *= corr[0]; o[j][1] *= corr[0];
                    o[j][2] *= corr[1]; o[j][3] *= corr[1];
                }
            }
            uint32_t pa[4] = {pack_half2(pv[0][0], pv[0][1]), pack_half2(pv[0][2], pv[0][3]),
                              pack_half2(pv[1][0], pv[1][1]), pack_half2(pv[1][2], pv[1][3])};
            // the P the products see (f16): rows r (words 0, 2) and r + 8 (1, 3)
            float2 f0 = __half22float2(*(__half2*)&pa[0]), f2 = __half22float2(*(__half2*)&pa[2]);
            float2 f1 = __half22float2(*(__half2*)&pa[1]), f3 = __half22float2(*(__half2*)&pa[3]);
            ps[0] += f0.x + f0.y + f2.x + f2.y;
            ps[1] += f1.x + f1.y + f3.x + f3.y;
            // O += P V
#pragma unroll
            for (int j = 0; j < NTD; j++) {
                uint32_t vw = *(const uint32_t*)(vp + j * 8 * 16);
                mma16816(o[j], pa, kv_half2(vw, 0x4140), kv_half2(vw, 0x4342));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[sl]);
        if (++sl == NSTG) { sl = 0; par ^= 1; }
    }

    // ---- the warps of a row tile merge pairwise in two rounds (1 -> 0 and 3 -> 2, then 2 -> 0) through the ring, which
    // is free: every stage was consumed
    named_bar_sync(1, C::CW * 32);
    for (int round = 1; round < KWARPS; round <<= 1) {
        const bool sender = (kw & (2 * round - 1)) == round, receiver = (kw & (2 * round - 1)) == 0;
        float* mb = (float*)ring + (size_t)(wt * (KWARPS / 2) + (kw >> 1) / round % (KWARPS / 2)) * C::MERGE_FLOATS;
        if (sender) {
#pragma unroll
            for (int j = 0; j < NTD; j++)
                *(float4*)(mb + (j * 32 + lane) * 4) = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
            float* t = mb + NTD * 32 * 4 + lane * 6;
            t[0] = m[0]; t[1] = m[1]; t[2] = l[0]; t[3] = l[1]; t[4] = ps[0]; t[5] = ps[1];
        }
        named_bar_sync(1, C::CW * 32);
        if (receiver) {
            const float* t = mb + NTD * 32 * 4 + lane * 6;
            float c0[2], c1[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                float m1 = t[h2], mn = fmaxf(m[h2], m1);
                c0[h2] = mn == -INFINITY ? 1.f : exp2f(m[h2] - mn);
                c1[h2] = mn == -INFINITY ? 1.f : exp2f(m1 - mn);
                m[h2] = mn;
                l[h2] = l[h2] * c0[h2] + t[2 + h2] * c1[h2];
                ps[h2] = ps[h2] * c0[h2] + t[4 + h2] * c1[h2];
            }
#pragma unroll
            for (int j = 0; j < NTD; j++) {
                float4 v = *(const float4*)(mb + (j * 32 + lane) * 4);
                o[j][0] = o[j][0] * c0[0] + v.x * c1[0]; o[j][1] = o[j][1] * c0[0] + v.y * c1[0];
                o[j][2] = o[j][2] * c0[1] + v.z * c1[1]; o[j][3] = o[j][3] * c0[1] + v.w * c1[1];
            }
        }
        named_bar_sync(1, C::CW * 32);
    }
    if (kw != 0) return;
#pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
        float L = l[h2], P = ps[h2];
        L += __shfl_xor_sync(0xffffffffu, L, 1);
        L += __shfl_xor_sync(0xffffffffu, L, 2);
        P += __shfl_xor_sync(0xffffffffu, P, 1);
        P += __shfl_xor_sync(0xffffffffu, P, 2);
        int row = wt * 16 + r + 8 * h2, tok = row / GROUP;
        if (tok >= nt) continue;
        int i = first + tok, t = token(tok), head = g * GROUP + row % GROUP;
        if (ns == 1) {
            float f = 1.f / L;
            float* op = out + (size_t)t * MIX + head * HD + 2 * t4;
#pragma unroll
            for (int j = 0; j < NTD; j++) {
                float2 gt = *(float2*)(op + j * 8);
                float2 res = make_float2(gt.x * (o[j][2 * h2] - KV_OFF * P) * f, gt.y * (o[j][2 * h2 + 1] - KV_OFF * P) * f);
                *(float2*)(op + j * 8) = res;
                if (TILES && mix) *(__half2*)(mix + (size_t)t * MIX + head * HD + 2 * t4 + j * 8) = __floats2half2_rn(res.x, res.y);
            }
        } else {
            size_t pi = ((size_t)i * NH + head) * z + s;
            float* pp = part_acc + pi * HD + 2 * t4;
#pragma unroll
            for (int j = 0; j < NTD; j++)
                *(float2*)(pp + j * 8) = make_float2(o[j][2 * h2] - KV_OFF * P, o[j][2 * h2 + 1] - KV_OFF * P);
            if (t4 == 0) { part_ml[pi * 2] = m[h2]; part_ml[pi * 2 + 1] = L; }
        }
    }
}

// ------------------------------------------------------------------------------------------------ decode attention
// Block (short segment, kv head, key split) of the decode / verify attention: 2 to 4 QUADS of four compute warps and a
// copy warp. The keys and values of the split arrive in 64-key stages through a ring fed by bulk copies; the quads
// take the stages in turn. Inside a quad the work of a stage is dealt so that no byte is converted twice:
//   scores   warp w multiplies all the rows (RT tiles of 16 (token, head) rows) by the keys 16 w .. 16 w + 15 of the
//            stage over the whole head dimension: one conversion of a key serves every row tile;
//   softmax  the four warps agree on the rows' running maxima through shared memory, so that all of them scale by the
//            same power of two, and exchange their 16-key slices of P (as f16 mma fragments) and of the row sums;
//   values   warp w accumulates the output dims 64 w .. 64 w + 63 over all 64 keys of the stage (for every row tile),
//            so the output accumulators of a row are spread over four warps (RT x 32 registers each).
// The int8 codes go to the tensor cores as 1152 + q halves (one prmt per pair) and the offset is folded out through the
// row sums, as in the reference (kernels/attn.cuh:38-40,198-234). The four quads' partial results meet in shared memory
// at the end; the block writes one (m, l, acc) partial per row, or the finished rows when the segment has one split.
template <int RT, int NQ>
struct Dec4Cfg {
    static constexpr int QUADS = NQ, CW = 4 * QUADS;   // compute warps
    static constexpr int THREADS = (CW + 1) * 32;       // + the copy warp
    static constexpr int SK = 64, NSTG = 5;             // keys per stage, ring depth
    static constexpr int STG_BYTES = SK * HD * 2 + SK * 8;
    static constexpr int Q_BYTES = RT * 16 * SROW * 2;
    // per quad: the warps' row maxima [4][RT][16], their P fragments [4][RT][32 lanes] x 16 B, their (sum, ps) [4][RT][16][2]
    static constexpr int X_MAX = 4 * RT * 16 * 4, X_P = 4 * RT * 32 * 16, X_SUM = 4 * RT * 16 * 8;
    static constexpr int X_BYTES = X_MAX + X_P + X_SUM;
    static constexpr int BAR_BYTES = 128;
    static constexpr int SMEM = BAR_BYTES + Q_BYTES + QUADS * X_BYTES + NSTG * STG_BYTES;
    static constexpr int MERGE_BYTES = 8 * 32 * (RT * 8 * 4 + RT * 6) * 4;   // two quads' registers at a time
    static_assert(MERGE_BYTES <= NSTG * STG_BYTES, "the merge buffers reuse the ring");
    static_assert(SMEM <= 227 * 1024, "shared memory");
};

template <int RT, int NQ>
__global__ void __launch_bounds__(Dec4Cfg<RT, NQ>::THREADS, 1)
attn_dec4_kernel(const float* q, const uint8_t* kc, const uint8_t* vc, const float* ks, const float* vs, const int* dseg,
                 const int* dtok, const int* tok_slot, const int* tok_pos, int cap, int z, int dsplits, int old_margin,
                 float* part_ml, float* part_acc, float* out, int* err) {
    using C = Dec4Cfg<RT, NQ>;
    constexpr int NSTG = C::NSTG, SK = C::SK, STG_BYTES = C::STG_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + NSTG;
    __half* qsh = (__half*)(smem + C::BAR_BYTES);
    uint8_t* xch = smem + C::BAR_BYTES + C::Q_BYTES;
    uint8_t* ring = xch + C::QUADS * C::X_BYTES;

    const int seg = blockIdx.x, g = blockIdx.y, s = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTG; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 4); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    // The step's token lists are uploaded before its first kernel, so they are read ahead of the kernel before (this
    // step's attn_prep), and so are the stages of keys and values that earlier steps wrote: whatever ends `old_margin`
    // positions or more before the segment's last key (0: nothing is read ahead).
    const int first = dseg[2 * seg], nt = dseg[2 * seg + 1];
    const int tlast = dtok[first + nt - 1], keys = tok_pos[tlast] + 1;
    const int chunk = dec_chunk(keys, dsplits), ns = (keys + chunk - 1) / chunk;
    if (s >= ns) return;
    const int kbeg = s * chunk, ke = min(keys, kbeg + chunk), nstg = (ke - kbeg + SK - 1) / SK;
    const int slot = tok_slot[tlast];

    if (warp == C::CW) {
        // ------------------------------------------------------------ the copy warp
        const uint64_t pol = policy_evict_first();
        const uint8_t* kh = kc + cache_head(slot, g, cap);
        const uint8_t* vh = vc + cache_head(slot, g, cap);
        const float* ksh = ks + scale_head(slot, g, cap);
        const float* vsh = vs + scale_head(slot, g, cap);
        bool waited = false;
        for (int j = 0; j < nstg; j++) {
            const int sl = j % NSTG;
            if (!waited && (old_margin <= 0 || kbeg + (j + 1) * SK > keys - old_margin)) {
                pdl_wait();
                waited = true;
            }
            if (j >= NSTG) {
                bool ok = true;
                if (lane == 0) ok = mbar_wait(&empty[sl], ((j / NSTG) - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) atomicExch(err, 3);
                    return;
                }
            }
            uint8_t* base = ring + sl * STG_BYTES;
            const int kb = kbeg + j * SK;
            if (lane == 0) mbar_expect_tx(&full[sl], STG_BYTES);
            __syncwarp();
            if (lane == 0) bulk_g2s(base, kh + (size_t)kb * HD, SK * HD, &full[sl], pol);
            if (lane == 1) bulk_g2s(base + SK * HD, vh + (size_t)kb * HD, SK * HD, &full[sl], pol);
            if (lane == 2) bulk_g2s(base + 2 * SK * HD, ksh + kb, SK * 4, &full[sl], pol);
            if (lane == 3) bulk_g2s(base + 2 * SK * HD + SK * 4, vsh + kb, SK * 4, &full[sl], pol);
        }
        return;
    }

    // ---------------------------------------------------------------- compute warps
    const int quad = warp >> 2, w = warp & 3, r = lane >> 2, t4 = lane & 3;
    constexpr int NCW = C::CW * 32;
    pdl_wait();  // q and the gates come from this step's attn_prep
    // Q of the segment's rows (row = token * GROUP + head) as f16
    for (int x = threadIdx.x; x < RT * 16 * HD / 4; x += NCW) {
        const int row = x / (HD / 4), d = (x % (HD / 4)) * 4, tok = row / GROUP;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tok < nt) v = *(const float4*)(q + ((size_t)dtok[first + tok] * NH + g * GROUP + row % GROUP) * HD + d);
        *(uint2*)&qsh[row * SROW + d] = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    }
    named_bar_sync(1, NCW);
    // this lane's rows 16 rt + r and + 8: the keys they may see end at lim; KV_OFF times the sums of their Q
    int lim[RT][2];
    float qoff[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        float qs = 0.f;
        const __half* qr = qsh + (rt * 16 + (lane & 15)) * SROW + (lane >> 4) * (HD / 2);
        for (int d = 0; d < HD / 2; d += 2) {
            const float2 f = __half22float2(*(const __half2*)(qr + d));
            qs += f.x + f.y;
        }
        qs += __shfl_xor_sync(0xffffffffu, qs, 16);
        qoff[rt][0] = KV_OFF * __shfl_sync(0xffffffffu, qs, r);
        qoff[rt][1] = KV_OFF * __shfl_sync(0xffffffffu, qs, r + 8);
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
            const int tok = (rt * 16 + r + 8 * h2) / GROUP;
            lim[rt][h2] = tok < nt ? min(ke, tok_pos[dtok[first + tok]] + 1) : 0;
        }
    }
    float m[RT][2], l[RT][2], ps[RT][2], o[RT][8][4];
#pragma unroll
    for (int rt = 0; rt < RT; rt++) {
        m[rt][0] = m[rt][1] = -INFINITY;
        l[rt][0] = l[rt][1] = ps[rt][0] = ps[rt][1] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) o[rt][j][0] = o[rt][j][1] = o[rt][j][2] = o[rt][j][3] = 0.f;
    }
    uint32_t qa[RT];
#pragma unroll
    for (int rt = 0; rt < RT; rt++) qa[rt] = smem_u32(qsh + (rt * 16 + (lane & 15)) * SROW + (lane >> 4) * 8);
    float* xmax = (float*)(xch + quad * C::X_BYTES);                 // [4][RT][16]
    uint4* xp = (uint4*)(xch + quad * C::X_BYTES + C::X_MAX);        // [4][RT][32]
    float2* xsum = (float2*)(xch + quad * C::X_BYTES + C::X_MAX + C::X_P);  // [4][RT][16]

    bool dead = false;
    for (int j = quad; j < nstg; j += C::QUADS) {
        const int sl = j % NSTG;
        const uint32_t par = (j / NSTG) & 1;
        if (!dead) {
            dead = !mbar_wait(&full[sl], par);
            if (dead && lane == 0) atomicExch(err, 4);
        } else {
            for (int k = 0; k < 1024 && !mbar_try_wait(&full[sl], par); k++) {}
        }
        const uint8_t* base = ring + sl * STG_BYTES;
        const int kb = kbeg + j * SK + 16 * w;  // this warp's 16 keys of the stage
        const uint8_t* kp = base + (16 * w + r) * HD + 16 * t4;
        const float* ksc_s = (const float*)(base + 2 * SK * HD) + 16 * w;
        const float* vsc_s = ksc_s + SK;
        float ksc[2][2], vsc[2][2];
#pragma unroll
        for (int nn = 0; nn < 2; nn++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int kk = 8 * nn + 2 * t4 + e;
                const bool in = kb + kk < ke;
                ksc[nn][e] = in ? ksc_s[kk] : 0.f;
                vsc[nn][e] = in ? vsc_s[kk] : 0.f;
            }
        // ---- scores: S = Q K^T for every row tile, this warp's 16 keys
        float sacc[RT][2][4];
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int nn = 0; nn < 2; nn++) sacc[rt][nn][0] = sacc[rt][nn][1] = sacc[rt][nn][2] = sacc[rt][nn][3] = 0.f;
#pragma unroll
        for (int b = 0; b < HD / 64; b++) {
            const uint4 kf0 = *(const uint4*)(kp + 64 * b), kf1 = *(const uint4*)(kp + 8 * HD + 64 * b);
            const uint32_t w0[4] = {kf0.x, kf0.y, kf0.z, kf0.w}, w1[4] = {kf1.x, kf1.y, kf1.z, kf1.w};
#pragma unroll
            for (int st = 0; st < 4; st++) {
                const uint32_t b00 = kv_half2(w0[st], 0x4140), b01 = kv_half2(w0[st], 0x4342);
                const uint32_t b10 = kv_half2(w1[st], 0x4140), b11 = kv_half2(w1[st], 0x4342);
#pragma unroll
                for (int rt = 0; rt < RT; rt++) {
                    uint32_t a[4];
                    ldsm_x4(a[0], a[1], a[2], a[3], qa[rt] + (b * 64 + st * 16) * 2);
                    mma16816(sacc[rt][0], a, b00, b01);
                    mma16816(sacc[rt][1], a, b10, b11);
                }
            }
        }
        // ---- the rows' maxima over this warp's keys, then over the quad's
        float v[RT][2][4];
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                float mx = -INFINITY;
#pragma unroll
                for (int nn = 0; nn < 2; nn++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int k = kb + 8 * nn + 2 * t4 + e;
                        const float sv = k < lim[rt][h2] ? (sacc[rt][nn][2 * h2 + e] - qoff[rt][h2]) * ksc[nn][e] : -INFINITY;
                        v[rt][nn][2 * h2 + e] = sv;
                        mx = fmaxf(mx, sv);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                if (t4 == 0) xmax[(w * RT + rt) * 16 + r + 8 * h2] = mx;
            }
        named_bar_sync(2 + quad, 128);
        float corr[RT][2];
        bool grew = false;
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                float mn = m[rt][h2];
#pragma unroll
                for (int ww = 0; ww < 4; ww++) mn = fmaxf(mn, xmax[(ww * RT + rt) * 16 + r + 8 * h2]);
                corr[rt][h2] = mn == -INFINITY ? 1.f : exp2f(m[rt][h2] - mn);
                m[rt][h2] = mn;
                grew |= corr[rt][h2] != 1.f;
            }
        // ---- P of this warp's keys (times the value scales, rounded to f16 as the products see it) and its row sums
#pragma unroll
        for (int rt = 0; rt < RT; rt++) {
            float pv[2][4], sum[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                sum[h2] = 0.f;
#pragma unroll
                for (int nn = 0; nn < 2; nn++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const float sv = v[rt][nn][2 * h2 + e];
                        const float pp = sv == -INFINITY ? 0.f : exp2f(sv - m[rt][h2]);
                        sum[h2] += pp;
                        pv[nn][2 * h2 + e] = pp * vsc[nn][e];
                    }
            }
            uint4 pa;
            pa.x = pack_half2(pv[0][0], pv[0][1]); pa.y = pack_half2(pv[0][2], pv[0][3]);
            pa.z = pack_half2(pv[1][0], pv[1][1]); pa.w = pack_half2(pv[1][2], pv[1][3]);
            xp[(w * RT + rt) * 32 + lane] = pa;
            __half2 h0, h1, h2v, h3;
            *(uint32_t*)&h0 = pa.x; *(uint32_t*)&h1 = pa.y; *(uint32_t*)&h2v = pa.z; *(uint32_t*)&h3 = pa.w;
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1), f2 = __half22float2(h2v), f3 = __half22float2(h3);
            float pr[2] = {f0.x + f0.y + f2.x + f2.y, f1.x + f1.y + f3.x + f3.y};
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                sum[h2] += __shfl_xor_sync(0xffffffffu, sum[h2], 1);
                sum[h2] += __shfl_xor_sync(0xffffffffu, sum[h2], 2);
                pr[h2] += __shfl_xor_sync(0xffffffffu, pr[h2], 1);
                pr[h2] += __shfl_xor_sync(0xffffffffu, pr[h2], 2);
                if (t4 == 0) xsum[(w * RT + rt) * 16 + r + 8 * h2] = make_float2(sum[h2], pr[h2]);
            }
        }
        named_bar_sync(2 + quad, 128);
#pragma unroll
        for (int rt = 0; rt < RT; rt++)
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++) {
                float sl2 = 0.f, sp2 = 0.f;
#pragma unroll
                for (int ww = 0; ww < 4; ww++) {  // in warp order: the same sum in all four warps
                    const float2 x = xsum[(ww * RT + rt) * 16 + r + 8 * h2];
                    sl2 += x.x;
                    sp2 += x.y;
                }
                l[rt][h2] = l[rt][h2] * corr[rt][h2] + sl2;
                ps[rt][h2] = ps[rt][h2] * corr[rt][h2] + sp2;
            }
        if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
            for (int rt = 0; rt < RT; rt++)
#pragma unroll
                for (int jd = 0; jd < 8; jd++) {
                    o[rt][jd][0] *= corr[rt][0]; o[rt][jd][1] *= corr[rt][0];
                    o[rt][jd][2] *= corr[rt][1]; o[rt][jd][3] *= corr[rt][1];
                }
        }
        // ---- values: O += P V over the stage's 64 keys, this warp's 64 output dims
#pragma unroll
        for (int kbk = 0; kbk < 4; kbk++) {
            uint32_t pa[RT][4];
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                const uint4 x = xp[(kbk * RT + rt) * 32 + lane];
                pa[rt][0] = x.x; pa[rt][1] = x.y; pa[rt][2] = x.z; pa[rt][3] = x.w;
            }
            const uint8_t* vp = base + SK * HD + kbk * 16 * HD + (64 * w + r) * 16 + t4 * 4;
#pragma unroll
            for (int jd = 0; jd < 8; jd++) {
                const uint32_t vw = *(const uint32_t*)(vp + jd * 8 * 16);
                const uint32_t b0 = kv_half2(vw, 0x4140), b1 = kv_half2(vw, 0x4342);
#pragma unroll
                for (int rt = 0; rt < RT; rt++) mma16816(o[rt][jd], pa[rt], b0, b1);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[sl]);
    }

    // ---- the quads merge pairwise through the ring, which is free (every stage was consumed): 1 -> 0 and 3 -> 2, then
    // 2 -> 0. A warp's registers go to the warp of the same index in the other quad (same rows, same dims).
    named_bar_sync(1, NCW);
    constexpr int MF = RT * 8 * 4 + RT * 6;  // floats per lane
    for (int round = 1; round < C::QUADS; round <<= 1) {
        const bool sender = (quad & (2 * round - 1)) == round;
        const bool receiver = (quad & (2 * round - 1)) == 0 && quad + round < C::QUADS;
        float* mb = (float*)ring + (size_t)(((quad >> 1) / round % 2) * 4 + w) * 32 * MF + lane;
        if (sender) {
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
#pragma unroll
                for (int jd = 0; jd < 8; jd++)
#pragma unroll
                    for (int e = 0; e < 4; e++) mb[((rt * 8 + jd) * 4 + e) * 32] = o[rt][jd][e];
#pragma unroll
                for (int h2 = 0; h2 < 2; h2++) {
                    mb[(RT * 32 + rt * 6 + h2) * 32] = m[rt][h2];
                    mb[(RT * 32 + rt * 6 + 2 + h2) * 32] = l[rt][h2];
                    mb[(RT * 32 + rt * 6 + 4 + h2) * 32] = ps[rt][h2];
                }
            }
        }
        named_bar_sync(1, NCW);
        if (receiver) {
#pragma unroll
            for (int rt = 0; rt < RT; rt++) {
                float c0[2], c1[2];
#pragma unroll
                for (int h2 = 0; h2 < 2; h2++) {
                    const float m1 = mb[(RT * 32 + rt * 6 + h2) * 32], mn = fmaxf(m[rt][h2], m1);
                    c0[h2] = mn == -INFINITY ? 1.f : exp2f(m[rt][h2] - mn);
                    c1[h2] = mn == -INFINITY ? 1.f : exp2f(m1 - mn);
                    m[rt][h2] = mn;
                    l[rt][h2] = l[rt][h2] * c0[h2] + mb[(RT * 32 + rt * 6 + 2 + h2) * 32] * c1[h2];
                    ps[rt][h2] = ps[rt][h2] * c0[h2] + mb[(RT * 32 + rt * 6 + 4 + h2) * 32] * c1[h2];
                }
#pragma unroll
                for (int jd = 0; jd < 8; jd++)
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        o[rt][jd][e] = o[rt][jd][e] * c0[e >> 1] + mb[((rt * 8 + jd) * 4 + e) * 32] * c1[e >> 1];
            }
        }
        named_bar_sync(1, NCW);
    }
    if (quad != 0) return;
#pragma unroll
    for (int rt = 0; rt < RT; rt++)
#pragma unroll
        for (int h2 = 0; h2 < 2; h2++) {
            const float L = l[rt][h2], P = ps[rt][h2];   // already whole-row sums, the same in the four warps
            const int row = rt * 16 + r + 8 * h2, tok = row / GROUP;
            if (tok >= nt) continue;
            const int i = first + tok, t = dtok[i], head = g * GROUP + row % GROUP;
            if (ns == 1) {
                const float f = 1.f / L;
                float* op = out + (size_t)t * MIX + head * HD + 64 * w + 2 * t4;
#pragma unroll
                for (int jd = 0; jd < 8; jd++) {
                    const float2 gt = *(float2*)(op + jd * 8);
                    *(float2*)(op + jd * 8) = make_float2(gt.x * (o[rt][jd][2 * h2] - KV_OFF * P) * f,
                                                          gt.y * (o[rt][jd][2 * h2 + 1] - KV_OFF * P) * f);
                }
            } else {
                const size_t pi = ((size_t)i * NH + head) * z + s;
                float* pp = part_acc + pi * HD + 64 * w + 2 * t4;
#pragma unroll
                for (int jd = 0; jd < 8; jd++)
                    *(float2*)(pp + jd * 8) = make_float2(o[rt][jd][2 * h2] - KV_OFF * P, o[rt][jd][2 * h2 + 1] - KV_OFF * P);
                if (w == 0 && t4 == 0) { part_ml[pi * 2] = m[rt][h2]; part_ml[pi * 2 + 1] = L; }
            }
        }
}

// Merge the ns key splits of one (token, head) in split order; *op *= result (the gate is there); optionally also the
// f16 copy of the product. HD threads, thread d owns dim d; the splits' maxima and sums go through shared memory once
// so that the accumulator loads of all splits are independent and in flight together.
__device__ __forceinline__ void combine_row(const float* part_ml, const float* part_acc, size_t base, int ns, float* op,
                                            __half* mp) {
    static_assert(DSPLITS <= 64 && TSPLITS <= 64, "two splits per lane");
    __shared__ float se[64];
    __shared__ float sL;
    const int d = threadIdx.x;
    float res;
    if (ns == 1) {
        res = *op;  // the attention kernel finished it
    } else {
        if (d < 32) {  // lane d: splits d and d + 32
            const float ms0 = d < ns ? part_ml[(base + d) * 2] : -INFINITY;
            const float ls0 = d < ns ? part_ml[(base + d) * 2 + 1] : 0.f;
            const float ms1 = d + 32 < ns ? part_ml[(base + d + 32) * 2] : -INFINITY;
            const float ls1 = d + 32 < ns ? part_ml[(base + d + 32) * 2 + 1] : 0.f;
            const float M = warp_max(fmaxf(ms0, ms1));
            const float e0 = ms0 == -INFINITY ? 0.f : exp2f(ms0 - M), e1 = ms1 == -INFINITY ? 0.f : exp2f(ms1 - M);
            se[d] = e0;
            se[d + 32] = e1;
            // the sum over splits in split order (not a tree: the same order whatever the lane count)
            float L = 0.f;
            for (int s = 0; s < ns; s++) L += __shfl_sync(0xffffffffu, s < 32 ? e0 * ls0 : e1 * ls1, s & 31);
            if (d == 0) sL = L;
        }
        __syncthreads();
        float A = 0.f;
        const float* pa = part_acc + base * HD + d;
#pragma unroll 8
        for (int s = 0; s < ns; s++) A += se[s] * pa[(size_t)s * HD];
        res = *op * A * (1.f / sL);
        *op = res;
    }
    if (mp) *mp = __float2half_rn(res);
}

// block (decode token, head)
__global__ void __launch_bounds__(HD)
attn_combine_kernel(const float* part_ml, const float* part_acc, const int* dtok, const int* dkeys, int z, int dsplits,
                    float* out, __half* mix) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x, h = blockIdx.y, t = dtok[i], d = threadIdx.x;
    const size_t o = (size_t)t * MIX + h * HD + d;
    combine_row(part_ml, part_acc, ((size_t)i * NH + h) * z, dec_splits(dkeys[i], dsplits), out + o, mix ? mix + o : nullptr);
}

// block (prompt tile * PTILE + row, head)
__global__ void __launch_bounds__(HD)
attn_combine_tiles_kernel(const float* part_ml, const float* part_acc, const int* ptile, const int* tok_pos, int z,
                          float* out, __half* mix) {
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x / PTILE, row = blockIdx.x % PTILE, h = blockIdx.y, d = threadIdx.x;
    const int t0 = ptile[2 * tile], len = ptile[2 * tile + 1];
    if (row >= len) return;
    const int keys = tok_pos[t0 + len - 1] + 1, chunk = tile_chunk(keys, z), t = t0 + row;
    const size_t o = (size_t)t * MIX + h * HD + d;
    combine_row(part_ml, part_acc, ((size_t)t * NH + h) * z, (keys + chunk - 1) / chunk, out + o, mix ? mix + o : nullptr);
}

}  // namespace qb

using namespace qb;

extern "C" {

int qb_attn_prep(qb_ctx* ctx, void* stream, const float* part, int splits, int n, const float* q_norm,
                 const float* k_norm, const float* inv_freq, float qscale, float* q, float* out, void* kc, void* vc,
                 float* ks, float* vs, const int* tok_slot, const int* tok_pos, int cap) {
    if (!ctx || !part || !q_norm || !k_norm || !inv_freq || !q || !out || !kc || !vc || !ks || !vs || !tok_slot ||
        !tok_pos || n <= 0 || splits < 1 || cap <= 0 || cap % 64)
        return QB_ERR_ARG;
    return launch(ctx, attn_prep_kernel, dim3(n, 2), dim3(32 * NH), 0, (cudaStream_t)stream, part, splits, n,
                  q_norm, k_norm, inv_freq, qscale, q, out, (uint8_t*)kc, (uint8_t*)vc, ks, vs, tok_slot, tok_pos, cap);
}

int qb_attn_dec_splits(int keys) { return keys > 0 ? dec_splits(keys, DSPLITS) : 0; }
int qb_attn_dec_splits_sm(int keys, int sms) { return keys > 0 && sms > 0 ? dec_splits(keys, dsplits_for(sms)) : 0; }

// ndseg short segments (dseg: first index into dtok, token count; at most 8 tokens each), ndec = their tokens in
// all, dmax = the longest segment's tokens, max_keys = the largest key count among them (sizes the grid).
int qb_attn_decode(qb_ctx* ctx, void* stream, const float* q, const void* kc, const void* vc, const float* ks,
                   const float* vs, const int* dseg, const int* dtok, const int* dkeys, const int* tok_slot,
                   const int* tok_pos, int cap, int ndseg, int ndec, int dmax, int max_keys, float* part_ml,
                   float* part_acc, float* out, void* mix_f16) {
    if (!ctx || !q || !kc || !vc || !ks || !vs || !dseg || !dtok || !dkeys || !tok_slot || !tok_pos || !part_ml ||
        !part_acc || !out || ndseg <= 0 || ndec <= 0 || dmax <= 0 || dmax > 8 || max_keys <= 0 || cap % 64 ||
        max_keys > cap)
        return QB_ERR_ARG;
    const int dsplits = dsplits_for(ctx->sms);
    const int z = dec_splits(max_keys, dsplits), rt = (dmax * GROUP + 15) / 16;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(ndseg, NKV, z);
    // a step has at most 64 decode tokens: whatever lies 64 positions or more before a segment's last key is from
    // earlier steps
    const int old_margin = ndec <= 64 ? 64 : 0;
    int rc;
#define QB_DEC(RT, NQ)                                                                                          \
    {                                                                                                           \
        using C = Dec4Cfg<RT, NQ>;                                                                              \
        rc = launch(ctx, attn_dec4_kernel<RT, NQ>, grid, dim3(C::THREADS), C::SMEM, st, q, (const uint8_t*)kc, \
                    (const uint8_t*)vc, ks, vs, dseg, dtok, tok_slot, tok_pos, cap, z, dsplits, old_margin, part_ml,   \
                    part_acc, out, ctx->err);                                                                             \
    }
    // quads per block: as many as leave every warp its registers (a warp holds RT x 32 output accumulators per lane);
    // measured at 5 rows: 2 quads 33.4 us, 3 quads (spills) 36.6 us, 4 quads 43.2 us
    if (rt == 1) QB_DEC(1, 4) else if (rt == 2) QB_DEC(2, 2) else QB_DEC(3, 2)
#undef QB_DEC
    if (rc) return rc;
    return launch(ctx, attn_combine_kernel, dim3(ndec, NH), dim3(HD), 0, st, (const float*)part_ml,
                  (const float*)part_acc, dtok, dkeys, z, dsplits, out, (__half*)mix_f16);
}

int qb_attn_tile_splits(int ntile, int max_keys) { return ntile > 0 && max_keys > 0 ? tile_splits(ntile, max_keys) : 0; }

// Prompt attention: ntile tiles of up to 10 consecutive tokens of one segment (the host's ptile array: first token,
// count), each against all the keys up to its last token; max_keys = the largest key count among them. `out` holds
// the gate on entry and the gated attention output on return; mix_f16 (optional) gets its f16 copy. One block per
// (tile, kv head, key split); part_ml / part_acc: scratch for n * 24 * qb_attn_tile_splits(ntile, max_keys) (m, l)
// pairs and accumulators of 256 floats, n = the step's tokens (unused with one split).
int qb_attn_prefill(qb_ctx* ctx, void* stream, const float* q, const void* kc, const void* vc, const float* ks,
                    const float* vs, const int* ptile, const int* tok_slot, const int* tok_pos, int cap, int ntile,
                    int max_keys, float* part_ml, float* part_acc, float* out, void* mix_f16) {
    if (!ctx || !q || !kc || !vc || !ks || !vs || !ptile || !tok_slot || !tok_pos || !out || ntile <= 0 || cap % 64 ||
        max_keys <= 0 || max_keys > cap)
        return QB_ERR_ARG;
    const int z = tile_splits(ntile, max_keys);
    if (z > 1 && (!part_ml || !part_acc)) return QB_ERR_ARG;
    if (z == 1) {  // many tiles: a pair of tiles per block on tcgen05 (attn_prefill_tc.cu)
        return qb_attn_prefill_tc_launch(ctx, (cudaStream_t)stream, q, kc, vc, ks, vs, ptile, ntile, tok_slot, tok_pos,
                                         cap, out, mix_f16);
    }
    using C = DecCfg<4, 2, 5>;  // 10 tokens x 6 heads = 60 rows: 4 row tiles; 2 warps each; 5 stages of 32 keys
    static_assert(PTILE * GROUP <= 64, "a prompt tile fills at most 4 row tiles");
    cudaStream_t st = (cudaStream_t)stream;
    int rc = launch(ctx, attn_decode_kernel<4, 2, 5, true>, dim3(ntile, NKV, z), dim3(C::THREADS), C::SMEM, st, q,
                    (const uint8_t*)kc, (const uint8_t*)vc, ks, vs, ptile, (const int*)nullptr, tok_slot, tok_pos, cap, z,
                    part_ml, part_acc, out, z == 1 ? (__half*)mix_f16 : (__half*)nullptr, ctx->err);
    if (rc || z == 1) return rc;
    return launch(ctx, attn_combine_tiles_kernel, dim3(ntile * PTILE, NH), dim3(HD), 0, st, (const float*)part_ml,
                  (const float*)part_acc, ptile, tok_pos, z, out, (__half*)mix_f16);
}

}  // extern "C"
