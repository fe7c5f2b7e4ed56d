// The GPU sampler: sample_rows and draft_sample of the reference (kernels/sampling.cuh:188-352; host definition
// src/sample.rs:88-211), in vLLM's order: repetition penalty, presence penalty, temperature, top-k, top-p, then the
// draw with the host's uniform numbers (with a draft: accept or resample).
//
// The reference gives a logit row to ONE block of 1024 threads, which reads the 248,320 logits (and their penalty
// bits) up to four times through a 4096-bin shared histogram. Here a row belongs to a CLUSTER of 8 blocks: each block
// reads an eighth of the row ONCE, applies the penalties and keeps the order-preserving keys in its shared memory
// (124 KB); the k-th largest key is then found by an 8-bit radix select whose histograms have one copy per lane (no
// two lanes of a warp ever add to the same word) and are merged over the cluster through distributed shared memory:
// one cluster barrier per level. The blocks append their candidates to the leading block's list with remote atomics;
// that block sorts them and draws. The arithmetic of the draw (exp of (v - vmax) / temperature, the shape of the
// prefix sums, every comparison) is the reference kernel's, so the tokens are identical draw for draw.
//
// Rows over the whole vocabulary (top_k 0) with a top-p cut, the common serving setting, are the host's in the reference
// (a full sort of 248,320 values per row and step). Here the blocks also sum the mass of all tokens, the cut is made
// among the 1024 most likely ones against that mass, and only a row whose cut lies beyond them goes to the host.
//
// Equal logits rank by index, exactly: when more values tie at the k-th place than the candidate list holds, the
// blocks take the first of them in index order (the reference's list keeps whichever its atomics reach first).
#include "common.cuh"
#include "launch.h"

namespace qb {
namespace {

constexpr int SCL = 8;       // blocks of a row's cluster
constexpr int STH = 1024;    // threads per block
constexpr int SCAP = 2048;   // candidates the leading block sorts at most
constexpr int QD = QB_QD, QCAP = QB_QCAP;

struct SamplerArgs {
    const float* logits;
    int W;           // logits per row
    long long ld;    // floats between rows
    const int* head_ids;
    const int *out_rows, *tok_slot, *ids, *row_first;
    const unsigned *seen, *outs;
    int set_words;   // words per slot of the two sets
    const float* params;
    int *qtok, *qn, *qid;
    float* qp;
    int *out_tok, *out_acc;
    int slice;       // logits per block (a multiple of 32)
};

struct SamplerSmem {
    unsigned hist[256 * 32];          // [bin][lane]
    unsigned long long cand[SCAP];    // leading block: (key << 32 | ~column), later (token << 32 | probability)
    unsigned tot[2][256];             // this block's histogram of a level, read by the whole cluster
    unsigned ctot[256];               // the cluster's
    unsigned long long best[33];      // argmax: per warp, [32] = this block's
    float sh[40];
    unsigned sv[12];
    unsigned eq;                      // values equal to the k-th, this block's count (ties path)
    unsigned wcnt[32];                // ties path: per warp, the equal values of the current chunk
    int chain[QD];
};

__device__ __forceinline__ float unordered(unsigned u) {
    return __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u);
}
__device__ __forceinline__ unsigned cluster_ld_u32(uint32_t addr) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ unsigned long long cluster_ld_u64(uint32_t addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cluster_st_u64(uint32_t addr, unsigned long long v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned cluster_atom_add(uint32_t addr, unsigned v) {
    unsigned r;
    asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(r) : "r"(addr), "r"(v) : "memory");
    return r;
}

// Inclusive prefix sum over the block's 1024 values: shuffles inside each warp, then the warps' totals by warp 0. The
// additions happen in the order of the reference's block_scan (kernels/sampling.cuh:48-68), so the sums have its bits.
__device__ __forceinline__ float scan1024(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float x = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += x;
    }
    if (lane == 31) sh[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = sh[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            float x = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += x;
        }
        sh[lane] = w;
    }
    __syncthreads();
    float r = v + (warp > 0 ? sh[warp - 1] : 0.f);
    __syncthreads();
    return r;
}

// Bitonic network over c[0 .. np), np a power of two: one compare-exchange per thread and step
template <bool ASC>
__device__ __forceinline__ void bitonic_sort(unsigned long long* c, int np, int tid) {
    for (int size = 2; size <= np; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < (np >> 1); t += STH) {
                const int i = ((t & ~(stride - 1)) << 1) | (t & (stride - 1)), o = i | stride;
                const bool up = (i & size) == 0;
                const unsigned long long a = c[i], b = c[o];
                if ((ASC ? a > b : a < b) == up) { c[i] = b; c[o] = a; }
            }
            __syncthreads();
        }
}

__device__ __forceinline__ float q_lookup(const int* qid, const float* qp, int n, int id) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1, v = qid[mid];
        if (v == id) return qp[mid];
        if (v < id) lo = mid + 1; else hi = mid - 1;
    }
    return 0.f;
}

template <bool DRAFT>
__global__ void __launch_bounds__(STH, 1) sampler_kernel(const SamplerArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SamplerSmem& S = *reinterpret_cast<SamplerSmem*>(smem_raw);
    unsigned* stepbits = reinterpret_cast<unsigned*>(smem_raw + sizeof(SamplerSmem));
    unsigned* vals = stepbits + a.slice / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = blockIdx.x, j = blockIdx.y;
    pdl_wait();

    const float* pr = a.params + j * 8;
    const float temp = pr[0], top_p = pr[2], rep = pr[3], u01 = pr[4], u2 = pr[5], pres = pr[7];
    const int top_k = (int)pr[1];
    const int row_tok = a.out_rows[j], slot = a.tok_slot[row_tok];
    int draft = -1, qrow = -1, first = 0, t = 0, k;
    bool greedy = false, wide = false;
    if (DRAFT) {
        t = (int)pr[5];
        k = min(top_k > 0 ? min(top_k, a.W) : QCAP, QCAP);
    } else {
        draft = (int)pr[6];
        first = a.row_first[j];
        if (draft <= -2) {  // a sampled draft: its distribution, if it is still the one stored for the row
            draft = -draft - 2;
            const int tt = row_tok - first, q = slot * QD + tt;
            if (tt < QD && a.qtok[q] == draft && a.qn[q] > 0) qrow = q;
        }
        greedy = temp <= 0.f || top_k == 1;
        // top_k 0 (the whole vocabulary) with a top-p cut: the cut is made among the QCAP most likely tokens against
        // the mass of ALL tokens, when it falls there (it does unless the distribution is nearly flat)
        wide = !greedy && top_k == 0 && top_p < 1.f;
        if (!greedy && !wide && (top_k == 0 || top_k > QCAP)) {  // more candidates than a block sorts: the host's row
            if (rank == 0 && tid == 0) a.out_acc[j] = -1;
            return;
        }
        k = greedy ? 1 : wide ? min(QCAP, a.W) : min(top_k, a.W);
    }

    // ---- this block's slice: penalised logits as order-preserving keys, read once
    const int lo_i = rank * a.slice, n_loc = max(0, min(a.W, lo_i + a.slice) - lo_i);
    const float* L = a.logits + (size_t)j * a.ld;
    const bool penal = rep != 1.f || pres != 0.f;
    const unsigned* sb = a.seen + (size_t)slot * a.set_words;
    const unsigned* ob = a.outs + (size_t)slot * a.set_words;
    if (penal) {
        if (DRAFT) {
            if (tid < QD) S.chain[tid] = tid < t ? a.qtok[slot * QD + tid] : -1;
        } else {
            // the step's tokens of the row's sequence after its first, up to the row's own (drafts fed so far)
            for (int w = tid; w < a.slice / 32; w += STH) stepbits[w] = 0;
            __syncthreads();
            for (int q = first + 1 + tid; q <= row_tok; q += STH) {
                const int x = a.ids[q] - lo_i;
                if (x >= 0 && x < n_loc) atomicOr(&stepbits[x >> 5], 1u << (x & 31));
            }
        }
        __syncthreads();
    }
    {
        const bool vec = (reinterpret_cast<uintptr_t>(L + lo_i) & 15) == 0;
        for (int i4 = tid * 4; i4 < n_loc; i4 += 4 * STH) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const int nv = min(4, n_loc - i4);
            if (vec && nv == 4) {
                const float4 f = *reinterpret_cast<const float4*>(L + lo_i + i4);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
                for (int e = 0; e < nv; e++) v[e] = L[lo_i + i4 + e];
            }
            if (penal) {
                if (DRAFT) {
                    for (int e = 0; e < nv; e++) {
                        const int x = a.head_ids ? a.head_ids[lo_i + i4 + e] : lo_i + i4 + e;
                        bool step = false;  // among the chain's drafts before this one
                        for (int c = 0; c < t; c++) step |= S.chain[c] == x;
                        if (rep != 1.f && (step || ((sb[x >> 5] >> (x & 31)) & 1))) v[e] = v[e] > 0.f ? v[e] / rep : v[e] * rep;
                        if (pres != 0.f && (step || ((ob[x >> 5] >> (x & 31)) & 1))) v[e] -= pres;
                    }
                } else {
                    const int w = (lo_i + i4) >> 5, bit = i4 & 31;
                    const unsigned st = stepbits[i4 >> 5];
                    const unsigned rw = rep != 1.f ? (sb[w] | st) >> bit : 0u;
                    const unsigned pw = pres != 0.f ? (ob[w] | st) >> bit : 0u;
                    for (int e = 0; e < nv; e++) {
                        if ((rw >> e) & 1) v[e] = v[e] > 0.f ? v[e] / rep : v[e] * rep;
                        if ((pw >> e) & 1) v[e] -= pres;
                    }
                }
            }
            for (int e = 0; e < nv; e++) vals[i4 + e] = ordered(v[e]);
        }
    }
    if (tid == 0) { S.sv[3] = 0; S.eq = 0; }
    __syncthreads();

    // ---- whole-vocabulary rows: the largest value, then the mass of all tokens at the temperature (the blocks' sums
    // added in rank order)
    float zall = 0.f;
    if (!DRAFT && wide) {
        unsigned mx = 0;
        for (int i = tid; i < n_loc; i += STH) mx = max(mx, vals[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) S.wcnt[warp] = mx;
        __syncthreads();
        if (warp == 0) {
            mx = S.wcnt[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) S.sv[10] = mx;
        }
        cluster_sync();
        if (warp == 0) {
            mx = lane < SCL ? cluster_ld_u32(cluster_map(&S.sv[10], lane)) : 0u;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) S.sv[11] = mx;
        }
        __syncthreads();
        const float vm = unordered(S.sv[11]);
        float z = 0.f;
        for (int i = tid; i < n_loc; i += STH) z += __expf((unordered(vals[i]) - vm) / temp);
        z = block_sum(z, S.sh);
        if (tid == 0) S.sh[36] = z;
        cluster_sync();
        if (rank == 0)
            for (int r = 0; r < SCL; r++) zall += __uint_as_float(cluster_ld_u32(cluster_map(&S.sh[36], r)));
    }

    // ---- greedy rows: the argmax of the penalised logits, ties to the lower index
    if (!DRAFT && greedy) {
        unsigned long long best = 0;
        for (int i = tid; i < n_loc; i += STH)
            best = max(best, ((unsigned long long)vals[i] << 32) | (0xffffffffu - (unsigned)(lo_i + i)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0) S.best[warp] = best;
        __syncthreads();
        if (warp == 0) {
            best = S.best[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
            if (lane == 0) S.best[32] = best;
        }
        cluster_sync();
        if (rank == 0 && warp == 0) {
            best = lane < SCL ? cluster_ld_u64(cluster_map(&S.best[32], lane)) : 0ull;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
            if (lane == 0) {
                const int tok = (int)(0xffffffffu - (unsigned)best);
                a.out_tok[j] = tok;
                a.out_acc[j] = draft >= 0 && tok == draft;
            }
        }
        cluster_sync();  // the others' shared memory stays until the leading block has read it
        return;
    }

    // ---- radix select: the bin of the k-th largest key, 8 bits per level, until the candidates fit the list
    const int cap = min(SCAP, max(256, 2 * k));
    unsigned prefix = 0, mask = 0, above = 0, in_bin = 0;
    bool fits = false;
    for (int level = 0; level < 4; level++) {
        const int shift = 24 - 8 * level;
        for (int w = tid; w < 256 * 32; w += STH) S.hist[w] = 0;
        __syncthreads();
        for (int i = tid; i < n_loc; i += STH) {
            const unsigned u = vals[i];
            if ((u & mask) == prefix) atomicAdd(&S.hist[(((u >> shift) & 255) << 5) + lane], 1u);
        }
        __syncthreads();
        if (tid < 256) {
            unsigned c = 0;
#pragma unroll 8
            for (int l = 0; l < 32; l++) c += S.hist[(tid << 5) + ((l + tid) & 31)];
            S.tot[level & 1][tid] = c;
        }
        cluster_sync();
        if (tid < 256) {
            unsigned c = 0;
#pragma unroll
            for (int r = 0; r < SCL; r++) c += cluster_ld_u32(cluster_map(&S.tot[level & 1][tid], r));
            S.ctot[tid] = c;
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns bins 255 - 8l down to 248 - 8l; counts from the top
            unsigned mine = 0;
#pragma unroll
            for (int q = 0; q < 8; q++) mine += S.ctot[255 - 8 * lane - q];
            unsigned incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned x = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += x;
            }
            unsigned c = above + incl - mine;
            if (c < (unsigned)k && above + incl >= (unsigned)k) {
                for (int q = 0; q < 8; q++) {
                    const int b = 255 - 8 * lane - q;
                    const unsigned h = S.ctot[b];
                    if (c + h >= (unsigned)k) { S.sv[0] = b; S.sv[1] = c; S.sv[2] = h; break; }
                    c += h;
                }
            }
        }
        __syncthreads();
        prefix |= S.sv[0] << shift;
        mask |= 255u << shift;
        above = S.sv[1];
        in_bin = S.sv[2];
        if (above + in_bin <= (unsigned)cap) { fits = true; break; }
    }

    // ---- candidates to the leading block's list
    const uint32_t r_cnt = cluster_map(&S.sv[3], 0), r_cand = cluster_map(&S.cand[0], 0);
    if (fits) {
        // every key at or above the lower edge of the bin
        for (int i = tid; i < n_loc; i += STH) {
            const unsigned u = vals[i];
            if (u >= prefix) {
                const unsigned at = cluster_atom_add(r_cnt, 1u);
                if (at < (unsigned)SCAP)
                    cluster_st_u64(r_cand + at * 8, ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)(lo_i + i)));
            }
        }
    } else {
        // more keys equal to the k-th (`prefix`, now exact) than the list holds: the keys above it and, in index
        // order, the first k - above of the equal ones. Blocks own ascending index ranges.
        unsigned mine = 0;
        for (int i = tid; i < n_loc; i += STH) mine += vals[i] == prefix;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        if (lane == 0 && mine) atomicAdd(&S.eq, mine);
        cluster_sync();
        unsigned before = 0;
        for (int r = 0; r < rank; r++) before += cluster_ld_u32(cluster_map(&S.eq, r));
        const unsigned need = (unsigned)k - above;
        const unsigned quota = before >= need ? 0u : min(need - before, S.eq);
        unsigned taken = 0;  // equal keys of earlier chunks
        for (int base = 0; base < n_loc; base += STH) {
            const int i = base + tid;
            const unsigned u = i < n_loc ? vals[i] : 0u;
            const bool eqv = i < n_loc && u == prefix;
            const unsigned bal = __ballot_sync(0xffffffffu, eqv);
            if (lane == 0) S.wcnt[warp] = __popc(bal);
            __syncthreads();
            unsigned wbefore = 0, chunk = 0;
            for (int w = 0; w < 32; w++) {
                const unsigned c = S.wcnt[w];
                if (w < warp) wbefore += c;
                chunk += c;
            }
            const unsigned pos = taken + wbefore + __popc(bal & ((1u << lane) - 1));
            if ((i < n_loc && u > prefix) || (eqv && pos < quota)) {
                const unsigned at = cluster_atom_add(r_cnt, 1u);
                if (at < (unsigned)SCAP)
                    cluster_st_u64(r_cand + at * 8, ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)(lo_i + i)));
            }
            taken += chunk;
            __syncthreads();
        }
    }
    cluster_sync();
    if (rank != 0) return;

    // ---- the leading block: sort the candidates (descending by value, ties to the lower index), softmax, cut, draw
    const int cnt = min((int)S.sv[3], SCAP);
    int np = 1;
    while (np < cnt) np <<= 1;
    for (int i = cnt + tid; i < np; i += STH) S.cand[i] = 0;
    __syncthreads();
    bitonic_sort<false>(S.cand, np, tid);
    k = min(k, cnt);
    auto column = [&](int r) { return (int)(0xffffffffu - (unsigned)S.cand[r]); };
    auto value = [&](int r) { return unordered((unsigned)(S.cand[r] >> 32)); };
    // softmax of the top k at the temperature, its prefix, the top-p cut (kernels/sampling.cuh:141-165)
    const float vmax = value(0);
    const float p = tid < k ? __expf((value(tid) - vmax) / temp) : 0.f;
    const float cum = scan1024(p, S.sh);
    if (tid == k - 1) S.sh[32] = cum;
    if (tid == 0) S.sv[4] = k;
    __syncthreads();
    const float total = wide ? zall : S.sh[32];
    if (wide && !(S.sh[32] / total >= top_p)) {  // the cut lies beyond the candidates: the host's row
        if (tid == 0) a.out_acc[j] = -1;
        return;
    }
    if (top_p < 1.f && tid < k && cum / total >= top_p) atomicMin(&S.sv[4], (unsigned)tid + 1);
    __syncthreads();
    const int keep = S.sv[4];
    if (tid == keep - 1) S.sh[33] = cum;
    __syncthreads();
    const float mass = S.sh[33];

    if (DRAFT) {
        // the draw: the first kept token whose prefix reaches u * mass; q = the kept tokens in ascending id order
        const int q = slot * QD + t;
        const float target = u01 * mass;
        if (tid == 0) S.sv[5] = keep - 1;
        __syncthreads();
        if (tid < keep && cum >= target) atomicMin(&S.sv[5], (unsigned)tid);
        __syncthreads();
        int x = 0x7fffffff;
        if (tid < keep) {
            const int c = column(tid);
            x = a.head_ids ? a.head_ids[c] : c;
        }
        const float prob = tid < keep ? p / mass : 0.f;
        if (tid == (int)S.sv[5]) { a.out_tok[j] = x; a.qtok[q] = x; a.qn[q] = keep; }
        __syncthreads();
        int nq = 1;
        while (nq < keep) nq <<= 1;
        for (int i = keep + tid; i < nq; i += STH) S.cand[i] = ~0ull;
        if (tid < keep) S.cand[tid] = ((unsigned long long)(unsigned)x << 32) | __float_as_uint(prob);
        __syncthreads();
        bitonic_sort<true>(S.cand, nq, tid);
        if (tid < keep) {
            a.qid[(size_t)q * QCAP + tid] = (int)(S.cand[tid] >> 32);
            a.qp[(size_t)q * QCAP + tid] = __uint_as_float((unsigned)S.cand[tid]);
        }
        return;
    }

    // the draft's probability among the kept tokens
    if (tid == 0) { S.sh[34] = 0.f; S.sv[6] = 0xffffffffu; }
    __syncthreads();
    if (draft >= 0 && tid < keep && column(tid) == draft) { S.sh[34] = p / mass; S.sv[6] = tid; }
    __syncthreads();
    const float pd = S.sh[34];
    const unsigned at_d = S.sv[6];
    if (qrow >= 0) {
        // d ~ q: accepted with probability min(1, p(d) / q(d)), else a draw from max(0, p - q) normalised
        const int* qi = a.qid + (size_t)qrow * QCAP;
        const float* qv = a.qp + (size_t)qrow * QCAP;
        const int nq = a.qn[qrow];
        const float qd = q_lookup(qi, qv, nq, draft);
        if (u01 * qd < pd) {
            if (tid == 0) { a.out_tok[j] = draft; a.out_acc[j] = 1; }
            return;
        }
        const float r = tid < keep ? fmaxf(p / mass - q_lookup(qi, qv, nq, column(tid)), 0.f) : 0.f;
        const float cr = scan1024(r, S.sh);
        if (tid == STH - 1) S.sh[35] = cr;
        if (tid == 0) { S.sv[7] = 0xffffffffu; S.sv[8] = 0; }
        __syncthreads();
        const float rtot = S.sh[35], target = u2 * rtot;
        if (r > 0.f && cr >= target) atomicMin(&S.sv[7], (unsigned)tid);
        if (r > 0.f) atomicMax(&S.sv[8], (unsigned)tid);
        __syncthreads();
        if (tid == 0) {
            // none crossed (rounding at the top end): the last token with residual mass; no residual mass at all
            // (rounding again): the most likely token
            const unsigned at = S.sv[7] != 0xffffffffu ? S.sv[7] : S.sv[8];
            a.out_tok[j] = column(rtot > 0.f ? (int)at : 0);
            a.out_acc[j] = 0;
        }
        return;
    }
    if (draft >= 0 && u01 < pd) {
        if (tid == 0) { a.out_tok[j] = draft; a.out_acc[j] = 1; }
        return;
    }
    // a draw from the kept tokens, without the rejected draft
    const float target = draft >= 0 ? u2 * (mass - pd * mass) : u01 * mass;
    const float c2 = cum - (at_d != 0xffffffffu && (unsigned)tid >= at_d ? pd * mass : 0.f);
    const bool live = tid < keep && (unsigned)tid != at_d;
    if (tid == 0) S.sv[9] = keep - 1;
    __syncthreads();
    if (live && c2 >= target) atomicMin(&S.sv[9], (unsigned)tid);
    __syncthreads();
    if (tid == 0) {
        int r = S.sv[9];
        if ((unsigned)r == at_d) r = r + 1 < keep ? r + 1 : r - 1;  // only when the draft was the last one left
        a.out_tok[j] = column(r);
        a.out_acc[j] = 0;
    }
}

template <bool DRAFT>
int launch_sampler(qb_ctx* ctx, void* stream, SamplerArgs a, int n_out) {
    if (!ctx || !a.logits || !a.params || !a.out_rows || !a.tok_slot || !a.seen || !a.outs || !a.out_tok || a.W <= 0 ||
        n_out < 0 || a.set_words <= 0)
        return QB_ERR_ARG;
    if (n_out == 0) return QB_OK;
    a.slice = ((a.W + SCL - 1) / SCL + 31) / 32 * 32;
    const size_t smem = sizeof(SamplerSmem) + (size_t)a.slice / 32 * 4 + (size_t)a.slice * 4;
    if (smem > 227 * 1024) return QB_ERR_TOO_LARGE;
    if (int rc = qb::prepare_kernel(ctx->device, (const void*)sampler_kernel<DRAFT>, 227 * 1024)) return rc;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(SCL, n_out);
    lc.blockDim = dim3(STH);
    lc.dynamicSmemBytes = smem;
    lc.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = SCL; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = ctx->pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, sampler_kernel<DRAFT>, a);
    return e == cudaSuccess ? QB_OK : (int)e;
}

}  // namespace
}  // namespace qb

extern "C" int qb_sample_rows(qb_ctx* ctx, void* stream, const float* logits, int width, int ld, int vocab, int n_out,
                              const int* out_rows, const int* tok_slot, const int* ids, const int* row_first,
                              const unsigned* seen, const unsigned* outs, const float* params, const int* qtok,
                              const int* qn, const int* qid, const float* qp, int* out_tok, int* out_acc) {
    if (!ids || !row_first || !qtok || !qn || !qid || !qp || !out_acc || vocab % 32 || width > vocab || ld < width)
        return QB_ERR_ARG;
    qb::SamplerArgs a = {};
    a.logits = logits; a.W = width; a.ld = ld; a.head_ids = nullptr;
    a.out_rows = out_rows; a.tok_slot = tok_slot; a.ids = ids; a.row_first = row_first;
    a.seen = seen; a.outs = outs; a.set_words = vocab / 32; a.params = params;
    a.qtok = const_cast<int*>(qtok); a.qn = const_cast<int*>(qn); a.qid = const_cast<int*>(qid);
    a.qp = const_cast<float*>(qp);
    a.out_tok = out_tok; a.out_acc = out_acc;
    return qb::launch_sampler<false>(ctx, stream, a, n_out);
}

extern "C" int qb_draft_sample(qb_ctx* ctx, void* stream, const float* logits, int width, int ld, const int* head_ids,
                               int vocab, int n_out, const int* out_rows, const int* tok_slot, const unsigned* seen,
                               const unsigned* outs, const float* params, int* drafts, int* qtok, int* qn, int* qid,
                               float* qp) {
    if (!qtok || !qn || !qid || !qp || vocab % 32 || ld < width || (!head_ids && width > vocab)) return QB_ERR_ARG;
    qb::SamplerArgs a = {};
    a.logits = logits; a.W = width; a.ld = ld; a.head_ids = head_ids;
    a.out_rows = out_rows; a.tok_slot = tok_slot; a.ids = nullptr; a.row_first = nullptr;
    a.seen = seen; a.outs = outs; a.set_words = vocab / 32; a.params = params;
    a.qtok = qtok; a.qn = qn; a.qid = qid; a.qp = qp;
    a.out_tok = drafts; a.out_acc = nullptr;
    return qb::launch_sampler<true>(ctx, stream, a, n_out);
}
