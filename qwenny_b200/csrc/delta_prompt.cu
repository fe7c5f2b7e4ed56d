// Gated DeltaNet for steps whose segments are not decode-sized (prompt chunks, long verify steps, and every step that
// does not take the one-launch mixer of deltanet.cu). Same entry points and buffers as the reference's three kernels
// (kernels/qwen_deltanet.cuh: delta_conv :84-131, delta_rule :172-288, delta_norm :295-315), another algorithm:
//
//  delta_prep_kernel        the causal depthwise conv, SiLU, the L2 norms of the q and k heads and the two gates. A
//                           thread owns ONE channel and slides along 16 tokens with the conv's four inputs in
//                           registers (each input row is read once, not four times); the 128 channels of a block are
//                           one q, k or v head, so the head's norm is a block reduction per token.
//  delta_chunk_prep_kernel  the part of the CHUNKED delta rule that does not depend on the state (the WY form the
//                           reference states for its MLX backend, src/mlx/delta.rs:6-15,85-137; chunks of 64 tokens):
//                           per chunk and key head K K^T and Q K^T once, then per value head the unit lower triangular
//                           system's inverse T = (I + A)^-1, A_ij = b_i (k_i . k_j) exp(G_i - G_j), and
//                           P_ij = (q_i . k_j) exp(G_i - G_j). All chunks of all segments in parallel.
//  delta_scan_kernel        a block per (half of a value head's columns, value head, segment) carries its 64 x 128 slice
//                           of the f32 state in shared memory from chunk to chunk: R = b (V - gam K S^T), D = T R,
//                           O = gam Q S^T + P D, S' = gam_C S + D^T (k_j exp(G_C - G_j)). The contractions run on the
//                           tensor cores as 3 x TF32 (every operand split into a TF32 head and tail, three products
//                           per term), which keeps f32 accuracy: the state stays within 1e-4 of the token recurrence
//                           over thousands of tokens. The last 16..79 tokens of a segment, any replayed tokens and
//                           short segments run in the token form with the operation order of the decode mixer, so the
//                           checkpoint, the replay bank and a later rollback see the bits a decode step would make.
//  delta_gate_norm_kernel   RMSNorm(w) * SiLU(z) per value head -> f16, then the slots' metadata.
#include "delta_common.cuh"
#include "launch.h"

namespace qb {

// ------------------------------------------------------------------------------------------------ delta_prep
constexpr int PREP_TOK = 16;  // tokens a block slides along

__device__ __forceinline__ float in_sum(const float* p, int splits, size_t stride, size_t at) {
    float v = p[at];
    for (int s = 1; s < splits; s++) v += p[at + s * stride];
    return v;
}

// grid (LQKV / 128, ceil(n / PREP_TOK)), block 128: thread c is channel 128 blockIdx.x + c
__global__ void __launch_bounds__(128)
delta_prep_kernel(const float* p, int splits, int n, const float* ba, int ba_splits, const float* cw,
                  const float* a_log, const float* dt_bias, const float* mem, long long sst, float* cv,
                  const int* tok_slot, const int* tok_pos) {
    __shared__ float ss_part[PREP_TOK][4];
    pdl_launch_dependents();
    const int head = blockIdx.x, ch = head * 128 + threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tb = blockIdx.y * PREP_TOK, cnt = min(PREP_TOK, n - tb);
    const float4 taps = ld4(cw + (size_t)ch * CONV_K);
    pdl_wait();
    const size_t stride = (size_t)n * DELTA_IN;
    // every load of the tile first (they are independent), the sliding window after
    float x[PREP_TOK], y[PREP_TOK];
    int slots[PREP_TOK], poss[PREP_TOK];
#pragma unroll
    for (int i = 0; i < PREP_TOK; i++) {
        const int t = min(tb + i, n - 1);
        x[i] = in_sum(p, splits, stride, (size_t)t * DELTA_IN + ch);
        slots[i] = tok_slot[t];
        poss[i] = tok_pos[t];
    }
    float h0 = 0.f, h1 = 0.f, h2 = 0.f;  // the conv inputs at the three positions before the current token
    int prev_slot = -1;
#pragma unroll
    for (int i = 0; i < PREP_TOK; i++) {
        y[i] = 0.f;
        if (i < cnt) {
            const int t = tb + i, slot = slots[i], pos = poss[i];
            if (slot != prev_slot) {
                // a segment starts in this tile (or the tile starts): fetch the history, from the step's own rows of
                // the same sequence or from the slot's ring
                auto hist = [&](int back) {
                    const int qp = pos - back, tt = t - back;
                    if (qp < 0) return 0.f;
                    if (tt >= 0 && tok_slot[tt] == slot) return in_sum(p, splits, stride, (size_t)tt * DELTA_IN + ch);
                    return mem[slot * sst + SLOT_RING + (size_t)(qp & (CR - 1)) * LQKV + ch];
                };
                h0 = hist(3); h1 = hist(2); h2 = hist(1);
                prev_slot = slot;
            }
            float a = taps.x * h0;
            a = fmaf(taps.y, h1, a);
            a = fmaf(taps.z, h2, a);
            a = fmaf(taps.w, x[i], a);
            y[i] = silu(a);
            h0 = h1; h1 = h2; h2 = x[i];
        }
    }
    if (head < 2 * LK_HEADS) {  // a q or k head: L2 norm over the block's 128 channels, q also / sqrt(128)
#pragma unroll
        for (int i = 0; i < PREP_TOK; i++) {
            float s = warp_sum(y[i] * y[i]);
            if (lane == 0) ss_part[i][warp] = s;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PREP_TOK; i++) {
            float sc = rsqrtf(((ss_part[i][0] + ss_part[i][1]) + (ss_part[i][2] + ss_part[i][3])) + 1e-6f);
            if (head < LK_HEADS) sc *= rsqrtf((float)LKD);
            y[i] *= sc;
        }
    }
#pragma unroll
    for (int i = 0; i < PREP_TOK; i++)
        if (i < cnt) cv[(size_t)(tb + i) * CVW + ch] = y[i];
    if (head == 0) {  // the gates of the tile's tokens: exp(g) and beta per value head
        for (int x = threadIdx.x; x < cnt * LV_HEADS; x += 128) {
            const int t = tb + x / LV_HEADS, v = x % LV_HEADS;
            float b = 0.f, a = 0.f;
            for (int s = 0; s < ba_splits; s++) {
                const float* r = ba + ((size_t)s * n + t) * (2 * LV_HEADS);
                b += r[v];
                a += r[LV_HEADS + v];
            }
            a += dt_bias[v];
            const float sp = a > 20.f ? a : log1pf(expf(a));
            cv[(size_t)t * CVW + LQKV + v] = expf(-expf(a_log[v]) * sp);
            cv[(size_t)t * CVW + LQKV + LV_HEADS + v] = 1.f / (1.f + expf(-b));
        }
    }
}

// ------------------------------------------------------------------------------------------------ the chunked form
constexpr int CH = 64;                   // tokens per chunk
constexpr int TP_FLOATS = 2 * CH * CH + CH;  // per (chunk, value head): T, P, the cumulative log decays
constexpr int KLD = LKD + 4;             // row stride of the q / k / state tiles (floats): fragment loads hit 32 banks
constexpr int TLD = CH + 4;              // ... of T and P
constexpr int RLD = 64 + 8;              // ... of R, D and V (read with the token index on the fragment's k side)

// tokens of a segment that run in chunks: whole chunks that end at least KEEP tokens before the segment's end (the
// checkpoint and the bank of the rollback plan are made in the token form)
__host__ __device__ __forceinline__ int chunked_tokens(int len) { return len >= CH + KEEP ? (len - KEEP) / CH * CH : 0; }

// ---- 3 x TF32 on mma.sync m16n8k8: x = hi + lo, hi the upper 19 bits of x (a TF32 value), lo = x - hi exactly (the
// tensor core ignores the 13 low bits of an operand, so lo enters with 11 more bits of x); a . b ~ lo_a hi_b + hi_a lo_b
// + hi_a hi_b. Products that only feed the step's outputs take operands rounded to TF32 once.
__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ uint32_t tf32_round(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
struct FragA { uint32_t hi[4], lo[4]; };
__device__ __forceinline__ FragA frag_a(float a0, float a1, float a2, float a3) {
    FragA f;
    tf32_split(a0, f.hi[0], f.lo[0]); tf32_split(a1, f.hi[1], f.lo[1]);
    tf32_split(a2, f.hi[2], f.lo[2]); tf32_split(a3, f.hi[3], f.lo[3]);
    return f;
}
__device__ __forceinline__ void mma3(float* c, const FragA& a, float b0, float b1) {
    uint32_t h0, l0, h1, l1;
    tf32_split(b0, h0, l0);
    tf32_split(b1, h1, l1);
    mma_tf32(c, a.lo, h0, h1);
    mma_tf32(c, a.hi, l0, l1);
    mma_tf32(c, a.hi, h0, h1);
}

// grid (chunks of the longest possible segment, LK_HEADS, segs), block 256. tp: [chunk index][LV_HEADS][TP_FLOATS],
// chunk index = first token of the chunk / 64 (distinct for disjoint 64-token ranges).
constexpr int CP_THREADS = 256;
constexpr int CP_SMEM = (2 * CH * KLD + 2 * CH * (CH + 1) + 6 * CH) * 4;  // 102 KB: two blocks per SM
static_assert(3 * CH * (CH + 1) <= 2 * CH * KLD, "the three A matrices reuse the q / k tiles");

__global__ void __launch_bounds__(CP_THREADS)
delta_chunk_prep_kernel(const float* cv, float* tp, const int* seg_start, const int* seg_len) {
    extern __shared__ __align__(16) float cps[];
    float* Ks = cps;                         // [64][KLD]; later A of the three value heads [3][64][65]
    float* Qs = Ks + CH * KLD;
    float* KK = Qs + CH * KLD;               // [64][65]; later scratch of the inverse
    float* QK = KK + CH * (CH + 1);
    float* gs = QK + CH * (CH + 1);          // [3][64] cumulative log decay
    float* bs = gs + 3 * CH;                 // [3][64] beta
    pdl_launch_dependents();
    const int c = blockIdx.x, kh = blockIdx.y, sg = blockIdx.z, tid = threadIdx.x;
    const int t0 = seg_start[sg], len = seg_len[sg];
    if (c * CH >= chunked_tokens(len)) return;
    const int tok = t0 + c * CH;
    const int G = LV_HEADS / LK_HEADS;
    pdl_wait();
    for (int x = tid; x < CH * (LKD / 4); x += CP_THREADS) {
        const int r = x / (LKD / 4), d = (x % (LKD / 4)) * 4;
        const float* row = cv + (size_t)(tok + r) * CVW + kh * LKD + d;
        cp_async16(Qs + r * KLD + d, row);
        cp_async16(Ks + r * KLD + d, row + LK_HEADS * LKD);
    }
    cp_async_commit();
    if (tid < 3 * 32) {  // a warp per value head: the gates, and the running sum of the log decays
        const int hv = tid >> 5, lane = tid & 31, h = kh * G + hv;
        float l0 = logf(cv[(size_t)(tok + 2 * lane) * CVW + LQKV + h]);
        float l1 = logf(cv[(size_t)(tok + 2 * lane + 1) * CVW + LQKV + h]);
        bs[hv * CH + 2 * lane] = cv[(size_t)(tok + 2 * lane) * CVW + LQKV + LV_HEADS + h];
        bs[hv * CH + 2 * lane + 1] = cv[(size_t)(tok + 2 * lane + 1) * CVW + LQKV + LV_HEADS + h];
        float run = l0 + l1;  // inclusive scan of the pair sums over the lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            float up = __shfl_up_sync(0xffffffffu, run, o);
            if (lane >= o) run += up;
        }
        gs[hv * CH + 2 * lane] = run - l1;
        gs[hv * CH + 2 * lane + 1] = run;
    }
    cp_async_wait_all();
    __syncthreads();
    // K K^T and Q K^T on the tensor cores (3 x TF32): warp (matrix, 16-row tile m) takes the column tiles of the lower
    // triangle, 0 .. 2 m + 1
    {
        const int warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
        const int m = warp & 3, nts = 2 * m + 2;
        const float* ar = (warp >> 2 ? Qs : Ks) + (16 * m + g8) * KLD + t4;
        const float* br = Ks + g8 * KLD + t4;
        float* dst = warp >> 2 ? QK : KK;
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        for (int k0 = 0; k0 < LKD; k0 += 8) {
            const FragA a = frag_a(ar[k0], ar[8 * KLD + k0], ar[k0 + 4], ar[8 * KLD + k0 + 4]);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (j < nts) mma3(acc[j], a, br[8 * j * KLD + k0], br[8 * j * KLD + k0 + 4]);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float* d0 = dst + (16 * m + g8) * (CH + 1) + 8 * j + 2 * t4;
            d0[0] = acc[j][0]; d0[1] = acc[j][1];
            d0[8 * (CH + 1)] = acc[j][2]; d0[8 * (CH + 1) + 1] = acc[j][3];
        }
    }
    __syncthreads();
    // A of the three value heads over the q / k tiles (done with), and P straight to global memory
    float* As = Ks;
    for (int x = tid; x < 3 * CH * CH; x += CP_THREADS) {
        const int hv = x / (CH * CH), i = (x / CH) % CH, j = x % CH;
        const float dec = j <= i ? expf(gs[hv * CH + i] - gs[hv * CH + j]) : 0.f;
        As[(hv * CH + i) * (CH + 1) + j] = j < i ? bs[hv * CH + i] * KK[i * (CH + 1) + j] * dec : 0.f;
        float* out = tp + ((size_t)(tok >> 6) * LV_HEADS + kh * G + hv) * TP_FLOATS;
        out[CH * CH + i * CH + j] = j <= i ? QK[i * (CH + 1) + j] * dec : 0.f;
        if (j == 0) out[2 * CH * CH + i] = gs[hv * CH + i];
    }
    __syncthreads();
    // T = (I + A)^-1, unit lower triangular, IN PLACE over A. The four 16 x 16 diagonal blocks by forward substitution,
    // a thread per column (T_ic = -sum_{c <= j < i} A_ij T_jc), into scratch and back; then blocks merge pairwise,
    // 16 -> 32 -> 64: for a block pair [[T11, 0], [T21, T22]] the lower left part is T21 = -T22 (A21 T11), two small
    // products spread over the block (X = A21 T11 goes through scratch, so T21 may overwrite A21).
    float* D0 = KK;                    // [3][4][16][17] the diagonal blocks' inverses
    float* Xs = KK + 3 * 4 * 16 * 17;  // [3][32][33] scratch of the merges (K K^T and Q K^T are done with)
    float* Ts = As;
    if (tid < 3 * CH) {
        const int hv = tid / CH, blk = (tid % CH) / 16, b0 = blk * 16, col = tid % 16;
        const float* A = As + hv * CH * (CH + 1);
        float* T = D0 + (hv * 4 + blk) * 16 * 17;
        for (int i = 0; i < col; i++) T[i * 17 + col] = 0.f;
        T[col * 17 + col] = 1.f;
        for (int i = col + 1; i < 16; i++) {
            float s0 = 0.f, s1 = 0.f;
            int j = col;
            for (; j + 1 < i; j += 2) {
                s0 = fmaf(A[(b0 + i) * (CH + 1) + b0 + j], T[j * 17 + col], s0);
                s1 = fmaf(A[(b0 + i) * (CH + 1) + b0 + j + 1], T[(j + 1) * 17 + col], s1);
            }
            if (j < i) s0 = fmaf(A[(b0 + i) * (CH + 1) + b0 + j], T[j * 17 + col], s0);
            T[i * 17 + col] = -(s0 + s1);
        }
    }
    __syncthreads();
    for (int x = tid; x < 3 * 4 * 256; x += CP_THREADS) {
        const int hv = x / 1024, blk = (x / 256) % 4, i = (x % 256) / 16, j = x % 16;
        Ts[(hv * CH + blk * 16 + i) * (CH + 1) + blk * 16 + j] = D0[((hv * 4 + blk) * 16 + i) * 17 + j];
    }
    __syncthreads();
    for (int half = 16; half < CH; half *= 2) {
        const int pairs = CH / (2 * half), per = half * half;
        // X = A21 T11 (T11 lower triangular: the sum over b starts at the column)
        for (int x = tid; x < 3 * pairs * per; x += CP_THREADS) {
            const int hv = x / (pairs * per), pr = (x / per) % pairs, i = (x % per) / half, j = x % half;
            const int base = pr * 2 * half;
            const float* A = As + hv * CH * (CH + 1) + (base + half + i) * (CH + 1) + base;
            const float* T = Ts + hv * CH * (CH + 1) + base * (CH + 1) + base + j;
            float s0 = 0.f, s1 = 0.f;
            int b = j;
            for (; b + 1 < half; b += 2) {
                s0 = fmaf(A[b], T[b * (CH + 1)], s0);
                s1 = fmaf(A[b + 1], T[(b + 1) * (CH + 1)], s1);
            }
            if (b < half) s0 = fmaf(A[b], T[b * (CH + 1)], s0);
            Xs[(hv * 32 + pr * half + i) * 33 + j] = s0 + s1;
        }
        __syncthreads();
        // T21 = -T22 X (T22 lower triangular: the sum over a ends at the row)
        for (int x = tid; x < 3 * pairs * per; x += CP_THREADS) {
            const int hv = x / (pairs * per), pr = (x / per) % pairs, i = (x % per) / half, j = x % half;
            const int base = pr * 2 * half;
            const float* T22 = Ts + hv * CH * (CH + 1) + (base + half + i) * (CH + 1) + base + half;
            const float* X = Xs + (hv * 32 + pr * half) * 33 + j;
            float s0 = 0.f, s1 = 0.f;
            int a2 = 0;
            for (; a2 + 1 <= i; a2 += 2) {
                s0 = fmaf(T22[a2], X[a2 * 33], s0);
                s1 = fmaf(T22[a2 + 1], X[(a2 + 1) * 33], s1);
            }
            if (a2 <= i) s0 = fmaf(T22[a2], X[a2 * 33], s0);
            Ts[hv * CH * (CH + 1) + (base + half + i) * (CH + 1) + base + j] = -(s0 + s1);
        }
        __syncthreads();
    }
    for (int x = tid; x < 3 * CH * CH; x += CP_THREADS) {
        const int hv = x / (CH * CH), i = (x / CH) % CH, j = x % CH;
        tp[((size_t)(tok >> 6) * LV_HEADS + kh * G + hv) * TP_FLOATS + i * CH + j] = Ts[(hv * CH + i) * (CH + 1) + j];
    }
}

constexpr int SC_THREADS = 512, SC_COLS = 64;   // threads of a scan block; value columns of its state slice
constexpr int SC_TAIL = 16;                      // tokens staged per round of the token form
struct ScanSmem {
    float kq[2 * CH][KLD];     // chunk: k rows 0..63, q rows 64..127; token form: q / k / v of a round
    float t[CH][TLD], pm[CH][TLD];
    float s[SC_COLS][KLD];     // the state slice [value column][key]
    float r[CH][RLD], d[CH][RLD];
    float g[CH], b[CH], gam[CH], dec[CH];
    float te[SC_TAIL], tb[SC_TAIL], tkq[SC_TAIL];
};

__global__ void __launch_bounds__(SC_THREADS, 1)
delta_scan_kernel(const float* p, int splits, int n, const float* cv, const float* tp, float* mem, long long sst,
                  const int* meta, float* out, const int* seg_start, const int* seg_len, const int* seg_slot,
                  const int* seg_pos0) {
    extern __shared__ __align__(16) uint8_t scan_raw[];
    ScanSmem& M = *(ScanSmem*)scan_raw;
    pdl_launch_dependents();
    const int vs = blockIdx.x, h = blockIdx.y, sg = blockIdx.z, kh = h / (LV_HEADS / LK_HEADS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
    const int lc = tid >> 3, sub = tid & 7, col = vs * SC_COLS + lc;   // token form: 8 lanes per value column
    const int t0 = seg_start[sg], len = seg_len[sg], slot = seg_slot[sg], p0 = seg_pos0[sg];
    const Plan pl = make_plan(meta, slot, p0, len);
    float* sm0 = mem + slot * sst;
    auto sbuf = [&](int b) { return sm0 + (size_t)b * SLOT_STATE + ((size_t)h * LVD + col) * LKD; };
    auto entry = [&](int b, int pos) { return sm0 + 2 * SLOT_STATE + (size_t)b * SLOT_BANK + (size_t)(pos % KEEP) * REP; };
    constexpr int RPT = LKD / 8;
    // ---- the state, and the replay of accepted tokens from the bank: nothing here depends on this step's kernels
    float S[RPT];
    if (pl.zero) {
#pragma unroll
        for (int i = 0; i < RPT; i++) S[i] = 0.f;
    } else {
        ld_rows<8>(S, sbuf(pl.in), sub);
    }
    for (int i = 0; i < pl.r; i++) {
        const float* e = entry(pl.in, pl.from + i);
        float k[RPT];
        ld_rows<8>(k, e + kh * LKD, sub);
        const float dk = dot_rows<8>(S, k);
        const float ex = e[LK_HEADS * LKD + LV_HEADS * LVD + h], be = e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h];
        const float delta = (e[LK_HEADS * LKD + h * LVD + col] - ex * dk) * be;
#pragma unroll
        for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
    }
    pdl_wait();

    const int l0 = chunked_tokens(len);
    if (l0 > 0) {
        // ================================================================ chunks
        st_rows<8>(&M.s[lc][0], S, sub);
        const int mq = warp >> 2, nq = warp & 3;   // a warp's 16-row tile and 16-column tile in G1, G2 and G3
        auto load_q = [&](int tok) {
            for (int x = tid; x < CH * (LKD / 4); x += SC_THREADS) {
                const int r = x / (LKD / 4), dd = (x % (LKD / 4)) * 4;
                cp_async16(&M.kq[CH + r][dd], cv + (size_t)(tok + r) * CVW + kh * LKD + dd);
            }
        };
        auto load_k = [&](int tok) {
            for (int x = tid; x < CH * (LKD / 4); x += SC_THREADS) {
                const int r = x / (LKD / 4), dd = (x % (LKD / 4)) * 4;
                cp_async16(&M.kq[r][dd], cv + (size_t)(tok + r) * CVW + LK_HEADS * LKD + kh * LKD + dd);
            }
        };
        auto load_tv = [&](int tok) {  // T, the block's value columns (into r), the gates
            const float* src = tp + ((size_t)(tok >> 6) * LV_HEADS + h) * TP_FLOATS;
            for (int x = tid; x < CH * (CH / 4); x += SC_THREADS) {
                const int r = x / (CH / 4), dd = (x % (CH / 4)) * 4;
                cp_async16(&M.t[r][dd], src + r * CH + dd);
                cp_async16(&M.r[r][dd], cv + (size_t)(tok + r) * CVW + 2 * LK_HEADS * LKD + h * LVD + vs * SC_COLS + dd);
            }
            if (tid < CH / 4) cp_async16(&M.g[tid * 4], src + 2 * CH * CH + tid * 4);
            if (tid >= 32 && tid < 32 + CH) cp_async4(&M.b[tid - 32], cv + (size_t)(tok + tid - 32) * CVW + LQKV + LV_HEADS + h);
        };
        auto load_p = [&](int tok) {
            const float* src = tp + ((size_t)(tok >> 6) * LV_HEADS + h) * TP_FLOATS + CH * CH;
            for (int x = tid; x < CH * (CH / 4); x += SC_THREADS) {
                const int r = x / (CH / 4), dd = (x % (CH / 4)) * 4;
                cp_async16(&M.pm[r][dd], src + r * CH + dd);
            }
        };
        load_q(t0); load_k(t0); load_tv(t0);
        cp_async_commit();
        load_p(t0);
        cp_async_commit();
        for (int c0 = 0; c0 < l0; c0 += CH) {
            const int tok = t0 + c0;
            const bool more = c0 + CH < l0;
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");  // everything but P
            __syncthreads();
            if (tid < CH) {
                M.gam[tid] = expf(M.g[tid]);
                M.dec[tid] = expf(M.g[CH - 1] - M.g[tid]);
            }
            // ---- G1: K S^T (3 x TF32: it feeds the state) and Q S^T (q rounded once, S split: it feeds outputs only);
            // warp (mq, nq) has rows 16 mq .. of both and the value columns 16 nq .. 16 nq + 15
            float acck[2][4], acc[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                acck[j][0] = acck[j][1] = acck[j][2] = acck[j][3] = 0.f;
                acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
            }
            {
                const float* ak = &M.kq[16 * mq + g8][t4];
                const float* aq = &M.kq[CH + 16 * mq + g8][t4];
                const float* br = &M.s[16 * nq + g8][t4];
#pragma unroll 4
                for (int k0 = 0; k0 < LKD; k0 += 8) {
                    const FragA a = frag_a(ak[k0], ak[8 * KLD + k0], ak[k0 + 4], ak[8 * KLD + k0 + 4]);
                    const uint32_t q4[4] = {tf32_round(aq[k0]), tf32_round(aq[8 * KLD + k0]), tf32_round(aq[k0 + 4]),
                                            tf32_round(aq[8 * KLD + k0 + 4])};
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        uint32_t h0, l0, h1, l1;
                        tf32_split(br[8 * j * KLD + k0], h0, l0);
                        tf32_split(br[8 * j * KLD + k0 + 4], h1, l1);
                        mma_tf32(acck[j], a.lo, h0, h1);
                        mma_tf32(acck[j], a.hi, l0, l1);
                        mma_tf32(acck[j], a.hi, h0, h1);
                        mma_tf32(acc[j], q4, l0, l1);
                        mma_tf32(acc[j], q4, h0, h1);
                    }
                }
            }
            __syncthreads();  // gam / dec visible (written above), every warp done with q and with S as an operand
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                // R = b (V - gam K S^T), over V in place; gam Q S^T stays in the registers until P D joins it
                const int i = 16 * mq + g8 + 8 * hh;
                const float bi = M.b[i], gi = M.gam[i];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    float2* rv = (float2*)&M.r[i][16 * nq + 8 * j + 2 * t4];
                    const float2 v = *rv;
                    *rv = make_float2(bi * (v.x - gi * acck[j][2 * hh]), bi * (v.y - gi * acck[j][2 * hh + 1]));
                    acc[j][2 * hh] *= gi;
                    acc[j][2 * hh + 1] *= gi;
                }
            }
            if (more) load_q(tok + CH);   // the q tile is free
            cp_async_commit();
            __syncthreads();
            // ---- G2: D = T R, 64 x 64 over the chunk's tokens (T is lower triangular: rows 16 m2 .. stop at 16 m2 + 15)
            {
                const int m2 = warp >> 2, np = warp & 3;
                float dacc[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++) dacc[j][0] = dacc[j][1] = dacc[j][2] = dacc[j][3] = 0.f;
                const float* ar = &M.t[16 * m2 + g8][t4];
                const float* br = &M.r[t4][16 * np + g8];
                for (int k0 = 0; k0 < 16 * (m2 + 1); k0 += 8) {
                    const FragA a = frag_a(ar[k0], ar[8 * TLD + k0], ar[k0 + 4], ar[8 * TLD + k0 + 4]);
#pragma unroll
                    for (int j = 0; j < 2; j++) mma3(dacc[j], a, br[k0 * RLD + 8 * j], br[(k0 + 4) * RLD + 8 * j]);
                }
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    *(float2*)&M.d[16 * m2 + g8][16 * np + 8 * j + 2 * t4] = make_float2(dacc[j][0], dacc[j][1]);
                    *(float2*)&M.d[16 * m2 + g8 + 8][16 * np + 8 * j + 2 * t4] = make_float2(dacc[j][2], dacc[j][3]);
                }
            }
            __syncthreads();
            if (more) load_tv(tok + CH);  // T, R (the value columns' place) and the gates are free: gam and dec hold what
            cp_async_commit();            // the rest of the chunk needs of them
            // ---- G4: S' = gam_C S + D^T (k_j dec_j), 64 value columns x 128 keys over the chunk's tokens
            {
                const int m4 = warp >> 2, nq = warp & 3;
                float sacc[4][4];
                const float gc = M.gam[CH - 1];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 a = *(const float2*)&M.s[16 * m4 + g8][32 * nq + 8 * j + 2 * t4];
                    const float2 b = *(const float2*)&M.s[16 * m4 + g8 + 8][32 * nq + 8 * j + 2 * t4];
                    sacc[j][0] = gc * a.x; sacc[j][1] = gc * a.y; sacc[j][2] = gc * b.x; sacc[j][3] = gc * b.y;
                }
                const float* ar = &M.d[t4][16 * m4 + g8];
                const float* br = &M.kq[t4][32 * nq + g8];
#pragma unroll 2
                for (int k0 = 0; k0 < CH; k0 += 8) {
                    const float d0 = M.dec[k0 + t4], d1 = M.dec[k0 + t4 + 4];
                    const FragA a = frag_a(ar[k0 * RLD] * d0, ar[k0 * RLD + 8] * d0, ar[(k0 + 4) * RLD] * d1, ar[(k0 + 4) * RLD + 8] * d1);
#pragma unroll
                    for (int j = 0; j < 4; j++) mma3(sacc[j], a, br[k0 * KLD + 8 * j], br[(k0 + 4) * KLD + 8 * j]);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    *(float2*)&M.s[16 * m4 + g8][32 * nq + 8 * j + 2 * t4] = make_float2(sacc[j][0], sacc[j][1]);
                    *(float2*)&M.s[16 * m4 + g8 + 8][32 * nq + 8 * j + 2 * t4] = make_float2(sacc[j][2], sacc[j][3]);
                }
            }
            asm volatile("cp.async.wait_group 2;\n" ::: "memory");  // this chunk's P (the two groups after it may fly)
            __syncthreads();
            if (more) load_k(tok + CH);   // the k tile is free
            cp_async_commit();
            // ---- G3: O = gam Q S^T + P D (operands rounded to TF32 once), straight to the output rows
            {
                const float* ar = &M.pm[16 * mq + g8][t4];
                const float* br = &M.d[t4][16 * nq + g8];
                for (int k0 = 0; k0 < 16 * (mq + 1); k0 += 8) {
                    const uint32_t a4[4] = {tf32_round(ar[k0]), tf32_round(ar[8 * TLD + k0]), tf32_round(ar[k0 + 4]),
                                            tf32_round(ar[8 * TLD + k0 + 4])};
#pragma unroll
                    for (int j = 0; j < 2; j++)
                        mma_tf32(acc[j], a4, tf32_round(br[k0 * RLD + 8 * j]), tf32_round(br[(k0 + 4) * RLD + 8 * j]));
                }
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    float* o = out + (size_t)(tok + 16 * mq + g8 + 8 * hh) * MIX + h * LVD + vs * SC_COLS + 16 * nq + 2 * t4;
#pragma unroll
                    for (int j = 0; j < 2; j++) *(float2*)(o + 8 * j) = make_float2(acc[j][2 * hh], acc[j][2 * hh + 1]);
                }
            }
            __syncthreads();
            if (more) load_p(tok + CH);
            cp_async_commit();
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();
        ld_rows<8>(S, &M.s[lc][0], sub);
    }

    // ================================================================ the token form: tokens l0 .. len - 1
    float* tq = &M.kq[0][0];                       // [SC_TAIL][128]
    float* tk = tq + SC_TAIL * LKD;                // [SC_TAIL][128]
    float* tv = tk + SC_TAIL * LKD;                // [SC_TAIL][64]
    for (int c0 = l0; c0 < len; c0 += SC_TAIL) {
        const int m = min(SC_TAIL, len - c0);
        __syncthreads();  // the previous round (or the chunks) is done with the staging area
        for (int x = tid; x < m * (LKD / 4); x += SC_THREADS) {
            const int r = x / (LKD / 4), dd = (x % (LKD / 4)) * 4;
            const float* row = cv + (size_t)(t0 + c0 + r) * CVW + kh * LKD + dd;
            *(float4*)(tq + r * LKD + dd) = ld4(row);
            *(float4*)(tk + r * LKD + dd) = ld4(row + LK_HEADS * LKD);
        }
        for (int x = tid; x < m * (SC_COLS / 4); x += SC_THREADS) {
            const int r = x / (SC_COLS / 4), dd = (x % (SC_COLS / 4)) * 4;
            *(float4*)(tv + r * SC_COLS + dd) = ld4(cv + (size_t)(t0 + c0 + r) * CVW + 2 * LK_HEADS * LKD + h * LVD + vs * SC_COLS + dd);
        }
        if (tid < 2 * m) {
            const int r = tid >> 1, which = tid & 1;
            (which ? M.tb : M.te)[r] = cv[(size_t)(t0 + c0 + r) * CVW + LQKV + which * LV_HEADS + h];
        }
        __syncthreads();
        for (int r = warp; r < m; r += SC_THREADS / 32) {  // k . q of each token
            const float4 a = ld4(tq + r * LKD + lane * 4), b = ld4(tk + r * LKD + lane * 4);
            const float x = warp_sum(a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w);
            if (lane == 0) M.tkq[r] = x;
        }
        // the inputs of the tokens from the new checkpoint on go to its bank, for a later restart: k once per key head,
        // v by each block for its columns, the gates once per value head
        for (int r = max(0, pl.ck - (p0 + c0)); r < m; r++) {
            float* e = entry(pl.cbuf, p0 + c0 + r);
            if (vs == 0 && h % (LV_HEADS / LK_HEADS) == 0 && tid < LKD) e[kh * LKD + tid] = tk[r * LKD + tid];
            if (tid >= 128 && tid < 128 + SC_COLS) e[LK_HEADS * LKD + h * LVD + vs * SC_COLS + tid - 128] = tv[r * SC_COLS + tid - 128];
            if (vs == 0 && tid == 256) {
                e[LK_HEADS * LKD + LV_HEADS * LVD + h] = M.te[r];
                e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS + h] = M.tb[r];
            }
        }
        __syncthreads();
        for (int r = 0; r < m; r++) {
            if (pl.wck && p0 + c0 + r == pl.ck) st_rows<8>(sbuf(pl.cbuf), S, sub);
            float k[RPT], q[RPT];
            ld_rows<8>(k, tk + r * LKD, sub);
            ld_rows<8>(q, tq + r * LKD, sub);
            const float dk = dot_rows<8>(S, k), dq = dot_rows<8>(S, q);
            const float ex = M.te[r], delta = (tv[r * SC_COLS + lc] - ex * dk) * M.tb[r];
            if (sub == 0) out[(size_t)(t0 + c0 + r) * MIX + h * LVD + col] = ex * dq + delta * M.tkq[r];
#pragma unroll
            for (int j = 0; j < RPT; j++) S[j] = ex * S[j] + k[j] * delta;
        }
    }
    st_rows<8>(sbuf(pl.ebuf), S, sub);
    // ---- the conv ring: the conv inputs of the segment's last CR tokens, this block's share of the channels (after
    // delta_prep, which read the ring, has finished: it is an earlier kernel of the stream)
    const int nb = gridDim.x * gridDim.y, share = (LQKV + nb - 1) / nb;
    const int cb = (h * gridDim.x + vs) * share, cnt = max(0, min(share, LQKV - cb)), mm = min(len, CR);
    for (int i = tid; i < mm * cnt; i += SC_THREADS) {
        const int r = len - mm + i / cnt, c = cb + i % cnt;
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += p[((size_t)s * n + t0 + r) * DELTA_IN + c];
        sm0[SLOT_RING + (size_t)((p0 + r) & (CR - 1)) * LQKV + c] = v;
    }
}

// ------------------------------------------------------------------------------------------------ delta_gate_norm
// grid (n), block 384: warp w normalises value heads 4 w .. 4 w + 3 of the token, a lane four columns of each
constexpr int GN_THREADS = 384;
__global__ void __launch_bounds__(GN_THREADS)
delta_gate_norm_kernel(const float* p, int splits, int n, const float* nw, const float* o, __half* y, int* meta,
                       const int* seg_len, const int* seg_slot, const int* seg_pos0, int segs) {
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float4 w = ld4(nw + lane * 4);
    pdl_wait();
    const size_t stride = (size_t)n * DELTA_IN;
#pragma unroll
    for (int i = 0; i < LV_HEADS / (GN_THREADS / 32); i++) {
        const int h = warp * (LV_HEADS / (GN_THREADS / 32)) + i;
        const size_t at = (size_t)t * MIX + h * LVD + lane * 4;
        const float4 v = ld4(o + at);
        const float* zp = p + (size_t)t * DELTA_IN + LQKV + h * LVD + lane * 4;
        float4 z = ld4(zp);
        for (int s = 1; s < splits; s++) {
            const float4 x = ld4(zp + s * stride);
            z.x += x.x; z.y += x.y; z.z += x.z; z.w += x.w;
        }
        const float r = rsqrtf(warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) / LVD + EPS);
        *(uint2*)(y + at) = make_uint2(pack_half2(w.x * (v.x * r) * silu(z.x), w.y * (v.y * r) * silu(z.y)),
                                       pack_half2(w.z * (v.z * r) * silu(z.z), w.w * (v.w * r) * silu(z.w)));
    }
    if (t == 0) {  // the step is recorded in the slots' metadata (every reader of the old values ran in earlier kernels)
        for (int s = threadIdx.x; s < segs; s += GN_THREADS) {
            const int slot = seg_slot[s], p0 = seg_pos0[s], len = seg_len[s];
            const Plan pl = make_plan(meta, slot, p0, len);
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
    return launch(ctx, delta_prep_kernel, dim3(LQKV / 128, (n + PREP_TOK - 1) / PREP_TOK), dim3(128), 0,
                  (cudaStream_t)stream, p, splits, n, ba, ba_splits, cw, a_log, dt_bias, mem, sst, cv, tok_slot, tok_pos);
}

// The scratch of the chunked form (T, P and the log decays of every chunk and value head of a step of up to 2048
// tokens, 52 MB) belongs to the context and is allocated by the first step that has a segment long enough to run in
// chunks: a prompt-sized step, which is never captured into a graph.
int qb_delta_rule(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* cv, float* mem,
                  long long sst, const int* meta, float* out, const int* seg_start, const int* seg_len,
                  const int* seg_slot, const int* seg_pos0, int segs) {
    if (!ctx || !p || !cv || !mem || !meta || !out || !seg_start || !seg_len || !seg_slot || !seg_pos0 || n <= 0 ||
        segs <= 0 || splits < 1)
        return QB_ERR_ARG;
    constexpr int MAX_TOK = 2048;
    cudaStream_t st = (cudaStream_t)stream;
    const int chunks = chunked_tokens(n) / CH;  // of the longest segment the step can hold
    if (chunks > 0) {
        if (n > MAX_TOK) return QB_ERR_TOO_LARGE;
        if (!ctx->delta_tp) {
            QB_CUDA(cudaMalloc(&ctx->delta_tp, (size_t)(MAX_TOK / CH + 1) * LV_HEADS * TP_FLOATS * sizeof(float)));
        }
        int rc = launch(ctx, delta_chunk_prep_kernel, dim3(chunks, LK_HEADS, segs), dim3(CP_THREADS), CP_SMEM, st, cv,
                        ctx->delta_tp, seg_start, seg_len);
        if (rc) return rc;
    }
    return launch(ctx, delta_scan_kernel, dim3(LVD / SC_COLS, LV_HEADS, segs), dim3(SC_THREADS), sizeof(ScanSmem), st, p,
                  splits, n, cv, (const float*)ctx->delta_tp, mem, sst, meta, out, seg_start, seg_len, seg_slot, seg_pos0);
}

int qb_delta_norm(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* nw, const float* out,
                  void* y, int* meta, const int* seg_len, const int* seg_slot, const int* seg_pos0, int segs) {
    if (!ctx || !p || !nw || !out || !y || !meta || !seg_len || !seg_slot || !seg_pos0 || n <= 0 || segs <= 0 ||
        splits < 1)
        return QB_ERR_ARG;
    return launch(ctx, delta_gate_norm_kernel, dim3(n), dim3(GN_THREADS), 0, (cudaStream_t)stream, p, splits, n, nw, out,
                  (__half*)y, meta, seg_len, seg_slot, seg_pos0, segs);
}

}  // extern "C"
