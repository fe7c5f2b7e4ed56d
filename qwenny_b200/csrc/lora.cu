// A LoRA adapter applied unmerged (kernels/lora.cuh, src/cuda/qwen/lora.rs of the reference): y = W x + s B (A x) per
// adapted module, s = alpha / r for the tokens of slots that use the adapter and nothing added for the others. The
// products that read one input share one stacked A, whose product xa = A x is a 16-bit matrix product of the step
// (qb_gemm_f16_plain: split-K partial sums [split][n][M], M = adapted modules * rank). The kernels here add s B xa to
// a plain product's first partial sums (lora_add), or apply SwiGLU to a plain [gate; up] product, in the SwiGLU
// epilogue's row order, with the delta added first (lora_silu).
//
// Tiling: a block covers 64 outputs x 32 tokens with 256 threads, thread = (output, token lane 0..3); a thread keeps
// its output's R values of B in registers and walks the tile's tokens 4 apart, so decode-sized steps spread over
// rows / 64 blocks and every B row is fetched once per 32 tokens. The tokens' xa are summed over the splits once per
// block into shared memory (tokens without the adapter are skipped there and cost a compare later). Per (output,
// token) the arithmetic is fixed by the reference's kernels, whose bits the results must have: splits added in
// ascending order, the rank's products as ONE chain of fused multiply-adds in rank order, then y += s * delta.
#include "common.cuh"
#include "launch.h"

namespace qb {
namespace {

constexpr int TILE_OUT = 64;     // outputs of a block
constexpr int TILE_TOK = 32;     // tokens of a block
constexpr int TOK_LANES = 4;     // threads that share an output
constexpr int LMAXM = 256;       // columns of xa at most (LORA_MAXM of the reference)

struct LoraArgs {
    const float* xa;
    int split, M;
    const __half* B;
    int rows;
    const int* tab;       // [0..3): ends of the modules' rows (ascending; unused INT_MAX); [4..8): their first column of xa
    const int* tok_slot;
    const float* slot_scale;
    int n;
    float* y;
    int ldy;
    __half* mid;
};

// R values of B's row `o` as floats
template <int R>
struct BRow {
    float b[R];
    __device__ __forceinline__ void load(const __half* B, int o) {
        const uint4* p = reinterpret_cast<const uint4*>(B + (size_t)o * R);
#pragma unroll
        for (int i = 0; i < R / 8; i++) {
            const uint4 u = p[i];
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __half22float2(h[q]);
                b[8 * i + 2 * q] = f.x;
                b[8 * i + 2 * q + 1] = f.y;
            }
        }
    }
    __device__ __forceinline__ float dot(const float* x) const {
        float d = 0.f;
#pragma unroll
        for (int q = 0; q < R; q++) d = fmaf(b[q], x[q], d);
        return d;
    }
};

// PAIRS = false: an output is a row of y, the delta is added in place. PAIRS = true (the SwiGLU form): an output j is
// an element of mid, made from the gate row 16 (j / 8) + j % 8 and the up row 8 below it of the plain product y.
template <int R, bool PAIRS>
__global__ void __launch_bounds__(TILE_OUT * TOK_LANES) lora_tile_kernel(const LoraArgs a) {
    __shared__ float xs[TILE_TOK][LMAXM];
    __shared__ float scale[TILE_TOK];
    pdl_wait();
    const int tid = threadIdx.x, tok0 = blockIdx.y * TILE_TOK, cnt = min(TILE_TOK, a.n - tok0);
    if (tid < TILE_TOK) scale[tid] = tid < cnt ? a.slot_scale[a.tok_slot[tok0 + tid]] : 0.f;
    __syncthreads();
    bool adapted = false;
    for (int i = 0; i < cnt; i++) adapted |= scale[i] != 0.f;
    if (!adapted && !PAIRS) return;  // nothing to add in this tile (the SwiGLU form still has to write mid)
    for (int i = tid; i < cnt * a.M; i += TILE_OUT * TOK_LANES) {
        const int tl = i / a.M, c = i - tl * a.M;
        float v = 0.f;
        if (scale[tl] != 0.f)
            for (int sp = 0; sp < a.split; sp++) v += a.xa[((size_t)sp * a.n + tok0 + tl) * a.M + c];
        xs[tl][c] = v;
    }
    __syncthreads();
    const int o = blockIdx.x * TILE_OUT + (tid % TILE_OUT), lane_tok = tid / TILE_OUT;
    if (!PAIRS) {
        if (o >= a.rows) return;
        // which stacked module the row belongs to, and where that module's columns of xa start
        int module = 0;
#pragma unroll
        for (int i = 0; i < 3; i++) module += o >= a.tab[i];
        const int off = a.tab[4 + module];
        if (off < 0) return;
        BRow<R> row;
        row.load(a.B, o);
        for (int tl = lane_tok; tl < cnt; tl += TOK_LANES) {
            const float s = scale[tl];
            if (s != 0.f) a.y[(size_t)(tok0 + tl) * a.ldy + o] += s * row.dot(&xs[tl][off]);
        }
        return;
    }
    if (o >= a.rows / 2) return;
    const int gate_row = 16 * (o / 8) + o % 8, up_row = gate_row + 8, off_gate = a.tab[4], off_up = a.tab[5];
    BRow<R> bg, bu;
    if (adapted && off_gate >= 0) bg.load(a.B, gate_row);
    if (adapted && off_up >= 0) bu.load(a.B, up_row);
    for (int tl = lane_tok; tl < cnt; tl += TOK_LANES) {
        const size_t at = (size_t)(tok0 + tl) * a.ldy;
        float gate = a.y[at + gate_row], up = a.y[at + up_row];
        const float s = scale[tl];
        if (s != 0.f) {
            if (off_gate >= 0) gate += s * bg.dot(&xs[tl][off_gate]);
            if (off_up >= 0) up += s * bu.dot(&xs[tl][off_up]);
        }
        a.mid[(size_t)(tok0 + tl) * (a.rows / 2) + o] = __float2half_rn(silu(gate) * up);  // every token, as the epilogue rounds it
    }
}

template <int R>
int run(qb_ctx* ctx, cudaStream_t st, const LoraArgs& a, bool pairs) {
    const int outs = pairs ? a.rows / 2 : a.rows;
    const dim3 grid((outs + TILE_OUT - 1) / TILE_OUT, (a.n + TILE_TOK - 1) / TILE_TOK);
    return pairs ? launch(ctx, lora_tile_kernel<R, true>, grid, dim3(TILE_OUT * TOK_LANES), 0, st, a)
                 : launch(ctx, lora_tile_kernel<R, false>, grid, dim3(TILE_OUT * TOK_LANES), 0, st, a);
}

int dispatch(qb_ctx* ctx, void* stream, LoraArgs a, int rank, bool with_silu) {
    if (!ctx || !a.xa || !a.B || !a.tab || !a.tok_slot || !a.slot_scale || !a.y || a.n < 0 || a.rows <= 0 || a.M <= 0 ||
        a.M > LMAXM || a.split < 1 || a.ldy < a.rows || (with_silu && (!a.mid || a.rows % 16)))
        return QB_ERR_ARG;
    if (a.n == 0) return QB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    switch (rank) {
        case 8: return run<8>(ctx, st, a, with_silu);
        case 16: return run<16>(ctx, st, a, with_silu);
        case 32: return run<32>(ctx, st, a, with_silu);
        case 64: return run<64>(ctx, st, a, with_silu);
    }
    return QB_ERR_UNSUPPORTED;  // the reference serves ranks 8, 16, 32, 64 (RANKS, src/cuda/qwen/lora.rs:21)
}

}  // namespace
}  // namespace qb

extern "C" int qb_lora_add(qb_ctx* ctx, void* stream, const float* xa, int split, int M, const void* B, int rows,
                           const int* tab, const int* tok_slot, const float* slot_scale, int n, float* y, int ldy,
                           int rank) {
    qb::LoraArgs a = {xa, split, M, (const __half*)B, rows, tab, tok_slot, slot_scale, n, y, ldy, nullptr};
    return qb::dispatch(ctx, stream, a, rank, false);
}

extern "C" int qb_lora_silu(qb_ctx* ctx, void* stream, const float* xa, int split, int M, const void* B, int rows,
                            const int* tab, const int* tok_slot, const float* slot_scale, int n, const float* y, int ldy,
                            void* mid, int rank) {
    qb::LoraArgs a = {xa, split, M, (const __half*)B, rows, tab, tok_slot, slot_scale, n, const_cast<float*>(y), ldy,
                      (__half*)mid};
    return qb::dispatch(ctx, stream, a, rank, true);
}
