// A LoRA adapter applied unmerged (kernels/lora.cuh, src/cuda/qwen/lora.rs of the reference): y = W x + s B (A x) per
// adapted module, s = alpha / r for the tokens of slots that use the adapter and nothing added for the others. The
// products that read one input share one stacked A, whose product xa = A x is a 16-bit matrix product of the step
// (qb_gemm_f16_plain: split-K partial sums [split][n][M], M = adapted modules * rank). The kernels here add s B xa to
// a plain product's first partial sums (lora_add), or apply SwiGLU to a plain [gate; up] product, in the SwiGLU
// epilogue's row order, with the delta added first (lora_silu).
//
// One thread owns one output row: its R halves of B sit in registers (128-bit loads, a warp reads 32 consecutive rows),
// the tokens' xa are summed over the splits once per block into shared memory, and tokens without the adapter cost a
// compare. The sums run in the reference's order (splits ascending; the rank's products as one fused multiply-add
// chain), so the results have the bits of its kernels.
#include "common.cuh"
#include "launch.h"

namespace qb {
namespace {

constexpr int LTT = 8;      // tokens per block (LORA_TT)
constexpr int LMAXM = 256;  // columns of xa at most (LORA_MAXM)

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

// One kernel for both forms. A thread owns one output of the block's tile: row o of y (the delta is added in place), or
// SwiGLU output j of mid, whose gate row og = 16 (j / 8) + j % 8 and up row og + 8 sit in the same 16-row tile of y.
// Grid (outputs / 256, n / 8).
template <int R, bool SWIGLU>
__global__ void __launch_bounds__(256) lora_kernel(const LoraArgs a) {
    __shared__ float xs[LTT][LMAXM];  // xa of the block's tokens, summed over the splits in split order
    __shared__ float sc[LTT];         // their slots' scales (0: the token does not use the adapter)
    pdl_wait();
    const int t0 = blockIdx.y * LTT, tid = threadIdx.x;
    if (tid < LTT) sc[tid] = t0 + tid < a.n ? a.slot_scale[a.tok_slot[t0 + tid]] : 0.f;
    __syncthreads();
    for (int i = tid; i < LTT * a.M; i += 256) {
        const int tl = i / a.M, c = i - tl * a.M;
        float v = 0.f;
        if (sc[tl] != 0.f)
            for (int s = 0; s < a.split; s++) v += a.xa[((size_t)s * a.n + t0 + tl) * a.M + c];
        xs[tl][c] = v;
    }
    __syncthreads();

    // a row of B as R floats (128-bit loads), and its product with a token's xa as ONE chain of fused multiply-adds in
    // rank order: the order the reference's kernels sum in
    auto row_of = [&](int o, float (&b)[R]) {
        const uint4* p = reinterpret_cast<const uint4*>(a.B + (size_t)o * R);
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
    };
    auto delta = [&](const float (&b)[R], int tl, int off) {
        const float* x = &xs[tl][off];
        float d = 0.f;
#pragma unroll
        for (int q = 0; q < R; q++) d = fmaf(b[q], x[q], d);
        return d;
    };

    const int out = blockIdx.x * 256 + tid;
    if (!SWIGLU) {
        bool any = false;
#pragma unroll
        for (int tl = 0; tl < LTT; tl++) any |= sc[tl] != 0.f;
        if (!any || out >= a.rows) return;
        // the stacked module of this row and its columns of xa
        const int off = a.tab[4 + (out >= a.tab[0]) + (out >= a.tab[1]) + (out >= a.tab[2])];
        if (off < 0) return;
        float b[R];
        row_of(out, b);
#pragma unroll
        for (int tl = 0; tl < LTT; tl++)
            if (sc[tl] != 0.f) a.y[(size_t)(t0 + tl) * a.ldy + out] += sc[tl] * delta(b, tl, off);
        return;
    }
    if (out >= a.rows / 2) return;
    const int og = 16 * (out / 8) + out % 8, ou = og + 8, offg = a.tab[4], offu = a.tab[5];
    float bg[R], bu[R];
    if (offg >= 0) row_of(og, bg);
    if (offu >= 0) row_of(ou, bu);
#pragma unroll
    for (int tl = 0; tl < LTT; tl++) {
        const int t = t0 + tl;
        if (t >= a.n) break;
        float g = a.y[(size_t)t * a.ldy + og], u = a.y[(size_t)t * a.ldy + ou];
        if (sc[tl] != 0.f) {
            if (offg >= 0) g += sc[tl] * delta(bg, tl, offg);
            if (offu >= 0) u += sc[tl] * delta(bu, tl, offu);
        }
        a.mid[(size_t)t * (a.rows / 2) + out] = __float2half_rn(silu(g) * u);  // every token, as the epilogue rounds it
    }
}

template <int R>
int run(qb_ctx* ctx, cudaStream_t st, const LoraArgs& a, bool with_silu) {
    const int per = with_silu ? 512 : 256;
    const dim3 grid((a.rows + per - 1) / per, (a.n + LTT - 1) / LTT);
    return with_silu ? launch(ctx, lora_kernel<R, true>, grid, dim3(256), 0, st, a)
                     : launch(ctx, lora_kernel<R, false>, grid, dim3(256), 0, st, a);
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
