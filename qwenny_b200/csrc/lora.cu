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

// the block's tokens: their scales, and the sum of xa's partial sums for those that use the adapter
__device__ __forceinline__ void stage_xa(const LoraArgs& a, int t0, float (*xs)[LMAXM], float* sc) {
    if (threadIdx.x < LTT) {
        const int t = t0 + threadIdx.x;
        sc[threadIdx.x] = t < a.n ? a.slot_scale[a.tok_slot[t]] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < LTT * a.M; i += blockDim.x) {
        const int tl = i / a.M, c = i - tl * a.M, t = t0 + tl;
        float v = 0.f;
        if (sc[tl] != 0.f)
            for (int s = 0; s < a.split; s++) v += a.xa[((size_t)s * a.n + t) * a.M + c];
        xs[tl][c] = v;
    }
    __syncthreads();
}

template <int R>
__device__ __forceinline__ void load_row(const __half* B, int o, float (&b)[R]) {
    const uint4* p = reinterpret_cast<const uint4*>(B + (size_t)o * R);
#pragma unroll
    for (int i = 0; i < R / 8; i++) {
        const uint4 u = p[i];
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            b[8 * i + 2 * j] = f.x;
            b[8 * i + 2 * j + 1] = f.y;
        }
    }
}

template <int R>
__device__ __forceinline__ float dot(const float (&b)[R], const float* x) {
    float d = 0.f;
#pragma unroll
    for (int j = 0; j < R; j++) d = fmaf(b[j], x[j], d);
    return d;
}

// y[t][o] += s_t * B[o] . xa[t][off(o) ..]; grid (rows / 256, n / 8)
template <int R>
__global__ void __launch_bounds__(256) lora_add_kernel(const LoraArgs a) {
    __shared__ float xs[LTT][LMAXM];
    __shared__ float sc[LTT];
    pdl_wait();
    const int t0 = blockIdx.y * LTT;
    stage_xa(a, t0, xs, sc);
    bool any = false;
#pragma unroll
    for (int i = 0; i < LTT; i++) any |= sc[i] != 0.f;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (!any || o >= a.rows) return;
    const int mod = (o >= a.tab[0]) + (o >= a.tab[1]) + (o >= a.tab[2]);
    const int off = a.tab[4 + mod];
    if (off < 0) return;
    float b[R];
    load_row<R>(a.B, o, b);
#pragma unroll
    for (int tl = 0; tl < LTT; tl++)
        if (sc[tl] != 0.f) a.y[(size_t)(t0 + tl) * a.ldy + o] += sc[tl] * dot<R>(b, &xs[tl][off]);
}

// mid[t][8p + g] = silu(gate + dg) * (up + du) of the plain [gate; up] product y in the SwiGLU row order (16-row tile p:
// gate rows 8p .. 8p + 7, then their up rows); every token, with or without the adapter. Grid (rows / 2 / 256, n / 8)
template <int R>
__global__ void __launch_bounds__(256) lora_silu_kernel(const LoraArgs a) {
    __shared__ float xs[LTT][LMAXM];
    __shared__ float sc[LTT];
    pdl_wait();
    const int t0 = blockIdx.y * LTT;
    stage_xa(a, t0, xs, sc);
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= a.rows / 2) return;
    const int og = 16 * (j / 8) + j % 8, ou = og + 8, offg = a.tab[4], offu = a.tab[5];
    float bg[R], bu[R];
    if (offg >= 0) load_row<R>(a.B, og, bg);
    if (offu >= 0) load_row<R>(a.B, ou, bu);
#pragma unroll
    for (int tl = 0; tl < LTT; tl++) {
        const int t = t0 + tl;
        if (t >= a.n) break;
        float g = a.y[(size_t)t * a.ldy + og], u = a.y[(size_t)t * a.ldy + ou];
        if (sc[tl] != 0.f) {
            if (offg >= 0) g += sc[tl] * dot<R>(bg, &xs[tl][offg]);
            if (offu >= 0) u += sc[tl] * dot<R>(bu, &xs[tl][offu]);
        }
        a.mid[(size_t)t * (a.rows / 2) + j] = __float2half_rn(silu(g) * u);
    }
}

template <int R>
int run(qb_ctx* ctx, cudaStream_t st, const LoraArgs& a, bool with_silu) {
    const int per = with_silu ? 512 : 256;
    const dim3 grid((a.rows + per - 1) / per, (a.n + LTT - 1) / LTT);
    return with_silu ? launch(ctx, lora_silu_kernel<R>, grid, dim3(256), 0, st, a)
                     : launch(ctx, lora_add_kernel<R>, grid, dim3(256), 0, st, a);
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
