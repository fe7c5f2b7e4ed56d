// Dense products of checkpoints that are not int4: 16-bit and int8 weights in the reference's tile form with the three
// epilogues (gemm_{f16,i8}_t*_{plain,silu,argmax}, kernels/gemm.cuh:118-304 of the reference; Gemm::run_split,
// src/cuda/core.rs:532-560). W: tiles of 16 rows in mma A-fragment order (f16: one k16 step per 16-byte load of a lane,
// qb_pack_f16; int8: codes q + 128, two k16 steps per load, one f32 scale per row and 128 columns stored
// [tile][group][16 rows], qb_pack_i8).
//
// A block is one (tile, k split, block of 8 NTT tokens). Its 4 warps take the 128-column groups of the split in turn
// (a group's weights are 8 or 4 loads per lane, the next group's in flight while this one is multiplied; int8 groups
// go through the tensor core as exact f16 integers and are scaled in f32 per group, as the reference does), add up in
// shared memory in warp order, and warp 0 runs the epilogue.
#include "common.cuh"
#include "launch.h"

namespace qb {
namespace {

// two bytes (q + 128) -> half2 (q, q), exactly: 0x64XX is 1024 + XX
__device__ __forceinline__ uint32_t bytes_half2(uint32_t w, uint32_t sel) {
    uint32_t h = __byte_perm(w, 0x64646464u, sel);
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&h), __half2half2(__float2half(1152.f)));
    return *reinterpret_cast<uint32_t*>(&r);
}

template <int WB, int NTT, int EPI>
__global__ void __launch_bounds__(128) gemm_dec_kernel(const uint4* __restrict__ W, const float* __restrict__ S,
                                                       const __half* __restrict__ X, const int* __restrict__ xrows,
                                                       int K, int ntiles, int n, int kper, void* __restrict__ Yv, int ldy,
                                                       unsigned long long* __restrict__ keys) {
    constexpr int LPG = WB == 16 ? 8 : 4;  // 16-byte loads per lane and 128-column group
    __shared__ float4 red[3][NTT][32];
    pdl_launch_dependents();
    const int tile = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3, tok0 = blockIdx.z * (8 * NTT);
    const int k0 = split * kper, k1 = min(K, k0 + kper), groups = (k1 - k0) / 128;
    const uint4* wp = W + ((size_t)tile * (K / 128) + k0 / 128) * LPG * 32 + lane;
    const float* sp = S ? S + ((size_t)tile * (K / 128) + k0 / 128) * 16 : nullptr;
    uint4 wc[LPG], wn[LPG];
    float sc[2] = {1.f, 1.f}, sn[2] = {1.f, 1.f};
    auto fetch = [&](int gi, uint4* w, float* s) {
        if (gi >= groups) return;
#pragma unroll
        for (int v = 0; v < LPG; v++) w[v] = __ldg(wp + (size_t)(gi * LPG + v) * 32);
        if (WB == 8) { s[0] = __ldg(sp + gi * 16 + g); s[1] = __ldg(sp + gi * 16 + g + 8); }
    };
    fetch(warp, wc, sc);  // the weights do not depend on the previous kernel
    pdl_wait();
    float acc[NTT][4];
#pragma unroll
    for (int j = 0; j < NTT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const __half* xr[NTT];
#pragma unroll
    for (int j = 0; j < NTT; j++) {
        const int tok = tok0 + 8 * j + g;
        xr[j] = tok < n ? X + (size_t)(xrows ? xrows[tok] : tok) * K + k0 + 2 * t : nullptr;
    }
    for (int gi = warp; gi < groups; gi += 4) {
        fetch(gi + 4, wn, sn);
        float tmp[NTT][4];
#pragma unroll
        for (int j = 0; j < NTT; j++) tmp[j][0] = tmp[j][1] = tmp[j][2] = tmp[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            uint32_t a[4];
            if (WB == 16) {
                a[0] = wc[ks].x; a[1] = wc[ks].y; a[2] = wc[ks].z; a[3] = wc[ks].w;
            } else {
                const uint4 u = wc[ks >> 1];
                const uint32_t lo = (ks & 1) ? u.z : u.x, hi = (ks & 1) ? u.w : u.y;
                a[0] = bytes_half2(lo, 0x4140); a[1] = bytes_half2(lo, 0x4342);
                a[2] = bytes_half2(hi, 0x4140); a[3] = bytes_half2(hi, 0x4342);
            }
#pragma unroll
            for (int j = 0; j < NTT; j++) {
                uint32_t b0 = 0, b1 = 0;
                if (xr[j]) {
                    b0 = *reinterpret_cast<const uint32_t*>(xr[j] + gi * 128 + ks * 16);
                    b1 = *reinterpret_cast<const uint32_t*>(xr[j] + gi * 128 + ks * 16 + 8);
                }
                mma16816(WB == 8 ? tmp[j] : acc[j], a, b0, b1);
            }
        }
        if (WB == 8) {
#pragma unroll
            for (int j = 0; j < NTT; j++) {
                acc[j][0] += sc[0] * tmp[j][0]; acc[j][1] += sc[0] * tmp[j][1];
                acc[j][2] += sc[1] * tmp[j][2]; acc[j][3] += sc[1] * tmp[j][3];
            }
        }
#pragma unroll
        for (int v = 0; v < LPG; v++) wc[v] = wn[v];
        sc[0] = sn[0]; sc[1] = sn[1];
    }
    if (warp > 0) {
#pragma unroll
        for (int j = 0; j < NTT; j++) red[warp - 1][j][lane] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int j = 0; j < NTT; j++)
#pragma unroll
        for (int w = 0; w < 3; w++) {
            const float4 v = red[w][j][lane];
            acc[j][0] += v.x; acc[j][1] += v.y; acc[j][2] += v.z; acc[j][3] += v.w;
        }
    // acc[j]: c0, c1 = row g, tokens 2t and 2t + 1 of token tile j; c2, c3 = row g + 8
    if (EPI == QB_EPI_SILU) {
        // tile p holds rows 8p .. 8p + 7 of gate, then of up: Y f16 [n][ldy], Y[tok][8p + g] = silu(gate) * up
        __half* y = reinterpret_cast<__half*>(Yv);
#pragma unroll
        for (int j = 0; j < NTT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int tok = tok0 + 8 * j + 2 * t + e;
                if (tok < n) y[(size_t)tok * ldy + tile * 8 + g] = __float2half_rn(silu(acc[j][e]) * acc[j][2 + e]);
            }
        return;
    }
    float* y = reinterpret_cast<float*>(Yv) + (EPI == QB_EPI_PLAIN ? (size_t)split * n * ldy : 0);
#pragma unroll
    for (int j = 0; j < NTT; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int tok = tok0 + 8 * j + 2 * t + (i & 1), r = tile * 16 + g + (i >> 1) * 8;
            if (tok < n) y[(size_t)tok * ldy + r] = acc[j][i];
        }
    if (EPI == QB_EPI_ARGMAX) {
#pragma unroll
        for (int j = 0; j < NTT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int r = tile * 16 + g;
                unsigned long long k = max(argmax_key(acc[j][e], r), argmax_key(acc[j][2 + e], r + 8));
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) k = max(k, __shfl_xor_sync(0xffffffffu, k, o));
                const int tok = tok0 + 8 * j + 2 * t + e;
                if (g == 0 && tok < n) atomicMax(keys + tok, k);
            }
    }
}

template <int WB, int NTT>
int go(qb_ctx* ctx, cudaStream_t st, dim3 grid, int epi, const void* W, const float* S, const void* X, const int* xrows,
       int K, int ntiles, int n, int kper, void* Y, int ldy, unsigned long long* keys) {
    const uint4* w = (const uint4*)W;
    const __half* x = (const __half*)X;
    switch (epi) {
        case QB_EPI_PLAIN:
            return launch(ctx, gemm_dec_kernel<WB, NTT, QB_EPI_PLAIN>, grid, dim3(128), 0, st, w, S, x, xrows, K, ntiles, n, kper, Y, ldy, keys);
        case QB_EPI_SILU:
            return launch(ctx, gemm_dec_kernel<WB, NTT, QB_EPI_SILU>, grid, dim3(128), 0, st, w, S, x, xrows, K, ntiles, n, kper, Y, ldy, keys);
        case QB_EPI_ARGMAX:
            return launch(ctx, gemm_dec_kernel<WB, NTT, QB_EPI_ARGMAX>, grid, dim3(128), 0, st, w, S, x, xrows, K, ntiles, n, kper, Y, ldy, keys);
    }
    return QB_ERR_ARG;
}

}  // namespace
}  // namespace qb

// wbits 16 (S null) or 8. Plain: Y f32 [K / kper splits][n][ldy] partial sums for the consumer to add; SwiGLU (rows in
// row_order(silu)): Y f16 [n][ldy], ldy >= ntiles * 8; argmax: Y f32 [n][ldy] and keys[t] maximised with
// (ordered(logit) << 32 | ~row). The last two need the whole sum: kper == K.
extern "C" int qb_gemm_dec(qb_ctx* ctx, void* stream, const void* W, const float* S, int wbits, const void* X,
                           const int* xrows, int K, int ntiles, int n, int kper, int epi, void* Y, int ldy,
                           unsigned long long* keys) {
    if (!ctx || !W || !X || !Y || (wbits != 16 && wbits != 8) || (wbits == 8 && !S) || K <= 0 || K % 128 || ntiles <= 0 ||
        n <= 0 || n > 65535 * 32 || kper <= 0 || kper % 128 || epi < QB_EPI_PLAIN || epi > QB_EPI_ARGMAX)
        return QB_ERR_ARG;
    if (epi != QB_EPI_PLAIN && kper < K) return QB_ERR_ARG;
    if (epi == QB_EPI_ARGMAX && !keys) return QB_ERR_ARG;
    if (ldy < (epi == QB_EPI_SILU ? ntiles * 8 : ntiles * 16)) return QB_ERR_ARG;
    const int split = (K + kper - 1) / kper;
    cudaStream_t st = (cudaStream_t)stream;
#define QB_DEC(NTT)                                                                                                   \
    {                                                                                                                 \
        const dim3 grid(ntiles, split, (n + 8 * NTT - 1) / (8 * NTT));                                                \
        return wbits == 16 ? qb::go<16, NTT>(ctx, st, grid, epi, W, S, X, xrows, K, ntiles, n, kper, Y, ldy, keys)    \
                           : qb::go<8, NTT>(ctx, st, grid, epi, W, S, X, xrows, K, ntiles, n, kper, Y, ldy, keys);    \
    }
    if (n <= 8) QB_DEC(1)
    if (n <= 16) QB_DEC(2)
    QB_DEC(4)
#undef QB_DEC
}
