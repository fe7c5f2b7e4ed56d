// Dense f16 skinny product for the few matrices a checkpoint keeps in 16 bits (the DeltaNet in_proj_b / in_proj_a
// pair, 96 x 5120): Y[split][t][r] = W[r] . X[t] over the split's k range. Replaces gemm_dec<16, NTT, EPI_PLAIN>
// (kernels/gemm.cuh:222-304 of the reference). W arrives in the reference's packed form: tiles of 16 rows, per k16
// step the 32 lanes' mma A fragments (8 halves each), so a warp's 128-bit loads are the fragments themselves.
// A block is one (tile, k split, block of 8 NTT tokens); its 4 warps take alternate k16 steps and add up in shared memory in warp order.
#include "common.cuh"
#include "launch.h"

namespace qb {

template <int NTT>
__global__ void __launch_bounds__(128) gemm_f16_plain_kernel(const uint4* __restrict__ W, const __half* __restrict__ X,
                                                             const int* __restrict__ xrows, int K, int ntiles, int n,
                                                             int kper, float* __restrict__ Y, int ldy) {
    __shared__ float4 red[3][NTT][32];
    pdl_launch_dependents();
    const int tile = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3, tok0 = blockIdx.z * (8 * NTT);
    const int k0 = split * kper, k1 = min(K, k0 + kper);
    const uint4* wp = W + ((size_t)tile * (K / 16) + k0 / 16) * 32 + lane;
    const int steps = (k1 - k0) / 16;
    // the weights do not depend on the previous kernel: all of this warp's fragments (up to MAXF k16 steps) are in
    // flight before it waits for that kernel; longer ranges fetch the rest as they go
    constexpr int MAXF = 16;
    uint4 wf[MAXF];
#pragma unroll
    for (int i = 0; i < MAXF; i++) {
        int sidx = warp + 4 * i;
        wf[i] = sidx < steps ? __ldg(wp + (size_t)sidx * 32) : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    float acc[NTT][4];
#pragma unroll
    for (int j = 0; j < NTT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const __half* xr[NTT];
#pragma unroll
    for (int j = 0; j < NTT; j++) {
        int tok = tok0 + 8 * j + g;
        xr[j] = tok < n ? X + (size_t)(xrows ? xrows[tok] : tok) * K + k0 + 2 * t : nullptr;
    }
    auto step = [&](int s, const uint4& w) {
        uint32_t a[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < NTT; j++) {
            uint32_t b0 = 0, b1 = 0;
            if (xr[j]) {
                b0 = *(const uint32_t*)(xr[j] + s * 16);
                b1 = *(const uint32_t*)(xr[j] + s * 16 + 8);
            }
            mma16816(acc[j], a, b0, b1);
        }
    };
#pragma unroll
    for (int i = 0; i < MAXF; i++)
        if (warp + 4 * i < steps) step(warp + 4 * i, wf[i]);
    for (int s = warp + 4 * MAXF; s < steps; s += 4) step(s, __ldg(wp + (size_t)s * 32));
    if (warp > 0) {
#pragma unroll
        for (int j = 0; j < NTT; j++) red[warp - 1][j][lane] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    }
    __syncthreads();
    if (warp == 0) {
        float* y = Y + (size_t)split * n * ldy;
#pragma unroll
        for (int j = 0; j < NTT; j++) {
#pragma unroll
            for (int w = 0; w < 3; w++) {
                float4 v = red[w][j][lane];
                acc[j][0] += v.x; acc[j][1] += v.y; acc[j][2] += v.z; acc[j][3] += v.w;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int tok = tok0 + 8 * j + 2 * t + (i & 1), r = tile * 16 + g + (i >> 1) * 8;
                if (tok < n) y[(size_t)tok * ldy + r] = acc[j][i];
            }
        }
    }
}

}  // namespace qb

using namespace qb;

extern "C" int qb_gemm_f16_plain(qb_ctx* ctx, void* stream, const void* W, const void* X, const int* xrows, int K,
                                 int ntiles, int n, int kper, float* Y, int ldy) {
    if (!ctx || !W || !X || !Y || K <= 0 || K % 16 || ntiles <= 0 || n <= 0 || n > 65535 * 32 || kper <= 0 || kper % 16 ||
        ldy < ntiles * 16)
        return QB_ERR_ARG;
    int split = (K + kper - 1) / kper;
    dim3 grid(ntiles, split, n <= 32 ? 1 : (n + 31) / 32);
    cudaStream_t st = (cudaStream_t)stream;
    const uint4* w = (const uint4*)W;
    const __half* x = (const __half*)X;
    if (n <= 8) return launch(ctx, gemm_f16_plain_kernel<1>, grid, dim3(128), 0, st, w, x, xrows, K, ntiles, n, kper, Y, ldy);
    if (n <= 16) return launch(ctx, gemm_f16_plain_kernel<2>, grid, dim3(128), 0, st, w, x, xrows, K, ntiles, n, kper, Y, ldy);
    return launch(ctx, gemm_f16_plain_kernel<4>, grid, dim3(128), 0, st, w, x, xrows, K, ntiles, n, kper, Y, ldy);
}
