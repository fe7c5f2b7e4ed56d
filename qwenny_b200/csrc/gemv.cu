// Host side of the W4A16 skinny product: picks a tile shape and split for the shape, launches the persistent grid.
#include "ctx.h"
#include <array>
#include <map>
#include "measure.h"
#include "w4a16_gemv.cuh"

namespace qb {

struct GemvPlan {
    int cg, kg, nstages, ctas;
    int cluster_s;  // > 0: clustered split K with this many ranks per column block
};

static int smem_of(int cg, int kg, int m, int nstages, int zp = 0) {  // GemvCfg<cg, kg, .>::smem
    int nw = cg * kg, tk = kg * 128, tn = cg * 64;
    int stage = (nw * 4096 + (1 + zp) * kg * tn * 2 + m * (tk + 8) * 2 + 127) / 128 * 128;
    return 128 + ((tk + 8) * 2 + 127) / 128 * 128 + nstages * stage;
}

// Blocks of the persistent grid and the most of them that can share one column block (the scratch stride).
static void grid_of(const qb_ctx* ctx, const GemvPlan& p, int n, int k, int* grid, int* maxc) {
    long long total = (long long)(n / (p.cg * 64)) * (k / (p.kg * 128));
    long long g = (long long)ctx->sms * p.ctas;
    if (g > total) g = total;
    int kst = k / (p.kg * 128);
    long long per = total / g;  // the shortest range
    *grid = (int)g;
    *maxc = (int)((kst + per - 1) / per) + 1;
}
// the kernel divides its (column block, k stage) list among the blocks in 32-bit arithmetic
static bool schedule_fits(const qb_ctx* ctx, const GemvPlan& p, int n, int k) {
    const long long total = (long long)(n / (p.cg * 64)) * (k / (p.kg * 128));
    return (total + 1) * ((long long)ctx->sms * p.ctas + 1) < (1ll << 31);
}

template <int CG, int KG, int NT, int EPI, int ZP = 0>
static int launch_cfg(qb_ctx* ctx, cudaStream_t st, GemvArgs a, const GemvPlan& p) {
    using C = GemvCfg<CG, KG, NT>;
    auto kern = w4a16_gemv_kernel<CG, KG, NT, EPI, ZP>;
    int smem = C::smem(p.nstages, a.m, a.zp);
    if (!schedule_fits(ctx, p, a.N, a.K)) return QB_ERR_TOO_LARGE;
    if (int rc = prepare_kernel(ctx->device, (const void*)kern, smem)) return rc;
    cudaLaunchConfig_t lc = {};
    cudaLaunchAttribute at[2];
    int nat = 0;
    // Clusters are placed inside one GPC each, so not every rank count packs the GPU in one wave: ask the driver how
    // many clusters of a size can be resident (cached per device, kernel, size and shared-memory footprint, so that the answer,
    // and with it the way k is split and summed, depends on the product's shape alone and not on the calls before it)
    // and take the most ranks whose column blocks all fit, then as few as give the same longest share of k stages.
    int cluster_s = 0;
    if (p.cluster_s > 0) {
        int* fits = attr_cache().clusters(ctx->device, (const void*)kern, smem);  // resident clusters of size s
        const int ncb = a.N / C::TN, kst = a.K / C::TK;
        int s = p.cluster_s;
        for (; s > 1; s--) {
            if (!fits[s]) {
                cudaLaunchConfig_t q = {};
                q.gridDim = dim3(s, ncb);
                q.blockDim = dim3(C::THREADS);
                q.dynamicSmemBytes = smem;
                cudaLaunchAttribute ca[1];
                ca[0].id = cudaLaunchAttributeClusterDimension;
                ca[0].val.clusterDim.x = s; ca[0].val.clusterDim.y = 1; ca[0].val.clusterDim.z = 1;
                q.attrs = ca; q.numAttrs = 1;
                int nc = 0;
                if (cudaOccupancyMaxActiveClusters(&nc, kern, &q) != cudaSuccess) nc = -1;
                fits[s] = nc > 0 ? nc : -1;
            }
            if (fits[s] >= ncb) break;
        }
        if (s > kst) s = kst;
        const int longest = (kst + s - 1) / s;
        while (s > 1 && (kst + s - 2) / (s - 1) == longest) s--;
        cluster_s = s;
    }
    a.cluster_s = cluster_s;
    a.early = ctx->early > 0 ? ctx->early : 1;
    if (cluster_s > 0) {

        a.maxc = 1;
        lc.gridDim = dim3(cluster_s, a.N / C::TN);
        at[nat].id = cudaLaunchAttributeClusterDimension;
        at[nat].val.clusterDim.x = cluster_s;
        at[nat].val.clusterDim.y = 1;
        at[nat].val.clusterDim.z = 1;
        nat++;
    } else {
        int grid, maxc;
        grid_of(ctx, p, a.N, a.K, &grid, &maxc);
        a.maxc = maxc;
        if ((size_t)(a.N / 64) * maxc * NT * 4 * 32 * 16 > ctx->scratch_bytes) return QB_ERR_ARG;
        lc.gridDim = dim3(grid);
    }
    lc.blockDim = dim3(C::THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    if (ctx->pdl) {
        at[nat].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[nat].val.programmaticStreamSerializationAllowed = 1;
        nat++;
    }
    lc.attrs = at;
    lc.numAttrs = nat;
    GemvMaps maps = {};
    EncodeTiled enc = encode_tiled();
    if (!enc) return QB_ERR_UNSUPPORTED;
    a.xmap = (!a.xrows && C::XTENSOR) ? 1 : 0;
    if (a.xmap) {
        // X: m rows of K halves = K/4 8-byte elements from row0 on; box: a padded row (XROW halves) x m rows
        const cuuint64_t xd[2] = {(cuuint64_t)(a.K / 4), (cuuint64_t)a.m}, xs[1] = {(cuuint64_t)a.K * 2};
        const cuuint32_t xb[2] = {(cuuint32_t)(C::XROW / 4), (cuuint32_t)a.m}, one[2] = {1, 1};
        if (enc(&maps.x, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void*)(a.X + (size_t)a.row0 * a.K), xd, xs, xb, one,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return QB_ERR_ARG;
    }
    if (C::TENSOR) {
        // weights: K/16 rows of 2N words = N 8-byte elements; a stage's box: CG x 64 elements x TK/16 rows
        const cuuint64_t wd[2] = {(cuuint64_t)a.N, (cuuint64_t)(a.K / 16)}, ws[1] = {(cuuint64_t)a.N * 8};
        const cuuint32_t wb[2] = {(cuuint32_t)(CG * 64), (cuuint32_t)(C::TK / 16)}, one[2] = {1, 1};
        // scales (and offsets): K/128 (x 2) rows of N halves; box TN x KG
        const cuuint64_t sd[2] = {(cuuint64_t)a.N, (cuuint64_t)((1 + a.zp) * (a.K / 128))}, ss[1] = {(cuuint64_t)a.N * 2};
        const cuuint32_t sb[2] = {(cuuint32_t)C::TN, (cuuint32_t)KG};
        if (enc(&maps.w, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void*)a.B, wd, ws, wb, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            enc(&maps.s, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)a.S, sd, ss, sb, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return QB_ERR_ARG;
    }
    QB_CUDA(cudaLaunchKernelEx(&lc, kern, maps, a));
    return QB_OK;
}

template <int NT, int EPI>
static int launch_shape(qb_ctx* ctx, cudaStream_t st, const GemvArgs& a, const GemvPlan& p) {
    if (a.zp) {  // the zero-point variants: the three shapes the built-in choice uses
        if (p.cg == 2 && p.kg == 4) return launch_cfg<2, 4, NT, EPI, 1>(ctx, st, a, p);
        if (p.cg == 4 && p.kg == 2) return launch_cfg<4, 2, NT, EPI, 1>(ctx, st, a, p);
        if (p.cg == 4 && p.kg == 1) return launch_cfg<4, 1, NT, EPI, 1>(ctx, st, a, p);
        return QB_ERR_UNSUPPORTED;
    }
    if (p.cg == 2 && p.kg == 4) return launch_cfg<2, 4, NT, EPI>(ctx, st, a, p);
    if (p.cg == 4 && p.kg == 2) return launch_cfg<4, 2, NT, EPI>(ctx, st, a, p);
    if (p.cg == 8 && p.kg == 1) return launch_cfg<8, 1, NT, EPI>(ctx, st, a, p);
    if (p.cg == 1 && p.kg == 8) return launch_cfg<1, 8, NT, EPI>(ctx, st, a, p);
    if (p.cg == 4 && p.kg == 1) return launch_cfg<4, 1, NT, EPI>(ctx, st, a, p);
    return QB_ERR_ARG;
}

// The built-in choice: wide matrices take 256 x 256 tiles (fewer, larger copies; a block's range crosses few column
// blocks), narrow ones 128 x 512 so that a column block is shared by few blocks; the ring as deep as the blocks per
// SM allow.
static GemvPlan pick(const qb_ctx* ctx, int n, int k, int m, int cg, int kg, int ctas, int zp = 0) {
    GemvPlan p;
    bool deep = false;  // equal shares of a persistent grid instead of a cluster per column block (long k that is no multiple of 512)
    if (cg) { p.cg = cg; p.kg = kg; }
    else if (n >= 65536 && n % 512 == 0 && !zp) { p.cg = 8; p.kg = 1; }  // the output layer: no k groups to add up per piece
    // wide, short k, and no more 64-output column blocks than block slots (the in-projections, 16384 and 14336 x 5120):
    // 64 x 1024 tiles, ONE block per column block: the eight k groups of a block add up in shared memory and nothing
    // crosses blocks. 4.72 ms per 64-layer step against 4.85 ms with 256 x 256 tiles in clusters of 4 / 5 ranks.
    else if (n >= 8192 && k % 1024 == 0 && n / 64 <= ctx->sms * 2 && !zp) { p.cg = 1; p.kg = 8; }
    else if (n >= 8192 && k % 256 == 0) { p.cg = 4; p.kg = 2; }
    // few outputs, long k (down, 5120 x 17408): 128 x 512 tiles, 40 column blocks in clusters of 7 ranks, like the
    // out-projection: 13.4 us on its own and 4.87 ms per 64-layer step, against 15.5 us and 5.03 ms as equal shares of
    // a persistent grid of 256 x 256 tiles (whose column blocks had some 15 sharers to add up) and 5.04 ms as 256 x 256
    // tiles in clusters of 8
    else if (k >= 16384 && k % 512 == 0 && n % 128 == 0) { p.cg = 2; p.kg = 4; }
    else if (k >= 16384 && k % 256 == 0 && n % 256 == 0) { p.cg = 4; p.kg = 2; deep = true; }
    else if (k % 512 == 0 && n % 128 == 0) { p.cg = 2; p.kg = 4; }
    else if (k % 256 == 0) { p.cg = 4; p.kg = 2; }
    else { p.cg = 4; p.kg = 1; }
    p.ctas = ctas ? ctas : 2;
    const int budget = (228 * 1024) / p.ctas - 1024;
    p.nstages = 2;
    while (p.nstages < GEMV_MAX_STAGES && smem_of(p.cg, p.kg, m, p.nstages + 1, zp) <= budget) p.nstages++;
    // Clustered split K when the column blocks x ranks fit one wave of blocks: the most ranks (at most 8, the
    // portable cluster size) that fit, then as few as give the same longest share. The in-block reduction buffer
    // doubles as the rank's parking space, so the tile must have kg > 1.
    p.cluster_s = 0;
    const int slots = ctx->sms * p.ctas, ncb = n / (p.cg * 64), kst = k / (p.kg * 128);
    if (!ctx->no_cluster && !deep && p.kg > 1 && ncb <= slots) {
        int s = slots / ncb;  // an upper bound; the launch asks the driver what really fits
        if (s > 8) s = 8;
        (void)kst;
        p.cluster_s = s;
    }
    return p;
}

}  // namespace qb

using namespace qb;

// Measurement only: the next products record per-block timestamps (4 x 1024 int64 each) into `buf` (device memory);
// null switches it off.
extern "C" int qb_marlin_trace(qb_ctx* ctx, long long* buf) {
    ctx->trace = buf;
    return QB_OK;
}

// Measurement only: 1 makes the products' consumers release every stage unread, which times the copy pipeline alone
// (results are then meaningless); 2 (tests) makes the copy warp leave out its second stage and cuts the consumers' wait
// to 1024 polls: the wait runs out, the warps record error 2, walk on and the kernel ends; 0 restores the product.
extern "C" int qb_marlin_probe(qb_ctx* ctx, int mode) {
    ctx->probe = mode;
    return QB_OK;
}

extern "C" int qb_marlin_early(qb_ctx* ctx, int stages) {
    if (!ctx || stages < 1 || stages > GEMV_MAX_STAGES) return QB_ERR_ARG;
    ctx->early = stages;
    return QB_OK;
}

extern "C" int qb_marlin_tune(qb_ctx* ctx, int cg, int kg, int nstages, int ctas) {
    // ctas < 0: as -ctas, and stream-K only (no clustered split K); nstages < 0: as -nstages, and no tensor-core
    // path for more than 16 rows (16-row slabs through the skinny kernel instead)
    ctx->no_tc = nstages < 0;
    if (nstages < 0) nstages = nstages == -1 ? 0 : -nstages;
    ctx->no_cluster = ctas < 0;
    if (ctas < 0) ctas = -ctas;
    ctx->tune_cg = cg; ctx->tune_kg = kg; ctx->tune_nstages = nstages; ctx->tune_ctas = ctas;
    return QB_OK;
}

static int gemm_rows(qb_ctx* ctx, cudaStream_t st, const void* X, const void* B, void* Y, const void* S, int m,
                     int n, int k, int row0, int epi, const int* xrows, unsigned long long* keys, int n_valid,
                     int zp = 0) {
    int nt = m <= 8 ? 1 : 2;
    GemvPlan p = pick(ctx, n, k, m, ctx->tune_cg, ctx->tune_kg, ctx->tune_ctas, zp);
    if (ctx->tune_nstages) p.nstages = ctx->tune_nstages;
    int tn = p.cg * 64, tk = p.kg * 128;
    if (n % tn || k % tk || p.nstages < 2 || p.nstages > GEMV_MAX_STAGES) return QB_ERR_ARG;
    if (smem_of(p.cg, p.kg, m, p.nstages, zp) > 227 * 1024 || (size_t)(n / 64) > ctx->ncounters) return QB_ERR_ARG;
    GemvArgs a;
    a.X = (const __half*)X; a.xrows = xrows; a.B = (const uint32_t*)B; a.S = (const __half*)S; a.Y = Y;
    a.m = m; a.N = n; a.K = k; a.row0 = row0;
    a.nstages = p.nstages; a.maxc = 1;
    a.probe = ctx->probe;
    a.wait_limit = ctx->probe == 2 ? 1024u : WAIT_LIMIT;
    a.trace = ctx->trace;
    if (ctx->trace) ctx->trace += 4 * 1024;  // the next product's slots
    a.scratch = (float4*)ctx->scratch; a.counters = ctx->counters; a.keys = keys; a.n_valid = n_valid; a.err = ctx->err;
    a.zp = zp;
#define QB_GO(NT)                                                              \
    switch (epi) {                                                             \
        case QB_EPI_PLAIN: return launch_shape<NT, EPI_PLAIN>(ctx, st, a, p);  \
        case QB_EPI_SILU: return launch_shape<NT, EPI_SILU>(ctx, st, a, p);    \
        case QB_EPI_ARGMAX: return launch_shape<NT, EPI_ARGMAX>(ctx, st, a, p);\
        default: return QB_ERR_ARG;                                            \
    }
    if (nt == 1) { QB_GO(1) } else { QB_GO(2) }
#undef QB_GO
}

extern "C" int qb_marlin_gemm(qb_ctx* ctx, void* stream, const void* X, const void* B, void* Y, const void* S, int m,
                              int n, int k, int row0, int epi, const int* xrows, unsigned long long* keys,
                              int n_valid) {
    if (!ctx || !X || !B || !Y || !S || m < 0 || n <= 0 || k <= 0 || n % 256 || k % 128) return QB_ERR_ARG;
    if (epi == QB_EPI_ARGMAX && !keys) return QB_ERR_ARG;
    if (epi == QB_EPI_SILU && (n % 16)) return QB_ERR_ARG;
    if (epi < 0 || epi > QB_EPI_ARGMAX) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // more than 16 rows: the tensor-core product (plain and SwiGLU epilogues, contiguous rows)
    if (m > 16 && epi != QB_EPI_ARGMAX && !xrows && !ctx->no_tc)
        return qb_gemm_tc_launch(ctx, st, X, B, Y, S, m, n, k, row0, epi, 0);
    // otherwise 16-row slabs through the skinny kernel
    for (int r = 0; r < m; r += 16) {
        int mm = m - r < 16 ? m - r : 16;
        int rc = gemm_rows(ctx, st, X, B, Y, S, mm, n, k, xrows ? 0 : row0 + r, epi, xrows ? xrows + r : nullptr,
                           keys ? keys + (xrows ? r : 0) : nullptr, n_valid);
        if (rc) return rc;
        if (xrows) {  // gathered rows land at output rows r..: shift Y by r rows
            Y = (char*)Y + (size_t)mm * (epi == QB_EPI_SILU ? n / 2 * 2 : (size_t)n * 4);
        }
    }
    return QB_OK;
}


// ------------------------------------------------------------------------------------------------ no-allocation variant
// The zero-point variants (marlin_*_z, kernels/marlin.cuh:126-133): S holds the scales [k/128][n] followed by a second
// table (8 - z) * scale in the same layout (pack_marlin with zeros, src/cuda/core.rs:262-285). Any row count: more than
// 16 contiguous rows with the plain or SwiGLU epilogue run on the tensor-core product, the rest as 16-row slabs.
extern "C" int qb_marlin_gemm_z(qb_ctx* ctx, void* stream, const void* X, const void* B, void* Y, const void* S, int m,
                                int n, int k, int row0, int epi, const int* xrows, unsigned long long* keys,
                                int n_valid) {
    if (!ctx || !X || !B || !Y || !S || m < 0 || n <= 0 || k <= 0 || n % 256 || k % 128) return QB_ERR_ARG;
    if (epi < 0 || epi > QB_EPI_ARGMAX) return QB_ERR_ARG;
    if (epi == QB_EPI_ARGMAX && !keys) return QB_ERR_ARG;
    if (epi == QB_EPI_SILU && (n % 16)) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (m > 16 && epi != QB_EPI_ARGMAX && !xrows && !ctx->no_tc)
        return qb_gemm_tc_launch(ctx, st, X, B, Y, S, m, n, k, row0, epi, 1);
    for (int r = 0; r < m; r += 16) {
        int mm = m - r < 16 ? m - r : 16;
        int rc = gemm_rows(ctx, st, X, B, Y, S, mm, n, k, xrows ? 0 : row0 + r, epi, xrows ? xrows + r : nullptr,
                           keys ? keys + (xrows ? r : 0) : nullptr, n_valid, 1);
        if (rc) return rc;
        if (xrows) Y = (char*)Y + (size_t)mm * (epi == QB_EPI_SILU ? n / 2 * 2 : (size_t)n * 4);
    }
    return QB_OK;
}

// Some hosts can never call cudaMalloc once they are serving: an engine that has handed all free device memory to its
// KV-cache page pool (the reference sizes that pool from what is left after loading, src/cuda/qwen/mod.rs:422-428), a
// plugin loaded into a process whose allocator is owned by someone else, code running inside a stream capture. For
// them the stream-K product's scratch (split-K partials, arrival tickets, error word) also exists as a fixed array
// inside the library image: every GPU that loads the library holds these QB_STATIC_SCRATCH_BYTES until exit.
namespace {

constexpr size_t STATIC_PARTIAL_BYTES = 16u << 20;  // [n / 64][sharers][4][32] float4 of one product
constexpr size_t STATIC_TICKETS = 4096;             // one per 64 outputs: n <= 262144
constexpr size_t STATIC_BYTES = STATIC_PARTIAL_BYTES + STATIC_TICKETS * sizeof(int) + 256;

static __device__ __align__(256) unsigned char qb_static_scratch[STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
// device address of the array on each device, resolved by the first call there (the array's name in host code is only
// a handle for cudaGetSymbolAddress, not an address a kernel could use)
unsigned char* g_static_ptr[MAX_DEVICES] = {nullptr};
int g_static_sms[MAX_DEVICES] = {0};

}  // namespace

extern "C" int qb_static_scratch_bytes(void) { return (int)STATIC_BYTES; }

// The error word of the allocation-free products on the current device: non-zero once one of them gave up a bounded
// wait (its output is then incomplete). Reads and clears it; waits for the device. 0 when no such product ran yet.
extern "C" int qb_static_device_error(void) {
    int dev = -1;
    QB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES || !g_static_ptr[dev]) return 0;
    int* err = (int*)(g_static_ptr[dev] + STATIC_PARTIAL_BYTES + STATIC_TICKETS * sizeof(int));
    int v = 0;
    QB_CUDA(cudaDeviceSynchronize());
    QB_CUDA(cudaMemcpy(&v, err, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) QB_CUDA(cudaMemset(err, 0, sizeof(int)));
    return v;
}

extern "C" int qb_marlin_gemm_noalloc(void* stream, const void* X, const void* B, void* Y, const void* S, int m, int n,
                                      int k, int row0, int epi, const int* xrows, unsigned long long* keys,
                                      int n_valid) {
    if (!X || !B || !Y || !S || m < 1 || m > 16 || n <= 0 || k <= 0 || n % 256 || k % 128) return QB_ERR_ARG;
    if (epi == QB_EPI_ARGMAX && !keys) return QB_ERR_ARG;
    int dev = -1;
    QB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return QB_ERR_ARG;
    if (!g_static_ptr[dev]) {
        // set-up, once per device, with that device current: the array's device address and the SM count
        unsigned char* ptr = nullptr;
        QB_CUDA(cudaGetSymbolAddress((void**)&ptr, qb_static_scratch));
        QB_CUDA(cudaDeviceGetAttribute(&g_static_sms[dev], cudaDevAttrMultiProcessorCount, dev));
        g_static_ptr[dev] = ptr;
    }
    // a context on the stack that points into the static array; stream-K only (the path that needs the scratch)
    qb_ctx c;
    c.device = dev;
    c.sms = g_static_sms[dev];
    c.scratch = (float*)g_static_ptr[dev];
    c.scratch_bytes = STATIC_PARTIAL_BYTES;
    c.counters = (int*)(g_static_ptr[dev] + STATIC_PARTIAL_BYTES);
    c.ncounters = STATIC_TICKETS;
    c.err = (int*)(g_static_ptr[dev] + STATIC_PARTIAL_BYTES + STATIC_TICKETS * sizeof(int));
    c.no_cluster = true;
    if (epi < 0 || epi > QB_EPI_ARGMAX) return QB_ERR_ARG;
    // sizes beyond the fixed array: refuse before anything is enqueued
    if ((size_t)(n / 64) > STATIC_TICKETS) return QB_ERR_TOO_LARGE;
    {
        int nt = m <= 8 ? 1 : 2;
        GemvPlan p = pick(&c, n, k, m, 0, 0, 0);
        int grid, maxc;
        grid_of(&c, p, n, k, &grid, &maxc);
        if ((size_t)(n / 64) * maxc * nt * 4 * 32 * 16 > STATIC_PARTIAL_BYTES) return QB_ERR_TOO_LARGE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // the tickets must start at zero; every call leaves them so, but the array is shared with whatever ran before
    QB_CUDA(cudaMemsetAsync(c.counters, 0, (size_t)(n / 64) * sizeof(int), st));
    return gemm_rows(&c, st, X, B, Y, S, m, n, k, xrows ? 0 : row0, epi, xrows, keys, n_valid);
}
