// Context creation and the error word.
#include "ctx.h"
#include "common.cuh"
#include <array>
#include <map>
#include <mutex>
#include <tuple>

namespace qb {

namespace {
std::mutex g_attr_mutex;
std::map<std::pair<int, const void*>, int> g_attr_smem;
std::map<std::tuple<int, const void*, int>, std::array<int, 9>> g_attr_clusters;
}  // namespace

bool AttrCache::need(int device, const void* kern, int smem) {
    std::lock_guard<std::mutex> lock(g_attr_mutex);
    auto it = g_attr_smem.find({device, kern});
    if (it == g_attr_smem.end()) {
        g_attr_smem[{device, kern}] = smem;
        return true;
    }
    if (it->second >= smem) return false;
    it->second = smem;
    return true;
}

int* AttrCache::clusters(int device, const void* kern, int smem) {
    std::lock_guard<std::mutex> lock(g_attr_mutex);
    return g_attr_clusters.try_emplace(std::make_tuple(device, kern, smem), std::array<int, 9>{}).first->second.data();
}

AttrCache& attr_cache() {
    static AttrCache c;
    return c;
}

int prepare_kernel(int device, const void* kern, int smem) {
    if (!attr_cache().need(device, kern, smem)) return QB_OK;
    // Every kernel asks for the same L1 / shared-memory split (all shared): the big streaming kernels need it, and an
    // SM whose split has to change between two kernels drains first, which would undo the overlap of neighbours.
    QB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    if (smem > 48 * 1024) QB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return QB_OK;
}

}  // namespace qb

extern "C" {

// Host-only check of the per-device attribute bookkeeping (no CUDA call): 0 when two devices each get their own
// opt-in for the same kernel, a larger request on one device asks again there only, and repeats ask for nothing.
int qb_attr_cache_selftest(void) {
    static int k1, k2;  // stand-ins for two kernels
    qb::AttrCache& c = qb::attr_cache();
    const int d0 = 1000, d1 = 1001;  // device numbers no real GPU has
    if (!c.need(d0, &k1, 100000)) return 1;
    if (c.need(d0, &k1, 100000)) return 2;
    if (c.need(d0, &k1, 50000)) return 3;
    if (!c.need(d1, &k1, 100000)) return 4;   // the second device has not been opted in by the first one's call
    if (!c.need(d0, &k2, 0)) return 5;
    if (c.need(d0, &k2, 0)) return 6;
    if (!c.need(d0, &k1, 200000)) return 7;
    if (c.need(d1, &k1, 100000)) return 8;
    int* a = c.clusters(d0, &k1, 4096);
    a[3] = 17;
    if (c.clusters(d1, &k1, 4096)[3] != 0 || c.clusters(d0, &k1, 4096)[3] != 17) return 9;
    return 0;
}

const char* qb_version(void) { return "qwenny_b200 0.1 (sm_100a)"; }

int qb_create(int device, qb_ctx** out) {
    if (!out) return QB_ERR_ARG;
    QB_CUDA(cudaSetDevice(device));
    qb_ctx* c = new qb_ctx();
    c->device = device;
    QB_CUDA(cudaDeviceGetAttribute(&c->sms, cudaDevAttrMultiProcessorCount, device));
    // the largest user: split-K partials of a 16-row product, [n/64][nsplit][2][4][32] float4; 32 MiB covers
    // n * nsplit up to 2^17 * 8 (the 27B shapes need under 6 MiB)
    c->scratch_bytes = 32u << 20;
    QB_CUDA(cudaMalloc(&c->scratch, c->scratch_bytes));
    c->ncounters = 1 << 14;
    QB_CUDA(cudaMalloc(&c->counters, c->ncounters * sizeof(int)));
    QB_CUDA(cudaMemset(c->counters, 0, c->ncounters * sizeof(int)));
    QB_CUDA(cudaMalloc(&c->err, 64));
    QB_CUDA(cudaMemset(c->err, 0, 64));
    *out = c;
    return QB_OK;
}

void qb_destroy(qb_ctx* c) {
    if (!c) return;
    cudaFree(c->scratch);
    cudaFree(c->counters);
    cudaFree(c->err);
    cudaFree(c->delta_tp);
    cudaFree(c->tc_part);
    cudaFree(c->tc_tickets);
    delete c;
}

int qb_device_error(qb_ctx* c) {
    if (!c) return QB_ERR_ARG;
    int v = 0;
    QB_CUDA(cudaDeviceSynchronize());
    QB_CUDA(cudaMemcpy(&v, c->err, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) QB_CUDA(cudaMemset(c->err, 0, sizeof(int)));
    return v;
}

int qb_sm_count(const qb_ctx* c) { return c ? c->sms : 0; }

int qb_set_pdl(qb_ctx* c, int on) {
    if (!c) return QB_ERR_ARG;
    c->pdl = on != 0;
    return QB_OK;
}

}  // extern "C"


namespace qb {
EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}
}  // namespace qb

// ---------------------------------------------------------------------------------------------------------------
// Test of the waits' way out: a block waits (with the library's bounded wait, here with a short poll limit) on an
// mbarrier that nothing ever arrives on; the wait runs out, the block records code 99 in the context's error word and
// returns. The host reads it with qb_device_error and the context stays usable.
namespace qb {
__global__ void wait_probe_kernel(int* err, uint32_t limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, limit);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok && threadIdx.x == 0) atomicExch(err, 99);
}
}  // namespace qb

extern "C" int qb_wait_probe(qb_ctx* ctx, void* stream, unsigned limit) {
    if (!ctx || limit == 0 || limit > (1u << 20)) return QB_ERR_ARG;
    qb::wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->err, limit);
    return (int)cudaGetLastError();
}
