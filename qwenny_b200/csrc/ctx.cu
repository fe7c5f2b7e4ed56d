// Context creation and the error word.
#include "ctx.h"

extern "C" {

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
    c->sq_groups = 1024;
    QB_CUDA(cudaMalloc(&c->sq, c->sq_groups * 16 * sizeof(float)));
    QB_CUDA(cudaMemset(c->sq, 0, c->sq_groups * 16 * sizeof(float)));
    QB_CUDA(cudaMalloc(&c->gbar, 64));
    QB_CUDA(cudaMemset(c->gbar, 0, 64));
    *out = c;
    return QB_OK;
}

void qb_destroy(qb_ctx* c) {
    if (!c) return;
    cudaFree(c->scratch);
    cudaFree(c->counters);
    cudaFree(c->err);
    cudaFree(c->gbar);
    cudaFree(c->sq);
    delete c;
}

int qb_device_error(qb_ctx* c) {
    int v = 0;
    QB_CUDA(cudaDeviceSynchronize());
    QB_CUDA(cudaMemcpy(&v, c->err, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) QB_CUDA(cudaMemset(c->err, 0, sizeof(int)));
    return v;
}

int qb_sm_count(const qb_ctx* c) { return c->sms; }

int qb_set_pdl(qb_ctx* c, int on) {
    c->pdl = on != 0;
    return QB_OK;
}

}  // extern "C"
