// The library context: what the reference's Gemm::load allocates once per model (src/cuda/core.rs:437-464) — the SM
// count and the scratch its blocks reduce through — plus the device error word of the bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/qwenny_b200.h"

struct qb_ctx {
    int device = 0;
    int sms = 0;
    // split-K partial sums of the skinny int4 products (L2 resident) and the per-64-output arrival tickets
    float* scratch = nullptr;
    size_t scratch_bytes = 0;
    int* counters = nullptr;
    size_t ncounters = 0;
    int* err = nullptr;  // device word
    float* sq = nullptr;       // sums of squares of the last residual product's rows: [sq_groups][16]
    size_t sq_groups = 0;
    unsigned* gbar = nullptr;  // grid-barrier counters of the persistent layer kernel (zero between launches)
    bool chain_pdl = true;     // that kernel's launch carries the programmatic-dependent-launch attribute too
    // measurement override of the GEMV plan (0: built-in choice)
    int tune_cg = 0, tune_kg = 0, tune_nstages = 0, tune_ctas = 0;
    bool no_cluster = false, no_tc = false;
    // programmatic dependent launch on the launches that support it
    bool pdl = false;
    int probe = 0;               // measurement: see qb_marlin_probe
    long long* trace = nullptr;  // measurement: per-block timestamps of the next products
};

#define QB_CUDA(x)                         \
    do {                                   \
        cudaError_t e_ = (x);              \
        if (e_ != cudaSuccess) return (int)e_; \
    } while (0)

// the prompt-sized W4A16 product on tcgen05 (w4a16_gemm_tc.cu); reached through qb_marlin_gemm for more than 16 rows
int qb_gemm_tc_launch(qb_ctx* ctx, cudaStream_t st, const void* X, const void* B, void* Y, const void* S, int m, int n,
                      int k, int row0, int epi);
