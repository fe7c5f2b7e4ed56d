// The library context: what the reference's Gemm::load allocates once per model (src/cuda/core.rs:437-464) — the SM
// count and the scratch its blocks reduce through — plus the device error word of the bounded waits.
#pragma once
#include <cuda.h>
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
    float* tc_part = nullptr;   // partial tiles of the tensor-core W4A16 product's stream-K shares (sms x 2 x 256 KB), taken with its first call
    int* tc_tickets = nullptr;  // its per-tile tickets (QB_TC_TICKETS, zero between launches)
    float* delta_tp = nullptr;  // scratch of the chunked delta rule (T, P, log decays per chunk and value head), taken by
                                // the first prompt-sized DeltaNet step
    // measurement override of the GEMV plan (0: built-in choice)
    int tune_cg = 0, tune_kg = 0, tune_nstages = 0, tune_ctas = 0;
    bool no_cluster = false, no_tc = false;
    // programmatic dependent launch on the launches that support it
    bool pdl = false;
    int probe = 0;               // measurement: see qb_marlin_probe
    int early = 1;               // stages of weights the next skinny product requests before it waits for the kernel
                                 // before it (set by the caller that knows what that kernel is; see model.cu)
    long long* trace = nullptr;  // measurement: per-block timestamps of the next products
};

constexpr int QB_TC_TICKETS = 1 << 16;  // tiles of one tensor-core W4A16 product (256 outputs x 256 tokens each)
#define QB_CUDA(x)                         \
    do {                                   \
        cudaError_t e_ = (x);              \
        if (e_ != cudaSuccess) return (int)e_; \
    } while (0)

namespace qb {

// cuTensorMapEncodeTiled, resolved through the runtime (the library does not link the driver); null when unavailable
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled();

// Kernel attributes (the opt-in to more than 48 KB of dynamic shared memory, the shared-memory carve-out) belong to the
// device that is current when cudaFuncSetAttribute runs, so what has been set is remembered per (device, kernel), not
// per process: a process that drives several GPUs opts every kernel in on each of them. AttrCache is the bookkeeping
// alone (no CUDA call), shared by all host threads behind one mutex.
class AttrCache {
  public:
    // true when `kern` on `device` has not yet been given at least `smem` bytes (or, smem == 0, has not been seen at
    // all); the new value is recorded, so the caller must then set the attribute
    bool need(int device, const void* kern, int smem);
    // the resident-cluster counts the driver reported for (device, kernel, shared memory), filled by the caller
    int* clusters(int device, const void* kern, int smem);
};
AttrCache& attr_cache();
// sets what `kern` needs on `device` (which must be current) before a launch with `smem` bytes of dynamic shared memory
int prepare_kernel(int device, const void* kern, int smem);

}  // namespace qb

// the many-tile prompt attention on tcgen05 (attn_prefill_tc.cu); reached through qb_attn_prefill
int qb_attn_prefill_tc_launch(qb_ctx* ctx, cudaStream_t st, const float* q, const void* kc, const void* vc, const float* ks,
                              const float* vs, const int* ptile, int ntile, const int* tok_slot, const int* tok_pos,
                              int cap, float* out, void* mix_f16);
// the prompt-sized W4A16 product on tcgen05 (w4a16_gemm_tc.cu); reached through qb_marlin_gemm / qb_marlin_gemm_z (zp:
// S carries the offsets' table after the scales) for more than 16 rows
int qb_gemm_tc_launch(qb_ctx* ctx, cudaStream_t st, const void* X, const void* B, void* Y, const void* S, int m, int n,
                      int k, int row0, int epi, int zp);
