/* Measurement-only entry points of libqwenny_b200.so: exported for the timing and profiling drivers, not part of the
 * public ABI (include/qwenny_b200.h) and not for a serving host. */
#pragma once
#include "ctx.h"
#ifdef __cplusplus
extern "C" {
#endif
/* Fixes the tile shape (cg x kg consumer warps), ring depth and blocks per SM of the next qb_marlin_gemm calls on the
 * context; zeros restore the built-in choice. ctas < 0: as -ctas, and stream-K only; nstages < 0: as -nstages, and no
 * tensor-core path for more than 16 rows. */
int qb_marlin_tune(qb_ctx* ctx, int cg, int kg, int nstages, int ctas_per_sm);
/* The following qb_marlin_gemm calls write per-block timestamps (ns of the global timer: start, first stage landed,
 * last stage consumed, end; 4 x 1024 int64 per call) into consecutive slices of `buf`; NULL switches it off. */
int qb_marlin_trace(qb_ctx* ctx, long long* buf);
/* mode 1 makes the products' consumers release every stage unread, so a launch times the copy pipeline alone (its
 * results are meaningless); mode 2 (tests) makes the copy warp leave out its second stage and cuts the consumers' wait
 * to 1024 polls: their wait runs out, they record error 2 and walk on, the kernel ends; 0 restores the product. */
int qb_marlin_probe(qb_ctx* ctx, int mode);
/* Tests: the next n graph captures of the model report out of memory without touching the GPU. */
struct qb_model;
int qb_model_fail_captures(struct qb_model* m, int n);
/* Host-only checks of the step-graph cache policy (with fakes behind its hooks) and of the per-device
 * kernel-attribute bookkeeping; 0 when they hold. */
int qb_graph_cache_selftest(void);
int qb_attr_cache_selftest(void);
/* Tests: one block waits on an mbarrier that nothing arrives on, with the library's bounded wait cut to `limit` polls
 * (at most 2^20); the wait runs out and the context's error word reads 99 (qb_device_error). */
int qb_wait_probe(qb_ctx* ctx, void* stream, unsigned limit);
#ifdef __cplusplus
}
#endif
