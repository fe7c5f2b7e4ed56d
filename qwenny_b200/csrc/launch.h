// One launch helper for every kernel: cudaLaunchKernelEx with the programmatic-dependent-launch attribute when the
// context asks for it. Every kernel of the library calls pdl_wait() before it touches anything an earlier kernel of
// the stream wrote, so the chain of dependencies stays transitive whichever launches carry the attribute.
#pragma once
#include "ctx.h"

namespace qb {

template <typename... KArgs, typename... Args>
static inline int launch(const qb_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t st, Args... args) {
    if (int rc = prepare_kernel(ctx->device, (const void*)kern, (int)smem)) return rc;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = ctx->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&lc, kern, static_cast<KArgs>(args)...);
    return e == cudaSuccess ? QB_OK : (int)e;
}

}  // namespace qb
