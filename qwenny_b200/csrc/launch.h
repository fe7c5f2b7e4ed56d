// One launch helper for every kernel: cudaLaunchKernelEx with the programmatic-dependent-launch attribute when the
// context asks for it. Every kernel of the library calls pdl_wait() before it touches anything an earlier kernel of
// the stream wrote, so the chain of dependencies stays transitive whichever launches carry the attribute.
#pragma once
#include <set>
#include "ctx.h"

namespace qb {

template <typename... KArgs, typename... Args>
static inline int launch(const qb_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t st, Args... args) {
    // Every kernel asks for the same L1 / shared-memory split (all shared): the big streaming kernels need it, and an
    // SM whose split has to change between two kernels drains first, which would undo the overlap of neighbours.
    static std::set<const void*> prepared;
    if (!prepared.count((const void*)kern)) {
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        prepared.insert((const void*)kern);
    }
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
