// A slot's state on the wire: the byte images the reference's host saves, swaps to the host and reloads
// (Model::save_kv / load_kv / save_state / load_state, src/cuda/qwen/mod.rs:993-1061; per layer Attn::layout / save /
// load, src/cuda/qwen/attn.rs:182-233, and DeltaNet::saved_bytes / save / load, src/cuda/qwen/deltanet.rs:181-226).
//
// The reference copies every region of every layer with a call of its own (per attention layer 4 kv heads x (keys,
// values, two scale rows); per DeltaNet layer the end state and three rows of the conv ring picked by the slot's
// metadata, which it first reads back). Here ONE kernel gathers all regions of all layers into a staging buffer in
// wire order (the DeltaNet regions resolved on the device from the metadata), and one copy moves the image over PCIe;
// loading is the mirror: one copy, one scatter kernel that also writes the DeltaNet metadata. The images are the
// reference's, byte for byte.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "launch.h"
#include "session.h"

namespace qb {
namespace {

constexpr unsigned long long CHUNK = 1ull << 16;  // bytes per block

template <bool SAVE>
__global__ void __launch_bounds__(256) session_copy_kernel(const Span* spans, int nspans, unsigned char* staging,
                                                           int* positions) {
    pdl_wait();
    // the span of this block's chunk: the last one whose first chunk is <= blockIdx.x
    int lo = 0, hi = nspans - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (spans[mid].chunk0 <= blockIdx.x) lo = mid; else hi = mid - 1;
    }
    const Span s = spans[lo];
    const unsigned long long at = (unsigned long long)(blockIdx.x - s.chunk0) * CHUNK;
    const unsigned long long n = s.bytes > at ? (s.bytes - at < CHUNK ? s.bytes - at : CHUNK) : 0;
    unsigned char* host_side = staging + s.off + at;
    unsigned char* dev = s.dev;
    bool zeros = false;
    if (s.kind == SPAN_STATE) {
        if (SAVE) dev += (size_t)s.meta[2] * SLOT_STATE * 4;  // the end state's buffer; a loaded state goes to buffer 0
    } else if (s.kind == SPAN_RING) {
        // row j of the conv ring's last CONV_K - 1 positions before `end`
        const int q = (SAVE ? s.meta[0] : s.pos) - (CONV_K - 1) + s.j;
        if (q < 0) {
            if (!SAVE) return;
            zeros = true;
        }
        dev += (size_t)SLOT_RING * 4 + (size_t)(q & (CR - 1)) * LQKV * 4;
    } else if (s.kind == SPAN_META) {
        if (threadIdx.x == 0) {
            if (SAVE) {
                positions[s.j] = s.meta[0];
            } else {
                int* m = reinterpret_cast<int*>(dev);
                m[0] = s.pos; m[1] = s.pos; m[2] = 0; m[3] = 0;
            }
        }
        return;
    }
    dev += at;
    unsigned char* src = SAVE ? dev : host_side;
    unsigned char* dst = SAVE ? host_side : dev;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | n) & 15) == 0) {
        for (unsigned long long i = threadIdx.x * 16ull; i < n; i += 256 * 16)
            *reinterpret_cast<uint4*>(dst + i) = zeros ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(src + i);
    } else {  // every region is whole 32-bit words
        for (unsigned long long i = threadIdx.x * 4ull; i < n; i += 256 * 4)
            *reinterpret_cast<unsigned*>(dst + i) = zeros ? 0u : *reinterpret_cast<const unsigned*>(src + i);
    }
}

}  // namespace

unsigned assign_chunks(std::vector<Span>& spans) {
    unsigned c = 0;
    for (auto& s : spans) {
        s.chunk0 = c;
        c += (unsigned)std::max<unsigned long long>(1, (s.bytes + CHUNK - 1) / CHUNK);
    }
    return c;
}

int launch_session_copy(qb_ctx* ctx, cudaStream_t st, bool save, const Span* d_spans, int nspans, unsigned chunks,
                        unsigned char* staging, int* positions) {
    if (nspans <= 0 || chunks == 0) return QB_OK;
    if (save) return launch(ctx, session_copy_kernel<true>, dim3(chunks), dim3(256), 0, st, d_spans, nspans, staging, positions);
    return launch(ctx, session_copy_kernel<false>, dim3(chunks), dim3(256), 0, st, d_spans, nspans, staging, positions);
}

}  // namespace qb
