// The regions of a slot's saved image (session.cu): where each lives on the device and in the image.
#pragma once
#include <vector>
#include "ctx.h"

namespace qb {

enum { SPAN_PLAIN = 0, SPAN_STATE = 1, SPAN_RING = 2, SPAN_META = 3 };

struct Span {
    unsigned char* dev;        // plain: the bytes; state / ring: the slot's DeltaNet memory; meta (load): its metadata
    const int* meta;           // state / ring / meta when saving: the slot's metadata {end, ck, ebuf, _}
    unsigned long long off;    // offset in the image
    unsigned long long bytes;
    int kind;
    int j;                     // ring: the row (0 .. CONV_K - 2); meta (save): the layer's index in `positions`
    int pos;                   // loading: the position the state is at
    unsigned chunk0;           // the span's first 64 KB chunk among all spans'
};

// numbers the spans' chunks; returns their count (the grid of the copy kernel)
unsigned assign_chunks(std::vector<Span>& spans);
// gathers (save) the spans into the image at `staging`, or scatters (load) the image into them; when saving, every
// SPAN_META span writes its layer's end position to positions[j]
int launch_session_copy(qb_ctx* ctx, cudaStream_t st, bool save, const Span* d_spans, int nspans, unsigned chunks,
                        unsigned char* staging, int* positions);

}  // namespace qb
