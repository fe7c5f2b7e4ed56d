// The host arrays of a step: Step::upload of the reference's host (src/cuda/core.rs:835-926), restated. Pure host
// code (no CUDA call), so that the checks and the arrays can be tested without a device: the model's runner copies what
// this fills to the device in one piece.
#pragma once
#include <cstddef>
#include <cstdint>
#include "../../include/qwenny_b200.h"

namespace qb {
namespace step {

constexpr int MAX_TOK = 2048, MAX_OUT = 64;     // src/cuda/core.rs:16-19
constexpr int SHORT_SEG = 8, MAX_DEC = 64;      // attn::segments, src/cuda/qwen/attn.rs:17-19
constexpr int DCUT = 2048;                      // short segments are cut where pos / DCUT changes (attn.rs:27)
constexpr int PTILE = 10;                       // tokens of a prompt tile: 64 rows / 6 query heads per kv head (attn.rs:18)
constexpr int MAX_MARK = MAX_TOK + 8 * MAX_OUT;  // tokens a step may add to the seen sets (core.rs:880)

// offsets (ints) of the step arrays inside the single step allocation
struct StepLayout {
    size_t ids, tok_slot, tok_pos, seg_start, seg_len, seg_slot, seg_pos0, dtok, dseg, dkeys, ptile, out_rows, mark,
        mark_at, mtp_rows, row_first, total;
    StepLayout() {
        size_t o = 0;
        auto take = [&](size_t n) { size_t r = o; o += (n + 3) / 4 * 4; return r; };
        ids = take(MAX_TOK); tok_slot = take(MAX_TOK); tok_pos = take(MAX_TOK);
        seg_start = take(MAX_TOK); seg_len = take(MAX_TOK); seg_slot = take(MAX_TOK); seg_pos0 = take(MAX_TOK);
        dtok = take(MAX_TOK); dseg = take(2 * MAX_TOK); dkeys = take(MAX_TOK); ptile = take(2 * MAX_TOK); out_rows = take(MAX_OUT);
        mark = take(MAX_MARK); mark_at = take(MAX_TOK + 1); mtp_rows = take(MAX_TOK); row_first = take(MAX_OUT);
        total = o;
    }
};

// the host-side shape of a step: what sizes its launches (Step's counts, core.rs:700-727)
struct StepShape {
    int n = 0, n_out = 0, segs = 0, ndec = 0, ntile = 0, ndseg = 0, dmax = 0, max_seg = 0, dec_max_pos = 0, tile_max_pos = 0;
};

// Fills h (StepLayout().total ints) from a step's tokens and logit rows. Tokens of one sequence must be contiguous
// and in order. rows (MTP steps, else null): per token the row of the residual stream of the step before that holds
// its hidden state. marks / marks_at (null: every token of a segment): the tokens to add to the seen set of segment
// s's slot are marks[marks_at[s] .. marks_at[s + 1]] (Step::upload's `marks`: a verify step marks the committed
// history, not its drafts). QB_ERR_ARG where the reference's ensure!s fail; nothing of h is then to be used.
inline int build_step_arrays(const qb_tok* toks, int n, const int* out, int n_out, const int* rows, const uint32_t* marks,
                             const int* marks_at, int slots, int max_ctx, int vocab_valid, int* h, StepShape* shape) {
    if (!toks || !h || !shape || n < 1 || n > MAX_TOK || n_out < 0 || n_out > MAX_OUT || (n_out && !out)) return QB_ERR_ARG;
    if ((marks != nullptr) != (marks_at != nullptr)) return QB_ERR_ARG;
    for (int i = 0; i < n_out; i++)
        if (out[i] < 0 || out[i] >= n) return QB_ERR_ARG;
    const StepLayout L;
    int segs = 0;
    for (int i = 0; i < n; i++) {
        const qb_tok& t = toks[i];
        if ((int)t.slot >= slots || (int)t.pos >= max_ctx || (int)t.id >= vocab_valid) return QB_ERR_ARG;
        h[L.ids + i] = (int)t.id; h[L.tok_slot + i] = (int)t.slot; h[L.tok_pos + i] = (int)t.pos;
        if (i > 0 && toks[i - 1].slot == t.slot) {
            if (toks[i - 1].pos + 1 != t.pos) return QB_ERR_ARG;  // positions of a slot not consecutive
            h[L.seg_len + segs - 1]++;
        } else {
            for (int s = 0; s < segs; s++)
                if (h[L.seg_slot + s] == (int)t.slot) return QB_ERR_ARG;  // a slot in two segments
            h[L.seg_start + segs] = i; h[L.seg_len + segs] = 1; h[L.seg_slot + segs] = (int)t.slot;
            h[L.seg_pos0 + segs] = (int)t.pos;
            segs++;
        }
    }
    int ndec = 0, ndseg = 0, ntile = 0, dmax = 0, max_seg = 0, dec_max_pos = 0, tile_max_pos = 0, nmark = 0;
    for (int s = 0; s < segs; s++) {
        int st = h[L.seg_start + s], len = h[L.seg_len + s];
        max_seg = len > max_seg ? len : max_seg;
        if (len <= SHORT_SEG && ndec + len <= MAX_DEC) {
            int a = st;
            while (a < st + len) {
                int part = (int)toks[a].pos / DCUT, e = a + 1;
                while (e < st + len && (int)toks[e].pos / DCUT == part) e++;
                h[L.dseg + 2 * ndseg] = ndec; h[L.dseg + 2 * ndseg + 1] = e - a;
                for (int t = a; t < e; t++) {
                    h[L.dtok + ndec] = t;
                    h[L.dkeys + ndec] = (int)toks[e - 1].pos + 1;
                    ndec++;
                }
                dmax = e - a > dmax ? e - a : dmax;
                dec_max_pos = (int)toks[e - 1].pos > dec_max_pos ? (int)toks[e - 1].pos : dec_max_pos;
                ndseg++;
                a = e;
            }
        } else {
            for (int o = 0; o < len; o += PTILE) {  // prompt tiles of 64 / GROUP consecutive tokens
                int cnt = len - o < PTILE ? len - o : PTILE, last = (int)toks[st + o + cnt - 1].pos;
                h[L.ptile + 2 * ntile] = st + o; h[L.ptile + 2 * ntile + 1] = cnt;
                tile_max_pos = last > tile_max_pos ? last : tile_max_pos;
                ntile++;
            }
        }
        h[L.mark_at + s] = nmark;
        if (marks) {
            const int a = marks_at[s], e = marks_at[s + 1];
            if (a < 0 || e < a || e - a > MAX_MARK - nmark) return QB_ERR_ARG;  // more marks than the step holds (core.rs:880)
            for (int t = a; t < e; t++) {
                if (marks[t] >= (uint32_t)vocab_valid) return QB_ERR_ARG;
                h[L.mark + nmark++] = (int)marks[t];
            }
        } else {
            for (int t = st; t < st + len; t++) h[L.mark + nmark++] = (int)toks[t].id;
        }
    }
    h[L.mark_at + segs] = nmark;
    for (int i = 0; i < n_out; i++) {
        h[L.out_rows + i] = out[i];
        int first = 0;  // the first token of the row's segment (Step::upload, src/cuda/core.rs:893-894)
        for (int sg = 0; sg < segs; sg++)
            if (h[L.seg_start + sg] <= out[i]) first = h[L.seg_start + sg];
        h[L.row_first + i] = first;
    }
    if (rows)
        for (int i = 0; i < n; i++) h[L.mtp_rows + i] = rows[i];
    shape->n = n; shape->n_out = n_out; shape->segs = segs; shape->ndec = ndec; shape->ntile = ntile; shape->ndseg = ndseg;
    shape->dmax = dmax; shape->max_seg = max_seg; shape->dec_max_pos = dec_max_pos; shape->tile_max_pos = tile_max_pos;
    return QB_OK;
}

}  // namespace step
}  // namespace qb
