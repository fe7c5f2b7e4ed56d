// The C entries of the draft head's bookkeeping (draft_vocab.h) and DraftHead::learn of the reference's host
// (src/cuda/qwen/draft.rs:55-68): the tokens a step commits go into the bookkeeping, and every tile of 16 rows that
// changed is packed from the stored output layer and written into the model's draft head in place.
#include <new>
#include <vector>
#include "../../include/qwenny_b200.h"
#include "draft_vocab.h"

struct qb_draft_vocab {
    qb::DraftRows* rows = nullptr;
};

extern "C" {

int qb_draft_vocab_create(int vocab, const uint32_t* ids, const float* score, int n, int cap, qb_draft_vocab** out) {
    if (!out || vocab <= 0 || n < 0 || cap <= 0 || (n && !ids)) return QB_ERR_ARG;
    std::vector<uint32_t> i(ids, ids + n);
    std::vector<float> s;
    if (score) s.assign(score, score + n);
    qb::DraftRows* r = new (std::nothrow) qb::DraftRows((size_t)vocab, std::move(i), std::move(s), (size_t)cap);
    if (!r || !r->ok()) { delete r; return QB_ERR_ARG; }
    *out = new qb_draft_vocab{r};
    return QB_OK;
}

int qb_draft_vocab_load(int vocab, const uint32_t* saved_ids, const float* saved_score, int n_saved,
                        const uint32_t* seed_ids, int n_seed, qb_draft_vocab** out) {
    if (!out || vocab <= 0 || n_saved < 0 || n_seed < 0 || (n_seed && !seed_ids)) return QB_ERR_ARG;
    qb::DraftRows* r = qb::DraftRows::load((size_t)vocab, saved_ids, saved_score, (size_t)n_saved, seed_ids, (size_t)n_seed);
    if (!r) return QB_ERR_ARG;
    *out = new qb_draft_vocab{r};
    return QB_OK;
}

void qb_draft_vocab_destroy(qb_draft_vocab* v) {
    if (!v) return;
    delete v->rows;
    delete v;
}

int qb_draft_vocab_rows(const qb_draft_vocab* v) { return v ? (int)v->rows->ids().size() : 0; }

int qb_draft_vocab_get(const qb_draft_vocab* v, uint32_t* ids, float* score, int cap) {
    if (!v || cap < 0 || (int)v->rows->ids().size() > cap) return QB_ERR_ARG;
    const size_t n = v->rows->ids().size();
    for (size_t r = 0; r < n; r++) {
        if (ids) ids[r] = v->rows->ids()[r];
        if (score) score[r] = v->rows->score()[r];
    }
    return QB_OK;
}

int qb_draft_vocab_row_of(const qb_draft_vocab* v, uint32_t token) {
    if (!v) return -1;
    const uint32_t r = v->rows->row_of(token);
    return r == qb::DraftRows::NONE ? -1 : (int)r;
}

int qb_draft_vocab_waiting(const qb_draft_vocab* v, uint32_t token) { return v && v->rows->waiting(token) ? 1 : 0; }
int qb_draft_vocab_pending(const qb_draft_vocab* v) { return v ? (int)v->rows->pending() : 0; }
int qb_draft_vocab_dirty(const qb_draft_vocab* v) { return v && v->rows->dirty() ? 1 : 0; }

int qb_draft_vocab_saved(qb_draft_vocab* v) {
    if (!v) return QB_ERR_ARG;
    v->rows->saved();
    return QB_OK;
}

int qb_draft_vocab_may_change(const qb_draft_vocab* v, const uint32_t* toks, int n) {
    return v && n > 0 && toks && v->rows->may_change(toks, (size_t)n) ? 1 : 0;
}

int qb_draft_vocab_learn(qb_draft_vocab* v, const uint32_t* toks, int n, qb_publish_fn publish, void* user, int* changed) {
    if (!v || n < 0 || (n && !toks)) return QB_ERR_ARG;
    return v->rows->learn(
        toks, (size_t)n,
        [&](const std::vector<uint32_t>& ids, const std::vector<int>& tiles) {
            return publish ? publish(user, ids.data(), (int)ids.size(), tiles.data(), (int)tiles.size()) : 0;
        },
        changed);
}

int qb_draft_ids_pt(const uint8_t* bytes, size_t len, int vocab, uint32_t* ids, int cap, int* n) {
    if (!bytes || vocab <= 0 || !n || cap < 0 || (cap && !ids)) return QB_ERR_ARG;
    std::vector<uint32_t> got;
    const int rc = qb::draft_ids_from_pt(bytes, len, (size_t)vocab, &got);
    if (rc) return rc;
    *n = (int)got.size();
    if ((int)got.size() > cap) return QB_ERR_TOO_LARGE;
    for (size_t i = 0; i < got.size(); i++) ids[i] = got[i];
    return QB_OK;
}

int qb_model_learn(qb_model* m, void* stream, qb_draft_vocab* v, const uint32_t* toks, int n, const uint32_t* h_q,
                   const float* h_scales, const uint8_t* h_zeros, int zero_points, int rows, int cols, int group,
                   int* grew) {
    if (!m || !v || n < 0 || (n && !toks) || !h_q || !h_scales || rows <= 0 || cols <= 0 || cols % 128 || group <= 0)
        return QB_ERR_ARG;
    if (grew) *grew = 0;
    std::vector<uint32_t> words((size_t)cols / 16 * 32);
    std::vector<uint16_t> sc((size_t)(zero_points ? 2 : 1) * cols / 128 * 16);
    return v->rows->learn(
        toks, (size_t)n,
        [&](const std::vector<uint32_t>& ids, const std::vector<int>& tiles) {
            for (int t : tiles) {
                int order[16];
                for (int i = 0; i < 16; i++) order[i] = (int)ids[(size_t)16 * t + i];
                int rc = qb_marlin_block(h_q, h_scales, h_zeros, zero_points, rows, cols, group, order, words.data(), sc.data());
                int g = 0;
                if (!rc) rc = qb_model_learn_block(m, stream, t, words.data(), sc.data(), order, &g);
                if (rc) return rc;
                if (g && grew) *grew = 1;
            }
            return 0;
        },
        nullptr);
}

}  // extern "C"
