// Which token has which row of the MTP's draft head, and how that changes while a server runs: the bookkeeping of the
// reference's host (Rows and Adaptive, src/draft_vocab.rs:22-201), restated. Every token a step commits adds 1 to the
// score of its row; all scores halve every DECAY committed tokens; a token without a row waits until 16 such tokens
// are there, which then get a new tile of 16 rows while the head has room and else the rows of the coldest tokens
// (score below 1: unused since the last halvings), rewritten in place. Pure host code: the head's weights are written
// by whoever publishes the changed tiles (qb_model_learn_block).
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <vector>

namespace qb {

class DraftRows {
  public:
    static constexpr uint32_t NONE = 0xffffffffu;
    static constexpr size_t DECAY = 20000;     // committed tokens between two halvings (draft_vocab.rs:17)
    static constexpr size_t MAX_ROWS = 65536;  // rows of a draft head at most (draft_vocab.rs:15)

    // Rows for `ids` with their scores (a score array of another length: all 0), a multiple of 16 of them, at most
    // `cap` (Rows::new, draft_vocab.rs:41-54). ok() is false when the arguments do not make a head.
    DraftRows(size_t vocab, std::vector<uint32_t> ids, std::vector<float> score, size_t cap)
        : ids_(std::move(ids)), score_(std::move(score)), row_of_(vocab, NONE), waiting_(vocab, 0), cap_(cap) {
        ok_ = ids_.size() % 16 == 0 && ids_.size() <= cap_ && cap_ % 16 == 0;
        for (size_t r = 0; ok_ && r < ids_.size(); r++) {
            const uint32_t t = ids_[r];
            if (t >= vocab || row_of_[t] != NONE) ok_ = false;  // a token twice or beyond the vocabulary
            else row_of_[t] = (uint32_t)r;
        }
        if (score_.size() != ids_.size()) score_.assign(ids_.size(), 0.f);
    }

    // The rows saved by an earlier run, if they fit this vocabulary (else none of them: read_saved,
    // draft_vocab.rs:134-146), then those of `seed` that are new while there is room; whole tiles only (Adaptive::load,
    // :158-176). Null when a seed token lies beyond the vocabulary or less than one tile comes of it.
    static DraftRows* load(size_t vocab, const uint32_t* saved, const float* saved_score, size_t n_saved,
                           const uint32_t* seed, size_t n_seed, size_t cap = MAX_ROWS) {
        std::vector<uint32_t> ids;
        std::vector<float> score;
        std::vector<char> have(vocab, 0);
        bool fits = saved && saved_score && n_saved <= MAX_ROWS;
        for (size_t i = 0; fits && i < n_saved; i++) {
            if (saved[i] >= vocab || have[saved[i]]) fits = false;
            else have[saved[i]] = 1;
        }
        if (fits) {
            ids.assign(saved, saved + n_saved);
            score.assign(saved_score, saved_score + n_saved);
        } else {
            std::fill(have.begin(), have.end(), 0);
        }
        for (size_t i = 0; i < n_seed; i++) {
            const uint32_t t = seed[i];
            if (t >= vocab) return nullptr;
            if (ids.size() < MAX_ROWS && !have[t]) {
                have[t] = 1;
                ids.push_back(t);
                score.push_back(0.f);
            }
        }
        const size_t whole = ids.size() / 16 * 16;
        ids.resize(whole);
        score.resize(whole);
        if (ids.empty()) return nullptr;
        DraftRows* r = new DraftRows(vocab, std::move(ids), std::move(score), cap);
        if (!r->ok()) { delete r; return nullptr; }
        return r;
    }

    bool ok() const { return ok_; }
    const std::vector<uint32_t>& ids() const { return ids_; }
    const std::vector<float>& score() const { return score_; }
    size_t vocab() const { return row_of_.size(); }
    size_t cap() const { return cap_; }
    size_t pending() const { return pending_.size(); }
    size_t since() const { return since_; }
    bool dirty() const { return dirty_; }
    void saved() { dirty_ = false; }
    // the row of a token, NONE without one
    uint32_t row_of(uint32_t t) const { return t < row_of_.size() ? row_of_[t] : NONE; }
    bool waiting(uint32_t t) const { return t < waiting_.size() && waiting_[t]; }

    // Whether take(toks) can change a tile: most steps only count and need no snapshot to roll back to
    // (draft_vocab.rs:57-68). Repeats count once; a token that waits already, has a row or lies beyond the vocabulary
    // is no new one.
    bool may_change(const uint32_t* toks, size_t n) const {
        std::vector<uint32_t> fresh;
        for (size_t i = 0; i < n; i++) {
            const uint32_t t = toks[i];
            if (t < row_of_.size() && row_of_[t] == NONE && !waiting_[t] &&
                std::find(fresh.begin(), fresh.end(), t) == fresh.end()) {
                fresh.push_back(t);
                if (pending_.size() + fresh.size() >= 16) return true;
            }
        }
        return false;
    }

    // Take in committed tokens; the tiles (of 16 rows) whose tokens changed, ascending (draft_vocab.rs:71-119)
    std::vector<int> take(const uint32_t* toks, size_t n) {
        for (size_t i = 0; i < n; i++) {
            const uint32_t t = toks[i];
            if (t >= row_of_.size()) continue;
            if (row_of_[t] != NONE) score_[row_of_[t]] += 1.f;
            else if (!waiting_[t]) {
                waiting_[t] = 1;
                pending_.push_back(t);
            }
        }
        since_ += n;
        if (since_ >= DECAY) {
            since_ = 0;
            for (float& s : score_) s *= 0.5f;
        }
        const size_t whole = pending_.size() / 16 * 16;
        std::vector<int> tiles;
        if (whole == 0) return tiles;
        const std::vector<uint32_t> fresh(pending_.begin(), pending_.begin() + whole);
        pending_.erase(pending_.begin(), pending_.begin() + whole);
        for (uint32_t t : fresh) waiting_[t] = 0;
        // new tiles while there is room ...
        const size_t room = std::min(cap_ - ids_.size(), whole);
        for (size_t tile = ids_.size() / 16; tile < (ids_.size() + room) / 16; tile++) tiles.push_back((int)tile);
        for (size_t i = 0; i < room; i++) {
            row_of_[fresh[i]] = (uint32_t)ids_.size();
            ids_.push_back(fresh[i]);
            score_.push_back(1.f);
        }
        // ... then the coldest rows, as many as there are; new tokens beyond those get no row (they may come again)
        std::vector<size_t> cold;
        for (size_t r = 0; r < ids_.size(); r++)
            if (score_[r] < 1.f) cold.push_back(r);
        const size_t k = std::min(whole - room, cold.size());
        if (k == 0) return tiles;
        // (among equal scores the lower rows go first: the reference's selection leaves that order open)
        std::stable_sort(cold.begin(), cold.end(), [&](size_t a, size_t b) { return score_[a] < score_[b]; });
        for (size_t i = 0; i < k; i++) {
            const size_t r = cold[i];
            const uint32_t t = fresh[room + i];
            row_of_[ids_[r]] = NONE;
            ids_[r] = t;
            score_[r] = 1.f;
            row_of_[t] = (uint32_t)r;
            tiles.push_back((int)(r / 16));
        }
        std::sort(tiles.begin(), tiles.end());
        tiles.erase(std::unique(tiles.begin(), tiles.end()), tiles.end());
        return tiles;
    }

    // Take in the tokens a step commits. When tiles change, publish(ids, tiles) puts them into the head; if it fails
    // (returns non-zero) the rows are as before and its code is returned (Adaptive::learn, draft_vocab.rs:185-201).
    // *changed (optional): the number of tiles published.
    int learn(const uint32_t* toks, size_t n,
              const std::function<int(const std::vector<uint32_t>&, const std::vector<int>&)>& publish, int* changed) {
        if (changed) *changed = 0;
        const bool snapshot = may_change(toks, n);
        Snapshot before;
        if (snapshot) before = {ids_, score_, row_of_, pending_, waiting_, since_};
        const std::vector<int> tiles = take(toks, n);
        if (tiles.empty()) return 0;
        if (const int rc = publish(ids_, tiles)) {
            if (snapshot) {  // (a change of tiles has its snapshot)
                ids_ = std::move(before.ids); score_ = std::move(before.score); row_of_ = std::move(before.row_of);
                pending_ = std::move(before.pending); waiting_ = std::move(before.waiting); since_ = before.since;
            }
            return rc;
        }
        dirty_ = true;
        if (changed) *changed = (int)tiles.size();
        return 0;
    }

  private:
    struct Snapshot {
        std::vector<uint32_t> ids;
        std::vector<float> score;
        std::vector<uint32_t> row_of, pending;
        std::vector<char> waiting;
        size_t since = 0;
    };
    std::vector<uint32_t> ids_;     // the token of each row
    std::vector<float> score_;      // the score of each row
    std::vector<uint32_t> row_of_;  // per vocabulary id: its row, or NONE
    std::vector<uint32_t> pending_; // ids without a row in the order they came
    std::vector<char> waiting_;     // which ids are in `pending_`
    size_t since_ = 0;              // committed tokens since the last halving
    size_t cap_;
    bool ok_ = false, dirty_ = false;
};

// The token ids of a draft vocabulary file (mtp_draft_vocab_ids.pt: a PyTorch int64 tensor, i.e. a zip archive whose
// stored entry */data/0 holds the values), repeats dropped (draft_ids, draft_vocab.rs:231-268). Returns 0 and the ids,
// 1: not a zip archive (or a truncated one), 2: no tensor data, 3: the entry is compressed or no whole int64s,
// 4: a token id beyond the vocabulary.
inline int draft_ids_from_pt(const uint8_t* b, size_t len, size_t vocab, std::vector<uint32_t>* ids) {
    bool bad = false;
    auto at = [&](size_t o, size_t n) -> size_t {  // little-endian field
        if (o + n > len || o + n < o) { bad = true; return 0; }
        size_t v = 0;
        for (size_t i = n; i-- > 0;) v = v << 8 | b[o + i];
        return v;
    };
    // the end of central directory record (no archive comment), then the central directory's entries
    if (len < 22) return 1;
    const size_t end = len - 22;
    if (!(b[end] == 'P' && b[end + 1] == 'K' && b[end + 2] == 5 && b[end + 3] == 6)) return 1;
    size_t c = at(end + 16, 4);
    const size_t entries = at(end + 10, 2);
    static const char tail[] = "/data/0";
    for (size_t e = 0; e < entries; e++) {
        const size_t method = at(c + 10, 2), size = at(c + 20, 4), nl = at(c + 28, 2), el = at(c + 30, 2),
                     cl = at(c + 32, 2), off = at(c + 42, 4);
        if (bad) return 1;
        const bool named = nl >= 7 && c + 46 + nl <= len && std::equal(tail, tail + 7, b + c + 46 + nl - 7);
        if (named) {
            if (method != 0 || size % 8) return 3;
            const size_t data = off + 30 + at(off + 26, 2) + at(off + 28, 2);
            if (bad || data + size > len || data + size < data) return 1;
            std::vector<char> seen(vocab, 0);
            ids->clear();
            for (size_t i = 0; i < size; i += 8) {
                uint64_t u = 0;
                for (int j = 7; j >= 0; j--) u = u << 8 | b[data + i + j];
                if (u >= vocab) return 4;  // (a negative id is a huge unsigned one)
                if (!seen[u]) {
                    seen[u] = 1;
                    ids->push_back((uint32_t)u);
                }
            }
            return 0;
        }
        c += 46 + nl + el + cl;
    }
    return bad ? 1 : 2;
}

}  // namespace qb
