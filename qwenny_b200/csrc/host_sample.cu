// The sampler's rows on the host: the reference hands a row with more candidates than its GPU kernel sorts (top_k 0,
// the whole vocabulary, or above 1024) to sample::sample_row / sample_row_q (src/sample.rs:88-211) through
// Step::sample_on_host (src/cuda/core.rs:1007-1032). qb_sample_rows marks the same rows (out_acc -1); this is their
// host side: float32 arithmetic in the host definition's order (a sequential prefix sum over the ranked tokens).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <vector>

#include "../../include/qwenny_b200.h"

namespace {

inline uint32_t okey(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Sets {
    const unsigned *seen, *outs;
    const int* step;
    int nstep;
    bool in_step(int t) const {
        for (int i = 0; i < nstep; i++)
            if (step[i] == t) return true;
        return false;
    }
    bool has(const unsigned* set, int t) const { return (set && ((set[t >> 5] >> (t & 31)) & 1)) || in_step(t); }
};

// The penalised logits and the top k tokens by value, ties to the lower index (k 0: all of them), src/sample.rs:88-115
void ranked(const float* logits, int n, const Sets& s, const float* row, int k, std::vector<float>& vals,
            std::vector<int>& idx) {
    const float rep = row[3], pres = row[7];
    vals.assign(logits, logits + n);
    if (rep != 1.f || pres != 0.f) {
        // the sets' members only: walk the words, then the step's tokens
        std::vector<int> touched;
        auto walk = [&](const unsigned* set) {
            if (!set) return;
            for (int w = 0; w < (n + 31) / 32; w++)
                for (unsigned b = set[w]; b; b &= b - 1) {
                    const int t = w * 32 + __builtin_ctz(b);
                    if (t < n) touched.push_back(t);
                }
        };
        if (rep != 1.f) walk(s.seen);
        if (pres != 0.f) walk(s.outs);
        for (int i = 0; i < s.nstep; i++)
            if (s.step[i] >= 0 && s.step[i] < n) touched.push_back(s.step[i]);
        std::sort(touched.begin(), touched.end());
        touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
        for (int t : touched) {
            float v = vals[t];
            if (rep != 1.f && s.has(s.seen, t)) v = v > 0.f ? v / rep : v * rep;
            if (pres != 0.f && s.has(s.outs, t)) v -= pres;
            vals[t] = v;
        }
    }
    k = k > 0 ? std::min(k, n) : n;
    if (k == n && n > 4096) {
        // the whole vocabulary in order: a stable radix sort of the inverted keys (ascending ~key = descending value;
        // stable = equal values keep their index order), three passes of 11 bits
        std::vector<uint32_t> key(n), key2(n);
        std::vector<int> id(n), id2(n);
        for (int i = 0; i < n; i++) { key[i] = ~okey(vals[i]); id[i] = i; }
        for (int shift = 0; shift < 33; shift += 11) {
            size_t count[2049] = {0};
            for (int i = 0; i < n; i++) count[((key[i] >> shift) & 2047) + 1]++;
            for (int b = 0; b < 2048; b++) count[b + 1] += count[b];
            for (int i = 0; i < n; i++) {
                const size_t at = count[(key[i] >> shift) & 2047]++;
                key2[at] = key[i];
                id2[at] = id[i];
            }
            key.swap(key2);
            id.swap(id2);
        }
        idx.swap(id);
        return;
    }
    std::vector<uint64_t> keys(n);
    for (int i = 0; i < n; i++) keys[i] = ((uint64_t)okey(vals[i]) << 32) | (0xffffffffu - (uint32_t)i);
    if (k < n) std::nth_element(keys.begin(), keys.begin() + (k - 1), keys.end(), std::greater<uint64_t>());
    keys.resize(k);
    std::sort(keys.begin(), keys.end(), std::greater<uint64_t>());
    idx.resize(k);
    for (int i = 0; i < k; i++) idx[i] = (int)(0xffffffffu - (uint32_t)keys[i]);
}

// Softmax of the ranked tokens at the temperature, its prefix, the top-p cut (src/sample.rs:119-135)
int kept(const std::vector<float>& vals, const std::vector<int>& idx, float temp, float top_p, std::vector<float>& p,
         std::vector<float>& cum) {
    const int n = (int)idx.size();
    const float vmax = vals[idx[0]];
    p.resize(n);
    cum.resize(n);
    float c = 0.f;
    for (int i = 0; i < n; i++) {
        p[i] = std::exp((vals[idx[i]] - vmax) / temp);
        c += p[i];
        cum[i] = c;
    }
    const float total = cum[n - 1];
    if (top_p < 1.f)
        for (int i = 0; i < n; i++)
            if (cum[i] / total >= top_p) return i + 1;
    return n;
}

}  // namespace

extern "C" int qb_host_sample_row(const float* logits, int n, const unsigned* seen, const unsigned* outs,
                                  const int* step, int nstep, const float* row_in, const int* q_ids, const float* q_p,
                                  int nq, int* tok, int* acc) {
    if (!logits || n <= 0 || !row_in || !tok || !acc || nstep < 0 || (nstep && !step)) return QB_ERR_ARG;
    float row[8];
    std::copy(row_in, row_in + 8, row);
    bool from_q = false;
    if (row[6] <= -2.f) {  // a sampled draft; without its stored distribution it counts as a draft of the argmax
        row[6] = -row[6] - 2.f;
        from_q = nq > 0 && q_ids && q_p;
    }
    const Sets s = {seen, outs, step, nstep};
    const float temp = row[0], top_p = row[2], u1 = row[4], u2 = row[5];
    const int top_k = (int)row[1];
    const bool has_draft = row[6] >= 0.f;
    const int d = has_draft ? (int)row[6] : -1;
    std::vector<float> vals, p, cum;
    std::vector<int> idx;
    if (from_q) {
        // src/sample.rs:177-200: accepted with min(1, p(d) / q(d)), else a draw from max(0, p - q) normalised
        ranked(logits, n, s, row, top_k, vals, idx);
        const int keep = kept(vals, idx, temp, top_p, p, cum);
        const float mass = cum[keep - 1];
        auto qof = [&](int t) {
            const int* e = std::lower_bound(q_ids, q_ids + nq, t);
            return e != q_ids + nq && *e == t ? q_p[e - q_ids] : 0.f;
        };
        float pd = 0.f;
        for (int i = 0; i < keep; i++) {
            p[i] = p[i] / mass;
            if (idx[i] == d) pd = p[i];
        }
        if (u1 * qof(d) < pd) { *tok = d; *acc = 1; return QB_OK; }
        std::vector<float> r(keep), cr(keep);
        float c = 0.f;
        for (int i = 0; i < keep; i++) {
            r[i] = std::max(p[i] - qof(idx[i]), 0.f);
            c += r[i];
            cr[i] = c;
        }
        *acc = 0;
        if (!(c > 0.f)) { *tok = idx[0]; return QB_OK; }
        const float target = u2 * c;
        int at = -1;
        for (int i = 0; i < keep && at < 0; i++)
            if (r[i] > 0.f && cr[i] >= target) at = i;
        for (int i = keep - 1; i >= 0 && at < 0; i--)
            if (r[i] > 0.f) at = i;
        *tok = idx[std::max(at, 0)];
        return QB_OK;
    }
    // src/sample.rs:141-172
    const bool greedy = temp <= 0.f || top_k == 1;
    ranked(logits, n, s, row, greedy ? 1 : top_k, vals, idx);
    if (greedy) { *tok = idx[0]; *acc = has_draft && d == idx[0]; return QB_OK; }
    const int keep = kept(vals, idx, temp, top_p, p, cum);
    const float mass = cum[keep - 1];
    int at_d = -1;
    if (has_draft)
        for (int i = 0; i < keep && at_d < 0; i++)
            if (idx[i] == d) at_d = i;
    const float pd = at_d >= 0 ? p[at_d] / mass : 0.f;
    if (has_draft && u1 < pd) { *tok = d; *acc = 1; return QB_OK; }
    const float target = has_draft ? u2 * (mass - pd * mass) : u1 * mass;
    int r = -1;
    for (int i = 0; i < keep && r < 0; i++)
        if (i != at_d && cum[i] - (at_d >= 0 && i >= at_d ? pd * mass : 0.f) >= target) r = i;
    if (r < 0) r = keep - 1;
    if (r == at_d) r = r + 1 < keep ? r + 1 : std::max(r - 1, 0);
    *tok = idx[r];
    *acc = 0;
    return QB_OK;
}
