// Host side of a decode / verify step: what the reference's Rust host does around its kernels, restated in C++ for
// this path only.
//   qb_model_create / set_layer / set_head   the layer stack's pointers and the step buffers
//                                            (Stack::load, Bufs: src/cuda/qwen/mod.rs:286-419)
//   qb_model_step                            Model::step (src/cuda/qwen/mod.rs:1125-1143): Step::upload
//                                            (src/cuda/core.rs:835-926), then Graphs::run (:1151-1192) of launch_step
//                                            (src/cuda/qwen/mod.rs:744-766): the step's kernels captured once per
//                                            step shape into a CUDA graph and replayed
//   qb_model_argmax                          Engine::argmax (src/cuda/core.rs:1100-1103): the greedy tokens
// Weights and per-slot caches belong to the caller (device pointers that stay valid for the model's life, as the
// reference's fixed-address regions do); activations and step arrays are allocated here once.
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>
#include "common.cuh"
#include "ctx.h"
#include "graphs.h"
#include "session.h"
#include "step_arrays.h"

using namespace qb;
using namespace qb::step;  // the step's limits (MAX_TOK, MAX_OUT, ...), its array layout and the builder of the arrays

namespace {

static_assert(PTILE == 64 / GROUP, "a prompt tile is 64 rows of (token, query head of a kv head)");
constexpr int GRAPH_TOK = 32;                   // steps of up to this many tokens are replayed as graphs (core.rs:27)
constexpr int PAIRS = 64 * 128;                 // (decode token, split) pairs of the partial buffers (attn.rs:29)

struct Layer {
    qb_layer w;
    bool set = false;
    bool has_lora = false;
    qb_lora_layer lora = {};
};

struct GraphKey {
    int v[10];
    bool operator<(const GraphKey& o) const { return std::memcmp(v, o.v, sizeof v) < 0; }
};

// a captured step and its kernel count
struct StepGraph {
    cudaGraphExec_t ex = nullptr;
    int kernels = 0;
};

// device memory outside the cache pool that the graphs leave free (GRAPH_FLOOR, src/cuda/core.rs:1108)
constexpr size_t GRAPH_FLOOR = (size_t)128 << 20;

}  // namespace

struct qb_model {
    qb_ctx* ctx = nullptr;
    int nlayers = 0, slots = 0, max_ctx = 0, vocab_rows = 0, vocab_valid = 0;
    std::vector<Layer> layers;
    const void* embed = nullptr;
    const float* final_norm = nullptr;
    const void *lm_w = nullptr, *lm_s = nullptr;
    // activations (Bufs)
    float *h = nullptr, *part = nullptr, *ba = nullptr, *o = nullptr, *cv = nullptr, *q = nullptr, *ml = nullptr,
          *acc = nullptr, *logits = nullptr;
    __half *xn = nullptr, *mix = nullptr, *mid = nullptr;
    unsigned long long* keys = nullptr;
    unsigned* seen = nullptr;
    // step arrays (Step), one device allocation and one pinned host mirror: a single copy per step
    int *d_step = nullptr, *h_step = nullptr;
    // two pinned mirrors in turn, each guarded by an event recorded after its copy: a caller may queue step after step
    // without waiting, and a mirror is rewritten only once the copy that read it has run
    int* h_mirror[2] = {nullptr, nullptr};
    cudaEvent_t h_event[2] = {nullptr, nullptr};
    int h_cur = 0;
    size_t step_ints = 0;
    int *ids, *tok_slot, *tok_pos, *seg_start, *seg_len, *seg_slot, *seg_pos0, *dtok, *dseg, *dkeys, *ptile, *out_rows,
        *mark, *mark_at, *row_first;
    unsigned long long* h_keys = nullptr;  // pinned
    // host-side shape of the uploaded step
    int n = 0, n_out = 0, segs = 0, ndec = 0, ntile = 0, ndseg = 0, dmax = 0, max_seg = 0, dec_max_pos = 0,
        tile_max_pos = 0;
    // MTP draft layer (optional): stored as layers[nlayers]; fc's input, the rows of the residual stream its tokens take
    // their hidden states from, the drafts of the running chains
    bool has_mtp = false;
    qb_mtp mtp = {};
    __half* xin2 = nullptr;
    int *mtp_rows = nullptr, *draft_ids = nullptr, *dchain = nullptr, *h_chain = nullptr;
    uint32_t* blk_words = nullptr;   // staging of a learned draft-head block: words, scales, tokens
    uint16_t* blk_sc = nullptr;
    int* blk_ids = nullptr;
    // the sampler's state (Step, src/cuda/core.rs:743-756), allocated with the first call that needs it: the slots'
    // generated-token sets, the rows' parameters and results, the stored draft distributions
    unsigned* outs = nullptr;
    float *sparams = nullptr, *qp = nullptr;
    int *sampled = nullptr, *qtok = nullptr, *qn = nullptr, *qid = nullptr;
    float* h_sparams = nullptr;  // pinned [MAX_OUT][8]
    int* h_sampled = nullptr;    // pinned: tokens [MAX_OUT], accepted [MAX_OUT], then the chains [slots][QB_QD]
    // LoRA served unmerged: the slots' scales (device + host mirror), the partial sums of A x, the plain [gate; up]
    // product of adapted layers; lora_step: the uploaded step has tokens of adapter slots
    float* slot_scale = nullptr;
    std::vector<float> h_scale;
    float *lpart = nullptr, *lgu = nullptr;
    bool any_lora = false, lora_step = false;
    // saved images (session.cu): the span table (pinned + device), the staging buffer (grows on demand)
    qb::Span *h_spans = nullptr, *d_spans = nullptr;
    unsigned char* staging = nullptr;
    size_t staging_bytes = 0;
    int *d_positions = nullptr, *h_positions = nullptr;
    // the captured steps (Graphs, src/cuda/core.rs:1117-1252): least recently used out when device memory runs short
    qb::GraphCache<GraphKey, StepGraph>* graphs = nullptr;
    qb_pool* pool = nullptr;   // the cache pool whose free pages go back to the driver when memory is shorter still
    int fail_captures = 0;     // measurement / tests: the next captures report out of memory without touching the GPU
    long long graphless = 0;   // steps that ran without a graph because theirs found no memory
    bool use_graphs = true, fused = true;
    // the DeltaNet layers' small 16-bit in-projection runs on a second stream, beside the int4 one (fork / join by
    // events; inside a captured graph the two become parallel branches)
    bool fork = true;
    cudaStream_t side = nullptr;
    std::vector<cudaEvent_t> ev;  // per layer: fork, join
    std::vector<cudaEvent_t> lev;  // per layer and adapted product: fork, join of xa = A x (created with the first adapter)
    long long launches = 0;  // kernels launched (or replayed) since creation
    int step_kernels = 0;    // kernels of the last step
    int ba_kper = 1024;      // k range of a split of the DeltaNet 16-bit in-projection in the current step
};

namespace {

template <class T>
int dalloc(T** p, size_t n) {
    QB_CUDA(cudaMalloc((void**)p, n * sizeof(T)));
    QB_CUDA(cudaMemset(*p, 0, n * sizeof(T)));
    return QB_OK;
}

#define QB_TRY(x)            \
    do {                     \
        int rc_ = (x);       \
        if (rc_) return rc_; \
    } while (0)

// A layer's in-projection(s): the small 16-bit product of a DeltaNet layer, then the int4 one (whose weight prefetch
// overlaps it).
int launch_in_proj(qb_model* m, cudaStream_t st, int layer, int& k) {
    qb_ctx* c = m->ctx;
    const qb_layer& L = m->layers[layer].w;
    const int n = m->n;
    void* s = (void*)st;
    if (L.kind == QB_LAYER_DELTA) {
        const int ba_tiles = 2 * LV_HEADS / 16;
        void* sb = s;
        if (m->fork) {
            QB_CUDA(cudaEventRecord(m->ev[2 * layer], st));
            QB_CUDA(cudaStreamWaitEvent(m->side, m->ev[2 * layer], 0));
            sb = (void*)m->side;
        }
        QB_TRY(qb_gemm_f16_plain(c, sb, L.in_ba, m->xn, nullptr, H, ba_tiles, n, m->ba_kper, m->ba, 2 * LV_HEADS)); k++;
        if (m->fork) QB_CUDA(cudaEventRecord(m->ev[2 * layer + 1], m->side));
    }
    const int rows = L.kind == QB_LAYER_DELTA ? DELTA_IN : ATTN_IN;
    // (one stage of weights before the wait, the default: as 64 x 1024 tiles the in-projection gains nothing from
    // two, 4679 against 4707 us per 64-layer step; gate_up, behind the other norm, does: see launch_layer_tail)
    QB_TRY(qb_marlin_gemm(c, s, m->xn, L.in_proj_w, m->part, L.in_proj_s, n, rows, H, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
    return QB_OK;
}

// A layer's mixer: m->part (+ m->ba) -> m->mix (f16)
int launch_mixer(qb_model* m, cudaStream_t st, int layer, int& k) {
    qb_ctx* c = m->ctx;
    const qb_layer& L = m->layers[layer].w;
    const int n = m->n;
    void* s = (void*)st;
    if (L.kind == QB_LAYER_DELTA) {
        const int ba_splits = H / m->ba_kper;
        if (m->fork) QB_CUDA(cudaStreamWaitEvent(st, m->ev[2 * layer + 1], 0));  // the 16-bit in-projection joins
        if (m->fused && n <= CR - CONV_K + 1) {
            QB_TRY(qb_delta_mixer(c, s, m->part, 1, n, m->ba, ba_splits, L.conv_w, L.a_log, L.dt_bias, L.norm_w, L.mem,
                                  L.sst, L.meta, nullptr, m->mix, m->seg_start, m->seg_len, m->seg_slot, m->seg_pos0,
                                  m->segs)); k++;
        } else {
            QB_TRY(qb_delta_conv(c, s, m->part, 1, n, m->ba, ba_splits, L.conv_w, L.a_log, L.dt_bias, L.mem, L.sst,
                                 m->cv, m->tok_slot, m->tok_pos)); k++;
            QB_TRY(qb_delta_rule(c, s, m->part, 1, n, m->cv, L.mem, L.sst, L.meta, m->o, m->seg_start, m->seg_len,
                                 m->seg_slot, m->seg_pos0, m->segs)); k++;
            QB_TRY(qb_delta_norm(c, s, m->part, 1, n, L.norm_w, m->o, m->mix, L.meta, m->seg_len, m->seg_slot,
                                 m->seg_pos0, m->segs)); k++;
        }
    } else {
        const float qscale = 1.4426950408889634f / 16.f;  // scores in base 2, over sqrt(HD)
        QB_TRY(qb_attn_prep(c, s, m->part, 1, n, L.q_norm, L.k_norm, L.inv_freq, qscale, m->q, m->o, L.kc, L.vc, L.ks,
                            L.vs, m->tok_slot, m->tok_pos, L.cap)); k++;
        if (m->ndec > 0) {
            QB_TRY(qb_attn_decode(c, s, m->q, L.kc, L.vc, L.ks, L.vs, m->dseg, m->dtok, m->dkeys, m->tok_slot, m->tok_pos,
                                  L.cap, m->ndseg, m->ndec, m->dmax, m->dec_max_pos + 1, m->ml, m->acc, m->o, m->mix));
            k += 2;
        }
        if (m->ntile > 0) {
            QB_TRY(qb_attn_prefill(c, s, m->q, L.kc, L.vc, L.ks, L.vs, m->ptile, m->tok_slot, m->tok_pos, L.cap, m->ntile,
                                   m->tile_max_pos + 1, m->ml, m->acc, m->o, m->mix));
            k += qb_attn_tile_splits(m->ntile, m->tile_max_pos + 1) > 1 ? 2 : 1;
        }
    }
    return QB_OK;
}

// The plain form of a layer after its mixer: out_proj, residual + norm, gate_up (SwiGLU), down, residual + norm
// (Stack::layer / mlp, src/cuda/qwen/mod.rs:498-575)
int launch_layer_tail(qb_model* m, cudaStream_t st, const qb_layer& L, const float* w_next, int& k) {
    qb_ctx* c = m->ctx;
    const int n = m->n;
    void* s = (void*)st;
    QB_TRY(qb_marlin_gemm(c, s, m->mix, L.out_w, m->part, L.out_s, n, H, MIX, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
    QB_TRY(qb_add_rmsnorm(c, s, m->h, m->part, 1, n, L.post_norm, m->xn, EPS)); k++;
    // gate_up waits some 2.5 us for the norm in front of it with the memory idle: it requests TWO stages of weights
    // before that wait (measured per position in the layer, 64 layers x 5 rows: some 40 us per step over one stage;
    // three, the whole ring, is slower than one)
    c->early = 2;
    int rc = qb_marlin_gemm(c, s, m->xn, L.gate_up_w, m->mid, L.gate_up_s, n, 2 * FF, H, 0, QB_EPI_SILU, nullptr, nullptr, 0);
    c->early = 1;  // down follows gate_up directly: nothing idle to fill (4842 against 4880 us per step with two)
    if (rc == QB_OK) { k++; rc = qb_marlin_gemm(c, s, m->mid, L.down_w, m->part, L.down_s, n, H, FF, 0, QB_EPI_PLAIN, nullptr, nullptr, 0); }
    c->early = 1;
    QB_TRY(rc); k++;
    QB_TRY(qb_add_rmsnorm(c, s, m->h, m->part, 1, n, w_next, m->xn, EPS)); k++;
    return QB_OK;
}

// xa = A x of a stacked product's adapter into m->lpart (split-K partial sums [split][n][M]); the split count
int lora_xa(qb_model* m, void* s, const qb_lora_prod& p, const void* x, int cols, int* split, int& k) {
    *split = (cols + 1023) / 1024;
    QB_TRY(qb_gemm_f16_plain(m->ctx, s, p.a, x, nullptr, cols, p.a_tiles, m->n, 1024, m->lpart, p.a_tiles * 16)); k++;
    return QB_OK;
}

// A layer with a LoRA in a step with adapter tokens (Stack::mix / mlp with `lo`, src/cuda/qwen/mod.rs:521-575): every
// adapted product is followed by xa = A x and the delta's kernel; [gate; up] runs plain and lora_silu applies SwiGLU.
int launch_layer_lora(qb_model* m, cudaStream_t st, int layer, const float* w_next, int& k) {
    qb_ctx* c = m->ctx;
    const qb_layer& L = m->layers[layer].w;
    const qb_lora_layer& A = m->layers[layer].lora;
    const int n = m->n, R = A.rank;
    void* s = (void*)st;
    int split = 0;
    // xa = A x reads the same input as the base product it accompanies: with the second stream it runs beside that
    // product (a parallel branch of the step's graph) and only the delta's kernel stays on the critical path.
    // `e`: the product's index in the layer (its pair of events); `forked`: the second stream already waits for the
    // input (the DeltaNet 16-bit in-projection's fork)
    auto xa_beside = [&](int e, const qb_lora_prod& P, const void* x, int cols, bool forked) -> int {
        if (!m->fork) return lora_xa(m, s, P, x, cols, &split, k);
        cudaEvent_t* ev = &m->lev[8 * layer + 2 * e];
        if (!forked) {
            QB_CUDA(cudaEventRecord(ev[0], st));
            QB_CUDA(cudaStreamWaitEvent(m->side, ev[0], 0));
        }
        QB_TRY(lora_xa(m, (void*)m->side, P, x, cols, &split, k));
        QB_CUDA(cudaEventRecord(ev[1], m->side));
        return QB_OK;
    };
    auto join = [&](int e) -> int {
        if (m->fork) QB_CUDA(cudaStreamWaitEvent(st, m->lev[8 * layer + 2 * e + 1], 0));
        return QB_OK;
    };
    if (A.inp.a && L.kind != QB_LAYER_DELTA) QB_TRY(xa_beside(0, A.inp, m->xn, H, false));
    QB_TRY(launch_in_proj(m, st, layer, k));
    if (A.inp.a) {
        const int rows = L.kind == QB_LAYER_DELTA ? DELTA_IN : ATTN_IN;
        if (L.kind == QB_LAYER_DELTA) QB_TRY(xa_beside(0, A.inp, m->xn, H, true));  // behind the 16-bit product there
        QB_TRY(join(0));
        if (A.inp.b) {
            QB_TRY(qb_lora_add(c, s, m->lpart, split, A.inp.a_tiles * 16, A.inp.b, rows, A.inp.tab, m->tok_slot,
                               m->slot_scale, n, m->part, rows, R)); k++;
        }
        if (A.inp.b2 && L.kind == QB_LAYER_DELTA) {
            QB_TRY(qb_lora_add(c, s, m->lpart, split, A.inp.a_tiles * 16, A.inp.b2, 2 * LV_HEADS, A.inp.tab2, m->tok_slot,
                               m->slot_scale, n, m->ba, 2 * LV_HEADS, R)); k++;
        }
    }
    QB_TRY(launch_mixer(m, st, layer, k));
    if (A.out.a) QB_TRY(xa_beside(1, A.out, m->mix, MIX, false));
    QB_TRY(qb_marlin_gemm(c, s, m->mix, L.out_w, m->part, L.out_s, n, H, MIX, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
    if (A.out.a) {
        QB_TRY(join(1));
        QB_TRY(qb_lora_add(c, s, m->lpart, split, A.out.a_tiles * 16, A.out.b, H, A.out.tab, m->tok_slot, m->slot_scale, n,
                           m->part, H, R)); k++;
    }
    QB_TRY(qb_add_rmsnorm(c, s, m->h, m->part, 1, n, L.post_norm, m->xn, EPS)); k++;
    if (A.gate_up.a) {
        QB_TRY(xa_beside(2, A.gate_up, m->xn, H, false));
        QB_TRY(qb_marlin_gemm(c, s, m->xn, L.gate_up_w, m->lgu, L.gate_up_s, n, 2 * FF, H, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
        QB_TRY(join(2));
        QB_TRY(qb_lora_silu(c, s, m->lpart, split, A.gate_up.a_tiles * 16, A.gate_up.b, 2 * FF, A.gate_up.tab, m->tok_slot,
                            m->slot_scale, n, m->lgu, 2 * FF, m->mid, R)); k++;
    } else {
        QB_TRY(qb_marlin_gemm(c, s, m->xn, L.gate_up_w, m->mid, L.gate_up_s, n, 2 * FF, H, 0, QB_EPI_SILU, nullptr, nullptr, 0)); k++;
    }
    if (A.down.a) QB_TRY(xa_beside(3, A.down, m->mid, FF, false));
    QB_TRY(qb_marlin_gemm(c, s, m->mid, L.down_w, m->part, L.down_s, n, H, FF, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
    if (A.down.a) {
        QB_TRY(join(3));
        QB_TRY(qb_lora_add(c, s, m->lpart, split, A.down.a_tiles * 16, A.down.b, H, A.down.tab, m->tok_slot, m->slot_scale,
                           n, m->part, H, R)); k++;
    }
    QB_TRY(qb_add_rmsnorm(c, s, m->h, m->part, 1, n, w_next, m->xn, EPS)); k++;
    return QB_OK;
}

// The kernels of one MTP step over the uploaded tokens (launch_mtp, src/cuda/qwen/mod.rs:799-840): the tokens'
// embeddings and their hidden states at mtp_rows of the residual stream (the target's with its final norm, or, `own`,
// the MTP layer's of the step before with the MTP's norm) through mtp_in, fc, the MTP's decoder layer, and the draft
// head (or the output layer) with the argmax epilogue. fc writes the MTP's residual stream in place of the
// reference's product + sum_parts (one split).
int launch_mtp(qb_model* m, cudaStream_t st, bool own) {
    qb_ctx* c = m->ctx;
    const int n = m->n;
    int k = 0;
    void* s = (void*)st;
    const qb_mtp& M = m->mtp;
    const qb_layer& L = m->layers[m->nlayers].w;
    m->ba_kper = 1024;
    QB_TRY(qb_embed(c, s, m->embed, m->ids, m->o, m->keys, m->n_out, n)); k++;
    QB_TRY(qb_mtp_in(c, s, m->o, m->h, m->mtp_rows, own ? M.norm : m->final_norm, M.pre_e, M.pre_h, m->xin2, EPS, n)); k++;
    QB_TRY(qb_marlin_gemm(c, s, m->xin2, M.fc_w, m->h, M.fc_s, n, H, 2 * H, 0, QB_EPI_PLAIN, nullptr, nullptr, 0)); k++;
    QB_TRY(qb_rmsnorm(c, s, m->h, L.input_norm, m->xn, EPS, n)); k++;
    QB_TRY(launch_in_proj(m, st, m->nlayers, k));
    QB_TRY(launch_mixer(m, st, m->nlayers, k));
    QB_TRY(launch_layer_tail(m, st, L, M.norm, k));
    if (m->n_out > 0) {
        const bool head = M.head_w != nullptr;
        auto product = head && M.head_zero_points ? qb_marlin_gemm_z : qb_marlin_gemm;
        QB_TRY(product(c, s, m->xn, head ? M.head_w : m->lm_w, m->logits, head ? M.head_s : m->lm_s, m->n_out,
                       head ? M.head_rows : m->vocab_rows, H, 0, QB_EPI_ARGMAX, m->out_rows, m->keys,
                       head ? M.head_valid : m->vocab_valid)); k++;
    }
    m->step_kernels = k;
    return QB_OK;
}

// The kernels of one step over the uploaded tokens, in the reference's order (launch_step).
int launch_step(qb_model* m, cudaStream_t st) {
    qb_ctx* c = m->ctx;
    const int n = m->n;
    int k = 0;
    void* s = (void*)st;
    // the reference splits the small 16-bit product 40 ways (split_for); 5 splits of 1024 columns leave its consumers
    // 8x fewer partial sums to add
    m->ba_kper = m->fused || n > 32 ? 1024 : H / qb_split_for(2 * LV_HEADS / 16, H, 16, 1024 * 8 / (n <= 8 ? 8 : n <= 16 ? 16 : 32));
    QB_TRY(qb_mark_seen(c, s, m->seen, m->mark, m->mark_at, m->seg_slot, m->seg_pos0, m->segs, m->vocab_rows)); k++;
    QB_TRY(qb_embed(c, s, m->embed, m->ids, m->h, m->keys, m->n_out, n)); k++;
    QB_TRY(qb_rmsnorm(c, s, m->h, m->layers[0].w.input_norm, m->xn, EPS, n)); k++;
    for (int i = 0; i < m->nlayers; i++) {
        const qb_layer& L = m->layers[i].w;
        const float* w_next = i + 1 < m->nlayers ? m->layers[i + 1].w.input_norm : m->final_norm;
        if (m->lora_step && m->layers[i].has_lora) {
            QB_TRY(launch_layer_lora(m, st, i, w_next, k));
            continue;
        }
        QB_TRY(launch_in_proj(m, st, i, k));
        QB_TRY(launch_mixer(m, st, i, k));
        QB_TRY(launch_layer_tail(m, st, L, w_next, k));
    }
    if (m->n_out > 0) {
        QB_TRY(qb_marlin_gemm(c, s, m->xn, m->lm_w, m->logits, m->lm_s, m->n_out, m->vocab_rows, H, 0, QB_EPI_ARGMAX,
                              m->out_rows, m->keys, m->vocab_valid)); k++;
    }
    m->step_kernels = k;
    return QB_OK;
}

}  // namespace

extern "C" {

int qb_model_create(qb_ctx* ctx, int nlayers, int slots, int max_ctx, int vocab_rows, int vocab_valid,
                    qb_model** out) {
    if (!ctx || !out || nlayers <= 0 || slots <= 0 || max_ctx <= 0 || vocab_rows % 256 || vocab_valid > vocab_rows ||
        vocab_valid <= 0)
        return QB_ERR_ARG;
    QB_CUDA(cudaSetDevice(ctx->device));
    qb_model* m = new qb_model();
    m->ctx = ctx; m->nlayers = nlayers; m->slots = slots; m->max_ctx = max_ctx;
    m->vocab_rows = vocab_rows; m->vocab_valid = vocab_valid;
    m->layers.resize(nlayers + 1);  // + the MTP layer's place
    {
        qb::GraphCache<GraphKey, StepGraph>::Hooks hk;
        hk.free_mem = []() -> size_t {
            size_t fr = 0, tot = 0;
            return cudaMemGetInfo(&fr, &tot) == cudaSuccess ? fr : (size_t)-1;
        };
        hk.destroy = [](StepGraph& g) { if (g.ex) cudaGraphExecDestroy(g.ex); g.ex = nullptr; };
        hk.sync = []() { cudaDeviceSynchronize(); };
        hk.release = [m](size_t bytes) -> size_t {
            if (!m->pool) return 0;
            size_t page = qb_pool_page(m->pool), given = 0;
            if (page) qb_pool_release(m->pool, (bytes + page - 1) / page, &given);
            return given;
        };
        m->graphs = new qb::GraphCache<GraphKey, StepGraph>(hk, GRAPH_FLOOR);
    }
    QB_CUDA(cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking));
    m->ev.resize(2 * (nlayers + 1));
    for (auto& e : m->ev) QB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    const size_t T = MAX_TOK;
    QB_TRY(dalloc(&m->h, T * H)); QB_TRY(dalloc(&m->xn, T * H));
    QB_TRY(dalloc(&m->part, T * (size_t)DELTA_IN));
    QB_TRY(dalloc(&m->ba, (size_t)40 * 32 * 2 * LV_HEADS + 5 * T * 2 * LV_HEADS));  // 40 splits of 32 rows or 5 of T
    QB_TRY(dalloc(&m->o, T * MIX)); QB_TRY(dalloc(&m->mix, T * MIX)); QB_TRY(dalloc(&m->mid, T * FF));
    QB_TRY(dalloc(&m->cv, T * CVW)); QB_TRY(dalloc(&m->q, T * NH * HD));
    QB_TRY(dalloc(&m->ml, (size_t)PAIRS * NH * 2)); QB_TRY(dalloc(&m->acc, (size_t)PAIRS * NH * HD));
    QB_TRY(dalloc(&m->logits, (size_t)MAX_OUT * vocab_rows)); QB_TRY(dalloc(&m->keys, (size_t)MAX_OUT));
    QB_TRY(dalloc(&m->seen, (size_t)slots * vocab_rows / 32));
    StepLayout L;
    m->step_ints = L.total;
    QB_TRY(dalloc(&m->d_step, L.total));
    for (int i = 0; i < 2; i++) {
        QB_CUDA(cudaMallocHost((void**)&m->h_mirror[i], L.total * sizeof(int)));
        std::memset(m->h_mirror[i], 0, L.total * sizeof(int));
        QB_CUDA(cudaEventCreateWithFlags(&m->h_event[i], cudaEventDisableTiming));
    }
    m->h_step = m->h_mirror[0];
    QB_CUDA(cudaMallocHost((void**)&m->h_keys, MAX_OUT * sizeof(unsigned long long)));
    int* d = m->d_step;
    m->ids = d + L.ids; m->tok_slot = d + L.tok_slot; m->tok_pos = d + L.tok_pos; m->seg_start = d + L.seg_start;
    m->seg_len = d + L.seg_len; m->seg_slot = d + L.seg_slot; m->seg_pos0 = d + L.seg_pos0; m->dtok = d + L.dtok;
    m->dseg = d + L.dseg; m->dkeys = d + L.dkeys; m->ptile = d + L.ptile; m->out_rows = d + L.out_rows; m->mark = d + L.mark;
    m->mark_at = d + L.mark_at;
    m->mtp_rows = d + L.mtp_rows;
    m->row_first = d + L.row_first;
    *out = m;
    return QB_OK;
}

void qb_model_destroy(qb_model* m) {
    if (!m) return;
    delete m->graphs;
    for (auto& e : m->ev) cudaEventDestroy(e);
    for (auto& e : m->lev) cudaEventDestroy(e);
    if (m->side) cudaStreamDestroy(m->side);
    if (m->h_chain) cudaFreeHost(m->h_chain);
    if (m->h_sparams) cudaFreeHost(m->h_sparams);
    if (m->h_sampled) cudaFreeHost(m->h_sampled);
    if (m->h_spans) cudaFreeHost(m->h_spans);
    if (m->h_positions) cudaFreeHost(m->h_positions);
    void* sb[] = {m->blk_words, m->blk_sc, m->blk_ids, m->outs, m->sparams, m->sampled, m->qtok, m->qn, m->qid, m->qp, m->d_spans, m->staging, m->d_positions, m->slot_scale, m->lpart, m->lgu};
    for (void* b : sb) cudaFree(b);
    void* bufs[] = {m->xin2, m->draft_ids, m->dchain, m->h, m->xn, m->part, m->ba, m->o, m->mix, m->mid, m->cv, m->q, m->ml, m->acc, m->logits, m->keys,
                    m->seen, m->d_step};
    for (void* b : bufs) cudaFree(b);
    for (int i = 0; i < 2; i++) {
        cudaFreeHost(m->h_mirror[i]);
        if (m->h_event[i]) cudaEventDestroy(m->h_event[i]);
    }
    cudaFreeHost(m->h_keys);
    delete m;
}

static int set_layer_at(qb_model* m, int i, const qb_layer* l);

int qb_model_set_layer(qb_model* m, int i, const qb_layer* l) {
    if (!m || !l || i < 0 || i >= m->nlayers) return QB_ERR_ARG;
    return set_layer_at(m, i, l);
}

// i == nlayers: the MTP layer's place
static int set_layer_at(qb_model* m, int i, const qb_layer* l) {
    if (!l->in_proj_w || !l->in_proj_s || !l->out_w || !l->out_s || !l->gate_up_w || !l->gate_up_s || !l->down_w ||
        !l->down_s || !l->input_norm || !l->post_norm)
        return QB_ERR_ARG;
    if (l->kind == QB_LAYER_DELTA) {
        if (!l->in_ba || !l->conv_w || !l->a_log || !l->dt_bias || !l->norm_w || !l->mem || !l->meta ||
            l->sst < (long long)SLOT_RING + CR * LQKV)
            return QB_ERR_ARG;
    } else if (l->kind == QB_LAYER_ATTN) {
        if (!l->q_norm || !l->k_norm || !l->inv_freq || !l->kc || !l->vc || !l->ks || !l->vs || l->cap < m->max_ctx ||
            l->cap % 64)
            return QB_ERR_ARG;
    } else {
        return QB_ERR_ARG;
    }
    m->layers[i].w = *l;
    m->layers[i].set = true;
    m->graphs->clear();  // captured steps hold the layer's old pointers
    return QB_OK;
}

int qb_model_set_head(qb_model* m, const void* embed_bf16, const float* final_norm, const void* lm_w,
                      const void* lm_s) {
    if (!m || !embed_bf16 || !final_norm || !lm_w || !lm_s) return QB_ERR_ARG;
    m->embed = embed_bf16; m->final_norm = final_norm; m->lm_w = lm_w; m->lm_s = lm_s;
    m->graphs->clear();
    return QB_OK;
}

int qb_model_use_graphs(qb_model* m, int on) {
    if (!m) return QB_ERR_ARG;
    m->use_graphs = on != 0;
    return QB_OK;
}


int qb_model_use_fork(qb_model* m, int on) {
    if (!m) return QB_ERR_ARG;
    if (m->fork != (on != 0)) {
        m->graphs->clear();
    }
    m->fork = on != 0;
    return QB_OK;
}


int qb_model_use_fused(qb_model* m, int on) {
    if (!m) return QB_ERR_ARG;
    if (m->fused != (on != 0)) {
        m->graphs->clear();
    }
    m->fused = on != 0;
    return QB_OK;
}

// Step::upload: the step's tokens (each sequence's contiguous and in order), the rows whose logits are wanted.
// Every token of a segment is added to its slot's seen set (the reference's `marks: None`).
static int upload_step(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out, const int* rows,
                       const uint32_t* marks = nullptr, const int* marks_at = nullptr);

int qb_model_upload(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out) {
    return upload_step(m, stream, toks, n, out, n_out, nullptr);
}

int qb_model_upload_marks(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out,
                          const uint32_t* marks, const int* marks_at) {
    if (!marks || !marks_at) return QB_ERR_ARG;
    return upload_step(m, stream, toks, n, out, n_out, nullptr, marks, marks_at);
}

// The arrays alone, on the host (no device, no model): what qb_model_upload would copy to the device
int qb_step_arrays(const qb_tok* toks, int n, const int* out, int n_out, const uint32_t* marks, const int* marks_at,
                   int slots, int max_ctx, int vocab_valid, int* h_arrays, long long* offsets, int* shape) {
    if (!h_arrays || !offsets || !shape) return QB_ERR_ARG;
    const StepLayout L;
    const size_t off[16] = {L.ids,  L.tok_slot, L.tok_pos, L.seg_start, L.seg_len,  L.seg_slot, L.seg_pos0, L.dtok,
                            L.dseg, L.dkeys,    L.ptile,   L.out_rows,  L.mark,     L.mark_at,  L.mtp_rows, L.row_first};
    for (int i = 0; i < 16; i++) offsets[i] = (long long)off[i];
    StepShape sh;
    QB_TRY(build_step_arrays(toks, n, out, n_out, nullptr, marks, marks_at, slots, max_ctx, vocab_valid, h_arrays, &sh));
    const int v[10] = {sh.n, sh.n_out, sh.segs, sh.ndec, sh.ntile, sh.ndseg, sh.dmax, sh.max_seg, sh.dec_max_pos, sh.tile_max_pos};
    for (int i = 0; i < 10; i++) shape[i] = v[i];
    return QB_OK;
}
int qb_step_ints(void) { return (int)StepLayout().total; }

// rows (MTP steps): per token the row of the residual stream of the step before that holds its hidden state
static int upload_step(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out, const int* rows,
                       const uint32_t* marks, const int* marks_at) {
    if (!m) return QB_ERR_ARG;
    if (!toks || n < 1 || n > MAX_TOK || n_out < 0 || n_out > MAX_OUT || (n_out && !out)) return QB_ERR_ARG;
    const int cur = m->h_cur ^ 1;
    QB_CUDA(cudaEventSynchronize(m->h_event[cur]));  // the copy that last read this mirror has run
    int* h = m->h_mirror[cur];
    StepShape sh;
    // (a step that is refused leaves the arrays and counts of the step before in place)
    QB_TRY(build_step_arrays(toks, n, out, n_out, rows, marks, marks_at, m->slots, m->max_ctx, m->vocab_valid, h, &sh));
    m->h_cur = cur;
    m->h_step = h;
    QB_CUDA(cudaMemcpyAsync(m->d_step, h, m->step_ints * sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    QB_CUDA(cudaEventRecord(m->h_event[m->h_cur], (cudaStream_t)stream));
    m->lora_step = false;
    if (m->any_lora && !rows)  // the MTP layer is not adapted (mtp_launch, src/cuda/qwen/mod.rs:933-934)
        for (int i = 0; i < n && !m->lora_step; i++) m->lora_step = m->h_scale[toks[i].slot] != 0.f;
    m->n = sh.n; m->n_out = sh.n_out; m->segs = sh.segs; m->ndec = sh.ndec; m->ntile = sh.ntile; m->ndseg = sh.ndseg;
    m->dmax = sh.dmax; m->max_seg = sh.max_seg; m->dec_max_pos = sh.dec_max_pos; m->tile_max_pos = sh.tile_max_pos;
    return QB_OK;
}

// Graphs::run: replay the step's graph, capturing it the first time its shape is seen; larger steps launch directly.
// kind: 0 the model's step, 1 an MTP step on the target's hidden states, 2 an MTP step on its own
static int run_kind(qb_model* m, void* stream, int kind) {
    if (!m || m->n <= 0 || !m->embed) return QB_ERR_ARG;
    for (int i = 0; i < m->nlayers; i++)
        if (!m->layers[i].set) return QB_ERR_ARG;
    if (kind && !m->has_mtp) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    auto launch_step = [kind](qb_model* mm, cudaStream_t s2) {
        return kind == 0 ? ::launch_step(mm, s2) : launch_mtp(mm, s2, kind == 2);
    };
    if (!m->use_graphs || m->n > GRAPH_TOK) {
        QB_TRY(launch_step(m, st));
        m->launches += m->step_kernels;
        return QB_OK;
    }
    GraphKey key = {{m->n, m->n_out, m->segs, m->ndec, m->ntile, m->max_seg,
                     (m->ndec ? qb_attn_dec_splits_sm(m->dec_max_pos + 1, m->ctx->sms) : 0) +
                         64 * (m->ntile ? qb_attn_tile_splits(m->ntile, m->tile_max_pos + 1) : 0),
                     m->ndseg, m->dmax, kind + (m->lora_step ? 4 : 0)}};
    if (StepGraph* g = m->graphs->find(key)) {
        QB_CUDA(cudaGraphLaunch(g->ex, st));
        m->step_kernels = g->kernels;
        m->launches += m->step_kernels;
        return QB_OK;
    }
    // A first run outside a capture sets the kernels' attributes (not allowed while capturing), warms the caches and
    // IS this step; the capture that follows only records. So a capture that fails costs the graph, never the step.
    QB_TRY(launch_step(m, st));
    m->launches += m->step_kernels;
    QB_CUDA(cudaStreamSynchronize(st));
    m->graphs->make_room();
    cudaError_t e = cudaSuccess;
    cudaGraphExec_t ex = nullptr;
    if (m->fail_captures > 0) {
        m->fail_captures--;
        e = cudaErrorMemoryAllocation;
    } else {
        cudaGraph_t g = nullptr;
        QB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        int rc = launch_step(m, st);
        e = cudaStreamEndCapture(st, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e == cudaSuccess) e = cudaGraphInstantiate(&ex, g, 0);
        if (g) cudaGraphDestroy(g);
    }
    if (e == cudaErrorMemoryAllocation) {
        // no memory for the graph: fewer graphs from now on, this step (already run) without one
        (void)cudaGetLastError();
        m->graphs->on_out_of_memory();
        m->graphless++;
        return QB_OK;
    }
    if (e != cudaSuccess) return (int)e;
    StepGraph sg;
    sg.ex = ex; sg.kernels = m->step_kernels;
    m->graphs->insert(key, sg);
    return QB_OK;
}

int qb_model_run(qb_model* m, void* stream) { return run_kind(m, stream, 0); }

// The MTP draft layer (Mtp, src/cuda/qwen/mod.rs:648-661): its decoder layer, fc [5120][10240], the two input norms
// and its final norm, and optionally a draft head (rows of the output layer for part of the vocabulary,
// src/cuda/qwen/draft.rs) with the token of each of its rows.
int qb_model_set_mtp(qb_model* m, const qb_mtp* mtp) {
    if (!m || !mtp || !mtp->fc_w || !mtp->fc_s || !mtp->pre_e || !mtp->pre_h || !mtp->norm) return QB_ERR_ARG;
    if (mtp->head_w && (!mtp->head_s || !mtp->head_ids || mtp->head_rows <= 0 || mtp->head_rows % 256 ||
                        mtp->head_valid <= 0 || mtp->head_valid > mtp->head_rows || mtp->head_rows > m->vocab_rows))
        return QB_ERR_ARG;
    QB_TRY(set_layer_at(m, m->nlayers, &mtp->layer));  // (drops the captured steps)
    m->mtp = *mtp;
    if (!m->xin2) {
        QB_TRY(dalloc(&m->xin2, (size_t)MAX_TOK * 2 * H));
        QB_TRY(dalloc(&m->draft_ids, (size_t)MAX_TOK));
        QB_TRY(dalloc(&m->dchain, (size_t)MAX_OUT * QB_MAX_DRAFTS));
        QB_CUDA(cudaMallocHost((void**)&m->h_chain, MAX_OUT * QB_MAX_DRAFTS * sizeof(int)));
    }
    if (mtp->head_w && !m->blk_words) {
        // the staging of a learned draft-head block (Gemm::block_stage, src/cuda/core.rs:672-676), taken once: no device
        // memory is taken while serving
        QB_TRY(dalloc(&m->blk_words, (size_t)H / 16 * 32));
        QB_TRY(dalloc(&m->blk_sc, (size_t)2 * (H / 128) * 16));
        QB_TRY(dalloc(&m->blk_ids, (size_t)16));
    }
    m->has_mtp = true;
    return QB_OK;
}

// DraftHead::learn for one 16-row block (src/cuda/qwen/draft.rs:56-72; Gemm::put_block, src/cuda/core.rs:614-671): the
// block's packed words and scales (qb_marlin_block's output, host) go through the staging buffers into rows
// 16 block .. 16 block + 15 of the draft head, its tokens into head_ids, and the rows count as valid from now on.
// *grew: the head's valid row count changed (the MTP steps' graphs carry it and were dropped).
int qb_model_learn_block(qb_model* m, void* stream, int block, const uint32_t* h_words, const uint16_t* h_sc,
                         const int* h_ids16, int* grew) {
    if (!m || !m->has_mtp || !m->mtp.head_w || !h_words || !h_sc || !h_ids16 || block < 0 ||
        (block + 1) * 16 > m->mtp.head_rows)
        return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int groups = H / 128, tables = m->mtp.head_zero_points ? 2 : 1;
    QB_CUDA(cudaMemcpyAsync(m->blk_words, h_words, (size_t)H / 16 * 32 * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    QB_CUDA(cudaMemcpyAsync(m->blk_sc, h_sc, (size_t)tables * groups * 16 * sizeof(uint16_t), cudaMemcpyHostToDevice, st));
    QB_CUDA(cudaMemcpyAsync(m->blk_ids, h_ids16, 16 * sizeof(int), cudaMemcpyHostToDevice, st));
    QB_TRY(qb_marlin_put_block(m->ctx, stream, (void*)m->mtp.head_w, (void*)m->mtp.head_s, m->blk_words, m->blk_sc,
                               m->mtp.head_rows, block / 4, block % 4, groups, tables, H / 16));
    QB_CUDA(cudaMemcpyAsync((int*)m->mtp.head_ids + 16 * block, m->blk_ids, 16 * sizeof(int), cudaMemcpyDeviceToDevice, st));
    QB_CUDA(cudaStreamSynchronize(st));  // the host buffers are the caller's again
    const int valid = m->mtp.head_valid > (block + 1) * 16 ? m->mtp.head_valid : (block + 1) * 16;
    if (grew) *grew = valid != m->mtp.head_valid;
    if (valid != m->mtp.head_valid) {
        m->mtp.head_valid = valid;
        m->graphs->retain([](const GraphKey& k) { return (k.v[9] & 3) == 0; });  // the MTP kinds are 1 and 2
    }
    return QB_OK;
}

int qb_model_set_pool(qb_model* m, qb_pool* pool) {
    if (!m) return QB_ERR_ARG;
    m->pool = pool;
    return QB_OK;
}

// graphs held now, the cap on them (-1: none yet), steps that ran without a graph for want of memory
int qb_model_graph_stats(const qb_model* m, long long* held, long long* cap, long long* graphless) {
    if (!m) return QB_ERR_ARG;
    if (held) *held = (long long)m->graphs->size();
    if (cap) *cap = m->graphs->cap() == qb::GraphCache<GraphKey, StepGraph>::NO_CAP ? -1 : (long long)m->graphs->cap();
    if (graphless) *graphless = m->graphless;
    return QB_OK;
}

// Tests: the next `n` graph captures behave as if the driver had no memory for them (nothing touches the GPU).
int qb_model_fail_captures(qb_model* m, int n) {
    if (!m || n < 0) return QB_ERR_ARG;
    m->fail_captures = n;
    return QB_OK;
}

// Engine::draft with greedy rows (draft_chains, src/cuda/qwen/mod.rs:870-896): k drafts for each of the n_out rows
// `out` of the MTP step over `toks`, whose hidden states are rows `rows` of the residual stream the last model step
// left. The first MTP step runs on the target's hidden states; each further one on the MTP's own, one position on,
// with the draft just made as its token (its id stays on the device). h_drafts: host [n_out][k]. Waits for the chain.
int qb_model_draft(qb_model* m, void* stream, const qb_tok* toks, int n, const int* rows, const int* out, int n_out,
                   int k, int* h_drafts) {
    if (!m || !m->has_mtp || !toks || !rows || n < 1 || n > MAX_TOK || n_out < 0 || n_out > MAX_OUT || k < 0 ||
        k > QB_MAX_DRAFTS || (n_out && (!out || !h_drafts)))
        return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const bool none = k == 0 || n_out == 0;
    QB_TRY(upload_step(m, stream, toks, n, out, none ? 0 : n_out, rows));
    QB_TRY(run_kind(m, stream, 1));
    if (none) return QB_OK;
    const int* head_ids = m->mtp.head_w ? m->mtp.head_ids : nullptr;
    QB_TRY(qb_draft_pick(m->ctx, stream, m->keys, head_ids, n_out, m->draft_ids, m->dchain, QB_MAX_DRAFTS, 0));
    std::vector<qb_tok> cur(n_out);
    std::vector<int> at(out, out + n_out), all(n_out);
    for (int i = 0; i < n_out; i++) { cur[i] = toks[out[i]]; all[i] = i; }
    for (int t = 1; t < k; t++) {
        for (auto& c : cur) { c.id = 0; c.pos += 1; }
        QB_TRY(upload_step(m, stream, cur.data(), n_out, all.data(), n_out, at.data()));
        // the step's token ids are the drafts just made (ids_from_drafts, src/cuda/core.rs:1077-1080)
        QB_CUDA(cudaMemcpyAsync(m->ids, m->draft_ids, n_out * sizeof(int), cudaMemcpyDeviceToDevice, st));
        QB_TRY(run_kind(m, stream, 2));
        QB_TRY(qb_draft_pick(m->ctx, stream, m->keys, head_ids, n_out, m->draft_ids, m->dchain, QB_MAX_DRAFTS, t));
        at = all;
    }
    QB_CUDA(cudaMemcpyAsync(m->h_chain, m->dchain, (size_t)n_out * QB_MAX_DRAFTS * sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    for (int i = 0; i < n_out; i++)
        for (int t = 0; t < k; t++) h_drafts[i * k + t] = m->h_chain[i * QB_MAX_DRAFTS + t];
    return QB_OK;
}

int qb_model_step(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out) {
    QB_TRY(qb_model_upload(m, stream, toks, n, out, n_out));
    return qb_model_run(m, stream);
}

// Model::step with `marks` (src/cuda/qwen/mod.rs:1125-1143): the tokens each segment adds to its slot's seen set
int qb_model_step_marks(qb_model* m, void* stream, const qb_tok* toks, int n, const int* out, int n_out,
                        const uint32_t* marks, const int* marks_at) {
    QB_TRY(qb_model_upload_marks(m, stream, toks, n, out, n_out, marks, marks_at));
    return qb_model_run(m, stream);
}

// Engine::argmax: the greedy token of each logit row of the last step (waits for the step)
int qb_model_argmax(qb_model* m, void* stream, int* h_tokens, int n_out) {
    if (!m || !h_tokens || n_out < 0 || n_out > m->n_out) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    QB_CUDA(cudaMemcpyAsync(m->h_keys, m->keys, n_out * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    for (int i = 0; i < n_out; i++) h_tokens[i] = (int)(0xffffffffu - (uint32_t)(m->h_keys[i] & 0xffffffffu));
    return QB_OK;
}

// ---- the sampler on the step's logits (Step::sample, set_outputs, draft_sample, draft_q: src/cuda/core.rs:977-1100)

static int ensure_sampler(qb_model* m) {
    if (m->outs) return QB_OK;
    const size_t q = (size_t)m->slots * QB_QD;
    QB_TRY(dalloc(&m->outs, (size_t)m->slots * m->vocab_rows / 32));
    QB_TRY(dalloc(&m->sparams, (size_t)MAX_OUT * 8));
    QB_TRY(dalloc(&m->sampled, (size_t)2 * MAX_OUT));
    QB_TRY(dalloc(&m->qtok, q)); QB_TRY(dalloc(&m->qn, q));
    QB_TRY(dalloc(&m->qid, q * QB_QCAP)); QB_TRY(dalloc(&m->qp, q * QB_QCAP));
    QB_CUDA(cudaMemset(m->qtok, 0xff, q * sizeof(int)));  // -1: no draft stored
    QB_CUDA(cudaMallocHost((void**)&m->h_sparams, (size_t)QB_MAX_DRAFTS * MAX_OUT * 8 * sizeof(float)));
    QB_CUDA(cudaMallocHost((void**)&m->h_sampled, (2 * MAX_OUT + q) * sizeof(int)));
    QB_CUDA(cudaDeviceSynchronize());
    return QB_OK;
}

// The tokens a slot's request generated so far, as a set of vocab_rows bits (the presence penalty's; host words)
int qb_model_set_outputs(qb_model* m, void* stream, int slot, const unsigned* words) {
    if (!m || !words || slot < 0 || slot >= m->slots) return QB_ERR_ARG;
    QB_TRY(ensure_sampler(m));
    const size_t w = (size_t)m->vocab_rows / 32;
    QB_CUDA(cudaMemcpyAsync(m->outs + slot * w, words, w * sizeof(unsigned), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    QB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));  // `words` is the caller's
    return QB_OK;
}

// Step::sample_on_host: row j of the last step on the host, from the logits and the sets on the device
static int sample_on_host(qb_model* m, cudaStream_t st, int j, const float* row, int* tok, int* acc) {
    StepLayout L;
    const int* h = m->h_step;
    const int rt = h[L.out_rows + j], first = h[L.row_first + j], slot = h[L.tok_slot + rt];
    const size_t w = (size_t)m->vocab_rows / 32;
    std::vector<float> logits(m->vocab_valid);
    std::vector<unsigned> seen(w), outs(w);
    std::vector<int> step(rt - first), qi;
    std::vector<float> qv;
    QB_CUDA(cudaMemcpyAsync(logits.data(), m->logits + (size_t)j * m->vocab_rows, logits.size() * sizeof(float),
                            cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaMemcpyAsync(seen.data(), m->seen + slot * w, w * sizeof(unsigned), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaMemcpyAsync(outs.data(), m->outs + slot * w, w * sizeof(unsigned), cudaMemcpyDeviceToHost, st));
    if (!step.empty())
        QB_CUDA(cudaMemcpyAsync(step.data(), m->ids + first + 1, step.size() * sizeof(int), cudaMemcpyDeviceToHost, st));
    int nq = 0;
    if (row[6] <= -2.f && rt - first < QB_QD) {
        const int q = slot * QB_QD + (rt - first);
        int head[2] = {0, 0};
        QB_CUDA(cudaMemcpyAsync(&head[0], m->qtok + q, sizeof(int), cudaMemcpyDeviceToHost, st));
        QB_CUDA(cudaMemcpyAsync(&head[1], m->qn + q, sizeof(int), cudaMemcpyDeviceToHost, st));
        QB_CUDA(cudaStreamSynchronize(st));
        if (head[0] == (int)(-row[6] - 2.f) && head[1] > 0) {
            nq = head[1];
            qi.resize(nq); qv.resize(nq);
            QB_CUDA(cudaMemcpyAsync(qi.data(), m->qid + (size_t)q * QB_QCAP, nq * sizeof(int), cudaMemcpyDeviceToHost, st));
            QB_CUDA(cudaMemcpyAsync(qv.data(), m->qp + (size_t)q * QB_QCAP, nq * sizeof(float), cudaMemcpyDeviceToHost, st));
        }
    }
    QB_CUDA(cudaStreamSynchronize(st));
    return qb_host_sample_row(logits.data(), m->vocab_valid, seen.data(), outs.data(), step.data(), (int)step.size(), row,
                              qi.data(), qv.data(), nq, tok, acc);
}

// Step::sample: the next token of each logit row of the last step under the rows' parameters (host [n_out][8], see
// qb_sample_rows), on the device; rows with more candidates than the kernel sorts on the host, from the same state.
// h_tok / h_acc: host [n_out]. Waits for the step.
int qb_model_sample(qb_model* m, void* stream, const float* params, int n_out, int* h_tok, int* h_acc) {
    if (!m || !params || !h_tok || !h_acc || n_out != m->n_out || n_out <= 0) return QB_ERR_ARG;
    QB_TRY(ensure_sampler(m));
    cudaStream_t st = (cudaStream_t)stream;
    std::memcpy(m->h_sparams, params, (size_t)n_out * 8 * sizeof(float));
    QB_CUDA(cudaMemcpyAsync(m->sparams, m->h_sparams, (size_t)n_out * 8 * sizeof(float), cudaMemcpyHostToDevice, st));
    QB_TRY(qb_sample_rows(m->ctx, stream, m->logits, m->vocab_valid, m->vocab_rows, m->vocab_rows, n_out, m->out_rows,
                          m->tok_slot, m->ids, m->row_first, m->seen, m->outs, m->sparams, m->qtok, m->qn, m->qid, m->qp,
                          m->sampled, m->sampled + MAX_OUT));
    m->launches++;
    QB_CUDA(cudaMemcpyAsync(m->h_sampled, m->sampled, 2 * MAX_OUT * sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    for (int j = 0; j < n_out; j++) {
        h_tok[j] = m->h_sampled[j];
        h_acc[j] = m->h_sampled[MAX_OUT + j];
        if (h_acc[j] < 0) QB_TRY(sample_on_host(m, st, j, params + 8 * j, &h_tok[j], &h_acc[j]));
    }
    return QB_OK;
}

// Engine::draft with sampled rows (draft_chains + launch_drafts, src/cuda/qwen/mod.rs:866-918): as qb_model_draft,
// but every step's drafts are drawn on the device by qb_draft_sample under the rows' draft parameters (`sampling`:
// host [n_out][8] as Params::draft_row gives them; a row with temperature <= 0 takes the argmax, argmax_draft_row)
// with the draws u (host [n_out][k]); the distribution of each draft is kept for (slot, t) for the target's
// qb_model_sample rows that mark it sampled. h_drafts: host [n_out][k].
int qb_model_draft_sampled(qb_model* m, void* stream, const qb_tok* toks, int n, const int* rows, const int* out,
                           int n_out, int k, const float* sampling, const float* u, int* h_drafts) {
    if (!m || !m->has_mtp || !toks || !rows || !sampling || !u || n < 1 || n > MAX_TOK || n_out < 1 || n_out > MAX_OUT ||
        k < 1 || k > QB_MAX_DRAFTS || !out || !h_drafts)
        return QB_ERR_ARG;
    QB_TRY(ensure_sampler(m));
    cudaStream_t st = (cudaStream_t)stream;
    const bool head = m->mtp.head_w != nullptr;
    const int width = head ? m->mtp.head_valid : m->vocab_valid, ld = head ? m->mtp.head_rows : m->vocab_rows;
    auto draw = [&](int t) -> int {
        float* hp = m->h_sparams + (size_t)t * MAX_OUT * 8;  // a region per step: the copies run later
        for (int i = 0; i < n_out; i++) {
            float* r = hp + 8 * i;
            if (sampling[8 * i] > 0.f) {
                std::memcpy(r, sampling + 8 * i, 8 * sizeof(float));
                r[4] = u[i * k + t];
            } else {
                const float g[8] = {1.f, 1.f, 1.f, 1.f, 0.5f, 0.f, -1.f, 0.f};
                std::memcpy(r, g, sizeof g);
            }
            r[5] = (float)t;
        }
        QB_CUDA(cudaMemcpyAsync(m->sparams, hp, (size_t)n_out * 8 * sizeof(float), cudaMemcpyHostToDevice, st));
        QB_TRY(qb_draft_sample(m->ctx, stream, m->logits, width, ld, head ? m->mtp.head_ids : nullptr, m->vocab_rows, n_out,
                               m->out_rows, m->tok_slot, m->seen, m->outs, m->sparams, m->draft_ids, m->qtok, m->qn, m->qid,
                               m->qp));
        m->launches++;
        return QB_OK;
    };
    QB_TRY(upload_step(m, stream, toks, n, out, n_out, rows));
    QB_TRY(run_kind(m, stream, 1));
    QB_TRY(draw(0));
    std::vector<qb_tok> cur(n_out);
    std::vector<int> at(out, out + n_out), all(n_out);
    for (int i = 0; i < n_out; i++) { cur[i] = toks[out[i]]; all[i] = i; }
    for (int t = 1; t < k; t++) {
        for (auto& c : cur) { c.id = 0; c.pos += 1; }
        QB_TRY(upload_step(m, stream, cur.data(), n_out, all.data(), n_out, at.data()));
        QB_CUDA(cudaMemcpyAsync(m->ids, m->draft_ids, n_out * sizeof(int), cudaMemcpyDeviceToDevice, st));
        QB_TRY(run_kind(m, stream, 2));
        QB_TRY(draw(t));
        at = all;
    }
    int* chains = m->h_sampled + 2 * MAX_OUT;
    QB_CUDA(cudaMemcpyAsync(chains, m->qtok, (size_t)m->slots * QB_QD * sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    for (int i = 0; i < n_out; i++)
        for (int t = 0; t < k; t++) h_drafts[i * k + t] = chains[(int)toks[out[i]].slot * QB_QD + t];
    return QB_OK;
}

// Step::draft_q: the distribution kept for slot `slot`'s draft at index t and the token drawn from it; ids / p: host
// [QB_QCAP]. Waits for the stream.
int qb_model_draft_q(qb_model* m, void* stream, int slot, int t, int* tok, int* n, int* ids, float* p) {
    if (!m || slot < 0 || slot >= m->slots || t < 0 || t >= QB_QD || !tok || !n || !ids || !p) return QB_ERR_ARG;
    QB_TRY(ensure_sampler(m));
    cudaStream_t st = (cudaStream_t)stream;
    const int q = slot * QB_QD + t;
    QB_CUDA(cudaMemcpyAsync(tok, m->qtok + q, sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaMemcpyAsync(n, m->qn + q, sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    if (*n < 0 || *n > QB_QCAP) return QB_ERR_DEVICE;
    QB_CUDA(cudaMemcpyAsync(ids, m->qid + (size_t)q * QB_QCAP, *n * sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaMemcpyAsync(p, m->qp + (size_t)q * QB_QCAP, *n * sizeof(float), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    return QB_OK;
}

// ---- a LoRA adapter served unmerged

static bool lora_prod_ok(const qb_lora_prod& p, bool needs_b) {
    if (!p.a) return true;
    return p.a_tiles > 0 && p.a_tiles * 16 <= 256 && (!needs_b || (p.b && p.tab)) && (!p.b || p.tab) && (!p.b2 || p.tab2);
}

int qb_model_set_adapter(qb_model* m, int layer, const qb_lora_layer* lora) {
    if (!m || layer < 0 || layer >= m->nlayers) return QB_ERR_ARG;
    Layer& L = m->layers[layer];
    if (!lora) {
        L.has_lora = false;
    } else {
        if ((lora->rank != 8 && lora->rank != 16 && lora->rank != 32 && lora->rank != 64) || !lora_prod_ok(lora->inp, false) ||
            !lora_prod_ok(lora->out, true) || !lora_prod_ok(lora->gate_up, true) || !lora_prod_ok(lora->down, true))
            return QB_ERR_ARG;
        if (!m->lpart) {
            // A x of the widest input (17 splits of 1024 columns) and the plain [gate; up] product of a whole step
            QB_TRY(dalloc(&m->lpart, (size_t)17 * MAX_TOK * 256));
            QB_TRY(dalloc(&m->lgu, (size_t)MAX_TOK * 2 * FF));
            m->lev.resize((size_t)8 * m->nlayers);
            for (auto& e : m->lev) QB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        L.lora = *lora;
        L.has_lora = true;
    }
    m->any_lora = false;
    for (int i = 0; i < m->nlayers; i++) m->any_lora |= m->layers[i].has_lora;
    m->graphs->clear();  // captured steps hold the old adapter's pointers and the layers' adapted / plain choice
    return QB_OK;
}

int qb_model_set_slot_scale(qb_model* m, void* stream, int slot, float scale) {
    if (!m || slot < 0 || slot >= m->slots) return QB_ERR_ARG;
    if (!m->slot_scale) {
        QB_TRY(dalloc(&m->slot_scale, (size_t)m->slots));
        m->h_scale.assign(m->slots, 0.f);
        QB_CUDA(cudaDeviceSynchronize());
    }
    m->h_scale[slot] = scale;
    QB_CUDA(cudaMemcpyAsync(m->slot_scale + slot, &m->h_scale[slot], sizeof(float), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    QB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return QB_OK;
}

// ---- a slot's saved images (Model::save_kv / load_kv / save_state / load_state, src/cuda/qwen/mod.rs:993-1061)

static int all_layers(const qb_model* m) { return m->nlayers + (m->has_mtp ? 1 : 0); }
static size_t kv_layer_bytes(int from, int to) {  // Attn::saved_bytes, src/cuda/qwen/attn.rs:198-200
    const size_t n = to - from, vl = (size_t)(to + 15) / 16 * 16 - from;
    return NKV * (n * HD + vl * HD + n * 4 + n * 4);
}
static constexpr size_t DELTA_BYTES = ((size_t)SLOT_STATE + (CONV_K - 1) * LQKV) * 4;  // DeltaNet::saved_bytes

static int ensure_session(qb_model* m, size_t image) {
    const size_t cap = (size_t)(m->nlayers + 1) * 16 + 2;
    if (!m->h_spans) {
        QB_CUDA(cudaMallocHost((void**)&m->h_spans, cap * sizeof(qb::Span)));
        QB_CUDA(cudaMalloc((void**)&m->d_spans, cap * sizeof(qb::Span)));
        QB_CUDA(cudaMalloc((void**)&m->d_positions, (m->nlayers + 1) * sizeof(int)));
        QB_CUDA(cudaMallocHost((void**)&m->h_positions, (m->nlayers + 1) * sizeof(int)));
    }
    if (image > m->staging_bytes) {
        if (m->staging) QB_CUDA(cudaFree(m->staging));
        m->staging = nullptr; m->staging_bytes = 0;
        QB_CUDA(cudaMalloc((void**)&m->staging, image));
        m->staging_bytes = image;
    }
    return QB_OK;
}

static int run_spans(qb_model* m, cudaStream_t st, bool save, std::vector<qb::Span>& spans) {
    const unsigned chunks = qb::assign_chunks(spans);
    std::memcpy(m->h_spans, spans.data(), spans.size() * sizeof(qb::Span));
    QB_CUDA(cudaMemcpyAsync(m->d_spans, m->h_spans, spans.size() * sizeof(qb::Span), cudaMemcpyHostToDevice, st));
    QB_TRY(qb::launch_session_copy(m->ctx, st, save, m->d_spans, (int)spans.size(), chunks, m->staging, m->d_positions));
    m->launches++;
    return QB_OK;
}

// the attention layers' regions of positions [from, to) of a slot, in wire order (Attn::layout)
static void kv_spans(const qb_model* m, int slot, int from, int to, std::vector<qb::Span>& spans) {
    const size_t n = to - from, vl = (size_t)(to + 15) / 16 * 16 - from;
    unsigned long long off = 0;
    auto put = [&](void* base, size_t at, size_t bytes) {
        qb::Span s = {};
        s.dev = (unsigned char*)base + at; s.off = off; s.bytes = bytes; s.kind = qb::SPAN_PLAIN;
        spans.push_back(s);
        off += bytes;
    };
    for (int i = 0; i < all_layers(m); i++) {
        const qb_layer& L = m->layers[i].w;
        if (L.kind != QB_LAYER_ATTN) continue;
        for (int g = 0; g < NKV; g++) {
            const size_t p = ((size_t)slot * NKV + g) * L.cap + from;
            put(L.kc, p * HD, n * HD); put(L.vc, p * HD, vl * HD); put(L.ks, p * 4, n * 4); put(L.vs, p * 4, n * 4);
        }
    }
}

static int kv_check(const qb_model* m, int slot, int from, int to, size_t bytes, size_t* image) {
    if (!m || slot < 0 || slot >= m->slots || from < 0 || from % 16 || from > to) return QB_ERR_ARG;
    size_t total = 0;
    for (int i = 0; i < all_layers(m); i++) {
        const qb_layer& L = m->layers[i].w;
        if (L.kind != QB_LAYER_ATTN) continue;
        if (to > L.cap) return QB_ERR_ARG;
        total += kv_layer_bytes(from, to);
    }
    *image = total;
    return bytes == total ? QB_OK : QB_ERR_ARG;
}

size_t qb_model_kv_bytes(const qb_model* m, int from, int to) {
    if (!m || from < 0 || from > to) return 0;
    size_t total = 0;
    for (int i = 0; i < all_layers(m); i++)
        if (m->layers[i].w.kind == QB_LAYER_ATTN) total += kv_layer_bytes(from, to);
    return total;
}

size_t qb_model_state_bytes(const qb_model* m) {
    if (!m) return 0;
    size_t total = (size_t)m->vocab_rows / 8;  // the seen set
    for (int i = 0; i < all_layers(m); i++)
        if (m->layers[i].w.kind == QB_LAYER_DELTA) total += DELTA_BYTES;
    return total;
}

// Model::save_kv: every attention layer's cache of slot `slot` for positions [from, to) (from a multiple of 16) into
// h_out (qb_model_kv_bytes(from, to) bytes). Waits for the stream.
int qb_model_save_kv(qb_model* m, void* stream, int slot, int from, int to, void* h_out, size_t bytes) {
    size_t image = 0;
    QB_TRY(kv_check(m, slot, from, to, bytes, &image));
    if (!h_out && image) return QB_ERR_ARG;
    if (!image) return QB_OK;
    QB_TRY(ensure_session(m, image));
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<qb::Span> spans;
    kv_spans(m, slot, from, to, spans);
    QB_TRY(run_spans(m, st, true, spans));
    QB_CUDA(cudaMemcpyAsync(h_out, m->staging, image, cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    return QB_OK;
}

// Model::load_kv: an image from qb_model_save_kv for positions [from, to) into slot `slot`
int qb_model_load_kv(qb_model* m, void* stream, int slot, int from, int to, const void* h_data, size_t bytes) {
    size_t image = 0;
    QB_TRY(kv_check(m, slot, from, to, bytes, &image));
    if (!h_data && image) return QB_ERR_ARG;
    if (!image) return QB_OK;
    QB_TRY(ensure_session(m, image));
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<qb::Span> spans;
    kv_spans(m, slot, from, to, spans);
    QB_CUDA(cudaMemcpyAsync(m->staging, h_data, image, cudaMemcpyHostToDevice, st));
    QB_TRY(run_spans(m, st, false, spans));
    QB_CUDA(cudaStreamSynchronize(st));  // h_data is the caller's
    return QB_OK;
}

static void state_spans(const qb_model* m, int slot, bool save, int pos, std::vector<qb::Span>& spans, int* ndelta) {
    unsigned long long off = 0;
    int nd = 0;
    for (int i = 0; i < all_layers(m); i++) {
        const qb_layer& L = m->layers[i].w;
        if (L.kind != QB_LAYER_DELTA) continue;
        qb::Span s = {};
        s.dev = (unsigned char*)(L.mem + (size_t)slot * L.sst);
        s.meta = L.meta + slot * META;
        s.pos = pos;
        s.kind = qb::SPAN_STATE; s.off = off; s.bytes = (size_t)SLOT_STATE * 4;
        spans.push_back(s);
        off += s.bytes;
        for (int j = 0; j < CONV_K - 1; j++) {
            s.kind = qb::SPAN_RING; s.j = j; s.off = off; s.bytes = (size_t)LQKV * 4;
            spans.push_back(s);
            off += s.bytes;
        }
        s.kind = qb::SPAN_META; s.j = nd; s.off = off; s.bytes = 0;
        if (!save) s.dev = (unsigned char*)(L.meta + slot * META);
        spans.push_back(s);
        nd++;
    }
    qb::Span s = {};
    s.dev = (unsigned char*)(m->seen + (size_t)slot * (m->vocab_rows / 32));
    s.kind = qb::SPAN_PLAIN; s.off = off; s.bytes = (size_t)m->vocab_rows / 8;
    spans.push_back(s);
    *ndelta = nd;
}

// Model::save_state: every DeltaNet layer's end state and the conv ring's last three positions, then the slot's seen
// set, into h_out (qb_model_state_bytes bytes); *pos = the position the state is at (every layer's must agree: else
// QB_ERR_DEVICE). Waits for the stream.
int qb_model_save_state(qb_model* m, void* stream, int slot, void* h_out, size_t bytes, int* pos) {
    if (!m || slot < 0 || slot >= m->slots || !h_out || !pos || bytes != qb_model_state_bytes(m)) return QB_ERR_ARG;
    QB_TRY(ensure_session(m, bytes));
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<qb::Span> spans;
    int nd = 0;
    state_spans(m, slot, true, 0, spans, &nd);
    QB_TRY(run_spans(m, st, true, spans));
    QB_CUDA(cudaMemcpyAsync(h_out, m->staging, bytes, cudaMemcpyDeviceToHost, st));
    if (nd) QB_CUDA(cudaMemcpyAsync(m->h_positions, m->d_positions, nd * sizeof(int), cudaMemcpyDeviceToHost, st));
    QB_CUDA(cudaStreamSynchronize(st));
    *pos = nd ? m->h_positions[0] : 0;
    for (int i = 1; i < nd; i++)
        if (m->h_positions[i] != *pos) return QB_ERR_DEVICE;
    return QB_OK;
}

// Model::load_state: an image from qb_model_save_state taken at position `pos` into slot `slot`: the next step of the
// slot continues there (state in buffer 0, metadata {pos, pos, 0, 0})
int qb_model_load_state(qb_model* m, void* stream, int slot, const void* h_data, size_t bytes, int pos) {
    if (!m || slot < 0 || slot >= m->slots || !h_data || pos < 0 || bytes != qb_model_state_bytes(m)) return QB_ERR_ARG;
    QB_TRY(ensure_session(m, bytes));
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<qb::Span> spans;
    int nd = 0;
    state_spans(m, slot, false, pos, spans, &nd);
    QB_CUDA(cudaMemcpyAsync(m->staging, h_data, bytes, cudaMemcpyHostToDevice, st));
    QB_TRY(run_spans(m, st, false, spans));
    QB_CUDA(cudaStreamSynchronize(st));
    return QB_OK;
}

// Device pointers of the step's results and activations (tests, samplers): logits f32 [n_out][vocab_rows], the
// residual stream h f32 [n][5120], the last matrix-product input xn f16 [n][5120]
float* qb_model_logits(qb_model* m) { return m ? m->logits : nullptr; }
float* qb_model_hidden(qb_model* m) { return m ? m->h : nullptr; }
void* qb_model_xn(qb_model* m) { return m ? (void*)m->xn : nullptr; }
unsigned* qb_model_seen(qb_model* m) { return m ? m->seen : nullptr; }
long long qb_model_launches(const qb_model* m) { return m ? m->launches : 0; }
int qb_model_step_kernels(const qb_model* m) { return m ? m->step_kernels : 0; }

}  // extern "C"
