// Host-side weight packers: the layouts the reference's loader produces (src/cuda/core.rs) and every kernel here
// reads. Load-time code, multi-threaded over the k16 steps / tiles as the reference's is.
#include <cuda_fp16.h>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>
#include "ctx.h"

namespace {

inline uint16_t f16_bits(float v) {
    __half h = __float2half_rn(v);
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}

template <class F>
void parallel_for(int n, F f) {
    int threads = (int)std::max(1u, std::thread::hardware_concurrency());
    threads = std::min(threads, std::max(1, n));
    int per = (n + threads - 1) / threads;
    std::vector<std::thread> pool;
    for (int i = 0; i < threads; i++) {
        int a = i * per, b = std::min(n, a + per);
        if (a >= b) break;
        pool.emplace_back([=] { for (int j = a; j < b; j++) f(j); });
    }
    for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// Packed row i holds source row order[i]; SwiGLU matrices interleave 8 gate rows with their 8 up rows per 16-row
// block (row_order, src/cuda/core.rs:106-114).
int qb_row_order(int rows, int silu, int* h_order) {
    if (rows < 0 || !h_order || (silu && rows % 16)) return QB_ERR_ARG;
    for (int i = 0; i < rows; i++)
        h_order[i] = silu ? (i / 16) * 8 + i % 8 + (i % 16 >= 8 ? rows / 2 : 0) : i;
    return QB_OK;
}

// A stored int4 matrix -> Marlin's layout (pack_marlin, src/cuda/core.rs:262-311; marlin_word :244-253).
//   h_q      u32 [rows][cols/8], value of column c at bits (c % 8) * 4, stored q + 8 (Quant, src/checkpoint.rs:20-31)
//   h_scales f32 [rows][cols/group], group a multiple of 128
//   h_order  n packed rows -> source row (n a multiple of 64)
//   h_words  out: u32 [cols/16][2n]; h_sc out: f16 bits [cols/128][n], output o of a 64-group at 8 (o % 8) + o / 8
static int pack_marlin(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int rows, int cols, int group,
                       const int* h_order, int n, uint32_t* h_words, uint16_t* h_sc);

int qb_pack_marlin(const uint32_t* h_q, const float* h_scales, int rows, int cols, int group, const int* h_order, int n,
                   uint32_t* h_words, uint16_t* h_sc) {
    return pack_marlin(h_q, h_scales, nullptr, rows, cols, group, h_order, n, h_words, h_sc);
}

// With zero points (h_zeros u8 [rows][cols/group], the stored value z of w = (q - z) * scale): h_sc gets 2 cols/128
// rows, the scales followed by (8 - z) * scale in the same layout (exact in f16: |8 - z| has at most 3 significant bits)
int qb_pack_marlin_z(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int rows, int cols, int group,
                     const int* h_order, int n, uint32_t* h_words, uint16_t* h_sc) {
    if (!h_zeros) return QB_ERR_ARG;
    return pack_marlin(h_q, h_scales, h_zeros, rows, cols, group, h_order, n, h_words, h_sc);
}

static int pack_marlin(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int rows, int cols, int group,
                       const int* h_order, int n, uint32_t* h_words, uint16_t* h_sc) {
    if (!h_q || !h_scales || !h_order || !h_words || !h_sc) return QB_ERR_ARG;
    if (n % 64 || cols % 128 || group % 128 || cols % group) return QB_ERR_ARG;
    for (int i = 0; i < n; i++)
        if (h_order[i] < 0 || h_order[i] >= rows) return QB_ERR_ARG;
    const int words = cols / 8, groups = cols / 128, qgroups = cols / group;
    for (int o = 0; o < n; o++) {
        int c64 = o / 64, c = o % 64, at = c64 * 64 + 8 * (c % 8) + c / 8;
        for (int gi = 0; gi < groups; gi++) {
            const size_t gq = (size_t)h_order[o] * qgroups + gi * 128 / group;
            h_sc[(size_t)gi * n + at] = f16_bits(h_scales[gq]);
            if (h_zeros) h_sc[(size_t)(groups + gi) * n + at] = f16_bits((8.f - (float)h_zeros[gq]) * h_scales[gq]);
        }
    }
    parallel_for(cols / 16, [&](int k16) {
        uint32_t* ws = h_words + (size_t)k16 * 2 * n;
        int k0 = k16 * 16;
        for (int c64 = 0; c64 < n / 64; c64++)
            for (int lane = 0; lane < 32; lane++) {
                int g = lane / 4, t = lane % 4;
                for (int blk = 0; blk < 4; blk++) {
                    const int* rws = h_order + c64 * 64 + blk * 16;
                    uint32_t word = 0;
                    for (int x = 0; x < 8; x++) {
                        int row = rws[g + 8 * ((x >> 1) & 1)], c = k0 + 2 * t + 8 * (x & 1) + (x >> 2);
                        uint32_t v = (h_q[(size_t)row * words + c / 8] >> ((c % 8) * 4)) & 15u;
                        word |= v << (4 * x);
                    }
                    ws[(c64 * 32 + lane) * 4 + blk] = word;
                }
            }
    });
    return QB_OK;
}

// One 16-row block of a Marlin matrix, as the draft head learns rows (the host half of Gemm::put_block,
// src/cuda/core.rs:614-656): the stored rows h_rows16[0..16) of the quantized matrix become the block's words
// [cols/16][32 lanes] (marlin_word, :244-253) and its scales [tables * cols/128][16] (marlin_scale, :255-260; tables = 2
// with zero points: the scales, then (8 - z) * scale). Without zero points every stored z must be 8 (QB_ERR_ARG).
int qb_marlin_block(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int zero_points, int rows,
                    int cols, int group, const int* h_rows16, uint32_t* h_words, uint16_t* h_sc) {
    if (!h_q || !h_scales || !h_rows16 || !h_words || !h_sc || cols % 128 || group % 128 || cols % group) return QB_ERR_ARG;
    if (zero_points && !h_zeros) return QB_ERR_ARG;
    const int words = cols / 8, groups = cols / 128, qgroups = cols / group;
    for (int r = 0; r < 16; r++) {
        if (h_rows16[r] < 0 || h_rows16[r] >= rows) return QB_ERR_ARG;
        if (!zero_points && h_zeros)
            for (int gi = 0; gi < qgroups; gi++)
                if (h_zeros[(size_t)h_rows16[r] * qgroups + gi] != 8) return QB_ERR_ARG;  // a symmetric matrix
    }
    for (int k16 = 0; k16 < cols / 16; k16++)
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane / 4, t = lane % 4;
            uint32_t word = 0;
            for (int x = 0; x < 8; x++) {
                const int row = h_rows16[g + 8 * ((x >> 1) & 1)], c = k16 * 16 + 2 * t + 8 * (x & 1) + (x >> 2);
                word |= ((h_q[(size_t)row * words + c / 8] >> ((c % 8) * 4)) & 15u) << (4 * x);
            }
            h_words[k16 * 32 + lane] = word;
        }
    for (int r = 0; r < 16; r++)
        for (int gi = 0; gi < groups; gi++) {
            const size_t gq = (size_t)h_rows16[r] * qgroups + gi * 128 / group;
            h_sc[gi * 16 + r] = f16_bits(h_scales[gq]);
            if (zero_points) h_sc[(groups + gi) * 16 + r] = f16_bits((8.f - (float)h_zeros[gq]) * h_scales[gq]);
        }
    return QB_OK;
}

// A dense matrix (f32 [rows][cols]) -> f16 tiles of 16 rows in mma A-fragment order, [tile][cols/16][32 lanes][8]
// (pack, src/cuda/core.rs:337-391, the f16 branch; frag :222-227). rows = n packed rows through h_order.
int qb_pack_f16(const float* h_w, int rows, int cols, const int* h_order, int n, uint16_t* h_out) {
    if (!h_w || !h_out || n % 16 || cols % 16) return QB_ERR_ARG;
    parallel_for(n / 16, [&](int tile) {
        uint16_t* o = h_out + (size_t)tile * 16 * cols;
        for (int k16 = 0; k16 < cols / 16; k16++)
            for (int lane = 0; lane < 32; lane++) {
                int g = lane / 4, t = lane % 4, c = k16 * 16 + 2 * t;
                int rc[8][2] = {{g, c}, {g, c + 1}, {g + 8, c}, {g + 8, c + 1},
                                {g, c + 8}, {g, c + 9}, {g + 8, c + 8}, {g + 8, c + 9}};
                for (int e = 0; e < 8; e++) {
                    int pr = tile * 16 + rc[e][0];
                    int row = h_order ? h_order[pr] : pr;
                    *o++ = f16_bits(h_w[(size_t)row * cols + rc[e][1]]);
                }
            }
    });
    (void)rows;
    return QB_OK;
}

// int8 weights of a 16-bit matrix in the reference's device form (pack with int8, src/cuda/core.rs:337-372,
// frags_int8 :233-244): per row and group of 128 columns scale = max |w| / 127 (1 for an all-zero group), codes
// round(w / scale) clamped to +-127 and stored + 128; tiles of 16 rows in mma A-fragment order, two k16 steps per
// 16-byte load of a lane; scales f32 [tile][group][16 rows].
int qb_pack_i8(const float* h_w, int rows, int cols, const int* h_order, int n, uint8_t* h_out, float* h_scales) {
    if (!h_w || !h_out || !h_scales || n % 16 || cols % 128) return QB_ERR_ARG;
    const int groups = cols / 128;
    parallel_for(n / 16, [&](int tile) {
        std::vector<uint8_t> q((size_t)16 * cols);
        float* st = h_scales + (size_t)tile * groups * 16;
        for (int r = 0; r < 16; r++) {
            const int pr = tile * 16 + r;
            const float* row = h_w + (size_t)(h_order ? h_order[pr] : pr) * cols;
            for (int gi = 0; gi < groups; gi++) {
                float mx = 0.f;
                for (int c = 0; c < 128; c++) mx = std::max(mx, std::fabs(row[gi * 128 + c]));
                const float scale = mx > 0.f ? mx / 127.f : 1.f;
                st[gi * 16 + r] = scale;
                for (int c = 0; c < 128; c++) {
                    float v = std::round(row[gi * 128 + c] / scale);
                    v = std::min(127.f, std::max(-127.f, v));
                    q[(size_t)r * cols + gi * 128 + c] = (uint8_t)((int)v + 128);
                }
            }
        }
        uint8_t* o = h_out + (size_t)tile * 16 * cols;
        for (int k32 = 0; k32 < cols / 32; k32++)
            for (int lane = 0; lane < 32; lane++)
                for (int ks = 0; ks < 2; ks++) {
                    const int g = lane / 4, t = lane % 4, c = k32 * 32 + ks * 16 + 2 * t;
                    const int rc[8][2] = {{g, c}, {g, c + 1}, {g + 8, c}, {g + 8, c + 1},
                                          {g, c + 8}, {g, c + 9}, {g + 8, c + 8}, {g + 8, c + 9}};
                    for (int e = 0; e < 8; e++) *o++ = q[(size_t)rc[e][0] * cols + rc[e][1]];
                }
    });
    (void)rows;
    return QB_OK;
}

// Split-K factor of the dense decode products (split_for, src/cuda/core.rs:393-398).
int qb_split_for(int tiles, int cols, int bits, int kd) {
    if (tiles <= 0 || cols <= 0 || bits <= 0 || bits > 2048 || kd <= 0) return 0;  // no split: the reference's host would stop on the division
    const int UNITS = 1024;
    int stage_cols = 2048 / bits, chunks = cols / stage_cols;
    int want = std::max((UNITS + tiles - 1) / tiles, (cols + kd - 1) / kd);
    for (int d = 1; d <= chunks; d++)
        if (chunks % d == 0 && d >= want) return d;
    return chunks;
}

}  // extern "C"
