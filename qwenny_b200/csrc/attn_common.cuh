// What the attention kernels share: the cache addressing and byte orders of the reference (kernels/attn.cuh:19-64),
// which its unchanged host saves, loads and swaps.
#pragma once
#include "common.cuh"

namespace qb {

constexpr float KV_OFF = 1152.f;
constexpr int SROW = HD + 8;   // Q row stride in halves (ldmatrix rows on distinct banks)
constexpr int DSPLITS = 37;    // most key splits of a decode token on a 148-SM part (qb_attn_dec_splits' default)
constexpr int TSPLITS = 32;    // most key splits of a prompt tile (a power of two)

__host__ __device__ inline size_t cache_head(int slot, int g, int cap) { return ((size_t)slot * NKV + g) * cap * HD; }
__host__ __device__ inline size_t scale_head(int slot, int g, int cap) { return ((size_t)slot * NKV + g) * cap; }

// Byte of dim d in a key row / of (position, dim) in a head's values: the reference's fragment orders
// (kslot, vslot: kernels/attn.cuh:23-37)
__device__ __forceinline__ int kslot(int d) {
    int b = d >> 6, w = d & 15, t4 = (w & 7) >> 1, e = (w & 1) | ((w >> 3) << 1);
    return b * 64 + t4 * 16 + ((d & 63) >> 4) * 4 + e;
}
__device__ __forceinline__ size_t vslot(int pos, int d) {
    int j = pos & 15, t4 = (j & 7) >> 1, e = (j & 1) | ((j >> 3) << 1);
    return ((size_t)(pos >> 4) * HD + d) * 16 + t4 * 4 + e;
}

// Keys per split of a token with `keys` keys: a multiple of 64, at most `dsplits` splits (SM count / kv heads), and the same for every key
// count between two multiples of 2048 (where the host cuts short segments: a token's splits must not depend on how
// many drafts follow it in the step), so it is sized for the end of that range.
__host__ __device__ inline int dec_chunk(int keys, int dsplits) {
    const int range_end = ((keys - 1) / 2048 + 1) * 2048;
    return max(64, ((range_end + dsplits - 1) / dsplits + 63) / 64 * 64);
}
__host__ __device__ inline int dec_splits(int keys, int dsplits) { int c = dec_chunk(keys, dsplits); return (keys + c - 1) / c; }
// the most key splits of a decode token on a part with `sms` SMs: one block per SM over the kv heads, at most 64
__host__ inline int dsplits_for(int sms) { return max(1, min(64, sms / NKV)); }

constexpr int PTILE = 64 / GROUP;  // tokens of a prompt tile at most

}  // namespace qb
