// Tile geometry and tensor strides shared by the host planners and the kernels.
//
// Sequences are cut into 128-row tiles; the last tile of a sequence may be ragged.  Which (query,
// key) pairs attend is a band around a diagonal that is aligned to the bottom-right corner of the
// score matrix, the FlashAttention convention:
//     query i sees key j  iff  i + off - left <= j <= i + off + right,   off = seqlen_k - seqlen_q.
// Full attention has both sides unbounded, a causal mask is right = 0, a sliding window bounds
// one or both sides.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define FA3B200_HD __host__ __device__
#else
#define FA3B200_HD
#endif

namespace fa3b200 {

constexpr int kTileRows = 128;
constexpr int kUnbounded = 1 << 29;  // larger than any supported sequence length
// Most CTAs a small problem is cut into when its key tiles are split: the size of the CTA table that
// travels in the GEMM kernel's parameters (the host planner keeps to it).
constexpr int kMaxSplitCtas = 512;

FA3B200_HD inline int tiles_of(int seqlen) { return (seqlen + kTileRows - 1) / kTileRows; }

struct Band {
    int off;    // seqlen_k - seqlen_q
    int left;   // keys up to `left` positions before the diagonal are visible (kUnbounded: all)
    int right;  // keys up to `right` positions after the diagonal are visible (kUnbounded: all)
    int seqlen_q;
    int seqlen_k;
};

// window_left / window_right: -1 = unbounded, as in the parameter block; causal forces right = 0.
FA3B200_HD inline Band make_band(int seqlen_q, int seqlen_k, bool causal, int window_left,
                                 int window_right) {
    Band b;
    b.off = seqlen_k - seqlen_q;
    b.left = window_left < 0 || window_left >= kUnbounded ? kUnbounded : window_left;
    b.right = causal ? 0 : (window_right < 0 || window_right >= kUnbounded ? kUnbounded : window_right);
    b.seqlen_q = seqlen_q;
    b.seqlen_k = seqlen_k;
    return b;
}

FA3B200_HD inline bool band_is_full(const Band& b) {
    return b.left >= kUnbounded && b.right >= kUnbounded;
}

// Query tiles [first, last] that see at least one key of key tile kt (empty when last < first).
FA3B200_HD inline int first_q_tile(int kt, const Band& b) {
    if (b.right >= kUnbounded) return 0;
    const int first_query = kt * kTileRows - b.off - b.right;  // sees the tile's first key
    return first_query <= 0 ? 0 : first_query / kTileRows;
}
FA3B200_HD inline int last_q_tile(int kt, const Band& b) {
    int last_query = b.seqlen_q - 1;
    if (b.left < kUnbounded) {
        int key_hi = kt * kTileRows + kTileRows - 1;
        if (key_hi > b.seqlen_k - 1) key_hi = b.seqlen_k - 1;
        const int q = key_hi - b.off + b.left;  // last query that still sees the tile's last key
        if (q < last_query) last_query = q;
    }
    return last_query < 0 ? -1 : last_query / kTileRows;
}
FA3B200_HD inline int q_tiles_of_k_tile(int kt, const Band& b) {
    const int n = last_q_tile(kt, b) - first_q_tile(kt, b) + 1;
    return n > 0 ? n : 0;
}

// Key tiles [first, last] that hold at least one key visible to query tile qt.
FA3B200_HD inline int first_k_tile(int qt, const Band& b) {
    if (b.left >= kUnbounded) return 0;
    const int first_key = qt * kTileRows + b.off - b.left;  // seen by the tile's first query
    return first_key <= 0 ? 0 : first_key / kTileRows;
}
FA3B200_HD inline int last_k_tile(int qt, const Band& b) {
    int last_key = b.seqlen_k - 1;
    if (b.right < kUnbounded) {
        int query_hi = qt * kTileRows + kTileRows - 1;
        if (query_hi > b.seqlen_q - 1) query_hi = b.seqlen_q - 1;
        const int k = query_hi + b.off + b.right;  // last key the tile's last query sees
        if (k < last_key) last_key = k;
    }
    return last_key < 0 ? -1 : last_key / kTileRows;
}
FA3B200_HD inline int k_tiles_of_q_tile(int qt, const Band& b) {
    const int n = last_k_tile(qt, b) - first_k_tile(qt, b) + 1;
    return n > 0 ? n : 0;
}

// True when tile (kt, qt) holds at least one masked (key, query) pair.
FA3B200_HD inline bool tile_needs_mask(int kt, int qt, const Band& b) {
    const int key_lo = kt * kTileRows, key_hi = key_lo + kTileRows - 1;
    const int query_lo = qt * kTileRows, query_hi = query_lo + kTileRows - 1;
    const bool ragged_keys = key_hi >= b.seqlen_k;
    const bool crosses_right = b.right < kUnbounded && key_hi > query_lo + b.off + b.right;
    const bool crosses_left = b.left < kUnbounded && key_lo < query_hi + b.off - b.left;
    return ragged_keys || crosses_right || crosses_left;
}

// For key `key` (absolute) in a tile whose first query is `query0`: the surviving queries of the
// tile are those with  lo <= (query - query0) <= hi.
FA3B200_HD inline void query_range_of_key(int key, int query0, const Band& b, int* lo, int* hi) {
    if (key >= b.seqlen_k) {
        *lo = kUnbounded;
        *hi = -kUnbounded;
        return;
    }
    *lo = b.right < kUnbounded ? key - b.off - b.right - query0 : -kUnbounded;
    *hi = b.left < kUnbounded ? key - b.off + b.left - query0 : kUnbounded;
}

// For query `query` (absolute) and a tile whose first key is `key0`: the surviving keys of the
// tile are those with  lo <= (key - key0) <= hi.
FA3B200_HD inline void key_range_of_query(int query, int key0, const Band& b, int* lo, int* hi) {
    *lo = b.left < kUnbounded ? query + b.off - b.left - key0 : -kUnbounded;
    int h = b.seqlen_k - 1 - key0;
    if (b.right < kUnbounded) {
        const int d = query + b.off + b.right - key0;
        if (d < h) h = d;
    }
    *hi = h;
}

// Element strides of a [batch, head, row, D] tensor whose innermost dimension is contiguous.
struct TensorStrides {
    int64_t batch;
    int64_t head;
    int64_t row;
};

// bshd == false: [B,H,S,D] contiguous; true: [B,S,H,D] contiguous.
FA3B200_HD inline TensorStrides strides_of(bool bshd, int heads, int seqlen, int d) {
    TensorStrides s;
    s.batch = int64_t(heads) * seqlen * d;
    s.head = bshd ? int64_t(d) : int64_t(seqlen) * d;
    s.row = bshd ? int64_t(heads) * d : int64_t(d);
    return s;
}

}  // namespace fa3b200
