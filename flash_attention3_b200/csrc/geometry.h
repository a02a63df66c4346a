// Tile geometry and tensor strides shared by the host planners and the kernels.
//
// Sequences are cut into 128-row tiles; the last tile of a sequence may be ragged.  With a causal
// mask and seqlen_q != seqlen_k the diagonal is aligned to the bottom-right corner, the FlashAttention
// convention: query i sees key j iff j <= i + (seqlen_k - seqlen_q).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define FA3B200_HD __host__ __device__
#else
#define FA3B200_HD
#endif

namespace fa3b200 {

constexpr int kTileRows = 128;

FA3B200_HD inline int tiles_of(int seqlen) { return (seqlen + kTileRows - 1) / kTileRows; }

// First query tile that sees any key of key tile kt.
FA3B200_HD inline int first_q_tile(int kt, int causal_off, bool causal) {
    if (!causal) return 0;
    const int first_query = kt * kTileRows - causal_off;  // sees key kt*128
    return first_query <= 0 ? 0 : first_query / kTileRows;
}

// Number of query tiles key tile kt has to visit (per query head).
FA3B200_HD inline int q_tiles_of_k_tile(int kt, int n_q_tiles, int causal_off, bool causal) {
    const int first = first_q_tile(kt, causal_off, causal);
    return first >= n_q_tiles ? 0 : n_q_tiles - first;
}

// Number of key tiles (0 .. n-1) query tile qt has to visit.
FA3B200_HD inline int k_tiles_of_q_tile(int qt, int n_k_tiles, int causal_off, bool causal) {
    if (!causal) return n_k_tiles;
    const int last_key = qt * kTileRows + kTileRows - 1 + causal_off;  // seen by the tile's last query
    if (last_key < 0) return 0;
    const int n = last_key / kTileRows + 1;
    return n < n_k_tiles ? n : n_k_tiles;
}

// True when tile (kt, qt) holds at least one masked (key, query) pair.
FA3B200_HD inline bool tile_needs_mask(int kt, int qt, int seqlen_k, int causal_off, bool causal) {
    const bool ragged_keys = (kt + 1) * kTileRows > seqlen_k;
    const bool crosses_diagonal = causal && kt * kTileRows + kTileRows - 1 > qt * kTileRows + causal_off;
    return ragged_keys || crosses_diagonal;
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
