// Host-side choice of the CTA launch order for the causal backward.
//
// A CTA that owns key tile kt walks the query tiles that see it (n_tiles - kt of
// them per query head when seqlen_q == seqlen_k), so work per CTA falls with kt.
// The B200 block scheduler hands the
// next block index to whichever SM frees up first, which is greedy list
// scheduling; the plan below simulates exactly that for a few candidate orders
// and keeps the one with the smallest modelled makespan.  This plays the role
// of the reference's choose_causal_cta_order / modeled_causal_max_work
// (reference src/fused_bwd_kernel.cpp:1285-1358), whose model is a fixed
// round-robin over 48 compute units; the permutation itself
// (remap_k_tile) keeps the reference's serpentine form as one candidate.
#pragma once

#include <algorithm>
#include <functional>
#include <queue>
#include <vector>

#include "geometry.h"

namespace fa3b200 {

// Tile grid of one head: which query tiles each key tile visits.
struct TileWork {
    int n_k_tiles = 0;
    Band band{};
    bool causal = false;  // the band is bounded: work differs between key tiles
    int steps(int kt) const { return q_tiles_of_k_tile(kt, band); }
    static TileWork of(const Band& band) {
        TileWork w;
        w.n_k_tiles = tiles_of(band.seqlen_k);
        w.band = band;
        w.causal = !band_is_full(band);
        return w;
    }
    static TileWork square(int n_tiles, bool causal) {
        return of(make_band(n_tiles * kTileRows, n_tiles * kTileRows, causal, -1, -1));
    }
};

enum CtaOrderMode : int {
    kOrderHeavyFirst = 0,  // key tile index ascending: longest work first (LPT)
    kOrderLightFirst = 1,
    kOrderSerpentine = 2,
};

// dQ-accumulator bytes that the CTAs running at the same time may spread over (about half of L2;
// 16 and 32 MB measured slower on the S=8192 shapes)
constexpr long long kDqL2BudgetBytes = 64LL << 20;

struct CtaOrderPlan {
    int mode = kOrderHeavyFirst;
    int width = 1;
    // Heads are taken in groups of `head_group`; inside a group the order is tile slot major, head
    // minor: block = (group * n_tiles + tile slot) * head_group + head in group.  head_group = all
    // heads is the globally heaviest-first order; a small group keeps the CTAs that run together on
    // a few heads, so their Q/dO tiles and the dQ-accumulator lines they add into stay in L2.
    int head_group = 1;
    long long makespan = 0;  // modelled, in query-tile steps
};

inline int host_remap_k_tile(int physical, int count, int mode, int width) {
    if (mode == kOrderHeavyFirst) return physical;
    if (mode == kOrderLightFirst) return count - 1 - physical;
    const int round = physical / width;
    const int base = round * width;
    const int slot = physical - base;
    const int span = std::min(width, count - base);
    return base + ((round & 1) == 0 ? slot : span - 1 - slot);
}

// Greedy list scheduling of blocks 0..n-1 (block = physical tile * bh + head)
// on `sms` machines; cost of a block = steps of its logical key tile + a fixed
// prologue/epilogue charge.
inline long long modelled_makespan(const TileWork& work, int bh_count, int group, int sms,
                                   int mode, int width, int head_group = 0) {
    const int n_tiles = work.n_k_tiles;
    if (head_group <= 0 || head_group > bh_count) head_group = bh_count;
    std::priority_queue<long long, std::vector<long long>, std::greater<long long>> free_at;
    for (int i = 0; i < sms; ++i) free_at.push(0);
    long long makespan = 0;
    const long long blocks = (long long)n_tiles * bh_count;
    const long long per_group = (long long)n_tiles * head_group;
    for (long long idx = 0; idx < blocks; ++idx) {
        const long long hg = idx / per_group;
        const int heads_here = int(std::min<long long>(head_group, bh_count - hg * head_group));
        const int physical = int((idx - hg * per_group) / heads_here);
        const int kt = host_remap_k_tile(physical, n_tiles, mode, width);
        const long long cost = 1 + (long long)group * work.steps(kt);
        const long long start = free_at.top();
        free_at.pop();
        free_at.push(start + cost);
        makespan = std::max(makespan, start + cost);
    }
    return makespan;
}

inline long long modelled_makespan(int n_tiles, int bh_count, int group, bool causal, int sms,
                                   int mode, int width, int head_group = 0) {
    return modelled_makespan(TileWork::square(n_tiles, causal), bh_count, group, sms, mode, width,
                             head_group);
}

// dq_bytes_per_head: bytes of fp32 dQ accumulator that the CTAs of one (batch, KV head) add into.
inline CtaOrderPlan plan_cta_order(const TileWork& work, int bh_count, int group, int sms,
                                   long long dq_bytes_per_head = 0) {
    const int n_tiles = work.n_k_tiles;
    const bool causal = work.causal;
    CtaOrderPlan best;
    best.head_group = bh_count;
    best.makespan = modelled_makespan(work, bh_count, group, sms, kOrderHeavyFirst, 1);
    const long long heavy_first = best.makespan;
    const int max_width = std::min(n_tiles, 16);
    for (int width = 2; causal && width <= max_width; ++width) {
        const long long m =
            modelled_makespan(work, bh_count, group, sms, kOrderSerpentine, width);
        if (m < best.makespan) {
            best.mode = kOrderSerpentine;
            best.width = width;
            best.makespan = m;
        }
    }
    // Cache-friendly grouping: the smallest head group (so the dQ-accumulator lines and Q/dO tiles of
    // the CTAs that run together stay in L2) whose modelled makespan is within 2 % of plain
    // heaviest-first, and whose accumulator share stays within the L2 budget.  Measured on B200:
    // +7..+14 % throughput on the S=4096..8192 shapes against the global heaviest-first order.
    if (dq_bytes_per_head > 0) {
        long long g_max = kDqL2BudgetBytes / dq_bytes_per_head;
        if (g_max < 1) g_max = 1;
        if (g_max > bh_count - 1) g_max = bh_count - 1;
        for (long long g = 1; g <= g_max; ++g) {
            const long long m = modelled_makespan(work, bh_count, group, sms, kOrderHeavyFirst, 1, int(g));
            if (m * 100 <= heavy_first * 102) {
                best.mode = kOrderHeavyFirst;
                best.width = 1;
                best.head_group = int(g);
                best.makespan = m;
                break;
            }
        }
    }
    return best;
}

inline CtaOrderPlan plan_cta_order(int n_tiles, int bh_count, int group, bool causal, int sms,
                                   long long dq_bytes_per_head = 0) {
    return plan_cta_order(TileWork::square(n_tiles, causal), bh_count, group, sms, dq_bytes_per_head);
}

}  // namespace fa3b200
