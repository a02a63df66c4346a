// Host-side choice of the CTA launch order for the causal backward.
//
// A CTA that owns key tile kt walks (n_tiles - kt) query tiles per query head,
// so work per CTA falls linearly with kt.  The B200 block scheduler hands the
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

namespace fa3b200 {

enum CtaOrderMode : int {
    kOrderHeavyFirst = 0,  // key tile index ascending: longest work first (LPT)
    kOrderLightFirst = 1,
    kOrderSerpentine = 2,
};

struct CtaOrderPlan {
    int mode = kOrderHeavyFirst;
    int width = 1;
    // Block index = head * n_tiles + tile slot when set, tile slot * heads + head otherwise.
    // Head-major keeps the CTAs that run together on a few heads, so their Q/dO tiles and
    // dQ-accumulator lines stay in L2; tile-major is the globally heaviest-first order.
    int head_major = 0;
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
inline long long modelled_makespan(int n_tiles, int bh_count, int group, bool causal, int sms,
                                   int mode, int width, bool head_major = false) {
    std::priority_queue<long long, std::vector<long long>, std::greater<long long>> free_at;
    for (int i = 0; i < sms; ++i) free_at.push(0);
    long long makespan = 0;
    const long long blocks = (long long)n_tiles * bh_count;
    for (long long idx = 0; idx < blocks; ++idx) {
        const int physical = head_major ? int(idx % n_tiles) : int(idx / bh_count);
        const int kt = host_remap_k_tile(physical, n_tiles, mode, width);
        const long long cost = 1 + (long long)group * (causal ? n_tiles - kt : n_tiles);
        const long long start = free_at.top();
        free_at.pop();
        free_at.push(start + cost);
        makespan = std::max(makespan, start + cost);
    }
    return makespan;
}

inline CtaOrderPlan plan_cta_order(int n_tiles, int bh_count, int group, bool causal, int sms) {
    CtaOrderPlan best;
    best.makespan = modelled_makespan(n_tiles, bh_count, group, causal, sms, kOrderHeavyFirst, 1);
    const long long heavy_first = best.makespan;
    const int max_width = std::min(n_tiles, 16);
    for (int width = 2; causal && width <= max_width; ++width) {
        const long long m =
            modelled_makespan(n_tiles, bh_count, group, causal, sms, kOrderSerpentine, width);
        if (m < best.makespan) {
            best.mode = kOrderSerpentine;
            best.width = width;
            best.makespan = m;
        }
    }
    // Prefer the cache-friendly head-major order (measured: +14 % throughput on S=4096..8192
    // MHA shapes) unless the model says its makespan is more than 8 % longer than
    // plain heaviest-first.
    const long long hm =
        modelled_makespan(n_tiles, bh_count, group, causal, sms, kOrderHeavyFirst, 1, true);
    if (hm * 100 <= heavy_first * 108) {
        best.mode = kOrderHeavyFirst;
        best.width = 1;
        best.head_major = 1;
        best.makespan = hm;
    }
    return best;
}

}  // namespace fa3b200
