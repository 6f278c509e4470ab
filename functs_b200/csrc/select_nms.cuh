// Block-level building blocks for "mask -> nonzero -> stable descending sort -> top-k -> greedy NMS".
//
// All of it is integer / exactly-rounded fp32 work: the selection orders 64-bit keys (score bits, inverted
// index), and the IoU test reproduces, operation by operation, what a scalar CPU loop over
//   inter / (area_i + area_j - inter) > thr
// computes in fp32 (every product, sum and quotient rounded on its own; no fused multiply-add).
#pragma once

#include "common.cuh"

namespace fb {

constexpr int kHistBits = 11;
constexpr int kHistBins = 1 << kHistBits;
constexpr int kBinListCap = 1024;  // keys of the boundary bin that are finished by a local sort

// ---- coarse score histogram shared by a candidate producer and the binned top-k ----------------------------
// Positive fp32 bit patterns are ordered like their values, so (bits - bits(thr)) >> shift is a monotone bucketing
// of the scores above thr; everything at or above the last bucket is clamped into it.
struct HistParams {
    uint32_t base;
    int shift;
};

inline HistParams hist_params_for(float thr) {
    HistParams h;
    uint32_t one_bits = 0x3F800000u;  // scores are products of probabilities: <= 1.0
    float t = thr > 0.0f ? thr : 0.0f;
    uint32_t b;
    static_assert(sizeof(float) == 4, "fp32");
    __builtin_memcpy(&b, &t, 4);
    h.base = b;
    uint32_t diff = one_bits > b ? one_bits - b : 1u;
    h.shift = 0;
    while (((diff - 1u) >> h.shift) > static_cast<uint32_t>(kHistBins - 1)) ++h.shift;
    return h;
}

#ifdef __CUDACC__
__device__ __forceinline__ int hist_digit(uint64_t key, uint32_t base, int shift) {
    uint32_t bits = static_cast<uint32_t>(key >> 32);
    uint32_t d = bits > base ? (bits - base) >> shift : 0u;
    return d > static_cast<uint32_t>(kHistBins - 1) ? kHistBins - 1 : static_cast<int>(d);
}
#endif

// ---- bitonic sort, descending, on `n` (power of two) 64-bit keys in shared memory -------------------
template <int NT>
__device__ __forceinline__ void bitonic_sort_desc(uint64_t* s, int n) {
    // one thread per compare-exchange pair: pair p of a (k, j) step is (i, i | j) with bit j of i clear
    const int pairs = n >> 1;
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int p = threadIdx.x; p < pairs; p += NT) {
                const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
                const int ixj = i | j;
                const uint64_t a = s[i], b = s[ixj];
                const bool desc_seg = (i & k) == 0;
                if (desc_seg ? (a < b) : (a > b)) {
                    s[i] = b;
                    s[ixj] = a;
                }
            }
            __syncthreads();
        }
    }
}

// Rank sort, descending, of n <= NT distinct keys: thread t counts the keys larger than s[t] (broadcast reads) and
// drops its key at that rank.  Cheaper than the bitonic network for a few hundred keys (no barrier per step).
// tmp: n more keys of shared memory; s must be 16-byte aligned.  Ends with a barrier; the sorted keys are back in s.
template <int NT>
__device__ __forceinline__ void rank_sort_desc(uint64_t* s, int n, uint64_t* tmp) {
    const int t = threadIdx.x;
    uint64_t mine = 0ull;
    int rank = 0;
    if (t < n) {
        mine = s[t];
        const ulonglong2* s2 = reinterpret_cast<const ulonglong2*>(s);  // two keys per (broadcast) load
#pragma unroll 4
        for (int j = 0; j < (n >> 1); ++j) {
            const ulonglong2 k = s2[j];
            rank += (k.x > mine) ? 1 : 0;
            rank += (k.y > mine) ? 1 : 0;
        }
        if (n & 1) rank += (s[n - 1] > mine) ? 1 : 0;
        tmp[rank] = mine;
    }
    __syncthreads();
    if (t < n) s[t] = tmp[t];
    __syncthreads();
}

__device__ __forceinline__ int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

template <int SELCAP>
struct SelectSmem {
    __align__(16) uint64_t sel[SELCAP];
    uint64_t binlist[kBinListCap];
    int hist[kHistBins];
    uint64_t red_min[32];
    uint64_t red_max[32];
    int red_cnt[32];
    // broadcast slots
    uint64_t kmin, kmax;
    int nvalid;
    int digit, above, inbin;
    int sel_cnt, bin_cnt;
};

// Adds 1 to hist[d] for every lane with valid != 0, one shared-memory atomic per distinct digit per warp.
__device__ __forceinline__ void warp_hist_add(int* hist, int d, bool valid) {
    int dd = valid ? d : -1;
    unsigned peers = __match_any_sync(kFullMask, dd);
    if (valid) {
        int leader = __ffs(peers) - 1;
        if ((threadIdx.x & 31) == leader) atomicAdd(&hist[d], __popc(peers));
    }
}

// Selects the `topk` largest non-zero keys among key(0..n-1) and leaves them sorted descending in sm.sel.
// Returns the number selected (min(#non-zero keys, topk)).  Keys must be distinct; key(i) == 0 means "absent".
// All NT threads of the block must call it; SELCAP is a power of two >= topk and NT a multiple of 32.
template <int NT, int SELCAP, int UNROLL, class KeyFn>
__device__ int block_select_topk(KeyFn key, int n, int topk, SelectSmem<SELCAP>& sm) {
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int NW = NT / 32;

    // pass 0: count, min and max of the present keys
    uint64_t lmin = ~0ull, lmax = 0ull;
    int lcnt = 0;
    for (int base = 0; base < n; base += NT * UNROLL) {
        uint64_t k[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int i = base + u * NT + tid;
            k[u] = (i < n) ? key(i) : 0ull;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (k[u] != 0ull) {
                lmin = k[u] < lmin ? k[u] : lmin;
                lmax = k[u] > lmax ? k[u] : lmax;
                ++lcnt;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        uint64_t omin = __shfl_xor_sync(kFullMask, lmin, o);
        uint64_t omax = __shfl_xor_sync(kFullMask, lmax, o);
        lcnt += __shfl_xor_sync(kFullMask, lcnt, o);
        lmin = omin < lmin ? omin : lmin;
        lmax = omax > lmax ? omax : lmax;
    }
    if (lane == 0) {
        sm.red_min[warp] = lmin;
        sm.red_max[warp] = lmax;
        sm.red_cnt[warp] = lcnt;
    }
    if (tid == 0) {
        sm.sel_cnt = 0;
        sm.bin_cnt = 0;
    }
    __syncthreads();
    if (warp == 0) {
        uint64_t a = lane < NW ? sm.red_min[lane] : ~0ull;
        uint64_t b = lane < NW ? sm.red_max[lane] : 0ull;
        int c = lane < NW ? sm.red_cnt[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            uint64_t oa = __shfl_xor_sync(kFullMask, a, o);
            uint64_t ob = __shfl_xor_sync(kFullMask, b, o);
            c += __shfl_xor_sync(kFullMask, c, o);
            a = oa < a ? oa : a;
            b = ob > b ? ob : b;
        }
        if (lane == 0) {
            sm.kmin = a;
            sm.kmax = b;
            sm.nvalid = c;
        }
    }
    __syncthreads();
    const int nvalid = sm.nvalid;
    const uint64_t kmin = sm.kmin, kmax = sm.kmax;
    if (nvalid == 0) return 0;

    int sort_n;
    int result;
    if (nvalid <= topk) {
        // everything is selected
        for (int base = 0; base < n; base += NT * UNROLL) {
            uint64_t k[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int i = base + u * NT + tid;
                k[u] = (i < n) ? key(i) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (k[u] != 0ull) {
                    int pos = atomicAdd(&sm.sel_cnt, 1);
                    if (pos < SELCAP) sm.sel[pos] = k[u];
                }
            }
        }
        __syncthreads();
        result = nvalid;
    } else {
        // radix descent from the highest bit in which the keys differ
        uint64_t diff = kmin ^ kmax;  // != 0 because nvalid >= 2 distinct keys
        int hb = 63 - __clzll(static_cast<long long>(diff));
        uint64_t mask = (hb >= 63) ? 0ull : ~((1ull << (hb + 1)) - 1ull);
        uint64_t prefix = kmax & mask;
        int want = topk;
        while (true) {
            int shift = hb - kHistBits + 1;
            if (shift < 0) shift = 0;
            const int nb = hb - shift + 1;
            const int nbins = 1 << nb;
            for (int i = tid; i < nbins; i += NT) sm.hist[i] = 0;
            __syncthreads();
            for (int base = 0; base < n; base += NT * UNROLL) {
                uint64_t k[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    int i = base + u * NT + tid;
                    k[u] = (i < n) ? key(i) : 0ull;
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    bool v = (k[u] != 0ull) && ((k[u] & mask) == prefix);
                    int d = static_cast<int>((k[u] >> shift) & static_cast<uint64_t>(nbins - 1));
                    warp_hist_add(sm.hist, d, v);
                }
            }
            __syncthreads();
            // warp 0 finds the largest digit d with (count of digits >= d) >= want
            if (warp == 0) {
                const int per = (nbins + 31) / 32;  // bins per lane, lane 31 holds the highest bins
                int lo = lane * per, hi = lo + per;
                if (hi > nbins) hi = nbins;
                int s = 0;
                for (int i = lo; i < hi; ++i) s += sm.hist[i];
                // suffix sum over lanes: suf = sum of s over lanes > lane
                int incl = s;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int t = __shfl_down_sync(kFullMask, incl, o);
                    if (lane + o < 32) incl += t;
                }
                int suf = incl - s;  // strictly higher lanes
                bool mine = (suf < want) && (incl >= want);
                if (mine) {
                    int cum = suf;
                    int d = hi - 1;
                    for (; d >= lo; --d) {
                        int h = sm.hist[d];
                        if (cum + h >= want) break;
                        cum += h;
                    }
                    sm.digit = d;
                    sm.above = cum;
                    sm.inbin = sm.hist[d];
                }
            }
            __syncthreads();
            const int digit = sm.digit, above = sm.above, inbin = sm.inbin;
            want -= above;
            mask |= static_cast<uint64_t>(nbins - 1) << shift;
            prefix |= static_cast<uint64_t>(digit) << shift;
            hb = shift - 1;
            if (inbin == want || shift == 0 || inbin <= kBinListCap) break;
            __syncthreads();
        }
        // collect: strictly above the boundary bin -> sel; inside the bin -> binlist
        for (int base = 0; base < n; base += NT * UNROLL) {
            uint64_t k[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                int i = base + u * NT + tid;
                k[u] = (i < n) ? key(i) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (k[u] != 0ull) {
                    uint64_t km = k[u] & mask;
                    if (km > prefix) {
                        int pos = atomicAdd(&sm.sel_cnt, 1);
                        if (pos < SELCAP) sm.sel[pos] = k[u];
                    } else if (km == prefix) {
                        int pos = atomicAdd(&sm.bin_cnt, 1);
                        if (pos < kBinListCap) sm.binlist[pos] = k[u];
                    }
                }
            }
        }
        __syncthreads();
        int bc = sm.bin_cnt < kBinListCap ? sm.bin_cnt : kBinListCap;
        int bn = next_pow2(bc);
        for (int i = bc + tid; i < bn; i += NT) sm.binlist[i] = 0ull;
        __syncthreads();
        bitonic_sort_desc<NT>(sm.binlist, bn);
        const int have = sm.sel_cnt;  // == topk - want
        for (int i = tid; i < want && i < bc; i += NT) {
            if (have + i < SELCAP) sm.sel[have + i] = sm.binlist[i];
        }
        __syncthreads();
        result = topk;
    }
    sort_n = next_pow2(result);
    for (int i = result + tid; i < sort_n; i += NT) sm.sel[i] = 0ull;
    __syncthreads();
    bitonic_sort_desc<NT>(sm.sel, sort_n);
    return result;
}

// The exact generic selection as an out-of-line call: it is the rare way out of the binned selections below, and its
// code (three passes, two sorts) should not sit in the middle of their instruction stream.
template <int NT, int SELCAP, int UNROLL, class KeyFn>
__device__ __noinline__ int block_select_topk_outlined(KeyFn key, int n, int topk, SelectSmem<SELCAP>* sm) {
    return block_select_topk<NT, SELCAP, UNROLL>(key, n, topk, *sm);
}

// Same result as block_select_topk, but in two passes for keys whose scores lie above a known threshold: one pass
// fills the coarse score histogram (hist_digit), the second collects the keys above / inside the boundary bucket,
// and only the boundary bucket is sorted.  Falls back to block_select_topk when that bucket exceeds kBinListCap.
// KeyFn::kDenseScores marks a key function over a plain fp32 score array (members s, thr, vec4: the array may be read
// four at a time): the two passes then read the scores directly and build keys only for the elements they keep.
template <int NT, int SELCAP, int UNROLL, class KeyFn>
__device__ int block_select_topk_binned(KeyFn key, int n, int topk, uint32_t hist_base, int hist_shift,
                                        SelectSmem<SELCAP>& sm) {
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < kHistBins; i += NT) sm.hist[i] = 0;
    if (tid == 0) {
        sm.sel_cnt = 0;
        sm.bin_cnt = 0;
        sm.digit = -1;
        sm.above = 0;
        sm.inbin = 0;
        sm.nvalid = 0;
    }
    __syncthreads();
    if constexpr (KeyFn::kDenseScores) {
        // fp32 scores, four per load: an element below the threshold costs a compare, nothing else
        const float thr = key.thr;
        auto add = [&](float v) {
            if (v > thr) atomicAdd(&sm.hist[hist_digit(static_cast<uint64_t>(__float_as_uint(v)) << 32, hist_base, hist_shift)], 1);
        };
        const int n4 = key.vec4 ? (n >> 2) : 0;
        const float4* s4 = reinterpret_cast<const float4*>(key.s);
        for (int c = tid; c < n4; c += NT) {
            const float4 q = s4[c];
            add(q.x);
            add(q.y);
            add(q.z);
            add(q.w);
        }
        for (int i = 4 * n4 + tid; i < n; i += NT) add(key.s[i]);
    } else {
        for (int base = 0; base < n; base += NT * UNROLL) {
            uint64_t k[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = base + u * NT + tid;
                k[u] = (i < n) ? key(i) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (k[u] != 0ull) atomicAdd(&sm.hist[hist_digit(k[u], hist_base, hist_shift)], 1);
            }
        }
    }
    __syncthreads();
    // boundary bucket: the largest digit d with (keys in buckets >= d) >= topk.  Every thread sums its share of the
    // buckets (higher thread = higher buckets), suffix sums over the block locate the thread that holds the boundary
    {
        static_assert(kHistBins % NT == 0, "the histogram must split evenly over the block");
        constexpr int per = kHistBins / NT;
        int h[per];
        int s = 0;
#pragma unroll
        for (int k = 0; k < per; ++k) {
            h[k] = sm.hist[tid * per + k];
            s += h[k];
        }
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_down_sync(kFullMask, incl, o);
            if (lane + o < 32) incl += t;
        }
        if (lane == 0) sm.red_cnt[warp] = incl;
        __syncthreads();
        int higher = 0, total = 0;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) {
            const int c = sm.red_cnt[w];
            total += c;
            higher += (w > warp) ? c : 0;
        }
        incl += higher;
        const int suf = incl - s;
        if (tid == 0) sm.nvalid = total;
        // the counts are not needed again: every bucket now holds the number of keys in the buckets above it, which
        // is where its keys start in the final descending order
        {
            int above_k = suf;
#pragma unroll
            for (int k = per - 1; k >= 0; --k) {
                sm.hist[tid * per + k] = above_k;
                above_k += h[k];
            }
        }
        if (total > topk && suf < topk && incl >= topk) {
            int cum = suf, dsel = 0, hsel = 0, above = 0;
            bool found = false;
#pragma unroll
            for (int k = per - 1; k >= 0; --k) {  // incl >= topk: one of the buckets is the boundary
                if (!found) {
                    if (cum + h[k] >= topk) {
                        found = true;
                        dsel = k;
                        hsel = h[k];
                        above = cum;
                    } else {
                        cum += h[k];
                    }
                }
            }
            sm.digit = tid * per + dsel;
            sm.above = above;
            sm.inbin = hsel;
        }
    }
    __syncthreads();
    const int nvalid = sm.nvalid;
    if (nvalid == 0) return 0;
    const int dstar = sm.digit;  // -1: everything is selected
    if (sm.inbin > kBinListCap) {
        __syncthreads();
        return block_select_topk_outlined<NT, SELCAP, UNROLL>(key, n, topk, &sm);
    }
    auto place = [&](uint64_t k) {
        const int d = hist_digit(k, hist_base, hist_shift);
        if (d > dstar) {
            const int pos = atomicAdd(&sm.sel_cnt, 1);
            if (pos < SELCAP) sm.sel[pos] = k;
        } else if (d == dstar) {
            const int pos = atomicAdd(&sm.bin_cnt, 1);
            if (pos < kBinListCap) sm.binlist[pos] = k;
        }
    };
    if constexpr (KeyFn::kDenseScores) {
        // a score can only reach bucket dstar or above if its bits reach the bucket's first value: one integer
        // compare per element, the few that pass take the exact path
        const float thr = key.thr;
        const uint32_t lo_bits = dstar > 0 ? hist_base + (static_cast<uint32_t>(dstar) << hist_shift) : 0u;
        auto look = [&](float v, int i) {
            if (v > thr && __float_as_uint(v) >= lo_bits) place(make_key(v, static_cast<uint32_t>(i)));
        };
        const int n4 = key.vec4 ? (n >> 2) : 0;
        const float4* s4 = reinterpret_cast<const float4*>(key.s);
        for (int c = tid; c < n4; c += NT) {
            const float4 q = s4[c];
            look(q.x, 4 * c);
            look(q.y, 4 * c + 1);
            look(q.z, 4 * c + 2);
            look(q.w, 4 * c + 3);
        }
        for (int i = 4 * n4 + tid; i < n; i += NT) look(key.s[i], i);
    } else {
        for (int base = 0; base < n; base += NT * UNROLL) {
            uint64_t k[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = base + u * NT + tid;
                k[u] = (i < n) ? key(i) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (k[u] != 0ull) place(k[u]);
            }
        }
    }
    __syncthreads();
    const int result = nvalid < topk ? nvalid : topk;
    if (dstar >= 0) {
        const int bc = sm.bin_cnt;
        const int bn = next_pow2(bc);
        for (int i = bc + tid; i < bn; i += NT) sm.binlist[i] = 0ull;
        __syncthreads();
        bitonic_sort_desc<NT>(sm.binlist, bn);
        const int have = sm.sel_cnt;
        const int want = topk - have;
        for (int i = tid; i < want && i < bc; i += NT) {
            if (have + i < SELCAP) sm.sel[have + i] = sm.binlist[i];
        }
        __syncthreads();
    }
    // Final order.  The boundary bucket's share already sits sorted behind the `have` keys of the higher buckets.
    // Those are ordered by a counting sort: a key of bucket d goes to the run that starts at hist[d] (keys in higher
    // buckets), in arrival order; afterwards hist[d] is the run's end and hist[d + 1] its start, and every key
    // counts the larger keys of its own run (a run holds a key or two unless many scores are nearly equal).
    static_assert(SELCAP <= kBinListCap, "the boundary list doubles as the scatter target");
    {
        const int have = dstar >= 0 ? (sm.sel_cnt < SELCAP ? sm.sel_cnt : SELCAP) : result;
        uint64_t* tmp = sm.binlist;  // not needed any more
        __syncthreads();
        for (int i = tid; i < have; i += NT) {
            const uint64_t k = sm.sel[i];
            tmp[atomicAdd(&sm.hist[hist_digit(k, hist_base, hist_shift)], 1)] = k;
        }
        __syncthreads();
        for (int i = tid; i < have; i += NT) {
            const uint64_t mine = tmp[i];
            const int d = hist_digit(mine, hist_base, hist_shift);
            const int lo = d + 1 < kHistBins ? sm.hist[d + 1] : 0, hi = sm.hist[d];
            int rank = lo;
            for (int q = lo; q < hi; ++q) rank += (tmp[q] > mine) ? 1 : 0;
            sm.sel[rank] = mine;
        }
        __syncthreads();
    }
    return result;
}

// A plain fp32 score array as a key function (key = score above thr, index); kDenseScores lets the binned selection
// read the array four scores at a time when vec4 says it is 16-byte aligned.
struct DenseScores {
    static constexpr bool kDenseScores = true;
    const float* s;
    float thr;
    bool vec4;
    __device__ __forceinline__ uint64_t operator()(int i) const {
        const float v = s[i];
        return (v > thr) ? make_key(v, static_cast<uint32_t>(i)) : 0ull;
    }
};

// Keys that already sit in a list (shared memory): the non-dense form of the key functions above.
struct ListKeys {
    static constexpr bool kDenseScores = false;
    const uint64_t* k;
    __device__ __forceinline__ uint64_t operator()(int i) const { return k[i]; }
};

constexpr int kCandCap = 1024;  // candidate keys block_select_topk_sampled may collect before it gives up

// The largest digit d with (entries of hist in buckets >= d) >= target, or -1 when the histogram holds fewer.
// hist is left as it is.  All NT threads must call it.
template <int NT>
__device__ int block_hist_rank_bucket(const int* hist, int* red_cnt, int* slot, int target) {
    static_assert(kHistBins % NT == 0, "the histogram must split evenly over the block");
    constexpr int per = kHistBins / NT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int h[per];
    int s = 0;
#pragma unroll
    for (int k = 0; k < per; ++k) {
        h[k] = hist[tid * per + k];
        s += h[k];
    }
    int incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_down_sync(kFullMask, incl, o);
        if (lane + o < 32) incl += t;
    }
    if (lane == 0) red_cnt[warp] = incl;
    if (tid == 0) *slot = -1;
    __syncthreads();
    int higher = 0;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) higher += (w > warp) ? red_cnt[w] : 0;
    incl += higher;
    const int suf = incl - s;
    if (suf < target && incl >= target) {
        int cum = suf, d = 0;
        bool found = false;
#pragma unroll
        for (int k = per - 1; k >= 0; --k) {
            if (!found) {
                if (cum + h[k] >= target) {
                    found = true;
                    d = k;
                } else {
                    cum += h[k];
                }
            }
        }
        *slot = tid * per + d;
    }
    __syncthreads();
    return *slot;
}

// the two-pass selection over a whole score array, out of line (the sampled selection's rare way out)
template <int NT, int SELCAP>
__device__ __noinline__ int block_select_dense_outlined(const float* s, bool vec4, float thr, int n, int topk, uint32_t hist_base,
                                                        int hist_shift, SelectSmem<SELCAP>* sm) {
    return block_select_topk_binned<NT, SELCAP, 8>(DenseScores{s, thr, vec4}, n, topk, hist_base, hist_shift, *sm);
}

// Same result as block_select_topk_binned for a plain fp32 score array in GLOBAL memory (key = score above thr, index),
// reading the array once: a spread sample of the scores (one 16-byte chunk per thread) gives a score floor that should
// leave a few hundred candidates; one pass collects every key at or above the floor into `cand` (kCandCap keys of
// shared memory, appended with one atomic per warp and round); the exact selection then runs on that list.  The floor
// is only a guess, the count decides: with fewer than topk candidates (while keys below the floor exist) or more than
// kCandCap, the two-pass selection over the whole array runs instead, so the result never depends on the sample.
template <int NT, int SELCAP>
__device__ int block_select_topk_sampled(const float* __restrict__ s, bool vec4, float thr, int n, int topk,
                                         uint32_t hist_base, int hist_shift, SelectSmem<SELCAP>& sm, uint64_t* cand) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n4 = vec4 ? (n >> 2) : 0;
    const float4* s4 = reinterpret_cast<const float4*>(s);
    uint32_t lo_bits = 0u;  // 0: every score above thr is a candidate
    if (n > kCandCap && n4 >= NT) {
        for (int i = tid; i < kHistBins; i += NT) sm.hist[i] = 0;
        __syncthreads();
        const float4 q = __ldg(s4 + static_cast<int>((static_cast<int64_t>(tid) * n4) / NT));
        auto add = [&](float v) {
            if (v > thr) atomicAdd(&sm.hist[hist_digit(static_cast<uint64_t>(__float_as_uint(v)) << 32, hist_base, hist_shift)], 1);
        };
        add(q.x);
        add(q.y);
        add(q.z);
        add(q.w);
        __syncthreads();
        // rank in the sample that corresponds to 1.8 * topk in the whole array (the spread of a count of a few dozen
        // sample hits is about a sixth of it: falling short of topk takes three standard deviations)
        const int target = static_cast<int>((static_cast<int64_t>(topk) * (4 * NT) * 9) / (static_cast<int64_t>(n) * 5)) + 4;
        const int d = block_hist_rank_bucket<NT>(sm.hist, sm.red_cnt, &sm.digit, target);
        if (d > 0) lo_bits = hist_base + (static_cast<uint32_t>(d) << hist_shift);
    }
    if (tid == 0) sm.bin_cnt = 0;
    __syncthreads();
    // collection: lane-local hit counts, a warp prefix sum, one atomic per warp and round
    auto append = [&](const uint64_t (&k)[4], int cnt) {
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        const int total = __shfl_sync(kFullMask, incl, 31);
        if (total != 0) {
            int base = 0;
            if (lane == 31) base = atomicAdd(&sm.bin_cnt, total);
            base = __shfl_sync(kFullMask, base, 31);
            int pos = base + incl - cnt;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (k[e] != 0ull) {
                    if (pos < kCandCap) cand[pos] = k[e];
                    ++pos;
                }
            }
        }
    };
    auto key_of = [&](float v, int i) -> uint64_t {
        return (v > thr && __float_as_uint(v) >= lo_bits) ? make_key(v, static_cast<uint32_t>(i)) : 0ull;
    };
    constexpr int UN = 3;
    for (int c0 = warp * 32 + lane; __any_sync(kFullMask, c0 < n4); c0 += NT * UN) {
        float4 q[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int c = c0 + u * NT;
            q[u] = c < n4 ? __ldg(s4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int c = c0 + u * NT;
            uint64_t k[4];
            k[0] = key_of(q[u].x, 4 * c);
            k[1] = key_of(q[u].y, 4 * c + 1);
            k[2] = key_of(q[u].z, 4 * c + 2);
            k[3] = key_of(q[u].w, 4 * c + 3);
            append(k, (k[0] != 0ull) + (k[1] != 0ull) + (k[2] != 0ull) + (k[3] != 0ull));
        }
    }
    for (int i0 = 4 * n4 + warp * 32; i0 < n; i0 += NT) {  // scalar tail (or the whole array when it is not 16-byte aligned)
        const int i = i0 + lane;
        uint64_t k[4] = {i < n ? key_of(__ldg(s + i), i) : 0ull, 0ull, 0ull, 0ull};
        append(k, k[0] != 0ull ? 1 : 0);
    }
    __syncthreads();
    const int c = sm.bin_cnt;
    __syncthreads();  // (the selections below reset the counter)
    if (c > kCandCap || (lo_bits != 0u && c < topk)) {
        return block_select_dense_outlined<NT, SELCAP>(s, vec4, thr, n, topk, hist_base, hist_shift, &sm);
    }
    return block_select_topk_binned<NT, SELCAP, 2>(ListKeys{cand}, c, topk, hist_base, hist_shift, sm);
}

// ---- IoU suppression test ------------------------------------------------------------------------
struct NmsBox {
    float x1, y1, x2, y2, area;
};

__device__ __forceinline__ NmsBox make_nms_box(float x1, float y1, float x2, float y2) {
    NmsBox b;
    b.x1 = x1;
    b.y1 = y1;
    b.x2 = x2;
    b.y2 = y2;
    b.area = __fmul_rn(__fsub_rn(x2, x1), __fsub_rn(y2, y1));
    return b;
}

// true iff fp32(inter / (area_i + area_j - inter)) > thr.  thr_lo / thr_hi bracket thr by a relative 1e-6:
// outside the bracket the comparison against thr * union decides without a division, inside it the
// correctly rounded quotient is formed, so the answer is always that of the division.
__device__ __forceinline__ bool iou_exceeds(const NmsBox& a, const NmsBox& b, float thr, float thr_lo, float thr_hi) {
    // x extent first: boxes of different classes sit in disjoint coordinate ranges, so most pairs end here
    float w = fmaxf(0.0f, __fsub_rn(fminf(a.x2, b.x2), fmaxf(a.x1, b.x1)));
    if (!(w > 0.0f)) return false;  // inter = w * h = 0: the quotient is 0 (or NaN): never above a positive threshold
    float h = fmaxf(0.0f, __fsub_rn(fminf(a.y2, b.y2), fmaxf(a.y1, b.y1)));
    float inter = __fmul_rn(w, h);
    if (!(inter > 0.0f)) return false;
    float uni = __fsub_rn(__fadd_rn(a.area, b.area), inter);
    if (uni > 0.0f && uni < 3.0e38f && inter < 3.0e38f) {
        if (inter > __fmul_rn(uni, thr_hi)) return true;
        if (inter < __fmul_rn(uni, thr_lo)) return false;
    }
    return __fdiv_rn(inter, uni) > thr;
}

// The same decision without branches, for callers that run several independent tests at once: verdict 0 = not above,
// 1 = above, 2 = inside the bracket (the caller forms the correctly rounded quotient inter / uni and compares it
// with thr, as iou_exceeds does).
struct IouQuick {
    float inter, uni;
    int verdict;
};
__device__ __forceinline__ IouQuick iou_quick(const NmsBox& a, const NmsBox& b, float thr_lo, float thr_hi) {
    IouQuick q;
    const float w = fmaxf(0.0f, __fsub_rn(fminf(a.x2, b.x2), fmaxf(a.x1, b.x1)));
    const float h = fmaxf(0.0f, __fsub_rn(fminf(a.y2, b.y2), fmaxf(a.y1, b.y1)));
    q.inter = __fmul_rn(w, h);
    q.uni = __fsub_rn(__fadd_rn(a.area, b.area), q.inter);
    const bool pos = (w > 0.0f) && (q.inter > 0.0f);
    const bool safe = q.uni > 0.0f && q.uni < 3.0e38f && q.inter < 3.0e38f;
    const bool yes = pos && safe && q.inter > __fmul_rn(q.uni, thr_hi);
    const bool no = !pos || (safe && q.inter < __fmul_rn(q.uni, thr_lo));
    q.verdict = yes ? 1 : (no ? 0 : 2);
    return q;
}

// For boxes with finite coordinates and areas below 1e37 (nms_box_is_tame) the guards of iou_exceeds are implied by a
// positive intersection: inter <= min(area) and max(area) <= union <= 2e37.  yes / unsure as in iou_quick.
__device__ __forceinline__ bool nms_box_is_tame(const NmsBox& b) {
    return fabsf(b.x1) < 1.0e18f && fabsf(b.y1) < 1.0e18f && fabsf(b.x2) < 1.0e18f && fabsf(b.y2) < 1.0e18f && b.area < 1.0e37f;
}
__device__ __forceinline__ void iou_quick_tame(const NmsBox& a, const NmsBox& b, float thr_lo, float thr_hi, bool& yes,
                                               bool& unsure) {
    const float w = __fsub_rn(fminf(a.x2, b.x2), fmaxf(a.x1, b.x1));
    const float h = __fsub_rn(fminf(a.y2, b.y2), fmaxf(a.y1, b.y1));
    const float inter = __fmul_rn(w, h);
    const float uni = __fsub_rn(__fadd_rn(a.area, b.area), inter);
    const bool pos = w > 0.0f && h > 0.0f && inter > 0.0f;
    yes = pos && inter > __fmul_rn(uni, thr_hi);
    unsure = pos && !yes && !(inter < __fmul_rn(uni, thr_lo));
}

// One word of a row of the suppression matrix: lane b tests box j = 32w + b against box i (valid = j > i && j < n).
// The x extents are compared first for the whole warp; only if some lane overlaps in x is the full test run.
// Must be called by all 32 lanes.
__device__ __forceinline__ uint32_t nms_row_word(const NmsBox& bi, const NmsBox* sb, int j, bool valid, float thr,
                                                 float thr_lo, float thr_hi) {
    bool cand = false;
    if (valid) cand = fminf(bi.x2, sb[j].x2) > fmaxf(bi.x1, sb[j].x1);  // positive overlap in x
    if (__ballot_sync(kFullMask, cand) == 0u) return 0u;
    bool pred = false;
    if (cand) pred = iou_exceeds(bi, sb[j], thr, thr_lo, thr_hi);
    return __ballot_sync(kFullMask, pred);
}

// Serial part of greedy NMS over a precomputed suppression bit matrix, run by ONE warp.
// mask: row i has `words` 32-bit words (row stride `row_stride` words); bit j of row i set iff j > i and box i
// suppresses box j.  keep_words[w] receives the keep bits of boxes 32w..32w+31.  words <= 32.
__device__ __forceinline__ void warp_nms_scan(const uint32_t* mask, int row_stride, int n, int words,
                                              uint32_t* keep_words) {
    const int lane = threadIdx.x & 31;
    uint32_t removed = 0u;  // lane l tracks word l
    for (int w = 0; w < words; ++w) {
        uint32_t r = __shfl_sync(kFullMask, removed, w);
        const int base = w * 32;
        const int rows = min(32, n - base);
        // loads first (none depends on a decision): the diagonal 32x32 block (broadcast reads, identical on every
        // lane) and this lane's column word of the 32 rows
        uint32_t diag[32], col[32];
#pragma unroll
        for (int b = 0; b < 32; ++b) {
            const bool in = b < rows;
            diag[b] = in ? mask[(base + b) * row_stride + w] : 0u;
            col[b] = (in && lane < words) ? mask[(base + b) * row_stride + lane] : 0u;
        }
        // Serial part.  Row b can only set bits above b, so bit b of r is final once the rows before b are done and
        // keepw = ~r (valid rows) at the end.  Only rows with a non-empty diagonal word can change r: when there
        // are few of them they are walked in order (re-read from shared memory by index), otherwise all 32 rows go
        // through the unrolled register chain.
        uint32_t nz = 0u;
#pragma unroll
        for (int b = 0; b < 32; ++b) nz |= (diag[b] != 0u) ? (1u << b) : 0u;
        if (__popc(nz) <= 10) {
            while (nz) {
                const int b = __ffs(nz) - 1;
                nz &= nz - 1u;
                if (!(r & (1u << b))) r |= mask[(base + b) * row_stride + w];
            }
        } else {
#pragma unroll
            for (int b = 0; b < 32; ++b) {
                const uint32_t alive = (r & (1u << b)) ? 0u : 0xffffffffu;
                r |= diag[b] & alive;
            }
        }
        const uint32_t valid_rows = rows >= 32 ? 0xffffffffu : ((1u << rows) - 1u);
        const uint32_t keepw = ~r & valid_rows;
        // kept rows of this block remove columns in the later words
#pragma unroll
        for (int b = 0; b < 32; ++b) removed |= (keepw & (1u << b)) ? col[b] : 0u;
        if (lane == 0) keep_words[w] = keepw;
    }
}

// Greedy NMS over a precomputed suppression bit matrix, resolved by the whole block in parallel rounds instead of a
// serial walk.  Thread i owns row i (NT == 32 * WORDS, n <= NT).  A box is certainly kept once every box that could
// suppress it is certainly removed, and certainly removed once a certainly kept box suppresses it; both sets only
// grow, every round settles at least the first undecided box, and the fixed point is the greedy result.  Random boxes
// need a handful of rounds.  or_words: 2 * WORDS words of shared memory.  keep_words[w] receives the keep bits.
template <int NT, int WORDS>
__device__ __forceinline__ void block_nms_resolve(const uint32_t* mask, int n, uint32_t* keep_words, uint32_t* or_words) {
    static_assert(NT == 32 * WORDS, "one thread per row, one warp per word");
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const bool valid = t < n;
    uint32_t row[WORDS];
    uint32_t any = 0u;
#pragma unroll
    for (int w = 0; w < WORDS; ++w) {
        row[w] = valid ? mask[t * WORDS + w] : 0u;
        any |= row[w];
    }
    uint32_t* maybe = or_words;            // boxes that a not-yet-removed box suppresses
    uint32_t* gone = or_words + WORDS;     // boxes that a kept box suppresses
    bool kept = false, removed = false;
    for (int round = 0; round <= n; ++round) {
        if (t < 2 * WORDS) or_words[t] = 0u;
        __syncthreads();
        if (__any_sync(kFullMask, any != 0u && !removed)) {
#pragma unroll
            for (int w = 0; w < WORDS; ++w) {
                const uint32_t v = __reduce_or_sync(kFullMask, removed ? 0u : row[w]);
                if (lane == w && v != 0u) atomicOr(&maybe[w], v);
            }
        }
        __syncthreads();
        kept = valid && !removed && ((maybe[warp] >> lane) & 1u) == 0u;
        if (__any_sync(kFullMask, any != 0u && kept)) {
#pragma unroll
            for (int w = 0; w < WORDS; ++w) {
                const uint32_t v = __reduce_or_sync(kFullMask, kept ? row[w] : 0u);
                if (lane == w && v != 0u) atomicOr(&gone[w], v);
            }
        }
        __syncthreads();
        removed = valid && ((gone[warp] >> lane) & 1u) != 0u;
        if (__syncthreads_or((valid && !kept && !removed) ? 1 : 0) == 0) break;
    }
    const uint32_t kw = __ballot_sync(kFullMask, kept);
    if (lane == 0) keep_words[warp] = kw;
}

}  // namespace fb
