// Masked index (threshold + compaction), top-k selection and greedy NMS as stand-alone launches.
// These are the un-fused ATen / torchvision steps that sit between the reference's fusion groups
// (nonzero, bool-mask index, sort, torchvision.ops.nms — reference call sites
// functs/benchmark/ai_model/yolov3/yolov3_bbox.py:122-134, 144-151, 177 and ssd/ssd_bbox.py:163-172, 212).
#include <atomic>

#include "select_nms.cuh"

namespace fb {

// ---- threshold + compaction -------------------------------------------------------------------
// grid.x = chunks per group, grid.y = group.  Each warp stages its hits in shared memory and reserves
// space in the group's list with one atomic per flush.
constexpr int kCompactThreads = 256;
constexpr int kCompactPerThread = 8;
constexpr int kWarpStage = 160;  // staged keys per warp; flushed when fewer than 32 slots remain

__device__ __forceinline__ void warp_stage_flush(uint64_t* stage, int& fill, uint64_t* keys, int32_t* count,
                                                 int64_t capacity, int32_t* status) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    int base = 0;
    if (lane == 0 && fill > 0) base = atomicAdd(count, fill);
    base = __shfl_sync(kFullMask, base, 0);
    for (int i = lane; i < fill; i += 32) {
        int64_t pos = static_cast<int64_t>(base) + i;
        if (pos < capacity) {
            keys[pos] = stage[i];
        } else if (status != nullptr) {
            atomicOr(status, FB_STATUS_CAND_OVERFLOW);
        }
    }
    __syncwarp();
    fill = 0;
}

// Appends key for lanes with pred, keeping `fill` identical on all lanes of the warp.
__device__ __forceinline__ void warp_stage_push(uint64_t* stage, int& fill, bool pred, uint64_t key) {
    unsigned m = __ballot_sync(kFullMask, pred);
    if (pred) {
        int off = __popc(m & ((1u << (threadIdx.x & 31)) - 1u));
        stage[fill + off] = key;
    }
    fill += __popc(m);
}

__global__ void __launch_bounds__(kCompactThreads)
threshold_compact_kernel(const float* __restrict__ scores, int64_t n, float thr, uint64_t* __restrict__ keys,
                         int32_t* __restrict__ counts, int64_t capacity, int32_t* status, int32_t* hist,
                         uint32_t hist_base, int hist_shift) {
    __shared__ uint64_t stage_all[kCompactThreads / 32][kWarpStage];
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    uint64_t* stage = stage_all[warp];
    int fill = 0;
    const float* s = scores + static_cast<int64_t>(g) * n;
    uint64_t* gkeys = keys + static_cast<int64_t>(g) * capacity;
    const int64_t chunk = static_cast<int64_t>(kCompactThreads) * kCompactPerThread;
    const int64_t start = static_cast<int64_t>(blockIdx.x) * chunk;
#pragma unroll
    for (int u = 0; u < kCompactPerThread; ++u) {
        int64_t i = start + static_cast<int64_t>(u) * kCompactThreads + threadIdx.x;
        float v = (i < n) ? s[i] : 0.0f;
        bool pred = (i < n) && (v > thr);
        const uint64_t key = make_key(v, static_cast<uint32_t>(i));
        if (pred && hist != nullptr) atomicAdd(hist + static_cast<int64_t>(g) * kHistBins + hist_digit(key, hist_base, hist_shift), 1);
        warp_stage_push(stage, fill, pred, key);
        if (fill + 32 > kWarpStage) warp_stage_flush(stage, fill, gkeys, counts + g, capacity, status);
    }
    warp_stage_flush(stage, fill, gkeys, counts + g, capacity, status);
}

// ---- top-k over candidate keys in global memory -----------------------------------------------
constexpr int kSelectThreads = 1024;
constexpr int kSelCap = 1024;

struct GlobalKeys {
    const uint64_t* p;
    __device__ __forceinline__ uint64_t operator()(int i) const { return p[i]; }
};

__global__ void __launch_bounds__(kSelectThreads)
select_topk_kernel(const uint64_t* __restrict__ in_keys, const int32_t* __restrict__ in_counts, int64_t capacity,
                   int32_t topk, uint64_t* __restrict__ out_keys, int32_t* __restrict__ out_counts) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SelectSmem<kSelCap>& sm = *reinterpret_cast<SelectSmem<kSelCap>*>(smem_raw);
    const int g = blockIdx.x;
    int64_t cnt = in_counts[g];
    if (cnt > capacity) cnt = capacity;
    if (cnt < 0) cnt = 0;
    GlobalKeys kf{in_keys + static_cast<int64_t>(g) * capacity};
    int m = block_select_topk<kSelectThreads, kSelCap, 4>(kf, static_cast<int>(cnt), topk, sm);
    for (int i = threadIdx.x; i < topk; i += kSelectThreads) {
        out_keys[static_cast<int64_t>(g) * topk + i] = (i < m) ? sm.sel[i] : 0ull;
    }
    if (threadIdx.x == 0) out_counts[g] = m;
}

// ---- NMS ----------------------------------------------------------------------------------------------------------
// The kernels work on the NMS-space boxes rebuilt from the selected keys: gather the box of every selected candidate,
// take the maximum coordinate over them, shift each box by label * (max + 1).
constexpr int kNmsMaxN = 1024;
constexpr int kNmsWords = kNmsMaxN / 32;
constexpr int kMaskThreads = 256;
constexpr int kMaskCtasMax = 16;       // CTAs per group in the matrix kernel (rows interleaved); the launcher picks
                                       // the largest count that keeps the whole grid resident at once
constexpr int kMaskMaxBuckets = 1024; // class buckets used for pruning (more classes than this: one bucket)
constexpr int kScanChunk = 256;       // non-empty matrix rows staged in shared memory at a time

// ---- suppression matrix ------------------------------------------------------------------------------------------
// Class pruning.  With class offsets, class c occupies the coordinate range [c*M + lo, c*M + hi] (M = hi + 1, lo / hi the
// extreme coordinates of the selected boxes), so boxes whose labels differ by more than K = floor((hi - lo) / M) + 1
// cannot intersect.  The candidates are bucketed by label (counting sort) and a row only tests the members of the
// buckets within K of its own label; every pair that can intersect is still tested with the exact IoU expression, so
// the matrix is the same as the one an all-pairs loop produces.
//
// nms_prepare_block (run by the CTA that finishes a group's top-k selection, or by nms_prepare_kernel when the selected
// keys come from elsewhere) gathers the selected boxes, applies the class offsets, and leaves the boxes, their buckets
// and the bucket order in scratch; nms_mask_scan_kernel (up to kMaskCtasMax CTAs per group) copies that into shared memory and
// computes its share of the rows; the CTA of a group that finishes last then runs the greedy scan.
struct NmsPrepHeader {
    int n, nb, reach, pad;
};
constexpr int64_t kPrepBoxesOff = 16;
constexpr int64_t kPrepLabelOff = kPrepBoxesOff + static_cast<int64_t>(kNmsMaxN) * sizeof(NmsBox);
constexpr int64_t kPrepOrderOff = kPrepLabelOff + kNmsMaxN * 2;
constexpr int64_t kPrepStartOff = kPrepOrderOff + kNmsMaxN * 2;
// one bit per candidate: its key named a box outside [0, num_boxes) (the candidate then takes no part in the NMS)
constexpr int64_t kPrepInvalidOff = kPrepStartOff + (kMaskMaxBuckets + 1) * 4;
constexpr int64_t kPrepBytes = (kPrepInvalidOff + kNmsWords * 4 + 255) / 256 * 256;
static_assert(sizeof(NmsBox) == 20 && kPrepBoxesOff % 16 == 0 && kPrepLabelOff % 16 == 0 && kPrepOrderOff % 16 == 0 &&
                  kPrepStartOff % 4 == 0 && kPrepInvalidOff % 4 == 0 && kPrepBytes % 256 == 0 && kPrepBytes == 28928,
              "prepared NMS input layout");

template <int NT>
struct NmsPrepSmem {
    uint16_t slabel[kNmsMaxN];
    int bcursor[kMaskMaxBuckets];
    float red_hi[NT / 32 + 1], red_lo[NT / 32 + 1];
};

// All NT threads of a CTA.  sel: the group's n selected keys, sorted (shared or global memory); boxes_g: the group's
// num_boxes boxes; prep: the group's prepared-input record; ticket: the group's arrival counter of the matrix kernel
// (cleared).  A key whose box index is not below num_boxes (a stale or malformed key: the keys are caller-supplied) is
// never used as an address: the candidate gets a zero box, is marked invalid in the record (the scan treats it as
// removed from the start, so it neither survives nor suppresses) and FB_STATUS_INDEX_RANGE is set in `status`.
template <int NT>
__device__ __forceinline__ void nms_prepare_block(const float* __restrict__ boxes_g, int64_t num_boxes, int num_classes,
                                                  int class_offset, const uint64_t* sel, int n,
                                                  unsigned char* __restrict__ prep, int32_t* ticket, int32_t* status,
                                                  NmsPrepSmem<NT>& ps) {
    uint16_t* slabel = ps.slabel;
    int* bcursor = ps.bcursor;
    float* red_hi = ps.red_hi;
    float* red_lo = ps.red_lo;
    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    NmsBox* pb = reinterpret_cast<NmsBox*>(prep + kPrepBoxesOff);
    uint16_t* plabel = reinterpret_cast<uint16_t*>(prep + kPrepLabelOff);
    uint16_t* porder = reinterpret_cast<uint16_t*>(prep + kPrepOrderOff);
    int* pstart = reinterpret_cast<int*>(prep + kPrepStartOff);
    uint32_t* pinvalid = reinterpret_cast<uint32_t*>(prep + kPrepInvalidOff);
    const int nb = (class_offset && num_classes <= kMaskMaxBuckets) ? num_classes : 1;
    static_assert(NT % 32 == 0, "a warp covers 32 consecutive candidates");

    // gather: thread t owns candidates t, t + NT, ...
    constexpr int kPer = kNmsMaxN / NT;
    float4 bx[kPer];
    int label[kPer];
    float lmax = -INFINITY, lmin = INFINITY;
    for (int i = t; i < nb; i += NT) bcursor[i] = 0;
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
        const int c = t + q * NT;
        bx[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        label[q] = 0;
        bool bad = false;
        if (c < n) {
            const uint32_t flat = key_index(sel[c]);
            const uint32_t box = flat / static_cast<uint32_t>(num_classes);
            label[q] = static_cast<int>(flat - box * static_cast<uint32_t>(num_classes));
            bad = static_cast<int64_t>(box) >= num_boxes;
            if (!bad) {
                bx[q] = reinterpret_cast<const float4*>(boxes_g)[box];
                lmax = fmaxf(lmax, fmaxf(fmaxf(bx[q].x, bx[q].y), fmaxf(bx[q].z, bx[q].w)));
                lmin = fminf(lmin, fminf(fminf(bx[q].x, bx[q].y), fminf(bx[q].z, bx[q].w)));
            }
        }
        const unsigned bad_word = __ballot_sync(kFullMask, bad);
        if (lane == 0) {
            pinvalid[(t >> 5) + q * (NT / 32)] = bad_word;
            if (bad_word != 0u && status != nullptr) atomicOr(status, FB_STATUS_INDEX_RANGE);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lmax = fmaxf(lmax, __shfl_xor_sync(kFullMask, lmax, o));
        lmin = fminf(lmin, __shfl_xor_sync(kFullMask, lmin, o));
    }
    if (lane == 0) {
        red_hi[warp] = lmax;
        red_lo[warp] = lmin;
    }
    __syncthreads();
    if (t < 32) {
        float v = (t < NT / 32) ? red_hi[t] : -INFINITY;
        float u = (t < NT / 32) ? red_lo[t] : INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
            u = fminf(u, __shfl_xor_sync(kFullMask, u, o));
        }
        if (t == 0) {
            red_hi[NT / 32] = v;
            red_lo[NT / 32] = u;
        }
    }
    __syncthreads();
    const float hi = red_hi[NT / 32], lo = red_lo[NT / 32];
    const float scale = __fadd_rn(hi, 1.0f);
    // label distance beyond which two boxes cannot intersect (one extra bucket covers the fp32 rounding of the shifts)
    int reach = nb;
    if (nb > 1 && scale > 0.0f) {
        const float r = floorf((hi - lo) / scale) + 1.0f;
        if (r < static_cast<float>(nb)) reach = static_cast<int>(r);
    }
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
        const int c = t + q * NT;
        if (c < n) {
            const float off = class_offset ? __fmul_rn(static_cast<float>(label[q]), scale) : 0.0f;
            pb[c] = make_nms_box(__fadd_rn(bx[q].x, off), __fadd_rn(bx[q].y, off), __fadd_rn(bx[q].z, off),
                                 __fadd_rn(bx[q].w, off));
            const int bucket = nb > 1 ? label[q] : 0;
            slabel[c] = static_cast<uint16_t>(bucket);
            plabel[c] = static_cast<uint16_t>(bucket);
            atomicAdd(&bcursor[bucket], 1);
        }
    }
    __syncthreads();
    // exclusive prefix of the bucket counts (one warp, contiguous chunk per lane), then the scatter
    if (warp == 0) {
        const int per = (nb + 31) / 32;
        const int b0 = lane * per, b1 = min(nb, b0 + per);
        int s = 0;
        for (int i = b0; i < b1; ++i) s += bcursor[i];
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += v;
        }
        int run = incl - s;
        for (int i = b0; i < b1; ++i) {
            const int c = bcursor[i];
            pstart[i] = run;
            bcursor[i] = run;
            run += c;
        }
        if (lane == 31) pstart[nb] = incl;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
        const int c = t + q * NT;
        if (c < n) porder[atomicAdd(&bcursor[slabel[c]], 1)] = static_cast<uint16_t>(c);
    }
    if (t == 0) {
        NmsPrepHeader h;
        h.n = n;
        h.nb = nb;
        h.reach = reach;
        h.pad = 0;
        *reinterpret_cast<NmsPrepHeader*>(prep) = h;
        *ticket = 0;
    }
}

// grid = groups; block = 256.  For selected keys that did not come from select_binned_kernel.
__global__ void __launch_bounds__(kMaskThreads)
nms_prepare_kernel(const float* __restrict__ boxes, int64_t num_boxes, int num_classes, const uint64_t* __restrict__ sel_keys,
                   const int32_t* __restrict__ sel_counts, int topk, int class_offset, unsigned char* __restrict__ prep_g,
                   int32_t* __restrict__ ticket_g, int32_t* status) {
    __shared__ NmsPrepSmem<kMaskThreads> ps;
    const int g = blockIdx.x;
    int n = sel_counts[g];
    if (n > topk) n = topk;
    if (n < 0) n = 0;
    nms_prepare_block<kMaskThreads>(boxes + static_cast<int64_t>(g) * num_boxes * 4, num_boxes, num_classes, class_offset,
                                    sel_keys + static_cast<int64_t>(g) * topk, n, prep_g + static_cast<int64_t>(g) * kPrepBytes,
                                    ticket_g + g, status, ps);
}



// ---- binned top-k: many CTAs per group collect, the last one to finish sorts --------------------------------
// Needs the coarse score histogram that the candidate producer filled (hist[g][kHistBins]).  Every CTA finds the
// boundary bucket d* (the largest d with count(digit >= d) >= topk), scans its share of the candidate list and
// appends keys above d* to the group's `sel` list and keys inside d* to its `bin` list.  CTAs then take a ticket;
// the one that draws the last ticket sorts the bin list, tops `sel` up from it and writes the sorted result (if the
// lists turn out not to fit the histogram, or the boundary bucket is too crowded, it runs the exact generic selection
// over the whole candidate list instead), and, when asked to, prepares the group's NMS input (nms_prepare_block).
// No CTA ever waits for another one.
constexpr int kBinThreads = 512;
constexpr int kBinSplit = 4;         // CTAs per group
constexpr int kBinListGlobal = 2048; // capacity of the boundary-bucket list; beyond it the generic selection runs

struct SelectCtr {
    int32_t sel_cnt, bin_cnt, ticket;
    int32_t fallback;  // set to 1 when the group was finished by the generic selection (observability only)
};

struct BinnedSmem {
    uint64_t sel[kSelCap];
    uint64_t bin[kBinListGlobal];
    int hist[kHistBins];
};

__global__ void __launch_bounds__(kBinThreads, 2)
select_binned_kernel(const uint64_t* __restrict__ in_keys, const int32_t* __restrict__ in_counts, int64_t capacity,
                     const int32_t* __restrict__ hist, uint32_t hist_base, int hist_shift, int32_t topk,
                     SelectCtr* ctr, uint64_t* sel_tmp, uint64_t* bin_tmp, uint64_t* __restrict__ out_keys,
                     int32_t* __restrict__ out_counts, const float* __restrict__ nms_boxes, int64_t num_boxes,
                     int num_classes, int class_offset, unsigned char* __restrict__ prep_g, int32_t* __restrict__ ticket_g,
                     int32_t* status) {
    constexpr size_t kRaw = sizeof(BinnedSmem) > sizeof(SelectSmem<kSelCap>) ? sizeof(BinnedSmem) : sizeof(SelectSmem<kSelCap>);
    static_assert(sizeof(uint64_t) * kSelCap + sizeof(NmsPrepSmem<kBinThreads>) <= kRaw, "NMS preparation reuses the buffer");
    __shared__ __align__(16) unsigned char raw[kRaw];
    BinnedSmem& sm = *reinterpret_cast<BinnedSmem*>(raw);  // .sel is the first member of both views
    __shared__ int s_dstar, s_above, s_inbin, s_last;
    const int g = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the group's histogram (four buckets per thread) does not depend on anything: ask for it first, together with
    // the candidate count, so that the two round trips overlap
    static_assert(kHistBins == 4 * kBinThreads, "four histogram buckets per thread");
    const int4 hv = __ldcg(reinterpret_cast<const int4*>(hist + static_cast<int64_t>(g) * kHistBins) + tid);
    int64_t cnt64 = in_counts[g];
    if (cnt64 > capacity) cnt64 = capacity;
    if (cnt64 < 0) cnt64 = 0;
    const int n = static_cast<int>(cnt64);
    const uint64_t* keys = in_keys + static_cast<int64_t>(g) * capacity;
    // this CTA's share of the keys: the first two batches are requested now and looked at once the boundary is known
    const int lo = static_cast<int>(static_cast<int64_t>(n) * blockIdx.x / gridDim.x);
    const int hi = static_cast<int>(static_cast<int64_t>(n) * (blockIdx.x + 1) / gridDim.x);
    constexpr int kPre = 8;
    uint64_t pre[kPre];
#pragma unroll
    for (int u = 0; u < kPre; ++u) {
        const int i = lo + u * kBinThreads + tid;
        pre[u] = (i < hi) ? __ldg(keys + i) : 0ull;
    }
    __shared__ int s_wsum[kBinThreads / 32];
    if (tid == 0) {
        s_dstar = -1;  // n <= topk: everything is "above"
        s_above = n;
        s_inbin = 0;
    }
    {
        // boundary bucket: the largest d with (keys in buckets >= d) >= topk; suffix sums over the block
        const int s4 = hv.x + hv.y + hv.z + hv.w;
        int incl = s4;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_down_sync(kFullMask, incl, o);
            if (lane + o < 32) incl += v;
        }
        if (lane == 0) s_wsum[warp] = incl;
        __syncthreads();
        for (int w = warp + 1; w < kBinThreads / 32; ++w) incl += s_wsum[w];
        const int suf = incl - s4;
        if (n > topk && suf < topk && incl >= topk) {
            int cum = suf, d = 3, inb = hv.w;
            if (cum + hv.w < topk) {
                cum += hv.w;
                d = 2;
                inb = hv.z;
                if (cum + hv.z < topk) {
                    cum += hv.z;
                    d = 1;
                    inb = hv.y;
                    if (cum + hv.y < topk) {
                        cum += hv.y;
                        d = 0;
                        inb = hv.x;
                    }
                }
            }
            s_dstar = tid * 4 + d;
            s_above = cum;
            s_inbin = inb;
        }
    }
    __shared__ int s_nsel, s_nbin, s_bsel, s_bbin;
    if (tid == 0) {
        s_nsel = 0;
        s_nbin = 0;
    }
    __syncthreads();
    const int dstar = s_dstar;
    SelectCtr* c = ctr + g;
    uint64_t* gsel = sel_tmp + static_cast<int64_t>(g) * kSelCap;
    uint64_t* gbin = bin_tmp + static_cast<int64_t>(g) * kBinListGlobal;
    // collect this CTA's share into shared-memory lists first (one shared atomic per warp and list), then reserve
    // space in the group's global lists with ONE atomic per list and copy
    {
        const unsigned lt = (1u << lane) - 1u;
        auto place = [&](uint64_t k) {  // called by whole warps
            const int d = k != 0ull ? hist_digit(k, hist_base, hist_shift) : -2;
            const bool up = d > dstar, in = d == dstar;
            const unsigned mu = __ballot_sync(kFullMask, up), mi = __ballot_sync(kFullMask, in);
            if (mu != 0u) {
                int base = 0;
                if (lane == 0) base = atomicAdd(&s_nsel, __popc(mu));
                base = __shfl_sync(kFullMask, base, 0);
                const int pos = base + __popc(mu & lt);
                if (up && pos < kSelCap) sm.sel[pos] = k;
            }
            if (mi != 0u) {
                int base = 0;
                if (lane == 0) base = atomicAdd(&s_nbin, __popc(mi));
                base = __shfl_sync(kFullMask, base, 0);
                const int pos = base + __popc(mi & lt);
                if (in && pos < kBinListGlobal) sm.bin[pos] = k;
            }
        };
#pragma unroll
        for (int u = 0; u < kPre; ++u) place(pre[u]);
        for (int base = lo + kPre * kBinThreads; base < hi; base += kBinThreads * 4) {
            uint64_t k[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * kBinThreads + tid;
                k[u] = (i < hi) ? __ldg(keys + i) : 0ull;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) place(k[u]);
        }
    }
    __syncthreads();
    if (tid == 0) {
        s_bsel = s_nsel > 0 ? atomicAdd(&c->sel_cnt, s_nsel) : 0;
        s_bbin = s_nbin > 0 ? atomicAdd(&c->bin_cnt, s_nbin) : 0;
    }
    __syncthreads();
    for (int i = tid; i < min(s_nsel, kSelCap); i += kBinThreads)
        if (s_bsel + i < kSelCap) gsel[s_bsel + i] = sm.sel[i];
    for (int i = tid; i < min(s_nbin, kBinListGlobal); i += kBinThreads)
        if (s_bbin + i < kBinListGlobal) gbin[s_bbin + i] = sm.bin[i];
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&c->ticket, 1) == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- the last CTA of the group finishes the selection ----
    const int sel_cnt = *reinterpret_cast<volatile int32_t*>(&c->sel_cnt);
    const int bin_cnt = *reinterpret_cast<volatile int32_t*>(&c->bin_cnt);
    const bool consistent = (n <= topk) ? (sel_cnt == n && sel_cnt <= kSelCap)
                                        : (sel_cnt == s_above && bin_cnt == s_inbin && sel_cnt < topk &&
                                           sel_cnt + bin_cnt >= topk && bin_cnt <= kBinListGlobal);
    int result = n < topk ? n : topk;
    if (!consistent) {
        // the boundary bucket is too crowded (many equal scores) or the histogram does not describe this list:
        // exact generic selection over the whole list (rare, slow)
        if (tid == 0) c->fallback = 1;
        __syncthreads();
        GlobalKeys kf{keys};
        result = block_select_topk<kBinThreads, kSelCap, 4>(kf, n, topk, *reinterpret_cast<SelectSmem<kSelCap>*>(raw));
        __syncthreads();
    } else {
        for (int i = tid; i < sel_cnt; i += kBinThreads) sm.sel[i] = __ldcg(gsel + i);
        if (n > topk) {
            const int bn = next_pow2(bin_cnt);
            for (int i = tid; i < bn; i += kBinThreads) sm.bin[i] = (i < bin_cnt) ? __ldcg(gbin + i) : 0ull;
            __syncthreads();
            bitonic_sort_desc<kBinThreads>(sm.bin, bn);
            const int want = topk - sel_cnt;
            for (int i = tid; i < want; i += kBinThreads) sm.sel[sel_cnt + i] = sm.bin[i];
        }
        // sm.sel[0 .. sel_cnt) holds the keys above the boundary bucket in arrival order, the sorted tail from the
        // boundary bucket follows.  Order the head by counting sort on the score buckets (higher bucket = higher
        // score) plus a rank count inside every bucket; a crowded bucket falls back to the bitonic network.
        __syncthreads();
        int* cnt = sm.hist;                                     // the staged histogram is not needed any more
        uint64_t* tmp = sm.bin;                                 // nor the boundary list: first half = keys,
        int* cursor = reinterpret_cast<int*>(sm.bin + kSelCap);  // second half = running positions
        for (int i = tid; i < kHistBins; i += kBinThreads) cnt[i] = 0;
        __syncthreads();
        for (int i = tid; i < sel_cnt; i += kBinThreads) atomicAdd(&cnt[hist_digit(sm.sel[i], hist_base, hist_shift)], 1);
        __syncthreads();
        constexpr int kPerThread = kHistBins / kBinThreads;
        int c[kPerThread];
        int mine = 0, crowded = 0;
#pragma unroll
        for (int q = 0; q < kPerThread; ++q) {
            c[q] = cnt[tid * kPerThread + q];
            mine += c[q];
            crowded |= c[q] > 32 ? 1 : 0;
        }
        // keys in higher buckets come first: exclusive suffix sum over threads (buckets ascend with tid)
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_down_sync(kFullMask, incl, o);
            if (lane + o < 32) incl += v;
        }
        __shared__ int warp_sum[kBinThreads / 32];
        if (lane == 0) warp_sum[warp] = incl;
        crowded = __syncthreads_or(crowded);
        int above = incl - mine;
        for (int w = warp + 1; w < kBinThreads / 32; ++w) above += warp_sum[w];
#pragma unroll
        for (int q = kPerThread - 1; q >= 0; --q) {
            cursor[tid * kPerThread + q] = above;
            above += c[q];
        }
        __syncthreads();
        if (!crowded) {
            for (int i = tid; i < sel_cnt; i += kBinThreads) {
                const uint64_t k = sm.sel[i];
                tmp[atomicAdd(&cursor[hist_digit(k, hist_base, hist_shift)], 1)] = k;
            }
            __syncthreads();
            // inside a bucket: every key counts the larger keys of its bucket's segment (keys are distinct) and
            // goes straight to its final place
            for (int i = tid; i < sel_cnt; i += kBinThreads) {
                const uint64_t k = tmp[i];
                const int bkt = hist_digit(k, hist_base, hist_shift);
                const int end = cursor[bkt], begin = end - cnt[bkt];
                int r = begin;
                for (int j = begin; j < end; ++j) r += tmp[j] > k ? 1 : 0;
                sm.sel[r] = k;
            }
            __syncthreads();
        } else {
            const int sn = next_pow2(result);
            for (int i = result + tid; i < sn; i += kBinThreads) sm.sel[i] = 0ull;
            __syncthreads();
            bitonic_sort_desc<kBinThreads>(sm.sel, sn);
        }
    }
    for (int i = tid; i < topk; i += kBinThreads) out_keys[static_cast<int64_t>(g) * topk + i] = (i < result) ? sm.sel[i] : 0ull;
    if (tid == 0) out_counts[g] = result;
    if (prep_g != nullptr) {
        __syncthreads();
        NmsPrepSmem<kBinThreads>& ps = *reinterpret_cast<NmsPrepSmem<kBinThreads>*>(raw + sizeof(uint64_t) * kSelCap);
        nms_prepare_block<kBinThreads>(nms_boxes + static_cast<int64_t>(g) * num_boxes * 4, num_boxes, num_classes,
                                       class_offset, sm.sel, result, prep_g + static_cast<int64_t>(g) * kPrepBytes,
                                       ticket_g + g, status, ps);
    }
}

// grid = (CTAs per group, groups); block = 256.  Rows are interleaved over the CTAs of a group (i = k * gridDim.x +
// blockIdx.x).  Each CTA writes its rows of the suppression matrix (and one flag per row: does the row suppress
// anything at all?), then takes a ticket; the CTA that draws the group's last ticket runs the greedy scan: only rows
// with at least one set bit can remove anything, so the flagged rows are listed in ascending order, staged in shared
// memory kScanChunk at a time, and one warp walks them (row i is applied unless box i has been removed already; lane l
// keeps the removed bits of boxes 32l .. 32l+31).  All threads of that CTA then write the compacted outputs.
// No CTA waits for another one.
struct NmsRowsSmem {
    __align__(16) NmsBox sb[kNmsMaxN];
    __align__(16) uint16_t slabel[kNmsMaxN];  // bucket of every candidate
    __align__(16) uint16_t order[kNmsMaxN];   // candidates grouped by bucket
    int bstart[kMaskMaxBuckets + 1];
    uint32_t rowbuf[kMaskThreads / 32][kNmsWords];
};
struct NmsScanSmem {
    uint32_t srow[kScanChunk][kNmsWords];
    uint16_t nzrow[kNmsMaxN];
    int part[kNmsMaxN / 32 + 1];
    uint32_t keep_words[kNmsWords];
    int word_prefix[kNmsWords + 1];
};

__global__ void __launch_bounds__(kMaskThreads)
nms_mask_scan_kernel(const unsigned char* __restrict__ prep_g, float thr, float thr_lo, float thr_hi,
                     uint32_t* __restrict__ mask_g, uint8_t* __restrict__ rowflag_g, int32_t* __restrict__ ticket_g,
                     const float* __restrict__ boxes, int64_t num_boxes, int num_classes,
                     const uint64_t* __restrict__ sel_keys, int topk, float* __restrict__ dets,
                     int64_t* __restrict__ labels, int64_t* __restrict__ flat_ids, int64_t* __restrict__ keep,
                     int32_t* __restrict__ out_counts, int4* __restrict__ records) {
    constexpr size_t kRaw = sizeof(NmsRowsSmem) > sizeof(NmsScanSmem) ? sizeof(NmsRowsSmem) : sizeof(NmsScanSmem);
    __shared__ __align__(16) unsigned char raw[kRaw];
    __shared__ int s_last;
    NmsRowsSmem& rs = *reinterpret_cast<NmsRowsSmem*>(raw);
    const int g = blockIdx.y;
    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    const unsigned char* prep = prep_g + static_cast<int64_t>(g) * kPrepBytes;
    const NmsPrepHeader h = *reinterpret_cast<const NmsPrepHeader*>(prep);
    // the record comes from memory: whatever it holds, nothing below indexes beyond the shared arrays
    const int n = min(max(h.n, 0), kNmsMaxN), nb = min(max(h.nb, 1), kMaskMaxBuckets), reach = max(h.reach, 0);
    const int rt = gridDim.x;
    uint32_t* gmask = mask_g + static_cast<int64_t>(g) * kNmsMaxN * kNmsWords;
    uint8_t* gflag = rowflag_g + static_cast<int64_t>(g) * kNmsMaxN;
    if (static_cast<int>(blockIdx.x) < n) {  // otherwise this CTA owns no row
        {
            // boxes (5 words each), buckets and order (8 candidates per 16 bytes), bucket starts: 16-byte copies
            // (rounded up: the record and the shared arrays are padded to multiples of 16 bytes)
            const uint4* src = reinterpret_cast<const uint4*>(prep + kPrepBoxesOff);
            uint4* dst = reinterpret_cast<uint4*>(rs.sb);
            for (int i = t; i < (n * 5 + 3) / 4; i += kMaskThreads) dst[i] = __ldg(src + i);
            const uint4* lsrc = reinterpret_cast<const uint4*>(prep + kPrepLabelOff);
            const uint4* osrc = reinterpret_cast<const uint4*>(prep + kPrepOrderOff);
            uint4* ldst = reinterpret_cast<uint4*>(rs.slabel);
            uint4* odst = reinterpret_cast<uint4*>(rs.order);
            for (int i = t; i < (n + 7) / 8; i += kMaskThreads) {
                ldst[i] = __ldg(lsrc + i);
                odst[i] = __ldg(osrc + i);
            }
            const int* ssrc = reinterpret_cast<const int*>(prep + kPrepStartOff);
            for (int i = t; i <= nb; i += kMaskThreads) rs.bstart[i] = __ldg(ssrc + i);
        }
        __syncthreads();
        uint32_t* myrow = rs.rowbuf[warp];
        for (int i = warp * rt + static_cast<int>(blockIdx.x); i < n; i += (kMaskThreads / 32) * rt) {
            const NmsBox bi = rs.sb[i];
            const int li = min(static_cast<int>(rs.slabel[i]), nb - 1);
            const int p0 = max(rs.bstart[max(li - reach, 0)], 0), p1 = min(rs.bstart[min(li + reach + 1, nb)], n);
            myrow[lane] = 0u;
            __syncwarp();
            for (int base = p0; base < p1; base += 32) {
                const int p = base + lane;
                if (p < p1) {
                    const int j = rs.order[p];
                    if (j > i && j < n && iou_exceeds(bi, rs.sb[j], thr, thr_lo, thr_hi)) atomicOr(&myrow[j >> 5], 1u << (j & 31));
                }
            }
            __syncwarp();
            const uint32_t mw = myrow[lane];
            gmask[i * kNmsWords + lane] = mw;
            const bool any = __any_sync(kFullMask, mw != 0u);
            if (lane == 0) gflag[i] = any ? 1 : 0;
            __syncwarp();
        }
    }
    __threadfence();
    __syncthreads();
    if (t == 0) s_last = (atomicAdd(ticket_g + g, 1) == rt - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- the group's last CTA: greedy scan + outputs ----
    NmsScanSmem& ss = *reinterpret_cast<NmsScanSmem*>(raw);
    const float* boxes_g = boxes + static_cast<int64_t>(g) * num_boxes * 4;
    const uint64_t* sel = sel_keys + static_cast<int64_t>(g) * topk;
    // ascending list of the non-empty rows (candidate c = q * 256 + t)
    constexpr int kRounds = kNmsMaxN / kMaskThreads;
    bool nz[kRounds];
    unsigned nzm[kRounds];
    // the output rows of this thread's candidates do not depend on the scan: fetch key and box now, use them after it
    uint64_t okey[kRounds];
    float4 obox[kRounds];
#pragma unroll
    for (int q = 0; q < kRounds; ++q) {
        const int c = q * kMaskThreads + t;
        okey[q] = c < n ? sel[c] : 0ull;
    }
#pragma unroll
    for (int q = 0; q < kRounds; ++q) {
        const int c = q * kMaskThreads + t;
        obox[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n) {
            // an out-of-range box index is never dereferenced; such a candidate is marked invalid and not written out
            const uint32_t box = key_index(okey[q]) / static_cast<uint32_t>(num_classes);
            if (static_cast<int64_t>(box) < num_boxes) obox[q] = reinterpret_cast<const float4*>(boxes_g)[box];
        }
    }
#pragma unroll
    for (int q = 0; q < kRounds; ++q) {
        const int c = q * kMaskThreads + t;
        nz[q] = c < n && __ldcg(gflag + c) != 0;
        nzm[q] = __ballot_sync(kFullMask, nz[q]);
        if (lane == 0) ss.part[q * (kMaskThreads / 32) + warp] = __popc(nzm[q]);
    }
    __syncthreads();
    int nz_total = 0;
    int before[kRounds];
#pragma unroll
    for (int q = 0; q < kRounds; ++q) before[q] = 0;
    for (int w = 0; w < kNmsMaxN / 32; ++w) {
        const int cnt = ss.part[w];
#pragma unroll
        for (int q = 0; q < kRounds; ++q) before[q] += (w < q * (kMaskThreads / 32) + warp) ? cnt : 0;
        nz_total += cnt;
    }
#pragma unroll
    for (int q = 0; q < kRounds; ++q)
        if (nz[q]) ss.nzrow[before[q] + __popc(nzm[q] & ((1u << lane) - 1u))] = static_cast<uint16_t>(q * kMaskThreads + t);
    __syncthreads();
    // warp 0: lane l holds the removed bits of boxes 32l .. 32l+31; invalid candidates start out removed
    uint32_t removed = (warp == 0) ? __ldcg(reinterpret_cast<const uint32_t*>(prep + kPrepInvalidOff) + lane) : 0u;
    for (int c0 = 0; c0 < nz_total; c0 += kScanChunk) {
        const int rows = min(kScanChunk, nz_total - c0);
        if (t < rows) {  // one thread per row: eight 16-byte loads (L2-resident: just written)
            const uint4* src = reinterpret_cast<const uint4*>(gmask + static_cast<int64_t>(ss.nzrow[c0 + t]) * kNmsWords);
            uint4* dst = reinterpret_cast<uint4*>(&ss.srow[t][0]);
#pragma unroll
            for (int q = 0; q < kNmsWords / 4; ++q) dst[q] = __ldcg(src + q);
        }
        __syncthreads();
        if (warp == 0) {
            for (int j0 = 0; j0 < rows; j0 += 32) {
                const int mine = (j0 + lane < rows) ? ss.nzrow[c0 + j0 + lane] : 0;  // row numbers of the next 32 entries
                const int cnt = min(32, rows - j0);
                for (int j = 0; j < cnt; ++j) {
                    const int i = __shfl_sync(kFullMask, mine, j);
                    const uint32_t rw = __shfl_sync(kFullMask, removed, i >> 5);
                    const uint32_t row = ss.srow[j0 + j][lane];
                    if (!((rw >> (i & 31)) & 1u)) removed |= row;
                }
            }
        }
        __syncthreads();
    }
    if (warp == 0) {
        const int lo = lane * 32;
        const uint32_t valid = n >= lo + 32 ? 0xffffffffu : (n > lo ? ((1u << (n - lo)) - 1u) : 0u);
        const uint32_t kw = ~removed & valid;
        ss.keep_words[lane] = kw;
        // exclusive prefix of the kept counts
        int incl = __popc(kw);
        const int own = incl;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += v;
        }
        ss.word_prefix[lane] = incl - own;
        if (lane == 31) {
            ss.word_prefix[kNmsWords] = incl;
            out_counts[g] = incl;
        }
    }
    __syncthreads();
    const int64_t obase = static_cast<int64_t>(g) * topk;
#pragma unroll
    for (int q = 0; q < kRounds; ++q) {
        const int c = q * kMaskThreads + t;
        if (c >= n) continue;
        const uint32_t kw = ss.keep_words[c >> 5];
        const int b = c & 31;
        if ((kw >> b) & 1u) {
            const uint64_t k = okey[q];
            const uint32_t flat = key_index(k);
            const uint32_t box = flat / static_cast<uint32_t>(num_classes);
            const float4 bx = obox[q];
            const int rank = ss.word_prefix[c >> 5] + __popc(kw & ((1u << b) - 1u));
            float* d = dets + (obase + rank) * 5;
            d[0] = bx.x;
            d[1] = bx.y;
            d[2] = bx.z;
            d[3] = bx.w;
            d[4] = key_score(k);
            labels[obase + rank] = static_cast<int64_t>(flat - box * static_cast<uint32_t>(num_classes));
            flat_ids[obase + rank] = static_cast<int64_t>(flat);
            if (keep != nullptr) keep[obase + rank] = c;
            if (records != nullptr) {  // the 32-byte record of the multi-GPU gather (layout of pack_detections_kernel)
                records[2 * (obase + rank)] = make_int4(__float_as_int(bx.x), __float_as_int(bx.y), __float_as_int(bx.z),
                                                        __float_as_int(bx.w));
                records[2 * (obase + rank) + 1] = make_int4(__float_as_int(key_score(k)),
                                                            static_cast<int>(flat - box * static_cast<uint32_t>(num_classes)),
                                                            static_cast<int>(flat), 1);
            }
        }
    }
    // zero the tail so that the padded outputs are deterministic
    const int total_kept = ss.word_prefix[kNmsWords];
    for (int i = total_kept + t; i < topk; i += kMaskThreads) {
        float* d = dets + (obase + i) * 5;
        d[0] = d[1] = d[2] = d[3] = d[4] = 0.0f;
        labels[obase + i] = -1;
        flat_ids[obase + i] = -1;
        if (keep != nullptr) keep[obase + i] = -1;
        if (records != nullptr) {
            records[2 * (obase + i)] = make_int4(0, 0, 0, 0);
            records[2 * (obase + i) + 1] = make_int4(0, -1, -1, 0);
        }
    }
}

// ---- host launchers (internal C++ API, used by the C ABI and by the YOLO pipeline) ----------------
int launch_threshold_compact(const float* scores, int groups, int64_t n, float thr, uint64_t* keys, int32_t* counts,
                             int64_t capacity, int zero_counts, int32_t* hist, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(scores && keys && counts, "threshold_compact: null pointer");
    FB_REQUIRE(groups > 0 && groups <= 65535 && n > 0 && n < (1ll << 32) && capacity > 0, "threshold_compact: bad sizes");
    FB_REQUIRE(thr > 0.0f, "threshold_compact: the threshold must be positive (keys need positive scores)");
    if (zero_counts) {
        FB_TRY(check_cuda(cudaMemsetAsync(counts, 0, sizeof(int32_t) * groups, st), "memset counts"));
        if (hist != nullptr)
            FB_TRY(check_cuda(cudaMemsetAsync(hist, 0, sizeof(int32_t) * groups * kHistBins, st), "memset hist"));
    }
    const HistParams hp = hist_params_for(thr);
    const int64_t chunk = static_cast<int64_t>(kCompactThreads) * kCompactPerThread;
    dim3 grid(static_cast<unsigned>((n + chunk - 1) / chunk), groups);
    threshold_compact_kernel<<<grid, kCompactThreads, 0, st>>>(scores, n, thr, keys, counts, capacity, status, hist, hp.base,
                                                               hp.shift);
    count_launch();
    return check_launch("threshold_compact_kernel");
}

int launch_select_topk(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, int groups, int topk,
                       uint64_t* out_keys, int32_t* out_counts, cudaStream_t st) {
    FB_REQUIRE(in_keys && in_counts && out_keys && out_counts, "select_topk: null pointer");
    FB_REQUIRE(groups > 0 && topk > 0 && topk <= kSelCap && capacity > 0 && capacity < (1ll << 31),
               "select_topk: bad sizes (topk must be in [1, %d])", kSelCap);
    const size_t smem = sizeof(SelectSmem<kSelCap>);
    FB_TRY(check_cuda(cudaFuncSetAttribute(select_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "select_topk attr"));
    select_topk_kernel<<<groups, kSelectThreads, smem, st>>>(in_keys, in_counts, capacity, topk, out_keys, out_counts);
    count_launch();
    return check_launch("select_topk_kernel");
}

// Work area of the binned selection: [SelectCtr x groups (padded to 256 B)][sel lists][bin lists].
int64_t select_binned_ctr_bytes(int groups) { return (static_cast<int64_t>(groups) * sizeof(SelectCtr) + 255) / 256 * 256; }
int64_t select_binned_lists_bytes(int groups) {
    return static_cast<int64_t>(groups) * (kSelCap + kBinListGlobal) * sizeof(uint64_t);
}

// Work area of batched NMS: [bit matrix: groups x 1024 x 32 words][row flags: groups x 1024 bytes]
// [prepared input: groups x kPrepBytes, 256-byte aligned][tickets: groups x int32].
struct NmsScratch {
    uint32_t* mask;
    uint8_t* rowflag;
    unsigned char* prep;
    int32_t* ticket;
};
static NmsScratch nms_scratch_views(void* base, int groups) {
    NmsScratch v;
    v.mask = static_cast<uint32_t*>(base);
    v.rowflag = reinterpret_cast<uint8_t*>(v.mask) + static_cast<int64_t>(groups) * kNmsMaxN * kNmsWords * sizeof(uint32_t);
    unsigned char* p = v.rowflag + static_cast<int64_t>(groups) * kNmsMaxN;
    p += (256 - (reinterpret_cast<uintptr_t>(p) & 255)) & 255;
    v.prep = p;
    v.ticket = reinterpret_cast<int32_t*>(p + static_cast<int64_t>(groups) * kPrepBytes);
    return v;
}
int64_t nms_mask_bytes(int groups) {
    return static_cast<int64_t>(groups) * (kNmsMaxN * kNmsWords * sizeof(uint32_t) + kNmsMaxN + kPrepBytes + 4) + 256;
}
int64_t nms_scratch_bytes(int groups, int topk) {
    (void)topk;
    return nms_mask_bytes(groups);
}

// ctr must be zero when the kernel starts (zero_ctr != 0 makes this call clear it).  With nms_scratch != nullptr the
// CTA that finishes a group also prepares the group's NMS input there (boxes [groups, num_boxes, 4], flat index =
// box * num_classes + label), so that launch_batched_nms(..., prepared = 1) can follow directly.
int launch_select_binned(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, const int32_t* hist,
                         float thr, int groups, int topk, uint64_t* out_keys, int32_t* out_counts, void* ctr,
                         void* lists, int zero_ctr, const float* nms_boxes, int64_t num_boxes, int num_classes,
                         int class_offset, void* nms_scratch, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(in_keys && in_counts && hist && out_keys && out_counts && ctr && lists, "select_topk_binned: null pointer");
    FB_REQUIRE(groups > 0 && groups <= 65535 && topk > 0 && topk <= kSelCap && capacity > 0 && capacity < (1ll << 31),
               "select_topk_binned: bad sizes (topk must be in [1, %d])", kSelCap);
    FB_REQUIRE(thr > 0.0f, "select_topk_binned: the threshold must be positive");
    FB_REQUIRE((reinterpret_cast<uintptr_t>(hist) & 15) == 0, "select_topk_binned: the histogram must be 16-byte aligned");
    FB_REQUIRE(nms_scratch == nullptr || (nms_boxes != nullptr && num_boxes > 0 && num_classes > 0 &&
                                          (reinterpret_cast<uintptr_t>(nms_boxes) & 15) == 0),
               "select_topk_binned: NMS preparation needs 16-byte aligned boxes");
    if (zero_ctr) FB_TRY(check_cuda(cudaMemsetAsync(ctr, 0, select_binned_ctr_bytes(groups), st), "memset select counters"));
    const HistParams hp = hist_params_for(thr);
    uint64_t* sel_tmp = static_cast<uint64_t*>(lists);
    uint64_t* bin_tmp = sel_tmp + static_cast<int64_t>(groups) * kSelCap;
    NmsScratch v{nullptr, nullptr, nullptr, nullptr};
    if (nms_scratch != nullptr) v = nms_scratch_views(nms_scratch, groups);
    dim3 grid(kBinSplit, groups);
    select_binned_kernel<<<grid, kBinThreads, 0, st>>>(in_keys, in_counts, capacity, hist, hp.base, hp.shift, topk,
                                                       static_cast<SelectCtr*>(ctr), sel_tmp, bin_tmp, out_keys, out_counts,
                                                       nms_boxes, num_boxes, num_classes, class_offset, v.prep, v.ticket,
                                                       status);
    count_launch();
    return check_launch("select_binned_kernel");
}

// prepared != 0: the group's NMS input is in the scratch already (launch_select_binned with the same scratch).
int launch_batched_nms(const float* boxes, int64_t num_boxes, int num_classes, const uint64_t* sel_keys,
                       const int32_t* sel_counts, int groups, int topk, float iou_thr, int class_offset, float* dets,
                       int64_t* labels, int64_t* flat_ids, int64_t* keep, int32_t* out_counts, void* mask, int prepared,
                       int32_t* status, cudaStream_t st, int32_t* records) {
    FB_REQUIRE(records == nullptr || (reinterpret_cast<uintptr_t>(records) & 15) == 0, "batched_nms: records must be 16-byte aligned");
    FB_REQUIRE(boxes && sel_keys && sel_counts && dets && labels && flat_ids && out_counts && mask,
               "batched_nms: null pointer");
    FB_REQUIRE(groups > 0 && groups <= 65535 && topk > 0 && topk <= kNmsMaxN && num_classes > 0 && num_boxes > 0,
               "batched_nms: bad sizes (topk must be in [1, %d])", kNmsMaxN);
    FB_REQUIRE(iou_thr > 0.0f && iou_thr < 1.0f, "batched_nms: iou threshold must be in (0, 1)");
    FB_REQUIRE((reinterpret_cast<uintptr_t>(boxes) & 15) == 0 && (reinterpret_cast<uintptr_t>(mask) & 15) == 0,
               "batched_nms: boxes and scratch must be 16-byte aligned");
    const float thr_lo = iou_thr * (1.0f - 1.0e-6f), thr_hi = iou_thr * (1.0f + 1.0e-6f);
    const NmsScratch v = nms_scratch_views(mask, groups);
    if (!prepared) {
        nms_prepare_kernel<<<groups, kMaskThreads, 0, st>>>(boxes, num_boxes, num_classes, sel_keys, sel_counts, topk,
                                                            class_offset, v.prep, v.ticket, status);
        count_launch();
        FB_TRY(check_launch("nms_prepare_kernel"));
    }
    // one wave: a second, partly filled wave costs more than longer row loops per warp
    static std::atomic<int> wave_cache[64];  // resident CTAs of this kernel per device: asked once (0 = not yet)
    int dev = 0;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    int wave = dev >= 0 && dev < 64 ? wave_cache[dev].load(std::memory_order_relaxed) : 0;
    if (wave == 0) {
        int sms = 0, per_sm = 0;
        FB_TRY(check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "SM count"));
        FB_TRY(check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, nms_mask_scan_kernel, kMaskThreads, 0),
                          "occupancy"));
        wave = sms * per_sm;
        if (dev >= 0 && dev < 64) wave_cache[dev].store(wave, std::memory_order_relaxed);
    }
    int ctas = wave / groups;
    ctas = ctas < 1 ? 1 : (ctas > kMaskCtasMax ? kMaskCtasMax : ctas);
    dim3 grid(ctas, groups);
    nms_mask_scan_kernel<<<grid, kMaskThreads, 0, st>>>(v.prep, iou_thr, thr_lo, thr_hi, v.mask, v.rowflag, v.ticket, boxes,
                                                        num_boxes, num_classes, sel_keys, topk, dets, labels, flat_ids, keep,
                                                        out_counts, reinterpret_cast<int4*>(records));
    count_launch();
    return check_launch("nms_mask_scan_kernel");
}

}  // namespace fb

// ---- C ABI ------------------------------------------------------------------------------------------
extern "C" {

int functs_b200_threshold_compact(const float* scores, int32_t groups, int64_t n, float thr, uint64_t* keys,
                                  int32_t* counts, int64_t capacity, int32_t zero_counts, int32_t* hist,
                                  int32_t* status, void* stream) {
    return fb::launch_threshold_compact(scores, groups, n, thr, keys, counts, capacity, zero_counts, hist, status,
                                        fb::as_stream(stream));
}

int functs_b200_select_topk(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, int32_t groups,
                            int32_t topk, uint64_t* out_keys, int32_t* out_counts, void* stream) {
    return fb::launch_select_topk(in_keys, in_counts, capacity, groups, topk, out_keys, out_counts,
                                  fb::as_stream(stream));
}

int32_t functs_b200_hist_bins(void) { return fb::kHistBins; }

int64_t functs_b200_select_binned_scratch_bytes(int32_t groups) {
    if (groups <= 0) return 0;
    return fb::select_binned_ctr_bytes(groups) + fb::select_binned_lists_bytes(groups);
}

int functs_b200_select_topk_binned(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity,
                                   const int32_t* hist, float thr, int32_t groups, int32_t topk, uint64_t* out_keys,
                                   int32_t* out_counts, void* scratch, void* stream) {
    if (scratch == nullptr || (reinterpret_cast<uintptr_t>(scratch) & 255) != 0) {
        fb::set_error("select_topk_binned: scratch must be non-null and 256-byte aligned");
        return FB_ERR_INVALID_ARGUMENT;
    }
    unsigned char* base = static_cast<unsigned char*>(scratch);
    return fb::launch_select_binned(in_keys, in_counts, capacity, hist, thr, groups, topk, out_keys, out_counts, base,
                                    base + fb::select_binned_ctr_bytes(groups > 0 ? groups : 1), 1, nullptr, 0, 0, 0, nullptr,
                                    nullptr, fb::as_stream(stream));
}

int64_t functs_b200_nms_scratch_bytes(int32_t groups, int32_t topk) {
    if (groups <= 0) return 0;
    return fb::nms_scratch_bytes(groups, topk);
}

int functs_b200_batched_nms(const float* boxes, int64_t num_boxes, int32_t num_classes, const uint64_t* sel_keys,
                            const int32_t* sel_counts, int32_t groups, int32_t topk, float iou_thr,
                            int32_t class_offset, float* dets, int64_t* labels, int64_t* flat_ids, int64_t* keep,
                            int32_t* out_counts, int32_t* status, void* scratch, void* stream) {
    if (scratch == nullptr || groups <= 0) {
        fb::set_error("batched_nms: null scratch or bad group count");
        return FB_ERR_INVALID_ARGUMENT;
    }
    return fb::launch_batched_nms(boxes, num_boxes, num_classes, sel_keys, sel_counts, groups, topk, iou_thr,
                                  class_offset, dets, labels, flat_ids, keep, out_counts, scratch, 0, status,
                                  fb::as_stream(stream), nullptr);
}

}  // extern "C"
