// C2: YOLOv3-style decode group + the post-process pipeline built on the select / NMS kernels.
//
// The decode kernel is the fusion group "permute -> reshape -> sigmoid on the xy / objectness / class slices
// (slice + sigmoid + slice_rev) -> xy grid offset -> exp * anchor -> corner form -> objectness * class score ->
// score mask" of functs/benchmark/ai_model/yolov3/yolov3_bbox.py:209-220 and :122-127, in one pass over the NCHW
// logits: threads run along the contiguous spatial axis (coalesced), every thread walks the 85 channels of one
// box, and the hits of a warp are staged in shared memory and appended to the image's candidate list.
#include <cstddef>

#include <atomic>

#include "select_nms.cuh"

namespace fb {

int64_t select_binned_ctr_bytes(int groups);
int64_t select_binned_lists_bytes(int groups);
int launch_select_binned(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, const int32_t* hist,
                         float thr, int groups, int topk, uint64_t* out_keys, int32_t* out_counts, void* ctr,
                         void* lists, int zero_ctr, const float* nms_boxes, int64_t num_boxes, int num_classes,
                         int class_offset, void* nms_scratch, int32_t* status, cudaStream_t st);
int64_t nms_mask_bytes(int groups);
int launch_batched_nms(const float* boxes, int64_t num_boxes, int num_classes, const uint64_t* sel_keys,
                       const int32_t* sel_counts, int groups, int topk, float iou_thr, int class_offset, float* dets,
                       int64_t* labels, int64_t* flat_ids, int64_t* keep, int32_t* out_counts, void* mask, int prepared,
                       int32_t* status, cudaStream_t st, int32_t* records = nullptr);

constexpr int kYoloThreads = 128;
constexpr int kYoloClasses = 80;
constexpr int kYoloAttrib = 85;
constexpr int kYoloChunk = 8;        // class logits per thread and step; the next step's loads are issued before this step is consumed
constexpr int kYoloSub = 8;          // logits whose hits are queued at once: <= 32 lanes * 8 = 256 new entries
constexpr int kYoloWarpStage = 96;   // staged candidate keys per warp (flushed when fewer than 32 slots remain)
constexpr int kYoloQueue = 512;      // circular queue of pending hits per warp (256 new + < 32 left over)

struct YoloParams {
    const float* map[3];
    int size[3];        // S
    int tiles[3];       // position tiles per (image, anchor) plane
    int tile_begin[4];  // first CTA of every level, [3] = total
    int live_begin[4];  // the same for the candidate-only kernel (tiles of (anchor, position) slots per image)
    int staged[3];      // level goes through the bulk-copy staged path (16-byte aligned planes)
    int prune_topk;     // > 0: the caller only needs the prune_topk best candidates per image (see prune_digit_regs)
    int box_begin[3];   // first box index of every level inside an image
    float stride[3];
    float anchor_w[3][3];
    float anchor_h[3][3];
    int batch;
    int num_boxes;
    float thr;
    float* boxes;
    float* obj_out;
    float* cls_out;
    uint64_t* keys;
    int32_t* counts;
    int64_t capacity;
    int32_t* status;
    int32_t* hist;       // optional [batch][kHistBins] histogram of candidate scores (for the binned top-k), or null
    int scan_in_staged;  // no level takes the plain-load form: the staged CTAs have to look at the histogram themselves
    int32_t* floor;      // optional [batch]: highest pruning bucket any CTA has found for the image so far (zero at launch)
    uint32_t hist_base;  // float bits of the score threshold
    int hist_shift;
};

struct __align__(8) YoloHit {
    float v;        // class logit
    uint32_t meta;  // owning lane << 8 | class
};

struct YoloWarpSmem {
    uint64_t stage[kYoloWarpStage];
    YoloHit queue[kYoloQueue];
    float vals[kYoloSub][32];  // the logits of the current sub-chunk, so that a hit can be fetched by a runtime index
    int qtail;                 // total entries ever pushed (the warp keeps the matching head in a register)
};

// Appends the staged keys of a warp to the image's candidate list (one atomic per flush).
__device__ __forceinline__ void yolo_flush(YoloWarpSmem& ws, int& fill, uint64_t* gkeys, int32_t* gcount, int64_t capacity,
                                           int32_t* status) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    int base = 0;
    if (lane == 0) base = atomicAdd(gcount, fill);
    base = __shfl_sync(kFullMask, base, 0);
    for (int i = lane; i < fill; i += 32) {
        const int64_t pos = static_cast<int64_t>(base) + i;
        if (pos < capacity) gkeys[pos] = ws.stage[i];
        else if (status != nullptr) atomicOr(status, FB_STATUS_CAND_OVERFLOW);
    }
    __syncwarp();
    fill = 0;
}

// One dense batch: lane i evaluates queue entry head + i (nb <= 32 entries).  Objectness comes from the owning
// lane by shuffle; hits go to the staging buffer and to the score histogram.
__device__ __forceinline__ void yolo_eval_batch(YoloWarpSmem& ws, int head, int nb, float so, uint32_t flat0,
                                                const YoloParams& P, int img, int& fill, uint64_t* gkeys,
                                                int32_t* gcount) {
    const int lane = threadIdx.x & 31;
    const bool act = lane < nb;
    YoloHit e;
    e.v = 0.0f;
    e.meta = static_cast<uint32_t>(lane) << 8;
    if (act) e = ws.queue[(head + lane) & (kYoloQueue - 1)];
    const int src = static_cast<int>(e.meta >> 8);
    const int cls = static_cast<int>(e.meta & 255u);
    const float so_src = __shfl_sync(kFullMask, so, src);
    const float s = __fmul_rn(so_src, sigmoid_f32(e.v));
    const bool pred = act && (s > P.thr);
    const unsigned m = __ballot_sync(kFullMask, pred);
    if (pred) {
        const int off = __popc(m & ((1u << lane) - 1u));
        const uint32_t flat_src = flat0 + static_cast<uint32_t>((src - lane) * 3 * kYoloClasses);
        ws.stage[fill + off] = make_key(s, flat_src + static_cast<uint32_t>(cls));
        if (P.hist != nullptr) {
            const int d = hist_digit(static_cast<uint64_t>(__float_as_uint(s)) << 32, P.hist_base, P.hist_shift);
            atomicAdd(P.hist + static_cast<int64_t>(img) * kHistBins + d, 1);
        }
    }
    fill += __popc(m);
    if (fill + 32 > kYoloWarpStage) yolo_flush(ws, fill, gkeys, gcount, P.capacity, P.status);
}

// Body for one pyramid level.  S_T > 0 fixes the map size at compile time (channel strides become immediates).
template <int S_T, bool DENSE>
__device__ __forceinline__ void yolo_decode_level(const YoloParams& P, const int lvl, const int local, YoloWarpSmem& ws) {
    const int S = S_T > 0 ? S_T : P.size[lvl];
    const int SS = S * S;
    const int plane = local / P.tiles[lvl];  // = image * 3 + anchor
    const int tile = local - plane * P.tiles[lvl];
    const int img = plane / 3;
    const int anc = plane - img * 3;
    const int p = tile * kYoloThreads + threadIdx.x;
    const int lane = threadIdx.x & 31;
    // Lanes past the end of the plane are clamped so that every lane loads a legal address.  A warp is then either
    // fully valid, or its tail lanes all alias position SS - 1; aliased lanes never produce candidates.
    const bool valid = p < SS;
    const int pp = valid ? p : (SS - 1);
    const float* __restrict__ src = P.map[lvl] + (static_cast<int64_t>(img) * 255 + anc * kYoloAttrib) * SS + pp;

    const float t0 = __ldg(src);
    const float t1 = __ldg(src + SS);
    const float t2 = __ldg(src + 2 * SS);
    const float t3 = __ldg(src + 3 * SS);
    const float t4 = __ldg(src + 4 * SS);
    const float* __restrict__ csrc = src + 5 * SS;
    float v[kYoloChunk];
#pragma unroll
    for (int u = 0; u < kYoloChunk; ++u) v[u] = __ldg(csrc + u * SS);

    const int gy = pp / S, gx = pp - gy * S;
    const float stride = P.stride[lvl];
    const float cx = __fmul_rn(__fadd_rn(sigmoid_f32(t0), static_cast<float>(gx)), stride);
    const float cy = __fmul_rn(__fadd_rn(sigmoid_f32(t1), static_cast<float>(gy)), stride);
    const float hw = __fmul_rn(__fmul_rn(expf(t2), P.anchor_w[lvl][anc]), 0.5f);
    const float hh = __fmul_rn(__fmul_rn(expf(t3), P.anchor_h[lvl][anc]), 0.5f);
    const float so = sigmoid_f32(t4);
    const int box = P.box_begin[lvl] + pp * 3 + anc;
    const int64_t gbox = static_cast<int64_t>(img) * P.num_boxes + box;
    if (valid) {
        reinterpret_cast<float4*>(P.boxes)[gbox] =
            make_float4(__fsub_rn(cx, hw), __fsub_rn(cy, hh), __fadd_rn(cx, hw), __fadd_rn(cy, hh));
        if (DENSE && P.obj_out != nullptr) P.obj_out[gbox] = so;
    }

    // Logit cut: score = so * sigmoid(v) can exceed thr only if sigmoid(v) > thr / so.  The cut is placed a
    // relative 1e-5 below that (hundreds of fp32 ulps, covering the rounding of sigmoid and of the product) and
    // another 0.02 lower in the logit domain (covering the rounding of the logit itself), so it never loses a
    // candidate; everything above the cut is evaluated exactly.
    float v_cut = INFINITY;
    if (valid && so > P.thr) {
        const float q = (P.thr / so) * (1.0f - 1.0e-5f);
        v_cut = logf(q / (1.0f - q)) - 0.02f;
    }

    int fill = 0;    // staged keys (warp-uniform)
    int head = 0;    // queue entries consumed so far (warp-uniform)
    int pushed = 0;  // queue entries pushed so far (warp-uniform copy of ws.qtail)
    if (lane == 0) ws.qtail = 0;
    __syncwarp();
    uint64_t* gkeys = P.keys + static_cast<int64_t>(img) * P.capacity;
    int32_t* gcount = P.counts + img;
    // flat index of class 0 of this lane's UNCLAMPED position (dense batches offset it to the owning lane)
    const uint32_t flat0 = static_cast<uint32_t>(P.box_begin[lvl] + p * 3 + anc) * kYoloClasses;

#pragma unroll 1
    for (int c0 = 0; c0 < kYoloClasses; c0 += kYoloChunk) {
        // software pipeline: the loads of the next step are in flight while this step's logits are consumed
        float vn[kYoloChunk];
        if (c0 + kYoloChunk < kYoloClasses) {
#pragma unroll
            for (int u = 0; u < kYoloChunk; ++u) vn[u] = __ldg(csrc + (c0 + kYoloChunk + u) * SS);
        } else {
#pragma unroll
            for (int u = 0; u < kYoloChunk; ++u) vn[u] = 0.0f;
        }
        if (DENSE) {
            if (valid && P.cls_out != nullptr) {
#pragma unroll
                for (int u = 0; u < kYoloChunk; ++u) P.cls_out[gbox * kYoloClasses + c0 + u] = sigmoid_f32(v[u]);
            }
        }
#pragma unroll
        for (int h = 0; h < kYoloChunk; h += kYoloSub) {
            uint32_t hits = 0u;
#pragma unroll
            for (int u = 0; u < kYoloSub; ++u) hits |= (v[h + u] > v_cut ? 1u : 0u) << u;
            const int cnt = __popc(hits);
            const int total = __reduce_add_sync(kFullMask, cnt);
            if (total > 0) {  // warp-uniform
                __syncwarp();
#pragma unroll
                for (int u = 0; u < kYoloSub; ++u) ws.vals[u][lane] = v[h + u];
                if (cnt > 0) {
                    int pos = atomicAdd(&ws.qtail, cnt);
                    const uint32_t meta0 = (static_cast<uint32_t>(lane) << 8) | static_cast<uint32_t>(c0 + h);
                    while (hits) {
                        const int u = __ffs(hits) - 1;
                        hits &= hits - 1u;
                        YoloHit e;
                        e.v = ws.vals[u][lane];
                        e.meta = meta0 + static_cast<uint32_t>(u);
                        ws.queue[pos & (kYoloQueue - 1)] = e;
                        ++pos;
                    }
                }
                __syncwarp();
                pushed += total;  // == ws.qtail
                while (pushed - head >= 32) {
                    yolo_eval_batch(ws, head, 32, so, flat0, P, img, fill, gkeys, gcount);
                    head += 32;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kYoloChunk; ++u) v[u] = vn[u];
    }
    const int rest = pushed - head;
    if (rest > 0) yolo_eval_batch(ws, head, rest, so, flat0, P, img, fill, gkeys, gcount);
    if (fill > 0) yolo_flush(ws, fill, gkeys, gcount, P.capacity, P.status);
}

template <int S0, int S1, int S2, bool DENSE>
__global__ void __launch_bounds__(kYoloThreads)
yolo_decode_kernel(const YoloParams P) {
    __shared__ YoloWarpSmem smem_all[kYoloThreads / 32];
    YoloWarpSmem& ws = smem_all[threadIdx.x >> 5];
    const int cta = blockIdx.x;
    if (cta >= P.tile_begin[2]) {
        yolo_decode_level<S2, DENSE>(P, 2, cta - P.tile_begin[2], ws);
    } else if (cta >= P.tile_begin[1]) {
        yolo_decode_level<S1, DENSE>(P, 1, cta - P.tile_begin[1], ws);
    } else {
        yolo_decode_level<S0, DENSE>(P, 0, cta, ws);
    }
}

// ---- candidate-only decode ("live box" form) ------------------------------------------------------------------
// Used when no dense objectness / class-score output is requested (the fused post-process).  A box whose objectness
// does not exceed the threshold cannot yield a candidate, so the class logits are only walked for the boxes that
// survive that test: a CTA decodes a tile of kLiveTile (anchor, position) slots of one image and level (two slots per
// thread), compacts the surviving slots into a shared list, and then lets thread k walk the 80 class logits of the
// k-th survivor.  Hits are packed with a ballot into the warp's queue and evaluated 32 at a time.
constexpr int kLiveThreads = 256;
constexpr int kLiveSlots = 2;  // slots per thread in the first phase
constexpr int kLiveTile = kLiveThreads * kLiveSlots;
constexpr int kLiveSub = 4;     // class steps between two looks at the queue: <= 128 new entries
constexpr int kLiveQueue = 256;  // > 128 new + 31 left over
constexpr int kLiveStage = 96;

// Pruning for callers that keep only the `need` best candidates of an image.  The image's score histogram only ever
// grows, so once some bucket d has at least `need` recorded candidates in the buckets >= d, a candidate of a lower
// bucket can never be among the `need` best and may be dropped unrecorded.  This returns such a d (0 = no pruning
// yet) from a possibly stale look at the histogram: stale counts are smaller, which only makes d more conservative.
// The second look (the owner lane's 64 buckets, two per lane) can only see larger counts than the first, which keeps
// the result conservative as well.  Called by one full warp; nothing waits for anybody.
__device__ __noinline__ int prune_digit_regs(const int32_t* __restrict__ h, int need) {
    const int lane = threadIdx.x & 31;
    constexpr int per = kHistBins / 32;
    static_assert(per == 64, "two buckets per lane in the second look");
    const int4* h4 = reinterpret_cast<const int4*>(h + lane * per);
    int sum = 0;
#pragma unroll 4
    for (int i = 0; i < per / 4; ++i) {
        const int4 x = __ldcg(h4 + i);
        sum += (x.x + x.y) + (x.z + x.w);
    }
    int incl = sum;  // this lane's buckets and all higher ones
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(kFullMask, incl, o);
        if (lane + o < 32) incl += v;
    }
    const unsigned who = __ballot_sync(kFullMask, incl - sum < need && incl >= need);
    if (who == 0u) return 0;  // fewer than `need` candidates recorded so far
    const int owner = __ffs(who) - 1;
    const int above = __shfl_sync(kFullMask, incl - sum, owner);
    const int b0 = owner * per + 2 * lane;
    const int2 c = __ldcg(reinterpret_cast<const int2*>(h + b0));
    int incl2 = c.x + c.y;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(kFullMask, incl2, o);
        if (lane + o < 32) incl2 += v;
    }
    const int hi = above + incl2 - (c.x + c.y);  // recorded candidates in the buckets above this lane's pair
    int d = 0;
    if (hi < need && hi + c.x + c.y >= need) d = (hi + c.y >= need) ? b0 + 1 : b0;
    return __reduce_max_sync(kFullMask, d);
}

// v > cut is necessary for so * sigmoid(v) to reach `floor_score` (> 0).  The cut sits a relative 1e-5 below the
// exact bound (hundreds of fp32 ulps: rounding of the sigmoid and of the product) and another 0.02 lower in the
// logit domain, so it never loses a candidate.  The 0.02 also covers the fast division and logarithm used here
// (errors of a few ulps, i.e. below 1e-5 in the logit): the cut is recomputed whenever the pruning floor rises, for
// every survivor, and must be cheap.
__device__ __forceinline__ float logit_cut(float so, float floor_score) {
    const float q = __fdividef(floor_score, so) * (1.0f - 1.0e-5f);
    if (!(q < 1.0f)) return INFINITY;
    return __logf(__fdividef(q, 1.0f - q)) - 0.02f;
}

struct __align__(16) YoloLive {
    float so;        // objectness score
    float v_cut;     // class logits at or below this cannot reach the threshold
    uint32_t chan;   // offset of the slot's class-0 logit inside the image's level map
    uint32_t flat0;  // flat (box, class 0) index inside the image
};

struct YoloLiveWarp {
    uint64_t stage[kLiveStage];
    YoloHit queue[kLiveQueue];  // meta = live index << 8 | class
};

struct YoloLiveSmem {
    int prune;  // latest pruning bucket published for this CTA
    int done_warps;  // consumer warps that have finished (the scanner warp stops at kLiveThreads / 32)
    YoloLive live[kLiveTile];
    YoloLiveWarp w[kLiveThreads / 32];
    int warp_cnt[kLiveThreads / 32];
};

// barrier of the kLiveThreads consumer threads of a plain-load CTA (the ninth warp does not take part)
__device__ __forceinline__ void live_sync() { asm volatile("bar.sync 1, %0;" ::"n"(256) : "memory"); }

__device__ __forceinline__ void live_flush(YoloLiveWarp& ws, int& fill, uint64_t* gkeys, int32_t* gcount, int64_t capacity,
                                           int32_t* status) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    int base = 0;
    if (lane == 0) base = atomicAdd(gcount, fill);
    base = __shfl_sync(kFullMask, base, 0);
    for (int i = lane; i < fill; i += 32) {
        const int64_t pos = static_cast<int64_t>(base) + i;
        if (pos < capacity) gkeys[pos] = ws.stage[i];
        else if (status != nullptr) atomicOr(status, FB_STATUS_CAND_OVERFLOW);
    }
    __syncwarp();
    fill = 0;
}

// lane i evaluates queue entry head + i (nb <= 32 entries): exact score, threshold, key, histogram.
__device__ __forceinline__ void live_eval_batch(const YoloLiveSmem& sm, YoloLiveWarp& ws, int head, int nb,
                                                const YoloParams& P, int32_t* ghist, int prune, int& fill,
                                                uint64_t* gkeys, int32_t* gcount) {
    const int lane = threadIdx.x & 31;
    const bool act = lane < nb;
    bool pred = false;
    float s = 0.0f;
    uint32_t flat = 0u;
    int digit = 0;
    if (act) {
        const YoloHit e = ws.queue[(head + lane) & (kLiveQueue - 1)];
        const YoloLive o = sm.live[e.meta >> 8];
        s = __fmul_rn(o.so, sigmoid_f32(e.v));
        flat = o.flat0 + (e.meta & 255u);
        digit = hist_digit(static_cast<uint64_t>(__float_as_uint(s)) << 32, P.hist_base, P.hist_shift);
        pred = s > P.thr && digit >= prune;
    }
    const unsigned m = __ballot_sync(kFullMask, pred);
    if (pred) {
        ws.stage[fill + __popc(m & ((1u << lane) - 1u))] = make_key(s, flat);
        if (ghist != nullptr) atomicAdd(ghist + digit, 1);
    }
    fill += __popc(m);
    if (fill + 32 > kLiveStage) live_flush(ws, fill, gkeys, gcount, P.capacity, P.status);
}

template <int S_T>
__device__ __forceinline__ void yolo_live_level(const YoloParams& P, const int lvl, const int local, YoloLiveSmem& sm) {
    const int S = S_T > 0 ? S_T : P.size[lvl];
    const int SS = S * S;
    const int nslots = 3 * SS;
    const int tiles = (nslots + kLiveTile - 1) / kLiveTile;
    const int img = local / tiles;
    const int tile = local - img * tiles;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const float* __restrict__ base = P.map[lvl] + static_cast<int64_t>(img) * 255 * SS;
    const float stride = P.stride[lvl];

    // ---- phase 1: box decode + objectness test for kLiveSlots slots per thread ----
    float so[kLiveSlots], vcut[kLiveSlots];
    uint32_t chan[kLiveSlots], flat0[kLiveSlots];
    bool alive[kLiveSlots];
    float tv[kLiveSlots][5];
    int anc_[kLiveSlots], p_[kLiveSlots];
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        const int slot = tile * kLiveTile + q * kLiveThreads + t;
        const bool valid = slot < nslots;
        const int sl = valid ? slot : 0;
        const int anc = sl / SS, p = sl - anc * SS;
        anc_[q] = anc;
        p_[q] = p;
        alive[q] = valid;
        const float* src = base + anc * kYoloAttrib * SS + p;
#pragma unroll
        for (int c = 0; c < 5; ++c) tv[q][c] = valid ? __ldg(src + c * SS) : 0.0f;
    }
    int32_t* ghist = P.hist != nullptr ? P.hist + static_cast<int64_t>(img) * kHistBins : nullptr;
    const bool pruning = P.prune_topk > 0 && ghist != nullptr;
    if (warp == 0) {
        // a bucket that an earlier CTA derived from the image's histogram stays valid: one load instead of a scan
        int d = 0;
        if (pruning) d = P.floor != nullptr ? __ldcg(P.floor + img) : prune_digit_regs(ghist, P.prune_topk);
        if (lane == 0) atomicMax(&sm.prune, d);  // (the scanner warp may have been there already)
    }
    live_sync();
    int prune = sm.prune;  // candidates of buckets below this are dropped
    // lowest score of bucket `prune`; 0 while nothing is pruned
    float floor_score = prune > 0 ? __uint_as_float(P.hist_base + (static_cast<uint32_t>(prune) << P.hist_shift)) : 0.0f;
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        const int anc = anc_[q], p = p_[q];
        const int gy = p / S, gx = p - gy * S;
        const float aw = anc == 0 ? P.anchor_w[lvl][0] : (anc == 1 ? P.anchor_w[lvl][1] : P.anchor_w[lvl][2]);
        const float ah = anc == 0 ? P.anchor_h[lvl][0] : (anc == 1 ? P.anchor_h[lvl][1] : P.anchor_h[lvl][2]);
        const float cx = __fmul_rn(__fadd_rn(sigmoid_f32(tv[q][0]), static_cast<float>(gx)), stride);
        const float cy = __fmul_rn(__fadd_rn(sigmoid_f32(tv[q][1]), static_cast<float>(gy)), stride);
        const float hw = __fmul_rn(__fmul_rn(expf(tv[q][2]), aw), 0.5f);
        const float hh = __fmul_rn(__fmul_rn(expf(tv[q][3]), ah), 0.5f);
        so[q] = sigmoid_f32(tv[q][4]);
        const int box = P.box_begin[lvl] + p * 3 + anc;
        if (alive[q]) {
            reinterpret_cast<float4*>(P.boxes)[static_cast<int64_t>(img) * P.num_boxes + box] =
                make_float4(__fsub_rn(cx, hw), __fsub_rn(cy, hh), __fadd_rn(cx, hw), __fadd_rn(cy, hh));
        }
        // a score is so * sigmoid(v) <= so: the box can only yield candidates if so itself clears both bars; the
        // class logits above logit_cut() are then evaluated exactly
        alive[q] = alive[q] && so[q] > P.thr && so[q] >= floor_score;
        vcut[q] = alive[q] ? logit_cut(so[q], fmaxf(P.thr, floor_score)) : INFINITY;
        chan[q] = static_cast<uint32_t>((anc * kYoloAttrib + 5) * SS + p);
        flat0[q] = static_cast<uint32_t>(box) * kYoloClasses;
    }
    // compaction: the survivors of a warp stay together (slot order inside each of its kLiveSlots runs)
    unsigned bal[kLiveSlots];
    int mine = 0;
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        bal[q] = __ballot_sync(kFullMask, alive[q]);
        mine += __popc(bal[q]);
    }
    if (lane == 0) sm.warp_cnt[warp] = mine;
    live_sync();
    int wbase = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kLiveThreads / 32; ++w) {
        const int c = sm.warp_cnt[w];
        if (w < warp) wbase += c;
        total += c;
    }
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        if (alive[q]) {
            YoloLive e;
            e.so = so[q];
            e.v_cut = vcut[q];
            e.chan = chan[q];
            e.flat0 = flat0[q];
            sm.live[wbase + __popc(bal[q] & ((1u << lane) - 1u))] = e;
        }
        wbase += __popc(bal[q]);
    }
    live_sync();

    // ---- phase 2: thread k walks the class logits of survivor k ----
    YoloLiveWarp& ws = sm.w[warp];
    uint64_t* gkeys = P.keys + static_cast<int64_t>(img) * P.capacity;
    int32_t* gcount = P.counts + img;
    const unsigned lt = (1u << lane) - 1u;
    int fill = 0, head = 0, tail = 0;  // warp-uniform
#pragma unroll 1
    for (int k0 = warp * 32; k0 < total; k0 += kLiveThreads) {
        const int k = k0 + lane;
        const bool has = k < total;
        YoloLive me;
        me.so = 0.0f;
        me.v_cut = INFINITY;
        me.chan = 0u;
        me.flat0 = 0u;
        if (has) me = sm.live[k];
        const float* __restrict__ csrc = base + me.chan;
        const uint32_t meta0 = static_cast<uint32_t>(k) << 8;
        float v[kYoloChunk];
#pragma unroll
        for (int u = 0; u < kYoloChunk; ++u) v[u] = has ? __ldg(csrc + u * SS) : 0.0f;
#pragma unroll 1
        for (int c0 = 0; c0 < kYoloClasses; c0 += kYoloChunk) {
            if (pruning) {
                // the CTA's spare warp looks at the histogram all the time (live_scanner) and leaves the bucket here
                const int now = *reinterpret_cast<volatile int*>(&sm.prune);
                if (now > prune) {
                    prune = now;
                    floor_score = __uint_as_float(P.hist_base + (static_cast<uint32_t>(prune) << P.hist_shift));
                    me.v_cut = (has && me.so >= floor_score) ? logit_cut(me.so, fmaxf(P.thr, floor_score)) : INFINITY;
                }
            }
            float vn[kYoloChunk];
            if (c0 + kYoloChunk < kYoloClasses) {
#pragma unroll
                for (int u = 0; u < kYoloChunk; ++u)
                    vn[u] = (has && me.v_cut < INFINITY) ? __ldg(csrc + (c0 + kYoloChunk + u) * SS) : 0.0f;
            } else {
#pragma unroll
                for (int u = 0; u < kYoloChunk; ++u) vn[u] = 0.0f;
            }
#pragma unroll
            for (int h = 0; h < kYoloChunk; h += kLiveSub) {
#pragma unroll
                for (int u = 0; u < kLiveSub; ++u) {
                    const bool pred = v[h + u] > me.v_cut;
                    const unsigned m = __ballot_sync(kFullMask, pred);
                    if (pred) {
                        YoloHit e;
                        e.v = v[h + u];
                        e.meta = meta0 | static_cast<uint32_t>(c0 + h + u);
                        ws.queue[(tail + __popc(m & lt)) & (kLiveQueue - 1)] = e;
                    }
                    tail += __popc(m);
                }
                __syncwarp();
                while (tail - head >= 32) {
                    live_eval_batch(sm, ws, head, 32, P, ghist, prune, fill, gkeys, gcount);
                    head += 32;
                }
            }
#pragma unroll
            for (int u = 0; u < kYoloChunk; ++u) v[u] = vn[u];
        }
    }
    __syncwarp();
    if (tail - head > 0) live_eval_batch(sm, ws, head, tail - head, P, ghist, prune, fill, gkeys, gcount);
    if (fill > 0) live_flush(ws, fill, gkeys, gcount, P.capacity, P.status);
    __syncwarp();
    if (lane == 0) atomicAdd(&sm.done_warps, 1);
}

// The ninth warp of a plain-load CTA (the staged CTAs use theirs as the copy producer): it looks at the image's histogram
// over and over while the other eight work and publishes every bucket it finds, for its own CTA (shared memory) and for
// all other CTAs of the image (P.floor).  The earlier the first buckets are out, the less the first wave of CTAs (which
// starts with nothing to prune by) has to walk and evaluate.  Bounded: it ends when the eight consumer warps are done,
// and after kLiveScans looks at the latest.
constexpr int kLiveScans = 256;
template <int S_T>
__device__ __forceinline__ void live_scanner(const YoloParams& P, const int lvl, const int local, YoloLiveSmem& sm) {
    const int S = S_T > 0 ? S_T : P.size[lvl];
    const int tiles = (3 * S * S + kLiveTile - 1) / kLiveTile;
    const int img = local / tiles;
    if (P.hist == nullptr || P.prune_topk <= 0) return;
    const int32_t* ghist = P.hist + static_cast<int64_t>(img) * kHistBins;
    const int lane = threadIdx.x & 31;
    for (int it = 0; it < kLiveScans; ++it) {
        if (*reinterpret_cast<volatile int*>(&sm.done_warps) >= kLiveThreads / 32) break;
        const int d = prune_digit_regs(ghist, P.prune_topk);
        if (lane == 0 && d > *reinterpret_cast<volatile int*>(&sm.prune)) {
            atomicMax(&sm.prune, d);
            if (P.floor != nullptr) atomicMax(P.floor + img, d);
        }
        __syncwarp();
    }
}

// ---- the same with the class planes staged through shared memory by the copy engine -------------------------
// Levels whose plane size is a multiple of 4 floats (16-byte aligned rows) take this path: the CTA's tile is
// kStTile (anchor, position) slots; for every step of kStClasses classes one thread issues bulk copies of the
// tile's piece of each class plane (1 or 2 contiguous segments, a tile can straddle an anchor boundary) into a ring
// of kStStages buffers, completion on an mbarrier.  The copies of the next steps are in flight while the survivors'
// logits of the current step are read from shared memory, so DRAM latency is not on the consumers' critical path.
constexpr int kStTile = 448;     // < 2 * kLiveThreads: about half the slots survive, one survivor per thread
constexpr int kStClasses = 8;
constexpr int kStStages = 3;
constexpr int kStSteps = kYoloClasses / kStClasses;
constexpr int kStSub = 2;
constexpr int kStQueue = 128;    // > 32 * kStSub new + 31 left over
constexpr int kStConsumerWarps = kLiveThreads / 32;
constexpr int kStThreads = kLiveThreads + 32;  // + the producer warp
static_assert(kYoloClasses % kStClasses == 0 && kStTile % 4 == 0 && kStTile <= kLiveTile, "staged decode layout");

// staged candidate keys per warp, flushed when fewer than 32 slots remain (224 slots, i.e. two flushes instead of five for
// the CTAs of the first wave, measured: no change)
constexpr int kStKeyStage = 96;

struct YoloStWarp {
    uint64_t stage[kStKeyStage];
    YoloHit queue[kStQueue];  // meta = live index << 8 | class
};

struct __align__(128) YoloStagedSmem {
    float ring[kStStages][kStClasses][kStTile];
    YoloLive live[kStTile];  // .chan holds the slot's index inside the tile
    YoloStWarp w[kLiveThreads / 32];
    uint64_t full[kStStages];   // copy engine -> consumers: the buffer's bytes have landed
    uint64_t empty[kStStages];  // consumers -> producer warp: every consumer warp is done with the buffer
    int warp_cnt[kLiveThreads / 32];
    int prune;  // latest pruning bucket published for this CTA
};
static_assert(sizeof(YoloStagedSmem) <= 75 * 1024, "three CTAs per SM");

static_assert(offsetof(YoloStagedSmem, live) % 16 == 0 &&
                  offsetof(YoloStagedSmem, full) % 8 == 0 && offsetof(YoloStagedSmem, empty) % 8 == 0 && offsetof(YoloStagedSmem, w) % 8 == 0,
              "shared-memory layout of the staged decode");

__device__ __forceinline__ void st_flush(YoloStWarp& ws, int& fill, uint64_t* gkeys, int32_t* gcount, int64_t capacity,
                                         int32_t* status) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    int base = 0;
    if (lane == 0) base = atomicAdd(gcount, fill);
    base = __shfl_sync(kFullMask, base, 0);
    for (int i = lane; i < fill; i += 32) {
        const int64_t pos = static_cast<int64_t>(base) + i;
        if (pos < capacity) gkeys[pos] = ws.stage[i];
        else if (status != nullptr) atomicOr(status, FB_STATUS_CAND_OVERFLOW);
    }
    __syncwarp();
    fill = 0;
}

// Everything the evaluation of queued hits needs, by value (the function below is not inlined).
struct StEvalArgs {
    float thr;
    uint32_t hist_base;
    int hist_shift;
    int32_t* ghist;
    uint64_t* gkeys;
    int32_t* gcount;
    int64_t capacity;
    int32_t* status;
};

// Lane i evaluates queue entry head + i (nb <= 32 entries): exact score, threshold and pruning bucket, key,
// histogram.  Returns the new fill level of the warp's key stage.  Kept out of line: it is called from several
// places of an unrolled loop and the copies would only bloat the instruction footprint.
__device__ __noinline__ int st_eval_batch(const YoloLive* live, YoloStWarp* wsp, int head, int nb, StEvalArgs a, int prune,
                                          int fill) {
    YoloStWarp& ws = *wsp;
    const int lane = threadIdx.x & 31;
    bool pred = false;
    float s = 0.0f;
    uint32_t flat = 0u;
    int digit = 0;
    if (lane < nb) {
        const YoloHit e = ws.queue[(head + lane) & (kStQueue - 1)];
        const YoloLive o = live[e.meta >> 8];
        s = __fmul_rn(o.so, sigmoid_f32(e.v));
        flat = o.flat0 + (e.meta & 255u);
        digit = hist_digit(static_cast<uint64_t>(__float_as_uint(s)) << 32, a.hist_base, a.hist_shift);
        pred = s > a.thr && digit >= prune;
    }
    const unsigned m = __ballot_sync(kFullMask, pred);
    if (pred) {
        ws.stage[fill + __popc(m & ((1u << lane) - 1u))] = make_key(s, flat);
        if (a.ghist != nullptr) atomicAdd(a.ghist + digit, 1);
    }
    fill += __popc(m);
    if (fill + 32 > kStKeyStage) st_flush(ws, fill, a.gkeys, a.gcount, a.capacity, a.status);
    return fill;
}

// One thread: copies of class step `step` of the tile [s0, s0 + n) into ring buffer `buf`.
__device__ __forceinline__ void st_issue(YoloStagedSmem& sm, const float* base, int SS, int s0, int n, int step, int buf) {
    mbar_arrive_expect_tx(&sm.full[buf], static_cast<uint32_t>(n) * 4u * kStClasses);
    const int a0 = s0 / SS;
    const int pa = s0 - a0 * SS;
    const int len0 = min(n, SS - pa);  // slots of the first anchor; the rest (if any) starts the next anchor's planes
#pragma unroll
    for (int c = 0; c < kStClasses; ++c) {
        const int ch = 5 + step * kStClasses + c;
        bulk_copy_g2s(&sm.ring[buf][c][0], base + static_cast<int64_t>(a0 * kYoloAttrib + ch) * SS + pa,
                      static_cast<uint32_t>(len0) * 4u, &sm.full[buf]);
        if (len0 < n)
            bulk_copy_g2s(&sm.ring[buf][c][len0], base + static_cast<int64_t>((a0 + 1) * kYoloAttrib + ch) * SS,
                          static_cast<uint32_t>(n - len0) * 4u, &sm.full[buf]);
    }
}

template <int S_T>
__device__ __forceinline__ void yolo_staged_level(const YoloParams& P, const int lvl, const int local, YoloStagedSmem& sm) {
    const int S = S_T > 0 ? S_T : P.size[lvl];
    const int SS = S * S;
    const int nslots = 3 * SS;
    const int tiles = (nslots + kStTile - 1) / kStTile;
    const int img = local / tiles;
    const int tile = local - img * tiles;
    const int s0 = tile * kStTile;
    const int n = min(kStTile, nslots - s0);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const bool producer = warp == kStConsumerWarps;  // the ninth warp only feeds the ring
    const float* __restrict__ base = P.map[lvl] + static_cast<int64_t>(img) * 255 * SS;
    const float stride = P.stride[lvl];
    int32_t* ghist = P.hist != nullptr ? P.hist + static_cast<int64_t>(img) * kHistBins : nullptr;
    const bool pruning = P.prune_topk > 0 && ghist != nullptr;

    if (t == 0) {
#pragma unroll
        for (int b = 0; b < kStStages; ++b) mbar_init(&sm.full[b], 1);  // (the empty barriers: after the first phase)
        fence_barrier_init();
    }
    __syncthreads();
    if (producer && lane == 0) {
#pragma unroll
        for (int b = 0; b < kStStages; ++b) st_issue(sm, base, SS, s0, n, b, b);
    }

    // ---- phase 1 (consumer warps): box decode + objectness test, two slots per thread, plain loads ----
    float so[kLiveSlots], vcut[kLiveSlots];
    uint32_t flat0[kLiveSlots];
    bool alive[kLiveSlots];
    float tv[kLiveSlots][5];
    int anc_[kLiveSlots], p_[kLiveSlots];
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        const int ls = q * kLiveThreads + t;
        const bool valid = !producer && ls < n;
        const int sl = valid ? s0 + ls : s0;
        const int anc = sl / SS, p = sl - anc * SS;
        anc_[q] = anc;
        p_[q] = p;
        alive[q] = valid;
        const float* src = base + anc * kYoloAttrib * SS + p;
#pragma unroll
        for (int c = 0; c < 5; ++c) tv[q][c] = valid ? __ldg(src + c * SS) : 0.0f;
    }
    if (producer) {  // idle until the first buffer comes back: look up the image's pruning bucket meanwhile
        // a bucket that an earlier CTA derived from the image's histogram stays valid: one load instead of a scan
        // (a scan here, in every CTA, was measured: the decode kernel went from 80 to 92 us)
        int d = 0;
        if (pruning) d = P.floor != nullptr ? __ldcg(P.floor + img) : prune_digit_regs(ghist, P.prune_topk);
        if (lane == 0) sm.prune = d;
    }
    // box decode (does not need the bucket)
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        const int anc = anc_[q], p = p_[q];
        const int gy = p / S, gx = p - gy * S;
        const float aw = anc == 0 ? P.anchor_w[lvl][0] : (anc == 1 ? P.anchor_w[lvl][1] : P.anchor_w[lvl][2]);
        const float ah = anc == 0 ? P.anchor_h[lvl][0] : (anc == 1 ? P.anchor_h[lvl][1] : P.anchor_h[lvl][2]);
        const float cx = __fmul_rn(__fadd_rn(sigmoid_f32(tv[q][0]), static_cast<float>(gx)), stride);
        const float cy = __fmul_rn(__fadd_rn(sigmoid_f32(tv[q][1]), static_cast<float>(gy)), stride);
        const float hw = __fmul_rn(__fmul_rn(expf(tv[q][2]), aw), 0.5f);
        const float hh = __fmul_rn(__fmul_rn(expf(tv[q][3]), ah), 0.5f);
        so[q] = sigmoid_f32(tv[q][4]);
        const int box = P.box_begin[lvl] + p * 3 + anc;
        if (alive[q]) {
            reinterpret_cast<float4*>(P.boxes)[static_cast<int64_t>(img) * P.num_boxes + box] =
                make_float4(__fsub_rn(cx, hw), __fsub_rn(cy, hh), __fadd_rn(cx, hw), __fadd_rn(cy, hh));
        }
        flat0[q] = static_cast<uint32_t>(box) * kYoloClasses;
    }
    __syncthreads();
    int prune = sm.prune;  // candidates of buckets below this are dropped
    // lowest score of bucket `prune`; 0 while nothing is pruned
    float floor_score = prune > 0 ? __uint_as_float(P.hist_base + (static_cast<uint32_t>(prune) << P.hist_shift)) : 0.0f;
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        // a score is so * sigmoid(v) <= so: the box can only yield candidates if so itself clears both bars
        alive[q] = alive[q] && so[q] > P.thr && so[q] >= floor_score;
        vcut[q] = alive[q] ? logit_cut(so[q], fmaxf(P.thr, floor_score)) : INFINITY;
    }
    unsigned bal[kLiveSlots];
    int mine = 0;
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        bal[q] = __ballot_sync(kFullMask, alive[q]);
        mine += __popc(bal[q]);
    }
    if (lane == 0 && !producer) sm.warp_cnt[warp] = mine;
    __syncthreads();
    int wbase = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kStConsumerWarps; ++w) {
        const int c = sm.warp_cnt[w];
        if (w < warp) wbase += c;
        total += c;
    }
#pragma unroll
    for (int q = 0; q < kLiveSlots; ++q) {
        if (alive[q]) {
            YoloLive e;
            e.so = so[q];
            e.v_cut = vcut[q];
            e.chan = static_cast<uint32_t>(q * kLiveThreads + t);
            e.flat0 = flat0[q];
            sm.live[wbase + __popc(bal[q] & ((1u << lane) - 1u))] = e;
        }
        wbase += __popc(bal[q]);
    }
    // Only the warps that hold survivors take part in the ring: the others would do nothing but poll its barriers (and a
    // polling warp competes with the working ones for issue slots and for the shared-memory pipe), so they leave here.
    const int nbusy = min(kStConsumerWarps, max(1, (total + 31) >> 5));
    if (t == 0) {
#pragma unroll
        for (int b = 0; b < kStStages; ++b) mbar_init(&sm.empty[b], static_cast<uint32_t>(nbusy));
        fence_barrier_init();
    }
    __syncthreads();  // the last CTA-wide barrier: from here on the warps only meet through the ring's mbarriers
    if (!producer && warp >= nbusy) return;

    if (producer) {
        // refill a buffer as soon as all consumer warps have released it
        int floor_seen = 0;
#pragma unroll 1
        for (int step = kStStages; step < kStSteps; ++step) {
            const int buf = step % kStStages;
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait_bounded(&sm.empty[buf], static_cast<uint32_t>((step / kStStages - 1) & 1), 100000u) ? 1 : 0;
                if (ok) st_issue(sm, base, SS, s0, n, step, buf);
                else if (P.status != nullptr) atomicOr(P.status, FB_STATUS_WAIT_TIMEOUT);
            }
            ok = __shfl_sync(kFullMask, ok, 0);
            if (!ok) break;
            // The image's bucket as other CTAs published it: this warp asks for the word after every refill and hands the
            // answer of the previous request on to the consumers through shared memory.  The request is in flight while
            // the warp waits for the next buffer, so nobody ever waits for it.  (The consumer warps used to load the word
            // themselves, one step ahead: every class step then took at least one L2 round trip, about a microsecond
            // under load, which was most of the kernel's time.)
            if (pruning && P.floor != nullptr && lane == 0) {
                if (floor_seen > *reinterpret_cast<volatile int*>(&sm.prune)) *reinterpret_cast<volatile int*>(&sm.prune) = floor_seen;
                floor_seen = __ldcg(P.floor + img);
            }
            // A look at the histogram delays this warp's next refill by several memory round trips, and measured end to
            // end it costs more than it saves; the CTAs of the plain-load levels take the looks instead and every other
            // CTA reads the bucket they publish (P.floor).  Only a pyramid without a plain-load level scans here (first
            // tile of every image and level, twice).
            if (pruning && P.scan_in_staged && tile == 0 && (step == 4 || step == 7)) {
                const int d = prune_digit_regs(ghist, P.prune_topk);
                if (lane == 0 && d > sm.prune) {
                    *reinterpret_cast<volatile int*>(&sm.prune) = d;
                    if (P.floor != nullptr) atomicMax(P.floor + img, d);
                }
            }
        }
        return;
    }

    // ---- phase 2 (consumer warps): per class step, lane k reads the logits of survivor k (k + 256, ... if more) ----
    YoloStWarp& ws = sm.w[warp];
    uint64_t* gkeys = P.keys + static_cast<int64_t>(img) * P.capacity;
    int32_t* gcount = P.counts + img;
    const unsigned lt = (1u << lane) - 1u;
    const StEvalArgs ea{P.thr, P.hist_base, P.hist_shift, ghist, gkeys, gcount, P.capacity, P.status};
    int fill = 0, head = 0, tail = 0;  // warp-uniform
#pragma unroll 1
    for (int step = 0; step < kStSteps; ++step) {
        const int buf = step % kStStages;
        if (pruning) {
            const int now = *reinterpret_cast<volatile int*>(&sm.prune);  // one broadcast read: the same for all lanes
            if (now > prune) {  // raise the cuts of this thread's survivors
                prune = now;
                floor_score = __uint_as_float(P.hist_base + (static_cast<uint32_t>(prune) << P.hist_shift));
                for (int k = t; k < total; k += kLiveThreads) {
                    const float so_k = sm.live[k].so;
                    sm.live[k].v_cut = so_k >= floor_score ? logit_cut(so_k, fmaxf(P.thr, floor_score)) : INFINITY;
                }
            }
        }
        const bool landed = mbar_wait_bounded(&sm.full[buf], static_cast<uint32_t>((step / kStStages) & 1), 100000u);
        if (!__all_sync(kFullMask, landed)) {  // the copy never landed: flag the call, read nothing more
            if (lane == 0 && P.status != nullptr) atomicOr(P.status, FB_STATUS_WAIT_TIMEOUT);
            break;
        }
#pragma unroll 1
        for (int k0 = warp * 32; k0 < total; k0 += kLiveThreads) {
            const int k = k0 + lane;
            const bool has = k < total;
            float vc = INFINITY;
            int ls = 0;
            if (has) {
                const YoloLive me = sm.live[k];
                vc = me.v_cut;
                ls = static_cast<int>(me.chan);
            }
            const uint32_t meta0 = (static_cast<uint32_t>(k) << 8) | static_cast<uint32_t>(step * kStClasses);
            float v[kStClasses];
#pragma unroll
            for (int u = 0; u < kStClasses; ++u) v[u] = sm.ring[buf][u][ls];
            // All votes of the step first (independent of one another), then one packing round: once the pruning floor is
            // up a step has a handful of hits per warp or none, and the warp's critical path is what a class step costs.
            unsigned m[kStClasses];
            int fresh = 0;
#pragma unroll
            for (int u = 0; u < kStClasses; ++u) {
                m[u] = __ballot_sync(kFullMask, v[u] > vc);
                fresh += __popc(m[u]);
            }
            if (fresh == 0) continue;
            if (tail - head + fresh <= kStQueue) {
                int off = tail;
#pragma unroll
                for (int u = 0; u < kStClasses; ++u) {
                    if (v[u] > vc) {
                        YoloHit e;
                        e.v = v[u];
                        e.meta = meta0 + static_cast<uint32_t>(u);
                        ws.queue[(off + __popc(m[u] & lt)) & (kStQueue - 1)] = e;
                    }
                    off += __popc(m[u]);
                }
                tail = off;
                __syncwarp();
                while (tail - head >= 32) {
                    fill = st_eval_batch(sm.live, &ws, head, 32, ea, prune, fill);
                    head += 32;
                }
                continue;
            }
            // more hits than the queue takes at once (no floor yet, or a dense image): kStSub classes at a time
#pragma unroll
            for (int h = 0; h < kStClasses; h += kStSub) {
#pragma unroll
                for (int u = 0; u < kStSub; ++u) {
                    if (v[h + u] > vc) {
                        YoloHit e;
                        e.v = v[h + u];
                        e.meta = meta0 + static_cast<uint32_t>(h + u);
                        ws.queue[(tail + __popc(m[h + u] & lt)) & (kStQueue - 1)] = e;
                    }
                    tail += __popc(m[h + u]);
                }
                __syncwarp();
                while (tail - head >= 32) {
                    fill = st_eval_batch(sm.live, &ws, head, 32, ea, prune, fill);
                    head += 32;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[buf]);  // this warp is done with ring[buf]
    }
    __syncwarp();
    if (tail - head > 0) fill = st_eval_batch(sm.live, &ws, head, tail - head, ea, prune, fill);
    if (fill > 0) st_flush(ws, fill, gkeys, gcount, P.capacity, P.status);
}

// Levels with 16-byte aligned planes go through the staged path, the others (13 x 13) through plain loads.
template <int S0, int S1, int S2>
__global__ void __launch_bounds__(kStThreads, 3)
yolo_decode_staged_kernel(const YoloParams P) {
    extern __shared__ __align__(128) unsigned char st_raw[];
    const int cta = blockIdx.x;
    const int lvl = cta >= P.live_begin[2] ? 2 : (cta >= P.live_begin[1] ? 1 : 0);
    const int local = cta - P.live_begin[lvl];
    if constexpr (S0 == 0 && S1 == 0 && S2 == 0) {  // sizes known only at run time: one body serves every level
        if (P.staged[lvl]) {
            yolo_staged_level<0>(P, lvl, local, *reinterpret_cast<YoloStagedSmem*>(st_raw));
        } else {
            YoloLiveSmem& sm = *reinterpret_cast<YoloLiveSmem*>(st_raw);
            if (threadIdx.x == 0) {
                sm.done_warps = 0;
                sm.prune = 0;
            }
            __syncthreads();
            if (threadIdx.x >= kLiveThreads) return live_scanner<0>(P, lvl, local, sm);
            yolo_live_level<0>(P, lvl, local, sm);
        }
    } else if (P.staged[lvl]) {
        YoloStagedSmem& sm = *reinterpret_cast<YoloStagedSmem*>(st_raw);
        if (lvl == 2) yolo_staged_level<S2>(P, 2, local, sm);
        else if (lvl == 1) yolo_staged_level<S1>(P, 1, local, sm);
        else yolo_staged_level<S0>(P, 0, local, sm);
    } else {
        YoloLiveSmem& sm = *reinterpret_cast<YoloLiveSmem*>(st_raw);
        if (threadIdx.x == 0) {
            sm.done_warps = 0;
            sm.prune = 0;
        }
        __syncthreads();
        if (threadIdx.x >= kLiveThreads) {  // the plain-load form has no copy producer: its ninth warp watches the histogram
            if (lvl == 2) live_scanner<S2>(P, 2, local, sm);
            else if (lvl == 1) live_scanner<S1>(P, 1, local, sm);
            else live_scanner<S0>(P, 0, local, sm);
            return;
        }
        if (lvl == 2) yolo_live_level<S2>(P, 2, local, sm);
        else if (lvl == 1) yolo_live_level<S1>(P, 1, local, sm);
        else yolo_live_level<S0>(P, 0, local, sm);
    }
}

// Development switch (functs_b200_debug_set "yolo_prune"): 0 keeps every candidate above the score threshold.
static std::atomic<int> g_yolo_prune{1};
void yolo_set_prune(int on) { g_yolo_prune.store(on ? 1 : 0, std::memory_order_relaxed); }

static const float kAnchors[3][3][2] = {{{116, 90}, {156, 198}, {373, 326}},
                                        {{30, 61}, {62, 45}, {59, 119}},
                                        {{10, 13}, {16, 30}, {33, 23}}};  // yolov3_bbox.py:191-193
static const float kStrides[3] = {32.f, 16.f, 8.f};

int launch_yolo_decode(const float* map0, const float* map1, const float* map2, int batch, int s0, int s1, int s2,
                       float score_thr, float* boxes, float* obj_out, float* cls_out, uint64_t* cand_keys,
                       int32_t* cand_counts, int64_t capacity, int32_t* hist, int zero_first, int prune_topk,
                       int32_t* floor, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(map0 && map1 && map2 && boxes && cand_keys && cand_counts, "yolo_decode: null pointer");
    FB_REQUIRE(batch > 0 && s0 > 0 && s1 > 0 && s2 > 0 && s0 <= 1024 && s1 <= 1024 && s2 <= 1024 && capacity > 0,
               "yolo_decode: bad sizes");
    FB_REQUIRE(score_thr > 0.0f, "yolo_decode: score threshold must be positive (keys require positive scores)");
    FB_REQUIRE((reinterpret_cast<uintptr_t>(boxes) & 15) == 0, "yolo_decode: boxes must be 16-byte aligned");
    YoloParams P;
    P.map[0] = map0;
    P.map[1] = map1;
    P.map[2] = map2;
    const int S[3] = {s0, s1, s2};
    int64_t tile_acc = 0;
    int box_acc = 0;
    for (int l = 0; l < 3; ++l) {
        P.size[l] = S[l];
        P.tiles[l] = (S[l] * S[l] + kYoloThreads - 1) / kYoloThreads;
        P.tile_begin[l] = static_cast<int>(tile_acc);
        tile_acc += static_cast<int64_t>(P.tiles[l]) * 3 * batch;
        P.box_begin[l] = box_acc;
        box_acc += S[l] * S[l] * 3;
        P.stride[l] = kStrides[l];
        for (int a = 0; a < 3; ++a) {
            P.anchor_w[l][a] = kAnchors[l][a][0];
            P.anchor_h[l][a] = kAnchors[l][a][1];
        }
    }
    FB_REQUIRE(tile_acc < (1ll << 31), "yolo_decode: too many tiles");
    FB_REQUIRE(static_cast<int64_t>(box_acc) * kYoloClasses < (1ll << 32), "yolo_decode: flat index exceeds 32 bits");
    P.tile_begin[3] = static_cast<int>(tile_acc);
    P.batch = batch;
    P.num_boxes = box_acc;
    P.thr = score_thr;
    P.boxes = boxes;
    P.obj_out = obj_out;
    P.cls_out = cls_out;
    P.keys = cand_keys;
    P.counts = cand_counts;
    P.capacity = capacity;
    P.status = status;
    P.hist = hist;
    P.prune_topk = (hist != nullptr && prune_topk > 0) ? prune_topk : 0;
    P.floor = P.prune_topk > 0 ? floor : nullptr;
    const HistParams hp = hist_params_for(score_thr);
    P.hist_base = hp.base;
    P.hist_shift = hp.shift;
    if (zero_first) {
        FB_TRY(check_cuda(cudaMemsetAsync(cand_counts, 0, sizeof(int32_t) * batch, st), "memset cand_counts"));
        if (hist != nullptr)
            FB_TRY(check_cuda(cudaMemsetAsync(hist, 0, sizeof(int32_t) * batch * kHistBins, st), "memset hist"));
    }
    const unsigned nblk = static_cast<unsigned>(tile_acc);
    const bool dense = obj_out != nullptr || cls_out != nullptr;
    const bool std_sizes = s0 == 13 && s1 == 26 && s2 == 52;  // the configured pyramid: strides compiled in
    if (dense) {
        if (std_sizes) yolo_decode_kernel<13, 26, 52, true><<<nblk, kYoloThreads, 0, st>>>(P);
        else yolo_decode_kernel<0, 0, 0, true><<<nblk, kYoloThreads, 0, st>>>(P);
        count_launch();
        return check_launch("yolo_decode_kernel");
    }
    FB_REQUIRE(255ll * S[0] * S[0] < (1ll << 32) && 255ll * S[1] * S[1] < (1ll << 32) && 255ll * S[2] * S[2] < (1ll << 32),
               "yolo_decode: level map too large");
    int64_t live_acc = 0;
    for (int l = 0; l < 3; ++l) {
        // a plane of S * S floats keeps every row 16-byte aligned iff S * S is a multiple of 4 (and the map itself is)
        // (and a plane at least as long as a tile, so that a tile touches at most two anchors)
        P.staged[l] = ((S[l] * S[l]) % 4 == 0 && S[l] * S[l] >= kStTile && (reinterpret_cast<uintptr_t>(P.map[l]) & 15) == 0) ? 1 : 0;
        const int tile = P.staged[l] ? kStTile : kLiveTile;
        P.live_begin[l] = static_cast<int>(live_acc);
        live_acc += static_cast<int64_t>((3 * S[l] * S[l] + tile - 1) / tile) * batch;
    }
    FB_REQUIRE(live_acc < (1ll << 31), "yolo_decode: too many tiles");
    P.live_begin[3] = static_cast<int>(live_acc);
    P.scan_in_staged = (P.staged[0] && P.staged[1] && P.staged[2]) ? 1 : 0;
    const unsigned nlive = static_cast<unsigned>(live_acc);
    const size_t smem = sizeof(YoloStagedSmem) > sizeof(YoloLiveSmem) ? sizeof(YoloStagedSmem) : sizeof(YoloLiveSmem);
    // the shared-memory opt-in is a per-device property of the kernel: set once, not on every call
    static unsigned char attr_done[2][64] = {};
    int dev = 0;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    const int slot = dev >= 0 && dev < 64 ? dev : 0;
    if (std_sizes) {
        if (!attr_done[0][slot] || dev >= 64) {
            FB_TRY(check_cuda(cudaFuncSetAttribute(yolo_decode_staged_kernel<13, 26, 52>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                              "yolo_decode attr"));
            attr_done[0][slot] = 1;
        }
        yolo_decode_staged_kernel<13, 26, 52><<<nlive, kStThreads, smem, st>>>(P);
    } else {
        if (!attr_done[1][slot] || dev >= 64) {
            FB_TRY(check_cuda(cudaFuncSetAttribute(yolo_decode_staged_kernel<0, 0, 0>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                              "yolo_decode attr"));
            attr_done[1][slot] = 1;
        }
        yolo_decode_staged_kernel<0, 0, 0><<<nlive, kStThreads, smem, st>>>(P);
    }
    count_launch();
    return check_launch("yolo_decode_staged_kernel");
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Scratch of the one-call post-process.  The first `zero_bytes` bytes hold everything that must be zero when a
// call starts (candidate counts, score histogram, selection counters) and are cleared by ONE memset.
struct YoloScratch {
    int64_t counts_off, hist_off, ctr_off, floor_off, zero_bytes;
    int64_t keys_off, sel_keys_off, sel_counts_off, lists_off, mask_off, total;
};

static YoloScratch yolo_scratch_layout(int batch, int64_t capacity, int topk) {
    YoloScratch L;
    int64_t off = 0;
    L.counts_off = off;
    off = align_up(off + static_cast<int64_t>(batch) * 4, 256);
    L.hist_off = off;
    off = align_up(off + static_cast<int64_t>(batch) * kHistBins * 4, 256);
    L.ctr_off = off;
    off = align_up(off + select_binned_ctr_bytes(batch), 256);
    L.floor_off = off;  // per image: the pruning bucket published by the decode kernel's CTAs
    off = align_up(off + static_cast<int64_t>(batch) * 4, 256);
    L.zero_bytes = off;
    L.keys_off = off;
    off = align_up(off + static_cast<int64_t>(batch) * capacity * 8, 256);
    L.sel_keys_off = off;
    off = align_up(off + static_cast<int64_t>(batch) * topk * 8, 256);
    L.sel_counts_off = off;
    off = align_up(off + static_cast<int64_t>(batch) * 4, 256);
    L.lists_off = off;
    off = align_up(off + select_binned_lists_bytes(batch), 256);
    L.mask_off = off;
    off = align_up(off + nms_mask_bytes(batch), 256);
    L.total = off;
    return L;
}

}  // namespace fb

extern "C" {

int functs_b200_yolo_decode(const float* map0, const float* map1, const float* map2, int32_t batch, int32_t s0,
                            int32_t s1, int32_t s2, float score_thr, float* boxes, float* obj_out, float* cls_out,
                            uint64_t* cand_keys, int32_t* cand_counts, int64_t capacity, int32_t* hist,
                            int32_t* status, void* stream) {
    return fb::launch_yolo_decode(map0, map1, map2, batch, s0, s1, s2, score_thr, boxes, obj_out, cls_out, cand_keys,
                                  cand_counts, capacity, hist, 1, 0, nullptr, status, fb::as_stream(stream));
}

int64_t functs_b200_yolo_scratch_bytes(int32_t batch, int32_t s0, int32_t s1, int32_t s2, int64_t capacity,
                                       int32_t topk) {
    (void)s0;
    (void)s1;
    (void)s2;
    if (batch <= 0 || capacity <= 0 || topk <= 0) return 0;
    return fb::yolo_scratch_layout(batch, capacity, topk).total;
}

int functs_b200_yolo_postprocess(const float* map0, const float* map1, const float* map2, int32_t batch, int32_t s0,
                                 int32_t s1, int32_t s2, float score_thr, int32_t topk, float iou_thr,
                                 int64_t capacity, float* boxes, float* dets, int64_t* labels, int64_t* flat_ids,
                                 int32_t* out_counts, int32_t* status, void* scratch, void* stream) {
    return functs_b200_yolo_postprocess_dense(map0, map1, map2, batch, s0, s1, s2, score_thr, topk, iou_thr, capacity,
                                              boxes, nullptr, nullptr, dets, labels, flat_ids, out_counts, nullptr,
                                              status, scratch, stream);
}

int functs_b200_yolo_postprocess_dense(const float* map0, const float* map1, const float* map2, int32_t batch,
                                       int32_t s0, int32_t s1, int32_t s2, float score_thr, int32_t topk,
                                       float iou_thr, int64_t capacity, float* boxes, float* obj_out, float* cls_out,
                                       float* dets, int64_t* labels, int64_t* flat_ids, int32_t* out_counts,
                                       int32_t* records, int32_t* status, void* scratch, void* stream) {
    using namespace fb;
    FB_REQUIRE(scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 255) == 0,
               "yolo_postprocess: scratch must be non-null and 256-byte aligned");
    FB_REQUIRE(batch > 0 && capacity > 0 && topk > 0, "yolo_postprocess: bad sizes");
    const YoloScratch L = yolo_scratch_layout(batch, capacity, topk);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    int32_t* counts = reinterpret_cast<int32_t*>(base + L.counts_off);
    int32_t* hist = reinterpret_cast<int32_t*>(base + L.hist_off);
    uint64_t* keys = reinterpret_cast<uint64_t*>(base + L.keys_off);
    uint64_t* sel_keys = reinterpret_cast<uint64_t*>(base + L.sel_keys_off);
    int32_t* sel_counts = reinterpret_cast<int32_t*>(base + L.sel_counts_off);
    cudaStream_t st = as_stream(stream);
    const int num_boxes = 3 * (s0 * s0 + s1 * s1 + s2 * s2);
    FB_TRY(check_cuda(cudaMemsetAsync(base, 0, static_cast<size_t>(L.zero_bytes), st), "memset yolo counters"));
    record_stage_event(0, st);
    // only the topk best candidates of an image are used below: let the decode kernel drop hopeless ones early
    // (with dense objectness / class-score outputs every score is formed anyway: the thread-per-box kernel, no pruning)
    FB_TRY(launch_yolo_decode(map0, map1, map2, batch, s0, s1, s2, score_thr, boxes, obj_out, cls_out, keys, counts,
                              capacity, hist, 0, g_yolo_prune.load(std::memory_order_relaxed) ? topk : 0,
                              reinterpret_cast<int32_t*>(base + L.floor_off), status, st));
    record_stage_event(1, st);
    // the CTA that finishes an image's selection also prepares the image's NMS input in the NMS work area
    FB_TRY(launch_select_binned(keys, counts, capacity, hist, score_thr, batch, topk, sel_keys, sel_counts,
                                base + L.ctr_off, base + L.lists_off, 0, boxes, num_boxes, kYoloClasses, 1,
                                base + L.mask_off, status, st));
    record_stage_event(2, st);
    const int rc = launch_batched_nms(boxes, num_boxes, kYoloClasses, sel_keys, sel_counts, batch, topk, iou_thr, 1, dets,
                                      labels, flat_ids, nullptr, out_counts, base + L.mask_off, 1, status, st, records);
    record_stage_event(3, st);
    return rc;
}

}  // extern "C"
