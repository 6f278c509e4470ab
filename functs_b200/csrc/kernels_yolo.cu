// C2: YOLOv3-style decode group + the post-process pipeline built on the select / NMS kernels.
//
// The decode kernel is the fusion group "permute -> reshape -> sigmoid on the xy / objectness / class slices
// (slice + sigmoid + slice_rev) -> xy grid offset -> exp * anchor -> corner form -> objectness * class score ->
// score mask" of functs/benchmark/ai_model/yolov3/yolov3_bbox.py:209-220 and :122-127, in one pass over the NCHW
// logits: threads run along the contiguous spatial axis (coalesced), every thread walks the 85 channels of one
// box, and the hits of a warp are staged in shared memory and appended to the image's candidate list.
#include "select_nms.cuh"

namespace fb {

int64_t select_binned_ctr_bytes(int groups);
int64_t select_binned_lists_bytes(int groups);
int launch_select_binned(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, const int32_t* hist,
                         float thr, int groups, int topk, uint64_t* out_keys, int32_t* out_counts, void* ctr,
                         void* lists, int zero_ctr, cudaStream_t st);
int64_t nms_mask_bytes(int groups);
int launch_batched_nms(const float* boxes, int64_t num_boxes, int num_classes, const uint64_t* sel_keys,
                       const int32_t* sel_counts, int groups, int topk, float iou_thr, int class_offset, float* dets,
                       int64_t* labels, int64_t* flat_ids, int64_t* keep, int32_t* out_counts, void* mask,
                       cudaStream_t st);

constexpr int kYoloThreads = 128;
constexpr int kYoloClasses = 80;
constexpr int kYoloAttrib = 85;
constexpr int kYoloChunk = 16;       // class logits loaded per thread before any is consumed
constexpr int kYoloSub = 8;          // logits whose hits are queued at once: <= 32 lanes * 8 = 256 new entries
constexpr int kYoloWarpStage = 96;   // staged candidate keys per warp (flushed when fewer than 32 slots remain)
constexpr int kYoloQueue = 512;      // circular queue of pending hits per warp (256 new + < 32 left over)

struct YoloParams {
    const float* map[3];
    int size[3];        // S
    int tiles[3];       // position tiles per (image, anchor) plane
    int tile_begin[4];  // first CTA of every level, [3] = total
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
        if (c0 > 0) {
#pragma unroll
            for (int u = 0; u < kYoloChunk; ++u) v[u] = __ldg(csrc + (c0 + u) * SS);
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

static const float kAnchors[3][3][2] = {{{116, 90}, {156, 198}, {373, 326}},
                                        {{30, 61}, {62, 45}, {59, 119}},
                                        {{10, 13}, {16, 30}, {33, 23}}};  // yolov3_bbox.py:191-193
static const float kStrides[3] = {32.f, 16.f, 8.f};

int launch_yolo_decode(const float* map0, const float* map1, const float* map2, int batch, int s0, int s1, int s2,
                       float score_thr, float* boxes, float* obj_out, float* cls_out, uint64_t* cand_keys,
                       int32_t* cand_counts, int64_t capacity, int32_t* hist, int zero_first, int32_t* status,
                       cudaStream_t st) {
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
    } else {
        if (std_sizes) yolo_decode_kernel<13, 26, 52, false><<<nblk, kYoloThreads, 0, st>>>(P);
        else yolo_decode_kernel<0, 0, 0, false><<<nblk, kYoloThreads, 0, st>>>(P);
    }
    count_launch();
    return check_launch("yolo_decode_kernel");
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Scratch of the one-call post-process.  The first `zero_bytes` bytes hold everything that must be zero when a
// call starts (candidate counts, score histogram, selection counters) and are cleared by ONE memset.
struct YoloScratch {
    int64_t counts_off, hist_off, ctr_off, zero_bytes;
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
                                  cand_counts, capacity, hist, 1, status, fb::as_stream(stream));
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
    FB_TRY(launch_yolo_decode(map0, map1, map2, batch, s0, s1, s2, score_thr, boxes, nullptr, nullptr, keys, counts,
                              capacity, hist, 0, status, st));
    record_stage_event(1, st);
    FB_TRY(launch_select_binned(keys, counts, capacity, hist, score_thr, batch, topk, sel_keys, sel_counts,
                                base + L.ctr_off, base + L.lists_off, 0, st));
    record_stage_event(2, st);
    const int rc = launch_batched_nms(boxes, num_boxes, kYoloClasses, sel_keys, sel_counts, batch, topk, iou_thr, 1, dets,
                                      labels, flat_ids, nullptr, out_counts, base + L.mask_off, st);
    record_stage_event(3, st);
    return rc;
}

}  // extern "C"
