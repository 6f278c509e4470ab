// Masked index (threshold + compaction), top-k selection and greedy NMS as stand-alone launches.
// These are the un-fused ATen / torchvision steps that sit between the reference's fusion groups
// (nonzero, bool-mask index, sort, torchvision.ops.nms — reference call sites
// functs/benchmark/ai_model/yolov3/yolov3_bbox.py:122-134, 144-151, 177 and ssd/ssd_bbox.py:163-172, 212).
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
                         int32_t* __restrict__ counts, int64_t capacity, int32_t* status) {
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
        warp_stage_push(stage, fill, pred, make_key(v, static_cast<uint32_t>(i)));
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

// ---- NMS: suppression bit matrix (many CTAs per group) + serial scan (one CTA per group) ---------
// Both kernels rebuild the same NMS-space boxes from the selected keys: gather the box of every selected
// candidate, take the maximum coordinate over them, shift each box by label * (max + 1).
constexpr int kNmsThreads = 1024;
constexpr int kNmsMaxN = 1024;
constexpr int kNmsWords = kNmsMaxN / 32;

struct NmsGather {
    float4 raw;  // un-shifted box
    float score;
    int label;
    uint32_t flat;
};

// Every thread t < n gathers candidate t; the block computes the maximum coordinate; returns the shifted box.
__device__ __forceinline__ NmsBox gather_nms_box(const float* __restrict__ boxes_g, const uint64_t* __restrict__ sel,
                                                  int n, int num_classes, int class_offset, float* red /*[33]*/,
                                                  NmsGather& out) {
    const int t = threadIdx.x;
    float4 bx = make_float4(0.f, 0.f, 0.f, 0.f);
    out.score = 0.f;
    out.label = 0;
    out.flat = 0;
    float lmax = -INFINITY;
    if (t < n) {
        uint64_t k = sel[t];
        uint32_t flat = key_index(k);
        uint32_t box = flat / static_cast<uint32_t>(num_classes);
        out.flat = flat;
        out.label = static_cast<int>(flat - box * static_cast<uint32_t>(num_classes));
        out.score = key_score(k);
        bx = reinterpret_cast<const float4*>(boxes_g)[box];
        lmax = fmaxf(fmaxf(bx.x, bx.y), fmaxf(bx.z, bx.w));
    }
    out.raw = bx;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(kFullMask, lmax, o));
    if ((t & 31) == 0) red[t >> 5] = lmax;
    __syncthreads();
    if (t < 32) {
        float v = (t < (blockDim.x >> 5)) ? red[t] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
        if (t == 0) red[32] = v;
    }
    __syncthreads();
    float off = 0.0f;
    if (class_offset) off = __fmul_rn(static_cast<float>(out.label), __fadd_rn(red[32], 1.0f));
    return make_nms_box(__fadd_rn(bx.x, off), __fadd_rn(bx.y, off), __fadd_rn(bx.z, off), __fadd_rn(bx.w, off));
}

// grid = (row tiles of 32 rows, groups); block = 1024 threads = 32 warps, one row of the bit matrix per warp.
__global__ void __launch_bounds__(kNmsThreads)
nms_mask_kernel(const float* __restrict__ boxes, int64_t num_boxes, int num_classes, const uint64_t* __restrict__ sel_keys,
                const int32_t* __restrict__ sel_counts, int topk, float thr, float thr_lo, float thr_hi,
                int class_offset, uint32_t* __restrict__ mask_out) {
    __shared__ NmsBox sb[kNmsMaxN];
    __shared__ float red[33];
    const int g = blockIdx.y;
    int n = sel_counts[g];
    if (n > topk) n = topk;
    const int row0 = blockIdx.x * 32;
    if (row0 >= n) return;
    NmsGather gth;
    NmsBox mine = gather_nms_box(boxes + static_cast<int64_t>(g) * num_boxes * 4, sel_keys + static_cast<int64_t>(g) * topk,
                                 n, num_classes, class_offset, red, gth);
    sb[threadIdx.x] = mine;
    __syncthreads();
    // warp r owns row row0 + r; lane b tests box 32w + b, so consecutive lanes read consecutive boxes
    const int r = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int i = row0 + r;
    const int words = (n + 31) >> 5;
    uint32_t bits = 0u;
    if (i < n) {
        const NmsBox bi = sb[i];
        for (int w = i >> 5; w < words; ++w) {
            const int j = w * 32 + lane;
            bool pred = false;
            if (j > i && j < n) pred = iou_exceeds(bi, sb[j], thr, thr_lo, thr_hi);
            unsigned m = __ballot_sync(kFullMask, pred);
            if (lane == w) bits = m;
        }
        mask_out[(static_cast<int64_t>(g) * kNmsMaxN + i) * kNmsWords + lane] = bits;
    }
}

// grid = groups; block = 1024.  Stages the group's bit matrix in shared memory, one warp scans, all threads
// write the compacted outputs.
__global__ void __launch_bounds__(kNmsThreads)
nms_scan_kernel(const float* __restrict__ boxes, int64_t num_boxes, int num_classes, const uint64_t* __restrict__ sel_keys,
                const int32_t* __restrict__ sel_counts, int topk, const uint32_t* __restrict__ mask_in,
                float* __restrict__ dets, int64_t* __restrict__ labels, int64_t* __restrict__ flat_ids,
                int64_t* __restrict__ keep, int32_t* __restrict__ out_counts) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* smask = reinterpret_cast<uint32_t*>(smem_raw);  // [n][32]
    __shared__ uint32_t keep_words[kNmsWords];
    __shared__ int word_prefix[kNmsWords + 1];
    const int g = blockIdx.x;
    const int t = threadIdx.x;
    int n = sel_counts[g];
    if (n > topk) n = topk;
    const int words = (n + 31) >> 5;
    // stage rows [0, n) (row stride 32 words), 16 bytes per thread per step
    {
        const uint4* src = reinterpret_cast<const uint4*>(mask_in + static_cast<int64_t>(g) * kNmsMaxN * kNmsWords);
        uint4* dst = reinterpret_cast<uint4*>(smask);
        const int total = n * (kNmsWords / 4);
        for (int i = t; i < total; i += kNmsThreads) dst[i] = src[i];
    }
    if (t < kNmsWords) keep_words[t] = 0u;
    __syncthreads();
    if (t < 32) warp_nms_scan(smask, kNmsWords, n, words, keep_words);
    __syncthreads();
    if (t == 0) {
        int acc = 0;
        for (int w = 0; w < kNmsWords; ++w) {
            word_prefix[w] = acc;
            acc += __popc(keep_words[w]);
        }
        word_prefix[kNmsWords] = acc;
        out_counts[g] = acc;
    }
    __syncthreads();
    const int64_t obase = static_cast<int64_t>(g) * topk;
    if (t < n) {
        uint32_t kw = keep_words[t >> 5];
        int b = t & 31;
        if ((kw >> b) & 1u) {
            int rank = word_prefix[t >> 5] + __popc(kw & ((1u << b) - 1u));
            uint64_t k = sel_keys[obase + t];
            uint32_t flat = key_index(k);
            uint32_t box = flat / static_cast<uint32_t>(num_classes);
            float4 bx = reinterpret_cast<const float4*>(boxes + static_cast<int64_t>(g) * num_boxes * 4)[box];
            float* d = dets + (obase + rank) * 5;
            d[0] = bx.x;
            d[1] = bx.y;
            d[2] = bx.z;
            d[3] = bx.w;
            d[4] = key_score(k);
            labels[obase + rank] = static_cast<int64_t>(flat - box * static_cast<uint32_t>(num_classes));
            flat_ids[obase + rank] = static_cast<int64_t>(flat);
            if (keep != nullptr) keep[obase + rank] = t;
        }
    }
    // zero the tail so that the padded outputs are deterministic
    const int total_kept = word_prefix[kNmsWords];
    for (int i = total_kept + t; i < topk; i += kNmsThreads) {
        float* d = dets + (obase + i) * 5;
        d[0] = d[1] = d[2] = d[3] = d[4] = 0.0f;
        labels[obase + i] = -1;
        flat_ids[obase + i] = -1;
        if (keep != nullptr) keep[obase + i] = -1;
    }
}

// ---- host launchers (internal C++ API, used by the C ABI and by the YOLO pipeline) ----------------
int launch_threshold_compact(const float* scores, int groups, int64_t n, float thr, uint64_t* keys, int32_t* counts,
                             int64_t capacity, int zero_counts, int32_t* status, cudaStream_t st) {
    FB_REQUIRE(scores && keys && counts, "threshold_compact: null pointer");
    FB_REQUIRE(groups > 0 && groups <= 65535 && n > 0 && n < (1ll << 32) && capacity > 0, "threshold_compact: bad sizes");
    if (zero_counts) FB_TRY(check_cuda(cudaMemsetAsync(counts, 0, sizeof(int32_t) * groups, st), "memset counts"));
    const int64_t chunk = static_cast<int64_t>(kCompactThreads) * kCompactPerThread;
    dim3 grid(static_cast<unsigned>((n + chunk - 1) / chunk), groups);
    threshold_compact_kernel<<<grid, kCompactThreads, 0, st>>>(scores, n, thr, keys, counts, capacity, status);
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

int64_t nms_scratch_bytes(int groups, int topk) {
    (void)topk;
    return static_cast<int64_t>(groups) * kNmsMaxN * kNmsWords * sizeof(uint32_t);
}

int launch_batched_nms(const float* boxes, int64_t num_boxes, int num_classes, const uint64_t* sel_keys,
                       const int32_t* sel_counts, int groups, int topk, float iou_thr, int class_offset, float* dets,
                       int64_t* labels, int64_t* flat_ids, int64_t* keep, int32_t* out_counts, void* scratch,
                       cudaStream_t st) {
    FB_REQUIRE(boxes && sel_keys && sel_counts && dets && labels && flat_ids && out_counts && scratch,
               "batched_nms: null pointer");
    FB_REQUIRE(groups > 0 && groups <= 65535 && topk > 0 && topk <= kNmsMaxN && num_classes > 0 && num_boxes > 0,
               "batched_nms: bad sizes (topk must be in [1, %d])", kNmsMaxN);
    FB_REQUIRE(iou_thr > 0.0f && iou_thr < 1.0f, "batched_nms: iou threshold must be in (0, 1)");
    FB_REQUIRE((reinterpret_cast<uintptr_t>(boxes) & 15) == 0 && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0,
               "batched_nms: boxes and scratch must be 16-byte aligned");
    const float thr_lo = iou_thr * (1.0f - 1.0e-6f), thr_hi = iou_thr * (1.0f + 1.0e-6f);
    uint32_t* mask = static_cast<uint32_t*>(scratch);
    dim3 grid((topk + 31) / 32, groups);
    nms_mask_kernel<<<grid, kNmsThreads, 0, st>>>(boxes, num_boxes, num_classes, sel_keys, sel_counts, topk, iou_thr,
                                                  thr_lo, thr_hi, class_offset, mask);
    count_launch();
    FB_TRY(check_launch("nms_mask_kernel"));
    const size_t smem = static_cast<size_t>(kNmsMaxN) * kNmsWords * sizeof(uint32_t);
    FB_TRY(check_cuda(cudaFuncSetAttribute(nms_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "nms_scan attr"));
    nms_scan_kernel<<<groups, kNmsThreads, smem, st>>>(boxes, num_boxes, num_classes, sel_keys, sel_counts, topk, mask,
                                                       dets, labels, flat_ids, keep, out_counts);
    count_launch();
    return check_launch("nms_scan_kernel");
}

}  // namespace fb

// ---- C ABI ------------------------------------------------------------------------------------------
extern "C" {

int functs_b200_threshold_compact(const float* scores, int32_t groups, int64_t n, float thr, uint64_t* keys,
                                  int32_t* counts, int64_t capacity, int32_t zero_counts, int32_t* status,
                                  void* stream) {
    return fb::launch_threshold_compact(scores, groups, n, thr, keys, counts, capacity, zero_counts, status,
                                        fb::as_stream(stream));
}

int functs_b200_select_topk(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, int32_t groups,
                            int32_t topk, uint64_t* out_keys, int32_t* out_counts, void* stream) {
    return fb::launch_select_topk(in_keys, in_counts, capacity, groups, topk, out_keys, out_counts,
                                  fb::as_stream(stream));
}

int64_t functs_b200_nms_scratch_bytes(int32_t groups, int32_t topk) { return fb::nms_scratch_bytes(groups, topk); }

int functs_b200_batched_nms(const float* boxes, int64_t num_boxes, int32_t num_classes, const uint64_t* sel_keys,
                            const int32_t* sel_counts, int32_t groups, int32_t topk, float iou_thr,
                            int32_t class_offset, float* dets, int64_t* labels, int64_t* flat_ids, int64_t* keep,
                            int32_t* out_counts, void* scratch, void* stream) {
    return fb::launch_batched_nms(boxes, num_boxes, num_classes, sel_keys, sel_counts, groups, topk, iou_thr,
                                  class_offset, dets, labels, flat_ids, keep, out_counts, scratch,
                                  fb::as_stream(stream));
}

}  // extern "C"
