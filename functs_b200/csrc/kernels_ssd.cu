// C3: SSD-style post-process in two launches.
//
// Group 1 (ssd_softmax_decode_kernel): softmax over every confidence row with the background column dropped
// (functs/benchmark/ai_model/ssd/ssd_bbox.py:268) fused with the box decode and its strided in-place clamp
// (ssd_bbox.py:121-154).  A CTA stages a tile of conf rows in shared memory with one bulk (TMA) copy when the
// tile is 16-byte aligned, each thread reduces one row (row stride 81 words: conflict-free), and the scores are
// written class-major so that group 2 reads contiguous runs.
//
// Group 2 (ssd_class_nms_kernel): the loop over classes (ssd_bbox.py:163-172 + :212 per class) with every
// (image, class) iteration mapped onto one CTA: mask > thr, top-k by (score desc, prior asc), gather boxes,
// greedy NMS, write the kept rows and their count.
#include "select_nms.cuh"

namespace fb {

constexpr int kSsdTile = 128;     // priors per CTA in group 1
constexpr int kSsdMaxRow = 96;    // maximum conf columns (C + 1) supported by the register/smem layout

// dynamic smem: [tile rows * ncol floats][8-byte mbarrier]
__global__ void __launch_bounds__(kSsdTile)
ssd_softmax_decode_kernel(const float* __restrict__ loc, const float* __restrict__ conf, const float* __restrict__ priors,
                          int num_priors, int num_classes, float clamp_max, float* __restrict__ boxes,
                          float* __restrict__ scores_cm, int use_bulk) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int ncol = num_classes + 1;
    float* tile = reinterpret_cast<float*>(smem_raw);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw + ((static_cast<size_t>(kSsdTile) * ncol * 4 + 15) / 16) * 16);
    const int img = blockIdx.y;
    const int p0 = blockIdx.x * kSsdTile;
    const int rows = min(kSsdTile, num_priors - p0);
    const int t = threadIdx.x;
    const float* gsrc = conf + (static_cast<int64_t>(img) * num_priors + p0) * ncol;
    const int nfl = rows * ncol;
    bool staged = false;
    if (use_bulk) {
        if (t == 0) {
            mbar_init(bar, 1);
            fence_barrier_init();
        }
        __syncthreads();
        if (t == 0) {
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nfl) * 4u);
            bulk_copy_g2s(tile, gsrc, static_cast<uint32_t>(nfl) * 4u, bar);
        }
        staged = mbar_wait_bounded(bar, 0, 200000u);
        // if the wait ran out (never observed), fall through to the plain loads below after the copy engine
        // had its chance; staged is uniform enough: every thread polls the same barrier
        staged = __syncthreads_and(staged ? 1 : 0) != 0;
    }
    if (!staged) {
        for (int i = t; i < nfl; i += kSsdTile) tile[i] = __ldg(gsrc + i);
        __syncthreads();
    }

    const int p = p0 + t;
    if (t < rows) {
        float* row = tile + t * ncol;
        float mx = row[0];
        for (int c = 1; c < ncol; ++c) mx = fmaxf(mx, row[c]);
        float sum = 0.0f;
        for (int c = 0; c < ncol; ++c) {
            float e = expf(__fsub_rn(row[c], mx));
            row[c] = e;
            sum = __fadd_rn(sum, e);
        }
        const float inv = __fdiv_rn(1.0f, sum);
        for (int c = 0; c < ncol; ++c) row[c] = __fmul_rn(row[c], inv);

        // decode (centre/size priors, variances 0.1 / 0.2), then clamp x to [0, max], y to [0, max]
        const float4 pr = __ldg(reinterpret_cast<const float4*>(priors) + p);
        const float4 d = __ldg(reinterpret_cast<const float4*>(loc) + static_cast<int64_t>(img) * num_priors + p);
        const float gx = __fadd_rn(pr.x, __fmul_rn(pr.z, __fmul_rn(d.x, 0.1f)));
        const float gy = __fadd_rn(pr.y, __fmul_rn(pr.w, __fmul_rn(d.y, 0.1f)));
        const float gw = __fmul_rn(pr.z, expf(__fmul_rn(d.z, 0.2f)));
        const float gh = __fmul_rn(pr.w, expf(__fmul_rn(d.w, 0.2f)));
        const float hw = __fmul_rn(gw, 0.5f), hh = __fmul_rn(gh, 0.5f);
        float4 o;
        o.x = fminf(fmaxf(__fsub_rn(gx, hw), 0.0f), clamp_max);
        o.y = fminf(fmaxf(__fsub_rn(gy, hh), 0.0f), clamp_max);
        o.z = fminf(fmaxf(__fadd_rn(gx, hw), 0.0f), clamp_max);
        o.w = fminf(fmaxf(__fadd_rn(gy, hh), 0.0f), clamp_max);
        reinterpret_cast<float4*>(boxes)[static_cast<int64_t>(img) * num_priors + p] = o;
    }
    __syncthreads();
    // class-major store: for a fixed class consecutive threads write consecutive priors
    if (t < rows) {
        const float* row = tile + t * ncol;
        float* dst = scores_cm + static_cast<int64_t>(img) * num_classes * num_priors + p;
        for (int c = 0; c < num_classes; ++c) dst[static_cast<int64_t>(c) * num_priors] = row[c];
    }
}

// ---- group 2 ------------------------------------------------------------------------------------------------
constexpr int kSsdNmsThreads = 256;
constexpr int kSsdNmsMinBlocks = 6;  // CTAs per SM the register allocation aims at (27 KB of shared memory each)
constexpr int kSsdSelCap = 256;
constexpr int kSsdWords = kSsdSelCap / 32;

constexpr size_t kSsdSelBytes = (sizeof(SelectSmem<kSsdSelCap>) + 127) / 128 * 128;
constexpr int kSsdRowBatch = 16;  // rows of the suppression matrix one warp tests at a time (4: 419 us, 8: 378, 16: 370)

// dynamic smem: [SelectSmem<256>][kCandCap candidate keys]; after the selection the NMS boxes and the 256 x 8 mask words
// live in the selection's boundary list and histogram, which are not needed any more.  The class's scores (one contiguous
// run of the class-major array) are read from global memory once: a sampled score floor, one collection pass, and the
// exact selection on the few hundred candidates (block_select_topk_sampled).
__global__ void __launch_bounds__(kSsdNmsThreads, kSsdNmsMinBlocks)
ssd_class_nms_kernel(const float* __restrict__ boxes, const float* __restrict__ scores_cm, int num_priors, int num_classes,
                     float score_thr, uint32_t hist_base, int hist_shift, int topk, float iou_thr, float thr_lo,
                     float thr_hi, float* __restrict__ dets, int64_t* __restrict__ prior_ids,
                     int32_t* __restrict__ out_counts) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    SelectSmem<kSsdSelCap>& sm = *reinterpret_cast<SelectSmem<kSsdSelCap>*>(smem_raw);
    static_assert(sizeof(NmsBox) * kSsdSelCap <= sizeof(sm.binlist) && sizeof(uint32_t) * kSsdSelCap * kSsdWords <= sizeof(sm.hist),
                  "the NMS work area must fit the parts of the selection state it reuses");
    // selected boxes as corners (one 16-byte shared load) + area, in the boundary list of the finished selection
    static_assert(sizeof(float4) * kSsdSelCap + sizeof(float) * kSsdSelCap <= sizeof(sm.binlist) &&
                      offsetof(SelectSmem<kSsdSelCap>, binlist) % 16 == 0,
                  "the corner / area arrays must fit (and be 16-byte aligned in) the boundary list");
    float4* sxy = reinterpret_cast<float4*>(sm.binlist);
    float* sarea = reinterpret_cast<float*>(sxy + kSsdSelCap);
    uint32_t* smask = reinterpret_cast<uint32_t*>(sm.hist);
    uint64_t* cand = reinterpret_cast<uint64_t*>(smem_raw + kSsdSelBytes);
    __shared__ uint32_t keep_words[kSsdWords];
    __shared__ int word_prefix[kSsdWords + 1];
    __shared__ uint32_t or_words[2 * kSsdWords];

    const int cls = blockIdx.x, img = blockIdx.y;
    const int t = threadIdx.x;
    const float* src = scores_cm + (static_cast<int64_t>(img) * num_classes + cls) * num_priors;
    const bool vec4 = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    const int n = block_select_topk_sampled<kSsdNmsThreads, kSsdSelCap>(src, vec4, score_thr, num_priors, topk, hist_base,
                                                                        hist_shift, sm, cand);
    // (block_select_topk ends with a barrier when n > 1; make the hand-over explicit)
    __syncthreads();

    const float* bimg = boxes + static_cast<int64_t>(img) * num_priors * 4;
    float4 mybox = make_float4(0.f, 0.f, 0.f, 0.f);
    uint64_t mykey = 0ull;
    bool tame_box = true;
    if (t < n) {
        mykey = sm.sel[t];
        mybox = __ldg(reinterpret_cast<const float4*>(bimg) + key_index(mykey));
        const NmsBox nb = make_nms_box(mybox.x, mybox.y, mybox.z, mybox.w);
        tame_box = nms_box_is_tame(nb);
        sxy[t] = mybox;
        sarea[t] = nb.area;
    }
    if (t < kSsdWords) keep_words[t] = 0u;
    const bool tame = __syncthreads_and(tame_box ? 1 : 0) != 0;  // also the barrier behind the box stores

    // suppression bit matrix.  A task is (column word w, batch of rows): lane b holds box j = 32w + b, the rows' boxes
    // are broadcast reads, the tests of a batch are independent and branch-free, and one ballot per row yields the
    // word, which a single lane stores: no atomics.  Word w only needs the rows i < 32w + 31; tasks are dealt
    // round-robin to the warps.
    const int lane = t & 31, warp = t >> 5;
    const int words = (n + 31) >> 5;
    for (int i = t; i < n * kSsdWords; i += kSsdNmsThreads) smask[i] = 0u;
    __syncthreads();
    {
        int total = 0;
        for (int w = 0; w < words; ++w) total += (min(n, 32 * w + 31) + kSsdRowBatch - 1) / kSsdRowBatch;
        for (int task = warp; task < total; task += kSsdNmsThreads / 32) {
            int w = 0, rb = task;
            for (;; ++w) {
                const int nb = (min(n, 32 * w + 31) + kSsdRowBatch - 1) / kSsdRowBatch;
                if (rb < nb) break;
                rb -= nb;
            }
            const int j = 32 * w + lane;
            const bool jv = j < n;
            const float4 cj = sxy[jv ? j : 0];
            const float aj = sarea[jv ? j : 0];
            const NmsBox bj{cj.x, cj.y, cj.z, cj.w, aj};
            const int i0 = rb * kSsdRowBatch;
            if (tame) {
                // Common case first: most pairs do not come near the threshold.  With the width clamped at zero the
                // product w * h is positive only for a real intersection, and for tame boxes the union is positive, so
                // "inter >= union * thr_lo" is necessary for the quotient to exceed the threshold: one vote per row on
                // that; the few pairs that pass are settled by the exact test, and a non-empty word (rare) is stored by
                // one lane.  The matrix was cleared above.
                // (Measured and dropped: the centre form (hw_a + hw_b) - |cx_a - cx_b| as an add / multiply upper bound of
                // the overlap.  It is loose when one box contains the other, which priors of one cell do all the time:
                // the exact test ran so often that the matrix took 24 us per list instead of 15.)
                // (Also measured and dropped: all votes of a batch first, then the rows with a candidate: 20 us.)
                // (And: the union test as a sum of per-box terms, inter >= c * a_i + c * a_j with c = thr / (1 + thr), plus a
                // row mask on the vote instead of the per-lane i < j test: two instructions fewer per pair on paper, 299 us
                // against 292 for the kernel.)
#pragma unroll
                for (int u = 0; u < kSsdRowBatch; ++u) {
                    const int i = i0 + u;
                    const int ii = i < n ? i : 0;
                    const float4 ci = sxy[ii];
                    const float ai = sarea[ii];
                    const float iw = fmaxf(0.0f, __fsub_rn(fminf(ci.z, cj.z), fmaxf(ci.x, cj.x)));
                    const float ih = __fsub_rn(fminf(ci.w, cj.w), fmaxf(ci.y, cj.y));
                    const float inter = __fmul_rn(iw, ih);
                    const float uni = __fsub_rn(__fadd_rn(ai, aj), inter);
                    const bool maybe = jv && i < j && !(inter < __fmul_rn(uni, thr_lo));  // i < j implies i < n
                    uint32_t bits = __ballot_sync(kFullMask, maybe);
                    if (bits != 0u) {
                        const NmsBox bi{ci.x, ci.y, ci.z, ci.w, ai};
                        bits = __ballot_sync(kFullMask, maybe && iou_exceeds(bi, bj, iou_thr, thr_lo, thr_hi));
                        if (lane == 0 && bits != 0u) smask[i * kSsdWords + w] = bits;
                    }
                }
            } else {
#pragma unroll 1
                for (int u = 0; u < kSsdRowBatch; ++u) {
                    const int i = i0 + u;
                    const int ii = i < n ? i : 0;
                    const float4 ci = sxy[ii];
                    const NmsBox bi{ci.x, ci.y, ci.z, ci.w, sarea[ii]};
                    const bool hit = jv && i < j && iou_exceeds(bi, bj, iou_thr, thr_lo, thr_hi);
                    const uint32_t bits = __ballot_sync(kFullMask, hit);
                    if (lane == 0 && bits != 0u) smask[i * kSsdWords + w] = bits;
                }
            }
        }
    }
    __syncthreads();
    block_nms_resolve<kSsdNmsThreads, kSsdWords>(smask, n, keep_words, or_words);
    __syncthreads();
    if (t == 0) {
        int acc = 0;
        for (int w = 0; w < kSsdWords; ++w) {
            word_prefix[w] = acc;
            acc += __popc(keep_words[w]);
        }
        word_prefix[kSsdWords] = acc;
        out_counts[img * num_classes + cls] = acc;
    }
    __syncthreads();
    const int64_t obase = (static_cast<int64_t>(img) * num_classes + cls) * topk;
    if (t < n) {
        const uint32_t kw = keep_words[t >> 5];
        const int b = t & 31;
        if ((kw >> b) & 1u) {
            const int rank = word_prefix[t >> 5] + __popc(kw & ((1u << b) - 1u));
            float* d = dets + (obase + rank) * 5;
            d[0] = mybox.x;
            d[1] = mybox.y;
            d[2] = mybox.z;
            d[3] = mybox.w;
            d[4] = key_score(mykey);
            prior_ids[obase + rank] = static_cast<int64_t>(key_index(mykey));
        }
    }
    const int kept = word_prefix[kSsdWords];
    for (int i = kept + t; i < topk; i += kSsdNmsThreads) {
        float* d = dets + (obase + i) * 5;
        d[0] = d[1] = d[2] = d[3] = d[4] = 0.0f;
        prior_ids[obase + i] = -1;
    }
}

}  // namespace fb

extern "C" {

int functs_b200_ssd_softmax_decode(const float* loc, const float* conf, const float* priors, int32_t batch,
                                   int32_t num_priors, int32_t num_classes, float clamp_max, float* boxes,
                                   float* scores_cm, void* stream) {
    using namespace fb;
    FB_REQUIRE(loc && conf && priors && boxes && scores_cm, "ssd_softmax_decode: null pointer");
    FB_REQUIRE(batch > 0 && batch <= 65535 && num_priors > 0 && num_classes > 0 && num_classes + 1 <= kSsdMaxRow,
               "ssd_softmax_decode: bad sizes (classes + 1 must be <= %d)", kSsdMaxRow);
    FB_REQUIRE(((reinterpret_cast<uintptr_t>(loc) | reinterpret_cast<uintptr_t>(priors) | reinterpret_cast<uintptr_t>(boxes)) & 15) == 0,
               "ssd_softmax_decode: loc, priors and boxes must be 16-byte aligned");
    const int ncol = num_classes + 1;
    // the bulk copy needs every tile start and length to be a multiple of 16 bytes
    const bool aligned = (reinterpret_cast<uintptr_t>(conf) & 15) == 0 && ((static_cast<int64_t>(num_priors) * ncol) % 4 == 0) &&
                         ((static_cast<int64_t>(kSsdTile) * ncol) % 4 == 0) &&
                         ((static_cast<int64_t>(num_priors % kSsdTile) * ncol) % 4 == 0);
    const size_t smem = ((static_cast<size_t>(kSsdTile) * ncol * 4 + 15) / 16) * 16 + 16;
    FB_TRY(check_cuda(cudaFuncSetAttribute(ssd_softmax_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "ssd_softmax_decode attr"));
    dim3 grid((num_priors + kSsdTile - 1) / kSsdTile, batch);
    ssd_softmax_decode_kernel<<<grid, kSsdTile, smem, as_stream(stream)>>>(loc, conf, priors, num_priors, num_classes,
                                                                           clamp_max, boxes, scores_cm, aligned ? 1 : 0);
    count_launch();
    return check_launch("ssd_softmax_decode_kernel");
}

int functs_b200_ssd_class_nms(const float* boxes, const float* scores_cm, int32_t batch, int32_t num_priors,
                              int32_t num_classes, float score_thr, int32_t topk, float iou_thr, float* dets,
                              int64_t* prior_ids, int32_t* out_counts, void* stream) {
    using namespace fb;
    FB_REQUIRE(boxes && scores_cm && dets && prior_ids && out_counts, "ssd_class_nms: null pointer");
    FB_REQUIRE(batch > 0 && batch <= 65535 && num_priors > 0 && num_classes > 0, "ssd_class_nms: bad sizes");
    FB_REQUIRE(topk > 0 && topk <= kSsdSelCap, "ssd_class_nms: topk must be in [1, %d]", kSsdSelCap);
    FB_REQUIRE(score_thr > 0.0f, "ssd_class_nms: score threshold must be positive");
    FB_REQUIRE(iou_thr > 0.0f && iou_thr < 1.0f, "ssd_class_nms: iou threshold must be in (0, 1)");
    FB_REQUIRE(((reinterpret_cast<uintptr_t>(boxes) | reinterpret_cast<uintptr_t>(scores_cm)) & 15) == 0,
               "ssd_class_nms: boxes and scores must be 16-byte aligned");
    const size_t smem = kSsdSelBytes + sizeof(uint64_t) * kCandCap;
    FB_TRY(check_cuda(cudaFuncSetAttribute(ssd_class_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)),
                      "ssd_class_nms attr"));
    const float thr_lo = iou_thr * (1.0f - 1.0e-6f), thr_hi = iou_thr * (1.0f + 1.0e-6f);
    dim3 grid(num_classes, batch);
    const HistParams hp = hist_params_for(score_thr);
    ssd_class_nms_kernel<<<grid, kSsdNmsThreads, smem, as_stream(stream)>>>(boxes, scores_cm, num_priors, num_classes,
                                                                            score_thr, hp.base, hp.shift, topk, iou_thr,
                                                                            thr_lo, thr_hi, dets, prior_ids, out_counts);
    count_launch();
    return check_launch("ssd_class_nms_kernel");
}

}  // extern "C"
