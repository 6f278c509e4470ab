// C5: YOLACT-style mask assembly in one launch.
//
// Reference structure (functs/benchmark/ai_model/yolact/yolact_mask.py:250-264, 306-333): per image
// mask = sigmoid(proto @ coef.T), cropped to each detection's sanitised box, here by slice assignment inside a
// loop over detections, then thresholded.  The loop iterations only differ in the detection index, so the loop
// is folded into the kernel.  A warp owns a 16 x 4 pixel tile; a thread keeps the 32 prototype channels of two
// horizontally adjacent pixels in registers and walks the detections.  Per 32 detections the warp ballots which crops touch its
// tile at all; for the others it only stores zeros, for those it evaluates the 32-term dot products (fixed k order,
// fp32 FMA) and the sigmoid-threshold test.  Coefficients and crop bounds live in shared memory and are read as
// warp broadcasts.
#include <cmath>

#include "common.cuh"

namespace fb {

constexpr int kYolactThreads = 128;
constexpr int kYolactK = 32;
constexpr int kYolactMaxDet = 256;
constexpr int kYolactTileW = 16, kYolactTileH = 4;  // pixels per warp tile: 8 lanes x 2 pixels wide, 4 rows

// sanitize_coordinates (yolact_mask.py:327-333) followed by "col >= x1 and col < x2" as integer bounds.
__device__ __forceinline__ void crop_range(float a, float b, int size, int& lo, int& hi) {
    float x1 = fminf(a, b);
    float x2 = fmaxf(x1, b);
    x1 = fmaxf(__fsub_rn(x1, 1.0f), 0.0f);
    x2 = fminf(__fadd_rn(x2, 1.0f), static_cast<float>(size));
    lo = static_cast<int>(ceilf(x1));
    hi = static_cast<int>(ceilf(x2));
}

// sigmoid(v) > thr.  Outside [v_lo, v_hi] (a band around logit(thr) that is far wider than the rounding of the fp32
// sigmoid) the answer is known from v alone; inside it the fp32 sigmoid is formed and compared, so the result is
// always that of the comparison on the fp32 sigmoid.
__device__ __forceinline__ bool sigmoid_exceeds(float v, float thr, float v_lo, float v_hi) {
    if (v > v_hi) return true;
    if (v < v_lo) return false;
    return sigmoid_f32(v) > thr;
}

template <bool LOGITS>
__global__ void __launch_bounds__(kYolactThreads, 5)
yolact_masks_kernel(const float* __restrict__ proto, const float* __restrict__ coef, const float* __restrict__ boxes,
                    int height, int width, int num_det, float thr, float v_lo, float v_hi, int tiles_x, int num_tiles,
                    uint8_t* __restrict__ masks, float* __restrict__ logits) {
    __shared__ __align__(16) float s_coef[kYolactMaxDet * kYolactK];
    __shared__ int4 s_bounds[kYolactMaxDet];
    const int img = blockIdx.y;
    const int hw = height * width;
    const int t = threadIdx.x;
    {
        const float4* csrc = reinterpret_cast<const float4*>(coef + static_cast<int64_t>(img) * num_det * kYolactK);
        float4* cdst = reinterpret_cast<float4*>(s_coef);
        for (int i = t; i < num_det * (kYolactK / 4); i += kYolactThreads) cdst[i] = __ldg(csrc + i);
        for (int d = t; d < num_det; d += kYolactThreads) {
            const float4 bx = __ldg(reinterpret_cast<const float4*>(boxes) + static_cast<int64_t>(img) * num_det + d);
            int xs, xe, ys, ye;
            crop_range(bx.x, bx.z, width, xs, xe);
            crop_range(bx.y, bx.w, height, ys, ye);
            s_bounds[d] = make_int4(xs, xe, ys, ye);
        }
    }
    __syncthreads();

    const int lane = t & 31;
    const int wt = blockIdx.x * (kYolactThreads / 32) + (t >> 5);  // warp tile
    if (wt >= num_tiles) return;
    const int ty = wt / tiles_x, tx = wt - ty * tiles_x;
    const int x0 = tx * kYolactTileW, y0 = ty * kYolactTileH;
    const int x = x0 + 2 * (lane & 7);   // this thread: pixels (y, x) and (y, x + 1); the width is even
    const int y = y0 + (lane >> 3);
    const bool vpix = x < width && y < height;

    float pr[2][kYolactK];
    {
        const float4* psrc = reinterpret_cast<const float4*>(proto + (static_cast<int64_t>(img) * hw + static_cast<int64_t>(y) * width + x) * kYolactK);
#pragma unroll
        for (int q = 0; q < 2 * (kYolactK / 4); ++q) {
            const float4 v = vpix ? __ldg(psrc + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            const int u = q / (kYolactK / 4), k4 = (q % (kYolactK / 4)) * 4;
            pr[u][k4 + 0] = v.x;
            pr[u][k4 + 1] = v.y;
            pr[u][k4 + 2] = v.z;
            pr[u][k4 + 3] = v.w;
        }
    }

    uint8_t* mrow = masks + static_cast<int64_t>(img) * num_det * hw + static_cast<int64_t>(y) * width + x;
    float* lrow = LOGITS ? logits + static_cast<int64_t>(img) * num_det * hw + static_cast<int64_t>(y) * width + x : nullptr;
#pragma unroll 1
    for (int c0 = 0; c0 < num_det; c0 += 32) {
        // which of the detections c0 .. c0+31 have a crop that touches this warp's tile?
        bool touch = false;
        if (c0 + lane < num_det) {
            const int4 bd = s_bounds[c0 + lane];
            touch = bd.x < x0 + kYolactTileW && bd.y > x0 && bd.z < y0 + kYolactTileH && bd.w > y0;
        }
        const unsigned word = LOGITS ? kFullMask : __ballot_sync(kFullMask, touch);
        const int dend = min(32, num_det - c0);
#pragma unroll 1
        for (int b = 0; b < dend; ++b) {
            const int d = c0 + b;
            uint32_t out = 0u;
            if ((word >> b) & 1u) {  // warp-uniform
                const int4 bd = s_bounds[d];
                float acc0 = 0.f, acc1 = 0.f;
                const float4* c4 = reinterpret_cast<const float4*>(s_coef + d * kYolactK);
#pragma unroll
                for (int q = 0; q < kYolactK / 4; ++q) {
                    const float4 c = c4[q];
                    acc0 = fmaf(pr[0][4 * q + 0], c.x, acc0);
                    acc1 = fmaf(pr[1][4 * q + 0], c.x, acc1);
                    acc0 = fmaf(pr[0][4 * q + 1], c.y, acc0);
                    acc1 = fmaf(pr[1][4 * q + 1], c.y, acc1);
                    acc0 = fmaf(pr[0][4 * q + 2], c.z, acc0);
                    acc1 = fmaf(pr[1][4 * q + 2], c.z, acc1);
                    acc0 = fmaf(pr[0][4 * q + 3], c.w, acc0);
                    acc1 = fmaf(pr[1][4 * q + 3], c.w, acc1);
                }
                const bool iny = y >= bd.z && y < bd.w;
                if (iny && x >= bd.x && x < bd.y && sigmoid_exceeds(acc0, thr, v_lo, v_hi)) out |= 1u;
                if (iny && x + 1 >= bd.x && x + 1 < bd.y && sigmoid_exceeds(acc1, thr, v_lo, v_hi)) out |= 0x100u;
                if (LOGITS && vpix) *reinterpret_cast<float2*>(lrow + static_cast<int64_t>(d) * hw) = make_float2(acc0, acc1);
            }
            if (vpix) *reinterpret_cast<uint16_t*>(mrow + static_cast<int64_t>(d) * hw) = static_cast<uint16_t>(out);
        }
    }
}

}  // namespace fb

extern "C" {

int functs_b200_yolact_masks(const float* proto, const float* coef, const float* boxes, int32_t batch, int32_t height,
                             int32_t width, int32_t num_det, float thr, uint8_t* masks, float* logits_out,
                             void* stream) {
    using namespace fb;
    FB_REQUIRE(proto && coef && boxes && masks, "yolact_masks: null pointer");
    FB_REQUIRE(batch > 0 && batch <= 65535 && height > 0 && width > 0, "yolact_masks: bad sizes");
    FB_REQUIRE(num_det > 0 && num_det <= kYolactMaxDet, "yolact_masks: detections per image must be in [1, %d]",
               kYolactMaxDet);
    FB_REQUIRE(width % 2 == 0, "yolact_masks: the mask width must be even (pixels are stored in pairs)");
    FB_REQUIRE(thr > 0.0f && thr < 1.0f, "yolact_masks: the threshold must be in (0, 1)");
    const int64_t hw = static_cast<int64_t>(height) * width;
    FB_REQUIRE(hw < (1ll << 30), "yolact_masks: mask too large");
    FB_REQUIRE(((reinterpret_cast<uintptr_t>(proto) | reinterpret_cast<uintptr_t>(coef) | reinterpret_cast<uintptr_t>(boxes)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(masks) & 1) == 0 &&
                   (logits_out == nullptr || (reinterpret_cast<uintptr_t>(logits_out) & 7) == 0),
               "yolact_masks: misaligned pointer");
    // band around logit(thr) inside which the fp32 sigmoid decides; far outside the sigmoid's rounding error
    float v_lo = 1.0f, v_hi = -1.0f;  // empty band position = "always evaluate"
    if (thr <= 0.999f && thr >= 0.001f) {
        const double l = std::log(static_cast<double>(thr) / (1.0 - static_cast<double>(thr)));
        v_lo = static_cast<float>(l - 1.0e-3);
        v_hi = static_cast<float>(l + 1.0e-3);
    } else {
        v_lo = -INFINITY;
        v_hi = INFINITY;
    }
    const int tiles_x = (width + kYolactTileW - 1) / kYolactTileW;
    const int tiles_y = (height + kYolactTileH - 1) / kYolactTileH;
    const int num_tiles = tiles_x * tiles_y;
    const int warps = kYolactThreads / 32;
    dim3 grid(static_cast<unsigned>((num_tiles + warps - 1) / warps), batch);
    if (logits_out != nullptr) {
        yolact_masks_kernel<true><<<grid, kYolactThreads, 0, as_stream(stream)>>>(proto, coef, boxes, height, width, num_det,
                                                                                  thr, v_lo, v_hi, tiles_x, num_tiles, masks,
                                                                                  logits_out);
    } else {
        yolact_masks_kernel<false><<<grid, kYolactThreads, 0, as_stream(stream)>>>(proto, coef, boxes, height, width, num_det,
                                                                                   thr, v_lo, v_hi, tiles_x, num_tiles, masks,
                                                                                   nullptr);
    }
    count_launch();
    return check_launch("yolact_masks_kernel");
}

}  // extern "C"
