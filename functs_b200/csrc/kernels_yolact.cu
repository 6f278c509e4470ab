// C5: YOLACT-style mask assembly in one launch.
//
// Reference structure (functs/benchmark/ai_model/yolact/yolact_mask.py:250-264, 306-333): per image
// mask = sigmoid(proto @ coef.T), cropped to each detection's sanitised box, here by slice assignment inside a
// loop over detections, then thresholded.  The loop iterations only differ in the detection index, so the loop
// is folded into the kernel: a thread keeps the 32 prototype channels of 4 consecutive pixels in registers,
// walks the detections, evaluates the 32-term dot product (fixed k order, fp32 FMA) only where the pixel lies
// inside the crop, and stores 4 mask bytes at once.  Coefficients and crop bounds live in shared memory and are
// read as warp broadcasts.
#include "common.cuh"

namespace fb {

constexpr int kYolactThreads = 128;
constexpr int kYolactPix = 4;                            // pixels per thread (consecutive in the flat H*W order)
constexpr int kYolactTile = kYolactThreads * kYolactPix;  // pixels per CTA
constexpr int kYolactK = 32;
constexpr int kYolactMaxDet = 256;

// sanitize_coordinates (yolact_mask.py:327-333) followed by "col >= x1 and col < x2" as integer bounds.
__device__ __forceinline__ void crop_range(float a, float b, int size, int& lo, int& hi) {
    float x1 = fminf(a, b);
    float x2 = fmaxf(x1, b);
    x1 = fmaxf(__fsub_rn(x1, 1.0f), 0.0f);
    x2 = fminf(__fadd_rn(x2, 1.0f), static_cast<float>(size));
    lo = static_cast<int>(ceilf(x1));
    hi = static_cast<int>(ceilf(x2));
}

template <bool LOGITS>
__global__ void __launch_bounds__(kYolactThreads, 3)
yolact_masks_kernel(const float* __restrict__ proto, const float* __restrict__ coef, const float* __restrict__ boxes,
                    int height, int width, int num_det, float thr, uint8_t* __restrict__ masks,
                    float* __restrict__ logits) {
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

    const int p0 = blockIdx.x * kYolactTile + t * kYolactPix;
    if (p0 >= hw) return;  // hw is a multiple of 4, so a thread's 4 pixels are all in or all out

    // prototype channels of the 4 pixels -> registers (each thread reads 512 contiguous bytes)
    float pr[kYolactPix][kYolactK];
    {
        const float4* psrc = reinterpret_cast<const float4*>(proto + (static_cast<int64_t>(img) * hw + p0) * kYolactK);
#pragma unroll
        for (int u = 0; u < kYolactPix; ++u) {
#pragma unroll
            for (int q = 0; q < kYolactK / 4; ++q) {
                const float4 v = __ldg(psrc + u * (kYolactK / 4) + q);
                pr[u][4 * q + 0] = v.x;
                pr[u][4 * q + 1] = v.y;
                pr[u][4 * q + 2] = v.z;
                pr[u][4 * q + 3] = v.w;
            }
        }
    }
    int px[kYolactPix], py[kYolactPix];
#pragma unroll
    for (int u = 0; u < kYolactPix; ++u) {
        py[u] = (p0 + u) / width;
        px[u] = (p0 + u) - py[u] * width;
    }

    uint8_t* mdst = masks + static_cast<int64_t>(img) * num_det * hw + p0;
    float* ldst = LOGITS ? logits + static_cast<int64_t>(img) * num_det * hw + p0 : nullptr;
#pragma unroll 1
    for (int d = 0; d < num_det; ++d) {
        const int4 bd = s_bounds[d];
        bool in[kYolactPix];
        bool any = false;
#pragma unroll
        for (int u = 0; u < kYolactPix; ++u) {
            in[u] = px[u] >= bd.x && px[u] < bd.y && py[u] >= bd.z && py[u] < bd.w;
            any = any || in[u];
        }
        uint32_t packed = 0u;
        if (any || LOGITS) {
            float acc[kYolactPix] = {0.f, 0.f, 0.f, 0.f};
            const float4* c4 = reinterpret_cast<const float4*>(s_coef + d * kYolactK);
#pragma unroll
            for (int q = 0; q < kYolactK / 4; ++q) {
                const float4 c = c4[q];
#pragma unroll
                for (int u = 0; u < kYolactPix; ++u) {
                    acc[u] = fmaf(pr[u][4 * q + 0], c.x, acc[u]);
                    acc[u] = fmaf(pr[u][4 * q + 1], c.y, acc[u]);
                    acc[u] = fmaf(pr[u][4 * q + 2], c.z, acc[u]);
                    acc[u] = fmaf(pr[u][4 * q + 3], c.w, acc[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < kYolactPix; ++u) {
                if (in[u] && sigmoid_f32(acc[u]) > thr) packed |= (1u << (8 * u));
            }
            if (LOGITS) {
                *reinterpret_cast<float4*>(ldst + static_cast<int64_t>(d) * hw) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            }
        }
        *reinterpret_cast<uint32_t*>(mdst + static_cast<int64_t>(d) * hw) = packed;
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
    const int64_t hw = static_cast<int64_t>(height) * width;
    FB_REQUIRE(hw % 4 == 0 && hw < (1ll << 30), "yolact_masks: height * width must be a multiple of 4");
    FB_REQUIRE(((reinterpret_cast<uintptr_t>(proto) | reinterpret_cast<uintptr_t>(coef) | reinterpret_cast<uintptr_t>(boxes)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(masks) & 3) == 0 &&
                   (logits_out == nullptr || (reinterpret_cast<uintptr_t>(logits_out) & 15) == 0),
               "yolact_masks: misaligned pointer");
    dim3 grid(static_cast<unsigned>((hw + kYolactTile - 1) / kYolactTile), batch);
    if (logits_out != nullptr) {
        yolact_masks_kernel<true><<<grid, kYolactThreads, 0, as_stream(stream)>>>(proto, coef, boxes, height, width, num_det,
                                                                                  thr, masks, logits_out);
    } else {
        yolact_masks_kernel<false><<<grid, kYolactThreads, 0, as_stream(stream)>>>(proto, coef, boxes, height, width, num_det,
                                                                                   thr, masks, nullptr);
    }
    count_launch();
    return check_launch("yolact_masks_kernel");
}

}  // extern "C"
