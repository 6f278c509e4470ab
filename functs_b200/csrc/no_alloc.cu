// functs_b200_batched_nms_static: batched NMS for callers that cannot hand the library a scratch buffer.
//
// Who needs it: a host that binds only this C ABI and owns no device allocator of its own — for example a serving
// process whose whole device memory was given to another framework's pool at start-up, or a post-processing step
// that runs in a latency-critical loop where a cudaMalloc (which synchronises the whole device) is not acceptable.
// Such a caller can still provide inputs and outputs (they are part of its fixed memory plan) but has nowhere to
// take the 157 KB-per-group work area (suppression matrix, row flags, prepared boxes) from.  Here it lives in a
// file-scope __device__ array.
//
// Cost and limits: the array is kStaticNmsGroups * 157 KB = 1258 KB (about 1.3 MB) of device memory on EVERY GPU that loads the
// library, held until the process exits.  At most kStaticNmsGroups groups per call.  All calls share the array:
// two calls whose kernels can overlap on the GPU (different streams, different host threads) race on it — serialise
// them.  Nothing in the array has to start at zero: the kernels write every word, flag and prepared box that a
// later kernel of the same call reads, so stale contents of an earlier call are never observed.
#include <mutex>

#include "common.cuh"

namespace fb {

int launch_batched_nms(const float* boxes, int64_t num_boxes, int num_classes, const uint64_t* sel_keys,
                       const int32_t* sel_counts, int groups, int topk, float iou_thr, int class_offset, float* dets,
                       int64_t* labels, int64_t* flat_ids, int64_t* keep, int32_t* out_counts, void* mask, int prepared,
                       int32_t* status, cudaStream_t st, int32_t* records = nullptr);
int64_t nms_mask_bytes(int groups);

constexpr int kStaticNmsGroups = 8;
// per group: the 1024 x 1024 bit matrix (128 KB), one flag byte per row (1 KB) and the prepared boxes / class buckets
// (28928 bytes) and an arrival counter (4 bytes); plus 256 bytes of alignment slack.  Checked against nms_mask_bytes() at every call.
constexpr size_t kStaticNmsBytes = static_cast<size_t>(kStaticNmsGroups) * (1024 * 32 * sizeof(uint32_t) + 1024 + 28928 + 4) + 256;  // 1258 KB

// In host code this name is only a handle for the symbol, not a device address: the address is looked up per device.
static __device__ __align__(256) unsigned char g_static_nms_scratch[kStaticNmsBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the CURRENT device (looked up once per device, then cached).
static int static_nms_scratch(void** out) {
    int dev = -1;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    FB_REQUIRE(dev >= 0 && dev < kMaxDevices, "batched_nms_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        FB_TRY(check_cuda(cudaGetSymbolAddress(&p, g_static_nms_scratch), "cudaGetSymbolAddress(static NMS scratch)"));
        FB_REQUIRE(p != nullptr && (reinterpret_cast<uintptr_t>(p) & 255) == 0, "batched_nms_static: bad symbol address");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return FB_OK;
}

}  // namespace fb

extern "C" {

int32_t functs_b200_batched_nms_static_max_groups(void) { return fb::kStaticNmsGroups; }

int functs_b200_batched_nms_static(const float* boxes, int64_t num_boxes, int32_t num_classes, const uint64_t* sel_keys,
                                   const int32_t* sel_counts, int32_t groups, int32_t topk, float iou_thr,
                                   int32_t class_offset, float* dets, int64_t* labels, int64_t* flat_ids,
                                   int64_t* keep, int32_t* out_counts, int32_t* status, void* stream) {
    using namespace fb;
    FB_REQUIRE(groups > 0 && groups <= kStaticNmsGroups,
               "batched_nms_static: %d groups requested, the built-in scratch holds at most %d (use "
               "functs_b200_batched_nms with caller-provided scratch for more)",
               groups, kStaticNmsGroups);
    FB_REQUIRE(static_cast<size_t>(nms_mask_bytes(groups)) <= kStaticNmsBytes, "batched_nms_static: scratch too small");
    void* scratch = nullptr;
    FB_TRY(static_nms_scratch(&scratch));
    return launch_batched_nms(boxes, num_boxes, num_classes, sel_keys, sel_counts, groups, topk, iou_thr, class_offset,
                              dets, labels, flat_ids, keep, out_counts, scratch, 0, status, as_stream(stream));
}

}  // extern "C"
