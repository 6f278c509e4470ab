// Library-level pieces of the C ABI: error text, launch accounting and the group registry that the
// tssa::ParallelFunctor operator binds to (reference: fait/passes/te_op.cpp:238-249 registers an operator
// whose Operation runs a compiled group; fait/fuser/graph_builder.cpp:714-927 is that Operation).
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace fb {

static thread_local char g_error[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return FB_OK;
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return FB_ERR_CUDA;
}

static thread_local cudaEvent_t g_stage_events[8];
static thread_local int g_num_stage_events = 0;

void record_stage_event(int index, cudaStream_t st) {
    if (index >= 0 && index < g_num_stage_events && g_stage_events[index] != nullptr) cudaEventRecord(g_stage_events[index], st);
}

// ---- group registry -----------------------------------------------------------------------------------
// A signature names the op sequence of a fusion group the way the group's subgraph prints it, outermost
// structure first.  Argument conventions are listed per entry; pointers are device pointers.
struct GroupEntry {
    const char* signature;
    int (*launch)(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void* scratch,
                  int32_t* status, void* stream);
};

static int g_rows(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void*, int32_t*,
                  void* stream) {
    // in: b; ia: rows, cols, n; fa: addend; out: result
    return functs_b200_rows_select_add_select_rev(static_cast<const float*>(in[0]), static_cast<float*>(out[0]), ia[0],
                                                  ia[1], ia[2], static_cast<float>(fa[0]), stream);
}

static int g_yolo_decode(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void*,
                         int32_t* status, void* stream) {
    // in: map0, map1, map2; ia: batch, s0, s1, s2, capacity; fa: score_thr; out: boxes, cand_keys, cand_counts
    return functs_b200_yolo_decode(static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                   static_cast<const float*>(in[2]), static_cast<int32_t>(ia[0]),
                                   static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]), static_cast<int32_t>(ia[3]),
                                   static_cast<float>(fa[0]), static_cast<float*>(out[0]), nullptr, nullptr,
                                   static_cast<uint64_t*>(out[1]), static_cast<int32_t*>(out[2]), ia[4], nullptr, status, stream);
}

static int g_yolo_post(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void* scratch,
                       int32_t* status, void* stream) {
    // in: map0, map1, map2; ia: batch, s0, s1, s2, topk, capacity; fa: score_thr, iou_thr;
    // out: boxes, obj (may be null), cls (may be null), dets, labels, flat_ids, counts, records (may be null)
    return functs_b200_yolo_postprocess_dense(
        static_cast<const float*>(in[0]), static_cast<const float*>(in[1]), static_cast<const float*>(in[2]),
        static_cast<int32_t>(ia[0]), static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]), static_cast<int32_t>(ia[3]),
        static_cast<float>(fa[0]), static_cast<int32_t>(ia[4]), static_cast<float>(fa[1]), ia[5],
        static_cast<float*>(out[0]), static_cast<float*>(out[1]), static_cast<float*>(out[2]), static_cast<float*>(out[3]),
        static_cast<int64_t*>(out[4]), static_cast<int64_t*>(out[5]), static_cast<int32_t*>(out[6]),
        static_cast<int32_t*>(out[7]), status, scratch, stream);
}

static int g_select_topk(const void* const* in, const int64_t* ia, const double*, void* const* out, void*, int32_t*,
                         void* stream) {
    // in: keys, counts; ia: capacity, groups, topk; out: sel_keys, sel_counts
    return functs_b200_select_topk(static_cast<const uint64_t*>(in[0]), static_cast<const int32_t*>(in[1]), ia[0],
                                   static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]),
                                   static_cast<uint64_t*>(out[0]), static_cast<int32_t*>(out[1]), stream);
}

static int g_batched_nms(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void* scratch,
                         int32_t* status, void* stream) {
    // in: boxes, sel_keys, sel_counts; ia: num_boxes, num_classes, groups, topk, class_offset; fa: iou_thr;
    // out: dets, labels, flat_ids, keep (may be null), out_counts
    return functs_b200_batched_nms(static_cast<const float*>(in[0]), ia[0], static_cast<int32_t>(ia[1]),
                                   static_cast<const uint64_t*>(in[1]), static_cast<const int32_t*>(in[2]),
                                   static_cast<int32_t>(ia[2]), static_cast<int32_t>(ia[3]), static_cast<float>(fa[0]),
                                   static_cast<int32_t>(ia[4]), static_cast<float*>(out[0]),
                                   static_cast<int64_t*>(out[1]), static_cast<int64_t*>(out[2]),
                                   static_cast<int64_t*>(out[3]), static_cast<int32_t*>(out[4]), status, scratch, stream);
}

static int g_ssd_softmax_decode(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void*,
                                int32_t*, void* stream) {
    // in: loc, conf, priors; ia: batch, num_priors, num_classes; fa: clamp_max; out: boxes, scores_cm
    return functs_b200_ssd_softmax_decode(static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                          static_cast<const float*>(in[2]), static_cast<int32_t>(ia[0]),
                                          static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]),
                                          static_cast<float>(fa[0]), static_cast<float*>(out[0]),
                                          static_cast<float*>(out[1]), stream);
}

static int g_ssd_class_nms(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void*,
                           int32_t*, void* stream) {
    // in: boxes, scores_cm; ia: batch, num_priors, num_classes, topk; fa: score_thr, iou_thr;
    // out: dets, prior_ids, out_counts
    return functs_b200_ssd_class_nms(static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                     static_cast<int32_t>(ia[0]), static_cast<int32_t>(ia[1]),
                                     static_cast<int32_t>(ia[2]), static_cast<float>(fa[0]), static_cast<int32_t>(ia[3]),
                                     static_cast<float>(fa[1]), static_cast<float*>(out[0]),
                                     static_cast<int64_t*>(out[1]), static_cast<int32_t*>(out[2]), stream);
}

static int g_yolact(const void* const* in, const int64_t* ia, const double* fa, void* const* out, void*, int32_t*,
                    void* stream) {
    // in: proto, coef, boxes; ia: batch, height, width, num_det; fa: thr; out: masks, logits [batch, N, H, W] (may be null)
    return functs_b200_yolact_masks(static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                    static_cast<const float*>(in[2]), static_cast<int32_t>(ia[0]),
                                    static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]), static_cast<int32_t>(ia[3]),
                                    static_cast<float>(fa[0]), static_cast<uint8_t*>(out[0]), static_cast<float*>(out[1]), stream);
}

static int g_lstm(const void* const* in, const int64_t* ia, const double*, void* const* out, void* scratch,
                  int32_t* status, void* stream) {
    // in: x, w_ih, w_hh, b_ih, b_hh; ia: T, B, I, H; out: hs, cs
    return functs_b200_lstm_forward(static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                    static_cast<const float*>(in[2]), static_cast<const float*>(in[3]),
                                    static_cast<const float*>(in[4]), static_cast<int32_t>(ia[0]),
                                    static_cast<int32_t>(ia[1]), static_cast<int32_t>(ia[2]), static_cast<int32_t>(ia[3]),
                                    static_cast<float*>(out[0]), static_cast<float*>(out[1]), status, scratch, stream);
}

static const GroupEntry kGroups[] = {
    {"loop[i<n]{immut::select(b,0,i)->aten::add(.,c)->immut::select_rev(b,.,0,i)}", g_rows},
    {"yolov3{permute->reshape->slice/sigmoid/slice_rev[xy,obj,cls]->add(grid)->mul(stride)->exp*anchor->corners->"
     "mul(obj,cls)->gt(thr)->nonzero}",
     g_yolo_decode},
    {"yolov3{decode->loop[b<B]{mul(obj,cls)->gt(thr)->nonzero->sort(desc,stable)->slice[:k]->class-offset nms}}", g_yolo_post},
    {"masked{sort(desc,stable)->slice[:k]}", g_select_topk},
    {"nms{max->mul(label)->add->torchvision::nms->index}", g_batched_nms},
    {"ssd{softmax(-1)->slice[:-1]->delta2bbox->slice_rev[0::2,1::2](clamp)}", g_ssd_softmax_decode},
    {"pmap[c<classes]{gt(thr)->nonzero->sort(desc,stable)->slice[:k]->index->torchvision::nms->index}", g_ssd_class_nms},
    {"loop[d<n]{matmul(proto,coef[d])->sigmoid->slice->slice_rev(crop)->gt(thr)}", g_yolact},
    {"loop[t<T]{matmul(x[t],w_ih)+matmul(h,w_hh)->immut::select[gates]->sigmoid/tanh->select_rev(hs,t)->select_rev(cs,t)}",
     g_lstm},
};
static const int kNumGroups = static_cast<int>(sizeof(kGroups) / sizeof(kGroups[0]));

}  // namespace fb

extern "C" {

int functs_b200_abi_version(void) { return 2; }
const char* functs_b200_last_error(void) { return fb::g_error; }
uint64_t functs_b200_launch_count(void) { return fb::g_launches.load(std::memory_order_relaxed); }

void functs_b200_set_stage_events(void* const* events, int32_t count) {
    if (events == nullptr || count <= 0) {
        fb::g_num_stage_events = 0;
        return;
    }
    if (count > 8) count = 8;
    for (int i = 0; i < count; ++i) fb::g_stage_events[i] = static_cast<cudaEvent_t>(events[i]);
    fb::g_num_stage_events = count;
}

int functs_b200_group_count(void) { return fb::kNumGroups; }

const char* functs_b200_group_signature(int group_id) {
    if (group_id < 0 || group_id >= fb::kNumGroups) return nullptr;
    return fb::kGroups[group_id].signature;
}

int functs_b200_group_lookup(const char* signature) {
    if (signature == nullptr) return FB_ERR_NOT_FOUND;
    for (int i = 0; i < fb::kNumGroups; ++i) {
        if (std::strcmp(signature, fb::kGroups[i].signature) == 0) return i;
    }
    fb::set_error("no precompiled kernel for group signature '%s'", signature);
    return FB_ERR_NOT_FOUND;
}

int functs_b200_group_launch(int group_id, const void* const* in_ptrs, const int64_t* int_args,
                             const double* float_args, void* const* out_ptrs, void* scratch, int32_t* status,
                             void* stream) {
    if (group_id < 0 || group_id >= fb::kNumGroups) {
        fb::set_error("group id %d outside [0, %d)", group_id, fb::kNumGroups);
        return FB_ERR_NOT_FOUND;
    }
    if (in_ptrs == nullptr || out_ptrs == nullptr || int_args == nullptr) {
        fb::set_error("group_launch: null argument array");
        return FB_ERR_INVALID_ARGUMENT;
    }
    static const double kNoFloats[4] = {0, 0, 0, 0};
    return fb::kGroups[group_id].launch(in_ptrs, int_args, float_args ? float_args : kNoFloats, out_ptrs, scratch, status,
                                        stream);
}

}  // extern "C"
