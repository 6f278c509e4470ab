/*
 * functs_b200 — C ABI of the B200 (sm_100a) executor for FuncTs fusion groups.
 *
 * Every entry point is a thin launcher over precompiled kernels: plain device pointers and
 * sizes in, an integer status out.  No entry point allocates device memory, synchronises
 * the device or touches a stream other than the one it is given (``stream`` is a
 * ``cudaStream_t`` passed as ``void*``; NULL = the legacy default stream).  Work that needs
 * temporary device memory takes a caller-allocated ``scratch`` pointer whose size the
 * matching ``*_scratch_bytes`` function reports.
 *
 * What each entry point replaces in the reference (paths inside the reference project):
 * the reference executes a fusion group through ``GraphBuilder::run``
 * (fait/fuser/graph_builder.cpp:714-927), which marshals IValues, allocates outputs and
 * calls one NVRTC-compiled kernel per group through ``CudaCodeGenTssa::call``
 * (fait/tensorexpr/cuda_codegen_tssa.cpp:1167-1290).  Here the group bodies are fixed,
 * hand-written kernels and the caller (the operator shim) owns allocation.
 *
 * Return value: FB_OK (0) or a negative FB_ERR_* code; ``functs_b200_last_error`` gives a
 * message for the calling thread.  Kernels never trap: data-dependent problems (a candidate
 * buffer that is too small) are reported through the int32 ``status`` word in device memory.
 */
#ifndef FUNCTS_B200_H_
#define FUNCTS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_OK 0
#define FB_ERR_INVALID_ARGUMENT (-1)
#define FB_ERR_CUDA (-2)
#define FB_ERR_UNSUPPORTED (-3)
#define FB_ERR_NOT_FOUND (-4)

/* bits of the device status word */
#define FB_STATUS_CAND_OVERFLOW 1 /* a candidate list was longer than its capacity; extra candidates were dropped */
#define FB_STATUS_WAIT_TIMEOUT 2  /* a bounded device-side wait ran out */
#define FB_STATUS_INDEX_RANGE 4   /* an index tensor (or a candidate key) named a row outside the indexed extent */

/* ---- library ------------------------------------------------------------------------- */

/* ABI version of this header (bumped on incompatible change). */
int functs_b200_abi_version(void);
/* Message of the last failing call made by this thread ("" if none). */
const char* functs_b200_last_error(void);
/* Kernels launched by this library in this process so far (the reference counts launches with
 * CUPTI, fait/util/profile.cpp:39-41; the "kernels per call" metric is a difference of two reads). */
uint64_t functs_b200_launch_count(void);

/* Profiling hook (the reference brackets regions with prof::Begin/End ops, fait/util/profile.cpp:123-149): arms up to
 * 8 caller-owned cudaEvent_t handles for the calling thread; multi-stage entry points record event k on their stream
 * before stage k and the next one after the last stage.  count = 0 disarms. */
void functs_b200_set_stage_events(void* const* events, int32_t count);

/* ---- C1: loop { select(b,0,i) -> add -> select_rev(b,.,0,i) } on a cloned, carried tensor -- */
/* Replaces the group printed in the reference README.md:284-299 (examples/get_started.py:10-15):
 * out = clone(b); out[i,:] = b[i,:] + addend for 0 <= i < n.  b, out: [rows, cols] fp32, contiguous.
 * One launch; loop iterations map onto CTAs. */
int functs_b200_rows_select_add_select_rev(const float* b, float* out, int64_t rows, int64_t cols, int64_t n,
                                           float addend, void* stream);

/* ---- masked index / top-k / NMS building blocks (shared by C2 and C3) ------------------- */
/* Candidate key = (float bits of the score) << 32 | (0xFFFFFFFF - flat index); descending key order is
 * "score descending, then index ascending", i.e. nonzero() followed by a stable descending sort
 * (functs/benchmark/ai_model/ssd/ssd_bbox.py:163-172).  Scores must be > 0. */

/* scores [groups, n] fp32 -> keys of the elements > thr, per group, in unspecified order.
 * keys [groups, capacity], counts [groups] int32 (must be zeroed by the caller or by zero_counts=1).
 * hist (optional, [groups, functs_b200_hist_bins()] int32, zeroed like counts): coarse histogram of the candidate
 * scores, the input of functs_b200_select_topk_binned. */
int32_t functs_b200_hist_bins(void);
int functs_b200_threshold_compact(const float* scores, int32_t groups, int64_t n, float thr, uint64_t* keys,
                                  int32_t* counts, int64_t capacity, int32_t zero_counts, int32_t* hist,
                                  int32_t* status, void* stream);

/* Per group: the topk largest keys, sorted descending. in_keys [groups, capacity] with in_counts valid
 * entries (clamped to capacity); out_keys [groups, topk]; out_counts [groups] = min(count, topk).  topk <= 1024. */
int functs_b200_select_topk(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity, int32_t groups,
                            int32_t topk, uint64_t* out_keys, int32_t* out_counts, void* stream);

/* The same selection for long candidate lists: 4 CTAs per group collect the keys above / inside the boundary
 * bucket of the score histogram `hist` (filled by the candidate producer with the same thr), the CTA that finishes
 * last sorts; if a group's boundary bucket holds more keys than the sort buffer, or the histogram and the keys
 * disagree, that CTA runs the exact generic selection over the whole list instead (1 launch either way).
 * hist must be 16-byte aligned.  scratch: functs_b200_select_binned_scratch_bytes(groups), 256-byte aligned. */
int64_t functs_b200_select_binned_scratch_bytes(int32_t groups);
int functs_b200_select_topk_binned(const uint64_t* in_keys, const int32_t* in_counts, int64_t capacity,
                                   const int32_t* hist, float thr, int32_t groups, int32_t topk, uint64_t* out_keys,
                                   int32_t* out_counts, void* scratch, void* stream);

/* Greedy IoU NMS over the selected candidates of every group, as torchvision.ops.nms does on CPU
 * (call sites yolov3_bbox.py:177, ssd_bbox.py:212), optionally class-wise through the coordinate-offset
 * trick of yolov3_bbox.py:144-146 (class_offset != 0: offset = label * (max coordinate of the selected boxes + 1)).
 * boxes [groups, num_boxes, 4]; sel_keys [groups, topk] sorted; flat index = box * num_classes + label.
 * Outputs (fixed capacity topk per group, first out_counts[g] rows valid, score-descending):
 *   dets [groups, topk, 5] (x1,y1,x2,y2,score), labels [groups, topk] int64, flat_ids [groups, topk] int64,
 *   keep [groups, topk] int64 (position in the selected list), out_counts [groups] int32.
 * A key whose box index (flat index / num_classes) is not below num_boxes is never used as an address: that candidate
 * takes no part in the NMS (it neither survives nor suppresses), and FB_STATUS_INDEX_RANGE is set in `status`
 * (optional device word, may be NULL).
 * scratch: functs_b200_nms_scratch_bytes(groups, topk). */
int64_t functs_b200_nms_scratch_bytes(int32_t groups, int32_t topk);
int functs_b200_batched_nms(const float* boxes, int64_t num_boxes, int32_t num_classes, const uint64_t* sel_keys,
                            const int32_t* sel_counts, int32_t groups, int32_t topk, float iou_thr,
                            int32_t class_offset, float* dets, int64_t* labels, int64_t* flat_ids, int64_t* keep,
                            int32_t* out_counts, int32_t* status, void* scratch, void* stream);

/* The same NMS for callers that cannot provide scratch memory.  No counterpart in the reference (its executor always
 * allocates through torch's caching allocator).  Meant for hosts that bind only this C ABI and own no device allocator
 * — all device memory belongs to another framework's pool, or a cudaMalloc (a device-wide synchronisation) is not
 * acceptable inside their loop.  The suppression matrix lives in a 1258 KB (about 1.3 MB) __device__ array inside the library (held on
 * every GPU that loads the library, until exit), so groups <= functs_b200_batched_nms_static_max_groups() (8); more
 * groups are rejected with FB_ERR_INVALID_ARGUMENT.  The entry point calls no cudaMalloc / cudaFree or any allocating
 * routine.  The first call on a device looks the array's address up (cudaGetSymbolAddress) with that device current:
 * make that first call before any stream capture.  All calls share the array; calls whose kernels can overlap on
 * the GPU race on it.  Inputs and outputs exactly as functs_b200_batched_nms. */
int32_t functs_b200_batched_nms_static_max_groups(void);
int functs_b200_batched_nms_static(const float* boxes, int64_t num_boxes, int32_t num_classes, const uint64_t* sel_keys,
                                   const int32_t* sel_counts, int32_t groups, int32_t topk, float iou_thr,
                                   int32_t class_offset, float* dets, int64_t* labels, int64_t* flat_ids,
                                   int64_t* keep, int32_t* out_counts, int32_t* status, void* stream);

/* Packs the padded outputs of batched_nms / yolo_postprocess into 32-byte records for the multi-GPU gather of final
 * detections (the step that follows the reference's per-image loop when the batch is sharded over GPUs; the reference
 * itself is single-device, its callers concatenate per-image results on the host: yolov3_bbox.py:236-243).
 * records [groups, topk, 8] int32: words 0..4 = x1, y1, x2, y2, score (fp32 bits), 5 = label, 6 = flat id,
 * 7 = 1 for a valid row (k < counts[g]) and 0 for padding.  16-byte aligned. */
int functs_b200_pack_detections(const float* dets, const int64_t* labels, const int64_t* flat_ids, const int32_t* counts,
                                int32_t groups, int32_t topk, int32_t* records, void* stream);

/* Pushes `bytes` of packed records from this GPU into a buffer that may live on another GPU of the box (a pointer this
 * process got by opening the owner's CUDA IPC handle): one asynchronous copy on `stream`, carried out by a copy engine
 * over NVLink, no kernel on either GPU.  The one-sided form of "only the final detections are gathered": every rank
 * pushes its shard into its slot of the destination rank's buffer; the caller confirms arrival with one small
 * collective per block of steps.  Both pointers 16-byte aligned, bytes a multiple of 16. */
int functs_b200_push_records(void* dst, const int32_t* records, int64_t bytes, void* stream);

/* ---- C2: YOLOv3-style decode + score mask + top-k + class-wise NMS ----------------------- */
/* Follows functs/benchmark/ai_model/yolov3/yolov3_bbox.py:195-243 at the configured shapes:
 * three NCHW logit maps [batch, 255, S, S]; box order is level, y, x, anchor. */

/* Decode group (one launch): permute/reshape, sigmoid on the xy / objectness / class slices, xy grid offset and
 * stride, wh = exp * anchor, corner form, score = obj * cls, mask score > thr, compaction into candidate keys.
 * boxes [batch, N, 4] with N = 3*(s0^2+s1^2+s2^2); obj_out [batch, N] and cls_out [batch, N, 80] are optional
 * (NULL = not written; they exist for value-parity checks); cand_keys [batch, capacity]; cand_counts [batch] and
 * the optional score histogram hist [batch, functs_b200_hist_bins()] are zeroed by the launch sequence. */
int functs_b200_yolo_decode(const float* map0, const float* map1, const float* map2, int32_t batch, int32_t s0,
                            int32_t s1, int32_t s2, float score_thr, float* boxes, float* obj_out, float* cls_out,
                            uint64_t* cand_keys, int32_t* cand_counts, int64_t capacity, int32_t* hist,
                            int32_t* status, void* stream);

/* Whole post-process: one memset + decode -> select_topk_binned -> batched_nms(class_offset=1): 3 kernel launches
 * (decode + mask + compaction; top-k selection, which also lays out the NMS input; NMS bit matrix + greedy scan).
 * Outputs as in batched_nms.
 * scratch: functs_b200_yolo_scratch_bytes(batch, s0, s1, s2, capacity, topk). */
int64_t functs_b200_yolo_scratch_bytes(int32_t batch, int32_t s0, int32_t s1, int32_t s2, int64_t capacity,
                                       int32_t topk);
int functs_b200_yolo_postprocess(const float* map0, const float* map1, const float* map2, int32_t batch, int32_t s0,
                                 int32_t s1, int32_t s2, float score_thr, int32_t topk, float iou_thr,
                                 int64_t capacity, float* boxes, float* dets, int64_t* labels, int64_t* flat_ids,
                                 int32_t* out_counts, int32_t* status, void* scratch, void* stream);

/* The same with the dense per-box outputs of the decode group kept: obj_out [batch, N] and cls_out [batch, N, 80]
 * (sigmoid of the objectness / class logits), as a program that returns them needs (the slices flat[..., 4] and
 * flat[..., 5:] of yolov3_bbox.py:217-219).  Every score is formed in that case, so the decode launch is the
 * thread-per-box kernel and nothing is pruned; still 3 launches.  NULL for both = functs_b200_yolo_postprocess.
 * records (optional, [batch, topk, 8] int32, 16-byte aligned): the NMS kernel also writes every output row as the
 * 32-byte record of functs_b200_pack_detections, so that a sharded caller can gather right away (no pack launch). */
int functs_b200_yolo_postprocess_dense(const float* map0, const float* map1, const float* map2, int32_t batch,
                                       int32_t s0, int32_t s1, int32_t s2, float score_thr, int32_t topk,
                                       float iou_thr, int64_t capacity, float* boxes, float* obj_out, float* cls_out,
                                       float* dets, int64_t* labels, int64_t* flat_ids, int32_t* out_counts,
                                       int32_t* records, int32_t* status, void* scratch, void* stream);

/* ---- C3: SSD-style post-process ----------------------------------------------------------- */
/* Follows functs/benchmark/ai_model/ssd/ssd_bbox.py:121-154 (decode with the strided clamp), :268 (softmax, last
 * column = background dropped) and :163-172 + :212 inside a loop over classes that is mapped onto CTAs. */

/* Group 1 (one launch): softmax over conf rows, box decode (variances 0.1 / 0.2, clamp to [0, clamp_max]).
 * loc [batch, P, 4]; conf [batch, P, C+1]; priors [P, 4] (cx, cy, w, h); boxes [batch, P, 4];
 * scores_cm [batch, C, P] (class-major). */
int functs_b200_ssd_softmax_decode(const float* loc, const float* conf, const float* priors, int32_t batch,
                                   int32_t num_priors, int32_t num_classes, float clamp_max, float* boxes,
                                   float* scores_cm, void* stream);
/* Group 2 (one launch, one CTA per (image, class) loop iteration): mask > thr, top-k, NMS.
 * dets [batch, C, topk, 5]; prior_ids [batch, C, topk] int64; out_counts [batch, C] int32.  topk <= 256. */
int functs_b200_ssd_class_nms(const float* boxes, const float* scores_cm, int32_t batch, int32_t num_priors,
                              int32_t num_classes, float score_thr, int32_t topk, float iou_thr, float* dets,
                              int64_t* prior_ids, int32_t* out_counts, void* stream);

/* ---- C4: imperative LSTM with slice-assigned outputs ---------------------------------------- */
/* Follows functs/benchmark/ai_model/lstm/lstm.py:79-98, 118-133 (one layer; hs[t] = h, cs[t] = c kept).
 * x [T, B, I]; w_ih [4, I, H]; w_hh [4, H, H]; b_ih, b_hh [4, H]; hs, cs [T, B, H]; gate order i, f, g, o;
 * h0 = c0 = 0.  scratch: functs_b200_lstm_scratch_bytes(T, B, I, H).
 * Three launches: operand split + pre-tiling, the hoisted input projection (tcgen05, 3xTF32), and one persistent
 * recurrent kernel. */
int64_t functs_b200_lstm_scratch_bytes(int32_t seq_len, int32_t batch, int32_t input, int32_t hidden);
int functs_b200_lstm_forward(const float* x, const float* w_ih, const float* w_hh, const float* b_ih,
                             const float* b_hh, int32_t seq_len, int32_t batch, int32_t input, int32_t hidden,
                             float* hs, float* cs, int32_t* status, void* scratch, void* stream);
/* Same, with the GEMM paths chosen by the caller: mode 0 = default; 1 = fp32 CUDA cores for the input projection and
 * the recurrence (the on-device check of the tensor-core results); 2 = tcgen05 (3xTF32) for both — the recurrence then
 * is one persistent kernel whose CTAs keep their slice of w_hh resident in shared memory and exchange h[t] as pre-tiled
 * TF32 hi / lo operands (needs batch == 64); 3 = tensor-core projection + CUDA-core recurrence.  A shape a tensor-core
 * path does not take falls back to the CUDA-core form of that GEMM. */
int functs_b200_lstm_forward_mode(const float* x, const float* w_ih, const float* w_hh, const float* b_ih,
                                  const float* b_hh, int32_t seq_len, int32_t batch, int32_t input, int32_t hidden,
                                  float* hs, float* cs, int32_t* status, void* scratch, void* stream, int32_t mode);

/* Debugging switches (name -> value); returns FB_ERR_NOT_FOUND for an unknown name.
 *   "yolo_prune": 0 makes functs_b200_yolo_postprocess keep every candidate above the score threshold instead of
 *                 dropping, inside the decode kernel, those that can no longer reach the top-k (default 1; the
 *                 outputs are the same either way). */
int functs_b200_debug_set(const char* name, int32_t value);

/* ---- C5: YOLACT-style mask assembly ------------------------------------------------------------ */
/* Follows functs/benchmark/ai_model/yolact/yolact_mask.py:250-264 and :306-333: per detection
 * sigmoid(proto @ coef) cropped to the sanitised box by slice assignment, thresholded.
 * proto [batch, H, W, K] (K = 32); coef [batch, N, K]; boxes [batch, N, 4] (x1, y1, x2, y2 in pixels);
 * masks [batch, N, H, W] uint8; logits_out optional [batch, N, H, W] fp32 (dense proto @ coef, for value checks).
 * W must be even.  One launch. */
int functs_b200_yolact_masks(const float* proto, const float* coef, const float* boxes, int32_t batch, int32_t height,
                             int32_t width, int32_t num_det, float thr, uint8_t* masks, float* logits_out,
                             void* stream);

/* ---- Access / Assign family as stand-alone launches ------------------------------------------- */
/* A strided gather description: out[ax] = src[offset + sum_d ((ax_d % mod_d) * stride_d)], rank <= 8.
 * It expresses immut::select / slice / squeeze / unsqueeze / view / reshape / permute / expand / expand_as /
 * repeat (index math of functs/csrc/jit/tensorexpr/nnc_ext.cpp:62-401).  elem_size in {1,2,4,8}. */
typedef struct {
    int32_t rank;
    int64_t out_shape[8];
    int64_t src_stride[8]; /* in elements */
    int64_t src_mod[8];    /* 0 = no modulo */
    int64_t src_offset;    /* in elements */
} functs_b200_access_desc;

int functs_b200_access(const void* src, void* out, const functs_b200_access_desc* desc, int32_t elem_size,
                       void* stream);

/* The reverse ("assign") forms: out = self everywhere except the region selected along ``dim``, which comes
 * from src (nnc_ext.cpp:112-164, 187-212).  self/out: contiguous, shape self_shape[rank]; src: contiguous.
 *   select_rev: region = { ax[dim] == index };  slice_rev: region = { start <= ax[dim] < end, (ax[dim]-start) % step == 0 }.
 * start/end/index are already normalised by the caller. */
int functs_b200_select_rev(const void* self, const void* src, void* out, const int64_t* self_shape, int32_t rank,
                           int32_t dim, int64_t index, int32_t elem_size, void* stream);
int functs_b200_slice_rev(const void* self, const void* src, void* out, const int64_t* self_shape, int32_t rank,
                          int32_t dim, int64_t start, int64_t end, int64_t step, int32_t elem_size, void* stream);
/* immut::index (first index tensor, dim 0, int64 indices): out[i, r] = self[idx[i], r]; index_rev is the row
 * scatter out = self; out[idx[i], r] = src[i, r] (which of several duplicate indices wins is unspecified,
 * as for index_put_). */
int functs_b200_index_rows(const void* self, const int64_t* idx, void* out, int64_t self_rows, int64_t num_idx,
                           int64_t row_elems, int32_t elem_size, int32_t* status, void* stream);
int functs_b200_index_rows_rev(const void* self, const void* src, const int64_t* idx, void* out, int64_t self_rows,
                               int64_t num_idx, int64_t row_elems, int32_t elem_size, int32_t* status, void* stream);

/* ---- generic group: one launch for a fusion group no precompiled kernel covers ------------------------ */
/* The reference generates one CUDA kernel per fusion group at run time (NVRTC, fait/fuser/graph_builder.cpp:259-712:
 * every output element is one inlined gather expression; map iterations sit on blockIdx.y,
 * fait/tensorexpr/functor_parallization.cpp:83-111).  Here the same expression is data: the host flattens the group into
 * a small postfix program over the output's multi-index, and ONE precompiled kernel evaluates it per element.
 *   - a LOAD reads input `tensor` at  base + sum_k coef[k] * x[k]  (x = the output element's multi-index): every Access
 *     op (select / slice / squeeze / unsqueeze / permute / expand) on the way to the output has been folded into those
 *     coefficients on the host.  Only a read below a strided assignment needs a division of a coordinate; such a load
 *     has general != 0 and is described by terms: base + sum_k stride_k * ((mul_k * x[dim_k] + add_k) / div_k);
 *   - a COND tests  lo <= v < hi  and  (v - lo) % step == 0  with  v = add + sum_k coef[k] * x[k]  (one non-zero
 *     coefficient) and either falls through or jumps: the Assign ops (select_rev / slice_rev) and cat / stack become
 *     COND ... JUMP ... chains, so only the selected operand is evaluated;
 *   - CONST / UNARY / BINARY work on a small value stack (fp32; comparisons give 1.0 / 0.0); a binary operator with a
 *     scalar operand is one *_IMM instruction (RSUB / RDIV: the scalar is the left operand).
 * One program per (map iteration, group output); grid.y walks the programs.  Everything is 32-bit: tensors of 2^31
 * elements or more are not taken.  div_magic / div_shift: the output shape's dimensions as multiply-shift divisors
 * (q = mulhi(magic, n); ((n - q) >> 1) + q >> shift; unused for extent 1), filled in by the host.
 * The dimensions need not be in the output's own order: thread e works on the element whose multi-index is the
 * decomposition of e over `shape` (last dimension fastest) and stores it at sum_k out_coef[k] * x[k].  The host orders
 * them so that the lanes of a warp run along a dimension no COND tests (one path per warp instead of one per lane), and
 * lets a thread take vec neighbouring elements of that dimension through the program in one pass. */
enum {
    FB_G_END = 0, FB_G_LOAD = 1, FB_G_CONST = 2, FB_G_COND = 3, FB_G_JUMP = 4,
    /* unary */ FB_G_EXP = 10, FB_G_SIGMOID = 11, FB_G_TANH = 12, FB_G_RELU = 13, FB_G_NEG = 14, FB_G_CLAMP_MIN = 15,
    FB_G_CLAMP_MAX = 16, FB_G_ABS = 17, FB_G_SQRT = 18, FB_G_LOG = 19,
    /* binary */ FB_G_ADD = 30, FB_G_SUB = 31, FB_G_MUL = 32, FB_G_DIV = 33, FB_G_MIN = 34, FB_G_MAX = 35, FB_G_GT = 36,
    FB_G_GE = 37, FB_G_LT = 38, FB_G_LE = 39, FB_G_EQ = 40, FB_G_NE = 41,
    /* binary with the scalar imm as right operand: FB_G_IMM + the binary code; the two with it as left operand */
    FB_G_IMM = 30, /* FB_G_ADD + FB_G_IMM = 60 ... FB_G_NE + FB_G_IMM = 71 */
    FB_G_RSUB_IMM = 80, FB_G_RDIV_IMM = 81
};
#define FB_G_MAX_INSTR 256
#define FB_G_MAX_LOADS 24
#define FB_G_MAX_PREDS 24
#define FB_G_MAX_TERMS 6
#define FB_G_MAX_INPUTS 16
#define FB_G_STACK 12
typedef struct {
    uint16_t op;   /* FB_G_* */
    uint16_t arg;  /* LOAD: load slot; COND: predicate slot (the jump target is in imm_i); JUMP: target */
    union { float f; int32_t i; } imm; /* CONST / CLAMP_* / *_IMM: the scalar; COND: jump target when the test fails */
} functs_b200_ginstr;
typedef struct {
    int16_t dim;  /* output dimension the coordinate follows, -1 = constant */
    int16_t div;  /* >= 1 */
    int32_t mul, add, stride;
} functs_b200_gterm;
typedef struct {
    int32_t tensor;  /* index into in_ptr */
    int32_t base;
    int32_t dtype;   /* 0 = float32, 1 = uint8 / bool, 2 = int64, 3 = int32 */
    int32_t general; /* 0: coef[]; else: nterms terms */
    int32_t coef[8];
    int32_t nterms;
    int32_t reserved;
    functs_b200_gterm term[FB_G_MAX_TERMS];
} functs_b200_gload;
typedef struct {
    int32_t coef[8];
    int32_t add, lo, hi, step;
} functs_b200_gpred;
typedef struct {
    int32_t rank;
    int32_t shape[8];
    int32_t numel;
    int32_t out_dtype;  /* 0 = float32, 1 = bool (uint8) */
    int32_t ninstr;
    uint32_t div_magic[8];
    uint32_t div_shift[8];
    int32_t out_coef[8];  /* the element's place in the output: sum_k out_coef[k] * x[k] */
    int32_t vec;          /* elements per thread: 1, or 4 along the fastest dimension (which no COND may test), 32 apart */
    int32_t lane_extent;  /* vec > 1: elements along the fastest dimension (shape holds the work items per row:
                             32 for every started block of 32 * vec elements) */
    int32_t work;         /* product of shape: thread work items */
    int32_t pad0;
    const void* in_ptr[FB_G_MAX_INPUTS];
    void* out_ptr;
    int32_t reserved[2];  /* keeps sizeof a multiple of 16 */
    functs_b200_ginstr instr[FB_G_MAX_INSTR];
    functs_b200_gload load[FB_G_MAX_LOADS];
    functs_b200_gpred pred[FB_G_MAX_PREDS];
} functs_b200_gprogram;
/* programs: `count` programs in HOST memory when on_device == 0 (count == 1: passed to the kernel by value) or in DEVICE
 * memory when on_device != 0; max_work / max_rank = the largest work / rank among them (a program of a higher rank
 * than max_rank is not run).  One launch. */
int functs_b200_generic_group_launch(const functs_b200_gprogram* programs, int32_t count, int32_t max_work,
                                     int32_t max_rank, int32_t on_device, void* stream);

/* ---- group registry: what the tssa::ParallelFunctor operator binds to ------------------------ */
/* The reference registers one JIT operator whose Operation runs a compiled group
 * (fait/passes/te_op.cpp:238-249).  Here a group is found by a canonical signature string and launched with
 * flat argument arrays; the typed entry points above are what the registry dispatches to.
 * Returns a group id >= 0 or FB_ERR_NOT_FOUND. */
int functs_b200_group_lookup(const char* signature);
int functs_b200_group_count(void);
const char* functs_b200_group_signature(int group_id);
int functs_b200_group_launch(int group_id, const void* const* in_ptrs, const int64_t* int_args,
                             const double* float_args, void* const* out_ptrs, void* scratch, int32_t* status,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FUNCTS_B200_H_ */
