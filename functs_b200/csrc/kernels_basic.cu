// C1 (the get_started scatter-map group) and the Access / Assign family as stand-alone launches.
//
// Index semantics follow the reference's lowerings (functs/csrc/jit/tensorexpr/nnc_ext.cpp:62-401):
// an access op is a pure index remap of a contiguous source, a *_rev op returns `self` with the accessed
// region replaced by `src`.
#include <type_traits>

#include "common.cuh"

namespace fb {

// ---- C1 -----------------------------------------------------------------------------------------
// Loop { t = select(b, 0, i); u = t + addend; b = select_rev(b, u, 0, i) } for i in [0, n) on a cloned b.
// Iteration i only reads and writes row i, so the iterations are independent: blockIdx.y = row (loop
// iteration for y < n, pass-through copy of the clone otherwise), blockIdx.x = 128-bit column tile.
constexpr int kRowsThreads = 256;

__global__ void __launch_bounds__(kRowsThreads)
rows_add_kernel_v4(const float4* __restrict__ b, float4* __restrict__ out, int64_t cols4, int64_t n, float addend) {
    const int64_t row = blockIdx.y;
    const int64_t c = static_cast<int64_t>(blockIdx.x) * kRowsThreads + threadIdx.x;
    if (c >= cols4) return;
    float4 v = __ldg(b + row * cols4 + c);
    if (row < n) {
        v.x = __fadd_rn(v.x, addend);
        v.y = __fadd_rn(v.y, addend);
        v.z = __fadd_rn(v.z, addend);
        v.w = __fadd_rn(v.w, addend);
    }
    out[row * cols4 + c] = v;
}

__global__ void __launch_bounds__(kRowsThreads)
rows_add_kernel_s(const float* __restrict__ b, float* __restrict__ out, int64_t cols, int64_t n, float addend) {
    const int64_t row = blockIdx.y;
    const int64_t c = static_cast<int64_t>(blockIdx.x) * kRowsThreads + threadIdx.x;
    if (c >= cols) return;
    float v = __ldg(b + row * cols + c);
    if (row < n) v = __fadd_rn(v, addend);
    out[row * cols + c] = v;
}

// ---- access: out[ax] = src[offset + sum_d (ax_d % mod_d) * stride_d] ------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
access_kernel(const T* __restrict__ src, T* __restrict__ out, const functs_b200_access_desc d, int64_t numel) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < numel; e += stride) {
        int64_t rem = e;
        int64_t off = d.src_offset;
#pragma unroll
        for (int k = 7; k >= 0; --k) {
            if (k < d.rank) {
                const int64_t sz = d.out_shape[k];
                int64_t ax = rem % sz;
                rem /= sz;
                if (d.src_mod[k] > 0) ax %= d.src_mod[k];
                off += ax * d.src_stride[k];
            }
        }
        out[e] = src[off];
    }
}

// The same gather with 32-bit index arithmetic (every extent, stride and offset below 2^31): a 64-bit division costs
// about ten times a 32-bit one, and a gather of rank r does r of them (plus the modulo) per element.  Dimensions are
// merged and the innermost run is widened to 16-byte elements on the host (simplify_access), so that a contiguous
// region moves as 128-bit loads and stores and the divisions are paid once per 16 bytes.
struct AccessDesc32 {
    int rank;
    unsigned shape[8];
    int stride[8];
    unsigned mod[8];  // 0 = none
    int offset;
};

template <typename T>
__global__ void __launch_bounds__(256)
access_kernel32(const T* __restrict__ src, T* __restrict__ out, const AccessDesc32 d, unsigned numel) {
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < numel; e += stride) {
        unsigned rem = e;
        int off = d.offset;
#pragma unroll
        for (int k = 7; k >= 0; --k) {
            if (k < d.rank) {
                const unsigned sz = d.shape[k];
                unsigned ax = rem % sz;
                rem /= sz;
                if (d.mod[k] > 0u) ax %= d.mod[k];
                off += static_cast<int>(ax) * d.stride[k];
            }
        }
        out[e] = src[off];
    }
}

// 16-byte elements of the region form of the Assign family: out = self except where dd = (e / inner) % D lies in the
// region (inner counted in 16-byte units).
__global__ void __launch_bounds__(256)
assign_region_kernel_v16(const uint4* __restrict__ self, const uint4* __restrict__ src, uint4* __restrict__ out,
                         unsigned numel, unsigned D, unsigned inner, unsigned start, unsigned end, unsigned step, unsigned L) {
    const unsigned gstride = gridDim.x * blockDim.x;
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < numel; e += gstride) {
        const unsigned od = e / inner, in = e - od * inner;
        const unsigned o = od / D, dd = od - o * D;
        const bool set = dd >= start && dd < end && ((dd - start) % step) == 0u;
        out[e] = set ? __ldg(src + (o * L + (dd - start) / step) * inner + in) : __ldg(self + e);
    }
}

// ---- select_rev / slice_rev over the (outer, D, inner) view of self ---------------------------------------
// region: start <= d < end and (d - start) % step == 0; src is contiguous [outer, L, inner] with
// L = ceil((end - start) / step) (select_rev: start = index, end = index + 1, step = 1, L = 1).
template <typename T>
__global__ void __launch_bounds__(256)
assign_region_kernel(const T* __restrict__ self, const T* __restrict__ src, T* __restrict__ out, int64_t numel,
                     int64_t D, int64_t inner, int64_t start, int64_t end, int64_t step, int64_t L) {
    const int64_t gstride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < numel; e += gstride) {
        const int64_t in = e % inner;
        const int64_t od = e / inner;
        const int64_t dd = od % D;
        const int64_t o = od / D;
        const bool set = dd >= start && dd < end && ((dd - start) % step) == 0;
        out[e] = set ? src[(o * L + (dd - start) / step) * inner + in] : self[e];
    }
}

// ---- row gather / scatter -------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
index_rows_kernel(const T* __restrict__ self, const int64_t* __restrict__ idx, T* __restrict__ out, int64_t self_rows,
                  int64_t num_idx, int64_t row_elems, int32_t* status) {
    const int64_t total = num_idx * row_elems;
    const int64_t gstride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += gstride) {
        const int64_t i = e / row_elems, r = e - i * row_elems;
        int64_t row = idx[i];
        if (row < 0) row += self_rows;
        if (row < 0 || row >= self_rows) {
            if (status != nullptr) atomicOr(status, FB_STATUS_INDEX_RANGE);
            out[e] = T(0);
        } else {
            out[e] = self[row * row_elems + r];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const T* __restrict__ src, const int64_t* __restrict__ idx, T* __restrict__ out, int64_t self_rows,
                    int64_t num_idx, int64_t row_elems, int32_t* status) {
    const int64_t total = num_idx * row_elems;
    const int64_t gstride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += gstride) {
        const int64_t i = e / row_elems, r = e - i * row_elems;
        int64_t row = idx[i];
        if (row < 0) row += self_rows;
        if (row < 0 || row >= self_rows) {
            if (status != nullptr) atomicOr(status, FB_STATUS_INDEX_RANGE);
        } else {
            out[row * row_elems + r] = src[e];
        }
    }
}

static inline unsigned grid_for(int64_t numel, int threads) {
    int64_t need = (numel + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;  // grid-stride loops take the rest
    if (need > cap) need = cap;
    if (need < 1) need = 1;
    return static_cast<unsigned>(need);
}

// Merges adjacent dimensions that the source walks contiguously (stride[k] == stride[k + 1] * shape[k + 1], no modulo) and
// drops extents of 1.  Returns the simplified description (same element order of the output).
static functs_b200_access_desc merge_dims(const functs_b200_access_desc& in) {
    functs_b200_access_desc d{};
    d.src_offset = in.src_offset;
    int r = 0;
    for (int k = 0; k < in.rank; ++k) {
        if (in.out_shape[k] == 1) continue;
        if (r > 0 && in.src_mod[k] == 0 && d.src_mod[r - 1] == 0 && d.src_stride[r - 1] == in.src_stride[k] * in.out_shape[k]) {
            d.out_shape[r - 1] *= in.out_shape[k];
            d.src_stride[r - 1] = in.src_stride[k];
        } else {
            d.out_shape[r] = in.out_shape[k];
            d.src_stride[r] = in.src_stride[k];
            d.src_mod[r] = in.src_mod[k];
            ++r;
        }
    }
    d.rank = r;
    return d;
}

// If the innermost output dimension reads a contiguous, 16-byte aligned run, re-expresses the gather in 16-byte
// elements.  Returns the new element size (16) or the old one.
static int widen_to_16(functs_b200_access_desc& d, int elem_size, const void* src, const void* out) {
    if (d.rank == 0 || elem_size >= 16) return elem_size;
    const int v = 16 / elem_size;
    const int last = d.rank - 1;
    if (d.src_stride[last] != 1 || d.src_mod[last] != 0 || d.out_shape[last] % v != 0 || d.src_offset % v != 0) return elem_size;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) return elem_size;
    for (int k = 0; k < last; ++k) {
        if (d.src_stride[k] % v != 0) return elem_size;
    }
    d.out_shape[last] /= v;
    d.src_offset /= v;
    for (int k = 0; k < last; ++k) d.src_stride[k] /= v;
    return 16;
}

static bool fits_32(const functs_b200_access_desc& d, int64_t numel) {
    if (numel >= (1ll << 31)) return false;
    int64_t reach = d.src_offset < 0 ? -d.src_offset : d.src_offset;
    for (int k = 0; k < d.rank; ++k) {
        const int64_t st = d.src_stride[k] < 0 ? -d.src_stride[k] : d.src_stride[k];
        if (d.out_shape[k] >= (1ll << 31) || st >= (1ll << 31) || d.src_mod[k] >= (1ll << 31)) return false;
        reach += st * (d.out_shape[k] - 1);
    }
    return reach < (1ll << 31);
}

template <typename F>
static int dispatch_elem(int elem_size, F&& f) {
    switch (elem_size) {
        case 1: return f(static_cast<uint8_t*>(nullptr));
        case 2: return f(static_cast<uint16_t*>(nullptr));
        case 4: return f(static_cast<uint32_t*>(nullptr));
        case 8: return f(static_cast<uint64_t*>(nullptr));
        default: set_error("element size %d is not one of 1, 2, 4, 8", elem_size); return FB_ERR_INVALID_ARGUMENT;
    }
}

}  // namespace fb

namespace fb {

// Detection records for the multi-GPU gather: one 32-byte record per output row, bit-preserving:
// words 0..4 = (x1, y1, x2, y2, score) as fp32 bits, 5 = label, 6 = flat id, 7 = 1 for a valid row / 0 for padding.
__global__ void __launch_bounds__(256)
pack_detections_kernel(const float* __restrict__ dets, const int64_t* __restrict__ labels,
                       const int64_t* __restrict__ flat_ids, const int32_t* __restrict__ counts, int topk, int64_t total,
                       int4* __restrict__ rec) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const int g = static_cast<int>(i / topk);
    const int k = static_cast<int>(i - static_cast<int64_t>(g) * topk);
    const float* d = dets + i * 5;
    int4 lo, hi;
    lo.x = __float_as_int(d[0]);
    lo.y = __float_as_int(d[1]);
    lo.z = __float_as_int(d[2]);
    lo.w = __float_as_int(d[3]);
    hi.x = __float_as_int(d[4]);
    hi.y = static_cast<int>(labels[i]);
    hi.z = static_cast<int>(flat_ids[i]);
    hi.w = k < counts[g] ? 1 : 0;
    rec[2 * i] = lo;
    rec[2 * i + 1] = hi;
}

}  // namespace fb

extern "C" {

int functs_b200_rows_select_add_select_rev(const float* b, float* out, int64_t rows, int64_t cols, int64_t n,
                                           float addend, void* stream) {
    using namespace fb;
    FB_REQUIRE(b && out, "rows_select_add_select_rev: null pointer");
    FB_REQUIRE(rows > 0 && rows <= 65535 && cols > 0, "rows_select_add_select_rev: rows must be in [1, 65535], cols > 0");
    FB_REQUIRE(n >= 0 && n <= rows, "rows_select_add_select_rev: n = %lld outside [0, rows = %lld] (select index out of range)",
               static_cast<long long>(n), static_cast<long long>(rows));
    cudaStream_t st = as_stream(stream);
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (vec) {
        const int64_t cols4 = cols / 4;
        dim3 grid(static_cast<unsigned>((cols4 + kRowsThreads - 1) / kRowsThreads), static_cast<unsigned>(rows));
        rows_add_kernel_v4<<<grid, kRowsThreads, 0, st>>>(reinterpret_cast<const float4*>(b), reinterpret_cast<float4*>(out),
                                                          cols4, n, addend);
    } else {
        dim3 grid(static_cast<unsigned>((cols + kRowsThreads - 1) / kRowsThreads), static_cast<unsigned>(rows));
        rows_add_kernel_s<<<grid, kRowsThreads, 0, st>>>(b, out, cols, n, addend);
    }
    count_launch();
    return check_launch("rows_add_kernel");
}

int functs_b200_access(const void* src, void* out, const functs_b200_access_desc* desc, int32_t elem_size,
                       void* stream) {
    using namespace fb;
    FB_REQUIRE(src && out && desc, "access: null pointer");
    FB_REQUIRE(desc->rank >= 0 && desc->rank <= 8, "access: rank %d outside [0, 8]", desc->rank);
    int64_t numel = 1;
    for (int k = 0; k < desc->rank; ++k) {
        FB_REQUIRE(desc->out_shape[k] >= 0, "access: negative extent");
        numel *= desc->out_shape[k];
    }
    if (numel == 0) return FB_OK;
    FB_REQUIRE(elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8, "element size %d is not one of 1, 2, 4, 8",
               elem_size);
    cudaStream_t st = as_stream(stream);
    functs_b200_access_desc d = merge_dims(*desc);
    const int width = widen_to_16(d, elem_size, src, out);
    const int64_t n = numel / (width / elem_size);
    if (fits_32(d, n)) {
        AccessDesc32 q{};
        q.rank = d.rank;
        q.offset = static_cast<int>(d.src_offset);
        for (int k = 0; k < d.rank; ++k) {
            q.shape[k] = static_cast<unsigned>(d.out_shape[k]);
            q.stride[k] = static_cast<int>(d.src_stride[k]);
            q.mod[k] = static_cast<unsigned>(d.src_mod[k]);
        }
        const unsigned grid = grid_for(n, 256);
        if (width == 16) {
            access_kernel32<uint4><<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(out), q,
                                                         static_cast<unsigned>(n));
        } else {
            int rc = dispatch_elem(elem_size, [&](auto* tag) {
                using T = typename std::remove_pointer<decltype(tag)>::type;
                access_kernel32<T><<<grid, 256, 0, st>>>(static_cast<const T*>(src), static_cast<T*>(out), q, static_cast<unsigned>(n));
                return FB_OK;
            });
            FB_TRY(rc);
        }
        count_launch();
        return check_launch("access_kernel32");
    }
    const functs_b200_access_desc d64 = *desc;
    int rc = dispatch_elem(elem_size, [&](auto* tag) {
        using T = typename std::remove_pointer<decltype(tag)>::type;
        access_kernel<T><<<grid_for(numel, 256), 256, 0, st>>>(static_cast<const T*>(src), static_cast<T*>(out), d64, numel);
        return FB_OK;
    });
    FB_TRY(rc);
    count_launch();
    return check_launch("access_kernel");
}

static int assign_region(const void* self, const void* src, void* out, const int64_t* self_shape, int32_t rank,
                         int32_t dim, int64_t start, int64_t end, int64_t step, int32_t elem_size, void* stream,
                         const char* what) {
    using namespace fb;
    FB_REQUIRE(self && out && self_shape, "%s: null pointer", what);
    FB_REQUIRE(rank >= 1 && rank <= 8 && dim >= 0 && dim < rank, "%s: dim %d outside rank %d", what, dim, rank);
    FB_REQUIRE(step >= 1, "%s: step must be >= 1", what);
    int64_t outer = 1, inner = 1;
    for (int k = 0; k < dim; ++k) outer *= self_shape[k];
    for (int k = dim + 1; k < rank; ++k) inner *= self_shape[k];
    const int64_t D = self_shape[dim];
    FB_REQUIRE(start >= 0 && start <= D && end <= D, "%s: region [%lld, %lld) outside extent %lld", what,
               static_cast<long long>(start), static_cast<long long>(end), static_cast<long long>(D));
    if (end < start) end = start;
    const int64_t L = (end - start + step - 1) / step;
    const int64_t numel = outer * D * inner;
    if (numel == 0) return FB_OK;
    FB_REQUIRE(src != nullptr || L == 0, "%s: null src", what);
    cudaStream_t st = as_stream(stream);
    // 16-byte elements when the inner run allows it (and everything indexes in 32 bits)
    if (elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8) {
        const int v = 16 / elem_size;
        const bool aligned = ((reinterpret_cast<uintptr_t>(self) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(src)) & 15) == 0;
        if (aligned && inner % v == 0 && numel / v < (1ll << 31) && D < (1ll << 31) && step < (1ll << 31)) {
            const unsigned n16 = static_cast<unsigned>(numel / v);
            assign_region_kernel_v16<<<grid_for(n16, 256), 256, 0, st>>>(
                static_cast<const uint4*>(self), static_cast<const uint4*>(src), static_cast<uint4*>(out), n16,
                static_cast<unsigned>(D), static_cast<unsigned>(inner / v), static_cast<unsigned>(start),
                static_cast<unsigned>(end), static_cast<unsigned>(step), static_cast<unsigned>(L));
            count_launch();
            return check_launch(what);
        }
    }
    int rc = dispatch_elem(elem_size, [&](auto* tag) {
        using T = typename std::remove_pointer<decltype(tag)>::type;
        assign_region_kernel<T><<<grid_for(numel, 256), 256, 0, st>>>(static_cast<const T*>(self), static_cast<const T*>(src),
                                                                       static_cast<T*>(out), numel, D, inner, start, end,
                                                                       step, L);
        return FB_OK;
    });
    FB_TRY(rc);
    count_launch();
    return check_launch(what);
}

int functs_b200_select_rev(const void* self, const void* src, void* out, const int64_t* self_shape, int32_t rank,
                           int32_t dim, int64_t index, int32_t elem_size, void* stream) {
    if (self_shape != nullptr && rank >= 1 && rank <= 8 && dim >= 0 && dim < rank) {
        if (index < 0 || index >= self_shape[dim]) {
            fb::set_error("select_rev: index %lld out of range for extent %lld", static_cast<long long>(index),
                          static_cast<long long>(self_shape[dim]));
            return FB_ERR_INVALID_ARGUMENT;
        }
    }
    return assign_region(self, src, out, self_shape, rank, dim, index, index + 1, 1, elem_size, stream, "select_rev");
}

int functs_b200_slice_rev(const void* self, const void* src, void* out, const int64_t* self_shape, int32_t rank,
                          int32_t dim, int64_t start, int64_t end, int64_t step, int32_t elem_size, void* stream) {
    return assign_region(self, src, out, self_shape, rank, dim, start, end, step, elem_size, stream, "slice_rev");
}

int functs_b200_index_rows(const void* self, const int64_t* idx, void* out, int64_t self_rows, int64_t num_idx,
                           int64_t row_elems, int32_t elem_size, int32_t* status, void* stream) {
    using namespace fb;
    FB_REQUIRE(self && idx && out, "index_rows: null pointer");
    FB_REQUIRE(self_rows > 0 && num_idx >= 0 && row_elems > 0, "index_rows: bad sizes");
    const int64_t total = num_idx * row_elems;
    if (total == 0) return FB_OK;
    cudaStream_t st = as_stream(stream);
    int rc = dispatch_elem(elem_size, [&](auto* tag) {
        using T = typename std::remove_pointer<decltype(tag)>::type;
        index_rows_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const T*>(self), idx, static_cast<T*>(out),
                                                                    self_rows, num_idx, row_elems, status);
        return FB_OK;
    });
    FB_TRY(rc);
    count_launch();
    return check_launch("index_rows_kernel");
}

int functs_b200_index_rows_rev(const void* self, const void* src, const int64_t* idx, void* out, int64_t self_rows,
                               int64_t num_idx, int64_t row_elems, int32_t elem_size, int32_t* status, void* stream) {
    using namespace fb;
    FB_REQUIRE(self && out, "index_rows_rev: null pointer");
    FB_REQUIRE(self_rows > 0 && num_idx >= 0 && row_elems > 0, "index_rows_rev: bad sizes");
    FB_REQUIRE(elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8, "index_rows_rev: bad element size");
    cudaStream_t st = as_stream(stream);
    if (self != out) {
        FB_TRY(check_cuda(cudaMemcpyAsync(out, self, static_cast<size_t>(self_rows * row_elems * elem_size),
                                          cudaMemcpyDeviceToDevice, st),
                          "index_rows_rev copy"));
    }
    const int64_t total = num_idx * row_elems;
    if (total == 0) return FB_OK;
    FB_REQUIRE(src && idx, "index_rows_rev: null pointer");
    int rc = dispatch_elem(elem_size, [&](auto* tag) {
        using T = typename std::remove_pointer<decltype(tag)>::type;
        scatter_rows_kernel<T><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const T*>(src), idx, static_cast<T*>(out),
                                                                      self_rows, num_idx, row_elems, status);
        return FB_OK;
    });
    FB_TRY(rc);
    count_launch();
    return check_launch("scatter_rows_kernel");
}

int functs_b200_pack_detections(const float* dets, const int64_t* labels, const int64_t* flat_ids, const int32_t* counts,
                                int32_t groups, int32_t topk, int32_t* records, void* stream) {
    using namespace fb;
    FB_REQUIRE(dets && labels && flat_ids && counts && records, "pack_detections: null pointer");
    FB_REQUIRE(groups > 0 && topk > 0, "pack_detections: bad sizes");
    FB_REQUIRE((reinterpret_cast<uintptr_t>(records) & 15) == 0, "pack_detections: records must be 16-byte aligned");
    const int64_t total = static_cast<int64_t>(groups) * topk;
    pack_detections_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        dets, labels, flat_ids, counts, topk, total, reinterpret_cast<int4*>(records));
    count_launch();
    return check_launch("pack_detections_kernel");
}

int functs_b200_push_records(void* dst, const int32_t* records, int64_t bytes, void* stream) {
    using namespace fb;
    FB_REQUIRE(dst != nullptr && records != nullptr && bytes > 0, "push_records: null pointer or empty copy");
    FB_REQUIRE(((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(records) | static_cast<uintptr_t>(bytes)) & 15) == 0,
               "push_records: pointers and size must be multiples of 16 bytes");
    return check_cuda(cudaMemcpyAsync(dst, records, static_cast<size_t>(bytes), cudaMemcpyDefault, as_stream(stream)),
                      "push_records copy");
}

}  // extern "C"
