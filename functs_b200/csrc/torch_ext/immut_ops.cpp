// Operator registrations of the immut:: Access / Assign family for TorchScript graphs.
//
// The schema strings are those of the reference (functs/csrc/jit/ir/symbol_ext.cpp:121-199), so graphs printed or
// parsed with them stay interchangeable.  Only CUDA kernels are registered: every op is one launch of the C-ABI
// library (libfuncts_b200.so) on the current stream and returns a fresh contiguous tensor (the pure meaning the
// functionalized graph gives these ops; the reference's eager kernels return views or write into `self` in place,
// symbol_ext.cpp:17-117).  A CPU tensor reaching one of these ops fails in the dispatcher: there is no CPU path.
#include <ATen/ATen.h>
#include <ATen/InferSize.h>
#include <ATen/WrapDimUtils.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <optional>
#include <vector>

#include "../../../include/functs_b200.h"

namespace functs_b200 {
namespace {

void* stream_of(const at::Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void check_rc(int rc) { TORCH_CHECK(rc == FB_OK, "functs_b200: ", functs_b200_last_error()); }

struct Desc {
    functs_b200_access_desc d{};
    std::vector<int64_t> shape;
    void finish() {
        d.rank = static_cast<int32_t>(shape.size());
        TORCH_CHECK(d.rank <= 8, "functs_b200: rank ", d.rank, " exceeds the supported maximum of 8");
        for (int i = 0; i < d.rank; ++i) d.out_shape[i] = shape[i];
    }
};

std::vector<int64_t> row_major_strides(at::IntArrayRef shape) {
    std::vector<int64_t> st(shape.size(), 1);
    for (int64_t i = static_cast<int64_t>(shape.size()) - 2; i >= 0; --i) st[i] = st[i + 1] * shape[i + 1];
    return st;
}

at::Tensor run_access(const at::Tensor& src_in, Desc& desc) {
    c10::cuda::CUDAGuard guard(src_in.device());  // launch on the tensor's device, whatever device is current
    at::Tensor src = src_in.contiguous();
    desc.finish();
    at::Tensor out = at::empty(desc.shape, src.options());
    if (out.numel() == 0) return out;
    check_rc(functs_b200_access(src.data_ptr(), out.data_ptr(), &desc.d, static_cast<int32_t>(src.element_size()),
                                stream_of(src)));
    return out;
}

// out axis k reads source axis `from[k]` (or -1: broadcast / new axis), with optional modulus
at::Tensor im_access(at::Tensor src) {
    Desc desc;
    desc.shape = src.sizes().vec();
    auto st = row_major_strides(src.sizes());
    for (size_t i = 0; i < st.size(); ++i) desc.d.src_stride[i] = st[i];
    return run_access(src, desc);
}

at::Tensor im_assign(at::Tensor self, at::Tensor src, std::optional<bool> n) {
    (void)self;
    (void)n;
    return im_access(src);
}

at::Tensor im_select(at::Tensor src, int64_t dim, int64_t index) {
    dim = at::maybe_wrap_dim(dim, src.dim());
    const int64_t size = src.size(dim);
    TORCH_CHECK_INDEX(index >= -size && index < size, "select(): index ", index, " out of range for tensor of size ",
                      src.sizes(), " at dimension ", dim);
    if (index < 0) index += size;
    auto st = row_major_strides(src.sizes());
    Desc desc;
    int k = 0;
    for (int64_t d = 0; d < src.dim(); ++d) {
        if (d == dim) continue;
        desc.shape.push_back(src.size(d));
        desc.d.src_stride[k++] = st[d];
    }
    desc.d.src_offset = index * st[dim];
    return run_access(src, desc);
}

struct SliceRange {
    int64_t start, end, len;
};

SliceRange normalize_slice(int64_t size, std::optional<c10::SymInt> start_, std::optional<c10::SymInt> end_, int64_t step) {
    TORCH_CHECK(step > 0, "slice step must be positive");
    int64_t start = start_.has_value() ? start_->expect_int() : 0;
    int64_t end = end_.has_value() ? end_->expect_int() : size;
    if (start < 0) start += size;
    if (end < 0) end += size;
    start = std::min(std::max<int64_t>(start, 0), size);
    end = std::min(std::max(end, start), size);
    return {start, end, (end - start + step - 1) / step};
}

at::Tensor im_slice(at::Tensor src, int64_t dim, std::optional<c10::SymInt> start, std::optional<c10::SymInt> end,
                 c10::SymInt step_) {
    dim = at::maybe_wrap_dim(dim, src.dim());
    const int64_t step = step_.expect_int();
    const SliceRange r = normalize_slice(src.size(dim), start, end, step);
    auto st = row_major_strides(src.sizes());
    Desc desc;
    desc.shape = src.sizes().vec();
    desc.shape[dim] = r.len;
    for (int64_t d = 0; d < src.dim(); ++d) desc.d.src_stride[d] = st[d];
    desc.d.src_stride[dim] = st[dim] * step;
    desc.d.src_offset = r.start * st[dim];
    return run_access(src, desc);
}

at::Tensor im_view(at::Tensor self, at::IntArrayRef size) {
    Desc desc;
    desc.shape = at::infer_size(size, self.numel());
    auto st = row_major_strides(desc.shape);
    for (size_t i = 0; i < st.size(); ++i) desc.d.src_stride[i] = st[i];
    return run_access(self, desc);
}

at::Tensor im_squeeze(at::Tensor self, int64_t dim) {
    if (self.dim() == 0) return im_access(self);
    dim = at::maybe_wrap_dim(dim, self.dim());
    auto shape = self.sizes().vec();
    if (shape[dim] == 1) shape.erase(shape.begin() + dim);
    return im_view(self, shape);
}

at::Tensor im_unsqueeze(at::Tensor self, int64_t dim) {
    dim = at::maybe_wrap_dim(dim, self.dim() + 1);
    auto shape = self.sizes().vec();
    shape.insert(shape.begin() + dim, 1);
    return im_view(self, shape);
}

at::Tensor im_permute(at::Tensor self, at::IntArrayRef dims) {
    TORCH_CHECK(static_cast<int64_t>(dims.size()) == self.dim(), "permute: number of dims does not match");
    auto st = row_major_strides(self.sizes());
    std::vector<bool> seen(self.dim(), false);
    Desc desc;
    for (size_t i = 0; i < dims.size(); ++i) {
        const int64_t d = at::maybe_wrap_dim(dims[i], self.dim());
        TORCH_CHECK(!seen[d], "permute: repeated dim");
        seen[d] = true;
        desc.shape.push_back(self.size(d));
        desc.d.src_stride[i] = st[d];
    }
    return run_access(self, desc);
}

// inverse permutation applied to self (self has the permuted shape)
at::Tensor im_permute_rev(at::Tensor self, at::IntArrayRef dims) {
    std::vector<int64_t> inv(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) inv[at::maybe_wrap_dim(dims[i], static_cast<int64_t>(dims.size()))] = static_cast<int64_t>(i);
    return im_permute(self, inv);
}

at::Tensor im_expand(at::Tensor self, at::IntArrayRef size, bool implicit) {
    (void)implicit;
    const int64_t orank = static_cast<int64_t>(size.size()), rank = self.dim();
    TORCH_CHECK(orank >= rank, "expand: the number of sizes must be >= the tensor rank");
    auto st = row_major_strides(self.sizes());
    const int64_t lead = orank - rank;
    Desc desc;
    for (int64_t d = 0; d < orank; ++d) {
        if (d < lead) {
            TORCH_CHECK(size[d] >= 0, "expand: -1 is not allowed in a leading, non-existing dimension");
            desc.shape.push_back(size[d]);
            desc.d.src_stride[d] = 0;
        } else {
            const int64_t in = self.size(d - lead);
            const int64_t want = size[d] == -1 ? in : size[d];
            TORCH_CHECK(want == in || in == 1, "expand: size ", want, " must match the existing size ", in);
            desc.shape.push_back(want);
            desc.d.src_stride[d] = (in == 1 && want != 1) ? 0 : st[d - lead];
        }
    }
    return run_access(self, desc);
}

at::Tensor im_expand_rev(at::Tensor self, at::IntArrayRef size, bool implicit) { return im_expand(self, size, implicit); }

at::Tensor im_expand_as(at::Tensor self, at::Tensor other) { return im_expand(self, other.sizes(), false); }

at::Tensor im_repeat(at::Tensor self, at::IntArrayRef reps) {
    const int64_t orank = static_cast<int64_t>(reps.size()), rank = self.dim();
    TORCH_CHECK(orank >= rank, "repeat: the number of repeats must be >= the tensor rank");
    auto st = row_major_strides(self.sizes());
    const int64_t lead = orank - rank;
    Desc desc;
    for (int64_t d = 0; d < orank; ++d) {
        TORCH_CHECK(reps[d] >= 0, "repeat: negative repeat");
        if (d < lead) {
            desc.shape.push_back(reps[d]);
        } else {
            const int64_t in = self.size(d - lead);
            desc.shape.push_back(in * reps[d]);
            desc.d.src_stride[d] = st[d - lead];
            desc.d.src_mod[d] = reps[d] != 1 ? in : 0;
        }
    }
    return run_access(self, desc);
}

at::Tensor im_select_rev(at::Tensor self, at::Tensor src, int64_t dim, int64_t index) {
    c10::cuda::CUDAGuard guard(self.device());
    TORCH_CHECK(src.device() == self.device(), "select_rev: self and src live on different devices");
    self = self.contiguous();
    dim = at::maybe_wrap_dim(dim, self.dim());
    const int64_t size = self.size(dim);
    TORCH_CHECK_INDEX(index >= -size && index < size, "select_rev(): index ", index, " out of range at dimension ", dim);
    if (index < 0) index += size;
    auto want = self.sizes().vec();
    want.erase(want.begin() + dim);
    src = src.to(self.scalar_type()).expand(want).contiguous();
    at::Tensor out = at::empty_like(self);
    auto shape = self.sizes().vec();
    check_rc(functs_b200_select_rev(self.data_ptr(), src.data_ptr(), out.data_ptr(), shape.data(), static_cast<int32_t>(self.dim()),
                                    static_cast<int32_t>(dim), index, static_cast<int32_t>(self.element_size()), stream_of(self)));
    return out;
}

at::Tensor im_slice_rev(at::Tensor self, at::Tensor src, int64_t dim, std::optional<c10::SymInt> start,
                     std::optional<c10::SymInt> end, c10::SymInt step_) {
    c10::cuda::CUDAGuard guard(self.device());
    TORCH_CHECK(src.device() == self.device(), "slice_rev: self and src live on different devices");
    self = self.contiguous();
    dim = at::maybe_wrap_dim(dim, self.dim());
    const int64_t step = step_.expect_int();
    const SliceRange r = normalize_slice(self.size(dim), start, end, step);
    auto want = self.sizes().vec();
    want[dim] = r.len;
    src = src.to(self.scalar_type()).expand(want).contiguous();
    at::Tensor out = at::empty_like(self);
    auto shape = self.sizes().vec();
    check_rc(functs_b200_slice_rev(self.data_ptr(), src.data_ptr(), out.data_ptr(), shape.data(), static_cast<int32_t>(self.dim()),
                                   static_cast<int32_t>(dim), r.start, r.end, step, static_cast<int32_t>(self.element_size()),
                                   stream_of(self)));
    return out;
}

// self.repeat(r) is a copy: assigning to it never reaches self (the reference's kernel returns self unchanged,
// functs/csrc/jit/ir/symbol_ext.cpp:94-101)
at::Tensor im_repeat_rev(at::Tensor self, at::Tensor src, at::IntArrayRef size) {
    (void)src;
    (void)size;
    return im_access(self);
}

at::Tensor im_expand_as_rev(at::Tensor self, at::Tensor src, at::Tensor other) {
    TORCH_CHECK(self.sizes() == other.sizes(),
                "expand_as_rev: destinations overlap (an extent of 1 was expanded); the assignment is ill-posed");
    return im_access(src.to(self.scalar_type()));
}

at::Tensor im_index_tensor(at::Tensor self, c10::List<std::optional<at::Tensor>> indices) {
    c10::cuda::CUDAGuard guard(self.device());
    TORCH_CHECK(indices.size() >= 1 && indices.get(0).has_value(), "immut::index supports one index tensor on dimension 0");
    for (size_t i = 1; i < indices.size(); ++i) TORCH_CHECK(!indices.get(i).has_value(), "immut::index: only dimension 0");
    at::Tensor idx = indices.get(0)->contiguous();
    TORCH_CHECK(idx.scalar_type() == at::kLong, "immut::index needs int64 indices (bool masks go through aten::index)");
    self = self.contiguous();
    auto shape = idx.sizes().vec();
    for (int64_t d = 1; d < self.dim(); ++d) shape.push_back(self.size(d));
    at::Tensor out = at::empty(shape, self.options());
    at::Tensor status = at::zeros({1}, self.options().dtype(at::kInt));
    const int64_t rows = self.size(0);
    const int64_t row_elems = rows > 0 ? self.numel() / rows : 0;
    if (out.numel() > 0) {
        check_rc(functs_b200_index_rows(self.data_ptr(), idx.data_ptr<int64_t>(), out.data_ptr(), rows, idx.numel(), row_elems,
                                        static_cast<int32_t>(self.element_size()), status.data_ptr<int32_t>(), stream_of(self)));
        TORCH_CHECK_INDEX(status.item<int32_t>() == 0, "index out of range in immut::index");
    }
    return out;
}

}  // namespace
}  // namespace functs_b200

TORCH_LIBRARY(immut, m) {
    m.def("immut::access(Tensor src) -> Tensor");
    m.def("immut::assign(Tensor self, Tensor src, bool? n=None) -> Tensor");
    m.def("immut::select(Tensor src, int dim, int index) -> Tensor");
    m.def("immut::select_rev(Tensor self, Tensor src, int dim, int index) -> Tensor");
    m.def("immut::slice(Tensor src, int dim=0, SymInt? start=None, SymInt? end=None, SymInt step=1) -> Tensor");
    m.def("immut::slice_rev(Tensor self, Tensor src, int dim=0, SymInt? start=None, SymInt? end=None, SymInt step=1) -> Tensor");
    m.def("immut::squeeze(Tensor self, int dim) -> Tensor");
    m.def("immut::unsqueeze(Tensor self, int dim) -> Tensor");
    m.def("immut::view(Tensor self, int[] size) -> Tensor");
    m.def("immut::reshape(Tensor self, int[] size) -> Tensor");
    m.def("immut::permute(Tensor self, int[] sizes) -> Tensor");
    m.def("immut::permute_rev(Tensor self, int[] size) -> Tensor");
    m.def("immut::expand(Tensor self, int[] size, *, bool implicit) -> Tensor");
    m.def("immut::expand_rev(Tensor self, int[] size, *, bool implicit) -> Tensor");
    m.def("immut::repeat(Tensor self, int[] size) -> Tensor");
    m.def("immut::repeat_rev(Tensor self, Tensor src, int[] size) -> Tensor");
    m.def("immut::expand_as(Tensor self, Tensor other) -> Tensor");
    m.def("immut::expand_as_rev(Tensor self, Tensor src, Tensor other) -> Tensor");
    m.def("immut::index.Tensor(Tensor self, Tensor?[] indices) -> Tensor");
}

TORCH_LIBRARY_IMPL(immut, CUDA, m) {
    using namespace functs_b200;
    m.impl("access", im_access);
    m.impl("assign", im_assign);
    m.impl("select", im_select);
    m.impl("select_rev", im_select_rev);
    m.impl("slice", im_slice);
    m.impl("slice_rev", im_slice_rev);
    m.impl("squeeze", im_squeeze);
    m.impl("unsqueeze", im_unsqueeze);
    m.impl("view", im_view);
    m.impl("reshape", im_view);
    m.impl("permute", im_permute);
    m.impl("permute_rev", im_permute_rev);
    m.impl("expand", im_expand);
    m.impl("expand_rev", im_expand_rev);
    m.impl("repeat", im_repeat);
    m.impl("repeat_rev", im_repeat_rev);
    m.impl("expand_as", im_expand_as);
    m.impl("expand_as_rev", im_expand_as_rev);
    m.impl("index.Tensor", im_index_tensor);
}
