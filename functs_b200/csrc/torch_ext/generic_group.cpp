// Generic fusion group: subgraph -> postfix program -> ONE launch of the precompiled interpreter kernel.
//
// The reference turns the subgraph of a tssa::ParallelFunctor into NNC tensors, inlines every intermediate and generates
// one kernel in which each output element is a single gather expression (fait/fuser/graph_builder.cpp:311-499; lowerings
// fait/fuser/custom_lowering_func.cpp:17-559, functs/csrc/jit/tensorexpr/nnc_ext.cpp:62-401).  The same inlining happens
// here on the host, at call time, when the shapes are known: the subgraph becomes an expression DAG, and emitting it pushes
// an index map from the output down to the leaves:
//   - Access ops (select / slice / squeeze / unsqueeze / permute / expand / expand_as) only rewrite the map: every
//     coordinate of an operand is (mul * x[dim] + add) / div of ONE output coordinate (or a constant);
//   - Assign ops (select_rev / slice_rev) and cat / stack become a predicate on one output coordinate plus two branches;
//   - a leaf becomes a LOAD whose address is linear in those coordinates; elementwise ops work on a value stack.
// Programs are rebuilt per call (a few microseconds of host work) and travel as a kernel parameter when there is one of
// them, otherwise through one small device buffer.  What the program format cannot express (reshape of an intermediate,
// reductions, integer arithmetic, tensors of 2^31 elements) is reported as unsupported and the caller falls back to the
// node-by-node interpreter.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/jit/ir/constants.h>
#include <torch/csrc/jit/ir/ir.h>

#include <cstring>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "../../../include/functs_b200.h"
#include "fusion.h"

namespace functs_b200 {

using namespace torch::jit;

namespace {

struct Unsupported : std::runtime_error {
    explicit Unsupported(const std::string& why) : std::runtime_error(why) {}
};
#define G_REQUIRE(cond, why)              \
    do {                                  \
        if (!(cond)) throw Unsupported(why); \
    } while (0)

struct Coord {
    int dim = -1;  // output dimension it follows, -1: constant
    int64_t mul = 0, add = 0, div = 1;
};
using Map = std::vector<Coord>;

struct Expr;
using ExprP = std::shared_ptr<Expr>;
struct Expr {
    enum Kind { Leaf, Const, Unary, Binary, Select, Slice, Squeeze, Unsqueeze, Permute, Expand, SelectRev, SliceRev, Cat, Stack };
    Kind kind = Const;
    std::vector<int64_t> shape;
    std::vector<ExprP> in;
    int op = 0;             // FB_G_* for Unary / Binary
    double f = 0.0;         // Const value, clamp bound
    std::vector<int64_t> iv;  // op parameters (dim, index, start, end, step, permutation ...)
    int tensor = -1;        // Leaf: input slot
    int dtype = 0;          // Leaf: load dtype code
    bool is_bool = false;   // value is a truth value (comparison result / bool tensor)
};

int64_t numelOf(const std::vector<int64_t>& s) {
    int64_t n = 1;
    for (int64_t v : s) n *= v;
    return n;
}

int64_t wrapDim(int64_t d, int64_t rank) {
    G_REQUIRE(d >= -rank && d < rank, "dimension out of range");
    return d < 0 ? d + rank : d;
}

std::vector<int64_t> broadcastShapes(const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
    const size_t r = std::max(a.size(), b.size());
    std::vector<int64_t> out(r, 1);
    for (size_t k = 0; k < r; ++k) {
        const int64_t x = k < r - a.size() ? 1 : a[k - (r - a.size())];
        const int64_t y = k < r - b.size() ? 1 : b[k - (r - b.size())];
        G_REQUIRE(x == y || x == 1 || y == 1, "shapes do not broadcast");
        out[k] = x == 1 ? y : x;
    }
    return out;
}

// ---- value environment while walking the subgraph -------------------------------------------------------------------
struct Val {
    enum Kind { None, Tensor, Int, Double, Bool, IntList, TensorList } kind = None;
    ExprP t;
    int64_t i = 0;
    double d = 0.0;
    std::vector<int64_t> il;
    std::vector<ExprP> tl;
};

struct Builder {
    std::vector<at::Tensor> inputs;  // contiguous device tensors, slot = index
    std::vector<std::pair<int, int>> sources;  // per slot: (argument of the node, position inside a list argument or -1)
    int cur_arg = -1, cur_pos = -1;            // where the values fromIValue() is looking at come from
    std::unordered_map<const Value*, Val> env;

    ExprP leaf(const at::Tensor& t_in) {
        G_REQUIRE(t_in.is_cuda(), "tensor input is not on a CUDA device");
        at::Tensor t = t_in.contiguous();
        int code = -1;
        switch (t.scalar_type()) {
            case at::kFloat: code = 0; break;
            case at::kBool: code = 1; break;
            default: break;
        }
        G_REQUIRE(code >= 0, "tensor dtype is neither float32 nor bool");
        G_REQUIRE(t.numel() < (1ll << 31), "tensor too large for 32-bit indexing");
        G_REQUIRE(inputs.size() < FB_G_MAX_INPUTS, "too many tensor inputs");
        auto e = std::make_shared<Expr>();
        e->kind = Expr::Leaf;
        e->shape = t.sizes().vec();
        e->tensor = static_cast<int>(inputs.size());
        e->dtype = code;
        e->is_bool = code == 1;
        inputs.push_back(t);
        sources.emplace_back(cur_arg, cur_pos);
        return e;
    }

    static ExprP constant(double v) {
        auto e = std::make_shared<Expr>();
        e->kind = Expr::Const;
        e->f = v;
        return e;
    }

    Val fromIValue(const c10::IValue& iv) {
        Val v;
        if (iv.isNone()) v.kind = Val::None;
        else if (iv.isTensor()) {
            v.kind = Val::Tensor;
            v.t = leaf(iv.toTensor());
        } else if (iv.isBool()) {
            v.kind = Val::Bool;
            v.i = iv.toBool();
        } else if (iv.isInt()) {
            v.kind = Val::Int;
            v.i = iv.toInt();
        } else if (iv.isDouble()) {
            v.kind = Val::Double;
            v.d = iv.toDouble();
        } else if (iv.isIntList()) {
            v.kind = Val::IntList;
            v.il = iv.toIntVector();
        } else if (iv.isTensorList()) {
            v.kind = Val::TensorList;
            int j = 0;
            for (const at::Tensor& t : iv.toTensorVector()) {
                cur_pos = j++;
                v.tl.push_back(leaf(t));
            }
        } else {
            throw Unsupported("input kind not supported");
        }
        return v;
    }

    const Val& get(const Value* v) {
        auto it = env.find(v);
        if (it != env.end()) return it->second;
        G_REQUIRE(v->node()->kind() == prim::Constant, "value defined outside the group");
        auto iv = toIValue(v);
        G_REQUIRE(iv.has_value(), "constant without a value");
        if (iv->isTensor()) {
            // a tensor constant of the subgraph: 0-d tensors act as scalars, others must already live on the device
            const at::Tensor& t = iv->toTensor();
            G_REQUIRE(t.dim() == 0 && t.scalar_type() == at::kFloat, "tensor constant inside the group");
            Val s;
            s.kind = Val::Double;
            s.d = t.item<double>();
            return env[v] = s;
        }
        return env[v] = fromIValue(*iv);
    }

    ExprP tensorOf(const Value* v) {
        const Val& x = get(v);
        G_REQUIRE(x.kind == Val::Tensor, "expected a tensor");
        return x.t;
    }
    int64_t intOf(const Value* v) {
        const Val& x = get(v);
        G_REQUIRE(x.kind == Val::Int || x.kind == Val::Bool, "expected an int");
        return x.i;
    }
    bool isNone(const Value* v) { return get(v).kind == Val::None; }
    double scalarOf(const Value* v) {
        const Val& x = get(v);
        if (x.kind == Val::Int || x.kind == Val::Bool) return static_cast<double>(x.i);
        G_REQUIRE(x.kind == Val::Double, "expected a scalar");
        return x.d;
    }
    bool isScalar(const Value* v) {
        const Val& x = get(v);
        return x.kind == Val::Int || x.kind == Val::Double || x.kind == Val::Bool;
    }

    void setTensor(const Value* v, ExprP e) {
        Val x;
        x.kind = Val::Tensor;
        x.t = std::move(e);
        env[v] = std::move(x);
    }

    ExprP unary(int op, ExprP a, double f = 0.0) {
        auto e = std::make_shared<Expr>();
        e->kind = Expr::Unary;
        e->op = op;
        e->f = f;
        e->shape = a->shape;
        e->in = {std::move(a)};
        return e;
    }
    ExprP binary(int op, ExprP a, ExprP b) {
        auto e = std::make_shared<Expr>();
        e->kind = Expr::Binary;
        e->op = op;
        e->shape = a->kind == Expr::Const ? b->shape : (b->kind == Expr::Const ? a->shape : broadcastShapes(a->shape, b->shape));
        e->is_bool = op >= FB_G_GT;
        e->in = {std::move(a), std::move(b)};
        return e;
    }

    ExprP operand(const Value* v) { return isScalar(v) ? constant(scalarOf(v)) : tensorOf(v); }

    void node(const Node* n) {
        const std::string kind = n->kind().toQualString();
        auto is = [&](const char* a, const char* b = nullptr) { return kind == a || (b != nullptr && kind == b); };
        if (n->kind() == prim::Constant) return;
        if (n->kind() == prim::ListConstruct) {
            Val v;
            if (n->output()->type()->isSubtypeOf(*c10::ListType::ofTensors())) {
                v.kind = Val::TensorList;
                for (const Value* in : n->inputs()) v.tl.push_back(tensorOf(in));
            } else {
                v.kind = Val::IntList;
                for (const Value* in : n->inputs()) v.il.push_back(intOf(in));
            }
            env[n->output()] = std::move(v);
            return;
        }
        auto out = [&](ExprP e) { setTensor(n->output(), std::move(e)); };
        static const std::unordered_map<std::string, int> unaries{
            {"aten::exp", FB_G_EXP}, {"aten::sigmoid", FB_G_SIGMOID}, {"aten::tanh", FB_G_TANH}, {"aten::relu", FB_G_RELU},
            {"aten::neg", FB_G_NEG}, {"aten::abs", FB_G_ABS}, {"aten::sqrt", FB_G_SQRT}, {"aten::log", FB_G_LOG}};
        static const std::unordered_map<std::string, int> binaries{
            {"aten::mul", FB_G_MUL}, {"aten::div", FB_G_DIV}, {"aten::minimum", FB_G_MIN}, {"aten::maximum", FB_G_MAX},
            {"aten::gt", FB_G_GT}, {"aten::ge", FB_G_GE}, {"aten::lt", FB_G_LT}, {"aten::le", FB_G_LE}, {"aten::eq", FB_G_EQ},
            {"aten::ne", FB_G_NE}};
        if (auto it = unaries.find(kind); it != unaries.end()) {
            ExprP a = tensorOf(n->input(0));
            G_REQUIRE(!a->is_bool, "arithmetic on a bool tensor");
            return out(unary(it->second, a));
        }
        if (auto it = binaries.find(kind); it != binaries.end()) {
            G_REQUIRE(n->inputs().size() == 2, "binary op with extra arguments");
            ExprP a = operand(n->input(0)), b = operand(n->input(1));
            G_REQUIRE(a->kind != Expr::Const || b->kind != Expr::Const, "scalar-only op");
            G_REQUIRE(!a->is_bool && !b->is_bool, "arithmetic on a bool tensor");
            if (it->second == FB_G_DIV && b->kind == Expr::Const) {
                // ATen divides a float tensor by a scalar as a multiplication with the reciprocal, formed in double and
                // rounded to fp32 once: same bits here
                const float inv = static_cast<float>(1.0 / b->f);
                return out(binary(FB_G_MUL, a, constant(static_cast<double>(inv))));
            }
            return out(binary(it->second, a, b));
        }
        if (is("aten::add") || is("aten::sub")) {
            ExprP a = operand(n->input(0)), b = operand(n->input(1));
            G_REQUIRE(a->kind != Expr::Const || b->kind != Expr::Const, "scalar-only op");
            G_REQUIRE(!a->is_bool && !b->is_bool, "arithmetic on a bool tensor");
            const double alpha = n->inputs().size() > 2 ? scalarOf(n->input(2)) : 1.0;
            if (alpha != 1.0) b = b->kind == Expr::Const ? constant(b->f * alpha) : binary(FB_G_MUL, b, constant(alpha));
            return out(binary(is("aten::add") ? FB_G_ADD : FB_G_SUB, a, b));
        }
        if (is("aten::clamp")) {
            ExprP a = tensorOf(n->input(0));
            if (!isNone(n->input(1))) a = unary(FB_G_CLAMP_MIN, a, scalarOf(n->input(1)));
            if (!isNone(n->input(2))) a = unary(FB_G_CLAMP_MAX, a, scalarOf(n->input(2)));
            return out(a);
        }
        if (is("aten::clone") || is("aten::contiguous") || is("immut::access")) return out(tensorOf(n->input(0)));
        if (is("immut::assign")) return out(tensorOf(n->input(1)));
        auto make = [&](Expr::Kind k, std::vector<ExprP> in, std::vector<int64_t> shape, std::vector<int64_t> iv) {
            auto e = std::make_shared<Expr>();
            e->kind = k;
            e->in = std::move(in);
            e->shape = std::move(shape);
            e->iv = std::move(iv);
            e->is_bool = e->in[0]->is_bool;
            return e;
        };
        if (is("immut::select", "aten::select")) {
            ExprP a = tensorOf(n->input(0));
            const int64_t rank = static_cast<int64_t>(a->shape.size());
            const int64_t dim = wrapDim(intOf(n->input(1)), rank);
            int64_t idx = intOf(n->input(2));
            if (idx < 0) idx += a->shape[dim];
            G_REQUIRE(idx >= 0 && idx < a->shape[dim], "select index out of range");
            std::vector<int64_t> shape = a->shape;
            shape.erase(shape.begin() + dim);
            return out(make(Expr::Select, {a}, shape, {dim, idx}));
        }
        auto sliceBounds = [&](const Node* nd, int first, int64_t size, int64_t& start, int64_t& end, int64_t& step) {
            start = isNone(nd->input(first)) ? 0 : intOf(nd->input(first));
            end = isNone(nd->input(first + 1)) ? size : intOf(nd->input(first + 1));
            step = intOf(nd->input(first + 2));
            G_REQUIRE(step >= 1, "slice step must be positive");
            if (start < 0) start += size;
            if (end < 0) end += size;
            start = std::min(std::max<int64_t>(start, 0), size);
            end = std::min(std::max(end, start), size);
        };
        if (is("immut::slice", "aten::slice")) {
            ExprP a = tensorOf(n->input(0));
            const int64_t dim = wrapDim(intOf(n->input(1)), static_cast<int64_t>(a->shape.size()));
            int64_t start, end, step;
            sliceBounds(n, 2, a->shape[dim], start, end, step);
            std::vector<int64_t> shape = a->shape;
            shape[dim] = (end - start + step - 1) / step;
            return out(make(Expr::Slice, {a}, shape, {dim, start, step}));
        }
        if (is("immut::squeeze", "aten::squeeze")) {
            ExprP a = tensorOf(n->input(0));
            G_REQUIRE(n->inputs().size() == 2, "squeeze without a dimension");
            const int64_t dim = wrapDim(intOf(n->input(1)), static_cast<int64_t>(a->shape.size()));
            if (a->shape[dim] != 1) return out(a);
            std::vector<int64_t> shape = a->shape;
            shape.erase(shape.begin() + dim);
            return out(make(Expr::Squeeze, {a}, shape, {dim}));
        }
        if (is("immut::unsqueeze", "aten::unsqueeze")) {
            ExprP a = tensorOf(n->input(0));
            const int64_t dim = wrapDim(intOf(n->input(1)), static_cast<int64_t>(a->shape.size()) + 1);
            std::vector<int64_t> shape = a->shape;
            shape.insert(shape.begin() + dim, 1);
            return out(make(Expr::Unsqueeze, {a}, shape, {dim}));
        }
        if (is("immut::permute", "aten::permute")) {
            ExprP a = tensorOf(n->input(0));
            const Val& dims = get(n->input(1));
            G_REQUIRE(dims.kind == Val::IntList && dims.il.size() == a->shape.size(), "bad permutation");
            std::vector<int64_t> shape, perm;
            for (int64_t d : dims.il) {
                perm.push_back(wrapDim(d, static_cast<int64_t>(a->shape.size())));
                shape.push_back(a->shape[perm.back()]);
            }
            return out(make(Expr::Permute, {a}, shape, perm));
        }
        if (is("immut::expand", "aten::expand") || is("immut::expand_as", "aten::expand_as")) {
            ExprP a = tensorOf(n->input(0));
            std::vector<int64_t> shape;
            if (kind.find("expand_as") != std::string::npos) {
                shape = tensorOf(n->input(1))->shape;
            } else {
                const Val& sz = get(n->input(1));
                G_REQUIRE(sz.kind == Val::IntList && sz.il.size() >= a->shape.size(), "bad expand size");
                shape = sz.il;
                const size_t lead = shape.size() - a->shape.size();
                for (size_t k = 0; k < shape.size(); ++k) {
                    if (shape[k] == -1) {
                        G_REQUIRE(k >= lead, "expand: -1 in a new leading dimension");
                        shape[k] = a->shape[k - lead];
                    }
                }
            }
            G_REQUIRE(broadcastShapes(a->shape, shape) == shape, "expand: shapes do not fit");
            return out(make(Expr::Expand, {a}, shape, {}));
        }
        if (is("immut::select_rev")) {
            ExprP self = tensorOf(n->input(0)), src = tensorOf(n->input(1));
            const int64_t dim = wrapDim(intOf(n->input(2)), static_cast<int64_t>(self->shape.size()));
            int64_t idx = intOf(n->input(3));
            if (idx < 0) idx += self->shape[dim];
            G_REQUIRE(idx >= 0 && idx < self->shape[dim], "select_rev index out of range");
            std::vector<int64_t> want = self->shape;
            want.erase(want.begin() + dim);
            G_REQUIRE(src->shape == want, "select_rev: src does not have the selected shape (broadcast not supported)");
            return out(make(Expr::SelectRev, {self, src}, self->shape, {dim, idx}));
        }
        if (is("immut::slice_rev")) {
            ExprP self = tensorOf(n->input(0)), src = tensorOf(n->input(1));
            const int64_t dim = wrapDim(intOf(n->input(2)), static_cast<int64_t>(self->shape.size()));
            int64_t start, end, step;
            sliceBounds(n, 3, self->shape[dim], start, end, step);
            std::vector<int64_t> want = self->shape;
            want[dim] = (end - start + step - 1) / step;
            G_REQUIRE(src->shape == want, "slice_rev: src does not have the sliced shape (broadcast not supported)");
            return out(make(Expr::SliceRev, {self, src}, self->shape, {dim, start, end, step}));
        }
        if (is("aten::cat") || is("aten::stack")) {
            const Val& list = get(n->input(0));
            G_REQUIRE(list.kind == Val::TensorList && !list.tl.empty(), "cat / stack of an empty or unknown list");
            const bool stack = is("aten::stack");
            const int64_t rank = static_cast<int64_t>(list.tl[0]->shape.size()) + (stack ? 1 : 0);
            const int64_t dim = wrapDim(intOf(n->input(1)), rank);
            std::vector<int64_t> shape = list.tl[0]->shape;
            std::vector<int64_t> iv{dim};
            if (stack) {
                for (const ExprP& e : list.tl) G_REQUIRE(e->shape == list.tl[0]->shape, "stack: shapes differ");
                shape.insert(shape.begin() + dim, static_cast<int64_t>(list.tl.size()));
            } else {
                int64_t total = 0;
                for (const ExprP& e : list.tl) {
                    G_REQUIRE(e->shape.size() == shape.size(), "cat: ranks differ");
                    for (size_t k = 0; k < shape.size(); ++k)
                        G_REQUIRE(static_cast<int64_t>(k) == dim || e->shape[k] == shape[k], "cat: shapes differ");
                    iv.push_back(total);  // first coordinate of this operand
                    total += e->shape[dim];
                }
                shape[dim] = total;
            }
            auto e = make(stack ? Expr::Stack : Expr::Cat, list.tl, shape, iv);
            for (const ExprP& x : list.tl) G_REQUIRE(x->is_bool == e->is_bool, "cat / stack of mixed dtypes");
            return out(e);
        }
        throw Unsupported("op " + kind + " has no generic lowering");
    }
};

// ---- program emission -------------------------------------------------------------------------------------------------
// d >= 2 as a multiply-shift divisor for 32-bit dividends: q = mulhi(magic, n); (((n - q) >> 1) + q) >> shift == n / d
// (the round-up variant of division by an invariant integer; exact for every n < 2^32).  d = 1 is not used by the kernel.
void divisorOf(uint32_t d, uint32_t& magic, uint32_t& shift) {
    magic = 0;
    shift = 0;
    if (d < 2) return;
    uint32_t log2d = 31;
    while (((d >> log2d) & 1u) == 0u) --log2d;
    if ((d & (d - 1)) == 0) {  // a power of two: magic 0 turns the expression into n >> log2d
        shift = log2d - 1;
        return;
    }
    const uint64_t two = 1ull << (32 + log2d);
    uint64_t m = two / d;
    const uint64_t rem = two - m * d;
    m += m;
    const uint64_t twice = rem + rem;
    if (twice >= d) m += 1;
    magic = static_cast<uint32_t>(m + 1);
    shift = log2d;
}

// Orders the dimensions the kernel decomposes the element number over: the lanes of a warp (fastest dimension) run
// along a dimension that no COND tests, so that a warp takes one path through the program instead of one per lane; the
// tested dimensions come next (their values still change close together in time, which keeps the rows they select from
// in cache), the others last.  Without a COND the output's own order stays.  Everything that names a dimension (loads,
// predicates, extents, divisors) is renumbered; out_coef keeps the element's place in the contiguous output.
void orderDimensionsForLanes(functs_b200_gprogram& P) {
    const int rank = P.rank;
    int64_t stride[8];
    {
        int64_t run = 1;
        for (int k = rank - 1; k >= 0; --k) {
            stride[k] = run;
            run *= P.shape[k];
        }
    }
    bool tested[8] = {false, false, false, false, false, false, false, false};
    bool any = false;
    for (int pc = 0; pc < P.ninstr; ++pc) {
        if (P.instr[pc].op != FB_G_COND) continue;
        const functs_b200_gpred& q = P.pred[P.instr[pc].arg];
        for (int k = 0; k < rank; ++k)
            if (q.coef[k] != 0 && P.shape[k] > 1) tested[k] = any = true;
    }
    int order[8];  // order[p] = the output dimension at position p (position rank - 1 is the fastest)
    for (int k = 0; k < rank; ++k) order[k] = k;
    if (any) {
        // lane dimension: the innermost untested one with at least a warp's worth of extent, else the largest untested
        int lane_dim = -1;
        for (int k = rank - 1; k >= 0 && lane_dim < 0; --k)
            if (!tested[k] && P.shape[k] >= 32) lane_dim = k;
        if (lane_dim < 0) {
            for (int k = 0; k < rank; ++k)
                if (!tested[k] && P.shape[k] > 1 && (lane_dim < 0 || P.shape[k] > P.shape[lane_dim])) lane_dim = k;
        }
        if (lane_dim >= 0) {
            int p = rank - 1;
            order[p--] = lane_dim;
            for (int k = rank - 1; k >= 0; --k)
                if (tested[k]) order[p--] = k;
            for (int k = rank - 1; k >= 0; --k)
                if (!tested[k] && k != lane_dim) order[p--] = k;
        }
    }
    int where[8];  // position of every output dimension
    for (int p = 0; p < rank; ++p) where[order[p]] = p;
    int32_t shape[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < rank; ++p) {
        shape[p] = P.shape[order[p]];
        P.out_coef[p] = static_cast<int32_t>(stride[order[p]]);
    }
    // A thread takes four neighbouring elements of the fastest dimension through the program in one pass when no COND
    // tests that dimension (decoding and predicates are then paid once for the four), the dimension is long enough to
    // matter, and a quarter of the threads still fills the GPU (a small output wants more threads, not longer ones:
    // the step-4 box decoding on [3000, 4] took 21 us with four elements per thread against 12.5 with one).
    P.vec = 1;
    P.lane_extent = rank > 0 ? shape[rank - 1] : 1;
    if (rank > 0 && !tested[order[rank - 1]] && shape[rank - 1] >= 8 && P.numel >= 4 * 148 * 256 * 2) {
        P.vec = 4;
        shape[rank - 1] = (shape[rank - 1] + 127) / 128 * 32;  // work items per row: blocks of 32 lanes x 4 elements
    }
    int64_t work = 1;
    for (int p = 0; p < 8; ++p) {
        P.shape[p] = shape[p];
        P.div_magic[p] = P.div_shift[p] = 0;
        if (p < rank) {
            divisorOf(static_cast<uint32_t>(shape[p]), P.div_magic[p], P.div_shift[p]);
            work *= shape[p];
        } else {
            P.out_coef[p] = 0;
        }
    }
    P.work = static_cast<int32_t>(work);
    auto renumber = [&](int32_t (&coef)[8]) {
        int32_t c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int p = 0; p < rank; ++p) c[p] = coef[order[p]];
        for (int p = 0; p < 8; ++p) coef[p] = c[p];
    };
    for (int k = 0; k < FB_G_MAX_LOADS; ++k) {
        renumber(P.load[k].coef);
        for (int t = 0; t < P.load[k].nterms; ++t)
            if (P.load[k].term[t].dim >= 0) P.load[k].term[t].dim = static_cast<int16_t>(where[P.load[k].term[t].dim]);
    }
    for (int k = 0; k < FB_G_MAX_PREDS; ++k) renumber(P.pred[k].coef);
}

struct Emitter {
    functs_b200_gprogram& P;
    int nloads = 0, npreds = 0;
    int depth = 0, max_depth = 0;

    int push(uint16_t op, uint16_t arg = 0) {
        G_REQUIRE(P.ninstr < FB_G_MAX_INSTR - 1, "program too long");
        P.instr[P.ninstr].op = op;
        P.instr[P.ninstr].arg = arg;
        P.instr[P.ninstr].imm.i = 0;
        return P.ninstr++;
    }
    void grow(int d) {
        depth += d;
        max_depth = std::max(max_depth, depth);
        G_REQUIRE(max_depth <= FB_G_STACK, "expression too deep for the value stack");
    }

    static Coord compose(const Coord& c, int64_t mul, int64_t add) {  // mul * c + add
        Coord r = c;
        if (c.div > 1) {
            // c = (m * x + a) / d is only evaluated where the division is exact (under the predicate of the strided
            // assignment that introduced it), so a factor that is a multiple of d cancels it: reading back the very
            // elements a strided slice_rev wrote (t[:, 1::2] = f(t[:, 1::2])) is the common case
            if (mul == 1 && add == 0) return r;
            G_REQUIRE(mul % c.div == 0, "index map needs a division inside a further map");
            mul /= c.div;
            r.div = 1;
        }
        r.mul = c.mul * mul;
        r.add = c.add * mul + add;
        return r;
    }
    static bool fits32(int64_t v) { return v > -(1ll << 31) && v < (1ll << 31); }

    // pushes "coordinate c in [lo, hi) and (c - lo) % step == 0"; returns -1 always true, -2 always false, else the slot
    int pred(const Coord& c, int64_t lo, int64_t hi, int64_t step) {
        G_REQUIRE(c.div == 1, "predicate on a divided coordinate");
        if (c.dim < 0) {
            const bool ok = c.add >= lo && c.add < hi && ((c.add - lo) % step) == 0;
            return ok ? -1 : -2;
        }
        // the coordinate runs over [0, extent) of its output dimension: a test that every value of v = mul * x + add
        // passes (an assignment to a whole dimension, `t[:] = ...`) or fails costs nothing and, more to the point, does
        // not duplicate the operand that both of its branches would otherwise carry
        {
            const int64_t extent = P.shape[c.dim];
            const int64_t v0 = c.add, v1 = c.mul * (extent - 1) + c.add;
            const int64_t vmin = std::min(v0, v1), vmax = std::max(v0, v1);
            if (vmax < lo || vmin >= hi) return -2;
            if (vmin >= lo && vmax < hi && (step == 1 || (c.mul % step == 0 && (c.add - lo) % step == 0))) return -1;
        }
        G_REQUIRE(npreds < FB_G_MAX_PREDS, "too many predicates");
        G_REQUIRE(fits32(c.mul) && fits32(c.add) && fits32(lo) && fits32(hi) && fits32(step), "predicate out of 32-bit range");
        functs_b200_gpred& q = P.pred[npreds];
        std::memset(&q, 0, sizeof(q));
        q.coef[c.dim] = static_cast<int32_t>(c.mul);
        q.add = static_cast<int32_t>(c.add);
        q.lo = static_cast<int32_t>(lo);
        q.hi = static_cast<int32_t>(hi);
        q.step = static_cast<int32_t>(step);
        return npreds++;
    }

    // if (p) A else B, where A and B each push one value
    template <typename FA, typename FB>
    void branch(int p, FA&& a, FB&& b) {
        if (p == -1) return a();
        if (p == -2) return b();
        const int cond = push(FB_G_COND, static_cast<uint16_t>(p));
        const int d0 = depth;
        a();
        const int jump = push(FB_G_JUMP);
        P.instr[cond].imm.i = P.ninstr;
        depth = d0;
        b();
        P.instr[jump].arg = static_cast<uint16_t>(P.ninstr);
    }

    void emit(const ExprP& e, const Map& m) {
        switch (e->kind) {
            case Expr::Const: {
                const int k = push(FB_G_CONST);
                P.instr[k].imm.f = static_cast<float>(e->f);
                grow(1);
                return;
            }
            case Expr::Leaf: {
                // described in a scratch slot first: a load equal to an earlier one (the same element of the same tensor,
                // reached again through another branch or a shared subexpression) reuses that slot
                functs_b200_gload L;
                std::memset(&L, 0, sizeof(L));
                L.tensor = e->tensor;
                L.dtype = e->dtype;
                L.nterms = 0;
                int64_t base = 0, stride = 1;
                for (int64_t q = static_cast<int64_t>(e->shape.size()) - 1; q >= 0; --q) {
                    const Coord& c = m[q];
                    if (e->shape[q] != 1) {
                        if (c.dim < 0) {
                            base += stride * (c.add / c.div);
                        } else {
                            G_REQUIRE(L.nterms < FB_G_MAX_TERMS, "too many index terms");
                            G_REQUIRE(fits32(c.mul) && fits32(c.add) && fits32(stride) && c.div < (1 << 15), "index term out of range");
                            functs_b200_gterm& t = L.term[L.nterms++];
                            t.dim = static_cast<int16_t>(c.dim);
                            t.div = static_cast<int16_t>(c.div);
                            t.mul = static_cast<int32_t>(c.mul);
                            t.add = static_cast<int32_t>(c.add);
                            t.stride = static_cast<int32_t>(stride);
                        }
                    }
                    stride *= e->shape[q];
                }
                G_REQUIRE(fits32(base), "offset out of range");
                L.base = static_cast<int32_t>(base);
                L.general = 0;
                for (int k = 0; k < L.nterms; ++k) L.general |= L.term[k].div > 1 ? 1 : 0;
                if (L.general == 0) {
                    // base + sum_k coef[k] * x[k]: constant parts of the terms go into the base
                    int64_t b2 = base, coef[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    for (int k = 0; k < L.nterms; ++k) {
                        const functs_b200_gterm& t = L.term[k];
                        b2 += static_cast<int64_t>(t.add) * t.stride;
                        if (t.dim >= 0) coef[t.dim] += static_cast<int64_t>(t.mul) * t.stride;
                    }
                    G_REQUIRE(fits32(b2), "offset out of range");
                    L.base = static_cast<int32_t>(b2);
                    for (int k = 0; k < 8; ++k) {
                        G_REQUIRE(fits32(coef[k]), "index coefficient out of range");
                        L.coef[k] = static_cast<int32_t>(coef[k]);
                    }
                    L.nterms = 0;
                    std::memset(L.term, 0, sizeof(L.term));
                }
                int slot = -1;
                for (int k = 0; k < nloads && slot < 0; ++k)
                    if (std::memcmp(&P.load[k], &L, sizeof(L)) == 0) slot = k;
                if (slot < 0) {
                    G_REQUIRE(nloads < FB_G_MAX_LOADS, "too many loads");
                    slot = nloads++;
                    P.load[slot] = L;
                }
                push(FB_G_LOAD, static_cast<uint16_t>(slot));
                grow(1);
                return;
            }
            case Expr::Unary: {
                emit(e->in[0], m);
                const int k = push(static_cast<uint16_t>(e->op));
                P.instr[k].imm.f = static_cast<float>(e->f);
                return;
            }
            case Expr::Binary: {
                const bool c0 = e->in[0]->kind == Expr::Const, c1 = e->in[1]->kind == Expr::Const;
                if (c0 != c1) {
                    // a scalar operand travels inside the instruction: no push, no pop
                    const ExprP& t = e->in[c0 ? 1 : 0];
                    const float imm = static_cast<float>(e->in[c0 ? 0 : 1]->f);
                    int op = e->op;
                    if (c0) {  // scalar on the left: commute, or mirror the comparison, or use the reversed forms
                        switch (e->op) {
                            case FB_G_SUB: op = FB_G_RSUB_IMM - FB_G_IMM; break;
                            case FB_G_DIV: op = FB_G_RDIV_IMM - FB_G_IMM; break;
                            case FB_G_GT: op = FB_G_LT; break;
                            case FB_G_GE: op = FB_G_LE; break;
                            case FB_G_LT: op = FB_G_GT; break;
                            case FB_G_LE: op = FB_G_GE; break;
                            default: break;  // add, mul, min, max, eq, ne commute
                        }
                    }
                    // (the operand has the result's shape or broadcasts into it: same rule as below)
                    Map ma(t->shape.size());
                    const size_t lead = e->shape.size() - t->shape.size();
                    for (size_t q = 0; q < t->shape.size(); ++q) {
                        if (t->shape[q] == 1 && e->shape[q + lead] != 1) ma[q] = Coord{};
                        else ma[q] = m[q + lead];
                    }
                    emit(t, ma);
                    const int k = push(static_cast<uint16_t>(op + FB_G_IMM));
                    P.instr[k].imm.f = imm;
                    return;
                }
                for (int side = 0; side < 2; ++side) {
                    const ExprP& a = e->in[side];
                    if (a->kind == Expr::Const) {
                        emit(a, {});
                        continue;
                    }
                    // broadcast: right-aligned dimensions, extent 1 reads coordinate 0
                    Map ma(a->shape.size());
                    const size_t lead = e->shape.size() - a->shape.size();
                    for (size_t q = 0; q < a->shape.size(); ++q) {
                        if (a->shape[q] == 1 && e->shape[q + lead] != 1) ma[q] = Coord{};
                        else ma[q] = m[q + lead];
                    }
                    emit(a, ma);
                }
                push(static_cast<uint16_t>(e->op));
                grow(-1);
                return;
            }
            case Expr::Select: {
                Map ma = m;
                Coord c;
                c.add = e->iv[1];
                ma.insert(ma.begin() + e->iv[0], c);
                return emit(e->in[0], ma);
            }
            case Expr::Slice: {
                Map ma = m;
                ma[e->iv[0]] = compose(m[e->iv[0]], e->iv[2], e->iv[1]);  // in = start + step * out
                return emit(e->in[0], ma);
            }
            case Expr::Squeeze: {
                Map ma = m;
                ma.insert(ma.begin() + e->iv[0], Coord{});
                return emit(e->in[0], ma);
            }
            case Expr::Unsqueeze: {
                Map ma = m;
                ma.erase(ma.begin() + e->iv[0]);
                return emit(e->in[0], ma);
            }
            case Expr::Permute: {
                Map ma(m.size());
                for (size_t i = 0; i < m.size(); ++i) ma[e->iv[i]] = m[i];
                return emit(e->in[0], ma);
            }
            case Expr::Expand: {
                const ExprP& a = e->in[0];
                Map ma(a->shape.size());
                const size_t lead = e->shape.size() - a->shape.size();
                for (size_t q = 0; q < a->shape.size(); ++q) ma[q] = (a->shape[q] == 1 && e->shape[q + lead] != 1) ? Coord{} : m[q + lead];
                return emit(a, ma);
            }
            case Expr::SelectRev: {
                const int64_t dim = e->iv[0], idx = e->iv[1];
                const int p = pred(m[dim], idx, idx + 1, 1);
                return branch(
                    p,
                    [&] {
                        Map ms = m;
                        ms.erase(ms.begin() + dim);
                        emit(e->in[1], ms);
                    },
                    [&] { emit(e->in[0], m); });
            }
            case Expr::SliceRev: {
                const int64_t dim = e->iv[0], start = e->iv[1], end = e->iv[2], step = e->iv[3];
                const int p = pred(m[dim], start, end, step);
                return branch(
                    p,
                    [&] {
                        Map ms = m;
                        Coord c = compose(m[dim], 1, -start);  // (coordinate - start) / step
                        G_REQUIRE(c.div == 1, "nested strided assignment");
                        c.div = step;
                        ms[dim] = c;
                        emit(e->in[1], ms);
                    },
                    [&] { emit(e->in[0], m); });
            }
            case Expr::Cat: {
                const int64_t dim = e->iv[0];
                std::function<void(size_t)> chain = [&](size_t k) {
                    const int64_t first = e->iv[1 + k];
                    auto self = [&] {
                        Map mk = m;
                        mk[dim] = compose(m[dim], 1, -first);
                        emit(e->in[k], mk);
                    };
                    if (k + 1 == e->in.size()) return self();
                    const int p = pred(m[dim], first, e->iv[2 + k], 1);
                    branch(p, self, [&] { chain(k + 1); });
                };
                return chain(0);
            }
            case Expr::Stack: {
                const int64_t dim = e->iv[0];
                std::function<void(size_t)> chain = [&](size_t k) {
                    auto self = [&] {
                        Map mk = m;
                        mk.erase(mk.begin() + dim);
                        emit(e->in[k], mk);
                    };
                    if (k + 1 == e->in.size()) return self();
                    const int p = pred(m[dim], static_cast<int64_t>(k), static_cast<int64_t>(k) + 1, 1);
                    branch(p, self, [&] { chain(k + 1); });
                };
                return chain(0);
            }
        }
    }
};

}  // namespace

// What a call leaves behind for the next one: the flattened programs and, for every tensor slot of every program, where
// the tensor came from.  key describes everything the programs depend on (shapes, dtypes, devices, scalar values).
struct GenericPlan {
    std::mutex mu;
    bool valid = false;
    std::string key;
    std::vector<functs_b200_gprogram> progs;                  // iterations x outputs (ninstr == 0: an empty output)
    std::vector<std::vector<std::pair<int, int>>> sources;    // per iteration
    std::vector<std::vector<int64_t>> out_shape;              // per program
    int32_t max_numel = 0;
};
std::shared_ptr<GenericPlan> NewGenericPlan() { return std::make_shared<GenericPlan>(); }

namespace {

void describe(const c10::IValue& iv, std::string& k) {
    if (iv.isTensor()) {
        const at::Tensor& t = iv.toTensor();
        k += 'T';
        k += std::to_string(static_cast<int>(t.scalar_type()));
        k += t.is_cuda() ? 'c' : 'h';
        k += std::to_string(t.is_cuda() ? t.get_device() : -1);
        for (int64_t d : t.sizes()) {
            k += ',';
            k += std::to_string(d);
        }
        k += ';';
    } else if (iv.isDouble()) {
        const double d = iv.toDouble();
        uint64_t bits;
        std::memcpy(&bits, &d, 8);
        k += 'D';
        k += std::to_string(bits);
        k += ';';
    } else if (iv.isInt()) {
        k += 'I';
        k += std::to_string(iv.toInt());
        k += ';';
    } else if (iv.isBool()) {
        k += iv.toBool() ? "B1;" : "B0;";
    } else if (iv.isNone()) {
        k += "N;";
    } else if (iv.isList()) {
        k += '[';
        for (const c10::IValue& e : iv.toListRef()) describe(e, k);
        k += ']';
    } else {
        k += "?;";  // the builder refuses such an input anyway
    }
}

at::Tensor sourceTensor(const std::vector<c10::IValue>& inputs, const std::pair<int, int>& src) {
    const c10::IValue& iv = inputs.at(static_cast<size_t>(src.first));
    if (src.second < 0) return iv.toTensor();
    return iv.toListRef().at(static_cast<size_t>(src.second)).toTensor();
}

// allocates the outputs, points the programs at this call's tensors and launches
void launchPrograms(std::vector<functs_b200_gprogram> progs, const std::vector<std::vector<std::pair<int, int>>>& sources,
                    const std::vector<std::vector<int64_t>>& out_shape, int32_t max_numel, size_t n_out, bool is_map,
                    const std::vector<c10::IValue>& inputs, std::vector<c10::IValue>& outputs) {
    const size_t iters = progs.size() / n_out;
    std::vector<std::vector<at::Tensor>> results(n_out);
    std::vector<at::Tensor> keep_alive;
    c10::Device device(c10::kCPU);
    bool have_device = false;
    for (size_t it = 0; it < iters; ++it) {
        std::vector<at::Tensor> ins;
        for (const auto& src : sources[it]) {
            at::Tensor t = sourceTensor(inputs, src).contiguous();
            if (!have_device) {
                device = t.device();
                have_device = true;
            }
            ins.push_back(t);
            keep_alive.push_back(std::move(t));
        }
        for (size_t o = 0; o < n_out; ++o) {
            functs_b200_gprogram& P = progs[it * n_out + o];
            at::Tensor out = at::empty(out_shape[it * n_out + o],
                                       at::TensorOptions().device(device).dtype(P.out_dtype == 1 ? at::kBool : at::kFloat));
            results[o].push_back(out);
            if (P.ninstr == 0) continue;
            P.out_ptr = out.data_ptr();
            for (size_t k = 0; k < ins.size(); ++k) P.in_ptr[k] = ins[k].data_ptr();
        }
    }
    std::vector<functs_b200_gprogram> live;  // programs of empty outputs are dropped (nothing to compute)
    int32_t max_rank = 0;
    for (const auto& P : progs) {
        if (P.ninstr > 0) {
            live.push_back(P);
            max_rank = std::max(max_rank, P.rank);
        }
    }
    if (!live.empty()) {
        c10::cuda::CUDAGuard guard(device);
        void* stream = at::cuda::getCurrentCUDAStream().stream();
        int rc;
        if (live.size() == 1) {
            rc = functs_b200_generic_group_launch(live.data(), 1, max_numel, max_rank, 0, stream);
        } else {
            const int64_t bytes = static_cast<int64_t>(live.size() * sizeof(functs_b200_gprogram));
            at::Tensor host = at::empty({bytes}, at::TensorOptions().dtype(at::kByte).pinned_memory(true));
            std::memcpy(host.data_ptr(), live.data(), static_cast<size_t>(bytes));
            at::Tensor table = host.to(device, /*non_blocking=*/true);  // (the pinned allocator defers the reuse of `host`)
            rc = functs_b200_generic_group_launch(static_cast<const functs_b200_gprogram*>(table.data_ptr()),
                                                  static_cast<int32_t>(live.size()), max_numel, max_rank, 1, stream);
        }
        TORCH_CHECK(rc == FB_OK, "functs_b200 generic group: ", functs_b200_last_error());
    }
    outputs.clear();
    for (size_t o = 0; o < n_out; ++o) {
        if (is_map) outputs.emplace_back(c10::List<at::Tensor>(results[o]));
        else outputs.emplace_back(results[o][0]);
    }
}

}  // namespace

// Runs the subgraph of a functor node as one launch.  stack_inputs: the node's inputs (for a map: lists for the parallel
// arguments).  Returns false when the group cannot be expressed as programs (nothing has been launched then).
bool RunGenericGroup(const std::shared_ptr<Graph>& sub, bool is_map, int64_t degree, const std::vector<int64_t>& par,
                     const std::vector<c10::IValue>& inputs, std::vector<c10::IValue>& outputs, std::string* why,
                     GenericPlan* plan) {
    const size_t n_out = sub->outputs().size();
    std::string key;
    if (plan != nullptr) {
        key.reserve(256);
        key += std::to_string(degree);
        key += '|';
        for (const c10::IValue& iv : inputs) describe(iv, key);
        std::unique_lock<std::mutex> lock(plan->mu);
        if (plan->valid && plan->key == key) {
            // same shapes, dtypes, devices and scalars as the call that built the programs: only the pointers change
            auto progs = plan->progs;
            auto sources = plan->sources;
            auto out_shape = plan->out_shape;
            const int32_t max_numel = plan->max_numel;
            lock.unlock();
            launchPrograms(std::move(progs), sources, out_shape, max_numel, n_out, is_map, inputs, outputs);
            return true;
        }
    }
    try {
        const int64_t iters = is_map ? degree : 1;
        G_REQUIRE(iters >= 1 && iters * static_cast<int64_t>(n_out) <= 4096, "too many programs");
        std::vector<functs_b200_gprogram> progs(static_cast<size_t>(iters) * n_out);
        std::vector<std::vector<std::pair<int, int>>> sources(static_cast<size_t>(iters));
        std::vector<std::vector<int64_t>> out_shape(progs.size());
        c10::Device device(c10::kCPU);
        bool have_device = false;
        int32_t max_numel = 0;
        for (int64_t it = 0; it < iters; ++it) {
            Builder b;
            // subgraph input 0: the iteration index (maps) or a None placeholder (plain groups)
            {
                Val v;
                if (is_map) {
                    v.kind = Val::Int;
                    v.i = it;
                }
                b.env[sub->inputs()[0]] = v;
            }
            G_REQUIRE(sub->inputs().size() == inputs.size() + 1 || (is_map && sub->inputs().size() == par.size() + 1),
                      "subgraph arity does not match the node");
            for (size_t k = 0; k + 1 < sub->inputs().size(); ++k) {
                c10::IValue iv = inputs[k];
                b.cur_arg = static_cast<int>(k);
                b.cur_pos = -1;
                if (is_map && k < par.size() && par[k]) {
                    iv = iv.toListRef().at(static_cast<size_t>(it));
                    b.cur_pos = static_cast<int>(it);
                }
                b.env[sub->inputs()[k + 1]] = b.fromIValue(iv);
            }
            b.cur_arg = -1;
            for (const Node* n : sub->nodes()) b.node(n);
            for (const at::Tensor& t : b.inputs) {
                if (!have_device) {
                    device = t.device();
                    have_device = true;
                }
                G_REQUIRE(t.device() == device, "tensor inputs on different devices");
            }
            G_REQUIRE(have_device, "a group without tensor inputs");
            for (const auto& src : b.sources) G_REQUIRE(src.first >= 0, "tensor constant inside the group");
            for (size_t o = 0; o < n_out; ++o) {
                ExprP e = b.tensorOf(sub->outputs()[o]);
                G_REQUIRE(e->shape.size() <= 8, "output rank above 8");
                const int64_t numel = numelOf(e->shape);
                G_REQUIRE(numel < (1ll << 31), "output too large for 32-bit indexing");
                functs_b200_gprogram& P = progs[static_cast<size_t>(it) * n_out + o];
                std::memset(&P, 0, sizeof(P));
                P.rank = static_cast<int32_t>(e->shape.size());
                for (size_t k = 0; k < e->shape.size(); ++k) P.shape[k] = static_cast<int32_t>(e->shape[k]);
                P.numel = static_cast<int32_t>(numel);
                P.out_dtype = e->is_bool ? 1 : 0;
                for (size_t k = 0; k < e->shape.size(); ++k) divisorOf(static_cast<uint32_t>(e->shape[k]), P.div_magic[k], P.div_shift[k]);
                out_shape[static_cast<size_t>(it) * n_out + o] = e->shape;
                if (numel == 0) {
                    P.ninstr = 0;
                    continue;
                }
                Emitter em{P};
                Map id(e->shape.size());
                for (size_t k = 0; k < id.size(); ++k) {
                    id[k].dim = static_cast<int>(k);
                    id[k].mul = 1;
                }
                em.emit(e, id);
                em.push(FB_G_END);
                orderDimensionsForLanes(P);
                max_numel = std::max(max_numel, P.work);
            }
            sources[static_cast<size_t>(it)] = b.sources;
        }
        if (plan != nullptr) {
            std::lock_guard<std::mutex> lock(plan->mu);
            plan->key = key;
            plan->progs = progs;
            plan->sources = sources;
            plan->out_shape = out_shape;
            plan->max_numel = max_numel;
            plan->valid = true;
        }
        launchPrograms(std::move(progs), sources, out_shape, max_numel, n_out, is_map, inputs, outputs);
        return true;
    } catch (const Unsupported& u) {
        if (why != nullptr) *why = u.what();
        return false;
    }
}

}  // namespace functs_b200
