// Static shapes / dtypes / devices for the values of a functionalized graph.
//
// Role of the reference's RefineInputTypes + InferDtypeAndDevice + InferShape (fait/passes/refine_types.cpp:179, 540,
// 670 with the per-op tables of fait/passes/tensor_type_funcs.cpp) for the part of the op set this build launches:
// graph inputs take the caller's type hints, TorchScript's own propagation supplies dtypes, devices and what sizes it can,
// and the tables below cover the immut:: Access / Assign family (which TorchScript does not know) and the shape-preserving
// and broadcasting aten:: operators of the fusable set.  A value whose shape cannot be
// derived (non-constant arguments, unknown operand shapes) simply stays unrefined; nothing is guessed.
#include <torch/csrc/jit/ir/constants.h>
#include <torch/csrc/jit/passes/shape_analysis.h>
#include <torch/csrc/jit/passes/symbolic_shape_analysis.h>

#include <functional>
#include <optional>
#include <unordered_map>
#include <unordered_set>

#include "fusion.h"

namespace functs_b200 {

using namespace torch::jit;

namespace {

using Sizes = std::vector<int64_t>;

std::optional<Sizes> knownSizes(const Value* v) {
    auto tt = v->type()->cast<c10::TensorType>();
    if (!tt) return std::nullopt;
    auto s = tt->sizes().concrete_sizes();
    if (!s) return std::nullopt;
    return *s;
}

std::optional<int64_t> constInt(const Value* v) { return constant_as<int64_t>(const_cast<Value*>(v)); }

std::optional<Sizes> constIntList(const Value* v) {
    auto iv = toIValue(v);
    if (iv && iv->isIntList()) return iv->toIntVector();
    if (v->node()->kind() == prim::ListConstruct) {
        Sizes out;
        for (const Value* e : v->node()->inputs()) {
            auto c = constInt(e);
            if (!c) return std::nullopt;
            out.push_back(*c);
        }
        return out;
    }
    return std::nullopt;
}

int64_t wrapDim(int64_t d, int64_t rank) { return d < 0 ? d + rank : d; }

// output sizes of one immut:: node from its operands' sizes, or nullopt
std::optional<Sizes> immutSizes(const Node* n) {
    const std::string kind = n->kind().toQualString();
    auto self = knownSizes(n->input(0));
    if (!self) return std::nullopt;
    const int64_t rank = static_cast<int64_t>(self->size());
    auto is = [&](const char* name) { return kind == name; };
    // every reverse op and assign returns a tensor of self's shape
    if (is("immut::assign") || is("immut::select_rev") || is("immut::slice_rev") || is("immut::repeat_rev") ||
        is("immut::expand_as_rev") || is("immut::access"))
        return self;
    if (is("immut::select")) {
        auto d = constInt(n->input(1));
        if (!d) return std::nullopt;
        const int64_t dim = wrapDim(*d, rank);
        if (dim < 0 || dim >= rank) return std::nullopt;
        Sizes out = *self;
        out.erase(out.begin() + dim);
        return out;
    }
    if (is("immut::slice")) {
        auto d = constInt(n->input(1));
        auto step = constInt(n->input(4));
        if (!d || !step || *step <= 0) return std::nullopt;
        const int64_t dim = wrapDim(*d, rank);
        if (dim < 0 || dim >= rank) return std::nullopt;
        const int64_t len = (*self)[dim];
        auto bound = [&](const Value* v, int64_t dflt) -> std::optional<int64_t> {
            if (v->type()->kind() == c10::TypeKind::NoneType) return dflt;
            auto iv = toIValue(v);
            if (iv && iv->isNone()) return dflt;
            auto c = constInt(v);
            if (!c) return std::nullopt;
            int64_t x = *c < 0 ? *c + len : *c;
            return x < 0 ? 0 : (x > len ? len : x);
        };
        auto lo = bound(n->input(2), 0), hi = bound(n->input(3), len);
        if (!lo || !hi) return std::nullopt;
        Sizes out = *self;
        out[dim] = *hi > *lo ? (*hi - *lo + *step - 1) / *step : 0;
        return out;
    }
    if (is("immut::squeeze")) {
        auto d = constInt(n->input(1));
        if (!d) return std::nullopt;
        const int64_t dim = wrapDim(*d, rank);
        if (dim < 0 || dim >= rank) return std::nullopt;
        Sizes out = *self;
        if (out[dim] == 1) out.erase(out.begin() + dim);
        return out;
    }
    if (is("immut::unsqueeze")) {
        auto d = constInt(n->input(1));
        if (!d) return std::nullopt;
        const int64_t dim = *d < 0 ? *d + rank + 1 : *d;
        if (dim < 0 || dim > rank) return std::nullopt;
        Sizes out = *self;
        out.insert(out.begin() + dim, 1);
        return out;
    }
    if (is("immut::view") || is("immut::reshape")) {
        auto size = constIntList(n->input(1));
        if (!size) return std::nullopt;
        int64_t numel = 1, known = 1, infer = -1;
        for (int64_t s : *self) numel *= s;
        for (size_t i = 0; i < size->size(); ++i) {
            if ((*size)[i] == -1) {
                if (infer >= 0) return std::nullopt;
                infer = static_cast<int64_t>(i);
            } else {
                known *= (*size)[i];
            }
        }
        Sizes out = *size;
        if (infer >= 0) {
            if (known == 0 || numel % known != 0) return std::nullopt;
            out[infer] = numel / known;
        } else if (known != numel) {
            return std::nullopt;
        }
        return out;
    }
    if (is("immut::permute")) {
        auto perm = constIntList(n->input(1));
        if (!perm || static_cast<int64_t>(perm->size()) != rank) return std::nullopt;
        Sizes out(rank);
        for (int64_t i = 0; i < rank; ++i) {
            const int64_t p = wrapDim((*perm)[i], rank);
            if (p < 0 || p >= rank) return std::nullopt;
            out[i] = (*self)[p];
        }
        return out;
    }
    if (is("immut::expand")) {
        auto size = constIntList(n->input(1));
        if (!size || static_cast<int64_t>(size->size()) < rank) return std::nullopt;
        Sizes out = *size;
        const int64_t lead = static_cast<int64_t>(size->size()) - rank;
        for (int64_t i = 0; i < static_cast<int64_t>(size->size()); ++i) {
            if (out[i] == -1) {
                if (i < lead) return std::nullopt;
                out[i] = (*self)[i - lead];
            }
        }
        return out;
    }
    if (is("immut::expand_as")) return knownSizes(n->input(1));
    if (is("immut::repeat")) {
        auto reps = constIntList(n->input(1));
        if (!reps || static_cast<int64_t>(reps->size()) < rank) return std::nullopt;
        Sizes out = *reps;
        const int64_t lead = static_cast<int64_t>(reps->size()) - rank;
        for (int64_t i = 0; i < rank; ++i) out[lead + i] *= (*self)[i];
        return out;
    }
    return std::nullopt;  // immut::index: data-independent only with index shapes; left to the caller
}

// aten:: operators of the fusable set whose result shape is that of operand 0 ...
bool isSameShapeUnary(Symbol k) {
    static const std::unordered_set<Symbol> kinds{aten::clone, aten::contiguous, aten::sigmoid, aten::exp, aten::tanh,
                                                  aten::relu,  aten::clamp,      aten::softmax};
    return kinds.count(k) != 0;
}
// ... or the broadcast of operands 0 and 1 (a Scalar operand does not change the shape); comparisons yield bool
bool isBroadcastBinary(Symbol k, bool& is_compare) {
    static const std::unordered_set<Symbol> arith{aten::add, aten::sub, aten::mul, aten::div, aten::minimum, aten::maximum,
                                                  aten::__and__};
    static const std::unordered_set<Symbol> cmp{aten::eq, aten::ne, aten::lt, aten::le, aten::gt, aten::ge};
    is_compare = cmp.count(k) != 0;
    return is_compare || arith.count(k) != 0;
}

std::optional<Sizes> broadcastSizes(const Sizes& a, const Sizes& b) {
    const size_t n = std::max(a.size(), b.size());
    Sizes out(n);
    for (size_t i = 0; i < n; ++i) {
        const int64_t x = i < n - a.size() ? 1 : a[i - (n - a.size())];
        const int64_t y = i < n - b.size() ? 1 : b[i - (n - b.size())];
        if (x != y && x != 1 && y != 1) return std::nullopt;
        out[i] = x == 1 ? y : x;
    }
    return out;
}

// ---- lists of tensors ---------------------------------------------------------------------------------------------------
// A List[Tensor] type cannot say what its elements look like, so lists are refined on the side: value -> tuple type with
// one tensor type per element (the reference's `refinedTypes` map, fait/passes/refine_types.h:8, 35-46; graph inputs get
// theirs from tuple type hints, refine_types.cpp:57-82, 179-195).
using Refined = std::unordered_map<Value*, c10::TypePtr>;

c10::TupleTypePtr refinedList(const Refined& refined, Value* v) {
    auto it = refined.find(v);
    return it == refined.end() ? nullptr : it->second->cast<c10::TupleType>();
}

// the most specific tensor type every element satisfies: dtype, device and rank if they agree, sizes where all agree
c10::TypePtr unifyElements(const c10::TupleTypePtr& tup) {
    c10::TensorTypePtr acc;
    for (const auto& e : tup->elements()) {
        auto tt = e->cast<c10::TensorType>();
        if (!tt) return nullptr;
        if (!acc) {
            acc = tt;
            continue;
        }
        if (acc->scalarType() != tt->scalarType() || acc->device() != tt->device() || acc->dim() != tt->dim() || !acc->dim())
            return c10::TensorType::get();
        auto a = acc->sizes().concrete_sizes(), b = tt->sizes().concrete_sizes();
        if (a && b && *a == *b) continue;
        std::vector<c10::ShapeSymbol> dims;
        for (size_t k = 0; k < *acc->dim(); ++k) {
            const auto x = acc->symbolic_sizes().at(k), y = tt->symbolic_sizes().at(k);
            dims.push_back(x.is_static() && y.is_static() && x.static_size() == y.static_size() ? x : c10::ShapeSymbol::newSymbol());
        }
        acc = acc->withSymbolicShapes(c10::SymbolicShape(dims));
    }
    return acc;
}

bool setRefined(Refined& refined, Value* v, c10::TypePtr t) {
    auto it = refined.find(v);
    if (it != refined.end() && *it->second == *t) return false;
    refined[v] = std::move(t);
    return true;
}

bool setTensorType(Value* v, const c10::TypePtr& t) {
    auto tt = t ? t->cast<c10::TensorType>() : nullptr;
    if (!tt || *v->type() == *tt) return false;
    auto cur = v->type()->cast<c10::TensorType>();
    if (cur && cur->sizes().concrete_sizes()) return false;  // already fully known
    v->setType(tt);
    return true;
}

bool refineLists(Block* block, Refined& refined) {
    static const Symbol kMap = Symbol::fromQualString("tssa::ParallelMap");
    bool changed = false;
    for (Node* n : block->nodes()) {
        if (n->kind() == prim::ListConstruct && n->output()->type()->isSubtypeOf(*c10::ListType::ofTensors())) {
            std::vector<c10::TypePtr> elems;
            for (Value* in : n->inputs()) elems.push_back(in->type());
            changed = setRefined(refined, n->output(), c10::TupleType::create(elems)) || changed;
        } else if (n->kind() == aten::__getitem__) {
            if (auto tup = refinedList(refined, n->input(0))) {
                auto idx = constInt(n->input(1));
                const int64_t count = static_cast<int64_t>(tup->elements().size());
                if (idx && *idx >= -count && *idx < count) {
                    changed = setTensorType(n->output(), tup->elements()[*idx < 0 ? *idx + count : *idx]) || changed;
                } else {
                    changed = setTensorType(n->output(), unifyElements(tup)) || changed;  // list[i] with a run-time index
                }
            }
        } else if (n->kind() == kMap) {
            Block* body = n->blocks()[0];
            for (size_t k = 1; k < n->inputs().size() && k < body->inputs().size(); ++k) {
                if (auto tup = refinedList(refined, n->input(k))) changed = setTensorType(body->inputs()[k], unifyElements(tup)) || changed;
            }
        } else if ((n->kind() == aten::cat || n->kind() == aten::stack) && n->inputs().size() == 2) {
            auto tup = refinedList(refined, n->input(0));
            auto dim = constInt(n->input(1));
            auto cur = n->output()->type()->cast<c10::TensorType>();
            if (tup && dim && !tup->elements().empty() && !(cur && cur->sizes().concrete_sizes())) {
                std::optional<Sizes> out;
                c10::TensorTypePtr first;
                bool ok = true;
                for (const auto& e : tup->elements()) {
                    auto tt = e->cast<c10::TensorType>();
                    auto s = tt ? tt->sizes().concrete_sizes() : std::nullopt;
                    if (!s) {
                        ok = false;
                        break;
                    }
                    if (!out) {
                        first = tt;
                        out = *s;
                        const int64_t rank = static_cast<int64_t>(s->size()) + (n->kind() == aten::stack ? 1 : 0);
                        const int64_t d = wrapDim(*dim, rank);
                        if (d < 0 || d >= rank) {
                            ok = false;
                            break;
                        }
                        if (n->kind() == aten::stack) out->insert(out->begin() + d, 1);
                    } else {
                        const int64_t d = wrapDim(*dim, static_cast<int64_t>(out->size()));
                        (*out)[d] += n->kind() == aten::stack ? 1 : (*s)[d];
                    }
                }
                if (ok && out && first->scalarType()) {
                    n->output()->setType(c10::TensorType::createContiguous(*first->scalarType(), first->device().value_or(c10::Device(c10::kCPU)), *out));
                    changed = true;
                }
            }
        }
        for (Block* b : n->blocks()) changed = refineLists(b, refined) || changed;
        // a map's result lists: `degree` elements of the body's result type
        if (n->kind() == kMap) {
            auto degree = constInt(n->input(0));
            Block* body = n->blocks()[0];
            if (degree && *degree >= 0 && *degree <= 4096) {
                for (size_t k = 0; k < n->outputs().size() && k < body->outputs().size(); ++k) {
                    if (!body->outputs()[k]->type()->cast<c10::TensorType>()) continue;
                    std::vector<c10::TypePtr> elems(static_cast<size_t>(*degree), body->outputs()[k]->type());
                    changed = setRefined(refined, n->output(k), c10::TupleType::create(elems)) || changed;
                }
            }
        }
    }
    return changed;
}

bool refineBlock(Block* block) {
    bool changed = false;
    for (Node* n : block->nodes()) {
        for (Block* b : n->blocks()) changed = refineBlock(b) || changed;
        if (n->outputs().size() != 1 || n->inputs().empty()) continue;
        auto out_t = n->output()->type()->cast<c10::TensorType>();
        auto in = n->input(0)->type()->cast<c10::TensorType>();
        if (!in || !out_t || out_t->sizes().concrete_sizes() || !in->scalarType()) continue;
        std::optional<Sizes> sizes;
        c10::ScalarType dtype = *in->scalarType();
        bool is_compare = false;
        if (std::string(n->kind().toQualString()).rfind("immut::", 0) == 0) {
            sizes = immutSizes(n);
        } else if (isSameShapeUnary(n->kind())) {
            sizes = knownSizes(n->input(0));
        } else if (isBroadcastBinary(n->kind(), is_compare) && n->inputs().size() >= 2) {
            auto a = knownSizes(n->input(0));
            if (a && n->input(1)->type()->cast<c10::TensorType>()) {
                auto b = knownSizes(n->input(1));
                if (b) sizes = broadcastSizes(*a, *b);
            } else if (a) {
                sizes = a;  // Scalar operand
            }
            if (is_compare) dtype = c10::kBool;
        }
        if (!sizes) continue;
        n->output()->setType(c10::TensorType::createContiguous(dtype, in->device().value_or(c10::Device(c10::kCPU)), *sizes));
        changed = true;
    }
    return changed;
}

}  // namespace

std::vector<std::pair<Value*, c10::TypePtr>> InferShapesRefined(const std::shared_ptr<Graph>& graph,
                                                                 const std::vector<c10::TypePtr>& type_hint) {
    Refined refined;
    for (size_t i = 0; i < type_hint.size() && i < graph->inputs().size(); ++i) {
        if (!type_hint[i]) continue;
        Value* in = graph->inputs()[i];
        // a tuple hint for a list input describes its elements: kept on the side, the list type itself cannot carry it
        if (type_hint[i]->cast<c10::TupleType>() && in->type()->cast<c10::ListType>()) refined[in] = type_hint[i];
        else in->setType(type_hint[i]);
    }
    // alternate between TorchScript's propagation (aten:: ops), the immut:: table and the list refinement until nothing
    // changes
    for (int round = 0; round < 8; ++round) {
        PropagateInputShapes(graph);     // dtypes, devices, ranks
        std::shared_ptr<Graph> gref = graph;
        try {
            PropagateShapesOnGraph(gref);  // concrete sizes through the aten:: shape functions
        } catch (const c10::Error&) {
            // TorchScript's symbolic shape analysis gives up on some list-taking operators (cat over a list input): the
            // tables below and the list refinement still run
        }
        // (TorchScript's propagation resets what it does not know, so the list results are re-derived first every round)
        bool any = false;
        for (int inner = 0; inner < 8; ++inner) {
            const bool l = refineLists(graph->block(), refined);
            const bool t = refineBlock(graph->block());
            any = any || t;
            if (!l && !t) break;
        }
        if (!any) break;
    }
    return std::vector<std::pair<Value*, c10::TypePtr>>(refined.begin(), refined.end());
}

void InferShapes(const std::shared_ptr<Graph>& graph, const std::vector<c10::TypePtr>& type_hint) {
    InferShapesRefined(graph, type_hint);
}

}  // namespace functs_b200
