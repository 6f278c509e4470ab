// Precompiled regions: how a functionalized TorchScript graph reaches the hand-written kernels of libfuncts_b200.so.
//
// The reference compiles whatever subgraph a tssa::ParallelFunctor node carries (GraphBuilder::compile,
// fait/fuser/graph_builder.cpp:259-712) and runs it (GraphBuilder::run, :714-927).  Here the kernels exist before the
// graph does, so the direction is reversed: every kernel sequence is described by the imperative program it replaces
// (a "pattern program", scripted and functionalized by the same passes as the user's program), and a region of the
// user's graph is handed to the kernels when its canonical signature equals the pattern's.
//
//   canonical signature   the nodes of a window of consecutive top-level nodes, nested blocks included, printed with
//                         values numbered by order of definition, outer values numbered by order of first use, constants
//                         by value.  Scalar constants the pattern declares free (thresholds, top-k) print as "?" and are
//                         collected; tensor constants (frozen module attributes: priors, anchor tables, weights) always
//                         print by dtype and rank only and are collected.  Shapes are not part of a signature: the
//                         kernels take sizes at run time and the operator checks what they cannot take.
//   match                 a pattern with n top-level nodes is compared with every window of n nodes of every block's
//                         top level; on equality the window is replaced by ONE tssa::ParallelFunctor node that carries
//                         the pattern's name (attribute `region`), the free constants as named attributes, the tensor
//                         constants (attribute `tparams`) and, as Subgraph, a copy of the window it replaced.
//   operator              a region functor never interprets its subgraph: it allocates outputs and scratch with torch,
//                         launches through functs_b200_group_launch on the current stream, reads the per-list counts
//                         back and narrows the padded outputs to the ragged lists the program returns.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/jit/ir/constants.h>
#include <torch/csrc/jit/ir/ir.h>
#include <torch/csrc/jit/runtime/operator.h>

#include <cmath>
#include <mutex>
#include <set>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

#include "../../../include/functs_b200.h"
#include "fusion.h"

namespace functs_b200 {

using namespace torch::jit;

namespace {

const Symbol kParallelFunctorSym = Symbol::fromQualString("tssa::ParallelFunctor");
const Symbol kAttrRegion = Symbol::attr("region");
const Symbol kAttrTParams = Symbol::attr("tparams");

// ---- canonical form ------------------------------------------------------------------------------------------------

struct Canon {
    std::ostringstream os;
    std::unordered_map<const Value*, std::string> names;
    std::unordered_set<const Node*> window;          // top-level nodes of the window
    std::vector<Value*> inputs;                      // outer non-constant values, by first use
    std::vector<double> fconsts;                     // every use of a float constant, in traversal order
    std::vector<int64_t> iconsts;                    // every use of an int constant
    std::vector<at::Tensor> tconsts;                 // every use of a tensor constant
    std::set<int> fwild, iwild;                      // slots (indices into fconsts / iconsts) that print as "?"
    int next_local = 0;

    bool inWindow(const Node* n) const {
        for (const Node* p = n; p != nullptr;) {
            if (window.count(p)) return true;
            const Block* b = p->owningBlock();
            p = b ? b->owningNode() : nullptr;
        }
        return false;
    }

    static std::string typeKind(const c10::TypePtr& t) {
        if (t->cast<c10::TensorType>()) return "Tensor";
        if (auto l = t->cast<c10::ListType>()) return typeKind(l->getElementType()) + "[]";
        if (auto o = t->cast<c10::OptionalType>()) return typeKind(o->getElementType()) + "?";
        if (auto tu = t->cast<c10::TupleType>()) {
            std::string s = "(";
            for (auto& e : tu->elements()) s += typeKind(e) + ",";
            return s + ")";
        }
        return t->str();
    }

    std::string constant(const Value* v) {
        const Node* n = v->node();
        if (v->type()->kind() == c10::TypeKind::NoneType) return "None";
        auto iv = toIValue(v);
        if (!iv) return "c<" + v->type()->str() + ">";
        std::ostringstream s;
        if (iv->isBool()) {
            s << (iv->toBool() ? "b1" : "b0");
        } else if (iv->isInt()) {
            const int slot = static_cast<int>(iconsts.size());
            iconsts.push_back(iv->toInt());
            if (iwild.count(slot)) s << "i?";
            else s << "i" << iv->toInt();
        } else if (iv->isDouble()) {
            const int slot = static_cast<int>(fconsts.size());
            fconsts.push_back(iv->toDouble());
            if (fwild.count(slot)) s << "f?";
            else {
                s.precision(17);
                s << "f" << iv->toDouble();
            }
        } else if (iv->isTensor()) {
            const at::Tensor& t = iv->toTensor();
            tconsts.push_back(t);
            s << "T<" << c10::toString(t.scalar_type()) << "," << t.dim() << ">";
        } else if (iv->isIntList()) {
            s << "[";
            for (int64_t e : iv->toIntVector()) s << e << ",";
            s << "]";
        } else if (iv->isString()) {
            s << "'" << iv->toStringRef() << "'";
        } else {
            s << "c<" << n->output()->type()->str() << ">";
        }
        return s.str();
    }

    std::string use(Value* v) {
        auto it = names.find(v);
        if (it != names.end()) return it->second;
        if (v->node()->kind() == prim::Constant) return constant(v);  // not cached: every use is its own slot
        // an outer value
        std::string nm = "$" + std::to_string(inputs.size()) + ":" + typeKind(v->type());
        inputs.push_back(v);
        names[v] = "$" + std::to_string(inputs.size() - 1);
        return nm;
    }

    void define(const Value* v) { names[v] = "%" + std::to_string(next_local++); }

    // In a graph without mutation a view and its immut:: copy mean the same; which of the two the functionalizer leaves
    // depends on whether the viewed tensor is a graph input (untracked) or an intermediate.  Both print as "access::".
    static std::string kindName(Symbol k) {
        static const std::unordered_set<std::string> access{"select", "slice", "squeeze", "unsqueeze", "permute", "view",
                                                             "reshape", "expand", "expand_as", "repeat"};
        const std::string q = k.toQualString();
        const size_t p = q.find("::");
        if (p != std::string::npos) {
            const std::string ns = q.substr(0, p), op = q.substr(p + 2);
            if ((ns == "aten" || ns == "immut") && access.count(op)) return "access::" + op;
        }
        return q;
    }

    void node(Node* n) {
        if (n->kind() == prim::Constant) return;
        std::vector<std::string> ins;
        for (Value* in : n->inputs()) ins.push_back(use(in));
        for (size_t k = 0; k < n->outputs().size(); ++k) {
            define(n->output(k));
            os << (k ? "," : "") << names[n->output(k)];
        }
        os << "=" << kindName(n->kind()) << "(";
        for (size_t k = 0; k < ins.size(); ++k) os << (k ? "," : "") << ins[k];
        os << ")";
        for (Block* b : n->blocks()) block(b);
        os << ";";
    }

    void block(Block* b) {
        os << "{(";
        for (size_t k = 0; k < b->inputs().size(); ++k) {
            define(b->inputs()[k]);
            os << (k ? "," : "") << names[b->inputs()[k]];
        }
        os << ")";
        for (Node* n : b->nodes()) node(n);
        os << "->(";
        for (size_t k = 0; k < b->outputs().size(); ++k) os << (k ? "," : "") << use(b->outputs()[k]);
        os << ")}";
    }
};

struct Described {
    std::string signature;
    std::vector<Value*> inputs, outputs;
    std::vector<double> fconsts;
    std::vector<int64_t> iconsts;
    std::vector<at::Tensor> tconsts;
};

Described describeWindow(const std::vector<Node*>& nodes, const std::set<int>& fwild, const std::set<int>& iwild) {
    Canon c;
    c.fwild = fwild;
    c.iwild = iwild;
    c.window.insert(nodes.begin(), nodes.end());
    for (Node* n : nodes) c.node(n);
    Described d;
    // live-outs: top-level results used outside the window (or returned by the enclosing block)
    c.os << "outs(";
    for (Node* n : nodes) {
        for (Value* o : n->outputs()) {
            bool outside = false;
            for (const Use& u : o->uses()) outside = outside || !c.inWindow(u.user);
            if (outside) {
                d.outputs.push_back(o);
                c.os << c.names[o] << ",";
            }
        }
    }
    c.os << ")";
    d.signature = c.os.str();
    d.inputs = std::move(c.inputs);
    d.fconsts = std::move(c.fconsts);
    d.iconsts = std::move(c.iconsts);
    d.tconsts = std::move(c.tconsts);
    return d;
}

// top-level nodes of a block that take part in windows: everything but constants and the tuple that only packs the
// block's return values
std::vector<Node*> windowNodes(Block* b) {
    std::vector<Node*> out;
    for (Node* n : b->nodes()) {
        if (n->kind() == prim::Constant) continue;
        out.push_back(n);
    }
    while (!out.empty() && out.back()->kind() == prim::TupleConstruct) {
        bool only_return = true;
        for (const Use& u : out.back()->output()->uses()) only_return = only_return && u.user == b->return_node();
        if (!only_return) break;
        out.pop_back();
    }
    return out;
}

// ---- pattern registry ------------------------------------------------------------------------------------------------

struct RegionPattern {
    std::string name;       // adapter name
    std::string signature;
    int num_nodes = 0;
    std::set<int> fwild, iwild;
    std::vector<std::pair<std::string, int>> froles, iroles;  // attribute name -> slot
    int num_inputs = 0, num_outputs = 0, num_tensors = 0;
};

std::mutex g_patterns_mutex;
std::vector<RegionPattern>& patterns() {
    static std::vector<RegionPattern> p;
    return p;
}

std::atomic<int64_t> g_interpreted_runs{0};
std::atomic<int64_t> g_generic_runs{0};

// ---- replacement --------------------------------------------------------------------------------------------------

void replaceWindow(const std::vector<Node*>& nodes, const Described& d, const RegionPattern& pat) {
    Node* last = nodes.back();
    Graph* g = last->owningGraph();
    Node* f = g->createWithSubgraph(kParallelFunctorSym);
    f->insertAfter(last);
    f->setSourceRange(nodes.front()->sourceRange());
    // Subgraph: a copy of the window (documentation and IR dumps; it is never interpreted)
    auto sub = f->g(attr::Subgraph);
    std::unordered_map<Value*, Value*> vmap;
    for (Value* in : d.inputs) {
        Value* si = sub->addInput();
        si->copyMetadata(in);
        vmap[in] = si;
        f->addInput(in);
    }
    auto lookup = [&](Value* v) -> Value* {
        auto it = vmap.find(v);
        if (it != vmap.end()) return it->second;
        TORCH_INTERNAL_ASSERT(v->node()->kind() == prim::Constant, "region window reads an unmapped value");
        Node* c = sub->createClone(v->node(), [](Value*) -> Value* { return nullptr; });
        sub->prependNode(c);
        vmap[v] = c->output();
        return c->output();
    };
    for (Node* n : nodes) {
        Node* c = sub->createClone(n, lookup);
        sub->appendNode(c);
        for (size_t k = 0; k < n->outputs().size(); ++k) vmap[n->output(k)] = c->output(k);
    }
    std::unordered_set<Node*> in_window(nodes.begin(), nodes.end());
    for (Value* o : d.outputs) {
        sub->registerOutput(vmap.at(o));
        Value* fo = f->addOutput();
        fo->copyMetadata(o);
    }
    for (size_t k = 0; k < d.outputs.size(); ++k) d.outputs[k]->replaceAllUsesWith(f->output(k));
    f->s_(kAttrRegion, pat.name);
    for (auto& r : pat.froles) f->f_(Symbol::attr(r.first), d.fconsts.at(static_cast<size_t>(r.second)));
    for (auto& r : pat.iroles) f->i_(Symbol::attr(r.first), d.iconsts.at(static_cast<size_t>(r.second)));
    f->ts_(kAttrTParams, d.tconsts);
    f->i_(Symbol::attr("parallel_degree"), -1);
    f->i_(Symbol::attr("is_parallel_map"), 0);
    f->is_(Symbol::attr("is_parallel_args"), std::vector<int64_t>(d.inputs.size(), 0));
    std::vector<c10::TypePtr> refine;
    for (Value* in : d.inputs) refine.push_back(in->type());
    f->tys_(Symbol::attr("input_refine_types"), refine);
    for (auto it = nodes.rbegin(); it != nodes.rend(); ++it) (*it)->destroy();
}

bool matchBlock(Block* b) {
    std::vector<RegionPattern> pats;
    {
        std::lock_guard<std::mutex> lock(g_patterns_mutex);
        pats = patterns();
    }
    bool any = false;
    for (bool again = true; again;) {
        again = false;
        std::vector<Node*> top = windowNodes(b);
        for (const RegionPattern& pat : pats) {
            const int n = pat.num_nodes;
            for (int s = 0; !again && s + n <= static_cast<int>(top.size()); ++s) {
                if (top[s]->kind() == kParallelFunctorSym) continue;
                std::vector<Node*> win(top.begin() + s, top.begin() + s + n);
                Described d = describeWindow(win, pat.fwild, pat.iwild);
                if (d.signature != pat.signature) continue;
                replaceWindow(win, d, pat);
                again = any = true;
            }
            if (again) break;
        }
    }
    for (Node* n : b->nodes()) {
        if (n->kind() == kParallelFunctorSym) continue;
        for (Block* nb : n->blocks()) any = matchBlock(nb) || any;
    }
    return any;
}

// ---- operator helpers ----------------------------------------------------------------------------------------------

void checkRc(int rc, const char* what) { TORCH_CHECK(rc == FB_OK, "functs_b200 ", what, ": ", functs_b200_last_error()); }

int lookupGroup(const char* sig) {
    const int id = functs_b200_group_lookup(sig);
    TORCH_CHECK(id >= 0, "functs_b200: the kernel library has no group '", sig, "'");
    return id;
}

at::Tensor cudaF32(const at::Tensor& t, const char* what) {
    TORCH_CHECK(t.is_cuda(), "functs_b200: ", what, " must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.scalar_type() == at::kFloat, "functs_b200: ", what, " must be float32");
    return t.contiguous();
}

void raiseOnStatus(const at::Tensor& status_host, const char* what) {
    const int bits = status_host.item<int>();
    TORCH_CHECK(bits == 0, "functs_b200 ", what, ": device status ", bits,
                (bits & FB_STATUS_CAND_OVERFLOW) ? " (a candidate list overflowed)" : "",
                (bits & FB_STATUS_WAIT_TIMEOUT) ? " (a bounded device-side wait ran out)" : "",
                (bits & FB_STATUS_INDEX_RANGE) ? " (an index was out of range)" : "");
}

// a frozen module attribute, moved to the device of the inputs once per device
struct DeviceConstants {
    std::mutex m;
    std::unordered_map<int, std::vector<at::Tensor>> per_device;
};

using Adapter = std::function<Operation(const Node*)>;

// ---- C2: YOLOv3-style post-process ---------------------------------------------------------------------------------
// Pattern outputs (in order of definition): bboxes, obj, cls, results   (dense = 1)
//                                       or: results                     (dense = 0)
// Tensor constants, by first use: grid and anchor table of level 0, 1, 2: [S*S*3, 2] each.
Operation makeYolo(const Node* node, bool dense) {
    const double thr = node->f(Symbol::attr("score_thr")), iou = node->f(Symbol::attr("iou_thr"));
    const int64_t topk = node->i(Symbol::attr("topk"));
    const std::vector<at::Tensor> tc = node->ts(kAttrTParams);
    TORCH_CHECK(tc.size() >= 6, "yolov3 region: expected the grid and anchor constants of three levels, got ", tc.size());
    // the kernels generate the cell grid and hold the reference's anchor table (yolov3_bbox.py:191-193): the program's
    // constants must be exactly those
    static const float kAnchors[3][3][2] = {{{116, 90}, {156, 198}, {373, 326}}, {{30, 61}, {62, 45}, {59, 119}},
                                            {{10, 13}, {16, 30}, {33, 23}}};
    std::vector<int64_t> sizes;
    for (int l = 0; l < 3; ++l) {
        at::Tensor grid = tc[2 * l].to(at::kCPU).contiguous(), anc = tc[2 * l + 1].to(at::kCPU).contiguous();
        TORCH_CHECK(grid.dim() == 2 && grid.size(1) == 2 && grid.sizes() == anc.sizes() && grid.size(0) % 3 == 0,
                    "yolov3 region: unexpected grid / anchor constants");
        const int64_t cells = grid.size(0) / 3;
        const int64_t s = static_cast<int64_t>(std::llround(std::sqrt(static_cast<double>(cells))));
        TORCH_CHECK(s * s == cells, "yolov3 region: the level is not square");
        sizes.push_back(s);
        const float* gp = grid.data_ptr<float>();
        const float* ap = anc.data_ptr<float>();
        for (int64_t i = 0; i < grid.size(0); ++i) {
            const int64_t cell = i / 3, a = i % 3;
            TORCH_CHECK(gp[2 * i] == static_cast<float>(cell % s) && gp[2 * i + 1] == static_cast<float>(cell / s) &&
                            ap[2 * i] == kAnchors[l][a][0] && ap[2 * i + 1] == kAnchors[l][a][1],
                        "yolov3 region: grid / anchor constants differ from the table the kernels hold");
        }
    }
    const int gid = lookupGroup(
        "yolov3{decode->loop[b<B]{mul(obj,cls)->gt(thr)->nonzero->sort(desc,stable)->slice[:k]->class-offset nms}}");
    return [=](Stack& stack) {
        c10::List<at::Tensor> list = pop(stack).toTensorList();
        TORCH_CHECK(list.size() == 3, "yolov3 region: expected three prediction maps");
        std::vector<at::Tensor> maps;
        for (size_t l = 0; l < 3; ++l) {
            at::Tensor m = cudaF32(list.get(l), "prediction map");
            TORCH_CHECK(m.dim() == 4 && m.size(1) == 255 && m.size(2) == sizes[l] && m.size(3) == sizes[l],
                        "yolov3 region: map ", l, " must be [B, 255, ", sizes[l], ", ", sizes[l], "]");
            maps.push_back(m);
        }
        c10::cuda::CUDAGuard guard(maps[0].device());
        const int64_t B = maps[0].size(0);
        const int64_t N = 3 * (sizes[0] * sizes[0] + sizes[1] * sizes[1] + sizes[2] * sizes[2]);
        const int64_t capacity = N * 80;
        auto f32 = maps[0].options();
        auto i64 = f32.dtype(at::kLong);
        at::Tensor boxes = at::empty({B, N, 4}, f32);
        at::Tensor obj, cls;
        if (dense) {
            obj = at::empty({B, N}, f32);
            cls = at::empty({B, N, 80}, f32);
        }
        at::Tensor dets = at::empty({B, topk, 5}, f32), labels = at::empty({B, topk}, i64), ids = at::empty({B, topk}, i64);
        at::Tensor counts = at::empty({B}, f32.dtype(at::kInt)), status = at::zeros({1}, f32.dtype(at::kInt));
        at::Tensor scratch = at::empty(
            {functs_b200_yolo_scratch_bytes(static_cast<int32_t>(B), static_cast<int32_t>(sizes[0]), static_cast<int32_t>(sizes[1]),
                                            static_cast<int32_t>(sizes[2]), capacity, static_cast<int32_t>(topk))},
            f32.dtype(at::kByte));
        const void* in_ptrs[] = {maps[0].data_ptr(), maps[1].data_ptr(), maps[2].data_ptr()};
        const int64_t ints[] = {B, sizes[0], sizes[1], sizes[2], topk, capacity};
        const double floats[] = {thr, iou};
        void* outs[] = {boxes.data_ptr(), dense ? obj.data_ptr() : nullptr, dense ? cls.data_ptr() : nullptr,
                        dets.data_ptr(), labels.data_ptr(), ids.data_ptr(), counts.data_ptr(), nullptr};
        checkRc(functs_b200_group_launch(gid, in_ptrs, ints, floats, outs, scratch.data_ptr(), status.data_ptr<int>(),
                                         at::cuda::getCurrentCUDAStream().stream()),
                "yolov3 post-process");
        // the only synchronisation: counts (and the status word) come back, the padded outputs are narrowed
        at::Tensor host = at::cat({counts, status}).cpu();
        raiseOnStatus(host[B], "yolov3 post-process");
        const int* cnt = host.data_ptr<int>();
        c10::impl::GenericList results(c10::TupleType::create({c10::TensorType::get(), c10::TensorType::get(), c10::TensorType::get()}));
        for (int64_t b = 0; b < B; ++b) {
            results.push_back(c10::ivalue::Tuple::create(
                {dets[b].narrow(0, 0, cnt[b]), labels[b].narrow(0, 0, cnt[b]), ids[b].narrow(0, 0, cnt[b])}));
        }
        if (dense) {
            push(stack, std::move(boxes), std::move(obj), std::move(cls));
        }
        stack.emplace_back(std::move(results));
    };
}

// ---- C3: SSD-style post-process --------------------------------------------------------------------------------------
// Pattern outputs: scores [B, P, C] (a view of the class-major buffer), results, bboxes.
// Tensor constants by first use: priors (w, h) [P, 2] and priors (cx, cy) [P, 2] (views of one [P, 4] table), several uses.
Operation makeSsd(const Node* node) {
    const double thr = node->f(Symbol::attr("score_thr")), iou = node->f(Symbol::attr("iou_thr"));
    const double clamp_max = node->f(Symbol::attr("clamp_max"));
    const int64_t topk = node->i(Symbol::attr("topk"));
    const std::vector<at::Tensor> tc = node->ts(kAttrTParams);
    TORCH_CHECK(tc.size() == 3, "ssd region: expected 3 uses of the prior table, got ", tc.size());
    // uses in program order: pwh (x mul), pxy (add), pwh (exp mul); the table is rebuilt as [P, 4] = (cx, cy, w, h)
    at::Tensor pwh = tc[0].to(at::kCPU), pxy = tc[1].to(at::kCPU);
    TORCH_CHECK(pwh.dim() == 2 && pwh.size(1) == 2 && pxy.sizes() == pwh.sizes() && at::equal(tc[2].to(at::kCPU), pwh),
                "ssd region: unexpected prior constants");
    at::Tensor priors_cpu = at::cat({pxy, pwh}, 1).contiguous();
    auto consts = std::make_shared<DeviceConstants>();
    const int g1 = lookupGroup("ssd{softmax(-1)->slice[:-1]->delta2bbox->slice_rev[0::2,1::2](clamp)}");
    const int g2 = lookupGroup("pmap[c<classes]{gt(thr)->nonzero->sort(desc,stable)->slice[:k]->index->torchvision::nms->index}");
    return [=](Stack& stack) {
        at::Tensor conf = cudaF32(pop(stack).toTensor(), "conf");
        at::Tensor loc = cudaF32(pop(stack).toTensor(), "loc");
        TORCH_CHECK(loc.dim() == 3 && loc.size(2) == 4 && conf.dim() == 3 && conf.size(0) == loc.size(0) &&
                        conf.size(1) == loc.size(1) && loc.size(1) == priors_cpu.size(0) && conf.size(2) >= 2,
                    "ssd region: loc [B, P, 4] / conf [B, P, C+1] do not fit the prior table");
        c10::cuda::CUDAGuard guard(loc.device());
        at::Tensor priors;
        {
            std::lock_guard<std::mutex> lock(consts->m);
            auto& v = consts->per_device[loc.get_device()];
            if (v.empty()) v.push_back(priors_cpu.to(loc.device()));
            priors = v[0];
        }
        const int64_t B = loc.size(0), P = loc.size(1), C = conf.size(2) - 1;
        auto f32 = loc.options();
        at::Tensor boxes = at::empty({B, P, 4}, f32), scores_cm = at::empty({B, C, P}, f32);
        at::Tensor dets = at::empty({B, C, topk, 5}, f32), ids = at::empty({B, C, topk}, f32.dtype(at::kLong));
        at::Tensor counts = at::empty({B, C}, f32.dtype(at::kInt));
        void* stream = at::cuda::getCurrentCUDAStream().stream();
        {
            const void* in_ptrs[] = {loc.data_ptr(), conf.data_ptr(), priors.data_ptr()};
            const int64_t ints[] = {B, P, C};
            const double floats[] = {clamp_max};
            void* outs[] = {boxes.data_ptr(), scores_cm.data_ptr()};
            checkRc(functs_b200_group_launch(g1, in_ptrs, ints, floats, outs, nullptr, nullptr, stream), "ssd softmax + decode");
        }
        {
            const void* in_ptrs[] = {boxes.data_ptr(), scores_cm.data_ptr()};
            const int64_t ints[] = {B, P, C, topk};
            const double floats[] = {thr, iou};
            void* outs[] = {dets.data_ptr(), ids.data_ptr(), counts.data_ptr()};
            checkRc(functs_b200_group_launch(g2, in_ptrs, ints, floats, outs, nullptr, nullptr, stream), "ssd class NMS");
        }
        // ragged results: one compaction over the whole batch, then per-image views
        at::Tensor valid = at::arange(topk, counts.options()).view({1, 1, topk}) < counts.unsqueeze(-1);  // [B, C, K]
        at::Tensor flat_valid = valid.reshape({-1});
        at::Tensor all_dets = dets.reshape({-1, 5}).index({flat_valid});
        at::Tensor all_ids = ids.reshape({-1}).index({flat_valid});
        at::Tensor all_labels = at::arange(C, ids.options()).view({1, C, 1}).expand({B, C, topk}).reshape({-1}).index({flat_valid});
        at::Tensor per_image = counts.sum({1}, false, at::kLong).cpu();
        const int64_t* pi = per_image.data_ptr<int64_t>();
        c10::impl::GenericList results(c10::TupleType::create({c10::TensorType::get(), c10::TensorType::get(), c10::TensorType::get()}));
        int64_t off = 0;
        for (int64_t b = 0; b < B; ++b) {
            results.push_back(c10::ivalue::Tuple::create(
                {all_dets.narrow(0, off, pi[b]), all_labels.narrow(0, off, pi[b]), all_ids.narrow(0, off, pi[b])}));
            off += pi[b];
        }
        push(stack, scores_cm.permute({0, 2, 1}));
        stack.emplace_back(std::move(results));
        push(stack, std::move(boxes));
    };
}

// ---- C4: imperative LSTM ----------------------------------------------------------------------------------------------
// Pattern outputs: hs, cs.  Tensor constants by first use: w_ih [4, I, H], b_ih [4, 1, H], w_hh [4, H, H], b_hh [4, 1, H].
Operation makeLstm(const Node* node) {
    const std::vector<at::Tensor> tc = node->ts(kAttrTParams);
    TORCH_CHECK(tc.size() == 4, "lstm region: expected 4 weight constants, got ", tc.size());
    const int64_t hidden = node->i(Symbol::attr("hidden"));
    TORCH_CHECK(tc[0].dim() == 3 && tc[0].size(0) == 4 && tc[0].size(2) == hidden && tc[2].dim() == 3 &&
                    tc[2].size(0) == 4 && tc[2].size(1) == hidden && tc[2].size(2) == hidden &&
                    tc[1].numel() == 4 * hidden && tc[3].numel() == 4 * hidden,
                "lstm region: weights must be gate-leading: w_ih [4, I, H], w_hh [4, H, H], biases [4, 1, H]");
    auto consts = std::make_shared<DeviceConstants>();
    const int gid = lookupGroup(
        "loop[t<T]{matmul(x[t],w_ih)+matmul(h,w_hh)->immut::select[gates]->sigmoid/tanh->select_rev(hs,t)->select_rev(cs,t)}");
    return [=](Stack& stack) {
        at::Tensor x = cudaF32(pop(stack).toTensor(), "x");
        TORCH_CHECK(x.dim() == 3 && x.size(2) == tc[0].size(1), "lstm region: x must be [T, B, ", tc[0].size(1), "]");
        c10::cuda::CUDAGuard guard(x.device());
        std::vector<at::Tensor> w;
        {
            std::lock_guard<std::mutex> lock(consts->m);
            auto& v = consts->per_device[x.get_device()];
            if (v.empty()) {
                for (const at::Tensor& t : tc) v.push_back(t.to(x.device(), at::kFloat).contiguous());
            }
            w = v;
        }
        const int64_t T = x.size(0), B = x.size(1), I = x.size(2);
        at::Tensor hs = at::empty({T, B, hidden}, x.options()), cs = at::empty({T, B, hidden}, x.options());
        at::Tensor status = at::zeros({1}, x.options().dtype(at::kInt));
        at::Tensor scratch = at::empty({functs_b200_lstm_scratch_bytes(static_cast<int32_t>(T), static_cast<int32_t>(B),
                                                                       static_cast<int32_t>(I), static_cast<int32_t>(hidden))},
                                       x.options().dtype(at::kByte));
        const void* in_ptrs[] = {x.data_ptr(), w[0].data_ptr(), w[2].data_ptr(), w[1].data_ptr(), w[3].data_ptr()};
        const int64_t ints[] = {T, B, I, hidden};
        void* outs[] = {hs.data_ptr(), cs.data_ptr()};
        checkRc(functs_b200_group_launch(gid, in_ptrs, ints, nullptr, outs, scratch.data_ptr(), status.data_ptr<int>(),
                                         at::cuda::getCurrentCUDAStream().stream()),
                "lstm");
        raiseOnStatus(status.cpu(), "lstm");
        push(stack, std::move(hs), std::move(cs));
    };
}

// ---- C5: YOLACT-style mask assembly ----------------------------------------------------------------------------------
// Pattern outputs (loop results in order): logits [B, H, W, N], masks [B, N, H, W]   (with_logits = 1)   or: masks.
Operation makeYolact(const Node* node, bool with_logits) {
    const double thr = node->f(Symbol::attr("thr"));
    const int gid = lookupGroup("loop[d<n]{matmul(proto,coef[d])->sigmoid->slice->slice_rev(crop)->gt(thr)}");
    return [=](Stack& stack) {
        at::Tensor boxes = cudaF32(pop(stack).toTensor(), "boxes");
        at::Tensor coef = cudaF32(pop(stack).toTensor(), "coef");
        at::Tensor proto = cudaF32(pop(stack).toTensor(), "proto");
        TORCH_CHECK(proto.dim() == 4 && proto.size(3) == 32 && coef.dim() == 3 && coef.size(2) == 32 && boxes.dim() == 3 &&
                        boxes.size(2) == 4 && coef.size(0) == proto.size(0) && boxes.size(0) == proto.size(0) &&
                        boxes.size(1) == coef.size(1),
                    "yolact region: proto [B, H, W, 32], coef [B, N, 32], boxes [B, N, 4] expected");
        c10::cuda::CUDAGuard guard(proto.device());
        const int64_t B = proto.size(0), H = proto.size(1), W = proto.size(2), N = coef.size(1);
        at::Tensor masks = at::empty({B, N, H, W}, proto.options().dtype(at::kByte));
        at::Tensor logits;
        if (with_logits) logits = at::empty({B, N, H, W}, proto.options());
        const void* in_ptrs[] = {proto.data_ptr(), coef.data_ptr(), boxes.data_ptr()};
        const int64_t ints[] = {B, H, W, N};
        const double floats[] = {thr};
        void* outs[] = {masks.data_ptr(), with_logits ? logits.data_ptr() : nullptr};
        checkRc(functs_b200_group_launch(gid, in_ptrs, ints, floats, outs, nullptr, nullptr,
                                         at::cuda::getCurrentCUDAStream().stream()),
                "yolact masks");
        if (with_logits) push(stack, logits.permute({0, 2, 3, 1}));
        push(stack, std::move(masks));
    };
}

const std::unordered_map<std::string, Adapter>& adapters() {
    static const std::unordered_map<std::string, Adapter> a{
        {"yolov3_post_dense", [](const Node* n) { return makeYolo(n, true); }},
        {"yolov3_post", [](const Node* n) { return makeYolo(n, false); }},
        {"ssd_post", [](const Node* n) { return makeSsd(n); }},
        {"lstm_seq", [](const Node* n) { return makeLstm(n); }},
        {"yolact_masks_logits", [](const Node* n) { return makeYolact(n, true); }},
        {"yolact_masks", [](const Node* n) { return makeYolact(n, false); }},
    };
    return a;
}

}  // namespace

// ---- public (fusion.h) ---------------------------------------------------------------------------------------------

bool isRegionFunctor(const Node* node) { return node->hasAttribute(kAttrRegion); }

Operation createRegionOperation(const Node* node) {
    const std::string name = node->s(kAttrRegion);
    auto it = adapters().find(name);
    TORCH_CHECK(it != adapters().end(), "tssa::ParallelFunctor: no kernel adapter named '", name, "'");
    return it->second(node);
}

void countInterpretedRun() { g_interpreted_runs.fetch_add(1, std::memory_order_relaxed); }
int64_t InterpretedFunctorRuns() { return g_interpreted_runs.load(std::memory_order_relaxed); }
void countGenericRun() { g_generic_runs.fetch_add(1, std::memory_order_relaxed); }
int64_t GenericGroupRuns() { return g_generic_runs.load(std::memory_order_relaxed); }

RegionDescription DescribeRegion(const std::shared_ptr<Graph>& graph, const std::vector<int64_t>& fwild,
                                 const std::vector<int64_t>& iwild) {
    std::vector<Node*> win = windowNodes(graph->block());
    TORCH_CHECK(!win.empty(), "DescribeRegion: the graph has no nodes");
    Described d = describeWindow(win, std::set<int>(fwild.begin(), fwild.end()), std::set<int>(iwild.begin(), iwild.end()));
    RegionDescription r;
    r.signature = d.signature;
    r.num_nodes = static_cast<int64_t>(win.size());
    r.num_inputs = static_cast<int64_t>(d.inputs.size());
    r.num_outputs = static_cast<int64_t>(d.outputs.size());
    r.fconsts = d.fconsts;
    r.iconsts = d.iconsts;
    r.num_tensors = static_cast<int64_t>(d.tconsts.size());
    return r;
}

void RegisterRegionPattern(const std::string& name, const std::shared_ptr<Graph>& graph,
                           const std::vector<std::pair<std::string, int64_t>>& froles,
                           const std::vector<std::pair<std::string, int64_t>>& iroles) {
    TORCH_CHECK(adapters().count(name), "RegisterRegionPattern: no kernel adapter named '", name, "'");
    RegionPattern p;
    p.name = name;
    for (auto& r : froles) {
        p.fwild.insert(static_cast<int>(r.second));
        p.froles.emplace_back(r.first, static_cast<int>(r.second));
    }
    for (auto& r : iroles) {
        p.iwild.insert(static_cast<int>(r.second));
        p.iroles.emplace_back(r.first, static_cast<int>(r.second));
    }
    std::vector<Node*> win = windowNodes(graph->block());
    Described d = describeWindow(win, p.fwild, p.iwild);
    p.signature = d.signature;
    p.num_nodes = static_cast<int>(win.size());
    p.num_inputs = static_cast<int>(d.inputs.size());
    p.num_outputs = static_cast<int>(d.outputs.size());
    p.num_tensors = static_cast<int>(d.tconsts.size());
    std::lock_guard<std::mutex> lock(g_patterns_mutex);
    for (RegionPattern& q : patterns()) {
        if (q.signature == p.signature) {
            q = p;  // registering the same program again replaces the entry
            return;
        }
    }
    patterns().push_back(std::move(p));
}

int64_t RegionPatternCount() {
    std::lock_guard<std::mutex> lock(g_patterns_mutex);
    return static_cast<int64_t>(patterns().size());
}

bool MatchPrecompiledRegions(const std::shared_ptr<Graph>& graph) { return matchBlock(graph->block()); }

std::string RegionSignature(const Node* functor) {
    TORCH_CHECK(functor->kind() == kParallelFunctorSym, "RegionSignature: not a tssa::ParallelFunctor node");
    return functor->hasAttribute(kAttrRegion) ? functor->s(kAttrRegion) : std::string();
}

}  // namespace functs_b200
