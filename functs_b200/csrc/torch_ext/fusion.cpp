// Loop parallelization, op grouping and the tssa::ParallelFunctor operator.
//
// Behaviour follows the reference's passes (fait/passes/parallelize_loops.cpp:12-145 for the loop test and the map
// form, fait/passes/fuse_ops.cpp:209-527 for what may be grouped, fait/passes/te_op.cpp:34-236 for the functor node and
// its attributes); the implementation is independent of them: groups are contiguous runs (nothing is reordered), and
// the functor operator runs a subgraph through a GraphExecutor unless a precompiled kernel is known for it.
#include "fusion.h"

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/jit/ir/constants.h>
#include <torch/csrc/jit/passes/common_subexpression_elimination.h>
#include <torch/csrc/jit/passes/constant_propagation.h>
#include <torch/csrc/jit/passes/dead_code_elimination.h>
#include <torch/csrc/jit/runtime/custom_operator.h>
#include <torch/csrc/jit/runtime/graph_executor.h>
#include <torch/csrc/jit/runtime/operator.h>

#include <cstdlib>
#include <fstream>
#include <atomic>
#include <functional>
#include <mutex>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

#include "../../../include/functs_b200.h"
#include "tensorssa.h"

namespace functs_b200 {

using namespace torch::jit;

namespace {

const Symbol kParallelMap = Symbol::fromQualString("tssa::ParallelMap");
const Symbol kParallelFunctor = Symbol::fromQualString("tssa::ParallelFunctor");
const Symbol kAttrDegree = Symbol::attr("parallel_degree");
const Symbol kAttrIsMap = Symbol::attr("is_parallel_map");
const Symbol kAttrParArgs = Symbol::attr("is_parallel_args");
const Symbol kAttrRefineTypes = Symbol::attr("input_refine_types");
const Symbol kAttrSignature = Symbol::attr("kernel_signature");

bool isInside(const Value* v, const Block* block) {
    for (const Block* b = v->node()->owningBlock(); b != nullptr;
         b = b->owningNode() ? b->owningNode()->owningBlock() : nullptr) {
        if (b == block) return true;
    }
    return false;
}

bool nodeInside(const Node* n, const Block* block) {
    for (const Block* b = n->owningBlock(); b != nullptr; b = b->owningNode() ? b->owningNode()->owningBlock() : nullptr) {
        if (b == block) return true;
    }
    return false;
}

bool isConstTrue(const Value* v) {
    auto iv = toIValue(v);
    return iv && iv->isBool() && iv->toBool();
}

void forEachNode(Block* block, const std::function<void(Node*)>& fn) {
    for (auto it = block->nodes().begin(); it != block->nodes().end();) {
        Node* n = *it;
        ++it;  // fn may destroy n
        for (Block* b : n->blocks()) forEachNode(b, fn);
        fn(n);
    }
}

// ---- ParallelizeLoops -----------------------------------------------------------------------------------------

struct LoopLists {
    std::vector<Node*> reads;    // top-level list[iter] reads of outer lists
    std::vector<Node*> appends;  // top-level appends to outer lists
};

// A loop may become a map when iterations cannot see one another: no carried values, constant-true conditions, outer
// lists only read by list[i] / list[const] / len(list) or extended by exactly one top-level append, appended lists born
// empty right in the loop's block and untouched before the loop ends, and no other side effect anywhere in the body.
bool loopIsParallel(Node* loop, LoopLists& lists) {
    if (loop->inputs().size() != 2 || !isConstTrue(loop->input(1))) return false;
    Block* body = loop->blocks()[0];
    if (body->outputs().size() != 1 || !isConstTrue(body->outputs()[0])) return false;
    Value* iter = body->inputs()[0];
    std::unordered_map<Value*, int> append_count;
    bool ok = true;
    std::function<void(Block*, bool)> visit = [&](Block* b, bool top) {
        for (Node* n : b->nodes()) {
            const bool is_append = n->kind() == aten::append;
            if (!is_append && n->kind() != prim::Loop && n->kind() != prim::If && n->hasSideEffects()) ok = false;
            if (const auto* schema = n->maybeSchema()) {
                if (!is_append && schema->is_mutable()) ok = false;  // a functionalized body has no such node left
            }
            for (size_t k = 0; k < n->inputs().size(); ++k) {
                Value* in = n->input(k);
                if (!in->type()->cast<c10::ListType>() || isInside(in, body)) continue;
                if (n->kind() == aten::__getitem__ && k == 0) {
                    Value* idx = n->input(1);
                    if (idx == iter) {
                        if (top) lists.reads.push_back(n);
                    } else if (idx->node()->kind() != prim::Constant) {
                        ok = false;
                    }
                } else if (is_append && k == 0 && top) {
                    append_count[in]++;
                    lists.appends.push_back(n);
                } else if (n->kind() == aten::len) {
                    // reading the length is harmless for a list that is not appended to (checked below)
                } else {
                    ok = false;
                }
            }
            for (Block* nb : n->blocks()) visit(nb, false);
        }
    };
    visit(body, true);
    if (!ok) return false;
    for (auto& kv : append_count) {
        Value* list = kv.first;
        if (kv.second != 1) return false;
        Node* def = list->node();
        if (def->kind() != prim::ListConstruct || !def->inputs().empty() || def->owningBlock() != loop->owningBlock())
            return false;
        for (const Use& u : list->uses()) {
            if (nodeInside(u.user, body)) {
                if (u.user->kind() != aten::append) return false;  // read of a list that the loop is filling
            } else if (u.user->owningBlock() != loop->owningBlock() || !u.user->isAfter(loop)) {
                return false;  // touched before the loop, or from another block
            }
        }
    }
    return true;
}

void convertLoopToMap(Node* loop, const LoopLists& lists) {
    Graph* g = loop->owningGraph();
    Block* body = loop->blocks()[0];
    std::vector<Value*> in_lists, out_lists;
    for (Node* r : lists.reads) in_lists.push_back(r->input(0));
    for (Node* a : lists.appends) out_lists.push_back(a->input(0));

    std::vector<Value*> args{loop->input(0)};
    args.insert(args.end(), in_lists.begin(), in_lists.end());
    Node* map = g->create(kParallelMap, args, out_lists.size());
    map->setSourceRange(loop->sourceRange());
    map->insertBefore(loop);
    Block* mb = map->addBlock();
    std::unordered_map<Value*, Value*> vmap;
    Value* idx = mb->addInput();
    idx->setType(c10::IntType::get());
    vmap[body->inputs()[0]] = idx;
    for (Node* r : lists.reads) {
        Value* p = mb->addInput();
        p->setType(r->output()->type());
        vmap[r->output()] = p;
    }
    auto lookup = [&](Value* v) -> Value* {
        auto it = vmap.find(v);
        return it == vmap.end() ? v : it->second;
    };
    std::unordered_set<Node*> skip(lists.reads.begin(), lists.reads.end());
    std::unordered_map<Node*, size_t> append_slot;
    for (size_t i = 0; i < lists.appends.size(); ++i) append_slot[lists.appends[i]] = i;
    std::vector<Value*> results(lists.appends.size(), nullptr);
    for (Node* n : body->nodes()) {
        if (skip.count(n)) continue;
        auto ap = append_slot.find(n);
        if (ap != append_slot.end()) {
            results[ap->second] = lookup(n->input(1));
            continue;
        }
        Node* c = g->createClone(n, lookup);
        mb->appendNode(c);
        for (size_t k = 0; k < n->outputs().size(); ++k) vmap[n->output(k)] = c->output(k);
    }
    for (Value* r : results) mb->registerOutput(r);
    for (size_t i = 0; i < out_lists.size(); ++i) {
        map->output(i)->setType(out_lists[i]->type());
        out_lists[i]->replaceAllUsesAfterNodeWith(loop, map->output(i));
    }
    loop->destroy();
    for (Value* l : out_lists) {
        if (!l->hasUses()) l->node()->destroy();
    }
}

// The inverse, for maps that did not end up as one fused group: a plain loop with list reads and appends.
void convertMapToLoop(Node* map) {
    Graph* g = map->owningGraph();
    WithInsertPoint guard(map);
    Block* mb = map->blocks()[0];
    std::vector<Value*> out_lists;
    for (Value* o : map->outputs()) {
        Node* lc = g->insertNode(g->createList(o->type()->expect<c10::ListType>()->getElementType(), {}));
        out_lists.push_back(lc->output());
    }
    Value* true_v = g->insertConstant(true);
    Node* loop = g->insertNode(g->create(prim::Loop, {map->input(0), true_v}, 0));
    loop->setSourceRange(map->sourceRange());
    Block* body = loop->addBlock();
    Value* iter = body->addInput();
    iter->setType(c10::IntType::get());
    std::unordered_map<Value*, Value*> vmap;
    vmap[mb->inputs()[0]] = iter;
    {
        WithInsertPoint in_body(body);
        for (size_t k = 1; k < mb->inputs().size(); ++k) {
            Node* get = g->insertNode(g->create(aten::__getitem__, {map->input(k), iter}, 1));
            get->output()->setType(mb->inputs()[k]->type());
            vmap[mb->inputs()[k]] = get->output();
        }
        auto lookup = [&](Value* v) -> Value* {
            auto it = vmap.find(v);
            return it == vmap.end() ? v : it->second;
        };
        for (Node* n : mb->nodes()) {
            Node* c = g->insertNode(g->createClone(n, lookup));
            for (size_t k = 0; k < n->outputs().size(); ++k) vmap[n->output(k)] = c->output(k);
        }
        for (size_t i = 0; i < out_lists.size(); ++i) {
            Node* ap = g->insertNode(g->create(aten::append, {out_lists[i], lookup(mb->outputs()[i])}, 1));
            ap->output()->setType(out_lists[i]->type());
        }
        body->registerOutput(g->insertConstant(true));
    }
    for (size_t i = 0; i < out_lists.size(); ++i) map->output(i)->replaceAllUsesWith(out_lists[i]);
    map->destroy();
}

}  // namespace

void ParallelizeLoops(const std::shared_ptr<Graph>& graph) {
    std::vector<Node*> loops;
    forEachNode(graph->block(), [&](Node* n) {
        if (n->kind() == prim::Loop) loops.push_back(n);  // inner loops first
    });
    for (Node* loop : loops) {
        LoopLists lists;
        if (loopIsParallel(loop, lists) && !lists.appends.empty()) convertLoopToMap(loop, lists);
    }
}

// the rest of the file: FuseOps, LowerToParallelFunctors, the operator
#include "fusion_groups.inc"

}  // namespace functs_b200
