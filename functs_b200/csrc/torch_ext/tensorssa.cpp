// TensorSSA functionalization for TorchScript graphs on torch 2.11: rewrite-mutation (pass-up / pass-down),
// block propagation, rename, remove-update.
//
// What the passes do follows the reference (functs/csrc/jit/passes/convert_to_tensorssa.cpp:105-481,
// functs/csrc/jit/passes/remove_inplace.cpp:20-73); how they find views does not: the reference forks PyTorch's
// AliasDb to read its private element map (functs/csrc/jit/ir/alias_analysis.h), which no longer builds against
// current PyTorch, so this file tracks views itself.  A tensor is TRACKED when its storage provably starts inside the
// graph (the output of an operator whose schema returns a fresh tensor) or when it is a supported view
// (select / slice / squeeze.dim / unsqueeze / permute / view — the aliasing ops whose write-back is well posed) of a
// tracked tensor.  A storage tree is
// dropped (left un-functionalized) as soon as one of its members is aliased in a way the passes do not model:
// an unsupported aliasing or mutating operator, a loop-carried or block-returned tensor, a container that is not
// only read.  This is the same conservative rule the reference applies to "ambiguous" aliases
// (convert_to_tensorssa.cpp:27-78): graph inputs, Loop/If outputs and containers are never functionalized.
#include "tensorssa.h"

#include <torch/csrc/jit/ir/ir.h>
#include <torch/csrc/jit/runtime/operator.h>

#include <algorithm>
#include <deque>
#include <functional>
#include <unordered_map>
#include <unordered_set>

namespace functs_b200 {

using namespace torch::jit;
using c10::Symbol;

namespace sym {
const Symbol update = Symbol::fromQualString("tssa::update");
const Symbol assign = Symbol::fromQualString("immut::assign");
const Symbol index = Symbol::fromQualString("immut::index");
const Symbol select_rev = Symbol::fromQualString("immut::select_rev");
const Symbol slice_rev = Symbol::fromQualString("immut::slice_rev");
}  // namespace sym

namespace {

struct ViewKind {
    Symbol aten, immut;
};

// aten view op -> immut access op.  expand / expand_as / reshape are not here: writing through them is ill posed
// (overlapping destinations) or may not alias at all, so a tree that uses them is left alone.
const std::vector<ViewKind>& view_kinds() {
    static const std::vector<ViewKind> kinds = {
        {aten::select, Symbol::fromQualString("immut::select")},
        {aten::slice, Symbol::fromQualString("immut::slice")},
        {aten::squeeze, Symbol::fromQualString("immut::squeeze")},
        {aten::unsqueeze, Symbol::fromQualString("immut::unsqueeze")},
        {aten::permute, Symbol::fromQualString("immut::permute")},
        {aten::view, Symbol::fromQualString("immut::view")},
    };
    return kinds;
}

const ViewKind* view_kind_of_aten(Symbol s) {
    for (auto& k : view_kinds())
        if (k.aten == s) return &k;
    return nullptr;
}
const ViewKind* view_kind_of_immut(Symbol s) {
    for (auto& k : view_kinds())
        if (k.immut == s) return &k;
    return nullptr;
}

bool is_tensor(const Value* v) { return v->type()->cast<c10::TensorType>() != nullptr; }

// true when the node is one of the tracked view ops in its tensor form (select.int, slice.Tensor, squeeze.dim ...)
bool is_supported_view(const Node* n) {
    if (view_kind_of_aten(n->kind()) == nullptr && view_kind_of_immut(n->kind()) == nullptr) return false;
    if (n->outputs().size() != 1 || n->inputs().empty() || !is_tensor(n->input(0)) || !is_tensor(n->output(0))) return false;
    if (n->kind() == aten::squeeze && n->inputs().size() != 2) return false;  // only squeeze.dim has a well-defined reverse
    return true;
}

void for_each_node(Block* b, const std::function<void(Node*)>& fn) {
    for (auto it = b->nodes().begin(); it != b->nodes().end();) {
        Node* n = *it;
        ++it;  // fn may destroy n
        for (Block* sub : n->blocks()) for_each_node(sub, fn);
        fn(n);
    }
}

// ---- view forest ------------------------------------------------------------------------------------------
class ViewForest {
  public:
    explicit ViewForest(Graph& g) { build(g); }

    bool tracked(const Value* v) const {
        auto it = info_.find(v);
        return it != info_.end() && !poisoned_.count(root_of(v));
    }
    Value* base_of(const Value* v) const { return info_.at(v).base; }
    const std::vector<Value*>& views_of(const Value* v) const { return info_.at(v).views; }
    bool is_write(const Node* n) const { return writes_.count(n) != 0 && tracked(n->input(0)); }

    // the immut:: twin of a view takes the place of the aten node
    void rename(Value* from, Value* to) {
        auto node = info_.extract(from);
        if (node.empty()) return;
        node.key() = to;
        Value* base = node.mapped().base;
        for (Value* v : node.mapped().views) info_.at(v).base = to;
        info_.insert(std::move(node));
        if (base != nullptr) {
            auto& sib = info_.at(base).views;
            std::replace(sib.begin(), sib.end(), from, to);
        }
        if (poisoned_.erase(from)) poisoned_.insert(to);
    }
    void rename_write(const Node* from, const Node* to) {
        if (writes_.erase(from)) writes_.insert(to);
    }

  private:
    struct Info {
        Value* base = nullptr;
        std::vector<Value*> views;
    };
    std::unordered_map<const Value*, Info> info_;
    std::unordered_set<const Value*> poisoned_;  // roots whose tree must be left alone
    std::unordered_set<const Node*> writes_;     // aten::copy_ nodes whose destination is in the forest

    const Value* root_of(const Value* v) const {
        const Value* r = v;
        while (true) {
            auto it = info_.find(r);
            if (it == info_.end() || it->second.base == nullptr) return r;
            r = it->second.base;
        }
    }
    void poison(const Value* v) {
        if (info_.count(v)) poisoned_.insert(root_of(v));
    }

    // Does output `out_idx` of a node with a schema own fresh storage?
    static bool returns_fresh_tensor(const Node* n, size_t out_idx) {
        const auto* schema = n->maybeSchema();
        if (schema == nullptr) return false;
        if (out_idx >= schema->returns().size()) return false;
        return schema->returns()[out_idx].alias_info() == nullptr;
    }

    void build(Graph& g) {
        // pass 1: membership (program order guarantees bases are seen before their views)
        for_each_node(g.block(), [&](Node* n) {
            if (is_supported_view(n) && info_.count(n->input(0))) {
                info_[n->output(0)].base = n->input(0);
                info_[n->input(0)].views.push_back(n->output(0));
                return;
            }
            if (n->kind() == prim::Constant || n->kind() == prim::Loop || n->kind() == prim::If) return;
            for (size_t i = 0; i < n->outputs().size(); ++i) {
                if (is_tensor(n->output(i)) && returns_fresh_tensor(n, i)) info_[n->output(i)];
            }
        });
        // pass 2: uses that the passes do not model poison the whole storage tree
        for_each_node(g.block(), [&](Node* n) {
            if (n->kind() == prim::Loop) {
                for (size_t i = 2; i < n->inputs().size(); ++i) poison(n->input(i));  // loop-carried: aliases a block param
            }
            for (Block* sub : n->blocks())
                for (Value* out : sub->outputs()) poison(out);  // escapes through a block return
            if (n->kind() == prim::ListConstruct || n->kind() == prim::TupleConstruct || n->kind() == prim::DictConstruct) {
                if (!container_only_read(n->output(0)))
                    for (Value* in : n->inputs()) poison(in);
                return;
            }
            const auto* schema = n->maybeSchema();
            if (schema == nullptr) {
                // structural nodes read their inputs; anything else without a schema is unknown
                const bool structural = n->kind() == prim::Loop || n->kind() == prim::If || n->kind() == prim::Return ||
                                        n->kind() == prim::Constant || n->kind() == sym::update;
                if (!structural)
                    for (Value* in : n->inputs()) poison(in);
                return;
            }
            for (size_t i = 0; i < n->inputs().size() && i < schema->arguments().size(); ++i) {
                Value* in = n->input(i);
                if (!info_.count(in)) continue;
                const auto* alias = schema->arguments()[i].alias_info();
                if (alias == nullptr) continue;  // pure read
                if (i == 0 && is_supported_view(n)) continue;
                if (i == 0 && n->kind() == aten::copy_) {
                    writes_.insert(n);
                    continue;
                }
                poison(in);  // aliasing or mutating operator outside the supported set
            }
        });
    }

    // a freshly constructed container is harmless if every user only reads it (or it is a result of the whole graph:
    // what the caller does with returned tensors happens after the graph has run)
    static bool container_only_read(const Value* c) {
        for (const Use& u : c->uses()) {
            if (u.user->kind() == prim::Return && u.user->owningBlock() == u.user->owningGraph()->block()) continue;
            const auto* schema = u.user->maybeSchema();
            if (schema == nullptr) return false;
            if (u.offset >= schema->arguments().size()) return false;
            if (schema->arguments()[u.offset].alias_info() != nullptr) return false;
            for (const auto& r : schema->returns())
                if (r.alias_info() != nullptr) return false;
        }
        return true;
    }
};

// ---- step 0: x.op_(args) -> t = x.op(args); x.copy_(t) ------------------------------------------------------
bool writes_first_input(const Node* n) {
    const auto* schema = n->maybeSchema();
    if (schema == nullptr || schema->arguments().empty() || n->inputs().empty()) return false;
    const auto* alias = schema->arguments()[0].alias_info();
    return alias != nullptr && alias->isWrite();
}

}  // namespace

void RemoveInplace(const std::shared_ptr<Graph>& graph) {
    for_each_node(graph->block(), [&](Node* n) {
        if (!writes_first_input(n) || !is_tensor(n->input(0)) || n->outputs().size() != 1) return;
        if (n->kind() == aten::copy_) {
            n->output()->replaceAllUsesWith(n->input(0));  // copy_ returns its destination
            return;
        }
        std::string name = n->kind().toUnqualString();
        if (name.empty() || name.back() != '_') return;
        name.pop_back();
        const Symbol pure = Symbol::fromQualString(std::string(n->kind().ns().toUnqualString()) + "::" + name);
        Graph* g = n->owningGraph();
        Node* twin = g->create(pure, n->inputs(), 1);
        twin->insertBefore(n);
        if (twin->maybeSchema() == nullptr) {  // no out-of-place overload with these arguments: leave the op alone
            twin->destroy();
            return;
        }
        // squeeze_ / unsqueeze_ / transpose_ / t_ ... change the tensor's metadata, not its values: their out-of-place twin
        // returns a VIEW, and "view, then copy_ back" would be another program.  Such ops stay as they are.
        if (!twin->schema().returns().empty() && twin->schema().returns()[0].alias_info() != nullptr) {
            twin->destroy();
            return;
        }
        twin->output()->setType(n->output()->type());
        twin->setSourceRange(n->sourceRange());
        Value* non_blocking;
        {
            WithInsertPoint guard(n);
            non_blocking = g->insertConstant(false);
        }
        Node* copy = g->create(aten::copy_, {n->input(0), twin->output(), non_blocking}, 1);
        copy->output()->setType(n->input(0)->type());
        copy->setSourceRange(n->sourceRange());
        copy->insertBefore(n);
        n->output()->replaceAllUsesWith(n->input(0));
        n->destroy();
    });
}

void DumbRemoveInterPrecedureMutation(const std::shared_ptr<Graph>& graph) {
    // graph inputs are aliases the caller can see: clone every tensor input once, at the top (the reference's
    // convert_to_tensorssa.cpp:308-320; functs/jit/_script.py:97-98 calls it for add_clone=True)
    Node* first = *graph->block()->nodes().begin();
    for (Value* input : graph->inputs()) {
        if (!is_tensor(input)) continue;
        WithInsertPoint guard(first);
        Value* none = graph->insertConstant(c10::IValue());
        Node* clone = graph->create(aten::clone, {input, none}, 1);
        clone->output()->copyMetadata(input);
        clone->insertBefore(first);
        input->replaceAllUsesAfterNodeWith(clone, clone->output());
    }
}

namespace {

// ---- step 2: aten view -> immut view, aten::copy_ -> immut::assign ------------------------------------------------
void immutablize(Graph& g, ViewForest& forest) {
    for_each_node(g.block(), [&](Node* n) {
        if (n->kind() == aten::copy_ && forest.is_write(n)) {
            Node* a = g.create(sym::assign, n->inputs(), 1);
            a->output()->setType(n->input(0)->type());
            a->setSourceRange(n->sourceRange());
            a->insertAfter(n);
            n->output()->replaceAllUsesWith(n->input(0));
            forest.rename_write(n, a);
            n->destroy();
            return;
        }
        const ViewKind* k = view_kind_of_aten(n->kind());
        if (k == nullptr || !is_supported_view(n) || !forest.tracked(n->output(0))) return;
        Node* v = g.create(k->immut, n->inputs(), 1);
        v->output()->setType(n->output()->type());
        v->setSourceRange(n->sourceRange());
        v->insertAfter(n);
        n->output()->replaceAllUsesWith(v->output());
        forest.rename(n->output(), v->output());
        n->destroy();
    });
}

// ---- step 3: one mutation -> pass-up to the storage root, pass-down to every live view ------------------------------
Node* make_update(Graph& g, Value* fresh, Value* stale, Node* after, MutateInfo& info) {
    Node* u = g.create(sym::update, {fresh, stale}, 0);
    u->insertAfter(after);
    info.add(u);
    return u;
}

// The node that turns a new value `fresh` of the view produced by `access` into a new value of its base.
// Inserted after `after` (helper nodes, if any, go in between).  The argument conventions are those of the
// reference's reverse table (functs/csrc/jit/ir/symbol_ext.h:72-85): select/slice keep the view arguments with the
// new value inserted after `self`; squeeze <-> unsqueeze and permute_rev act on the new value alone; the reverse of a
// view is a view back to the base's shape.
Node* make_reverse(Graph& g, Node* access, Value* base, Value* fresh, Node* after) {
    static const Symbol k_select = Symbol::fromQualString("immut::select"), k_select_rev = Symbol::fromQualString("immut::select_rev");
    static const Symbol k_slice = Symbol::fromQualString("immut::slice"), k_slice_rev = Symbol::fromQualString("immut::slice_rev");
    static const Symbol k_squeeze = Symbol::fromQualString("immut::squeeze"), k_unsqueeze = Symbol::fromQualString("immut::unsqueeze");
    static const Symbol k_permute = Symbol::fromQualString("immut::permute"), k_permute_rev = Symbol::fromQualString("immut::permute_rev");
    static const Symbol k_view = Symbol::fromQualString("immut::view");
    const Symbol kind = access->kind();
    Node* rev = nullptr;
    if (kind == k_select || kind == k_slice) {
        rev = g.create(kind == k_select ? k_select_rev : k_slice_rev, access->inputs(), 1);
        rev->insertInput(1, fresh);
    } else if (kind == k_squeeze || kind == k_unsqueeze || kind == k_permute) {
        rev = g.create(kind == k_squeeze ? k_unsqueeze : (kind == k_unsqueeze ? k_squeeze : k_permute_rev), access->inputs(), 1);
        rev->replaceInput(0, fresh);
    } else if (kind == k_view) {
        Node* size = g.create(aten::size, {base}, 1);
        size->output()->setType(c10::ListType::ofInts());
        size->insertAfter(after);
        after = size;
        rev = g.create(k_view, {fresh, size->output()}, 1);
    } else {
        return nullptr;
    }
    rev->insertAfter(after);
    return rev;
}

void rewrite_one_mutation(Node* write, ViewForest& forest, MutateInfo& info) {
    Graph& g = *write->owningGraph();
    // immut::assign(dst, src, non_blocking): its output is the new value of dst
    Value* dst = write->input(0);
    Value* fresh = write->output(0);
    Node* tail = write;

    // pass-up: rebuild every enclosing view's base from the new value, up to the root
    Value* cur = dst;
    while (Value* base = forest.base_of(cur)) {
        Node* access = cur->node();  // immut view producing `cur` from `base`
        Node* rev = make_reverse(g, access, base, fresh, tail);
        TORCH_CHECK(rev != nullptr, "functs_b200: unknown view operator in pass-up: ", access->kind().toQualString());
        rev->output()->setType(base->type());
        rev->setSourceRange(write->sourceRange());
        tail = rev;
        fresh = rev->output();
        cur = base;
    }
    Value* root = cur;
    Node* root_update = make_update(g, fresh, root, tail, info);

    // pass-down: re-derive every view that exists before the write and dominates it (depth first from the root)
    struct Item {
        Value* stale;   // tracked tensor whose views are to be refreshed
        Value* fresh;   // its new value
        Node* update;   // update marker after which the children's markers go
    };
    std::deque<Item> work{{root, fresh, root_update}};
    while (!work.empty()) {
        Item it = work.back();
        work.pop_back();
        for (Value* view : forest.views_of(it.stale)) {
            Node* access = view->node();
            if (!(access->isBefore(write) && write->isDominatedBy(access))) continue;
            Node* again = g.create(access->kind(), access->inputs(), 1);
            again->replaceInput(0, it.fresh);
            again->output()->copyMetadata(view);
            again->setSourceRange(write->sourceRange());
            again->insertAfter(it.fresh->node());
            Node* u = make_update(g, again->output(), view, it.update, info);
            work.push_back({view, again->output(), u});
        }
    }
}

void rewrite_mutations(Graph& g, ViewForest& forest, MutateInfo& info) {
    std::vector<Node*> writes;
    for_each_node(g.block(), [&](Node* n) {
        if (n->kind() == sym::assign && forest.is_write(n)) writes.push_back(n);
    });
    for (Node* w : writes) rewrite_one_mutation(w, forest, info);
}

// ---- step 4: thread mutated values through the blocks between their definition and their updates ---------------------
void add_mutated_to_block(Value* mutated, Block* block, std::unordered_set<Block*>& seen, bool add_node_output) {
    if (!seen.insert(block).second) return;
    Node* owner = block->owningNode();
    Graph& g = *owner->owningGraph();
    block->insertOutput(block->outputs().size(), mutated);
    if (add_node_output) {
        Value* out = owner->addOutput();
        out->setType(mutated->type());
        g.create(sym::update, {out, mutated}, 0)->insertAfter(owner);
    }
    if (owner->kind() == prim::Loop) {
        Value* param = block->addInput();
        param->setType(mutated->type());
        g.create(sym::update, {param, mutated}, 0)->insertBefore(*block->nodes().begin());
        owner->addInput(mutated);
    } else if (owner->kind() == prim::If) {
        Block* other = owner->blocks()[block == owner->blocks()[0] ? 1 : 0];
        add_mutated_to_block(mutated, other, seen, false);
    }
}

void rename_in(Block* block) {
    for (Node* n : block->nodes()) {
        if (n->kind() == sym::update) n->input(1)->replaceAllUsesAfterNodeWith(n, n->input(0));
        for (Block* sub : n->blocks()) rename_in(sub);
    }
}

}  // namespace

void MutateInfo::add(Node* update) {
    Value* mutated = update->input(1);
    if (!mutNodes.count(mutated)) mutValues.push_back(mutated);
    mutNodes[mutated].push_back(update);
}

void TensorSSARewriteMutation(const std::shared_ptr<Graph>& graph, MutateInfo& info) {
    RemoveInplace(graph);
    ViewForest forest(*graph);
    immutablize(*graph, forest);
    rewrite_mutations(*graph, forest, info);
}

void TensorSSAPropagation(const std::shared_ptr<Graph>& graph, MutateInfo& info) {
    (void)graph;
    for (Value* mutated : info.mutValues) {
        Block* def_block = mutated->node()->owningBlock();
        std::unordered_set<Block*> seen;
        // copy: add_mutated_to_block appends to nothing we iterate, but keep the list stable anyway
        const std::vector<Node*> updates = info.mutNodes[mutated];
        for (Node* u : updates)
            for (Block* b = u->owningBlock(); b != def_block; b = b->owningNode()->owningBlock())
                add_mutated_to_block(mutated, b, seen, true);
    }
}

void TensorSSARename(const std::shared_ptr<Graph>& graph) { rename_in(graph->block()); }

void TensorSSARemoveUpdate(const std::shared_ptr<Graph>& graph) {
    for_each_node(graph->block(), [&](Node* n) {
        if (n->kind() == sym::update) {
            n->destroy();
        } else if (n->kind() == sym::assign) {
            // assign(self, src) stands for "self now holds src".  Where the result only feeds the src operand of
            // select_rev / slice_rev, those ops broadcast and cast src to their destination themselves, so src can take its
            // place.  Anywhere else (a write to a whole tensor: x.copy_(row), or through a squeeze / permute / view) the
            // value must have self's shape and dtype: src is used as it is only when both static types are known and
            // equal, otherwise a cast and an expand_as are inserted (copy_ broadcasts and converts, so must this).
            Value* self = n->input(0);
            Value* src = n->input(1);
            bool only_rev_src = true;
            for (const Use& u : n->output()->uses()) {
                const bool rev = u.user->kind() == sym::select_rev || u.user->kind() == sym::slice_rev;
                only_rev_src = only_rev_src && rev && u.offset == 1;
            }
            bool same = only_rev_src;
            if (!same) {
                auto ts = self->type()->cast<c10::TensorType>(), td = src->type()->cast<c10::TensorType>();
                same = ts && td && ts->scalarType() && td->scalarType() && *ts->scalarType() == *td->scalarType() &&
                       ts->sizes().concrete_sizes() && td->sizes().concrete_sizes() &&
                       *ts->sizes().concrete_sizes() == *td->sizes().concrete_sizes();
            }
            Value* repl = src;
            if (!same) {
                Graph* g = n->owningGraph();
                WithInsertPoint guard(n);
                Value* f = g->insertConstant(false);
                Value* none = g->insertConstant(c10::IValue());
                Node* to = g->insertNode(g->create(aten::to, {src, self, f, f, none}, 1));
                to->output()->setType(c10::TensorType::get());
                Node* ex = g->insertNode(g->create(aten::expand_as, {to->output(), self}, 1));
                ex->output()->setType(self->type());
                repl = ex->output();
            }
            n->output()->replaceAllUsesWith(repl);
            n->destroy();
        }
    });
}

void ConvertToTensorSSA(const std::shared_ptr<Graph>& graph) {
    MutateInfo info;
    TensorSSARewriteMutation(graph, info);
    TensorSSAPropagation(graph, info);
    TensorSSARename(graph);
}

}  // namespace functs_b200
