// TensorSSA functionalization passes (see tensorssa.cpp).  Names follow the reference's pass API
// (functs/csrc/jit/passes/convert_to_tensorssa.h:31-36).
#pragma once

#include <torch/csrc/jit/ir/ir.h>

#include <memory>
#include <unordered_map>
#include <vector>

namespace functs_b200 {

// Mutated values and, per value, the tssa::update markers that announce a new version of it
// (reference: TensorSSAMutateInfo, convert_to_tensorssa.h:12-30).
struct MutateInfo {
    std::vector<torch::jit::Value*> mutValues;
    std::unordered_map<torch::jit::Value*, std::vector<torch::jit::Node*>> mutNodes;
    void add(torch::jit::Node* update);
};

// x.op_(args) -> t = x.op(args); x.copy_(t)   for every in-place operator that has an out-of-place twin
void RemoveInplace(const std::shared_ptr<torch::jit::Graph>& graph);
// clone every tensor input at the top of the graph, so that the program only mutates memory it owns
void DumbRemoveInterPrecedureMutation(const std::shared_ptr<torch::jit::Graph>& graph);
// views -> immut:: access ops, copy_ -> immut::assign, every mutation rewritten by pass-up / pass-down, with
// tssa::update(new, old) markers
void TensorSSARewriteMutation(const std::shared_ptr<torch::jit::Graph>& graph, MutateInfo& info);
// add the mutated values as block parameters / returns of the Loop and If nodes between definition and mutation
void TensorSSAPropagation(const std::shared_ptr<torch::jit::Graph>& graph, MutateInfo& info);
// at every tssa::update(new, old): uses of `old` after the marker become `new`
void TensorSSARename(const std::shared_ptr<torch::jit::Graph>& graph);
// drop the markers; immut::assign(self, src) -> src
void TensorSSARemoveUpdate(const std::shared_ptr<torch::jit::Graph>& graph);
// RewriteMutation + Propagation + Rename
void ConvertToTensorSSA(const std::shared_ptr<torch::jit::Graph>& graph);

}  // namespace functs_b200
