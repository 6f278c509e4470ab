// Loop parallelization, op grouping and the tssa::ParallelFunctor operator (see fusion.cpp).
//
// These passes play the role of the reference's fait/passes/{parallelize_loops,fuse_ops,te_op}.cpp on a graph that
// the TensorSSA passes have already made free of tensor mutation:
//   ParallelizeLoops         prim::Loop without carried values, whose outer lists are only read by list[i] and written by
//                            one append each            ->  tssa::ParallelMap(n, in lists...) -> out lists
//   FuseOps                  contiguous runs of fusable tensor ops (>= 2 working ops)  ->  prim::FusionGroup
//   LowerToParallelFunctors  map whose body is one group -> tssa::ParallelFunctor(is_parallel_map = 1);
//                            other groups -> tssa::ParallelFunctor(is_parallel_map = 0); other maps -> loops again
//   MatchPrecompiledLoops    known whole-loop patterns -> tssa::ParallelFunctor carrying a kernel signature
// tssa::ParallelFunctor is a registered JIT operator: it launches the precompiled kernel of libfuncts_b200.so when the
// node carries the signature of one, and otherwise interprets its subgraph (per parallel index) on the immut:: kernels.
#pragma once

#include <torch/csrc/jit/ir/ir.h>
#include <torch/csrc/jit/runtime/operator.h>

#include <memory>
#include <string>
#include <vector>

namespace functs_b200 {

void ParallelizeLoops(const std::shared_ptr<torch::jit::Graph>& graph);
// whole loops that a precompiled kernel of the C-ABI library covers -> tssa::ParallelFunctor carrying its signature
void MatchPrecompiledLoops(const std::shared_ptr<torch::jit::Graph>& graph);
// loops with carried values, a constant trip count (<= 16) and a small body are unrolled completely
void UnrollLoopsWithDeps(const std::shared_ptr<torch::jit::Graph>& graph);
void FuseOps(const std::shared_ptr<torch::jit::Graph>& graph);
// a map whose body is more than one fusion group -> a chain of maps, one group (or one run of other nodes) each
void SplitParallelMaps(const std::shared_ptr<torch::jit::Graph>& graph);
// maps with a constant trip count and a self-contained body, written out iteration by iteration (not in the default pipeline)
void UnrollSimpleMaps(const std::shared_ptr<torch::jit::Graph>& graph);
void LowerToParallelFunctors(const std::shared_ptr<torch::jit::Graph>& graph);
// TensorSSA conversion (+ marker removal) followed by the three passes above and dead-code elimination
void FaitPipeline(const std::shared_ptr<torch::jit::Graph>& graph);
// graph inputs take `type_hint` (null entries are skipped); shapes, dtypes and devices are then propagated through the
// aten:: operators (TorchScript's own propagation) and the immut:: family (shape_infer.cpp)
void InferShapes(const std::shared_ptr<torch::jit::Graph>& graph, const std::vector<c10::TypePtr>& type_hint);
// the same, returning the refined list types: (list value, tuple type with one tensor type per element).  A tuple hint for
// a List[Tensor] graph input describes the list's elements.
std::vector<std::pair<torch::jit::Value*, c10::TypePtr>> InferShapesRefined(const std::shared_ptr<torch::jit::Graph>& graph,
                                                                            const std::vector<c10::TypePtr>& type_hint);
// number of tssa::ParallelFunctor nodes in the graph (all blocks): the unit the launch-count metric counts
int64_t CountParallelFunctors(const std::shared_ptr<torch::jit::Graph>& graph);
// the normalisation every graph goes through before regions are matched: TensorSSA conversion, marker removal, CSE,
// constant propagation, dead-code elimination (pattern programs and user programs alike)
void PrepareForMatching(const std::shared_ptr<torch::jit::Graph>& graph);

// ---- precompiled regions (regions.cpp) --------------------------------------------------------------------------------
// Canonical description of the whole top level of `graph` (a pattern program after PrepareForMatching).  fwild / iwild:
// slots of the float / int constant lists that print as "?" instead of by value.
struct RegionDescription {
    std::string signature;
    int64_t num_nodes = 0, num_inputs = 0, num_outputs = 0, num_tensors = 0;
    std::vector<double> fconsts;
    std::vector<int64_t> iconsts;
};
RegionDescription DescribeRegion(const std::shared_ptr<torch::jit::Graph>& graph, const std::vector<int64_t>& fwild,
                                 const std::vector<int64_t>& iwild);
// `graph`: a pattern program after PrepareForMatching; `name`: the kernel adapter that runs it; froles / iroles: (attribute
// name, constant slot) of the scalar constants a matching program may choose freely
void RegisterRegionPattern(const std::string& name, const std::shared_ptr<torch::jit::Graph>& graph,
                           const std::vector<std::pair<std::string, int64_t>>& froles,
                           const std::vector<std::pair<std::string, int64_t>>& iroles);
int64_t RegionPatternCount();
// windows of top-level nodes whose canonical signature equals a registered pattern -> one tssa::ParallelFunctor each
bool MatchPrecompiledRegions(const std::shared_ptr<torch::jit::Graph>& graph);
// name of the kernel adapter a functor node is bound to ("" = none: its subgraph is interpreted)
std::string RegionSignature(const torch::jit::Node* functor);
bool isRegionFunctor(const torch::jit::Node* node);
torch::jit::Operation createRegionOperation(const torch::jit::Node* node);
// functor runs that went through the subgraph interpreter instead of a precompiled kernel, in this process
void countInterpretedRun();
int64_t InterpretedFunctorRuns();
// ---- generic group (generic_group.cpp): the subgraph of a functor as ONE launch of the program-interpreting kernel ----
// inputs: the node's inputs (lists for the parallel arguments of a map); outputs: one IValue per subgraph output (a list
// of `degree` tensors for a map).  Returns false, with the reason in *why, when the group cannot be expressed as programs.
// plan: per-functor cache of the flattened programs (opaque; created with NewGenericPlan, one per functor node).  A call
// whose inputs have the shapes, dtypes, devices and scalar values of the previous one only patches the pointers.
struct GenericPlan;
std::shared_ptr<GenericPlan> NewGenericPlan();
bool RunGenericGroup(const std::shared_ptr<torch::jit::Graph>& sub, bool is_map, int64_t degree,
                     const std::vector<int64_t>& par, const std::vector<c10::IValue>& inputs,
                     std::vector<c10::IValue>& outputs, std::string* why, GenericPlan* plan = nullptr);
void countGenericRun();
int64_t GenericGroupRuns();
std::string LastGenericRefusal();

}  // namespace functs_b200
