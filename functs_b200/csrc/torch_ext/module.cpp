// Python module functs_b200._C: the pass entry points under the names the reference binds
// (functs/csrc/jit/python/init.cpp:31-76).  Graphs are mutated in place; every function returns None.
#include <torch/csrc/jit/python/pybind_utils.h>
#include <torch/extension.h>

#include <torch/csrc/jit/api/compilation_unit.h>
#include <torch/csrc/jit/api/module.h>
#include <torch/csrc/jit/passes/freeze_module.h>
#include <torch/csrc/jit/passes/shape_analysis.h>

#include "fusion.h"
#include "tensorssa.h"

namespace py = pybind11;
using torch::jit::Graph;

PYBIND11_MODULE(_C, m) {
    m.doc() = "functs_b200: TensorSSA functionalization passes + immut:: operator registrations (loaded as a side effect)";
    py::class_<functs_b200::MutateInfo, std::shared_ptr<functs_b200::MutateInfo>>(m, "TensorSSAMutateInfo")
        .def(py::init<>())
        .def_property_readonly("mutValues", [](functs_b200::MutateInfo& self) { return self.mutValues; })
        .def_property_readonly("mutNodes", [](functs_b200::MutateInfo& self) { return self.mutNodes; });
    m.def("_jit_pass_remove_inplace", [](std::shared_ptr<Graph> g) { functs_b200::RemoveInplace(g); });
    m.def("_jit_pass_dumb_remove_inter_precedure_mutation",
          [](std::shared_ptr<Graph> g) { functs_b200::DumbRemoveInterPrecedureMutation(g); });
    m.def("_jit_pass_convert_to_tensorssa", [](std::shared_ptr<Graph> g) { functs_b200::ConvertToTensorSSA(g); });
    m.def("_jit_pass_tensorssa_remove_update", [](std::shared_ptr<Graph> g) { functs_b200::TensorSSARemoveUpdate(g); });
    m.def("_jit_pass_rewrite_mutation", [](std::shared_ptr<Graph> g, std::shared_ptr<functs_b200::MutateInfo> info) {
        functs_b200::TensorSSARewriteMutation(g, *info);
    });
    m.def("_jit_pass_block_propagation", [](std::shared_ptr<Graph> g, std::shared_ptr<functs_b200::MutateInfo> info) {
        functs_b200::TensorSSAPropagation(g, *info);
    });
    m.def("_jit_pass_rename", [](std::shared_ptr<Graph> g) { functs_b200::TensorSSARename(g); });
    // loop parallelization, grouping, functor lowering (reference: fait passes behind _jit_pass_fait_pipeline)
    m.def("_jit_pass_parallelize_loops", [](std::shared_ptr<Graph> g) { functs_b200::ParallelizeLoops(g); });
    m.def("_jit_pass_fait_fuse_ops", [](std::shared_ptr<Graph> g, py::object /*refined_types*/) { functs_b200::FuseOps(g); },
          py::arg("graph"), py::arg("refined_types") = py::none());
    // the reference's grouper for graphs that did not go through the ParallelMap pipeline (functs.jit.script(backend="jit"),
    // functs/csrc/jit/python/init.cpp:40-42 -> FuncTsFuseTensorExprs): here the same entry point groups the fusable ops of a
    // functionalized graph and lowers the groups to tssa::ParallelFunctor nodes, which run as one launch each
    m.def("_jit_pass_fuse_tensorexpr", [](std::shared_ptr<Graph> g) {
        functs_b200::FuseOps(g);
        functs_b200::LowerToParallelFunctors(g);
    });
    m.def("_jit_pass_match_precompiled_loops", [](std::shared_ptr<Graph> g) { functs_b200::MatchPrecompiledLoops(g); });
    m.def("_jit_pass_unroll_loops_with_deps", [](std::shared_ptr<Graph> g) { functs_b200::UnrollLoopsWithDeps(g); });
    m.def("_jit_pass_split_parallel_maps", [](std::shared_ptr<Graph> g) { functs_b200::SplitParallelMaps(g); });
    m.def("_jit_pass_unroll_simple_maps", [](std::shared_ptr<Graph> g) { functs_b200::UnrollSimpleMaps(g); });
    m.def("_jit_pass_lower_to_parallel_functors", [](std::shared_ptr<Graph> g) { functs_b200::LowerToParallelFunctors(g); });
    m.def("_jit_pass_fait_pipeline",
          [](std::shared_ptr<Graph> g, std::vector<c10::TypePtr> type_hint) {
              // the type hints refine the graph inputs (shapes / dtypes), as the reference's pipeline does first
              for (size_t i = 0; i < type_hint.size() && i < g->inputs().size(); ++i) {
                  // (a tuple hint describes the elements of a list input; the list type itself cannot carry it)
                  if (type_hint[i] && !(type_hint[i]->cast<c10::TupleType>() && g->inputs()[i]->type()->cast<c10::ListType>()))
                      g->inputs()[i]->setType(type_hint[i]);
              }
              functs_b200::FaitPipeline(g);
          },
          py::arg("graph"), py::arg("type_hint") = std::vector<c10::TypePtr>());
    m.def("_jit_pass_fait_shape_infer",
          [](std::shared_ptr<Graph> g, std::vector<c10::TypePtr> type_hint, py::object refined_types) {
              // refined_types (a dict, as in the reference's binding): filled with value -> tuple type of every list of
              // tensors whose elements' types are known; the same pairs are returned keyed by the values' debug names
              auto pairs = functs_b200::InferShapesRefined(g, type_hint);
              py::dict by_name;
              for (auto& kv : pairs) {
                  by_name[py::str(kv.first->debugName())] = kv.second;
                  if (!refined_types.is_none()) refined_types[py::cast(kv.first)] = kv.second;
              }
              return by_name;
          },
          py::arg("graph"), py::arg("type_hint") = std::vector<c10::TypePtr>(), py::arg("refined_types") = py::none());
    // precompiled regions: pattern programs are registered from Python (functs_b200/patterns.py)
    m.def("_jit_pass_prepare_for_matching", [](std::shared_ptr<Graph> g) { functs_b200::PrepareForMatching(g); });
    m.def("_jit_pass_match_precompiled_regions", [](std::shared_ptr<Graph> g) { return functs_b200::MatchPrecompiledRegions(g); });
    m.def("_describe_region",
          [](std::shared_ptr<Graph> g, std::vector<int64_t> fwild, std::vector<int64_t> iwild) {
              auto d = functs_b200::DescribeRegion(g, fwild, iwild);
              py::dict out;
              out["signature"] = d.signature;
              out["num_nodes"] = d.num_nodes;
              out["num_inputs"] = d.num_inputs;
              out["num_outputs"] = d.num_outputs;
              out["num_tensors"] = d.num_tensors;
              out["fconsts"] = d.fconsts;
              out["iconsts"] = d.iconsts;
              return out;
          },
          py::arg("graph"), py::arg("fwild") = std::vector<int64_t>(), py::arg("iwild") = std::vector<int64_t>());
    m.def("_register_region_pattern",
          [](const std::string& name, std::shared_ptr<Graph> g, std::vector<std::pair<std::string, int64_t>> froles,
             std::vector<std::pair<std::string, int64_t>> iroles) { functs_b200::RegisterRegionPattern(name, g, froles, iroles); });
    m.def("_region_pattern_count", []() { return functs_b200::RegionPatternCount(); });
    m.def("_interpreted_functor_runs", []() { return functs_b200::InterpretedFunctorRuns(); });
    m.def("_generic_group_runs", []() { return functs_b200::GenericGroupRuns(); });
    m.def("_last_generic_refusal", []() { return functs_b200::LastGenericRefusal(); });
    m.def("_functor_regions", [](std::shared_ptr<Graph> g) {
        // adapter name of every tssa::ParallelFunctor node ("" = interpreted), in graph order
        std::vector<std::string> out;
        std::function<void(torch::jit::Block*)> visit = [&](torch::jit::Block* b) {
            for (torch::jit::Node* n : b->nodes()) {
                if (n->kind() == c10::Symbol::fromQualString("tssa::ParallelFunctor")) out.push_back(functs_b200::RegionSignature(n));
                for (torch::jit::Block* nb : n->blocks()) visit(nb);
            }
        };
        visit(g->block());
        return out;
    });
    m.def("_count_parallel_functors", [](std::shared_ptr<Graph> g) { return functs_b200::CountParallelFunctors(g); });
    m.def("_jit_pass_freeze", [](torch::jit::Module& module) { return torch::jit::freeze_module(module); });
    m.def("_jit_pass_clone", [](torch::jit::Module& module) { return module.clone(); });
    m.def("_create_function_from_graph", [](const std::string& qualname, std::shared_ptr<Graph> graph) {
        auto cu = std::make_shared<torch::jit::CompilationUnit>();
        auto* fn = cu->create_function(c10::QualifiedName(qualname), graph);
        return torch::jit::StrongFunctionPtr(std::move(cu), fn);
    });
}
