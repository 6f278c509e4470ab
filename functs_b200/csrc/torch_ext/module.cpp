// Python module functs_b200._C: the pass entry points under the names the reference binds
// (functs/csrc/jit/python/init.cpp:31-76).  Graphs are mutated in place; every function returns None.
#include <torch/csrc/jit/python/pybind_utils.h>
#include <torch/extension.h>

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
}
