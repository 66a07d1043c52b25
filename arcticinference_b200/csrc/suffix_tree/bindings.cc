// pybind11 module `arcticinference_b200.suffix_decoding._C`: SuffixTree and Draft with the
// method names of the reference's nanobind module (csrc/suffix_decoding/bindings.cc:79-103):
// extend / extend_ndarray / speculate / speculate_ndarray / remove / num_seqs /
// check_integrity / estimate_memory. The *_ndarray overloads read int32 numpy arrays in place.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "suffix_tree.h"

namespace py = pybind11;
using ab200::Draft;
using ab200::SuffixTree;

using I32Array = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;

PYBIND11_MODULE(_C, m) {
  m.doc() = "Host-side suffix tree for suffix decoding";

  py::class_<Draft>(m, "Draft")
      .def(py::init<>())
      .def_readwrite("token_ids", &Draft::token_ids)
      .def_readwrite("parents", &Draft::parents)
      .def_readwrite("probs", &Draft::probs)
      .def_readwrite("score", &Draft::score)
      .def_readwrite("match_len", &Draft::match_len);

  py::class_<SuffixTree>(m, "SuffixTree")
      .def(py::init<int32_t>(), py::arg("max_depth"))
      .def("num_seqs", &SuffixTree::num_seqs)
      .def("num_nodes", &SuffixTree::num_nodes)
      .def("max_depth", &SuffixTree::max_depth)
      .def("contains", &SuffixTree::contains)
      .def("append", &SuffixTree::append, py::arg("seq_id"), py::arg("token"))
      .def("extend",
           [](SuffixTree& t, int32_t seq_id, const std::vector<int32_t>& tokens) {
             t.extend(seq_id, tokens.data(), tokens.size());
           },
           py::arg("seq_id"), py::arg("tokens"))
      .def("extend_ndarray",
           [](SuffixTree& t, int32_t seq_id, I32Array tokens) {
             t.extend(seq_id, tokens.data(), (size_t)tokens.size());
           },
           py::arg("seq_id"), py::arg("tokens"))
      .def("remove", &SuffixTree::remove, py::arg("seq_id"))
      .def("speculate",
           [](const SuffixTree& t, const std::vector<int32_t>& context, int32_t max_spec_tokens,
              float max_spec_factor, float max_spec_offset, float min_token_prob,
              bool use_tree_spec) {
             return t.speculate(context.data(), context.size(), max_spec_tokens, max_spec_factor,
                                max_spec_offset, min_token_prob, use_tree_spec);
           },
           py::arg("context"), py::arg("max_spec_tokens"), py::arg("max_spec_factor") = 1.0f,
           py::arg("max_spec_offset") = 0.0f, py::arg("min_token_prob") = 0.1f,
           py::arg("use_tree_spec") = false)
      .def("speculate_ndarray",
           [](const SuffixTree& t, I32Array context, int32_t max_spec_tokens, float max_spec_factor,
              float max_spec_offset, float min_token_prob, bool use_tree_spec) {
             py::gil_scoped_release nogil;
             return t.speculate(context.data(), (size_t)context.size(), max_spec_tokens,
                                max_spec_factor, max_spec_offset, min_token_prob, use_tree_spec);
           },
           py::arg("context"), py::arg("max_spec_tokens"), py::arg("max_spec_factor") = 1.0f,
           py::arg("max_spec_offset") = 0.0f, py::arg("min_token_prob") = 0.1f,
           py::arg("use_tree_spec") = false)
      .def("check_integrity", &SuffixTree::check_integrity)
      .def("estimate_memory", &SuffixTree::estimate_memory);
}
