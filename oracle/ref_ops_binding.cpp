// Test-infrastructure binding: exposes the reference's five MoE ops, compiled unmodified from the
// reference source tree, as the Python module ``ref_ops`` so that GPU tests can compare them with
// libb200moe on the same inputs.  The declarations come from the reference's own src/include/ops.h.
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "ops.h"

PYBIND11_MODULE(ref_ops, m) {
  m.doc() = "electrock-infer reference MoE ops (oracle build)";
  m.def("silu_and_mul", &electrock_infer::silu_and_mul, pybind11::arg("out"), pybind11::arg("input"));
  m.def("topk_softmax", &electrock_infer::topk_softmax, pybind11::arg("topk_weights"),
        pybind11::arg("topk_indices"), pybind11::arg("gating_output"));
  m.def("moe_sum", &electrock_infer::moe_sum, pybind11::arg("input"), pybind11::arg("output"));
  m.def("moe_sum_efficient", &electrock_infer::moe_sum_efficient, pybind11::arg("input"),
        pybind11::arg("output"));
  m.def("moe_align_block_size", &electrock_infer::moe_align_block_size, pybind11::arg("topk_ids"),
        pybind11::arg("num_experts"), pybind11::arg("block_size"),
        pybind11::arg("sorted_token_ids"), pybind11::arg("expert_ids"),
        pybind11::arg("num_tokens_post_pad"));
}
