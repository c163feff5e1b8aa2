// pybind11 shim over the C ABI of libb200moe (include/b200moe.h): the thin Python binding the operator's host side
// uses on its hot call. Pointers cross as integers (torch's data_ptr()), nothing here owns memory or touches torch.
// Counterpart of the reference's CPython fast-call extension (candidate/nvfp4_fast.c:153-295), which exists to keep
// the per-call host cost of moe_run low.
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>

#include "../../include/b200moe.h"

namespace py = pybind11;

static void check(int code, const char* what) {
  if (code == 0) return;
  std::string msg = std::string(what) + ": " + b200moe_last_error() + " (code " + std::to_string(code) + ")";
  if (code >= 700 && code < 800) throw py::value_error(msg);
  throw std::runtime_error(msg);
}

template <class T>
static T* ptr(uintptr_t v) { return reinterpret_cast<T*>(v); }

PYBIND11_MODULE(_b200moe_shim, m) {
  m.doc() = "pybind11 binding of libb200moe's layer entry points";
  m.def("abi_version", &b200moe_abi_version);
  m.def("create", [](int hidden, int intermediate, int num_experts, int top_k, int num_shared_experts, int max_tokens, int tile_n,
                     int graph_cache) {
    b200moe_config c{};
    c.struct_size = (int32_t)sizeof(c);
    c.hidden = hidden; c.intermediate = intermediate; c.num_experts = num_experts; c.top_k = top_k;
    c.num_shared_experts = num_shared_experts; c.max_tokens = max_tokens; c.tile_n = tile_n; c.graph_cache = graph_cache;
    b200moe_handle h = nullptr;
    check(b200moe_create(&c, &h), "b200moe_create");
    return reinterpret_cast<uintptr_t>(h);
  });
  m.def("destroy", [](uintptr_t h) { check(b200moe_destroy(ptr<b200moe_layer>(h)), "b200moe_destroy"); });
  // One positional call per forward: every argument is an int (device address, 0 = null) or a small scalar.
  m.def("run", [](uintptr_t h, int num_tokens, uintptr_t ids, uintptr_t weights, uintptr_t hidden_states, uintptr_t hidden_scale,
                  int scale_layout, int activation_type, uintptr_t w1, uintptr_t s1, uintptr_t w2, uintptr_t s2, uintptr_t alpha,
                  uintptr_t beta, uintptr_t limit, uintptr_t scale_up, uintptr_t scale_gate, uintptr_t scale_out, int expert_offset,
                  int direct_rows, uintptr_t output, int64_t output_stride, uintptr_t stream, int64_t hidden_states_stride,
                  int64_t hidden_states_scale_stride, int64_t topk_stride) {
    b200moe_args a{};
    a.struct_size = (int32_t)sizeof(a);
    a.num_tokens = num_tokens;
    a.topk_ids = ptr<const int32_t>(ids);
    a.topk_weights = ptr<const float>(weights);
    a.hidden_states = ptr<const void>(hidden_states);
    a.hidden_states_scale = ptr<const void>(hidden_scale);
    a.hidden_states_scale_layout = scale_layout;
    a.activation_type = activation_type;
    a.gemm1_weights = ptr<const void>(w1);
    a.gemm1_weights_scale = ptr<const void>(s1);
    a.gemm2_weights = ptr<const void>(w2);
    a.gemm2_weights_scale = ptr<const void>(s2);
    a.gemm1_alpha = ptr<const float>(alpha);
    a.gemm1_beta = ptr<const float>(beta);
    a.gemm1_clamp_limit = ptr<const float>(limit);
    a.output1_scale_scalar = ptr<const float>(scale_up);
    a.output1_scale_gate_scalar = ptr<const float>(scale_gate);
    a.output2_scale_scalar = ptr<const float>(scale_out);
    a.local_expert_offset = expert_offset;
    a.direct_rows = direct_rows;
    a.output = ptr<void>(output);
    a.output_stride = output_stride;
    a.hidden_states_stride = hidden_states_stride;
    a.hidden_states_scale_stride = hidden_states_scale_stride;
    a.topk_stride = topk_stride;
    check(b200moe_run(ptr<b200moe_layer>(h), &a, ptr<void>(stream)), "b200moe_run");
  }, py::arg("handle"), py::arg("num_tokens"), py::arg("ids"), py::arg("weights"), py::arg("hidden_states"), py::arg("hidden_scale"),
     py::arg("scale_layout"), py::arg("activation_type"), py::arg("w1"), py::arg("s1"), py::arg("w2"), py::arg("s2"), py::arg("alpha"),
     py::arg("beta"), py::arg("limit"), py::arg("scale_up"), py::arg("scale_gate"), py::arg("scale_out"), py::arg("expert_offset"),
     py::arg("direct_rows"), py::arg("output"), py::arg("output_stride"), py::arg("stream"), py::arg("hidden_states_stride") = 0,
     py::arg("hidden_states_scale_stride") = 0, py::arg("topk_stride") = 0);
  // Repeat call with an argument block the caller keeps alive (address of a b200moe_args): no marshalling at all.
  m.def("run_packed", [](uintptr_t h, uintptr_t args, uintptr_t stream) {
    check(b200moe_run(ptr<b200moe_layer>(h), ptr<const b200moe_args>(args), ptr<void>(stream)), "b200moe_run");
  });
  m.def("handle_null", []() { return (uintptr_t)0; });
  m.def("status", [](uintptr_t h, uintptr_t stream) {
    int32_t code = 0;
    check(b200moe_status(ptr<b200moe_layer>(h), ptr<void>(stream), &code), "b200moe_status");
    return (int)code;
  });
}
