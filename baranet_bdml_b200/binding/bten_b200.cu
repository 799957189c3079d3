// `bten` as a superset: everything the reference's module binds (src/bindings.cu:12-25, through its own
// src/py_tensor_shim.hh, compiled from the reference tree where it lies) plus thin entries that hand a TensorF's
// pointer, strides and sizes to libbn_attn.so (include/bn_attn.h).  With this module in place of the reference's
// `bten`, the unmodified `mygrad` package runs as before and GroupedQueryAttention can be switched to the fused
// kernel by rebinding its __call__ (baranet_bdml_b200/mygrad_dropin.py) - no change to the model code.
//
// The new entries follow the reference's operator convention (src/ops/op_rope.cuh:101-126 is representative): the
// binding allocates the output tensor, shape or device errors become std::runtime_error (RuntimeError in Python),
// the launch goes to the legacy default stream and returns immediately.
//
// Build: `make -C oracle bten REF=<reference tree>` (oracle/Makefile).
#include <pybind11/pybind11.h>
#include <pybind11/numpy.h>

#include "ops/op_elemwise.cuh"
#include "py_tensor_shim.hh"
#include "llama/llama_bindings.hpp"

#include "bn_attn.h"

namespace py = pybind11;

extern unsigned long long randgen_seed;   // src/randgen.cu of the reference, compiled into this module

namespace {

inline void bn_ok(int status) {
    if (status != BN_OK) throw std::runtime_error(bn_last_error());
}

using TF = PyTensor<float>;
using TU = PyTensor<uint32_t>;

inline const float* ptr(const TF& x) { return x.t.rawp + x.t.offset; }

void need_device(const TF& x, const char* what) {
    if (!x.t.on_device) throw std::runtime_error(std::string(what) + ": only GPU implementation available");
}

void add_b200_entries(py::module_& m) {
    auto cls = py::reinterpret_borrow<py::class_<TF>>(m.attr("TensorF"));

    // The attention core of GroupedQueryAttention.__call__ (mygrad/llama/llama_layers.py:161-183) in one launch;
    // takes the slot of op_attention_fused (src/ops/op_attention_fused.cuh:109-118): (Q, K, V, out, scale, causal,
    // seq_offset).  heads_mode 0 = the reference layer's own result (heads collapsed into one softmax).
    cls.def("attention_fused",
            [](const TF& q, const TF& k, const TF& v, float scale, bool causal, int seq_offset, int num_heads,
               int num_kv_heads, int head_dim, float theta, int heads_mode) {
                need_device(q, "Attention");
                need_device(k, "Attention");
                need_device(v, "Attention");
                if (k.t.h != q.t.h || v.t.h != q.t.h || q.t.w != num_heads * head_dim ||
                    k.t.w != num_kv_heads * head_dim || v.t.w != k.t.w)
                    throw std::runtime_error("Attention: hidden size mismatch");
                TF out(q.t.h, q.t.w, true);
                bn_ok(bn_attn_prefill_f32(ptr(q), q.t.stride_h, q.t.stride_w, ptr(k), k.t.stride_h, k.t.stride_w, ptr(v),
                                          v.t.stride_h, v.t.stride_w, out.t.rawp, out.t.stride_h, out.t.stride_w, q.t.h,
                                          num_heads, num_kv_heads, head_dim, scale, theta, seq_offset, causal ? 1 : 0,
                                          heads_mode, /*apply_rope=*/1, /*stream=*/nullptr));
                return out;
            },
            py::arg("key"), py::arg("value"), py::arg("scale"), py::arg("causal") = false, py::arg("seq_offset") = 0,
            py::arg("num_heads") = 32, py::arg("num_kv_heads") = 4, py::arg("head_dim") = 64,
            py::arg("theta") = 10000.0f, py::arg("heads_mode") = (int)BN_HEADS_COLLAPSED);

    // Bit-compatible replacements of op_mm, op_rope, op_rmsnorm and op_argmax under names of their own, so that the
    // reference's operators stay reachable in the same process (the parity tests run both).
    cls.def("matmul_b200",
            [](const TF& a, const TF& b) {
                need_device(a, "Matrix multiply");
                need_device(b, "Matrix multiply");
                if (a.t.w != b.t.h) throw std::runtime_error("MatMul: inner dimensions mismatch");
                TF out(a.t.h, b.t.w, true);
                bn_ok(bn_mm_f32(ptr(a), a.t.stride_h, a.t.stride_w, ptr(b), b.t.stride_h, b.t.stride_w, out.t.rawp,
                                out.t.stride_h, out.t.stride_w, a.t.h, a.t.w, b.t.w, nullptr));
                return out;
            },
            py::arg("other"));
    cls.def("rope_b200",
            [](const TF& x, int position_offset, int head_dim, float theta) {
                need_device(x, "RoPE");
                TF out(x.t.h, x.t.w, true);
                bn_ok(bn_rope_f32(ptr(x), x.t.stride_h, x.t.stride_w, out.t.rawp, out.t.stride_h, out.t.stride_w, x.t.h,
                                  x.t.w, head_dim, theta, position_offset, nullptr));
                return out;
            },
            py::arg("position_offset") = 0, py::arg("head_dim") = 64, py::arg("theta") = 10000.0f);
    cls.def("rmsnorm_b200",
            [](const TF& x, const TF& weight, float eps) {
                need_device(x, "RMSNorm");
                if (weight.t.h != 1 || weight.t.w != x.t.w)
                    throw std::runtime_error("RMSNorm: weight shape must be (1, hidden_dim)");
                TF out(x.t.h, x.t.w, true);
                bn_ok(bn_rmsnorm_f32(ptr(x), x.t.stride_h, x.t.stride_w, ptr(weight), weight.t.stride_w, out.t.rawp,
                                     out.t.stride_h, out.t.stride_w, x.t.h, x.t.w, eps, nullptr));
                return out;
            },
            py::arg("weight"), py::arg("eps") = 1e-6f);
    // hidden = residual + hidden; hidden = norm(hidden) of LLaMADecoderLayer (llama_layers.py:279-283) in one launch
    cls.def("add_rmsnorm",
            [](const TF& a, const TF& b, const TF& weight, float eps) {
                need_device(a, "RMSNorm");
                need_device(b, "RMSNorm");
                if (a.t.h != b.t.h || a.t.w != b.t.w) throw std::runtime_error("Add: shape mismatch");
                if (weight.t.h != 1 || weight.t.w != a.t.w)
                    throw std::runtime_error("RMSNorm: weight shape must be (1, hidden_dim)");
                TF sum(a.t.h, a.t.w, true), out(a.t.h, a.t.w, true);
                bn_ok(bn_add_rmsnorm_f32(ptr(a), a.t.stride_h, a.t.stride_w, ptr(b), b.t.stride_h, b.t.stride_w,
                                         ptr(weight), weight.t.stride_w, sum.t.rawp, sum.t.stride_h, sum.t.stride_w,
                                         out.t.rawp, out.t.stride_h, out.t.stride_w, a.t.h, a.t.w, eps, nullptr));
                return py::make_tuple(sum, out);
            },
            py::arg("other"), py::arg("weight"), py::arg("eps") = 1e-6f);
    cls.def("argmax_b200", [](const TF& x) {
        need_device(x, "Argmax");
        TU out(x.t.h, 1, true);
        bn_ok(bn_argmax_rows_f32(ptr(x), x.t.stride_h, x.t.stride_w, out.t.rawp, x.t.h, x.t.w, nullptr));
        return out;
    });
    // rows of an embedding table picked on the device (LLaMAModel.embed, llama_model.py:58-78, gathers on the host)
    cls.def("gather_rows",
            [](const TF& table, const TU& ids) {
                need_device(table, "Embedding");
                if (!ids.t.on_device) throw std::runtime_error("Embedding: only GPU implementation available");
                if (table.t.stride_w != 1 || ids.t.stride_w != 1 || (ids.t.h != 1 && ids.t.w != 1))
                    throw std::runtime_error("Embedding: table rows must be contiguous and ids a vector");
                const int n = ids.t.h * ids.t.w;
                TF out(n, table.t.w, true);
                bn_ok(bn_embedding_gather_f32(ptr(table), table.t.stride_h, ids.t.rawp + ids.t.offset, out.t.rawp,
                                              out.t.stride_h, n, table.t.w, table.t.h, nullptr, nullptr));
                return out;
            },
            py::arg("ids"));
}

}  // namespace

PYBIND11_MODULE(bten, m) {
    m.doc() = "BareNet tensor bindings (float32 / uint32) with the B200 attention entries";
    m.def("randgen_seed", [](unsigned long long seed) { ::randgen_seed = seed; }, "Set random seed");
    bind_tensor_type<float>(m, "TensorF");
    bind_tensor_type<uint32_t>(m, "TensorU32");
    bind_llama_model(m);
    add_b200_entries(m);
    m.attr("has_b200_attention") = true;
    m.def("bn_version", []() { return bn_version(); });
}
