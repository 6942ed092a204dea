// pybind11 module over the C ABI of libavefp4 (include/ave_fp4.h): the native-module form of the binding.
//
// The reference keeps its native Python module in python/src (python/src/avelang_bindings.cc:493-529, one
// PYBIND11_MODULE that exposes the compiler).  This file is the counterpart for the FP4 path: it exposes the
// C-ABI entry points one for one, with device pointers and the stream passed as integers (what
// torch.Tensor.data_ptr() and torch.cuda.current_stream().cuda_stream give), so that the operators in
// python/avelang_kernels can call the library without ctypes.  It holds no logic of its own: every function
// forwards to libavefp4.so, and a non-zero return code becomes a RuntimeError carrying ave_fp4_last_error(),
// which is how the reference surfaces driver errors (python/avelang/backends/nvidia/driver.py:68-81).
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/ave_fp4.h"

namespace py = pybind11;

namespace {

void* P(std::uintptr_t v) { return reinterpret_cast<void*>(v); }

void check(int rc) {
    if (rc != 0) {
        std::string msg = ave_fp4_last_error();
        if (msg.rfind("ave-lang Error", 0) != 0) msg = "ave-lang Error [CUDA]: " + msg;
        throw std::runtime_error(msg + " (code " + std::to_string(rc) + ")");
    }
}

ave_fp4_epilogue make_epilogue(std::uintptr_t bias, int activation) {
    ave_fp4_epilogue e{};
    e.bias_bf16 = P(bias);
    e.activation = activation;
    return e;
}

}  // namespace

PYBIND11_MODULE(_avefp4_shim, m) {
    m.doc() = "libavefp4 C ABI (block-scaled FP4 GEMM and quantise for sm_100a) as a native Python module";

    m.def("init", [](int device) { check(ave_fp4_init(device)); }, py::arg("device"));
    m.def("last_error", []() { return std::string(ave_fp4_last_error()); });
    m.def("sm_count", []() { return ave_fp4_sm_count(); });
    m.def("sf_bytes", &ave_fp4_sf_bytes, py::arg("rows"), py::arg("k"), py::arg("fmt"), py::arg("sf_layout"));
    m.def("workspace_bytes", &ave_fp4_workspace_bytes, py::arg("m"), py::arg("n"), py::arg("k"), py::arg("fmt"), py::arg("variant"),
          py::arg("device"));
    m.def("linear_decode_workspace_bytes", &ave_fp4_linear_decode_workspace_bytes, py::arg("m"), py::arg("n"), py::arg("k"),
          py::arg("fmt"), py::arg("device"));

    m.def("quantize",
          [](std::uintptr_t x, std::int64_t rows, std::int64_t k, std::int64_t ldx, int fmt, std::uintptr_t amax, std::uintptr_t gs,
             std::uintptr_t packed, std::uintptr_t scales, int sf_layout, std::uintptr_t stream) {
              check(ave_fp4_quantize(P(x), rows, k, ldx, fmt, P(amax), P(gs), P(packed), P(scales), sf_layout, P(stream)));
          },
          py::arg("x_bf16"), py::arg("rows"), py::arg("k"), py::arg("ldx"), py::arg("fmt"), py::arg("amax_f32"), py::arg("global_scale"),
          py::arg("packed"), py::arg("scales"), py::arg("sf_layout"), py::arg("stream"));
    m.def("quantize_nvfp4_dynamic",
          [](std::uintptr_t x, std::int64_t rows, std::int64_t k, std::int64_t ldx, std::uintptr_t gs, std::uintptr_t packed,
             std::uintptr_t scales, int sf_layout, std::uintptr_t amax_scratch, std::uintptr_t stream) {
              check(ave_fp4_quantize_nvfp4_dynamic(P(x), rows, k, ldx, P(gs), P(packed), P(scales), sf_layout, P(amax_scratch), P(stream)));
          },
          py::arg("x_bf16"), py::arg("rows"), py::arg("k"), py::arg("ldx"), py::arg("global_scale"), py::arg("packed"), py::arg("scales"),
          py::arg("sf_layout"), py::arg("amax_scratch"), py::arg("stream"));

    m.def("gemm",
          [](std::uintptr_t a, std::uintptr_t sfa, std::uintptr_t ags, std::uintptr_t b, std::uintptr_t sfb, std::uintptr_t bgs,
             std::uintptr_t d, std::int64_t mm, std::int64_t n, std::int64_t k, std::int64_t ldd, int fmt, int variant, std::uintptr_t ws,
             std::int64_t ws_bytes, std::uintptr_t stream, std::uintptr_t bias, int activation) {
              if (bias == 0 && activation == AVE_FP4_ACT_NONE) {
                  check(ave_fp4_gemm(P(a), P(sfa), P(ags), P(b), P(sfb), P(bgs), P(d), mm, n, k, ldd, fmt, variant, P(ws), ws_bytes, P(stream)));
              } else {
                  const ave_fp4_epilogue e = make_epilogue(bias, activation);
                  check(ave_fp4_gemm_epilogue(P(a), P(sfa), P(ags), P(b), P(sfb), P(bgs), P(d), mm, n, k, ldd, fmt, variant, P(ws), ws_bytes,
                                              P(stream), &e));
              }
          },
          py::arg("a_packed"), py::arg("a_scales"), py::arg("a_global_scale"), py::arg("b_packed"), py::arg("b_scales"),
          py::arg("b_global_scale"), py::arg("d_bf16"), py::arg("m"), py::arg("n"), py::arg("k"), py::arg("ldd"), py::arg("fmt"),
          py::arg("variant") = 0, py::arg("workspace") = 0, py::arg("workspace_bytes") = 0, py::arg("stream") = 0, py::arg("bias_bf16") = 0,
          py::arg("activation") = 0);

    m.def("linear_decode",
          [](std::uintptr_t x, std::int64_t ldx, std::uintptr_t b, std::uintptr_t sfb, std::uintptr_t bgs, std::uintptr_t d, std::int64_t mm,
             std::int64_t n, std::int64_t k, std::int64_t ldd, int fmt, int flags, std::uintptr_t ws, std::int64_t ws_bytes,
             std::uintptr_t stream, std::uintptr_t bias, int activation) {
              const ave_fp4_epilogue e = make_epilogue(bias, activation);
              const bool plain = (bias == 0 && activation == AVE_FP4_ACT_NONE);
              check(ave_fp4_linear_decode(P(x), ldx, P(b), P(sfb), P(bgs), P(d), mm, n, k, ldd, fmt, flags, P(ws), ws_bytes, P(stream),
                                          plain ? nullptr : &e));
          },
          py::arg("x_bf16"), py::arg("ldx"), py::arg("b_packed"), py::arg("b_scales"), py::arg("b_global_scale"), py::arg("d_bf16"),
          py::arg("m"), py::arg("n"), py::arg("k"), py::arg("ldd"), py::arg("fmt"), py::arg("flags") = 0, py::arg("workspace") = 0,
          py::arg("workspace_bytes") = 0, py::arg("stream") = 0, py::arg("bias_bf16") = 0, py::arg("activation") = 0);

    m.def("bf16_gemm",
          [](std::uintptr_t a, std::uintptr_t b, std::uintptr_t d, std::int64_t mm, std::int64_t n, std::int64_t k, std::int64_t ldd,
             int variant, std::uintptr_t stream) { check(ave_bf16_gemm(P(a), P(b), P(d), mm, n, k, ldd, variant, P(stream))); },
          py::arg("a_bf16"), py::arg("b_bf16"), py::arg("d_bf16"), py::arg("m"), py::arg("n"), py::arg("k"), py::arg("ldd"),
          py::arg("variant") = 0, py::arg("stream") = 0);

    m.def("check", [](std::uintptr_t stream) { check(ave_fp4_check(P(stream))); }, py::arg("stream") = 0);
}
