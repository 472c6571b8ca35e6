// Python extension `tk_kernel` with one function `dispatch_micro`, the module and function names the
// reference's harness imports (kernels/gemm/bf16fp32/256_256_64_32_with16x32.cpp:389-393, bench.py:34).
// Like the reference's binding (include/pyutils/pyutils.cuh:15-47) it duck-types torch tensors --
// class name, is_contiguous(), device.type, shape, data_ptr() -- and does not link against torch.
// It adds the dtype / shape cross-checks the reference leaves out and forwards to the C ABI.
#include <pybind11/pybind11.h>

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "mxfp6.h"

namespace py = pybind11;

namespace {

struct TensorView {
    uint64_t ptr;
    std::array<int64_t, 4> shape;   // left-padded with 1s, as the reference's gl<> descriptors are
    std::string dtype;
    int device;
};

TensorView view_of(const py::object& obj) {
    if (!(py::hasattr(obj, "__class__") && obj.attr("__class__").attr("__name__").cast<std::string>() == "Tensor"))
        throw std::runtime_error("Expected a torch.Tensor");
    if (!obj.attr("is_contiguous")().cast<bool>()) throw std::runtime_error("Tensor must be contiguous");
    if (obj.attr("device").attr("type").cast<std::string>() == "cpu") throw std::runtime_error("Tensor must be on CUDA device");
    TensorView v{};
    v.shape = {1, 1, 1, 1};
    auto shp = obj.attr("shape").cast<py::tuple>();
    const size_t dims = shp.size();
    if (dims > 4) throw std::runtime_error("Expected Tensor.ndim <= 4");
    for (size_t i = 0; i < dims; ++i) v.shape[4 - dims + i] = py::cast<int64_t>(shp[i]);
    v.ptr = obj.attr("data_ptr")().cast<uint64_t>();
    v.dtype = py::str(obj.attr("dtype")).cast<std::string>();
    py::object idx = obj.attr("device").attr("index");
    v.device = idx.is_none() ? 0 : idx.cast<int>();
    return v;
}

void dispatch_micro(py::object A, py::object B, py::object C, py::object scale_A, py::object scale_B, int fmt) {
    const TensorView a = view_of(A), b = view_of(B), c = view_of(C), sa = view_of(scale_A), sb = view_of(scale_B);
    if (a.dtype != "torch.uint8" || b.dtype != "torch.uint8") throw std::runtime_error("A and B must be packed fp6 as torch.uint8");
    if (sa.dtype != "torch.uint8" || sb.dtype != "torch.uint8") throw std::runtime_error("scales must be E8M0 bytes as torch.uint8");
    if (c.dtype != "torch.bfloat16") throw std::runtime_error("C must be torch.bfloat16");
    for (const TensorView* t : {&a, &b, &c, &sa, &sb})
        if (t->shape[0] != 1 || t->shape[1] != 1) throw std::runtime_error("Expected 2-D tensors");
    // M from A, N from C, K from A -- the reference's rule (256_256_64_32_with16x32.cpp:52-54)
    const int64_t M = a.shape[2], N = c.shape[3];
    const bool fp8 = fmt == MXFP8_E4M3 || fmt == MXFP8_E5M2;
    if (!fp8 && a.shape[3] % 3 != 0) throw std::runtime_error("A.shape[1] must be 3K/4 bytes");
    const int64_t K = fp8 ? a.shape[3] : a.shape[3] / 3 * 4;
    if (K % 128 != 0) throw std::runtime_error("K must be a multiple of 128");
    if (c.shape[2] != M) throw std::runtime_error("C.shape[0] must equal A.shape[0]");
    if (b.shape[2] != N || b.shape[3] != a.shape[3]) throw std::runtime_error("B must be [N, 3K/4] (fp6) or [N, K] (fp8)");
    if (sa.shape[2] != M || sa.shape[3] != K / 32) throw std::runtime_error("scale_A must be [M, K/32]");
    if (sb.shape[2] != N || sb.shape[3] != K / 32) throw std::runtime_error("scale_B must be [N, K/32]");
    if (a.device != b.device || a.device != c.device || a.device != sa.device || a.device != sb.device)
        throw std::runtime_error("all tensors must be on the same device");
    if (fmt < 0 || fmt > 3) throw std::runtime_error("fmt must be 0 (E2M3), 1 (E3M2), 2 (fp8 E4M3) or 3 (fp8 E5M2)");

    // launch on torch's current stream of the tensors' device, with that device current
    py::module_ cuda = py::module_::import("torch").attr("cuda");
    py::object guard = cuda.attr("device")(a.device);
    guard.attr("__enter__")();
    int rc;
    try {
        const uint64_t stream = cuda.attr("current_stream")().attr("cuda_stream").cast<uint64_t>();
        rc = mxfp6_gemm(reinterpret_cast<const void*>(a.ptr), reinterpret_cast<const void*>(sa.ptr),
                        reinterpret_cast<const void*>(b.ptr), reinterpret_cast<const void*>(sb.ptr),
                        reinterpret_cast<void*>(c.ptr), M, N, K, fmt, fmt, reinterpret_cast<void*>(stream));
    } catch (...) {
        guard.attr("__exit__")(py::none(), py::none(), py::none());
        throw;
    }
    guard.attr("__exit__")(py::none(), py::none(), py::none());
    if (rc != MXFP6_OK) throw std::runtime_error(std::string("mxfp6_gemm failed: ") + mxfp6_last_error());
}

}  // namespace

PYBIND11_MODULE(tk_kernel, m) {
    m.doc() = "MX-FP6 GEMM for B200: C[M,N] (bf16) = A[M,K] * B[N,K]^T with packed fp6 operands and E8M0 block scales";
    m.def("dispatch_micro", &dispatch_micro, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("scale_A"),
          py::arg("scale_B"), py::arg("fmt") = 0);
    m.def("version", []() { return mxfp6_version(); });
}
