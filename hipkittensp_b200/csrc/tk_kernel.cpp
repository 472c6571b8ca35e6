// Python extension `tk_kernel` with one function `dispatch_micro`, the module and function names the
// reference's harness imports (kernels/gemm/bf16fp32/256_256_64_32_with16x32.cpp:389-393, bench.py:34).
// Like the reference's binding (include/pyutils/pyutils.cuh:15-47) it duck-types torch tensors --
// class name, is_contiguous(), is_cuda, shape, data_ptr() -- and does not link against torch.
// It adds the dtype / shape cross-checks the reference leaves out and forwards to the C ABI.
#include <cuda_runtime_api.h>
#include <pybind11/pybind11.h>

#include <array>
#include <cstring>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "mxfp6.h"

namespace py = pybind11;

namespace {

enum class DType { U8, BF16, Other };

struct TensorView {
    uint64_t ptr;
    std::array<int64_t, 4> shape;   // left-padded with 1s, as the reference's gl<> descriptors are
    DType dtype;
    int device;
};

// Objects looked up once: the two dtypes the operator accepts and torch's accessor of the current stream handle.
struct TorchHandles {
    py::object u8, bf16, raw_stream, cuda;
    TorchHandles() {
        py::module_ torch = py::module_::import("torch");
        u8 = torch.attr("uint8");
        bf16 = torch.attr("bfloat16");
        cuda = torch.attr("cuda");
        py::object c = torch.attr("_C");
        if (py::hasattr(c, "_cuda_getCurrentRawStream")) raw_stream = c.attr("_cuda_getCurrentRawStream");
    }
    uint64_t current_stream(int device) const {
        if (raw_stream) return raw_stream(device).cast<uint64_t>();
        return cuda.attr("current_stream")(device).attr("cuda_stream").cast<uint64_t>();
    }
};
const TorchHandles& handles() {
    static TorchHandles* h = new TorchHandles();   // never destroyed: outlives interpreter shutdown order problems
    return *h;
}

TensorView view_of(const py::object& obj) {
    if (std::strcmp(Py_TYPE(obj.ptr())->tp_name, "Tensor") != 0) throw std::runtime_error("Expected a torch.Tensor");
    if (!obj.attr("is_contiguous")().cast<bool>()) throw std::runtime_error("Tensor must be contiguous");
    if (!obj.attr("is_cuda").cast<bool>()) throw std::runtime_error("Tensor must be on CUDA device");
    TensorView v{};
    v.shape = {1, 1, 1, 1};
    auto shp = obj.attr("shape").cast<py::tuple>();
    const size_t dims = shp.size();
    if (dims > 4) throw std::runtime_error("Expected Tensor.ndim <= 4");
    for (size_t i = 0; i < dims; ++i) v.shape[4 - dims + i] = py::cast<int64_t>(shp[i]);
    v.ptr = obj.attr("data_ptr")().cast<uint64_t>();
    const TorchHandles& h = handles();
    py::object dt = obj.attr("dtype");
    v.dtype = dt.is(h.u8) ? DType::U8 : dt.is(h.bf16) ? DType::BF16 : DType::Other;
    v.device = obj.attr("get_device")().cast<int>();
    return v;
}

// Makes `device` current for the lifetime of the object and restores the previous one.
struct DeviceGuard {
    int prev = -1, changed = 0;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) throw std::runtime_error("cudaGetDevice failed");
        if (prev != device) {
            if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
            changed = 1;
        }
    }
    ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

void dispatch_micro(py::object A, py::object B, py::object C, py::object scale_A, py::object scale_B, int fmt) {
    const TensorView a = view_of(A), b = view_of(B), c = view_of(C), sa = view_of(scale_A), sb = view_of(scale_B);
    if (a.dtype != DType::U8 || b.dtype != DType::U8) throw std::runtime_error("A and B must be packed fp6 as torch.uint8");
    if (sa.dtype != DType::U8 || sb.dtype != DType::U8) throw std::runtime_error("scales must be E8M0 bytes as torch.uint8");
    if (c.dtype != DType::BF16) throw std::runtime_error("C must be torch.bfloat16");
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
    int rc;
    {
        DeviceGuard guard(a.device);
        const uint64_t stream = handles().current_stream(a.device);
        rc = mxfp6_gemm(reinterpret_cast<const void*>(a.ptr), reinterpret_cast<const void*>(sa.ptr),
                        reinterpret_cast<const void*>(b.ptr), reinterpret_cast<const void*>(sb.ptr),
                        reinterpret_cast<void*>(c.ptr), M, N, K, fmt, fmt, reinterpret_cast<void*>(stream));
    }
    if (rc != MXFP6_OK) throw std::runtime_error(std::string("mxfp6_gemm failed: ") + mxfp6_last_error());
}

}  // namespace

PYBIND11_MODULE(tk_kernel, m) {
    m.doc() = "MX-FP6 GEMM for B200: C[M,N] (bf16) = A[M,K] * B[N,K]^T with packed fp6 operands and E8M0 block scales";
    m.def("dispatch_micro", &dispatch_micro, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("scale_A"),
          py::arg("scale_B"), py::arg("fmt") = 0);
    m.def("version", []() { return mxfp6_version(); });
}
