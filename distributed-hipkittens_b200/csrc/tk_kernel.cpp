// Python module `tk_kernel`: the reference's one callable,
//   dispatch_micro(A, B, C, iris_view, M_local, N, K, row_offset)
// (distributed-kernels/bf16_gemm/kernel.cpp:253-265, bound through kittens::py::bind_function,
// include/pyutils/pyutils.cuh:66-71), plus the entry points the named hot path adds, in the same
// style: positional torch tensors -> raw pointers -> C ABI (include/dk_b200.h) -> CUDA.
//
// Tensor arguments go through the same checks, with the same messages, as the reference's
// from_object<GL>::make (include/pyutils/pyutils.cuh:14-47): class name "Tensor", contiguous, not
// on the CPU, at most 4 dimensions. Added here: a dtype check, and launches go on torch's current
// stream instead of the NULL stream. No torch headers are needed: tensors are read through their
// Python attributes, exactly as the reference does.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <map>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "dk_b200.h"

namespace py = pybind11;

namespace {

void throw_on(int rc, const char* what) {
    if (rc != DK_OK) {
        std::string msg = std::string(what) + ": " + dk_strerror(rc);
        const char* d = dk_last_error_string();
        if (d && *d) msg += std::string(" (") + d + ")";
        if (rc == DK_ERR_DEVICE) {
            unsigned st[4] = {0, 0, 0, 0};
            dk_last_device_status(st);
            msg += " [code " + std::to_string(st[0]) + " block " + std::to_string(st[1]) + " site " +
                   std::to_string(st[2]) + " detail " + std::to_string(st[3]) + "]";
        }
        throw std::runtime_error(msg);
    }
}

struct TensorArg {
    void* ptr = nullptr;
    std::vector<int64_t> shape;
    std::string dtype;  // e.g. "torch.bfloat16"
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

TensorArg tensor_arg(const py::object& obj, const char* want_dtype = nullptr) {
    if (py::hasattr(obj, "__class__") &&
        obj.attr("__class__").attr("__name__").cast<std::string>() == "Tensor") {
        if (!obj.attr("is_contiguous")().cast<bool>()) throw std::runtime_error("Tensor must be contiguous");
        if (obj.attr("device").attr("type").cast<std::string>() == "cpu")
            throw std::runtime_error("Tensor must be on CUDA device");
        auto py_shape = obj.attr("shape").cast<py::tuple>();
        if (py_shape.size() > 4) throw std::runtime_error("Expected Tensor.ndim <= 4");
        TensorArg t;
        for (size_t i = 0; i < py_shape.size(); ++i) t.shape.push_back(py::cast<int64_t>(py_shape[i]));
        t.ptr = reinterpret_cast<void*>(obj.attr("data_ptr")().cast<uint64_t>());
        t.dtype = py::str(obj.attr("dtype")).cast<std::string>();
        if (want_dtype != nullptr && t.dtype != want_dtype)
            throw std::runtime_error(std::string("Expected dtype ") + want_dtype + ", got " + t.dtype);
        return t;
    }
    throw std::runtime_error("Expected a torch.Tensor");
}

const dk_view* view_arg(const py::object& obj) {
    if (obj.is_none()) return nullptr;
    if (!py::hasattr(obj, "_addr")) throw std::runtime_error("Expected an iris_py.IrisDeviceView");
    return reinterpret_cast<const dk_view*>(obj.attr("_addr")().cast<uintptr_t>());
}

void* current_stream() {
    py::object torch = py::module_::import("torch");
    return reinterpret_cast<void*>(
        torch.attr("cuda").attr("current_stream")().attr("cuda_stream").cast<uintptr_t>());
}

void dispatch_micro(py::object A, py::object B, py::object C, py::object view, int M_local, int N,
                    int K, int row_offset) {
    (void)row_offset;  // accepted and unused, as in the reference (kernel.cpp:80)
    TensorArg a = tensor_arg(A, "torch.bfloat16");
    TensorArg b = tensor_arg(B, "torch.bfloat16");
    TensorArg c = tensor_arg(C, "torch.bfloat16");
    if (a.numel() != static_cast<int64_t>(M_local) * K) throw std::runtime_error("A must hold M_local*K elements");
    if (b.numel() != static_cast<int64_t>(N) * K) throw std::runtime_error("B must hold N*K elements");
    if (c.numel() != static_cast<int64_t>(M_local) * N) throw std::runtime_error("C must hold M_local*N elements");
    const dk_view* v = view_arg(view);
    throw_on(dk_gemm_bf16(a.ptr, b.ptr, c.ptr, M_local, N, K, v, -1, current_stream()), "dispatch_micro");
}

// One reduce-scatter workspace per (heap, M, N), allocated from the heap on first use. Every rank
// makes the same calls in the same order, so the offsets agree.
std::map<std::tuple<uintptr_t, int, int>, void*> g_rs_workspaces;

void gemm_rs(py::object A, py::object Bt, py::object Out, py::object view) {
    TensorArg a = tensor_arg(A, "torch.bfloat16");
    TensorArg b = tensor_arg(Bt, "torch.bfloat16");
    TensorArg o = tensor_arg(Out, "torch.bfloat16");
    if (a.shape.size() != 2 || b.shape.size() != 2 || o.shape.size() != 2)
        throw std::runtime_error("gemm_rs expects 2-D tensors A[M,K/P], Bt[N,K/P], Out[M/P,N]");
    const int M = static_cast<int>(a.shape[0]), Kloc = static_cast<int>(a.shape[1]);
    const int N = static_cast<int>(b.shape[0]);
    if (b.shape[1] != Kloc) throw std::runtime_error("A and Bt disagree on K");
    const dk_view* v = view_arg(view);
    const int world = v ? v->world : 1;
    if (o.shape[0] * world != M || o.shape[1] != N) throw std::runtime_error("Out must be [M/world, N]");
    void* ws = nullptr;
    void* stream = current_stream();
    if (world > 1) {
        auto key = std::make_tuple(reinterpret_cast<uintptr_t>(v->heap), M, N);
        auto it = g_rs_workspaces.find(key);
        if (it == g_rs_workspaces.end()) {
            const size_t bytes = dk_gemm_rs_workspace_bytes(M, N, world);
            ws = dk_heap_alloc(static_cast<dk_heap*>(v->heap), bytes, 1024);
            if (ws == nullptr) throw std::runtime_error("Failed to allocate iris memory");
            throw_on(dk_gemm_rs_workspace_init(ws, bytes, v, stream), "gemm_rs workspace");
            g_rs_workspaces[key] = ws;
        } else {
            ws = it->second;
        }
    }
    throw_on(dk_gemm_rs(a.ptr, b.ptr, o.ptr, M, N, Kloc, ws, v, stream), "gemm_rs");
}

void allreduce(py::object X, py::object Out, py::object view, int algo) {
    TensorArg x = tensor_arg(X, "torch.bfloat16");
    TensorArg o = tensor_arg(Out, "torch.bfloat16");
    if (x.numel() != o.numel()) throw std::runtime_error("X and Out must hold the same number of elements");
    throw_on(dk_allreduce(x.ptr, o.ptr, static_cast<size_t>(x.numel()), algo, view_arg(view), current_stream()),
             "allreduce");
}

py::tuple device_status() {
    unsigned st[4] = {0, 0, 0, 0};
    throw_on(dk_last_device_status(st), "device_status");
    return py::make_tuple(st[0], st[1], st[2], st[3]);
}

}  // namespace

PYBIND11_MODULE(tk_kernel, m) {
    m.doc() = "B200 kernels behind the reference's tk_kernel interface";
    m.def("dispatch_micro", &dispatch_micro,
          "C[M_local,N] = A[M_local,K] @ B[N,K]^T (bf16, fp32 accumulate). Positional arguments: "
          "A, B, C, iris_view, M_local, N, K, row_offset");
    m.def("gemm_rs", &gemm_rs,
          "Out[M/P,N] = reduce-scatter over ranks of A[M,K/P] @ Bt[N,K/P]^T. Positional: A, Bt, Out, view");
    m.def("allreduce", &allreduce, py::arg("X"), py::arg("Out"), py::arg("view"), py::arg("algo") = -1,
          "Out = sum over ranks of X (bf16). algo: -1 auto, 0 one-shot, 1 two-shot, 2 NVLS");
    m.def("device_status", &device_status,
          "(code, block, site, detail) of the first device-side wait that gave up; clears it");
}
