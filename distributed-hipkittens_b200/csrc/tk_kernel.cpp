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

#include <stdexcept>
#include <string>
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

// The single-GPU form of the reference's GEMM module: dispatch_micro(A[M,K], Bt[N,K], C[M,N])
// (kernels/cdna4/gemm/bf16fp32/256_256_64_32_with16x32.cpp:329-339, called that way by its
// test.py:28 and bench.py:34). M, N, K come from the tensors, as there (g.M, g.N, g.K are the
// globals' runtime dimensions).
void dispatch_micro3(py::object A, py::object Bt, py::object C) {
    TensorArg a = tensor_arg(A, "torch.bfloat16");
    TensorArg b = tensor_arg(Bt, "torch.bfloat16");
    TensorArg c = tensor_arg(C, "torch.bfloat16");
    if (a.shape.size() != 2 || b.shape.size() != 2 || c.shape.size() != 2)
        throw std::runtime_error("dispatch_micro expects 2-D tensors A[M,K], Bt[N,K], C[M,N]");
    const int M = static_cast<int>(a.shape[0]), K = static_cast<int>(a.shape[1]);
    const int N = static_cast<int>(b.shape[0]);
    if (b.shape[1] != K) throw std::runtime_error("A and Bt disagree on K");
    if (c.shape[0] != M || c.shape[1] != N) throw std::runtime_error("C must be [M, N]");
    throw_on(dk_gemm_bf16(a.ptr, b.ptr, c.ptr, M, N, K, nullptr, -1, current_stream()), "dispatch_micro");
}

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
    // the workspace for this (M, N) belongs to the heap of the view: made on first use (every rank
    // makes the same calls in the same order, so the offsets agree), gone when the heap goes
    throw_on(dk_gemm_rs_workspace_get(v, M, N, stream, &ws), "gemm_rs workspace");
    throw_on(dk_gemm_rs(a.ptr, b.ptr, o.ptr, M, N, Kloc, ws, v, stream), "gemm_rs");
}

// Column-parallel GEMM fused with the all-gather of its activations (dk_ag_gemm): every rank passes
// its row shard of A and its own columns of the weight and gets all rows of its output columns.
void ag_gemm(py::object A, py::object Bt, py::object Cout, py::object view) {
    TensorArg a = tensor_arg(A, "torch.bfloat16");
    TensorArg b = tensor_arg(Bt, "torch.bfloat16");
    TensorArg c = tensor_arg(Cout, "torch.bfloat16");
    if (a.shape.size() != 2 || b.shape.size() != 2 || c.shape.size() != 2)
        throw std::runtime_error("ag_gemm expects 2-D tensors A[M/P,K], Bt[N,K], C[M,N]");
    const dk_view* v = view_arg(view);
    const int world = v ? v->world : 1;
    const int M = static_cast<int>(a.shape[0]) * world, K = static_cast<int>(a.shape[1]);
    const int N = static_cast<int>(b.shape[0]);
    if (b.shape[1] != K) throw std::runtime_error("A and Bt disagree on K");
    if (c.shape[0] != M || c.shape[1] != N) throw std::runtime_error("C must be [M/P * world, N]");
    void* ws = nullptr;
    void* stream = current_stream();
    throw_on(dk_ag_gemm_workspace_get(v, M, K, stream, &ws), "ag_gemm workspace");
    throw_on(dk_ag_gemm(a.ptr, b.ptr, c.ptr, M, N, K, ws, v, stream), "ag_gemm");
}

void allreduce(py::object X, py::object Out, py::object view, int algo) {
    TensorArg x = tensor_arg(X, "torch.bfloat16");
    TensorArg o = tensor_arg(Out, "torch.bfloat16");
    if (x.numel() != o.numel()) throw std::runtime_error("X and Out must hold the same number of elements");
    throw_on(dk_allreduce(x.ptr, o.ptr, static_cast<size_t>(x.numel()), algo, view_arg(view), current_stream()),
             "allreduce");
}

// ---- MoE entry points. Outputs are torch tensors created through torch's Python API.
py::object torch_empty(std::vector<int64_t> shape, const char* dtype, const py::object& like) {
    py::object torch = py::module_::import("torch");
    py::tuple shp(shape.size());
    for (size_t i = 0; i < shape.size(); ++i) shp[i] = py::int_(shape[i]);
    return torch.attr("empty")(shp, py::arg("dtype") = torch.attr(dtype), py::arg("device") = like.attr("device"));
}
void* tptr(const py::object& t) { return reinterpret_cast<void*>(t.attr("data_ptr")().cast<uint64_t>()); }

py::tuple moe_route(py::object logits, int k) {
    TensorArg l = tensor_arg(logits, "torch.float32");
    if (l.shape.size() != 2) throw std::runtime_error("logits must be [T, E]");
    const int T = static_cast<int>(l.shape[0]), E = static_cast<int>(l.shape[1]);
    py::object idx = torch_empty({T, k}, "int32", logits);
    py::object w = torch_empty({T, k}, "float32", logits);
    throw_on(dk_moe_route(static_cast<const float*>(l.ptr), T, E, k, static_cast<int*>(tptr(idx)),
                          static_cast<float*>(tptr(w)), current_stream()), "moe_route");
    return py::make_tuple(idx, w);
}

py::tuple moe_permute(py::object topk_idx, int E, int pad, int experts_per_segment) {
    TensorArg ti = tensor_arg(topk_idx, "torch.int32");
    if (ti.shape.size() != 2) throw std::runtime_error("topk_idx must be [T, k]");
    const int T = static_cast<int>(ti.shape[0]), k = static_cast<int>(ti.shape[1]);
    const int seg = experts_per_segment > 0 ? experts_per_segment : E;
    if (seg < 1 || E % seg != 0) throw std::runtime_error("experts_per_segment must divide E");
    const int nseg = E / seg;
    const int64_t cap = static_cast<int64_t>(dk_moe_rows_capacity(T, k, seg, pad));
    py::object rop = torch_empty({T, k}, "int32", topk_idx);
    py::object por = torch_empty({nseg, cap}, "int32", topk_idx);
    py::object offs = torch_empty({nseg, seg + 1}, "int32", topk_idx);
    py::object counts = torch_empty({E}, "int32", topk_idx);
    const size_t sb = dk_moe_permute_scratch_bytes(T, k, E);
    py::object scratch = torch_empty({static_cast<int64_t>(sb)}, "uint8", topk_idx);
    throw_on(dk_moe_permute(static_cast<const int*>(ti.ptr), T, k, E, pad, seg, static_cast<int*>(tptr(rop)),
                            static_cast<int*>(tptr(por)), static_cast<int>(cap), static_cast<int*>(tptr(offs)),
                            static_cast<int*>(tptr(counts)), tptr(scratch), sb, current_stream()),
             "moe_permute");
    if (nseg == 1) return py::make_tuple(rop, por[py::int_(0)], offs[py::int_(0)], counts);
    return py::make_tuple(rop, por, offs, counts);
}

py::tuple moe_quant(py::object X, py::object row_map, int map_mode, int k) {
    TensorArg x = tensor_arg(X, "torch.bfloat16");
    if (x.shape.size() != 2) throw std::runtime_error("X must be [rows, C]");
    const int C = static_cast<int>(x.shape[1]);
    int R = static_cast<int>(x.shape[0]);
    const int* map = nullptr;
    if (!row_map.is_none()) {
        TensorArg m = tensor_arg(row_map, "torch.int32");
        map = static_cast<const int*>(m.ptr);
        R = static_cast<int>(m.numel());
        if (map_mode == 0) map_mode = 1;
    }
    py::object q = torch_empty({R, C}, "uint8", X);
    py::object s = torch_empty({R / 128, C / 128}, "float32", X);
    throw_on(dk_quant_block128(x.ptr, R, C, map, map_mode, k, tptr(q), static_cast<float*>(tptr(s)),
                               current_stream()), "moe_quant");
    return py::make_tuple(q, s);
}

py::object moe_ffn_fp8(py::object Xq, py::object Xs, py::object W13q, py::object W13s, py::object W2q,
                       py::object W2s, py::object offsets) {
    TensorArg xq = tensor_arg(Xq, "torch.uint8"), xs = tensor_arg(Xs, "torch.float32");
    TensorArg w13q = tensor_arg(W13q, "torch.uint8"), w13s = tensor_arg(W13s, "torch.float32");
    TensorArg w2q = tensor_arg(W2q, "torch.uint8"), w2s = tensor_arg(W2s, "torch.float32");
    TensorArg off = tensor_arg(offsets, "torch.int32");
    if (xq.shape.size() != 2 || w13q.shape.size() != 3 || w2q.shape.size() != 3)
        throw std::runtime_error("expected Xq [R,H], W13q [E,2F,H], W2q [E,H,F]");
    const int R = static_cast<int>(xq.shape[0]), H = static_cast<int>(xq.shape[1]);
    const int E = static_cast<int>(w13q.shape[0]), F = static_cast<int>(w13q.shape[1] / 2);
    if (w13q.shape[2] != H || w2q.shape[0] != E || w2q.shape[1] != H || w2q.shape[2] != F || off.numel() != E + 1)
        throw std::runtime_error("MoE weight / offset shapes disagree");
    py::object hq = torch_empty({R, F}, "uint8", Xq);
    py::object hs = torch_empty({R / 128, F / 128}, "float32", Xq);
    py::object y = torch_empty({R, H}, "bfloat16", Xq);
    void* st = current_stream();
    throw_on(dk_moe_grouped_gemm_fp8(xq.ptr, static_cast<const float*>(xs.ptr), w13q.ptr,
                                     static_cast<const float*>(w13s.ptr), static_cast<const int*>(off.ptr), E, R,
                                     F, H, 1, tptr(hq), static_cast<float*>(tptr(hs)), st), "moe_ffn_fp8 (gate/up)");
    throw_on(dk_moe_grouped_gemm_fp8(tptr(hq), static_cast<const float*>(tptr(hs)), w2q.ptr,
                                     static_cast<const float*>(w2s.ptr), static_cast<const int*>(off.ptr), E, R,
                                     H, F, 0, tptr(y), nullptr, st), "moe_ffn_fp8 (down)");
    return y;
}

// ---- MXFP8 (1x32 e8m0 block scales) and the MoE path with power-of-two 128x128 scales
py::tuple mx_quant(py::object X) {
    TensorArg x = tensor_arg(X);
    const bool f32 = x.dtype == "torch.float32";
    if (!f32 && x.dtype != "torch.bfloat16") throw std::runtime_error("Expected dtype torch.bfloat16 or torch.float32, got " + x.dtype);
    if (x.shape.size() != 2) throw std::runtime_error("X must be [R, K]");
    const int R = static_cast<int>(x.shape[0]), K = static_cast<int>(x.shape[1]);
    if (K % 128 != 0) throw std::runtime_error("K must be a multiple of 128");
    py::object q = torch_empty({R, K}, "uint8", X);
    py::object s = torch_empty({R, K / 32}, "uint8", X);
    py::object atoms = torch_empty({(R + 127) / 128, K / 128, 512}, "uint8", X);
    throw_on(dk_mx_quant(x.ptr, f32 ? 1 : 0, R, K, tptr(q), tptr(s), tptr(atoms), current_stream()), "mx_quant");
    return py::make_tuple(q, s, atoms);
}

py::object gemm_mxfp8(py::object Aq, py::object Asf, py::object Bq, py::object Bsf, bool out_f32) {
    TensorArg a = tensor_arg(Aq, "torch.uint8"), sa = tensor_arg(Asf, "torch.uint8");
    TensorArg b = tensor_arg(Bq, "torch.uint8"), sb = tensor_arg(Bsf, "torch.uint8");
    if (a.shape.size() != 2 || b.shape.size() != 2 || a.shape[1] != b.shape[1])
        throw std::runtime_error("expected Aq [M,K] and Bq [N,K] e4m3 bytes");
    const int M = static_cast<int>(a.shape[0]), K = static_cast<int>(a.shape[1]), N = static_cast<int>(b.shape[0]);
    if (K % 128 != 0) throw std::runtime_error("K must be a multiple of 128");
    if (static_cast<size_t>(sa.numel()) < dk_mx_sf_bytes(M, K) || static_cast<size_t>(sb.numel()) < dk_mx_sf_bytes(N, K))
        throw std::runtime_error("scale atom arrays are too small for these operands");
    py::object c = torch_empty({M, N}, out_f32 ? "float32" : "bfloat16", Aq);
    throw_on(dk_gemm_mxfp8(a.ptr, sa.ptr, b.ptr, sb.ptr, tptr(c), M, N, K, out_f32 ? 1 : 0, current_stream()),
             "gemm_mxfp8");
    return c;
}

py::tuple moe_quant_pow2(py::object X, py::object row_map, int map_mode, int k) {
    TensorArg x = tensor_arg(X, "torch.bfloat16");
    if (x.shape.size() != 2) throw std::runtime_error("X must be [rows, C]");
    const int C = static_cast<int>(x.shape[1]);
    int R = static_cast<int>(x.shape[0]);
    const int* map = nullptr;
    if (!row_map.is_none()) {
        TensorArg m = tensor_arg(row_map, "torch.int32");
        map = static_cast<const int*>(m.ptr);
        R = static_cast<int>(m.numel());
        if (map_mode == 0) map_mode = 1;
    }
    py::object q = torch_empty({R, C}, "uint8", X);
    py::object e8 = torch_empty({R / 128, C / 128}, "uint8", X);
    py::object atoms = torch_empty({R / 128, (C / 128 + 3) / 4, 512}, "uint8", X);
    throw_on(dk_quant_block128_pow2(x.ptr, R, C, map, map_mode, k, tptr(q), nullptr, tptr(e8), tptr(atoms),
                                    current_stream()), "moe_quant_pow2");
    return py::make_tuple(q, e8, atoms);
}

py::object moe_ffn_mxfp8(py::object Xq, py::object Xa, py::object W13q, py::object W13a, py::object W2q,
                         py::object W2a, py::object offsets) {
    TensorArg xq = tensor_arg(Xq, "torch.uint8"), xa = tensor_arg(Xa, "torch.uint8");
    TensorArg w13q = tensor_arg(W13q, "torch.uint8"), w13a = tensor_arg(W13a, "torch.uint8");
    TensorArg w2q = tensor_arg(W2q, "torch.uint8"), w2a = tensor_arg(W2a, "torch.uint8");
    TensorArg off = tensor_arg(offsets, "torch.int32");
    if (xq.shape.size() != 2 || w13q.shape.size() != 3 || w2q.shape.size() != 3)
        throw std::runtime_error("expected Xq [R,H], W13q [E,2F,H], W2q [E,H,F]");
    const int R = static_cast<int>(xq.shape[0]), H = static_cast<int>(xq.shape[1]);
    const int E = static_cast<int>(w13q.shape[0]), F = static_cast<int>(w13q.shape[1] / 2);
    if (w13q.shape[2] != H || w2q.shape[0] != E || w2q.shape[1] != H || w2q.shape[2] != F || off.numel() != E + 1)
        throw std::runtime_error("MoE weight / offset shapes disagree");
    const int64_t hk = (H / 128 + 3) / 4, fk = (F / 128 + 3) / 4;  // atoms per 128-row block
    if (xa.numel() != static_cast<int64_t>(R / 128) * hk * 512 ||
        w13a.numel() != static_cast<int64_t>(E) * (2 * F / 128) * hk * 512 ||
        w2a.numel() != static_cast<int64_t>(E) * (H / 128) * fk * 512)
        throw std::runtime_error("scale atom arrays do not match the operands");
    py::object hq = torch_empty({R, F}, "uint8", Xq);
    py::object he = torch_empty({R / 128, F / 128}, "uint8", Xq);
    py::object ha = torch_empty({R / 128, fk, 512}, "uint8", Xq);
    py::object y = torch_empty({R, H}, "bfloat16", Xq);
    void* st = current_stream();
    throw_on(dk_moe_grouped_gemm_mxfp8(xq.ptr, xa.ptr, w13q.ptr, w13a.ptr, static_cast<const int*>(off.ptr), E, R, F,
                                       H, 1, tptr(hq), tptr(he), tptr(ha), st), "moe_ffn_mxfp8 (gate/up)");
    throw_on(dk_moe_grouped_gemm_mxfp8(tptr(hq), tptr(ha), w2q.ptr, w2a.ptr, static_cast<const int*>(off.ptr), E, R,
                                       H, F, 0, tptr(y), nullptr, nullptr, st), "moe_ffn_mxfp8 (down)");
    return y;
}

void moe_dispatch(py::object X, py::object topk_idx, py::object row_of_pair, int experts_per_rank,
                  py::object Xrecv, py::object view) {
    TensorArg x = tensor_arg(X, "torch.bfloat16"), ti = tensor_arg(topk_idx, "torch.int32");
    TensorArg rp = tensor_arg(row_of_pair, "torch.int32"), xr = tensor_arg(Xrecv, "torch.bfloat16");
    if (x.shape.size() != 2 || ti.shape.size() != 2 || rp.numel() != ti.numel())
        throw std::runtime_error("expected X [T_loc,H], topk_idx [T_loc,k], row_of_pair [T_loc,k]");
    throw_on(dk_moe_dispatch(x.ptr, static_cast<const int*>(ti.ptr), static_cast<const int*>(rp.ptr),
                             static_cast<int>(ti.shape[0]), static_cast<int>(ti.shape[1]),
                             static_cast<int>(x.shape[1]), experts_per_rank, xr.ptr, view_arg(view), 1,
                             current_stream()), "moe_dispatch");
}

py::object moe_combine(py::object Y, py::object topk_idx, py::object row_of_pair, py::object topk_w,
                       int experts_per_rank, py::object view) {
    TensorArg y = tensor_arg(Y, "torch.bfloat16"), ti = tensor_arg(topk_idx, "torch.int32");
    TensorArg rp = tensor_arg(row_of_pair, "torch.int32"), w = tensor_arg(topk_w, "torch.float32");
    if (y.shape.size() != 2 || ti.shape.size() != 2 || rp.numel() != ti.numel() || w.numel() != ti.numel())
        throw std::runtime_error("expected Y [R,H], topk_idx / row_of_pair / topk_w [T_loc,k]");
    const int T = static_cast<int>(ti.shape[0]), k = static_cast<int>(ti.shape[1]), H = static_cast<int>(y.shape[1]);
    py::object out = torch_empty({T, H}, "bfloat16", Y);
    const dk_view* v = view_arg(view);
    if (v == nullptr || v->world <= 1) {
        throw_on(dk_moe_combine(y.ptr, static_cast<const int*>(rp.ptr), static_cast<const float*>(w.ptr), T, k, H,
                                tptr(out), current_stream()), "moe_combine");
    } else {
        throw_on(dk_moe_combine_ep(y.ptr, static_cast<const int*>(ti.ptr), static_cast<const int*>(rp.ptr),
                                   static_cast<const float*>(w.ptr), T, k, H, experts_per_rank, tptr(out), v, 1,
                                   current_stream()), "moe_combine");
    }
    return out;
}

// One expert-parallel MoE layer through a single call (dk_moe_ep_layer). `Workspace` is a uint8 tensor
// of moe_ep_workspace_bytes(...) bytes; with more than one rank it must come from the symmetric heap
// (iris.empty([bytes], "uint8")), allocated at the same point of every rank's program.
int64_t moe_ep_workspace_bytes(int T_loc, int k, int E, int H, int F, int world) {
    return static_cast<int64_t>(dk_moe_ep_workspace_bytes(T_loc, k, E, H, F, world));
}

py::object moe_layer_ep(py::object X, py::object logits, int k, py::object W13q, py::object W13s, py::object W2q,
                        py::object W2s, py::object Out, py::object Workspace, py::object view, int scale_mode,
                        py::object counts, bool device_epoch) {
    TensorArg x = tensor_arg(X, "torch.bfloat16"), lg = tensor_arg(logits, "torch.float32");
    TensorArg w13q = tensor_arg(W13q, "torch.uint8"), w2q = tensor_arg(W2q, "torch.uint8");
    TensorArg w13s = tensor_arg(W13s, scale_mode != 0 ? "torch.uint8" : "torch.float32");
    TensorArg w2s = tensor_arg(W2s, scale_mode != 0 ? "torch.uint8" : "torch.float32");
    TensorArg out = tensor_arg(Out, "torch.bfloat16"), ws = tensor_arg(Workspace, "torch.uint8");
    if (x.shape.size() != 2 || lg.shape.size() != 2 || w13q.shape.size() != 3 || w2q.shape.size() != 3)
        throw std::runtime_error("expected X [T_loc,H], logits [T_loc,E], W13q [E/P,2F,H], W2q [E/P,H,F]");
    const dk_view* v = view_arg(view);
    const int world = v ? v->world : 1;
    dk_moe_ep_args a{};
    a.T_loc = static_cast<int>(x.shape[0]);
    a.H = static_cast<int>(x.shape[1]);
    a.E = static_cast<int>(lg.shape[1]);
    a.k = k;
    a.F = static_cast<int>(w2q.shape[2]);
    a.scale_mode = scale_mode;
    if (lg.shape[0] != a.T_loc || w13q.shape[0] * world != a.E || w13q.shape[1] != 2 * a.F || w13q.shape[2] != a.H ||
        w2q.shape[0] * world != a.E || w2q.shape[1] != a.H || out.numel() != x.numel())
        throw std::runtime_error("MoE layer shapes disagree");
    const size_t need = dk_moe_ep_workspace_bytes(a.T_loc, a.k, a.E, a.H, a.F, world);
    if (need == 0) throw std::runtime_error("unsupported MoE layer shape");
    if (static_cast<size_t>(ws.numel()) < need)
        throw std::runtime_error("workspace too small: " + std::to_string(ws.numel()) + " < " + std::to_string(need));
    a.x = x.ptr;
    a.logits = static_cast<const float*>(lg.ptr);
    a.w13q = w13q.ptr;
    a.w13s = w13s.ptr;
    a.w2q = w2q.ptr;
    a.w2s = w2s.ptr;
    a.out = out.ptr;
    a.workspace = ws.ptr;
    a.counts_out = nullptr;
    if (!counts.is_none()) {
        TensorArg c = tensor_arg(counts, "torch.int32");
        if (c.numel() * world != a.E) throw std::runtime_error("counts must hold E / world entries");
        a.counts_out = static_cast<int*>(c.ptr);
    }
    throw_on(dk_moe_ep_layer(&a, v, device_epoch ? DK_EPOCH_DEVICE : 0u, 15, current_stream()), "moe_layer_ep");
    return Out;
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
    m.def("dispatch_micro", &dispatch_micro3,
          "C[M,N] = A[M,K] @ Bt[N,K]^T (bf16, fp32 accumulate), the single-GPU form. Positional: A, Bt, C");
    m.def("gemm_rs", &gemm_rs,
          "Out[M/P,N] = reduce-scatter over ranks of A[M,K/P] @ Bt[N,K/P]^T. Positional: A, Bt, Out, view");
    m.def("ag_gemm", &ag_gemm,
          "C[M,N] = (all-gather over ranks of A[M/P,K]) @ Bt[N,K]^T, gather fused into the GEMM. Positional: A, Bt, C, view");
    m.def("allreduce", &allreduce, py::arg("X"), py::arg("Out"), py::arg("view"), py::arg("algo") = -1,
          "Out = sum over ranks of X (bf16). algo: -1 auto, 0 one-shot, 1 two-shot, 2 NVLS");
    m.def("moe_route", &moe_route, "(topk_idx int32 [T,k], topk_w fp32 [T,k]) from fp32 logits [T,E]");
    m.def("moe_permute", &moe_permute, py::arg("topk_idx"), py::arg("E"), py::arg("pad") = 128,
          py::arg("experts_per_segment") = 0,
          "(row_of_pair, pair_of_row, expert_offsets, counts), int32, deterministic");
    m.def("moe_quant", &moe_quant, py::arg("X"), py::arg("row_map") = py::none(), py::arg("map_mode") = 0,
          py::arg("k") = 1, "(Xq e4m3 bytes, Xs fp32) with 128x128 block scales; optional row gather");
    m.def("moe_ffn_fp8", &moe_ffn_fp8,
          "Y[R,H] bf16 from Xq, Xs, W13q[E,2F,H], W13s, W2q[E,H,F], W2s, expert_offsets");
    m.def("mx_quant", &mx_quant, "(q e4m3 bytes [R,K], s e8m0 [R,K/32], scale atoms) from bf16 or fp32 X, 1x32 blocks");
    m.def("gemm_mxfp8", &gemm_mxfp8, py::arg("Aq"), py::arg("Asf"), py::arg("Bq"), py::arg("Bsf"),
          py::arg("out_f32") = false, "C[M,N] = dequant(A) @ dequant(B)^T, e4m3 with 1x32 e8m0 scale atoms");
    m.def("moe_quant_pow2", &moe_quant_pow2, py::arg("X"), py::arg("row_map") = py::none(), py::arg("map_mode") = 0,
          py::arg("k") = 1, "(Xq e4m3 bytes, e8m0 per 128x128 block, scale atoms) with power-of-two block scales");
    m.def("moe_ffn_mxfp8", &moe_ffn_mxfp8,
          "Y[R,H] bf16 from Xq, X atoms, W13q[E,2F,H], W13 atoms, W2q[E,H,F], W2 atoms, expert_offsets "
          "(power-of-two block scales applied by the tensor core)");
    m.def("moe_dispatch", &moe_dispatch, "push local tokens into the destination ranks' receive rows");
    m.def("moe_combine", &moe_combine, "Out[T_loc,H] = sum_j w_j * Y_dest[row_j]; pulls from peers when world > 1");
    m.def("moe_ep_workspace_bytes", &moe_ep_workspace_bytes, "bytes of workspace moe_layer_ep needs");
    m.def("moe_layer_ep", &moe_layer_ep, py::arg("X"), py::arg("logits"), py::arg("k"), py::arg("W13q"),
          py::arg("W13s"), py::arg("W2q"), py::arg("W2s"), py::arg("Out"), py::arg("Workspace"), py::arg("view"),
          py::arg("scale_mode") = 0, py::arg("counts") = py::none(), py::arg("device_epoch") = false,
          "One fp8 MoE layer, expert-parallel over the ranks of the view, in one call: route, exchange, "
          "dispatch (once per token and GPU), quantise, gate/up + SiLU*mul, down, combine. "
          "scale_mode 0: fp32 block scales; 1: power-of-two block scales on the block-scaled MMA; "
          "2: as 1, tokens quantised per 128 channels at home and dispatched as fp8. device_epoch: the call "
          "number lives in device memory, so the call can be captured into a CUDA graph (after one eager call) "
          "and replayed, every rank the same number of times");
    m.def("device_status", &device_status,
          "(code, block, site, detail) of the first device-side wait that gave up; clears it");
}
