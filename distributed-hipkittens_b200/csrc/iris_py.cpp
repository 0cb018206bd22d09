// Python module `iris_py`: same classes, methods, defaults and error strings as the reference's
// distributed-kernels/iris_py.cpp:109-155, on top of the C ABI in include/dk_b200.h.
//
//   iris_py.Iris(heap_size_mb=1024, verbose=False)   .rank() .world_size() .barrier()
//                                                   .empty(shape, dtype="bfloat16") .get_device_view()
//   iris_py.Tensor           .data_ptr() .shape .dtype .numel() .nbytes()
//   iris_py.IrisDeviceView   .cur_rank() .world_size()
//   iris_py.mpi_init() -> (rank, world_size)        iris_py.mpi_finalize()
//
// Differences, all additive: no MPI is needed (rank and world size come from RANK/WORLD_SIZE or
// OMPI_COMM_WORLD_*; world 1 when unset); `empty` also accepts float8_e4m3fn / uint8 / int32;
// a Tensor keeps its heap alive (the reference keeps a raw pointer, iris_py.cpp:17,24, so that
// destroying Iris first is a use-after-free there); Tensor exposes __cuda_array_interface__ so that
// `torch.as_tensor(t, device="cuda")` is a zero-copy view.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dk_b200.h"

namespace py = pybind11;

static void throw_on(int rc, const char* what) {
    if (rc != DK_OK) {
        std::string msg = std::string(what) + ": " + dk_strerror(rc);
        const char* d = dk_last_error_string();
        if (d && *d) msg += std::string(" (") + d + ")";
        throw std::runtime_error(msg);
    }
}

// Owns the dk_heap; shared by the Iris object and every Tensor cut from it.
struct HeapHolder {
    dk_heap* h = nullptr;
    ~HeapHolder() {
        if (h) dk_heap_destroy(h);
    }
};

struct DkDeviceView {
    dk_view v{};
    std::shared_ptr<HeapHolder> keep;
    int cur_rank() const { return v.rank; }
    int world_size() const { return v.world; }
    uintptr_t addr() const { return reinterpret_cast<uintptr_t>(&v); }
};

class IrisTensor {
public:
    void* data;
    std::vector<int64_t> shape;
    size_t dtype_size;
    std::string dtype;
    std::shared_ptr<HeapHolder> heap;

    IrisTensor(void* ptr, std::vector<int64_t> s, size_t ds, const std::string& dt,
               std::shared_ptr<HeapHolder> hp)
        : data(ptr), shape(std::move(s)), dtype_size(ds), dtype(dt), heap(std::move(hp)) {}
    ~IrisTensor() {
        if (data && heap && heap->h) dk_heap_free(heap->h, data);
    }
    uintptr_t data_ptr() const { return reinterpret_cast<uintptr_t>(data); }
    std::vector<int64_t> get_shape() const { return shape; }
    std::string get_dtype() const { return dtype; }
    size_t numel() const {
        size_t total = 1;
        for (auto d : shape) total *= static_cast<size_t>(d);
        return total;
    }
    size_t nbytes() const { return numel() * dtype_size; }
    py::dict cuda_array_interface() const {
        std::string typestr;
        if (dtype == "float32" || dtype == "float") typestr = "<f4";
        else if (dtype == "float16" || dtype == "half") typestr = "<f2";
        else if (dtype == "int32") typestr = "<i4";
        else if (dtype_size == 1) typestr = "|u1";
        else typestr = "<u2";  // bfloat16 travels as uint16; view it as torch.bfloat16
        py::dict d;
        py::tuple shp(shape.size());
        for (size_t i = 0; i < shape.size(); ++i) shp[i] = py::int_(shape[i]);
        d["shape"] = shp;
        d["typestr"] = typestr;
        d["data"] = py::make_tuple(data_ptr(), false);
        d["version"] = 3;
        d["strides"] = py::none();
        return d;
    }
};

class IrisInstance {
    std::shared_ptr<HeapHolder> heap_;
    int rank_ = 0;
    int world_size_ = 1;
    bool verbose_ = false;

public:
    IrisInstance(size_t heap_size_mb = 1024, bool verbose = false) : verbose_(verbose) {
        int local = 0;
        throw_on(dk_bootstrap_env(&rank_, &world_size_, &local), "bootstrap");
        if (world_size_ > 1) {
            int ndev = 0;
            throw_on(dk_device_count(&ndev), "device count");
            if (ndev <= 0) throw std::runtime_error("no CUDA device");
            throw_on(dk_device_set(local % ndev), "set device");
        }
        heap_ = std::make_shared<HeapHolder>();
        // DK_HEAP_MB raises (never lowers) the heap size an unmodified script asks for: the fused
        // kernels take their workspaces from the same heap as the script's own tensors.
        if (const char* e = std::getenv("DK_HEAP_MB")) {
            const long long want = std::atoll(e);
            if (want > 0 && static_cast<size_t>(want) > heap_size_mb) heap_size_mb = static_cast<size_t>(want);
        }
        if (verbose_ && std::getenv("DK_LOG") == nullptr) dk_set_log_level(1);
        const size_t heap_size_bytes = heap_size_mb * 1024 * 1024;
        throw_on(dk_heap_create(heap_size_bytes, rank_, world_size_, nullptr, &heap_->h),
                 "Failed to create iris heap");
        if (verbose_)
            py::print("[iris_py] rank", rank_, "of", world_size_, "heap", heap_size_mb, "MiB");
    }

    int rank() const { return rank_; }
    int world_size() const { return world_size_; }

    std::shared_ptr<IrisTensor> empty(std::vector<int64_t> shape, const std::string& dtype = "bfloat16") {
        size_t total_elements = 1;
        for (auto dim : shape) {
            if (dim < 0) throw std::runtime_error("negative dimension");
            total_elements *= static_cast<size_t>(dim);
        }
        size_t dtype_size;
        if (dtype == "bfloat16" || dtype == "bf16") dtype_size = 2;
        else if (dtype == "float32" || dtype == "float") dtype_size = 4;
        else if (dtype == "float16" || dtype == "half") dtype_size = 2;
        else if (dtype == "float8_e4m3fn" || dtype == "uint8") dtype_size = 1;
        else if (dtype == "int32") dtype_size = 4;
        else throw std::runtime_error("Unsupported dtype: " + dtype);

        void* ptr = dk_heap_alloc(heap_->h, total_elements * dtype_size, 256);
        if (!ptr) throw std::runtime_error("Failed to allocate iris memory");
        return std::make_shared<IrisTensor>(ptr, shape, dtype_size, dtype, heap_);
    }

    void barrier() {
        throw_on(dk_device_synchronize(), "barrier");
        throw_on(dk_heap_barrier(heap_->h), "barrier");
    }

    DkDeviceView get_device_view() {
        DkDeviceView dv;
        throw_on(dk_heap_view(heap_->h, &dv.v), "get_device_view");
        dv.keep = heap_;
        return dv;
    }

    // Collective: map the NVLink multicast object over all ranks' heaps. False when unavailable.
    bool enable_multicast() {
        const int rc = dk_heap_enable_multicast(heap_->h);
        if (rc == DK_OK) return true;
        if (rc == DK_ERR_UNSUPPORTED) return false;
        throw_on(rc, "enable_multicast");
        return false;
    }

    uintptr_t heap_handle() const { return reinterpret_cast<uintptr_t>(heap_->h); }
};

PYBIND11_MODULE(iris_py, m) {
    m.doc() = "Iris Python bindings for distributed GPU memory management (B200 build)";

    py::class_<DkDeviceView>(m, "IrisDeviceView")
        .def("cur_rank", &DkDeviceView::cur_rank, "Get current rank")
        .def("world_size", &DkDeviceView::world_size, "Get world size")
        .def("_addr", &DkDeviceView::addr, "Address of the dk_view struct (valid while this object lives)");

    py::class_<IrisInstance, std::shared_ptr<IrisInstance>>(m, "Iris")
        .def(py::init<size_t, bool>(), py::arg("heap_size_mb") = 1024, py::arg("verbose") = false,
             "Create iris instance (rank and world size from the environment)\n\n"
             "Args:\n"
             "    heap_size_mb: Size of distributed heap in megabytes (default: 1024)\n"
             "    verbose: Enable verbose logging (default: False)")
        .def("rank", &IrisInstance::rank, "Get current rank")
        .def("world_size", &IrisInstance::world_size, "Get total number of ranks")
        .def("empty", &IrisInstance::empty, py::arg("shape"), py::arg("dtype") = "bfloat16",
             "Create empty tensor allocated with iris\n\n"
             "Args:\n"
             "    shape: Tuple or list of tensor dimensions\n"
             "    dtype: Data type ('bfloat16', 'float32', 'float16', 'float8_e4m3fn', 'uint8', 'int32')\n\n"
             "Returns:\n"
             "    IrisTensor: Iris tensor object")
        .def("barrier", &IrisInstance::barrier, "Synchronize the device, then all ranks")
        .def("get_device_view", &IrisInstance::get_device_view, "Get device view for kernel usage")
        .def("enable_multicast", &IrisInstance::enable_multicast,
             "Collective over all ranks: map the NVLink multicast object over the heaps (NVLS all-reduce).\n"
             "Returns False when the system has no multicast support. Not in the reference.")
        .def("_heap", &IrisInstance::heap_handle, "dk_heap* as an integer");

    py::class_<IrisTensor, std::shared_ptr<IrisTensor>>(m, "Tensor")
        .def("data_ptr", &IrisTensor::data_ptr, "Get raw data pointer as integer")
        .def_property_readonly("shape", &IrisTensor::get_shape, "Get tensor shape")
        .def_property_readonly("dtype", &IrisTensor::get_dtype, "Get tensor dtype")
        .def("numel", &IrisTensor::numel, "Get total number of elements")
        .def("nbytes", &IrisTensor::nbytes, "Get total size in bytes")
        .def_property_readonly("__cuda_array_interface__", &IrisTensor::cuda_array_interface);

    m.def("mpi_init", []() {
        int r = 0, w = 1, l = 0;
        throw_on(dk_bootstrap_env(&r, &w, &l), "mpi_init");
        return py::make_tuple(r, w);
    }, "Read (rank, world_size) from the environment");

    m.def("mpi_finalize", []() {}, "No-op: there is no MPI to finalize");
}
