// pybind module torch_spyre._C: same names as the reference's module
// (torch_spyre/csrc/module.cpp:174-204): start_runtime, free_runtime, launch_kernel,
// SpyreTensorLayout with its StickFormat enum.  The runtime underneath is CUDA.
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <mutex>
#include <sstream>

#include "../../../include/spyre_b200.h"
#include "spyre_storage.h"

namespace spyre {

void register_hooks();  // spyre_backend.cpp

namespace {

// SpyreTensorLayout, as torch_spyre/csrc/spyre_tensor_impl.h:29-93.
struct SpyreTensorLayout {
  enum StickFormat { Dense = 0, Sparse, SparseMulti };
  std::vector<int64_t> device_size, device_strides;
  std::vector<int32_t> dim_map;
  int32_t num_stick_dims = 1;
  StickFormat format = Dense;

  SpyreTensorLayout(std::vector<int64_t> host_size, c10::ScalarType dtype) {
    std::vector<int32_t> order(host_size.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = (int32_t)i;
    init(host_size, dtype, order, Dense);
  }
  SpyreTensorLayout(std::vector<int64_t> host_size, c10::ScalarType dtype,
                    std::vector<int32_t> dim_order, StickFormat fmt = Dense) {
    init(host_size, dtype, dim_order, fmt);
  }
  SpyreTensorLayout(std::vector<int64_t> size, std::vector<int64_t> strides, std::vector<int32_t> map,
                    int32_t nstick, StickFormat fmt)
      : device_size(std::move(size)), device_strides(std::move(strides)), dim_map(std::move(map)),
        num_stick_dims(nstick), format(fmt) {}

  void init(const std::vector<int64_t>& host_size, c10::ScalarType dtype,
            const std::vector<int32_t>& dim_order, StickFormat fmt) {
    const int rank = (int)host_size.size();
    TORCH_CHECK(rank >= 1 && rank + 1 <= TS_MAX_DIMS, "Unsupported tensor rank: ", rank);
    TORCH_CHECK((int)dim_order.size() == rank, "dim_order must have one entry per host dim");
    device_size.assign(rank + 1, 0);
    device_strides.assign(rank + 1, 0);
    dim_map.assign(rank + 1, 0);
    const int n = ts_layout_init(host_size.data(), rank, (int)c10::elementSize(dtype), dim_order.data(),
                                 device_size.data(), device_strides.data(), dim_map.data());
    TORCH_CHECK(n == rank + 1, "ts_layout_init failed: ", ts_status_string(n));
    format = fmt;
    num_stick_dims = 1;
  }

  std::string to_string() const {  // spyre_tensor_impl.cpp:76-111
    auto list = [](const auto& v) {
      std::string out;
      for (size_t i = 0; i < v.size(); ++i) {
        out += std::to_string(v[i]);
        if (i + 1 < v.size()) out += ", ";
      }
      return out;
    };
    std::string s = "SpyreTensorLayout(device_size=[" + list(device_size) + "], device_strides=[" +
                    list(device_strides) + "], dim_map =[" + list(dim_map) +
                    "], num_stick_dims=" + std::to_string(num_stick_dims) + ", format=\"";
    s += format == Dense ? "Dense" : (format == Sparse ? "Sparse" : "SparseMulti");
    s += "\")";
    return s;
  }
};

std::once_flag g_runtime_once;
bool g_runtime_started = false;

void start_runtime() {
  std::call_once(g_runtime_once, [] {
    register_debug_flag();
    register_hooks();
    g_runtime_started = true;
  });
}
void free_runtime() {}

// launch_kernel(spec, args): the reference deserialises a compiled graph and runs it
// (torch_spyre/csrc/module.cpp:64-170).  Here a kernel spec is resolved to a C-ABI call
// by the Python runtime, which registers its dispatcher once at import.
py::object& kernel_launcher() {
  static py::object* fn = new py::object(py::none());
  return *fn;
}

}  // namespace
}  // namespace spyre

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using spyre::SpyreTensorLayout;
  m.doc() = "Spyre C++ bindings (CUDA-backed)";
  m.def("start_runtime", &spyre::start_runtime);
  m.def("free_runtime", &spyre::free_runtime);
  m.def("set_kernel_launcher", [](py::object fn) { spyre::kernel_launcher() = std::move(fn); });
  m.def("launch_kernel", [](py::object spec, py::object args) {
    TORCH_CHECK(!spyre::kernel_launcher().is_none(), "no kernel launcher registered");
    return spyre::kernel_launcher()(spec, args);
  });
  m.def("is_available", [] { return c10::cuda::device_count() > 0; });
  m.def("device_count", [] { return (int)c10::cuda::device_count(); });
  m.def("current_device", [] { return (int)c10::cuda::current_device(); });
  m.def("set_device", [](int i) { c10::cuda::set_device((c10::DeviceIndex)i); });
  m.def("synchronize", [](int i) {
    c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)(i < 0 ? c10::cuda::current_device() : i))
        .synchronize();
  });
  // helpers for the Python op layer
  m.def("is_canonical", &spyre::is_canonical);
  // test hook: False sends device-to-device copies of views through the two-pass route
  m.def("set_restickify_enabled", &spyre::set_restickify_enabled);
  m.def("base_shape", [](const at::Tensor& t) { return spyre::storage_ctx(t)->base_shape; });
  m.def("storage_ptr", [](const at::Tensor& t) { return (uintptr_t)spyre::storage_ctx(t)->ptr; });
  m.def("storage_as_cuda_bytes", &spyre::storage_as_cuda_bytes);
  m.def("stick_nbytes", [](std::vector<int64_t> shape, int64_t elem_bytes) {
    return spyre::stick_nbytes(shape, elem_bytes);
  });

  py::class_<SpyreTensorLayout> layout(m, "SpyreTensorLayout");
  py::enum_<SpyreTensorLayout::StickFormat>(layout, "StickFormat")
      .value("Dense", SpyreTensorLayout::Dense)
      .value("Sparse", SpyreTensorLayout::Sparse)
      .value("SparseMulti", SpyreTensorLayout::SparseMulti);
  layout
      .def(py::init([](std::vector<int64_t> host_size, py::object dtype) {
             return SpyreTensorLayout(host_size, torch::python::detail::py_object_to_dtype(dtype));
           }),
           py::arg("host_size"), py::arg("dtype"))
      .def(py::init([](std::vector<int64_t> host_size, py::object dtype, std::vector<int32_t> order,
                       SpyreTensorLayout::StickFormat fmt) {
             return SpyreTensorLayout(host_size, torch::python::detail::py_object_to_dtype(dtype),
                                      order, fmt);
           }),
           py::arg("host_size"), py::arg("dtype"), py::arg("dim_order"),
           py::arg("format") = SpyreTensorLayout::Dense)
      .def(py::init<std::vector<int64_t>, std::vector<int64_t>, std::vector<int32_t>, int32_t,
                    SpyreTensorLayout::StickFormat>(),
           py::arg("device_size"), py::arg("device_strides"), py::arg("dim_map"),
           py::arg("num_stick_dims"), py::arg("format"))
      .def_readwrite("device_size", &SpyreTensorLayout::device_size)
      .def_readwrite("device_strides", &SpyreTensorLayout::device_strides)
      .def_readwrite("dim_map", &SpyreTensorLayout::dim_map)
      .def_readwrite("num_stick_dims", &SpyreTensorLayout::num_stick_dims)
      .def_readwrite("format", &SpyreTensorLayout::format)
      .def("__str__", &SpyreTensorLayout::to_string)
      .def("__repr__", &SpyreTensorLayout::to_string);
}
