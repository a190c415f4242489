// pybind11 / torch extension over the C ABI: the binding a maintainer of the reference would put
// in place of the bodies of src/aihwkit/simulator/rpu_base_src/rpu_base_tiles_cuda.cpp, compiled.
// The bound class keeps an ab200_tile handle where the reference keeps an RPUCudaPulsed<float>;
// every method is the reference's lambda of the same name with its call into the tile replaced by
// the C-ABI entry point (cited per method). Only `include/aihwkit_b200.h` is used: no header of
// the library's own C++ classes.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "aihwkit_b200.h"

namespace {

void check(int code) {
  if (code != 0) {
    throw std::runtime_error(ab200_last_error());
  }
}

const float *fptr(const torch::Tensor &t) { return t.data_ptr<float>(); }

struct B200Tile {
  ab200_tile *h = nullptr;
  int device = -1;

  // the configuration struct travels as bytes (ab200_tile_config, checked against the library's
  // own sizeof); createRPUArray + the CudaAnalogTile constructor, rpu_base_devices.cpp:453-467,
  // rpu_base_tiles_cuda.cpp:532-538
  B200Tile(const py::bytes &config, int cuda_device) : device(cuda_device) {
    const std::string raw = config;
    if (raw.size() != ab200_sizeof(4) || raw.size() != sizeof(ab200_tile_config)) {
      throw std::runtime_error("ab200_tile_config: size mismatch between the caller and the library");
    }
    ab200_tile_config cfg;
    std::memcpy(&cfg, raw.data(), sizeof(cfg));
    check(ab200_tile_create(&cfg, cuda_device, &h));
  }
  ~B200Tile() { ab200_tile_destroy(h); }
  B200Tile(const B200Tile &) = delete;
  B200Tile &operator=(const B200Tile &) = delete;

  int x_size() const { return ab200_tile_get_x_size(h); }
  int d_size() const { return ab200_tile_get_d_size(h); }

  void expect(const torch::Tensor &t, const char *what) const {
    if (!t.is_cuda() || t.get_device() != device || t.scalar_type() != torch::kFloat32) {
      throw std::runtime_error(std::string(what) + ": expected a float32 CUDA tensor on the tile's device");
    }
  }

  // rpu_base_tiles_cuda.cpp:160-205
  torch::Tensor forward(const torch::Tensor &x_input, bool bias, bool x_trans, bool d_trans, bool is_test,
                        bool non_blocking) {
    expect(x_input, "forward");
    auto x = x_input.contiguous();
    const int in_size = (int)(x_trans ? x.size(0) : x.size(-1));
    if (in_size != x_size() - (bias ? 1 : 0)) {
      throw std::runtime_error("x_input size mismatch");
    }
    const int m_batch = (int)(x.numel() / in_size);
    std::vector<int64_t> dims(x.sizes().begin(), x.sizes().end());
    dims[d_trans ? 0 : dims.size() - 1] = d_size();
    torch::Tensor d = torch::empty(dims, x.options());
    auto stream = at::cuda::getCurrentCUDAStream(device);
    check(ab200_tile_forward(h, fptr(x), d.data_ptr<float>(), bias, m_batch, x_trans, d_trans, is_test,
                             stream.stream()));
    if (!non_blocking) {
      stream.synchronize();
    }
    return d;
  }

  // rpu_base_tiles_cuda.cpp:217-262
  torch::Tensor backward(const torch::Tensor &d_input, bool bias, bool d_trans, bool x_trans, bool non_blocking) {
    expect(d_input, "backward");
    auto d = d_input.contiguous();
    const int out_size = (int)(d_trans ? d.size(0) : d.size(-1));
    if (out_size != d_size()) {
      throw std::runtime_error("d_input size mismatch");
    }
    const int m_batch = (int)(d.numel() / out_size);
    std::vector<int64_t> dims(d.sizes().begin(), d.sizes().end());
    dims[x_trans ? 0 : dims.size() - 1] = x_size() - (bias ? 1 : 0);
    torch::Tensor x = torch::empty(dims, d.options());
    auto stream = at::cuda::getCurrentCUDAStream(device);
    check(ab200_tile_backward(h, fptr(d), x.data_ptr<float>(), bias, m_batch, d_trans, x_trans, stream.stream()));
    if (!non_blocking) {
      stream.synchronize();
    }
    return x;
  }

  // rpu_base_tiles_cuda.cpp:274-330
  void update(const torch::Tensor &x_input, const torch::Tensor &d_input, bool bias, bool x_trans, bool d_trans,
              bool non_blocking) {
    expect(x_input, "update");
    expect(d_input, "update");
    auto x = x_input.contiguous();
    auto d = d_input.contiguous();
    const int in_size = (int)(x_trans ? x.size(0) : x.size(-1));
    const int m_batch = (int)(x.numel() / in_size);
    auto stream = at::cuda::getCurrentCUDAStream(device);
    check(ab200_tile_update(h, fptr(x), fptr(d), bias, m_batch, x_trans, d_trans, stream.stream()));
    if (!non_blocking) {
      stream.synchronize();
    }
  }

  // rpu_base_tiles.cpp:150-205
  void set_weights(const torch::Tensor &w) {
    auto c = w.detach().cpu().contiguous().to(torch::kFloat32);
    if (c.dim() != 2 || c.size(0) != d_size() || c.size(1) != x_size()) {
      throw std::runtime_error("Invalid weights dimensions: expected [d_size, x_size] array");
    }
    check(ab200_tile_set_weights(h, fptr(c)));
  }
  torch::Tensor get_weights() {
    torch::Tensor w = torch::empty({d_size(), x_size()}, torch::kFloat32);
    check(ab200_tile_get_weights(h, w.data_ptr<float>()));
    return w;
  }
  void set_learning_rate(float lr) { check(ab200_tile_set_learning_rate(h, lr)); }
  float get_learning_rate() {
    float lr = 0.0f;
    check(ab200_tile_get_learning_rate(h, &lr));
    return lr;
  }

  // rpu_base_tiles.cpp:764-825
  std::vector<std::string> get_hidden_parameter_names() {
    std::vector<std::string> names;
    const int n = ab200_tile_hidden_parameter_count(h);
    for (int k = 0; k < n; k++) {
      names.emplace_back(ab200_tile_hidden_parameter_name(h, k));
    }
    return names;
  }
  torch::Tensor get_hidden_parameters() {
    const int n = ab200_tile_hidden_parameter_count(h);
    torch::Tensor p = torch::empty({n, d_size(), x_size()}, torch::kFloat32);
    if (n > 0) {
      check(ab200_tile_get_hidden_parameters(h, p.data_ptr<float>()));
    }
    return p;
  }
  void set_hidden_parameters(const torch::Tensor &p) {
    auto c = p.detach().cpu().contiguous().to(torch::kFloat32);
    const int n = ab200_tile_hidden_parameter_count(h);
    if (c.dim() != 3 || c.size(0) != n || c.size(1) != d_size() || c.size(2) != x_size()) {
      throw std::runtime_error("Invalid hidden parameter dimensions");
    }
    if (n > 0) {
      check(ab200_tile_set_hidden_parameters(h, fptr(c)));
    }
  }
};

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "pybind11 binding of the B200 analog tile over its C ABI";
  m.def("version", []() { return std::string(ab200_version()); });
  py::class_<B200Tile>(m, "CudaAnalogTile")
      .def(py::init<const py::bytes &, int>(), py::arg("config"), py::arg("cuda_device") = 0)
      .def("get_x_size", &B200Tile::x_size)
      .def("get_d_size", &B200Tile::d_size)
      .def("forward", &B200Tile::forward, py::arg("x_input"), py::arg("bias") = false, py::arg("x_trans") = false,
           py::arg("d_trans") = false, py::arg("is_test") = false, py::arg("non_blocking") = false)
      .def("backward", &B200Tile::backward, py::arg("d_input"), py::arg("bias") = false,
           py::arg("d_trans") = false, py::arg("x_trans") = false, py::arg("non_blocking") = false)
      .def("update", &B200Tile::update, py::arg("x_input"), py::arg("d_input"), py::arg("bias") = false,
           py::arg("x_trans") = false, py::arg("d_trans") = false, py::arg("non_blocking") = false)
      .def("set_weights", &B200Tile::set_weights)
      .def("get_weights", &B200Tile::get_weights)
      .def("set_learning_rate", &B200Tile::set_learning_rate)
      .def("get_learning_rate", &B200Tile::get_learning_rate)
      .def("get_hidden_parameter_names", &B200Tile::get_hidden_parameter_names)
      .def("get_hidden_parameters", &B200Tile::get_hidden_parameters)
      .def("set_hidden_parameters", &B200Tile::set_hidden_parameters);
}
