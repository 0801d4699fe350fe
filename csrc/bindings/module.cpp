// pybind11 module `orthon_b200._C`: Tensor, Device, free operators, runtime diagnostics.
//
// Surface parity (reference project paths): bindings/module.cpp:28-96,
// bindings/tensor_bindings.cpp:349-787, bindings/ops_bindings.cpp:68-363.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "ob/ops.h"

namespace py = pybind11;
using namespace ob;

namespace ob {
namespace cu {
Tensor pinned_empty(const Shape& shape, DType dtype);
void copy_h2d_async(Tensor& dst, const Tensor& src, int stream_kind);
void copy_d2h_async(Tensor& dst, const Tensor& src);
unsigned int take_index_errors();
int take_gemm_error(int device);
void set_gemm_route(int route);
void set_float32_matmul_precision(int level);
int float32_matmul_precision();
int last_gemm_route();
void set_conv_route(int route);
int last_conv_route();
uint64_t kernel_launch_count();
}  // namespace cu
void bind_distributed(py::module_& m);
}  // namespace ob

namespace {

DType dtype_from_py(const py::object& o) {
  if (o.is_none()) return DType::F32;
  if (py::isinstance<py::str>(o)) return parse_dtype(o.cast<std::string>());
  return o.cast<DType>();
}

Device device_from_py(const py::object& o) {
  if (py::isinstance<py::str>(o)) return Device::parse(o.cast<std::string>());
  return o.cast<Device>();
}

Shape shape_from_py(const py::object& o) {
  if (py::isinstance<py::int_>(o)) return Shape{o.cast<int64_t>()};
  Shape s;
  for (auto h : o) s.push_back(py::cast<int64_t>(h));
  return s;
}

std::optional<int> opt_dim(const py::object& o) {
  if (o.is_none()) return std::nullopt;
  return o.cast<int>();
}

Tensor host_copy(const Tensor& t) {
  NoGradGuard g;
  Tensor c = t.device().is_cuda() ? ops::to(t.detach(), Device()) : ops::contiguous(t.detach());
  return c;
}

py::list tolist_flat(const Tensor& t) {
  Tensor h = host_copy(t);
  py::list out;
  const size_t esz = dtype_size(h.dtype());
  const char* p = static_cast<const char*>(h.data());
  const int64_t n = h.numel();
  const DType d = h.dtype();
  for (int64_t i = 0; i < n; ++i) {
    if (d == DType::Bool) out.append(py::bool_(p[i] != 0));
    else if (d == DType::I64) { int64_t v; std::memcpy(&v, p + i * 8, 8); out.append(py::int_(v)); }
    else if (!dtype_is_floating(d)) out.append(py::int_(static_cast<int64_t>(load_as_double(p + i * esz, d))));
    else out.append(py::float_(load_as_double(p + i * esz, d)));
  }
  return out;
}

py::object scalar_to_py(const Tensor& t) {
  if (t.numel() != 1) throw std::invalid_argument("item(): tensor must hold exactly one element");
  return tolist_flat(t)[0];
}

Tensor from_numpy(const py::array& arr_in, const py::object& dtype_o) {
  py::array arr = py::array::ensure(arr_in, py::array::c_style);
  if (!arr) throw std::invalid_argument("from_numpy: expected a C-contiguous numpy array");
  const py::dtype dt = arr.dtype();
  DType src;
  const char kind = dt.kind();
  const auto isz = dt.itemsize();
  if (kind == 'f' && isz == 4) src = DType::F32;
  else if (kind == 'f' && isz == 8) src = DType::F64;
  else if (kind == 'f' && isz == 2) src = DType::F16;
  else if (kind == 'i' && isz == 4) src = DType::I32;
  else if (kind == 'i' && isz == 8) src = DType::I64;
  else if (kind == 'u' && isz == 1) src = DType::U8;
  else if (kind == 'i' && isz == 1) src = DType::I8;
  else if (kind == 'b') src = DType::Bool;
  else throw std::invalid_argument("from_numpy: unsupported numpy dtype");
  Shape shape;
  for (py::ssize_t i = 0; i < arr.ndim(); ++i) shape.push_back(arr.shape(i));
  if (shape.empty()) shape = {1};
  Tensor t = Tensor::empty(shape, src, Device());
  if (t.numel()) std::memcpy(t.data(), arr.data(), t.nbytes());
  if (!dtype_o.is_none()) {
    const DType want = dtype_from_py(dtype_o);
    if (want != src) {
      NoGradGuard g;
      t = ops::cast(t, want);
    }
  }
  return t;
}

py::array to_numpy(const Tensor& t) {
  Tensor h = host_copy(t);
  if (h.dtype() == DType::BF16) {
    NoGradGuard g;
    h = ops::cast(h, DType::F32);
  }
  py::dtype dt;
  switch (h.dtype()) {
    case DType::F32: dt = py::dtype("float32"); break;
    case DType::F64: dt = py::dtype("float64"); break;
    case DType::F16: dt = py::dtype("float16"); break;
    case DType::I32: dt = py::dtype("int32"); break;
    case DType::I64: dt = py::dtype("int64"); break;
    case DType::U8: dt = py::dtype("uint8"); break;
    case DType::I8: dt = py::dtype("int8"); break;
    default: dt = py::dtype("bool"); break;
  }
  std::vector<py::ssize_t> shape(h.shape().begin(), h.shape().end());
  py::array out(dt, shape);
  if (h.numel()) std::memcpy(out.mutable_data(), h.data(), h.nbytes());
  return out;
}

py::bytes tensor_to_bytes(const Tensor& t) {
  Tensor h = host_copy(t);
  return py::bytes(static_cast<const char*>(h.data()), h.nbytes());
}

Tensor tensor_from_bytes(const py::bytes& b, const py::object& shape_o, const py::object& dtype_o) {
  const Shape shape = shape_from_py(shape_o);
  const DType d = dtype_from_py(dtype_o);
  const std::string s = b;
  const int64_t n = Layout::checked_numel(shape);
  if (static_cast<size_t>(n) * dtype_size(d) != s.size())
    throw std::invalid_argument("_tensor_from_bytes: byte count does not match shape and dtype");
  Tensor t = Tensor::empty(shape, d, Device());
  if (n) std::memcpy(t.data(), s.data(), s.size());
  return t;
}

Tensor targets_from_py(const py::object& o) {
  if (py::isinstance<Tensor>(o)) return o.cast<Tensor>();
  std::vector<int64_t> v = o.cast<std::vector<int64_t>>();
  Tensor t = Tensor::empty({static_cast<int64_t>(v.size())}, DType::I64, Device());
  if (!v.empty()) std::memcpy(t.data(), v.data(), v.size() * 8);
  return t;
}

py::object numel_object(int64_t n) {
  static py::object cls = py::module_::import("orthon_b200._numel").attr("_Numel");
  return cls(n);
}

Tensor getitem(const Tensor& t, const py::object& key) {
  if (py::isinstance<py::int_>(key)) return ops::index(t, key.cast<int64_t>());
  if (py::isinstance<py::tuple>(key)) {
    Tensor cur = t;
    for (auto h : key.cast<py::tuple>()) {
      if (!py::isinstance<py::int_>(h)) throw py::type_error("Tensor indices must be integers");
      cur = ops::index(cur, py::cast<int64_t>(h));
    }
    return cur;
  }
  throw py::type_error("Tensor indices must be integers");
}

void setitem(Tensor& t, const py::object& key, double value) {
  if (grad_enabled() && t.requires_grad() && !t.is_leaf())
    throw std::runtime_error("__setitem__: in-place modification of a tensor with autograd history is only allowed under no_grad()");
  NoGradGuard g;
  Tensor view = getitem(t, key);
  const bool full_index = (py::isinstance<py::tuple>(key) ? static_cast<int>(key.cast<py::tuple>().size()) : 1) == t.ndim();
  if (t.device().is_cuda() && !full_index) throw std::invalid_argument("__setitem__: CUDA tensors require a full index");
  ops::fill_raw(view, value);
  t.bump_version();
}

int64_t flat_index(const Tensor& t, const py::object& key) {
  if (py::isinstance<py::int_>(key)) return key.cast<int64_t>();
  std::vector<int64_t> idx = key.cast<std::vector<int64_t>>();
  if (static_cast<int>(idx.size()) != t.ndim()) throw std::invalid_argument("index rank does not match the tensor");
  int64_t flat = 0;
  for (int d = 0; d < t.ndim(); ++d) {
    int64_t i = idx[d];
    if (i < 0) i += t.shape()[d];
    if (i < 0 || i >= t.shape()[d]) throw std::out_of_range("index out of range");
    flat = flat * t.shape()[d] + i;
  }
  return flat;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "orthon_b200 native runtime (sm_100a)";

  py::enum_<DType>(m, "DType")
      .value("float32", DType::F32).value("float64", DType::F64).value("float16", DType::F16)
      .value("bfloat16", DType::BF16).value("int32", DType::I32).value("int64", DType::I64)
      .value("uint8", DType::U8).value("int8", DType::I8).value("bool", DType::Bool);
  py::enum_<DeviceType>(m, "DeviceType").value("CPU", DeviceType::CPU).value("CUDA", DeviceType::CUDA);

  py::class_<Device>(m, "Device")
      .def(py::init([](const std::string& s) { return Device::parse(s); }))
      .def(py::init([](DeviceType t, int i) { return Device(t, i); }), py::arg("type"), py::arg("index") = 0)
      .def_property_readonly("type", [](const Device& d) { return d.type; })
      .def_property_readonly("index", [](const Device& d) { return d.index; })
      .def("is_cuda", &Device::is_cuda)
      .def("is_cpu", &Device::is_cpu)
      .def("__str__", &Device::str)
      .def("__repr__", [](const Device& d) { return "Device('" + d.str() + "')"; })
      .def("__hash__", [](const Device& d) { return std::hash<std::string>()(d.str()); })
      .def("__eq__", [](const Device& d, const py::object& o) {
        if (py::isinstance<Device>(o)) return d == o.cast<Device>();
        if (py::isinstance<py::str>(o)) {
          try { return d == Device::parse(o.cast<std::string>()); } catch (...) { return false; }
        }
        return false;
      });

  py::class_<Tensor> T(m, "Tensor");
  T.attr("__array_ufunc__") = py::none();
  T.def_property_readonly("shape", [](const Tensor& t) { return py::tuple(py::cast(t.shape())); })
      .def_property_readonly("strides", [](const Tensor& t) { return py::tuple(py::cast(t.strides())); })
      .def_property_readonly("numel", [](const Tensor& t) { return numel_object(t.numel()); })
      .def_property_readonly("ndim", &Tensor::ndim)
      .def_property_readonly("is_contiguous", &Tensor::is_contiguous)
      .def_property_readonly("dtype", [](const Tensor& t) { return std::string(dtype_name(t.dtype())); })
      .def_property_readonly("storage_offset", &Tensor::offset)
      .def_property_readonly("device", &Tensor::device)
      .def_property("requires_grad", &Tensor::requires_grad, [](Tensor& t, bool on) { t.requires_grad_(on); })
      .def_property_readonly("is_leaf", &Tensor::is_leaf)
      .def_property_readonly("grad", [](const Tensor& t) -> py::object {
        Tensor g = t.grad();
        if (!g.defined()) return py::none();
        return py::cast(g);
      })
      .def_property_readonly("_impl_id", [](const Tensor& t) { return reinterpret_cast<uintptr_t>(t.raw()); })
      .def_property_readonly("_buffer_id", [](const Tensor& t) { return reinterpret_cast<uintptr_t>(t.impl()->buffer().get()); })
      .def_property_readonly("_storage_version", &Tensor::version)
      .def_property_readonly("_has_grad_fn", [](const Tensor& t) { return !t.is_leaf(); })
      .def_property_readonly("_grad_fn_name", [](const Tensor& t) -> py::object {
        if (t.is_leaf()) return py::none();
        return py::str(t.grad_fn()->name());
      })
      .def_property_readonly("_data_ptr", [](const Tensor& t) { return reinterpret_cast<uintptr_t>(t.data()); })
      .def("requires_grad_", [](Tensor& t, bool on) { t.requires_grad_(on); return t; }, py::arg("requires_grad") = true)
      .def("set_grad", [](Tensor& t, const py::object& g) { t.set_grad(g.is_none() ? Tensor() : g.cast<Tensor>()); })
      .def("zero_grad", &Tensor::zero_grad)
      .def("backward", [](const Tensor& t, bool retain) { t.backward(retain); }, py::arg("retain_graph") = false)
      .def("detach", &Tensor::detach)
      .def("tolist", &tolist_flat)
      .def("numpy", &to_numpy)
      .def("item", &scalar_to_py)
      .def("get_item", [](const Tensor& t, const py::object& key) { return ops::read_scalar(t, flat_index(t, key)); })
      .def("set_item", [](Tensor& t, const py::object& key, double v) {
        if (grad_enabled() && t.requires_grad() && !t.is_leaf())
          throw std::runtime_error("set_item: in-place modification of a tensor with autograd history is only allowed under no_grad()");
        ops::write_scalar(t, flat_index(t, key), v);
      })
      .def("fill_", [](Tensor& t, double v) { ops::fill_(t, v); return t; })
      .def("add_", [](Tensor& t, const Tensor& o, double alpha) { ops::add_(t, o, alpha); return t; }, py::arg("other"), py::arg("alpha") = 1.0)
      .def("mul_", [](Tensor& t, double alpha) { ops::mul_(t, alpha); return t; })
      .def("_copy_flat_range_from", [](Tensor& dst, int64_t dst_off, const Tensor& src, int64_t src_off, int64_t n) {
        ops::copy_range(dst, dst_off, src, src_off, n);
      })
      .def("_copy_flat_range_to", [](const Tensor& src, int64_t src_off, Tensor& dst, int64_t dst_off, int64_t n) {
        ops::copy_range(dst, dst_off, src, src_off, n);
      })
      .def("_copy_data_", [](Tensor& dst, const Tensor& src) {
        NoGradGuard g;
        Tensor s = src.detach();
        if (s.dtype() != dst.dtype()) s = ops::cast(s, dst.dtype());
        ops::copy_(dst, s);
      })
      .def("_model_value_reference", [](const Tensor& t) { return t.detach(); })
      .def("_rebind_model_value_", [](Tensor& t, const Tensor& value) {
        if (grad_enabled()) throw std::runtime_error("_rebind_model_value_ requires no_grad()");
        t.impl()->rebind(*value.impl());
        t.impl()->ag().grad.reset();
      })
      .def("_set_grad_slot", [](Tensor& t, const py::object& slot) {
        if (slot.is_none()) { t.impl()->ag().grad_slot.reset(); return; }
        Tensor s = slot.cast<Tensor>();
        if (s.shape() != t.shape() || s.dtype() != t.dtype() || s.device() != t.device())
          throw std::invalid_argument("_set_grad_slot: slot must match the parameter's shape, dtype and device");
        t.impl()->ag().grad_slot = s.detach().impl();
      })
      .def("reshape", [](const Tensor& t, py::args a) {
        return ops::reshape(t, a.size() == 1 && !py::isinstance<py::int_>(a[0]) ? shape_from_py(a[0]) : shape_from_py(a));
      })
      .def("flatten", &ops::flatten, py::arg("start_dim") = 0, py::arg("end_dim") = -1)
      .def("transpose", &ops::transpose, py::arg("dim0") = 0, py::arg("dim1") = 1)
      .def("slice", &ops::slice, py::arg("dim"), py::arg("start"), py::arg("end"))
      .def("contiguous", &ops::contiguous)
      .def("__getitem__", &getitem)
      .def("__setitem__", &setitem)
      .def("__len__", [](const Tensor& t) { if (t.ndim() == 0) throw py::type_error("len() of a rank-0 tensor"); return t.shape()[0]; })
      .def("to", [](const Tensor& t, const py::object& dev) { return ops::to(t, device_from_py(dev)); })
      .def("cpu", [](const Tensor& t) { return ops::to(t, Device()); })
      .def("cuda", [](const Tensor& t, int idx) { return ops::to(t, Device(DeviceType::CUDA, idx)); }, py::arg("index") = 0)
      .def("cast", [](const Tensor& t, const py::object& d) { return ops::cast(t, dtype_from_py(d)); })
      .def("sum", [](const Tensor& t, const py::object& dim, bool keep) { return ops::sum(t, opt_dim(dim), keep); }, py::arg("dim") = py::none(), py::arg("keepdim") = false)
      .def("mean", [](const Tensor& t, const py::object& dim, bool keep) { return ops::mean(t, opt_dim(dim), keep); }, py::arg("dim") = py::none(), py::arg("keepdim") = false)
      // Values only, as in the reference (bindings/tensor_bindings.cpp:693-697); indices come from argmax.
      .def("max", [](const Tensor& t, const py::object& dim, bool keep) { return ops::max(t, opt_dim(dim), keep).first; },
           py::arg("dim") = py::none(), py::arg("keepdim") = false)
      .def("argmax", [](const Tensor& t, const py::object& dim, bool keep) { return ops::argmax(t, opt_dim(dim), keep); }, py::arg("dim") = py::none(), py::arg("keepdim") = false)
      .def("neg", &ops::neg).def("relu", &ops::relu).def("sigmoid", &ops::sigmoid).def("tanh", &ops::tanh)
      .def("leaky_relu", &ops::leaky_relu, py::arg("negative_slope") = 0.01)
      .def("gelu", &ops::gelu).def("exp", &ops::exp).def("sqrt", &ops::sqrt).def("reciprocal", &ops::reciprocal).def("log", &ops::log)
      .def("softmax", &ops::softmax, py::arg("dim") = -1)
      .def("log_softmax", &ops::log_softmax, py::arg("dim") = -1)
      .def("matmul", &ops::matmul)
      .def("__matmul__", [](const Tensor& a, const py::object& b) -> py::object {
        if (!py::isinstance<Tensor>(b)) return py::reinterpret_borrow<py::object>(Py_NotImplemented);
        return py::cast(ops::matmul(a, b.cast<Tensor>()));
      })
      .def("__neg__", &ops::neg)
      .def("_register_post_accumulate_grad_hook", [](Tensor& t, std::function<void()> fn) {
        t.impl()->ag().post_accumulate_hooks.push_back(std::move(fn));
      })
      .def("_register_backward_finalizer", [](Tensor& t, uint64_t key, std::function<void()> fn) {
        auto& list = t.is_leaf() ? t.impl()->ag().finalizers : t.grad_fn()->finalizers;
        for (auto& f : list)
          if (f.first == key) { f.second = std::move(fn); return; }
        list.emplace_back(key, std::move(fn));
      })
      .def("_clear_hooks", [](Tensor& t) {
        t.impl()->ag().post_accumulate_hooks.clear();
        t.impl()->ag().finalizers.clear();
      })
      .def("__repr__", [](const Tensor& t) {
        return "Tensor(shape=" + shape_str(t.shape()) + ", dtype=" + dtype_name(t.dtype()) + ", device=" + t.device().str() +
               (t.requires_grad() ? ", requires_grad=True)" : ")");
      });

  // Arithmetic operators: Tensor or Python scalar operands; anything else is NotImplemented.
  auto is_scalar = [](const py::object& o) { return py::isinstance<py::float_>(o) || (py::isinstance<py::int_>(o) && !py::isinstance<py::bool_>(o)); };
#define BINOP(NAME, TENSOR_EXPR, SCALAR_EXPR)                                                   \
  T.def(NAME, [is_scalar](const Tensor& a, const py::object& o) -> py::object {                 \
    if (py::isinstance<Tensor>(o)) { const Tensor b = o.cast<Tensor>(); return py::cast(TENSOR_EXPR); } \
    if (is_scalar(o)) { const double s = o.cast<double>(); return py::cast(SCALAR_EXPR); }       \
    return py::reinterpret_borrow<py::object>(Py_NotImplemented);                                \
  })
  BINOP("__add__", ops::add(a, b), ops::add_scalar(a, s));
  BINOP("__radd__", ops::add(b, a), ops::add_scalar(a, s));
  BINOP("__sub__", ops::sub(a, b), ops::add_scalar(a, -s));
  BINOP("__rsub__", ops::sub(b, a), ops::add_scalar(ops::neg(a), s));
  BINOP("__mul__", ops::mul(a, b), ops::mul_scalar(a, s));
  BINOP("__rmul__", ops::mul(b, a), ops::mul_scalar(a, s));
  BINOP("__truediv__", ops::div(a, b), ops::mul_scalar(a, 1.0 / s));
  BINOP("__rtruediv__", ops::div(b, a), ops::mul_scalar(ops::reciprocal(a), s));
#undef BINOP

  // ------------------------------------------------------------- factories
  auto cpu_only = [](const py::object& dev) {
    if (!dev.is_none() && !device_from_py(dev).is_cpu())
      throw std::invalid_argument("factories create CPU tensors; move the result with .to(device)");
  };
  m.def("empty", [cpu_only](const py::object& shape, const py::object& dtype, const py::object& dev) {
    cpu_only(dev); return Tensor::empty(shape_from_py(shape), dtype_from_py(dtype), Device());
  }, py::arg("shape"), py::arg("dtype") = py::none(), py::arg("device") = py::none());
  m.def("zeros", [cpu_only](const py::object& shape, const py::object& dtype, const py::object& dev) {
    cpu_only(dev); return Tensor::zeros(shape_from_py(shape), dtype_from_py(dtype), Device());
  }, py::arg("shape"), py::arg("dtype") = py::none(), py::arg("device") = py::none());
  m.def("ones", [cpu_only](const py::object& shape, const py::object& dtype, const py::object& dev) {
    cpu_only(dev); return Tensor::full(shape_from_py(shape), 1.0, dtype_from_py(dtype), Device());
  }, py::arg("shape"), py::arg("dtype") = py::none(), py::arg("device") = py::none());
  m.def("full", [cpu_only](const py::object& shape, double v, const py::object& dtype, const py::object& dev) {
    cpu_only(dev); return Tensor::full(shape_from_py(shape), v, dtype_from_py(dtype), Device());
  }, py::arg("shape"), py::arg("value"), py::arg("dtype") = py::none(), py::arg("device") = py::none());
  // Private device-side factories (used by optimizers and reducers to avoid host staging).
  m.def("_zeros_on", [](const py::object& shape, const py::object& dtype, const py::object& dev) {
    return Tensor::zeros(shape_from_py(shape), dtype_from_py(dtype), device_from_py(dev));
  });
  m.def("_empty_on", [](const py::object& shape, const py::object& dtype, const py::object& dev) {
    return Tensor::empty(shape_from_py(shape), dtype_from_py(dtype), device_from_py(dev));
  });
  m.def("_full_on", [](const py::object& shape, double v, const py::object& dtype, const py::object& dev) {
    return Tensor::full(shape_from_py(shape), v, dtype_from_py(dtype), device_from_py(dev));
  });
  m.def("_view_flat", [](const Tensor& base, int64_t offset, const py::object& shape) {
    // Contiguous view of `shape` starting `offset` elements into a contiguous 1-D tensor.
    if (!base.is_contiguous()) throw std::invalid_argument("_view_flat: base must be contiguous");
    Shape s = shape_from_py(shape);
    return Tensor::view_of(base, Layout(s, Layout::contiguous_strides(s), base.offset() + offset));
  });
  m.def("_pinned_empty", [](const py::object& shape, const py::object& dtype) {
    return cu::pinned_empty(shape_from_py(shape), dtype_from_py(dtype));
  });
  m.def("_copy_h2d_async", &cu::copy_h2d_async, py::arg("dst"), py::arg("src"), py::arg("stream_kind") = 0);
  m.def("_copy_d2h_async", &cu::copy_d2h_async);
  m.def("from_numpy", &from_numpy, py::arg("array"), py::arg("dtype") = py::none());
  m.def("_tensor_to_bytes", &tensor_to_bytes);
  m.def("_tensor_from_bytes", &tensor_from_bytes);

  // ------------------------------------------------------------- operators
  m.def("add", &ops::add); m.def("mul", &ops::mul); m.def("sub", &ops::sub); m.def("div", &ops::div);
  m.def("fill_", [](Tensor& t, double v) { ops::fill_(t, v); return t; });
  m.def("reshape", [](const Tensor& t, const py::object& s) { return ops::reshape(t, shape_from_py(s)); });
  m.def("transpose", &ops::transpose, py::arg("tensor"), py::arg("dim0") = 0, py::arg("dim1") = 1);
  m.def("contiguous", &ops::contiguous);
  m.def("sum", [](const Tensor& t, const py::object& dim, bool keep) { return ops::sum(t, opt_dim(dim), keep); }, py::arg("tensor"), py::arg("dim") = py::none(), py::arg("keepdim") = false);
  m.def("mean", [](const Tensor& t, const py::object& dim, bool keep) { return ops::mean(t, opt_dim(dim), keep); }, py::arg("tensor"), py::arg("dim") = py::none(), py::arg("keepdim") = false);
  m.def("max", [](const Tensor& t, const py::object& dim, bool keep) { return ops::max(t, opt_dim(dim), keep).first; },
        py::arg("tensor"), py::arg("dim") = py::none(), py::arg("keepdim") = false);
  m.def("argmax", [](const Tensor& t, const py::object& dim, bool keep) { return ops::argmax(t, opt_dim(dim), keep); }, py::arg("tensor"), py::arg("dim") = py::none(), py::arg("keepdim") = false);
  m.def("neg", &ops::neg); m.def("relu", &ops::relu); m.def("sigmoid", &ops::sigmoid); m.def("tanh", &ops::tanh);
  m.def("leaky_relu", &ops::leaky_relu, py::arg("tensor"), py::arg("negative_slope") = 0.01);
  m.def("gelu", &ops::gelu); m.def("exp", &ops::exp); m.def("sqrt", &ops::sqrt); m.def("reciprocal", &ops::reciprocal);
  m.def("log", &ops::log);
  m.def("dropout", [](const Tensor& t, double p, const py::int_& seed) {
    return ops::dropout(t, p, static_cast<uint64_t>(seed.cast<py::int_>().attr("__and__")(py::int_(0xFFFFFFFFFFFFFFFFull)).cast<uint64_t>()));
  }, py::arg("tensor"), py::arg("p"), py::arg("seed"));
  m.def("embedding", &ops::embedding, py::arg("indices"), py::arg("weight"));
  m.def("to", [](const Tensor& t, const py::object& dev) { return ops::to(t, device_from_py(dev)); });
  m.def("cast", [](const Tensor& t, const py::object& d) { return ops::cast(t, dtype_from_py(d)); });
  m.def("matmul", &ops::matmul);
  m.def("fused_linear_relu", &ops::fused_linear_relu);
  m.def("linear", [](const Tensor& x, const Tensor& w, const py::object& b, const std::string& act, const py::object& res) {
    ops::Act a = ops::Act::None;
    if (act == "relu") a = ops::Act::Relu;
    else if (act == "gelu") a = ops::Act::Gelu;
    else if (act != "none" && !act.empty()) throw std::invalid_argument("linear: activation must be 'none', 'relu' or 'gelu'");
    return ops::linear(x, w, b.is_none() ? Tensor() : b.cast<Tensor>(), a, res.is_none() ? Tensor() : res.cast<Tensor>());
  }, py::arg("input"), py::arg("weight"), py::arg("bias") = py::none(), py::arg("activation") = "none", py::arg("residual") = py::none());
  m.def("softmax", &ops::softmax, py::arg("tensor"), py::arg("dim") = -1);
  m.def("log_softmax", &ops::log_softmax, py::arg("tensor"), py::arg("dim") = -1);
  m.def("cross_entropy", [](const Tensor& logits, const py::object& targets) { return ops::cross_entropy(logits, targets_from_py(targets)); });
  m.def("nll_loss", [](const Tensor& lp, const py::object& targets, const std::string& red) {
    return ops::nll_loss(lp, targets_from_py(targets), red);
  }, py::arg("log_probs"), py::arg("targets"), py::arg("reduction") = "mean");
  m.def("conv2d", [](const Tensor& x, const Tensor& w, const py::object& b, int sh, int sw, int ph, int pw) {
    return ops::conv2d(x, w, b.is_none() ? Tensor() : b.cast<Tensor>(), sh, sw, ph, pw);
  }, py::arg("input"), py::arg("weight"), py::arg("bias") = py::none(), py::arg("stride_h") = 1, py::arg("stride_w") = 1, py::arg("pad_h") = 0, py::arg("pad_w") = 0);
  m.def("maxpool2d", &ops::maxpool2d, py::arg("input"), py::arg("kernel_h"), py::arg("kernel_w"), py::arg("stride_h"), py::arg("stride_w"), py::arg("pad_h") = 0, py::arg("pad_w") = 0);
  m.def("_layer_norm", [](const Tensor& x, const py::object& w, const py::object& b, double eps) {
    return ops::layer_norm(x, w.is_none() ? Tensor() : w.cast<Tensor>(), b.is_none() ? Tensor() : b.cast<Tensor>(), eps);
  });
  m.def("_attention", [](const Tensor& q, const Tensor& k, const Tensor& v, const py::object& mask, bool causal, double scale, double p, const py::int_& seed) {
    return ops::attention(q, k, v, mask.is_none() ? Tensor() : mask.cast<Tensor>(), causal, scale, p,
                          seed.attr("__and__")(py::int_(0xFFFFFFFFFFFFFFFFull)).cast<uint64_t>());
  }, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("mask") = py::none(), py::arg("causal") = false, py::arg("scale") = 1.0, py::arg("dropout_p") = 0.0, py::arg("seed") = py::int_(0));
  m.def("_attention_qkv", [](const Tensor& qkv, int64_t heads, const py::object& mask, bool causal, double scale, double p, const py::int_& seed) {
    return ops::attention_packed(qkv, heads, mask.is_none() ? Tensor() : mask.cast<Tensor>(), causal, scale, p,
                                 seed.attr("__and__")(py::int_(0xFFFFFFFFFFFFFFFFull)).cast<uint64_t>());
  }, py::arg("qkv"), py::arg("heads"), py::arg("mask") = py::none(), py::arg("causal") = false, py::arg("scale") = 1.0,
     py::arg("dropout_p") = 0.0, py::arg("seed") = py::int_(0));
  // Diagnostics (reference project: bindings/ops_bindings.cpp:300-363, src/diagnostics/matmul.cpp).
  m.def("set_float32_matmul_precision", [](const std::string& level) {
    if (level == "highest") cu::set_float32_matmul_precision(0);
    else if (level == "high") cu::set_float32_matmul_precision(1);
    else throw std::invalid_argument("set_float32_matmul_precision: expected 'highest' or 'high'");
  }, "float32 matmul / linear on CUDA: 'highest' = float32 FMA kernel (default), 'high' = large products as bfloat16 piece products on the tensor cores");
  m.def("get_float32_matmul_precision", [] { return std::string(cu::float32_matmul_precision() ? "high" : "highest"); });
  m.def("_matmul_force_route", [](const std::string& route) {
    if (route == "auto") cu::set_gemm_route(0);
    else if (route == "simt") cu::set_gemm_route(1);
    else if (route == "tcgen05") cu::set_gemm_route(2);
    else throw std::invalid_argument("matmul route must be 'auto', 'simt' or 'tcgen05'");
  });
  m.def("_matmul_last_route", [] {
    static const char* names[] = {"none", "simt", "tcgen05_128x128", "tcgen05_128x256"};
    return std::string(names[cu::last_gemm_route() & 3]);
  });
  m.def("_conv2d_force_route", [](const std::string& route) {
    if (route == "auto") cu::set_conv_route(0);
    else if (route == "direct") cu::set_conv_route(1);
    else throw std::invalid_argument("conv2d route must be 'auto' or 'direct'");
  });
  m.def("_conv2d_last_route", [] {
    static const char* names[] = {"none", "direct", "tcgen05_lowering", "none"};
    return std::string(names[cu::last_conv_route() & 3]);
  });
  m.def("_attention_qkv_fused", [](const Tensor& qkv, int64_t heads) { return cu::flash_attention_supported(qkv, heads); });
  m.def("_mlp_gelu", [](const Tensor& x, const Tensor& w1, const py::object& b1, const Tensor& w2, const py::object& b2,
                        const py::object& residual) {
    auto opt = [](const py::object& o) { return o.is_none() ? Tensor() : o.cast<Tensor>(); };
    return ops::mlp_gelu(x, w1, opt(b1), w2, opt(b2), opt(residual));
  }, py::arg("x"), py::arg("w1"), py::arg("b1"), py::arg("w2"), py::arg("b2"), py::arg("residual") = py::none());
  m.def("_gemm", &ops::gemm, py::arg("a"), py::arg("trans_a"), py::arg("b"), py::arg("trans_b"));
  m.def("isfinite_all", &ops::isfinite_all);
  m.def("_isfinite_into", [](const Tensor& t, Tensor& flag) { ops::isfinite_into(t, flag); });
  m.def("_amp_unscale_to_float32_and_check", [](const Tensor& g, double inv) {
    auto r = ops::amp_unscale_to_f32_and_check(g, inv);
    return py::make_tuple(r.first, r.second);
  });
  m.def("_amp_unscale_into", [](const Tensor& g, double inv, Tensor& flag) { return ops::amp_unscale_into(g, inv, flag); });
  m.def("_amp_copy_master_to_model_", [](Tensor& model, const Tensor& master) { ops::amp_copy_master_to_model_(model, master); });
  m.def("_adam_step_", [](Tensor& master, Tensor& mm, Tensor& vv, const Tensor& grad, const py::object& model, double lr, double b1,
                          double b2, double eps, double wd, double bc1, double bc2, double gs) {
    Tensor mdl = model.is_none() ? Tensor() : model.cast<Tensor>();
    ops::adam_step_(master, mm, vv, grad, mdl, ops::AdamHyper{lr, b1, b2, eps, wd, bc1, bc2, gs});
  });
  m.def("_sgd_step_", [](Tensor& master, const Tensor& grad, const py::object& model, double lr, double wd, double gs) {
    Tensor mdl = model.is_none() ? Tensor() : model.cast<Tensor>();
    ops::sgd_step_(master, grad, mdl, lr, wd, gs);
  });

  // --------------------------------------------------------------- runtime
  m.def("cuda_enabled", [] { return true; });
  m.def("cuda_available", [] { return Runtime::instance().cuda_available(); });
  m.def("cuda_device_count", [] { return Runtime::instance().cuda_device_count(); });
  m.def("cuda_synchronize", [] {
    Runtime::instance().synchronize_all();
    const int n = Runtime::instance().cuda_device_count();
    for (int d = 0; d < n; ++d) {
      const int e = cu::take_gemm_error(d);
      if (e) throw std::runtime_error("device cuda:" + std::to_string(d) + " reported a kernel wait timeout (code " + std::to_string(e) + ")");
    }
  });
  m.def("_cuda_stream_handle", [](int device) {
    // cudaStream_t of the device's current stream, as an integer, for foreign callers.
    return reinterpret_cast<uintptr_t>(Runtime::instance().cuda(device).current_stream());
  }, py::arg("device") = 0);
  m.def("_kernel_launch_count", [] { return cu::kernel_launch_count(); });
  m.def("_cuda_index_errors", [] { return cu::take_index_errors(); });
  m.def("_cuda_device_facts", [](int idx) {
    CudaContext& c = Runtime::instance().cuda(idx);
    py::dict d;
    d["sm_count"] = c.sm_count();
    d["cc_major"] = c.cc_major();
    d["cc_minor"] = c.cc_minor();
    d["total_memory"] = c.total_memory();
    return d;
  });
  // Timing event recorded on a device's current stream (CUDA events under the hood).
  py::class_<CompletionToken>(m, "CudaEvent")
      .def_static("record", [](int device) {
        CudaContext& c = Runtime::instance().cuda(device);
        DeviceGuard g(device);
        return CompletionToken::record_on(device, c.current_stream(), true);
      }, py::arg("device") = 0)
      .def("ready", &CompletionToken::ready)
      .def("synchronize", &CompletionToken::wait_host)
      .def("elapsed_ms_since", &CompletionToken::elapsed_ms_since);
  m.def("_flush_l2", [](int device) {
    // Overwrites a buffer larger than the 126 MB L2 so the next kernel starts cold.
    static Tensor scratch;
    if (!scratch.defined() || scratch.device().index != device)
      scratch = Tensor::empty({256LL << 20}, DType::U8, Device(DeviceType::CUDA, device));
    ops::fill_raw(scratch, 1.0);
  }, py::arg("device") = 0);
  m.def("is_grad_enabled", &grad_enabled);
  m.def("set_grad_enabled", &set_grad_enabled);
  m.def("_memory_pool_stats", [] {
    const MemoryPoolStats s = MemoryPool::instance().stats();
    py::dict d;
    d["total_requests"] = s.total_requests; d["raw_allocations"] = s.raw_allocations; d["reused_blocks"] = s.reused_blocks;
    d["current_bytes"] = s.current_bytes; d["peak_bytes"] = s.peak_bytes; d["cached_bytes"] = s.cached_bytes;
    d["reserved_bytes"] = s.reserved_bytes;
    return d;
  });
  m.def("_memory_pool_clear", [] { MemoryPool::instance().clear(); });
  m.def("_memory_pool_reset_peak", [] { MemoryPool::instance().reset_peak(); });
  m.def("_memory_pool_set_enabled", [](bool on) { MemoryPool::instance().set_enabled(on); });
  m.def("_memory_pool_enabled", [] { return MemoryPool::instance().enabled(); });
  m.def("_memory_pool_set_max_cached_bytes", [](uint64_t n) { MemoryPool::instance().set_max_cached_bytes(n); });
  m.def("_memory_pool_max_cached_bytes", [] { return MemoryPool::instance().max_cached_bytes(); });
  // Names of the reference's diagnostics surface (python/orthon/_diagnostics.py:8-17).
  m.def("_memory_pool_clear_cache", [] { MemoryPool::instance().clear(); });
  m.def("_memory_pool_reset_stats", [] { MemoryPool::instance().reset_peak(); });
  m.def("_scratch_pool_stats", [] {
    const ScratchPoolStats s = ScratchLease::stats();
    py::dict d;
    d["leases"] = s.leases; d["bytes_in_use"] = s.bytes_in_use; d["peak_bytes"] = s.peak_bytes;
    return d;
  });
  m.def("_dispatch_kernels", [] {
    py::list out;
    const KernelRegistry& r = default_dispatcher().registry();
    for (const KernelRecord& k : r.kernels()) {
      py::dict d;
      d["op"] = r.schema(k.op).name;
      d["backend"] = k.constraints.backend == Backend::CPU ? "cpu" : "cuda";
      py::list dts;
      for (int i = 0; i < static_cast<int>(DType::COUNT); ++i)
        if (k.constraints.dtypes & (1u << i)) dts.append(dtype_name(static_cast<DType>(i)));
      d["dtypes"] = dts;
      d["layouts"] = static_cast<int>(k.constraints.layouts);
      d["name"] = k.name;
      out.append(d);
    }
    return out;
  });
  m.def("_dispatch_resolve", [](const std::string& op, const py::object& dev, const py::object& dtype, int layout) {
    const KernelRegistry& r = default_dispatcher().registry();
    for (int i = 0; i < static_cast<int>(OperatorId::COUNT); ++i) {
      const OperatorId id = static_cast<OperatorId>(i);
      if (std::string(r.schema(id).name) == op) {
        const KernelRecord* k = r.find(id, backend_of(device_from_py(dev)), dtype_from_py(dtype), static_cast<uint8_t>(layout));
        return k ? py::object(py::str(k->name)) : py::object(py::none());
      }
    }
    throw std::invalid_argument("unknown operator '" + op + "'");
  }, py::arg("op"), py::arg("device"), py::arg("dtype"), py::arg("layout") = 1);
  m.def("_set_dispatch_trace", [](const py::object& fn) {
    if (fn.is_none()) { default_dispatcher().set_observer(nullptr); return; }
    py::function f = fn.cast<py::function>();
    default_dispatcher().set_observer([f](const DispatchRequest& r, const KernelRecord& k) {
      py::gil_scoped_acquire gil;
      f(py::str(default_dispatcher().registry().schema(r.op).name), py::str(k.name));
    });
  });
  py::register_exception<UnsupportedOperation>(m, "UnsupportedOperation", PyExc_RuntimeError);

  bind_distributed(m);
}
