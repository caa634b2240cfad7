// pybind11 module over the C++ Sampler class (include/etb200_sampler.hpp), in the style of the
// reference's runner bindings (extension/llm/runner/pybindings.cpp: errors become
// std::runtime_error, the GIL is released around calls that wait for the GPU). Device
// buffers are passed as integer addresses (tensor.data_ptr()), so the module depends on
// neither torch nor numpy.
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/etb200_sampler.hpp"

namespace py = pybind11;
using executorch_b200::Error;
using executorch_b200::ScalarType;
using executorch_b200::extension::llm::Sampler;

namespace {

void throw_if_error(Error e) {
  if (e != Error::Ok) {
    throw std::runtime_error("etb200 error 0x" + std::to_string(static_cast<uint32_t>(e)) + ": " +
                             Sampler::last_error_message());
  }
}

void* ptr(uintptr_t p) { return reinterpret_cast<void*>(p); }

}  // namespace

PYBIND11_MODULE(_sampler_pybind, m) {
  m.doc() = "B200 token sampler (pybind11 binding of executorch_b200::extension::llm::Sampler)";
  m.attr("kTopp") = executorch_b200::extension::llm::kTopp;

  py::class_<Sampler>(m, "Sampler")
      .def(py::init([](int32_t vocab_size, float temperature, float topp, unsigned long long rng_seed,
                       int32_t device) {
             auto s = std::make_unique<Sampler>(vocab_size, temperature, topp, rng_seed, device);
             throw_if_error(s->status());
             return s;
           }),
           py::arg("vocab_size"), py::arg("temperature"), py::arg("topp"), py::arg("rng_seed"),
           py::arg("device") = 0)
      .def(py::init([](int32_t vocab_size, float temperature, int32_t device) {
             auto s = std::make_unique<Sampler>(vocab_size, temperature, device);
             throw_if_error(s->status());
             return s;
           }),
           py::arg("vocab_size"), py::arg("temperature"), py::arg("device") = 0)
      .def("set_temperature", &Sampler::set_temperature, py::arg("temperature"))
      .def("set_topk", &Sampler::set_topk, py::arg("topk"))
      .def_property("rng_state", &Sampler::rng_state, &Sampler::set_rng_state)
      .def_property_readonly("vocab_size", &Sampler::vocab_size)
      .def(
          "sample",
          [](Sampler& s, uintptr_t logits, int32_t dtype, uintptr_t stream) {
            int32_t token = 0;
            py::gil_scoped_release release;
            // same call as Sampler::sample<T>, with the dtype chosen at run time
            Error e = Error::Ok;
            switch (static_cast<ScalarType>(dtype)) {
              case ScalarType::Float:
                token = s.sample(static_cast<float*>(ptr(logits)), ptr(stream));
                break;
              case ScalarType::Half:
                token = s.sample(static_cast<executorch_b200::Half*>(ptr(logits)), ptr(stream));
                break;
              case ScalarType::BFloat16:
                token = s.sample(static_cast<executorch_b200::BFloat16*>(ptr(logits)), ptr(stream));
                break;
              case ScalarType::UInt16:
                token = s.sample(static_cast<uint16_t*>(ptr(logits)), ptr(stream));
                break;
              default:
                e = Error::NotSupported;
            }
            if (e != Error::Ok) throw std::runtime_error("unsupported logits dtype code");
            return token;
          },
          py::arg("logits_ptr"), py::arg("dtype"), py::arg("stream") = 0)
      .def(
          "sample_rows",
          [](Sampler& s, uintptr_t logits, int32_t dtype, int64_t rows, int64_t row_stride,
             uintptr_t rng_states, uintptr_t out_ids, uintptr_t stream) {
            Error e;
            {
              py::gil_scoped_release release;
              e = s.sample_rows(ptr(logits), static_cast<ScalarType>(dtype), rows, row_stride,
                                static_cast<uint64_t*>(ptr(rng_states)),
                                static_cast<int64_t*>(ptr(out_ids)), ptr(stream));
            }
            throw_if_error(e);
          },
          py::arg("logits_ptr"), py::arg("dtype"), py::arg("rows"), py::arg("row_stride"),
          py::arg("rng_states_ptr"), py::arg("out_ids_ptr"), py::arg("stream") = 0);
}
