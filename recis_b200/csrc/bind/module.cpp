// Python module definition: each bind_*.cpp registers its functions here.
#include <torch/extension.h>

void init_sparse(pybind11::module& m);
void init_dense(pybind11::module& m);
void init_comm(pybind11::module& m);
void init_ragged(pybind11::module& m);
void init_serialize(pybind11::module& m);
void init_metrics(pybind11::module& m);
void init_io(pybind11::module& m);
void init_exchange(pybind11::module& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "recis_b200 native extension (sm_100a kernels + CPU implementations)";
  init_sparse(m);
  init_dense(m);
  init_comm(m);
  init_ragged(m);
  init_serialize(m);
  init_metrics(m);
  init_io(m);
  init_exchange(m);
}
