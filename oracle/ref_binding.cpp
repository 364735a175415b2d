// Python binding for the reference project's own CPU sources, compiled unmodified
// from where they lie (see build_ref.py).  TEST INFRASTRUCTURE ONLY: this module is
// the checker / timed CPU baseline and is never imported by the product package.
//
// Exposes the same names the reference registers in torchsparse/backend/pybind_cpu.cpp:12-23
// (minus hash_query_cpu, which needs the absent third-party sparsehash headers).
#include <torch/extension.h>

#include "convolution/convolution_gather_scatter_cpu.h"
#include "devoxelize/devoxelize_cpu.h"
#include "hash/hash_cpu.h"
#include "others/count_cpu.h"
#include "voxelize/voxelize_cpu.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("conv_forward_gather_scatter_cpu", &conv_forward_gather_scatter_cpu);
  m.def("conv_backward_gather_scatter_cpu", &conv_backward_gather_scatter_cpu);
  m.def("voxelize_forward_cpu", &voxelize_forward_cpu);
  m.def("voxelize_backward_cpu", &voxelize_backward_cpu);
  m.def("devoxelize_forward_cpu", &devoxelize_forward_cpu);
  m.def("devoxelize_backward_cpu", &devoxelize_backward_cpu);
  m.def("hash_cpu", &hash_cpu);
  m.def("kernel_hash_cpu", &kernel_hash_cpu);
  m.def("count_cpu", &count_cpu);
}
