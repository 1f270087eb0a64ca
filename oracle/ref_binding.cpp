// pybind11 module over the UNMODIFIED reference sources (compiled in place from the reference tree by
// oracle/build_ref.py).  Test infrastructure: lets the GPU tests compare this library against the reference's
// own CUDA kernels and lets tests/golden/make_golden.py record their outputs.  Declarations come from the
// reference's own headers.
#include <torch/extension.h>

#include "sphconv/rules.h"
#include "sphconv/tensor.h"
#ifdef SPH_REF_WITH_CONV
#include "sphconv/rule_conv.h"
#endif

PYBIND11_MODULE(sphconv_ref, m) {
  m.def("get_rules_subm", &sphconv::get_rules_subm, "");
  m.def("get_rules", &sphconv::get_rules, "");
  m.def("init_tensor", &sphconv::init_tensor, "");
  m.def("to_dense", &sphconv::to_dense, "");
#ifdef SPH_REF_WITH_CONV
  m.def("rule_conv", &sphconv::device::rule_conv, "");
  m.def("rule_conv_backward", &sphconv::device::rule_conv_backward, "");
  m.attr("has_conv") = true;
#else
  m.attr("has_conv") = false;
#endif
}
