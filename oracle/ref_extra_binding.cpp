// Test infrastructure: exposes the reference's fused_add_rms_norm host function (csrc/norm.cu:100-113), which the
// reference's own module table (csrc/ffi.cpp:4-8) leaves out, so that the GPU parity tests can call the reference
// kernel (csrc/norm.cu:59-83) itself.  Compiled by oracle/build_ref.py next to the reference's norm.cu, read in
// place from the reference tree; nothing of the reference is copied here.
#include <pybind11/pybind11.h>
#include <torch/extension.h>

void fused_add_rms_norm(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, float epsilon);

PYBIND11_MODULE(_csrc_ref_extra, m) {
  m.def("fused_add_rms_norm", &fused_add_rms_norm, "in-place residual add + RMS norm (reference kernel)");
}
