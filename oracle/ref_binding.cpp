// Test infrastructure only: pybind front door for the UNMODIFIED reference CPU
// implementation of the deformable-convolution path. The four reference
// translation units are compiled from where they lie in the reference checkout
// (mmcv/ops/csrc/pytorch/{modulated_deform_conv,deform_conv}.cpp and
// mmcv/ops/csrc/pytorch/cpu/{modulated_deform_conv,deform_conv}.cpp); this file
// only re-declares their entry points and gives them the keyword names of the
// reference's own module definition (mmcv/ops/csrc/pytorch/pybind.cpp:525-545
// and :641-656), so that the reference's Python wrappers can call it unchanged.
#include <torch/extension.h>

using at::Tensor;

void deform_conv_forward(Tensor input, Tensor weight, Tensor offset,
                         Tensor output, Tensor columns, Tensor ones, int kW,
                         int kH, int dW, int dH, int padW, int padH,
                         int dilationW, int dilationH, int group,
                         int deformable_group, int im2col_step);
void deform_conv_backward_input(Tensor input, Tensor offset, Tensor gradOutput,
                                Tensor gradInput, Tensor gradOffset,
                                Tensor weight, Tensor columns, int kW, int kH,
                                int dW, int dH, int padW, int padH,
                                int dilationW, int dilationH, int group,
                                int deformable_group, int im2col_step);
void deform_conv_backward_parameters(Tensor input, Tensor offset,
                                     Tensor gradOutput, Tensor gradWeight,
                                     Tensor columns, Tensor ones, int kW,
                                     int kH, int dW, int dH, int padW, int padH,
                                     int dilationW, int dilationH, int group,
                                     int deformable_group, float scale,
                                     int im2col_step);
void modulated_deform_conv_forward(
    Tensor input, Tensor weight, Tensor bias, Tensor ones, Tensor offset,
    Tensor mask, Tensor output, Tensor columns, int kernel_h, int kernel_w,
    const int stride_h, const int stride_w, const int pad_h, const int pad_w,
    const int dilation_h, const int dilation_w, const int group,
    const int deformable_group, const bool with_bias);
void modulated_deform_conv_backward(
    Tensor input, Tensor weight, Tensor bias, Tensor ones, Tensor offset,
    Tensor mask, Tensor columns, Tensor grad_input, Tensor grad_weight,
    Tensor grad_bias, Tensor grad_offset, Tensor grad_mask, Tensor grad_output,
    int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
    int pad_w, int dilation_h, int dilation_w, int group, int deformable_group,
    const bool with_bias);

namespace py = pybind11;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("deform_conv_forward", &deform_conv_forward, py::arg("input"),
        py::arg("weight"), py::arg("offset"), py::arg("output"),
        py::arg("columns"), py::arg("ones"), py::arg("kW"), py::arg("kH"),
        py::arg("dW"), py::arg("dH"), py::arg("padW"), py::arg("padH"),
        py::arg("dilationW"), py::arg("dilationH"), py::arg("group"),
        py::arg("deformable_group"), py::arg("im2col_step"));
  m.def("deform_conv_backward_input", &deform_conv_backward_input,
        py::arg("input"), py::arg("offset"), py::arg("gradOutput"),
        py::arg("gradInput"), py::arg("gradOffset"), py::arg("weight"),
        py::arg("columns"), py::arg("kW"), py::arg("kH"), py::arg("dW"),
        py::arg("dH"), py::arg("padW"), py::arg("padH"), py::arg("dilationW"),
        py::arg("dilationH"), py::arg("group"), py::arg("deformable_group"),
        py::arg("im2col_step"));
  m.def("deform_conv_backward_parameters", &deform_conv_backward_parameters,
        py::arg("input"), py::arg("offset"), py::arg("gradOutput"),
        py::arg("gradWeight"), py::arg("columns"), py::arg("ones"),
        py::arg("kW"), py::arg("kH"), py::arg("dW"), py::arg("dH"),
        py::arg("padW"), py::arg("padH"), py::arg("dilationW"),
        py::arg("dilationH"), py::arg("group"), py::arg("deformable_group"),
        py::arg("scale"), py::arg("im2col_step"));
  m.def("modulated_deform_conv_forward", &modulated_deform_conv_forward,
        py::arg("input"), py::arg("weight"), py::arg("bias"), py::arg("ones"),
        py::arg("offset"), py::arg("mask"), py::arg("output"),
        py::arg("columns"), py::arg("kernel_h"), py::arg("kernel_w"),
        py::arg("stride_h"), py::arg("stride_w"), py::arg("pad_h"),
        py::arg("pad_w"), py::arg("dilation_h"), py::arg("dilation_w"),
        py::arg("group"), py::arg("deformable_group"), py::arg("with_bias"));
  m.def("modulated_deform_conv_backward", &modulated_deform_conv_backward,
        py::arg("input"), py::arg("weight"), py::arg("bias"), py::arg("ones"),
        py::arg("offset"), py::arg("mask"), py::arg("columns"),
        py::arg("grad_input"), py::arg("grad_weight"), py::arg("grad_bias"),
        py::arg("grad_offset"), py::arg("grad_mask"), py::arg("grad_output"),
        py::arg("kernel_h"), py::arg("kernel_w"), py::arg("stride_h"),
        py::arg("stride_w"), py::arg("pad_h"), py::arg("pad_w"),
        py::arg("dilation_h"), py::arg("dilation_w"), py::arg("group"),
        py::arg("deformable_group"), py::arg("with_bias"));
}
