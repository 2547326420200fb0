// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own CPU convolutions, compiled from the reference's source
// files where they lie (the Makefile passes their directories with -I; nothing is copied).
// Wrapped: repro_conv_cuda/repro_conv_cpu.h:25 (cpu_conv2d), :45 (cpu_conv2d_grad_weight),
// :72 (cpu_conv2d_grad_input).  shape = {N, C, H, W, F, KH, KW, SY, SX, PY, PX}.
#include "repro_conv_cpu.h"

static repro_conv::ConvShape shape_of(const int* s) {
    repro_conv::ConvShape g;
    g.N = s[0]; g.C = s[1]; g.H = s[2]; g.W = s[3]; g.F = s[4]; g.KH = s[5]; g.KW = s[6];
    g.SY = s[7]; g.SX = s[8]; g.PY = s[9]; g.PX = s[10];
    return g;
}

extern "C" {

void ref_cpu_conv2d(const float* x, const float* w, float* out, const int* shape, int S) {
    repro_conv::cpu_conv2d(x, w, out, shape_of(shape), S);
}
void ref_cpu_conv2d_grad_weight(const float* dy, const float* x, float* dw, const int* shape, int S) {
    repro_conv::cpu_conv2d_grad_weight(dy, x, dw, shape_of(shape), S);
}
void ref_cpu_conv2d_grad_input(const float* dy, const float* w, float* dx, const int* shape, int S) {
    repro_conv::cpu_conv2d_grad_input(dy, w, dx, shape_of(shape), S);
}

}
