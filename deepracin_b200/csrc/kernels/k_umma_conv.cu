/* Tensor-core (tcgen05) convolution path -- placeholder until the kernel lands: reports every shape as unsupported. */
#include "k_common.cuh"
extern "C" int dRk_tensor_conv_supported(int W, int H, int Cin, int Cout, int kw, int kh) { (void)W; (void)H; (void)Cin; (void)Cout; (void)kw; (void)kh; return 0; }
extern "C" dRk_TensorConvPlan *dRk_tensor_conv_plan(const float *in, const float *wT, const float *bias, float *out, int n, int W, int H, int Cin,
                                                    int Cout, int kw, int kh, int act, int ldo, int coff, int *status)
{ (void)in; (void)wT; (void)bias; (void)out; (void)n; (void)W; (void)H; (void)Cin; (void)Cout; (void)kw; (void)kh; (void)act; (void)ldo; (void)coff; (void)status; return NULL; }
extern "C" int dRk_tensor_conv_run(dRk_stream stream, dRk_TensorConvPlan *plan) { (void)stream; (void)plan; return -1; }
extern "C" void dRk_tensor_conv_free(dRk_TensorConvPlan *plan) { (void)plan; }
