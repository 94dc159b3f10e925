/*
 * CPU oracle for the thnets forward pass -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU operators (NCHW float tensors,
 * fp32 arithmetic, same formulas and the same quirks) plus its uint8 "lowp"
 * scheme.  Only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg may link or load this; the product library never does.
 *
 * Every function names the reference file:line it restates.  All tensors are
 * dense row-major; image tensors are [N][C][H][W].
 */
#ifndef THB200_ORACLE_H
#define THB200_ORACLE_H
#ifdef __cplusplus
extern "C" {
#endif

/* ---- fp32 operators (oracle_fp32.c) ---- */
void orc_normalize(float *x, int N, int C, int H, int W, const float *mean, const float *std);
void orc_images_to_float(const unsigned char *const *images, int N, int W, int H, int stride, int cp,
                         const float *mean, const float *std, int bgr, float *dst);
int  orc_conv_out(int in, int k, int d, int pad);
int  orc_pool_out(int in, int k, int d, int pad, int ceil_mode);
void orc_conv2d(const float *x, int N, int C, int H, int W, const float *w, const float *bias,
                int Cout, int kH, int kW, int dH, int dW, int padH, int padW, float *y);
void orc_fullconv2d(const float *x, int N, int C, int H, int W, const float *w, const float *bias,
                    int Cout, int kH, int kW, int dH, int dW, int padH, int padW, int adjH, int adjW,
                    int strict_bias, float *y);
void orc_linear(const float *x, int N, int K, const float *w, const float *bias, int M, float *y);
void orc_batchnorm(const float *x, int N, int C, int HW, const float *mean, const float *var,
                   const float *weight, const float *bias, double eps, float *y);
void orc_threshold(const float *x, long n, float threshold, float val, float alpha, float *y);
void orc_prelu(const float *x, int N, int C, int HW, const float *w, int nOutputPlane, float *y);
void orc_maxpool(const float *x, int N, int C, int H, int W, int kH, int kW, int dH, int dW,
                 int padH, int padW, int ceil_mode, float *y);
void orc_avgpool(const float *x, int N, int C, int H, int W, int kH, int kW, int dH, int dW,
                 int padH, int padW, int ceil_mode, int count_include_pad, float *y);
double orc_exp_minus_approx(double x);
void orc_softmax(const float *x, int nframe, int dim, int stride, float *y);
void orc_caddtable(const float *const *ins, const long *n, int nin, int is_csub, float *y);
void orc_join_channels(const float *const *ins, const int *C, int nin, int N, int HW, float *y);

/* ---- uint8 "lowp" scheme (oracle_lowp.c) ---- */
void orc_lowp_quantize(const float *x, long n, unsigned char *q, float *sub, float *mult);
void orc_lowp_dequantize(const unsigned char *q, long n, float sub, float mult, float *x);
unsigned char orc_lowp_scale_float(float sub, float mult, float value);
void orc_lowp_gemm_params(float w_sub, float w_mult, float in_sub, float in_mult, float out_sub,
                          float out_mult, int *a_offset, int *b_offset, int *c_offset, int *c_mult,
                          int *c_shift);
void orc_lowp_conv_acc(const unsigned char *x, int C, int H, int W, const unsigned char *w, int Cout,
                       int kH, int kW, int dH, int dW, int padH, int padW, int zero, int a_offset,
                       int b_offset, int *acc);
void orc_lowp_conv(const unsigned char *x, int N, int C, int H, int W, float in_sub, float in_mult,
                   const unsigned char *w, float w_sub, float w_mult, const unsigned char *bias,
                   float b_sub, float b_mult, int Cout, int kH, int kW, int dH, int dW, int padH,
                   int padW, float out_sub, float out_mult, unsigned char *y);
void orc_lowp_maxpool(const unsigned char *x, int N, int C, int H, int W, int kH, int kW, int dH,
                      int dW, int padH, int padW, int ceil_mode, unsigned char *y);
void orc_lowp_threshold(const unsigned char *x, long n, unsigned char threshold, unsigned char val,
                        unsigned char *y);
void orc_lowp_images(const unsigned char *const *images, int N, int W, int H, int stride,
                     const float *mean, const float *std, int bgr, unsigned char *dst, float *sub,
                     float *mult);

/* the 8-bit GEMM contract (lowpgemm_contract.c) */
void lowpgemm(const int is_a_transposed, const int is_b_transposed, const int is_c_transposed,
              const int m, const int n, const int k, const unsigned char *a, const unsigned char *b,
              unsigned char *c, const int lda, const int ldb, const int ldc, const int a_offset,
              const int b_offset, const int c_offset, const int c_mult, const int c_shift);
unsigned char orc_lowp_requant(int acc, int c_offset, int c_mult, int c_shift);

/* ---- the remaining operators (oracle_shape.c) ---- */
void orc_upsample2x(const float *x, int N, int C, int H, int W, float *y);
void orc_zero_pad(const float *x, int N, int C, int H, int W, int pad_l, int pad_r, int pad_t, int pad_b, float *y);
void orc_slice(const float *x, const long *size, int ndim, int axis, long from, long to, float *y);
void orc_cmax(const float *const *ins, int nin, long n, float *y);
void orc_logsoftmax(const float *x, long nframe, long dim, long stride, int first_frame_quirk, float *y);
void orc_l2_normalize(const float *x, long rows, long row_len, int per_row, float *y);
void orc_max_unpool(const float *v, const float *pool_in, int N, int C, int H, int W, int kH, int kW, int dH, int dW, int padH,
                    int padW, int oH, int oW, float *y);

#ifdef __cplusplus
}
#endif
#endif
