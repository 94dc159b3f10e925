/*
 * Host-side arithmetic of the uint8 ("lowp") engine: everything the reference derives in float on
 * the CPU before or around its 8-bit GEMM -- quantisation ranges, zero points, the requantisation
 * multiplier and shift, the per-channel bias addends.  These are evaluated here with the same C
 * float expressions, roundf and log calls, in the same order, because the device kernels must
 * reproduce the reference's integers bit for bit and a different rounding of one of these scalars
 * changes every output byte.
 */
#include <math.h>
#include "thb_internal.h"

/* lowp/lowp_basic.c:15-35: range always contains 0, mult = 255.0/(max-min) narrowed to float, each
 * element roundf(x*mult) - roundf(min*mult); the largest element may come out as 256 and is then stored
 * as 0 (conversion through int keeps the low byte) */
void thb_lowp_quantize(const float *x, long n, unsigned char *q, float *sub, float *mult)
{
    float lo = 0, hi = 0, m;
    for (long i = 0; i < n; i++) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
    }
    m = hi - lo > 0 ? (float)(255.0 / (hi - lo)) : 0;
    const float zero_term = roundf(lo * m);
    for (long i = 0; i < n; i++) q[i] = (unsigned char)(int)(roundf(x[i] * m) - zero_term);
    *sub = lo;
    *mult = m;
}

/* lowp/lowp_basic.c:214-222: clamp to [0,255], then truncate */
unsigned char thb_lowp_scale_float(float sub, float mult, float value)
{
    float s = (value - sub) * mult;
    return s < 0 ? 0 : s > 255 ? 255 : (unsigned char)s;
}

/* lowp/lowp_basic.c:309-320 */
void thb_lowp_gemm_params(float w_sub, float w_mult, float in_sub, float in_mult, float out_sub, float out_mult,
                          int *a_offset, int *b_offset, int *c_offset, int *c_mult, int *c_shift)
{
    float scaling = w_mult * in_mult / out_mult;
    int shift = roundf((log(scaling) / log(2))) + 10;
    int mult = roundf((1 << shift) / scaling);
    *c_offset = roundf(-out_sub * w_mult * in_mult);
    *a_offset = roundf(w_sub * w_mult);
    *b_offset = roundf(in_sub * in_mult);
    *c_mult = mult;
    *c_shift = shift;
}

/* lowp/lowp_SpatialConvolution.c:112-119 */
void thb_lowp_bias_addends(const unsigned char *qbias, int n, float b_sub, float b_mult, float out_mult, int *addend)
{
    float mult = out_mult / b_mult;
    int add = roundf(b_sub * out_mult);
    for (int i = 0; i < n; i++) {
        int a = qbias[i];
        addend[i] = (int)roundf(a * mult) + add;
    }
}
