/*
 * uint8 "lowp" CPU oracle -- TEST INFRASTRUCTURE ONLY (see oracle.h).
 *
 * Restates the lowp/ directory of the reference.  Batches are defined PER IMAGE: the
 * reference's lowp convolution addresses byte buffers with float-sized offsets
 * for every image after the first, so it is only meaningful at batch 1; a batch
 * here is the batch-1 algorithm applied to each image with shared quantisation
 * parameters.  The GEMM core is the contract in lowpgemm_contract.c (parity
 * unpinned there); everything else is pinned against the reference's own lowp
 * sources compiled around that contract (oracle/_ref/libthnets_ref_lowp.so).
 */
#include <math.h>
#include <string.h>
#include <stdlib.h>
#include <stdint.h>
#include "oracle.h"

/*
 * lowp_basic.c:5-38.  The range always contains 0 (min = max = 0 to start);
 * mult = 255.0 / (max - min) evaluated in double then narrowed; each element is
 * roundf(x*mult) - roundf(min*mult), the two terms rounded separately, so the top
 * element can come out as 256: the float -> unsigned char conversion of 256.0 is
 * undefined in C; gcc on x86-64 converts through int and keeps the low byte (0),
 * which is what this does.
 */
void orc_lowp_quantize(const float *x, long n, unsigned char *q, float *sub, float *mult)
{
    float mn = 0, mx = 0, m;
    for (long i = 0; i < n; i++) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
    }
    if (mx - mn > 0) m = 255.0 / (mx - mn);
    else m = 0;
    float zr = roundf(mn * m);
    for (long i = 0; i < n; i++) q[i] = (unsigned char)(int)(roundf(x[i] * m) - zr);
    *sub = mn;
    *mult = m;
}

/* lowp_basic.c:40-58 */
void orc_lowp_dequantize(const unsigned char *q, long n, float sub, float mult, float *x)
{
    float inv = mult ? 1.0 / mult : 0;
    for (long i = 0; i < n; i++) x[i] = q[i] * inv + sub;
}

/* lowp_basic.c:214-222: clamp then TRUNCATE (not round). */
unsigned char orc_lowp_scale_float(float sub, float mult, float value)
{
    float scaled = (value - sub) * mult;
    if (scaled < 0) return 0;
    if (scaled > 255) return 255;
    return (unsigned char)scaled;
}

/* lowp_basic.c:299-321: the float expressions, roundf and log calls in the reference's order. */
void orc_lowp_gemm_params(float w_sub, float w_mult, float in_sub, float in_mult, float out_sub,
                          float out_mult, int *a_offset, int *b_offset, int *c_offset, int *c_mult,
                          int *c_shift)
{
    float scaling = w_mult * in_mult / out_mult;
    int shift = roundf((log(scaling) / log(2))) + 10;
    int mult = roundf((1 << shift) / scaling);
    int offset = roundf(-out_sub * w_mult * in_mult);
    *a_offset = roundf(w_sub * w_mult);
    *b_offset = roundf(in_sub * in_mult);
    *c_offset = offset;
    *c_mult = mult;
    *c_shift = shift;
}

/* lowp_SpatialConvolution.c:5-69: u8 im2col of ONE image, rows ordered (channel, kh, kw),
 * out-of-image taps filled with the byte `zero`. */
static void unfold_u8(const unsigned char *x, int C, int H, int W, int kH, int kW, int dH, int dW,
                      int padH, int padW, int oH, int oW, unsigned char zero, unsigned char *col)
{
    for (long k = 0; k < (long)C * kH * kW; k++) {
        int c = (int)(k / (kH * kW)), rest = (int)(k % (kH * kW)), kh = rest / kW, kw = rest % kW;
        unsigned char *dst = col + k * oH * oW;
        const unsigned char *src = x + (long)c * H * W;
        for (int y = 0; y < oH; y++) {
            int iy = y * dH - padH + kh;
            for (int xx = 0; xx < oW; xx++) {
                int ix = xx * dW - padW + kw;
                dst[y * oW + xx] = (iy < 0 || iy >= H || ix < 0 || ix >= W) ? zero : src[iy * W + ix];
            }
        }
    }
}

/* The int32 accumulators of one image before requantisation: what "int32 accumulators
 * bit-exact" refers to.  acc is [Cout][oH*oW]. */
void orc_lowp_conv_acc(const unsigned char *x, int C, int H, int W, const unsigned char *w, int Cout,
                       int kH, int kW, int dH, int dW, int padH, int padW, int zero, int a_offset,
                       int b_offset, int *acc)
{
    int oH = orc_conv_out(H, kH, dH, padH), oW = orc_conv_out(W, kW, dW, padW);
    long K = (long)C * kH * kW, P = (long)oH * oW;
    unsigned char *col = (unsigned char *)malloc(K * P);
    unfold_u8(x, C, H, W, kH, kW, dH, dW, padH, padW, oH, oW, (unsigned char)zero, col);
#pragma omp parallel for
    for (int co = 0; co < Cout; co++) {
        uint32_t *row = (uint32_t *)(acc + (long)co * P);
        memset(row, 0, sizeof(int) * P);
        for (long k = 0; k < K; k++) {
            int av = w[(long)co * K + k] + a_offset;
            const unsigned char *cr = col + k * P;
            for (long p = 0; p < P; p++) row[p] += (uint32_t)(av * (cr[p] + b_offset));
        }
    }
    free(col);
}

/* lowp_SpatialConvolution.c:71-88: the groups of 8 clamp to [0,255]; the len%8 tail only
 * clamps at 255, so a negative sum there wraps modulo 256. */
static void lowpadd(unsigned char *dst, int add, int len)
{
    int i;
    for (i = 0; i < len - 7; i += 8)
        for (int j = 0; j < 8; j++) {
            int v = dst[i + j] + add;
            dst[i + j] = v > 255 ? 255 : v < 0 ? 0 : v;
        }
    for (; i < len; i++) {
        int v = dst[i] + add;
        dst[i] = v > 255 ? 255 : (unsigned char)v;
    }
}

/*
 * lowp_SpatialConvolution.c:90-122,124-187 for every image of the batch: padding byte
 * zero = roundf(-in_sub*in_mult) (:101), GEMM with the parameters of lowp_basic.c:299-321,
 * then per output plane the saturating add of
 * roundf(qbias * (out_mult / b_mult)) + roundf(b_sub * out_mult)   (:112-119).
 */
void orc_lowp_conv(const unsigned char *x, int N, int C, int H, int W, float in_sub, float in_mult,
                   const unsigned char *w, float w_sub, float w_mult, const unsigned char *bias,
                   float b_sub, float b_mult, int Cout, int kH, int kW, int dH, int dW, int padH,
                   int padW, float out_sub, float out_mult, unsigned char *y)
{
    int oH = orc_conv_out(H, kH, dH, padH), oW = orc_conv_out(W, kW, dW, padW);
    long K = (long)C * kH * kW, P = (long)oH * oW;
    int zero = roundf(-in_sub * in_mult);
    int a_off, b_off, c_off, c_mult, c_shift;
    orc_lowp_gemm_params(w_sub, w_mult, in_sub, in_mult, out_sub, out_mult, &a_off, &b_off, &c_off,
                         &c_mult, &c_shift);
    float bm = out_mult / b_mult;
    int add = roundf(b_sub * out_mult);
    unsigned char *col = (unsigned char *)malloc(K * P);
    for (int n = 0; n < N; n++) {
        unsigned char *yn = y + (long)n * Cout * P;
        unfold_u8(x + (long)n * C * H * W, C, H, W, kH, kW, dH, dW, padH, padW, oH, oW,
                  (unsigned char)zero, col);
        lowpgemm(1, 1, 1, Cout, (int)P, (int)K, w, col, yn, (int)K, (int)P, (int)P, a_off, b_off, c_off,
                 c_mult, c_shift);
        for (int co = 0; co < Cout; co++) {
            int addend = bias[co];
            addend = roundf(addend * bm) + add;
            lowpadd(yn + (long)co * P, addend, (int)P);
        }
    }
    free(col);
}

/* lowp_SpatialMaxPooling.c:4-43,45-108: u8 maximum starting from 0. */
void orc_lowp_maxpool(const unsigned char *x, int N, int C, int H, int W, int kH, int kW, int dH,
                      int dW, int padH, int padW, int ceil_mode, unsigned char *y)
{
    int oH = orc_pool_out(H, kH, dH, padH, ceil_mode), oW = orc_pool_out(W, kW, dW, padW, ceil_mode);
    for (long p = 0; p < (long)N * C; p++) {
        const unsigned char *ip = x + p * H * W;
        unsigned char *op = y + p * oH * oW;
        for (int i = 0; i < oH; i++)
            for (int j = 0; j < oW; j++) {
                int hs = i * dH - padH, ws = j * dW - padW;
                int he = hs + kH < H ? hs + kH : H, we = ws + kW < W ? ws + kW : W;
                if (hs < 0) hs = 0;
                if (ws < 0) ws = 0;
                unsigned char m = 0;
                for (int yy = hs; yy < he; yy++)
                    for (int xx = ws; xx < we; xx++)
                        if (ip[yy * W + xx] > m) m = ip[yy * W + xx];
                op[i * oW + j] = m;
            }
    }
}

/* lowp_Threshold.c:3-28: q > threshold ? q : val, both bytes from orc_lowp_scale_float. */
void orc_lowp_threshold(const unsigned char *x, long n, unsigned char threshold, unsigned char val,
                        unsigned char *y)
{
    for (long i = 0; i < n; i++) y[i] = x[i] > threshold ? x[i] : val;
}

/* lowp_basic.c:60-131: u8 HWC images straight to planar u8 with a static range from mean/std. */
void orc_lowp_images(const unsigned char *const *images, int N, int W, int H, int stride,
                     const float *mean, const float *std, int bgr, unsigned char *dst, float *sub,
                     float *mult)
{
    float mn = 1e30, mx = -1e30, m, mul[3];
    int isub[3];
    for (int i = 0; i < 3; i++) {
        if (-mean[i] / std[i] < mn) mn = -mean[i] / std[i];
        if ((1 - mean[i]) / std[i] > mx) mx = (1 - mean[i]) / std[i];
    }
    if (mx - mn) m = 255 / (mx - mn);
    else m = 0;
    for (int i = 0; i < 3; i++) {
        isub[i] = roundf(255 * (mean[i] + std[i] * mn));
        mul[i] = m / (255 * std[i]);
    }
    for (int n = 0; n < N; n++)
        for (int c = 0; c < 3; c++)
            for (int i = 0; i < H; i++)
                for (int j = 0; j < W; j++) {
                    int sc = bgr ? 2 - c : c;
                    dst[(((long)n * 3 + c) * H + i) * W + j] =
                        (unsigned char)(int)roundf((images[n][sc + 3 * j + stride * i] - isub[c]) * mul[c]);
                }
    *sub = mn;
    *mult = m;
}
