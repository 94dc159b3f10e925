/*
 * fp32 CPU oracle -- TEST INFRASTRUCTURE ONLY (see oracle.h).
 *
 * Restates, operator by operator, what the reference's CPU engine computes on
 * NCHW float tensors.  Pinned against the reference itself: tests compare every
 * function here with the unmodified reference sources compiled into
 * oracle/_ref/ and with the golden vectors generated from them.
 */
#include <math.h>
#include <string.h>
#include <float.h>
#include <stdlib.h>
#include "oracle.h"

/* thapi.c:396-403 -- THProcessFloat normalises in place with a true division. */
void orc_normalize(float *x, int N, int C, int H, int W, const float *mean, const float *std)
{
    long hw = (long)H * W;
    for (int n = 0; n < N; n++)
        for (int c = 0; c < C; c++) {
            float *p = x + ((long)n * C + c) * hw;
            for (long i = 0; i < hw; i++) p[i] = (p[i] - mean[c]) / std[c];
        }
}

/* thapi.c:20-46 (rgb2float / bgr2float) -- multiplies by 0.003921568f and by 1/std. */
void orc_images_to_float(const unsigned char *const *images, int N, int W, int H, int stride, int cp,
                         const float *mean, const float *std, int bgr, float *dst)
{
    float inv[3];
    for (int c = 0; c < cp; c++) inv[c] = 1 / std[c];
    for (int n = 0; n < N; n++)
        for (int c = 0; c < cp; c++)
            for (int i = 0; i < H; i++)
                for (int j = 0; j < W; j++) {
                    int sc = bgr ? cp - 1 - c : c;
                    dst[(((long)n * cp + c) * H + i) * W + j] =
                        (images[n][sc + cp * j + stride * i] * 0.003921568f - mean[c]) * inv[c];
                }
}

/* SpatialConvolutionMM.c:159-160 */
int orc_conv_out(int in, int k, int d, int pad) { return (in + 2 * pad - k) / d + 1; }

/* SpatialMaxPooling.c:196-210, SpatialAveragePooling.c:120-139 */
int orc_pool_out(int in, int k, int d, int pad, int ceil_mode)
{
    int o;
    if (ceil_mode) o = (int)ceilf((float)(in - k + 2 * pad) / d) + 1;
    else o = (int)floorf((float)(in - k + 2 * pad) / d) + 1;
    if (pad && (o - 1) * d >= in + pad) --o;
    return o;
}

/*
 * SpatialConvolutionMM.c:75-109,126-225 with thbasic.c:1073-1103: cross-correlation,
 * symmetric zero padding; every output plane starts from its bias value and the
 * products are added in K order (channel, kernel row, kernel column), all in fp32.
 */
void orc_conv2d(const float *x, int N, int C, int H, int W, const float *w, const float *bias,
                int Cout, int kH, int kW, int dH, int dW, int padH, int padW, float *y)
{
    int oH = orc_conv_out(H, kH, dH, padH), oW = orc_conv_out(W, kW, dW, padW);
    long work = (long)N * Cout;
#pragma omp parallel for schedule(dynamic, 1)
    for (long t = 0; t < work; t++) {
        int n = (int)(t / Cout), co = (int)(t % Cout);
        float *yp = y + t * oH * oW;
        float b = bias ? bias[co] : 0.f;
        for (int i = 0; i < oH * oW; i++) yp[i] = b;
        for (int c = 0; c < C; c++) {
            const float *xp = x + ((long)n * C + c) * H * W;
            for (int kh = 0; kh < kH; kh++)
                for (int kw = 0; kw < kW; kw++) {
                    float wv = w[(((long)co * C + c) * kH + kh) * kW + kw];
                    for (int oh = 0; oh < oH; oh++) {
                        int ih = oh * dH - padH + kh;
                        if (ih < 0 || ih >= H) continue;
                        /* valid ow range: 0 <= ow*dW - padW + kw < W */
                        int lo = padW - kw; lo = lo > 0 ? (lo + dW - 1) / dW : 0;
                        int hi = (W - 1 + padW - kw); hi = hi < 0 ? -1 : hi / dW;
                        if (hi > oW - 1) hi = oW - 1;
                        const float *xr = xp + (long)ih * W - padW + kw;
                        float *yr = yp + (long)oh * oW;
                        for (int ow = lo; ow <= hi; ow++) yr[ow] += wv * xr[ow * dW];
                    }
                }
        }
    }
}

/*
 * SpatialFullConvolution.c:99-127 (col2im) and :129-251.  weight is
 * [Cin][Cout][kH][kW]; out = (in-1)*d - 2*pad + k + adj.  When a bias tensor with
 * storage exists the reference's bias GEMM runs with beta = 11, so the result is
 * 11*deconv + bias (:229-238); strict_bias != 0 gives the intended deconv + bias.
 */
void orc_fullconv2d(const float *x, int N, int C, int H, int W, const float *w, const float *bias,
                    int Cout, int kH, int kW, int dH, int dW, int padH, int padW, int adjH, int adjW,
                    int strict_bias, float *y)
{
    int oH = (H - 1) * dH - 2 * padH + kH + adjH, oW = (W - 1) * dW - 2 * padW + kW + adjW;
    long work = (long)N * Cout;
#pragma omp parallel for schedule(dynamic, 1)
    for (long t = 0; t < work; t++) {
        int n = (int)(t / Cout), co = (int)(t % Cout);
        float *yp = y + t * oH * oW;
        memset(yp, 0, sizeof(float) * oH * oW);
        /* columns[(co,kh,kw)][h,w] = sum_c W[c][co][kh][kw] * x[c][h][w]; scattered in (kh,kw) order */
        float *col = (float *)malloc(sizeof(float) * H * W);
        for (int kh = 0; kh < kH; kh++)
            for (int kw = 0; kw < kW; kw++) {
                memset(col, 0, sizeof(float) * H * W);
                for (int c = 0; c < C; c++) {
                    float wv = w[(((long)c * Cout + co) * kH + kh) * kW + kw];
                    const float *xp = x + ((long)n * C + c) * H * W;
                    for (int i = 0; i < H * W; i++) col[i] += wv * xp[i];
                }
                for (int h = 0; h < H; h++) {
                    int oh = h * dH - padH + kh;
                    if (oh < 0 || oh >= oH) continue;
                    for (int ww = 0; ww < W; ww++) {
                        int ow = ww * dW - padW + kw;
                        if (ow >= 0 && ow < oW) yp[(long)oh * oW + ow] += col[h * W + ww];
                    }
                }
            }
        free(col);
        if (bias) {
            float beta = strict_bias ? 1.f : 11.f;
            for (int i = 0; i < oH * oW; i++) yp[i] = beta * yp[i] + bias[co];
        }
    }
}

/* Linear.c:72-113: y = W x + b, W is [M][K] row-major, fp32 accumulation over K. */
void orc_linear(const float *x, int N, int K, const float *w, const float *bias, int M, float *y)
{
#pragma omp parallel for
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            const float *xr = x + (long)n * K, *wr = w + (long)m * K;
            float acc = 0;
            for (int k = 0; k < K; k++) acc += wr[k] * xr[k];
            y[(long)n * M + m] = acc + (bias ? bias[m] : 0.f);
        }
}

/* SpatialBatchNormalization.c:57-116: invstd computed in double then narrowed. */
void orc_batchnorm(const float *x, int N, int C, int HW, const float *mean, const float *var,
                   const float *weight, const float *bias, double eps, float *y)
{
    for (int c = 0; c < C; c++) {
        float m = mean[c];
        float invstd = 1 / sqrt(var[c] + eps);
        float wv = weight ? weight[c] : 1, bv = bias ? bias[c] : 0;
        for (int n = 0; n < N; n++) {
            const float *xp = x + ((long)n * C + c) * HW;
            float *yp = y + ((long)n * C + c) * HW;
            for (int i = 0; i < HW; i++) yp[i] = ((xp[i] - m) * invstd) * wv + bv;
        }
    }
}

/* Threshold.c:38-63: leaky form when alpha != 0, else x > threshold ? x : val. */
void orc_threshold(const float *x, long n, float threshold, float val, float alpha, float *y)
{
    if (alpha)
        for (long i = 0; i < n; i++) y[i] = x[i] >= 0 ? x[i] : x[i] * alpha;
    else
        for (long i = 0; i < n; i++) y[i] = x[i] > threshold ? x[i] : val;
}

/* PReLU.c:32-92: one shared slope when nOutputPlane == 0, else one per channel. */
void orc_prelu(const float *x, int N, int C, int HW, const float *w, int nOutputPlane, float *y)
{
    for (int n = 0; n < N; n++)
        for (int c = 0; c < C; c++) {
            float s = nOutputPlane ? w[c] : w[0];
            const float *xp = x + ((long)n * C + c) * HW;
            float *yp = y + ((long)n * C + c) * HW;
            for (int i = 0; i < HW; i++) yp[i] = xp[i] > 0 ? xp[i] : s * xp[i];
        }
}

/* SpatialMaxPooling.c:74-119,168-247: window clipped to the image, strict '>' from -FLT_MAX. */
void orc_maxpool(const float *x, int N, int C, int H, int W, int kH, int kW, int dH, int dW,
                 int padH, int padW, int ceil_mode, float *y)
{
    int oH = orc_pool_out(H, kH, dH, padH, ceil_mode), oW = orc_pool_out(W, kW, dW, padW, ceil_mode);
#pragma omp parallel for
    for (long p = 0; p < (long)N * C; p++) {
        const float *ip = x + p * H * W;
        float *op = y + p * oH * oW;
        for (int i = 0; i < oH; i++)
            for (int j = 0; j < oW; j++) {
                int hs = i * dH - padH, ws = j * dW - padW;
                int he = hs + kH < H ? hs + kH : H, we = ws + kW < W ? ws + kW : W;
                if (hs < 0) hs = 0;
                if (ws < 0) ws = 0;
                float m = -FLT_MAX;
                for (int yy = hs; yy < he; yy++)
                    for (int xx = ws; xx < we; xx++)
                        if (ip[yy * W + xx] > m) m = ip[yy * W + xx];
                op[i * oW + j] = m;
            }
    }
}

/* SpatialAveragePooling.c:71-207: kW/kH == 0 means global; divisor is the clipped window
 * unless count_include_pad; sequential fp32 sum then one division. */
void orc_avgpool(const float *x, int N, int C, int H, int W, int kH, int kW, int dH, int dW,
                 int padH, int padW, int ceil_mode, int count_include_pad, float *y)
{
    if (kW == 0) kW = W;
    if (kH == 0) kH = H;
    int oH = orc_pool_out(H, kH, dH, padH, ceil_mode), oW = orc_pool_out(W, kW, dW, padW, ceil_mode);
#pragma omp parallel for
    for (long p = 0; p < (long)N * C; p++) {
        const float *ip = x + p * H * W;
        float *op = y + p * oH * oW;
        for (int yy = 0; yy < oH; yy++)
            for (int xx = 0; xx < oW; xx++) {
                int hs = yy * dH - padH, ws = xx * dW - padW;
                int he = hs + kH < H + padH ? hs + kH : H + padH;
                int we = ws + kW < W + padW ? ws + kW : W + padW;
                int pool = (he - hs) * (we - ws);
                if (hs < 0) hs = 0;
                if (ws < 0) ws = 0;
                if (he > H) he = H;
                if (we > W) we = W;
                float sum = 0;
                int div = count_include_pad ? pool : (he - hs) * (we - ws);
                for (int ky = hs; ky < he; ky++)
                    for (int kx = ws; kx < we; kx++) sum += ip[ky * W + kx];
                op[yy * oW + xx] = 0.f + sum / div;
            }
    }
}

/* thbasic.c:462-491: exp(-x) as 1/(degree-4 polynomial)^8 in double, exactly 0 from 13 up. */
double orc_exp_minus_approx(double x)
{
    if (x < 13.0) {
        double y = 1.0 + x * (0.125 + x * (0.0078125 + x * (0.00032552083 + x * 1.0172526e-5)));
        y *= y;
        y *= y;
        y *= y;
        return 1 / y;
    }
    return 0;
}

/* SoftMax.c:24-90: softmax over `dim` entries spaced `stride` apart, per frame and position. */
void orc_softmax(const float *x, int nframe, int dim, int stride, float *y)
{
    for (long t = 0; t < (long)stride * nframe; t++) {
        const float *ip = x + (t / stride) * dim * stride + t % stride;
        float *op = y + (t / stride) * dim * stride + t % stride;
        float mx = -FLT_MAX, sum = 0;
        for (int d = 0; d < dim; d++)
            if (ip[(long)d * stride] >= mx) mx = ip[(long)d * stride];
        for (int d = 0; d < dim; d++) {
            float z = orc_exp_minus_approx(mx - ip[(long)d * stride]);
            op[(long)d * stride] = z;
            sum += z;
        }
        for (int d = 0; d < dim; d++) op[(long)d * stride] *= 1 / sum;
    }
}

/*
 * CAddTable.c:32-86.  With exactly two inputs a CAddTable SUBTRACTS (a - b) and a
 * CSubTable adds; elements of a beyond b's length are copied.  With any other count
 * the output starts as input 0 and then every input (0 included) is added (or
 * subtracted for CSubTable), so input 0 is counted twice.
 */
void orc_caddtable(const float *const *ins, const long *n, int nin, int is_csub, float *y)
{
    long j;
    if (nin == 2) {
        if (is_csub) for (j = 0; j < n[1]; j++) y[j] = ins[0][j] + ins[1][j];
        else for (j = 0; j < n[1]; j++) y[j] = ins[0][j] - ins[1][j];
        for (; j < n[0]; j++) y[j] = ins[0][j];
        return;
    }
    for (j = 0; j < n[0]; j++) y[j] = ins[0][j];
    for (int i = 0; i < nin; i++)
        for (j = 0; j < n[i]; j++) {
            if (is_csub) y[j] -= ins[i][j];
            else y[j] += ins[i][j];
        }
}

/* JoinTable.c:34-86 / Concat.c:21-76 along the channel dimension of [N][C][HW] tensors. */
void orc_join_channels(const float *const *ins, const int *C, int nin, int N, int HW, float *y)
{
    int Ctot = 0;
    for (int i = 0; i < nin; i++) Ctot += C[i];
    for (int n = 0; n < N; n++) {
        long off = 0;
        for (int i = 0; i < nin; i++) {
            memcpy(y + ((long)n * Ctot + off) * HW, ins[i] + (long)n * C[i] * HW,
                   sizeof(float) * (long)C[i] * HW);
            off += C[i];
        }
    }
}
