/* CPU restatement of the reference's remaining operators -- TEST INFRASTRUCTURE ONLY (see oracle.h).
 * NCHW fp32 throughout, each function citing the reference lines it follows. */
#include <math.h>
#include <string.h>
#include "oracle.h"

/* modules/Upsample.c:18-63: every input element fills a 2 x 2 block */
void orc_upsample2x(const float *x, int N, int C, int H, int W, float *y)
{
    for (long p = 0; p < (long)N * C; p++)
        for (int h = 0; h < H; h++)
            for (int w = 0; w < W; w++) {
                const float v = x[(p * H + h) * W + w];
                float *o = y + (p * 2 * H + 2 * h) * 2 * W + 2 * w;
                o[0] = o[1] = o[2 * W] = o[2 * W + 1] = v;
            }
}

/* modules/SpatialZeroPadding.c:17-60 as it is meant: out[h + pad_t][w + pad_l] = in[h][w], zero elsewhere, negative
 * pads crop.  (The reference's loop strides input rows by the HEIGHT and clears pad_r floats past the row's end instead
 * of the right padding, so its own result is only defined for square maps with pad_r <= 0; there it equals this.) */
void orc_zero_pad(const float *x, int N, int C, int H, int W, int pad_l, int pad_r, int pad_t, int pad_b, float *y)
{
    const int oH = H + pad_t + pad_b, oW = W + pad_l + pad_r;
    for (long p = 0; p < (long)N * C; p++)
        for (int oh = 0; oh < oH; oh++)
            for (int ow = 0; ow < oW; ow++) {
                const int h = oh - pad_t, w = ow - pad_l;
                y[(p * oH + oh) * oW + ow] = (h >= 0 && h < H && w >= 0 && w < W) ? x[(p * H + h) * W + w] : 0.f;
            }
}

/* modules/Slice.c:34-39, thbasic.c:192-209: elements [from, to) along `axis` of a contiguous tensor of `ndim` sizes */
void orc_slice(const float *x, const long *size, int ndim, int axis, long from, long to, float *y)
{
    long outer = 1, inner = 1;
    for (int i = 0; i < axis; i++) outer *= size[i];
    for (int i = axis + 1; i < ndim; i++) inner *= size[i];
    for (long o = 0; o < outer; o++)
        memcpy(y + o * (to - from) * inner, x + (o * size[axis] + from) * inner, sizeof(float) * (to - from) * inner);
}

/* modules/Cmax.c:20-68 for inputs of one size: a > b ? a : b, left to right */
void orc_cmax(const float *const *ins, int nin, long n, float *y)
{
    for (long j = 0; j < n; j++) {
        float v = ins[0][j];
        for (int i = 1; i < nin; i++) v = v > ins[i][j] ? v : ins[i][j];
        y[j] = v;
    }
}

/* modules/LogSoftMax.c:19-81, including its last loop, which subtracts logSum from input_data[d*stride] -- the values at
 * the START of the input -- for every frame and position (:77); first_frame_quirk = 0 subtracts from the position's own */
void orc_logsoftmax(const float *x, long nframe, long dim, long stride, int first_frame_quirk, float *y)
{
    for (long t = 0; t < stride * nframe; t++) {
        const float *ip = x + (t / stride) * dim * stride + t % stride;
        float *op = y + (t / stride) * dim * stride + t % stride;
        float logSum = 0, inputMax = -INFINITY;
        for (long d = 0; d < dim; d++)
            if (ip[d * stride] >= inputMax) inputMax = ip[d * stride];
        for (long d = 0; d < dim; d++) logSum += exp(ip[d * stride] - inputMax);
        logSum = inputMax + log(logSum);
        for (long d = 0; d < dim; d++) op[d * stride] = (first_frame_quirk ? x[d * stride] : ip[d * stride]) - logSum;
    }
}

/* modules/Normalize.c:12-44: rows of a 2-D tensor, or the whole tensor */
void orc_l2_normalize(const float *x, long rows, long row_len, int per_row, float *y)
{
    if (per_row) {
        for (long i = 0; i < rows; i++) {
            float sum = 0;
            for (long j = 0; j < row_len; j++) sum += x[i * row_len + j] * x[i * row_len + j];
            sum = sqrtf(sum);
            for (long j = 0; j < row_len; j++) y[i * row_len + j] = x[i * row_len + j] / sum;
        }
    } else {
        float sum = 0;
        for (long j = 0; j < rows * row_len; j++) sum += x[j] * x[j];
        sum = sqrtf(sum);
        for (long j = 0; j < rows * row_len; j++) y[j] = x[j] / sum;
    }
}

/* modules/SpatialMaxPooling.c:74-119 (the indices it records) + modules/SpatialMaxUnpooling.c:14-40: output zeroed, then
 * every pooled-size value v[i][j] written at the position of the maximum of window (i, j) of the pooling's input, windows
 * in row-major order (a later window overwrites an earlier one) */
void orc_max_unpool(const float *v, const float *pool_in, int N, int C, int H, int W, int kH, int kW, int dH, int dW, int padH,
                    int padW, int oH, int oW, float *y)
{
    memset(y, 0, sizeof(float) * (size_t)N * C * H * W);
    for (long p = 0; p < (long)N * C; p++) {
        const float *ip = pool_in + p * H * W, *vp = v + p * oH * oW;
        float *op = y + p * H * W;
        for (int i = 0; i < oH; i++)
            for (int j = 0; j < oW; j++) {
                long hstart = (long)i * dH - padH, wstart = (long)j * dW - padW;
                long hend = hstart + kH < H ? hstart + kH : H, wend = wstart + kW < W ? wstart + kW : W;
                if (hstart < 0) hstart = 0;
                if (wstart < 0) wstart = 0;
                long maxindex = -1;
                float maxval = -INFINITY;
                for (long a = hstart; a < hend; a++)
                    for (long b = wstart; b < wend; b++)
                        if (ip[a * W + b] > maxval) { maxval = ip[a * W + b]; maxindex = a * W + b; }
                if (maxindex >= 0) op[maxindex] = vp[i * oW + j];
            }
    }
}
