// Operators outside the benchmark networks that complete the module coverage: 2x upsampling, zero padding / cropping,
// slicing, elementwise maximum, LogSoftMax, L2 normalisation and max unpooling.  All of them move or compare data
// (HBM-bound); they work on channels-innermost tensors of fp32, fp16 or bf16, one thread per (pixel, 16-byte chunk)
// where the access pattern allows it and per element otherwise.
#include "common.cuh"
#include <math.h>

namespace {

inline int nblk(long n, int bs = 256) { return (int)((n + bs - 1) / bs); }

#define SHAPE_DISPATCH(dtype, CALL)                                \
    switch (dtype) {                                               \
    case THB_F32: { using T = float; CALL; break; }                \
    case THB_F16: { using T = __half; CALL; break; }               \
    case THB_BF16: { using T = __nv_bfloat16; CALL; break; }       \
    default: return THB_ERR_UNSUPPORTED;                           \
    }

// y[n][oh][ow][c] = x[n][oh + top][ow + left][c] inside the source, 0 outside (top/left may be negative = padding, or
// positive = cropping); up2 = 1: nearest-neighbour 2x upsampling instead (source pixel (oh/2, ow/2)); up2 = 2: reflection
// padding (positions outside mirror about the first / last row and column, the border itself not repeated).
template <typename T>
__global__ void window_copy_kernel(const T *__restrict__ x, int N, int H, int W, int C, int x_ld, int top, int left, int up2,
                                   int oH, int oW, T *__restrict__ y, int y_ld)
{
    const int vec = 16 / (int)sizeof(T), chunks = (C + vec - 1) / vec;
    const long total = (long)N * oH * oW * chunks;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int ck = (int)(i % chunks);
    long pix = i / chunks;
    const int ow = (int)(pix % oW);
    pix /= oW;
    const int oh = (int)(pix % oH), n = (int)(pix / oH);
    int ih = up2 == 1 ? oh >> 1 : oh + top, iw = up2 == 1 ? ow >> 1 : ow + left;
    if (up2 == 2) {
        ih = ih < 0 ? -ih : ih >= H ? 2 * H - 2 - ih : ih;
        iw = iw < 0 ? -iw : iw >= W ? 2 * W - 2 - iw : iw;
    }
    uint4 v = make_uint4(0, 0, 0, 0);
    if ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W)
        v = *reinterpret_cast<const uint4 *>(x + (((long)n * H + ih) * W + iw) * x_ld + ck * vec);
    *reinterpret_cast<uint4 *>(y + (((long)n * oH + oh) * oW + ow) * y_ld + ck * vec) = v;
}

// channels [from, from + C) of x -> channels [0, C) of y, any `from` (element accesses); padded channels of y become 0
template <typename T>
__global__ void channel_slice_kernel(const T *__restrict__ x, long pixels, int from, int C, int x_ld, T *__restrict__ y, int y_ld, int y_pad)
{
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pixels * y_pad) return;
    const int c = (int)(i % y_pad);
    const long p = i / y_pad;
    dt<T>::st(y + p * y_ld + c, c < C ? dt<T>::ld(x + p * x_ld + from + c) : 0.f);
}

// y[n][p][c] = x[n][c * HW + p]: a vector per image in (channel, row, column) order becomes a channels-innermost map;
// padded channels of y become 0
template <typename T>
__global__ void from_nchw_kernel(const T *__restrict__ x, int x_ld, long images_pixels, long HW, int C, T *__restrict__ y, int y_ld, int y_pad)
{
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= images_pixels * y_pad) return;
    const int c = (int)(i % y_pad);
    const long np = i / y_pad, n = np / HW, p = np % HW;
    dt<T>::st(y + np * y_ld + c, c < C ? dt<T>::ld(x + n * x_ld + c * HW + p) : 0.f);
}

struct MaxIn {
    const void *x[8];
    int ld[8];
};
// Cmax.c:33-66: elementwise maximum over the inputs (all of one shape here)
template <typename T>
__global__ void cmax_kernel(MaxIn in, int nin, long pixels, int C, T *__restrict__ y, int y_ld, int y_pad)
{
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pixels * y_pad) return;
    const int c = (int)(i % y_pad);
    const long p = i / y_pad;
    float v = 0.f;
    if (c < C) {
        v = dt<T>::ld(reinterpret_cast<const T *>(in.x[0]) + p * in.ld[0] + c);
        for (int k = 1; k < nin; k++) {
            const float w = dt<T>::ld(reinterpret_cast<const T *>(in.x[k]) + p * in.ld[k] + c);
            v = v > w ? v : w;   // MAX(a, b) = a > b ? a : b
        }
    }
    dt<T>::st(y + p * y_ld + c, v);
}

// LogSoftMax.c:56-79 over the channels of each pixel, one warp per pixel: max (with >=), sum of exp(x - max) accumulated
// in float, logSum = max + log(sum).  The reference's last loop reads the values it subtracts logSum from at the START of
// the whole input (frame 0, position 0) for every frame and position; quirk = 1 reproduces that, 0 subtracts from the
// pixel's own values.
template <typename T>
__global__ void logsoftmax_kernel(const T *__restrict__ x, long pixels, int C, int x_ld, T *__restrict__ y, int y_ld, int quirk)
{
    const long p = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (p >= pixels) return;
    const T *row = x + p * x_ld;
    float mx = -INFINITY;
    for (int c = lane; c < C; c += 32) mx = fmaxf(mx, dt<T>::ld(row + c));
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int c = lane; c < C; c += 32) sum += (float)exp((double)(dt<T>::ld(row + c) - mx));
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float logsum = mx + (float)log((double)sum);
    const T *src = quirk ? x : row;
    for (int c = lane; c < C; c += 32) dt<T>::st(y + p * y_ld + c, dt<T>::ld(src + c) - logsum);
}

// sum of squares of `len` consecutive elements per row (padding elements are zero and change nothing): one block per row
template <typename T>
__global__ void sumsq_rows_kernel(const T *__restrict__ x, long row_len, float *__restrict__ out)
{
    __shared__ float part[32];
    const T *row = x + (long)blockIdx.x * row_len;
    float s = 0.f;
    for (long i = threadIdx.x; i < row_len; i += blockDim.x) {
        const float v = dt<T>::ld(row + i);
        s = fmaf(v, v, s);
    }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (threadIdx.x == 0) out[blockIdx.x] = s;
    }
}
// y = x / sqrtf(sum), sum = sums[row] (per_row) or the total of all rows' sums (Normalize.c:21-41)
template <typename T>
__global__ void normalize_scale_kernel(const T *__restrict__ x, long rows, long row_len, const float *__restrict__ sums, int per_row,
                                       T *__restrict__ y)
{
    __shared__ float total;
    if (!per_row) {
        if (threadIdx.x == 0) {
            float t = 0.f;
            for (long r = 0; r < rows; r++) t += sums[r];
            total = t;
        }
        __syncthreads();
    }
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * row_len) return;
    const float nrm = sqrtf(per_row ? sums[i / row_len] : total);
    dt<T>::st(y + i, dt<T>::ld(x + i) / nrm);
}

// SpatialMaxUnpooling.c:14-40 as a gather.  v: pooled-size values [N][oH][oW][C]; xin: the pooling's input [N][H][W][C];
// y: [N][H][W][C].  The reference zeroes the output and scatters every pooled value to the position of its window's
// maximum (first maximum in row-major window order, strict >, SpatialMaxPooling.c:95-112), later windows overwriting
// earlier ones.  Here each output element looks at the windows that contain it, from the last one in row-major order to
// the first, and takes the value of the first whose maximum sits on it.
template <typename T>
__global__ void max_unpool_kernel(const T *__restrict__ v, const T *__restrict__ xin, int N, int H, int W, int C, int x_ld, int v_ld,
                                  int kH, int kW, int dH, int dW, int padH, int padW, int oH, int oW, T *__restrict__ y, int y_ld, int y_pad)
{
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long total = (long)N * H * W * y_pad;
    if (i >= total) return;
    const int c = (int)(i % y_pad);
    long pix = i / y_pad;
    const int w = (int)(pix % W);
    pix /= W;
    const int h = (int)(pix % H), n = (int)(pix / H);
    float out = 0.f;
    if (c < C) {
        // windows (i, j) with i*dH - padH <= h < i*dH - padH + kH
        int i1 = (h + padH) / dH, j1 = (w + padW) / dW;
        int i0 = (h + padH - kH + dH) / dH, j0 = (w + padW - kW + dW) / dW;
        if (h + padH - kH + 1 <= 0) i0 = 0;
        if (w + padW - kW + 1 <= 0) j0 = 0;
        if (i1 > oH - 1) i1 = oH - 1;
        if (j1 > oW - 1) j1 = oW - 1;
        bool found = false;
        for (int wi = i1; wi >= i0 && !found; wi--)
            for (int wj = j1; wj >= j0 && !found; wj--) {
                int hs = wi * dH - padH, ws = wj * dW - padW;
                const int he = min(hs + kH, H), we = min(ws + kW, W);
                hs = max(hs, 0);
                ws = max(ws, 0);
                if (h < hs || h >= he || w < ws || w >= we) continue;
                float best = -INFINITY;
                int bh = -1, bw = -1;
                for (int a = hs; a < he; a++)
                    for (int b = ws; b < we; b++) {
                        const float val = dt<T>::ld(xin + (((long)n * H + a) * W + b) * x_ld + c);
                        if (val > best) { best = val; bh = a; bw = b; }
                    }
                if (bh == h && bw == w) {
                    out = dt<T>::ld(v + (((long)n * oH + wi) * oW + wj) * v_ld + c);
                    found = true;
                }
            }
    }
    dt<T>::st(y + (((long)n * H + h) * W + w) * y_ld + c, out);
}

}  // namespace

extern "C" {

int thb_upsample2x(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, int y_ld, thb_stream s)
{
    const int vec = dtype == THB_F32 ? 4 : 8;
    if (x_ld % vec || y_ld % vec) return THB_ERR_ARG;
    const long total = (long)N * 2 * H * 2 * W * ((C + vec - 1) / vec);
    if (total == 0) return THB_OK;
    SHAPE_DISPATCH(dtype, (window_copy_kernel<T><<<nblk(total), 256, 0, (cudaStream_t)s>>>((const T *)x, N, H, W, C, x_ld, 0, 0, 1, 2 * H,
                                                                                           2 * W, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("window_copy_kernel (upsample)");
}

int thb_zero_pad(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int pad_l, int pad_r, int pad_t, int pad_b, void *y,
                 int y_ld, thb_stream s)
{
    const int vec = dtype == THB_F32 ? 4 : 8;
    const int oH = H + pad_t + pad_b, oW = W + pad_l + pad_r;
    if (x_ld % vec || y_ld % vec || oH < 1 || oW < 1) return THB_ERR_ARG;
    const long total = (long)N * oH * oW * ((C + vec - 1) / vec);
    SHAPE_DISPATCH(dtype, (window_copy_kernel<T><<<nblk(total), 256, 0, (cudaStream_t)s>>>((const T *)x, N, H, W, C, x_ld, -pad_t, -pad_l, 0,
                                                                                           oH, oW, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("window_copy_kernel (zero padding)");
}

int thb_reflect_pad(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int pad_l, int pad_r, int pad_t, int pad_b, void *y,
                    int y_ld, thb_stream s)
{
    const int vec = dtype == THB_F32 ? 4 : 8;
    const int oH = H + pad_t + pad_b, oW = W + pad_l + pad_r;
    if (x_ld % vec || y_ld % vec || pad_l < 0 || pad_r < 0 || pad_t < 0 || pad_b < 0 || pad_t >= H || pad_b >= H || pad_l >= W || pad_r >= W)
        return THB_ERR_ARG;
    const long total = (long)N * oH * oW * ((C + vec - 1) / vec);
    SHAPE_DISPATCH(dtype, (window_copy_kernel<T><<<nblk(total), 256, 0, (cudaStream_t)s>>>((const T *)x, N, H, W, C, x_ld, -pad_t, -pad_l, 2,
                                                                                           oH, oW, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("window_copy_kernel (reflection padding)");
}

int thb_slice_channels(int dtype, const void *x, long pixels, int from, int C, int x_ld, void *y, int y_ld, thb_stream s)
{
    const int al = dtype == THB_F32 ? 4 : 8, y_pad = (C + al - 1) / al * al;
    if (pixels == 0) return THB_OK;
    if (from < 0 || C < 1 || y_pad > y_ld) return THB_ERR_ARG;
    SHAPE_DISPATCH(dtype, (channel_slice_kernel<T><<<nblk(pixels * y_pad), 256, 0, (cudaStream_t)s>>>((const T *)x, pixels, from, C, x_ld,
                                                                                                      (T *)y, y_ld, y_pad)));
    return THB_LAUNCH_CHECK("channel_slice_kernel");
}

int thb_from_nchw(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, int y_ld, thb_stream s)
{
    const int al = dtype == THB_F32 ? 4 : 8, y_pad = (C + al - 1) / al * al;
    const long HW = (long)H * W;
    if (N < 1 || C < 1 || HW < 1 || y_pad > y_ld || (long)C * HW > x_ld) return THB_ERR_ARG;
    SHAPE_DISPATCH(dtype, (from_nchw_kernel<T><<<nblk(N * HW * y_pad), 256, 0, (cudaStream_t)s>>>((const T *)x, x_ld, N * HW, HW, C, (T *)y,
                                                                                                 y_ld, y_pad)));
    return THB_LAUNCH_CHECK("from_nchw_kernel");
}

int thb_cmax(int dtype, int nin, const void *const *x_host, const int *ld_host, long pixels, int C, void *y, int y_ld, thb_stream s)
{
    if (nin < 1 || nin > 8) return THB_ERR_UNSUPPORTED;
    const int al = dtype == THB_F32 ? 4 : 8, y_pad = (C + al - 1) / al * al;
    if (pixels == 0) return THB_OK;
    MaxIn in;
    for (int k = 0; k < nin; k++) { in.x[k] = x_host[k]; in.ld[k] = ld_host[k]; }
    SHAPE_DISPATCH(dtype, (cmax_kernel<T><<<nblk(pixels * y_pad), 256, 0, (cudaStream_t)s>>>(in, nin, pixels, C, (T *)y, y_ld, y_pad)));
    return THB_LAUNCH_CHECK("cmax_kernel");
}

int thb_logsoftmax(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, int first_frame_quirk, thb_stream s)
{
    if (pixels == 0) return THB_OK;
    SHAPE_DISPATCH(dtype, (logsoftmax_kernel<T><<<nblk(pixels * 32), 256, 0, (cudaStream_t)s>>>((const T *)x, pixels, C, x_ld, (T *)y, y_ld,
                                                                                                first_frame_quirk)));
    return THB_LAUNCH_CHECK("logsoftmax_kernel");
}

int thb_l2_normalize(int dtype, const void *x, long rows, long row_len, int per_row, float *scratch_rows, void *y, thb_stream s)
{
    if (rows < 1 || row_len < 1) return THB_OK;
    SHAPE_DISPATCH(dtype, (sumsq_rows_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)s>>>((const T *)x, row_len, scratch_rows)));
    int rc = THB_LAUNCH_CHECK("sumsq_rows_kernel");
    if (rc) return rc;
    SHAPE_DISPATCH(dtype, (normalize_scale_kernel<T><<<nblk(rows * row_len), 256, 0, (cudaStream_t)s>>>((const T *)x, rows, row_len,
                                                                                                        scratch_rows, per_row, (T *)y)));
    return THB_LAUNCH_CHECK("normalize_scale_kernel");
}

int thb_max_unpool(int dtype, const void *v, int v_ld, const void *pool_in, int x_ld, int N, int H, int W, int C, int kH, int kW, int dH,
                   int dW, int padH, int padW, int oH, int oW, void *y, int y_ld, thb_stream s)
{
    const int al = dtype == THB_F32 ? 4 : 8, y_pad = (C + al - 1) / al * al;
    const long total = (long)N * H * W * y_pad;
    if (total == 0) return THB_OK;
    if (kH < 1 || kW < 1 || dH < 1 || dW < 1 || y_pad > y_ld) return THB_ERR_ARG;
    SHAPE_DISPATCH(dtype, (max_unpool_kernel<T><<<nblk(total), 256, 0, (cudaStream_t)s>>>((const T *)v, (const T *)pool_in, N, H, W, C, x_ld,
                                                                                          v_ld, kH, kW, dH, dW, padH, padW, oH, oW, (T *)y,
                                                                                          y_ld, y_pad)));
    return THB_LAUNCH_CHECK("max_unpool_kernel");
}

}  // extern "C"
