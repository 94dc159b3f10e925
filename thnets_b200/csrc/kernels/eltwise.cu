// HBM-bound kernels of the forward pass: layout/precision boundary, pooling, per-channel affine +
// activation, tensor combination, channel-slice copies, softmax, col2im gather, u8 helpers.
// All of them walk channels-innermost tensors in 16-byte channel vectors so that every global access
// of a warp is a run of full sectors.
#include "common.cuh"
#include <float.h>
#include <math.h>

namespace {

// ---- 16-byte channel vectors --------------------------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float *p, float (&v)[4])
    {
        float4 t = *reinterpret_cast<const float4 *>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4])
    {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half *p, float (&v)[8])
    {
        uint4 t = *reinterpret_cast<const uint4 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[8])
    {
        uint4 t;
        __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = t;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8])
    {
        uint4 t = *reinterpret_cast<const uint4 *>(p);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[8])
    {
        uint4 t;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = t;
    }
};
template <> struct Vec<uint8_t> {
    static constexpr int N = 16;
    static __device__ __forceinline__ void load(const uint8_t *p, float (&v)[16])
    {
        uint4 t = *reinterpret_cast<const uint4 *>(p);
        const uint8_t *b = reinterpret_cast<const uint8_t *>(&t);
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = (float)b[i];
    }
    static __device__ __forceinline__ void store(uint8_t *p, const float (&v)[16])
    {
        uint4 t;
        uint8_t *b = reinterpret_cast<uint8_t *>(&t);
#pragma unroll
        for (int i = 0; i < 16; i++) b[i] = (uint8_t)(int)v[i];
        *reinterpret_cast<uint4 *>(p) = t;
    }
};

inline int nblocks(long n, int bs = 256) { return (int)((n + bs - 1) / bs); }

#define DISPATCH_FLOAT_DTYPE(dtype, CALL)                         \
    switch (dtype) {                                               \
    case THB_F32: { using T = float; CALL; break; }                \
    case THB_F16: { using T = __half; CALL; break; }               \
    case THB_BF16: { using T = __nv_bfloat16; CALL; break; }       \
    default: return THB_ERR_UNSUPPORTED;                           \
    }
#define DISPATCH_ANY_DTYPE(dtype, CALL)                            \
    switch (dtype) {                                               \
    case THB_F32: { using T = float; CALL; break; }                \
    case THB_F16: { using T = __half; CALL; break; }               \
    case THB_BF16: { using T = __nv_bfloat16; CALL; break; }       \
    case THB_U8: { using T = uint8_t; CALL; break; }               \
    default: return THB_ERR_UNSUPPORTED;                           \
    }

// ---- preprocess: NCHW fp32 -> normalised NHWC T ---------------------------------------------------
template <typename T>
__global__ void preprocess_kernel(const float *x, float *x_inplace, int N, int C, long HW, float3 mean, float3 std_,
                                  T *y, int y_ld, float q_min, float q_mult)
{
    constexpr int VN = Vec<T>::N;
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= (long)N * HW) return;
    const long n = pix / HW, hw = pix - n * HW;
    const float m[3] = {mean.x, mean.y, mean.z}, sd[3] = {std_.x, std_.y, std_.z};
    const float zr = roundf(q_min * q_mult);
    // every stored channel of the pixel is written (y_ld may exceed the rounded channel count: zeros there)
    for (int c0 = 0; c0 < y_ld; c0 += VN) {
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; i++) {
            const int c = c0 + i;
            float val = 0.f;
            if (c < C) {
                const long idx = (n * C + c) * HW + hw;
                val = x[idx];
                if (c < 3) val = __fdiv_rn(__fsub_rn(val, m[c]), sd[c]);
                if (x_inplace) x_inplace[idx] = val;
                if (sizeof(T) == 1) val = (float)(((int)(roundf(val * q_mult) - zr)) & 255);
            }
            v[i] = val;
        }
        Vec<T>::store(y + pix * y_ld + c0, v);
    }
}

// Space-to-depth variant for a stride-2 first convolution on very few channels: the 2x2 pixel block
// (ph, pw) of channel c becomes channel (ph*2 + pw)*C + c of a half-resolution tensor, so the convolution
// turns into a stride-1 one over 4*C channels whose gathered 16-byte chunks are fully used.
// Rows may be stored row_pitch pixels apart with pad_left zero pixels in front (and zeros behind): every pixel of such
// a row is written here, the padding as zeros.
template <typename T>
__global__ void preprocess_s2d_kernel(const float *x, float *x_inplace, int N, int C, int H, int W, float3 mean,
                                      float3 std_, T *y, int y_ld, int row_pitch, int pad_left, float q_min, float q_mult)
{
    const float zr = roundf(q_min * q_mult);  // uint8 only: the quantisation of preprocess_kernel
    constexpr int VN = Vec<T>::N;
    const int H2 = H / 2, W2 = W / 2;
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;  // over the stored (padded) pixels
    if (pix >= (long)N * H2 * row_pitch) return;
    const long n = pix / ((long)H2 * row_pitch);
    const int rem = (int)(pix - n * (long)H2 * row_pitch), bh = rem / row_pitch, bw = rem - bh * row_pitch - pad_left;
    const bool real = bw >= 0 && bw < W2;
    const float m[3] = {mean.x, mean.y, mean.z}, sd[3] = {std_.x, std_.y, std_.z};
    const int Cs = 4 * C, Cpad = (Cs + VN - 1) / VN * VN;
    // Three planes (every benchmark network): the block's 2 x 2 pixels of every plane as two 8-byte loads per plane (W is
    // even, so a pixel pair never straddles a row and is 8-byte aligned), all issued before any is used, every index
    // known at compile time.  Other plane counts take the element-wise loop below.
    if (C != 3) {
        for (int c0 = 0; c0 < Cpad; c0 += VN) {
            float v[VN];
#pragma unroll
            for (int i = 0; i < VN; i++) {
                const int cs = c0 + i;
                float val = 0.f;
                if (real && cs < Cs) {
                    const int blk = cs / C, c = cs - blk * C;
                    const long idx = ((n * C + c) * H + (2 * bh + (blk >> 1))) * W + 2 * bw + (blk & 1);
                    val = x[idx];
                    if (c < 3) val = __fdiv_rn(__fsub_rn(val, m[c]), sd[c]);
                    if (x_inplace) x_inplace[idx] = val;
                    if (sizeof(T) == 1) val = (float)(((int)(roundf(val * q_mult) - zr)) & 255);
                }
                v[i] = val;
            }
            Vec<T>::store(y + pix * y_ld + c0, v);
        }
        return;
    }
    float vals[16];
#pragma unroll
    for (int i = 0; i < 16; i++) vals[i] = 0.f;
    if (real) {
#pragma unroll
        for (int c = 0; c < 3; c++) {
#pragma unroll
            for (int ph = 0; ph < 2; ph++) {
                const long idx = ((n * C + c) * H + (2 * bh + ph)) * W + 2 * bw;
                float2 v = *reinterpret_cast<const float2 *>(x + idx);
                if (c < 3) {
                    v.x = __fdiv_rn(__fsub_rn(v.x, m[c]), sd[c]);
                    v.y = __fdiv_rn(__fsub_rn(v.y, m[c]), sd[c]);
                }
                if (x_inplace) *reinterpret_cast<float2 *>(x_inplace + idx) = v;
                if (sizeof(T) == 1) {
                    v.x = (float)(((int)(roundf(v.x * q_mult) - zr)) & 255);
                    v.y = (float)(((int)(roundf(v.y * q_mult) - zr)) & 255);
                }
                // channel (ph*2 + pw)*3 + c of the regrouped pixel
                vals[(ph * 2) * 3 + c] = v.x;
                vals[(ph * 2 + 1) * 3 + c] = v.y;
            }
        }
    }
#pragma unroll
    for (int c0 = 0; c0 < 16; c0 += VN) {
        if (c0 >= Cpad) break;   // (12 channels rounded up to the type's 16-byte group: 12 for fp32, 16 otherwise)
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; i++) v[i] = vals[c0 + i];
        Vec<T>::store(y + pix * y_ld + c0, v);
    }
}

// uint8 engine, 3x3 / stride 1 / pad 1 first convolution on a three-plane float batch: every pixel's 27 neighbours,
// normalised and quantised as preprocess_kernel does, become the channels of that pixel of an [N][H][W][32] byte tensor
// (channel (r*3 + s)*3 + c = plane c of pixel (h - 1 + r, w - 1 + s)); neighbours outside the image hold the byte that 0.0
// quantises to -- with the input zero point b_offset = roundf(q_min * q_mult) of the convolution (lowp_basic.c:15-29) such a
// byte plus b_offset is exactly 0, so the tap contributes nothing, as in the reference, which never visits it.  The layer
// is then a 1x1 convolution over 27 channels.  The in-place side effect writes each pixel once, as the centre tap.
__global__ void preprocess_neigh_u8_kernel(const float *x, float *x_inplace, int N, int H, int W, float3 mean, float3 std_,
                                           uint8_t *y, int y_ld, float q_min, float q_mult)
{
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long HW = (long)H * W;
    if (pix >= (long)N * HW) return;
    const long n = pix / HW;
    const int hw = (int)(pix - n * HW), h = hw / W, w = hw - h * W;
    const float m[3] = {mean.x, mean.y, mean.z}, sd[3] = {std_.x, std_.y, std_.z};
    const float zr = roundf(q_min * q_mult);
    const uint32_t zp = (uint32_t)(-(int)zr) & 255u;
    uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int r = 0; r < 3; r++)
#pragma unroll
        for (int q = 0; q < 3; q++) {
            const int ih = h - 1 + r, iw = w - 1 + q;
            const bool inside = (unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W;
#pragma unroll
            for (int c = 0; c < 3; c++) {
                const int k = (r * 3 + q) * 3 + c;
                uint32_t byte = zp;
                if (inside) {
                    const long idx = (n * 3 + c) * HW + (long)ih * W + iw;
                    float val = __fdiv_rn(__fsub_rn(x[idx], m[c]), sd[c]);
                    if (x_inplace && r == 1 && q == 1) x_inplace[idx] = val;
                    byte = (uint32_t)(((int)(roundf(val * q_mult) - zr)) & 255);
                }
                words[k >> 2] |= byte << (8 * (k & 3));
            }
        }
    uint4 *dst = reinterpret_cast<uint4 *>(y + pix * y_ld);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
    for (int c0 = 32; c0 < y_ld; c0 += 16) *reinterpret_cast<uint4 *>(y + pix * y_ld + c0) = make_uint4(0, 0, 0, 0);
}

// u8 HWC images -> normalised NHWC T (thapi.c:20-46: multiply by 0.003921568f and by 1/std)
template <typename T>
__global__ void preprocess_images_kernel(const uint8_t *img, int N, int H, int W, int stride, int cp, int bgr, float3 mean,
                                         float3 istd, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= (long)N * H * W) return;
    const long n = pix / ((long)H * W);
    const int hw = (int)(pix - n * (long)H * W), h = hw / W, w = hw - h * W;
    const uint8_t *src = img + ((size_t)n * H + h) * stride + (size_t)w * cp;
    const float m[3] = {mean.x, mean.y, mean.z}, is[3] = {istd.x, istd.y, istd.z};
    float v[VN];
#pragma unroll
    for (int i = 0; i < VN; i++) {
        float val = 0.f;
        if (i < cp) {
            const int sc = bgr ? cp - 1 - i : i;
            val = __fmul_rn(__fsub_rn(__fmul_rn((float)src[sc], 0.003921568f), m[i]), is[i]);
        }
        v[i] = val;
    }
    Vec<T>::store(y + pix * y_ld, v);
    // (a pixel stored with more channels than one group: zeros behind)
#pragma unroll
    for (int i = 0; i < VN; i++) v[i] = 0.f;
    for (int c0 = VN; c0 < y_ld; c0 += VN) Vec<T>::store(y + pix * y_ld + c0, v);
}

// u8 HWC RGB images -> normalised space-to-depth NHWC T: the layout preprocess_s2d_kernel writes (channel (ph*2 + pw)*3 + c
// of block (bh, bw) = pixel (2bh + ph, 2bw + pw), rows row_pitch pixels apart with pad_left zero pixels in front), with the
// arithmetic of the image loader (thapi.c:20-46)
template <typename T>
__global__ void preprocess_images_s2d_kernel(const uint8_t *img, int N, int H, int W, int stride, int bgr, float3 mean, float3 istd,
                                             T *y, int y_ld, int row_pitch, int pad_left)
{
    constexpr int VN = Vec<T>::N;
    const int H2 = H / 2, W2 = W / 2;
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;  // over the stored (padded) pixels
    if (pix >= (long)N * H2 * row_pitch) return;
    const long n = pix / ((long)H2 * row_pitch);
    const int rem = (int)(pix - n * (long)H2 * row_pitch), bh = rem / row_pitch, bw = rem - bh * row_pitch - pad_left;
    const bool real = bw >= 0 && bw < W2;
    const float m[3] = {mean.x, mean.y, mean.z}, is[3] = {istd.x, istd.y, istd.z};
    constexpr int Cs = 12, Cpad = (Cs + VN - 1) / VN * VN;
    for (int c0 = 0; c0 < Cpad; c0 += VN) {
        float v[VN];
#pragma unroll
        for (int i = 0; i < VN; i++) {
            const int cs = c0 + i;
            float val = 0.f;
            if (real && cs < Cs) {
                const int blk = cs / 3, c = cs - blk * 3;
                const uint8_t *src = img + ((size_t)n * H + 2 * bh + (blk >> 1)) * stride + (size_t)(2 * bw + (blk & 1)) * 3;
                val = __fmul_rn(__fsub_rn(__fmul_rn((float)src[bgr ? 2 - c : c], 0.003921568f), m[c]), is[c]);
            }
            v[i] = val;
        }
        Vec<T>::store(y + pix * y_ld + c0, v);
    }
}

// One YUYV frame (Y0 U Y1 V per pixel pair) -> normalised NHWC T with three channels, the arithmetic of the reference's
// table-driven converter (thapi.c:48-117): Y' = (Y-16)*298/256, R = sat(Y' + 459*(V-128)/256),
// G = sat(Y' - 137*(U-128)/256 - 55*(V-128)/256), B = sat(Y' + 541*(U-128)/256), every quotient truncated towards zero
// as C integer division does, then (byte * 0.003921568f - mean) * (1/std).  One thread per pixel pair.
template <typename T>
__global__ void preprocess_yuyv_kernel(const uint8_t *frame, int H, int W, float3 mean, float3 istd, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const long pair = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int W2 = W / 2;
    if (pair >= (long)H * W2) return;
    const uchar4 q = *reinterpret_cast<const uchar4 *>(frame + pair * 4);  // Y0 U Y1 V
    const int u = (int)q.y - 128, v = (int)q.w - 128;
    const int yur = 459 * v / 256, yub = 541 * u / 256, yg = -137 * u / 256 + -55 * v / 256;
    const int ys[2] = {((int)q.x - 16) * 298 / 256, ((int)q.z - 16) * 298 / 256};
    const float m[3] = {mean.x, mean.y, mean.z}, is[3] = {istd.x, istd.y, istd.z};
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const int rgb[3] = {min(255, max(0, ys[k] + yur)), min(255, max(0, ys[k] + yg)), min(255, max(0, ys[k] + yub))};
        float out[VN > 4 ? VN : 4];
#pragma unroll
        for (int c = 0; c < (VN > 4 ? VN : 4); c++)
            out[c] = c < 3 ? __fmul_rn(__fsub_rn(__fmul_rn((float)rgb[c], 0.003921568f), m[c]), is[c]) : 0.f;
        // (the row of W pixels is contiguous: pixel index = 2 * pair + k)
        float vv[VN];
#pragma unroll
        for (int c = 0; c < VN; c++) vv[c] = out[c];
        Vec<T>::store(y + (pair * 2 + k) * y_ld, vv);
#pragma unroll
        for (int c = 0; c < VN; c++) vv[c] = 0.f;
        for (int c0 = VN; c0 < y_ld; c0 += VN) Vec<T>::store(y + (pair * 2 + k) * y_ld + c0, vv);
    }
}

// u8 HWC images -> quantised NHWC u8 with the static input range of the lowp image loader
// (lowp/lowp_basic.c:82-131, lowp/lowp_images.c): q = (unsigned char)(int)roundf((px - sub[c]) * mult[c])
__global__ void preprocess_images_u8_kernel(const uint8_t *img, int N, int H, int W, int stride, int bgr, int3 sub, float3 mult,
                                            uint8_t *y, int y_ld)
{
    const long pix = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= (long)N * H * W) return;
    const long n = pix / ((long)H * W);
    const int hw = (int)(pix - n * (long)H * W), h = hw / W, w = hw - h * W;
    const uint8_t *src = img + ((size_t)n * H + h) * stride + (size_t)w * 3;
    const int sb[3] = {sub.x, sub.y, sub.z};
    const float ml[3] = {mult.x, mult.y, mult.z};
    uint32_t word = 0;
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const int sc = bgr ? 2 - c : c;
        const int q = (int)roundf(__fmul_rn((float)((int)src[sc] - sb[c]), ml[c]));
        word |= (uint32_t)(q & 0xff) << (8 * c);
    }
    *reinterpret_cast<uint4 *>(y + pix * y_ld) = make_uint4(word, 0, 0, 0);
}

// Range of the normalised input (lowp_basic.c:15-29 starts both ends at 0).  A block scans a piece of one (image, channel)
// plane for its raw extremes with 16-byte loads and normalises only those two: subtraction and division by a positive
// deviation are monotone, so the extremes of the normalised values are the normalised extremes, bit for bit.
__global__ void __launch_bounds__(256) minmax_kernel(const float *x, int C, long HW, int pieces, float3 mean, float3 std_, float *minmax)
{
    const long plane = blockIdx.x / pieces;
    const int piece = blockIdx.x % pieces, c = (int)(plane % C);
    const long per = (HW + pieces - 1) / pieces, i0 = piece * per, i1 = min(HW, i0 + per);
    const float *p = x + plane * HW;
    float mn = INFINITY, mx = -INFINITY;
    if (((HW | per) & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        for (long i = i0 + threadIdx.x * 4; i < i1; i += 1024) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(p + i));
            mn = fminf(fminf(mn, fminf(v.x, v.y)), fminf(v.z, v.w));
            mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        }
    } else {
        for (long i = i0 + threadIdx.x; i < i1; i += 256) {
            const float v = p[i];
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0 && mn <= mx) {
        if (c < 3) {
            const float m = c == 0 ? mean.x : c == 1 ? mean.y : mean.z, sd = c == 0 ? std_.x : c == 1 ? std_.y : std_.z;
            const float a = __fdiv_rn(__fsub_rn(mn, m), sd), b = __fdiv_rn(__fsub_rn(mx, m), sd);
            mn = fminf(a, b);
            mx = fmaxf(a, b);
        }
        // mn <= 0 <= mx is all that matters: negative floats order like their unsigned bit patterns, non-negative like signed ints
        if (mn < 0.f) atomicMax(reinterpret_cast<unsigned int *>(minmax), __float_as_uint(mn));
        if (mx > 0.f) atomicMax(reinterpret_cast<int *>(minmax + 1), __float_as_int(mx));
    }
}

// ---- NHWC Tin -> NCHW Tout through a 32x32 shared-memory transpose ---------------------------------
template <typename Tin, typename Tout>
__global__ void nhwc_to_nchw_kernel(const Tin *x, int HW, int C, int x_ld, float q_sub, float q_invmult, Tout *y)
{
    __shared__ float tile[32][33];
    const int n = blockIdx.z, hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int hw = hw0 + r, c = c0 + threadIdx.x;
        float v = 0.f;
        if (hw < HW && c < C) {
            v = dt<Tin>::ld(x + ((size_t)n * HW + hw) * x_ld + c);
            if (sizeof(Tin) == 1) v = __fadd_rn(__fmul_rn(v, q_invmult), q_sub);
        }
        tile[r][threadIdx.x] = v;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int c = c0 + r, hw = hw0 + threadIdx.x;
        if (hw < HW && c < C) {
            dt<Tout>::st(y + ((size_t)n * C + c) * HW + hw, tile[threadIdx.x][r]);
        }
    }
}

// ---- pooling ------------------------------------------------------------------------------------------
template <typename T, bool IS_MAX>
__global__ void pool_kernel(const T *x, int N, int H, int W, int C, int x_ld, int kH, int kW, int dH, int dW, int padH,
                            int padW, int oH, int oW, int count_include_pad, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const int cvecs = (C + VN - 1) / VN;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)N * oH * oW * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long opix = idx / cvecs;
    const int ow = (int)(opix % oW), oh = (int)((opix / oW) % oH);
    const long n = opix / ((long)oW * oH);
    int hs = oh * dH - padH, ws = ow * dW - padW;
    float acc[VN];
    int he, we, div = 1;
    if (IS_MAX) {
        he = min(hs + kH, H); we = min(ws + kW, W);
        hs = max(hs, 0); ws = max(ws, 0);
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] = sizeof(T) == 1 ? 0.f : -FLT_MAX;
    } else {
        he = min(hs + kH, H + padH); we = min(ws + kW, W + padW);
        const int pool = (he - hs) * (we - ws);
        hs = max(hs, 0); ws = max(ws, 0);
        he = min(he, H); we = min(we, W);
        div = count_include_pad ? pool : (he - hs) * (we - ws);
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] = 0.f;
    }
    for (int h = hs; h < he; h++)
#pragma unroll 4
        for (int w = ws; w < we; w++) {  // (unrolled: four independent loads in flight; a 7x7 global pool is latency-bound)
            float v[VN];
            Vec<T>::load(x + ((size_t)(n * H + h) * W + w) * x_ld + cv * VN, v);
#pragma unroll
            for (int i = 0; i < VN; i++) {
                if (IS_MAX) acc[i] = v[i] > acc[i] ? v[i] : acc[i];
                else acc[i] += v[i];
            }
        }
    if (!IS_MAX) {
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] = acc[i] / (float)div;
    }
    Vec<T>::store(y + (size_t)opix * y_ld + cv * VN, acc);
}

// Global average pooling (the window is the whole map): the generic kernel would walk the map's pixels one after the
// other in each thread, a chain of dependent load latencies.  Here a block owns one image and 32 channel vectors; its
// eight warps take every eighth pixel (independent loads in flight) and their partial sums meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) global_avgpool_kernel(const T *x, int HW, int C, int x_ld, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    __shared__ float part[8][32][VN + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cvecs = (C + VN - 1) / VN, cv = blockIdx.y * 32 + lane;
    const long n = blockIdx.x;
    float acc[VN];
#pragma unroll
    for (int i = 0; i < VN; i++) acc[i] = 0.f;
    if (cv < cvecs)
        for (int p = warp; p < HW; p += 8) {
            float v[VN];
            Vec<T>::load(x + ((size_t)n * HW + p) * x_ld + cv * VN, v);
#pragma unroll
            for (int i = 0; i < VN; i++) acc[i] += v[i];
        }
#pragma unroll
    for (int i = 0; i < VN; i++) part[warp][lane][i] = acc[i];
    __syncthreads();
    if (warp == 0 && cv < cvecs) {
        float out[VN];
#pragma unroll
        for (int i = 0; i < VN; i++) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) s += part[w][lane][i];
            out[i] = s / (float)HW;
        }
        Vec<T>::store(y + (size_t)n * y_ld + cv * VN, out);
    }
}

// 3x3 stride-2 max pooling of a 16-bit type, without a conversion and with each input row reduced once: a thread owns one
// output column of one 8-channel group and walks down a strip of output rows; of the three input rows of a window the
// first is the last one of the window above, so every step reads two new rows of three pixels, takes their
// horizontal maxima, and combines them with the carried one.  Neighbouring threads read neighbouring pixels, so the
// shared column of adjacent windows is served by L1.
template <typename T2> __device__ __forceinline__ uint4 max8(const uint4 &a, const uint4 &b)
{
    uint4 r;
    const T2 *pa = reinterpret_cast<const T2 *>(&a), *pb = reinterpret_cast<const T2 *>(&b);
    T2 *pr = reinterpret_cast<T2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; i++) pr[i] = __hmax2(pa[i], pb[i]);
    return r;
}
struct U8x4 {};  // sixteen uint8 channels per 16-byte vector, maxima by __vmaxu4
template <> __device__ __forceinline__ uint4 max8<U8x4>(const uint4 &a, const uint4 &b)
{
    return make_uint4(__vmaxu4(a.x, b.x), __vmaxu4(a.y, b.y), __vmaxu4(a.z, b.z), __vmaxu4(a.w, b.w));
}
template <typename T2>
__global__ void maxpool3s2_kernel(const uint4 *__restrict__ x, int N, int H, int W, int cvecs, int x_ld8, int padH, int padW,
                                  int oH, int oW, int strip, int nstrips, uint32_t neg_inf2, uint4 *__restrict__ y, int y_ld8)
{
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)N * nstrips * oW * cvecs) return;
    const int cv = (int)(idx % cvecs);
    long r = idx / cvecs;
    const int ow = (int)(r % oW);
    r /= oW;
    const int st = (int)(r % nstrips);
    const long n = r / nstrips;
    const uint4 ninf = make_uint4(neg_inf2, neg_inf2, neg_inf2, neg_inf2);
    const int iw0 = ow * 2 - padW;
    const uint4 *img = x + (size_t)n * H * W * x_ld8 + cv;
    auto hrow = [&](int ih) {
        uint4 m = ninf;
        if ((unsigned)ih < (unsigned)H) {
            const uint4 *row = img + (size_t)ih * W * x_ld8;
#pragma unroll
            for (int k = 0; k < 3; k++)
                if ((unsigned)(iw0 + k) < (unsigned)W) m = max8<T2>(m, __ldg(row + (size_t)(iw0 + k) * x_ld8));
        }
        return m;
    };
    const int oh0 = st * strip, oh1 = min(oH, oh0 + strip);
    uint4 carried = hrow(oh0 * 2 - padH);
    uint4 *out = y + ((size_t)n * oH * oW + ow) * y_ld8 + cv;
    for (int oh = oh0; oh < oh1; oh++) {
        const uint4 r1 = hrow(oh * 2 - padH + 1), r2 = hrow(oh * 2 - padH + 2);
        out[(size_t)oh * oW * y_ld8] = max8<T2>(max8<T2>(carried, r1), r2);
        carried = r2;
    }
}

// ---- y = act(x*scale[c] + shift[c]) ----------------------------------------------------------------------
template <typename T>
__global__ void affine_act_kernel(const T *x, long pixels, int C, int x_ld, const float *scale, const float *shift,
                                  thb_act act, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const int cvecs = (C + VN - 1) / VN;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pixels * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long pix = idx / cvecs;
    float v[VN];
    Vec<T>::load(x + pix * x_ld + cv * VN, v);
#pragma unroll
    for (int i = 0; i < VN; i++) {
        const int c = cv * VN + i;
        if (c < C) {
            float t = v[i];
            if (scale) t = t * scale[c] + (shift ? shift[c] : 0.f);
            else if (shift) t = t + shift[c];
            v[i] = thb_apply_act(t, act.kind, act.threshold, act.value, act.alpha,
                                 act.kind == THB_ACT_PRELU ? act.slope[c] : 0.f);
        } else v[i] = 0.f;
    }
    Vec<T>::store(y + pix * y_ld + cv * VN, v);
}

__global__ void u8_threshold_kernel(const uint8_t *x, long pixels, int C, int x_ld, int thr, int val, uint8_t *y, int y_ld)
{
    const int cvecs = (C + 15) / 16;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pixels * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long pix = idx / cvecs;
    uint4 t = *reinterpret_cast<const uint4 *>(x + pix * x_ld + cv * 16);
    uint8_t *b = reinterpret_cast<uint8_t *>(&t);
#pragma unroll
    for (int i = 0; i < 16; i++) b[i] = (cv * 16 + i < C) ? (b[i] > thr ? b[i] : (uint8_t)val) : 0;
    *reinterpret_cast<uint4 *>(y + pix * y_ld + cv * 16) = t;
}

// uint8 a*ca + b*cb with ca, cb in {+1, -1}, both inputs and the output on the same static quantisation
// (sub = -range/2, mult = 255/range, so sub*mult = -127.5): the byte a dequantise -> float combine -> requantise chain
// gives in exact arithmetic, floor(ca*qa + cb*qb - (ca + cb - 1)*127.5) saturated to [0, 255] = `add2`/2 folded into an
// integer addend; an optional Threshold (bytes thr, val; thr < 0: none) follows.  No counterpart in the reference, whose
// lowp engine has no CAddTable.
__global__ void u8_combine_kernel(const uint8_t *a, int a_ld, const uint8_t *b, int b_ld, int ca, int cb, int addend,
                                  int thr, int val, long pixels, int C, uint8_t *y, int y_ld)
{
    const int cvecs = (C + 15) / 16;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pixels * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long pix = idx / cvecs;
    uint4 ta = __ldg(reinterpret_cast<const uint4 *>(a + pix * a_ld + cv * 16));
    uint4 tb = __ldg(reinterpret_cast<const uint4 *>(b + pix * b_ld + cv * 16));
    const uint8_t *pa = reinterpret_cast<const uint8_t *>(&ta), *pb = reinterpret_cast<const uint8_t *>(&tb);
    uint4 t;
    uint8_t *o = reinterpret_cast<uint8_t *>(&t);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int v = ca * (int)pa[i] + cb * (int)pb[i] + addend;
        v = min(255, max(0, v));
        if (thr >= 0) v = v > thr ? v : val;
        o[i] = (cv * 16 + i < C) ? (uint8_t)v : 0;
    }
    *reinterpret_cast<uint4 *>(y + pix * y_ld + cv * 16) = t;
}

struct CombineArgs {
    const void *x[8];
    int ld[8];
    float coef[8];
    int nin;
};
template <typename T>
__global__ void combine_kernel(CombineArgs a, long pixels, int C, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const int cvecs = (C + VN - 1) / VN;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pixels * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long pix = idx / cvecs;
    float acc[VN], v[VN];
    Vec<T>::load(reinterpret_cast<const T *>(a.x[0]) + pix * a.ld[0] + cv * VN, v);
#pragma unroll
    for (int i = 0; i < VN; i++) acc[i] = a.coef[0] * v[i];
    for (int k = 1; k < a.nin; k++) {
        Vec<T>::load(reinterpret_cast<const T *>(a.x[k]) + pix * a.ld[k] + cv * VN, v);
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] = fmaf(a.coef[k], v[i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < VN; i++)
        if (cv * VN + i >= C) acc[i] = 0.f;
    Vec<T>::store(y + pix * y_ld + cv * VN, acc);
}

template <typename T>
__global__ void copy_channels_kernel(const T *x, long pixels, int cvecs, int x_ld, T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= pixels * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long pix = idx / cvecs;
    *reinterpret_cast<uint4 *>(y + pix * y_ld + cv * VN) = *reinterpret_cast<const uint4 *>(x + pix * x_ld + cv * VN);
}

// ---- softmax over channels, one warp per pixel; exp(-d) = 1/(poly(d))^8 in double, 0 from 13 up ------------
__device__ __forceinline__ float exp_minus_approx(float d)
{
    const double x = (double)d;
    if (x < 13.0) {
        double y = 1.0 + x * (0.125 + x * (0.0078125 + x * (0.00032552083 + x * 1.0172526e-5)));
        y *= y; y *= y; y *= y;
        return (float)(1 / y);
    }
    return 0.f;
}
template <typename T>
__global__ void softmax_kernel(const T *x, long pixels, int C, int x_ld, T *y, int y_ld)
{
    const long pix = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (pix >= pixels) return;
    const T *xp = x + pix * x_ld;
    T *yp = y + pix * y_ld;
    float mx = -FLT_MAX;
    for (int c = lane; c < C; c += 32) mx = fmaxf(mx, dt<T>::ld(xp + c));
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int c = lane; c < C; c += 32) sum += exp_minus_approx(mx - dt<T>::ld(xp + c));
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1 / sum;
    for (int c = lane; c < C; c += 32) dt<T>::st(yp + c, exp_minus_approx(mx - dt<T>::ld(xp + c)) * inv);
}

// ---- col2im gather for the transposed convolution ---------------------------------------------------------
template <typename T>
__global__ void col2im_kernel(const T *cols, int N, int H, int W, int Cout, int kH, int kW, int dH, int dW, int padH,
                              int padW, int oH, int oW, int cols_ld, int Cp, float beta, const float *bias, thb_act act,
                              T *y, int y_ld)
{
    constexpr int VN = Vec<T>::N;
    const int cvecs = Cp / VN;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)N * oH * oW * cvecs) return;
    const int cv = (int)(idx % cvecs);
    const long opix = idx / cvecs;
    const int ow = (int)(opix % oW), oh = (int)((opix / oW) % oH);
    const long n = opix / ((long)oW * oH);
    float acc[VN];
#pragma unroll
    for (int i = 0; i < VN; i++) acc[i] = 0.f;
    for (int kh = 0; kh < kH; kh++) {
        const int hn = oh + padH - kh;
        if (hn < 0 || hn % dH) continue;
        const int h = hn / dH;
        if (h >= H) continue;
        for (int kw = 0; kw < kW; kw++) {
            const int wn = ow + padW - kw;
            if (wn < 0 || wn % dW) continue;
            const int w = wn / dW;
            if (w >= W) continue;
            float v[VN];
            Vec<T>::load(cols + ((size_t)(n * H + h) * W + w) * cols_ld + (size_t)(kh * kW + kw) * Cp + cv * VN, v);
#pragma unroll
            for (int i = 0; i < VN; i++) acc[i] += v[i];
        }
    }
#pragma unroll
    for (int i = 0; i < VN; i++) {
        const int c = cv * VN + i;
        if (c < Cout) {
            float t = acc[i];
            if (bias) t = beta * t + bias[c];
            acc[i] = thb_apply_act(t, act.kind, act.threshold, act.value, act.alpha,
                                   act.kind == THB_ACT_PRELU ? act.slope[c] : 0.f);
        } else acc[i] = 0.f;
    }
    Vec<T>::store(y + (size_t)opix * y_ld + cv * VN, acc);
}

// G lanes per pixel (a power of two up to 32): neighbouring lanes read neighbouring 16-byte chunks, so a warp's load covers
// whole pixels' contiguous bytes; bytes are summed four at a time (dp4a against ones) and the G partial sums by shuffles.
template <int G>
__global__ void u8_channel_sum_kernel(const uint8_t *x, long pixels, int C, int x_ld, int *csum)
{
    const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long pix = t / G;
    const int g = (int)(t % G);
    int s = 0;
    if (pix < pixels) {
        const uint8_t *p = x + pix * x_ld;
        for (int c0 = g * 16; c0 < C; c0 += G * 16) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p + c0));
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
            if (c0 + 16 > C) {
                // the last chunk: bytes beyond channel C do not count
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int nreal = C - c0 - 4 * i;
                    w[i] &= nreal >= 4 ? 0xffffffffu : nreal <= 0 ? 0u : (1u << (8 * nreal)) - 1u;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) s = (int)__dp4a(w[i], 0x01010101u, (uint32_t)s);
        }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (pix < pixels && g == 0) csum[pix] = s;
}

// the same with a whole block per pixel, for the few-pixel, many-channel inputs of Linear layers
__global__ void u8_channel_sum_wide_kernel(const uint8_t *x, int C, int x_ld, int *csum)
{
    const uint8_t *p = x + (size_t)blockIdx.x * x_ld;
    int s = 0;
    for (int c0 = threadIdx.x * 16; c0 < C; c0 += blockDim.x * 16) {
        const uint4 t = *reinterpret_cast<const uint4 *>(p + c0);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (c0 + i < C) s += (w[i >> 2] >> ((i & 3) * 8)) & 0xff;
    }
    __shared__ int part[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += part[i];
        csum[blockIdx.x] = tot;
    }
}

}  // namespace

// =================================================================================================
extern "C" {

int thb_channel_align(int dtype) { return dtype == THB_F32 ? 4 : dtype == THB_U8 ? 16 : 8; }

int thb_preprocess(const float *x, float *x_inplace, int N, int C, int H, int W, const float *mean3, const float *std3,
                   int dtype, void *y, int y_ld, float q_sub, float q_mult, thb_stream s)
{
    const long HW = (long)H * W, pix = (long)N * HW;
    if (pix == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]), sd = make_float3(std3[0], std3[1], std3[2]);
    DISPATCH_ANY_DTYPE(dtype, (preprocess_kernel<T><<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(
                                  x, x_inplace, N, C, HW, m, sd, (T *)y, y_ld, q_sub, q_mult)));
    return THB_LAUNCH_CHECK("preprocess_kernel");
}

int thb_preprocess_s2d_padded(const float *x, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                              const float *std3, int dtype, void *y, int y_ld, int row_pitch, int pad_left, thb_stream s)
{
    if (((H | W) & 1) || pad_left < 0 || row_pitch < pad_left + W / 2) return THB_ERR_ARG;
    const long pix = (long)N * (H / 2) * row_pitch;
    if (pix == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]), sd = make_float3(std3[0], std3[1], std3[2]);
    DISPATCH_FLOAT_DTYPE(dtype, (preprocess_s2d_kernel<T><<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(
                                    x, x_inplace, N, C, H, W, m, sd, (T *)y, y_ld, row_pitch, pad_left, 0.f, 0.f)));
    return THB_LAUNCH_CHECK("preprocess_s2d_kernel");
}

int thb_preprocess_s2d_u8(const float *x, float *x_inplace, int N, int C, int H, int W, const float *mean3, const float *std3,
                          void *y, int y_ld, float q_sub, float q_mult, thb_stream s)
{
    if ((H | W) & 1) return THB_ERR_ARG;
    const long pix = (long)N * (H / 2) * (W / 2);
    if (pix == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]), sd = make_float3(std3[0], std3[1], std3[2]);
    preprocess_s2d_kernel<uint8_t><<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(x, x_inplace, N, C, H, W, m, sd, (uint8_t *)y, y_ld,
                                                                              W / 2, 0, q_sub, q_mult);
    return THB_LAUNCH_CHECK("preprocess_s2d_kernel<u8>");
}

int thb_preprocess_neigh_u8(const float *x, float *x_inplace, int N, int H, int W, const float *mean3, const float *std3, void *y,
                            int y_ld, float q_sub, float q_mult, thb_stream s)
{
    if (y_ld < 32 || y_ld % 16) return THB_ERR_ARG;
    const long pix = (long)N * H * W;
    if (pix == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]), sd = make_float3(std3[0], std3[1], std3[2]);
    preprocess_neigh_u8_kernel<<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(x, x_inplace, N, H, W, m, sd, (uint8_t *)y, y_ld, q_sub, q_mult);
    return THB_LAUNCH_CHECK("preprocess_neigh_u8_kernel");
}

int thb_preprocess_s2d(const float *x, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                       const float *std3, int dtype, void *y, int y_ld, thb_stream s)
{
    return thb_preprocess_s2d_padded(x, x_inplace, N, C, H, W, mean3, std3, dtype, y, y_ld, W / 2, 0, s);
}

int thb_preprocess_images(const unsigned char *img, int N, int H, int W, int stride, int cp, int bgr, const float *mean3,
                          const float *std3, int dtype, void *y, int y_ld, thb_stream s)
{
    const long pix = (long)N * H * W;
    if (pix == 0) return THB_OK;
    if (cp != 1 && cp != 3) return THB_ERR_ARG;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]);
    float3 is = make_float3(1 / std3[0], 1 / std3[1], 1 / std3[2]);
    DISPATCH_FLOAT_DTYPE(dtype, (preprocess_images_kernel<T><<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(
                                    img, N, H, W, stride, cp, bgr, m, is, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("preprocess_images_kernel");
}

int thb_preprocess_yuyv(const unsigned char *frame, int H, int W, const float *mean3, const float *std3, int dtype, void *y,
                        int y_ld, thb_stream s)
{
    if (H < 1 || W < 2 || (W & 1) || y_ld < 3) return THB_ERR_ARG;
    if (dtype == THB_U8) return THB_ERR_UNSUPPORTED;  // (the reference refuses this entry point on its lowp engine)
    const long pairs = (long)H * (W / 2);
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]);
    float3 is = make_float3(1 / std3[0], 1 / std3[1], 1 / std3[2]);
    DISPATCH_FLOAT_DTYPE(dtype, (preprocess_yuyv_kernel<T><<<nblocks(pairs), 256, 0, (cudaStream_t)s>>>(frame, H, W, m, is, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("preprocess_yuyv_kernel");
}

int thb_preprocess_images_s2d(const unsigned char *img, int N, int H, int W, int stride, int bgr, const float *mean3, const float *std3,
                              int dtype, void *y, int y_ld, int row_pitch, int pad_left, thb_stream s)
{
    if (((H | W) & 1) || pad_left < 0 || row_pitch < pad_left + W / 2 || y_ld < 12) return THB_ERR_ARG;
    if (dtype != THB_F16 && dtype != THB_BF16) return THB_ERR_UNSUPPORTED;
    const long pix = (long)N * (H / 2) * row_pitch;
    if (pix == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]);
    float3 is = make_float3(1 / std3[0], 1 / std3[1], 1 / std3[2]);
    DISPATCH_FLOAT_DTYPE(dtype, (preprocess_images_s2d_kernel<T><<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(
                                    img, N, H, W, stride, bgr, m, is, (T *)y, y_ld, row_pitch, pad_left)));
    return THB_LAUNCH_CHECK("preprocess_images_s2d_kernel");
}

int thb_preprocess_images_lowp(const unsigned char *img, int N, int H, int W, int stride, int bgr, const float *mean3,
                               const float *std3, void *y, int y_ld, float *q_sub, float *q_mult, thb_stream s)
{
    if (y_ld % 16) return THB_ERR_ARG;
    // the loader's float expressions, in its order (lowp_basic.c:102-119)
    float mn = 1e30f, mx = -1e30f, m;
    for (int i = 0; i < 3; i++) {
        if (-mean3[i] / std3[i] < mn) mn = -mean3[i] / std3[i];
        if ((1 - mean3[i]) / std3[i] > mx) mx = (1 - mean3[i]) / std3[i];
    }
    m = (mx - mn) ? 255 / (mx - mn) : 0;
    int sub[3];
    float mul[3];
    for (int i = 0; i < 3; i++) {
        sub[i] = (int)roundf(255 * (mean3[i] + std3[i] * mn));
        mul[i] = m / (255 * std3[i]);
    }
    *q_sub = mn;
    *q_mult = m;
    const long pix = (long)N * H * W;
    if (pix == 0) return THB_OK;
    preprocess_images_u8_kernel<<<nblocks(pix), 256, 0, (cudaStream_t)s>>>(img, N, H, W, stride, bgr, make_int3(sub[0], sub[1], sub[2]),
                                                                            make_float3(mul[0], mul[1], mul[2]), (uint8_t *)y, y_ld);
    return THB_LAUNCH_CHECK("preprocess_images_u8_kernel");
}

int thb_minmax_normalized(const float *x, int N, int C, int H, int W, const float *mean3, const float *std3,
                          float *minmax2, thb_stream s)
{
    const long HW = (long)H * W, total = (long)N * C * HW;
    cudaError_t e = cudaMemsetAsync(minmax2, 0, 2 * sizeof(float), (cudaStream_t)s);
    if (e != cudaSuccess) return thb_note_launch(e, "minmax memset");
    if (total == 0) return THB_OK;
    float3 m = make_float3(mean3[0], mean3[1], mean3[2]), sd = make_float3(std3[0], std3[1], std3[2]);
    // pieces of a plane per block: enough blocks for a few waves, pieces a multiple of four elements long where possible
    const long planes = (long)N * C;
    int pieces = (int)((148L * 16 + planes - 1) / planes);
    if (pieces < 1) pieces = 1;
    while (pieces > 1 && ((HW + pieces - 1) / pieces < 4096 || (HW % (4L * pieces)))) pieces--;
    if (planes * pieces > 0x7fffffffL) return THB_ERR_UNSUPPORTED;
    minmax_kernel<<<(unsigned)(planes * pieces), 256, 0, (cudaStream_t)s>>>(x, C, HW, pieces, m, sd, minmax2);
    return THB_LAUNCH_CHECK("minmax_kernel");
}

int thb_postprocess(const void *x, int dtype, int N, int H, int W, int C, int x_ld, float q_sub, float q_invmult,
                    float *y, thb_stream s)
{
    const int HW = H * W;
    if ((long)N * HW * C == 0) return THB_OK;
    dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
    DISPATCH_ANY_DTYPE(dtype, (nhwc_to_nchw_kernel<T, float><<<grid, block, 0, (cudaStream_t)s>>>(
                                  (const T *)x, HW, C, x_ld, q_sub, q_invmult, y)));
    return THB_LAUNCH_CHECK("nhwc_to_nchw_kernel");
}

int thb_to_nchw(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, thb_stream s)
{
    const int HW = H * W;
    if ((long)N * HW * C == 0) return THB_OK;
    dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
    DISPATCH_ANY_DTYPE(dtype, (nhwc_to_nchw_kernel<T, T><<<grid, block, 0, (cudaStream_t)s>>>(
                                  (const T *)x, HW, C, x_ld, 0.f, 1.f, (T *)y)));
    return THB_LAUNCH_CHECK("nhwc_to_nchw_kernel");
}

int thb_maxpool(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int kH, int kW, int dH, int dW, int padH,
                int padW, int oH, int oW, void *y, int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    const long total = (long)N * oH * oW * ((C + al - 1) / al);
    if (total == 0) return THB_OK;
    if ((dtype == THB_F16 || dtype == THB_BF16) && kH == 3 && kW == 3 && dH == 2 && dW == 2 && x_ld % 8 == 0 && y_ld % 8 == 0) {
        const int cvecs = (C + 7) / 8;
        // strips of output rows: long enough to amortise the carried row, short enough for several waves of CTAs (measured:
        // strips of 4-7 rows are 7 % faster than 14 on the 112x112 ResNet stem output)
        int strip = oH;
        while (strip > 4 && (long)N * ((oH + strip - 1) / strip) * oW * cvecs < 24L * 148 * 256) strip = (strip + 1) / 2;
        const int nstrips = (oH + strip - 1) / strip;
        const long items = (long)N * nstrips * oW * cvecs;
        if (dtype == THB_F16)
            maxpool3s2_kernel<__half2><<<nblocks(items), 256, 0, (cudaStream_t)s>>>(
                (const uint4 *)x, N, H, W, cvecs, x_ld / 8, padH, padW, oH, oW, strip, nstrips, 0xFC00FC00u, (uint4 *)y, y_ld / 8);
        else
            maxpool3s2_kernel<__nv_bfloat162><<<nblocks(items), 256, 0, (cudaStream_t)s>>>(
                (const uint4 *)x, N, H, W, cvecs, x_ld / 8, padH, padW, oH, oW, strip, nstrips, 0xFF80FF80u, (uint4 *)y, y_ld / 8);
        return THB_LAUNCH_CHECK("maxpool3s2_kernel");
    }
    if (dtype == THB_U8 && kH == 3 && kW == 3 && dH == 2 && dW == 2 && x_ld % 16 == 0 && y_ld % 16 == 0) {
        // the same kernel on 16-channel vectors; the maximum starts from byte 0 as lowp_SpatialMaxPooling.c does
        const int cvecs = (C + 15) / 16;
        int strip = oH;
        while (strip > 4 && (long)N * ((oH + strip - 1) / strip) * oW * cvecs < 24L * 148 * 256) strip = (strip + 1) / 2;
        const int nstrips = (oH + strip - 1) / strip;
        const long items = (long)N * nstrips * oW * cvecs;
        maxpool3s2_kernel<U8x4><<<nblocks(items), 256, 0, (cudaStream_t)s>>>(
            (const uint4 *)x, N, H, W, cvecs, x_ld / 16, padH, padW, oH, oW, strip, nstrips, 0u, (uint4 *)y, y_ld / 16);
        return THB_LAUNCH_CHECK("maxpool3s2_kernel");
    }
    DISPATCH_ANY_DTYPE(dtype, (pool_kernel<T, true><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(
                                  (const T *)x, N, H, W, C, x_ld, kH, kW, dH, dW, padH, padW, oH, oW, 0, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("pool_kernel<max>");
}

int thb_avgpool(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int kH, int kW, int dH, int dW, int padH,
                int padW, int oH, int oW, int count_include_pad, void *y, int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    const long total = (long)N * oH * oW * ((C + al - 1) / al);
    if (total == 0) return THB_OK;
    if (kH == H && kW == W && padH == 0 && padW == 0 && oH == 1 && oW == 1 && x_ld % al == 0 && y_ld % al == 0) {
        const dim3 grid((unsigned)N, (unsigned)(((C + al - 1) / al + 31) / 32));
        DISPATCH_ANY_DTYPE(dtype, (global_avgpool_kernel<T><<<grid, 256, 0, (cudaStream_t)s>>>((const T *)x, H * W, C, x_ld, (T *)y, y_ld)));
        return THB_LAUNCH_CHECK("global_avgpool_kernel");
    }
    DISPATCH_ANY_DTYPE(dtype, (pool_kernel<T, false><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(
                                    (const T *)x, N, H, W, C, x_ld, kH, kW, dH, dW, padH, padW, oH, oW,
                                    count_include_pad, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("pool_kernel<avg>");
}

int thb_affine_act(int dtype, const void *x, long pixels, int C, int x_ld, const float *scale, const float *shift,
                   const thb_act *act, void *y, int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    const long total = pixels * ((C + al - 1) / al);
    if (total == 0) return THB_OK;
    thb_act a = {THB_ACT_NONE, 0, 0, 0, nullptr};
    if (act) a = *act;
    DISPATCH_FLOAT_DTYPE(dtype, (affine_act_kernel<T><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(
                                    (const T *)x, pixels, C, x_ld, scale, shift, a, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("affine_act_kernel");
}

int thb_u8_threshold(const void *x, long pixels, int C, int x_ld, int thr, int val, void *y, int y_ld, thb_stream s)
{
    const long total = pixels * ((C + 15) / 16);
    if (total == 0) return THB_OK;
    u8_threshold_kernel<<<nblocks(total), 256, 0, (cudaStream_t)s>>>((const uint8_t *)x, pixels, C, x_ld, thr, val,
                                                                     (uint8_t *)y, y_ld);
    return THB_LAUNCH_CHECK("u8_threshold_kernel");
}

int thb_u8_combine(const void *a, int a_ld, const void *b, int b_ld, int ca, int cb, int thr, int val, long pixels, int C,
                   void *y, int y_ld, thb_stream s)
{
    if ((ca != 1 && ca != -1) || (cb != 1 && cb != -1)) return THB_ERR_UNSUPPORTED;
    const long total = pixels * ((C + 15) / 16);
    if (total == 0) return THB_OK;
    /* floor(-(ca + cb - 1) * 127.5): +1+1 -> -128, +1-1 -> +127, -1-1 -> +382 */
    const int twice = -(ca + cb - 1) * 255;
    const int addend = twice >= 0 ? twice / 2 : -((-twice + 1) / 2);
    u8_combine_kernel<<<nblocks(total), 256, 0, (cudaStream_t)s>>>((const uint8_t *)a, a_ld, (const uint8_t *)b, b_ld, ca, cb,
                                                                   addend, thr, val, pixels, C, (uint8_t *)y, y_ld);
    return THB_LAUNCH_CHECK("u8_combine_kernel");
}

int thb_combine(int dtype, int nin, const void *const *x_host, const int *ld_host, const float *coef_host, long pixels,
                int C, void *y, int y_ld, thb_stream s)
{
    if (nin < 1 || nin > 8) return THB_ERR_UNSUPPORTED;
    CombineArgs a;
    a.nin = nin;
    for (int i = 0; i < nin; i++) {
        a.x[i] = x_host[i];
        a.ld[i] = ld_host[i];
        a.coef[i] = coef_host[i];
    }
    const int al = thb_channel_align(dtype);
    const long total = pixels * ((C + al - 1) / al);
    if (total == 0) return THB_OK;
    DISPATCH_FLOAT_DTYPE(dtype, (combine_kernel<T><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(a, pixels, C, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("combine_kernel");
}

int thb_copy_channels(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    const int cvecs = (C + al - 1) / al;
    const long total = pixels * cvecs;
    if (total == 0) return THB_OK;
    DISPATCH_ANY_DTYPE(dtype, (copy_channels_kernel<T><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(
                                  (const T *)x, pixels, cvecs, x_ld, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("copy_channels_kernel");
}

int thb_softmax(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, thb_stream s)
{
    if (pixels == 0) return THB_OK;
    DISPATCH_FLOAT_DTYPE(dtype, (softmax_kernel<T><<<nblocks(pixels * 32), 256, 0, (cudaStream_t)s>>>(
                                    (const T *)x, pixels, C, x_ld, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("softmax_kernel");
}

int thb_col2im(int dtype, const void *cols, int N, int H, int W, int Cout, int kH, int kW, int dH, int dW, int padH,
               int padW, int oH, int oW, int cols_ld, float beta, const float *bias, const thb_act *act, void *y,
               int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    const int Cp = (Cout + al - 1) / al * al;
    const long total = (long)N * oH * oW * (Cp / al);
    if (total == 0) return THB_OK;
    thb_act a = {THB_ACT_NONE, 0, 0, 0, nullptr};
    if (act) a = *act;
    DISPATCH_FLOAT_DTYPE(dtype, (col2im_kernel<T><<<nblocks(total), 256, 0, (cudaStream_t)s>>>(
                                    (const T *)cols, N, H, W, Cout, kH, kW, dH, dW, padH, padW, oH, oW, cols_ld, Cp, beta,
                                    bias, a, (T *)y, y_ld)));
    return THB_LAUNCH_CHECK("col2im_kernel");
}

int thb_u8_channel_sum(const void *x, long pixels, int C, int x_ld, int *csum, thb_stream s)
{
    if (pixels == 0) return THB_OK;
    if (C >= 2048 && pixels <= 65535) {
        u8_channel_sum_wide_kernel<<<(unsigned)pixels, 256, 0, (cudaStream_t)s>>>((const uint8_t *)x, C, x_ld, csum);
        return THB_LAUNCH_CHECK("u8_channel_sum_wide_kernel");
    }
    const int chunks = (C + 15) / 16;
#define CSUM_CASE(G)                                                                                                      \
    u8_channel_sum_kernel<G><<<nblocks(pixels * G), 256, 0, (cudaStream_t)s>>>((const uint8_t *)x, pixels, C, x_ld, csum)
    if (chunks <= 1) CSUM_CASE(1);
    else if (chunks <= 2) CSUM_CASE(2);
    else if (chunks <= 4) CSUM_CASE(4);
    else if (chunks <= 8) CSUM_CASE(8);
    else if (chunks <= 16) CSUM_CASE(16);
    else CSUM_CASE(32);
#undef CSUM_CASE
    return THB_LAUNCH_CHECK("u8_channel_sum_kernel");
}

}  // extern "C"
