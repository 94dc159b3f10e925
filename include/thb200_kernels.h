/*
 * thb200_kernels.h -- thin C ABI of the sm_100a kernels behind the thnets forward pass.
 *
 * Plain pointers, sizes and POD descriptors only; no C++ or framework types cross
 * this boundary.  Every pointer is a DEVICE pointer unless its name ends in _host.
 * Every function returns 0 on success, a negative thb_status otherwise, and never
 * falls back to the CPU: an unsupported case is an error.
 *
 * Activation tensors are channels-innermost: element (n, h, w, c) of a tensor with
 * pixel stride `ld` lives at ((n*H + h)*W + w)*ld + c.  `ld` may exceed C (padding,
 * or a channel slice of a wider concatenation buffer).  ld and every channel offset
 * are multiples of thb_channel_align(dtype) so that 16-byte accesses stay aligned.
 *
 * Each entry point names the reference operator it replaces (file:line within the
 * reference project).
 *
 * Threading: the launch functions keep small host-side caches (TMA descriptors by buffer
 * and shape, per-device kernel attributes) without locks, as the reference's engines
 * keep their state: call them from one host thread at a time.  Everything they enqueue
 * goes to the stream they are given; nothing synchronises the device.
 */
#ifndef THB200_KERNELS_H
#define THB200_KERNELS_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef enum { THB_F32 = 0, THB_F16 = 1, THB_BF16 = 2, THB_U8 = 3 } thb_dtype;

typedef enum {
    THB_OK = 0,
    THB_ERR_UNSUPPORTED = -1, /* shape / dtype combination has no kernel */
    THB_ERR_CUDA = -2,        /* a CUDA runtime call failed; see thb_last_cuda_error() */
    THB_ERR_TIMEOUT = -3,     /* a bounded device-side wait ran out (kernel status word) */
    THB_ERR_ARG = -4
} thb_status;

typedef void *thb_stream; /* cudaStream_t */

/* fused activation, applied last.  Threshold.c:38-63, PReLU.c:32-92 */
typedef enum {
    THB_ACT_NONE = 0, THB_ACT_THRESHOLD = 1, THB_ACT_LEAKY = 2, THB_ACT_PRELU = 3,
    THB_ACT_SIGMOID = 4, /* 1/(1 + expf(-x)), modules/Sigmoid.c:24 */
    THB_ACT_TANH = 5     /* tanhf(x), modules/Tanh.c */
} thb_act_kind;
typedef struct thb_act {
    int kind;
    float threshold, value, alpha; /* x > threshold ? x : value   |   x >= 0 ? x : alpha*x */
    const float *slope;            /* THB_ACT_PRELU: one slope per output channel: x > 0 ? x : slope[c]*x */
} thb_act;

/* 128-byte opaque TMA descriptor (CUtensorMap) of a packed weight matrix */
typedef struct __attribute__((aligned(64))) thb_tmap { unsigned long long opaque[16]; } thb_tmap;

/* ------------------------------------------------------------------------------------------
 * Convolution: replaces nn_SpatialConvolutionMM_updateOutput (modules/SpatialConvolutionMM.c:126-225),
 * THFloatTensor_convmm / sgemmargs (thbasic.c:1073-1103, OpenBLAS-stripped/sgemm.c:953-1036) and, in
 * THB_U8, Lowp_SpatialConvolution_updateOutput + THLowpTensor_mm (lowp/lowp_SpatialConvolution.c:90-187,
 * lowp/lowp_basic.c:299-321).  Implicit GEMM, no im2col buffer.  A Linear layer is the H=W=kH=kW=1 case.
 *
 * Floating-point epilogue (F32/F16/BF16), per output channel c:
 *     y = act( self_coef * (acc*scale[c] + shift[c]) + res_coef * res )
 * which covers bias, folded SpatialBatchNormalization and a fused two-input CAddTable/CSubTable.
 *
 * uint8 epilogue: exact int32 accumulator of sum (W+a_offset)*(X+b_offset) over the in-image taps,
 * gemmlowp-style requantisation ((acc+c_offset)*c_mult + round) >> c_shift saturated to u8, the
 * reference's per-plane saturating bias add (tail positions >= tail_start wrap below zero instead of
 * clamping, lowp_SpatialConvolution.c:71-88), then the u8 threshold q > relu_thr ? q : relu_val.
 * ---------------------------------------------------------------------------------------- */
typedef struct thb_conv_desc {
    int dtype;
    int N, H, W, Cin, in_ld;
    int Cout, kH, kW, dH, dW, padH, padW, oH, oW, out_ld;
    /* fp epilogue */
    const float *scale, *shift; /* NULL: 1 / 0.  Device arrays of Cout floats ROUNDED UP TO A MULTIPLE OF 64 (the kernels read them
                                 * in 16-byte groups and per 64-column block; the values behind Cout are ignored); the same
                                 * holds for act.slope.  (wsat and bias_add are read with clamped indices: Cout entries.) */
    const void *res;            /* NULL: none; same dtype and spatial shape as the output */
    int res_ld;
    float self_coef, res_coef;
    thb_act act;
    /* u8 epilogue */
    int a_offset, b_offset, c_offset, c_mult, c_shift;
    const int *wsat;     /* [Cout][(kH+1)*(kW+1)] summed-area table over taps of per-tap weight channel sums */
    const int *bias_add; /* [Cout] addend of the saturating bias add */
    const int *csum;     /* [N*H*W] per input pixel: sum of its Cin bytes (thb_u8_channel_sum) */
    int tail_start;      /* oH*oW - (oH*oW % 8) */
    int relu_thr, relu_val; /* relu_thr < 0: no threshold */
    int *acc_out;        /* optional: raw corrected int32 accumulators [N*oH*oW][Cout] (tests) */
    /* packed weights */
    const void *w;        /* F32: [Ktot][Cout4] ; tensor-core dtypes: [Cout_pad][Ktot_pad], K = tap*Cin_pad + c */
    const int *kinfo;     /* tensor-core dtypes: one word per 16-byte K chunk (thb_conv_pack_*) */
    const thb_tmap *tmap; /* tensor-core dtypes: TMA descriptor of w (host pointer) */
    int Cin_pad, Ktot_pad, Cout_pad, BN;
    int *status;          /* device word: set non-zero when a bounded wait gave up */
    /* Rows stored with their horizontal zero padding (0, 0: plain [N][H][W][ld] input).  in_row_pitch > 0: row h of
     * image n starts at pixel (n*H + h)*in_row_pitch of x and holds in_pad_left zero pixels, the W real pixels, then
     * at least kW - 1 - padW zero pixels; in_pad_left must equal padW.  When a row's kW taps then fill exactly
     * 128 bytes (kW * Cin_pad elements) and dW is 1, the tensor-core path fetches all of them with one copy. */
    int in_row_pitch, in_pad_left;
    /* Second activation operand (NULL: none; fp16 / bf16 only).  A 1x1 stride-1 unpadded convolution whose Cin input
     * channels come from TWO tensors: the first cin1 from x, the remaining Cin - cin1 from x2, an [N][x2_H][x2_W][x2_ld]
     * tensor sampled with stride x2_d (x2_H, x2_W must give the same oH x oW).  With the weights of two 1x1
     * convolutions side by side along K this computes their sum in one accumulator: a bottleneck block's last
     * convolution and its projection shortcut, without writing either addend.  cin1 and Cin - cin1 are multiples of 64.
     * No counterpart in the reference, which runs the two convolutions and a CAddTable. */
    const void *x2;
    int x2_ld, x2_H, x2_W, x2_d, cin1;
    /* uint8, optional: the convolution also leaves, per output pixel, the sum of its Cout output bytes -- what
     * thb_u8_channel_sum would compute for the next convolution.  When one tile covers all output channels
     * (Cout_pad == BN) the sums are stored; otherwise each column tile ADDS its part, and the caller clears the buffer
     * before the launch. */
    int *csum_out;
    /* Optional host copies of scale / shift (NULL: none), Cout floats each.  The patch convolution (thb_conv_patch_fwd,
     * thb_conv_maxpool_fwd) hands the per-channel constants to its kernel as launch parameters: with the host copies it
     * takes them from here; without them it reads the device arrays back with a blocking copy at EVERY launch, which is
     * fine for a test and must not happen inside a stream capture. */
    const float *scale_host, *shift_host;
    /* Split K (F16 / BF16, optional; 0 or 1: none).  A convolution of few tiles leaves most SMs idle: with splits = S the K
     * blocks of every tile are shared by S CTAs, which store fp32 partial tiles to splitk_scratch ([S][N*oH*oW][Cout_pad]
     * floats, thb_conv_splitk_plan gives S and the size), and a second launch adds them in split order and runs the
     * epilogue.  The launcher falls back to one launch when the layer's operand layout has no split form. */
    int splits;
    float *splitk_scratch;
} thb_conv_desc;

int thb_channel_align(int dtype);               /* 4 (F32), 8 (F16/BF16), 16 (U8) */
int thb_conv_geometry(thb_conv_desc *d);        /* fills Cin_pad, Ktot_pad, Cout_pad, BN from the shape */
size_t thb_conv_weight_bytes(const thb_conv_desc *d);
size_t thb_conv_kinfo_words(const thb_conv_desc *d);
/* host-side packing of OIHW fp32 weights (or pre-quantised u8 weights) into the kernel layout */
int thb_conv_pack_weights_host(const thb_conv_desc *d, const float *w_oihw, const unsigned char *wq_oihw,
                               void *packed_host, int *kinfo_host, int *wsat_host);
int thb_conv_make_tmap(const thb_conv_desc *d, thb_tmap *out);
int thb_conv_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s);
/* the split count that suits a convolution's tile count (1: none) and the scratch bytes it needs; THB200_NO_SPLITK=1: always 1 */
int thb_conv_splitk_plan(const thb_conv_desc *d, size_t *scratch_bytes);

/* Convolution + epilogue as above (no residual) + max pooling with a pk x pk window (2 or 3), stride 2 and padding ppad
 * in ONE launch: the convolution's own output is never written, only the [N][pH][pW][y_ld] pooled tensor.  Replaces
 * nn_SpatialConvolutionMM_updateOutput followed by nn_SpatialMaxPooling_updateOutput (modules/SpatialMaxPooling.c:168-247:
 * windows clipped to the image, maximum from the smallest value).  F16 / BF16, Cout <= 64 with BN = 64, stride-1
 * convolution on 16 or 64 (padded) input channels with a kernel of at most 8 x 8.  pH, pW: the pooled size the caller
 * derived (every window must start inside the convolution output).
 * thb_conv_maxpool_supported answers whether a descriptor qualifies (THB200_NO_CONV_POOL=1 makes it answer 0). */
int thb_conv_maxpool_supported(const thb_conv_desc *d, int pk, int ps, int ppad);
int thb_conv_maxpool_fwd(const thb_conv_desc *d, int pk, int ps, int ppad, int pH, int pW, const void *x, void *y, int y_ld,
                         thb_stream s);

/* The patch kernel behind both: thb_conv_fwd itself takes this route for the same class of convolutions (kernel larger
 * than 1 x 1; a fused residual with self_coef = +-1 is allowed here, not with the pooling) -- the raw input patch of a
 * rectangle of outputs is loaded once and every tap reads it in place.  THB200_NO_PATCH=1 switches the route off. */
int thb_conv_patch_supported(const thb_conv_desc *d);
int thb_conv_patch_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s);

/* Batch-small Linear: y[n][m] = sum_k W[m][k]*x[n][k] (+ epilogue as above), N <= 8, weights read once.
 * Replaces nn_Linear_updateOutput's addmv path (modules/Linear.c:86-90, OpenBLAS-stripped/sgemv.c:48-105). */
int thb_gemv_fwd(int dtype, const void *x, int N, int K, int x_ld, const void *w /*[M][K]*/, int M,
                 const float *scale, const float *shift, const thb_act *act, void *y, int y_ld, thb_stream s);

/* ---- layout / precision boundary (thapi.c:363-450, :452-573; lowp/lowp_basic.c:5-58) ---- */
/* NCHW fp32 -> normalised NHWC dtype; also writes the normalised fp32 values back over `x` when inplace != 0 */
int thb_preprocess(const float *x_nchw, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                   const float *std3, int dtype, void *y, int y_ld, float q_sub, float q_mult, thb_stream s);
/* same normalisation, but space-to-depth: output is [N][H/2][W/2][4*C] with channel (ph*2 + pw)*C + c holding pixel
 * (2h + ph, 2w + pw) of channel c -- the input layout of a stride-2 first convolution rewritten as stride 1 */
int thb_preprocess_s2d(const float *x_nchw, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                       const float *std3, int dtype, void *y, int y_ld, thb_stream s);
/* the same into rows of row_pitch >= pad_left + W/2 pixels that start with pad_left zero pixels and end in zero
 * pixels (the layout thb_conv_desc.in_row_pitch describes); every pixel of y, padding included, is written */
int thb_preprocess_s2d_padded(const float *x_nchw, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                              const float *std3, int dtype, void *y, int y_ld, int row_pitch, int pad_left, thb_stream s);
/* the same for the uint8 engine: normalise, quantise with the batch's measured range exactly as thb_preprocess does
 * (lowp/lowp_basic.c:15-35), store space-to-depth.  Zero weights quantise to the weights' zero point, whose products
 * vanish exactly (lowp_basic.c:310-320: the offsets are the rounded zero points), so the rewritten stride-1 convolution
 * gives the accumulators of the stride-2 one bit for bit. */
/* uint8, a 3x3 / stride 1 / pad 1 first convolution on three planes: NCHW fp32 -> [N][H][W][y_ld >= 32] bytes whose channel
 * (r*3 + s)*3 + c is plane c of pixel (h - 1 + r, w - 1 + s), normalised and quantised like thb_preprocess does (the
 * byte of 0.0 outside the image): the convolution becomes a 1x1 one over 27 channels with weights in the same order.
 * No counterpart in the reference (nn_unfolded_copy, modules/SpatialConvolutionMM.c:11-60, unfolds floats for every layer). */
int thb_preprocess_neigh_u8(const float *x_nchw, float *x_inplace, int N, int H, int W, const float *mean3, const float *std3,
                            void *y, int y_ld, float q_sub, float q_mult, thb_stream s);
int thb_preprocess_s2d_u8(const float *x_nchw, float *x_inplace, int N, int C, int H, int W, const float *mean3,
                          const float *std3, void *y, int y_ld, float q_sub, float q_mult, thb_stream s);
/* 1 when the device and driver accept the single-copy row fetch described at thb_conv_desc.in_row_pitch */
int thb_conv_padded_rows_supported(int dtype);
/* u8 HWC images (already on the device, row stride `stride`) -> normalised NHWC dtype (thapi.c:20-46) */
int thb_preprocess_images(const unsigned char *img, int N, int H, int W, int stride, int cp, int bgr,
                          const float *mean3, const float *std3, int dtype, void *y, int y_ld, thb_stream s);
/* one YUYV frame (already on the device, 2 bytes per pixel, W even) -> normalised NHWC dtype with 3 channels: the
 * table-driven conversion of yuyv2fRGB (thapi.c:48-117) computed per pixel pair.  F32 / F16 / BF16; U8 is refused as the
 * reference refuses THProcessYUYV on its lowp engine (thapi.c:588-591). */
int thb_preprocess_yuyv(const unsigned char *frame, int H, int W, const float *mean3, const float *std3, int dtype, void *y,
                        int y_ld, thb_stream s);
/* u8 HWC RGB images -> normalised, space-to-depth NHWC dtype in the padded-row layout of thb_preprocess_s2d_padded
 * (F16 / BF16): THProcessImages feeding a stride-2 first convolution (thapi.c:20-46 arithmetic) */
int thb_preprocess_images_s2d(const unsigned char *img, int N, int H, int W, int stride, int bgr, const float *mean3,
                              const float *std3, int dtype, void *y, int y_ld, int row_pitch, int pad_left, thb_stream s);
/* u8 HWC RGB images -> quantised NHWC u8 with the static input range the lowp image loader derives from mean/std
 * (lowp/lowp_basic.c:82-131); returns that range as *q_sub, *q_mult (host) */
int thb_preprocess_images_lowp(const unsigned char *img, int N, int H, int W, int stride, int bgr, const float *mean3,
                               const float *std3, void *y, int y_ld, float *q_sub_host, float *q_mult_host, thb_stream s);
/* min and max (both seeded with 0) of the normalised input, for the dynamic input quantisation */
int thb_minmax_normalized(const float *x_nchw, int N, int C, int H, int W, const float *mean3,
                          const float *std3, float *minmax2, thb_stream s);
/* NHWC dtype -> NCHW fp32 (dequantising u8 with q*inv_mult + sub) */
int thb_postprocess(const void *x, int dtype, int N, int H, int W, int C, int x_ld, float q_sub, float q_invmult,
                    float *y_nchw, thb_stream s);

/* ---- pooling: SpatialMaxPooling.c:74-247, SpatialAveragePooling.c:71-207, lowp_SpatialMaxPooling.c ---- */
int thb_maxpool(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int kH, int kW, int dH, int dW,
                int padH, int padW, int oH, int oW, void *y, int y_ld, thb_stream s);
int thb_avgpool(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int kH, int kW, int dH, int dW,
                int padH, int padW, int oH, int oW, int count_include_pad, void *y, int y_ld, thb_stream s);

/* ---- elementwise: SpatialBatchNormalization.c:57-116 / Threshold.c / PReLU.c / Dropout.c as y = act(x*scale[c]+shift[c]) ---- */
int thb_affine_act(int dtype, const void *x, long pixels, int C, int x_ld, const float *scale, const float *shift,
                   const thb_act *act, void *y, int y_ld, thb_stream s);
/* u8 threshold: q > thr ? q : val (lowp/lowp_Threshold.c:3-28) */
int thb_u8_threshold(const void *x, long pixels, int C, int x_ld, int thr, int val, void *y, int y_ld, thb_stream s);
/* uint8 ca*a + cb*b (ca, cb = +1 or -1) of tensors on the static quantisation sub = -range/2, mult = 255/range, then an
 * optional Threshold (thr < 0: none): y = sat_u8(floor(ca*qa + cb*qb - (ca + cb - 1)*127.5)).  No counterpart in the
 * reference (its lowp engine converts no CAddTable, lowp/lowp_basic.c:150-208); an extension for residual networks. */
int thb_u8_combine(const void *a, int a_ld, const void *b, int b_ld, int ca, int cb, int thr, int val, long pixels, int C,
                   void *y, int y_ld, thb_stream s);
/* y = sum_i coef[i]*x[i], evaluated left to right (CAddTable.c:32-86) */
int thb_combine(int dtype, int nin, const void *const *x_host, const int *ld_host, const float *coef_host,
                long pixels, int C, void *y, int y_ld, thb_stream s);
/* copy a C-channel tensor into a channel slice of a wider buffer (JoinTable.c:34-86, Concat.c:21-76) */
int thb_copy_channels(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, thb_stream s);
/* softmax over channels per pixel with the reference's polynomial exp (SoftMax.c:24-90, thbasic.c:462-491) */
int thb_softmax(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, thb_stream s);
/* col2im gather of a transposed convolution's column matrix [N*H*W][Cout*kH*kW] (SpatialFullConvolution.c:99-127),
 * then y = act(beta*y + bias[c]) (:229-238: beta is 11 in the reference whenever a bias exists) */
int thb_col2im(int dtype, const void *cols, int N, int H, int W, int Cout, int kH, int kW, int dH, int dW, int padH,
               int padW, int oH, int oW, int cols_ld, float beta, const float *bias, const thb_act *act, void *y,
               int y_ld, thb_stream s);
/* ---- operators outside the benchmark networks (fp32 / fp16 / bf16) ---- */
/* 2x nearest-neighbour upsampling (modules/Upsample.c:18-63): y is [N][2H][2W][y_ld] */
int thb_upsample2x(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, int y_ld, thb_stream s);
/* zero padding by pad_l/r/t/b pixels, negative values crop (modules/SpatialZeroPadding.c:17-60, as intended: the
 * reference's own loop strides rows by the height and leaves the right padding unwritten): y is [N][H+pad_t+pad_b][W+pad_l+pad_r][y_ld] */
int thb_zero_pad(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int pad_l, int pad_r, int pad_t, int pad_b, void *y,
                 int y_ld, thb_stream s);
/* reflection padding (what an ONNX Pad node of mode "reflect" in front of a convolution asks for; the reference parses it
 * into SpatialConvolution.refl_pad and no engine of its own honours it: used only when THB200_HONOUR_PADS=1) */
int thb_reflect_pad(int dtype, const void *x, int N, int H, int W, int C, int x_ld, int pad_l, int pad_r, int pad_t, int pad_b, void *y,
                    int y_ld, thb_stream s);
/* channels [from, from + C) of every pixel of x -> y (modules/Slice.c:34-39 along the channel dimension, any `from`) */
int thb_slice_channels(int dtype, const void *x, long pixels, int from, int C, int x_ld, void *y, int y_ld, thb_stream s);
/* Reshape to three dimensions (modules/Reshape.c:22-36): row n of x (x_ld elements apart) holds C*H*W values in (channel,
 * row, column) order; they become the channels-innermost map y[n][h][w][c] (fp32, fp16, bf16; padded channels 0) */
int thb_from_nchw(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, int y_ld, thb_stream s);
/* elementwise maximum of up to 8 tensors of one shape (modules/Cmax.c:20-68) */
int thb_cmax(int dtype, int nin, const void *const *x_host, const int *ld_host, long pixels, int C, void *y, int y_ld, thb_stream s);
/* log-softmax over the channels of each pixel (modules/LogSoftMax.c:19-81).  first_frame_quirk = 1 reproduces the
 * reference's last loop, which subtracts each position's log-sum from the values at the START of the input (:77) */
int thb_logsoftmax(int dtype, const void *x, long pixels, int C, int x_ld, void *y, int y_ld, int first_frame_quirk, thb_stream s);
/* x / ||x||_2 over each of `rows` contiguous rows of row_len elements (per_row = 1: a 2-D tensor) or over all of them
 * together (modules/Normalize.c:12-44); scratch_rows: `rows` floats of device scratch; y may be x */
int thb_l2_normalize(int dtype, const void *x, long rows, long row_len, int per_row, float *scratch_rows, void *y, thb_stream s);
/* max unpooling (modules/SpatialMaxUnpooling.c:14-121): v holds one value per pooling window ([N][oH][oW][v_ld]), pool_in is
 * the tensor that pooling read ([N][H][W][x_ld]); y ([N][H][W][y_ld]) gets each value at the position of its window's
 * maximum (the index SpatialMaxPooling.c:95-112 records) and zero elsewhere; later windows win where windows overlap */
int thb_max_unpool(int dtype, const void *v, int v_ld, const void *pool_in, int x_ld, int N, int H, int W, int C, int kH, int kW, int dH,
                   int dW, int padH, int padW, int oH, int oW, void *y, int y_ld, thb_stream s);

/* per-pixel sum of the first C bytes (zero-point correction term of the u8 convolution) */
int thb_u8_channel_sum(const void *x, long pixels, int C, int x_ld, int *csum, thb_stream s);
/* channels-innermost -> plain NCHW flatten order of the same dtype (View feeding anything but a Linear) */
int thb_to_nchw(int dtype, const void *x, int N, int H, int W, int C, int x_ld, void *y, thb_stream s);

/* ---- no counterpart in the reference ----
 * thb_conv_fwd for THB_U8 that allocates nothing and needs no caller-provided d->csum: the per-pixel channel sums
 * go into a fixed array of THB_STATIC_CSUM_MAX_PIXELS int32 that is part of the library's device image
 * (d->csum is ignored).  N*H*W input pixels beyond that limit are refused with THB_ERR_ARG and a message in
 * thb_last_cuda_error().  The first call on each device looks the array's address up and caches it; make that call
 * before starting a stream capture.  All calls on a device share the array: nothing in it needs to start at zero
 * (each call rewrites the entries it reads, in stream order), but calls that may execute concurrently race on it. */
#define THB_STATIC_CSUM_MAX_PIXELS 1048576
int thb_conv_u8_fwd_static(const thb_conv_desc *d, const void *x, void *y, thb_stream s);

/* the launchers read their diagnostic THB200_* environment switches once; this re-reads them */
void thb_conv_reload_knobs(void);
const char *thb_last_cuda_error(void);
int thb_kernel_launch_count(void); /* launches issued through this ABI since load (bench bookkeeping) */
void thb_count_launches(int n);    /* add launches that were replayed from a captured graph of calls to this ABI */

#ifdef __cplusplus
}
#endif
#endif
