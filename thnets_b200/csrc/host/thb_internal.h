/* Internal interfaces of the host library (not installed). */
#ifndef THB_INTERNAL_H
#define THB_INTERNAL_H
#include <stddef.h>
#include "thnets.h"
#include "thb200_kernels.h"

/* ---- Torch7 table access (t7_reader.c) ---- */
double thb_t7_number(struct table *t, const char *name);
int thb_t7_boolean(struct table *t, const char *name);
THFloatTensor *thb_t7_tensor(struct table *t, const char *name);
void *thb_t7_storage(struct table *t, const char *name, int *nelem);
struct nnmodule *thb_t7_nnmodule(struct table *t, const char *name);

/* ---- device-neutral model: a flat, topologically ordered operator list (model.c) ---- */
enum thb_op {
    OP_INPUT, OP_CONV, OP_DECONV, OP_LINEAR, OP_BN, OP_ACT, OP_MAXPOOL, OP_AVGPOOL, OP_COMBINE, OP_CONCAT,
    OP_SOFTMAX, OP_VIEW, OP_ALIAS, OP_SCALE,
    OP_UPSAMPLE,   /* Upsample.c: 2x nearest neighbour */
    OP_ZEROPAD,    /* SpatialZeroPadding.c: pad_l/r/t/b, negative values crop */
    OP_SLICE,      /* Slice.c: elements [from, to) along one dimension of the tensor as the reference ranks it */
    OP_CMAX,       /* Cmax.c: elementwise maximum of the inputs */
    OP_LOGSOFTMAX, /* LogSoftMax.c */
    OP_NORMALIZE,  /* Normalize.c: x / ||x||_2 per row of a 2-D tensor, over the whole tensor otherwise */
    OP_UNPOOL,     /* SpatialMaxUnpooling.c: in[0] pooled-size values, in[1] the input of the pooling it undoes */
    OP_RESHAPE     /* Reshape.c: a vector per image becomes a [C, H, W] map (one-dimensional targets are OP_VIEW) */
};
#define THB_MAXIN 16

typedef struct thb_node {
    int op;
    int nin, in[THB_MAXIN];
    /* conv / deconv / linear */
    int Cin, Cout, kH, kW, dH, dW, padH, padW, adjH, adjW;
    /* convolution attributes the reference parses and ignores (ending pads, dilation, auto_pad 1 upper / 2 lower, reflection) */
    int pad2H, pad2W, dlH, dlW, autopad, refl_pad;
    float *weight, *bias; /* owned copies; conv OIHW, deconv IOHW, linear [out][in]; bias may be NULL */
    /* batch norm: folded to per-channel scale / shift at load time */
    float *scale, *shift;
    int C;
    /* activation */
    int act_kind;
    float act_threshold, act_value, act_alpha;
    float *slope;
    int nslope; /* 0 = one shared slope */
    /* pooling */
    int ceil_mode, count_include_pad;
    /* combine: out = sum coef[i] * in[i], left to right */
    float coef[THB_MAXIN];
    /* concat */
    int dim;
    /* view */
    int numElements;
    /* scale (non-v2 Dropout): y = x * factor */
    float factor;
    /* zero padding / slice */
    int pad_l, pad_r, pad_t, pad_b;
    int slice_axis, slice_from, slice_to;
    /* reshape: the target [C, H, W] and the module's batchMode (-1 absent, 0 false, 1 true) */
    int reshape[3], batch_mode;
} thb_node;

typedef struct thb_model {
    int nnodes, cap;
    thb_node *nodes;
    int output;
    int refs;
} thb_model;

thb_model *thb_model_from_network(THNETWORK *net, char *err, size_t errlen);
thb_model *thb_model_from_module(struct module *m, char *err, size_t errlen);
void thb_model_release(thb_model *m);

/* ---- execution plan + runtime (plan.c) ---- */
typedef struct thb_engine thb_engine; /* a converted network's device state */

enum { THB_MODE_F32 = 0, THB_MODE_F16 = 1, THB_MODE_BF16 = 2, THB_MODE_U8 = 3 };

thb_engine *thb_engine_create(thb_model *model, int mode, float lowp_range, int ngpus);
void thb_engine_destroy(thb_engine *e);
/* Forward on a host batch.  input_rank 4: [N,C,H,W]; 3: [C,H,W] (N == 1).  Either `x` (fp32 NCHW, normalised in
 * place when inplace != 0) or `images` (u8 HWC) is given.  Returns element count, fills dims of the result. */
typedef struct thb_result {
    float *data; /* network-owned pinned host memory */
    long count;
    int ndim;
    long size[4];
} thb_result;
void thb_set_pipeline_chunks(int n);
int thb_engine_forward(thb_engine *e, float *x, unsigned char **images, int stride, int bgr, int cp, int N, int C,
                       int H, int W, int input_rank, const float *mean, const float *std, int inplace, thb_result *res);
float thb_engine_last_ms(thb_engine *e);
float thb_engine_time_forward(thb_engine *e, int iters);
int thb_engine_profile(thb_engine *e, int iters, int max_steps, int *kinds, float *ms, double *flops);
int thb_engine_profile_bytes(thb_engine *e, int max_steps, double *bytes);
void thb_slice_batch(int N, int G, int g, int *offset, int *count);
void thb_slice_sub_batches(int n, int S, int c, int *offset, int *count);
const char *thb_engine_error(void);
void thb_set_error(const char *fmt, ...);

unsigned short thb_float_to_half_bits(float v, int bf16); /* round to nearest even (conv_host.cu) */
void *thb_host_alloc_pinned(size_t bytes);
void thb_host_free_pinned(void *p);

/* ---- lowp host arithmetic (lowp_host.c): the reference's float expressions, evaluated on the host ---- */
void thb_lowp_quantize(const float *x, long n, unsigned char *q, float *sub, float *mult);
unsigned char thb_lowp_scale_float(float sub, float mult, float value);
void thb_lowp_gemm_params(float w_sub, float w_mult, float in_sub, float in_mult, float out_sub, float out_mult,
                          int *a_offset, int *b_offset, int *c_offset, int *c_mult, int *c_shift);
void thb_lowp_bias_addends(const unsigned char *qbias, int n, float b_sub, float b_mult, float out_mult, int *addend);

/* ---- single-module execution (api.c) ---- */
THFloatTensor *thb_module_updateOutput(struct module *m, THFloatTensor *in);
void thb_module_forget(struct module *m);

/* private tail of a THNETWORK allocated by this library */
typedef struct thb_netx {
    THNETWORK pub;
    unsigned magic;
    thb_engine *engine; /* NULL until converted / first forward */
    int mode;           /* THB_MODE_* requested for this network */
    float lowp_range;
    int owns_graph;     /* this handle owns pub.net / pub.pynet / objects */
} thb_netx;
#define THB_NETX_MAGIC 0xB2000001u

/* fills f->module from the operator name and the parameter list of a graph function (PyTorch-dump names) */
void thb_build_py_module(const char *fname, struct pyfunction *f);
/* ONNX file -> the same node tree (onnx_reader.c); NULL on failure with a message in err */
struct pyelement *loadonnx(const char *path, struct pyelement **allpynodes, char *err, size_t errlen);

#endif
