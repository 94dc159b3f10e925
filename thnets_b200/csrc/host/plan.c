/*
 * Execution planner and runtime of a converted network.
 *
 * The reference's engines swap one function pointer per module and allocate every activation on
 * every forward (cudnn/cudnn_basic.c:189-303, thapi.c:203-210, :405-416).  Here a network becomes,
 * once per input shape and per GPU, a list of kernel launches over two resident arenas:
 *   1. shape inference over the flat model (ranks and sizes as the reference's operators produce them);
 *   2. fusion: convolution/Linear + BatchNorm + two-input CAddTable + Threshold/PReLU collapse into one
 *      launch when each intermediate has a single consumer; BatchNorm + activation otherwise;
 *   3. liveness-based packing of all activations into one arena; weights packed and uploaded once;
 *   4. a batch is cut into contiguous slices, one per GPU; every GPU runs the whole list on its slice
 *      and the slices of the result are gathered by peer copies into GPU 0 (nothing is reduced).
 * Activations are channels-innermost ([N][H][W][ld]); the API's NCHW fp32 tensors are converted at the
 * two ends by the pre/postprocess kernels.
 */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include "thb_internal.h"

static char g_error[512];
const char *thb_engine_error(void) { return g_error; }
void thb_set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    if (th_debug) fprintf(stderr, "thb200: %s\n", g_error);
}
#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            thb_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return -1;                                                                             \
        }                                                                                          \
    } while (0)

void *thb_host_alloc_pinned(size_t bytes)
{
    void *p = 0;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable) != cudaSuccess) return 0;
    return p;
}
void thb_host_free_pinned(void *p)
{
    if (p) cudaFreeHost(p);
}

/* ------------------------------------------------------------------------------------------------ */
typedef struct {
    int N, C, H, W, rank;
    int flat, fC, fH, fW; /* flat: logical [N, C] view of a channels-innermost [N, fH, fW, fC] tensor */
} shape;

typedef struct {
    int buf;   /* activation buffer id, -1: not materialised */
    int ld;    /* pixel stride in elements */
    int coff;  /* channel offset inside the buffer */
    shape s;
    int csum_buf;        /* u8 mode: 1 + the buffer holding this tensor's per-pixel channel sums once a convolution asked for them; 0: none yet */
    float q_sub, q_mult; /* u8 mode */
    int q_dyn;           /* u8 mode: the scale is measured per forward (network input) */
    int row_pitch, pad_left; /* rows stored with horizontal zero padding (the staged network input only), else 0 */
} value;

typedef struct {
    size_t bytes, offset;
    int first, last;
} abuf;

enum step_kind {
    ST_CONV, ST_GEMV, ST_MAXPOOL, ST_AVGPOOL, ST_AFFINE, ST_U8THR, ST_U8COMBINE, ST_COMBINE, ST_COPY, ST_SOFTMAX, ST_COL2IM,
    ST_CSUM, ST_TO_NCHW, ST_ZERO, ST_UPSAMPLE, ST_ZEROPAD, ST_REFLECTPAD, ST_SLICEC, ST_CMAX, ST_LOGSOFTMAX, ST_NORMALIZE, ST_UNPOOL, ST_FROM_NCHW
};

typedef struct {
    int kind, dtype;
    int scratch_buf; /* fp32 partial tiles of a convolution whose K blocks are split over several CTAs (-1: none) */
    int nin, in_buf[8], in_ld[8], in_coff[8];
    int out_buf, out_ld, out_coff;
    int aux_buf; /* csum scratch (conv u8) */
    int aux2_buf; /* conv u8: channel sums of its OUTPUT, written by the convolution itself for the next one (-1: none) */
    float coef[8];
    int N, H, W, C, oH, oW, kH, kW, dH, dW, padH, padW, flag;
    long pixels;
    const float *scale, *shift, *bias;
    thb_act act;
    float beta;
    int thr, val;
    thb_conv_desc conv;
    thb_tmap *tmap;
    const void *w; /* gemv weights */
    int K, M;
    int dyn_quant; /* conv u8 whose input scale is only known per forward (first layer) */
    /* u8 conv constants needed to derive the per-forward parameters */
    float w_sub, w_mult, out_sub, out_mult;
    int flops_node; /* model node index of the conv (profiling) */
    int dual;       /* convolution with a second activation operand (in_buf[1]) instead of a residual */
    long out_pixels; int out_C; /* extent of the output tensor (th_minmax) */
    long in_off0, out_off0; /* element offsets added to the first input / the output (slices and joins along the batch dimension) */
    int pool_k, pool_pad, pool_oH, pool_oW; /* pool_k > 0: the max pooling that follows runs inside the convolution launch */
    double flops_extra; /* FLOPs of the second convolution computed by the same launch */
} step;

typedef struct instance {
    int device, slice_n, slice_off;
    cudaStream_t stream;
    cudaEvent_t ev0, ev1;
    cudaStream_t wb_stream; /* carries the copy of the normalised input back to the caller, beside the forward (made on first use) */
    cudaEvent_t ev_wb;
    int wb_pending;
    void **allocs;
    int nallocs, capallocs;
    void **hostmem; /* host arrays the launches' descriptors point to */
    int nhost, caphost;
    unsigned char *arena;
    size_t arena_bytes;
    float *d_in;          /* staged NCHW fp32 input */
    unsigned char *d_img; /* staged u8 HWC images */
    float *d_out;         /* NCHW fp32 result */
    float *d_minmax;
    float h_minmax[2];    /* host copy of the slice's input extremes (uint8 engine) */
    int *d_status;
    abuf *bufs;
    int nbufs;
    step *steps;
    int nsteps;
    value in_val, out_val;
    shape out_shape;
    long out_count;
    float last_ms;
    /* the planned launches as one CUDA graph: captured from the second forward on (the first runs them directly,
     * which also sets every kernel's attributes), replayed with a single launch afterwards */
    cudaGraphExec_t graph;
    int runs, graph_state; /* graph_state: 0 not tried, 1 usable, -1 capture failed or switched off */
    int graph_from;        /* first launch inside the graph (the ones before it are issued directly every forward) */
    int graph_launches;    /* kernel launches one replay stands for */
} instance;

struct thb_engine {
    thb_model *model;
    int mode, dtype, ngpus;
    float range;
    int strict_math;
    /* shape the instances were planned for */
    int N, C, H, W, rank, cp;
    int built;
    int input_s2d; /* the network input is staged space-to-depth for a stride-2 first convolution */
    int input_neigh; /* uint8 engine, 3x3 / stride 1 / pad 1 first convolution on a three-plane float batch: the boundary kernel
                      * stages every pixel's 27 quantised neighbours as the channels of that pixel (taps outside the image: the
                      * byte of 0.0), and the layer runs as a 1x1 convolution over them -- no gather, no border classes */
    int input_pad16; /* the network input is staged with 16 channels per pixel (zeros behind the real ones) for a stride-1
                      * first convolution, which then runs as a 16-channel convolution through the patch kernel */
    instance inst[8];
    /* Host-input forwards are pipelined: the batch slice of each GPU is cut into `chunks` sub-batches, each with its own
     * plan instance and stream on that GPU, so that the host-to-device copy of one sub-batch runs under the kernels of
     * the one before it.  Built on the first such forward; chunk c of GPU g is pipe[g * chunks + c]. */
    instance pipe[32];
    int chunks, pipe_built, pipe_chunks;
    float *h_out;
    size_t h_out_bytes;
    float *h_stage; /* pinned staging buffer for float batches that arrive in pageable host memory */
    size_t h_stage_bytes;
    float last_ms;
    int peer_gather;
    /* arguments of the last forward, for the device-resident timing loop */
    int honour_pads; /* THB200_HONOUR_PADS=1: ending pads, dilation, auto_pad and reflection padding of ONNX convolutions are computed */
    int whole_batch; /* the model has an operator that looks across the batch: one GPU, no sub-batches */
    int last_has_x, last_cp, last_bgr;
    float last_mean[3], last_std[3];
};

static int align_of(int dtype) { return thb_channel_align(dtype); }
static int esize_of(int dtype) { return dtype == THB_F32 ? 4 : dtype == THB_U8 ? 1 : 2; }
static int ru(int v, int m) { return (v + m - 1) / m * m; }

/* ---- device allocations owned by an instance ---- */
static void *dalloc(instance *I, size_t bytes)
{
    void *p = 0;
    if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) {
        thb_set_error("cudaMalloc of %zu bytes failed on device %d", bytes, I->device);
        return 0;
    }
    if (I->nallocs == I->capallocs) {
        I->capallocs = I->capallocs ? I->capallocs * 2 : 64;
        I->allocs = realloc(I->allocs, I->capallocs * sizeof(void *));
    }
    I->allocs[I->nallocs++] = p;
    return p;
}
/* host memory that lives as long as the instance */
static void host_keep(instance *I, void *p)
{
    if (I->nhost == I->caphost) {
        I->caphost = I->caphost ? I->caphost * 2 : 64;
        I->hostmem = realloc(I->hostmem, I->caphost * sizeof(void *));
    }
    I->hostmem[I->nhost++] = p;
}
static void *dupload(instance *I, const void *host, size_t bytes)
{
    void *p = dalloc(I, bytes);
    if (p && cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        thb_set_error("upload of %zu bytes failed", bytes);
        return 0;
    }
    return p;
}

/* ---- shape rules ---- */
static int conv_out(int in, int k, int d, int pad) { return (in + 2 * pad - k) / d + 1; }
/* SpatialMaxPooling.c:196-210 / SpatialAveragePooling.c:120-139 */
static int pool_out(int in, int k, int d, int pad, int ceil_mode, int any_pad)
{
    int o = ceil_mode ? (int)ceilf((float)(in - k + 2 * pad) / d) + 1 : (int)floorf((float)(in - k + 2 * pad) / d) + 1;
    if (any_pad && (o - 1) * d >= in + pad) --o; /* the last window must start inside the image */
    return o;
}

typedef struct {
    thb_engine *E;
    instance *I;
    thb_model *M;
    value *val;
    int *uses;      /* consumer count per node (+1 for the output) */
    int *absorbed;  /* node folded into an earlier launch */
    int *leader;    /* node index at which the value of node i is produced */
    int capbufs, capsteps;
} planner;

static int new_buf(planner *P, size_t bytes)
{
    instance *I = P->I;
    if (I->nbufs == P->capbufs) {
        P->capbufs = P->capbufs ? P->capbufs * 2 : 64;
        I->bufs = realloc(I->bufs, P->capbufs * sizeof(abuf));
    }
    abuf *b = &I->bufs[I->nbufs];
    b->bytes = (bytes + 255) & ~(size_t)255;
    b->offset = 0;
    b->first = b->last = -1;
    return I->nbufs++;
}
static step *new_step(planner *P, int kind)
{
    instance *I = P->I;
    if (I->nsteps == P->capsteps) {
        P->capsteps = P->capsteps ? P->capsteps * 2 : 64;
        I->steps = realloc(I->steps, P->capsteps * sizeof(step));
    }
    step *s = &I->steps[I->nsteps++];
    memset(s, 0, sizeof(*s));
    s->kind = kind;
    s->dtype = P->E->dtype;
    s->out_buf = s->aux_buf = s->aux2_buf = s->scratch_buf = -1;
    for (int i = 0; i < 8; i++) s->in_buf[i] = -1;
    s->flops_node = -1;
    return s;
}
static void step_in(step *s, const value *v)
{
    s->in_buf[s->nin] = v->buf;
    s->in_ld[s->nin] = v->ld;
    s->in_coff[s->nin] = v->coff;
    s->nin++;
}
/* fresh dense activation buffer for a value of shape `sh` */
static void materialise(planner *P, value *v, shape sh)
{
    int al = align_of(P->E->dtype);
    long pixels = (long)sh.N * sh.H * sh.W;
    v->s = sh;
    v->ld = ru(sh.C, al);
    v->coff = 0;
    v->buf = new_buf(P, (size_t)pixels * v->ld * esize_of(P->E->dtype));
}
static void step_out(step *s, const value *v)
{
    s->out_buf = v->buf;
    s->out_ld = v->ld;
    s->out_coff = v->coff;
    /* extent of the result, for the per-launch min/max report (th_minmax) */
    s->out_pixels = v->s.flat ? (long)v->s.N * v->s.fH * v->s.fW : (long)v->s.N * v->s.H * v->s.W;
    s->out_C = v->s.flat ? v->s.fC : v->s.C;
}

/* host-side value of one stored element (th_minmax report only) */
static float element_as_float(const void *p, long i, int dtype)
{
    if (dtype == THB_F32) return ((const float *)p)[i];
    if (dtype == THB_U8) return ((const unsigned char *)p)[i];
    unsigned short h = ((const unsigned short *)p)[i];
    unsigned int bits;
    if (dtype == THB_BF16) bits = (unsigned int)h << 16;
    else {
        const unsigned int sign = (h & 0x8000u) << 16, exp = (h >> 10) & 31, man = h & 1023;
        if (exp == 0) {
            float f = (float)man * (1.0f / 16777216.0f); /* subnormal: man * 2^-24 */
            return sign ? -f : f;
        }
        bits = exp == 31 ? sign | 0x7f800000u | (man << 13) : sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Joining without a copy: when every launch that writes a value's buffer takes an output pitch (convolutions, pooling,
 * elementwise kernels) and every reader takes an input pitch and a channel offset (the concatenation itself,
 * convolutions, pooling), those launches are pointed at the value's channel slice of the joined buffer instead
 * (thb_conv_desc.in_ld / out_ld and the kernels' x_ld / y_ld exist for this), and the value's own buffer is never
 * allocated.  Returns 1 when done, 0 when the value has to be copied.  THB200_JOIN_COPY=1 keeps the copies (diagnostic). */
static int write_into_slice(planner *P, int node, value *v, int jbuf, int jld, int coff)
{
    const char *e = getenv("THB200_JOIN_COPY"); /* (read while planning, not per launch) */
    const int keep_copies = e && atoi(e);
    instance *I = P->I;
    if (keep_copies || node == P->M->output || v->buf < 0 || v->coff || v->row_pitch || v->s.flat || v->buf == I->in_val.buf)
        return 0;
    /* readers still to be planned will see the slice: all of them must be able to */
    for (int j = 0; j < P->M->nnodes; j++) {
        const thb_node *c = &P->M->nodes[j];
        for (int q = 0; q < c->nin; q++)
            if (c->in[q] == node && !(c->op == OP_CONCAT || c->op == OP_MAXPOOL || c->op == OP_AVGPOOL || (c->op == OP_CONV && q == 0)))
                return 0;
    }
    /* no other value may live in the buffer (views and aliases), launches of the same fused chain apart */
    for (int i = 0; i < P->M->nnodes; i++)
        if (i != node && P->val[i].buf == v->buf && !P->absorbed[i]) return 0;
    int writers = 0;
    for (int t = 0; t < I->nsteps; t++) {
        const step *s = &I->steps[t];
        for (int k = 0; k < s->nin; k++)
            if (s->in_buf[k] == v->buf) {
                /* an earlier reader: its first operand, through a kernel that takes pitch and offset */
                if (k != 0 || s->out_buf == v->buf || s->in_coff[0] || s->in_off0 || s->in_ld[0] != v->ld || s->dual ||
                    !(s->kind == ST_CONV || s->kind == ST_MAXPOOL || s->kind == ST_AVGPOOL || s->kind == ST_CSUM || s->kind == ST_COPY))
                    return 0;
                if (s->kind == ST_CONV && (s->conv.in_ld != v->ld || s->conv.in_row_pitch)) return 0;
            }
        if (s->aux_buf == v->buf || s->aux2_buf == v->buf) return 0;
        if (s->out_buf != v->buf) continue;
        if (s->out_coff || s->out_off0 || s->out_ld != v->ld) return 0;
        switch (s->kind) {
        case ST_CONV: case ST_MAXPOOL: case ST_AVGPOOL: case ST_AFFINE: case ST_COMBINE: case ST_U8COMBINE: case ST_U8THR:
        case ST_UPSAMPLE: case ST_COL2IM:
            writers++;
            break;
        default:
            return 0;
        }
    }
    if (!writers) return 0;
    for (int t = 0; t < I->nsteps; t++) {
        step *s = &I->steps[t];
        if (s->nin > 0 && s->in_buf[0] == v->buf) {
            s->in_buf[0] = jbuf; s->in_ld[0] = jld; s->in_coff[0] = coff;
            if (s->kind == ST_CONV) s->conv.in_ld = jld;
        }
        if (s->out_buf != v->buf) continue;
        s->out_buf = jbuf; s->out_ld = jld; s->out_coff = coff;
        if (s->kind == ST_CONV) s->conv.out_ld = jld;
    }
    v->buf = jbuf; v->ld = jld; v->coff = coff;
    return 1;
}

static int sole_consumer(planner *P, int node)
{
    if (P->uses[node] != 1 || node == P->M->output) return -1;
    for (int j = node + 1; j < P->M->nnodes; j++)
        for (int k = 0; k < P->M->nodes[j].nin; k++)
            if (P->M->nodes[j].in[k] == node) return j;
    return -1;
}

static float *upload_floats(planner *P, const float *src, int n, int padded)
{
    float *tmp = calloc(padded, sizeof(float));
    memcpy(tmp, src, sizeof(float) * n);
    float *d = dupload(P->I, tmp, sizeof(float) * padded);
    free(tmp);
    return d;
}

static int fill_act(planner *P, thb_act *a, const thb_node *n, int C)
{
    a->kind = n->act_kind;
    a->threshold = n->act_threshold;
    a->value = n->act_value;
    a->alpha = n->act_alpha;
    a->slope = 0;
    if (n->act_kind == THB_ACT_PRELU) {
        /* the kernels read per-channel arrays in 16-byte groups and per 64-column block: a multiple of 64 floats */
        const int padded = ru(C, 64);
        float *tmp = calloc(padded, sizeof(float));
        if (!tmp || (n->nslope && n->nslope != C)) {
            free(tmp);
            thb_set_error("wrong number of input planes for PReLU (%d slopes, %d channels)", n->nslope, C);
            return -1;
        }
        for (int i = 0; i < C; i++) tmp[i] = n->nslope ? n->slope[i] : n->slope[0];
        a->slope = dupload(P->I, tmp, sizeof(float) * padded);
        free(tmp);
        if (!a->slope) return -1;
    }
    return 0;
}

/* Emit the launch(es) of a convolution / Linear / transposed convolution and whatever folds into it.
 * Returns the node whose value the launch produces. */
static int plan_gemm_group(planner *P, int i)
{
    thb_engine *E = P->E;
    thb_model *M = P->M;
    thb_node *n = &M->nodes[i];
    const value *in = &P->val[n->in[0]];
    const int dtype = E->dtype, al = align_of(dtype);
    shape is = in->s, os = is;
    int is_linear = n->op == OP_LINEAR, is_deconv = n->op == OP_DECONV;
    /* stride-2 first convolution on a space-to-depth input (see instance_build): rewritten as a stride-1 convolution
     * over 4*Cin channels.  Input row 2*oh - pad + r is block row oh + floor((r - pad)/2), phase (r - pad) mod 2. */
    const int s2d = E->input_s2d && n->in[0] == 0 && n->op == OP_CONV;
    const int pad16 = E->input_pad16 && n->in[0] == 0 && n->op == OP_CONV;  /* 16 stored channels, zeros behind the real ones */
    const int neigh = E->input_neigh && n->in[0] == 0 && n->op == OP_CONV;  /* 27 neighbours per pixel: a 1x1 convolution */
    const int s2d_padH = (n->padH + 1) / 2, s2d_padW = (n->padW + 1) / 2;
    const int s2d_kH = (n->kH - 1 - n->padH) / 2 + s2d_padH + 1, s2d_kW = (n->kW - 1 - n->padW) / 2 + s2d_padW + 1;

    /* ---- geometry ---- */
    int kH = n->kH, kW = n->kW, Cin = n->Cin, H = is.H, W = is.W, in_ld = in->ld, permute_hw = 0;
    int honour = 0, ekH = n->kH, ekW = n->kW, padT = n->padH, padB = n->padH, padL = n->padW, padR = n->padW;
    value refl_val;
    if (is_linear) {
        long feat = is.flat ? (long)is.fC * is.fH * is.fW : (long)is.C * is.H * is.W;
        if (feat != n->Cin) { thb_set_error("Linear expects %d inputs, got %ld", n->Cin, feat); return -1; }
        if (is.flat || is.H * is.W > 1) {
            /* the features are an NCHW flatten of a channels-innermost tensor: permute the weight's K axis */
            int fH = is.flat ? is.fH : is.H, fW = is.flat ? is.fW : is.W;
            if (in->coff) { thb_set_error("Linear on a channel slice is not supported"); return -1; }
            permute_hw = fH * fW;
            Cin = permute_hw * in->ld;
            in_ld = Cin;
        }
        H = W = 1;
        os.rank = is.N == 1 ? 1 : 2;
        os.C = n->Cout; os.H = os.W = 1; os.flat = 0;
    } else if (is_deconv) {
        if (is.rank < 3) { thb_set_error("3D or 4D (batch mode) tensor is expected"); return -1; }
        if (is.C != n->Cin) { thb_set_error("input channels and nInputPlane dont match"); return -1; }
        os.C = n->Cout;
        os.H = (is.H - 1) * n->dH - 2 * n->padH + n->kH + n->adjH;
        os.W = (is.W - 1) * n->dW - 2 * n->padW + n->kW + n->adjW;
    } else if (neigh) {
        os.C = n->Cout;  /* same spatial size (3x3, pad 1, stride 1) */
        Cin = 27;
        kH = kW = 1;
    } else if (s2d) {
        /* the logical input is still [N, Cin, 2H', 2W']: output size from the original geometry */
        os.C = n->Cout;
        os.H = conv_out(E->H, n->kH, 2, n->padH);
        os.W = conv_out(E->W, n->kW, 2, n->padW);
        Cin = 4 * n->Cin;
        kH = s2d_kH; kW = s2d_kW;
    } else {
        if (is.rank < 3) { thb_set_error("convolution needs a 3D or 4D input"); return -1; }
        if (is.C != n->Cin) { thb_set_error("nInputPlane %d does not match input planes %d", n->Cin, is.C); return -1; }
        os.C = n->Cout;
        /* Ending pads that differ from the leading ones, dilation, auto_pad and reflection padding: the reference's ONNX
         * loader parses them and none of its engines reads them (SpatialConvolution.c:88-109, onnx.cc:677-690), so by
         * default they are ignored here too -- and said so.  THB200_HONOUR_PADS=1 computes what the ONNX model asks for:
         * auto_pad resolved from the input size, a reflection-padded copy of the input, the output size from both pads
         * (the kernels pad with zeros wherever a window leaves the image, so only the size changes), and a dilated
         * kernel written out with zeros between its taps. */
        const int dlH = n->dlH > 0 ? n->dlH : 1, dlW = n->dlW > 0 ? n->dlW : 1;
        const int nontrivial = n->op == OP_CONV && (n->pad2H != n->padH || n->pad2W != n->padW || dlH != 1 || dlW != 1 || n->autopad || n->refl_pad);
        if (nontrivial && !(E->honour_pads && dtype != THB_U8)) {
            static int told = 0;
            if (!told++)
                fprintf(stderr, "thb200: a convolution's ending pads / dilation / auto_pad / reflection padding are ignored, as by the "
                                "reference (THB200_HONOUR_PADS=1 honours them)\n");
        }
        if (nontrivial && E->honour_pads && dtype != THB_U8) {
            honour = 1;
            ekH = (kH - 1) * dlH + 1; ekW = (kW - 1) * dlW + 1;
            padT = n->padH; padB = n->pad2H; padL = n->padW; padR = n->pad2W;
            if (n->autopad) {
                /* SAME_UPPER (1): the odd pixel of padding goes to the end; SAME_LOWER (2): to the beginning */
                int th_ = ((is.H + n->dH - 1) / n->dH - 1) * n->dH + ekH - is.H, tw_ = ((is.W + n->dW - 1) / n->dW - 1) * n->dW + ekW - is.W;
                if (th_ < 0) th_ = 0;
                if (tw_ < 0) tw_ = 0;
                padT = n->autopad == 1 ? th_ / 2 : th_ - th_ / 2; padB = th_ - padT;
                padL = n->autopad == 1 ? tw_ / 2 : tw_ - tw_ / 2; padR = tw_ - padL;
            }
            if (n->refl_pad && (padT || padB || padL || padR)) {
                if (padT >= is.H || padB >= is.H || padL >= is.W || padR >= is.W) { thb_set_error("reflection padding larger than the image"); return -1; }
                shape ps = is;
                ps.H = is.H + padT + padB; ps.W = is.W + padL + padR;
                memset(&refl_val, 0, sizeof(refl_val));
                materialise(P, &refl_val, ps);
                step *rs = new_step(P, ST_REFLECTPAD);
                step_in(rs, in); step_out(rs, &refl_val);
                rs->N = is.N; rs->H = is.H; rs->W = is.W; rs->C = is.C;
                rs->padW = padL; rs->kW = padR; rs->padH = padT; rs->kH = padB;
                in = &refl_val;
                is = ps; H = is.H; W = is.W; in_ld = in->ld;
                padT = padB = padL = padR = 0;
            }
            os.H = (is.H + padT + padB - ekH) / n->dH + 1;
            os.W = (is.W + padL + padR - ekW) / n->dW + 1;
            kH = ekH; kW = ekW;
        } else {
            os.H = conv_out(is.H, kH, n->dH, n->padH);
            os.W = conv_out(is.W, kW, n->dW, n->padW);
        }
        if (os.H < 1 || os.W < 1) { thb_set_error("Given input size: (%dx%dx%d). Output size is too small", is.C, is.H, is.W); return -1; }
    }

    /* ---- what folds in ---- */
    int cur = i, bn = -1, comb = -1, act = -1, j;
    /* In uint8 mode a batch normalisation that follows is folded into the weights and the bias BEFORE they are
     * quantised (w' = w * scale[co], b' = b * scale[co] + shift[co], the algebra of the reference's ONNX loader,
     * onnx.cc:537-548): the reference's lowp engine itself refuses the module (lowp/lowp_basic.c:194-196). */
    if (!is_deconv && (j = sole_consumer(P, cur)) >= 0 && M->nodes[j].op == OP_BN) { bn = j; cur = j; }
    if (bn >= 0 && M->nodes[bn].C != n->Cout) { thb_set_error("batch-norm width mismatch"); return -1; }
    int res_node = -1;
    float self_coef = 1.f, res_coef = 0.f;
    /* uint8: the fused residual needs what thb_u8_combine needs (two tensors on the static range, coefficients +-1)
     * and the table-driven epilogue (at most 13 border classes, the image at least as large as the kernel) */
    const char *nofuse = getenv("THB200_U8_NO_FUSED_RESIDUAL");
    const int u8_res_ok = dtype == THB_U8 && !in->q_dyn && (1 + 2 * n->padH) * (1 + 2 * n->padW) <= 13 && H >= kH && W >= kW &&
                          n->padH < kH && n->padW < kW && !is_linear && !(nofuse && atoi(nofuse));
    if ((dtype != THB_U8 || u8_res_ok) && !is_deconv && (j = sole_consumer(P, cur)) >= 0 && M->nodes[j].op == OP_COMBINE && M->nodes[j].nin == 2) {
        int pos = M->nodes[j].in[0] == cur ? 0 : 1, other = M->nodes[j].in[1 - pos];
        const float c0 = M->nodes[j].coef[0], c1 = M->nodes[j].coef[1];
        const int u8_ok = dtype != THB_U8 || ((c0 == 1.f || c0 == -1.f) && (c1 == 1.f || c1 == -1.f) && !P->val[other].q_dyn &&
                                              P->val[other].q_sub == -E->range / 2 && P->val[other].q_mult == 255 / E->range);
        if (u8_ok && other != cur && other < i && P->val[other].buf >= 0 && !P->val[other].s.flat &&
            (long)P->val[other].s.C == os.C && P->val[other].s.H == os.H && P->val[other].s.W == os.W) {
            comb = j; cur = j; res_node = other;
            self_coef = M->nodes[j].coef[pos];
            res_coef = M->nodes[j].coef[1 - pos];
        }
    }
    /* Two 1x1 convolutions whose (batch-normalised) outputs meet in a two-input sum -- a bottleneck block's last
     * convolution and its projection shortcut -- run as ONE convolution over both inputs: the weights side by side
     * along K (each scaled by its batch-norm and its coefficient of the sum), one accumulator, neither addend written.
     * 16-bit tensor-core modes only; the second convolution must not have been planned yet and must be used nowhere else. */
    int dual_conv = -1, dual_bn = -1;
    {
        const char *nodual = getenv("THB200_NO_DUAL");
        if (comb < 0 && (dtype == THB_F16 || dtype == THB_BF16) && !is_deconv && !is_linear && !s2d && n->kH == 1 && n->kW == 1 &&
            n->dH == 1 && n->dW == 1 && n->padH == 0 && n->padW == 0 && n->Cin % 64 == 0 && n->Cout >= 64 && !in->row_pitch &&
            in->coff == 0 && !(nodual && atoi(nodual)) && (j = sole_consumer(P, cur)) >= 0 && M->nodes[j].op == OP_COMBINE &&
            M->nodes[j].nin == 2) {
            const int pos = M->nodes[j].in[0] == cur ? 0 : 1, other = M->nodes[j].in[1 - pos];
            int ob = -1, oc = other;
            if (other > cur && other < j && M->nodes[other].op == OP_BN && P->uses[other] == 1) { ob = other; oc = M->nodes[other].in[0]; }
            if (oc > cur && oc < j && P->uses[oc] == 1 && M->nodes[oc].op == OP_CONV && oc != M->output && other != M->output) {
                const thb_node *c2 = &M->nodes[oc];
                const value *v2 = &P->val[c2->in[0]];
                if (c2->kH == 1 && c2->kW == 1 && c2->padH == 0 && c2->padW == 0 && c2->dH == c2->dW && c2->dH >= 1 && c2->dH <= 8 &&
                    c2->Cout == n->Cout && c2->Cin % 64 == 0 && c2->in[0] <= i && v2->buf >= 0 && !v2->s.flat && v2->s.rank >= 3 &&
                    v2->s.C == c2->Cin && v2->coff == 0 && !v2->row_pitch && v2->s.N == is.N &&
                    conv_out(v2->s.H, 1, c2->dH, 0) == os.H && conv_out(v2->s.W, 1, c2->dW, 0) == os.W &&
                    (ob < 0 || M->nodes[ob].C == n->Cout)) {
                    dual_conv = oc; dual_bn = ob;
                    comb = j; cur = j;
                    self_coef = M->nodes[j].coef[pos];
                    res_coef = M->nodes[j].coef[1 - pos];
                }
            }
        }
    }
    if ((j = sole_consumer(P, cur)) >= 0 && M->nodes[j].op == OP_ACT &&
        (dtype != THB_U8 || M->nodes[j].act_kind == THB_ACT_THRESHOLD)) { act = j; cur = j; }
    for (int k = i + 1; k <= cur; k++)
        if (k == bn || k == comb || k == act || k == dual_conv || k == dual_bn) { P->absorbed[k] = 1; P->leader[k] = i; }
    /* A stride-2 max pooling as the only consumer of this convolution (after its batch-norm and activation) can run
     * inside the convolution's launch, which then stores the pooled tensor only: decided below, once the kernel
     * geometry is known (16-bit types, at most 64 output channels, stride-1 convolution). */
    int pool = -1;
    if ((dtype == THB_F16 || dtype == THB_BF16) && !is_linear && !is_deconv && comb < 0 && dual_conv < 0 && n->Cout <= 64 &&
        (j = sole_consumer(P, cur)) >= 0 && M->nodes[j].op == OP_MAXPOOL) {
        const thb_node *pn = &M->nodes[j];
        if (pn->kH == pn->kW && pn->dH == 2 && pn->dW == 2 && pn->padH == pn->padW) pool = j;
    }

    /* ---- per-channel scale / shift ---- */
    float *scale = 0, *shift = 0;
    float *scale_h = 0, *shift_h = 0; /* host copies, owned by the instance (thb_conv_desc.scale_host / shift_host) */
    if (dtype != THB_U8) {
        int Cp = ru(n->Cout, 64);
        float *hs = calloc(Cp, sizeof(float)), *hh = calloc(Cp, sizeof(float));
        for (int c = 0; c < n->Cout; c++) {
            float b = n->bias ? n->bias[c] : 0.f;
            hs[c] = bn >= 0 ? M->nodes[bn].scale[c] : 1.f;
            hh[c] = bn >= 0 ? M->nodes[bn].scale[c] * b + M->nodes[bn].shift[c] : b;
        }
        if (bn >= 0 && M->nodes[bn].C != n->Cout) { free(hs); free(hh); thb_set_error("batch-norm width mismatch"); return -1; }
        if (dual_conv >= 0) {
            /* both scales go into the weights (below); what is left is the sum of the two shifts */
            const thb_node *c2 = &M->nodes[dual_conv];
            for (int c = 0; c < n->Cout; c++) {
                const float b2 = c2->bias ? c2->bias[c] : 0.f;
                const float h2 = dual_bn >= 0 ? M->nodes[dual_bn].scale[c] * b2 + M->nodes[dual_bn].shift[c] : b2;
                hh[c] = self_coef * hh[c] + res_coef * h2;
                hs[c] = 1.f;
            }
        }
        if (bn >= 0 && dual_conv < 0) { scale = dupload(P->I, hs, sizeof(float) * Cp); scale_h = hs; }
        if ((dual_conv >= 0 || bn >= 0 || n->bias) && !is_deconv) { shift = dupload(P->I, hh, sizeof(float) * Cp); shift_h = hh; }
        if (scale_h) host_keep(P->I, hs); else free(hs);
        if (shift_h) host_keep(P->I, hh); else free(hh);
    }

    value *out = &P->val[cur];

    /* ---- small-batch Linear: weight-streaming GEMV ---- */
    if (is_linear && dtype != THB_U8 && is.N <= 8) {
        materialise(P, out, os);
        step *s = new_step(P, ST_GEMV);
        step_in(s, in);
        step_out(s, out);
        /* weight rows are as long as the physical feature vector (channel padding included, zero weights there) */
        const int Kp = permute_hw ? Cin : in->ld;
        s->N = is.N; s->K = Kp; s->M = n->Cout; s->in_ld[0] = permute_hw ? in_ld : in->ld;
        s->scale = scale; s->shift = shift;
        if (act >= 0 && fill_act(P, &s->act, &M->nodes[act], n->Cout)) return -1;
        size_t es = esize_of(dtype);
        unsigned char *hw = calloc((size_t)n->Cout * Kp, es);
        for (int o = 0; o < n->Cout; o++)
            for (int k = 0; k < n->Cin; k++) {
                long dst = k;
                if (permute_hw) { int c = k / permute_hw, hw_ = k % permute_hw; dst = (long)hw_ * in->ld + c; }
                float v = n->weight[(size_t)o * n->Cin + k];
                if (dtype == THB_F32) ((float *)hw)[(size_t)o * Kp + dst] = v;
                else ((unsigned short *)hw)[(size_t)o * Kp + dst] = thb_float_to_half_bits(v, dtype == THB_BF16);
            }
        s->w = dupload(P->I, hw, (size_t)n->Cout * Kp * es);
        free(hw);
        if (!s->w) return -1;
        s->flops_node = i;
        return cur;
    }

    /* ---- implicit-GEMM convolution launch ---- */
    int csum_buf = -1;
    if (dtype == THB_U8) {
        /* per-pixel channel sums of the input feed the zero-point correction of the convolution */
        /* (several convolutions reading one tensor share one pass; csum_buf holds buffer index + 1, 0 = none yet) */
        value *inw = &P->val[n->in[0]];
        if (inw->csum_buf > 0 && !is_linear) csum_buf = inw->csum_buf - 1;
        else {
            csum_buf = new_buf(P, sizeof(int) * (size_t)is.N * H * W);
            step *cs = new_step(P, ST_CSUM);
            step_in(cs, in);
            cs->in_ld[0] = in_ld;
            cs->pixels = (long)is.N * H * W; cs->C = Cin; cs->out_buf = csum_buf;
            if (!is_linear) inw->csum_buf = csum_buf + 1;
        }
    }
    /* uint8: a place-holder launch in front of the convolution; it becomes the clearing of the output's channel-sum
     * buffer when the convolution has several column tiles, which then add their partial sums into it */
    int zero_step = -1;
    if (dtype == THB_U8 && !is_linear) {
        new_step(P, ST_ZERO)->pixels = 0;
        zero_step = P->I->nsteps - 1;
    }
    step *s = new_step(P, ST_CONV);
    thb_conv_desc *d = &s->conv;
    s->aux_buf = csum_buf;
    d->dtype = dtype;
    d->N = is.N; d->H = H; d->W = W; d->Cin = Cin; d->in_ld = in_ld;
    d->in_row_pitch = in->row_pitch; d->in_pad_left = in->pad_left;
    d->kH = kH; d->kW = kW; d->dH = n->dH; d->dW = n->dW; d->padH = n->padH; d->padW = n->padW;
    if (neigh) d->padH = d->padW = 0;
    d->self_coef = 1.f; d->res_coef = 0.f; d->relu_thr = -1;
    int Cp_out = ru(n->Cout, al);
    float *w_oihw = n->weight, *w_tmp = 0;
    float *w_fold = 0, *b_fold = 0; /* uint8: weights and bias with the batch normalisation folded in */
    const float *bias_eff = n->bias;
    if (dtype == THB_U8 && bn >= 0) {
        const size_t per = (size_t)n->Cin * n->kH * n->kW;
        w_fold = malloc(sizeof(float) * per * n->Cout);
        b_fold = malloc(sizeof(float) * n->Cout);
        for (int co = 0; co < n->Cout; co++) {
            const float sc = M->nodes[bn].scale[co];
            for (size_t k = 0; k < per; k++) w_fold[co * per + k] = n->weight[co * per + k] * sc;
            b_fold[co] = (n->bias ? n->bias[co] * sc : 0.f) + M->nodes[bn].shift[co];
        }
        w_oihw = w_fold;
        bias_eff = b_fold;
    }
    if (is_deconv) {
        /* column matrix [N*H*W][kH*kW*Cp]: column (kh*kW + kw)*Cp + co  <-  W[ci][co][kh][kw] */
        d->Cout = kH * kW * Cp_out; d->kH = d->kW = 1; d->dH = d->dW = 1; d->padH = d->padW = 0;
        d->oH = H; d->oW = W;
        w_tmp = calloc((size_t)d->Cout * Cin, sizeof(float));
        for (int ci = 0; ci < Cin; ci++)
            for (int co = 0; co < n->Cout; co++)
                for (int t = 0; t < kH * kW; t++)
                    w_tmp[((size_t)t * Cp_out + co) * Cin + ci] = n->weight[((size_t)ci * n->Cout + co) * kH * kW + t];
        w_oihw = w_tmp;
    } else if (is_linear) {
        d->Cout = n->Cout; d->oH = d->oW = 1;
        if (permute_hw && w_fold) { free(w_fold); free(b_fold); thb_set_error("batch-norm after a flattened Linear is not supported in Lowp"); return -1; }
        if (permute_hw) {
            w_tmp = calloc((size_t)n->Cout * Cin, sizeof(float));
            for (int o = 0; o < n->Cout; o++)
                for (int k = 0; k < n->Cin; k++) {
                    int c = k / permute_hw, hw_ = k % permute_hw;
                    w_tmp[(size_t)o * Cin + (size_t)hw_ * in->ld + c] = n->weight[(size_t)o * n->Cin + k];
                }
            w_oihw = w_tmp;
        }
    } else if (s2d) {
        d->Cout = n->Cout; d->oH = os.H; d->oW = os.W;
        d->dH = d->dW = 1; d->padH = s2d_padH; d->padW = s2d_padW;
        /* W'[co][(ph*2 + pw)*Cin + c][dh][dw] = W[co][c][2*(dh - pad') + ph + pad][...] where that row exists */
        w_tmp = calloc((size_t)n->Cout * Cin * kH * kW, sizeof(float));
        for (int co = 0; co < n->Cout; co++)
            for (int c = 0; c < n->Cin; c++)
                for (int r = 0; r < n->kH; r++)
                    for (int q = 0; q < n->kW; q++) {
                        int tr = r - n->padH + 2 * s2d_padH, tq = q - n->padW + 2 * s2d_padW; /* >= 0 */
                        int dh = tr / 2, ph = tr % 2, dw = tq / 2, pw = tq % 2;
                        w_tmp[(((size_t)co * Cin + (ph * 2 + pw) * n->Cin + c) * kH + dh) * kW + dw] =
                            (w_fold ? w_fold : n->weight)[(((size_t)co * n->Cin + c) * n->kH + r) * n->kW + q];
                    }
        w_oihw = w_tmp;
    } else if (neigh) {
        /* W'[co][(r*3 + s)*3 + c] = W[co][c][r][s]: the order the boundary kernel stores a pixel's neighbours in */
        d->Cout = n->Cout; d->oH = os.H; d->oW = os.W;
        const float *src = w_fold ? w_fold : n->weight;
        w_tmp = calloc((size_t)n->Cout * 27, sizeof(float));
        for (int co = 0; co < n->Cout; co++)
            for (int c = 0; c < 3; c++)
                for (int r = 0; r < 3; r++)
                    for (int q = 0; q < 3; q++)
                        w_tmp[(size_t)co * 27 + (r * 3 + q) * 3 + c] = src[(((size_t)co * 3 + c) * 3 + r) * 3 + q];
        w_oihw = w_tmp;
    } else if (pad16) {
        /* the same convolution over 16 input channels, the added ones with zero weights */
        d->Cout = n->Cout; d->oH = os.H; d->oW = os.W;
        d->Cin = 16;
        d->BN = 64; /* (the patch kernel's tile, also below 33 output channels) */
        const float *src = w_fold ? w_fold : n->weight;
        w_tmp = calloc((size_t)n->Cout * 16 * kH * kW, sizeof(float));
        for (int co = 0; co < n->Cout; co++)
            memcpy(w_tmp + (size_t)co * 16 * kH * kW, src + (size_t)co * n->Cin * kH * kW, sizeof(float) * n->Cin * kH * kW);
        w_oihw = w_tmp;
    } else {
        d->Cout = n->Cout; d->oH = os.H; d->oW = os.W;
        if (honour) {
            d->padH = padT; d->padW = padL;
            if (ekH != n->kH || ekW != n->kW) {
                /* dilation: the kernel written out at its full extent, zeros between the taps */
                const float *src = w_fold ? w_fold : n->weight;
                const int dlH = n->dlH > 0 ? n->dlH : 1, dlW = n->dlW > 0 ? n->dlW : 1;
                w_tmp = calloc((size_t)n->Cout * Cin * ekH * ekW, sizeof(float));
                for (long oc = 0; oc < (long)n->Cout * Cin; oc++)
                    for (int r = 0; r < n->kH; r++)
                        for (int q = 0; q < n->kW; q++)
                            w_tmp[(oc * ekH + r * dlH) * ekW + q * dlW] = src[(oc * n->kH + r) * n->kW + q];
                w_oihw = w_tmp;
            }
        }
    }
    if (dual_conv >= 0) {
        /* [Cout][cin1 + cin2] weights: each convolution's rows scaled by its batch-norm and its coefficient of the sum */
        const thb_node *c2 = &M->nodes[dual_conv];
        const value *v2 = &P->val[c2->in[0]];
        const int c1n = n->Cin, c2n = c2->Cin;
        w_tmp = malloc(sizeof(float) * (size_t)n->Cout * (c1n + c2n));
        for (int co = 0; co < n->Cout; co++) {
            const float s1 = self_coef * (bn >= 0 ? M->nodes[bn].scale[co] : 1.f);
            const float s2 = res_coef * (dual_bn >= 0 ? M->nodes[dual_bn].scale[co] : 1.f);
            float *row = w_tmp + (size_t)co * (c1n + c2n);
            for (int ci = 0; ci < c1n; ci++) row[ci] = s1 * n->weight[(size_t)co * c1n + ci];
            for (int ci = 0; ci < c2n; ci++) row[c1n + ci] = s2 * c2->weight[(size_t)co * c2n + ci];
        }
        w_oihw = w_tmp;
        d->Cin = c1n + c2n;
        d->cin1 = c1n;
        d->x2_ld = v2->ld; d->x2_H = v2->s.H; d->x2_W = v2->s.W; d->x2_d = c2->dH;
    }
    if (pool >= 0) d->BN = 64;
    if (thb_conv_geometry(d)) { free(w_tmp); thb_set_error("unsupported convolution geometry %dx%d", kH, kW); return -1; }
    if (pool >= 0 && !thb_conv_maxpool_supported(d, M->nodes[pool].kH, 2, M->nodes[pool].padH)) {
        pool = -1;
        d->BN = 0;
        thb_conv_geometry(d);
    }
    if (dual_conv < 0 && in_ld < d->Cin_pad) { free(w_tmp); thb_set_error("internal: input stride %d below padded channels %d", in_ld, d->Cin_pad); return -1; }
    /* Splitting a reduction over CTAs changes the order in which its fp32 partial sums are added, and whether a layer is
     * split depends on how many tiles the (sub-)batch gives it: with it, a batch sharded over GPUs or cut into sub-batches
     * no longer reproduces the whole batch bit for bit.  That identity is worth more than the few-tile layers' time, so
     * the 16-bit engines split only on request (THB200_SPLITK=1). */
    const char *ske = getenv("THB200_SPLITK");
    const int want_split = ske && atoi(ske);
    if (want_split && is_linear && (dtype == THB_F16 || dtype == THB_BF16) && d->BN < 128 && d->Cout >= 128) {
        /* A Linear on a batch of rows is a handful of tiles with a very long reduction.  The geometry rule narrows its tiles
         * so that more SMs get a share of the weights; where the reduction can be split over CTAs instead, wide tiles
         * move four times the weight bytes per barrier round (25088 -> 4096 on 32 rows: 135 -> about 40 us). */
        const int bn_narrow = d->BN;
        size_t bytes = 0;
        d->BN = 128;
        if (thb_conv_geometry(d) || thb_conv_splitk_plan(d, &bytes) < 2) {
            d->BN = bn_narrow;
            thb_conv_geometry(d);
        }
    }
    if (want_split && pool < 0 && dual_conv < 0 && (dtype == THB_F16 || dtype == THB_BF16) && !thb_conv_patch_supported(d)) {
        /* a launch of few tiles: several CTAs share each tile's reduction, through an fp32 scratch that lives for this launch */
        size_t sk_bytes = 0;
        const int S = thb_conv_splitk_plan(d, &sk_bytes);
        if (S > 1) {
            d->splits = S;
            s->scratch_buf = new_buf(P, sk_bytes);
        }
    }

    size_t wbytes = thb_conv_weight_bytes(d), kwords = thb_conv_kinfo_words(d);
    void *packed = malloc(wbytes);
    int *kinfo = malloc(kwords * sizeof(int)), *wsat = 0;
    unsigned char *wq = 0;
    if (dtype == THB_U8) {
        /* lowp/lowp_basic.c:156-157: weights and bias quantised over their own ranges */
        long wn = (long)d->Cout * d->Cin * d->kH * d->kW;
        wq = malloc(wn);
        thb_lowp_quantize(w_oihw, wn, wq, &s->w_sub, &s->w_mult);
        wsat = malloc(sizeof(int) * d->Cout * (d->kH + 1) * (d->kW + 1));
    }
    int rc = thb_conv_pack_weights_host(d, dtype == THB_U8 ? 0 : w_oihw, wq, packed, kinfo, wsat);
    free(w_tmp); free(w_fold);
    if (!rc) {
        d->w = dupload(P->I, packed, wbytes);
        d->kinfo = dupload(P->I, kinfo, kwords * sizeof(int));
        if (wsat) d->wsat = dupload(P->I, wsat, sizeof(int) * d->Cout * (d->kH + 1) * (d->kW + 1));
    }
    free(packed); free(kinfo); free(wsat); free(wq);
    if (rc || !d->w || !d->kinfo) { if (rc) thb_set_error("weight packing failed (%d)", rc); return -1; }
    if (dtype != THB_F32) {
        s->tmap = aligned_alloc(64, sizeof(thb_tmap));
        if (thb_conv_make_tmap(d, s->tmap)) { thb_set_error("TMA descriptor creation failed"); return -1; }
        d->tmap = s->tmap;
    }
    d->status = P->I->d_status;
    step_in(s, in);
    s->in_ld[0] = in_ld;
    s->flops_node = i;
    if (dual_conv >= 0) {
        step_in(s, &P->val[M->nodes[dual_conv].in[0]]);
        s->dual = 1;
        s->flops_extra = 2.0 * is.N * os.H * os.W * (double)n->Cout * M->nodes[dual_conv].Cin;
    }

    if (dtype == THB_U8) {
        if (!bias_eff) { thb_set_error("the lowp engine needs a bias on every convolution"); return -1; }
        unsigned char *bq = malloc(n->Cout);
        float b_sub, b_mult;
        thb_lowp_quantize(bias_eff, n->Cout, bq, &b_sub, &b_mult);
        free(b_fold);
        if (b_mult == 0) { free(bq); thb_set_error("an all-zero bias has no quantisation range in the lowp engine"); return -1; }
        float out_sub = -E->range / 2, out_mult = 255 / E->range; /* lowp_basic.c:137-138 */
        int *addend = malloc(sizeof(int) * n->Cout);
        thb_lowp_bias_addends(bq, n->Cout, b_sub, b_mult, out_mult, addend);
        d->bias_add = dupload(P->I, addend, sizeof(int) * n->Cout);
        free(addend); free(bq);
        s->out_sub = out_sub; s->out_mult = out_mult;
        int ohw = d->oH * d->oW;
        d->tail_start = ohw - ohw % 8;
        if (in->q_dyn) s->dyn_quant = 1;
        else {
            thb_lowp_gemm_params(s->w_sub, s->w_mult, in->q_sub, in->q_mult, out_sub, out_mult, &d->a_offset, &d->b_offset,
                                 &d->c_offset, &d->c_mult, &d->c_shift);
        }
        if (act >= 0) {
            /* lowp_Threshold.c:7-8: both bytes scaled with the (conv output) quantisation parameters */
            d->relu_thr = thb_lowp_scale_float(out_sub, out_mult, M->nodes[act].act_threshold);
            d->relu_val = thb_lowp_scale_float(out_sub, out_mult, M->nodes[act].act_value);
        }
        out->q_sub = out_sub; out->q_mult = out_mult;
        /* one column tile: the epilogue sees every output byte of a pixel and leaves their sum for the next convolution */
        const char *nocs = getenv("THB200_U8_NO_CSUM_OUT");
        if (!is_linear && zero_step >= 0 && !(nocs && atoi(nocs) == 1) && (d->Cout_pad == d->BN || !(nocs && atoi(nocs) == 2))) {
            s->aux2_buf = new_buf(P, sizeof(int) * (size_t)is.N * os.H * os.W);
            out->csum_buf = s->aux2_buf + 1;
            if (d->Cout_pad != d->BN) {
                step *z = &P->I->steps[zero_step];
                z->out_buf = s->aux2_buf;
                z->pixels = (long)is.N * os.H * os.W;
            }
        }
        if (res_node >= 0) {
            const value *rv = &P->val[res_node];
            step_in(s, rv);
            d->res_ld = rv->ld;
            d->self_coef = self_coef; d->res_coef = res_coef;
        }
    } else {
        d->scale = scale; d->shift = shift;
        d->scale_host = scale_h; d->shift_host = shift_h;
        if (act >= 0 && !is_deconv && fill_act(P, &d->act, &M->nodes[act], n->Cout)) return -1;
        if (res_node >= 0) {
            const value *rv = &P->val[res_node];
            step_in(s, rv);
            d->res_ld = rv->ld;
            d->self_coef = self_coef; d->res_coef = res_coef;
        }
    }

    if (is_deconv) {
        value cols;
        shape cs = is; cs.C = d->Cout;
        memset(&cols, 0, sizeof(cols));
        materialise(P, &cols, cs);
        s = &P->I->steps[P->I->nsteps - 1];
        step_out(s, &cols);
        s->conv.out_ld = cols.ld;
        materialise(P, out, os);
        step *g = new_step(P, ST_COL2IM);
        step_in(g, &cols);
        step_out(g, out);
        g->N = is.N; g->H = is.H; g->W = is.W; g->C = n->Cout; g->kH = kH; g->kW = kW; g->dH = n->dH; g->dW = n->dW;
        g->padH = n->padH; g->padW = n->padW; g->oH = os.H; g->oW = os.W;
        /* SpatialFullConvolution.c:229-238: the bias GEMM runs with beta = 11 whenever a bias exists */
        g->beta = E->strict_math ? 1.f : 11.f;
        if (n->bias) g->bias = upload_floats(P, n->bias, n->Cout, ru(n->Cout, 64));
        if (act >= 0 && fill_act(P, &g->act, &M->nodes[act], n->Cout)) return -1;
        return cur;
    }
    if (pool >= 0) {
        const thb_node *pn = &M->nodes[pool];
        shape ps = os;
        ps.H = pool_out(os.H, pn->kH, 2, pn->padH, pn->ceil_mode, pn->padH || pn->padW);
        ps.W = pool_out(os.W, pn->kW, 2, pn->padW, pn->ceil_mode, pn->padH || pn->padW);
        if (ps.H < 1 || ps.W < 1) { thb_set_error("input image smaller than kernel size"); return -1; }
        P->absorbed[pool] = 1;
        P->leader[pool] = i;
        out = &P->val[pool];
        os = ps;
        cur = pool;
    }
    materialise(P, out, os);
    s = &P->I->steps[P->I->nsteps - 1];
    step_out(s, out);
    s->conv.out_ld = out->ld;
    if (pool >= 0) {
        s->pool_k = M->nodes[pool].kH; s->pool_pad = M->nodes[pool].padH; s->pool_oH = os.H; s->pool_oW = os.W;
    }
    return cur;
}

static int plan_node(planner *P, int i)
{
    thb_engine *E = P->E;
    thb_model *M = P->M;
    thb_node *n = &M->nodes[i];
    const int dtype = E->dtype, al = align_of(dtype);
    value *out = &P->val[i];
    const value *in = n->nin ? &P->val[n->in[0]] : 0;
    step *s;
    int j;

    if (dtype == THB_U8 && n->op != OP_CONV && n->op != OP_LINEAR && n->op != OP_ACT && n->op != OP_MAXPOOL &&
        n->op != OP_VIEW && n->op != OP_ALIAS && n->op != OP_AVGPOOL && !(n->op == OP_COMBINE && n->nin == 2)) {
        /* the reference's lowp conversion rejects these module types too (lowp_basic.c:160-208); beyond it, this engine
         * takes what a residual network needs: a batch normalisation folded into the convolution before it, the
         * two-input CAddTable / CSubTable and the average pooling, each on the static output quantisation */
        thb_set_error("operator %d not supported in Lowp", n->op);
        return -1;
    }
    switch (n->op) {
    case OP_CONV: case OP_LINEAR: case OP_DECONV:
        return plan_gemm_group(P, i) < 0 ? -1 : 0;
    case OP_BN: case OP_ACT: case OP_SCALE: {
        int act = -1, C = in->s.C;
        if (in->s.flat) { thb_set_error("elementwise operator on a flattened spatial tensor is not supported"); return -1; }
        value *dst = out;
        if (dtype == THB_U8) {
            if (n->act_kind != THB_ACT_THRESHOLD) { thb_set_error("only Threshold is supported in Lowp"); return -1; }
            materialise(P, out, in->s);
            out->q_sub = in->q_sub; out->q_mult = in->q_mult;
            s = new_step(P, ST_U8THR);
            step_in(s, in); step_out(s, out);
            s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = C;
            s->thr = thb_lowp_scale_float(in->q_sub, in->q_mult, n->act_threshold);
            s->val = thb_lowp_scale_float(in->q_sub, in->q_mult, n->act_value);
            if (in->q_dyn) { thb_set_error("Threshold directly on the network input is not supported in Lowp"); return -1; }
            return 0;
        }
        if (n->op == OP_BN && (j = sole_consumer(P, i)) >= 0 && M->nodes[j].op == OP_ACT) {
            act = j; P->absorbed[j] = 1; P->leader[j] = i; dst = &P->val[j];
        }
        materialise(P, dst, in->s);
        s = new_step(P, ST_AFFINE);
        step_in(s, in); step_out(s, dst);
        s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = C;
        if (n->op == OP_BN) {
            if (n->C != C) { thb_set_error("batch-norm over %d channels applied to %d", n->C, C); return -1; }
            s->scale = upload_floats(P, n->scale, C, ru(C, 64));
            s->shift = upload_floats(P, n->shift, C, ru(C, 64));
            if (act >= 0 && fill_act(P, &s->act, &M->nodes[act], C)) return -1;
        } else if (n->op == OP_SCALE) {
            float *f = malloc(sizeof(float) * C);
            for (int c = 0; c < C; c++) f[c] = n->factor;
            s->scale = upload_floats(P, f, C, ru(C, 64));
            free(f);
        } else if (fill_act(P, &s->act, n, C))
            return -1;
        return 0;
    }
    case OP_MAXPOOL: case OP_AVGPOOL: {
        shape os = in->s;
        int kH = n->kH, kW = n->kW;
        if (in->s.rank < 3 || in->s.flat) { thb_set_error("3D or 4D (batch mode) tensor expected"); return -1; }
        if (n->op == OP_AVGPOOL) {
            if (kW == 0) kW = in->s.W;
            if (kH == 0) kH = in->s.H;
            if (!(kW / 2 >= n->padW && kH / 2 >= n->padH)) { thb_set_error("pad should be smaller than half of kernel size"); return -1; }
        }
        if (dtype == THB_U8 && n->op == OP_AVGPOOL && (n->padH || n->padW || in->q_dyn)) {
            thb_set_error("padded average pooling is not supported in Lowp");
            return -1;
        }
        os.H = pool_out(in->s.H, kH, n->dH, n->padH, n->ceil_mode, n->padH || n->padW);
        os.W = pool_out(in->s.W, kW, n->dW, n->padW, n->ceil_mode, n->padH || n->padW);
        if (os.H < 1 || os.W < 1) { thb_set_error("input image smaller than kernel size"); return -1; }
        materialise(P, out, os);
        out->q_sub = in->q_sub; out->q_mult = in->q_mult; out->q_dyn = in->q_dyn;
        s = new_step(P, n->op == OP_MAXPOOL ? ST_MAXPOOL : ST_AVGPOOL);
        step_in(s, in); step_out(s, out);
        s->N = in->s.N; s->H = in->s.H; s->W = in->s.W; s->C = in->s.C; s->kH = kH; s->kW = kW; s->dH = n->dH; s->dW = n->dW;
        s->padH = n->padH; s->padW = n->padW; s->oH = os.H; s->oW = os.W; s->flag = n->count_include_pad;
        return 0;
    }
    case OP_COMBINE: {
        if (dtype == THB_U8) {
            const value *b = &P->val[n->in[1]];
            int act = -1;
            if (in->q_dyn || b->q_dyn || in->q_sub != b->q_sub || in->q_mult != b->q_mult ||
                in->q_sub != -E->range / 2 || in->s.flat || b->s.flat) {
                thb_set_error("CAddTable in Lowp needs two tensors on the static output quantisation");
                return -1;
            }
            if (b->s.C != in->s.C || b->s.H != in->s.H || b->s.W != in->s.W || b->s.N != in->s.N) {
                thb_set_error("Sum of tensors of different sizes");
                return -1;
            }
            if ((n->coef[0] != 1.f && n->coef[0] != -1.f) || (n->coef[1] != 1.f && n->coef[1] != -1.f)) {
                thb_set_error("only sums and differences are supported in Lowp");
                return -1;
            }
            value *dst = out;
            if ((j = sole_consumer(P, i)) >= 0 && M->nodes[j].op == OP_ACT && M->nodes[j].act_kind == THB_ACT_THRESHOLD) {
                act = j; P->absorbed[j] = 1; P->leader[j] = i; dst = &P->val[j];
            }
            materialise(P, dst, in->s);
            dst->q_sub = in->q_sub; dst->q_mult = in->q_mult;
            s = new_step(P, ST_U8COMBINE);
            step_in(s, in); step_in(s, b); step_out(s, dst);
            s->coef[0] = n->coef[0]; s->coef[1] = n->coef[1];
            s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = in->s.C;
            s->thr = -1; s->val = 0;
            if (act >= 0) {
                s->thr = thb_lowp_scale_float(in->q_sub, in->q_mult, M->nodes[act].act_threshold);
                s->val = thb_lowp_scale_float(in->q_sub, in->q_mult, M->nodes[act].act_value);
            }
            return 0;
        }
        materialise(P, out, in->s);
        s = new_step(P, ST_COMBINE);
        for (int k = 0; k < n->nin; k++) {
            const value *v = &P->val[n->in[k]];
            if (v->s.C != in->s.C || v->s.H != in->s.H || v->s.W != in->s.W || v->s.N != in->s.N) {
                thb_set_error("Sum of tensors of different sizes");
                return -1;
            }
            step_in(s, v);
            s->coef[k] = n->coef[k];
        }
        step_out(s, out);
        s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = in->s.C;
        return 0;
    }
    case OP_CONCAT: {
        /* JoinTable.c:43-44: dimension 1 of a 1-D or 3-D input means dimension 0; only the channel
         * (feature) dimension is supported here */
        int dim = n->dim;
        if (dim == 1 && (in->s.rank == 1 || in->s.rank == 3)) dim--;
        int chan_dim = (in->s.rank == 4 || in->s.rank == 2) ? 1 : 0;
        if (dim == 0 && chan_dim == 1) {
            /* JoinTable.c:46-57 / Concat.c:21-76 along the batch dimension: the inputs' images one after the other */
            if (P->I->slice_n != E->N) { thb_set_error("concatenation along the batch dimension needs the whole batch on one GPU"); return -1; }
            shape os = in->s;
            os.N = 0;
            for (int k = 0; k < n->nin; k++) {
                const value *v = &P->val[n->in[k]];
                if (v->s.rank != in->s.rank || v->s.flat) { thb_set_error("Concatenation of tensors of different dimensionality"); return -1; }
                if (v->s.H != in->s.H || v->s.W != in->s.W || v->s.C != in->s.C) { thb_set_error("Concatenation of tensors of different sizes"); return -1; }
                os.N += v->s.N;
            }
            materialise(P, out, os);
            long img = 0;
            for (int k = 0; k < n->nin; k++) {
                const value *v = &P->val[n->in[k]];
                s = new_step(P, ST_COPY);
                step_in(s, v); step_out(s, out);
                s->pixels = (long)v->s.N * os.H * os.W; s->C = v->s.C;
                s->out_off0 = img * os.H * os.W * out->ld;
                img += v->s.N;
            }
            return 0;
        }
        if (dim != chan_dim) { thb_set_error("concatenation along dimension %d is not supported", n->dim); return -1; }
        shape os = in->s;
        os.C = 0;
        for (int k = 0; k < n->nin; k++) {
            const value *v = &P->val[n->in[k]];
            if (v->s.rank != in->s.rank) { thb_set_error("Concatenation of tensors of different dimensionality"); return -1; }
            if (v->s.H != in->s.H || v->s.W != in->s.W || v->s.N != in->s.N || v->s.flat) {
                thb_set_error("Concatenation of tensors of different sizes");
                return -1;
            }
            if (k < n->nin - 1 && v->s.C % al) {
                thb_set_error("concatenation of %d channels is not aligned to %d", v->s.C, al);
                return -1;
            }
            os.C += v->s.C;
        }
        materialise(P, out, os);
        int coff = 0;
        for (int k = 0; k < n->nin; k++) {
            value *v = &P->val[n->in[k]];
            const int C = v->s.C;
            if (!write_into_slice(P, n->in[k], v, out->buf, out->ld, coff)) {
                s = new_step(P, ST_COPY);
                step_in(s, v); step_out(s, out);
                s->out_coff = coff;
                s->pixels = (long)os.N * os.H * os.W; s->C = C;
            }
            coff += C;
        }
        return 0;
    }
    case OP_SOFTMAX: {
        if (in->s.flat) { thb_set_error("SoftMax on a flattened spatial tensor is not supported"); return -1; }
        materialise(P, out, in->s);
        s = new_step(P, ST_SOFTMAX);
        step_in(s, in); step_out(s, out);
        s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = in->s.C;
        return 0;
    }
    case OP_VIEW: {
        /* View.c:86-97: batch > 1 gives [batch, numElements], otherwise a 1-D tensor */
        long total = (long)in->s.N * in->s.C * in->s.H * in->s.W, per = n->numElements;
        long batch = in->s.rank == 4 || in->s.rank == 2 ? in->s.N : 1;
        if (per == -1) per = total / batch; else batch = total / per;
        if (batch != in->s.N || per * batch != total) { thb_set_error("View to %d elements does not keep the batch dimension", n->numElements); return -1; }
        *out = *in;
        out->s.rank = batch > 1 ? 2 : 1;
        if (in->s.flat) return 0;
        if (in->s.H * in->s.W > 1) {
            /* consumers that are Linear read the channels-innermost data through a permuted weight; anything
             * else (and the network output) gets the data reordered to the NCHW flatten it expects */
            int all_linear = i != M->output;
            for (int k = i + 1; k < M->nnodes && all_linear; k++)
                for (int q = 0; q < M->nodes[k].nin; q++)
                    if (M->nodes[k].in[q] == i && M->nodes[k].op != OP_LINEAR) all_linear = 0;
            if (all_linear && in->coff == 0 && dtype != THB_U8) {
                out->s.flat = 1; out->s.fC = in->s.C; out->s.fH = in->s.H; out->s.fW = in->s.W;
                out->s.C = (int)per; out->s.H = out->s.W = 1;
                return 0;
            }
            if (i == M->output) {
                /* the postprocess kernel emits NCHW order anyway: keep the spatial form, remember the rank */
                out->s.flat = 2;
                return 0;
            }
            shape os = in->s;
            os.C = (int)per; os.H = os.W = 1; os.rank = out->s.rank;
            materialise(P, out, os);
            out->q_sub = in->q_sub; out->q_mult = in->q_mult; out->q_dyn = in->q_dyn;
            s = new_step(P, ST_TO_NCHW);
            step_in(s, in); step_out(s, out);
            s->N = in->s.N; s->H = in->s.H; s->W = in->s.W; s->C = in->s.C;
            return 0;
        }
        out->s.C = (int)per; out->s.H = out->s.W = 1;
        return 0;
    }
    case OP_RESHAPE: {
        /* Reshape.c:22-36: the elements of each image, in the reference's (channel, row, column) order, become a
         * [C, H, W] map.  Without a batch dimension (3-D result) when batchMode is false, or absent while the tensor has
         * exactly numElements elements and its first dimension is not 1; with the input's batch in front otherwise. */
        if (dtype == THB_U8) { thb_set_error("Reshape is not supported in Lowp"); return -1; }
        const int rC = n->reshape[0], rH = n->reshape[1], rW = n->reshape[2];
        const long total = (long)in->s.N * in->s.C * in->s.H * in->s.W, per = (long)rC * rH * rW;
        const int size0 = in->s.rank == 4 || in->s.rank == 2 ? in->s.N : in->s.C;
        const int nonbatch = n->batch_mode == 0 || (n->batch_mode == -1 && total == n->numElements && size0 != 1);
        if (rC < 1 || rH < 1 || rW < 1 || per != n->numElements || per * in->s.N != total || (nonbatch && in->s.N != 1)) {
            thb_set_error("Reshape to %dx%dx%d does not fit %ld elements in %d image(s)", rC, rH, rW, total, in->s.N);
            return -1;
        }
        if (in->s.flat || in->s.H * in->s.W != 1) { thb_set_error("Reshape of a spatial tensor to three dimensions is not supported"); return -1; }
        shape os = in->s;
        os.C = rC; os.H = rH; os.W = rW; os.rank = nonbatch ? 3 : 4;
        materialise(P, out, os);
        s = new_step(P, ST_FROM_NCHW);
        step_in(s, in); step_out(s, out);
        s->N = in->s.N; s->H = rH; s->W = rW; s->C = rC;
        return 0;
    }
    case OP_UPSAMPLE: {
        /* Upsample.c:18-63 */
        if (in->s.rank < 3 || in->s.flat) { thb_set_error("Only 3D and 4D input is supported"); return -1; }
        shape os = in->s;
        os.H *= 2; os.W *= 2;
        materialise(P, out, os);
        s = new_step(P, ST_UPSAMPLE);
        step_in(s, in); step_out(s, out);
        s->N = in->s.N; s->H = in->s.H; s->W = in->s.W; s->C = in->s.C;
        return 0;
    }
    case OP_ZEROPAD: {
        /* SpatialZeroPadding.c:17-60 (negative pads crop) */
        if (in->s.rank < 3 || in->s.flat) { thb_set_error("input dimension must be 3 or 4"); return -1; }
        shape os = in->s;
        os.H = in->s.H + n->pad_t + n->pad_b; os.W = in->s.W + n->pad_l + n->pad_r;
        if (os.H < 1 || os.W < 1) { thb_set_error("zero padding leaves an empty tensor"); return -1; }
        materialise(P, out, os);
        s = new_step(P, ST_ZEROPAD);
        step_in(s, in); step_out(s, out);
        s->N = in->s.N; s->H = in->s.H; s->W = in->s.W; s->C = in->s.C;
        s->padW = n->pad_l; s->kW = n->pad_r; s->padH = n->pad_t; s->kH = n->pad_b;
        return 0;
    }
    case OP_SLICE: {
        /* Slice.c:34-39 + THFloatTensor_slice (thbasic.c:192-209): [from, to) along dimension `axis` of the tensor as the
         * reference ranks it ([N,C,H,W], [C,H,W], [N,C] or [C]) */
        if (in->s.flat) { thb_set_error("Slice of a flattened spatial tensor is not supported"); return -1; }
        const int rank = in->s.rank, ax = n->slice_axis;
        int which = -1; /* 0 batch, 1 channels, 2 rows, 3 columns */
        if (rank == 4) which = ax;
        else if (rank == 3) which = ax + 1;
        else if (rank == 2) which = ax;
        else if (rank == 1) which = ax == 0 ? 1 : -1;
        const int size = which == 0 ? in->s.N : which == 1 ? in->s.C : which == 2 ? in->s.H : which == 3 ? in->s.W : -1;
        if (which < 0 || which > 3 || (rank <= 2 && which > 1) || n->slice_from < 0 || n->slice_to <= n->slice_from || n->slice_to > size) {
            thb_set_error("Slice [%d, %d) along dimension %d does not fit the tensor", n->slice_from, n->slice_to, ax);
            return -1;
        }
        shape os = in->s;
        const int len = n->slice_to - n->slice_from;
        if (which == 1) {
            os.C = len;
            materialise(P, out, os);
            s = new_step(P, ST_SLICEC);
            step_in(s, in); step_out(s, out);
            s->pixels = (long)os.N * os.H * os.W; s->C = len; s->flag = n->slice_from;
        } else if (which == 0) {
            if (P->I->slice_n != E->N) { thb_set_error("a slice along the batch dimension needs the whole batch on one GPU"); return -1; }
            os.N = len;
            materialise(P, out, os);
            s = new_step(P, ST_COPY);
            step_in(s, in); step_out(s, out);
            s->pixels = (long)len * os.H * os.W; s->C = os.C;
            s->in_off0 = (long)n->slice_from * os.H * os.W * in->ld;
        } else {
            if (which == 2) os.H = len; else os.W = len;
            materialise(P, out, os);
            s = new_step(P, ST_ZEROPAD);
            step_in(s, in); step_out(s, out);
            s->N = in->s.N; s->H = in->s.H; s->W = in->s.W; s->C = in->s.C;
            s->padW = which == 3 ? -n->slice_from : 0; s->kW = which == 3 ? n->slice_to - in->s.W : 0;
            s->padH = which == 2 ? -n->slice_from : 0; s->kH = which == 2 ? n->slice_to - in->s.H : 0;
        }
        return 0;
    }
    case OP_CMAX: {
        /* Cmax.c:20-68 (inputs of one shape; the reference also takes shorter later inputs, which nothing here produces) */
        if (n->nin > 8) { thb_set_error("Cmax of %d tensors is not supported", n->nin); return -1; }
        for (int k = 0; k < n->nin; k++) {
            const value *v = &P->val[n->in[k]];
            if (v->s.rank != in->s.rank) { thb_set_error("Cmax of tensors of different dimensionality"); return -1; }
            if (v->s.C != in->s.C || v->s.H != in->s.H || v->s.W != in->s.W || v->s.N != in->s.N || v->s.flat) {
                thb_set_error("Cmax of tensors of different sizes");
                return -1;
            }
        }
        materialise(P, out, in->s);
        s = new_step(P, ST_CMAX);
        for (int k = 0; k < n->nin; k++) step_in(s, &P->val[n->in[k]]);
        step_out(s, out);
        s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = in->s.C;
        return 0;
    }
    case OP_LOGSOFTMAX: {
        if (in->s.flat) { thb_set_error("LogSoftMax on a flattened spatial tensor is not supported"); return -1; }
        if (P->I->slice_n != E->N && !E->strict_math) { thb_set_error("LogSoftMax as the reference computes it needs the whole batch on one GPU"); return -1; }
        materialise(P, out, in->s);
        s = new_step(P, ST_LOGSOFTMAX);
        step_in(s, in); step_out(s, out);
        s->pixels = (long)in->s.N * in->s.H * in->s.W; s->C = in->s.C;
        /* LogSoftMax.c:77 subtracts from the values at the start of the whole input; THB200_STRICT_MATH=1: from each position's own */
        s->flag = !E->strict_math;
        return 0;
    }
    case OP_NORMALIZE: {
        /* Normalize.c:12-44: per row of a 2-D tensor, over the whole tensor (batch included) otherwise */
        if (in->s.flat || in->coff || in->ld != ru(in->s.C, al)) { thb_set_error("Normalize needs a dense tensor"); return -1; }
        const int per_row = in->s.rank == 2;
        if (!per_row && P->I->slice_n != E->N) { thb_set_error("Normalize over a whole batch tensor needs the batch on one GPU"); return -1; }
        materialise(P, out, in->s);
        s = new_step(P, ST_NORMALIZE);
        step_in(s, in); step_out(s, out);
        s->N = in->s.N; s->pixels = (long)in->s.H * in->s.W * in->ld; s->flag = per_row;
        s->aux_buf = new_buf(P, sizeof(float) * (size_t)(in->s.N > 0 ? in->s.N : 1));
        return 0;
    }
    case OP_UNPOOL: {
        /* SpatialMaxUnpooling.c:42-121: input 0 has the size of the pooling's output, the result that of its input */
        const value *xin = &P->val[n->in[1]];
        if (in->s.rank != 3 && in->s.rank != 4) { thb_set_error("3D or 4D (batch mode) tensor is expected"); return -1; }
        if (in->s.flat || xin->s.flat || xin->buf < 0) { thb_set_error("SpatialMaxUnpooling needs spatial tensors"); return -1; }
        const int oH = pool_out(xin->s.H, n->kH, n->dH, n->padH, n->ceil_mode, n->padH || n->padW);
        const int oW = pool_out(xin->s.W, n->kW, n->dW, n->padW, n->ceil_mode, n->padH || n->padW);
        if (in->s.H != oH || in->s.W != oW || in->s.C != xin->s.C || in->s.N != xin->s.N) {
            thb_set_error("Invalid input size w.r.t current indices size");
            return -1;
        }
        shape os = xin->s;
        os.rank = in->s.rank;
        materialise(P, out, os);
        s = new_step(P, ST_UNPOOL);
        step_in(s, in); step_in(s, xin); step_out(s, out);
        s->N = os.N; s->H = os.H; s->W = os.W; s->C = os.C; s->oH = oH; s->oW = oW;
        s->kH = n->kH; s->kW = n->kW; s->dH = n->dH; s->dW = n->dW; s->padH = n->padH; s->padW = n->padW;
        return 0;
    }
    case OP_ALIAS:
        *out = *in;
        return 0;
    }
    thb_set_error("internal: unknown operator %d", n->op);
    return -1;
}

/* liveness-based packing of the activation buffers into one arena */
static size_t pack_arena(instance *I)
{
    for (int t = 0; t < I->nsteps; t++) {
        step *s = &I->steps[t];
        int ids[12], n = 0;
        for (int k = 0; k < s->nin; k++) ids[n++] = s->in_buf[k];
        ids[n++] = s->out_buf;
        ids[n++] = s->aux_buf;
        ids[n++] = s->aux2_buf;
        ids[n++] = s->scratch_buf;
        for (int k = 0; k < n; k++)
            if (ids[k] >= 0) {
                abuf *b = &I->bufs[ids[k]];
                if (b->first < 0) b->first = t;
                b->last = t;
            }
    }
    /* the network input lives from the preprocess launch (before step 0); the output until the postprocess */
    if (I->in_val.buf >= 0) I->bufs[I->in_val.buf].first = -1;
    if (I->out_val.buf >= 0) I->bufs[I->out_val.buf].last = I->nsteps;
    size_t top = 0;
    for (int b = 0; b < I->nbufs; b++) {
        abuf *B = &I->bufs[b];
        if (B->last < 0 && b != I->in_val.buf) { B->offset = 0; continue; }
        size_t off = 0;
        for (;;) {
            int moved = 0;
            for (int o = 0; o < b; o++) {
                abuf *O = &I->bufs[o];
                if (O->last < 0 && o != I->in_val.buf) continue;
                int overlap_time = !(O->last < B->first || B->last < O->first);
                if (overlap_time && off < O->offset + O->bytes && O->offset < off + B->bytes) {
                    off = O->offset + O->bytes;
                    moved = 1;
                }
            }
            if (!moved) break;
        }
        B->offset = off;
        if (off + B->bytes > top) top = off + B->bytes;
    }
    return top;
}

static void instance_free(instance *I)
{
    if (!I->allocs && !I->steps) return;
    for (int i = 0; i < I->nhost; i++) free(I->hostmem[i]);
    free(I->hostmem);
    cudaSetDevice(I->device);
    if (I->stream) cudaStreamSynchronize(I->stream);
    for (int i = 0; i < I->nallocs; i++) cudaFree(I->allocs[i]);
    for (int i = 0; i < I->nsteps; i++) free(I->steps[i].tmap);
    if (I->graph) cudaGraphExecDestroy(I->graph);
    if (I->ev0) cudaEventDestroy(I->ev0);
    if (I->ev1) cudaEventDestroy(I->ev1);
    if (I->ev_wb) cudaEventDestroy(I->ev_wb);
    if (I->wb_stream) cudaStreamDestroy(I->wb_stream);
    if (I->stream) cudaStreamDestroy(I->stream);
    free(I->allocs); free(I->steps); free(I->bufs);
    memset(I, 0, sizeof(*I));
}

static int instance_build(thb_engine *E, instance *I, int device, int slice_off, int slice_n)
{
    thb_model *M = E->model;
    memset(I, 0, sizeof(*I));
    I->device = device; I->slice_off = slice_off; I->slice_n = slice_n;
    CU(cudaSetDevice(device));
    CU(cudaStreamCreateWithFlags(&I->stream, cudaStreamNonBlocking));
    CU(cudaEventCreate(&I->ev0));
    CU(cudaEventCreate(&I->ev1));
    I->d_status = dalloc(I, sizeof(int));
    I->d_minmax = dalloc(I, 2 * sizeof(float));
    if (!I->d_status || !I->d_minmax) return -1;
    CU(cudaMemset(I->d_status, 0, sizeof(int)));

    planner P;
    memset(&P, 0, sizeof(P));
    P.E = E; P.I = I; P.M = M;
    P.val = calloc(M->nnodes, sizeof(value));
    P.uses = calloc(M->nnodes, sizeof(int));
    P.absorbed = calloc(M->nnodes, sizeof(int));
    P.leader = calloc(M->nnodes, sizeof(int));
    for (int i = 0; i < M->nnodes; i++) {
        P.val[i].buf = -1;
        P.leader[i] = i;
        for (int k = 0; k < M->nodes[i].nin; k++) P.uses[M->nodes[i].in[k]]++;
    }
    P.uses[M->output]++;

    shape in = {slice_n, E->C, E->H, E->W, E->rank, 0, 0, 0, 0};
    {
        /* a stride-2 convolution on very few channels as the only consumer of the float input: stage the input
         * space-to-depth so that the gathered 16-byte chunks carry four times as many useful channels */
        thb_node *c1 = M->nnodes > 1 ? &M->nodes[1] : 0;
        const char *off = getenv("THB200_NO_S2D"), *u8off = getenv("THB200_NO_S2D_U8");
        E->input_s2d = c1 && c1->op == OP_CONV && c1->in[0] == 0 && P.uses[0] == 1 && c1->dH == 2 && c1->dW == 2 &&
                       4 * E->C <= 16 && c1->Cin == E->C && E->H % 2 == 0 && E->W % 2 == 0 && E->rank == 4 &&
                       /* a float batch, or three-plane byte images (converted and regrouped by one kernel) in the 16-bit modes */
                       (E->cp == 0 || (E->cp == 3 && E->dtype != THB_U8)) &&
                       (E->dtype == THB_F16 || E->dtype == THB_BF16 || (E->dtype == THB_U8 && !(u8off && atoi(u8off)))) &&
                       c1->padH <= c1->kH - 1 && c1->padW <= c1->kW - 1 &&
                       !(E->honour_pads && (c1->pad2H != c1->padH || c1->pad2W != c1->padW || c1->dlH > 1 || c1->dlW > 1 || c1->autopad || c1->refl_pad)) &&
                       !(off && atoi(off));
        if (E->input_s2d) { in.C = 4 * E->C; in.H = E->H / 2; in.W = E->W / 2; }
    }
    {
        /* A stride-1 convolution with at most 64 output channels on very few input channels (VGG, the segmentation net):
         * with 32-byte pixels it is a case for the patch kernel (one copy per input patch) instead of a gather of
         * 16-byte chunks that are mostly padding. */
        thb_node *c1 = M->nnodes > 1 ? &M->nodes[1] : 0;
        const char *off = getenv("THB200_NO_PAD16");
        E->input_pad16 = !E->input_s2d && c1 && c1->op == OP_CONV && c1->in[0] == 0 && P.uses[0] == 1 && c1->dH == 1 && c1->dW == 1 &&
                         E->C <= 8 && c1->Cin == E->C && c1->Cout <= 64 && c1->kH <= 8 && c1->kW <= 8 && c1->kH * c1->kW > 1 &&
                         c1->padH < c1->kH && c1->padW < c1->kW && (E->dtype == THB_F16 || E->dtype == THB_BF16) &&
                         !(E->honour_pads && (c1->pad2H != c1->padH || c1->pad2W != c1->padW || c1->dlH > 1 || c1->dlW > 1 || c1->autopad || c1->refl_pad)) &&
                         !(off && atoi(off));
    }
    {
        /* uint8: a 3x3 / stride 1 / pad 1 first convolution on three planes of a float batch */
        thb_node *c1 = M->nnodes > 1 ? &M->nodes[1] : 0;
        const char *off = getenv("THB200_NO_NEIGH_U8");
        E->input_neigh = E->dtype == THB_U8 && !E->input_s2d && E->cp == 0 && E->C == 3 && E->rank == 4 && c1 && c1->op == OP_CONV &&
                         c1->in[0] == 0 && P.uses[0] == 1 && c1->Cin == 3 && c1->kH == 3 && c1->kW == 3 && c1->dH == 1 && c1->dW == 1 &&
                         c1->padH == 1 && c1->padW == 1 &&
                         !(E->honour_pads && (c1->pad2H != c1->padH || c1->pad2W != c1->padW || c1->dlH > 1 || c1->dlW > 1 || c1->autopad || c1->refl_pad)) &&
                         !(off && atoi(off));
        if (E->input_neigh) in.C = 27;
    }
    materialise(&P, &P.val[0], in);
    if (E->input_pad16) {
        value *v = &P.val[0];
        v->ld = 16;
        I->nbufs--; /* re-create the buffer with 16 channels per pixel */
        v->buf = new_buf(&P, (size_t)in.N * in.H * in.W * v->ld * esize_of(E->dtype));
    }
    if (E->input_s2d) {
        /* When the rewritten convolution's kernel row fills one 128-byte K block, store the staged rows with their
         * zero padding: one copy then fetches a whole kernel row of an output pixel (thb_conv_desc.in_row_pitch). */
        thb_node *c1 = &M->nodes[1];
        const int padW = (c1->padW + 1) / 2, kW = (c1->kW - 1 - c1->padW) / 2 + padW + 1;
        const char *off = getenv("THB200_NO_PADDED_ROWS");
        value *v = &P.val[0];
        /* (16-bit types only: the uint8 loader and the channel-sum pass write and read dense rows) */
        if (E->dtype != THB_U8 && kW * v->ld * esize_of(E->dtype) == 128 && thb_conv_padded_rows_supported(E->dtype) &&
            !(off && atoi(off))) {
            v->pad_left = padW;
            v->row_pitch = (padW + in.W + kW - 1 + 3) & ~3;
            I->nbufs--; /* re-create the buffer at its padded size */
            v->buf = new_buf(&P, (size_t)in.N * in.H * v->row_pitch * v->ld * esize_of(E->dtype));
        }
    }
    P.val[0].q_dyn = E->dtype == THB_U8;
    int rc = 0;
    for (int i = 1; i < M->nnodes && !rc; i++) {
        if (P.absorbed[i]) continue;
        rc = plan_node(&P, i);
    }
    if (!rc && P.val[M->output].buf < 0) { thb_set_error("internal: the output was not materialised"); rc = -1; }
    if (!rc) {
        I->in_val = P.val[0];
        I->out_val = P.val[M->output];
        I->out_shape = I->out_val.s;
        I->out_count = (long)I->out_shape.N * I->out_shape.C * I->out_shape.H * I->out_shape.W;
        I->arena_bytes = pack_arena(I);
        I->arena = dalloc(I, I->arena_bytes);
        size_t in_bytes = (size_t)slice_n * E->C * E->H * E->W * sizeof(float);
        I->d_in = dalloc(I, in_bytes);
        I->d_img = dalloc(I, (size_t)slice_n * E->H * E->W * 4);
        I->d_out = dalloc(I, (size_t)(I->out_count ? I->out_count : 1) * sizeof(float));
        if (!I->arena || !I->d_in || !I->d_out || !I->d_img) rc = -1;
        /* padded channels are never read as data, but stale NaN/Inf bit patterns would poison the
         * zero-weight products: start from a clean arena */
        if (!rc && cudaMemset(I->arena, 0, I->arena_bytes) != cudaSuccess) { thb_set_error("arena memset failed"); rc = -1; }
    }
    free(P.val); free(P.uses); free(P.absorbed); free(P.leader);
    if (th_debug && !rc)
        fprintf(stderr, "thb200: device %d: %d launches per forward, arena %.1f MiB, %d buffers\n", device, I->nsteps,
                I->arena_bytes / 1048576.0, I->nbufs);
    return rc;
}

static void *bufptr(instance *I, int buf, int coff, int dtype)
{
    return buf < 0 ? 0 : I->arena + I->bufs[buf].offset + (size_t)coff * esize_of(dtype);
}

static int run_steps_ev(thb_engine *E, instance *I, cudaEvent_t *evs, int from, int to)
{
    thb_stream st = I->stream;
    for (int t = from; t < to; t++) {
        step *s = &I->steps[t];
        const int dt = s->dtype;
        void *x0 = bufptr(I, s->in_buf[0], s->in_coff[0], dt);
        if (x0 && s->in_off0) x0 = (char *)x0 + s->in_off0 * esize_of(dt);
        void *y = bufptr(I, s->out_buf, s->out_coff, dt);
        if (y && s->out_off0) y = (char *)y + s->out_off0 * esize_of(dt);
        int rc = 0;
        double t0 = 0;
        if (th_profile) { cudaStreamSynchronize(I->stream); t0 = th_seconds(); }
        switch (s->kind) {
        case ST_CONV: {
            thb_conv_desc *d = &s->conv;
            if (s->dual) d->x2 = bufptr(I, s->in_buf[1], s->in_coff[1], dt);
            else if (s->nin > 1) d->res = bufptr(I, s->in_buf[1], s->in_coff[1], dt);
            if (s->aux_buf >= 0) d->csum = (const int *)bufptr(I, s->aux_buf, 0, THB_U8);
            if (s->aux2_buf >= 0) d->csum_out = (int *)bufptr(I, s->aux2_buf, 0, THB_U8);
            if (s->scratch_buf >= 0) d->splitk_scratch = (float *)bufptr(I, s->scratch_buf, 0, THB_U8);
            rc = s->pool_k ? thb_conv_maxpool_fwd(d, s->pool_k, 2, s->pool_pad, s->pool_oH, s->pool_oW, x0, y, s->out_ld, st)
                           : thb_conv_fwd(d, x0, y, st);
            break;
        }
        case ST_GEMV:
            rc = thb_gemv_fwd(dt, x0, s->N, s->K, s->in_ld[0], s->w, s->M, s->scale, s->shift, &s->act, y, s->out_ld, st);
            break;
        case ST_MAXPOOL:
            rc = thb_maxpool(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], s->kH, s->kW, s->dH, s->dW, s->padH, s->padW, s->oH,
                             s->oW, y, s->out_ld, st);
            break;
        case ST_AVGPOOL:
            rc = thb_avgpool(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], s->kH, s->kW, s->dH, s->dW, s->padH, s->padW, s->oH,
                             s->oW, s->flag, y, s->out_ld, st);
            break;
        case ST_AFFINE:
            rc = thb_affine_act(dt, x0, s->pixels, s->C, s->in_ld[0], s->scale, s->shift, &s->act, y, s->out_ld, st);
            break;
        case ST_U8COMBINE:
            rc = thb_u8_combine(x0, s->in_ld[0], bufptr(I, s->in_buf[1], s->in_coff[1], THB_U8), s->in_ld[1], (int)s->coef[0],
                                (int)s->coef[1], s->thr, s->val, s->pixels, s->C, y, s->out_ld, st);
            break;
        case ST_U8THR:
            rc = thb_u8_threshold(x0, s->pixels, s->C, s->in_ld[0], s->thr, s->val, y, s->out_ld, st);
            break;
        case ST_COMBINE: {
            const void *xs[8];
            for (int k = 0; k < s->nin; k++) xs[k] = bufptr(I, s->in_buf[k], s->in_coff[k], dt);
            rc = thb_combine(dt, s->nin, xs, s->in_ld, s->coef, s->pixels, s->C, y, s->out_ld, st);
            break;
        }
        case ST_COPY:
            rc = thb_copy_channels(dt, x0, s->pixels, s->C, s->in_ld[0], y, s->out_ld, st);
            break;
        case ST_SOFTMAX:
            rc = thb_softmax(dt, x0, s->pixels, s->C, s->in_ld[0], y, s->out_ld, st);
            break;
        case ST_COL2IM:
            rc = thb_col2im(dt, x0, s->N, s->H, s->W, s->C, s->kH, s->kW, s->dH, s->dW, s->padH, s->padW, s->oH, s->oW,
                            s->in_ld[0], s->beta, s->bias, &s->act, y, s->out_ld, st);
            break;
        case ST_ZERO:
            if (s->pixels > 0 && cudaMemsetAsync(bufptr(I, s->out_buf, 0, THB_U8), 0, sizeof(int) * (size_t)s->pixels, (cudaStream_t)st) != cudaSuccess) rc = -1;
            break;
        case ST_CSUM:
            rc = thb_u8_channel_sum(x0, s->pixels, s->C, s->in_ld[0], (int *)bufptr(I, s->out_buf, 0, THB_U8), st);
            break;
        case ST_TO_NCHW:
            rc = thb_to_nchw(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], y, st);
            break;
        case ST_FROM_NCHW:
            rc = thb_from_nchw(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], y, s->out_ld, st);
            break;
        case ST_UPSAMPLE:
            rc = thb_upsample2x(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], y, s->out_ld, st);
            break;
        case ST_ZEROPAD:
            rc = thb_zero_pad(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], s->padW, s->kW, s->padH, s->kH, y, s->out_ld, st);
            break;
        case ST_REFLECTPAD:
            rc = thb_reflect_pad(dt, x0, s->N, s->H, s->W, s->C, s->in_ld[0], s->padW, s->kW, s->padH, s->kH, y, s->out_ld, st);
            break;
        case ST_SLICEC:
            rc = thb_slice_channels(dt, x0, s->pixels, s->flag, s->C, s->in_ld[0], y, s->out_ld, st);
            break;
        case ST_CMAX: {
            const void *xs[8];
            for (int k = 0; k < s->nin; k++) xs[k] = bufptr(I, s->in_buf[k], s->in_coff[k], dt);
            rc = thb_cmax(dt, s->nin, xs, s->in_ld, s->pixels, s->C, y, s->out_ld, st);
            break;
        }
        case ST_LOGSOFTMAX:
            rc = thb_logsoftmax(dt, x0, s->pixels, s->C, s->in_ld[0], y, s->out_ld, s->flag, st);
            break;
        case ST_NORMALIZE:
            rc = thb_l2_normalize(dt, x0, s->N, s->pixels, s->flag, (float *)bufptr(I, s->aux_buf, 0, THB_U8), y, st);
            break;
        case ST_UNPOOL:
            rc = thb_max_unpool(dt, x0, s->in_ld[0], bufptr(I, s->in_buf[1], s->in_coff[1], dt), s->in_ld[1], s->N, s->H, s->W, s->C,
                                s->kH, s->kW, s->dH, s->dW, s->padH, s->padW, s->oH, s->oW, y, s->out_ld, st);
            break;
        }
        if (rc) { thb_set_error("kernel launch %d (kind %d) failed: %d %s", t, s->kind, rc, thb_last_cuda_error()); return -1; }
        if (evs) cudaEventRecord(evs[t + 1], I->stream);
        if (th_minmax && y && s->out_pixels > 0 && s->out_C > 0 && s->kind != ST_ZERO && s->kind != ST_CSUM) {
            /* thapi.c:141-154, :197-202: smallest and largest value of every layer's output -- how a caller picks the
             * lowp range.  A diagnostic: the tensor is read back and scanned on the host (uint8 tensors: their bytes). */
            const size_t es = esize_of(dt), bytes = (size_t)s->out_pixels * s->out_ld * es;
            unsigned char *hb = malloc(bytes ? bytes : 1);
            if (hb && cudaStreamSynchronize(I->stream) == cudaSuccess && cudaMemcpy(hb, y, bytes, cudaMemcpyDeviceToHost) == cudaSuccess) {
                float mn = INFINITY, mx = -INFINITY;
                for (long px = 0; px < s->out_pixels; px++)
                    for (int c = 0; c < s->out_C; c++) {
                        const float v = element_as_float(hb, px * s->out_ld + c, dt);
                        if (v > mx) mx = v;
                        if (v < mn) mn = v;
                    }
                printf("Layer %d output: min=%f, max=%f\n", t + 1, mn, mx);
            }
            free(hb);
        }
        if (th_profile) {
            /* thapi.c:211-233: wall clock per module, GFLOP/s for convolutions (serialises the stream) */
            cudaStreamSynchronize(I->stream);
            double dtm = th_seconds() - t0;
            if (s->kind == ST_CONV && s->flops_node >= 0) {
                thb_node *n = &E->model->nodes[s->flops_node];
                double flops = 2.0 * s->conv.N * s->conv.oH * s->conv.oW * (double)n->Cout * n->Cin * n->kH * n->kW;
                printf("%f seconds for launch %d, %f Gflops/s\n", dtm, t + 1, flops * 1e-9 / dtm);
                th_convtot += dtm; th_convflops += flops;
            } else printf("%f seconds for launch %d\n", dtm, t + 1);
        }
    }
    return 0;
}

/* The launches of one forward on the instance's stream: directly the first time, from then on as a replay of the
 * graph captured from them.  In the uint8 engine the convolutions that read the network input take kernel arguments
 * that change every forward (the input's quantisation is measured per batch, lowp_basic.c:299-321): the launches up to
 * and including the last of them are always issued directly and the graph holds the rest.  THB200_NO_GRAPH=1 and the
 * per-module profile mode launch everything directly. */
static int run_steps(thb_engine *E, instance *I)
{
    if (I->graph_state == 0 && I->runs >= 1) {
        const char *ng = getenv("THB200_NO_GRAPH");
        I->graph_state = -1;
        I->graph_from = 0;
        for (int t = 0; t < I->nsteps; t++)
            if (I->steps[t].kind == ST_CONV && I->steps[t].dyn_quant) I->graph_from = t + 1;
        if (I->graph_from < I->nsteps && !(ng && atoi(ng)) && !th_profile && !th_minmax) {
            cudaGraph_t g = 0;
            if (cudaStreamBeginCapture(I->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                const int l0 = thb_kernel_launch_count();
                const int rc = run_steps_ev(E, I, 0, I->graph_from, I->nsteps);
                I->graph_launches = thb_kernel_launch_count() - l0; /* kernels in the graph (its memset nodes are not launches) */
                thb_count_launches(-I->graph_launches);             /* they have not run yet: the replay below counts them */
                const cudaError_t ce = cudaStreamEndCapture(I->stream, &g);
                if (!rc && ce == cudaSuccess && g && cudaGraphInstantiate(&I->graph, g, 0) == cudaSuccess) I->graph_state = 1;
                if (g) cudaGraphDestroy(g);
                cudaGetLastError();
            }
        }
    }
    I->runs++;
    if (I->graph_state == 1 && !th_profile && !th_minmax) {
        if (I->graph_from && run_steps_ev(E, I, 0, 0, I->graph_from)) return -1;
        if (cudaGraphLaunch(I->graph, I->stream) == cudaSuccess) {
            thb_count_launches(I->graph_launches);
            return 0;
        }
        thb_set_error("graph launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    return run_steps_ev(E, I, 0, 0, I->nsteps);
}

static int lowp_input_range(thb_engine *E, instance *set, int G, int has_x, int cp, int C, int H, int W, const float *mean,
                            const float *std, float *q_sub, float *q_mult);
static int boundary_in(thb_engine *E, instance *I, int has_x, int inplace, int cp, int bgr, int C, int H, int W,
                       const float *mean, const float *std, float q_sub, float q_mult);
static int boundary_out(thb_engine *E, instance *I, float *dst);

/* Per-launch device times of one forward on the first GPU from the batch staged by the last THProcess* call (events
 * around every launch on the launching stream, averaged over `iters` passes).  Entry 0 is the boundary kernel in
 * (NCHW fp32 or HWC bytes -> the engine's layout), entries 1..n the planned launches, entry n+1 the boundary kernel
 * out.  kinds: 0 tensor-core/FFMA convolution, 1 GEMV, 2 any other planned launch, 3 boundary kernel.
 * flops: algorithmic FLOPs of the launch (2 * MACs of the convolution / Linear it computes), 0 otherwise. */
int thb_engine_profile(thb_engine *E, int iters, int max_steps, int *kinds, float *ms, double *flops)
{
    if (!E || !E->built || iters < 1 || (!E->last_has_x && !E->last_cp)) return -1;
    instance *I = &E->inst[0];
    if (cudaSetDevice(I->device) != cudaSuccess) return -1;
    const int total = I->nsteps + 2;
    const int n = total < max_steps ? total : max_steps;
    cudaEvent_t *evs = calloc(total + 1, sizeof(cudaEvent_t));
    for (int t = 0; t <= total; t++) cudaEventCreate(&evs[t]);
    for (int t = 0; t < n; t++) ms[t] = 0;
    int rc = 0;
    for (int it = 0; it < iters && !rc; it++) {
        float q_sub = 0, q_mult = 0;
        rc = lowp_input_range(E, E->inst, 1, E->last_has_x, E->last_cp, E->C, E->H, E->W, E->last_mean, E->last_std, &q_sub, &q_mult);
        cudaEventRecord(evs[0], I->stream);
        if (!rc) rc = boundary_in(E, I, E->last_has_x, 0, E->last_cp, E->last_bgr, E->C, E->H, E->W, E->last_mean, E->last_std, q_sub, q_mult);
        cudaEventRecord(evs[1], I->stream);
        if (!rc) rc = run_steps_ev(E, I, evs + 1, 0, I->nsteps);
        if (!rc) rc = boundary_out(E, I, I->d_out);
        cudaEventRecord(evs[total], I->stream);
        if (cudaStreamSynchronize(I->stream) != cudaSuccess) rc = -1;
        for (int t = 0; t < n && !rc; t++) {
            float m = 0;
            cudaEventElapsedTime(&m, evs[t], evs[t + 1]);
            ms[t] += m / iters;
        }
    }
    for (int t = 0; t < n; t++) {
        kinds[t] = 3;
        flops[t] = 0;
        if (t == 0 || t == total - 1) continue;
        step *s = &I->steps[t - 1];
        kinds[t] = s->kind == ST_CONV ? 0 : s->kind == ST_GEMV ? 1 : 2;
        if (s->flops_node >= 0) {
            thb_node *nd = &E->model->nodes[s->flops_node];
            double pix = s->kind == ST_CONV ? (double)s->conv.N * s->conv.oH * s->conv.oW : (double)s->N;
            if (nd->op == OP_DECONV) pix = (double)s->conv.N * s->conv.H * s->conv.W;
            flops[t] = 2.0 * pix * nd->Cout * nd->Cin * nd->kH * nd->kW + s->flops_extra;
        }
    }
    for (int t = 0; t <= total; t++) cudaEventDestroy(evs[t]);
    free(evs);
    return rc ? -1 : n;
}

/* Algorithmic bytes of each entry of thb_engine_profile: every tensor the launch names counted once (input, output,
 * residual, weights) at the storage type's size; 0 for launches that are neither a convolution nor a GEMV.  The
 * companion of thb_engine_profile's flops for a per-launch "slower of the two roofs" bound. */
int thb_engine_profile_bytes(thb_engine *E, int max_steps, double *bytes)
{
    if (!E || !E->built) return -1;
    instance *I = &E->inst[0];
    const int total = I->nsteps + 2;
    const int n = total < max_steps ? total : max_steps;
    for (int t = 0; t < n; t++) {
        bytes[t] = 0;
        if (t == 0 || t == total - 1) continue;
        step *s = &I->steps[t - 1];
        const double el = s->dtype == THB_F32 ? 4 : s->dtype == THB_U8 ? 1 : 2;
        if (s->kind == ST_CONV) {
            const thb_conv_desc *d = &s->conv;
            const double out = s->pool_k ? (double)d->N * s->pool_oH * s->pool_oW * d->Cout : (double)d->N * d->oH * d->oW * d->Cout;
            const double in_elems = s->dual ? (double)d->N * d->H * d->W * d->cin1 + (double)d->N * d->x2_H * d->x2_W * (d->Cin - d->cin1)
                                            : (double)d->N * d->H * d->W * d->Cin;
            bytes[t] = el * (in_elems + out * (d->res ? 2 : 1) + (double)d->Cout * d->Cin * d->kH * d->kW);
        } else if (s->kind == ST_GEMV) {
            bytes[t] = el * ((double)s->M * s->K + (double)s->N * (s->K + s->M));
        }
    }
    return n;
}

/* ================================================================================================ */
thb_engine *thb_engine_create(thb_model *model, int mode, float lowp_range, int ngpus)
{
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) {
        thb_set_error("no CUDA device: this library has no CPU engine");
        return 0;
    }
    thb_engine *E = calloc(1, sizeof(*E));
    E->model = model;
    model->refs++;
    E->mode = mode;
    E->dtype = mode == THB_MODE_F16 ? THB_F16 : mode == THB_MODE_BF16 ? THB_BF16 : mode == THB_MODE_U8 ? THB_U8 : THB_F32;
    E->range = lowp_range;
    E->ngpus = ngpus < 1 ? 1 : ngpus > ndev ? ndev : ngpus > 8 ? 8 : ngpus;
    const char *sm = getenv("THB200_STRICT_MATH");
    E->strict_math = sm && atoi(sm);
    const char *hp = getenv("THB200_HONOUR_PADS");
    E->honour_pads = hp && atoi(hp);
    /* Operators that look across the images of a batch (a slice or a join along the batch dimension, the whole-tensor
     * Normalize, the reference's LogSoftMax, which reads frame 0 for every frame) keep the batch on one GPU in one piece. */
    for (int i = 0; i < model->nnodes; i++) {
        const thb_node *nd = &model->nodes[i];
        if ((nd->op == OP_SLICE && nd->slice_axis == 0) || (nd->op == OP_CONCAT && nd->dim == 0) || nd->op == OP_NORMALIZE ||
            (nd->op == OP_LOGSOFTMAX && !E->strict_math))
            E->whole_batch = 1;
    }
    if (E->whole_batch) E->ngpus = 1;
    const char *g = getenv("THB200_GATHER");
    E->peer_gather = !(g && !strcmp(g, "host"));
    return E;
}

void thb_engine_destroy(thb_engine *E)
{
    if (!E) return;
    for (int g = 0; g < 8; g++) instance_free(&E->inst[g]);
    for (int g = 0; g < 32; g++) instance_free(&E->pipe[g]);
    thb_host_free_pinned(E->h_out);
    thb_host_free_pinned(E->h_stage);
    thb_model_release(E->model);
    free(E);
}

/* contiguous batch slices, one per GPU; the remainder images go to the lowest ranks */
void thb_slice_batch(int N, int G, int g, int *offset, int *count)
{
    int base = N / G, extra = N % G;
    *count = base + (g < extra ? 1 : 0);
    *offset = g * base + (g < extra ? g : extra);
}

/* The pipelined sub-batches of one GPU's slice of n images: sub-batch c of S.  Up to four of them grow from the first to
 * the last: a small first one starts the kernels sooner, and the copy of each later one still ends before the kernels
 * ahead of it do (ResNet-50 batch 256 in two: 96 + 160 images).  Boundaries in sixteenths of the slice; slices too small
 * for that, and more than four sub-batches, are cut evenly. */
void thb_slice_sub_batches(int n, int S, int c, int *offset, int *count)
{
    static const int cut[5][5] = {{0}, {0, 16}, {0, 6, 16}, {0, 3, 8, 16}, {0, 2, 6, 11, 16}};
    if (S < 1 || S > 4 || n < 8 * S) {
        thb_slice_batch(n, S < 1 ? 1 : S, c, offset, count);
        return;
    }
    *offset = (n * cut[S][c] + 8) / 16;
    *count = (n * cut[S][c + 1] + 8) / 16 - *offset;
}

static int engine_build(thb_engine *E, int N, int C, int H, int W, int rank, int cp)
{
    for (int g = 0; g < 8; g++) instance_free(&E->inst[g]);
    for (int g = 0; g < 32; g++) instance_free(&E->pipe[g]);
    E->built = 0;
    E->pipe_built = 0;
    E->N = N; E->C = C; E->H = H; E->W = W; E->rank = rank; E->cp = cp;
    int G = E->ngpus < N ? E->ngpus : N;
    if (G < 1) G = 1;
    int dev0 = 0;
    const char *d0 = getenv("THB200_DEVICE");
    if (d0) dev0 = atoi(d0);
    for (int g = 0; g < G; g++) {
        int off, n;
        thb_slice_batch(N, G, g, &off, &n);
        if (instance_build(E, &E->inst[g], dev0 + g, off, n)) return -1;
    }
    /* gather target: GPU 0 holds the whole result when peer copies are usable */
    if (G > 1 && E->peer_gather) {
        for (int g = 1; g < G; g++) {
            int can = 0;
            cudaDeviceCanAccessPeer(&can, E->inst[0].device, E->inst[g].device);
            if (!can) E->peer_gather = 0;
        }
        if (E->peer_gather) {
            /* direct copies over NVLink need the access switched on from the sending GPU's side (a second request is
             * answered with cudaErrorPeerAccessAlreadyEnabled, which is fine) */
            for (int g = 1; g < G; g++) {
                cudaSetDevice(E->inst[g].device);
                const cudaError_t pe = cudaDeviceEnablePeerAccess(E->inst[0].device, 0);
                if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) E->peer_gather = 0;
                cudaGetLastError();
            }
        }
        if (E->peer_gather) {
            long total = 0;
            for (int g = 0; g < G; g++) total += E->inst[g].out_count;
            cudaSetDevice(E->inst[0].device);
            E->inst[0].d_out = dalloc(&E->inst[0], (size_t)total * sizeof(float));
            if (!E->inst[0].d_out) return -1;
        }
    }
    E->built = G;
    /* Sub-batches per GPU for pipelined host-input forwards.  Two sub-batches hide about 0.6 of the input copy (measured
     * at ~50 GB/s from pinned memory) and cost every launch's fill and drain a second time (~6 us each, with a margin):
     * worth it for a float batch of ResNet-50 (154 MB, 2.8 ms of copy), not for the same batch as byte images (38 MB).
     * The uint8 engine needs the input range of the whole batch before any kernel can start. */
    const int per_gpu = N / G;
    const double in_mb = (double)per_gpu * (cp ? (double)H * W * cp : (double)C * H * W * 4) / 1e6;
    const double copy_ms = in_mb / 50.0, refill_ms = E->inst[0].nsteps * 0.006 * 1.5 + 0.1;
    E->chunks = E->dtype == THB_U8 || per_gpu < 32 || copy_ms * 0.6 <= refill_ms ? 1 : 2;
    const char *ce = getenv("THB200_CHUNKS");
    if (ce) E->chunks = atoi(ce) < 1 || E->dtype == THB_U8 ? 1 : atoi(ce) > 4 ? 4 : atoi(ce);
    if (E->chunks > per_gpu || E->whole_batch) E->chunks = 1;
    return 0;
}

static int g_chunks_override; /* 0 = the engine's own choice */
void thb_set_pipeline_chunks(int n) { g_chunks_override = n < 0 ? 0 : n > 4 ? 4 : n; }

/* plan instances of the sub-batches (first pipelined forward of this shape with S sub-batches per GPU) */
static int pipe_build(thb_engine *E, int S)
{
    const int G = E->built;
    for (int g = 0; g < 32; g++) instance_free(&E->pipe[g]);
    E->pipe_built = 0;
    for (int g = 0; g < G; g++)
        for (int c = 0; c < S; c++) {
            int off, n;
            thb_slice_sub_batches(E->inst[g].slice_n, S, c, &off, &n);
            if (instance_build(E, &E->pipe[g * S + c], E->inst[g].device, E->inst[g].slice_off + off, n)) return -1;
        }
    E->pipe_built = G * S;
    E->pipe_chunks = S;
    return 0;
}

/* per-forward parameters of a u8 convolution whose input scale is measured on the fly */
static void set_dynamic_quant(instance *I, float in_sub, float in_mult)
{
    for (int t = 0; t < I->nsteps; t++) {
        step *s = &I->steps[t];
        if (s->kind == ST_CONV && s->dyn_quant)
            thb_lowp_gemm_params(s->w_sub, s->w_mult, in_sub, in_mult, s->out_sub, s->out_mult, &s->conv.a_offset,
                                 &s->conv.b_offset, &s->conv.c_offset, &s->conv.c_mult, &s->conv.c_shift);
    }
}

/* The uint8 engine's input range.  A float batch: lowp_basic.c:15-29 takes one range over the WHOLE batch tensor, so
 * the slices' extremes are reduced on the host (one 8-byte read-back per GPU) and every instance's first convolution
 * gets the parameters that follow from it.  Byte images: the loader's range is static (lowp_basic.c:82-131), nothing
 * is measured here. */
static int lowp_input_range(thb_engine *E, instance *set, int G, int has_x, int cp, int C, int H, int W, const float *mean,
                            const float *std, float *q_sub, float *q_mult)
{
    *q_sub = *q_mult = 0;
    if (E->dtype != THB_U8) return 0;
    if (!has_x) {
        if (cp != 3) { thb_set_error("the lowp image loader takes 3-plane images"); return -1; }
        return 0;
    }
    float lo = 0, hi = 0;
    for (int g = 0; g < G; g++) {
        instance *I = &set[g];
        CU(cudaSetDevice(I->device));
        if (thb_minmax_normalized(I->d_in, I->slice_n, C, H, W, mean, std, I->d_minmax, I->stream)) return -1;
        CU(cudaMemcpyAsync(I->h_minmax, I->d_minmax, 2 * sizeof(float), cudaMemcpyDeviceToHost, I->stream));
    }
    for (int g = 0; g < G; g++) {
        instance *I = &set[g];
        CU(cudaSetDevice(I->device));
        CU(cudaStreamSynchronize(I->stream));
        if (I->h_minmax[0] < lo) lo = I->h_minmax[0];
        if (I->h_minmax[1] > hi) hi = I->h_minmax[1];
    }
    *q_sub = lo;
    *q_mult = hi - lo > 0 ? (float)(255.0 / (hi - lo)) : 0;
    for (int g = 0; g < G; g++) set_dynamic_quant(&set[g], *q_sub, *q_mult);
    return 0;
}

/* The boundary kernel in: the staged input (I->d_in: NCHW fp32, or I->d_img: HWC bytes) -> the engine's layout and type. */
static int boundary_in(thb_engine *E, instance *I, int has_x, int inplace, int cp, int bgr, int C, int H, int W,
                       const float *mean, const float *std, float q_sub, float q_mult)
{
    int rc;
    void *in_ptr = bufptr(I, I->in_val.buf, 0, E->dtype);
    if (has_x && E->input_neigh)
        rc = thb_preprocess_neigh_u8(I->d_in, inplace ? I->d_in : 0, I->slice_n, H, W, mean, std, in_ptr, I->in_val.ld, q_sub, q_mult,
                                     I->stream);
    else if (has_x && E->input_s2d && E->dtype == THB_U8)
        rc = thb_preprocess_s2d_u8(I->d_in, inplace ? I->d_in : 0, I->slice_n, C, H, W, mean, std, in_ptr, I->in_val.ld, q_sub,
                                   q_mult, I->stream);
    else if (has_x && E->input_s2d)
        rc = thb_preprocess_s2d_padded(I->d_in, inplace ? I->d_in : 0, I->slice_n, C, H, W, mean, std, E->dtype, in_ptr,
                                       I->in_val.ld, I->in_val.row_pitch ? I->in_val.row_pitch : W / 2,
                                       I->in_val.pad_left, I->stream);
    else if (has_x)
        rc = thb_preprocess(I->d_in, inplace ? I->d_in : 0, I->slice_n, C, H, W, mean, std, E->dtype, in_ptr, I->in_val.ld,
                            q_sub, q_mult, I->stream);
    else if (cp == 2) /* one YUYV frame (THProcessYUYV) */
        rc = E->dtype == THB_U8 ? THB_ERR_UNSUPPORTED
                                : thb_preprocess_yuyv(I->d_img, H, W, mean, std, E->dtype, in_ptr, I->in_val.ld, I->stream);
    else if (E->dtype == THB_U8) {
        rc = thb_preprocess_images_lowp(I->d_img, I->slice_n, H, W, W * cp, bgr, mean, std, in_ptr, I->in_val.ld, &q_sub,
                                        &q_mult, I->stream);
        set_dynamic_quant(I, q_sub, q_mult);
    } else if (E->input_s2d)
        rc = thb_preprocess_images_s2d(I->d_img, I->slice_n, H, W, W * cp, bgr, mean, std, E->dtype, in_ptr, I->in_val.ld,
                                       I->in_val.row_pitch ? I->in_val.row_pitch : W / 2, I->in_val.pad_left, I->stream);
    else
        rc = thb_preprocess_images(I->d_img, I->slice_n, H, W, W * cp, cp, bgr, mean, std, E->dtype, in_ptr,
                                   I->in_val.ld, I->stream);
    if (rc) { thb_set_error("preprocess launch failed: %s", thb_last_cuda_error()); return -1; }
    return 0;
}

/* The boundary kernel out: the network's last tensor -> NCHW fp32 at `dst`. */
static int boundary_out(thb_engine *E, instance *I, float *dst)
{
    const value *ov = &I->out_val;
    float inv = ov->q_mult ? (float)(1.0 / ov->q_mult) : 0;
    if (thb_postprocess(bufptr(I, ov->buf, ov->coff, E->dtype), E->dtype, ov->s.N, ov->s.H, ov->s.W, ov->s.C, ov->ld,
                        ov->q_sub, inv, dst, I->stream)) { thb_set_error("postprocess launch failed"); return -1; }
    return 0;
}

/* Everything one GPU does between its staged input and its NCHW fp32 result, on the instance's stream: the boundary
 * kernel in, the planned launches, the boundary kernel out.  ev0 marks the start of the planned launches.
 * `writeback`: host address the normalised input slice is copied back to (THProcessFloat's in-place side effect), or
 * NULL; `dst`: where the result goes (I->d_out, or this GPU's part of the gathered result). */
static int device_forward(thb_engine *E, instance *I, int has_x, int inplace, int cp, int bgr, int C, int H, int W,
                          const float *mean, const float *std, float q_sub, float q_mult, float *writeback, float *dst)
{
    if (boundary_in(E, I, has_x, inplace, cp, bgr, C, H, W, mean, std, q_sub, q_mult)) return -1;
    if (writeback) {
        /* the normalised values go back to the caller on a stream of their own: the link is full duplex and the forward does
         * not wait for them (the caller does, before THProcessFloat returns) */
        if (!I->wb_stream) {
            CU(cudaStreamCreateWithFlags(&I->wb_stream, cudaStreamNonBlocking));
            CU(cudaEventCreateWithFlags(&I->ev_wb, cudaEventDisableTiming));
        }
        CU(cudaEventRecord(I->ev_wb, I->stream));
        CU(cudaStreamWaitEvent(I->wb_stream, I->ev_wb, 0));
        CU(cudaMemcpyAsync(writeback, I->d_in, (size_t)I->slice_n * C * H * W * sizeof(float), cudaMemcpyDeviceToHost, I->wb_stream));
        I->wb_pending = 1;
    }
    CU(cudaEventRecord(I->ev0, I->stream));
    if (run_steps(E, I)) return -1;
    return boundary_out(E, I, dst);
}

/* 1 when `p` is ordinary (pageable) host memory: a copy from it is staged by the driver at a fraction of the link rate and
 * blocks the calling thread */
static int host_is_pageable(const void *p)
{
    struct cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return 0; }
    return a.type == cudaMemoryTypeUnregistered;
}

/* host-to-host copy by all the host threads OpenMP gives this process (1 MB blocks) */
static void parallel_copy(void *dst, const void *src, size_t bytes)
{
    const size_t blk = (size_t)1 << 20;
    const long nb = (long)((bytes + blk - 1) / blk);
#pragma omp parallel for schedule(static)
    for (long b = 0; b < nb; b++) {
        const size_t o = (size_t)b * blk;
        memcpy((char *)dst + o, (const char *)src + o, bytes - o < blk ? bytes - o : blk);
    }
}

/* The same for planes [p0, p1) of an NCHW float batch (plane p = image p / C, channel p % C, HW floats), normalising the
 * first three channels on the way exactly as the boundary kernels do -- (x - mean) / std, a subtraction and a division in
 * fp32 -- and writing the normalised values back over the caller's planes: THProcessFloat's in-place side effect
 * (thapi.c:396-403) done where the reference does it, on the host, instead of a 12-bytes-per-pixel copy back from the
 * device. */
static void stage_planes_normalised(float *dst, float *src, long p0, long p1, int C, long HW, const float *mean, const float *std)
{
#pragma omp parallel for schedule(static)
    for (long p = p0; p < p1; p++) {
        const int c = (int)(p % C);
        float *s = src + p * HW, *d = dst + p * HW;
        if (c < 3) {
            const float m = mean[c], sd = std[c];
            for (long i = 0; i < HW; i++) {
                const float v = (s[i] - m) / sd;
                s[i] = v;
                d[i] = v;
            }
        } else
            memcpy(d, s, (size_t)HW * sizeof(float));
    }
}

int thb_engine_forward(thb_engine *E, float *x, unsigned char **images, int stride, int bgr, int cp, int N, int C, int H,
                       int W, int rank, const float *mean, const float *std, int inplace, thb_result *res)
{
    if (N < 1 || C < 1 || H < 1 || W < 1) { thb_set_error("empty input"); return -1; }
    if (E->dtype == THB_U8 && !x) rank = 4; /* the lowp image loader always builds a 4-D tensor (lowp_basic.c:87-92) */
    if (!E->built || E->N != N || E->C != C || E->H != H || E->W != W || E->rank != rank || E->cp != cp) {
        if (engine_build(E, N, C, H, W, rank, cp)) return -1;
    }
    /* host input (a float batch or byte images): run the sub-batch instances so that copies and kernels overlap */
    instance *set = E->inst;
    int G = E->built;
    int peer_gather = E->peer_gather;
    int S = g_chunks_override ? g_chunks_override : E->chunks;
    if (E->dtype == THB_U8 || S > E->inst[0].slice_n || E->whole_batch) S = 1;
    if (S > 1) {
        if ((!E->pipe_built || E->pipe_chunks != S) && pipe_build(E, S)) return -1;
        set = E->pipe;
        G = E->pipe_built;
    }
    /* Peer gather: every GPU's part of the result ends up in GPU 0's result buffer (the first instance's, sized for the
     * whole batch), which goes to the host in one copy.  Instances on GPU 0 write their part there directly; the others
     * send theirs with cudaMemcpyPeerAsync on their own stream -- also when a GPU's slice runs as pipelined sub-batches. */
    float *gather = E->built > 1 && peer_gather ? E->inst[0].d_out : 0;
    const int dev0 = E->inst[0].device;
    const size_t img_elems = (size_t)C * H * W;
    float q_sub = 0, q_mult = 0;

    long total = 0;
    for (int g = 0; g < G; g++) total += set[g].out_count;
    if ((size_t)total * sizeof(float) > E->h_out_bytes) {
        thb_host_free_pinned(E->h_out);
        E->h_out_bytes = (size_t)total * sizeof(float);
        E->h_out = thb_host_alloc_pinned(E->h_out_bytes);
        if (!E->h_out) { thb_set_error("pinned result allocation failed"); return -1; }
    }
    /* A float batch in pageable memory (what a caller of the reference passes) goes through a pinned buffer of the
     * library, filled slice by slice by the host's threads, so that the copy to the device runs at link speed and under
     * the previous slice's kernels (THB200_NO_STAGING=1: hand the caller's pointer to the driver as it is). */
    int staged = 0;
    const size_t in_bytes = x ? (size_t)N * img_elems * sizeof(float) : (size_t)N * H * W * cp;
    if (in_bytes >= ((size_t)8 << 20) && (x || (size_t)stride == (size_t)W * cp) && host_is_pageable(x ? (const void *)x : images[0])) {
        const char *ns = getenv("THB200_NO_STAGING");
        staged = !(ns && atoi(ns));
        if (staged && in_bytes > E->h_stage_bytes) {
            thb_host_free_pinned(E->h_stage);
            E->h_stage_bytes = in_bytes;
            E->h_stage = thb_host_alloc_pinned(E->h_stage_bytes);
            if (!E->h_stage) { E->h_stage_bytes = 0; staged = 0; }
        }
    }
    /* A staged float batch that is to be normalised in place is normalised by the host threads while they stage it: the
     * device then gets normalised values (identity statistics from here on) and copies nothing back. */
    static const float zero3[3] = {0, 0, 0}, one3[3] = {1, 1, 1};
    const float *host_mean = mean, *host_std = std;
    const int host_norm = staged && x && inplace;
    if (host_norm) { mean = zero3; std = one3; inplace = 0; }
    /* what the device-resident timing loop needs to repeat this forward from the staged input */
    E->last_has_x = x != 0; E->last_cp = cp; E->last_bgr = bgr;
    for (int k = 0; k < 3; k++) { E->last_mean[k] = mean[k]; E->last_std[k] = std[k]; }

    /* The uint8 engine needs the input range of the whole batch before any kernel can start: it stages every slice, then
     * measures, then launches.  The other modes launch a slice's kernels as soon as its copy is queued. */
    const int two_phase = E->dtype == THB_U8;
    cudaEvent_t ev_call = 0;
    if (th_debug > 1 && cudaSetDevice(set[0].device) == cudaSuccess && cudaEventCreate(&ev_call) == cudaSuccess)
        cudaEventRecord(ev_call, set[0].stream);
    for (int phase = 0; phase < 2; phase++) {
        if (phase == 1) {
            if (!two_phase) break;
            if (lowp_input_range(E, set, G, x != 0, cp, C, H, W, mean, std, &q_sub, &q_mult)) return -1;
        }
        for (int g = 0; g < G; g++) {
            instance *I = &set[g];
            CU(cudaSetDevice(I->device));
            if (phase == 0) {
                /* stage the input slice */
                if (x) {
                    const size_t bytes = (size_t)I->slice_n * img_elems * sizeof(float);
                    const float *src = x + (size_t)I->slice_off * img_elems;
                    if (staged) {
                        /* in pieces of about 16 MB (whole planes): the copy to the device of one piece runs while the host
                         * threads fill the next */
                        float *st = E->h_stage + (size_t)I->slice_off * img_elems;
                        float *xs = x + (size_t)I->slice_off * img_elems;
                        const long HW = (long)H * W, planes = (long)I->slice_n * C;
                        long per_piece = (((long)16 << 20) / (long)sizeof(float)) / HW;
                        if (per_piece < 1) per_piece = 1;
                        for (long p0 = 0; p0 < planes; p0 += per_piece) {
                            const long p1 = p0 + per_piece < planes ? p0 + per_piece : planes;
                            const size_t o = (size_t)p0 * HW, cnt = (size_t)(p1 - p0) * HW;
                            if (host_norm) stage_planes_normalised(st, xs, p0, p1, C, HW, host_mean, host_std);
                            else parallel_copy(st + o, xs + o, cnt * sizeof(float));
                            CU(cudaMemcpyAsync(I->d_in + o, st + o, cnt * sizeof(float), cudaMemcpyHostToDevice, I->stream));
                        }
                    } else
                        CU(cudaMemcpyAsync(I->d_in, src, bytes, cudaMemcpyHostToDevice, I->stream));
                } else if ((size_t)stride == (size_t)W * cp) {
                    /* tightly packed rows: one copy per run of images that also follow one another in host memory */
                    const size_t img_bytes = (size_t)H * W * cp;
                    for (int n = 0; n < I->slice_n;) {
                        int run = 1;
                        while (n + run < I->slice_n && images[I->slice_off + n + run] == images[I->slice_off + n + run - 1] + img_bytes) run++;
                        const unsigned char *src = images[I->slice_off + n];
                        if (staged) {
                            unsigned char *st = (unsigned char *)E->h_stage + (size_t)(I->slice_off + n) * img_bytes;
                            parallel_copy(st, src, (size_t)run * img_bytes);
                            src = st;
                        }
                        CU(cudaMemcpyAsync(I->d_img + (size_t)n * img_bytes, src, (size_t)run * img_bytes, cudaMemcpyHostToDevice, I->stream));
                        n += run;
                    }
                } else {
                    for (int n = 0; n < I->slice_n; n++)
                        CU(cudaMemcpy2DAsync(I->d_img + (size_t)n * H * W * cp, (size_t)W * cp, images[I->slice_off + n], stride,
                                             (size_t)W * cp, H, cudaMemcpyHostToDevice, I->stream));
                }
                if (two_phase) continue;
            }
            long off = 0;
            for (int k = 0; k < g; k++) off += set[k].out_count;
            float *dst = gather && I->device == dev0 ? gather + off : I->d_out;
            if (device_forward(E, I, x != 0, inplace, cp, bgr, C, H, W, mean, std, q_sub, q_mult,
                               x && inplace ? x + (size_t)I->slice_off * img_elems : 0, dst)) return -1;
            CU(cudaEventRecord(I->ev1, I->stream));
            if (gather) {
                if (I->device != dev0)
                    CU(cudaMemcpyPeerAsync(gather + off, dev0, I->d_out, I->device, (size_t)I->out_count * sizeof(float), I->stream));
            } else
                CU(cudaMemcpyAsync(E->h_out + off, I->d_out, (size_t)I->out_count * sizeof(float), cudaMemcpyDeviceToHost, I->stream));
        }
    }
    float ms_max = 0;
    for (int g = G - 1; g >= 0; g--) {
        instance *I = &set[g];
        CU(cudaSetDevice(I->device));
        /* every other stream has been waited for by now: the gathered result is complete */
        if (g == 0 && gather)
            CU(cudaMemcpyAsync(E->h_out, gather, (size_t)total * sizeof(float), cudaMemcpyDeviceToHost, I->stream));
        CU(cudaStreamSynchronize(I->stream));
        if (I->wb_pending) {
            CU(cudaStreamSynchronize(I->wb_stream));
            I->wb_pending = 0;
        }
        float ms = 0;
        cudaEventElapsedTime(&ms, I->ev0, I->ev1);
        if (ev_call && I->device == set[0].device) {
            /* debug level 2: when each sub-batch's planned launches began and ended, from the start of the call */
            float a = 0, b = 0;
            cudaEventElapsedTime(&a, ev_call, I->ev0);
            cudaEventElapsedTime(&b, ev_call, I->ev1);
            fprintf(stderr, "thb200: sub-batch %d (%d images): launches from %.3f to %.3f ms\n", g, I->slice_n, a, b);
        }
        I->last_ms = ms;
        if (ms > ms_max) ms_max = ms;
        int status = 0;
        CU(cudaMemcpy(&status, I->d_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (status) {
            cudaMemset(I->d_status, 0, sizeof(int));
            thb_set_error("a device-side wait timed out (code %d) on device %d", status, I->device);
            return -1;
        }
    }
    E->last_ms = ms_max;
    if (ev_call) cudaEventDestroy(ev_call);

    shape os = set[0].out_shape;
    res->data = E->h_out;
    res->count = total;
    int rk = os.rank;
    if (os.flat == 2) { /* a trailing View over a spatial tensor: rank from the View, data already in NCHW order */
        res->ndim = rk;
        if (rk == 2) { res->size[0] = N; res->size[1] = total / N; }
        else res->size[0] = total;
        return 0;
    }
    res->ndim = rk;
    switch (rk) {
    case 4: res->size[0] = N; res->size[1] = os.C; res->size[2] = os.H; res->size[3] = os.W; break;
    case 3: res->size[0] = os.C; res->size[1] = os.H; res->size[2] = os.W; break;
    case 2: res->size[0] = N; res->size[1] = os.C; break;
    default: res->size[0] = os.C; break;
    }
    return 0;
}

float thb_engine_last_ms(thb_engine *E) { return E ? E->last_ms : -1.f; }

/* Device-resident timing loop: the whole forward from the batch staged in device memory by the last THProcess* call
 * (NCHW fp32 or HWC bytes) to the NCHW fp32 result in device memory -- boundary kernels, the uint8 engine's input
 * range (with its 8-byte read-back) and the planned launches -- `iters` times back to back per GPU, timed with events
 * on the launching stream; max over GPUs.  No host<->device copy of the batch or the result is inside. */
float thb_engine_time_forward(thb_engine *E, int iters)
{
    if (!E || !E->built || iters < 1 || (!E->last_has_x && !E->last_cp)) return -1.f;
    const int G = E->built;
    cudaEvent_t t0[8], t1[8];
    for (int g = 0; g < G; g++) {
        if (cudaSetDevice(E->inst[g].device) != cudaSuccess) return -1.f;
        cudaEventCreate(&t0[g]);
        cudaEventCreate(&t1[g]);
        cudaEventRecord(t0[g], E->inst[g].stream);
    }
    int rc = 0;
    for (int it = 0; it < iters && !rc; it++) {
        float q_sub = 0, q_mult = 0;
        rc = lowp_input_range(E, E->inst, G, E->last_has_x, E->last_cp, E->C, E->H, E->W, E->last_mean, E->last_std, &q_sub, &q_mult);
        for (int g = 0; g < G && !rc; g++) {
            instance *I = &E->inst[g];
            if (cudaSetDevice(I->device) != cudaSuccess) rc = -1;
            else rc = device_forward(E, I, E->last_has_x, 0, E->last_cp, E->last_bgr, E->C, E->H, E->W, E->last_mean, E->last_std,
                                     q_sub, q_mult, 0, I->d_out);
        }
    }
    float worst = 0;
    for (int g = 0; g < G; g++) {
        instance *I = &E->inst[g];
        cudaSetDevice(I->device);
        cudaEventRecord(t1[g], I->stream);
        if (cudaStreamSynchronize(I->stream) != cudaSuccess) rc = -1;
        float ms = 0;
        if (!rc) cudaEventElapsedTime(&ms, t0[g], t1[g]);
        if (ms > worst) worst = ms;
        cudaEventDestroy(t0[g]);
        cudaEventDestroy(t1[g]);
    }
    return rc ? -1.f : worst / iters;
}
