/*
 * The public thnets API on top of the B200 engine (reference thapi.c:237-796).
 *
 * Same entry points, argument meaning, ownership and error conventions as the reference:
 *   - THLoadNetwork returns NULL and sets THLastError() on a load failure (thapi.c:244-333);
 *   - THProcessFloat normalises the CALLER's buffer in place, (x - mean)/std (thapi.c:396-403), and
 *     returns a pointer into network-owned memory that stays valid until the next call (thapi.c:443-449);
 *   - THCreateCudaNetwork / THCreateLowpNetwork return a new handle that owns everything it needs, the
 *     source may be freed at once (thnets-test.c:128-149); half precision is the process-wide switch
 *     THCudaHalfFloat, read at conversion time (thapi.c:744-755);
 *   - anything else that goes wrong is fatal: message on stderr and exit(-1) (thbasic.c:172-181), unless
 *     THB200_NO_EXIT=1 is set, in which case the call returns 0 / NULL and THB200_LastErrorString() tells why.
 * What differs: every forward pass runs on the GPU, also for a network that was never converted
 * (fp32 mode) and for PyTorch-dump networks, which the reference cannot convert at all.
 */
#include <math.h>
#include <stdarg.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include <strings.h>
#include "thb_internal.h"

static int lasterror;
static int g_half_mode;  /* THCudaHalfFloat / THB200_SetPrecision */
static int g_ngpus = 1;  /* THB200_SetDevices */

static int fatal_or(int rc)
{
    const char *ne = getenv("THB200_NO_EXIT");
    if (!(ne && atoi(ne))) THError("%s", thb_engine_error());
    return rc;
}

static thb_netx *netx(THNETWORK *n)
{
    thb_netx *x = (thb_netx *)n;
    if (!n || x->magic != THB_NETX_MAGIC) THError("this THNETWORK was not created by this library");
    return x;
}

void THInit(void)
{
    static int done;
    if (done) return;
    done = 1;
    const char *g = getenv("THB200_GPUS");
    if (g && atoi(g) > 0) g_ngpus = atoi(g);
    const char *p = getenv("THB200_PRECISION");
    if (p) g_half_mode = !strcasecmp(p, "fp16") ? 1 : !strcasecmp(p, "bf16") ? 2 : 0;
}

int THLastError(void) { return lasterror; }
const char *THB200_LastErrorString(void) { return thb_engine_error(); }
int THB200_KernelLaunches(void) { return thb_kernel_launch_count(); }

int THCudaHalfFloat(int enable)
{
    g_half_mode = enable ? 1 : 0;
    return 0;
}
int THB200_SetPrecision(int mode)
{
    if (mode < 0 || mode > 2) return ERR_NOTIMPLEMENTED;
    g_half_mode = mode;
    return 0;
}
int THB200_SetPipelineChunks(int chunks)
{
    thb_set_pipeline_chunks(chunks);
    return 0;
}

int THB200_SetDevices(int ngpus)
{
    if (ngpus < 1 || ngpus > 8) return ERR_NOTIMPLEMENTED;
    g_ngpus = ngpus;
    return 0;
}
int THOpenCLHalfFloat(int enable) { (void)enable; return ERR_NOTIMPLEMENTED; }
THNETWORK *THCreateOpenCLNetwork(THNETWORK *net) { (void)net; return 0; }
void *THB200_HostAlloc(size_t bytes) { return thb_host_alloc_pinned(bytes); }
void THB200_HostFree(void *p) { thb_host_free_pinned(p); }

/* ------------------------------------------------------------------------------------------------ loading */
THNETWORK *THLoadNetwork(const char *path)
{
    char tmp[1024];
    thb_netx *x = calloc(1, sizeof(*x));
    THNETWORK *net = &x->pub;
    x->magic = THB_NETX_MAGIC;
    x->owns_graph = 1;
    for (int i = 0; i < 3; i++) net->std[i] = 1;
    lasterror = 0;

    net->allpynodes = calloc(MAXPYNODES, sizeof(*net->allpynodes));
    /* 0. an ONNX model, by the file name's ending (thapi.c:254-262); the result is held as a graph-dump network */
    {
        size_t n = strlen(path);
        if ((n > 3 && !strcasecmp(path + n - 3, ".pb")) || (n > 6 && !strcasecmp(path + n - 6, ".proto")) ||
            (n > 5 && !strcasecmp(path + n - 5, ".onnx"))) {
            char why[256] = "";
            net->pynet = loadonnx(path, net->allpynodes, why, sizeof(why));
            if (net->pynet) return net;
            if (*why) thb_set_error("%s: %s", path, why);
            memset(net->allpynodes, 0, MAXPYNODES * sizeof(*net->allpynodes));
        }
    }
    /* 1. a PyTorch graph dump, either the file itself or <path>/pymodel.net (thapi.c:264-271) */
    net->pynet = loadpytorch(path, net->allpynodes);
    if (!net->pynet) {
        snprintf(tmp, sizeof(tmp), "%s/pymodel.net", path);
        net->pynet = loadpytorch(tmp, net->allpynodes);
    }
    if (net->pynet) return net;
    free(net->allpynodes);
    net->allpynodes = 0;

    /* 2. a Torch7 directory: model.net (+ optional stat.t7 with mean / std) */
    int longsize = 8;
    snprintf(tmp, sizeof(tmp), "%s/model.net", path);
    net->netobj = malloc(sizeof(*net->netobj));
    lasterror = loadtorch(tmp, net->netobj, longsize);
    if (lasterror == ERR_CORRUPTED) lasterror = loadtorch(tmp, net->netobj, longsize = 4);
    if (lasterror) goto fail_obj;
    if (net->netobj->type != TYPE_NNMODULE) { lasterror = ERR_WRONGOBJECT; freeobject(net->netobj); goto fail_obj; }
    net->net = Module2Network(net->netobj->nnmodule);
    if (!net->net) { lasterror = ERR_WRONGOBJECT; freeobject(net->netobj); goto fail_obj; }

    snprintf(tmp, sizeof(tmp), "%s/stat.t7", path);
    net->statobj = malloc(sizeof(*net->statobj));
    int rc = loadtorch(tmp, net->statobj, longsize);
    if (rc) {
        free(net->statobj);
        net->statobj = 0;
    } else {
        struct thobject *st = net->statobj;
        if (st->type != TYPE_TABLE || st->table->nelem != 2) {
            lasterror = ERR_WRONGOBJECT;
            freenetwork(net->net);
            freeobject(net->netobj);
            freeobject(st);
            free(st);
            goto fail_obj;
        }
        for (int i = 0; i < st->table->nelem; i++) {
            struct threcord *r = &st->table->records[i];
            if (r->name.type != TYPE_STRING || r->value.type != TYPE_TENSOR || !r->value.tensor->storage) continue;
            float *dst = !strcmp(r->name.string.data, "mean") ? net->mean : !strcmp(r->name.string.data, "std") ? net->std : 0;
            if (dst && r->value.tensor->storage->nelem >= 3) memcpy(dst, r->value.tensor->storage->data, 3 * sizeof(float));
        }
    }
    THUseSpatialConvolutionMM(net, 2);
    return net;

fail_obj:
    free(net->netobj);
    free(x);
    return 0;
}

void THFreeNetwork(THNETWORK *network)
{
    thb_netx *x = netx(network);
    if (x->engine) thb_engine_destroy(x->engine);
    if (x->owns_graph) {
        if (network->pynet) freepynet(network->pynet);
        free(network->allpynodes);
        if (network->net) freenetwork(network->net);
        if (network->netobj) { freeobject(network->netobj); free(network->netobj); }
        if (network->statobj) { freeobject(network->statobj); free(network->statobj); }
    } else if (network->net) {
        free(network->net); /* the shell of a converted network */
    }
    if (network->out) THFloatTensor_free(network->out);
    x->magic = 0;
    free(x);
}

/* thapi.c:692-728: only the module type tags change here; there is one convolution algorithm on the device */
int THUseSpatialConvolutionMM(THNETWORK *network, int mm_type)
{
    if (!network->net) return ERR_NOTIMPLEMENTED;
    int rc = 0;
    for (int i = 0; i < network->net->nelem; i++) {
        struct module *m = &network->net->modules[i];
        if (mm_type && m->type == MT_SpatialConvolution) m->type = MT_SpatialConvolutionMM;
        else if (!mm_type && (m->type == MT_SpatialConvolutionMM || m->type == MT_SpatialConvolutionVirtMM)) {
            if (m->SpatialConvolution.padW || m->SpatialConvolution.padH) { rc = ERR_NOTIMPLEMENTED; continue; }
            m->type = MT_SpatialConvolution;
        }
        if (mm_type == 2 && m->type == MT_SpatialConvolutionMM) m->type = MT_SpatialConvolutionVirtMM;
        else if (mm_type == 1 && m->type == MT_SpatialConvolutionVirtMM) m->type = MT_SpatialConvolutionMM;
    }
    return rc;
}

/*
 * thapi.c:642-690: make a classifier slide over larger images.  `size` is the spatial size of the INPUT the
 * classifier was trained for; it is tracked through convolutions and poolings.  View / Reshape modules
 * vanish and every Linear becomes a size x size convolution (1 x 1 after the first).
 */
void THMakeSpatial(THNETWORK *network, int size)
{
    thb_netx *x = netx(network);
    struct network *net = network->net;
    if (!net) { thb_set_error("THMakeSpatial needs a Torch7 network"); return; }
    int planes = 3;
    for (int i = 0; i < net->nelem; i++) {
        struct module *m = &net->modules[i];
        switch (m->type) {
        case MT_View: case MT_Reshape:
            THFloatTensor_free(m->output);
            memmove(m, m + 1, sizeof(*m) * (net->nelem - i - 1));
            net->nelem--;
            i--;
            break;
        case MT_Linear: {
            THFloatTensor *w = m->Linear.weight, *b = m->Linear.bias;
            THFloatTensor_free(m->Linear.addBuffer);
            struct SpatialConvolution *c = &m->SpatialConvolution;
            memset(c, 0, sizeof(*c));
            m->type = MT_SpatialConvolutionVirtMM;
            c->bias = b; c->weight = w; c->finput = THFloatTensor_new();
            c->dW = c->dH = 1;
            c->kW = c->kH = size;
            c->nInputPlane = planes;
            planes = c->nOutputPlane = (int)w->size[0];
            size = 1;
            break;
        }
        case MT_SpatialConvolution: case MT_SpatialConvolutionMM: case MT_SpatialConvolutionVirtMM: {
            struct SpatialConvolution *c = &m->SpatialConvolution;
            size = (size + 2 * c->padW - c->kW) / c->dW + 1;
            planes = c->nOutputPlane;
            break;
        }
        case MT_SpatialMaxPooling: {
            struct SpatialMaxPooling *p = &m->SpatialMaxPooling;
            float q = (float)(size - p->kH + 2 * p->padH) / p->dH;
            size = (int)(p->ceil_mode ? ceilf(q) : floorf(q)) + 1;
            break;
        }
        case MT_SpatialZeroPadding:
            size += m->SpatialZeroPadding.pad_l + m->SpatialZeroPadding.pad_r;
            break;
        }
    }
    if (x->engine) { thb_engine_destroy(x->engine); x->engine = 0; }
}

/* ------------------------------------------------------------------------------------------------ conversion */
static THNETWORK *convert(THNETWORK *src, int mode, float range, int engine_tag)
{
    char err[256] = "";
    THInit();
    thb_model *model = thb_model_from_network(src, err, sizeof(err));
    if (!model) { thb_set_error("%s", err); fatal_or(0); return 0; }
    thb_netx *x = calloc(1, sizeof(*x));
    x->magic = THB_NETX_MAGIC;
    x->pub = *src;
    x->pub.netobj = x->pub.statobj = 0;
    x->pub.pynet = 0;
    x->pub.allpynodes = 0;
    x->pub.out = 0;
    x->pub.net = calloc(1, sizeof(struct network)); /* shell: callers read net->engine */
    x->pub.net->engine = engine_tag;
    x->mode = mode;
    x->lowp_range = range;
    x->engine = thb_engine_create(model, mode, range, g_ngpus);
    thb_model_release(model);
    if (!x->engine) { free(x->pub.net); free(x); fatal_or(0); return 0; }
    return &x->pub;
}

THNETWORK *THCreateCudaNetwork(THNETWORK *net) { return convert(net, g_half_mode, 0, ENGINE_CUDA); }

THNETWORK *THCreateLowpNetwork(THNETWORK *net, float range)
{
    if (!(range > 0)) { thb_set_error("the lowp range must be positive"); fatal_or(0); return 0; }
    return convert(net, THB_MODE_U8, range, ENGINE_LOWP);
}

static int ensure_engine(thb_netx *x)
{
    if (x->engine) return 0;
    char err[256] = "";
    THInit();
    thb_model *model = thb_model_from_network(&x->pub, err, sizeof(err));
    if (!model) { thb_set_error("%s", err); return -1; }
    x->engine = thb_engine_create(model, THB_MODE_F32, 0, g_ngpus);
    thb_model_release(model);
    return x->engine ? 0 : -1;
}

/* ------------------------------------------------------------------------------------------------ forward */
static int publish(THNETWORK *network, const thb_result *r, float **result, int *outwidth, int *outheight)
{
    if (network->out) THFloatTensor_free(network->out);
    THFloatTensor *t = network->out = THFloatTensor_new();
    t->nDimension = r->ndim;
    long stride = 1;
    for (int i = r->ndim - 1; i >= 0; i--) {
        t->size[i] = r->size[i];
        t->stride[i] = stride;
        stride *= r->size[i];
    }
    t->storage = THFloatStorage_newwithbuffer(r->data);
    if (result) *result = r->data;
    if (outwidth && outheight) {
        if (r->ndim >= 3) {
            *outwidth = (int)r->size[r->ndim - 1];
            *outheight = (int)r->size[r->ndim - 2];
        } else
            *outwidth = *outheight = 1;
    }
    return (int)r->count;
}

int THProcessFloat(THNETWORK *network, float *data, int batchsize, int width, int height, int nplanes, float **result,
                   int *outwidth, int *outheight)
{
    thb_netx *x = netx(network);
    thb_result r;
    if (ensure_engine(x)) return fatal_or(0);
    /* the reference leaves the normalised values in the caller's buffer; identity statistics need no write-back */
    int trivial = 1;
    for (int c = 0; c < 3; c++)
        if (network->mean[c] != 0 || network->std[c] != 1) trivial = 0;
    const char *keep = getenv("THB200_KEEP_INPUT");
    int inplace = !trivial && !(keep && atoi(keep));
    if (thb_engine_forward(x->engine, data, 0, 0, 0, 0, batchsize, nplanes, height, width, 4, network->mean, network->std,
                           inplace, &r))
        return fatal_or(0);
    return publish(network, &r, result, outwidth, outheight);
}

int THProcessImages(THNETWORK *network, unsigned char **images, int batchsize, int width, int height, int stride,
                    float **result, int *outwidth, int *outheight, int bgr)
{
    thb_netx *x = netx(network);
    thb_result r;
    int cp = stride < width * 3 ? 1 : 3; /* thapi.c:458-459 */
    if (ensure_engine(x)) return fatal_or(0);
    if (thb_engine_forward(x->engine, 0, images, stride, bgr, cp, batchsize, cp, height, width, batchsize == 1 ? 3 : 4,
                           network->mean, network->std, 0, &r))
        return fatal_or(0);
    return publish(network, &r, result, outwidth, outheight);
}

int THProcessYUYV(THNETWORK *network, unsigned char *image, int width, int height, float **results, int *outwidth,
                  int *outheight)
{
    /* thapi.c:575-612: one YUYV frame -> a 3 x height x width tensor (yuyv2fRGB with the network's mean / std) -> forward.
     * The reference refuses this entry point on its converted (cuDNN, OpenCL, lowp) networks and so does this library;
     * a network as THLoadNetwork returned it takes the frame: the bytes are copied as they are and converted on the GPU. */
    thb_netx *x = netx(network);
    thb_result r;
    if (network->net && network->net->engine != ENGINE_CPU) {
        thb_set_error(network->net->engine == ENGINE_LOWP ? "This function is not supported with Lowp"
                                                          : "This function is not supported with CUDNN");
        return fatal_or(0);
    }
    if (width < 2 || (width & 1) || height < 1) { thb_set_error("THProcessYUYV needs an even width"); return fatal_or(0); }
    if (ensure_engine(x)) return fatal_or(0);
    if (thb_engine_forward(x->engine, 0, &image, width * 2, 0, 2, 1, 3, height, width, 3, network->mean, network->std, 0, &r))
        return fatal_or(0);
    return publish(network, &r, results, outwidth, outheight);
}

THFloatTensor *THForward(THNETWORK *network, THFloatTensor *in)
{
    thb_netx *x = netx(network);
    static const float zero[3] = {0, 0, 0}, one[3] = {1, 1, 1};
    thb_result r;
    if (ensure_engine(x)) { fatal_or(0); return 0; }
    if (in->nDimension != 3 && in->nDimension != 4) { thb_set_error("THForward needs a 3D or 4D tensor"); fatal_or(0); return 0; }
    int o = in->nDimension == 4;
    int N = o ? (int)in->size[0] : 1, C = (int)in->size[o], H = (int)in->size[o + 1], W = (int)in->size[o + 2];
    if (thb_engine_forward(x->engine, THFloatTensor_data(in), 0, 0, 0, 0, N, C, H, W, in->nDimension, zero, one, 0, &r)) {
        fatal_or(0);
        return 0;
    }
    publish(network, &r, 0, 0, 0);
    return network->out;
}

/* One module on the device: host tensor in, the module's `output` tensor out (the operator-level boundary external code
 * uses, examples/thnets-tf.cc:113-138).  The lowered model, its plan and its uploaded weights are kept per module record
 * (a small table keyed by the record's address and a signature of its contents), so that calling a module again costs a
 * forward, not a conversion; a record whose contents changed, or another record at the same address, gets a new engine. */
typedef struct {
    struct module *m;
    unsigned long long sig;
    thb_engine *e;
    unsigned long long used;
} module_slot;
static module_slot g_slots[64];
static unsigned long long g_slot_clock;

static unsigned long long module_signature(const struct module *m)
{
    /* FNV-1a over the record minus its output tensor: type, function pointers, parameter union (tensor pointers included) */
    unsigned long long h = 1469598103934665603ull;
    const unsigned char *p = (const unsigned char *)m;
    const size_t lo = offsetof(struct module, output), hi = lo + sizeof(m->output);
    for (size_t i = 0; i < sizeof(*m); i++) {
        if (i >= lo && i < hi) continue;
        h = (h ^ p[i]) * 1099511628211ull;
    }
    return h;
}

/* forget the engine kept for a module record (called when a loader-built record is released) */
void thb_module_forget(struct module *m)
{
    for (int i = 0; i < 64; i++)
        if (g_slots[i].m == m) {
            thb_engine_destroy(g_slots[i].e);
            memset(&g_slots[i], 0, sizeof(g_slots[i]));
        }
}

THFloatTensor *thb_module_updateOutput(struct module *m, THFloatTensor *in)
{
    static const float zero[3] = {0, 0, 0}, one[3] = {1, 1, 1};
    char err[256] = "";
    thb_result r;
    THInit();
    const unsigned long long sig = module_signature(m);
    module_slot *slot = 0, *victim = &g_slots[0];
    for (int i = 0; i < 64; i++) {
        if (g_slots[i].m == m && g_slots[i].e) {
            if (g_slots[i].sig == sig) slot = &g_slots[i];
            else { thb_engine_destroy(g_slots[i].e); memset(&g_slots[i], 0, sizeof(g_slots[i])); }
        }
        if (g_slots[i].used < victim->used) victim = &g_slots[i];
    }
    if (!slot) {
        thb_model *model = thb_model_from_module(m, err, sizeof(err));
        if (!model) THError("%s", err);
        thb_engine *e = thb_engine_create(model, THB_MODE_F32, 0, 1);
        thb_model_release(model);
        if (!e) THError("%s", thb_engine_error());
        if (victim->e) thb_engine_destroy(victim->e);   /* the least recently used record makes room */
        victim->m = m; victim->sig = sig; victim->e = e;
        slot = victim;
    }
    slot->used = ++g_slot_clock;
    int rank = in->nDimension, N = 1, C = 1, H = 1, W = 1;
    if (rank == 4) { N = in->size[0]; C = in->size[1]; H = in->size[2]; W = in->size[3]; }
    else if (rank == 3) { C = in->size[0]; H = in->size[1]; W = in->size[2]; }
    else if (rank == 2) { N = in->size[0]; C = in->size[1]; }
    else if (rank == 1) { C = in->size[0]; }
    else THError("updateOutput needs a 1D to 4D tensor");
    /* 1-D and 2-D inputs are [C] / [N, C] feature vectors: planned as 1 x 1 images of rank 3 / 4 */
    if (thb_engine_forward(slot->e, THFloatTensor_data(in), 0, 0, 0, 0, N, C, H, W, rank >= 3 ? rank : rank + 2, zero, one, 0, &r))
        THError("%s", thb_engine_error());
    if (!m->output) m->output = THFloatTensor_new();
    THFloatTensor_resize(m->output, r.size, r.ndim);
    memcpy(THFloatTensor_data(m->output), r.data, sizeof(float) * r.count);
    return m->output;
}

/* Text dump of the lowered operator list (one line per node): used by host-side tests and for debugging. */
/* bounded formatted append: never writes past buf[len - 1]; returns the new length (at most len - 1) */
static int describe_append(char *buf, int len, int pos, const char *fmt, ...)
{
    if (pos >= len - 1) return len - 1;
    va_list ap;
    va_start(ap, fmt);
    int w = vsnprintf(buf + pos, (size_t)(len - pos), fmt, ap);
    va_end(ap);
    if (w < 0) return pos;
    return pos + w >= len ? len - 1 : pos + w;
}

int THB200_DescribeNetwork(THNETWORK *network, char *buf, int len)
{
    static const char *names[] = {"input", "conv", "deconv", "linear", "bn", "act", "maxpool", "avgpool", "combine",
                                  "concat", "softmax", "view", "alias", "scale", "upsample", "zeropad", "slice", "cmax",
                                  "logsoftmax", "normalize", "unpool", "reshape"};
    char err[256] = "";
    if (!buf || len < 2) return -1;
    thb_model *m = thb_model_from_network(network, err, sizeof(err));
    if (!m) { snprintf(buf, len, "error: %s", err); return -1; }
    int pos = 0;
    buf[0] = 0;
    for (int i = 0; i < m->nnodes; i++) {
        thb_node *n = &m->nodes[i];
        pos = describe_append(buf, len, pos, "%d %s in=", i, names[n->op]);
        for (int k = 0; k < n->nin; k++) pos = describe_append(buf, len, pos, "%s%d", k ? "," : "", n->in[k]);
        if (n->op == OP_CONV || n->op == OP_DECONV || n->op == OP_LINEAR)
            pos = describe_append(buf, len, pos, " %d->%d k%dx%d s%d,%d p%d,%d bias=%d", n->Cin, n->Cout, n->kH, n->kW, n->dH, n->dW,
                                  n->padH, n->padW, n->bias != 0);
        else if (n->op == OP_MAXPOOL || n->op == OP_AVGPOOL)
            pos = describe_append(buf, len, pos, " k%dx%d s%d,%d p%d,%d ceil=%d", n->kH, n->kW, n->dH, n->dW, n->padH, n->padW, n->ceil_mode);
        else if (n->op == OP_COMBINE)
            for (int k = 0; k < n->nin; k++) pos = describe_append(buf, len, pos, " %+g", n->coef[k]);
        else if (n->op == OP_VIEW) pos = describe_append(buf, len, pos, " %d", n->numElements);
        else if (n->op == OP_ACT) pos = describe_append(buf, len, pos, " kind=%d th=%g val=%g", n->act_kind, n->act_threshold, n->act_value);
        else if (n->op == OP_CONCAT) pos = describe_append(buf, len, pos, " dim=%d", n->dim);
        else if (n->op == OP_ZEROPAD) pos = describe_append(buf, len, pos, " l%d r%d t%d b%d", n->pad_l, n->pad_r, n->pad_t, n->pad_b);
        else if (n->op == OP_SLICE) pos = describe_append(buf, len, pos, " axis=%d [%d,%d)", n->slice_axis, n->slice_from, n->slice_to);
        else if (n->op == OP_RESHAPE) pos = describe_append(buf, len, pos, " %dx%dx%d", n->reshape[0], n->reshape[1], n->reshape[2]);
        pos = describe_append(buf, len, pos, "%s\n", i == m->output ? " <- output" : "");
    }
    thb_model_release(m);
    return pos;
}

int THB200_ProfileForward(THNETWORK *network, int iters, int max_steps, int *kinds, float *ms, double *flops)
{
    return thb_engine_profile(netx(network)->engine, iters, max_steps, kinds, ms, flops);
}
int THB200_ProfileForwardBytes(THNETWORK *network, int max_steps, double *bytes)
{
    return thb_engine_profile_bytes(netx(network)->engine, max_steps, bytes);
}
void THB200_SliceBatch(int N, int G, int g, int *offset, int *count) { thb_slice_batch(N, G, g, offset, count); }
void THB200_SliceSubBatches(int n, int S, int c, int *offset, int *count) { thb_slice_sub_batches(n, S, c, offset, count); }
float THB200_LastDeviceMs(THNETWORK *network) { return thb_engine_last_ms(netx(network)->engine); }
float THB200_TimeForward(THNETWORK *network, int iters) { return thb_engine_time_forward(netx(network)->engine, iters); }
