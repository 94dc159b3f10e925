/*
 * Builders of `struct module` records from the two model formats:
 *   * Torch7 nn.* objects  -> Module2Network   (reference thload.c:712-781 and the nnload_* functions
 *     of the modules directory: same field names, same defaults);
 *   * "PyTorch Graph Dump 1.00" functions -> loadpytorch  (reference pytorch.c:113-299 and the pyload_*
 *     functions of the modules directory: positional tensors are weight then bias).
 * A module record only carries parameters.  Its updateOutput runs that one operator on the device.
 */
#include <stdio.h>
#include <string.h>
#include "thnets.h"
#include "thb_internal.h"

/* ================================================================================================
 * Torch7
 * ============================================================================================== */
static void release_tensors(struct module *m)
{
    thb_module_forget(m);   /* an engine kept for single-module execution goes with the record */
    switch (m->type) {
    case MT_SpatialConvolution: case MT_SpatialConvolutionMM: case MT_SpatialConvolutionVirtMM:
        THFloatTensor_free(m->SpatialConvolution.bias);
        THFloatTensor_free(m->SpatialConvolution.weight);
        THFloatTensor_free(m->SpatialConvolution.finput);
        break;
    case MT_SpatialFullConvolution:
        THFloatTensor_free(m->SpatialFullConvolution.bias);
        THFloatTensor_free(m->SpatialFullConvolution.weight);
        THFloatTensor_free(m->SpatialFullConvolution.ones);
        THFloatTensor_free(m->SpatialFullConvolution.columns);
        break;
    case MT_Linear:
        THFloatTensor_free(m->Linear.bias);
        THFloatTensor_free(m->Linear.weight);
        THFloatTensor_free(m->Linear.addBuffer);
        break;
    case MT_SpatialBatchNormalization:
        THFloatTensor_free(m->SpatialBatchNormalization.running_mean);
        THFloatTensor_free(m->SpatialBatchNormalization.running_var);
        THFloatTensor_free(m->SpatialBatchNormalization.weight);
        THFloatTensor_free(m->SpatialBatchNormalization.bias);
        break;
    case MT_SpatialMaxPooling: THFloatTensor_free(m->SpatialMaxPooling.indices); break;
    case MT_PReLU: THFloatTensor_free(m->PReLU.weight); break;
    case MT_Sequential: case MT_ConcatTable:
        if (m->Sequential.net) freenetwork(m->Sequential.net);
        break;
    case MT_Concat:
        if (m->Concat.net) freenetwork(m->Concat.net);
        break;
    }
}

static void view_as_matrix(THFloatTensor *w)
{
    if (w->nDimension == 4) {
        long rows = w->size[0], cols = w->size[1] * w->size[2] * w->size[3];
        w->nDimension = 2;
        w->size[0] = rows; w->size[1] = cols;
        w->stride[0] = cols; w->stride[1] = 1;
    }
}

static void geometry(struct table *t, int *padW, int *padH, int *dW, int *dH, int *kW, int *kH)
{
    *padW = thb_t7_number(t, "padW"); *padH = thb_t7_number(t, "padH");
    *dW = thb_t7_number(t, "dW"); *dH = thb_t7_number(t, "dH");
    *kW = thb_t7_number(t, "kW"); *kH = thb_t7_number(t, "kH");
}

/* returns 0 when the Torch class is known */
static int build_torch_module(struct module *m, struct nnmodule *n)
{
    struct table *t = n->table;
    const char *cls = n->name;
    m->nnfree = release_tensors;
    m->updateOutput = thb_module_updateOutput;
    if (!strcmp(cls, "nn.SpatialConvolutionMM") || !strcmp(cls, "nn.SpatialConvolution")) {
        struct SpatialConvolution *c = &m->SpatialConvolution;
        m->type = MT_SpatialConvolutionMM;
        geometry(t, &c->padW, &c->padH, &c->dW, &c->dH, &c->kW, &c->kH);
        if (!c->padW && !c->padH) c->padW = c->padH = thb_t7_number(t, "padding");
        c->nInputPlane = thb_t7_number(t, "nInputPlane");
        c->nOutputPlane = thb_t7_number(t, "nOutputPlane");
        c->bias = thb_t7_tensor(t, "bias");
        c->weight = thb_t7_tensor(t, "weight");
        view_as_matrix(c->weight);
        c->finput = THFloatTensor_new();
        c->padH2 = c->padH; c->padW2 = c->padW; c->dlH = c->dlW = 1;
    } else if (!strcmp(cls, "nn.SpatialFullConvolution")) {
        struct SpatialFullConvolution *c = &m->SpatialFullConvolution;
        m->type = MT_SpatialFullConvolution;
        geometry(t, &c->padW, &c->padH, &c->dW, &c->dH, &c->kW, &c->kH);
        c->adjW = thb_t7_number(t, "adjW"); c->adjH = thb_t7_number(t, "adjH");
        c->nInputPlane = thb_t7_number(t, "nInputPlane");
        c->nOutputPlane = thb_t7_number(t, "nOutputPlane");
        c->bias = thb_t7_tensor(t, "bias");
        c->weight = thb_t7_tensor(t, "weight");
        c->columns = THFloatTensor_new();
        c->ones = THFloatTensor_new();
    } else if (!strcmp(cls, "nn.SpatialMaxPooling")) {
        struct SpatialMaxPooling *p = &m->SpatialMaxPooling;
        m->type = MT_SpatialMaxPooling;
        geometry(t, &p->padW, &p->padH, &p->dW, &p->dH, &p->kW, &p->kH);
        p->ceil_mode = thb_t7_number(t, "ceil_mode");
        p->indices = THFloatTensor_new();
    } else if (!strcmp(cls, "nn.SpatialAveragePooling")) {
        struct SpatialAveragePooling *p = &m->SpatialAveragePooling;
        m->type = MT_SpatialAveragePooling;
        geometry(t, &p->padW, &p->padH, &p->dW, &p->dH, &p->kW, &p->kH);
        p->ceil_mode = thb_t7_number(t, "ceil_mode");
        p->count_include_pad = thb_t7_number(t, "count_include_pad");
    } else if (!strcmp(cls, "nn.Linear")) {
        m->type = MT_Linear;
        m->Linear.weight = thb_t7_tensor(t, "weight");
        m->Linear.addBuffer = thb_t7_tensor(t, "addBuffer");
        m->Linear.bias = thb_t7_tensor(t, "bias");
    } else if (!strcmp(cls, "nn.SoftMax")) {
        m->type = MT_SoftMax;
    } else if (!strcmp(cls, "nn.Threshold") || !strcmp(cls, "nn.ReLU")) {
        m->type = MT_Threshold;
        m->Threshold.threshold = thb_t7_number(t, "threshold");
        m->Threshold.val = thb_t7_number(t, "val");
        m->Threshold.inplace = thb_t7_boolean(t, "inplace");
    } else if (!strcmp(cls, "nn.View")) {
        m->type = MT_View;
        m->View.numElements = thb_t7_number(t, "numElements");
    } else if (!strcmp(cls, "nn.Dropout") || !strcmp(cls, "nn.SpatialDropout") || !strcmp(cls, "nn.Identity") ||
               !strcmp(cls, "nn.Padding")) {
        /* the reference loads all four through its Dropout constructor (thload.c:721-726) */
        m->type = MT_Dropout;
        m->Dropout.inplace = thb_t7_boolean(t, "inplace");
        m->Dropout.v2 = thb_t7_boolean(t, "v2");
        m->Dropout.p = thb_t7_number(t, "p");
    } else if (!strcmp(cls, "nn.Reshape")) {
        int n1 = 0;
        m->type = MT_Reshape;
        m->Reshape.numElements = thb_t7_number(t, "nelement");
        m->Reshape.batchMode = thb_t7_boolean(t, "batchMode");
        void *d = thb_t7_storage(t, "size", &n1);
        if (d && n1 <= 4) { memcpy(m->Reshape.size, d, sizeof(long) * n1); m->Reshape.nsize = n1; }
        d = thb_t7_storage(t, "batchsize", &n1);
        if (d && n1 <= 4) { memcpy(m->Reshape.batchsize, d, sizeof(long) * n1); m->Reshape.nbatchsize = n1; }
    } else if (!strcmp(cls, "nn.SpatialBatchNormalization")) {
        struct SpatialBatchNormalization *b = &m->SpatialBatchNormalization;
        m->type = MT_SpatialBatchNormalization;
        b->running_mean = thb_t7_tensor(t, "running_mean");
        b->running_var = thb_t7_tensor(t, "running_var");
        b->weight = thb_t7_tensor(t, "weight");
        b->bias = thb_t7_tensor(t, "bias");
        b->eps = thb_t7_number(t, "eps");
    } else if (!strcmp(cls, "nn.Sequential")) {
        m->type = MT_Sequential;
        m->Sequential.net = Module2Network(n);
    } else if (!strcmp(cls, "nn.ConcatTable")) {
        m->type = MT_ConcatTable;
        m->ConcatTable.net = Module2Network(n);
    } else if (!strcmp(cls, "nn.Concat")) {
        m->type = MT_Concat;
        m->Concat.dimension = thb_t7_number(t, "dimension") - 1;
        m->Concat.net = Module2Network(n);
    } else if (!strcmp(cls, "nn.JoinTable")) {
        m->type = MT_JoinTable;
        m->JoinTable.dimension = thb_t7_number(t, "dimension") - 1;
    } else if (!strcmp(cls, "nn.CAddTable")) {
        m->type = MT_CAddTable;
    } else if (!strcmp(cls, "nn.PReLU")) {
        m->type = MT_PReLU;
        m->PReLU.nOutputPlane = thb_t7_number(t, "nOutputPlane");
        m->PReLU.weight = thb_t7_tensor(t, "weight");
    } else if (!strcmp(cls, "nn.SpatialZeroPadding")) { /* SpatialZeroPadding.c:4-15 */
        m->type = MT_SpatialZeroPadding;
        m->SpatialZeroPadding.pad_l = thb_t7_number(t, "pad_l");
        m->SpatialZeroPadding.pad_r = thb_t7_number(t, "pad_r");
        m->SpatialZeroPadding.pad_t = thb_t7_number(t, "pad_t");
        m->SpatialZeroPadding.pad_b = thb_t7_number(t, "pad_b");
    } else if (!strcmp(cls, "nn.Normalize") || !strcmp(cls, "nn.L2Normalize")) { /* thload.c:729-730 */
        m->type = MT_Normalize;
    } else if (!strcmp(cls, "nn.LogSoftMax")) {
        m->type = MT_LogSoftMax;
    } else if (!strcmp(cls, "nn.SpatialMaxUnpooling")) { /* SpatialMaxUnpooling.c:4-12 */
        m->type = MT_SpatialMaxUnpooling;
        m->SpatialMaxUnpooling.pooling = thb_t7_nnmodule(t, "pooling");
    } else
        return -1;
    return 0;
}

struct network *Module2Network(struct nnmodule *obj)
{
    if (strcmp(obj->name, "nn.Sequential") && strcmp(obj->name, "nn.Concat") && strcmp(obj->name, "nn.ConcatTable"))
        return 0;
    struct table *list = 0;
    for (int i = 0; i < obj->table->nelem; i++) {
        struct threcord *r = &obj->table->records[i];
        if (r->name.type == TYPE_STRING && !strcmp(r->name.string.data, "modules") && r->value.type == TYPE_TABLE) {
            list = r->value.table;
            break;
        }
    }
    if (!list) return 0;
    struct network *net = malloc(sizeof(*net));
    net->engine = ENGINE_CPU;
    net->nelem = list->nelem;
    net->modules = calloc(list->nelem ? list->nelem : 1, sizeof(struct module));
    for (int i = 0; i < list->nelem; i++) {
        struct module *m = &net->modules[i];
        if (list->records[i].value.type != TYPE_NNMODULE) THError("Entry %d of a modules table is not a module", i + 1);
        struct nnmodule *child = list->records[i].value.nnmodule;
        m->output = THFloatTensor_new();
        m->net = net;
        m->nnmodule = child;
        if (build_torch_module(m, child)) THError("Unknown module type %s", child->name);
    }
    return net;
}

void freenetwork(struct network *net)
{
    for (int i = 0; i < net->nelem; i++) {
        struct module *m = &net->modules[i];
        if (m->nnfree) m->nnfree(m);
        THFloatTensor_free(m->output);
        free(m->outputname);
    }
    free(net->modules);
    free(net);
}

/* ================================================================================================
 * PyTorch graph dump
 * ============================================================================================== */
static int rd_cstr(FILE *fp, char *s, int cap)
{
    for (int i = 0; i < cap; i++) {
        int c = fgetc(fp);
        if (c == EOF) return -1;
        s[i] = (char)c;
        if (!c) return 0;
    }
    return -1;
}
static int rd_ivec(FILE *fp, int *v)
{
    int n;
    if (fread(&n, 4, 1, fp) != 1 || n < 1 || n > 4) return -1;
    memset(v, 0, 4 * sizeof(int));
    return fread(v, 4, n, fp) == (size_t)n ? 0 : -1;
}
static THFloatTensor *rd_pytensor(FILE *fp)
{
    int ndim, dims[4];
    long long count;
    if (fread(&ndim, 4, 1, fp) != 1 || ndim < 1 || ndim > 4) return 0;
    if (fread(dims, 4, ndim, fp) != (size_t)ndim || fread(&count, 8, 1, fp) != 1 || count < 0) return 0;
    THFloatTensor *t = THFloatTensor_new();
    long stride = 1;
    t->nDimension = ndim;
    for (int i = ndim - 1; i >= 0; i--) {
        t->size[i] = dims[i];
        t->stride[i] = stride;
        stride *= dims[i];
    }
    t->storage = THFloatStorage_new((long)count);
    if (count && fread(t->storage->data, 4, (size_t)count, fp) != (size_t)count) {
        THFloatTensor_free(t);
        return 0;
    }
    return t;
}

static struct pyelement *param(struct elemlist *l, const char *name, int skip)
{
    for (; l; l = l->next)
        if (!strcmp(l->elem->name, name) && skip-- == 0) return l->elem;
    return 0;
}
static THFloatTensor *param_tensor(struct elemlist *l, const char *name, int skip)
{
    THFloatTensor *t = THFloatTensor_new();
    struct pyelement *e = param(l, name, skip);
    if (e && e->type == ELTYPE_TENSOR) THFloatTensor_set(t, e->tensor);
    return t;
}
static void ivec2(struct elemlist *l, const char *name, int *h, int *w)
{
    struct pyelement *e = param(l, name, 0);
    if (e && e->type == ELTYPE_INTVECT) { *h = e->ivect[0]; *w = e->ivect[1]; }
}
static int ival(struct elemlist *l, const char *name, int dflt)
{
    struct pyelement *e = param(l, name, 0);
    return (e && e->type == ELTYPE_INT) ? e->ivalue : dflt;
}
static float fval(struct elemlist *l, const char *name, float dflt)
{
    struct pyelement *e = param(l, name, 0);
    return (e && e->type == ELTYPE_FLOAT) ? e->fvalue : dflt;
}

void thb_build_py_module(const char *fname, struct pyfunction *f)
{
    const char *op = strrchr(fname, '.');
    op = op ? op + 1 : fname;
    struct module *m = &f->module;
    struct elemlist *p = f->params;
    m->output = THFloatTensor_new();
    m->nnfree = release_tensors;
    m->updateOutput = thb_module_updateOutput;
    if (!strcmp(op, "ConvNd")) {
        struct SpatialConvolution *c = &m->SpatialConvolution;
        m->type = MT_SpatialConvolutionVirtMM;
        c->weight = param_tensor(p, "", 0);
        c->bias = param_tensor(p, "", 1);
        c->finput = THFloatTensor_new();
        c->nOutputPlane = c->weight->size[0]; c->nInputPlane = c->weight->size[1];
        c->kH = c->weight->size[2]; c->kW = c->weight->size[3];
        ivec2(p, "padding", &c->padH, &c->padW);
        ivec2(p, "stride", &c->dH, &c->dW);
        /* the ONNX reader also passes the attributes the reference parses and ignores (SpatialConvolution.c:88-109) */
        c->padH2 = c->padH; c->padW2 = c->padW; c->dlH = c->dlW = 1;
        ivec2(p, "padding2", &c->padH2, &c->padW2);
        ivec2(p, "dilation", &c->dlH, &c->dlW);
        c->autopad = ival(p, "autopad", 0);
        c->refl_pad = ival(p, "refl_pad", 0);
    } else if (!strcmp(op, "ConvTransposedNd")) {
        struct SpatialFullConvolution *c = &m->SpatialFullConvolution;
        m->type = MT_SpatialFullConvolution;
        c->weight = param_tensor(p, "", 0);
        c->bias = param_tensor(p, "", 1);
        c->nInputPlane = c->weight->size[0]; c->nOutputPlane = c->weight->size[1];
        c->kH = c->weight->size[2]; c->kW = c->weight->size[3];
        ivec2(p, "padding", &c->padH, &c->padW);
        ivec2(p, "output_padding", &c->adjH, &c->adjW);
        ivec2(p, "stride", &c->dH, &c->dW);
        c->columns = THFloatTensor_new();
        c->ones = THFloatTensor_new();
    } else if (!strcmp(op, "Linear")) {
        m->type = MT_Linear;
        m->Linear.weight = param_tensor(p, "", 0);
        m->Linear.bias = param_tensor(p, "", 1);
        m->Linear.addBuffer = THFloatTensor_new();
    } else if (!strcmp(op, "BatchNorm")) {
        struct SpatialBatchNormalization *b = &m->SpatialBatchNormalization;
        m->type = MT_SpatialBatchNormalization;
        b->weight = param_tensor(p, "", 0);
        b->bias = param_tensor(p, "", 1);
        b->running_mean = param_tensor(p, "running_mean", 0);
        b->running_var = param_tensor(p, "running_var", 0);
        b->eps = fval(p, "eps", 0);
    } else if (!strcmp(op, "MaxPool2d")) {
        struct SpatialMaxPooling *q = &m->SpatialMaxPooling;
        m->type = MT_SpatialMaxPooling;
        q->indices = THFloatTensor_new();
        ivec2(p, "padding", &q->padH, &q->padW);
        ivec2(p, "stride", &q->dH, &q->dW);
        ivec2(p, "kernel_size", &q->kH, &q->kW);
        q->ceil_mode = ival(p, "ceil_mode", 0);
    } else if (!strcmp(op, "AvgPool2d")) {
        struct SpatialAveragePooling *q = &m->SpatialAveragePooling;
        m->type = MT_SpatialAveragePooling;
        ivec2(p, "padding", &q->padH, &q->padW);
        ivec2(p, "stride", &q->dH, &q->dW);
        ivec2(p, "kernel_size", &q->kH, &q->kW);
        q->ceil_mode = ival(p, "ceil_mode", 0);
    } else if (!strcmp(op, "Threshold")) {
        m->type = MT_Threshold;
        m->Threshold.threshold = fval(p, "threshold", 0);
        m->Threshold.val = fval(p, "value", 0);
        m->Threshold.inplace = ival(p, "inplace", 0);
        m->Threshold.alpha = fval(p, "alpha", 0);    /* the ONNX reader's LeakyRelu only (Threshold.c:30-35) */
    } else if (!strcmp(op, "PReLU")) {               /* the ONNX reader only (onnx.cc:35, PReLU.c:21-29) */
        m->type = MT_PReLU;
        m->PReLU.weight = param_tensor(p, "", 0);
        m->PReLU.nOutputPlane = m->PReLU.weight ? (int)m->PReLU.weight->size[0] : 0;
    } else if (!strcmp(op, "Dropout")) {
        m->type = MT_Dropout;
        m->Dropout.inplace = 1; m->Dropout.v2 = 1; m->Dropout.p = 0;
    } else if (!strcmp(op, "Softmax")) {
        m->type = MT_SoftMax;
    } else if (!strcmp(op, "View")) {
        struct pyelement *e = param(p, "sizes", 0);
        m->type = MT_View;
        if (e && e->type == ELTYPE_INTVECT) m->View.numElements = e->ivect[1];
    } else if (!strcmp(op, "Add")) {
        m->type = MT_CAddTable;
    } else if (!strcmp(op, "Sigmoid")) { /* these two: the ONNX reader only (onnx.cc:59-60) */
        m->type = MT_Sigmoid;
    } else if (!strcmp(op, "Tanh")) {
        m->type = MT_Tanh;
    } else if (!strcmp(op, "Sub")) { /* only the ONNX reader produces it (onnx.cc:45) */
        m->type = MT_CSubTable;
    } else if (!strcmp(op, "Concat")) {
        m->type = MT_JoinTable;
        m->JoinTable.dimension = ival(p, "dim", 0);
    } else if (!strcmp(op, "Slice")) {
        /* Slice.c:3-14: the graph dump carries "index" = {from, to} and no axis (dimension 0); the ONNX reader passes all three */
        struct pyelement *e = param(p, "index", 0);
        m->type = MT_Slice;
        if (e && e->type == ELTYPE_INTVECT) { m->Slice.from = e->ivect[0]; m->Slice.to = e->ivect[1]; }
        else { m->Slice.axis = ival(p, "axis", 0); m->Slice.from = ival(p, "from", 0); m->Slice.to = ival(p, "to", 0); }
    } else if (!strcmp(op, "Cmax")) {
        m->type = MT_Cmax;
    } else if (!strcmp(op, "LogSoftmax")) { /* ONNX reader only (onnx.cc:41) */
        m->type = MT_LogSoftMax;
    } else if (!strcmp(op, "Upsample")) {   /* ONNX reader only (onnx.cc:54, Upsample.c:4-16) */
        m->type = MT_Upsample;
        m->Upsample.width_scale = fval(p, "width_scale", 0);
        m->Upsample.height_scale = fval(p, "height_scale", 0);
    } else
        THError("Unsupported function %s", fname);
}

static void append(struct elemlist **head, struct pyelement *e)
{
    struct elemlist *n = calloc(1, sizeof(*n));
    n->elem = e;
    while (*head) head = &(*head)->next;
    *head = n;
}

static struct pyelement *rd_element(FILE *fp, struct pyelement **nodes)
{
    char name[100];
    int tag = fgetc(fp);
    if (tag == EOF) return 0;
    struct pyelement *e = calloc(1, sizeof(*e));
    e->type = tag;
    switch (tag) {
    case ELTYPE_END: case ELTYPE_INPUT: return e;
    case ELTYPE_OUTPUTID:
        if (fread(&e->ivalue, 4, 1, fp) != 1 || (unsigned)e->ivalue >= MAXPYNODES || !nodes[e->ivalue]) break;
        return e;
    case ELTYPE_INT:
        if (rd_cstr(fp, name, sizeof(name)) || fread(&e->ivalue, 4, 1, fp) != 1) break;
        e->name = strdup(name);
        return e;
    case ELTYPE_FLOAT:
        if (rd_cstr(fp, name, sizeof(name)) || fread(&e->fvalue, 4, 1, fp) != 1) break;
        e->name = strdup(name);
        return e;
    case ELTYPE_INTVECT:
        if (rd_cstr(fp, name, sizeof(name)) || rd_ivec(fp, e->ivect)) break;
        e->name = strdup(name);
        return e;
    case ELTYPE_TENSOR:
        if (rd_cstr(fp, name, sizeof(name)) || !(e->tensor = rd_pytensor(fp))) break;
        e->name = strdup(name);
        return e;
    case ELTYPE_FUNCTION: {
        if (fread(&e->function.id, 4, 1, fp) != 1 || (unsigned)e->function.id >= MAXPYNODES) break;
        if (rd_cstr(fp, name, sizeof(name))) break;
        e->name = strdup(name);
        nodes[e->function.id] = e;
        for (;;) {
            struct pyelement *child = rd_element(fp, nodes);
            if (!child) return 0; /* truncated file: the partial tree is abandoned */
            if (child->type == ELTYPE_END) {
                free(child);
                break;
            }
            if (child->type == ELTYPE_FUNCTION || child->type == ELTYPE_INPUT || child->type == ELTYPE_OUTPUTID) {
                append(&e->function.inputs, child);
                e->function.ninputs++;
            } else
                append(&e->function.params, child);
        }
        thb_build_py_module(name, &e->function);
        return e;
    }
    }
    free(e);
    return 0;
}

struct pyelement *loadpytorch(const char *path, struct pyelement **allpynodes)
{
    static const char magic[24] = "PyTorch Graph Dump 1.00";
    char header[24];
    FILE *fp = fopen(path, "rb");
    if (!fp) return 0;
    struct pyelement *root = 0;
    if (fread(header, 1, 24, fp) == 24 && !memcmp(header, magic, 24)) root = rd_element(fp, allpynodes);
    fclose(fp);
    if (root && root->type != ELTYPE_FUNCTION) {
        freepynet(root);
        root = 0;
    }
    return root;
}

void freepynet(struct pyelement *e)
{
    if (!e) return;
    free(e->name);
    if (e->type == ELTYPE_FUNCTION) {
        struct elemlist *lists[2] = {e->function.params, e->function.inputs};
        for (int k = 0; k < 2; k++)
            for (struct elemlist *l = lists[k], *next; l; l = next) {
                next = l->next;
                freepynet(l->elem);
                free(l);
            }
        THFloatTensor_free(e->function.module.output);
        if (e->function.module.nnfree) e->function.module.nnfree(&e->function.module);
    } else if (e->type == ELTYPE_TENSOR)
        THFloatTensor_free(e->tensor);
    free(e);
}
