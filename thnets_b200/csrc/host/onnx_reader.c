/* ONNX model loader without protobuf: a reader of the protobuf wire format for the handful of ONNX messages a
 * convolutional network uses, producing the same node tree the PyTorch-dump loader produces (struct pyelement), so
 * that everything downstream of a loaded network is shared.
 *
 * Replaces the reference's loadonnx (onnx.cc:572-834, which needs protoc-generated classes of onnx.proto) for the
 * operators of the benchmark configurations.  Field numbers (onnx.proto): ModelProto.graph = 7; GraphProto.node = 1,
 * initializer = 5, input = 11, output = 12; NodeProto.input = 1, output = 2, name = 3, op_type = 4, attribute = 5;
 * AttributeProto.name = 1, f = 2, i = 3, s = 4, t = 5, floats = 7, ints = 8; TensorProto.dims = 1, data_type = 2
 * (1 = float, 7 = int64), float_data = 4, int64_data = 7, name = 8, raw_data = 9; ValueInfoProto.name = 1.
 *
 * Behaviour kept from the reference's loader: a BatchNormalization whose input is a Conv / ConvTranspose is folded into
 * that convolution's weights and bias in fp32 (absorb_bn, onnx.cc:472-570); an Add of a constant to a convolution's
 * output becomes (part of) its bias (onnx.cc:605-660); a constant-mode Pad in front of a Conv adds to its padding
 * (onnx.cc:667-700); Add / Sum become CAddTable and Sub CSubTable (with the two-input arithmetic those modules have);
 * dilations, groups' absence, auto_pad and the end pads of a convolution are not looked at (modules/SpatialConvolution.c
 * onnxload).  Unknown operators are an error here (the reference substitutes a Dropout and warns). */
#include "thb_internal.h"
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------- wire format */
typedef struct { const uint8_t *p, *end; } pbuf;

static int pb_varint(pbuf *c, uint64_t *v)
{
    uint64_t r = 0;
    for (int shift = 0; shift < 64 && c->p < c->end; shift += 7) {
        uint8_t b = *c->p++;
        r |= (uint64_t)(b & 0x7f) << shift;
        if (!(b & 0x80)) { *v = r; return 0; }
    }
    return -1;
}

/* next field of a message: its number and wire type; varint / fixed values in *val, length-delimited payloads in *sub */
static int pb_next(pbuf *c, int *field, int *wt, uint64_t *val, pbuf *sub)
{
    uint64_t key, len;
    if (pb_varint(c, &key)) return -1;
    *field = (int)(key >> 3);
    *wt = (int)(key & 7);
    switch (*wt) {
    case 0: return pb_varint(c, val);
    case 1:
        if (c->end - c->p < 8) return -1;
        memcpy(val, c->p, 8); c->p += 8;
        return 0;
    case 2:
        if (pb_varint(c, &len) || (uint64_t)(c->end - c->p) < len) return -1;
        sub->p = c->p; sub->end = c->p + len; c->p += len;
        return 0;
    case 5: {
        uint32_t v;
        if (c->end - c->p < 4) return -1;
        memcpy(&v, c->p, 4); c->p += 4;
        *val = v;
        return 0;
    }
    }
    return -1; /* groups are not used by ONNX */
}

static char *pb_strdup(const pbuf *s)
{
    size_t n = (size_t)(s->end - s->p);
    char *r = malloc(n + 1);
    memcpy(r, s->p, n);
    r[n] = 0;
    return r;
}

/* ------------------------------------------------------------------------------------------- ONNX messages */
#define OX_MAXDIMS 8
#define OX_MAXIO 8
#define OX_MAXATTR 16
#define OX_MAXINTS 16

typedef struct {
    char *name;
    int ndims, data_type;
    long dims[OX_MAXDIMS];
    long count;     /* elements decoded */
    float *f;       /* data_type 1 */
    int64_t *i64;   /* data_type 7 */
} ox_tensor;

typedef struct {
    char *name;
    int has_i, has_f, nints, nfloats;
    int64_t i, ints[OX_MAXINTS];
    float f, floats[OX_MAXINTS];
    char *s;
    ox_tensor *t;
} ox_attr;

typedef struct {
    char *op, *in[OX_MAXIO], *out[OX_MAXIO];
    int nin, nout, nattr;
    ox_attr attr[OX_MAXATTR];
} ox_node;

typedef struct {
    ox_node *nodes;
    int nnodes, capnodes;
    ox_tensor **inits;
    int ninits, capinits;
    char **inputs;
    int ninputs, capinputs;
    char *output;
} ox_graph;

static void ox_tensor_free(ox_tensor *t)
{
    if (!t) return;
    free(t->name); free(t->f); free(t->i64); free(t);
}

static ox_tensor *ox_parse_tensor(pbuf m)
{
    ox_tensor *t = calloc(1, sizeof(*t));
    pbuf raw = {0, 0};
    long nf = 0, capf = 0, ni = 0, capi = 0;
    int field, wt;
    uint64_t v;
    pbuf sub;
    while (m.p < m.end) {
        if (pb_next(&m, &field, &wt, &v, &sub)) goto bad;
        if (field == 1) { /* dims: packed or one by one */
            if (wt == 2) {
                while (sub.p < sub.end) {
                    if (pb_varint(&sub, &v) || t->ndims >= OX_MAXDIMS) goto bad;
                    t->dims[t->ndims++] = (long)v;
                }
            } else if (wt == 0) {
                if (t->ndims >= OX_MAXDIMS) goto bad;
                t->dims[t->ndims++] = (long)v;
            }
        } else if (field == 2 && wt == 0)
            t->data_type = (int)v;
        else if (field == 4) { /* float_data */
            long add = wt == 2 ? (long)(sub.end - sub.p) / 4 : 1;
            if (nf + add > capf) { capf = (nf + add) * 2; t->f = realloc(t->f, capf * sizeof(float)); }
            if (wt == 2) memcpy(t->f + nf, sub.p, (size_t)add * 4);
            else if (wt == 5) { uint32_t u = (uint32_t)v; memcpy(t->f + nf, &u, 4); }
            else goto bad;
            nf += add;
        } else if (field == 7) { /* int64_data */
            if (wt == 2) {
                while (sub.p < sub.end) {
                    if (pb_varint(&sub, &v)) goto bad;
                    if (ni >= capi) { capi = capi ? capi * 2 : 16; t->i64 = realloc(t->i64, capi * sizeof(int64_t)); }
                    t->i64[ni++] = (int64_t)v;
                }
            } else if (wt == 0) {
                if (ni >= capi) { capi = capi ? capi * 2 : 16; t->i64 = realloc(t->i64, capi * sizeof(int64_t)); }
                t->i64[ni++] = (int64_t)v;
            }
        } else if (field == 8 && wt == 2) {
            free(t->name);
            t->name = pb_strdup(&sub);
        } else if (field == 9 && wt == 2)
            raw = sub;
    }
    if (raw.p) {
        size_t bytes = (size_t)(raw.end - raw.p);
        if (t->data_type == 1) {
            free(t->f);
            t->f = malloc(bytes ? bytes : 4);
            memcpy(t->f, raw.p, bytes);
            nf = (long)(bytes / 4);
        } else if (t->data_type == 7) {
            free(t->i64);
            t->i64 = malloc(bytes ? bytes : 8);
            memcpy(t->i64, raw.p, bytes);
            ni = (long)(bytes / 8);
        }
    }
    t->count = t->data_type == 7 ? ni : nf;
    return t;
bad:
    ox_tensor_free(t);
    return 0;
}

static int ox_parse_attr(pbuf m, ox_attr *a)
{
    int field, wt;
    uint64_t v;
    pbuf sub;
    memset(a, 0, sizeof(*a));
    while (m.p < m.end) {
        if (pb_next(&m, &field, &wt, &v, &sub)) return -1;
        if (field == 1 && wt == 2) { free(a->name); a->name = pb_strdup(&sub); }
        else if (field == 2 && wt == 5) { uint32_t u = (uint32_t)v; memcpy(&a->f, &u, 4); a->has_f = 1; }
        else if (field == 3 && wt == 0) { a->i = (int64_t)v; a->has_i = 1; }
        else if (field == 4 && wt == 2) { free(a->s); a->s = pb_strdup(&sub); }
        else if (field == 5 && wt == 2) { ox_tensor_free(a->t); a->t = ox_parse_tensor(sub); if (!a->t) return -1; }
        else if (field == 7) { /* floats: packed or one by one */
            if (wt == 2) {
                while (sub.end - sub.p >= 4) {
                    if (a->nfloats < OX_MAXINTS) memcpy(&a->floats[a->nfloats++], sub.p, 4);
                    sub.p += 4;
                }
            } else if (wt == 5 && a->nfloats < OX_MAXINTS) { uint32_t u = (uint32_t)v; memcpy(&a->floats[a->nfloats++], &u, 4); }
        }
        else if (field == 8) { /* ints: packed or one by one */
            if (wt == 2) {
                while (sub.p < sub.end) {
                    if (pb_varint(&sub, &v)) return -1;
                    if (a->nints < OX_MAXINTS) a->ints[a->nints++] = (int64_t)v;
                }
            } else if (wt == 0 && a->nints < OX_MAXINTS)
                a->ints[a->nints++] = (int64_t)v;
        }
    }
    return a->name ? 0 : -1;
}

static int ox_parse_node(pbuf m, ox_node *n)
{
    int field, wt;
    uint64_t v;
    pbuf sub;
    memset(n, 0, sizeof(*n));
    while (m.p < m.end) {
        if (pb_next(&m, &field, &wt, &v, &sub)) return -1;
        if (wt != 2) continue;
        if (field == 1) { if (n->nin >= OX_MAXIO) return -1; n->in[n->nin++] = pb_strdup(&sub); }
        else if (field == 2) { if (n->nout >= OX_MAXIO) return -1; n->out[n->nout++] = pb_strdup(&sub); }
        else if (field == 4) { free(n->op); n->op = pb_strdup(&sub); }
        else if (field == 5) {
            if (n->nattr >= OX_MAXATTR) return -1;
            if (ox_parse_attr(sub, &n->attr[n->nattr])) return -1;
            n->nattr++;
        }
    }
    return n->op && n->nout ? 0 : -1;
}

static char *ox_valueinfo_name(pbuf m)
{
    int field, wt;
    uint64_t v;
    pbuf sub;
    while (m.p < m.end) {
        if (pb_next(&m, &field, &wt, &v, &sub)) return 0;
        if (field == 1 && wt == 2) return pb_strdup(&sub);
    }
    return 0;
}

static void ox_graph_free(ox_graph *g)
{
    for (int i = 0; i < g->nnodes; i++) {
        ox_node *n = &g->nodes[i];
        free(n->op);
        for (int k = 0; k < n->nin; k++) free(n->in[k]);
        for (int k = 0; k < n->nout; k++) free(n->out[k]);
        for (int k = 0; k < n->nattr; k++) { free(n->attr[k].name); free(n->attr[k].s); ox_tensor_free(n->attr[k].t); }
    }
    free(g->nodes);
    for (int i = 0; i < g->ninits; i++) ox_tensor_free(g->inits[i]);
    free(g->inits);
    for (int i = 0; i < g->ninputs; i++) free(g->inputs[i]);
    free(g->inputs);
    free(g->output);
    memset(g, 0, sizeof(*g));
}

static int ox_parse_graph(pbuf m, ox_graph *g)
{
    int field, wt;
    uint64_t v;
    pbuf sub;
    while (m.p < m.end) {
        if (pb_next(&m, &field, &wt, &v, &sub)) return -1;
        if (wt != 2) continue;
        if (field == 1) {
            if (g->nnodes >= g->capnodes) { g->capnodes = g->capnodes ? g->capnodes * 2 : 64; g->nodes = realloc(g->nodes, g->capnodes * sizeof(ox_node)); }
            if (ox_parse_node(sub, &g->nodes[g->nnodes])) { g->nnodes++; return -1; }
            g->nnodes++;
        } else if (field == 5) {
            ox_tensor *t = ox_parse_tensor(sub);
            if (!t) return -1;
            if (g->ninits >= g->capinits) { g->capinits = g->capinits ? g->capinits * 2 : 64; g->inits = realloc(g->inits, g->capinits * sizeof(*g->inits)); }
            g->inits[g->ninits++] = t;
        } else if (field == 11) {
            char *nm = ox_valueinfo_name(sub);
            if (!nm) return -1;
            if (g->ninputs >= g->capinputs) { g->capinputs = g->capinputs ? g->capinputs * 2 : 16; g->inputs = realloc(g->inputs, g->capinputs * sizeof(char *)); }
            g->inputs[g->ninputs++] = nm;
        } else if (field == 12 && !g->output)
            g->output = ox_valueinfo_name(sub);
    }
    return g->nnodes > 0 ? 0 : -1;
}

/* ------------------------------------------------------------------------------------------- look-ups */
static ox_tensor *ox_init(const ox_graph *g, const char *name)
{
    if (!name || !*name) return 0;
    for (int i = 0; i < g->ninits; i++)
        if (g->inits[i]->name && !strcmp(g->inits[i]->name, name)) return g->inits[i];
    /* Constant nodes carry their tensor as attribute "value" */
    for (int i = 0; i < g->nnodes; i++)
        if (!strcmp(g->nodes[i].op, "Constant") && !strcmp(g->nodes[i].out[0], name))
            for (int k = 0; k < g->nodes[i].nattr; k++)
                if (!strcmp(g->nodes[i].attr[k].name, "value")) return g->nodes[i].attr[k].t;
    return 0;
}
static int ox_producer(const ox_graph *g, const char *name)
{
    for (int i = 0; i < g->nnodes; i++)
        for (int k = 0; k < g->nodes[i].nout; k++)
            if (!strcmp(g->nodes[i].out[k], name)) return i;
    return -1;
}
static const ox_attr *ox_attr_of(const ox_node *n, const char *name)
{
    for (int k = 0; k < n->nattr; k++)
        if (!strcmp(n->attr[k].name, name)) return &n->attr[k];
    return 0;
}
static long ox_int(const ox_node *n, const char *name, long dflt)
{
    const ox_attr *a = ox_attr_of(n, name);
    return a && a->has_i ? (long)a->i : dflt;
}
static float ox_float(const ox_node *n, const char *name, float dflt)
{
    const ox_attr *a = ox_attr_of(n, name);
    return a && a->has_f ? a->f : dflt;
}
static void ox_ints2(const ox_node *n, const char *name, int first, int dflt, int *h, int *w)
{
    const ox_attr *a = ox_attr_of(n, name);
    *h = *w = dflt;
    if (a && a->nints >= first + 2) { *h = (int)a->ints[first]; *w = (int)a->ints[first + 1]; }
    else if (a && a->nints == 1) *h = *w = (int)a->ints[0];
}

/* ------------------------------------------------------------------------------------------- node tree */
typedef struct {
    ox_graph *g;
    struct pyelement **all;   /* allpynodes of the network: id -> function element */
    int *built;               /* ONNX node -> id of the element that stands for it (0: not built yet) */
    char err[256];
} ox_build;

static struct pyelement *el_new(int type, const char *name)
{
    struct pyelement *e = calloc(1, sizeof(*e));
    e->type = type;
    if (name) e->name = strdup(name);
    return e;
}
static void el_append(struct elemlist **head, struct pyelement *e)
{
    struct elemlist *n = calloc(1, sizeof(*n));
    n->elem = e;
    while (*head) head = &(*head)->next;
    *head = n;
}
static void par_ivec(struct pyfunction *f, const char *name, int a, int b)
{
    struct pyelement *e = el_new(ELTYPE_INTVECT, name);
    e->ivect[0] = a; e->ivect[1] = b;
    el_append(&f->params, e);
}
static void par_int(struct pyfunction *f, const char *name, int v)
{
    struct pyelement *e = el_new(ELTYPE_INT, name);
    e->ivalue = v;
    el_append(&f->params, e);
}
static void par_float(struct pyfunction *f, const char *name, float v)
{
    struct pyelement *e = el_new(ELTYPE_FLOAT, name);
    e->fvalue = v;
    el_append(&f->params, e);
}
/* a float tensor parameter of the given shape (rank <= 4) holding a copy of `data` */
static void par_tensor(struct pyfunction *f, const char *name, const float *data, const long *dims, int ndims)
{
    struct pyelement *e = el_new(ELTYPE_TENSOR, name);
    THFloatTensor *t = THFloatTensor_new();
    long count = 1, stride = 1;
    for (int i = 0; i < ndims; i++) count *= dims[i];
    t->nDimension = ndims;
    for (int i = ndims - 1; i >= 0; i--) { t->size[i] = dims[i]; t->stride[i] = stride; stride *= dims[i]; }
    t->storage = THFloatStorage_new(count);
    if (count) memcpy(t->storage->data, data, (size_t)count * sizeof(float));
    e->tensor = t;
    el_append(&f->params, e);
}

static int ox_fail(ox_build *b, const char *fmt, const char *a)
{
    snprintf(b->err, sizeof(b->err), fmt, a);
    return -1;
}

static struct pyelement *ox_value(ox_build *b, const char *name);

/* the function element of ONNX node `idx` under the PyTorch-dump operator name `pyop`; activations `ins` become its
 * inputs (built recursively, in order), the caller then adds parameters and calls thb_build_py_module */
static struct pyelement *ox_function(ox_build *b, int idx, const char *pyop, const char *const *ins, int nins)
{
    if (idx + 1 >= MAXPYNODES) { ox_fail(b, "too many nodes%s", ""); return 0; }
    struct pyelement *e = el_new(ELTYPE_FUNCTION, pyop);
    e->function.id = idx + 1;
    for (int k = 0; k < nins; k++) {
        struct pyelement *c = ox_value(b, ins[k]);
        if (!c) { freepynet(e); return 0; }
        el_append(&e->function.inputs, c);
        e->function.ninputs++;
    }
    return e;
}

/* weights and bias of a convolution with, optionally, a batch normalisation folded in (absorb_bn, onnx.cc:472-570:
 * invstd = 1/sqrtf(var + eps); w *= invstd; bias = (bias - mean)*invstd; then w *= gamma; bias = bias*gamma + beta)
 * and a constant added to the bias */
static int ox_conv_params(ox_build *b, struct pyfunction *f, const ox_node *cn, int transposed, const ox_node *bn,
                          const ox_tensor *extra_bias)
{
    const ox_tensor *w = ox_init(b->g, cn->in[1]), *bias = cn->nin > 2 ? ox_init(b->g, cn->in[2]) : 0;
    if (!w || w->data_type != 1 || w->ndims != 4) return ox_fail(b, "convolution %s has no 4-D float weight", cn->out[0]);
    const long cout = transposed ? w->dims[1] : w->dims[0];
    const long per_o = transposed ? w->dims[2] * w->dims[3] : w->dims[1] * w->dims[2] * w->dims[3];
    long wcount = w->dims[0] * w->dims[1] * w->dims[2] * w->dims[3];
    if (w->count < wcount || (bias && bias->count < cout)) return ox_fail(b, "short tensor data in %s", cn->out[0]);
    float *wd = malloc((size_t)wcount * sizeof(float)), *bd = 0;
    memcpy(wd, w->f, (size_t)wcount * sizeof(float));
    if (bias || bn || extra_bias) {
        bd = calloc((size_t)cout, sizeof(float));
        if (bias) memcpy(bd, bias->f, (size_t)cout * sizeof(float));
    }
    if (bn) {
        const ox_tensor *gm = ox_init(b->g, bn->in[1]), *bt = ox_init(b->g, bn->in[2]), *mn = ox_init(b->g, bn->in[3]),
                        *vr = ox_init(b->g, bn->in[4]);
        const float eps = ox_float(bn, "epsilon", 1e-5f);
        if (!gm || !bt || !mn || !vr || gm->count < cout || bt->count < cout || mn->count < cout || vr->count < cout) {
            free(wd); free(bd);
            return ox_fail(b, "batch normalisation %s lacks its four tensors", bn->out[0]);
        }
        for (long o = 0; o < cout; o++) {
            const float invstd = 1 / sqrtf(vr->f[o] + eps);
            if (transposed) {
                for (long i = 0; i < w->dims[0]; i++)
                    for (long j = 0; j < per_o; j++) {
                        float *p = &wd[(i * cout + o) * per_o + j];
                        *p *= invstd;
                        *p *= gm->f[o];
                    }
            } else
                for (long j = 0; j < per_o; j++) {
                    wd[o * per_o + j] *= invstd;
                    wd[o * per_o + j] *= gm->f[o];
                }
            bd[o] = (bd[o] - mn->f[o]) * invstd;
            bd[o] = bd[o] * gm->f[o] + bt->f[o];
        }
    }
    if (extra_bias) {
        if (extra_bias->data_type != 1 || extra_bias->count != cout) {
            free(wd); free(bd);
            return ox_fail(b, "Add of a constant to %s: number of elements mismatch", cn->out[0]);
        }
        for (long o = 0; o < cout; o++) bd[o] += extra_bias->f[o];
    }
    par_tensor(f, "", wd, w->dims, 4);
    if (bd) par_tensor(f, "", bd, &cout, 1);
    free(wd); free(bd);
    return 0;
}

/* first activation (non-constant) input of a node, skipping Constant producers and initializers */
static const char *ox_act_input(const ox_build *b, const ox_node *n, int skip)
{
    for (int k = 0; k < n->nin; k++)
        if (*n->in[k] && !ox_init(b->g, n->in[k]) && skip-- == 0) return n->in[k];
    return 0;
}

static struct pyelement *ox_conv(ox_build *b, int idx, const ox_node *bn, const ox_tensor *extra_bias)
{
    const ox_node *n = &b->g->nodes[idx];
    const int transposed = !strcmp(n->op, "ConvTranspose");
    int padH, padW, padH2, padW2, dH, dW, dlH, dlW, aH = 0, aW = 0, refl = 0, autopad = 0;
    ox_ints2(n, "pads", 0, 0, &padH, &padW);
    /* onnx: pads = {top, left, bottom, right}; SpatialConvolution.c:94-97 keeps the ending pair as padH2 / padW2 */
    padH2 = padH; padW2 = padW;
    {
        const ox_attr *pa = ox_attr_of(n, "pads");
        if (pa && pa->nints >= 4) { padH2 = (int)pa->ints[2]; padW2 = (int)pa->ints[3]; }
        const ox_attr *ap = ox_attr_of(n, "auto_pad");
        if (ap && ap->s) autopad = !strcmp(ap->s, "SAME_UPPER") ? 1 : !strcmp(ap->s, "SAME_LOWER") ? 2 : 0;   /* :88-93 */
    }
    ox_ints2(n, "dilations", 0, 1, &dlH, &dlW);
    ox_ints2(n, "strides", 0, 1, &dH, &dW);
    if (transposed) ox_ints2(n, "output_padding", 0, 0, &aH, &aW);
    /* a constant-mode Pad in front of a Conv adds to its padding and disappears (onnx.cc:667-700) */
    const char *src = n->in[0];
    int pidx = ox_producer(b->g, src);
    if (!transposed && pidx >= 0 && !strcmp(b->g->nodes[pidx].op, "Pad")) {
        const ox_node *pn = &b->g->nodes[pidx];
        const ox_attr *mode = ox_attr_of(pn, "mode"), *pads = ox_attr_of(pn, "pads");
        const ox_tensor *pt = pn->nin > 1 ? ox_init(b->g, pn->in[1]) : 0;
        /* onnx.cc:677-690: "reflect" is noted in refl_pad, anything but "constant" and "reflect" is an error */
        if (mode && mode->s && !strcmp(mode->s, "reflect")) refl = 1;
        else if (mode && mode->s && *mode->s && strcmp(mode->s, "constant")) { ox_fail(b, "Unsupported padding type %s", mode->s); return 0; }
        if (pads && pads->nints >= 4) {
            padH += (int)pads->ints[2]; padW += (int)pads->ints[3];
            if (pads->nints >= 8) { padH2 += (int)pads->ints[6]; padW2 += (int)pads->ints[7]; }
            else { padH2 += (int)pads->ints[2]; padW2 += (int)pads->ints[3]; }
        } else if (pt && pt->data_type == 7 && pt->count >= 4) {
            padH += (int)pt->i64[2]; padW += (int)pt->i64[3];
            if (pt->count >= 8) { padH2 += (int)pt->i64[6]; padW2 += (int)pt->i64[7]; }
            else { padH2 += (int)pt->i64[2]; padW2 += (int)pt->i64[3]; }
        } else { ox_fail(b, "Pad %s without pads", pn->out[0]); return 0; }
        src = pn->in[0];
    }
    struct pyelement *e = ox_function(b, idx, transposed ? "ConvTransposedNd" : "ConvNd", &src, 1);
    if (!e) return 0;
    if (ox_conv_params(b, &e->function, n, transposed, bn, extra_bias)) { freepynet(e); return 0; }
    par_ivec(&e->function, "padding", padH, padW);
    par_ivec(&e->function, "stride", dH, dW);
    if (transposed) par_ivec(&e->function, "output_padding", aH, aW);
    else {
        /* what the reference's loader parses and none of its engines reads (SpatialConvolution.c:88-109) */
        par_ivec(&e->function, "padding2", padH2, padW2);
        par_ivec(&e->function, "dilation", dlH, dlW);
        par_int(&e->function, "autopad", autopad);
        par_int(&e->function, "refl_pad", refl);
    }
    return e;
}

/* the element that delivers tensor `name`: the network input, a reference to an element built earlier, or a new one */
static struct pyelement *ox_value(ox_build *b, const char *name)
{
    ox_graph *g = b->g;
    int idx = ox_producer(g, name);
    if (idx < 0) {
        for (int i = 0; i < g->ninputs; i++)
            if (!strcmp(g->inputs[i], name) && !ox_init(g, name)) return el_new(ELTYPE_INPUT, 0);
        ox_fail(b, "tensor %s has no producer", name);
        return 0;
    }
    if (b->built[idx]) {
        struct pyelement *r = el_new(ELTYPE_OUTPUTID, 0);
        r->ivalue = b->built[idx];
        return r;
    }
    const ox_node *n = &g->nodes[idx];
    const char *op = n->op;
    struct pyelement *e = 0;
    int stands_for = -1; /* a second ONNX node this element also stands for (a folded producer) */

    if (!strcmp(op, "Conv") || !strcmp(op, "ConvTranspose"))
        e = ox_conv(b, idx, 0, 0);
    else if (!strcmp(op, "BatchNormalization")) {
        int c = ox_producer(g, n->in[0]);
        if (c >= 0 && !b->built[c] && (!strcmp(g->nodes[c].op, "Conv") || !strcmp(g->nodes[c].op, "ConvTranspose"))) {
            e = ox_conv(b, c, n, 0);   /* absorbed: the convolution's element stands for both nodes */
            stands_for = c;
        } else {
            const ox_tensor *gm = ox_init(g, n->in[1]), *bt = ox_init(g, n->in[2]), *mn = ox_init(g, n->in[3]), *vr = ox_init(g, n->in[4]);
            if (!gm || !bt || !mn || !vr) { ox_fail(b, "batch normalisation %s lacks its four tensors", n->out[0]); return 0; }
            if (!(e = ox_function(b, idx, "BatchNorm", (const char *const *)&n->in[0], 1))) return 0;
            par_tensor(&e->function, "", gm->f, &gm->count, 1);
            par_tensor(&e->function, "", bt->f, &bt->count, 1);
            par_tensor(&e->function, "running_mean", mn->f, &mn->count, 1);
            par_tensor(&e->function, "running_var", vr->f, &vr->count, 1);
            par_float(&e->function, "eps", ox_float(n, "epsilon", 1e-5f));
        }
    } else if ((!strcmp(op, "Add") || !strcmp(op, "Sum")) && n->nin == 2 && (ox_init(g, n->in[0]) || ox_init(g, n->in[1]))) {
        /* a constant added to the output of a convolution is (part of) its bias (onnx.cc:605-660) */
        const int ci = ox_init(g, n->in[0]) ? 0 : 1;
        int c = ox_producer(g, n->in[!ci]);
        if (c < 0 || b->built[c] || (strcmp(g->nodes[c].op, "Conv") && strcmp(g->nodes[c].op, "ConvTranspose"))) {
            ox_fail(b, "Add of a constant to %s, which is not a convolution", n->in[!ci]);
            return 0;
        }
        e = ox_conv(b, c, 0, ox_init(g, n->in[ci]));
        stands_for = c;
    } else if (!strcmp(op, "Add") || !strcmp(op, "Sum") || !strcmp(op, "Sub") || !strcmp(op, "Concat")) {
        e = ox_function(b, idx, !strcmp(op, "Concat") ? "Concat" : !strcmp(op, "Sub") ? "Sub" : "Add", (const char *const *)n->in, n->nin);
        if (e && !strcmp(op, "Concat")) par_int(&e->function, "dim", (int)ox_int(n, "axis", 1));
    } else if (!strcmp(op, "Gemm") || !strcmp(op, "MatMul")) {
        const ox_tensor *w = ox_init(g, n->in[1]), *bias = n->nin > 2 ? ox_init(g, n->in[2]) : 0;
        if (!w || w->data_type != 1 || w->ndims != 2 || w->count < w->dims[0] * w->dims[1]) { ox_fail(b, "Gemm %s needs a constant 2-D weight", n->out[0]); return 0; }
        if (!(e = ox_function(b, idx, "Linear", (const char *const *)&n->in[0], 1))) return 0;
        /* Linear.c onnxload: the weight is [out][in]; without transB it arrives as [in][out] and is transposed */
        const int transB = !strcmp(op, "Gemm") && ox_int(n, "transB", 0);
        long dims[2] = {transB ? w->dims[0] : w->dims[1], transB ? w->dims[1] : w->dims[0]};
        float *wd = malloc((size_t)w->count * sizeof(float));
        if (transB) memcpy(wd, w->f, (size_t)(dims[0] * dims[1]) * sizeof(float));
        else
            for (long o = 0; o < dims[0]; o++)
                for (long i = 0; i < dims[1]; i++) wd[o * dims[1] + i] = w->f[i * dims[0] + o];
        par_tensor(&e->function, "", wd, dims, 2);
        free(wd);
        if (bias && bias->count >= dims[0] && ox_float(n, "beta", 1.f) != 0.f) par_tensor(&e->function, "", bias->f, &dims[0], 1);
    } else if (!strcmp(op, "MaxPool") || !strcmp(op, "AveragePool") || !strcmp(op, "GlobalAveragePool") || !strcmp(op, "ReduceMean")) {
        int kH = 0, kW = 0, dH = 1, dW = 1, padH = 0, padW = 0;
        if (!strcmp(op, "ReduceMean")) {
            /* onnx.cc:50, SpatialAveragePooling.c:47-51: the mean over rows and columns is an average pooling over the
             * whole map (no kernel_shape: kernel 0); any other axes are refused with the reference's message */
            const ox_attr *ax = ox_attr_of(n, "axes");
            if (ax && !(ax->nints == 0 || (ax->nints == 2 && ax->ints[0] == 2 && ax->ints[1] == 3))) {
                ox_fail(b, "ReduceMean along channel is not supported (%s)", n->out[0]);
                return 0;
            }
        } else if (strcmp(op, "GlobalAveragePool")) {
            ox_ints2(n, "kernel_shape", 0, 1, &kH, &kW);
            ox_ints2(n, "strides", 0, 1, &dH, &dW);
            ox_ints2(n, "pads", 0, 0, &padH, &padW);
        }
        if (!(e = ox_function(b, idx, !strcmp(op, "MaxPool") ? "MaxPool2d" : "AvgPool2d", (const char *const *)&n->in[0], 1))) return 0;
        par_ivec(&e->function, "padding", padH, padW);
        par_ivec(&e->function, "stride", dH, dW);
        par_ivec(&e->function, "kernel_size", kH, kW);
        par_int(&e->function, "ceil_mode", (int)ox_int(n, "ceil_mode", 0));
    } else if (!strcmp(op, "Relu")) {
        if (!(e = ox_function(b, idx, "Threshold", (const char *const *)&n->in[0], 1))) return 0;
        par_float(&e->function, "threshold", 0.f);
        par_float(&e->function, "value", 0.f);
        par_int(&e->function, "inplace", 0);
    } else if (!strcmp(op, "LeakyRelu")) {
        /* onnx.cc:36, Threshold.c:30-35: a Threshold record with the node's alpha -- 0 when the attribute is absent, which
         * makes it a ReLU (Threshold.c:55-60), not the 0.01 the operator's specification gives */
        if (!(e = ox_function(b, idx, "Threshold", (const char *const *)&n->in[0], 1))) return 0;
        par_float(&e->function, "threshold", 0.f);
        par_float(&e->function, "value", 0.f);
        par_int(&e->function, "inplace", 0);
        par_float(&e->function, "alpha", ox_float(n, "alpha", 0.f));
    } else if (!strcmp(op, "PRelu")) {
        /* onnx.cc:35, PReLU.c:21-29: the slopes are the second input, one per plane: its first dimension */
        const ox_tensor *w = n->nin > 1 ? ox_init(g, n->in[1]) : 0;
        if (!w || w->data_type != 1 || w->ndims < 1 || w->count < w->dims[0]) { ox_fail(b, "PRelu %s needs a constant slope tensor", n->out[0]); return 0; }
        if (!(e = ox_function(b, idx, "PReLU", (const char *const *)&n->in[0], 1))) return 0;
        par_tensor(&e->function, "", w->f, &w->dims[0], 1);
    } else if (!strcmp(op, "Dropout") || !strcmp(op, "Identity"))
        e = ox_function(b, idx, "Dropout", (const char *const *)&n->in[0], 1);
    else if (!strcmp(op, "Softmax") || !strcmp(op, "Sigmoid") || !strcmp(op, "Tanh") || !strcmp(op, "LogSoftmax"))
        e = ox_function(b, idx, op, (const char *const *)&n->in[0], 1);
    else if (!strcmp(op, "Max"))            /* onnx.cc:52: elementwise maximum of all inputs */
        e = ox_function(b, idx, "Cmax", (const char *const *)n->in, n->nin);
    else if (!strcmp(op, "Slice")) {        /* Slice.c:17-32: first entry of axes / starts / ends */
        int ax = 0, from = 0, to = 0, unused = 0;
        ox_ints2(n, "axes", 0, 0, &ax, &unused);
        ox_ints2(n, "starts", 0, 0, &from, &unused);
        ox_ints2(n, "ends", 0, 0, &to, &unused);
        if (!(e = ox_function(b, idx, "Slice", (const char *const *)&n->in[0], 1))) return 0;
        par_int(&e->function, "axis", ax);
        par_int(&e->function, "from", from);
        par_int(&e->function, "to", to);
    } else if (!strcmp(op, "Upsample")) {   /* Upsample.c:4-16: width_scale / height_scale, else scales[3] / scales[2] */
        float ws = ox_float(n, "width_scale", 0.f), hs = ox_float(n, "height_scale", 0.f);
        if (ws == 0.f && hs == 0.f) {
            const ox_attr *sa = ox_attr_of(n, "scales");
            if (sa && sa->nfloats >= 4) { hs = sa->floats[2]; ws = sa->floats[3]; }
        }
        if (!(e = ox_function(b, idx, "Upsample", (const char *const *)&n->in[0], 1))) return 0;
        par_float(&e->function, "width_scale", ws);
        par_float(&e->function, "height_scale", hs);
    }
    else if (!strcmp(op, "Flatten") || !strcmp(op, "Reshape")) {
        /* View.c: the batch dimension stays, everything else becomes one dimension */
        if (!strcmp(op, "Reshape")) {
            const ox_tensor *shp = n->nin > 1 ? ox_init(g, n->in[1]) : 0;
            const ox_attr *sa = ox_attr_of(n, "shape");
            const long nd = shp ? shp->count : sa ? sa->nints : 0;
            if (nd != 2) { ox_fail(b, "Reshape %s to other than [batch, features] is not supported", n->out[0]); return 0; }
        }
        if (!(e = ox_function(b, idx, "View", (const char *const *)&n->in[0], 1))) return 0;
        struct pyelement *sz = el_new(ELTYPE_INTVECT, "sizes");
        sz->ivect[0] = -1; sz->ivect[1] = -1;
        el_append(&e->function.params, sz);
    } else {
        ox_fail(b, "Unsupported node type %s", op);
        return 0;
    }
    if (!e) return 0;
    b->all[e->function.id] = e;
    b->built[idx] = e->function.id;
    if (stands_for >= 0) b->built[stands_for] = e->function.id;
    thb_build_py_module(e->name, &e->function);
    return e;
}

struct pyelement *loadonnx(const char *path, struct pyelement **allpynodes, char *err, size_t errlen)
{
    FILE *fp = fopen(path, "rb");
    if (!fp) return 0;
    fseek(fp, 0, SEEK_END);
    long size = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    uint8_t *buf = size > 0 ? malloc((size_t)size) : 0;
    if (!buf || fread(buf, 1, (size_t)size, fp) != (size_t)size) { fclose(fp); free(buf); return 0; }
    fclose(fp);

    ox_graph g;
    memset(&g, 0, sizeof(g));
    pbuf m = {buf, buf + size}, sub, graph = {0, 0};
    int field, wt, ok = 1;
    uint64_t v;
    while (m.p < m.end && ok) {
        if (pb_next(&m, &field, &wt, &v, &sub)) ok = 0;
        else if (field == 7 && wt == 2) graph = sub;
    }
    struct pyelement *root = 0;
    ox_build b;
    memset(&b, 0, sizeof(b));
    if (!ok || !graph.p || ox_parse_graph(graph, &g))
        snprintf(b.err, sizeof(b.err), "not an ONNX model (no readable graph)");
    else if (!g.output)
        snprintf(b.err, sizeof(b.err), "the ONNX graph names no output");
    else {
        b.g = &g;
        b.all = allpynodes;
        b.built = calloc((size_t)g.nnodes, sizeof(int));
        root = ox_value(&b, g.output);
        if (root && root->type != ELTYPE_FUNCTION) { freepynet(root); root = 0; snprintf(b.err, sizeof(b.err), "the ONNX graph computes nothing"); }
        free(b.built);
    }
    if (!root && err && errlen) snprintf(err, errlen, "%s", b.err);
    ox_graph_free(&g);
    free(buf);
    return root;
}
