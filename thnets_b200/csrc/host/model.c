/*
 * Lowering of a loaded network into a flat operator list.
 *
 * The reference executes its networks by walking containers (thapi.c:158-235, modules/Sequential.c,
 * Concat.c, ConcatTable.c) or the PyTorch element tree (pytorch.c:301-328).  Here both shapes are
 * flattened once into a topologically ordered list of `thb_node`s with explicit input edges and
 * private copies of every parameter, so that a converted network owns everything it needs after the
 * source network is freed.  The list keeps the reference's evaluation order (depth first, inputs in
 * file order), which is what defines operand order for CAddTable's a - b.
 */
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include "thb_internal.h"

typedef struct { int n, is_table, id[THB_MAXIN]; } val;

typedef struct {
    thb_model *m;
    char *err;
    size_t errlen;
    int memo[MAXPYNODES];
    /* max-pooling modules lowered so far (Torch7 route): an unpooling finds the pooling it undoes by identity */
    struct nnmodule *pool_mod[64];
    int pool_node[64], npools;
} builder;

static int fail(builder *b, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    if (b->err && b->errlen) vsnprintf(b->err, b->errlen, fmt, ap);
    va_end(ap);
    return -1;
}

static thb_node *new_node(builder *b, int op, int nin, const int *in)
{
    thb_model *m = b->m;
    if (m->nnodes == m->cap) {
        m->cap = m->cap ? m->cap * 2 : 64;
        m->nodes = realloc(m->nodes, m->cap * sizeof(thb_node));
    }
    thb_node *n = &m->nodes[m->nnodes++];
    memset(n, 0, sizeof(*n));
    n->op = op;
    n->nin = nin;
    for (int i = 0; i < nin; i++) n->in[i] = in[i];
    return n;
}
static int last_id(builder *b) { return b->m->nnodes - 1; }

/* contiguous private copy of a tensor's elements; NULL when the tensor has no storage */
static float *copy_tensor(THFloatTensor *t, long *count)
{
    long n = THFloatTensor_nElement(t);
    if (count) *count = n;
    if (!t || !t->storage || !t->storage->data || n <= 0) return 0;
    float *dst = malloc(sizeof(float) * n);
    const float *src = THFloatTensor_data(t);
    /* loaded tensors are dense; honour strides anyway for up to 4 dimensions */
    long idx = 0, s[4] = {1, 1, 1, 1}, st[4] = {0, 0, 0, 0};
    int off = 4 - t->nDimension;
    for (int i = 0; i < t->nDimension; i++) { s[off + i] = t->size[i]; st[off + i] = t->stride[i]; }
    for (long a = 0; a < s[0]; a++)
        for (long c = 0; c < s[1]; c++)
            for (long d = 0; d < s[2]; d++)
                for (long e = 0; e < s[3]; e++) dst[idx++] = src[a * st[0] + c * st[1] + d * st[2] + e * st[3]];
    return dst;
}

static int lower_leaf(builder *b, struct module *m, val in, val *out)
{
    thb_node *n;
    long cnt;
    out->n = 1;
    out->is_table = 0;
    if (in.is_table && m->type != MT_JoinTable && m->type != MT_CAddTable && m->type != MT_CSubTable && m->type != MT_Cmax)
        return fail(b, "module type %d cannot take a table of tensors", m->type);
    switch (m->type) {
    case MT_SpatialConvolution: case MT_SpatialConvolutionMM: case MT_SpatialConvolutionVirtMM: {
        struct SpatialConvolution *c = &m->SpatialConvolution;
        n = new_node(b, OP_CONV, 1, in.id);
        n->Cin = c->nInputPlane; n->Cout = c->nOutputPlane;
        n->kH = c->kH; n->kW = c->kW; n->dH = c->dH ? c->dH : 1; n->dW = c->dW ? c->dW : 1;
        n->padH = c->padH; n->padW = c->padW;
        n->pad2H = c->padH2; n->pad2W = c->padW2; n->dlH = c->dlH ? c->dlH : 1; n->dlW = c->dlW ? c->dlW : 1;
        n->autopad = c->autopad; n->refl_pad = c->refl_pad;
        if (!c->dlH && !c->dlW) { n->pad2H = n->padH; n->pad2W = n->padW; } /* a record no loader of ours filled: symmetric */
        n->weight = copy_tensor(c->weight, &cnt);
        if (!n->weight || cnt != (long)n->Cin * n->Cout * n->kH * n->kW)
            return fail(b, "convolution weight has %ld elements, expected %dx%dx%dx%d", cnt, n->Cout, n->Cin, n->kH, n->kW);
        n->bias = copy_tensor(c->bias, &cnt);
        if (n->bias && cnt != n->Cout) return fail(b, "convolution bias has %ld elements, expected %d", cnt, n->Cout);
        break;
    }
    case MT_SpatialFullConvolution: {
        struct SpatialFullConvolution *c = &m->SpatialFullConvolution;
        n = new_node(b, OP_DECONV, 1, in.id);
        n->Cin = (int)c->weight->size[0]; n->Cout = (int)c->weight->size[1];
        n->kH = c->kH; n->kW = c->kW; n->dH = c->dH ? c->dH : 1; n->dW = c->dW ? c->dW : 1;
        n->padH = c->padH; n->padW = c->padW; n->adjH = c->adjH; n->adjW = c->adjW;
        n->weight = copy_tensor(c->weight, &cnt);
        if (!n->weight || cnt != (long)n->Cin * n->Cout * n->kH * n->kW) return fail(b, "bad full-convolution weight");
        n->bias = copy_tensor(c->bias, &cnt);
        if (n->bias && cnt != n->Cout) return fail(b, "bad full-convolution bias");
        break;
    }
    case MT_Linear: {
        struct Linear *l = &m->Linear;
        if (l->commute) return fail(b, "Linear with commuted operands is not supported");
        n = new_node(b, OP_LINEAR, 1, in.id);
        n->Cout = (int)l->weight->size[0]; n->Cin = (int)l->weight->size[1];
        n->kH = n->kW = n->dH = n->dW = 1;
        n->weight = copy_tensor(l->weight, &cnt);
        if (!n->weight || cnt != (long)n->Cin * n->Cout) return fail(b, "bad Linear weight");
        n->bias = copy_tensor(l->bias, &cnt);
        if (n->bias && cnt != n->Cout) return fail(b, "bad Linear bias");
        break;
    }
    case MT_SpatialBatchNormalization: {
        /* ((x - mean) * invstd) * w + b with invstd = 1/sqrt(var + eps) taken in double
         * (SpatialBatchNormalization.c:80-85), folded to x*scale + shift */
        struct SpatialBatchNormalization *s = &m->SpatialBatchNormalization;
        long c1, c2;
        float *mean = copy_tensor(s->running_mean, &c1), *var = copy_tensor(s->running_var, &c2);
        float *w = copy_tensor(s->weight, 0), *bb = copy_tensor(s->bias, 0);
        if (!mean || !var || c1 != c2) { free(mean); free(var); free(w); free(bb); return fail(b, "bad batch-norm statistics"); }
        n = new_node(b, OP_BN, 1, in.id);
        n->C = (int)c1;
        n->scale = malloc(sizeof(float) * c1);
        n->shift = malloc(sizeof(float) * c1);
        for (long i = 0; i < c1; i++) {
            float invstd = 1 / sqrt(var[i] + s->eps);
            n->scale[i] = invstd * (w ? w[i] : 1.f);
            n->shift[i] = (bb ? bb[i] : 0.f) - mean[i] * n->scale[i];
        }
        free(mean); free(var); free(w); free(bb);
        break;
    }
    case MT_Threshold:
        n = new_node(b, OP_ACT, 1, in.id);
        if (m->Threshold.alpha) { n->act_kind = THB_ACT_LEAKY; n->act_alpha = m->Threshold.alpha; }
        else { n->act_kind = THB_ACT_THRESHOLD; n->act_threshold = m->Threshold.threshold; n->act_value = m->Threshold.val; }
        break;
    case MT_Sigmoid: case MT_Tanh: /* reachable through the ONNX reader only, as in the reference (onnx.cc:59-60) */
        n = new_node(b, OP_ACT, 1, in.id);
        n->act_kind = m->type == MT_Sigmoid ? THB_ACT_SIGMOID : THB_ACT_TANH;
        break;
    case MT_PReLU:
        n = new_node(b, OP_ACT, 1, in.id);
        n->act_kind = THB_ACT_PRELU;
        n->slope = copy_tensor(m->PReLU.weight, &cnt);
        n->nslope = m->PReLU.nOutputPlane;
        if (!n->slope || (n->nslope && cnt != n->nslope)) return fail(b, "bad PReLU weight");
        break;
    case MT_SpatialMaxPooling: {
        struct SpatialMaxPooling *p = &m->SpatialMaxPooling;
        n = new_node(b, OP_MAXPOOL, 1, in.id);
        n->kH = p->kH; n->kW = p->kW; n->dH = p->dH; n->dW = p->dW; n->padH = p->padH; n->padW = p->padW;
        n->ceil_mode = p->ceil_mode;
        if (n->dH < 1 || n->dW < 1 || n->kH < 1 || n->kW < 1) return fail(b, "max pooling needs kernel and stride >= 1");
        break;
    }
    case MT_SpatialAveragePooling: {
        struct SpatialAveragePooling *p = &m->SpatialAveragePooling;
        n = new_node(b, OP_AVGPOOL, 1, in.id);
        n->kH = p->kH; n->kW = p->kW; n->dH = p->dH; n->dW = p->dW; n->padH = p->padH; n->padW = p->padW;
        n->ceil_mode = p->ceil_mode; n->count_include_pad = p->count_include_pad;
        if (n->dH < 1 || n->dW < 1) return fail(b, "average pooling needs an explicit stride >= 1");
        break;
    }
    case MT_SoftMax: new_node(b, OP_SOFTMAX, 1, in.id); break;
    case MT_View:
        n = new_node(b, OP_VIEW, 1, in.id);
        n->numElements = m->View.numElements;
        break;
    case MT_Reshape:
        /* Reshape.c:22-36: to `size` without a batch dimension, or to `batchsize` with the input's batch in front; built
         * for a one-dimensional target (the flatten in front of a classifier), where it is what View does */
        if (m->Reshape.nsize == 3) {
            n = new_node(b, OP_RESHAPE, 1, in.id);
            n->numElements = m->Reshape.numElements;
            n->batch_mode = m->Reshape.batchMode;
            for (int k = 0; k < 3; k++) n->reshape[k] = (int)m->Reshape.size[k];
            break;
        }
        if (m->Reshape.nsize > 1) return fail(b, "Reshape to two or four dimensions is not supported by the B200 engine");
        n = new_node(b, OP_VIEW, 1, in.id);
        n->numElements = m->Reshape.numElements;
        break;
    case MT_Dropout: {
        /* identity for v2 dropout; anything else scales by 1 - p (Dropout.c:46-51) */
        float f = m->Dropout.v2 != 1 ? 1 - m->Dropout.p : 1.f;
        n = new_node(b, f == 1.f ? OP_ALIAS : OP_SCALE, 1, in.id);
        n->factor = f;
        break;
    }
    case MT_JoinTable:
        if (!in.is_table) return fail(b, "JoinTable needs a table of tensors");
        n = new_node(b, OP_CONCAT, in.n, in.id);
        n->dim = m->JoinTable.dimension;
        break;
    case MT_CAddTable: case MT_CSubTable: {
        /* CAddTable.c:59-83: two inputs -> a - b (a + b for CSubTable); otherwise start from input 0 and
         * add (subtract) every input, input 0 included */
        if (!in.is_table) return fail(b, "CAddTable needs a table of tensors");
        int sub = m->type == MT_CSubTable;
        if (in.n == 2) {
            n = new_node(b, OP_COMBINE, 2, in.id);
            n->coef[0] = 1.f;
            n->coef[1] = sub ? 1.f : -1.f;
        } else {
            int ids[THB_MAXIN];
            if (in.n + 1 > 8) return fail(b, "CAddTable with %d inputs is not supported", in.n);
            ids[0] = in.id[0];
            for (int i = 0; i < in.n; i++) ids[i + 1] = in.id[i];
            n = new_node(b, OP_COMBINE, in.n + 1, ids);
            n->coef[0] = 1.f;
            for (int i = 1; i <= in.n; i++) n->coef[i] = sub ? -1.f : 1.f;
        }
        break;
    }
    case MT_Upsample:
        if (m->Upsample.height_scale != 2 || m->Upsample.width_scale != 2) return fail(b, "Only 2x upsampling is supported");
        new_node(b, OP_UPSAMPLE, 1, in.id);
        break;
    case MT_SpatialZeroPadding:
        n = new_node(b, OP_ZEROPAD, 1, in.id);
        n->pad_l = m->SpatialZeroPadding.pad_l; n->pad_r = m->SpatialZeroPadding.pad_r;
        n->pad_t = m->SpatialZeroPadding.pad_t; n->pad_b = m->SpatialZeroPadding.pad_b;
        break;
    case MT_Slice:
        n = new_node(b, OP_SLICE, 1, in.id);
        n->slice_axis = m->Slice.axis; n->slice_from = m->Slice.from; n->slice_to = m->Slice.to;
        break;
    case MT_Cmax:
        if (!in.is_table || in.n < 1) return fail(b, "Cmax needs a table of tensors");
        new_node(b, OP_CMAX, in.n, in.id);
        break;
    case MT_LogSoftMax: new_node(b, OP_LOGSOFTMAX, 1, in.id); break;
    case MT_Normalize: new_node(b, OP_NORMALIZE, 1, in.id); break;
    case MT_SpatialMaxUnpooling: {
        /* SpatialMaxUnpooling.c:60-71: the pooling module it undoes is found by identity among the modules seen so far;
         * the unpooling reads that pooling's input again to locate each window's maximum */
        int pool = -1;
        for (int k = 0; k < b->npools; k++)
            if (b->pool_mod[k] == m->SpatialMaxUnpooling.pooling) pool = b->pool_node[k];
        if (pool < 0 || !m->SpatialMaxUnpooling.pooling) return fail(b, "SpatialMaxUnpooling refers to no SpatialMaxPooling of this network");
        int ids[2] = {in.id[0], b->m->nodes[pool].in[0]};
        const thb_node pn = b->m->nodes[pool];
        n = new_node(b, OP_UNPOOL, 2, ids);
        n->kH = pn.kH; n->kW = pn.kW; n->dH = pn.dH; n->dW = pn.dW; n->padH = pn.padH; n->padW = pn.padW; n->ceil_mode = pn.ceil_mode;
        break;
    }
    default: return fail(b, "module type %d is not supported by the B200 engine", m->type);
    }
    out->id[0] = last_id(b);
    if (m->type == MT_SpatialMaxPooling && m->nnmodule && b->npools < 64) {
        b->pool_mod[b->npools] = m->nnmodule;
        b->pool_node[b->npools++] = out->id[0];
    }
    return 0;
}

static int lower_module(builder *b, struct module *m, val in, val *out);

static int lower_chain(builder *b, struct network *net, val in, val *out)
{
    val cur = in;
    for (int i = 0; i < net->nelem; i++) {
        val next;
        if (lower_module(b, &net->modules[i], cur, &next)) return -1;
        cur = next;
    }
    *out = cur;
    return 0;
}

static int lower_module(builder *b, struct module *m, val in, val *out)
{
    if (m->type == MT_Sequential) return lower_chain(b, m->Sequential.net, in, out);
    if (m->type == MT_ConcatTable || m->type == MT_Concat) {
        struct network *sub = m->type == MT_Concat ? m->Concat.net : m->ConcatTable.net;
        val table = {0, 1, {0}};
        if (sub->nelem > THB_MAXIN) return fail(b, "container with %d branches", sub->nelem);
        for (int i = 0; i < sub->nelem; i++) {
            val branch;
            if (lower_module(b, &sub->modules[i], in, &branch)) return -1;
            if (branch.is_table) return fail(b, "nested tables are not supported");
            table.id[table.n++] = branch.id[0];
        }
        if (m->type == MT_ConcatTable) { *out = table; return 0; }
        thb_node *n = new_node(b, OP_CONCAT, table.n, table.id);
        n->dim = m->Concat.dimension;
        out->n = 1; out->is_table = 0; out->id[0] = last_id(b);
        return 0;
    }
    return lower_leaf(b, m, in, out);
}

static int lower_py(builder *b, struct pyelement *e, int *id)
{
    if (e->type == ELTYPE_INPUT) { *id = 0; return 0; }
    if (e->type == ELTYPE_OUTPUTID) {
        if ((unsigned)e->ivalue >= MAXPYNODES || b->memo[e->ivalue] < 0) return fail(b, "reference to an unknown node %d", e->ivalue);
        *id = b->memo[e->ivalue];
        return 0;
    }
    if (e->type != ELTYPE_FUNCTION) return fail(b, "unexpected element type %d in the graph", e->type);
    val in = {0, 0, {0}}, out;
    for (struct elemlist *l = e->function.inputs; l; l = l->next) {
        if (in.n >= THB_MAXIN) return fail(b, "too many inputs");
        if (lower_py(b, l->elem, &in.id[in.n])) return -1;
        in.n++;
    }
    int t = e->function.module.type;
    in.is_table = (t == MT_CAddTable || t == MT_CSubTable || t == MT_JoinTable || t == MT_Cmax);
    if (!in.is_table && in.n != 1) return fail(b, "function %s has %d inputs", e->name, in.n);
    if (lower_leaf(b, &e->function.module, in, &out)) return -1;
    b->memo[e->function.id] = out.id[0];
    *id = out.id[0];
    return 0;
}

static builder *builder_new(char *err, size_t errlen)
{
    builder *b = calloc(1, sizeof(*b));
    b->m = calloc(1, sizeof(thb_model));
    b->m->refs = 1;
    b->err = err;
    b->errlen = errlen;
    for (int i = 0; i < MAXPYNODES; i++) b->memo[i] = -1;
    new_node(b, OP_INPUT, 0, 0);
    return b;
}

thb_model *thb_model_from_network(THNETWORK *net, char *err, size_t errlen)
{
    builder *b = builder_new(err, errlen);
    int rc, out = 0;
    if (net->pynet) rc = lower_py(b, net->pynet, &out);
    else if (net->net) {
        val in = {1, 0, {0}}, o;
        rc = lower_chain(b, net->net, in, &o);
        if (!rc && o.is_table) rc = fail(b, "the network ends in a table of tensors");
        out = o.id[0];
    } else
        rc = fail(b, "the network holds no graph");
    thb_model *m = b->m;
    free(b);
    if (rc) { thb_model_release(m); return 0; }
    m->output = out;
    return m;
}

thb_model *thb_model_from_module(struct module *mod, char *err, size_t errlen)
{
    builder *b = builder_new(err, errlen);
    val in = {1, 0, {0}}, o;
    int rc = lower_module(b, mod, in, &o);
    thb_model *m = b->m;
    free(b);
    if (rc || o.is_table) { thb_model_release(m); return 0; }
    m->output = o.id[0];
    return m;
}

void thb_model_release(thb_model *m)
{
    if (!m || --m->refs > 0) return;
    for (int i = 0; i < m->nnodes; i++) {
        free(m->nodes[i].weight); free(m->nodes[i].bias); free(m->nodes[i].scale);
        free(m->nodes[i].shift); free(m->nodes[i].slope);
    }
    free(m->nodes);
    free(m);
}
