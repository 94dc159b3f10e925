/*
 * Reader of Torch7's binary serialisation (what `torch.save` writes): produces the thobject tree of
 * the public header.  Same format rules as the reference's loader (thload.c:119-406): little endian,
 * every table / torch object carries an index, an index seen before is a back-reference, `long` is
 * 8 bytes (or 4 on files written by 32-bit Torch), function objects are skipped.
 */
#include <stdio.h>
#include <string.h>
#include "thnets.h"
#include "thb_internal.h"

struct reader {
    FILE *fp;
    int next_idx, longsize, cap;
    struct thobject *seen; /* header copy (type + pointer) of every indexed object, by index */
};

static int rd_object(struct reader *r, struct thobject *obj);

static int rd_i32(struct reader *r, int *v) { return fread(v, 4, 1, r->fp) == 1 ? 0 : ERR_READFILE; }
static int rd_f64(struct reader *r, double *v) { return fread(v, 8, 1, r->fp) == 1 ? 0 : ERR_READFILE; }
static int rd_long(struct reader *r, long *v)
{
    if (r->longsize == 4) {
        int t;
        if (fread(&t, 4, 1, r->fp) != 1) return ERR_READFILE;
        *v = t;
        return 0;
    }
    long long t;
    if (fread(&t, 8, 1, r->fp) != 1) return ERR_READFILE;
    *v = (long)t;
    return 0;
}
static int rd_string(struct reader *r, char **s, int *len)
{
    if (rd_i32(r, len)) return ERR_READFILE;
    if (*len < 0 || *len > (1 << 24)) return ERR_CORRUPTED;
    *s = malloc(*len + 1);
    if (*len && fread(*s, *len, 1, r->fp) != 1) {
        free(*s);
        *s = 0;
        return ERR_READFILE;
    }
    (*s)[*len] = 0;
    return 0;
}

static void remember(struct reader *r, int idx, const struct thobject *obj)
{
    if (idx >= r->cap) {
        int ncap = r->cap * 2 > idx + 1 ? r->cap * 2 : idx + 1;
        r->seen = realloc(r->seen, ncap * sizeof(*r->seen));
        memset(r->seen + r->cap, 0, (ncap - r->cap) * sizeof(*r->seen));
        r->cap = ncap;
    }
    r->seen[idx] = *obj;
}

static int scalar_type(const char *name)
{
    static const struct { const char *n; int t; } map[] = {
        {"Byte", TYPE_BYTE}, {"Char", TYPE_CHAR}, {"Short", TYPE_SHORT}, {"Int", TYPE_INT}, {"Long", TYPE_LONG},
        {"Float", TYPE_FLOAT}, {"Cuda", TYPE_FLOAT}, {"Double", TYPE_DOUBLE}};
    for (unsigned i = 0; i < sizeof(map) / sizeof(map[0]); i++)
        if (!strcmp(name, map[i].n)) return map[i].t;
    return ERR_CORRUPTED;
}
static int scalar_size(int t)
{
    switch (t) {
    case TYPE_BYTE: case TYPE_CHAR: return 1;
    case TYPE_SHORT: return 2;
    case TYPE_INT: case TYPE_FLOAT: return 4;
    case TYPE_LONG: case TYPE_DOUBLE: return 8;
    }
    return ERR_CORRUPTED;
}

/* a back-reference shares the object it points at */
static int share(struct reader *r, int idx, struct thobject *obj, int want_table)
{
    if (idx < 1 || idx >= r->next_idx || idx >= r->cap || !r->seen[idx].type) return ERR_CORRUPTED;
    const struct thobject *o = &r->seen[idx];
    if (want_table) {
        if (o->type != TYPE_TABLE) return ERR_CORRUPTED;
        obj->type = TYPE_TABLE;
        obj->table = o->table;
        obj->table->nrefs++;
        return 0;
    }
    *obj = *o;
    switch (o->type) {
    case TYPE_TENSOR: obj->tensor->nrefs++; return 0;
    case TYPE_STORAGE: obj->storage->nrefs++; return 0;
    case TYPE_NNMODULE: obj->nnmodule->nrefs++; return 0;
    }
    return ERR_CORRUPTED;
}

static int rd_table(struct reader *r, struct thobject *obj)
{
    int idx, rc;
    if (rd_i32(r, &idx)) return ERR_READFILE;
    if (idx != r->next_idx) return share(r, idx, obj, 1);
    r->next_idx++;
    obj->type = TYPE_TABLE;
    obj->table = calloc(1, sizeof(*obj->table));
    obj->table->idx = idx;
    obj->table->nrefs = 1;
    remember(r, idx, obj);
    int n;
    if (rd_i32(r, &n)) return ERR_READFILE;
    if (n < 0 || n > (1 << 24)) return ERR_CORRUPTED;
    obj->table->records = calloc(n ? n : 1, sizeof(struct threcord));
    for (int i = 0; i < n; i++) {
        obj->table->nelem = i + 1;
        if ((rc = rd_object(r, &obj->table->records[i].name))) return rc;
        if ((rc = rd_object(r, &obj->table->records[i].value))) return rc;
    }
    obj->table->nelem = n;
    return 0;
}

static int rd_storage(struct reader *r, struct thobject *obj, int idx, const char *scalar)
{
    obj->type = TYPE_STORAGE;
    struct storage *s = obj->storage = calloc(1, sizeof(*s));
    s->idx = idx;
    s->nrefs = 1;
    s->scalartype = scalar_type(scalar);
    remember(r, idx, obj);
    int es = scalar_size(s->scalartype);
    if (es < 0) return es;
    if (rd_long(r, &s->nelem)) return ERR_READFILE;
    if (s->nelem < 0) return ERR_CORRUPTED;
    {
        /* a storage cannot hold more elements than the file has bytes left for (truncated or forged length) */
        const long here = ftell(r->fp);
        if (here >= 0 && !fseek(r->fp, 0, SEEK_END)) {
            const long end = ftell(r->fp);
            fseek(r->fp, here, SEEK_SET);
            const long per = s->scalartype == TYPE_LONG && r->longsize == 4 ? 4 : es;
            if (end >= here && s->nelem > (end - here) / per) return ERR_CORRUPTED;
        }
    }
    s->data = malloc((size_t)(s->nelem ? s->nelem : 1) * es);
    if (!s->data) THError("Out of memory loading a storage of %ld elements", s->nelem);
    if (s->scalartype == TYPE_LONG && r->longsize == 4) {
        for (long i = 0; i < s->nelem; i++) {
            int t;
            if (fread(&t, 4, 1, r->fp) != 1) return ERR_READFILE;
            ((long *)s->data)[i] = t;
        }
    } else if (s->nelem && fread(s->data, es, s->nelem, r->fp) != (size_t)s->nelem)
        return ERR_READFILE;
    return 0;
}

static int rd_tensor(struct reader *r, struct thobject *obj, int idx, const char *scalar)
{
    obj->type = TYPE_TENSOR;
    struct tensor *t = obj->tensor = calloc(1, sizeof(*t));
    t->idx = idx;
    t->nrefs = 1;
    t->scalartype = scalar_type(scalar);
    remember(r, idx, obj);
    if (rd_i32(r, &t->ndim)) return ERR_READFILE;
    if (t->ndim < 0 || t->ndim > 16) return ERR_CORRUPTED;
    t->size = calloc(t->ndim ? t->ndim : 1, sizeof(long));
    t->stride = calloc(t->ndim ? t->ndim : 1, sizeof(long));
    for (int i = 0; i < t->ndim; i++)
        if (rd_long(r, &t->size[i])) return ERR_READFILE;
    for (int i = 0; i < t->ndim; i++)
        if (rd_long(r, &t->stride[i])) return ERR_READFILE;
    if (rd_long(r, &t->storageoffset)) return ERR_READFILE;
    t->storageoffset--; /* Lua offsets start at 1 */
    struct thobject st;
    int rc = rd_object(r, &st);
    if (rc) {
        freeobject(&st);
        return rc;
    }
    if (st.type == TYPE_STORAGE) t->storage = st.storage;
    else if (st.type != TYPE_NIL) {
        freeobject(&st);
        return ERR_CORRUPTED;
    }
    return 0;
}

static int ends_with(const char *s, const char *suffix)
{
    size_t a = strlen(s), b = strlen(suffix);
    return a >= b && !strcmp(s + a - b, suffix);
}

static int rd_torch(struct reader *r, struct thobject *obj)
{
    int idx, len, rc;
    char *version = 0, *cls = 0;
    if (rd_i32(r, &idx)) return ERR_READFILE;
    if (idx != r->next_idx) return share(r, idx, obj, 0);
    r->next_idx++;
    if (rd_string(r, &version, &len)) return ERR_READFILE;
    free(version);
    if (rd_string(r, &cls, &len)) return ERR_READFILE;
    if (!strncmp(cls, "torch.", 6) && ends_with(cls, "Tensor")) {
        cls[strlen(cls) - 6] = 0;
        rc = rd_tensor(r, obj, idx, cls + 6);
    } else if (!strncmp(cls, "torch.", 6) && ends_with(cls, "Storage")) {
        cls[strlen(cls) - 7] = 0;
        rc = rd_storage(r, obj, idx, cls + 6);
    } else if (!strncmp(cls, "nn.", 3)) {
        obj->type = TYPE_NNMODULE;
        obj->nnmodule = calloc(1, sizeof(*obj->nnmodule));
        obj->nnmodule->idx = idx;
        obj->nnmodule->nrefs = 1;
        obj->nnmodule->name = cls;
        cls = 0;
        remember(r, idx, obj);
        struct thobject fields;
        rc = rd_object(r, &fields);
        if (!rc && fields.type != TYPE_TABLE) rc = ERR_CORRUPTED;
        if (rc) freeobject(&fields);
        else obj->nnmodule->table = fields.table;
    } else
        rc = ERR_NOTIMPLEMENTED;
    free(cls);
    return rc;
}

static int rd_object(struct reader *r, struct thobject *obj)
{
    int rc, skip;
    memset(obj, 0, sizeof(*obj));
    if (rd_i32(r, &obj->type)) return ERR_READFILE;
    switch (obj->type) {
    case TYPE_NIL: return 0;
    case TYPE_NUMBER: return rd_f64(r, &obj->number);
    case TYPE_STRING: return rd_string(r, &obj->string.data, &obj->string.size);
    case TYPE_BOOLEAN: return rd_i32(r, &obj->boolean);
    case TYPE_TABLE: return rd_table(r, obj);
    case TYPE_TORCH: return rd_torch(r, obj);
    case LEGACY_TYPE_RECUR_FUNCTION:
    case TYPE_RECUR_FUNCTION: {
        /* a dumped Lua closure: index, byte length, bytecode, then its upvalue table -- all dropped */
        struct thobject upvalues;
        if (rd_i32(r, &skip) || rd_i32(r, &skip)) return ERR_READFILE;
        if (fseek(r->fp, skip, SEEK_CUR)) return ERR_READFILE;
        r->next_idx++;
        rc = rd_object(r, &upvalues);
        freeobject(&upvalues);
        obj->type = TYPE_NIL;
        return rc;
    }
    case TYPE_FUNCTION: return ERR_NOTIMPLEMENTED;
    }
    return ERR_CORRUPTED;
}

int loadtorch(const char *path, struct thobject *obj, int longsize)
{
    struct reader r;
    memset(obj, 0, sizeof(*obj));
    r.fp = fopen(path, "rb");
    if (!r.fp) return ERR_OPENFILE;
    r.next_idx = 1;
    r.longsize = longsize == 4 ? 4 : 8;
    r.cap = 1024;
    r.seen = calloc(r.cap, sizeof(*r.seen));
    int rc = rd_object(&r, obj);
    fclose(r.fp);
    free(r.seen);
    if (rc) {
        freeobject(obj);
        memset(obj, 0, sizeof(*obj));
    }
    return rc;
}

static void free_table(struct table *t)
{
    if (!t || --t->nrefs > 0) return;
    for (int i = 0; i < t->nelem; i++) {
        freeobject(&t->records[i].name);
        freeobject(&t->records[i].value);
    }
    free(t->records);
    free(t);
}
static void free_storage(struct storage *s)
{
    if (!s || --s->nrefs > 0) return;
    free(s->data);
    free(s);
}

int freeobject(struct thobject *obj)
{
    switch (obj->type) {
    case TYPE_STRING: free(obj->string.data); break;
    case TYPE_TABLE: free_table(obj->table); break;
    case TYPE_STORAGE: free_storage(obj->storage); break;
    case TYPE_TENSOR:
        if (obj->tensor && --obj->tensor->nrefs <= 0) {
            free(obj->tensor->size);
            free(obj->tensor->stride);
            free_storage(obj->tensor->storage);
            free(obj->tensor);
        }
        break;
    case TYPE_NNMODULE:
        if (obj->nnmodule && --obj->nnmodule->nrefs <= 0) {
            free(obj->nnmodule->name);
            free_table(obj->nnmodule->table);
            free(obj->nnmodule);
        }
        break;
    }
    memset(obj, 0, sizeof(*obj));
    return 0;
}

/* ---- field access on a module's table ---------------------------------------------------------- */
static struct thobject *field(struct table *t, const char *name, int type)
{
    for (int i = 0; t && i < t->nelem; i++)
        if (t->records[i].name.type == TYPE_STRING && !strcmp(t->records[i].name.string.data, name) &&
            t->records[i].value.type == type)
            return &t->records[i].value;
    return 0;
}
double thb_t7_number(struct table *t, const char *name)
{
    struct thobject *o = field(t, name, TYPE_NUMBER);
    return o ? o->number : 0;
}
int thb_t7_boolean(struct table *t, const char *name)
{
    struct thobject *o = field(t, name, TYPE_BOOLEAN);
    return o ? o->boolean : -1;
}
/* float tensor view of a field; an absent field or a tensor without storage gives an empty tensor */
THFloatTensor *thb_t7_tensor(struct table *t, const char *name)
{
    THFloatTensor *th = THFloatTensor_new();
    struct thobject *o = field(t, name, TYPE_TENSOR);
    if (!o || o->tensor->ndim > 4 || o->tensor->scalartype != TYPE_FLOAT) return th;
    struct tensor *src = o->tensor;
    {
        /* the view must lie inside its storage: no negative size or stride, largest element index below nelem */
        long last = src->storageoffset;
        int bad = src->ndim < 0 || src->storageoffset < 0;
        for (int i = 0; i < src->ndim && !bad; i++) {
            if (src->size[i] < 0 || src->stride[i] < 0) bad = 1;
            else if (src->size[i] > 0) last += (src->size[i] - 1) * src->stride[i];
        }
        if (!bad && src->storage && src->ndim > 0 && last >= src->storage->nelem) bad = 1;
        if (bad) {
            fprintf(stderr, "thb200: tensor field %s does not fit its storage; treated as absent\n", name);
            return th;
        }
    }
    th->nDimension = src->ndim;
    memcpy(th->size, src->size, sizeof(long) * src->ndim);
    memcpy(th->stride, src->stride, sizeof(long) * src->ndim);
    th->storageOffset = src->storageoffset;
    if (src->storage) th->storage = THFloatStorage_newwithbuffer(src->storage->data);
    return th;
}
/* the nn module object a field refers to (SpatialMaxUnpooling.pooling), or NULL */
struct nnmodule *thb_t7_nnmodule(struct table *t, const char *name)
{
    struct thobject *o = field(t, name, TYPE_NNMODULE);
    return o ? o->nnmodule : 0;
}
void *thb_t7_storage(struct table *t, const char *name, int *nelem)
{
    struct thobject *o = field(t, name, TYPE_STORAGE);
    if (!o) return 0;
    *nelem = (int)o->storage->nelem;
    return o->storage->data;
}
