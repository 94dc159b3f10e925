/*
 * Host tensors and storages of the public ABI (reference thbasic.c:17-460, types thnets.h:104-120).
 * Only bookkeeping lives here: reference counting, shapes, strides.  No arithmetic -- every
 * operator of the forward pass runs on the device.
 */
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <time.h>
#include "thnets.h"
#include "thb_internal.h"

int th_debug, th_profile, th_minmax;
double th_convtot, th_convflops;

/* fatal error convention of the library: message on stderr, exit(-1)  (thbasic.c:172-181) */
void THError(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vfprintf(stderr, fmt, ap);
    va_end(ap);
    fputc('\n', stderr);
    exit(-1);
}

double th_seconds(void)
{
    static double origin;
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    double now = ts.tv_sec + ts.tv_nsec * 1e-9;
    if (!origin) origin = now;
    return now - origin;
}

THFloatStorage *THFloatStorage_new(long size)
{
    THFloatStorage *s = malloc(sizeof(*s));
    s->data = malloc(sizeof(float) * (size > 0 ? size : 1));
    if (!s || !s->data) THError("Out of memory allocating %ld floats", size);
    s->nref = 1;
    s->mustfree = 1;
    return s;
}

THFloatStorage *THFloatStorage_newwithbuffer(void *buffer)
{
    THFloatStorage *s = malloc(sizeof(*s));
    s->data = buffer;
    s->nref = 1;
    s->mustfree = 0;
    return s;
}

static void storage_release(THFloatStorage *s)
{
    if (__sync_sub_and_fetch(&s->nref, 1) == 0) {
        if (s->mustfree == 1) free(s->data);
        else if (s->mustfree == 2) thb_host_free_pinned(s->data);
        free(s);
    }
}

THFloatTensor *THFloatTensor_new(void) { return calloc(1, sizeof(THFloatTensor)); }

void THFloatTensor_free(THFloatTensor *t)
{
    if (!t) return;
    if (t->storage) storage_release(t->storage);
    free(t);
}

long THFloatTensor_nElement(THFloatTensor *t)
{
    if (!t || t->nDimension == 0) return 0;
    long n = 1;
    for (int i = 0; i < t->nDimension; i++) n *= t->size[i];
    return n;
}

float *THFloatTensor_data(THFloatTensor *t)
{
    return (t && t->storage && t->storage->data) ? t->storage->data + t->storageOffset : 0;
}

/* contiguous resize; a dimension of -1 drops the storage (thbasic.c:58-87) */
void THFloatTensor_resize(THFloatTensor *t, long *size, int nDimension)
{
    long before = THFloatTensor_nElement(t), stride = 1;
    int nostorage = 0;
    t->nDimension = nDimension;
    for (int i = nDimension - 1; i >= 0; i--) {
        t->size[i] = size[i];
        t->stride[i] = stride;
        stride *= size[i];
        if (size[i] == -1) nostorage = 1;
    }
    if (before == THFloatTensor_nElement(t)) return;
    if (nostorage) {
        if (t->storage) storage_release(t->storage);
        t->storage = 0;
    } else if (t->storage)
        t->storage->data = realloc(t->storage->data, sizeof(float) * stride);
    else
        t->storage = THFloatStorage_new(stride);
}

void THFloatTensor_resize4d(THFloatTensor *t, long s0, long s1, long s2, long s3)
{
    long sz[4] = {s0, s1, s2, s3};
    THFloatTensor_resize(t, sz, 4);
}
void THFloatTensor_resize3d(THFloatTensor *t, long s0, long s1, long s2)
{
    long sz[3] = {s0, s1, s2};
    THFloatTensor_resize(t, sz, 3);
}
void THFloatTensor_resize2d(THFloatTensor *t, long s0, long s1)
{
    long sz[2] = {s0, s1};
    THFloatTensor_resize(t, sz, 2);
}
void THFloatTensor_resize1d(THFloatTensor *t, long s0) { THFloatTensor_resize(t, &s0, 1); }

void THFloatTensor_set(THFloatTensor *dst, THFloatTensor *src)
{
    if (dst == src) return;
    if (dst->storage) storage_release(dst->storage);
    *dst = *src;
    if (dst->storage) __sync_fetch_and_add(&dst->storage->nref, 1);
}

THFloatTensor *THFloatTensor_newWithStorage1d(THFloatStorage *storage, long off, long size0, long stride0)
{
    THFloatTensor *t = THFloatTensor_new();
    t->nDimension = 1;
    t->size[0] = size0;
    t->stride[0] = stride0 == -1 ? 1 : stride0;
    t->storage = storage;
    t->storageOffset = off;
    __sync_fetch_and_add(&storage->nref, 1);
    return t;
}

THFloatTensor *THFloatTensor_newWithStorage2d(THFloatStorage *storage, long off, long size0, long stride0, long size1,
                                              long stride1)
{
    THFloatTensor *t = THFloatTensor_new();
    t->nDimension = 2;
    t->size[0] = size0;
    t->size[1] = size1;
    t->stride[0] = stride0 == -1 ? size1 : stride0;
    t->stride[1] = stride1 == -1 ? 1 : stride1;
    t->storage = storage;
    t->storageOffset = off;
    __sync_fetch_and_add(&storage->nref, 1);
    return t;
}

/* view of a loaded Torch7 tensor object; the object keeps ownership of the data (thload.c:700-710) */
THFloatTensor *THFloatTensor_newFromObject(struct thobject *obj)
{
    THFloatTensor *t = THFloatTensor_new();
    struct tensor *src = obj->tensor;
    t->nDimension = src->ndim;
    memcpy(t->size, src->size, sizeof(long) * src->ndim);
    memcpy(t->stride, src->stride, sizeof(long) * src->ndim);
    t->storage = THFloatStorage_newwithbuffer(src->storage->data);
    return t;
}
