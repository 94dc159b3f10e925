/*
 * thnets.h -- public header of the B200 build of the thnets inference library.
 *
 * Drop-in for the reference project's header of the same name: the entry points at
 * the bottom (THInit ... THLastError, the th_* globals) and the layout of every
 * structure a caller can reach through them (THNETWORK, struct network, struct
 * module and its parameter union, THFloatTensor, THFloatStorage, the Torch7 object
 * tree) are binary compatible with the reference's CPU build (reference
 * thnets.h:104-120, :122-248, :292-336, :401-407, :571-598).  What differs is
 * underneath: every forward pass runs as sm_100a CUDA kernels; there is no CPU
 * engine in this library, and a machine without a CUDA device gets an error, not
 * a slow answer.
 *
 * Layout rule: field order and types below are the ABI.  Do not reorder.
 */
#ifndef THNETS_B200_THNETS_H
#define THNETS_B200_THNETS_H

#include <float.h>
#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ error codes (THLastError) */
enum therror { ERR_OPENFILE = -1, ERR_READFILE = -2, ERR_NOTIMPLEMENTED = -3, ERR_CORRUPTED = -4, ERR_WRONGOBJECT = -5 };

/* ------------------------------------------------------------------ tensors */
typedef struct THFloatStorage {
    float *data;
    int nref;
    int mustfree; /* 0 = memory owned elsewhere, 1 = free(), 2 = device memory */
} THFloatStorage;

typedef struct THFloatTensor {
    long size[4];
    long stride[4];
    int nDimension;
    THFloatStorage *storage;
    long storageOffset;
} THFloatTensor;

/* ------------------------------------------------------------------ Torch7 object tree (loadtorch) */
enum thtype {
    TYPE_NIL = 0, TYPE_NUMBER = 1, TYPE_STRING = 2, TYPE_TABLE = 3, TYPE_TORCH = 4, TYPE_BOOLEAN = 5,
    TYPE_FUNCTION = 6, LEGACY_TYPE_RECUR_FUNCTION = 7, TYPE_RECUR_FUNCTION = 8,
    TYPE_BYTE = 100, TYPE_CHAR = 101, TYPE_SHORT = 102, TYPE_INT = 103, TYPE_LONG = 104, TYPE_FLOAT = 105,
    TYPE_DOUBLE = 106, TYPE_STORAGE = 200, TYPE_TENSOR = 201, TYPE_NNMODULE = 202
};

struct threcord;
struct table    { int idx, nrefs, nelem; struct threcord *records; };
struct nnmodule { int idx, nrefs; char *name; struct table *table; };
struct storage  { int idx, nrefs, scalartype; long nelem; void *data; };
struct tensor   { int idx, nrefs, scalartype, ndim; long *size, *stride, storageoffset; struct storage *storage; };

struct thobject {
    int type;
    union {
        double number;
        struct { int size; char *data; } string;
        struct table *table;
        struct storage *storage;
        struct tensor *tensor;
        struct nnmodule *nnmodule;
        int boolean;
    };
};
struct threcord { struct thobject name, value; };

/* ------------------------------------------------------------------ per-module parameters */
struct SpatialConvolution {
    THFloatTensor *bias, *weight, *finput;
    int dW, dH, padW, padH, kW, kH, nInputPlane, nOutputPlane;
    int refl_pad, padW2, padH2, autopad, dlH, dlW; /* parsed by loaders, honoured by no engine */
};
struct SpatialFullConvolution {
    THFloatTensor *bias, *weight;
    int dW, dH, padW, padH, kW, kH, nInputPlane, nOutputPlane, adjW, adjH;
    THFloatTensor *ones, *columns;
};
struct SpatialMaxPooling {
    int padW, padH, dW, dH, kW, kH, ceil_mode, iwidth, iheight;
    THFloatTensor *indices;
    int padW2, padH2;
};
struct SpatialAveragePooling {
    int padW, padH, dW, dH, kW, kH, ceil_mode, iwidth, iheight, count_include_pad, padW2, padH2;
};
struct Linear     { THFloatTensor *bias, *weight, *addBuffer; int commute; };
struct Threshold  { float threshold, val, alpha; int inplace; };
struct View       { int numElements, nDimension; long size[4]; };
struct Dropout    { float p; int inplace, v2; };
struct SpatialZeroPadding { int pad_l, pad_r, pad_t, pad_b; };
struct Reshape    { int numElements, batchMode; long size[4], batchsize[4]; int nsize, nbatchsize; };
struct SpatialMaxUnpooling { struct nnmodule *pooling; };
struct SpatialBatchNormalization { THFloatTensor *running_mean, *running_var, *weight, *bias; double eps; };
struct network;
struct Concat     { struct network *net; int dimension; };
struct Sequential { struct network *net; };
struct PReLU      { THFloatTensor *weight; int nOutputPlane; };
struct Padding    { float dim, pad, nInputDim, index, value; };
struct Slice      { int axis, from, to; };
struct Upsample   { float width_scale, height_scale; };
struct LSTM       { THFloatTensor *W, *R, *B; };
struct GRU        { THFloatTensor *W, *R, *B; };
struct Squeeze    { int naxes; int axes[4]; };

enum moduletype {
    MT_Nil, MT_SpatialConvolutionMM, MT_SpatialConvolutionVirtMM, MT_SpatialConvolution, MT_SpatialMaxPooling,
    MT_SpatialAveragePooling, MT_Linear, MT_SoftMax, MT_Threshold, MT_View, MT_Dropout, MT_SpatialZeroPadding,
    MT_Reshape, MT_Normalize, MT_SpatialFullConvolution, MT_SpatialMaxUnpooling, MT_SpatialBatchNormalization,
    MT_Sequential, MT_Concat, MT_ConcatTable, MT_JoinTable, MT_CAddTable, MT_CSubTable, MT_PReLU, MT_Identity,
    MT_Padding, MT_LogSoftMax, MT_Slice, MT_Cmax, MT_Upsample, MT_LSTM, MT_GRU, MT_Squeeze, MT_Unsqueeze,
    MT_Sigmoid, MT_Tanh, MT_Transpose
};

#define MAXMODULEINPUTS 16

/* The operator record.  updateOutput runs this one module on the device: host tensor in, host tensor out. */
struct module {
    int type;
    THFloatTensor *(*updateOutput)(struct module *m, THFloatTensor *in);
    void (*nnfree)(struct module *m);
    THFloatTensor *output;
    struct network *net;
    struct nnmodule *nnmodule;
    char *outputname;
    int ninputs;
    int inputs[MAXMODULEINPUTS];
    union {
        struct SpatialConvolution SpatialConvolution;
        struct SpatialMaxPooling SpatialMaxPooling;
        struct SpatialAveragePooling SpatialAveragePooling;
        struct Linear Linear;
        struct Threshold Threshold;
        struct View View;
        struct Dropout Dropout;
        struct SpatialZeroPadding SpatialZeroPadding;
        struct Reshape Reshape;
        struct SpatialFullConvolution SpatialFullConvolution;
        struct SpatialMaxUnpooling SpatialMaxUnpooling;
        struct SpatialBatchNormalization SpatialBatchNormalization;
        struct Sequential Sequential;
        struct Concat Concat;
        struct Sequential ConcatTable;
        struct Concat JoinTable;
        struct PReLU PReLU;
        struct Slice Slice;
        struct Upsample Upsample;
        struct LSTM LSTM;
        struct GRU GRU;
        struct Squeeze Squeeze;
    };
};

enum { ENGINE_CPU, ENGINE_CUDA, ENGINE_OPENCL, ENGINE_OPENCLINIT, ENGINE_LOWP };

struct network {
    int nelem, engine;
    struct module *modules;
};

/* ------------------------------------------------------------------ "PyTorch Graph Dump 1.00" tree */
#define MAXPYNODES 10000
enum eltype {
    ELTYPE_END = 0, ELTYPE_INPUT = 1, ELTYPE_FUNCTION = 2, ELTYPE_TENSOR = 3, ELTYPE_INT = 4, ELTYPE_FLOAT = 5,
    ELTYPE_INTVECT = 6, ELTYPE_OUTPUTID = 7
};
struct elemlist;
struct pyfunction {
    int id, ninputs;
    struct elemlist *inputs, *params;
    struct module module;
};
struct pyelement {
    enum eltype type;
    char *name;
    union {
        struct pyfunction function;
        int ivalue;
        float fvalue;
        int ivect[4];
        THFloatTensor *tensor;
    };
};
struct elemlist { struct pyelement *elem; struct elemlist *next; };

/* ------------------------------------------------------------------ high level API */
typedef struct thnetwork {
    struct thobject *netobj;
    struct thobject *statobj;
    struct network *net;          /* Torch7 route; NULL for PyTorch-dump networks */
    struct pyelement *pynet;      /* PyTorch-dump route: root = network output */
    struct pyelement **allpynodes;
    THFloatTensor *out;           /* last result; owned by the network */
    float mean[3], std[3];
} THNETWORK;

void THInit(void);
THNETWORK *THLoadNetwork(const char *path);
THFloatTensor *THForward(THNETWORK *net, THFloatTensor *in);
void THMakeSpatial(THNETWORK *network, int size);
int THProcessFloat(THNETWORK *network, float *data, int batchsize, int width, int height, int nplanes,
                   float **result, int *outwidth, int *outheight);
int THProcessImages(THNETWORK *network, unsigned char **images, int batchsize, int width, int height, int stride,
                    float **result, int *outwidth, int *outheight, int bgr);
int THProcessYUYV(THNETWORK *network, unsigned char *image, int width, int height, float **results,
                  int *outwidth, int *outheight);
THNETWORK *THCreateCudaNetwork(THNETWORK *net);
THNETWORK *THCreateOpenCLNetwork(THNETWORK *net);
THNETWORK *THCreateLowpNetwork(THNETWORK *net, float range);
int THCudaHalfFloat(int enable);
int THOpenCLHalfFloat(int enable);
int THUseSpatialConvolutionMM(THNETWORK *network, int mm_type);
void THFreeNetwork(THNETWORK *network);
int THLastError(void);
extern int th_debug, th_profile, th_minmax;
extern double th_convtot, th_convflops;

/* ------------------------------------------------------------------ helpers callers of the reference use */
void THError(const char *fmt, ...);
int loadtorch(const char *path, struct thobject *obj, int longsize);
int freeobject(struct thobject *obj);
void freenetwork(struct network *net);
struct network *Module2Network(struct nnmodule *obj);
struct pyelement *loadpytorch(const char *path, struct pyelement **allpynodes);
void freepynet(struct pyelement *node);
double th_seconds(void);

THFloatTensor *THFloatTensor_new(void);
THFloatStorage *THFloatStorage_new(long size);
THFloatStorage *THFloatStorage_newwithbuffer(void *buffer);
THFloatTensor *THFloatTensor_newFromObject(struct thobject *obj);
THFloatTensor *THFloatTensor_newWithStorage1d(THFloatStorage *storage, long storageOffset, long size0, long stride0);
THFloatTensor *THFloatTensor_newWithStorage2d(THFloatStorage *storage, long storageOffset, long size0, long stride0,
                                              long size1, long stride1);
void THFloatTensor_free(THFloatTensor *t);
float *THFloatTensor_data(THFloatTensor *tensor);
long THFloatTensor_nElement(THFloatTensor *t);
void THFloatTensor_resize(THFloatTensor *t, long *size, int nDimension);
void THFloatTensor_resize4d(THFloatTensor *t, long size0, long size1, long size2, long size3);
void THFloatTensor_resize3d(THFloatTensor *t, long size0, long size1, long size2);
void THFloatTensor_resize2d(THFloatTensor *t, long size0, long size1);
void THFloatTensor_resize1d(THFloatTensor *t, long size0);
void THFloatTensor_set(THFloatTensor *tdst, THFloatTensor *tsrc);

/* ------------------------------------------------------------------ B200 extensions (no reference counterpart) */
/* 0 = fp32 (default), 1 = fp16, 2 = bf16: same switch as THCudaHalfFloat, read when a network is converted */
int THB200_SetPrecision(int mode);
/* number of GPUs a converted network shards its batch over (1..8); read when a network is converted */
int THB200_SetDevices(int ngpus);
/* THProcessFloat cuts each GPU's batch slice into sub-batches so that the host-to-device copy of one runs under the
 * kernels of the one before; 0 = chosen from the input size (default, also THB200_CHUNKS), 1 = off, up to 4 */
int THB200_SetPipelineChunks(int chunks);
/* pinned host memory for input batches, so that THProcessFloat's copies run at full PCIe speed */
void *THB200_HostAlloc(size_t bytes);
void THB200_HostFree(void *p);
/* device time in milliseconds of the last forward (kernels only, between the input and output copies) */
float THB200_LastDeviceMs(THNETWORK *network);
/* Device-resident benchmark loop: the whole forward from the batch the last THProcessFloat / THProcessImages call
 * left in device memory (NCHW fp32, or HWC bytes) to the NCHW fp32 result in device memory -- the boundary kernels at
 * both ends, the uint8 engine's input-range pass and the planned launches -- `iters` times back to back; returns the
 * mean device time per forward in milliseconds (< 0 on error).  No host<->device copy of batch or result is inside. */
float THB200_TimeForward(THNETWORK *network, int iters);
/* Per-launch device time (ms, averaged over `iters` passes) of the same forward on the first GPU.  Entry 0 is the
 * boundary kernel in, the last entry the boundary kernel out, the planned launches lie between.  kinds[t] is 0 for a
 * convolution / Linear-as-convolution launch, 1 for a GEMV, 2 for another planned launch, 3 for a boundary kernel;
 * flops[t] its algorithmic FLOPs.  Returns the number of entries described (<= max_steps), < 0 on error. */
int THB200_ProfileForward(THNETWORK *network, int iters, int max_steps, int *kinds, float *ms, double *flops);
/* bytes[t]: algorithmic bytes of entry t of the same list (input, output, residual and weights counted once each at the
 * storage type's size) for convolution and GEMV launches, 0 for the others.  Returns the number described. */
int THB200_ProfileForwardBytes(THNETWORK *network, int max_steps, double *bytes);
/* the contiguous slice [offset, offset+count) of an N-image batch that GPU g of G processes */
void THB200_SliceBatch(int N, int G, int g, int *offset, int *count);
/* sub-batch c of the S pipelined sub-batches that a GPU's slice of n images is cut into (THB200_SetPipelineChunks) */
void THB200_SliceSubBatches(int n, int S, int c, int *offset, int *count);
int THB200_KernelLaunches(void);
/* one text line per operator of the lowered network; returns the length written, < 0 on error */
int THB200_DescribeNetwork(THNETWORK *network, char *buf, int len);
const char *THB200_LastErrorString(void);

#ifdef __cplusplus
}
#endif
#endif
