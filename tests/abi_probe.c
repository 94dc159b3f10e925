#include <stdio.h>
#include <stddef.h>
#include "thnets.h"
#define P(x) printf("%s=%zu\n", #x, (size_t)(x))
int main(){
P(sizeof(THFloatTensor)); P(sizeof(THFloatStorage)); P(sizeof(struct module)); P(sizeof(struct network)); P(sizeof(THNETWORK));
P(sizeof(struct thobject)); P(sizeof(struct pyelement)); P(sizeof(struct pyfunction));
P(offsetof(struct module, updateOutput)); P(offsetof(struct module, output)); P(offsetof(struct module, inputs)); P(offsetof(struct module, SpatialConvolution));
P(offsetof(struct module, SpatialConvolution.weight)); P(offsetof(struct module, SpatialConvolution.nOutputPlane)); P(offsetof(struct module, Linear.weight));
P(offsetof(struct module, SpatialMaxPooling.ceil_mode)); P(offsetof(struct module, SpatialBatchNormalization.eps)); P(offsetof(struct module, Reshape.batchsize));
P(offsetof(THNETWORK, net)); P(offsetof(THNETWORK, pynet)); P(offsetof(THNETWORK, out)); P(offsetof(THNETWORK, mean)); P(offsetof(THNETWORK, std));
P(offsetof(struct network, engine)); P(offsetof(struct network, modules)); P(offsetof(THFloatTensor, storage)); P(offsetof(THFloatTensor, storageOffset));
P(offsetof(struct pyelement, function.module)); P(offsetof(struct pyfunction, params));
P(MT_SpatialConvolutionVirtMM); P(MT_CSubTable); P(MT_Transpose); P(ENGINE_LOWP); P(MAXPYNODES); P(MAXMODULEINPUTS);
return 0;}
