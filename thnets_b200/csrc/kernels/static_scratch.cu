// thb_conv_u8_fwd_static: the uint8 convolution with its per-pixel channel-sum scratch held in a fixed
// array of device memory that belongs to this library image, so that the call allocates nothing.
//
// The uint8 convolution corrects its raw u8*u8 accumulators for the two zero points; one term of that
// correction is, per input pixel, the sum of the pixel's Cin bytes.  thb_conv_fwd reads those sums from a
// caller-provided buffer (thb_conv_desc.csum) that thb_u8_channel_sum filled.  Here the sums go into
// `g_csum_scratch` below instead and the convolution is pointed at it.
//
// Set-up: the first call on each device looks the array's address up (cudaGetSymbolAddress, which also
// makes the runtime load this module's image on that device); later calls on that device reuse the cached
// address.  Make that first call before any stream capture begins.
//
// Sharing: every call on a device uses the same array.  Nothing in it has to start at zero: each call
// overwrites entries [0, N*H*W) before its convolution reads them, in stream order.  Two calls whose
// execution can overlap (different streams without an ordering between them, or different host threads
// on different streams) race on the array and give wrong sums; keep such calls on one stream or order
// them with events.
#include <cuda_runtime.h>
#include <stdint.h>
#include "common.cuh"
#include <stdio.h>

/* THB_STATIC_CSUM_MAX_PIXELS (thb200_kernels.h) = 1048576 entries: 4 MiB of int32, e.g. 20 images of 224x224 */
static __device__ __align__(256) int g_csum_scratch[THB_STATIC_CSUM_MAX_PIXELS];

namespace {

#define THB_MAX_DEVICES 64
int *g_scratch_addr[THB_MAX_DEVICES]; /* device address of g_csum_scratch, per device ordinal; NULL = not looked up yet */

// per input pixel: sum of its first C bytes, written to the static array
__global__ void u8_channel_sum_static_kernel(const uint8_t *__restrict__ x, int pixels, int C, int x_ld)
{
    const int pix = blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= pixels) return;
    const uint4 *p = reinterpret_cast<const uint4 *>(x + (size_t)pix * x_ld);
    int s = 0;
    for (int c0 = 0; c0 < C; c0 += 16) {
        const uint4 t = p[c0 >> 4];
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 16; i++)
            if (c0 + i < C) s += (w[i >> 2] >> ((i & 3) * 8)) & 0xff;
    }
    g_csum_scratch[pix] = s;
}

int fail(cudaError_t e, const char *what) { return thb_note_launch(e, what); }

}  // namespace

extern "C" int thb_conv_u8_fwd_static(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    if (!d || !x || !y) return THB_ERR_ARG;
    if (d->dtype != THB_U8) {
        fail(cudaErrorInvalidValue, "thb_conv_u8_fwd_static: descriptor dtype is not THB_U8");
        return THB_ERR_ARG;
    }
    const long long pixels = (long long)d->N * d->H * d->W;
    if (pixels < 0 || pixels > THB_STATIC_CSUM_MAX_PIXELS) {
        char msg[160];
        snprintf(msg, sizeof(msg), "thb_conv_u8_fwd_static: N*H*W = %lld input pixels exceeds the static scratch of %d",
                 pixels, THB_STATIC_CSUM_MAX_PIXELS);
        fail(cudaErrorInvalidValue, msg);
        return THB_ERR_ARG;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(e, "thb_conv_u8_fwd_static: cudaGetDevice");
    if (dev < 0 || dev >= THB_MAX_DEVICES) {
        fail(cudaErrorInvalidDevice, "thb_conv_u8_fwd_static: device ordinal beyond the address cache");
        return THB_ERR_ARG;
    }
    int *scratch = g_scratch_addr[dev];
    if (!scratch) {
        e = cudaGetSymbolAddress((void **)&scratch, g_csum_scratch);
        if (e != cudaSuccess) return fail(e, "thb_conv_u8_fwd_static: cudaGetSymbolAddress(g_csum_scratch)");
        if (!scratch) return fail(cudaErrorInvalidSymbol, "thb_conv_u8_fwd_static: g_csum_scratch has no device address");
        g_scratch_addr[dev] = scratch;
    }
    if (pixels == 0) return THB_OK;
    const int threads = 256;
    u8_channel_sum_static_kernel<<<(unsigned)((pixels + threads - 1) / threads), threads, 0, (cudaStream_t)s>>>(
        (const uint8_t *)x, (int)pixels, d->Cin, d->in_ld);
    int rc = THB_LAUNCH_CHECK("u8_channel_sum_static_kernel");
    if (rc) return rc;
    thb_conv_desc local = *d;
    local.csum = scratch;
    return thb_conv_fwd(&local, x, y, s);
}
