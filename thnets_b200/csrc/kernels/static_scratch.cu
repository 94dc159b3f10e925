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

extern "C" int thb_conv_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s);
extern "C" int thb_u8_channel_sum(const void *x, long pixels, int C, int x_ld, int *csum, thb_stream s);

namespace {

#define THB_MAX_DEVICES 64
int *g_scratch_addr[THB_MAX_DEVICES]; /* device address of g_csum_scratch, per device ordinal; NULL = not looked up yet */

int refuse(int code, const char *why)
{
    thb_note_launch(cudaErrorInvalidValue, why);
    return code;
}

}  // namespace

extern "C" int thb_conv_u8_fwd_static(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    // Everything is checked before the first launch: the channel-sum kernels read whole 16-byte vectors of every pixel,
    // so a descriptor they cannot digest must come back as an error code, not as a device fault.
    if (!d || !x || !y) return THB_ERR_ARG;
    if (d->dtype != THB_U8) return refuse(THB_ERR_ARG, "thb_conv_u8_fwd_static: descriptor dtype is not THB_U8");
    if (d->N < 1 || d->H < 1 || d->W < 1 || d->Cin < 1 || d->Cout < 1)
        return refuse(THB_ERR_ARG, "thb_conv_u8_fwd_static: N, H, W, Cin and Cout must be positive");
    if (d->in_ld % 16 || d->in_ld < ((d->Cin + 15) & ~15) || (reinterpret_cast<uintptr_t>(x) & 15))
        return refuse(THB_ERR_ARG, "thb_conv_u8_fwd_static: input needs a 16-byte aligned base and in_ld = multiple of 16 >= Cin rounded up to 16");
    if (!d->w || !d->kinfo || !d->tmap || !d->wsat || !d->status)
        return refuse(THB_ERR_ARG, "thb_conv_u8_fwd_static: w, kinfo, tmap, wsat and status must be set");
    // Rows stored with their horizontal padding are not summed here: the sums are indexed densely as [n][H][W].
    if (d->in_row_pitch) return refuse(THB_ERR_UNSUPPORTED, "thb_conv_u8_fwd_static: in_row_pitch (rows stored with padding) is not supported");
    const long long pixels = (long long)d->N * d->H * d->W;
    if (pixels > THB_STATIC_CSUM_MAX_PIXELS) {
        char msg[160];
        snprintf(msg, sizeof(msg), "thb_conv_u8_fwd_static: N*H*W = %lld input pixels exceeds the static scratch of %d",
                 pixels, THB_STATIC_CSUM_MAX_PIXELS);
        return refuse(THB_ERR_ARG, msg);
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return thb_note_launch(e, "thb_conv_u8_fwd_static: cudaGetDevice");
    if (dev < 0 || dev >= THB_MAX_DEVICES) return refuse(THB_ERR_ARG, "thb_conv_u8_fwd_static: device ordinal beyond the address cache");
    int *scratch = g_scratch_addr[dev];
    if (!scratch) {
        e = cudaGetSymbolAddress((void **)&scratch, g_csum_scratch);
        if (e != cudaSuccess) return thb_note_launch(e, "thb_conv_u8_fwd_static: cudaGetSymbolAddress(g_csum_scratch)");
        if (!scratch) return thb_note_launch(cudaErrorInvalidSymbol, "thb_conv_u8_fwd_static: g_csum_scratch has no device address");
        g_scratch_addr[dev] = scratch;
    }
    // the same channel-sum kernels as the ordinary route, writing into the static array (no allocation on either)
    int rc = thb_u8_channel_sum(x, (long)pixels, d->Cin, d->in_ld, scratch, s);
    if (rc) return rc;
    thb_conv_desc local = *d;
    local.csum = scratch;
    return thb_conv_fwd(&local, x, y, s);
}
