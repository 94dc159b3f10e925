// Host side of the convolution ABI: tile geometry, weight packing into the kernel layouts,
// dispatch between the fp32 FFMA kernel and the tcgen05 kernel, and launch bookkeeping.
#include "common.cuh"
#include <stdio.h>
#include <string.h>
#include <stdlib.h>
#include <vector>

extern "C" int thb_conv_fwd_tc(const thb_conv_desc *d, const void *x, void *y, thb_stream s);
extern "C" int thb_conv_fwd_simt(const thb_conv_desc *d, const void *x, void *y, thb_stream s);
extern "C" int thb_conv_patch_supported(const thb_conv_desc *d);
extern "C" int thb_conv_patch_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s);

static char g_last_error[256] = "";
static int g_launches = 0;

extern "C" int thb_note_launch(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) {
        g_launches++;
        return THB_OK;
    }
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    fprintf(stderr, "thb200: %s\n", g_last_error);
    return THB_ERR_CUDA;
}
extern "C" const char *thb_last_cuda_error(void) { return g_last_error; }
extern "C" int thb_kernel_launch_count(void) { return g_launches; }
// launches replayed through a captured graph are counted by whoever replays it
extern "C" void thb_count_launches(int n) { g_launches += n; }

static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

/* K blocks from which a 256-channel tile is preferred to two 128-channel ones (diagnostic override: THB200_BN256_MIN_KB) */
static int bn256_min_kb()
{
    static int v = 0;
    if (!v) {
        const char *e = getenv("THB200_BN256_MIN_KB");
        v = e && atoi(e) > 0 ? atoi(e) : 4;
    }
    return v;
}

extern "C" int thb_conv_geometry(thb_conv_desc *d)
{
    if (d->kH < 1 || d->kW < 1 || d->kH > 127 || d->kW > 255 || d->dH < 1 || d->dW < 1 || d->Cin < 1 || d->Cout < 1)
        return THB_ERR_ARG;
    const int al = thb_channel_align(d->dtype);
    d->Cin_pad = round_up(d->Cin, al);
    if (d->Cin_pad / al > 0xffff) return THB_ERR_UNSUPPORTED;
    const int taps = d->kH * d->kW;
    if (d->dtype == THB_F32) {
        d->Ktot_pad = round_up(taps * d->Cin_pad, 16);
        d->BN = 64;
        d->Cout_pad = round_up(d->Cout, 64);
        return THB_OK;
    }
    const int bke = d->dtype == THB_U8 ? 128 : 64;
    d->Ktot_pad = round_up(taps * d->Cin_pad, bke);
    if (d->BN != 32 && d->BN != 64 && d->BN != 128 && d->BN != 256) {
        const long mtiles = ((long)d->N * d->oH * d->oW + 127) / 128;
        if (d->Cout <= 32) d->BN = 32;
        else if (d->Cout <= 64) d->BN = 64;
        else if (d->Cout <= 128) d->BN = 128;
        else if (d->Ktot_pad / bke >= bn256_min_kb() && mtiles * ((d->Cout + 255) / 256) >= 148 &&
                 round_up(d->Cout, 256) == round_up(d->Cout, 128)) d->BN = 256; /* wide tiles pay once the K loop outweighs the epilogue and every SM gets a tile */
        else d->BN = 128;
        /* a launch of a few tiles only (a Linear on a batch of pixels): narrower tiles give more SMs a share of the weights */
        if (d->BN == 128 && mtiles * ((d->Cout + 127) / 128) * 4 <= 148) d->BN = 64;
        /* (a Linear proper -- 1x1 maps, so neither a second operand nor a residual tile will be asked of the narrow tiles'
         * staged epilogue: 2048->1000 on 256 rows went from 24 to 17 us) */
        if (d->BN == 64 && d->Cout > 64 && d->H == 1 && d->W == 1 && taps == 1 && mtiles * ((d->Cout + 63) / 64) * 2 <= 148) d->BN = 32;
    }
    d->Cout_pad = round_up(d->Cout, d->BN);
    return THB_OK;
}

extern "C" size_t thb_conv_weight_bytes(const thb_conv_desc *d)
{
    const size_t es = d->dtype == THB_F32 ? 4 : d->dtype == THB_U8 ? 1 : 2;
    return (size_t)d->Ktot_pad * d->Cout_pad * es;
}
extern "C" size_t thb_conv_kinfo_words(const thb_conv_desc *d) { return (size_t)d->Ktot_pad / thb_channel_align(d->dtype); }

extern "C" int thb_conv_pack_weights_host(const thb_conv_desc *d, const float *w, const unsigned char *wq, void *packed,
                                          int *kinfo, int *wsat)
{
    const int al = thb_channel_align(d->dtype), taps = d->kH * d->kW;
    const int Cin = d->Cin, Cp = d->Cin_pad, Cout = d->Cout;
    // one word per 16-byte K chunk: kernel row << 24 | kernel column << 16 | channel offset in 16-byte units
    for (int g = 0; g < d->Ktot_pad / al; g++) {
        const int k = g * al, tap = k / Cp, c = k % Cp;
        kinfo[g] = tap < taps ? (int)(((unsigned)(tap / d->kW) << 24) | ((unsigned)(tap % d->kW) << 16) | (unsigned)(c / al))
                              : (int)0x80000000u;
    }
    memset(packed, 0, thb_conv_weight_bytes(d));
    if (d->dtype == THB_U8) {
        if (!wq || !wsat) return THB_ERR_ARG;
        unsigned char *p = (unsigned char *)packed;
        const int sw = d->kW + 1, sn = (d->kH + 1) * sw;
        for (int co = 0; co < Cout; co++) {
            int *sat = wsat + (size_t)co * sn;
            memset(sat, 0, sizeof(int) * sn);
            for (int r = 0; r < d->kH; r++)
                for (int s = 0; s < d->kW; s++) {
                    int t = 0;
                    for (int c = 0; c < Cin; c++) {
                        const unsigned char v = wq[(((size_t)co * Cin + c) * d->kH + r) * d->kW + s];
                        p[(size_t)co * d->Ktot_pad + (size_t)(r * d->kW + s) * Cp + c] = v;
                        t += v;
                    }
                    sat[(r + 1) * sw + s + 1] = t + sat[r * sw + s + 1] + sat[(r + 1) * sw + s] - sat[r * sw + s];
                }
        }
        return THB_OK;
    }
    if (!w) return THB_ERR_ARG;
    for (int co = 0; co < Cout; co++)
        for (int c = 0; c < Cin; c++)
            for (int t = 0; t < taps; t++) {
                const float v = w[((size_t)co * Cin + c) * taps + t];
                const size_t k = (size_t)t * Cp + c;
                if (d->dtype == THB_F32) ((float *)packed)[k * d->Cout_pad + co] = v;
                else if (d->dtype == THB_F16) ((__half *)packed)[(size_t)co * d->Ktot_pad + k] = __float2half_rn(v);
                else ((__nv_bfloat16 *)packed)[(size_t)co * d->Ktot_pad + k] = __float2bfloat16_rn(v);
            }
    return THB_OK;
}

extern "C" unsigned short thb_float_to_half_bits(float v, int bf16)
{
    if (bf16) {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        return *reinterpret_cast<unsigned short *>(&h);
    }
    __half h = __float2half_rn(v);
    return *reinterpret_cast<unsigned short *>(&h);
}

extern "C" int thb_conv_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    if (d->x2) {
        if (d->dtype != THB_F16 && d->dtype != THB_BF16) return THB_ERR_UNSUPPORTED;
        if (d->in_ld < d->cin1 || d->x2_ld < d->Cin - d->cin1) return THB_ERR_ARG;
        return thb_conv_fwd_tc(d, x, y, s);
    }
    if (d->in_ld < d->Cin_pad) return THB_ERR_ARG;
    if (d->in_row_pitch) {
        // rows stored with their padding: tensor-core dtypes only
        if (d->dtype == THB_F32) return THB_ERR_UNSUPPORTED;
        if (d->in_pad_left != d->padW || d->in_row_pitch < d->W + d->kW - 1) return THB_ERR_ARG;
    }
    if (d->dtype == THB_F32) return thb_conv_fwd_simt(d, x, y, s);
    // stride-1 layers with 16 or 64 channels per pixel and a kernel larger than 1x1: the raw input patch is loaded once
    // and every tap reads it in place (conv_patch_tc.cu)
    if (d->kH * d->kW > 1 && thb_conv_patch_supported(d)) return thb_conv_patch_fwd(d, x, y, s);
    return thb_conv_fwd_tc(d, x, y, s);
}
