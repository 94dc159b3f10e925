// fp32 implicit-GEMM convolution with exact FFMA accumulation (the fp32 mode's 1e-4 parity path).
//
// D[pixel][cout] = sum_k A[pixel][k] * Wk[k][cout], k = tap*Cin_pad + c over NHWC fp32 activations.
// Block tile (16*TM) pixels x 64 output channels, K step 16, 256 threads, TM x 4 outputs per thread.
// The A tile is gathered as float4 channel chunks (zero outside the image) and stored transposed in
// shared memory; global loads of the next K step are issued before the current one is consumed.
//
// Few pixels (batch 1): the tile grid alone leaves most SMs idle and each CTA walks the whole reduction alone.  Then the
// K steps are split over the CTAs of a thread-block cluster (grid z, up to 8): every CTA accumulates its share, the
// others leave their partial tiles in their own shared memory, and the cluster's first CTA adds them up through
// distributed shared memory in rank order (so the result does not depend on timing) and runs the epilogue.
#include "common.cuh"
#include <cooperative_groups.h>
#include <string.h>
namespace cg = cooperative_groups;

namespace {

struct ConvSimtParams {
    const float *x, *w;
    float *y;
    const int *kinfo;
    int P, H, W, in_ld, oW, oHW, dH, dW, padH, padW, Cout, Cout_pad, out_ld, nkb, n_kchunks;
    const float *scale, *shift, *slope, *res;
    int res_ld;
    float self_coef, res_coef;
    int act_kind;
    float act_th, act_val, act_alpha;
};

int g_no_split = -1;  // THB200_NO_SPLITK, read once

template <int TM, bool SPLIT>
__global__ void __launch_bounds__(256) conv_simt_kernel(const ConvSimtParams p)
{
    constexpr int BMT = 16 * TM, BNT = 64, BK = 16;
    constexpr int A_LOADS = (BMT * 4 + 255) / 256;
    __shared__ __align__(16) float As[BK][BMT + 4];
    __shared__ __align__(16) float Bs[BK][BNT];
    __shared__ float red[SPLIT ? TM * 4 : 1][SPLIT ? 256 : 1];  // this CTA's partial tile, read by the cluster's first CTA

    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.x * BMT, n0 = blockIdx.y * BNT;

    // gather bookkeeping for this thread's A chunks
    int a_row[A_LOADS], a_ih0[A_LOADS], a_iw0[A_LOADS], a_pix[A_LOADS];
    const int a_chunk = t & 3;
#pragma unroll
    for (int i = 0; i < A_LOADS; i++) {
        int idx = t + i * 256;
        int r = idx >> 2;
        a_row[i] = r;
        int pm = m0 + r;
        if (idx < BMT * 4 && pm < p.P) {
            int n = pm / p.oHW, rem = pm - n * p.oHW;
            int oh = rem / p.oW, ow = rem - oh * p.oW;
            a_ih0[i] = oh * p.dH - p.padH;
            a_iw0[i] = ow * p.dW - p.padW;
            a_pix[i] = n * p.H * p.W;
        } else {
            a_ih0[i] = a_iw0[i] = 0;
            a_pix[i] = -1;
        }
    }
    const int b_k = t >> 4, b_c = (t & 15) * 4;

    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    float4 a_reg[A_LOADS], b_reg;
    auto load_global = [&](int kb) {
        const int g = kb * 4 + a_chunk;
        const int ki = g < p.n_kchunks ? p.kinfo[g] : -1;
        const int dh = (ki >> 24) & 0x7f, dw = (ki >> 16) & 0xff, coff = (ki & 0xffff) * 4;
#pragma unroll
        for (int i = 0; i < A_LOADS; i++) {
            const int ih = a_ih0[i] + dh, iw = a_iw0[i] + dw;
            const bool ok = ki >= 0 && a_pix[i] >= 0 && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W;
            a_reg[i] = ok ? *reinterpret_cast<const float4 *>(p.x + (size_t)(a_pix[i] + ih * p.W + iw) * p.in_ld + coff)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        b_reg = *reinterpret_cast<const float4 *>(p.w + (size_t)(kb * BK + b_k) * p.Cout_pad + n0 + b_c);
    };
    auto store_smem = [&]() {
#pragma unroll
        for (int i = 0; i < A_LOADS; i++) {
            if (t + i * 256 < BMT * 4) {
                const int r = a_row[i], k = a_chunk * 4;
                As[k + 0][r] = a_reg[i].x;
                As[k + 1][r] = a_reg[i].y;
                As[k + 2][r] = a_reg[i].z;
                As[k + 3][r] = a_reg[i].w;
            }
        }
        *reinterpret_cast<float4 *>(&Bs[b_k][b_c]) = b_reg;
    };

    // this CTA's share of the K steps
    const int kb0 = SPLIT ? (int)((long)p.nkb * blockIdx.z / gridDim.z) : 0;
    const int kb1 = SPLIT ? (int)((long)p.nkb * (blockIdx.z + 1) / gridDim.z) : p.nkb;
    if (kb0 < kb1) load_global(kb0);
    for (int kb = kb0; kb < kb1; kb++) {
        store_smem();
        __syncthreads();
        if (kb + 1 < kb1) load_global(kb + 1);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM];
            const float4 b = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int i = 0; i < TM; i++) {
                acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
                acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
                acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
                acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
            }
        }
        __syncthreads();
    }

    if (SPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        if (blockIdx.z != 0) {
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) red[i * 4 + j][t] = acc[i][j];
        }
        cluster.sync();
        if (blockIdx.z == 0) {
            for (unsigned r = 1; r < gridDim.z; r++) {
                const float *remote = cluster.map_shared_rank(&red[0][0], r);
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] += remote[(i * 4 + j) * 256 + t];
            }
        }
        cluster.sync();  // the others' shared memory must outlive the reads above
        if (blockIdx.z != 0) return;
    }
    const int c0 = n0 + tx * 4;
    if (c0 >= p.Cout) return;
    float sc[4], sh[4], sl[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int c = c0 + j;
        sc[j] = c < p.Cout ? (p.scale ? p.scale[c] : 1.f) : 0.f;
        sh[j] = c < p.Cout ? (p.shift ? p.shift[c] : 0.f) : 0.f;
        sl[j] = (c < p.Cout && p.slope) ? p.slope[c] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int pm = m0 + ty * TM + i;
        if (pm >= p.P) continue;
        float v[4];
        float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.res) r = *reinterpret_cast<const float4 *>(p.res + (size_t)pm * p.res_ld + c0);
        const float rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float val = acc[i][j] * sc[j] + sh[j];
            if (p.res) val = p.self_coef * val + p.res_coef * rr[j];
            val = thb_apply_act(val, p.act_kind, p.act_th, p.act_val, p.act_alpha, sl[j]);
            v[j] = (c0 + j < p.Cout) ? val : 0.f;
        }
        *reinterpret_cast<float4 *>(p.y + (size_t)pm * p.out_ld + c0) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

}  // namespace

// (library-internal: thb_conv_reload_knobs() calls it so that a test can switch THB200_NO_SPLITK between cases)
extern "C" void thb_simt_reload_knobs(void) { g_no_split = -1; }

extern "C" int thb_conv_fwd_simt(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    if (!d->w || !d->kinfo) return THB_ERR_ARG;
    if (d->in_ld % 4 || d->out_ld % 4 || (d->res && d->res_ld % 4)) return THB_ERR_ARG;
    ConvSimtParams p;
    memset(&p, 0, sizeof(p));
    p.x = (const float *)x; p.w = (const float *)d->w; p.y = (float *)y; p.kinfo = d->kinfo;
    p.P = d->N * d->oH * d->oW;
    p.H = d->H; p.W = d->W; p.in_ld = d->in_ld; p.oW = d->oW; p.oHW = d->oH * d->oW;
    p.dH = d->dH; p.dW = d->dW; p.padH = d->padH; p.padW = d->padW;
    p.Cout = d->Cout; p.Cout_pad = d->Cout_pad; p.out_ld = d->out_ld;
    p.nkb = d->Ktot_pad / 16; p.n_kchunks = d->Ktot_pad / 4;
    p.scale = d->scale; p.shift = d->shift; p.slope = d->act.kind == THB_ACT_PRELU ? d->act.slope : nullptr;
    p.res = (const float *)d->res; p.res_ld = d->res_ld; p.self_coef = d->self_coef; p.res_coef = d->res_coef;
    p.act_kind = d->act.kind; p.act_th = d->act.threshold; p.act_val = d->act.value; p.act_alpha = d->act.alpha;
    if (p.P <= 0) return THB_OK;
    const int gy = d->Cout_pad / 64;
    cudaStream_t st = (cudaStream_t)s;
    if ((long)((p.P + 127) / 128) * gy >= 120) {
        conv_simt_kernel<8, false><<<dim3((p.P + 127) / 128, gy), 256, 0, st>>>(p);
    } else {
        // how many CTAs share one tile's reduction: enough to give every SM about two CTAs, at least four K steps each
        const long ctas = (long)((p.P + 31) / 32) * gy;
        static int sms = 0;
        int &no_split = g_no_split;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        if (no_split < 0) {
            const char *e = getenv("THB200_NO_SPLITK");
            no_split = e && atoi(e) ? 1 : 0;
        }
        int split = 1;
        while (split < 8 && ctas * split * 2 <= 2L * sms && p.nkb / (split * 2) >= 4) split *= 2;
        if (split == 1 || no_split) {
            conv_simt_kernel<2, false><<<dim3((p.P + 31) / 32, gy), 256, 0, st>>>(p);
        } else {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((p.P + 31) / 32, gy, split);
            cfg.blockDim = dim3(256);
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = split;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            const cudaError_t le = cudaLaunchKernelEx(&cfg, conv_simt_kernel<2, true>, p);
            if (le != cudaSuccess) return thb_note_launch(le, "conv_simt_kernel (split K)");
        }
    }
    return THB_LAUNCH_CHECK("conv_simt_kernel");
}
