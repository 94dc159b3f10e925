// Implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// GEMM view: D[pixel][cout] = sum_k A[pixel][k] * Wt[cout][k], k = tap*Cin_pad + c.
//   * one CTA computes 128 consecutive output pixels (flat over n, oh, ow -- tiles may span rows and
//     images, so small feature maps waste nothing) times BN output channels;
//   * A (the im2col rows) is never materialised: four producer warps gather 16-byte channel chunks of
//     the NHWC activation straight into the 128-byte-swizzled K-major tile layout with zero-filling
//     cp.async (out-of-image taps and ragged tiles become zeros);
//   * Wt (packed weights, K-major) arrives by 2-D TMA with SWIZZLE_128B, no multicast;
//   * one elected thread issues tcgen05.mma (kind::f16 for fp16/bf16 with fp32 accumulation, kind::i8
//     for u8 x u8 with int32 accumulation), stages are recycled through tcgen05.commit -> mbarrier;
//   * the producer warps turn into the epilogue: tcgen05.ld the accumulator rows (TMEM lane = pixel),
//     apply bias/BN scale-shift, residual, activation -- or the exact lowp requantisation -- and store
//     channels-innermost vectors.
// Every wait is bounded: a wait that runs out records a code in *status and the CTA drains and exits.
#include "common.cuh"
#include <cuda.h>
#include <string.h>
#include <stdio.h>

namespace {

constexpr int BM = 128;          // pixels per CTA tile (= TMEM lanes)
constexpr int A_STAGE_BYTES = BM * 128;
constexpr int LAG = 2;           // cp.async groups a producer thread keeps in flight

struct ConvTcParams {
    const uint8_t *x;
    uint8_t *y;
    const int *kinfo;
    int P, H, W, in_ld, oW, oHW, dH, dW, padH, padW, kH, kW, Cin, Cout, out_ld, nkb, n_kchunks;
    const float *scale, *shift, *slope;
    const uint8_t *res;
    int res_ld;
    float self_coef, res_coef;
    int act_kind;
    float act_th, act_val, act_alpha;
    int a_off, b_off, c_off, c_mult, c_shift;
    const int *wsat, *bias_add, *csum;
    int tail_start, relu_thr, relu_val;
    int *acc_out;
    int *status;
};

template <int KIND> struct kind_traits;             // 0 = fp16, 1 = bf16, 2 = u8
template <> struct kind_traits<0> { static constexpr int esize = 2; };
template <> struct kind_traits<1> { static constexpr int esize = 2; };
template <> struct kind_traits<2> { static constexpr int esize = 1; };

__device__ __forceinline__ uint32_t pack2(float a, float b, int kind)
{
    if (kind == 0) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float2 unpack2(uint32_t v, int kind)
{
    if (kind == 0) return __half22float2(*reinterpret_cast<__half2 *>(&v));
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&v));
}

template <int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1) conv_tc_kernel(const __grid_constant__ CUtensorMap tmapW, const ConvTcParams p)
{
    constexpr int ES = kind_traits<KIND>::esize;
    constexpr int BKE = 128 / ES;                 // K elements per 128-byte stage row
    constexpr int B_STAGE_BYTES = BN * 128;
    constexpr uint32_t IDESC = make_idesc(KIND == 2 ? 2u : 1u, KIND == 1 ? 1u : 0u, BN);
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sA = smem;
    uint8_t *sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sB + STAGES * B_STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + STAGES, *tmem_full = bars + 2 * STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *ep0 = reinterpret_cast<float *>(tmem_slot + 2);   // scale   | wtot (int)
    float *ep1 = ep0 + BN;                                    // shift   | bias_add (int)
    float *ep2 = ep1 + BN;                                    // slope

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full[s]), 128 + 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(tmem_full), 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 4 && lane == 0) tma_prefetch_desc(&tmapW);
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    if (warp < 4) {
        for (int i = tid; i < BN; i += 128) {
            int c = n0 + i;
            if (KIND == 2) {
                int tot = 0, ba = 0;
                if (c < p.Cout) {
                    tot = p.wsat[(size_t)c * (p.kH + 1) * (p.kW + 1) + (p.kH + 1) * (p.kW + 1) - 1];
                    ba = p.bias_add ? p.bias_add[c] : 0;
                }
                reinterpret_cast<int *>(ep0)[i] = tot;
                reinterpret_cast<int *>(ep1)[i] = ba;
            } else {
                ep0[i] = c < p.Cout ? (p.scale ? p.scale[c] : 1.f) : 0.f;
                ep1[i] = c < p.Cout ? (p.shift ? p.shift[c] : 0.f) : 0.f;
                ep2[i] = (c < p.Cout && p.slope) ? p.slope[c] : 0.f;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------------------------ A producer
        const int chunk = lane & 7;
        int ih0[8], iw0[8], pixbase[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int r = warp * 32 + j * 4 + (lane >> 3);
            int pm = m0 + r;
            if (pm < p.P) {
                int n = pm / p.oHW, rem = pm - n * p.oHW;
                int oh = rem / p.oW, ow = rem - oh * p.oW;
                ih0[j] = oh * p.dH - p.padH;
                iw0[j] = ow * p.dW - p.padW;
                pixbase[j] = n * p.H * p.W;
            } else {
                ih0[j] = iw0[j] = 0;
                pixbase[j] = -1;
            }
        }
        bool alive = true;
        for (int kb = 0; kb < p.nkb && alive; kb++) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1)) {
                if (lane == 0) atomicExch(p.status, 1);
                *abort_flag = 1;
                alive = false;
                break;
            }
            const int g = kb * 8 + chunk;
            const int ki = g < p.n_kchunks ? p.kinfo[g] : -1;
            const int dh = (ki >> 24) & 0x7f, dw = (ki >> 16) & 0xff;
            const size_t coff = (size_t)(ki & 0xffff) * 16;
            const uint32_t a_stage = smem_u32(sA + s * A_STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int r = warp * 32 + j * 4 + (lane >> 3);
                const int ih = ih0[j] + dh, iw = iw0[j] + dw;
                const bool ok = ki >= 0 && pixbase[j] >= 0 && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W;
                const uint8_t *src = ok ? p.x + ((size_t)(pixbase[j] + ih * p.W + iw) * p.in_ld) * ES + coff : p.x;
                cp_async16(a_stage + r * 128 + ((chunk ^ (r & 7)) << 4), src, ok ? 16u : 0u);
            }
            cp_async_commit();
            if (kb >= LAG) {
                cp_async_wait<LAG>();
                fence_proxy_async_smem();
                mbar_arrive(smem_u32(&full[(kb - LAG) % STAGES]));
            }
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (alive)
            for (int kb = (p.nkb > LAG ? p.nkb - LAG : 0); kb < p.nkb; kb++) mbar_arrive(smem_u32(&full[kb % STAGES]));

        // ------------------------------------------------------------------ epilogue
        const int row = warp * 32 + lane;
        const int pm = m0 + row;
        const bool valid = pm < p.P;
        bool have_acc = alive && !*abort_flag;
        if (have_acc && !mbar_wait_bounded(smem_u32(tmem_full), 0)) {
            if (lane == 0) atomicExch(p.status, 2);
            *abort_flag = 1;
            have_acc = false;
        }
        have_acc = __all_sync(0xffffffffu, have_acc);
        if (have_acc) {
            tc_fence_after();
            // per-pixel terms of the u8 zero-point correction
            int corr_pix = 0, r0 = 0, r1 = 0, s0 = 0, s1 = 0, plane_pos = 0;
            bool interior = true;
            if (KIND == 2 && valid) {
                int n = pm / p.oHW, rem = pm - n * p.oHW;
                int oh = rem / p.oW, ow = rem - oh * p.oW;
                plane_pos = rem;
                int ihb = oh * p.dH - p.padH, iwb = ow * p.dW - p.padW;
                r0 = max(0, -ihb); r1 = min(p.kH, p.H - ihb);
                s0 = max(0, -iwb); s1 = min(p.kW, p.W - iwb);
                interior = r0 == 0 && s0 == 0 && r1 == p.kH && s1 == p.kW;
                int xsum = 0;
                const int *cs = p.csum + (size_t)n * p.H * p.W;
                for (int r = r0; r < r1; r++)
                    for (int s = s0; s < s1; s++) xsum += cs[(ihb + r) * p.W + iwb + s];
                int nvalid = max(0, r1 - r0) * max(0, s1 - s0);
                corr_pix = p.a_off * (xsum + p.b_off * nvalid * p.Cin);
            }
            const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; cc++) {
                uint32_t acc[32];
                __syncwarp();
                tmem_ld32(lane_addr + cc * 32, acc);
                tmem_ld_wait();
                const int c0 = n0 + cc * 32;
                if (!valid || c0 >= p.Cout) continue;
                if (KIND == 2) {
                    const int *wtot = reinterpret_cast<const int *>(ep0) + cc * 32;
                    const int *badd = reinterpret_cast<const int *>(ep1) + cc * 32;
                    const int satw = p.kW + 1, satn = (p.kH + 1) * (p.kW + 1);
                    uint32_t outw[8];
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int c = c0 + i;
                        int q = 0;
                        if (c < p.Cout) {
                            int wv;
                            if (interior) wv = wtot[i];
                            else {
                                const int *t = p.wsat + (size_t)c * satn;
                                wv = t[r1 * satw + s1] - t[r0 * satw + s1] - t[r1 * satw + s0] + t[r0 * satw + s0];
                            }
                            const int a = (int)acc[i] + p.b_off * wv + corr_pix;
                            if (p.acc_out) p.acc_out[(size_t)pm * p.Cout + c] = a;
                            uint32_t v = ((uint32_t)a + (uint32_t)p.c_off) * (uint32_t)p.c_mult;
                            if (p.c_shift >= 1) v += 1u << (p.c_shift - 1);
                            int sres = (int)v;
                            if (p.c_shift > 0) sres >>= p.c_shift;
                            q = min(255, max(0, sres));
                            int t2 = q + badd[i];
                            if (plane_pos < p.tail_start) t2 = min(255, max(0, t2));
                            else t2 = t2 > 255 ? 255 : (t2 & 255);
                            q = t2;
                            if (p.relu_thr >= 0) q = q > p.relu_thr ? q : p.relu_val;
                        }
                        if ((i & 3) == 0) outw[i >> 2] = 0;
                        outw[i >> 2] |= (uint32_t)q << (8 * (i & 3));
                    }
                    uint8_t *dst = p.y + (size_t)pm * p.out_ld + c0;
#pragma unroll
                    for (int v4 = 0; v4 < 2; v4++)
                        if (c0 + v4 * 16 < p.Cout)
                            *reinterpret_cast<uint4 *>(dst + v4 * 16) =
                                make_uint4(outw[v4 * 4], outw[v4 * 4 + 1], outw[v4 * 4 + 2], outw[v4 * 4 + 3]);
                } else {
                    const float *sc = ep0 + cc * 32, *sh = ep1 + cc * 32, *sl = ep2 + cc * 32;
                    const uint8_t *rsrc = p.res ? p.res + ((size_t)pm * p.res_ld + c0) * 2 : nullptr;
                    uint8_t *dst = p.y + ((size_t)pm * p.out_ld + c0) * 2;
#pragma unroll
                    for (int v8 = 0; v8 < 4; v8++) {
                        if (c0 + v8 * 8 >= p.Cout) break;
                        uint4 rv = make_uint4(0, 0, 0, 0);
                        if (rsrc) rv = *reinterpret_cast<const uint4 *>(rsrc + v8 * 16);
                        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            const int i = v8 * 8 + h * 2;
                            float v0 = __uint_as_float(acc[i]) * sc[i] + sh[i];
                            float v1 = __uint_as_float(acc[i + 1]) * sc[i + 1] + sh[i + 1];
                            if (rsrc) {
                                float2 rr = unpack2(rw[h], KIND);
                                v0 = p.self_coef * v0 + p.res_coef * rr.x;
                                v1 = p.self_coef * v1 + p.res_coef * rr.y;
                            }
                            v0 = thb_apply_act(v0, p.act_kind, p.act_th, p.act_val, p.act_alpha, sl[i]);
                            v1 = thb_apply_act(v1, p.act_kind, p.act_th, p.act_val, p.act_alpha, sl[i + 1]);
                            if (c0 + i >= p.Cout) v0 = 0.f;
                            if (c0 + i + 1 >= p.Cout) v1 = 0.f;
                            ow[h] = pack2(v0, v1, KIND);
                        }
                        *reinterpret_cast<uint4 *>(dst + v8 * 16) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------------ weight (B) TMA producer
        if (lane == 0) {
            for (int kb = 0; kb < p.nkb; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1)) {
                    atomicExch(p.status, 3);
                    *abort_flag = 1;
                    break;
                }
                mbar_arrive_expect_tx(smem_u32(&full[s]), B_STAGE_BYTES);
                tma_load_2d(smem_u32(sB + s * B_STAGE_BYTES), &tmapW, smem_u32(&full[s]), kb * BKE, n0);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < p.nkb; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait_bounded(smem_u32(&full[s]), ph)) {
                    atomicExch(p.status, 4);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                fence_proxy_async_smem();
                const uint64_t adesc = make_sw128_kmajor_desc(smem_u32(sA + s * A_STAGE_BYTES));
                const uint64_t bdesc = make_sw128_kmajor_desc(smem_u32(sB + s * B_STAGE_BYTES));
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const uint32_t accum = (kb | k) != 0;
                    if (KIND == 2) tc_mma_i8(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, accum);
                    else tc_mma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, accum);
                }
                tc_commit(smem_u32(&empty[s]));
            }
            if (ok) tc_commit(smem_u32(tmem_full));
        }
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BN, int STAGES> constexpr size_t conv_tc_smem()
{
    return 1024 + (size_t)STAGES * (A_STAGE_BYTES + BN * 128) + (2 * STAGES + 1) * 8 + 8 + 3 * BN * 4 + 64;
}

template <int KIND, int BN, int STAGES>
int launch_tc(const CUtensorMap &tm, const ConvTcParams &p, int gx, int gy, cudaStream_t st)
{
    static bool configured = false;
    auto kern = conv_tc_kernel<KIND, BN, STAGES>;
    constexpr size_t smem = conv_tc_smem<BN, STAGES>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return thb_note_launch(e, "conv_tc smem attribute");
        configured = true;
    }
    kern<<<dim3(gx, gy), 192, smem, st>>>(tm, p);
    return THB_LAUNCH_CHECK("conv_tc_kernel");
}

template <int KIND>
int dispatch_bn(int BN, const CUtensorMap &tm, const ConvTcParams &p, int gx, int gy, cudaStream_t st)
{
    switch (BN) {
    case 32: return launch_tc<KIND, 32, 4>(tm, p, gx, gy, st);
    case 64: return launch_tc<KIND, 64, 4>(tm, p, gx, gy, st);
    case 128: return launch_tc<KIND, 128, 3>(tm, p, gx, gy, st);
    case 256: return launch_tc<KIND, 256, 4>(tm, p, gx, gy, st);
    }
    return THB_ERR_UNSUPPORTED;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode_fn()
{
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(sym);
    }
    return fn;
}

}  // namespace

extern "C" int thb_conv_make_tmap(const thb_conv_desc *d, thb_tmap *out)
{
    if (d->dtype == THB_F32) return THB_ERR_ARG;
    encode_tiled_fn enc = get_encode_fn();
    if (!enc) return thb_note_launch(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    const int es = d->dtype == THB_U8 ? 1 : 2;
    CUtensorMapDataType t = d->dtype == THB_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                            : d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {(cuuint64_t)d->Ktot_pad, (cuuint64_t)d->Cout_pad};
    cuuint64_t strides[1] = {(cuuint64_t)d->Ktot_pad * es};
    cuuint32_t box[2] = {(cuuint32_t)(128 / es), (cuuint32_t)d->BN};
    cuuint32_t estr[2] = {1, 1};
    static_assert(sizeof(CUtensorMap) == sizeof(thb_tmap), "tensor map size");
    CUresult r = enc(reinterpret_cast<CUtensorMap *>(out), t, 2, const_cast<void *>(d->w), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "thb200: cuTensorMapEncodeTiled failed (%d)\n", (int)r);
        return THB_ERR_CUDA;
    }
    return THB_OK;
}

extern "C" int thb_conv_fwd_tc(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    if (!d->tmap || !d->w || !d->kinfo) return THB_ERR_ARG;
    const int es = d->dtype == THB_U8 ? 1 : 2, ce = 16 / es;
    if (d->in_ld % ce || d->out_ld % ce || (d->res && d->res_ld % ce)) return THB_ERR_ARG;
    ConvTcParams p;
    memset(&p, 0, sizeof(p));
    p.x = (const uint8_t *)x;
    p.y = (uint8_t *)y;
    p.kinfo = d->kinfo;
    p.P = d->N * d->oH * d->oW;
    p.H = d->H; p.W = d->W; p.in_ld = d->in_ld; p.oW = d->oW; p.oHW = d->oH * d->oW;
    p.dH = d->dH; p.dW = d->dW; p.padH = d->padH; p.padW = d->padW; p.kH = d->kH; p.kW = d->kW;
    p.Cin = d->Cin; p.Cout = d->Cout; p.out_ld = d->out_ld;
    p.nkb = d->Ktot_pad / (128 / es);
    p.n_kchunks = d->Ktot_pad / ce;
    p.scale = d->scale; p.shift = d->shift; p.slope = d->act.kind == THB_ACT_PRELU ? d->act.slope : nullptr;
    p.res = (const uint8_t *)d->res; p.res_ld = d->res_ld;
    p.self_coef = d->self_coef; p.res_coef = d->res_coef;
    p.act_kind = d->act.kind; p.act_th = d->act.threshold; p.act_val = d->act.value; p.act_alpha = d->act.alpha;
    p.a_off = d->a_offset; p.b_off = d->b_offset; p.c_off = d->c_offset; p.c_mult = d->c_mult; p.c_shift = d->c_shift;
    p.wsat = d->wsat; p.bias_add = d->bias_add; p.csum = d->csum;
    p.tail_start = d->tail_start; p.relu_thr = d->relu_thr; p.relu_val = d->relu_val;
    p.acc_out = d->acc_out;
    p.status = d->status;
    if (!p.status) return THB_ERR_ARG;
    if (d->dtype == THB_U8 && (!p.wsat || !p.csum)) return THB_ERR_ARG;
    if (p.P <= 0) return THB_OK;
    const int gx = (p.P + BM - 1) / BM, gy = d->Cout_pad / d->BN;
    const CUtensorMap &tm = *reinterpret_cast<const CUtensorMap *>(d->tmap);
    cudaStream_t st = (cudaStream_t)s;
    switch (d->dtype) {
    case THB_F16: return dispatch_bn<0>(d->BN, tm, p, gx, gy, st);
    case THB_BF16: return dispatch_bn<1>(d->BN, tm, p, gx, gy, st);
    case THB_U8: return dispatch_bn<2>(d->BN, tm, p, gx, gy, st);
    }
    return THB_ERR_UNSUPPORTED;
}
