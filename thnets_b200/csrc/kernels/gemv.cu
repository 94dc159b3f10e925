// Batch-small Linear (N <= 8 rows of x): y[n][m] = act((sum_k W[m][k] x[n][k]) * scale[m] + shift[m]).
// HBM-bound on the weight matrix: one warp per output row streams W[m][:] once with 16-byte loads
// (four in flight per lane), keeps the x rows in L1/L2, accumulates in fp32 and reduces by shuffles.
#include "common.cuh"

namespace {

template <typename T> struct V16;
template <> struct V16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4 &t, float (&v)[4])
    {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y); v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
};
template <> struct V16<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4 &t, float (&v)[8])
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};
template <> struct V16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4 &t, float (&v)[8])
    {
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};

template <typename T, int NB>
__global__ void __launch_bounds__(256) gemv_kernel(const T *x, int K, int x_ld, const T *w, int M, const float *scale,
                                                   const float *shift, thb_act act, T *y, int y_ld)
{
    constexpr int VN = V16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x * 8 + warp;
    if (m >= M) {
        // channels of the padded tail of y are kept at exact zero
        if (m < (M + VN - 1) / VN * VN && m < y_ld && lane == 0)
            for (int n = 0; n < NB; n++) dt<T>::st(y + (size_t)n * y_ld + m, 0.f);
        return;
    }
    const uint4 *wr = reinterpret_cast<const uint4 *>(w + (size_t)m * K);
    const int nvec = K / VN;
    float acc[NB];
#pragma unroll
    for (int n = 0; n < NB; n++) acc[n] = 0.f;
    for (int v0 = lane; v0 < nvec; v0 += 128) {
        uint4 wv[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            wv[u] = (v0 + u * 32 < nvec) ? __ldcs(wr + v0 + u * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (v0 + u * 32 >= nvec) break;
            float wf[VN];
            V16<T>::unpack(wv[u], wf);
#pragma unroll
            for (int n = 0; n < NB; n++) {
                float xf[VN];
                V16<T>::unpack(*reinterpret_cast<const uint4 *>(x + (size_t)n * x_ld + (size_t)(v0 + u * 32) * VN), xf);
#pragma unroll
                for (int i = 0; i < VN; i++) acc[n] = fmaf(wf[i], xf[i], acc[n]);
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NB; n++)
        for (int o = 16; o > 0; o >>= 1) acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], o);
    if (lane == 0) {
        const float sc = scale ? scale[m] : 1.f, sh = shift ? shift[m] : 0.f;
        const float sl = act.kind == THB_ACT_PRELU ? act.slope[m] : 0.f;
#pragma unroll
        for (int n = 0; n < NB; n++)
            dt<T>::st(y + (size_t)n * y_ld + m, thb_apply_act(acc[n] * sc + sh, act.kind, act.threshold, act.value, act.alpha, sl));
    }
}

template <typename T>
int launch_gemv(const void *x, int N, int K, int x_ld, const void *w, int M, const float *scale, const float *shift,
                thb_act a, void *y, int y_ld, cudaStream_t st)
{
    const int grid = (M + 7) / 8 + 1;
#define GEMV_CASE(NB)                                                                                                   \
    case NB:                                                                                                            \
        gemv_kernel<T, NB><<<grid, 256, 0, st>>>((const T *)x, K, x_ld, (const T *)w, M, scale, shift, a, (T *)y, y_ld); \
        break;
    switch (N) {
        GEMV_CASE(1) GEMV_CASE(2) GEMV_CASE(3) GEMV_CASE(4) GEMV_CASE(5) GEMV_CASE(6) GEMV_CASE(7) GEMV_CASE(8)
    default: return THB_ERR_UNSUPPORTED;
    }
#undef GEMV_CASE
    return THB_LAUNCH_CHECK("gemv_kernel");
}

}  // namespace

extern "C" int thb_gemv_fwd(int dtype, const void *x, int N, int K, int x_ld, const void *w, int M, const float *scale,
                            const float *shift, const thb_act *act, void *y, int y_ld, thb_stream s)
{
    const int al = thb_channel_align(dtype);
    if (N < 1 || N > 8 || K % al || x_ld % al) return THB_ERR_UNSUPPORTED;
    thb_act a = {THB_ACT_NONE, 0, 0, 0, nullptr};
    if (act) a = *act;
    cudaStream_t st = (cudaStream_t)s;
    switch (dtype) {
    case THB_F32: return launch_gemv<float>(x, N, K, x_ld, w, M, scale, shift, a, y, y_ld, st);
    case THB_F16: return launch_gemv<__half>(x, N, K, x_ld, w, M, scale, shift, a, y, y_ld, st);
    case THB_BF16: return launch_gemv<__nv_bfloat16>(x, N, K, x_ld, w, M, scale, shift, a, y, y_ld, st);
    }
    return THB_ERR_UNSUPPORTED;
}
