// Batch-small Linear (N <= 8 rows of x): y[n][m] = act((sum_k W[m][k] x[n][k]) * scale[m] + shift[m]).
// HBM-bound on the weight matrix: W is streamed once with 16-byte loads (four to eight in flight per thread), the x rows
// stay in L1/L2, sums are fp32.
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

// One CTA per weight row at a time, rows taken with a grid stride by a grid that is resident all at once.  Each thread owns
// the vectors tid, tid+256, ... of a row in batches of U; the batch after the one being accumulated is already in flight
// (two register buffers, running on into the CTA's next row), so the stream of loads never drains at a row's end.
template <typename T, int NB>
struct GemvWalk {
    static constexpr int U = 4;
    const uint4 *w;
    int nvec, nbatch, M, stride;
    int row, b;  // next batch to load: row and batch index inside the row
    __device__ __forceinline__ void load(uint4 (&buf)[U])
    {
        if (row >= M) return;
        const uint4 *wr = w + (size_t)row * nvec;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = (b * U + u) * 256 + threadIdx.x;
            buf[u] = v < nvec ? __ldcs(wr + v) : make_uint4(0, 0, 0, 0);
        }
        if (++b == nbatch) { b = 0; row += stride; }
    }
};

template <typename T, int NB>
__global__ void __launch_bounds__(256, 4) gemv_kernel(const T *x, int K, int x_ld, const T *w, int M, const float *scale,
                                                      const float *shift, thb_act act, T *y, int y_ld)
{
    constexpr int VN = V16<T>::N, U = GemvWalk<T, NB>::U;
    __shared__ float part[2][8][NB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = K / VN;
    GemvWalk<T, NB> walk{reinterpret_cast<const uint4 *>(w), nvec, (nvec + U * 256 - 1) / (U * 256), M, (int)gridDim.x,
                         (int)blockIdx.x, 0};
    uint4 buf0[U], buf1[U];
    // Programmatic dependent launch: the weights do not depend on the kernel before this one, so the first batch of
    // every CTA is on its way while that kernel drains (and the next kernel of the stream may start its own in the same
    // way); x is read and y written only after the wait.
    walk.load(buf0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (blockIdx.x == 0) {
        // channels of the padded tail of y are kept at exact zero
        const int m = M + threadIdx.x;
        if (m < (M + VN - 1) / VN * VN && m < y_ld)
            for (int n = 0; n < NB; n++) dt<T>::st(y + (size_t)n * y_ld + m, 0.f);
    }
    float acc[NB];
#pragma unroll
    for (int n = 0; n < NB; n++) acc[n] = 0.f;
    int crow = blockIdx.x, cb = 0, parity = 0;

    auto consume = [&](const uint4 (&buf)[U]) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = (cb * U + u) * 256 + threadIdx.x;
            if (v < nvec) {
                float wf[VN];
                V16<T>::unpack(buf[u], wf);
#pragma unroll
                for (int n = 0; n < NB; n++) {
                    float xf[VN];
                    V16<T>::unpack(*reinterpret_cast<const uint4 *>(x + (size_t)n * x_ld + (size_t)v * VN), xf);
#pragma unroll
                    for (int i = 0; i < VN; i++) acc[n] = fmaf(wf[i], xf[i], acc[n]);
                }
            }
        }
        if (++cb < walk.nbatch) return;
        // the row is complete: warp sums, then warp 0 adds the eight partial sums (buffers alternate between rows, so
        // one barrier per row is enough)
#pragma unroll
        for (int n = 0; n < NB; n++) {
            for (int o = 16; o > 0; o >>= 1) acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], o);
            if (lane == 0) part[parity][warp][n] = acc[n];
            acc[n] = 0.f;
        }
        __syncthreads();
        if (threadIdx.x < NB) {
            const int n = threadIdx.x, m = crow;
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) s += part[parity][q][n];
            const float sc = scale ? scale[m] : 1.f, sh = shift ? shift[m] : 0.f;
            const float sl = act.kind == THB_ACT_PRELU ? act.slope[m] : 0.f;
            dt<T>::st(y + (size_t)n * y_ld + m, thb_apply_act(s * sc + sh, act.kind, act.threshold, act.value, act.alpha, sl));
        }
        parity ^= 1;
        cb = 0;
        crow += gridDim.x;
    };

    while (crow < M) {
        walk.load(buf1);
        consume(buf0);
        if (crow >= M) break;
        walk.load(buf0);
        consume(buf1);
    }
}

template <typename T>
int launch_gemv(const void *x, int N, int K, int x_ld, const void *w, int M, const float *scale, const float *shift,
                thb_act a, void *y, int y_ld, cudaStream_t st)
{
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int grid = M < 4 * sms ? M : 4 * sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaSuccess;
#define GEMV_CASE(NB)                                                                                                   \
    case NB:                                                                                                            \
        le = cudaLaunchKernelEx(&cfg, gemv_kernel<T, NB>, (const T *)x, K, x_ld, (const T *)w, M, scale, shift, a, (T *)y, y_ld); \
        break;
    switch (N) {
        GEMV_CASE(1) GEMV_CASE(2) GEMV_CASE(3) GEMV_CASE(4) GEMV_CASE(5) GEMV_CASE(6) GEMV_CASE(7) GEMV_CASE(8)
    default: return THB_ERR_UNSUPPORTED;
    }
#undef GEMV_CASE
    if (le != cudaSuccess) return thb_note_launch(le, "gemv_kernel");
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
