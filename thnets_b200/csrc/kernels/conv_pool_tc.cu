// Convolution + bias/BatchNorm + activation + 2-strided max pooling in ONE launch (fp16 / bf16, tcgen05).
//
// The reference runs SpatialMaxPooling as a pass of its own over the convolution's output
// (modules/SpatialMaxPooling.c:168-247).  Here the convolution's output never reaches global memory: a CTA
// computes a rectangular PATCH of convolution outputs that holds whole pooling windows, pools it on chip and
// stores only the pooled tile.  For a ResNet stem that removes a 411 MB write, the 411 MB read and a launch.
//
// Work unit: a tile of PR x PC pooled pixels of one image = a patch of CR x CC convolution outputs
// (CR = 2(PR-1)+kp, CC = 2(PC-1)+kp, CR*CC <= 256; 3x3/s2 pooling: 7 x 8 pooled from 15 x 17, 2x2/s2: 8 x 8 from
// 16 x 16).  Neighbouring patches of a 3x3 pooling overlap by one row and column, which are computed twice (12 %).
// The patch is the M dimension of TWO 128-row accumulators in TMEM; its row m = cr*CC + cc.
//
// Per K block ONE tiled 4-D TMA copy fetches the whole patch's activation rows (box {64 channels, CC, CR, 1} of the
// channels-innermost input at the tap's offset; rows and columns outside the image read as zeros), and one 2-D copy
// fetches the 64 x 128-byte weight tile.  K blocks are either 128-byte channel slabs of one tap (Cin_pad a multiple
// of 64), or -- for an input whose rows are stored with their zero padding and whose kW taps fill 128 bytes -- one
// whole kernel row per copy through overlapping 128-byte windows (the space-to-depth first layer).
//
// Warps: 0 TMA producer, 1 MMA issuer (8 x tcgen05.mma 128x64x16 per K block), 2-9 epilogue.  An epilogue thread
// owns one patch row: TMEM -> scale/shift/activation -> fp16 row in a shared-memory patch tile; after a barrier
// among the 256 epilogue threads each of them pools 16-byte channel chunks (windows clipped to the image as the
// reference clips them) into the pooled tile, which one thread hands to a 4-D TMA store.
// Every wait is bounded; a wait that runs out records a code in *status and the CTA drains and exits.
#include "common.cuh"
#include <cuda.h>
#include <string.h>
#include <stdio.h>
#include <stdlib.h>

namespace {

constexpr int CP_THREADS = 320;
constexpr int CP_MAX_STAGES = 4;
constexpr int CP_A_BYTES = 256 * 128;   // patch rows of one K block
constexpr int CP_B_BYTES = 64 * 128;    // 64 output channels x one K block
constexpr int CP_STAGE_BYTES = CP_A_BYTES + CP_B_BYTES;
constexpr int CP_CT_BYTES = 256 * 128;  // activated patch, one 128-byte row per convolution output
constexpr int CP_PT_BYTES = 64 * 128;   // pooled tile (at most 64 pooled pixels), two of them
constexpr size_t CP_SMEM = 1024 + 1024 + (size_t)CP_MAX_STAGES * CP_STAGE_BYTES + CP_CT_BYTES + 2 * CP_PT_BYTES + 1024;

struct ConvPoolParams {
    int N, oH, oW;         // convolution output
    int pH, pW;            // pooled output
    int kp, pp;            // pooling window (2 or 3) and padding; stride 2
    int PR, PC, CR, CC;    // pooled tile, convolution patch
    int tiles_r, tiles_c;  // pooled tiles per image
    int nkb, window_rows;  // K blocks; 1: a K block is a kernel row fetched through overlapping windows
    int kW, padH, padW, slabs;
    int Cout;
    const float *scale, *shift, *slope;
    int act_kind;
    float act_th, act_val, act_alpha;
    int kind;  // 0 fp16, 1 bf16
    int pdl;
    int *status;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
        "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void *tmap, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tmap), "r"(src),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
// barrier among the 256 epilogue threads only
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_pair(float a, float b, int kind)
{
    if (kind == 0) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t max_pair(uint32_t a, uint32_t b, int kind)
{
    if (kind == 0) {
        __half2 r = __hmax2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

struct Unit {
    int n, pr0, pc0;
};
__device__ __forceinline__ Unit unit_of(const ConvPoolParams &p, int u)
{
    const int per_img = p.tiles_r * p.tiles_c;
    Unit q;
    q.n = u / per_img;
    const int rem = u - q.n * per_img;
    const int tr = rem / p.tiles_c;
    q.pr0 = tr * p.PR;
    q.pc0 = (rem - tr * p.tiles_c) * p.PC;
    return q;
}

__global__ void __launch_bounds__(CP_THREADS, 1)
conv_pool_tc_kernel(const __grid_constant__ CUtensorMap tmapW, const __grid_constant__ CUtensorMap tmapA,
                    const __grid_constant__ CUtensorMap tmapP, const ConvPoolParams p, const int nst)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem), *empty = full + CP_MAX_STAGES;
    uint64_t *acc_full = empty + CP_MAX_STAGES, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *s_scale = reinterpret_cast<float *>(smem + 256), *s_shift = s_scale + 64, *s_slope = s_shift + 64;
    uint8_t *sA = smem + 1024;                          // per stage: the patch's rows, then the weight tile
    uint8_t *ct = sA + nst * CP_STAGE_BYTES;            // (1024-byte aligned: both sizes are multiples of 1024)
    uint8_t *pt = ct + CP_CT_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int units = p.N * p.tiles_r * p.tiles_c;
    const int mine = (int)blockIdx.x < units ? (units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    constexpr uint32_t TMEM_COLS = 256;  // two units x two 64-column accumulators

    if (tid == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 256);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (tid < 64) {
        // per-channel epilogue constants (host memory written before any launch: not produced by the previous kernel)
        const bool real = tid < p.Cout;
        s_scale[tid] = real ? (p.scale ? p.scale[tid] : 1.f) : 0.f;
        s_shift[tid] = real ? (p.shift ? p.shift[tid] : 0.f) : 0.f;
        s_slope[tid] = real && p.slope ? p.slope[tid] : 0.f;
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmapW);
        tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapP);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (warp == 0) {
        // ================================================================== TMA producer
        if (lane == 0) {
            int ring_s = 0;
            uint32_t ring_ph = 0;
            bool alive = true;
            for (int u = 0; u < mine && alive; u++) {
                const Unit q = unit_of(p, blockIdx.x + u * gridDim.x);
                const int r0 = 2 * q.pr0 - p.pp - p.padH, c0 = 2 * q.pc0 - p.pp;  // input row of tap row 0; first patch column
                int tap_r = 0, tap_s = 0, slab = 0;
                for (int kb = 0; kb < p.nkb; kb++) {
                    const int s = ring_s;
                    const uint32_t ph = ring_ph;
                    if (++ring_s == nst) { ring_s = 0; ring_ph ^= 1; }
                    if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1)) {
                        atomicExch(p.status, 3);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full[s]);
                    mbar_arrive_expect_tx(bar, (uint32_t)(p.CR * p.CC * 128 + CP_B_BYTES));
                    uint8_t *stage = sA + s * CP_STAGE_BYTES;
                    if (p.window_rows) {
                        // window position w = the kW taps of output column w (rows stored with their padding)
                        tma_load_4d(smem_u32(stage), &tmapA, bar, 0, c0, r0 + kb, q.n);
                    } else {
                        tma_load_4d(smem_u32(stage), &tmapA, bar, slab * 64, c0 - p.padW + tap_s, r0 + tap_r, q.n);
                        if (++slab == p.slabs) {
                            slab = 0;
                            if (++tap_s == p.kW) { tap_s = 0; tap_r++; }
                        }
                    }
                    tma_load_2d(smem_u32(stage + CP_A_BYTES), &tmapW, bar, kb * 64, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC_F16 = make_idesc(1u, 0u, 64), IDESC_BF16 = make_idesc(1u, 1u, 64);
            const uint32_t idesc = p.kind == 1 ? IDESC_BF16 : IDESC_F16;
            int ring_s = 0;
            uint32_t ring_ph = 0;
            bool alive = true;
            for (int u = 0; u < mine && alive; u++) {
                const int ab = u & 1;
                if (!mbar_wait_bounded(smem_u32(&acc_empty[ab]), ((u >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 6);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + ab * 128, d1 = d0 + 64;
                for (int kb = 0; kb < p.nkb; kb++) {
                    const int s = ring_s;
                    const uint32_t ph = ring_ph;
                    if (++ring_s == nst) { ring_s = 0; ring_ph ^= 1; }
                    if (!mbar_wait_bounded(smem_u32(&full[s]), ph)) {
                        atomicExch(p.status, 4);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t adesc = make_sw128_kmajor_desc(smem_u32(sA + s * CP_STAGE_BYTES));
                    const uint64_t bdesc = make_sw128_kmajor_desc(smem_u32(sA + s * CP_STAGE_BYTES + CP_A_BYTES));
#pragma unroll
                    for (int k = 0; k < 4; k++) tc_mma_f16(d0, adesc + 2 * k, bdesc + 2 * k, idesc, (uint32_t)((kb | k) != 0));
#pragma unroll
                    for (int k = 0; k < 4; k++)  // patch rows 128..255 lie 16 KB further on (1024 sixteen-byte units)
                        tc_mma_f16(d1, adesc + 1024 + 2 * k, bdesc + 2 * k, idesc, (uint32_t)((kb | k) != 0));
                    tc_commit(smem_u32(&empty[s]));
                }
                if (alive) tc_commit(smem_u32(&acc_full[ab]));
            }
        }
        __syncwarp();
    } else {
        // ================================================================== epilogue: activate, pool, store
        const int et = tid - 64;                 // 0..255
        const int quad = warp & 3;               // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;        // accumulator half: patch rows 0..127 / 128..255
        const int m = half * 128 + quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + half * 64;
        const int act_mode = p.act_kind == THB_ACT_NONE ? 0
                             : p.act_kind != THB_ACT_THRESHOLD ? 2
                             : (p.act_th == 0.f && p.act_val == 0.f) ? 3 : 1;
        const int items = p.PR * p.PC * 8;       // (pooled pixel, 16-byte channel chunk)
        const uint32_t neg_inf2 = p.kind == 0 ? 0xFC00FC00u : 0xFF80FF80u;
        uint8_t *row_smem = ct + m * 128;
        const int rsw = m & 7;
        for (int u = 0; u < mine; u++) {
            const int ab = u & 1;
            const Unit q = unit_of(p, blockIdx.x + u * gridDim.x);
            if (!mbar_wait_bounded(smem_u32(&acc_full[ab]), (u >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 2);
                *abort_flag = 1;
            }
            tc_fence_after();
            uint32_t acc0[32], acc1[32];
            __syncwarp();
            tmem_ld32(lane_addr + ab * 128, acc0);
            tmem_ld32(lane_addr + ab * 128 + 32, acc1);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&acc_empty[ab]));
            // this thread's convolution output: 64 channels -> eight 16-byte chunks of its patch-tile row
#pragma unroll
            for (int cj = 0; cj < 8; cj++) {
                const uint32_t *a = cj < 4 ? acc0 + cj * 8 : acc1 + (cj - 4) * 8;
                uint32_t ow[4];
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    const int c = cj * 8 + h * 2;
                    float v0 = fmaf(__uint_as_float(a[h * 2]), s_scale[c], s_shift[c]);
                    float v1 = fmaf(__uint_as_float(a[h * 2 + 1]), s_scale[c + 1], s_shift[c + 1]);
                    if (act_mode == 3) {
                        v0 = fmaxf(v0, 0.f);
                        v1 = fmaxf(v1, 0.f);
                    } else if (act_mode != 0) {
                        v0 = c < p.Cout ? thb_apply_act(v0, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c]) : 0.f;
                        v1 = c + 1 < p.Cout ? thb_apply_act(v1, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c + 1]) : 0.f;
                    }
                    ow[h] = pack_pair(v0, v1, p.kind);
                }
                *reinterpret_cast<uint4 *>(row_smem + ((cj ^ rsw) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
            epi_bar_sync();                       // the activated patch is complete
            if (*abort_flag) break;               // (read after the barrier: every thread sees the same value)
            uint8_t *ptile = pt + (u & 1) * CP_PT_BYTES;
            for (int it = et; it < items; it += 256) {
                const int px = it >> 3, j = it & 7;
                const int pr = px / p.PC, pc = px - pr * p.PC;
                // window of pooled pixel (pr0 + pr, pc0 + pc), clipped to the convolution output
                const int gr0 = 2 * (q.pr0 + pr) - p.pp, gc0 = 2 * (q.pc0 + pc) - p.pp;
                uint32_t mx[4] = {neg_inf2, neg_inf2, neg_inf2, neg_inf2};
                for (int dr = 0; dr < p.kp; dr++) {
                    if ((unsigned)(gr0 + dr) >= (unsigned)p.oH) continue;
                    for (int dc = 0; dc < p.kp; dc++) {
                        if ((unsigned)(gc0 + dc) >= (unsigned)p.oW) continue;
                        const int mm = (2 * pr + dr) * p.CC + 2 * pc + dc;
                        const uint4 v = *reinterpret_cast<const uint4 *>(ct + mm * 128 + ((j ^ (mm & 7)) << 4));
                        mx[0] = max_pair(mx[0], v.x, p.kind);
                        mx[1] = max_pair(mx[1], v.y, p.kind);
                        mx[2] = max_pair(mx[2], v.z, p.kind);
                        mx[3] = max_pair(mx[3], v.w, p.kind);
                    }
                }
                *reinterpret_cast<uint4 *>(ptile + px * 128 + j * 16) = make_uint4(mx[0], mx[1], mx[2], mx[3]);
            }
            fence_proxy_async_smem();             // the pooled rows must be visible to the copy engine
            epi_bar_sync();                       // pooled tile complete; the patch tile may be overwritten
            if (et == 0) {
                tma_store_4d(&tmapP, smem_u32(ptile), 0, q.pc0, q.pr0, q.n);  // clips pooled pixels beyond the map
                bulk_commit_group();
                bulk_wait_group_read<1>();        // the OTHER pooled tile's store has read it out
            }
        }
        if (et == 0) bulk_wait_group<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn cp_encode_fn()
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

// geometry of the pooled tile and its patch
void pool_tile(int kp, int *PR, int *PC)
{
    if (kp == 3) { *PR = 7; *PC = 8; }   // patch 15 x 17 = 255 rows
    else { *PR = 8; *PC = 8; }           // patch 16 x 16 = 256 rows
}

// Tensor map of the convolution input for patch boxes of CR x CC positions.  Plain input: {C, W, H, N}.  Rows stored
// with their padding: {128-byte window, window position, H, N} with windows one pixel (in_ld elements) apart, so that
// position w is the kW taps of output column w -- the windows overlap, which the encoder has to accept.
bool encode_input_map(const thb_conv_desc *d, const void *x, int CR, int CC, CUtensorMap *out)
{
    encode_tiled_fn enc = cp_encode_fn();
    if (!enc) return false;
    const CUtensorMapDataType t = d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint32_t estr[4] = {1, 1, 1, 1};
    cuuint64_t dims[4] = {(cuuint64_t)d->Cin_pad, (cuuint64_t)d->W, (cuuint64_t)d->H, (cuuint64_t)d->N};
    cuuint64_t strides[3] = {(cuuint64_t)d->in_ld * 2, (cuuint64_t)d->W * d->in_ld * 2, (cuuint64_t)d->H * d->W * d->in_ld * 2};
    if (d->in_row_pitch) {
        dims[0] = 64;
        dims[1] = (cuuint64_t)d->oW;
        strides[1] = (cuuint64_t)d->in_row_pitch * d->in_ld * 2;
        strides[2] = (cuuint64_t)d->H * d->in_row_pitch * d->in_ld * 2;
    }
    cuuint32_t box[4] = {64, (cuuint32_t)CC, (cuuint32_t)CR, 1};
    return enc(out, t, 4, const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct CpMapEntry {
    const void *x, *y;
    int key[16];
    alignas(64) CUtensorMap a, p;
};

bool geometry_ok(const thb_conv_desc *d, int pk, int ps, int ppad)
{
    if (d->dtype != THB_F16 && d->dtype != THB_BF16) return false;
    if (d->Cout > 64 || d->BN != 64 || d->dH != 1 || d->dW != 1 || d->x2 || d->res) return false;
    if ((pk != 2 && pk != 3) || ps != 2 || ppad < 0 || ppad >= pk) return false;
    if (d->padH >= d->kH || d->padW >= d->kW) return false;
    if (d->in_row_pitch) {
        // one kernel row per K block through overlapping windows
        return d->in_pad_left == d->padW && d->kW * d->Cin_pad == 64 && d->Ktot_pad == d->kH * 64 &&
               d->in_row_pitch >= d->oW + d->kW - 1 && d->in_ld == d->Cin_pad;
    }
    return d->Cin_pad % 64 == 0 && d->Ktot_pad == d->kH * d->kW * d->Cin_pad;
}

}  // namespace

// 1 when thb_conv_maxpool_fwd can run this convolution followed by a pk x pk max pooling of stride ps and padding ppad
extern "C" int thb_conv_maxpool_supported(const thb_conv_desc *d, int pk, int ps, int ppad)
{
    static int disabled = -1;
    if (disabled < 0) {
        const char *e = getenv("THB200_NO_CONV_POOL");
        disabled = e && atoi(e) ? 1 : 0;
    }
    if (disabled || !geometry_ok(d, pk, ps, ppad)) return 0;
    if (d->in_row_pitch) {
        // the overlapping-window descriptor: ask the encoder once per type (only its checks matter: dummy address)
        static int ok[4] = {-1, -1, -1, -1};
        if (ok[d->dtype] < 0) {
            if (cudaFree(0) != cudaSuccess) return 0;
            int PR, PC;
            pool_tile(pk, &PR, &PC);
            alignas(64) CUtensorMap tmp;
            ok[d->dtype] = encode_input_map(d, reinterpret_cast<const void *>(uintptr_t(1) << 20), 2 * (PR - 1) + pk, 2 * (PC - 1) + pk, &tmp) ? 1 : 0;
        }
        return ok[d->dtype];
    }
    return 1;
}

extern "C" int thb_conv_maxpool_fwd(const thb_conv_desc *d, int pk, int ps, int ppad, int pH, int pW, const void *x, void *y,
                                    int y_ld, thb_stream s)
{
    if (!d || !x || !y || !d->tmap || !d->status) return THB_ERR_ARG;
    if (!geometry_ok(d, pk, ps, ppad)) return THB_ERR_UNSUPPORTED;
    if (pH < 1 || pW < 1 || y_ld % 8 || d->in_ld % 8) return THB_ERR_ARG;
    // every pooling window must start inside the convolution output (SpatialMaxPooling.c:196-210 guarantees it)
    if (2 * (pH - 1) - ppad >= d->oH || 2 * (pW - 1) - ppad >= d->oW) return THB_ERR_ARG;
    encode_tiled_fn enc = cp_encode_fn();
    if (!enc) return thb_note_launch(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");

    ConvPoolParams p;
    memset(&p, 0, sizeof(p));
    p.N = d->N; p.oH = d->oH; p.oW = d->oW; p.pH = pH; p.pW = pW; p.kp = pk; p.pp = ppad;
    pool_tile(pk, &p.PR, &p.PC);
    p.CR = 2 * (p.PR - 1) + pk;
    p.CC = 2 * (p.PC - 1) + pk;
    p.tiles_r = (pH + p.PR - 1) / p.PR;
    p.tiles_c = (pW + p.PC - 1) / p.PC;
    p.nkb = d->Ktot_pad / 64;
    p.window_rows = d->in_row_pitch ? 1 : 0;
    p.kW = d->kW; p.padH = d->padH; p.padW = d->padW; p.slabs = d->Cin_pad / 64;
    p.Cout = d->Cout;
    p.scale = d->scale; p.shift = d->shift; p.slope = d->act.kind == THB_ACT_PRELU ? d->act.slope : nullptr;
    p.act_kind = d->act.kind; p.act_th = d->act.threshold; p.act_val = d->act.value; p.act_alpha = d->act.alpha;
    p.kind = d->dtype == THB_BF16 ? 1 : 0;
    p.status = d->status;

    // tensor maps of the input (patch box) and the pooled output (tile box), cached by buffer and shape
    static CpMapEntry cache[64];
    static int used = 0, next = 0;
    const int key[16] = {d->dtype, d->N, d->H, d->W, d->Cin_pad, d->in_ld, d->in_row_pitch, d->oW, pH, pW, y_ld, d->Cout, p.CR, p.CC, p.PR, p.PC};
    CpMapEntry *e = nullptr;
    for (int i = 0; i < used; i++)
        if (cache[i].x == x && cache[i].y == y && !memcmp(cache[i].key, key, sizeof(key))) { e = &cache[i]; break; }
    if (!e) {
        e = &cache[used < 64 ? used++ : (next++ % 64)];
        e->x = nullptr;
        const CUtensorMapDataType t = d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (!encode_input_map(d, x, p.CR, p.CC, &e->a)) return thb_note_launch(cudaErrorInvalidValue, "conv_pool: input tensor map");
        {
            const int c8 = (d->Cout + 7) & ~7;
            cuuint64_t dims[4] = {(cuuint64_t)c8, (cuuint64_t)pW, (cuuint64_t)pH, (cuuint64_t)d->N};
            cuuint64_t strides[3] = {(cuuint64_t)y_ld * 2, (cuuint64_t)pW * y_ld * 2, (cuuint64_t)pH * pW * y_ld * 2};
            cuuint32_t box[4] = {64, (cuuint32_t)p.PC, (cuuint32_t)p.PR, 1};
            if (enc(&e->p, t, 4, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return thb_note_launch(cudaErrorInvalidValue, "conv_pool: pooled output tensor map");
        }
        e->x = x; e->y = y;
        memcpy(e->key, key, sizeof(key));
    }

    static bool configured[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    if (!configured[dev]) {
        cudaError_t ce = cudaFuncSetAttribute(conv_pool_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CP_SMEM);
        if (ce != cudaSuccess) return thb_note_launch(ce, "conv_pool smem attribute");
        configured[dev] = true;
    }
    static int sms[16] = {0};
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    const int units = p.N * p.tiles_r * p.tiles_c;
    const int grid = units < sms[dev] ? units : (sms[dev] > 0 ? sms[dev] : 148);
    const int nst = p.nkb < CP_MAX_STAGES ? (p.nkb < 2 ? 2 : p.nkb) : CP_MAX_STAGES;
    static int use_pdl = -1;
    if (use_pdl < 0) {
        const char *ev = getenv("THB200_PDL");
        use_pdl = ev ? atoi(ev) : 1;
    }
    p.pdl = use_pdl;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(CP_THREADS);
    cfg.dynamicSmemBytes = CP_SMEM;
    cfg.stream = (cudaStream_t)s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, conv_pool_tc_kernel, *reinterpret_cast<const CUtensorMap *>(d->tmap), e->a, e->p, p, nst);
    return thb_note_launch(le != cudaSuccess ? le : cudaGetLastError(), "conv_pool_tc_kernel");
}
