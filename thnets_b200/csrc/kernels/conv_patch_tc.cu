// Patch convolution for stride-1 layers with few channels per pixel (fp16 / bf16, tcgen05): the raw input patch is
// loaded ONCE and every kernel tap reads it in place.
//
// The general kernel (conv_tc.cu) stages one activation tile per K block, so a 3x3 layer pushes every input pixel
// through shared memory nine times and pays a barrier round per tap.  Here a work unit is a rectangular patch of
// CR x CC convolution outputs of one image.  ONE tiled 4-D TMA copy brings the (CR+kH-1) x (CC+kW-1) input pixels the
// patch needs into shared memory as rows of one pixel each (32 bytes for 16 channels, 128 bytes for 64; pixels outside
// the image read as zeros).  With P = CC+kW-1 pixels per patch row, output (cr, cc) of tap (r, s) reads pixel
// (cr+r)*P + cc+s: for a fixed tap that is the SAME sequence of rows shifted by r*P+s pixels, so the A operand of tap
// (r, s) is simply the patch buffer's matrix descriptor advanced by (r*P+s) pixel rows -- the swizzle pattern follows
// the shared-memory address, so any row offset is valid.  The GEMM M index is m = cr*P + cc (256 rows = two 128-row
// accumulators; the kW-1 columns at the end of each patch row compute garbage that is never stored).  The weights of
// all taps stay resident in shared memory for the whole launch.  Per patch: one copy, one barrier round, and
// kH*kW*(pixel bytes / 32) back-to-back tcgen05.mma per accumulator.
//
// Epilogue (8 warps, one thread per patch row): TMEM -> scale/shift/activation -> a 128-byte row of a shared-memory
// tile, then either a 4-D TMA store of the CR x CC outputs, or -- when a stride-2 max pooling follows
// (modules/SpatialMaxPooling.c:168-247) -- the patch holds whole pooling windows (CR = 2(PR-1)+kp), the 256 epilogue
// threads pool it on chip with windows clipped to the image as the reference clips them, and only the PR x PC pooled
// tile is stored: the convolution's own output never reaches global memory.
// Every wait is bounded; a wait that runs out records a code in *status and the CTA drains and exits.
#include "common.cuh"
#include <cuda.h>
#include <string.h>
#include <stdio.h>
#include <stdlib.h>

namespace {

constexpr int PT_THREADS = 640;        // warps: 0 copy producer, 1-2 MMA issuers, 3 idle, 4-19 epilogue
constexpr int PT_MAX_STAGES = 4;
constexpr int PT_NACC = 2;              // accumulator pairs in TMEM: the MMA issuers run one patch ahead of the epilogue (four measured no faster)
constexpr int PT_CT_BYTES = 256 * 128;  // activated outputs of one patch, one 128-byte row each
constexpr int PT_PT_BYTES = 64 * 128;   // pooled tile (at most 64 pooled pixels)
constexpr size_t PT_SMEM_MAX = 232448;

struct PatchParams {
    int N, oH, oW;          // convolution output
    int CR, CC, P;          // patch: output rows, output columns, pixels per patch row (CC + kW - 1)
    int tiles_r, tiles_c;   // patches per image
    int kH, kW, padH, padW;
    int px_bytes;           // bytes per input pixel in shared memory: 32 (16 channels) or 128 (64 channels)
    int xoff;               // zero pixels stored in front of each input row
    int stage_bytes, nst;   // raw patch buffers
    int w_bytes;            // resident weights: kH*kW tiles of 64 rows x px_bytes
    int ct_bufs;            // output tiles without pooling: 2, or 1 when shared memory is short
    int Cout;
    int kp, pp, PR, PC;     // max pooling fused behind the convolution (kp = 0: none): window, padding, pooled tile
    const float *slope;
    float cscale[64], cshift[64];   // per-channel epilogue constants, read straight from the kernel-parameter bank
    int act_kind;
    float act_th, act_val, act_alpha;
    int kind;               // 0 fp16, 1 bf16
    int pdl;
    int has_res;            // a residual tensor (the output's shape) is added before the activation: y = act(conv' + res_coef * r)
    float res_coef;         // (the convolution's own coefficient, +-1, is folded into cscale / cshift)
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
// barrier among the 512 epilogue threads only
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// K-major operand whose rows are `row_bytes` (32 or 128) long and consecutive, swizzled with the pattern of that width:
// 8-row groups 8*row_bytes apart.  The start address may be any multiple of 16 bytes; the pattern follows the address.
__device__ __forceinline__ uint64_t make_rows_desc(uint32_t smem_addr, int row_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8 * row_bytes) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(row_bytes == 128 ? 2 : 6) << 61;   // SWIZZLE_128B : SWIZZLE_32B
    return d;
}

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
    int n, tr, tc, r0, c0;  // image, patch indices, first output row / column of the patch (may be -1 with pooling)
};
__device__ __forceinline__ Unit unit_of(const PatchParams &p, int u)
{
    const int per_img = p.tiles_r * p.tiles_c;
    Unit q;
    q.n = u / per_img;
    const int rem = u - q.n * per_img;
    q.tr = rem / p.tiles_c;
    q.tc = rem - q.tr * p.tiles_c;
    if (p.kp) {
        q.r0 = 2 * q.tr * p.PR - p.pp;
        q.c0 = 2 * q.tc * p.PC - p.pp;
    } else {
        q.r0 = q.tr * p.CR;
        q.c0 = q.tc * p.CC;
    }
    return q;
}

// All tcgen05.mma of ONE tap into one accumulator (KSTEPS instructions of K = 16 elements), descriptors given as
// (low word, high word).  An issuing thread is a single thread whose instruction latency is the kernel's critical
// path: the low word (the 14-bit start-address field, in 16-byte units) is advanced with adds, nothing else is
// recomputed, and the statement carries no memory clobber so that the compiler may fetch the next tap's offset early
// (the operands were made visible by the mbarrier wait and the fence before the loop).
template <int KSTEPS>
__device__ __forceinline__ void mma_tap(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t accumulate)
{
    if (KSTEPS == 1) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %5, 0;\n\t"
            "mov.b64 da, {%1, %3};\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
            "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate));
    } else {
        // four K steps along a 128-byte row: 32 bytes = 2 address units each; `hi` is never zero, so q is always true
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %5, 0;\n\t"
            "setp.ne.b32 q, %3, 0;\n\t"
            "mov.b64 da, {%1, %3};\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
            "add.s64 da, da, 2;\n\t"
            "add.s64 db, db, 2;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t"
            "add.s64 da, da, 2;\n\t"
            "add.s64 db, db, 2;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t"
            "add.s64 da, da, 2;\n\t"
            "add.s64 db, db, 2;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, q;\n\t}" ::"r"(d_tmem),
            "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate));
    }
}

// One thread's 32 accumulator columns (channels CH*32 .. CH*32+31 of its output pixel) -> four 16-byte chunks:
// y = act(acc * scale[c] + shift[c]).  CH is a template argument so that every index into the constants is known at
// compile time: they are then operands of the FFMA itself (kernel-parameter bank), not loads.
template <int CH>
__device__ __forceinline__ void activate_half(const uint32_t (&acc)[32], const PatchParams &p, int act_mode, const float *s_slope,
                                              uint4 (&o)[4])
{
#pragma unroll
    for (int cj = 0; cj < 4; cj++) {
        uint32_t ow[4];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const int c = CH * 32 + cj * 8 + h * 2;
            float v0 = fmaf(__uint_as_float(acc[cj * 8 + h * 2]), p.cscale[c], p.cshift[c]);
            float v1 = fmaf(__uint_as_float(acc[cj * 8 + h * 2 + 1]), p.cscale[c + 1], p.cshift[c + 1]);
            if (act_mode == 3) {
                v0 = fmaxf(v0, 0.f);
                v1 = fmaxf(v1, 0.f);
            } else if (act_mode != 0) {
                v0 = c < p.Cout ? thb_apply_act(v0, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c]) : 0.f;
                v1 = c + 1 < p.Cout ? thb_apply_act(v1, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c + 1]) : 0.f;
            }
            ow[h] = pack_pair(v0, v1, p.kind);
        }
        o[cj] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// the same with a residual: r holds the thread's 32 channels of the residual pixel (the four chunks its result replaces)
template <int CH>
__device__ __forceinline__ void activate_half_res(const uint32_t (&acc)[32], const PatchParams &p, int act_mode, const float *s_slope,
                                                  const uint4 (&r)[4], uint4 (&o)[4])
{
#pragma unroll
    for (int cj = 0; cj < 4; cj++) {
        const uint32_t rw[4] = {r[cj].x, r[cj].y, r[cj].z, r[cj].w};
        uint32_t ow[4];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const int c = CH * 32 + cj * 8 + h * 2;
            float2 rr;
            if (p.kind == 0) rr = __half22float2(*reinterpret_cast<const __half2 *>(&rw[h]));
            else rr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&rw[h]));
            float v0 = fmaf(p.res_coef, rr.x, fmaf(__uint_as_float(acc[cj * 8 + h * 2]), p.cscale[c], p.cshift[c]));
            float v1 = fmaf(p.res_coef, rr.y, fmaf(__uint_as_float(acc[cj * 8 + h * 2 + 1]), p.cscale[c + 1], p.cshift[c + 1]));
            if (act_mode == 3) {
                v0 = fmaxf(v0, 0.f);
                v1 = fmaxf(v1, 0.f);
            } else if (act_mode != 0) {
                v0 = thb_apply_act(v0, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c]);
                v1 = thb_apply_act(v1, p.act_kind, p.act_th, p.act_val, p.act_alpha, s_slope[c + 1]);
            }
            if (c >= p.Cout) v0 = 0.f;       // padded channels stay exact zeros
            if (c + 1 >= p.Cout) v1 = 0.f;
            ow[h] = pack_pair(v0, v1, p.kind);
        }
        o[cj] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// PX: bytes per input pixel in shared memory (32 or 128); KP: pooling window fused behind the convolution (0: none)
template <int PX, int KP>
__global__ void __launch_bounds__(PT_THREADS, 1)
conv_patch_tc_kernel(const __grid_constant__ CUtensorMap tmapW, const __grid_constant__ CUtensorMap tmapA,
                     const __grid_constant__ CUtensorMap tmapY, const __grid_constant__ CUtensorMap tmapR, const PatchParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem), *empty = full + PT_MAX_STAGES;
    uint64_t *acc_full = empty + PT_MAX_STAGES, *acc_empty = acc_full + PT_NACC, *w_full = acc_empty + PT_NACC;
    uint64_t *res_full = w_full + 1;                    // residual tile landed in output tile 0 / 1
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(res_full + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    // header of 2048 bytes: [0, 256) mbarriers, the TMEM slot and the abort flag; [512, 768) PReLU slopes
    static_assert((2 * PT_MAX_STAGES + 2 * PT_NACC + 1 + 2) * 8 + 8 <= 256, "the barriers outgrow their part of the header");
    float *s_slope = reinterpret_cast<float *>(smem + 512);
    uint8_t *sW = smem + 2048;                          // resident weights: tap t at sW + t * 64 * PX
    uint8_t *sP = sW + p.w_bytes;                       // raw patch buffers
    uint8_t *ct = sP + p.nst * p.stage_bytes;           // output tile(s): one with pooling, two without
    uint8_t *pt = ct + p.ct_bufs * PT_CT_BYTES;         // pooled tiles (pooling only)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int units = p.N * p.tiles_r * p.tiles_c;
    const int mine = (int)blockIdx.x < units ? (units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int taps = p.kH * p.kW;
    constexpr uint32_t TMEM_COLS = PT_NACC * 128;  // per unit two 64-column accumulators

    if (tid == 0) {
        for (int s = 0; s < p.nst; s++) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 2);            // one commit per MMA issuer
        }
        for (int b = 0; b < PT_NACC; b++) {
            mbar_init(smem_u32(&acc_full[b]), 2);          // one commit per MMA issuer
            mbar_init(smem_u32(&acc_empty[b]), 16);        // one arrival per epilogue warp
        }
        mbar_init(smem_u32(w_full), 1);
        mbar_init(smem_u32(&res_full[0]), 1);
        mbar_init(smem_u32(&res_full[1]), 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (tid < 64) {
        // per-channel epilogue constants (uploaded when the network was planned: no kernel of this stream writes them)
        const bool real = tid < p.Cout;
        s_slope[tid] = real && p.slope ? p.slope[tid] : 0.f;
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmapW);
        tma_prefetch_desc(&tmapA);
        tma_prefetch_desc(&tmapY);
        if (p.has_res) tma_prefetch_desc(&tmapR);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the weights do not depend on the kernel before this one: fetch them while it drains
    if (warp == 0 && lane == 0 && mine > 0) {
        mbar_arrive_expect_tx(smem_u32(w_full), (uint32_t)p.w_bytes);
        for (int t = 0; t < taps; t++) tma_load_2d(smem_u32(sW + t * 64 * PX), &tmapW, smem_u32(w_full), t * (PX / 2), 0);
    }
    if (p.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (warp == 0) {
        // ================================================================== TMA producer: one raw patch per unit
        if (lane == 0) {
            int ring_s = 0;
            uint32_t ring_ph = 0;
            const uint32_t box_bytes = (uint32_t)((p.CR + p.kH - 1) * p.P * PX);
            for (int u = 0; u < mine; u++) {
                const Unit q = unit_of(p, blockIdx.x + u * gridDim.x);
                const int s = ring_s;
                const uint32_t ph = ring_ph;
                if (++ring_s == p.nst) { ring_s = 0; ring_ph ^= 1; }
                if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1)) {
                    atomicExch(p.status, 3);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t bar = smem_u32(&full[s]);
                mbar_arrive_expect_tx(bar, box_bytes);
                tma_load_4d(smem_u32(sP + s * p.stage_bytes), &tmapA, bar, 0, q.c0 - p.padW + p.xoff, q.r0 - p.padH, q.n);
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 2) {
        // ================================================================== MMA issuers: warp 1 feeds the accumulator of GEMM
        // rows 0..127, warp 2 that of rows 128..255 (an instruction of N = 64 takes the tensor pipe 48 cycles, which
        // one issuing thread cannot sustain)
        if (lane == 0 && mine > 0) {
            constexpr uint32_t IDESC_F16 = make_idesc(1u, 0u, 64), IDESC_BF16 = make_idesc(1u, 1u, 64);
            const uint32_t idesc = p.kind == 1 ? IDESC_BF16 : IDESC_F16;
            constexpr int KSTEPS = PX / 32;      // tcgen05.mma of K = 16 elements per tap
            constexpr uint32_t HALF = 128u * PX / 16, BSTEP = 64u * PX / 16;   // descriptor steps: second accumulator's rows, next tap's weights
            constexpr uint32_t PXU = PX / 16;
            const int hsel = warp - 1, kW = p.kW;
            const uint32_t rowstep = (uint32_t)(p.P - p.kW + 1) * PXU;
            const uint64_t proto = make_rows_desc(0u, PX);
            const uint32_t hi = (uint32_t)(proto >> 32), lo_flags = (uint32_t)proto;
            const uint32_t b_lo0 = lo_flags | ((smem_u32(sW) >> 4) & 0x3FFFu);
            const int ntaps = taps;
            int ring_s = 0;
            uint32_t ring_ph = 0;
            bool alive = mbar_wait_bounded(smem_u32(w_full), 0);
            if (!alive) {
                atomicExch(p.status, 10);
                *abort_flag = 1;
            }
            for (int u = 0; u < mine && alive; u++) {
                const int ab = u % PT_NACC;
                if (!mbar_wait_bounded(smem_u32(&acc_empty[ab]), ((u / PT_NACC) & 1) ^ 1)) {
                    atomicExch(p.status, 6);
                    *abort_flag = 1;
                    break;
                }
                const int s = ring_s;
                const uint32_t ph = ring_ph;
                if (++ring_s == p.nst) { ring_s = 0; ring_ph ^= 1; }
                if (!mbar_wait_bounded(smem_u32(&full[s]), ph)) {
                    atomicExch(p.status, 4);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + ab * 128 + hsel * 64;
                const uint32_t a_lo0 = (lo_flags | ((smem_u32(sP + s * p.stage_bytes) >> 4) & 0x3FFFu)) + hsel * HALF;
                // tap (r, s) reads the patch from pixel row r*P + s on: one pixel (PXU address units) further per tap, and
                // P - kW + 1 pixels further at the end of a kernel row -- all in registers, the loop touches no memory
                uint32_t b_lo = b_lo0, a_lo = a_lo0;
                int sx = 1;
                mma_tap<KSTEPS>(d, a_lo, b_lo, hi, idesc, 0u);   // first tap: the accumulator starts from zero
#pragma unroll 4
                for (int t = 1; t < ntaps; t++) {
                    b_lo += BSTEP;
                    if (sx == kW) { sx = 1; a_lo += rowstep; } else { sx++; a_lo += PXU; }
                    mma_tap<KSTEPS>(d, a_lo, b_lo, hi, idesc, 1u);
                }
                tc_commit(smem_u32(&empty[s]));
                tc_commit(smem_u32(&acc_full[ab]));
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ================================================================== epilogue: activate, (pool,) store
        // 16 warps: a thread owns one GEMM row (TMEM lane) and 32 of its 64 output channels
        const int et = tid - 128;                // 0..511
        const int e = warp - 4;
        const int quad = warp & 3;               // TMEM lane quadrant this warp may read
        const int half = (e >> 2) & 1;           // accumulator half: GEMM rows 0..127 / 128..255
        const int ch = e >> 3;                   // channels 0..31 / 32..63
        const int m = half * 128 + quad * 32 + lane;
        const int cr = m / p.P, cc = m - cr * p.P;
        const bool valid = cr < p.CR && cc < p.CC;
        const int ci = cr * p.CC + cc;           // row of the output tile (valid rows only)
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + half * 64 + ch * 32;
        const int act_mode = p.act_kind == THB_ACT_NONE ? 0
                             : p.act_kind != THB_ACT_THRESHOLD ? 2
                             : (p.act_th == 0.f && p.act_val == 0.f) ? 3 : 1;
        const uint32_t neg_inf2 = p.kind == 0 ? 0xFC00FC00u : 0xFF80FF80u;
        const int kind = p.kind;
        // pooling: this thread's (pooled pixel, 16-byte channel chunk) item; its patch coordinates never change
        const int items = KP ? p.PR * p.PC * 8 : 0;
        const int it_px = et >> 3, it_j = et & 7;
        const int it_pr = KP ? it_px / p.PC : 0, it_pc = it_px - it_pr * p.PC;
        // Fused residual (no pooling, two output tiles): the residual tile of unit u is copied into the output tile the unit
        // will fill -- same box, same swizzle -- one unit ahead, so a thread finds its residual chunks where its result goes.
        const bool with_res = !KP && p.has_res;
        const uint32_t res_tile_bytes = (uint32_t)(p.CR * p.CC * 128);
        int res_issued = 0;
        if (with_res && et == 0 && mine > 0) {
            const Unit q0 = unit_of(p, blockIdx.x);
            mbar_arrive_expect_tx(smem_u32(&res_full[0]), res_tile_bytes);
            tma_load_4d(smem_u32(ct), &tmapR, smem_u32(&res_full[0]), 0, q0.c0, q0.r0, q0.n);
            res_issued = 1;
        }
        int u = 0;
        for (; u < mine; u++) {
            const int ab = u % PT_NACC;
            const Unit q = unit_of(p, blockIdx.x + u * gridDim.x);
            if (!mbar_wait_bounded(smem_u32(&acc_full[ab]), (u / PT_NACC) & 1)) {
                if (lane == 0) atomicExch(p.status, 2);
                *abort_flag = 1;
            }
            tc_fence_after();
            uint32_t acc[32];
            __syncwarp();
            tmem_ld32(lane_addr + ab * 128, acc);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[ab]));
            // the tile about to be written was the source of the store two units ago (of the last one with a single tile)
            if (et == 0 && !with_res) {   // (with a residual the wait came before the residual copy into this tile was issued)
                if (!KP && p.ct_bufs == 1) bulk_wait_group_read<0>();
                else bulk_wait_group_read<1>();
            }
            uint8_t *tile = KP || p.ct_bufs == 1 ? ct : ct + (u & 1) * PT_CT_BYTES;
            if (!KP) epi_bar_sync();
            if (with_res) {
                if (!mbar_wait_bounded(smem_u32(&res_full[u & 1]), (u >> 1) & 1)) {
                    if (lane == 0) atomicExch(p.status, 6);
                    *abort_flag = 1;
                }
            }
            if (valid) {
                uint4 o[4];
                uint8_t *row_smem = tile + ci * 128;
                const int rsw = ci & 7;
                if (with_res) {
                    uint4 r[4];
#pragma unroll
                    for (int cj = 0; cj < 4; cj++) r[cj] = *reinterpret_cast<const uint4 *>(row_smem + (((ch * 4 + cj) ^ rsw) << 4));
                    if (ch == 0) activate_half_res<0>(acc, p, act_mode, s_slope, r, o);
                    else activate_half_res<1>(acc, p, act_mode, s_slope, r, o);
                } else if (ch == 0) activate_half<0>(acc, p, act_mode, s_slope, o);
                else activate_half<1>(acc, p, act_mode, s_slope, o);
#pragma unroll
                for (int cj = 0; cj < 4; cj++) *reinterpret_cast<uint4 *>(row_smem + (((ch * 4 + cj) ^ rsw) << 4)) = o[cj];
            }
            if (!KP) {
                fence_proxy_async_smem();         // the rows must be visible to the copy engine
                epi_bar_sync();                   // the tile is complete
                if (*abort_flag) break;           // (read after the barrier: every thread sees the same value)
                if (et == 0) {
                    tma_store_4d(&tmapY, smem_u32(tile), 0, q.c0, q.r0, q.n);  // clips rows and columns beyond the map
                    bulk_commit_group();
                    if (with_res && u + 1 < mine) {
                        // the other tile was the source of the store of unit u - 1: once that has been read out, the
                        // residual of unit u + 1 may land there
                        bulk_wait_group_read<1>();
                        const Unit qn = unit_of(p, blockIdx.x + (u + 1) * gridDim.x);
                        const uint32_t bar = smem_u32(&res_full[(u + 1) & 1]);
                        mbar_arrive_expect_tx(bar, res_tile_bytes);
                        tma_load_4d(smem_u32(ct + ((u + 1) & 1) * PT_CT_BYTES), &tmapR, bar, 0, qn.c0, qn.r0, qn.n);
                        res_issued = u + 2;
                    }
                }
                continue;
            }
            epi_bar_sync();                       // the activated patch is complete
            if (*abort_flag) break;
            uint8_t *ptile = pt + (u & 1) * PT_PT_BYTES;
            if (et < items) {
                // window of this thread's pooled pixel, clipped to the convolution output
                const int gr0 = q.r0 + 2 * it_pr, gc0 = q.c0 + 2 * it_pc;
                uint32_t mx[4] = {neg_inf2, neg_inf2, neg_inf2, neg_inf2};
                const int m00 = 2 * it_pr * p.CC + 2 * it_pc;
#pragma unroll
                for (int dr = 0; dr < KP; dr++) {
                    const bool rok = (unsigned)(gr0 + dr) < (unsigned)p.oH;
#pragma unroll
                    for (int dc = 0; dc < KP; dc++) {
                        const int mm = m00 + dr * p.CC + dc;
                        const uint4 v = *reinterpret_cast<const uint4 *>(ct + mm * 128 + ((it_j ^ (mm & 7)) << 4));
                        if (rok && (unsigned)(gc0 + dc) < (unsigned)p.oW) {
                            mx[0] = max_pair(mx[0], v.x, kind);
                            mx[1] = max_pair(mx[1], v.y, kind);
                            mx[2] = max_pair(mx[2], v.z, kind);
                            mx[3] = max_pair(mx[3], v.w, kind);
                        }
                    }
                }
                *reinterpret_cast<uint4 *>(ptile + it_px * 128 + it_j * 16) = make_uint4(mx[0], mx[1], mx[2], mx[3]);
            }
            fence_proxy_async_smem();
            epi_bar_sync();                       // pooled tile complete; the patch tile may be overwritten
            if (et == 0) {
                tma_store_4d(&tmapY, smem_u32(ptile), 0, q.tc * p.PC, q.tr * p.PR, q.n);  // clips pooled pixels beyond the map
                bulk_commit_group();
            }
        }
        if (et == 0) bulk_wait_group<0>();
        // (after a give-up: a residual copy that nobody waited for must land before the CTA's shared memory goes away)
        if (with_res && et == 0 && u < mine && res_issued > u)
            for (int k = u; k < res_issued; k++) mbar_wait_bounded(smem_u32(&res_full[k & 1]), (k >> 1) & 1);
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
encode_tiled_fn pt_encode_fn()
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

struct Geometry {
    int CR, CC, P, tiles_r, tiles_c, PR, PC;
    int stage_bytes, nst, ct_bufs, w_bytes;
    size_t smem;
};

// shared-memory plan of a candidate patch: resident weights, raw patch buffers, output tile(s), pooled tiles
bool plan_smem(int kH, int kW, int px_bytes, int kp, bool two_tiles, Geometry *g)
{
    g->w_bytes = (kH * kW * 64 * px_bytes + 1023) & ~1023;
    // a patch buffer holds the copied pixels and whatever the 256 GEMM rows of the last tap reach beyond them
    const int box_px = (g->CR + kH - 1) * g->P, reach_px = (kH - 1) * g->P + kW - 1 + 256;
    g->stage_bytes = ((box_px > reach_px ? box_px : reach_px) * px_bytes + 1023) & ~1023;
    // without pooling the output tile is the source of an asynchronous store: two of them when room allows
    for (g->ct_bufs = kp ? 1 : 2; g->ct_bufs >= 1; g->ct_bufs--) {
        const size_t fixed = 1024 + 2048 + (size_t)g->w_bytes + (size_t)g->ct_bufs * PT_CT_BYTES + (kp ? 2 * PT_PT_BYTES : 0);
        if (fixed + 2 * (size_t)g->stage_bytes > PT_SMEM_MAX) continue;
        g->nst = (int)((PT_SMEM_MAX - fixed) / g->stage_bytes);
        if (g->nst > PT_MAX_STAGES) g->nst = PT_MAX_STAGES;
        if (two_tiles && g->ct_bufs != 2) return false; // (a fused residual is copied into the tile of the NEXT unit)
        if (!two_tiles && g->nst < 3 && g->ct_bufs == 2) continue;   // a third patch in flight is worth more than a second output tile
        g->smem = fixed + (size_t)g->nst * g->stage_bytes;
        return true;
    }
    return false;
}

// The patch that covers the map with the fewest units: CR output rows x CC output columns with CR * (CC + kW - 1) <= 256
// GEMM rows; with a pooling behind the convolution the patch is made of whole windows (CR = 2(PR-1)+kp, CC likewise).
bool choose_patch(int oH, int oW, int kH, int kW, int px_bytes, int kp, int pH, int pW, bool two_tiles, Geometry *best)
{
    long best_tiles = -1;
    for (int a = 1; a <= 64; a++) {
        Geometry g;
        memset(&g, 0, sizeof(g));
        g.CR = kp ? 2 * (a - 1) + kp : a;
        if (g.CR > 256) break;
        if (kp) {
            // largest PC with CR * (2(PC-1) + kp + kW - 1) <= 256, at most 64 pooled pixels per tile
            g.PR = a;
            g.PC = ((256 / g.CR) - (kW - 1) - kp) / 2 + 1;
            if (g.PC > pW) g.PC = pW;
            if (a * g.PC > 64) g.PC = 64 / a;
            if (g.PC < 1) continue;
            g.CC = 2 * (g.PC - 1) + kp;
        } else {
            g.CC = 256 / g.CR - (kW - 1);
            if (g.CC > oW) g.CC = oW;
            if (g.CC < 1) continue;
        }
        g.P = g.CC + kW - 1;
        if (g.P > 256 || g.CR + kH - 1 > 256 || g.CR * g.P > 256) continue;
        g.tiles_r = kp ? (pH + a - 1) / a : (oH + g.CR - 1) / g.CR;
        g.tiles_c = kp ? (pW + g.PC - 1) / g.PC : (oW + g.CC - 1) / g.CC;
        if (!plan_smem(kH, kW, px_bytes, kp, two_tiles, &g)) continue;
        const long tiles = (long)g.tiles_r * g.tiles_c;
        if (best_tiles < 0 || tiles < best_tiles || (tiles == best_tiles && g.nst > best->nst)) {
            best_tiles = tiles;
            *best = g;
        }
        if ((kp ? a >= pH : g.CR >= oH)) break;
    }
    return best_tiles > 0;
}

bool patch_geometry_ok(const thb_conv_desc *d, int pk, int ps, int ppad)
{
    if (d->dtype != THB_F16 && d->dtype != THB_BF16) return false;
    if (d->Cout > 64 || d->BN != 64 || d->dH != 1 || d->dW != 1 || d->x2) return false;
    // a fused residual: without pooling, coefficients of +-1 for the convolution's own term, rows of whole 16-byte chunks
    if (d->res && (pk || d->res_ld % 8 || ((uintptr_t)d->res & 15) || (d->self_coef != 1.f && d->self_coef != -1.f))) return false;
    if (d->Cin_pad != 16 && d->Cin_pad != 64) return false;
    if (d->in_ld < d->Cin_pad || d->in_ld % 8) return false;
    if (d->kH < 1 || d->kW < 1 || d->kH > 8 || d->kW > 8 || d->padH >= d->kH || d->padW >= d->kW) return false;
    if (d->Ktot_pad != (d->kH * d->kW * d->Cin_pad + 63) / 64 * 64) return false;
    if (d->in_row_pitch && d->in_pad_left != d->padW) return false;
    if (pk && ((pk != 2 && pk != 3) || ps != 2 || ppad < 0 || ppad >= pk)) return false;
    const size_t w_bytes = ((size_t)d->kH * d->kW * 64 * d->Cin_pad * 2 + 1023) & ~(size_t)1023;
    if (w_bytes > 98304) return false;
    return true;
}

// (the cache holds tensor maps only, i.e. addresses and shapes: nothing in it can go stale when memory is reused)
struct PtMapEntry {
    const void *x, *y, *wptr, *res;
    int key[20];
    alignas(64) CUtensorMap w, a, y_map, r_map;
};

int patch_launch(const thb_conv_desc *d, int pk, int ppad, int pH, int pW, const void *x, void *y, int y_ld, thb_stream s)
{
    encode_tiled_fn enc = pt_encode_fn();
    if (!enc) return thb_note_launch(cudaErrorUnknown, "cuTensorMapEncodeTiled entry point");
    PatchParams p;
    memset(&p, 0, sizeof(p));
    Geometry g;
    if (!choose_patch(d->oH, d->oW, d->kH, d->kW, d->Cin_pad * 2, pk, pH, pW, d->res != nullptr, &g)) return THB_ERR_UNSUPPORTED;
    p.N = d->N; p.oH = d->oH; p.oW = d->oW;
    p.CR = g.CR; p.CC = g.CC; p.P = g.P; p.tiles_r = g.tiles_r; p.tiles_c = g.tiles_c; p.PR = g.PR; p.PC = g.PC;
    p.kH = d->kH; p.kW = d->kW; p.padH = d->padH; p.padW = d->padW;
    p.px_bytes = d->Cin_pad * 2;
    p.xoff = d->in_row_pitch ? d->in_pad_left : 0;
    p.kp = pk; p.pp = ppad;
    p.Cout = d->Cout;
    p.slope = d->act.kind == THB_ACT_PRELU ? d->act.slope : nullptr;
    p.act_kind = d->act.kind; p.act_th = d->act.threshold; p.act_val = d->act.value; p.act_alpha = d->act.alpha;
    p.kind = d->dtype == THB_BF16 ? 1 : 0;
    p.status = d->status;
    p.w_bytes = g.w_bytes; p.stage_bytes = g.stage_bytes; p.nst = g.nst; p.ct_bufs = g.ct_bufs;
    const size_t smem = g.smem;

    // tensor maps of the weights (one tap per box), the input (patch box) and the output (tile box), cached by buffer and shape
    static PtMapEntry cache[128];
    static int used = 0, next = 0;
    const int key[20] = {d->dtype, d->N, d->H, d->W, d->Cin_pad, d->in_ld, d->in_row_pitch, d->oH, d->oW, pH, pW, y_ld, d->Cout,
                         p.CR, p.CC, p.PR, p.PC, d->kH * 16 + d->kW, d->res ? d->res_ld : 0, d->Ktot_pad};
    PtMapEntry *e = nullptr;
    for (int i = 0; i < used; i++)
        if (cache[i].x == x && cache[i].y == y && cache[i].wptr == d->w && cache[i].res == d->res && !memcmp(cache[i].key, key, sizeof(key))) { e = &cache[i]; break; }
    if (!e) {
        e = &cache[used < 128 ? used++ : (next++ % 128)];
        e->x = nullptr;
        const CUtensorMapDataType t = d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        const CUtensorMapSwizzle sw = p.px_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B;
        cuuint32_t estr[4] = {1, 1, 1, 1};
        {
            cuuint64_t dims[2] = {(cuuint64_t)d->Ktot_pad, (cuuint64_t)d->Cout_pad};
            cuuint64_t strides[1] = {(cuuint64_t)d->Ktot_pad * 2};
            cuuint32_t box[2] = {(cuuint32_t)d->Cin_pad, 64};
            if (enc(&e->w, t, 2, const_cast<void *>(d->w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return thb_note_launch(cudaErrorInvalidValue, "conv_patch: weight tensor map");
        }
        {
            const int Wst = d->in_row_pitch ? d->in_row_pitch : d->W;   // stored pixels per row
            cuuint64_t dims[4] = {(cuuint64_t)d->Cin_pad, (cuuint64_t)Wst, (cuuint64_t)d->H, (cuuint64_t)d->N};
            cuuint64_t strides[3] = {(cuuint64_t)d->in_ld * 2, (cuuint64_t)Wst * d->in_ld * 2, (cuuint64_t)d->H * Wst * d->in_ld * 2};
            cuuint32_t box[4] = {(cuuint32_t)d->Cin_pad, (cuuint32_t)p.P, (cuuint32_t)(p.CR + p.kH - 1), 1};
            if (enc(&e->a, t, 4, const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return thb_note_launch(cudaErrorInvalidValue, "conv_patch: input tensor map");
        }
        {
            const int c8 = (d->Cout + 7) & ~7;
            const int yH = pk ? pH : d->oH, yW = pk ? pW : d->oW;
            cuuint64_t dims[4] = {(cuuint64_t)c8, (cuuint64_t)yW, (cuuint64_t)yH, (cuuint64_t)d->N};
            cuuint64_t strides[3] = {(cuuint64_t)y_ld * 2, (cuuint64_t)yW * y_ld * 2, (cuuint64_t)yH * yW * y_ld * 2};
            cuuint32_t box[4] = {64, (cuuint32_t)(pk ? p.PC : p.CC), (cuuint32_t)(pk ? p.PR : p.CR), 1};
            // the pooled tile is written as plain rows; the convolution tile carries the 128-byte XOR pattern
            if (enc(&e->y_map, t, 4, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    pk ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return thb_note_launch(cudaErrorInvalidValue, "conv_patch: output tensor map");
        }
        if (d->res) {
            // the residual: the output's shape and box with its own pitch
            const int c8 = (d->Cout + 7) & ~7;
            cuuint64_t dims[4] = {(cuuint64_t)c8, (cuuint64_t)d->oW, (cuuint64_t)d->oH, (cuuint64_t)d->N};
            cuuint64_t strides[3] = {(cuuint64_t)d->res_ld * 2, (cuuint64_t)d->oW * d->res_ld * 2, (cuuint64_t)d->oH * d->oW * d->res_ld * 2};
            cuuint32_t box[4] = {64, (cuuint32_t)p.CC, (cuuint32_t)p.CR, 1};
            if (enc(&e->r_map, t, 4, const_cast<void *>(d->res), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return thb_note_launch(cudaErrorInvalidValue, "conv_patch: residual tensor map");
        }
        e->x = x; e->y = y; e->wptr = d->w; e->res = d->res;
        memcpy(e->key, key, sizeof(key));
    }

    // The per-channel constants travel as kernel parameters: from the descriptor's host copies when it has them, else
    // read back from the device (a blocking copy at every launch: callers that capture streams give the host copies).
    for (int c = 0; c < 64; c++) { p.cscale[c] = c < d->Cout ? 1.f : 0.f; p.cshift[c] = 0.f; }
    if (d->scale) {
        if (d->scale_host) memcpy(p.cscale, d->scale_host, sizeof(float) * d->Cout);
        else if (cudaMemcpy(p.cscale, d->scale, sizeof(float) * d->Cout, cudaMemcpyDeviceToHost) != cudaSuccess)
            return thb_note_launch(cudaGetLastError(), "conv_patch: reading the scale constants");
    }
    if (d->shift) {
        if (d->shift_host) memcpy(p.cshift, d->shift_host, sizeof(float) * d->Cout);
        else if (cudaMemcpy(p.cshift, d->shift, sizeof(float) * d->Cout, cudaMemcpyDeviceToHost) != cudaSuccess)
            return thb_note_launch(cudaGetLastError(), "conv_patch: reading the shift constants");
    }
    p.has_res = d->res != nullptr;
    p.res_coef = d->res_coef;
    if (p.has_res) {
        if (p.ct_bufs != 2) return THB_ERR_UNSUPPORTED;   // (the residual copy runs one unit ahead: it needs the second tile)
        if (d->self_coef != 1.f)                          // the convolution's own +-1 goes into its constants (exact)
            for (int c = 0; c < 64; c++) { p.cscale[c] *= d->self_coef; p.cshift[c] *= d->self_coef; }
    }
    static bool configured[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    typedef void (*kern_t)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const PatchParams);
    static const kern_t kerns[6] = {conv_patch_tc_kernel<32, 0>,  conv_patch_tc_kernel<32, 2>,  conv_patch_tc_kernel<32, 3>,
                                    conv_patch_tc_kernel<128, 0>, conv_patch_tc_kernel<128, 2>, conv_patch_tc_kernel<128, 3>};
    if (!configured[dev]) {
        for (int i = 0; i < 6; i++) {
            cudaError_t ce = cudaFuncSetAttribute(kerns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PT_SMEM_MAX);
            if (ce != cudaSuccess) return thb_note_launch(ce, "conv_patch smem attribute");
        }
        configured[dev] = true;
    }
    const kern_t kern = kerns[(p.px_bytes == 128 ? 3 : 0) + (pk == 0 ? 0 : pk == 2 ? 1 : 2)];
    static int sms[16] = {0};
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    const int units = p.N * p.tiles_r * p.tiles_c;
    const int nsm = sms[dev] > 0 ? sms[dev] : 148;
    const int grid = units < nsm ? units : nsm;
    static int use_pdl = -1;
    if (use_pdl < 0) {
        const char *ev = getenv("THB200_PDL");
        use_pdl = ev ? atoi(ev) : 1;
    }
    p.pdl = use_pdl;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(PT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, e->w, e->a, e->y_map, p.has_res ? e->r_map : e->y_map, p);
    return thb_note_launch(le != cudaSuccess ? le : cudaGetLastError(), "conv_patch_tc_kernel");
}

bool patch_disabled()
{
    static int disabled = -1;
    if (disabled < 0) {
        const char *e = getenv("THB200_NO_PATCH");
        disabled = e && atoi(e) ? 1 : 0;
    }
    return disabled != 0;
}

}  // namespace

// 1 when the patch kernel can run this convolution (plain store of its output)
extern "C" int thb_conv_patch_supported(const thb_conv_desc *d)
{
    Geometry g;
    return !patch_disabled() && patch_geometry_ok(d, 0, 0, 0) &&
           choose_patch(d->oH, d->oW, d->kH, d->kW, d->Cin_pad * 2, 0, 0, 0, d->res != nullptr, &g) ? 1 : 0;
}

extern "C" int thb_conv_patch_fwd(const thb_conv_desc *d, const void *x, void *y, thb_stream s)
{
    if (!d || !x || !y || !d->w || !d->status) return THB_ERR_ARG;
    if (!patch_geometry_ok(d, 0, 0, 0)) return THB_ERR_UNSUPPORTED;
    if (d->out_ld % 8) return THB_ERR_ARG;
    return patch_launch(d, 0, 0, 0, 0, x, y, d->out_ld, s);
}

// 1 when thb_conv_maxpool_fwd can run this convolution followed by a pk x pk max pooling of stride ps and padding ppad
extern "C" int thb_conv_maxpool_supported(const thb_conv_desc *d, int pk, int ps, int ppad)
{
    static int disabled = -1;
    if (disabled < 0) {
        const char *e = getenv("THB200_NO_CONV_POOL");
        disabled = e && atoi(e) ? 1 : 0;
    }
    Geometry g;
    return !disabled && !patch_disabled() && pk > 0 && patch_geometry_ok(d, pk, ps, ppad) &&
           choose_patch(d->oH, d->oW, d->kH, d->kW, d->Cin_pad * 2, pk, d->oH / 2 + 1, d->oW / 2 + 1, false, &g) ? 1 : 0;
}

extern "C" int thb_conv_maxpool_fwd(const thb_conv_desc *d, int pk, int ps, int ppad, int pH, int pW, const void *x, void *y,
                                    int y_ld, thb_stream s)
{
    if (!d || !x || !y || !d->w || !d->status) return THB_ERR_ARG;
    if (pk < 1 || !patch_geometry_ok(d, pk, ps, ppad)) return THB_ERR_UNSUPPORTED;
    if (pH < 1 || pW < 1 || y_ld % 8) return THB_ERR_ARG;
    // every pooling window must start inside the convolution output (SpatialMaxPooling.c:196-210 guarantees it)
    if (2 * (pH - 1) - ppad >= d->oH || 2 * (pW - 1) - ppad >= d->oW) return THB_ERR_ARG;
    return patch_launch(d, pk, ppad, pH, pW, x, y, y_ld, s);
}
