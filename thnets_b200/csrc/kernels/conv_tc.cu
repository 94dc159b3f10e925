// Implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// GEMM view: D[pixel][cout] = sum_k A[pixel][k] * Wt[cout][k], k = tap*Cin_pad + c.
// One PERSISTENT CTA per SM walks output tiles of 128 consecutive pixels (flat over n, oh, ow: tiles
// may span rows and images, so small feature maps waste nothing) x BN output channels.  Fifteen warps:
//   warp  4    TMA producer: packed weights (K-major, SWIZZLE_128B, no multicast) and -- whenever a K block is
//              one whole 128-byte channel slab of one tap -- the activation operand too: a plain 2-D load for
//              1x1 stride-1 convolutions, an im2col-mode load (the copy engine walks the 128 output pixels,
//              applies stride, tap offset and zero padding) for everything else;
//   warps 0-3  otherwise (few input channels, e.g. a first layer) gather 16-byte channel chunks of the NHWC
//              activation into the swizzled stage layout with zero-filling cp.async; in the TMA modes they
//              are a third epilogue group;
//   warp  5    MMA issuer: one elected thread issues tcgen05.mma (kind::f16: fp16/bf16 -> fp32,
//              kind::i8: u8 x u8 -> int32) into one of 2-4 TMEM accumulators, recycles stages through
//              tcgen05.commit -> mbarrier, and hands finished accumulators to the epilogue.  With narrow
//              tiles it works on two pixel tiles at once (pair mode), which share every weight tile and
//              every barrier round;
//   warps 6-13 two epilogue groups; a thread owns one pixel row (TMEM lane): it reads 64 accumulator
//              columns with tcgen05.ld, applies bias/BN scale-shift, residual and activation, and leaves the
//              fp16/bf16 row in a swizzled shared-memory tile.  It never waits on global memory or on the
//              other threads of its group.  The uint8 path (exact lowp requantisation) and BN = 32 stage
//              through shared memory and write out with plain stores;
//   warp 14    epilogue agents, one thread per group: TMA load of the fused residual tile into the group's
//              shared-memory tile, TMA store of the finished tile, recycling of the tile.
// No im2col buffer exists anywhere.  Every wait is bounded: a wait that runs out records a code in
// *status and the CTA drains and exits.
#include "common.cuh"
#include <cuda.h>
#include <string.h>
#include <stdio.h>
#include <stdlib.h>

namespace {

constexpr int BM = 128;                  // pixels per tile (= TMEM lanes)
constexpr int A_STAGE_BYTES = BM * 128;  // 128 rows of one 128-byte K block
constexpr int NTHREADS = 480;           // 4 producer/epilogue + 1 TMA + 1 MMA + 2 x 4 epilogue warps + 1 warp of agents
constexpr int EPI_TILE_BYTES = BM * 128;  // one 128-row x 64-column fp16 tile of the TMA epilogue

struct ConvTcParams {
    const uint8_t *x;
    uint8_t *y;
    const int *kinfo;
    int P, H, W, in_ld, oH, oW, oHW, dH, dW, padH, padW, kH, kW, Cin, Cout, out_ld, nkb, n_kchunks;
    int m_tiles, n_tiles;
    const float *scale, *shift, *slope;
    const uint8_t *res;
    int res_ld;
    float self_coef, res_coef;
    int act_kind;
    float act_th, act_val, act_alpha;
    int a_off, b_off, c_off, c_mult, c_shift;
    const int *wsat, *bias_add, *csum;
    int tail_start, relu_thr, relu_val;
    int a_tma;   // 1: 1x1 stride-1 convolution, the activation operand is a plain [pixels][Cin] matrix loaded by 2-D TMA;
                 // 2: whole 128-byte channel slabs per tap, loaded by im2col-mode TMA (any kernel size, stride, padding)
    int pdl;                   // launched with programmatic stream serialisation
    int pair;                  // TMA modes, BN <= 128: the CTA works on two vertically adjacent 128-pixel tiles at once.  Every
                               // pipeline stage carries both activation tiles and ONE weight tile, and the MMA thread feeds two
                               // accumulators per barrier round: that round costs the thread ~250 cycles whatever it carries,
                               // which a single narrow tile (192-256 tensor cycles per K block) cannot hide.
    int *csum_out;             // uint8, one column tile: per output pixel the sum of its output bytes (the next layer's channel sums)
    int res_addend;            // uint8 fused residual: the constant of ca*q + cb*r + addend (see thb_u8_combine)
    int u8_classes;            // uint8: > 0 when the border classes of the kernel window ((1 + 2 padH) x (1 + 2 padW) of them)
                               // fit the epilogue's shared-memory table; 0: every row looks its window up in global memory
    int reverse;               // TMA modes with the TMA epilogue: pixel tiles are walked from the tensor's end, so that a layer
                               // starts on what the layer before it wrote last and the L2 still holds
    int stages;                // TMA epilogue: pipeline stages (the launcher sizes them against the epilogue tiles)
    int epi_groups, epi_bufs;  // TMA epilogue: groups at work (2 or 3) and 16 KB tiles each of them cycles through
    int row_pitch, pad_left;  // gather: pixels between input rows, zero pixels in front of each row (W, 0 when plain)
    int tma_kw, tma_padw;     // a_tma == 2: taps per kernel row that need a load of their own, and the padding the
                              // descriptor's coordinates see (1, 0 when one copy fetches a padded row's kW taps)
    int slabs;   // a_tma == 2: 128-byte channel slabs per tap (K block kb = tap * slabs + slab)
    int nkb1, a2_mode, a2_d;  // second activation operand (a_tma == 1 only): K blocks nkb1.. come from it, through the fourth
                              // tensor map (no residual then); a2_mode 1: plain matrix, 2: 1x1 im2col sampling with stride a2_d
    int half, ntaps;  // a_tma == 2, half: a tap is 64 bytes of channels; a K block holds two taps as two tiles of 64-byte rows
                      // (SWIZZLE_64B), each loaded by its own activation and weight copy and fed to two MMAs of K = 32 bytes
    int use_l1;  // gather through L1: neighbouring taps of one tile re-read the same input pixels
    int *acc_out;
    int *status;
    int splits;                // > 1: the K blocks of every tile are shared by this many CTAs (units of work = tiles x splits, the
                               // split index innermost); each stores its raw fp32 partial tile to `partial` and
                               // splitk_finish_kernel adds them up in split order and runs the epilogue
    float *partial;            // [splits][P][partial_ld] fp32
    int partial_ld;
    long long wait_limit;      // SM cycles a bounded wait may take before it gives up (about two seconds by default)
    int test_withhold;         // tests only: the producer never delivers the last K block of the CTA's last tile
};

template <int KIND> struct kind_traits;  // 0 = fp16, 1 = bf16, 2 = u8
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

// One 16-byte output chunk (8 channels of one pixel) of the floating-point epilogue:
//   y = act( self * (acc*scale + shift) + res_coef * residual ), channels >= Cout forced to 0.
// ACT: 0 none, 1 threshold, 2 anything (leaky / PReLU), 3 plain ReLU (threshold 0, value 0).
template <int KIND, bool HAS_RES, int ACT, bool CHECK>
__device__ __forceinline__ uint4 epi_chunk(const float4 &a0, const float4 &a1, const float (&sc)[8], const float (&sh)[8],
                                           const float (&sl)[8], const uint4 &rv, const ConvTcParams &p, int c0)
{
    const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
#pragma unroll
    for (int h = 0; h < 4; h++) {
        float v0 = fmaf(av[h * 2], sc[h * 2], sh[h * 2]);
        float v1 = fmaf(av[h * 2 + 1], sc[h * 2 + 1], sh[h * 2 + 1]);
        if (HAS_RES) {
            // self_coef is +-1 in every fused CAddTable/CSubTable; the launcher folds it into scale and shift
            // (exact), so only the residual's own coefficient is left here
            const float2 rr = unpack2(rw[h], KIND);
            v0 = fmaf(p.res_coef, rr.x, v0);
            v1 = fmaf(p.res_coef, rr.y, v1);
        }
        if (ACT == 3) {  // x > 0 ? x : 0
            v0 = fmaxf(v0, 0.f);
            v1 = fmaxf(v1, 0.f);
        } else if (ACT == 1) {
            v0 = v0 > p.act_th ? v0 : p.act_val;
            v1 = v1 > p.act_th ? v1 : p.act_val;
        } else if (ACT == 2) {
            v0 = thb_apply_act(v0, p.act_kind, p.act_th, p.act_val, p.act_alpha, sl[h * 2]);
            v1 = thb_apply_act(v1, p.act_kind, p.act_th, p.act_val, p.act_alpha, sl[h * 2 + 1]);
        }
        if (CHECK) {
            if (c0 + h * 2 >= p.Cout) v0 = 0.f;
            if (c0 + h * 2 + 1 >= p.Cout) v1 = 0.f;
        }
        ow[h] = pack2(v0, v1, KIND);
    }
    return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// One pixel row of a 64-channel block of the TMA epilogue: the thread's 64 accumulator columns -> eight 16-byte chunks
// of its row of the swizzled shared-memory tile, which holds the residual row on entry when HAS_RES.  One variant is
// chosen per block, so that only the code of that variant is fetched.
template <int KIND, bool HAS_RES, int ACT, bool CHECK>
__device__ __forceinline__ void epi_block(const uint32_t (&acc0)[32], const uint32_t (&acc1)[32], uint8_t *row_smem, int rsw,
                                          int nsub0, const ConvTcParams &p)
{
    const float *scale = p.scale, *shift = p.shift, *slope = ACT == 2 ? p.slope : nullptr;
    const int cout = p.Cout;
    const float self = HAS_RES ? p.self_coef : 1.f;
#pragma unroll
    for (int cj = 0; cj < 8; cj++) {
        const int c0 = nsub0 + cj * 8;
        uint4 *slot = reinterpret_cast<uint4 *>(row_smem + ((cj ^ rsw) << 4));
        uint4 o = make_uint4(0, 0, 0, 0);
        if (!CHECK || c0 < cout) {
            float sc[8], sh[8], sl[8];
            const float4 one = make_float4(self, self, self, self), zero = make_float4(0.f, 0.f, 0.f, 0.f);
            float4 t0 = one, t1 = one;
            if (scale) {
                t0 = __ldg(reinterpret_cast<const float4 *>(scale + c0));
                t1 = __ldg(reinterpret_cast<const float4 *>(scale + c0 + 4));
                if (HAS_RES) { t0.x *= self; t0.y *= self; t0.z *= self; t0.w *= self; t1.x *= self; t1.y *= self; t1.z *= self; t1.w *= self; }
            }
            sc[0] = t0.x; sc[1] = t0.y; sc[2] = t0.z; sc[3] = t0.w; sc[4] = t1.x; sc[5] = t1.y; sc[6] = t1.z; sc[7] = t1.w;
            t0 = zero; t1 = zero;
            if (shift) {
                t0 = __ldg(reinterpret_cast<const float4 *>(shift + c0));
                t1 = __ldg(reinterpret_cast<const float4 *>(shift + c0 + 4));
                if (HAS_RES) { t0.x *= self; t0.y *= self; t0.z *= self; t0.w *= self; t1.x *= self; t1.y *= self; t1.z *= self; t1.w *= self; }
            }
            sh[0] = t0.x; sh[1] = t0.y; sh[2] = t0.z; sh[3] = t0.w; sh[4] = t1.x; sh[5] = t1.y; sh[6] = t1.z; sh[7] = t1.w;
            t0 = zero; t1 = zero;
            if (ACT == 2 && slope) {
                t0 = __ldg(reinterpret_cast<const float4 *>(slope + c0));
                t1 = __ldg(reinterpret_cast<const float4 *>(slope + c0 + 4));
            }
            sl[0] = t0.x; sl[1] = t0.y; sl[2] = t0.z; sl[3] = t0.w; sl[4] = t1.x; sl[5] = t1.y; sl[6] = t1.z; sl[7] = t1.w;
            const uint32_t *a = cj < 4 ? acc0 + cj * 8 : acc1 + (cj - 4) * 8;
            const float4 a0 = make_float4(__uint_as_float(a[0]), __uint_as_float(a[1]), __uint_as_float(a[2]), __uint_as_float(a[3]));
            const float4 a1 = make_float4(__uint_as_float(a[4]), __uint_as_float(a[5]), __uint_as_float(a[6]), __uint_as_float(a[7]));
            const uint4 rv = HAS_RES ? *slot : make_uint4(0, 0, 0, 0);
            o = epi_chunk<KIND, HAS_RES, ACT, CHECK>(a0, a1, sc, sh, sl, rv, p, c0);
        }
        *slot = o;
    }
}

// shared-memory plan of one CTA
template <int KIND, int BN, int STAGES> struct Smem {
    static constexpr bool TMA_EPI = KIND != 2 && BN >= 64;                        // epilogue through TMA loads/stores
    static constexpr int SUBN = BN >= 256 ? 32 : (BN >= 64 ? 64 : BN);           // staged epilogue: columns at a time
    static constexpr int B_STAGE_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr size_t STAGING = KIND == 2 ? (size_t)BM * (SUBN + 16) : (size_t)BM * (SUBN + 4) * 4;
    static constexpr size_t STAGING_PAD = (STAGING + 127) / 128 * 128;  // one staging tile per epilogue group
    static constexpr size_t BAR_BYTES = 1024;                           // mbarriers and the TMEM slot, ahead of the tiles
    // The TMA epilogue takes the whole 227 KB: the launcher splits what the barriers leave between pipeline stages
    // (at least STAGES of them) and 16 KB epilogue tiles.  The staged epilogue has STAGES stages and two staging tiles.
    static constexpr size_t AVAIL = 232448 - 1024 - BAR_BYTES;
    // uint8: per epilogue group a table of zero-point correction terms per (border class, channel) and the bias addends
    static constexpr int TBL_ROW = BN + 4;                                 // ints between the rows of two classes
    static constexpr int TBL_CAP = 3400;                                   // ints the class table may take
    // (after the class rows: 256 bias addends as ints, then the same addends as 128 words of two 16-bit halves)
    static constexpr size_t TBL_BYTES = KIND == 2 ? (size_t)(TBL_CAP + 256 + 128) * 4 + 64 : 0;
    static constexpr size_t TOTAL =
        TMA_EPI ? 232448 : 1024 + BAR_BYTES + (size_t)STAGES * STAGE_BYTES + 3 * STAGING_PAD + 3 * TBL_BYTES;
    static_assert(TOTAL <= 232448, "shared memory plan exceeds the 227 KB a CTA can have");
};
constexpr int MAX_STAGES = 12;

// position of an epilogue group in its sequence of 64-column blocks
struct EpiCursor {
    int j, sb;  // j-th tile of this group, block sb of that tile
};

// The CTA's own sequence of 128-pixel tiles ("local tiles" 0, 1, 2, ...).  Plain mode: global tile blockIdx.x +
// lt*gridDim.x of the (pixel tile, column tile) grid.  Pair mode: the CTA takes UNITS of two vertically adjacent pixel
// tiles with the same column tile; local tiles 2i and 2i+1 are the halves of its i-th unit.  A second half beyond
// the last pixel tile (odd tile count) is a phantom: it is computed from zero-filled loads and never stored.
template <int BN, bool SPLIT = false> struct TileMap {
    int pair, n_tiles, n_local, last_um, splits, nkb;
    __device__ TileMap(const ConvTcParams &p)
    {
        pair = p.pair;
        n_tiles = p.n_tiles;
        splits = SPLIT && p.splits > 1 ? p.splits : 1;   // (never with pair mode or a reversed walk)
        nkb = p.nkb;
        last_um = p.reverse ? (pair ? (p.m_tiles + 1) >> 1 : p.m_tiles) - 1 : -1;
        const int units = (pair ? (p.m_tiles + 1) >> 1 : p.m_tiles) * n_tiles * splits;
        const int mine = (int)blockIdx.x < units ? (units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        n_local = pair ? 2 * mine : mine;
    }
    // split index of local tile lt, and the K blocks [kb0, kb1) it covers
    __device__ int split_of(int lt) const { return SPLIT && splits > 1 ? (int)((blockIdx.x + lt * gridDim.x) % splits) : 0; }
    __device__ void kblocks(int lt, int &kb0, int &kb1) const
    {
        const int sp = split_of(lt);
        kb0 = (int)((long)nkb * sp / splits);
        kb1 = (int)((long)nkb * (sp + 1) / splits);
    }
    __device__ void coords(int lt, int &m0, int &n0) const
    {
        int u = blockIdx.x + (pair ? lt >> 1 : lt) * gridDim.x;
        if (SPLIT && splits > 1) u /= splits;
        int um = u / n_tiles;
        n0 = (u - um * n_tiles) * BN;
        if (last_um >= 0) um = last_um - um;  // walk the pixel tiles from the end of the tensor
        m0 = (pair ? 2 * um + (lt & 1) : um) * BM;
    }
};

// The sequence of 64-channel blocks an epilogue group walks: every ngrp-th local tile of this CTA, and of each tile
// the blocks that hold real channels.
template <int BN, bool SPLIT = false> struct EpiWalk {
    TileMap<BN, SPLIT> map;
    int grp, ngrp, my_tiles, cout8;
    __device__ EpiWalk(const ConvTcParams &p, int g) : map(p)
    {
        grp = g;
        ngrp = p.epi_groups;
        my_tiles = map.n_local > grp ? (map.n_local - 1 - grp) / ngrp + 1 : 0;
        cout8 = (p.Cout + 7) & ~7;
    }
    __device__ int local(int j) const { return grp + j * ngrp; }
    __device__ int blocks_of(int j) const
    {
        int m0, n0;
        map.coords(local(j), m0, n0);
        return min(BN / 64, (cout8 - n0 + 63) >> 6);
    }
    __device__ void advance(EpiCursor &c) const
    {
        if (++c.sb == blocks_of(c.j)) { c.sb = 0; c.j++; }
    }
};

// uint8 epilogue arithmetic of one pixel row over 32 accumulator columns (the table-driven path).  Per column: zero-point
// correction (table word of the row's border class + the row's own term, with c_offset folded in), gemmlowp
// requantisation ((x * c_mult + round) >> c_shift, saturated), the reference's saturating bias add, an optional fused
// residual ca*q + cb*r + addend (saturated) and the Threshold.  GENERAL = false assumes what almost every warp sees: no
// row in the image plane's tail (where the reference's bias add wraps instead of clamping at 0) and a Threshold whose
// replacement byte equals its threshold (max suffices); the integer pipe is what bounds this loop.
struct U8Epi {
    uint32_t rc;     // (corr_pix + c_offset) * c_mult + rounding term of this row, modulo 2^32
    uint32_t mult;
    int shift, tailmask, thr, rval, ca, cb, addend;
};
template <bool GENERAL, bool HAS_RES>
__device__ __forceinline__ void u8_chunk32(const uint32_t (&acc)[32], const int *trow, const int *brow, const U8Epi &e,
                                           const uint4 &res0, const uint4 &res1, uint32_t (&words)[8])
{
    const uint32_t rw[8] = {res0.x, res0.y, res0.z, res0.w, res1.x, res1.y, res1.z, res1.w};
#pragma unroll
    for (int g4 = 0; g4 < 8; g4++) {
        const int4 t4 = *reinterpret_cast<const int4 *>(trow + g4 * 4);
        const int4 b4 = *reinterpret_cast<const int4 *>(brow + g4 * 4);
        const int tv[4] = {t4.x, t4.y, t4.z, t4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
        int q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // (acc + t + corr) * mult + rnd in the ring of 32-bit words, with t * mult taken from the table
            const int sres = (int)(acc[g4 * 4 + i] * e.mult + (uint32_t)tv[i] + e.rc) >> e.shift;
            const int q1 = __vimin_s32_relu(sres, 255);
            int v;
            if (GENERAL) {
                const int t2 = q1 + bv[i];
                v = max(__vimin_s32_relu(t2, 255), t2 & e.tailmask);
            } else {
                v = __viaddmin_s32_relu(q1, bv[i], 255);
            }
            if (HAS_RES) {
                const int r = (int)((rw[g4] >> (8 * i)) & 255u);
                v = __vimin_s32_relu(e.ca * v + e.cb * r + e.addend, 255);
            }
            if (GENERAL) v = v > e.thr ? v : e.rval;
            else v = max(v, e.rval);
            q[i] = v;
        }
        const uint32_t lo = __byte_perm((uint32_t)q[0], (uint32_t)q[1], 0x0040), hi = __byte_perm((uint32_t)q[2], (uint32_t)q[3], 0x0040);
        words[g4] = __byte_perm(lo, hi, 0x5410);
    }
}

// The common case of u8_chunk32 (GENERAL = false) with the arithmetic after the shift done on two 16-bit halves per
// instruction.  What bounds this loop is the integer pipes: shifts, byte permutes, packing conversions and multiply-adds
// issue every second cycle per scheduler, minimum / maximum (also on halfword pairs) and plain adds every cycle; so the
// clamps are minima and maxima on pairs and every add is a plain 32-bit add of words whose halves cannot carry.
// That needs non-negative halves, hence an offset: the bias words hold addend + OFF (addends clamped to +-255, which
// saturates the same way), OFF = 256 without a residual and 384 with one, and
//   pair = min(pack_u16(shifted values), 255)                 in [0, 255]
//   S1   = clamp(pair + bias word, OFF (+ threshold byte when there is no residual), OFF + 255)
//   S2   = clamp(S1 + R, 512 + threshold byte, 512 + 255)     R = 255 - r for q - r + 127 (RES 1), r for q + r - 128 (RES 3)
// and the low bytes of the halves (offsets 256 and 512 leave them alone) are the result.
template <int RES>
__device__ __forceinline__ void u8_chunk32_pairs(const uint32_t (&acc)[32], const int *trow, const int *b2, const U8Epi &e,
                                                 const uint4 &res0, const uint4 &res1, uint32_t (&words)[8])
{
    const uint32_t rw[8] = {res0.x, res0.y, res0.z, res0.w, res1.x, res1.y, res1.z, res1.w};
    constexpr uint32_t OFF = RES ? 384u : 256u;
    const uint32_t rv2 = (uint32_t)e.rval * 0x00010001u;
    const uint32_t lo1 = OFF * 0x00010001u + (RES ? 0u : rv2), hi1 = (OFF + 255u) * 0x00010001u;
    const uint32_t lo2 = 512u * 0x00010001u + rv2, hi2 = 767u * 0x00010001u;
#pragma unroll
    for (int g4 = 0; g4 < 8; g4++) {
        const int4 t4 = *reinterpret_cast<const int4 *>(trow + g4 * 4);
        const int2 bb = *reinterpret_cast<const int2 *>(b2 + g4 * 2);
        const int tv[4] = {t4.x, t4.y, t4.z, t4.w};
        int sr[4];
#pragma unroll
        for (int i = 0; i < 4; i++) sr[i] = (int)(acc[g4 * 4 + i] * e.mult + (uint32_t)tv[i] + e.rc) >> e.shift;
        uint32_t s[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t v;
            asm("cvt.pack.sat.u16.s32 %0, %1, %2;" : "=r"(v) : "r"(sr[2 * h + 1]), "r"(sr[2 * h]));
            asm("min.u16x2 %0, %0, %1;" : "+r"(v) : "r"(0x00ff00ffu));
            v += (uint32_t)(h ? bb.y : bb.x);
            asm("max.s16x2 %0, %0, %1;" : "+r"(v) : "r"(lo1));
            asm("min.s16x2 %0, %0, %1;" : "+r"(v) : "r"(hi1));
            if (RES != 0) {
                const uint32_t r = RES == 1 ? ~rw[g4] : rw[g4];
                v += __byte_perm(r, 0, h ? 0x4342 : 0x4140);
                asm("max.s16x2 %0, %0, %1;" : "+r"(v) : "r"(lo2));
                asm("min.s16x2 %0, %0, %1;" : "+r"(v) : "r"(hi2));
            }
            s[h] = v;
        }
        words[g4] = __byte_perm(s[0], s[1], 0x6420);
    }
}

// The TMA epilogue of one group of four warps (fp16 / bf16, BN >= 64).  The group walks its tiles in blocks of 64
// output channels through `nbuf` shared-memory tiles of 128 rows x 128 bytes (SWIZZLE_128B).  Each thread owns one
// pixel row and never waits on another thread of its group or on global memory: it waits until the block's tile is
// available (for a fused residual that is the arrival of the residual tile, loaded by the group's agent), reads its 64
// accumulator columns from TMEM, combines them with its residual row in place, leaves the converted row in the tile
// and arrives on the tile's rows_ready barrier.  The agent (epilogue_agent) does the rest.
template <int KIND, int BN, int NACC, bool SPLIT>
__device__ __forceinline__ void epilogue_tma(const ConvTcParams &p, int grp, int warp, int lane, uint32_t tmem_base,
                                             uint8_t *tiles, uint64_t *acc_full, uint64_t *acc_empty, uint64_t *rows_ready,
                                             uint64_t *avail, volatile int *abort_flag)
{
    const int ngrp = p.epi_groups, nbuf = p.epi_bufs;
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool has_res = p.res != nullptr;
    const int act_mode = p.act_kind == THB_ACT_NONE ? 0
                         : p.act_kind != THB_ACT_THRESHOLD ? 2
                         : (p.act_th == 0.f && p.act_val == 0.f) ? 3 : 1;
    const EpiWalk<BN, SPLIT> walk(p, grp);
    EpiCursor cur = {0, 0};
    int b = 0;            // tile of the current block, and how often the ring of tiles has wrapped
    uint32_t wrap = 0;
    bool alive = true;
    while (cur.j < walk.my_tiles) {
        const int lt = grp + cur.j * ngrp;
        int m0, n0;
        walk.map.coords(lt, m0, n0);
        const int nsub0 = n0 + cur.sb * 64;
        const int ab = lt % NACC;
        const bool last_block = cur.sb == walk.blocks_of(cur.j) - 1;
        uint8_t *tile_smem = tiles + b * EPI_TILE_BYTES;
        if (cur.sb == 0) {
            if (!mbar_wait_bounded(smem_u32(&acc_full[ab]), (lt / NACC) & 1, p.wait_limit)) {
                if (lane == 0) atomicExch(p.status, 2);
                *abort_flag = 1;
                alive = false;
            }
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
        }
        uint32_t acc0[32], acc1[32];
        __syncwarp();
        tmem_ld32(lane_base + ab * BN + cur.sb * 64, acc0);
        tmem_ld32(lane_base + ab * BN + cur.sb * 64 + 32, acc1);
        tmem_ld_wait();
        if (last_block) {  // every column of this accumulator has been read: hand it back to the MMA warp
            tc_fence_before();
            mbar_arrive(smem_u32(&acc_empty[ab]));
        }
        if constexpr (SPLIT) {
            // split K: this CTA holds a partial sum of the tile.  The thread's 64 columns go to the fp32 scratch of its split
            // as they are; splitk_finish_kernel adds the splits and runs the epilogue.  No shared-memory tile, no agent.
            const int pm = m0 + row;
            if (pm < p.P) {
                float4 *dst = reinterpret_cast<float4 *>(p.partial + ((size_t)walk.map.split_of(lt) * p.P + pm) * p.partial_ld + nsub0);
#pragma unroll
                for (int q = 0; q < 8; q++) dst[q] = make_float4(__uint_as_float(acc0[4 * q]), __uint_as_float(acc0[4 * q + 1]),
                                                                 __uint_as_float(acc0[4 * q + 2]), __uint_as_float(acc0[4 * q + 3]));
#pragma unroll
                for (int q = 0; q < 8; q++) dst[8 + q] = make_float4(__uint_as_float(acc1[4 * q]), __uint_as_float(acc1[4 * q + 1]),
                                                                     __uint_as_float(acc1[4 * q + 2]), __uint_as_float(acc1[4 * q + 3]));
            }
            walk.advance(cur);
            continue;
        }
        // the tile is ours once its previous store has read it out and, with a residual, the residual rows are in it
        if (!mbar_wait_bounded(smem_u32(&avail[b]), wrap & 1, p.wait_limit)) {
            if (lane == 0) atomicExch(p.status, 8);
            *abort_flag = 1;
            alive = false;
        }
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        {
            uint8_t *row_smem = tile_smem + row * 128;
            const int rsw = row & 7;
            if (nsub0 + 64 > p.Cout || act_mode == 2 || act_mode == 1) {  // ragged channel edge or a general activation
                if (has_res) epi_block<KIND, true, 2, true>(acc0, acc1, row_smem, rsw, nsub0, p);
                else epi_block<KIND, false, 2, true>(acc0, acc1, row_smem, rsw, nsub0, p);
            } else if (has_res) {
                if (act_mode) epi_block<KIND, true, 3, false>(acc0, acc1, row_smem, rsw, nsub0, p);
                else epi_block<KIND, true, 0, false>(acc0, acc1, row_smem, rsw, nsub0, p);
            } else {
                if (act_mode) epi_block<KIND, false, 3, false>(acc0, acc1, row_smem, rsw, nsub0, p);
                else epi_block<KIND, false, 0, false>(acc0, acc1, row_smem, rsw, nsub0, p);
            }
        }
        fence_proxy_async_smem();  // this thread's row must be visible to the copy engine
        mbar_arrive(smem_u32(&rows_ready[b]));
        if (++b == nbuf) { b = 0; wrap++; }
        walk.advance(cur);
    }
}

// The agent of an epilogue group: one thread that owns the group's global-memory traffic.  It makes a tile available
// to the group (arming the tile's barrier with the TMA load of the residual tile when one is fused), waits until all
// 128 rows of a block are in its tile, hands the tile to a TMA store (which clips rows and channels beyond the tensor),
// waits until the store has read the tile out and makes it available for the block nbuf ahead.
template <int BN>
__device__ __forceinline__ void epilogue_agent(const ConvTcParams &p, const CUtensorMap *tmY, const CUtensorMap *tmR, int grp,
                                               uint8_t *tiles, uint64_t *rows_ready, uint64_t *avail,
                                               volatile int *abort_flag)
{
    const int nbuf = p.epi_bufs;
    const bool has_res = p.res != nullptr;
    const EpiWalk<BN> walk(p, grp);
    auto make_available = [&](const EpiCursor &c, int b) {
        int m0, n0;
        walk.map.coords(walk.local(c.j), m0, n0);
        if (has_res && m0 < p.P) {  // (a phantom half tile has no residual rows)
            mbar_arrive_expect_tx(smem_u32(&avail[b]), EPI_TILE_BYTES);
            tma_load_2d(smem_u32(tiles + b * EPI_TILE_BYTES), tmR, smem_u32(&avail[b]), n0 + c.sb * 64, m0);
        } else
            mbar_arrive(smem_u32(&avail[b]));
    };
    EpiCursor cur = {0, 0}, pre = {0, 0};  // block whose rows are awaited / next block to make a tile available for
    int q_pre = 0;
    for (; q_pre < nbuf && pre.j < walk.my_tiles; q_pre++) {
        make_available(pre, q_pre);
        walk.advance(pre);
    }
    int b = 0, q = 0;
    uint32_t wrap = 0;
    bool alive = true;
    for (; cur.j < walk.my_tiles; q++) {
        int m0, n0;
        walk.map.coords(walk.local(cur.j), m0, n0);
        if (!mbar_wait_bounded(smem_u32(&rows_ready[b]), wrap & 1, p.wait_limit)) {
            atomicExch(p.status, 5);
            *abort_flag = 1;
            alive = false;
            break;
        }
        if (m0 < p.P) tma_store_2d(tmY, smem_u32(tiles + b * EPI_TILE_BYTES), n0 + cur.sb * 64, m0);
        bulk_commit_group();
        bulk_wait_group_read<0>();
        if (pre.j < walk.my_tiles) {
            make_available(pre, b);
            walk.advance(pre);
            q_pre++;
        }
        if (++b == nbuf) { b = 0; wrap++; }
        walk.advance(cur);
    }
    bulk_wait_group<0>();
    // after an early exit, residual loads still in flight must land before the CTA may leave
    if (!alive && has_res)
        for (int k = q; k < q_pre; k++) mbar_wait_bounded(smem_u32(&avail[k % nbuf]), (k / nbuf) & 1, p.wait_limit);
}

template <int KIND, int BN, int STAGES, bool SPLIT>
__global__ void __launch_bounds__(NTHREADS, 1) conv_tc_kernel(const __grid_constant__ CUtensorMap tmapW, const __grid_constant__ CUtensorMap tmapA,
                                                               const __grid_constant__ CUtensorMap tmapY, const __grid_constant__ CUtensorMap tmapR,
                                                               const ConvTcParams p)
{
    using L = Smem<KIND, BN, STAGES>;
    constexpr int ES = kind_traits<KIND>::esize;
    constexpr int BKE = 128 / ES;  // K elements per 128-byte stage row
    constexpr int B_STAGE_BYTES = L::B_STAGE_BYTES;
    constexpr int SUBN = L::SUBN;
    constexpr int LAG = STAGES >= 4 ? STAGES - 2 : STAGES - 1;  // cp.async groups a producer thread keeps in flight
    constexpr uint32_t IDESC = make_idesc(KIND == 2 ? 2u : 1u, KIND == 1 ? 1u : 0u, BN);
    constexpr int NACC = BN >= 256 ? 2 : 4;  // TMEM accumulators: the MMA warp runs this many tiles ahead of the epilogue
    constexpr uint32_t TMEM_COLS = NACC * BN < 32 ? 32 : NACC * BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int nst = L::TMA_EPI ? p.stages : STAGES;  // pipeline stages in use
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    const bool pair = L::TMA_EPI && p.pair;
    const int a_stage_bytes = pair ? 2 * A_STAGE_BYTES : A_STAGE_BYTES;  // pair mode: both halves' activation tiles
    uint8_t *sA = smem + L::BAR_BYTES;
    uint8_t *sB = sA + nst * a_stage_bytes;
    uint8_t *stage_buf = sB + nst * B_STAGE_BYTES;
    uint64_t *full = bars, *empty = bars + MAX_STAGES;
    uint64_t *acc_full = bars + 2 * MAX_STAGES, *acc_empty = acc_full + 4;
    uint64_t *rows_ready = acc_empty + 4, *avail = rows_ready + 9;   // TMA epilogue: a pair per group and tile
    uint64_t *stg_ready = rows_ready, *stg_free = rows_ready + 3;    // staged epilogue: a pair per group
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(avail + 9);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (tid == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(smem_u32(&full[s]), p.a_tma ? 1 : 128 + 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < NACC; b++) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 128);
        }
        for (int g = 0; g < 9; g++) {
            mbar_init(smem_u32(&rows_ready[g]), 128);
            mbar_init(smem_u32(&avail[g]), 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmapW);
        if (p.a_tma) tma_prefetch_desc(&tmapA);
        if (L::TMA_EPI) {
            tma_prefetch_desc(&tmapY);
            if (p.res || p.nkb1) tma_prefetch_desc(&tmapR);
        }
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: this grid may have been started while the previous kernel of the stream was
    // still draining, so that the set-up above overlaps its tail.  Nothing before this point touches memory that
    // kernel could write or read; from here on it must have finished.  The next kernel may start its own set-up as
    // soon as this grid's CTAs leave their SMs.
    if (p.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (warp == 14) {
        // ================================================================== epilogue agents (TMA epilogue only)
        if constexpr (L::TMA_EPI)
            if (lane < p.epi_groups && !SPLIT)   // (split K: the partial tiles go straight to the fp32 scratch)
                epilogue_agent<BN>(p, &tmapY, &tmapR, lane, stage_buf + lane * p.epi_bufs * EPI_TILE_BYTES, rows_ready + lane * 3,
                                   avail + lane * 3, abort_flag);
        __syncwarp();
    } else if (warp < 4 && !(!L::TMA_EPI && p.a_tma && p.epi_groups == 3)) {
        // ================================================================== A producer (gather mode)
        // (with the staged epilogue and nothing to gather, these warps are its third group: the last branch below)
        if (p.a_tma) {
            // nothing to gather: these four warps are the third epilogue group
            if constexpr (L::TMA_EPI)
                if (p.epi_groups == 3)
                    epilogue_tma<KIND, BN, NACC, SPLIT>(p, 2, warp, lane, tmem_base, stage_buf + 2 * p.epi_bufs * EPI_TILE_BYTES,
                                                 acc_full, acc_empty, rows_ready + 6, avail + 6, abort_flag);
            goto done;
        }
        const int chunk = lane & 7;
        bool alive = true;
        int it = 0;  // K blocks issued so far by this CTA, over all its tiles
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
            const int m0 = (tile / p.n_tiles) * BM;
            // this thread's eight rows are 4 pixels apart: decompose the first, then step
            int ih0[8], iw0[8], pixbase[8];
            {
                int pm = m0 + warp * 32 + (lane >> 3);
                int n = pm / p.oHW, rem = pm - n * p.oHW;
                int oh = rem / p.oW, ow = rem - oh * p.oW;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (pm < p.P) {
                        ih0[j] = oh * p.dH - p.padH;
                        iw0[j] = ow * p.dW - p.padW;
                        pixbase[j] = n * p.H * p.row_pitch + p.pad_left;
                    } else {
                        ih0[j] = iw0[j] = 0;
                        pixbase[j] = -1;
                    }
                    pm += 4;
                    ow += 4;
                    while (ow >= p.oW) {
                        ow -= p.oW;
                        if (++oh == p.oH) { oh = 0; n++; }
                    }
                }
            }
            int ki_next = chunk < p.n_kchunks ? __ldg(p.kinfo + chunk) : -1;
            for (int kb = 0; kb < p.nkb; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const int ki = ki_next;
                {
                    const int g = (kb + 1) * 8 + chunk;
                    ki_next = (kb + 1 < p.nkb && g < p.n_kchunks) ? __ldg(p.kinfo + g) : -1;
                }
                if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1, p.wait_limit)) {
                    if (lane == 0) atomicExch(p.status, 1);
                    *abort_flag = 1;
                    alive = false;
                    break;
                }
                const int dh = (ki >> 24) & 0x7f, dw = (ki >> 16) & 0xff;
                const size_t coff = (size_t)(ki & 0xffff) * 16;
                const uint32_t a_stage = smem_u32(sA + s * A_STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int r = warp * 32 + j * 4 + (lane >> 3);
                    const int ih = ih0[j] + dh, iw = iw0[j] + dw;
                    const bool ok = ki >= 0 && pixbase[j] >= 0 && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W;
                    const uint8_t *src = ok ? p.x + ((size_t)(pixbase[j] + ih * p.row_pitch + iw) * p.in_ld) * ES + coff : p.x;
                    const uint32_t dst = a_stage + r * 128 + ((chunk ^ (r & 7)) << 4);
                    if (p.use_l1) cp_async16_ca(dst, src, ok ? 16u : 0u);
                    else cp_async16(dst, src, ok ? 16u : 0u);
                }
                cp_async_commit();
                if (it >= LAG) {
                    cp_async_wait<LAG>();
                    fence_proxy_async_smem();
                    mbar_arrive(smem_u32(&full[(it - LAG) % STAGES]));
                }
            }
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (alive)
            for (int k = (it > LAG ? it - LAG : 0); k < it; k++) mbar_arrive(smem_u32(&full[k % STAGES]));
    } else if (warp == 4) {
        // ================================================================== TMA producer: per K block the weight tile
        // and, in the TMA modes, the activation tile (both halves' tiles in pair mode)
        if (lane == 0) {
            const TileMap<BN, SPLIT> map(p);
            const int halves = pair ? 2 : 1;
            int ring_s = 0;  // stage and phase in the ring of nst stages
            uint32_t ring_ph = 0;
            bool alive = true;
            for (int lt = 0; lt < map.n_local && alive; lt += halves) {
                int m0, n0;
                map.coords(lt, m0, n0);
                // im2col mode: input position of each half's first output pixel for tap (0, 0)
                int iw[2] = {0, 0}, ih[2] = {0, 0}, in[2] = {0, 0}, tap_w = 0, tap_h = 0, slab = 0;
                if (p.nkb1 && p.a2_mode == 2)
                    for (int h = 0; h < halves; h++) {   // where the second operand is sampled for each half's first pixel
                        const int m = m0 + h * BM;
                        in[h] = m / p.oHW;
                        const int rem = m - in[h] * p.oHW;
                        const int oh = rem / p.oW;
                        ih[h] = oh * p.a2_d;
                        iw[h] = (rem - oh * p.oW) * p.a2_d;
                    }
                if (p.a_tma == 2)
                    for (int h = 0; h < halves; h++) {
                        const int m = m0 + h * BM;
                        in[h] = m / p.oHW;
                        const int rem = m - in[h] * p.oHW;
                        const int oh = rem / p.oW;
                        ih[h] = oh * p.dH - p.padH;
                        iw[h] = (rem - oh * p.oW) * p.dW - p.tma_padw;
                    }
                // split K: this unit covers the K blocks [kb0, kb1) of its tile, starting at the tap and slab of kb0
                int kb0 = 0, kb1 = p.nkb;
                if (SPLIT) {
                    map.kblocks(lt, kb0, kb1);
                    if (p.a_tma == 2) {
                        const int tap = kb0 / p.slabs;
                        slab = kb0 - tap * p.slabs;
                        tap_h = tap / p.tma_kw;
                        tap_w = tap - tap_h * p.tma_kw;
                    }
                }
                for (int kb = kb0; kb < kb1; kb++) {
                    const int s = ring_s;
                    const uint32_t ph = ring_ph;
                    if (++ring_s == nst) { ring_s = 0; ring_ph ^= 1; }
                    if (!mbar_wait_bounded(smem_u32(&empty[s]), ph ^ 1, p.wait_limit)) {
                        atomicExch(p.status, 3);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    // (tests of the give-up path: every earlier copy has been consumed by then, nothing is in flight)
                    if (p.test_withhold && kb == kb1 - 1 && lt + halves >= map.n_local) break;
                    const uint32_t bar = smem_u32(&full[s]);
                    if (p.half) {
                        const int nh = 2 * kb + 1 < p.ntaps ? 2 : 1;
                        mbar_arrive_expect_tx(bar, (uint32_t)(nh * (A_STAGE_BYTES / 2 + B_STAGE_BYTES / 2)));
                        for (int h = 0; h < nh; h++) {
                            tma_load_im2col_4d(smem_u32(sA + s * a_stage_bytes + h * (A_STAGE_BYTES / 2)), &tmapA, bar, 0, iw[0], ih[0],
                                               in[0], (uint16_t)tap_w, (uint16_t)tap_h);
                            tma_load_2d(smem_u32(sB + s * B_STAGE_BYTES + h * (B_STAGE_BYTES / 2)), &tmapW, bar, (2 * kb + h) * (BKE / 2), n0);
                            if (++tap_w == p.tma_kw) { tap_w = 0; tap_h++; }
                        }
                        continue;
                    }
                    mbar_arrive_expect_tx(bar, (uint32_t)(B_STAGE_BYTES + (p.a_tma ? a_stage_bytes : 0)));
                    if (p.a_tma == 1 && p.nkb1 && kb >= p.nkb1) {
                        for (int h = 0; h < halves; h++) {
                            const uint32_t dst = smem_u32(sA + s * a_stage_bytes + h * A_STAGE_BYTES);
                            if (p.a2_mode == 1) tma_load_2d(dst, &tmapR, bar, (kb - p.nkb1) * BKE, m0 + h * BM);
                            else tma_load_im2col_4d(dst, &tmapR, bar, (kb - p.nkb1) * BKE, iw[h], ih[h], in[h], 0, 0);
                        }
                    } else if (p.a_tma == 1) {
                        for (int h = 0; h < halves; h++)
                            tma_load_2d(smem_u32(sA + s * a_stage_bytes + h * A_STAGE_BYTES), &tmapA, bar, kb * BKE, m0 + h * BM);
                    } else if (p.a_tma == 2) {
                        for (int h = 0; h < halves; h++)
                            tma_load_im2col_4d(smem_u32(sA + s * a_stage_bytes + h * A_STAGE_BYTES), &tmapA, bar, slab * BKE, iw[h],
                                               ih[h], in[h], (uint16_t)tap_w, (uint16_t)tap_h);
                        if (++slab == p.slabs) {
                            slab = 0;
                            if (++tap_w == p.tma_kw) { tap_w = 0; tap_h++; }
                        }
                    }
                    tma_load_2d(smem_u32(sB + s * B_STAGE_BYTES), &tmapW, bar, kb * BKE, n0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            const TileMap<BN, SPLIT> map(p);
            const int halves = pair ? 2 : 1;
            int ring_s = 0;
            uint32_t ring_ph = 0;
            bool alive = true;
            for (int lt = 0; lt < map.n_local && alive; lt += halves) {
                // the accumulators of this unit's local tiles (two in pair mode) must have been drained
                for (int h = 0; h < halves && alive; h++)
                    if (!mbar_wait_bounded(smem_u32(&acc_empty[(lt + h) % NACC]), (((lt + h) / NACC) & 1) ^ 1, p.wait_limit)) {
                        atomicExch(p.status, 6);
                        *abort_flag = 1;
                        alive = false;
                    }
                if (!alive) break;
                tc_fence_after();
                const uint32_t d0 = tmem_base + (lt % NACC) * BN, d1 = tmem_base + ((lt + 1) % NACC) * BN;
                int kb0 = 0, kb1 = p.nkb;
                if (SPLIT) map.kblocks(lt, kb0, kb1);
                for (int kb = kb0; kb < kb1; kb++) {
                    const int s = ring_s;
                    const uint32_t ph = ring_ph;
                    if (++ring_s == nst) { ring_s = 0; ring_ph ^= 1; }
                    if (!mbar_wait_bounded(smem_u32(&full[s]), ph, p.wait_limit)) {
                        atomicExch(p.status, 4);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    fence_proxy_async_smem();
                    if (p.half) {
                        const int nh = 2 * kb + 1 < p.ntaps ? 2 : 1;
                        for (int h = 0; h < nh; h++) {
                            const uint64_t ad = make_sw64_kmajor_desc(smem_u32(sA + s * a_stage_bytes + h * (A_STAGE_BYTES / 2)));
                            const uint64_t bd = make_sw64_kmajor_desc(smem_u32(sB + s * B_STAGE_BYTES + h * (B_STAGE_BYTES / 2)));
#pragma unroll
                            for (int k = 0; k < 2; k++) {
                                const uint32_t accum = ((kb - kb0) | h | k) != 0;
                                if (KIND == 2) tc_mma_i8(d0, ad + 2 * k, bd + 2 * k, IDESC, accum);
                                else tc_mma_f16(d0, ad + 2 * k, bd + 2 * k, IDESC, accum);
                            }
                        }
                        tc_commit(smem_u32(&empty[s]));
                        continue;
                    }
                    const uint64_t adesc = make_sw128_kmajor_desc(smem_u32(sA + s * a_stage_bytes));
                    const uint64_t bdesc = make_sw128_kmajor_desc(smem_u32(sB + s * B_STAGE_BYTES));
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const uint32_t accum = ((kb - kb0) | k) != 0;
                        if (KIND == 2) tc_mma_i8(d0, adesc + 2 * k, bdesc + 2 * k, IDESC, accum);
                        else tc_mma_f16(d0, adesc + 2 * k, bdesc + 2 * k, IDESC, accum);
                    }
                    if (pair) {
                        // the second half's tile lies A_STAGE_BYTES further on (1024 in the descriptor's 16-byte units)
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            tc_mma_f16(d1, adesc + (A_STAGE_BYTES >> 4) + 2 * k, bdesc + 2 * k, IDESC, (uint32_t)((kb | k) != 0));
                    }
                    tc_commit(smem_u32(&empty[s]));
                }
                if (alive)
                    for (int h = 0; h < halves; h++) tc_commit(smem_u32(&acc_full[(lt + h) % NACC]));
            }
        }
        __syncwarp();
    } else {
        // ================================================================== epilogue (warps 6-13)
        // Two groups of four warps; group g owns TMEM accumulator g and every second tile of this CTA, so the
        // write-out of one tile overlaps the accumulator drain of the next.
        const int grp = warp < 4 ? 2 : (warp - 6) >> 2;
        const int et = warp < 4 ? tid : tid - 192 - grp * 128;  // 0..127 within the group
        const int ngrp = L::TMA_EPI ? 2 : (p.epi_groups == 3 ? 3 : 2);  // groups sharing the staged epilogue's tiles
        if constexpr (L::TMA_EPI) {
            epilogue_tma<KIND, BN, NACC, SPLIT>(p, grp, warp, lane, tmem_base, stage_buf + grp * p.epi_bufs * EPI_TILE_BYTES, acc_full,
                                         acc_empty, rows_ready + grp * 3, avail + grp * 3, abort_flag);
            goto done;
        }
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int row = quad * 32 + lane;      // tile row (= pixel) owned in phase 1
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        uint8_t *stg = stage_buf + grp * L::STAGING_PAD;
        const uint32_t bar_ready = smem_u32(&stg_ready[grp]), bar_free = smem_u32(&stg_free[grp]);
        const bool has_res = KIND != 2 && p.res != nullptr;
        const int act_mode = p.act_kind == THB_ACT_NONE ? 0
                             : p.act_kind != THB_ACT_THRESHOLD ? 2
                             : (p.act_th == 0.f && p.act_val == 0.f) ? 3 : 1;
        bool alive = true;
        int sub_it = 0;                        // staging blocks this group has processed
        int *tbl = reinterpret_cast<int *>(stage_buf + 3 * L::STAGING_PAD + grp * L::TBL_BYTES);  // uint8 only
        const uint32_t bar_tbl = smem_u32(&rows_ready[6 + grp]);
        int tbl_n0 = -1;
        uint32_t tbl_phase = 0;
        for (int lt = grp; alive; lt += ngrp) {
            const int tile = blockIdx.x + lt * gridDim.x;
            if (tile >= total_tiles) break;
            const int m0 = (tile / p.n_tiles) * BM, n0 = (tile % p.n_tiles) * BN;
            const int ab = lt % NACC;  // accumulator holding this tile
            const uint32_t lane_addr = lane_base + ab * BN;
            const int pm = m0 + row;
            const bool valid = pm < p.P;
            const bool check = n0 + BN > p.Cout;  // the tile reaches beyond the last real channel
            // per-pixel terms of the u8 zero-point correction
            int corr_pix = 0, r0 = 0, r1 = 0, s0 = 0, s1 = 0, plane_pos = 0;
            bool interior = true;
            if (KIND == 2 && valid) {
                const int n = pm / p.oHW, rem = pm - n * p.oHW;
                const int oh = rem / p.oW, ow = rem - oh * p.oW;
                plane_pos = rem;
                const int ihb = oh * p.dH - p.padH, iwb = ow * p.dW - p.padW;
                r0 = max(0, -ihb); r1 = min(p.kH, p.H - ihb);
                s0 = max(0, -iwb); s1 = min(p.kW, p.W - iwb);
                interior = r0 == 0 && s0 == 0 && r1 == p.kH && s1 == p.kW;
                int xsum = 0;
                const int *cs = p.csum + (size_t)n * p.H * p.W;
                for (int r = r0; r < r1; r++)
                    for (int s = s0; s < s1; s++) xsum += __ldg(cs + (ihb + r) * p.W + iwb + s);
                const int nvalid = max(0, r1 - r0) * max(0, s1 - s0);
                corr_pix = p.a_off * (xsum + p.b_off * nvalid * p.Cin);
            }
            // uint8 fast path: the window's border class of this row selects a row of the group's table
            // T[class][channel] = b_off * (sum of the weights of channel `channel` over the taps inside the image)
            int cls = 0;
            bool fast = KIND == 2 && p.u8_classes > 0;
            if (KIND == 2 && fast) {
                if (valid) {
                    const int ct = r0, cb = p.kH - r1, cl = s0, cr = p.kW - s1;  // taps clipped at each side
                    if ((ct > 0 && cb > 0) || (cl > 0 && cr > 0) || ct > p.padH || cb > p.padH || cl > p.padW || cr > p.padW ||
                        r1 <= r0 || s1 <= s0)
                        fast = false;  // clipped on two opposite sides (image smaller than the kernel): no class for that
                    else
                        cls = (ct > 0 ? ct : cb > 0 ? p.padH + cb : 0) * (1 + 2 * p.padW) + (cl > 0 ? cl : cr > 0 ? p.padW + cr : 0);
                }
                fast = __all_sync(0xffffffffu, fast);
                if (n0 != tbl_n0) {
                    // (re)build the table for this tile's channels: all four warps of the group, between two group barriers
                    bool ok = true;
                    mbar_arrive(bar_tbl);
                    ok = mbar_wait_bounded(bar_tbl, tbl_phase & 1, p.wait_limit);
                    tbl_phase++;
                    if (ok) {
                        const int ncc = 1 + 2 * p.padW, satw = p.kW + 1, satn = (p.kH + 1) * (p.kW + 1);
                        for (int idx = et; idx < p.u8_classes * BN; idx += 128) {
                            const int k = idx / BN, col = idx - k * BN;
                            const int rc = k / ncc, cc = k - rc * ncc;
                            const int tr0 = rc >= 1 && rc <= p.padH ? rc : 0, tr1 = rc > p.padH ? p.kH - (rc - p.padH) : p.kH;
                            const int ts0 = cc >= 1 && cc <= p.padW ? cc : 0, ts1 = cc > p.padW ? p.kW - (cc - p.padW) : p.kW;
                            const int *t = p.wsat + (size_t)min(n0 + col, p.Cout - 1) * satn;
                            // (stored times c_mult, modulo 2^32: the requantisation multiplies the corrected sum by it)
                            tbl[k * L::TBL_ROW + col] = (int)((uint32_t)(p.b_off * (__ldg(t + tr1 * satw + ts1) - __ldg(t + tr0 * satw + ts1) -
                                                                                    __ldg(t + tr1 * satw + ts0) + __ldg(t + tr0 * satw + ts0))) *
                                                              (uint32_t)p.c_mult);
                        }
                        for (int col = et; col < BN; col += 128)
                            tbl[L::TBL_CAP + col] = p.bias_add ? __ldg(p.bias_add + min(n0 + col, p.Cout - 1)) : 0;
                        // the addends once more for the paired arithmetic (u8_chunk32_pairs): two per word, each clamped
                        // to +-255 and raised by the offset that keeps the halves non-negative
                        const int off2 = p.res ? 384 : 256;
                        for (int pr = et; pr < BN / 2; pr += 128) {
                            const int ba = p.bias_add ? __ldg(p.bias_add + min(n0 + 2 * pr, p.Cout - 1)) : 0;
                            const int bb = p.bias_add ? __ldg(p.bias_add + min(n0 + 2 * pr + 1, p.Cout - 1)) : 0;
                            tbl[L::TBL_CAP + 256 + pr] = (min(max(ba, -255), 255) + off2) | ((min(max(bb, -255), 255) + off2) << 16);
                        }
                        mbar_arrive(bar_tbl);
                        ok = mbar_wait_bounded(bar_tbl, tbl_phase & 1, p.wait_limit);
                        tbl_phase++;
                    }
                    if (!ok) {
                        if (lane == 0) atomicExch(p.status, 8);
                        *abort_flag = 1;
                        alive = false;
                    }
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    tbl_n0 = n0;
                }
            }
            bool have_acc = false;
            uint32_t rowsum = 0;  // uint8: sum of this row's output bytes over the tile's columns
#pragma unroll 1
            for (int sb = 0; sb < BN / SUBN; sb++, sub_it++) {
                const int nsub0 = n0 + sb * SUBN;
                // the residual chunks this thread will need in phase 2: issued now, consumed after the staging
                // round trip, so their latency hides behind the accumulator drain
                constexpr int CPRF = SUBN / 8, RPI = 128 / CPRF;
                const int cg = et % CPRF, rbase = et / CPRF, c0f = nsub0 + cg * 8;
                uint4 rv[CPRF];
                if (KIND != 2) {
#pragma unroll
                    for (int u = 0; u < CPRF; u++) {
                        const int pm2 = m0 + rbase + u * RPI;
                        rv[u] = make_uint4(0, 0, 0, 0);
                        if (has_res && pm2 < p.P && c0f < p.Cout)
                            rv[u] = __ldg(reinterpret_cast<const uint4 *>(p.res + ((size_t)pm2 * p.res_ld + c0f) * 2));
                    }
                }
                if (!have_acc) {
                    if (!mbar_wait_bounded(smem_u32(&acc_full[ab]), (lt / NACC) & 1, p.wait_limit)) {
                        if (lane == 0) atomicExch(p.status, 2);
                        *abort_flag = 1;
                        alive = false;
                    }
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    tc_fence_after();
                    have_acc = true;
                }
                // ---- phase 1: this thread's pixel row, SUBN accumulator columns -> staging tile
                // (uint8: a warp stages and writes out its own 32 rows, so it synchronises with nobody but itself)
                if (KIND != 2) {
                    if (!mbar_wait_bounded(bar_free, (sub_it & 1) ^ 1, p.wait_limit)) {
                        if (lane == 0) atomicExch(p.status, 7);
                        *abort_flag = 1;
                        alive = false;
                    }
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                }
                if (KIND == 2 && fast) {
                    // 32 accumulator columns per TMEM load; per column one table word (the row's border class) and one bias
                    // addend from shared memory, then integer arithmetic only (u8_chunk32).
                    const int *trow = tbl + cls * L::TBL_ROW + sb * SUBN;
                    const int *brow = tbl + L::TBL_CAP + sb * SUBN;
                    U8Epi e;
                    e.mult = (uint32_t)p.c_mult;
                    e.rc = (uint32_t)(corr_pix + p.c_off) * e.mult + (p.c_shift >= 1 ? 1u << (p.c_shift - 1) : 0u);
                    e.shift = p.c_shift > 0 ? p.c_shift : 0;
                    e.tailmask = plane_pos < p.tail_start ? 0 : 255;  // the reference's tail adds without the lower clamp
                    e.thr = p.relu_thr;                               // < 0: every byte passes
                    e.rval = p.relu_thr < 0 ? 0 : p.relu_val;
                    e.ca = (int)p.self_coef; e.cb = (int)p.res_coef; e.addend = p.res_addend;
                    const bool u8res = p.res != nullptr;
                    // the form the fused residual takes in the paired arithmetic (0: neither, the scalar code does it)
                    const int res_mode = e.ca == 1 && e.cb == -1 ? 1 : e.ca == 1 && e.cb == 1 ? 3 : 0;
                    const int *b2row = tbl + L::TBL_CAP + 256 + sb * (SUBN / 2);
                    // the common case per warp: no tail row, Threshold replaces by its own threshold byte (or none)
                    const bool general = __any_sync(0xffffffffu, e.tailmask != 0) || (p.relu_thr >= 0 && p.relu_val != p.relu_thr);
                    const uint8_t *rrow = p.res + (size_t)(valid ? pm : 0) * p.res_ld + nsub0;
#pragma unroll 1
                    for (int cc = 0; cc < SUBN / 32; cc++) {
                        uint32_t acc[32];
                        uint4 res0 = make_uint4(0, 0, 0, 0), res1 = res0;
                        if (u8res && nsub0 + cc * 32 < p.res_ld) {
                            // residual bytes of this row: issued before the accumulator wait
                            res0 = __ldg(reinterpret_cast<const uint4 *>(rrow + cc * 32));
                            if (nsub0 + cc * 32 + 16 < p.res_ld) res1 = __ldg(reinterpret_cast<const uint4 *>(rrow + cc * 32 + 16));
                        }
                        __syncwarp();
                        tmem_ld32(lane_addr + sb * SUBN + cc * 32, acc);
                        tmem_ld_wait();
                        if (p.acc_out && valid) {
                            // raw corrected accumulators (tests only)
#pragma unroll
                            for (int i = 0; i < 32; i++) {
                                const int c = nsub0 + cc * 32 + i;
                                if (c < p.Cout) {
                                    // the row's own tap rectangle, from the summed-area table of the channel's weights
                                    const int satw = p.kW + 1;
                                    const int *t = p.wsat + (size_t)c * (p.kH + 1) * satw;
                                    const int wsum = __ldg(t + r1 * satw + s1) - __ldg(t + r0 * satw + s1) - __ldg(t + r1 * satw + s0) +
                                                     __ldg(t + r0 * satw + s0);
                                    p.acc_out[(size_t)pm * p.Cout + c] = (int)acc[i] + p.b_off * wsum + corr_pix;
                                }
                            }
                        }
                        uint32_t words[8];
                        if (u8res) {
                            if (general) u8_chunk32<true, true>(acc, trow + cc * 32, brow + cc * 32, e, res0, res1, words);
                            else if (res_mode == 1) u8_chunk32_pairs<1>(acc, trow + cc * 32, b2row + cc * 16, e, res0, res1, words);
                            else if (res_mode == 3) u8_chunk32_pairs<3>(acc, trow + cc * 32, b2row + cc * 16, e, res0, res1, words);
                            else u8_chunk32<false, true>(acc, trow + cc * 32, brow + cc * 32, e, res0, res1, words);
                        } else {
                            if (general) u8_chunk32<true, false>(acc, trow + cc * 32, brow + cc * 32, e, res0, res1, words);
                            else u8_chunk32_pairs<0>(acc, trow + cc * 32, b2row + cc * 16, e, res0, res1, words);
                        }
                        if (check) {
                            // channels beyond the last real one are stored as zero bytes
#pragma unroll
                            for (int g4 = 0; g4 < 8; g4++) {
                                const int nreal = p.Cout - (nsub0 + cc * 32 + g4 * 4);
                                words[g4] &= nreal >= 4 ? 0xffffffffu : nreal <= 0 ? 0u : (1u << (8 * nreal)) - 1u;
                            }
                        }
#pragma unroll
                        for (int g4 = 0; g4 < 8; g4++) rowsum = __dp4a(words[g4], 0x01010101u, rowsum);  // (dead code unless csum_out)
                        uint4 *dst = reinterpret_cast<uint4 *>(stg + row * (SUBN + 16) + cc * 32);
                        dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
                        dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
                    }
                } else if (KIND == 2) {
                    if (p.res && lane == 0) atomicExch(p.status, 9);  // a fused residual exists on the table-driven path only
                    // Eight columns at a time in a rolled loop (compact code: the unrolled 32-column form was bound by
                    // instruction fetch).  Per-channel constants are loaded once per group; only rows whose window is
                    // clipped by the image border look their own tap rectangle up in the summed-area table.
                    const int satw = p.kW + 1, satn = (p.kH + 1) * (p.kW + 1);
                    const bool clipped = valid && !interior;
                    const uint32_t rnd = p.c_shift >= 1 ? 1u << (p.c_shift - 1) : 0u;
                    const int cmax = p.Cout - 1;
#pragma unroll 1
                    for (int c8 = 0; c8 < SUBN / 8; c8++) {
                        uint32_t a8[8];
                        __syncwarp();
                        tmem_ld8(lane_addr + sb * SUBN + c8 * 8, a8);
                        tmem_ld_wait();
                        const int c0 = nsub0 + c8 * 8;
                        uint32_t lo = 0, hi = 0;
                        if (c0 < p.Cout) {
                            int wv[8], badd[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int c = min(c0 + i, cmax);
                                wv[i] = __ldg(p.wsat + (size_t)c * satn + satn - 1);
                                badd[i] = p.bias_add ? __ldg(p.bias_add + c) : 0;
                            }
                            if (clipped) {
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    const int *t = p.wsat + (size_t)min(c0 + i, cmax) * satn;
                                    wv[i] = __ldg(t + r1 * satw + s1) - __ldg(t + r0 * satw + s1) - __ldg(t + r1 * satw + s0) +
                                            __ldg(t + r0 * satw + s0);
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const int c = c0 + i;
                                int q = 0;
                                if (valid && c < p.Cout) {
                                    const int a = (int)a8[i] + p.b_off * wv[i] + corr_pix;
                                    if (p.acc_out) p.acc_out[(size_t)pm * p.Cout + c] = a;
                                    const uint32_t v = ((uint32_t)a + (uint32_t)p.c_off) * (uint32_t)p.c_mult + rnd;
                                    int sres = (int)v;
                                    if (p.c_shift > 0) sres >>= p.c_shift;
                                    q = min(255, max(0, sres));
                                    int t2 = q + badd[i];
                                    if (plane_pos < p.tail_start) t2 = min(255, max(0, t2));
                                    else t2 = t2 > 255 ? 255 : (t2 & 255);
                                    q = t2;
                                    if (p.relu_thr >= 0) q = q > p.relu_thr ? q : p.relu_val;
                                }
                                if (i < 4) lo |= (uint32_t)q << (8 * i);
                                else hi |= (uint32_t)q << (8 * (i - 4));
                            }
                        }
                        rowsum = __dp4a(hi, 0x01010101u, __dp4a(lo, 0x01010101u, rowsum));
                        *reinterpret_cast<uint2 *>(stg + row * (SUBN + 16) + c8 * 8) = make_uint2(lo, hi);
                    }
                } else {
#pragma unroll
                    for (int cc = 0; cc < SUBN / 32; cc++) {
                        uint32_t acc[32];
                        __syncwarp();
                        tmem_ld32(lane_addr + sb * SUBN + cc * 32, acc);
                        tmem_ld_wait();
                        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<float *>(stg) + row * (SUBN + 4) + cc * 32);
#pragma unroll
                        for (int q = 0; q < 8; q++) dst[q] = make_uint4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
                    }
                }
                if (sb == BN / SUBN - 1) {
                    // every column of this accumulator has been read: hand it back to the MMA warp
                    tc_fence_before();
                    mbar_arrive(smem_u32(&acc_empty[ab]));
                }
                if (KIND == 2) {
                    __syncwarp();
                } else {
                    mbar_arrive(bar_ready);
                    if (!mbar_wait_bounded(bar_ready, sub_it & 1, p.wait_limit)) {
                        if (lane == 0) atomicExch(p.status, 5);
                        *abort_flag = 1;
                        alive = false;
                    }
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                }
                // ---- phase 2: coalesced write-out of the staged block
                if (KIND == 2) {
                    // the warp's own 32 rows, 16-byte chunks: each instruction stores whole rows' worth of contiguous bytes
                    constexpr int CPR = SUBN / 16;
#pragma unroll
                    for (int u = 0; u < CPR; u++) {
                        const int idx = lane + u * 32, r = quad * 32 + idx / CPR, cg2 = idx % CPR;
                        const int pm2 = m0 + r, c0 = nsub0 + cg2 * 16;
                        if (pm2 < p.P && c0 < p.Cout)
                            *reinterpret_cast<uint4 *>(p.y + (size_t)pm2 * p.out_ld + c0) =
                                *reinterpret_cast<const uint4 *>(stg + r * (SUBN + 16) + cg2 * 16);
                    }
                    __syncwarp();
                } else if (c0f < p.Cout) {
                    const float *stage = reinterpret_cast<const float *>(stg);
                    float sc[8], sh[8], sl[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) { sc[i] = 1.f; sh[i] = 0.f; sl[i] = 0.f; }
                    if (p.scale) {
                        const float4 t0 = __ldg(reinterpret_cast<const float4 *>(p.scale + c0f)), t1 = __ldg(reinterpret_cast<const float4 *>(p.scale + c0f + 4));
                        sc[0] = t0.x; sc[1] = t0.y; sc[2] = t0.z; sc[3] = t0.w; sc[4] = t1.x; sc[5] = t1.y; sc[6] = t1.z; sc[7] = t1.w;
                    }
                    if (p.shift) {
                        const float4 t0 = __ldg(reinterpret_cast<const float4 *>(p.shift + c0f)), t1 = __ldg(reinterpret_cast<const float4 *>(p.shift + c0f + 4));
                        sh[0] = t0.x; sh[1] = t0.y; sh[2] = t0.z; sh[3] = t0.w; sh[4] = t1.x; sh[5] = t1.y; sh[6] = t1.z; sh[7] = t1.w;
                    }
                    if (p.slope) {
                        const float4 t0 = __ldg(reinterpret_cast<const float4 *>(p.slope + c0f)), t1 = __ldg(reinterpret_cast<const float4 *>(p.slope + c0f + 4));
                        sl[0] = t0.x; sl[1] = t0.y; sl[2] = t0.z; sl[3] = t0.w; sl[4] = t1.x; sl[5] = t1.y; sl[6] = t1.z; sl[7] = t1.w;
                    }
                    if (has_res && p.self_coef != 1.f) {
#pragma unroll
                        for (int i = 0; i < 8; i++) { sc[i] *= p.self_coef; sh[i] *= p.self_coef; }
                    }
#pragma unroll
                    for (int u = 0; u < CPRF; u++) {
                        const int r = rbase + u * RPI, pm2 = m0 + r;
                        if (pm2 >= p.P) continue;
                        const float4 a0 = *reinterpret_cast<const float4 *>(stage + r * (SUBN + 4) + cg * 8);
                        const float4 a1 = *reinterpret_cast<const float4 *>(stage + r * (SUBN + 4) + cg * 8 + 4);
                        uint4 o;
                        if (check || act_mode == 2 || act_mode == 1) o = epi_chunk<KIND, true, 2, true>(a0, a1, sc, sh, sl, rv[u], p, c0f);
                        else if (has_res) o = act_mode ? epi_chunk<KIND, true, 3, false>(a0, a1, sc, sh, sl, rv[u], p, c0f)
                                                       : epi_chunk<KIND, true, 0, false>(a0, a1, sc, sh, sl, rv[u], p, c0f);
                        else o = act_mode ? epi_chunk<KIND, false, 3, false>(a0, a1, sc, sh, sl, rv[u], p, c0f)
                                          : epi_chunk<KIND, false, 0, false>(a0, a1, sc, sh, sl, rv[u], p, c0f);
                        *reinterpret_cast<uint4 *>(p.y + ((size_t)pm2 * p.out_ld + c0f) * 2) = o;
                    }
                }
                if (KIND != 2) mbar_arrive(bar_free);
            }
            if (KIND == 2 && alive && p.csum_out && valid) {
                if (p.n_tiles == 1) p.csum_out[pm] = (int)rowsum;
                else atomicAdd(p.csum_out + pm, (int)rowsum);  // several column tiles: the buffer was cleared before the launch
            }
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Split K, second launch: one thread per pixel and 8-channel chunk adds the partial sums of the splits in split order (the
// result does not depend on timing) and runs the floating-point epilogue of epi_chunk on the sum.
template <int KIND, bool HAS_RES>
__global__ void __launch_bounds__(256) splitk_finish_kernel(const ConvTcParams p)
{
    const int chunks = (p.Cout + 7) >> 3;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.P * chunks) return;
    const long pm = idx / chunks;
    const int c0 = (int)(idx - pm * chunks) * 8;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    for (int sp = 0; sp < p.splits; sp++) {
        const float4 *src = reinterpret_cast<const float4 *>(p.partial + ((size_t)sp * p.P + pm) * p.partial_ld + c0);
        const float4 t0 = src[0], t1 = src[1];
        a0.x += t0.x; a0.y += t0.y; a0.z += t0.z; a0.w += t0.w;
        a1.x += t1.x; a1.y += t1.y; a1.z += t1.z; a1.w += t1.w;
    }
    const float self = HAS_RES ? p.self_coef : 1.f;
    float sc[8], sh[8], sl[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        // (the per-channel arrays are padded to multiples of 64 floats: reading a chunk's eight is always in bounds)
        sc[i] = (p.scale ? p.scale[c0 + i] : 1.f) * self;
        sh[i] = (p.shift ? p.shift[c0 + i] : 0.f) * self;
        sl[i] = p.slope ? p.slope[c0 + i] : 0.f;
    }
    uint4 rv = make_uint4(0, 0, 0, 0);
    if (HAS_RES) rv = __ldg(reinterpret_cast<const uint4 *>(p.res + ((size_t)pm * p.res_ld + c0) * 2));
    const uint4 o = epi_chunk<KIND, HAS_RES, 2, true>(a0, a1, sc, sh, sl, rv, p, c0);
    *reinterpret_cast<uint4 *>(p.y + ((size_t)pm * p.out_ld + c0) * 2) = o;
}

// Diagnostic launcher switches (THB200_* environment variables), read ONCE: a launch costs no getenv call.
// thb_conv_reload_knobs() re-reads them (the tests change them between cases).  -1 = not set.
struct ConvKnobs {
    int pair_min_kb, u8_fast, reverse, epi_groups, epi_bufs, pdl, conv_l1, half_taps, a_tma, test_withhold;
    long pair_min_units;
    long long wait_limit;
};
ConvKnobs g_knobs;
bool g_knobs_read = false;
int env_int(const char *name, int unset)
{
    const char *e = getenv(name);
    return e ? atoi(e) : unset;
}
void read_knobs()
{
    g_knobs.pair_min_kb = env_int("THB200_PAIR_MIN_KB", -1);
    const char *u = getenv("THB200_PAIR_MIN_UNITS");
    g_knobs.pair_min_units = u ? atol(u) : -1;
    g_knobs.u8_fast = env_int("THB200_U8_FAST", 1);
    g_knobs.reverse = env_int("THB200_REVERSE", 1);
    g_knobs.epi_groups = env_int("THB200_EPI_GROUPS", -1);
    g_knobs.epi_bufs = env_int("THB200_EPI_BUFS", -1);
    g_knobs.pdl = env_int("THB200_PDL", 1);
    g_knobs.conv_l1 = env_int("THB200_CONV_L1", -1);
    g_knobs.half_taps = env_int("THB200_HALF_TAPS", -1);
    g_knobs.a_tma = env_int("THB200_A_TMA", -1);
    g_knobs.test_withhold = env_int("THB200_TEST_WITHHOLD", 0);
    const char *wl = getenv("THB200_WAIT_LIMIT_CYCLES");
    g_knobs.wait_limit = wl && atoll(wl) > 0 ? atoll(wl) : 4000000000ll;
    g_knobs_read = true;
}
const ConvKnobs &knobs()
{
    if (!g_knobs_read) read_knobs();
    return g_knobs;
}

int num_sms()
{
    static int n[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    return n[dev] > 0 ? n[dev] : 148;
}

struct ConvTmaps {
    const CUtensorMap *w, *a, *y, *r;  // weights, activation operand, output, residual (unused ones alias w)
};

template <int KIND, int BN, int STAGES>
int launch_tc(const ConvTmaps &tm, ConvTcParams p, cudaStream_t st)
{
    static bool configured[16] = {false};
    // (the split-K variant is a kernel of its own, so that the ordinary one carries none of its code)
    constexpr bool CAN_SPLIT = Smem<KIND, BN, STAGES>::TMA_EPI;
    auto kern_plain = conv_tc_kernel<KIND, BN, STAGES, false>;
    auto kern_split = conv_tc_kernel<KIND, BN, STAGES, CAN_SPLIT>;
    constexpr size_t smem = Smem<KIND, BN, STAGES>::TOTAL;
    static_assert(smem <= 232448, "shared memory plan exceeds the 227 KB a CTA can have");
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern_plain, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess && CAN_SPLIT) e = cudaFuncSetAttribute(kern_split, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return thb_note_launch(e, "conv_tc smem attribute");
        configured[dev] = true;
    }
    using L = Smem<KIND, BN, STAGES>;
    // Pair mode (see ConvTcParams::pair): narrow tiles with a K loop long enough to be bound by the MMA thread's barrier
    // rounds, and at least two units of work per SM.
    const ConvKnobs &kn = knobs();
    const int pair_min_kb = kn.pair_min_kb >= 0 ? kn.pair_min_kb : 1;
    const long pair_min_units = kn.pair_min_units >= 0 ? kn.pair_min_units : 2L * num_sms();  // (tests exercise the mode on small shapes)
    p.u8_classes = 0;
    if (KIND == 2) {
        const int fast_mode = kn.u8_fast;
        const int ncls = (1 + 2 * p.padH) * (1 + 2 * p.padW);
        if (fast_mode && p.wsat && p.padH < p.kH && p.padW < p.kW && ncls * L::TBL_ROW <= L::TBL_CAP) p.u8_classes = ncls;
        // a fused residual exists on the table-driven path only, and that path needs windows clipped on one side at most
        if (p.res && (!p.u8_classes || p.H < p.kH || p.W < p.kW)) return thb_note_launch(cudaErrorInvalidValue, "conv_tc: uint8 residual");
    }
    p.pair = L::TMA_EPI && p.a_tma && !p.half && BN <= 128 && p.nkb >= pair_min_kb && (long)(p.m_tiles / 2) * p.n_tiles >= pair_min_units;
    {
        // Every second convolution launch of a host thread walks its pixel tiles backwards: consecutive layers then
        // start on the end of the tensor the layer before has just written, which the L2 still holds (1.3 % of a
        // ResNet-50 forward).  THB200_REVERSE=0 switches it off, 2 reverses every launch.
        static thread_local unsigned flip = 0;
        const int rev_mode = kn.reverse;
        p.reverse = L::TMA_EPI && p.a_tma && (rev_mode == 1 ? (flip++ & 1) : rev_mode == 2);
    }
    if (p.splits > 1) {
        // split K needs both operands through TMA (the K block -> tap decoding of the producer), whole 128-byte taps, one
        // activation operand and the TMA epilogue's accumulator walk; otherwise the launch runs unsplit
        if (!L::TMA_EPI || !p.a_tma || p.half || p.nkb1 || p.nkb < 4 * p.splits) p.splits = 1;
        else p.pair = 0, p.reverse = 0;
    }
    const int tiles = (p.pair ? (p.m_tiles + 1) / 2 : p.m_tiles) * p.n_tiles * (p.splits > 1 ? p.splits : 1);  // units of work
    int grid = tiles < num_sms() ? tiles : num_sms();
    // uint8: an epilogue group rebuilds its correction table whenever its next tile has other channels; with a grid that is a
    // multiple of the column tiles every CTA stays on one column tile (148 -> 144 CTAs for 8 or 16 column tiles)
    if (KIND == 2 && p.u8_classes > 0 && p.n_tiles > 1 && tiles > grid && grid % p.n_tiles && grid > 2 * p.n_tiles && knobs().u8_fast != 2)
        grid -= grid % p.n_tiles;
    if (!L::TMA_EPI) {
        // staged epilogue: uint8 with nothing to gather runs a third group on warps 0-3 (a fourth accumulator exists below 256 columns)
        p.epi_groups = KIND == 2 && p.a_tma && BN < 256 ? 3 : 2;
        if (kn.epi_groups >= 0) p.epi_groups = kn.epi_groups == 3 && KIND == 2 && p.a_tma && BN < 256 ? 3 : 2;
    }
    if (L::TMA_EPI) {
        if (!tm.y || (p.res && !tm.r)) return thb_note_launch(cudaErrorUnknown, "conv_tc: output tensor map");
        // Shared memory is split between pipeline stages and the epilogue's 16 KB tiles (groups x tiles per group); which
        // split wins was measured per layer shape.  A single K block with 128 output channels per tile lives off its
        // epilogue: three groups (warps 0-3 join when they have nothing to gather) of two tiles.  One or two K blocks with
        // a residual, and a single K block on 64-channel tiles: two groups of three tiles, whose deeper ring keeps
        // residual loads and stores in flight.  Up to eight K blocks: two groups of two tiles.  Longer reductions live
        // off loads in flight: one tile per group, the rest in stages.
        const bool short_k = p.nkb <= 2;
        p.epi_groups = p.a_tma && BN >= 128 && BN < 256 && p.nkb == 1 && !p.res ? 3 : 2;
        if (kn.epi_groups >= 0) p.epi_groups = kn.epi_groups == 3 && p.a_tma && BN < 256 ? 3 : 2;
        p.epi_bufs = p.epi_groups == 3 ? 2 : ((short_k && p.res) || p.nkb == 1) && BN < 256 ? 3 : p.nkb <= 8 ? 2 : 1;
        if (kn.epi_bufs >= 0) p.epi_bufs = kn.epi_bufs < 1 ? 1 : kn.epi_bufs > 3 ? 3 : kn.epi_bufs;
        const size_t stage_bytes = L::STAGE_BYTES + (p.pair ? A_STAGE_BYTES : 0);
        const int min_stages = p.pair ? 2 : STAGES;
        while (min_stages * stage_bytes + (size_t)p.epi_groups * p.epi_bufs * EPI_TILE_BYTES > L::AVAIL) p.epi_bufs--;
        if (p.epi_bufs < 1) return thb_note_launch(cudaErrorUnknown, "conv_tc: shared-memory plan");
        p.stages = (int)((L::AVAIL - (size_t)p.epi_groups * p.epi_bufs * EPI_TILE_BYTES) / stage_bytes);
        if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
        if (!p.a_tma) p.stages = STAGES;  // the gather's cp.async depth is tied to the compile-time count
    }
    const int use_pdl = kn.pdl;
    p.pdl = use_pdl;
    p.wait_limit = kn.wait_limit;
    p.test_withhold = kn.test_withhold && p.a_tma;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, p.splits > 1 ? kern_split : kern_plain, *tm.w, *tm.a, tm.y ? *tm.y : *tm.w,
                                              tm.r ? *tm.r : *tm.w, p);
    const int rc = thb_note_launch(le != cudaSuccess ? le : cudaGetLastError(), "conv_tc_kernel");
    if (rc != THB_OK || p.splits <= 1) return rc;
    if constexpr (KIND != 2) {
        // the partial tiles of the splits -> the layer's output
        const long items = (long)p.P * ((p.Cout + 7) >> 3);
        const unsigned blocks = (unsigned)((items + 255) / 256);
        if (p.res) splitk_finish_kernel<KIND, true><<<blocks, 256, 0, st>>>(p);
        else splitk_finish_kernel<KIND, false><<<blocks, 256, 0, st>>>(p);
        return thb_note_launch(cudaGetLastError(), "splitk_finish_kernel");
    }
    return rc;
}

template <int KIND>
int dispatch_bn(int BN, const ConvTmaps &tm, const ConvTcParams &p, cudaStream_t st)
{
    switch (BN) {
    case 32: return launch_tc<KIND, 32, 6>(tm, p, st);
    case 64: return launch_tc<KIND, 64, 5>(tm, p, st);
    case 128: return launch_tc<KIND, 128, 4>(tm, p, st);
    case 256: return launch_tc<KIND, 256, 3>(tm, p, st);
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

typedef CUresult (*encode_im2col_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_im2col_fn get_encode_im2col_fn()
{
    static encode_im2col_fn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_im2col_fn>(sym);
    }
    return fn;
}

// TMA descriptors of plain row-major matrices [rows][cols] with a row pitch (activation operand of a 1x1
// convolution, output and residual tensors), keyed by what they encode and built once per buffer and shape.
struct MTmapEntry {
    const void *x;
    long rows;
    int cols, ld, dtype, box_cols;
    alignas(64) CUtensorMap map;
};
const CUtensorMap *matrix_tmap(const void *x, long rows, int cols, int ld, int dtype, int box_cols)
{
    static MTmapEntry cache[1024];
    static int used = 0, next = 0;
    for (int i = 0; i < used; i++) {
        MTmapEntry &e = cache[i];
        if (e.x == x && e.rows == rows && e.cols == cols && e.ld == ld && e.dtype == dtype && e.box_cols == box_cols) return &e.map;
    }
    encode_tiled_fn enc = get_encode_fn();
    if (!enc) return nullptr;
    MTmapEntry &e = cache[used < 1024 ? used++ : (next++ % 1024)];
    e.x = nullptr;
    const int es = dtype == THB_U8 ? 1 : 2;
    CUtensorMapDataType t = dtype == THB_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                            : dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * es};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)BM};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&e.map, t, 2, const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    e.x = x; e.rows = rows; e.cols = cols; e.ld = ld; e.dtype = dtype; e.box_cols = box_cols;
    return &e.map;
}

// TMA descriptors of activation operands, keyed by what they encode (built once per buffer and shape).
// mode 1: the plain [pixels][Cin] matrix of a 1x1 stride-1 convolution; mode 2: im2col over {C, W, H, N}.
struct ATmapEntry {
    const void *x;
    int mode, N, H, W, cin_pad, in_ld, dtype, geom[8];
    alignas(64) CUtensorMap map;
};
const CUtensorMap *activation_tmap(const thb_conv_desc *d, const void *x, int mode)
{
    if (mode == 1)
        return matrix_tmap(x, (long)d->N * d->H * d->W, d->Cin_pad, d->in_ld, d->dtype, d->dtype == THB_U8 ? 128 : 64);
    static ATmapEntry cache[512];
    static int used = 0, next = 0;
    const int geom[8] = {d->kH, d->kW, d->dH, d->dW, d->padH, mode == 3 ? d->in_row_pitch : d->padW, d->oH, d->oW};
    for (int i = 0; i < used; i++) {
        ATmapEntry &e = cache[i];
        if (e.x == x && e.mode == mode && e.N == d->N && e.H == d->H && e.W == d->W && e.cin_pad == d->Cin_pad &&
            e.in_ld == d->in_ld && e.dtype == d->dtype && (mode == 1 || !memcmp(e.geom, geom, sizeof(geom))))
            return &e.map;
    }
    ATmapEntry &e = cache[used < 512 ? used++ : (next++ % 512)];
    e.x = nullptr;
    const int es = d->dtype == THB_U8 ? 1 : 2;
    CUtensorMapDataType t = d->dtype == THB_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                            : d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    {
        encode_im2col_fn enc = get_encode_im2col_fn();
        if (!enc) return nullptr;
        // The bounding box that base pixels (tap (0,0) positions) live in: from -pad up to the position of the last
        // output pixel (dim + pad - (k - 1) for a full convolution), so that stepping by the convolution stride visits
        // exactly oW x oH positions per image.
        cuuint64_t dims[4] = {(cuuint64_t)d->Cin_pad, (cuuint64_t)d->W, (cuuint64_t)d->H, (cuuint64_t)d->N};
        cuuint64_t strides[3] = {(cuuint64_t)d->in_ld * es, (cuuint64_t)d->W * d->in_ld * es,
                                 (cuuint64_t)d->H * d->W * d->in_ld * es};
        int lower[2] = {-d->padW, -d->padH};
        int upper[2] = {(d->oW - 1) * d->dW + 1 - d->W - d->padW, (d->oH - 1) * d->dH + 1 - d->H - d->padH};
        if (mode == 3) {
            // Rows stored with their zero padding, kW taps = 128 bytes, stride 1: "pixel" w of this tensor is the
            // 128-byte window that starts at stored pixel w, i.e. the kW taps of output column w.  Windows overlap
            // (the pixel stride is smaller than the window), there are oW of them per row, and no horizontal
            // padding is left for the copy engine to supply.
            dims[0] = (cuuint64_t)(128 / es);
            dims[1] = (cuuint64_t)d->oW;
            strides[1] = (cuuint64_t)d->in_row_pitch * d->in_ld * es;
            strides[2] = (cuuint64_t)d->H * d->in_row_pitch * d->in_ld * es;
            lower[0] = 0;
            upper[0] = 0;
        }
        cuuint32_t estr[4] = {1, (cuuint32_t)d->dW, (cuuint32_t)d->dH, 1};
        // mode 4: a tap is 64 bytes of channels; the box is 64 bytes wide and lands as rows of 64 bytes with the 64-byte swizzle
        if (enc(&e.map, t, 4, const_cast<void *>(x), dims, strides, lower, upper, (cuuint32_t)((mode == 4 ? 64 : 128) / es),
                (cuuint32_t)BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                mode == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return nullptr;
        // Drivers up to CUDA 13.1 encode im2col descriptors of tensors smaller than 128 KiB with a flag (bit 21 of
        // the second 64-bit word) that makes the load misbehave; CUTLASS clears it for those drivers, and so do we.
        int drv = 0;
        if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
            (size_t)d->N * d->H * (mode == 3 ? d->in_row_pitch : d->W) * d->in_ld * es < 131072)
            reinterpret_cast<uint64_t *>(&e.map)[1] &= ~(1ull << 21);
    }
    e.x = x; e.mode = mode; e.N = d->N; e.H = d->H; e.W = d->W; e.cin_pad = d->Cin_pad; e.in_ld = d->in_ld; e.dtype = d->dtype;
    memcpy(e.geom, geom, sizeof(geom));
    return &e.map;
}

// Descriptor of the packed weights read in boxes 64 bytes wide (SWIZZLE_64B), for convolutions whose taps are 64 bytes.
struct WHalfEntry {
    const void *w;
    int ktot, cout_pad, bn, dtype;
    alignas(64) CUtensorMap map;
};
const CUtensorMap *weights_half_tmap(const thb_conv_desc *d)
{
    static WHalfEntry cache[256];
    static int used = 0, next = 0;
    for (int i = 0; i < used; i++) {
        WHalfEntry &e = cache[i];
        if (e.w == d->w && e.ktot == d->Ktot_pad && e.cout_pad == d->Cout_pad && e.bn == d->BN && e.dtype == d->dtype) return &e.map;
    }
    encode_tiled_fn enc = get_encode_fn();
    if (!enc) return nullptr;
    WHalfEntry &e = cache[used < 256 ? used++ : (next++ % 256)];
    e.w = nullptr;
    const int es = d->dtype == THB_U8 ? 1 : 2;
    CUtensorMapDataType t = d->dtype == THB_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                            : d->dtype == THB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {(cuuint64_t)d->Ktot_pad, (cuuint64_t)d->Cout_pad};
    cuuint64_t strides[1] = {(cuuint64_t)d->Ktot_pad * es};
    cuuint32_t box[2] = {(cuuint32_t)(64 / es), (cuuint32_t)d->BN};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&e.map, t, 2, const_cast<void *>(d->w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    e.w = d->w; e.ktot = d->Ktot_pad; e.cout_pad = d->Cout_pad; e.bn = d->BN; e.dtype = d->dtype;
    return &e.map;
}

}  // namespace

extern "C" void thb_simt_reload_knobs(void);
extern "C" void thb_conv_reload_knobs(void)
{
    read_knobs();
    thb_simt_reload_knobs();
}

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

// upper corner of the im2col bounding box: representable, and leaving a box of at least one position
static bool box_corner_ok(int upper, int dim_plus_pad) { return upper >= -128 && upper <= 127 && dim_plus_pad + upper >= 1; }

extern "C" int thb_conv_padded_rows_supported(int dtype)
{
    if (dtype != THB_F16 && dtype != THB_BF16 && dtype != THB_U8) return 0;
    static int ok[4] = {-1, -1, -1, -1};
    if (ok[dtype] < 0) {
        // encode a descriptor of the overlapping-window kind over a dummy address: only the encoder's checks matter
        if (cudaFree(0) != cudaSuccess) return 0;  // the encoder needs an initialised driver
        thb_conv_desc d;
        memset(&d, 0, sizeof(d));
        const int es = dtype == THB_U8 ? 1 : 2;
        d.dtype = dtype;
        d.N = 2; d.H = 8; d.W = 8; d.kH = d.kW = 4; d.dH = d.dW = 1; d.padH = d.padW = 2; d.oH = d.oW = 8;
        d.Cin_pad = d.in_ld = 32 / es;
        d.in_row_pitch = 12; d.in_pad_left = 2;
        ok[dtype] = activation_tmap(&d, reinterpret_cast<const void *>(uintptr_t(1) << 20), 3) != nullptr;
    }
    return ok[dtype];
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
    p.H = d->H; p.W = d->W; p.in_ld = d->in_ld; p.oH = d->oH; p.oW = d->oW; p.oHW = d->oH * d->oW;
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
    if (d->csum_out) {
        if (d->dtype != THB_U8) return THB_ERR_UNSUPPORTED;
        p.csum_out = d->csum_out;
    }
    if (d->dtype == THB_U8 && d->res) {
        const int ca = (int)d->self_coef, cb = (int)d->res_coef;
        if ((ca != 1 && ca != -1) || (cb != 1 && cb != -1) || (float)ca != d->self_coef || (float)cb != d->res_coef) return THB_ERR_UNSUPPORTED;
        const int twice = -(ca + cb - 1) * 255;  // floor(-(ca + cb - 1) * 127.5), as thb_u8_combine
        p.res_addend = twice >= 0 ? twice / 2 : -((-twice + 1) / 2);
    }
    p.tail_start = d->tail_start; p.relu_thr = d->relu_thr; p.relu_val = d->relu_val;
    p.acc_out = d->acc_out;
    if (d->splits > 1 && d->splitk_scratch && d->dtype != THB_U8 && !d->x2) {
        p.splits = d->splits > 8 ? 8 : d->splits;
        p.partial = d->splitk_scratch;
        p.partial_ld = d->Cout_pad;
    }
    p.use_l1 = d->kH * d->kW > 1;
    const ConvKnobs &kn = knobs();
    if (kn.conv_l1 >= 0) p.use_l1 = kn.conv_l1;
    p.status = d->status;
    if (!p.status) return THB_ERR_ARG;
    if (d->dtype == THB_U8 && (!p.wsat || !p.csum)) return THB_ERR_ARG;
    if (p.P <= 0) return THB_OK;
    p.m_tiles = (p.P + BM - 1) / BM;
    p.n_tiles = d->Cout_pad / d->BN;
    const CUtensorMap &tm = *reinterpret_cast<const CUtensorMap *>(d->tmap);
    const CUtensorMap *ta = &tm;
    // a 1x1 stride-1 unpadded convolution (and every Linear) reads a plain [pixels][Cin] matrix: TMA loads it
    p.a_tma = d->kH == 1 && d->kW == 1 && d->dH == 1 && d->dW == 1 && d->padH == 0 && d->padW == 0 &&
              d->oH == d->H && d->oW == d->W;
    // anything else whose taps are whole 128-byte channel slabs goes through im2col-mode TMA, within the limits of
    // a rank-4 descriptor: box corners in [-128, 127], traversal strides up to 8, tap offsets below 256
    const int bke = 128 / es;
    const bool im2col_ok = d->dH <= 8 && d->dW <= 8 && d->padH <= 127 && d->padW <= 127 &&
                           d->kH <= 256 && d->kW <= 256 && d->oH >= 1 && d->oW >= 1 &&
                           box_corner_ok((d->oH - 1) * d->dH + 1 - d->H - d->padH, d->H + d->padH) &&
                           box_corner_ok((d->oW - 1) * d->dW + 1 - d->W - d->padW, d->W + d->padW);
    if (!p.a_tma && im2col_ok && d->Cin_pad % bke == 0 && d->Ktot_pad == d->kH * d->kW * d->Cin_pad) p.a_tma = 2;
    // taps of 64 bytes (uint8 with 64 channels, 16-bit types with 32): half a K block; two taps per block, each as its own
    // 64-byte-wide copy
    p.ntaps = d->kH * d->kW;
    const bool half_ok = !p.a_tma && im2col_ok && d->Cin_pad * 2 == bke && !d->in_row_pitch &&
                         d->Ktot_pad == (p.ntaps * d->Cin_pad + bke - 1) / bke * bke;
    if (half_ok) p.a_tma = 2, p.half = 1;
    p.slabs = d->Cin_pad / bke;
    p.tma_kw = d->kW;
    p.tma_padw = d->padW;
    p.row_pitch = d->in_row_pitch ? d->in_row_pitch : d->W;
    p.pad_left = d->in_row_pitch ? d->in_pad_left : 0;
    int tmap_mode = p.a_tma;
    if (d->in_row_pitch) {
        // padded rows: the plain-matrix and per-tap descriptors do not describe this layout; the single-copy row
        // fetch does when a row's taps fill one 128-byte K block
        p.a_tma = 0;
        if (im2col_ok && d->dW == 1 && d->kW * d->Cin_pad == bke && d->Ktot_pad == d->kH * bke) {
            p.a_tma = 2;
            tmap_mode = 3;
            p.slabs = 1;
            p.tma_kw = 1;
            p.tma_padw = 0;
        }
    }
    if (p.half) {
        tmap_mode = 4;
        p.slabs = 1;
        if (kn.half_taps == 0) p.half = 0, p.a_tma = 0;
    }
    if (kn.a_tma >= 0) {
        const int allow = kn.a_tma;  // 0: gather only, 1: plain-matrix TMA only, 2 (default): im2col too
        if (p.a_tma > allow) p.a_tma = 0, p.half = 0;
        if (allow == 22 && p.a_tma == 1) p.a_tma = 2;  // experiment: im2col mode for a plain matrix too
    }
    if (p.a_tma) {
        ta = activation_tmap(d, x, tmap_mode);
        if (!ta) p.a_tma = 0, p.half = 0, ta = &tm;
    }
    ConvTmaps maps = {&tm, ta, nullptr, nullptr};
    if (p.half) {
        maps.w = weights_half_tmap(d);
        if (!maps.w) return thb_note_launch(cudaErrorUnknown, "conv_tc: weight tensor map");
    }
    if (d->dtype != THB_U8 && d->BN >= 64) {
        // output and residual go through TMA: [pixels][channels rounded up to 8] matrices with their own pitch
        const int c8 = (d->Cout + 7) & ~7;
        maps.y = matrix_tmap(y, p.P, c8, d->out_ld, d->dtype, 64);
        if (d->res) maps.r = matrix_tmap(d->res, p.P, c8, d->res_ld, d->dtype, 64);
        if (d->x2) {
            // second activation operand: its descriptor travels in the residual's slot (there is no residual then)
            const int cin2 = d->Cin - d->cin1;
            if (d->res || p.a_tma != 1 || d->in_row_pitch || d->cin1 <= 0 || d->cin1 % 64 || cin2 <= 0 || cin2 % 64 || d->x2_d < 1 ||
                d->x2_d > 8 || d->Cin_pad != d->Cin || (d->x2_H - 1) / d->x2_d + 1 != d->oH || (d->x2_W - 1) / d->x2_d + 1 != d->oW)
                return THB_ERR_UNSUPPORTED;
            p.nkb1 = d->cin1 / 64;
            p.a2_d = d->x2_d;
            maps.a = matrix_tmap(x, p.P, d->cin1, d->in_ld, d->dtype, 64);
            if (d->x2_d == 1) {
                p.a2_mode = 1;
                maps.r = matrix_tmap(d->x2, p.P, cin2, d->x2_ld, d->dtype, 64);
            } else {
                thb_conv_desc d2;
                memset(&d2, 0, sizeof(d2));
                d2.dtype = d->dtype;
                d2.N = d->N; d2.H = d->x2_H; d2.W = d->x2_W; d2.Cin = d2.Cin_pad = cin2; d2.in_ld = d->x2_ld;
                d2.kH = d2.kW = 1; d2.dH = d2.dW = d->x2_d; d2.oH = d->oH; d2.oW = d->oW;
                p.a2_mode = 2;
                maps.r = activation_tmap(&d2, d->x2, 2);
            }
            if (!maps.a || !maps.r) return thb_note_launch(cudaErrorUnknown, "conv_tc: second operand tensor map");
        }
    }
    if (d->x2 && !p.nkb1) return THB_ERR_UNSUPPORTED;  // (narrow tiles and uint8 have no second operand)
    cudaStream_t st = (cudaStream_t)s;
    switch (d->dtype) {
    case THB_F16: return dispatch_bn<0>(d->BN, maps, p, st);
    case THB_BF16: return dispatch_bn<1>(d->BN, maps, p, st);
    case THB_U8: return dispatch_bn<2>(d->BN, maps, p, st);
    }
    return THB_ERR_UNSUPPORTED;
}

// How many CTAs should share the K blocks of each tile of this convolution (1: no split), and the bytes of fp32 scratch
// that takes.  A launch of fewer tiles than SMs, or of a wave and a bit, leaves SMs idle for most of its duration: with
// the tiles' reductions cut in S parts the units fill the machine in ceil(tiles * S / SMs) rounds of 1/S the length.
// S minimises rounds / S plus a charge for the second launch's extra traffic; every part keeps at least four K blocks.
extern "C" int thb_conv_splitk_plan(const thb_conv_desc *d, size_t *scratch_bytes)
{
    if (scratch_bytes) *scratch_bytes = 0;
    static int off = -1;
    if (off < 0) {
        const char *e = getenv("THB200_NO_SPLITK");
        off = e && atoi(e) ? 1 : 0;
    }
    if (off || (d->dtype != THB_F16 && d->dtype != THB_BF16) || d->BN < 64 || d->x2 || d->csum_out) return 1;
    const long P = (long)d->N * d->oH * d->oW;
    const long tiles = ((P + BM - 1) / BM) * (d->Cout_pad / d->BN);
    const int nkb = d->Ktot_pad / 64, sms = num_sms();
    // (the partial tiles cost S x 8 bytes of traffic per output element: only launches that leave at least half the SMs
    // idle and whose whole scratch stays small gain from the split -- 100-200 tiles of a 14 x 14 layer at batch 64 do not)
    if (tiles <= 0 || 2 * tiles > sms || nkb < 8) return 1;
    int best = 1;
    double best_cost = (double)((tiles + sms - 1) / sms);
    for (int S = 2; S <= 8 && nkb / S >= 4; S++) {
        const double cost = (double)((tiles * S + sms - 1) / sms) / S + 0.04 * (S - 1);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = S; }
    }
    const size_t bytes = (size_t)best * P * d->Cout_pad * sizeof(float);
    if (best > 1 && bytes > ((size_t)16 << 20)) return 1;
    if (best > 1 && scratch_bytes) *scratch_bytes = bytes;
    return best;
}
