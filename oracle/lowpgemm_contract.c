/*
 * The 8-bit GEMM behind the reference's "lowp" engine -- TEST INFRASTRUCTURE ONLY.
 *
 * PARITY UNPINNED at this boundary.  The reference calls
 * gemmlowp::eight_bit_int_gemm::EightBitIntGemm (A8B8 bit depth) from
 * lowp/gemm8.cc:4-17; gemmlowp is a third-party library that the reference does
 * not vendor and pins to no version (README.md:32, Makefile:33,173-178), and it is
 * not present on this machine.  This file restates that routine's published
 * contract in our own code:
 *
 *   acc(i,j) = sum_k (A(i,k) + a_offset) * (B(k,j) + b_offset)            (int32)
 *   C(i,j)   = saturate_u8( ((acc + c_offset) * c_mult + round) >> c_shift )
 *   round    = c_shift < 1 ? 0 : 1 << (c_shift - 1)
 *
 * with 32-bit wrap-around arithmetic and an arithmetic right shift.  The reference
 * has no test or golden vector at this boundary, so the contract is an assumption;
 * everything around it (parameter derivation, im2col, bias add, pooling, ReLU) is
 * checked against the reference's own lowp sources built on top of this function.
 *
 * Signature = the reference's lowpgemm (lowp/lowp_basic.c:289-297).  The three
 * "transposed" flags select row-major storage (flag 1) or column-major (flag 0).
 */
#include <stdint.h>
#include "oracle.h"

unsigned char orc_lowp_requant(int acc, int c_offset, int c_mult, int c_shift)
{
    uint32_t v = ((uint32_t)acc + (uint32_t)c_offset) * (uint32_t)c_mult;
    if (c_shift >= 1) v += (uint32_t)1 << (c_shift - 1);
    int32_t s = (int32_t)v;
    if (c_shift > 0) s = s >> (c_shift > 31 ? 31 : c_shift); /* arithmetic shift on two's complement */
    return s < 0 ? 0 : s > 255 ? 255 : (unsigned char)s;
}

void lowpgemm(const int is_a_transposed, const int is_b_transposed, const int is_c_transposed,
              const int m, const int n, const int k, const unsigned char *a, const unsigned char *b,
              unsigned char *c, const int lda, const int ldb, const int ldc, const int a_offset,
              const int b_offset, const int c_offset, const int c_mult, const int c_shift)
{
#pragma omp parallel for
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            uint32_t acc = 0;
            for (int l = 0; l < k; l++) {
                int av = is_a_transposed ? a[(long)i * lda + l] : a[(long)l * lda + i];
                int bv = is_b_transposed ? b[(long)l * ldb + j] : b[(long)j * ldb + l];
                acc += (uint32_t)((av + a_offset) * (bv + b_offset));
            }
            unsigned char r = orc_lowp_requant((int32_t)acc, c_offset, c_mult, c_shift);
            if (is_c_transposed) c[(long)i * ldc + j] = r;
            else c[(long)j * ldc + i] = r;
        }
}
