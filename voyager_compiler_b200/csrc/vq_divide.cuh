// fp32 division by a scale that many elements share, prepared once per scale.
#pragma once
#include <cstdint>

// x / s, correctly rounded, with the channel's scale prepared once (DivPlan):
//   * s a power of two with a normal inverse: x * (1 / s) is exact scaling;
//   * otherwise y = RN(1 / s), q = RN(x y), r = fma(-s, q, x), q' = fma(r, y, q): with a correctly
//     rounded reciprocal and a first quotient within one ulp the corrected quotient is the correctly
//     rounded one (Markstein's theorem), as long as nothing leaves the normal range: used for
//     2^-30 <= s <= 2^30 and 2^-60 <= |x| < 2^61; a zero keeps its sign through x * y;
//   * everything else: the IEEE division.
struct DivPlan {
    float s, y;
    int kind;      // 0 divide, 1 exact reciprocal, 2 corrected reciprocal
};
__device__ __forceinline__ DivPlan plan_division(float s) {
    DivPlan d;
    d.s = s;
    const uint32_t sb = __float_as_uint(s), ex = (sb >> 23) & 0xFFu;
    if ((sb & 0x807FFFFFu) == 0u && ex >= 2u && ex <= 252u) {
        d.y = __uint_as_float((254u - ex) << 23);
        d.kind = 1;
    } else if ((sb >> 31) == 0u && ex >= 97u && ex <= 157u) {
        d.y = __frcp_rn(s);
        d.kind = 2;
    } else {
        d.y = 0.0f;
        d.kind = 0;
    }
    return d;
}
__device__ __forceinline__ float divide(const DivPlan& d, float x) {
    if (d.kind == 1) return __fmul_rn(x, d.y);
    const uint32_t ax = __float_as_uint(x) & 0x7FFFFFFFu;
    if (d.kind == 2) {
        if (ax - 0x21800000u < 0x3D000000u) {           // exponent field 67 .. 188
            const float q = __fmul_rn(x, d.y);
            const float r = __fmaf_rn(-d.s, q, x);
            return __fmaf_rn(r, d.y, q);
        }
        if (ax == 0u) return __fmul_rn(x, d.y);
    }
    return __fdiv_rn(x, d.s);
}
