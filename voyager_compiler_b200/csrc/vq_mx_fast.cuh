// Compile-time specialised per-vector body of the fused MX scale + quantize kernels.
//
// The generic body (vq_mx_body.cuh) spends ~70 thread instructions per element, which makes the
// kernel issue bound at 15 % of the HBM roofline.  This body is specialised on dtype, scale rule,
// table kind and output set so that per element only these remain:
//   unpack, 1-3 multiply/FMA for x / scale, half a cvt.rn.bf16x2, one shared-memory lookup,
//   one pack op; per 16-byte vector: packed |x| maxima (max.u16x2 on bf16 pairs), the lane-group
//   shuffle reduction and the scale rule.
//
// x / scale without an IEEE division per element:
//   * scale is a power of two with a normal reciprocal: x * (1/scale) is the same correctly
//     rounded value (exact scaling).
//   * bf16 data, any scale: r = rcp.approx(scale), q0 = x*r, e = fma(-q0, scale, x),
//     q = fma(e, r, q0).  Operands have 8-bit significands, so the exact quotient is either
//     exactly representable (then q is exact: the residual e is exact and the correction lands on
//     it) or at least 2^-17 (relative) away from every bf16 rounding boundary, far more than the
//     ~2^-23 error of q; rounding q to bf16 therefore equals rounding the IEEE fp32 quotient to
//     bf16, which is what the CPU reference computes.  Used only when the scale comes straight
//     from the block maximum (so |q| stays bounded) and the scale and every non-zero element of
//     the vector are at least 2^-60 away from the subnormal range, so that e is computed exactly.
//   * everything else: __fdiv_rn.
#pragma once
#include "vq_mx_body.cuh"

namespace {

enum { OUT_FLOAT = 0, OUT_PACK4 = 1, OUT_PACK8 = 2 };
enum { TK_LUT = 0, TK_INT = 1 };

template <typename T>
struct Raw {
    uint32_t w[4];
    __device__ __forceinline__ void load_stream(const T* p) {
        uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
        w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    }
    __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0u; }
};

__device__ __forceinline__ uint32_t cvt_bf16x2(float hi, float lo) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float rcp_approx(float s) {
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(s));
    return r;
}

// per-thread |x| maximum of one raw vector as fp32 bits (bf16: pattern << 16), plus, for bf16,
// the smallest (|pattern| - 1) over the vector (0xFFFF for zeros) used by the safety test
template <typename T>
__device__ __forceinline__ uint32_t raw_amax(const Raw<T>& x, uint32_t& min_nz);
template <>
__device__ __forceinline__ uint32_t raw_amax<bf16_t>(const Raw<bf16_t>& x, uint32_t& min_nz) {
    uint32_t a0 = x.w[0] & 0x7FFF7FFFu, a1 = x.w[1] & 0x7FFF7FFFu, a2 = x.w[2] & 0x7FFF7FFFu, a3 = x.w[3] & 0x7FFF7FFFu;
    uint32_t m = __vmaxu2(__vmaxu2(a0, a1), __vmaxu2(a2, a3));
    uint32_t t = __vminu2(__vminu2(__vsub2(a0, 0x00010001u), __vsub2(a1, 0x00010001u)),
                          __vminu2(__vsub2(a2, 0x00010001u), __vsub2(a3, 0x00010001u)));
    min_nz = min(t & 0xFFFFu, t >> 16);
    return max(m & 0xFFFFu, m >> 16) << 16;
}
template <>
__device__ __forceinline__ uint32_t raw_amax<float>(const Raw<float>& x, uint32_t& min_nz) {
    min_nz = 0xFFFFu;
    return max(max(x.w[0] & 0x7FFFFFFFu, x.w[1] & 0x7FFFFFFFu), max(x.w[2] & 0x7FFFFFFFu, x.w[3] & 0x7FFFFFFFu));
}

template <typename T, int RULE>
__device__ __forceinline__ float fast_scale(const ScaleRule& r, uint32_t amax_bits) {
    if (amax_bits > 0x7F800000u) return 1.0f;
    if (RULE == 1) {
        if (amax_bits == 0x7F800000u) return __uint_as_float(0x7F800000u);
        uint32_t b = amax_bits ? amax_bits : 0x00800000u;
        int e = (b >= 0x00800000u) ? (int)(b >> 23) - 127 : (31 - __clz(b)) - 149;
        int i = e + 149;
        i += (b >= __ldg(r.bump_at + i)) ? 1 : 0;
        return __ldg(r.scale_of + i);
    }
    float a = __uint_as_float(amax_bits);
    float s = (r.qmax == 1.0f) ? a : Arith<T>::rnd(__fdiv_rn(a, r.qmax));
    if (r.stab.kind != VQ_TABLE_NONE) {
        uint32_t pat;
        s = table_value(r.stab, r.sres, s, pat);
    }
    return (s > 0.0f) ? s : 1.0f;
}

struct FastTab {
    const uint16_t* lut16;   // shared or global
    const uint8_t* lut8;
    float lo, hi;
    int lo_is_zero;
};

template <bool SM>
__device__ __forceinline__ uint32_t ld_u16(const uint16_t* base, uint32_t idx) {
    if (SM) {
        uint32_t v;
        uint32_t a = (uint32_t)__cvta_generic_to_shared(base) + idx * 2u;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
        return v;
    }
    return __ldg(base + idx);
}
template <bool SM>
__device__ __forceinline__ uint32_t ld_u8(const uint8_t* base, uint32_t idx) {
    if (SM) {
        uint32_t v;
        uint32_t a = (uint32_t)__cvta_generic_to_shared(base) + idx;
        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
        return v;
    }
    return __ldg(base + idx);
}

// clamp(rint(v)) of a bf16-representable value, NaN kept, -0 kept when lo == 0
__device__ __forceinline__ float int_round(const FastTab& t, float vb) {
    float q = rintf(vb);
    if (t.lo_is_zero) {
        q = (q < t.lo) ? t.lo : q;
        q = (q > t.hi) ? t.hi : q;
    } else {
        q = fminf(fmaxf(q, t.lo), t.hi);
    }
    return (vb != vb) ? vb : q;
}

// One 16-byte vector: quantize with block scale `s`, write the outputs of kind OUT at vector
// index `vi` of this tensor.
template <typename T, int TK, int OUT, bool SM>
__device__ __forceinline__ void fast_vector(const FastTab& t, const Raw<T>& x, float s, uint32_t min_nz,
                                            bool allow_refine, size_t vi, T* out_codes, uint8_t* codes8) {
    constexpr int N = sizeof(T) == 2 ? 8 : 4;
    float v[N];
    if (sizeof(T) == 2) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __uint_as_float(x.w[k] << 16);
            v[2 * k + 1] = __uint_as_float(x.w[k] & 0xFFFF0000u);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __uint_as_float(x.w[k]);
    }
    const uint32_t sb = __float_as_uint(s);
    const uint32_t ex = (sb >> 23) & 0xFFu;
    if ((sb & 0x807FFFFFu) == 0u && ex >= 2u && ex <= 252u) {
        const float r = __uint_as_float((254u - ex) << 23);
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = __fmul_rn(v[j], r);
    } else if (sizeof(T) == 2 && allow_refine && (sb >> 31) == 0u && ex >= 64u && ex <= 190u && min_nz >= 0x217Fu) {
        const float r = rcp_approx(s);
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float q0 = __fmul_rn(v[j], r);
            float e = __fmaf_rn(-q0, s, v[j]);
            v[j] = __fmaf_rn(e, r, q0);
        }
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = __fdiv_rn(v[j], s);
    }
    // bf16 patterns of the quotients, two per word (NaN -> 0x7FFF; the host only selects this
    // body for tables that give every NaN pattern the same output)
    uint32_t p2[N / 2];
#pragma unroll
    for (int k = 0; k < N / 2; ++k) p2[k] = cvt_bf16x2(v[2 * k + 1], v[2 * k]);

    if (OUT == OUT_FLOAT) {
        uint32_t o16[N];   // output bf16 patterns
#pragma unroll
        for (int k = 0; k < N / 2; ++k) {
            if (TK == TK_LUT) {
                o16[2 * k] = ld_u16<SM>(t.lut16, p2[k] & 0xFFFFu);
                o16[2 * k + 1] = ld_u16<SM>(t.lut16, p2[k] >> 16);
            } else {
                o16[2 * k] = __float_as_uint(int_round(t, __uint_as_float(p2[k] << 16))) >> 16;
                o16[2 * k + 1] = __float_as_uint(int_round(t, __uint_as_float(p2[k] & 0xFFFF0000u))) >> 16;
            }
        }
        if (sizeof(T) == 2) {
            uint4 o;
            o.x = o16[0] | (o16[1] << 16); o.y = o16[2] | (o16[3] << 16);
            o.z = o16[4 % N] | (o16[5 % N] << 16); o.w = o16[6 % N] | (o16[7 % N] << 16);
            __stcs(reinterpret_cast<uint4*>(out_codes + vi * N), o);
        } else {
            uint4 o = make_uint4(o16[0] << 16, o16[1] << 16, o16[2] << 16, o16[3] << 16);
            __stcs(reinterpret_cast<uint4*>(out_codes + vi * N), o);
        }
    } else {
        uint32_t c[N];
#pragma unroll
        for (int k = 0; k < N / 2; ++k) {
            if (TK == TK_LUT) {
                c[2 * k] = ld_u8<SM>(t.lut8, p2[k] & 0xFFFFu);
                c[2 * k + 1] = ld_u8<SM>(t.lut8, p2[k] >> 16);
            } else {
                float a = int_round(t, __uint_as_float(p2[k] << 16));
                float b = int_round(t, __uint_as_float(p2[k] & 0xFFFF0000u));
                c[2 * k] = (a != a) ? 0u : ((uint32_t)(int)a & 0xFFu);
                c[2 * k + 1] = (b != b) ? 0u : ((uint32_t)(int)b & 0xFFu);
            }
        }
        if (OUT == OUT_PACK4) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < N; ++j) w |= (c[j] & 0xFu) << (4 * j);
            if (N == 8) __stcs(reinterpret_cast<uint32_t*>(codes8 + vi * 4), w);
            else *reinterpret_cast<uint16_t*>(codes8 + vi * 2) = (uint16_t)w;
        } else {
            uint32_t* dst = reinterpret_cast<uint32_t*>(codes8 + vi * N);
#pragma unroll
            for (int k = 0; k < N / 4; ++k)
                __stcs(dst + k, c[4 * k] | (c[4 * k + 1] << 8) | (c[4 * k + 2] << 16) | (c[4 * k + 3] << 24));
        }
    }
}

}  // namespace
