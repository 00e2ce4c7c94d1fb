// Compile-time specialised per-chunk body of the fused MX scale + quantize kernels.
//
// The generic body (vq_mx_body.cuh) spends ~70 thread instructions per element, which makes the
// kernel issue bound at 15 % of the HBM roofline.  Here each thread owns a 32-byte chunk (16 bf16 /
// 8 fp32, one 256-bit load) and the code is specialised on dtype, scale rule, table kind and
// output set, so that per element only these remain: unpack, 1-3 multiply/FMA for x / scale, one
// cvt.rn.bf16 (pattern lands zero-extended in a register, ready to be a shared-memory offset),
// one shared-memory lookup, one multiply-add to pack; per 32-bit word three SIMD integer ops for
// the |x| extrema; per chunk the lane-group shuffle reduction and the scale rule.
//
// x / scale without an IEEE division per element:
//   * scale is a power of two with a normal reciprocal: x * (1/scale) is the same correctly
//     rounded value (exact scaling).
//   * bf16 data, any scale: q = x * rcp.approx(scale).  Both operands have significands of at
//     most 8 bits, x = mx * 2^a and scale = ms * 2^b with mx, ms <= 255.  A bf16 rounding boundary
//     is an odd multiple (2k+1) >= 257 of half an ulp; mx * 2^j * 256 = (2k+1) * ms has no solution
//     (the odd part of the right side exceeds 255), and since both sides are integers the exact
//     quotient stays at least 1 / (256 * ms) > 2^-17 (relative) away from every boundary, the
//     overflow boundary included.  q carries a relative error below 2^-22 (rcp.approx is within one
//     ulp), so rounding q to bf16 equals rounding the IEEE fp32 quotient to bf16, which is what the
//     CPU reference computes.  The argument needs q to be a normal number: the path is taken when
//     the scale lies in [2^-63, 2^63] and either the table cannot tell apart quotients below 2^-119
//     (`flat_tiny`) or no non-zero element of the chunk lies below 2^-60.
//   * everything else: __fdiv_rn.
#pragma once
#include "vq_mx_body.cuh"

namespace {

enum { OUT_FLOAT = 0, OUT_PACK4 = 1, OUT_PACK8 = 2, OUT_SCALE = 3, OUT_FAKEQ = 4 };
// OUT_SCALE: block scales only.  OUT_FAKEQ: the quantized value times the scale (quantize + dequantize).
enum { TK_LUT = 0, TK_INT = 1 };

// 32 bytes of input as raw words
struct Chunk {
    uint32_t w[8];
    __device__ __forceinline__ void load(const void* p) {
        asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                     : "l"(p));
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = 0u;
    }
};

__device__ __forceinline__ void store32(void* p, const uint32_t* o) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                 "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
}

// bf16 pattern of v, zero-extended (NaN -> 0x7FFF)
__device__ __forceinline__ uint32_t bf16_pattern(float v) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(0.0f), "f"(v));
    return d;
}
__device__ __forceinline__ float rcp_approx(float s) {
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(s));
    return r;
}

// {a, b} *= r as one packed fp32x2 multiply (two correctly rounded IEEE products, one issue slot).
__device__ __forceinline__ void mul2(float& a, float& b, float r) {
    asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %2};\n\tmul.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
        : "+f"(a), "+f"(b)
        : "f"(r));
}
// {d0, d1} = {a0, a1} * b + {c0, c1}: two fused multiply-adds, each rounded once, one issue slot.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c0, float c1) {
    asm("{\n\t.reg .b64 a, b, c;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tmov.b64 c, {%5, %6};\n\t"
        "fma.rn.f32x2 a, a, b, c;\n\tmov.b64 {%0, %1}, a;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c0), "f"(c1));
}

// |x| maximum of a chunk as fp32 bits.  For bf16 also whether the reciprocal path is safe for this
// chunk: no non-zero element below 2^-60 (pattern 0x2180).
template <typename T>
__device__ __forceinline__ uint32_t chunk_amax(const Chunk& x, bool& safe, bool need_safe);
// max(|a|, |b|) / min(|a|, |b|) per bf16 half; the sign bit of the result is garbage (xor of the
// input signs) and is masked off at the end.  .NaN: a NaN input gives NaN (0x7FFF), as torch.max.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t absmin_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("min.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

template <>
__device__ __forceinline__ uint32_t chunk_amax<bf16_t>(const Chunk& x, bool& safe, bool need_safe) {
    const uint32_t* w = x.w;
    uint32_t mx = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(w[0], w[1]), absmax_bf16x2(w[2], w[3])),
                                absmax_bf16x2(absmax_bf16x2(w[4], w[5]), absmax_bf16x2(w[6], w[7])));
    mx &= 0x7FFF7FFFu;
    safe = true;
    if (!need_safe) return max(mx & 0xFFFFu, mx >> 16) << 16;
    uint32_t mn = absmin_bf16x2(absmin_bf16x2(absmin_bf16x2(w[0], w[1]), absmin_bf16x2(w[2], w[3])),
                                absmin_bf16x2(absmin_bf16x2(w[4], w[5]), absmin_bf16x2(w[6], w[7])));
    mn &= 0x7FFF7FFFu;
    // smallest magnitude at least 2^-60 (pattern 0x2180): the reciprocal path is exact.  A NaN makes
    // the minimum unreliable, but then the block scale is 1 (a power of two) and the path is unused.
    safe = min(mn & 0xFFFFu, mn >> 16) >= 0x2180u;
    if (!safe) {
        // zeros are harmless: look at the smallest NON-zero magnitude (0 - 1 wraps to 0xFFFF)
        uint32_t t = 0xFFFFFFFFu;
#pragma unroll
        for (int k = 0; k < 8; ++k) t = __vminu2(t, __vsub2(w[k] & 0x7FFF7FFFu, 0x00010001u));
        safe = min(t & 0xFFFFu, t >> 16) >= 0x217Fu;
    }
    return max(mx & 0xFFFFu, mx >> 16) << 16;
}
template <>
__device__ __forceinline__ uint32_t chunk_amax<float>(const Chunk& x, bool& safe, bool) {
    safe = false;
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) m = max(m, x.w[k] & 0x7FFFFFFFu);
    return m;
}

// RULE 0: amax / quant_max (optionally through a scale table); 1: power of two; 2: quant_max is 1 and
// there is no scale table, so the scale is the block maximum itself (1 where that is 0 or NaN).
template <typename T, int RULE>
__device__ __forceinline__ float fast_scale(const ScaleRule& r, uint32_t amax_bits) {
    if (RULE == 2) {
        const float a = __uint_as_float(amax_bits);
        return (a > 0.0f) ? a : 1.0f;                   // NaN compares false
    }
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
    int flat_tiny;           // quotients below 2^-119 all give the same output: no scan for tiny elements
};

template <bool SM>
__device__ __forceinline__ uint32_t ld_u16(const uint16_t* base, uint32_t idx) {
    if (SM) {
        uint32_t v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(base) + idx * 2u));
        return v;
    }
    return __ldg(base + idx);
}
template <bool SM>
__device__ __forceinline__ uint32_t ld_u8(const uint8_t* base, uint32_t idx) {
    if (SM) {
        uint32_t v;
        asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(base) + idx));
        return v;
    }
    return __ldg(base + idx);
}
// The same reads for a table that sits at the very start of the kernel's dynamic shared memory:
// `stab` is that array itself, so the compiler addresses the table as symbol + index and the byte
// offset of the table costs no instruction.
template <bool SM>
__device__ __forceinline__ uint32_t tab_u16(const uint16_t* stab, const uint16_t* gtab, uint32_t idx) {
    return SM ? (uint32_t)stab[idx] : (uint32_t)__ldg(gtab + idx);
}
template <bool SM>
__device__ __forceinline__ uint32_t tab_u8(const uint8_t* stab, const uint8_t* gtab, uint32_t idx) {
    return SM ? (uint32_t)stab[idx] : (uint32_t)__ldg(gtab + idx);
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

// One 32-byte chunk: quantize with block scale `s`, write outputs of kind OUT at chunk index `ci`
// of this tensor (element offset ci * N).
template <typename T, int TK, int OUT, bool SM>
__device__ __forceinline__ void fast_chunk(const FastTab& t, const void* stab, const Chunk& x, float s, bool refine_ok, size_t ci,
                                           T* out_codes, uint8_t* codes8) {
    const uint16_t* s16 = reinterpret_cast<const uint16_t*>(stab);
    const uint8_t* s8 = reinterpret_cast<const uint8_t*>(stab);
    constexpr int N = sizeof(T) == 2 ? 16 : 8;
    float v[N];
    if (sizeof(T) == 2) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            v[(2 * k) % N] = __uint_as_float(x.w[k] << 16);
            v[(2 * k + 1) % N] = __uint_as_float(x.w[k] & 0xFFFF0000u);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(x.w[k]);
    }
    const uint32_t sb = __float_as_uint(s);
    const uint32_t ex = (sb >> 23) & 0xFFu;
    // bf16 data, positive scale in [2^-63, 2^63], no tiny element: one reciprocal multiply (see the
    // header; a power-of-two scale is just a special case of it).  sb - 2^-63 < 2^63 - 2^-63 as
    // unsigned integers is that range test (a negative scale wraps to the top).
    if (sizeof(T) == 2 && refine_ok && sb - 0x20000000u < 0x3F800000u) {
        const float r = rcp_approx(s);
#pragma unroll
        for (int j = 0; j < N; j += 2) mul2(v[j], v[j + 1], r);
    } else if ((sb & 0x807FFFFFu) == 0u && ex >= 2u && ex <= 252u) {
        const float r = __uint_as_float((254u - ex) << 23);
#pragma unroll
        for (int j = 0; j < N; j += 2) mul2(v[j], v[j + 1], r);
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = __fdiv_rn(v[j], s);
    }
    // bf16 pattern of every quotient (NaN -> 0x7FFF; the host only selects this body for tables
    // that give every NaN pattern the same output)
    uint32_t p[N];
#pragma unroll
    for (int j = 0; j < N; ++j) p[j] = bf16_pattern(v[j]);

    if (OUT == OUT_FLOAT || OUT == OUT_FAKEQ) {
        uint32_t o[8];
        if (sizeof(T) == 2) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                uint32_t a, b;
                if (TK == TK_LUT) {
                    a = tab_u16<SM>(s16, t.lut16, p[(2 * k) % N]);
                    b = tab_u16<SM>(s16, t.lut16, p[(2 * k + 1) % N]);
                } else {
                    a = __float_as_uint(int_round(t, __uint_as_float(p[(2 * k) % N] << 16))) >> 16;
                    b = __float_as_uint(int_round(t, __uint_as_float(p[(2 * k + 1) % N] << 16))) >> 16;
                }
                o[k] = b * 65536u + a;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (TK == TK_LUT) o[k] = tab_u16<SM>(s16, t.lut16, p[k]) << 16;
                else o[k] = __float_as_uint(int_round(t, __uint_as_float(p[k] << 16)));
            }
        }
        if (OUT == OUT_FAKEQ) {
            if (sizeof(T) == 2) {
                const uint32_t s2 = (__float_as_uint(s) >> 16) * 0x00010001u;
#pragma unroll
                for (int k = 0; k < 8; ++k) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[k]) : "r"(o[k]), "r"(s2));
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __float_as_uint(__fmul_rn(__uint_as_float(o[k]), s));
            }
        }
        store32(out_codes + ci * N, o);
    } else {
        uint32_t c[N];
#pragma unroll
        for (int j = 0; j < N; ++j) {
            if (TK == TK_LUT) {
                c[j] = tab_u8<SM>(s8, t.lut8, p[j]);
            } else {
                float a = int_round(t, __uint_as_float(p[j] << 16));
                c[j] = (a != a) ? 0u : ((uint32_t)(int)a & (OUT == OUT_PACK4 ? 0xFu : 0xFFu));
            }
        }
        if (OUT == OUT_PACK4) {
            // LUT codes of a <=16-level table are < 16 already
            uint32_t w[N / 8];
#pragma unroll
            for (int g = 0; g < N / 8; ++g) {
                uint32_t acc = c[8 * g];
#pragma unroll
                for (int j = 1; j < 8; ++j) acc = c[8 * g + j] * (1u << (4 * j)) + acc;
                w[g] = acc;
            }
            if (N == 16) __stcs(reinterpret_cast<uint2*>(codes8 + ci * 8), make_uint2(w[0], w[(N / 8) - 1]));
            else __stcs(reinterpret_cast<uint32_t*>(codes8 + ci * 4), w[0]);
        } else {
            uint32_t w[N / 4];
#pragma unroll
            for (int g = 0; g < N / 4; ++g)
                w[g] = ((c[4 * g + 3] * 256u + c[4 * g + 2]) * 256u + c[4 * g + 1]) * 256u + c[4 * g];
            if (N == 16) __stcs(reinterpret_cast<uint4*>(codes8 + ci * 16), make_uint4(w[0], w[1], w[2 % (N / 4)], w[3 % (N / 4)]));
            else __stcs(reinterpret_cast<uint2*>(codes8 + ci * 8), make_uint2(w[0], w[1]));
        }
    }
}

}  // namespace
