// Group-wise affine fake-quantize: GroupWiseAffineFakeQuantFunction.forward,
// src/voyager_compiler/quantization/fake_quantize.py:160-207, for blocks along the last (contiguous) axis.
//
//   min, max over each block (the zero padding of a ragged last block takes part, mx_utils.py:81-101;
//   a NaN in the block makes both NaN, as torch.amin / torch.amax do)
//   sf = (max - min) / (quant_max - quant_min);  sf = sf > 0 ? sf : 1
//   zp = -min / sf + quant_min;  optionally both through the scale table (vmap)
//   q  = clamp(round_half_even(x / sf + zp), quant_min, quant_max);  out = (q - zp) * sf
//
// Every operation is the IEEE operation upstream's expression performs, rounded to the tensor dtype after
// each step for bf16.  One launch: a group of G lanes takes a block, sweeps it once for the extrema and once
// (from L1/L2) for the values; HBM sees sizeof(T) read + sizeof(T) written per element plus two numbers per block.
//
// Blocks of exactly four 16-byte pieces per lane (block sizes 32 ... 512 that divide the row) take
// group_affine_held_kernel: the block stays in registers between the two sweeps, two elements go through every
// rounding, addition and multiplication together (cvt.rn.bf16x2, fma.rn.f32x2), the clamp is min.NaN / max.NaN,
// and x / sf is a multiplication wherever that gives the same rounded quotient:
//   * fp32: the corrected reciprocal of vq_divide.cuh (checked per element);
//   * bf16: x * rcp.approx(sf) rounded to bf16.  x and sf carry 8-bit significands, so the exact quotient stays at
//     least 2^-17 (relative) away from every bf16 rounding boundary while the product is within 2^-22 of it (the
//     argument at the top of vq_mx_fast.cuh); it needs a normal quotient: 2^-63 <= sf <= 2^63 and |x| >= 2^-60 or zero.
#include "vq_common.cuh"
#include "vq_divide.cuh"
#include <cstdlib>
#include <cstring>

namespace {

struct GroupAffineParams {
    const void* in;
    void* out;
    void* scale;
    void* zero_point;
    const uint16_t* table;     // optional 65 536-entry bf16 table for scale and zero point
    int64_t rows, K, n_blocks; // n_blocks = rows * blocks_per_row
    int block, blocks_per_row;
    int lanes;                 // lanes per block: a power of two <= 32
    int vec;                   // 16-byte accesses
    float qmin, qmax, qrange;  // qrange = float(quant_max - quant_min)
};

// Rounding to the tensor dtype after every operation; bf16 by the hardware conversion (round to nearest even; a NaN
// stays a NaN, whose payload nothing downstream reads).
template <typename T>
__device__ __forceinline__ float rnd(float v);
template <>
__device__ __forceinline__ float rnd<float>(float v) { return v; }
template <>
__device__ __forceinline__ float rnd<bf16_t>(float v) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(0.0f), "f"(v));
    return __uint_as_float(d << 16);
}

template <typename T>
__device__ __forceinline__ float through_table(const uint16_t* table, float v) {
    return table ? bf16_bits_to_f32(__ldg(table + f32_to_bf16_bits(v))) : v;
}

template <typename T>
__device__ __forceinline__ float fake_quant_one(float x, float sf, float zp, float lo, float hi) {
    float t = rnd<T>(__fdiv_rn(x, sf));
    t = rnd<T>(__fadd_rn(t, zp));
    float r = rintf(t);
    r = (r < lo) ? lo : r;             // comparisons keep a NaN, as torch.clamp does
    r = (r > hi) ? hi : r;
    return rnd<T>(__fmul_rn(rnd<T>(__fsub_rn(r, zp)), sf));
}

template <typename T>
__global__ void __launch_bounds__(256) group_affine_kernel(const GroupAffineParams p) {
    constexpr int V = Vec<T>::N;
    const T* x = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    const int G = p.lanes;
    const int lane = threadIdx.x & 31, sub = lane & (G - 1);
    const uint32_t gmask = (G == 32) ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int64_t groups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int64_t rounds = (p.n_blocks + groups - 1) / groups;
    const int64_t g0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const float lo = rnd<T>(p.qmin), hi = rnd<T>(p.qmax);      // clamp bounds in the tensor dtype
    for (int64_t r = 0; r < rounds; ++r) {               // all lanes of a warp stay in the loop together
        const int64_t b = g0 + r * groups;
        const bool live = b < p.n_blocks;
        const int64_t row = live ? b / p.blocks_per_row : 0;
        const int kb = live ? (int)(b - row * p.blocks_per_row) : 0;
        const int64_t base = row * p.K + (int64_t)kb * p.block;
        const int len = live ? (int)min((int64_t)p.block, p.K - (int64_t)kb * p.block) : 0;
        float mn = __uint_as_float(0x7F800000u), mx = __uint_as_float(0xFF800000u);
        bool nan = false;
        if (p.vec) {
#pragma unroll 4
            for (int c = sub * V; c < len; c += G * V) {
                Vec<T> v;
                v.load(x + base + c);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    nan |= v.v[j] != v.v[j];
                    mn = fminf(mn, v.v[j]);
                    mx = fmaxf(mx, v.v[j]);
                }
            }
        } else {
            for (int c = sub; c < len; c += G) {
                const float e = load_one<T>(x + base + c);
                nan |= e != e;
                mn = fminf(mn, e);
                mx = fmaxf(mx, e);
            }
        }
        if (len < p.block) {               // zero padding of a ragged block
            mn = fminf(mn, 0.0f);
            mx = fmaxf(mx, 0.0f);
        }
        for (int o = G >> 1; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(gmask, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, o));
            nan |= (__shfl_xor_sync(gmask, nan ? 1 : 0, o) != 0);
        }
        if (nan) mn = mx = __uint_as_float(0x7FC00000u);
        // -0 and +0 compare equal in fminf/fmaxf, and only enter the results through max - min and -min / sf,
        // where the sign of a zero extremum cannot change a finite non-zero outcome; a zero range gives sf = 1.
        float sf = rnd<T>(__fdiv_rn(rnd<T>(__fsub_rn(mx, mn)), p.qrange));
        sf = (sf > 0.0f) ? sf : 1.0f;
        float zp = rnd<T>(__fadd_rn(rnd<T>(__fdiv_rn(-mn, sf)), p.qmin));
        sf = through_table<T>(p.table, sf);
        zp = through_table<T>(p.table, zp);
        if (live && sub == 0) {
            store_one<T>(reinterpret_cast<T*>(p.scale) + b, sf);
            store_one<T>(reinterpret_cast<T*>(p.zero_point) + b, zp);
        }
        if (p.vec) {
#pragma unroll 4
            for (int c = sub * V; c < len; c += G * V) {
                Vec<T> v;
                v.load(x + base + c);
#pragma unroll
                for (int j = 0; j < V; ++j) v.v[j] = fake_quant_one<T>(v.v[j], sf, zp, lo, hi);
                v.store(out + base + c);
            }
        } else {
            for (int c = sub; c < len; c += G) store_one<T>(out + base + c, fake_quant_one<T>(load_one<T>(x + base + c), sf, zp, lo, hi));
        }
    }
}

__device__ __forceinline__ float min_nan(float a, float b) {
    float d;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float max_nan(float a, float b) {
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
// {a, b} = {a, b} * m + c as one packed fp32x2 operation (two correctly rounded results)
__device__ __forceinline__ void fma_pair(float& a, float& b, float m, float c) {
    asm("{\n\t.reg .b64 x, y, z;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %2};\n\tmov.b64 z, {%3, %3};\n\t"
        "fma.rn.f32x2 x, x, y, z;\n\tmov.b64 {%0, %1}, x;\n\t}"
        : "+f"(a), "+f"(b)
        : "f"(m), "f"(c));
}
__device__ __forceinline__ void mul_pair(float& a, float& b, float m) {
    asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %2};\n\tmul.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
        : "+f"(a), "+f"(b)
        : "f"(m));
}
// both values rounded to the tensor dtype; `packed` receives the two bf16 patterns (a low, b high)
template <typename T>
__device__ __forceinline__ void rnd_pair(float& a, float& b, uint32_t& packed);
template <>
__device__ __forceinline__ void rnd_pair<float>(float&, float&, uint32_t&) {}
template <>
__device__ __forceinline__ void rnd_pair<bf16_t>(float& a, float& b, uint32_t& packed) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(b), "f"(a));
    a = __uint_as_float(packed << 16);
    b = __uint_as_float(packed & 0xFFFF0000u);
}

// x / sf for all elements of a block, prepared once
template <typename T>
struct BlockQuotient;
template <>
struct BlockQuotient<float> {
    DivPlan d;
    __device__ __forceinline__ explicit BlockQuotient(float sf) : d(plan_division(sf)) {}
    __device__ __forceinline__ void pair(float& a, float& b) const {
        a = divide(d, a);
        b = divide(d, b);
    }
};
template <>
struct BlockQuotient<bf16_t> {
    float sf, y;
    bool mul;
    __device__ __forceinline__ explicit BlockQuotient(float s) : sf(s) {
        const uint32_t sb = __float_as_uint(s), ex = (sb >> 23) & 0xFFu;
        mul = (sb >> 31) == 0u && ex >= 64u && ex <= 190u;
        asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(s));
    }
    // the caller rounds the results to bf16
    __device__ __forceinline__ void pair(float& a, float& b) const {
        const uint32_t aa = __float_as_uint(a) & 0x7FFFFFFFu, ab = __float_as_uint(b) & 0x7FFFFFFFu;
        // zero, or at least 2^-60 (a NaN or an infinity gives the same through the product)
        if (mul && (aa - 1u) >= 0x217FFFFFu && (ab - 1u) >= 0x217FFFFFu) {
            mul_pair(a, b, y);
        } else {
            a = __fdiv_rn(a, sf);
            b = __fdiv_rn(b, sf);
        }
    }
};

// Blocks of exactly 4 * G 16-byte pieces, K a multiple of the block: see the head of the file.
template <typename T>
__global__ void __launch_bounds__(256, sizeof(T) == 4 ? 4 : 2) group_affine_held_kernel(const GroupAffineParams p) {
    constexpr int V = Vec<T>::N;
    const T* x = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    const int G = p.lanes;
    const int lane = threadIdx.x & 31, sub = lane & (G - 1);
    const uint32_t gmask = (G == 32) ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int64_t groups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int64_t rounds = (p.n_blocks + groups - 1) / groups;
    const int64_t g0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const float lo = rnd<T>(p.qmin), hi = rnd<T>(p.qmax);
    for (int64_t r = 0; r < rounds; ++r) {               // all lanes of a warp stay in the loop together
        const int64_t b = g0 + r * groups;
        const bool live = b < p.n_blocks;
        const T* src = x + (live ? b : 0) * (int64_t)p.block + sub * V;     // rows are whole blocks: block b starts at b * block
        Vec<T> v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k].load_stream(src + k * G * V);
        float mn = v[0].v[0], mx = v[0].v[0];
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int j = 0; j < V; ++j) {
                mn = min_nan(mn, v[k].v[j]);
                mx = max_nan(mx, v[k].v[j]);
            }
        for (int o = G >> 1; o > 0; o >>= 1) {
            mn = min_nan(mn, __shfl_xor_sync(gmask, mn, o));
            mx = max_nan(mx, __shfl_xor_sync(gmask, mx, o));
        }
        if (mn != mn || mx != mx) mn = mx = __uint_as_float(0x7FC00000u);
        float sf = rnd<T>(__fdiv_rn(rnd<T>(__fsub_rn(mx, mn)), p.qrange));
        sf = (sf > 0.0f) ? sf : 1.0f;
        float zp = rnd<T>(__fadd_rn(rnd<T>(__fdiv_rn(-mn, sf)), p.qmin));
        sf = through_table<T>(p.table, sf);
        zp = through_table<T>(p.table, zp);
        if (live && sub == 0) {
            store_one<T>(reinterpret_cast<T*>(p.scale) + b, sf);
            store_one<T>(reinterpret_cast<T*>(p.zero_point) + b, zp);
        }
        const BlockQuotient<T> quot(sf);
        const float nzp = -zp;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t w[V / 2];
#pragma unroll
            for (int j = 0; j < V; j += 2) {
                float a = v[k].v[j], c = v[k].v[j + 1];
                uint32_t& pk = w[j / 2];
                quot.pair(a, c);
                rnd_pair<T>(a, c, pk);
                fma_pair(a, c, 1.0f, zp);                  // t + zp (the product with one is exact)
                rnd_pair<T>(a, c, pk);
                a = rintf(a);
                c = rintf(c);
                a = (a < lo) ? lo : a;                     // comparisons keep a NaN and the sign of a zero, as torch.clamp does
                c = (c < lo) ? lo : c;
                a = (a > hi) ? hi : a;
                c = (c > hi) ? hi : c;
                fma_pair(a, c, 1.0f, nzp);                 // q - zp
                rnd_pair<T>(a, c, pk);
                mul_pair(a, c, sf);
                rnd_pair<T>(a, c, pk);
                v[k].v[j] = a;
                v[k].v[j + 1] = c;
            }
            if (live) {
                T* dst = out + b * (int64_t)p.block + sub * V + k * G * V;
                if (sizeof(T) == 2) __stcs(reinterpret_cast<uint4*>(dst), make_uint4(w[0], w[1], w[(V / 2) > 2 ? 2 : 0], w[(V / 2) > 3 ? 3 : 0]));
                else v[k].store(dst);
            }
        }
    }
}

// ---- bf16 blocks in packed arithmetic -----------------------------------------------------------------------------
// After the quotient every step of the expression is one bf16 operation on bf16 operands, so it can run on both
// halves of a 32-bit word at once with the same results: add / sub / mul.rn.bf16x2 round the exact result once, as
// the fp32 operation followed by the conversion does (a sum of two bf16 numbers that does not fit fp32 is further
// than 2^16 ulps from any bf16 rounding boundary; a product always fits).  Three things need care:
//   * clamp(round(t)) is computed as round(clamp(t)): the same for integer bounds;
//   * round to integer: for quant_max - quant_min <= 126 by adding and subtracting an even M with 128 <= q + M <= 255
//     (bf16 numbers in [128, 256) are the integers, ties go to the even one, M even keeps the parity), then the sign
//     of t is put back (a zero result keeps the sign of what was rounded, as rint does); otherwise through fp32;
//   * a negative zero in front of a lower bound of +0 would lose its sign in max(): without a scale table t is never
//     negative when quant_min is 0 (x >= min gives x / sf + zp >= 0 after the monotone roundings), so this kernel is
//     used without a table and with quant_min <= 0 < quant_max or quant_min > 0 only.
__device__ __forceinline__ uint32_t bf2_min_nan(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf2_max_nan(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t u16x2_min(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("min.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf2_both(float v) {       // v is a bf16 number: its pattern in both halves
    const uint32_t h = __float_as_uint(v) >> 16;
    return h | (h << 16);
}

__global__ void __launch_bounds__(256, 4) group_affine_packed_kernel(const GroupAffineParams p, float magic) {
    const uint4* x = reinterpret_cast<const uint4*>(p.in);
    uint4* out = reinterpret_cast<uint4*>(p.out);
    const int G = p.lanes;
    const int lane = threadIdx.x & 31, sub = lane & (G - 1);
    const uint32_t gmask = (G == 32) ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int64_t groups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int64_t rounds = (p.n_blocks + groups - 1) / groups;
    const int64_t g0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const uint32_t lo2 = bf2_both(p.qmin), hi2 = bf2_both(p.qmax), m2 = bf2_both(magic);
    const int per_block = p.block / 8;                   // 16-byte pieces of a block
    for (int64_t r = 0; r < rounds; ++r) {               // all lanes of a warp stay in the loop together
        const int64_t b = g0 + r * groups;
        const bool live = b < p.n_blocks;
        const uint4* src = x + (live ? b : 0) * per_block + sub;
        uint32_t w[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint4 t = __ldcs(src + k * G);
            w[4 * k] = t.x; w[4 * k + 1] = t.y; w[4 * k + 2] = t.z; w[4 * k + 3] = t.w;
        }
        // extrema of both halves, and the smallest non-zero magnitude as a 16-bit key (|h| - 1, a zero wraps to 0xFFFF)
        uint32_t mn2 = w[0], mx2 = w[0], key = 0xFFFFFFFFu;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            mn2 = bf2_min_nan(mn2, w[k]);
            mx2 = bf2_max_nan(mx2, w[k]);
            key = u16x2_min(key, (((w[k] & 0x7FFF7FFFu) | 0x80008000u) - 0x00010001u) ^ 0x80008000u);
        }
        float mn = min_nan(__uint_as_float(mn2 << 16), __uint_as_float(mn2 & 0xFFFF0000u));
        float mx = max_nan(__uint_as_float(mx2 << 16), __uint_as_float(mx2 & 0xFFFF0000u));
        uint32_t smallest = min(key & 0xFFFFu, key >> 16);
        for (int o = G >> 1; o > 0; o >>= 1) {
            mn = min_nan(mn, __shfl_xor_sync(gmask, mn, o));
            mx = max_nan(mx, __shfl_xor_sync(gmask, mx, o));
            smallest = min(smallest, __shfl_xor_sync(gmask, smallest, o));
        }
        if (mn != mn || mx != mx) mn = mx = __uint_as_float(0x7FC00000u);
        float sf = rnd<bf16_t>(__fdiv_rn(rnd<bf16_t>(__fsub_rn(mx, mn)), p.qrange));
        sf = (sf > 0.0f) ? sf : 1.0f;
        const float zp = rnd<bf16_t>(__fadd_rn(rnd<bf16_t>(__fdiv_rn(-mn, sf)), p.qmin));
        if (live && sub == 0) {
            store_one<bf16_t>(reinterpret_cast<bf16_t*>(p.scale) + b, sf);
            store_one<bf16_t>(reinterpret_cast<bf16_t*>(p.zero_point) + b, zp);
        }
        // x / sf as a product: sf in [2^-63, 2^63] and no element of the block below 2^-60 other than zeros
        const uint32_t sb = __float_as_uint(sf), ex = (sb >> 23) & 0xFFu;
        const bool by_product = ex >= 64u && ex <= 190u && smallest >= 0x217Fu;
        float y;
        asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(sf));
        const uint32_t sf2 = bf2_both(sf), zp2 = bf2_both(zp);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float a = __uint_as_float(w[k] << 16), c = __uint_as_float(w[k] & 0xFFFF0000u);
            if (by_product) {                              // the same for the whole block
                mul_pair(a, c, y);
            } else {
                a = __fdiv_rn(a, sf);
                c = __fdiv_rn(c, sf);
            }
            uint32_t t;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(t) : "f"(c), "f"(a));
            t = bf2_min_nan(bf2_max_nan(bf2_add(t, zp2), lo2), hi2);
            if (magic != 0.0f) {
                t = bf2_sub(bf2_add(t, m2), m2) | (t & 0x80008000u);
            } else {
                a = rintf(__uint_as_float(t << 16));
                c = rintf(__uint_as_float(t & 0xFFFF0000u));
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(t) : "f"(c), "f"(a));
            }
            w[k] = bf2_mul(bf2_sub(t, zp2), sf2);
        }
        if (live) {
            uint4* dst = out + b * per_block + sub;
#pragma unroll
            for (int k = 0; k < 4; ++k) __stcs(dst + k * G, make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]));
        }
    }
}

}  // namespace

extern "C" int vq_group_affine_fake_quantize(const void* in, int dtype, int64_t rows, int64_t K, int64_t block, double quant_min,
                                             double quant_max, const uint16_t* scale_table, void* out_scale, void* out_zero_point,
                                             void* out, void* stream) {
    const char* name = "vq_group_affine_fake_quantize";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(rows >= 0 && K >= 0 && block >= 1 && block < (1ll << 30), "%s: bad shape or block size", name);
    VQ_REQUIRE(quant_max > quant_min, "%s: quant_max must exceed quant_min", name);
    if (rows == 0 || K == 0) return 0;
    VQ_REQUIRE(in && out && out_scale && out_zero_point, "%s: null tensor", name);
    GroupAffineParams p{};
    p.in = in; p.out = out; p.scale = out_scale; p.zero_point = out_zero_point; p.table = scale_table;
    p.rows = rows; p.K = K;
    p.block = (int)block;
    p.blocks_per_row = (int)((K + block - 1) / block);
    p.n_blocks = rows * p.blocks_per_row;
    p.qmin = (float)quant_min; p.qmax = (float)quant_max; p.qrange = (float)(quant_max - quant_min);
    const int V = dtype == VQ_F32 ? 4 : 8;
    p.vec = (K % V == 0 && block % V == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0) ? 1 : 0;
    const int64_t chunks = p.vec ? (block + V - 1) / V : block;
    int lanes = 1;
    while (lanes * 2 <= 32 && lanes * 2 * 4 <= chunks) lanes *= 2;      // about four 16-byte pieces per lane: loads in flight
    p.lanes = lanes;
    const int threads = 256;
    const int64_t want = (p.n_blocks * lanes + threads - 1) / threads;
    const int64_t cap = (int64_t)vq_sm_count() * 8;
    const int blocks = (int)(want < cap ? want : cap);
    // the block held in registers: exactly four pieces per lane and rows of whole blocks (VOYAGER_B200_GROUP_AFFINE=sweeps: never)
    const char* form = getenv("VOYAGER_B200_GROUP_AFFINE");
    const bool held = p.vec && K % block == 0 && chunks == 4ll * lanes && !(form && !strcmp(form, "sweeps"));
    // bf16 in packed arithmetic: integer bounds of at most 256 in magnitude, no scale table, the zero not an upper bound
    const bool packed = held && dtype == VQ_BF16 && !scale_table && quant_min == (double)(int64_t)quant_min &&
                        quant_max == (double)(int64_t)quant_max && quant_min >= -256.0 && quant_max <= 256.0 && quant_max > 0.0 &&
                        !(form && !strcmp(form, "held"));
    if (packed) {
        // round to integer by an even M with 128 <= quant_min + M and quant_max + M <= 255; 0: through fp32
        double magic = 0.0;
        if (quant_max - quant_min <= 126.0) {
            magic = 128.0 - quant_min;
            if ((int64_t)magic & 1) magic += 1.0;
        }
        const int64_t resident = (int64_t)vq_sm_count() * 4;                  // four CTAs of this kernel fit an SM
        group_affine_packed_kernel<<<(int)(want < resident ? want : resident), threads, 0, (cudaStream_t)stream>>>(p, (float)magic);
    } else if (held) {
        const int64_t resident = (int64_t)vq_sm_count() * 4;
        if (dtype == VQ_F32) group_affine_held_kernel<float><<<(int)(want < resident ? want : resident), threads, 0, (cudaStream_t)stream>>>(p);
        else group_affine_held_kernel<bf16_t><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
    } else {
        if (dtype == VQ_F32) group_affine_kernel<float><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
        else group_affine_kernel<bf16_t><<<blocks, threads, 0, (cudaStream_t)stream>>>(p);
    }
    VQ_LAUNCH_CHECK("group_affine_kernel");
    return 0;
}
