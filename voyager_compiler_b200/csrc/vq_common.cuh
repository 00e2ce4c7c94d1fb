// Shared device/host helpers for the voyager_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/voyager_b200.h"

// ------------------------------------------------------------------------------------------
// Host side: error reporting, launch accounting, device properties
// ------------------------------------------------------------------------------------------
int vq_set_error(int code, const char* fmt, ...);
void vq_count_launch();
int vq_sm_count();               // SMs of the current device (cached per device)
int vq_max_smem_optin();         // max opt-in dynamic shared memory per block of the current device

#define VQ_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return vq_set_error(VQ_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define VQ_CUDA(call)                                                                         \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return vq_set_error(VQ_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define VQ_LAUNCH_CHECK(name)                                                                  \
    do {                                                                                       \
        cudaError_t e__ = cudaGetLastError();                                                  \
        if (e__ != cudaSuccess)                                                                \
            return vq_set_error(VQ_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
        vq_count_launch();                                                                     \
    } while (0)

// Tries the compile-time specialised fused MX kernel on `items` (host array; one item is passed by
// value, several need the device `workspace`).  Returns 1 when it launched, 0 when the arguments
// are outside its domain (the caller then uses the generic kernels), a negative status on error.
int vq_mx_fast_try(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max, int pow2,
                   const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                   void* workspace, cudaStream_t st);

// Tries the specialised element-wise kernel (op 0 map, 1 quantize, 2 dequantize).  Returns 1 when
// it launched, 0 when the arguments are outside its domain, a negative status on error.
int vq_ew_fast_try(int op, const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                   const vq_scale_layout* layout, const vq_table* t0, const vq_table* t1, void* out, uint8_t* codes,
                   cudaStream_t st);

// Division of a 31-bit index by a run-time constant: q = (umulhi(n, m) + n) >> s, valid for
// 0 <= n < 2^31 and 1 <= d < 2^31.
struct FastDiv {
    uint32_t d, m, s;
};
FastDiv make_fastdiv(uint32_t d);

__host__ __device__ __forceinline__ uint32_t fd_div(uint32_t n, const FastDiv& f) {
#ifdef __CUDA_ARCH__
    return (__umulhi(n, f.m) + n) >> f.s;
#else
    return (uint32_t)((((uint64_t)n * f.m) >> 32) + n) >> f.s;
#endif
}

// ------------------------------------------------------------------------------------------
// Device side
// ------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// Device copy of vq_table with the lookup pointer already resolved (global or shared).
struct TableDev {
    int kind;
    int n_runs;
    const uint16_t* lut16;
    const uint8_t* lut8;
    float lo, hi;
    const uint16_t* run_keys;
    const uint16_t* run_vals;
    const uint8_t* run_codes;
    uint16_t nan_val, pinf_val, ninf_val;
    uint8_t nan_code, pinf_code, ninf_code;
    uint8_t flat_tiny;
    const float* levels2;
};

#define VQ_MAX_RUNS 512

inline TableDev to_dev(const vq_table* t) {
    TableDev d{};
    if (!t) return d;
    d.kind = t->kind;
    d.n_runs = t->n_runs;
    d.lut16 = t->lut16;
    d.lut8 = t->lut8;
    d.lo = t->lo;
    d.hi = t->hi;
    d.run_keys = t->run_keys;
    d.run_vals = t->run_vals;
    d.run_codes = t->run_codes;
    d.nan_val = t->nan_val;
    d.pinf_val = t->pinf_val;
    d.ninf_val = t->ninf_val;
    d.nan_code = t->nan_code;
    d.pinf_code = t->pinf_code;
    d.ninf_code = t->ninf_code;
    d.levels2 = t->levels2;
    d.flat_tiny = (t->kind == VQ_TABLE_INT) ? (t->lo <= 0.0f && t->hi >= 0.0f) : t->flat_tiny;
    return d;
}

// fp32 -> bf16 bit pattern, round to nearest even.  Every NaN becomes 0xFFFF, the pattern the
// vectorised CPU conversion produces, so a NaN always selects the same table entry.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
    uint32_t u = __float_as_uint(v);
    uint32_t r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    return (v != v) ? 0xFFFFu : r;
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// Arithmetic in the tensor's dtype: fp32 keeps fp32; bf16 rounds every op's fp32 result to bf16,
// which is what the CPU reference does (operands widened, one IEEE op, RNE back).
template <typename T>
struct Arith;
template <>
struct Arith<float> {
    static __device__ __forceinline__ float rnd(float v) { return v; }
};
struct bf16_t {
    uint16_t bits;
};
template <>
struct Arith<bf16_t> {
    static __device__ __forceinline__ float rnd(float v) {
        // NaN payloads do not matter downstream: any NaN indexes entry 0xFFFF / compares false
        return bf16_bits_to_f32(f32_to_bf16_bits(v));
    }
};

template <typename T>
struct Vec;  // 16-byte vector of T
template <>
struct Vec<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void load_stream(const float* p) {
        float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const {
        __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <>
struct Vec<bf16_t> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void unpack(uint4 t) {
        uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ __forceinline__ void load(const bf16_t* p) { unpack(*reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void load_stream(const bf16_t* p) {
        unpack(__ldcs(reinterpret_cast<const uint4*>(p)));
    }
    // values are bf16-representable, so truncation is exact
    __device__ __forceinline__ void store(bf16_t* p) const {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xFFFF0000u);
        __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
    }
};

template <typename T>
__device__ __forceinline__ float load_one(const T* p);
template <>
__device__ __forceinline__ float load_one<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_one<bf16_t>(const bf16_t* p) { return bf16_bits_to_f32(p->bits); }
template <typename T>
__device__ __forceinline__ void store_one(T* p, float v);
template <>
__device__ __forceinline__ void store_one<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_one<bf16_t>(bf16_t* p, float v) { p->bits = (uint16_t)(__float_as_uint(v) >> 16); }

// Order-preserving 16-bit key of a bf16 pattern: ascending key == ascending value, -0 just below +0.
__device__ __forceinline__ uint32_t bf16_key(uint32_t bits) { return bits ^ ((bits & 0x8000u) ? 0xFFFFu : 0x8000u); }

// Index of the run that holds `key`: number of run starts <= key.  `keys` has n_runs-1 entries
// padded with 0xFFFF up to the next power of two minus one (pad never compares <= a real key
// because keys of finite inputs are <= 0xFF7F).
__device__ __forceinline__ uint32_t run_search(const uint16_t* keys, int steps_pow2, uint32_t key) {
    uint32_t idx = 0;
    for (uint32_t step = (uint32_t)steps_pow2; step > 0; step >>= 1) {
        uint32_t probe = idx + step;                 // candidate count
        uint32_t k = keys[probe - 1];
        idx = (k <= key) ? probe : idx;
    }
    return idx;
}

// Output value of a table for the value v (already in the op's arithmetic; rounded to bf16 here).
// `lut` is the resolved LUT16 pointer (shared or global), `rk`/`rv` the resolved run arrays.
struct TableRes {
    const uint16_t* lut;
    const uint16_t* rk;
    const uint16_t* rv;
    int steps;  // RUNS: largest power of two <= padded key count
};

// Result of one table lookup.
struct Looked {
    float val;
    uint32_t code;
};

// Output value and/or packed code for the bf16 pattern `pat`.
__device__ __forceinline__ Looked table_lookup(const TableDev& t, const TableRes& r, uint32_t pat, bool want_val,
                                               bool want_code) {
    Looked o{0.0f, 0u};
    if (t.kind == VQ_TABLE_INT) {
        float vb = bf16_bits_to_f32(pat);
        // comparisons, not fmaxf/fminf: clamp(-0, 0, hi) must stay -0 as it does on the CPU
        float q = rintf(vb);
        q = (q < t.lo) ? t.lo : q;
        q = (q > t.hi) ? t.hi : q;
        o.val = (vb != vb) ? vb : q;
        o.code = (vb != vb) ? 0u : ((uint32_t)(int)q & 0xFFu);
    } else if (t.kind == VQ_TABLE_RUNS) {
        if ((pat & 0x7F80u) == 0x7F80u) {  // inf / NaN inputs are kept out of the search
            const bool nan = (pat & 0x7Fu) != 0u, neg = (pat & 0x8000u) != 0u;
            o.val = bf16_bits_to_f32(nan ? t.nan_val : (neg ? t.ninf_val : t.pinf_val));
            o.code = nan ? t.nan_code : (neg ? t.ninf_code : t.pinf_code);
        } else {
            uint32_t idx = run_search(r.rk, r.steps, bf16_key(pat));
            o.val = bf16_bits_to_f32(r.rv[idx]);
            if (want_code && t.run_codes) o.code = t.run_codes[idx];
        }
    } else {
        if (want_val) o.val = bf16_bits_to_f32(r.lut[pat]);
        if (want_code && t.lut8) o.code = t.lut8[pat];
    }
    return o;
}

// Output value of a table for the value v (rounded to bf16 here).
__device__ __forceinline__ float table_value(const TableDev& t, const TableRes& r, float v, uint32_t& pat) {
    pat = f32_to_bf16_bits(v);
    return table_lookup(t, r, pat, true, false).val;
}

// |x| reduction that propagates NaN the way torch.max does: the fp32 bit patterns of |x| order
// finite < inf < NaN as unsigned integers.
__device__ __forceinline__ uint32_t abs_bits(float v) { return __float_as_uint(v) & 0x7FFFFFFFu; }

// Scale of one block from its |x| maximum (as fp32 bits), in the arithmetic of dtype T.
struct ScaleRule {
    int pow2;                   // 0: amax / qmax, 1: power of two, 2: the block maximum itself
    float qmax;                 // (float)quant_max
    const uint32_t* bump_at;    // pow2
    const float* scale_of;      // pow2
    TableDev stab;              // non-pow2: optional scale table (global LUT16 / INT / RUNS)
    TableRes sres;
};

template <typename T>
__device__ __forceinline__ float block_scale(const ScaleRule& r, uint32_t amax_bits) {
    if (r.pow2 == 2) return __uint_as_float(amax_bits);  // raw block maximum (NaN kept)
    if (amax_bits > 0x7F800000u) return 1.0f;  // NaN amax: every comparison fails -> 1
    if (r.pow2) {
        if (amax_bits == 0x7F800000u) return __uint_as_float(0x7F800000u);
        uint32_t b = amax_bits ? amax_bits : 0x00800000u;  // amax == 0 is replaced by 2^-126
        int e = (b >= 0x00800000u) ? (int)(b >> 23) - 127 : (31 - __clz(b)) - 149;
        int i = e + 149;
        i += (b >= __ldg(r.bump_at + i)) ? 1 : 0;
        return __ldg(r.scale_of + i);
    }
    float s = Arith<T>::rnd(__fdiv_rn(__uint_as_float(amax_bits), r.qmax));
    if (r.stab.kind != VQ_TABLE_NONE) {
        uint32_t pat;
        s = table_value(r.stab, r.sres, s, pat);
    }
    return (s > 0.0f) ? s : 1.0f;
}

// x / s in dtype T.  When s is a power of two whose reciprocal is a normal number the exact
// product x * (1/s) is the same correctly rounded result as the division.
struct Divider {
    float s, r;
    bool mul;
    __device__ __forceinline__ explicit Divider(float scale) : s(scale) {
        uint32_t b = __float_as_uint(scale);
        uint32_t ex = (b >> 23) & 0xFFu;
        mul = ((b & 0x807FFFFFu) == 0u) && ex >= 2u && ex <= 252u;
        r = __uint_as_float((254u - ex) << 23);
    }
    __device__ __forceinline__ float operator()(float x) const { return mul ? __fmul_rn(x, r) : __fdiv_rn(x, s); }
};

#endif  // __CUDACC__
