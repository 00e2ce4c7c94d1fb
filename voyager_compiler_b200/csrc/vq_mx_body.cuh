// Pieces shared by the single-tensor and the multi-tensor MX kernels.
#pragma once
#include "vq_common.cuh"

namespace {

struct MxParams {
    const void* in;
    int64_t outer, L, inner, block, nblk;   // nblk = ceil(L / block)
    int64_t n;
    ScaleRule rule;
    TableDev tab;          // kind NONE: scale only
    void* out_scale;
    void* out_codes;
    float* scale_f32;
    int8_t* exp_e8;
    uint8_t* codes;
    int code_bits;
    void* dequant;
    int group_shift;       // fast path: log2(lanes per block)
    int smem_lut16, smem_lut8;
};

__device__ __forceinline__ int pow2_steps_mx(int n_runs) {
    int keys = n_runs - 1, p = 1;
    while (p <= keys) p <<= 1;
    return p >> 1;
}

// Shared-memory staging: [lut16 128 KB][lut8 64 KB][run keys/vals/codes 2.5 KB]
__device__ __forceinline__ void stage_mx(const MxParams& p, uint4* smem, TableDev& tab, TableRes& res) {
    tab = p.tab;
    res = TableRes{p.tab.lut16, p.tab.run_keys, p.tab.run_vals, 0};
    uint8_t* s8 = reinterpret_cast<uint8_t*>(smem);
    if (p.smem_lut16) {
        const uint4* src = reinterpret_cast<const uint4*>(p.tab.lut16);
        uint4* dst = reinterpret_cast<uint4*>(s8);
        for (int i = threadIdx.x; i < 8192; i += blockDim.x) dst[i] = __ldg(src + i);
        res.lut = reinterpret_cast<const uint16_t*>(s8);
        s8 += 131072;
    }
    if (p.smem_lut8) {
        const uint4* src = reinterpret_cast<const uint4*>(p.tab.lut8);
        uint4* dst = reinterpret_cast<uint4*>(s8);
        for (int i = threadIdx.x; i < 4096; i += blockDim.x) dst[i] = __ldg(src + i);
        tab.lut8 = s8;
        s8 += 65536;
    }
    if (p.tab.kind == VQ_TABLE_RUNS) {
        uint16_t* keys = reinterpret_cast<uint16_t*>(s8);
        uint16_t* vals = keys + VQ_MAX_RUNS;
        uint8_t* rc = s8 + 4 * VQ_MAX_RUNS;
        for (int i = threadIdx.x; i < VQ_MAX_RUNS; i += blockDim.x) {
            keys[i] = (i < p.tab.n_runs - 1) ? p.tab.run_keys[i] : (uint16_t)0xFFFF;
            vals[i] = (i < p.tab.n_runs) ? p.tab.run_vals[i] : (uint16_t)0;
            rc[i] = (p.tab.run_codes && i < p.tab.n_runs) ? p.tab.run_codes[i] : (uint8_t)0;
        }
        res.rk = keys;
        res.rv = vals;
        res.steps = pow2_steps_mx(p.tab.n_runs);
        if (p.tab.run_codes) tab.run_codes = rc;
    }
    __syncthreads();
}

__device__ __forceinline__ int scale_exponent(float s) {
    uint32_t b = __float_as_uint(s);
    if (b >= 0x7F800000u) return 127;
    int e = (b >= 0x00800000u) ? (int)(b >> 23) - 127 : (b ? (31 - __clz(b)) - 149 : -127);
    return e < -127 ? -127 : (e > 127 ? 127 : e);
}

template <typename T>
__device__ __forceinline__ void emit_scale(const MxParams& p, int64_t idx, float s) {
    if (p.out_scale) store_one<T>(reinterpret_cast<T*>(p.out_scale) + idx, s);
    if (p.scale_f32) p.scale_f32[idx] = s;
    if (p.exp_e8) p.exp_e8[idx] = (int8_t)scale_exponent(s);
}


// Quantize one 16-byte vector whose block scale is `s` and write the requested outputs at element
// offset `base` of the given destinations.
template <typename T>
__device__ __forceinline__ void mx_emit_vector(const TableDev& tab, const TableRes& res, Vec<T>& x, float s, size_t base,
                                               T* out_codes, T* dequant, uint8_t* codes8, int code_bits) {
    constexpr int N = Vec<T>::N;
    const Divider dv(s);
    uint32_t codes[N];
    Vec<T> dq;
    const bool want_val = out_codes != nullptr || dequant != nullptr;
    const bool want_code = codes8 != nullptr;
#pragma unroll
    for (int j = 0; j < N; ++j) {
        float q = Arith<T>::rnd(dv(x.v[j]));
        Looked lk = table_lookup(tab, res, f32_to_bf16_bits(q), want_val, want_code);
        x.v[j] = lk.val;
        codes[j] = lk.code;
        dq.v[j] = Arith<T>::rnd(__fmul_rn(lk.val, s));
    }
    if (out_codes) x.store(out_codes + base);
    if (dequant) dq.store(dequant + base);
    if (codes8) {
        if (code_bits == 8) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(codes8 + base);
#pragma unroll
            for (int j = 0; j < N / 4; ++j)
                __stcs(dst + j, codes[4 * j] | (codes[4 * j + 1] << 8) | (codes[4 * j + 2] << 16) | (codes[4 * j + 3] << 24));
        } else {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < N; ++j) w |= (codes[j] & 0xFu) << (4 * j);
            if (N == 8) __stcs(reinterpret_cast<uint32_t*>(codes8 + base / 2), w);
            else *reinterpret_cast<uint16_t*>(codes8 + base / 2) = (uint16_t)w;
        }
    }
}

}  // namespace
