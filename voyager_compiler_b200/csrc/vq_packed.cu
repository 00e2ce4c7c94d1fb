// Dequantization of the packed views (8-bit or 4-bit codes + one fp32 scale or E8 exponent per
// block): out[i] = levels[code[i]] * scale[i / block], rounded once in the output dtype.  This is
// what `weight_code[idx] * expand(scale)` computes in the reference (ops/quantized.py:313-326) on
// float index tensors; here the codes are read at 1 or 0.5 bytes per element.
// HBM bound: code_bits/8 + 4/block bytes read, sizeof(T) written per element.
#include "vq_common.cuh"

namespace {

struct PackedParams {
    const uint8_t* codes;
    const float* levels;
    int n_levels;
    const float* scale_f32;
    const int8_t* exp_e8;
    void* out;
    uint32_t nchunk;        // chunks of 16 elements
    uint32_t block16;       // block size / 16
};

template <typename T, int BITS>
__global__ void __launch_bounds__(512) dequant_packed_kernel(const PackedParams p) {
    __shared__ float lv[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lv[i] = i < p.n_levels ? __ldg(p.levels + i) : 0.0f;
    __syncthreads();
    T* out = reinterpret_cast<T*>(p.out);
    const uint32_t nthreads = gridDim.x * blockDim.x;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < p.nchunk; c += nthreads) {
        uint32_t w[4];
        if (BITS == 8) {
            uint4 t = __ldcs(reinterpret_cast<const uint4*>(p.codes) + c);
            w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
        } else {
            uint2 t = __ldcs(reinterpret_cast<const uint2*>(p.codes) + c);
            w[0] = t.x; w[1] = t.y; w[2] = w[3] = 0;
        }
        const uint32_t b = c / p.block16;
        float s;
        if (p.scale_f32) s = __ldg(p.scale_f32 + b);
        else {
            const int e = __ldg(p.exp_e8 + b);
            s = (e >= -126) ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(1u << (e + 149 < 0 ? 0 : e + 149));
        }
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t code = BITS == 8 ? (w[j >> 2] >> (8 * (j & 3))) & 0xFFu : (w[j >> 3] >> (4 * (j & 7))) & 0xFu;
            v[j] = Arith<T>::rnd(__fmul_rn(lv[code], s));
        }
        if (sizeof(T) == 4) {
            float4* dst = reinterpret_cast<float4*>(out + (size_t)c * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) __stcs(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
        } else {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xFFFF0000u);
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t)c * 16);
            __stcs(dst, make_uint4(o[0], o[1], o[2], o[3]));
            __stcs(dst + 1, make_uint4(o[4], o[5], o[6], o[7]));
        }
    }
}

}  // namespace

extern "C" int vq_dequantize_packed(const uint8_t* codes, int code_bits, const float* levels, int n_levels,
                                    const float* scale_f32, const int8_t* exp_e8, int64_t n, int64_t block, void* out,
                                    int dtype, void* stream) {
    const char* name = "vq_dequantize_packed";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(code_bits == 8 || code_bits == 4, "%s: code_bits must be 8 or 4", name);
    VQ_REQUIRE(n >= 0, "%s: negative element count", name);
    if (n == 0) return 0;
    VQ_REQUIRE(codes && levels && out && (scale_f32 || exp_e8), "%s: null pointer", name);
    VQ_REQUIRE(n_levels >= 1 && n_levels <= (code_bits == 8 ? 256 : 16), "%s: n_levels out of range for %d-bit codes", name, code_bits);
    VQ_REQUIRE(block > 0 && block % 16 == 0 && n % block == 0, "%s: block must be a multiple of 16 that divides n", name);
    VQ_REQUIRE(n < (1ll << 35), "%s: tensor too large", name);
    VQ_REQUIRE((uintptr_t)codes % 16 == 0 && (uintptr_t)out % 16 == 0, "%s: buffers must be 16-byte aligned", name);
    PackedParams p{};
    p.codes = codes; p.levels = levels; p.n_levels = n_levels;
    p.scale_f32 = scale_f32; p.exp_e8 = exp_e8; p.out = out;
    p.nchunk = (uint32_t)(n / 16);
    p.block16 = (uint32_t)(block / 16);
    const int sms = vq_sm_count();
    const int threads = 512;
    int64_t want = ((int64_t)p.nchunk + threads - 1) / threads;
    int blocks = (int)(want > (int64_t)sms * 4 ? (int64_t)sms * 4 : want);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VQ_F32) {
        if (code_bits == 8) dequant_packed_kernel<float, 8><<<blocks, threads, 0, st>>>(p);
        else dequant_packed_kernel<float, 4><<<blocks, threads, 0, st>>>(p);
    } else {
        if (code_bits == 8) dequant_packed_kernel<bf16_t, 8><<<blocks, threads, 0, st>>>(p);
        else dequant_packed_kernel<bf16_t, 4><<<blocks, threads, 0, st>>>(p);
    }
    VQ_LAUNCH_CHECK("dequant_packed_kernel");
    return 0;
}
