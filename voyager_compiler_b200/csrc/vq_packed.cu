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
    uint32_t nword;         // 32-bit code words: 4 elements (8-bit codes) or 8 elements (4-bit codes)
    uint32_t block_words;   // words per block
};

// One 32-bit code word per thread and pass, so that a warp reads 128 contiguous bytes and writes
// 256 B - 1 KB contiguous; UNROLL independent words per thread keep enough bytes in flight.
template <typename T, int BITS, int UNROLL>
__global__ void __launch_bounds__(512) dequant_packed_kernel(const PackedParams p) {
    constexpr int EPW = 32 / BITS;
    __shared__ float lv[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lv[i] = i < p.n_levels ? __ldg(p.levels + i) : 0.0f;
    __syncthreads();
    T* out = reinterpret_cast<T*>(p.out);
    const uint32_t* words = reinterpret_cast<const uint32_t*>(p.codes);
    const uint32_t span = blockDim.x * UNROLL;
    for (uint32_t base = blockIdx.x * span + threadIdx.x; base < p.nword; base += gridDim.x * span) {
        uint32_t w[UNROLL];
        float s[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint32_t c = base + u * blockDim.x;
            if (c < p.nword) {
                w[u] = __ldcs(words + c);
                const uint32_t b = c / p.block_words;
                if (p.scale_f32) s[u] = __ldg(p.scale_f32 + b);
                else {
                    const int e = __ldg(p.exp_e8 + b);
                    s[u] = (e >= -126) ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(1u << (e + 149 < 0 ? 0 : e + 149));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint32_t c = base + u * blockDim.x;
            if (c >= p.nword) break;
            float v[EPW];
#pragma unroll
            for (int j = 0; j < EPW; ++j) {
                const uint32_t code = (w[u] >> (BITS * j)) & ((1u << BITS) - 1u);
                v[j] = __fmul_rn(lv[code], s[u]);
            }
            if constexpr (sizeof(T) == 4) {
                float4* dst = reinterpret_cast<float4*>(out + (size_t)c * EPW);
#pragma unroll
                for (int j = 0; j < EPW / 4; ++j) __stcs(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
            } else {
                uint32_t o[EPW / 2];
#pragma unroll
                for (int j = 0; j < EPW / 2; ++j)      // one rounding of the fp32 product, two values per instruction
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(v[2 * j + 1]), "f"(v[2 * j]));
                if constexpr (EPW == 8) __stcs(reinterpret_cast<uint4*>(out + (size_t)c * EPW), make_uint4(o[0], o[1], o[2], o[3]));
                else __stcs(reinterpret_cast<uint2*>(out + (size_t)c * EPW), make_uint2(o[0], o[1]));
            }
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
    const int epw = 32 / code_bits;
    p.nword = (uint32_t)(n / epw);
    p.block_words = (uint32_t)(block / epw);
    const int sms = vq_sm_count();
    const int threads = 512;
    constexpr int UNROLL = 4;
    int64_t want = ((int64_t)p.nword + threads * UNROLL - 1) / (threads * UNROLL);
    int blocks = (int)(want > (int64_t)sms * 4 ? (int64_t)sms * 4 : want);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VQ_F32) {
        if (code_bits == 8) dequant_packed_kernel<float, 8, UNROLL><<<blocks, threads, 0, st>>>(p);
        else dequant_packed_kernel<float, 4, UNROLL><<<blocks, threads, 0, st>>>(p);
    } else {
        if (code_bits == 8) dequant_packed_kernel<bf16_t, 8, UNROLL><<<blocks, threads, 0, st>>>(p);
        else dequant_packed_kernel<bf16_t, 4, UNROLL><<<blocks, threads, 0, st>>>(p);
    }
    VQ_LAUNCH_CHECK("dequant_packed_kernel");
    return 0;
}
