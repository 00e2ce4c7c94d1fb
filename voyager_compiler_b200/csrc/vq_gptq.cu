// One microscaling block of the GPTQ column walk (upstream: src/voyager_compiler/quantization/gptq.py:238-259,
// block_scale :79-137).  Within a block every output row is independent: its scale comes from its own (already
// compensated) weights, and each column's rounding error moves only the same row's later columns, weighted by one
// row of the inverse-Hessian factor that all rows share.  So one thread takes one row, keeps the row's block in
// registers and walks the columns; the factor's block sits in shared memory (every thread reads the same entry:
// broadcasts).  All arithmetic is fp32 in the order upstream's tensor expressions evaluate it (divide, round to
// bf16, table, multiply; subtract, divide; multiply, subtract), so a block is reproduced bit for bit.
#include "vq_common.cuh"

namespace {

constexpr int kGptqThreads = 64;
constexpr float kGptqEps = 1e-12f;                               // quantization/lcq.py:34, as fp32
constexpr int kShrinkSteps = 5;
__constant__ float kShrinkGrid[kShrinkSteps] = {1.0f, 0.93f, 0.86f, 0.79f, 0.72f};   // gptq.py:76

struct GptqParams {
    const float* work;           // [rows, ld]: the running weights; columns start..start+bw are read
    int64_t ld;
    int64_t rows;
    int64_t start;
    int bw;                      // columns in this block (<= BW)
    const float* hinv;           // upper factor of the inverse Hessian, [K, ldh]
    int64_t ldh;
    const float* salience;       // [K] diag(H), the weights of the shrink search (may be NULL without shrink)
    int shrink;
    float qmax;
    const uint16_t* lut;         // value table: bf16 pattern -> bf16 pattern
    const uint16_t* slut;        // scale table or NULL
    float* out;                  // [rows, ldo]: the reconstruction, columns start..start+bw written
    int64_t ldo;
    float* deltas;               // [rows, bw]: error / diagonal per column
    float* scale_out;            // [rows] or NULL: the scale each row used
};

__device__ __forceinline__ float through(const uint16_t* lut, float v) {
    return bf16_bits_to_f32(__ldg(lut + f32_to_bf16_bits(v)));
}

__device__ __forceinline__ float on_grid(const uint16_t* lut, float v, float s) {
    return __fmul_rn(through(lut, __fdiv_rn(v, s)), s);
}

template <int BW>
__global__ void __launch_bounds__(kGptqThreads) gptq_block_kernel(const __grid_constant__ GptqParams p) {
    __shared__ float hs[BW * BW];                                // hs[j * BW + i] = hinv[start + j, start + i], 0 beyond bw
    __shared__ float dg[BW], sal[BW];
    for (int t = threadIdx.x; t < BW * BW; t += blockDim.x) {
        const int j = t / BW, i = t % BW;
        hs[t] = (j < p.bw && i < p.bw) ? p.hinv[(p.start + j) * p.ldh + p.start + i] : 0.0f;
    }
    for (int t = threadIdx.x; t < BW; t += blockDim.x) {
        dg[t] = t < p.bw ? fmaxf(p.hinv[(p.start + t) * p.ldh + p.start + t], kGptqEps) : 1.0f;
        sal[t] = (t < p.bw && p.salience) ? p.salience[p.start + t] : 0.0f;
    }
    __syncthreads();
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= p.rows) return;
    float w[BW];
    const float* src = p.work + row * p.ld + p.start;
    uint32_t amax_bits = 0;
#pragma unroll
    for (int j = 0; j < BW; ++j) {
        w[j] = j < p.bw ? src[j] : 0.0f;
        amax_bits = max(amax_bits, abs_bits(w[j]));
    }
    // calculate_mx_qparam without the power-of-two rule (ops/quantized.py:489-498), then clamp_min(EPS)
    float s = 1.0f;
    if (amax_bits <= 0x7F800000u) {
        s = __fdiv_rn(__uint_as_float(amax_bits), p.qmax);
        if (p.slut) s = through(p.slut, s);
        s = s > 0.0f ? s : 1.0f;
    }
    s = fmaxf(s, kGptqEps);
    if (p.shrink) {
        // gptq.py:120-137: the factor with the lowest salience-weighted squared error, first wins ties;
        // the row sum runs over the columns in order
        const float base = s;
        float lowest = 0.0f;
        for (int f = 0; f < kShrinkSteps; ++f) {
            float sf = base;
            if (f > 0) sf = fmaxf(through(p.slut, __fmul_rn(base, kShrinkGrid[f])), kGptqEps);
            float err = 0.0f;
#pragma unroll
            for (int j = 0; j < BW; ++j) {
                if (j < p.bw) {
                    const float d = __fsub_rn(w[j], on_grid(p.lut, w[j], sf));
                    err = __fadd_rn(err, __fmul_rn(__fmul_rn(d, d), sal[j]));
                }
            }
            if (f == 0 || err < lowest) { lowest = err; s = sf; }
        }
    }
    if (p.scale_out) p.scale_out[row] = s;
    float* dst = p.out + row * p.ldo + p.start;
    float* dl = p.deltas + row * p.bw;
#pragma unroll
    for (int j = 0; j < BW; ++j) {
        if (j < p.bw) {
            const float v = w[j];
            const float q = on_grid(p.lut, v, s);
            const float delta = __fdiv_rn(__fsub_rn(v, q), dg[j]);
            dst[j] = q;
            dl[j] = delta;
#pragma unroll
            for (int i = j + 1; i < BW; ++i) w[i] = __fsub_rn(w[i], __fmul_rn(delta, hs[j * BW + i]));
        }
    }
}

template <int BW>
int launch_gptq(const GptqParams& p, cudaStream_t st) {
    const int blocks = (int)((p.rows + kGptqThreads - 1) / kGptqThreads);
    gptq_block_kernel<BW><<<blocks, kGptqThreads, 0, st>>>(p);
    VQ_LAUNCH_CHECK("gptq_block_kernel");
    return 0;
}

}  // namespace

extern "C" int vq_gptq_block(const float* work, int64_t ld, int64_t rows, int64_t start, int bw, const float* hinv, int64_t ldh,
                             const float* salience, int shrink, double quant_max, const vq_table* table,
                             const vq_table* scale_table, float* out, int64_t ldo, float* deltas, float* scale_out,
                             void* stream) {
    const char* name = "vq_gptq_block";
    VQ_REQUIRE(rows >= 0 && start >= 0 && bw >= 1, "%s: bad sizes", name);
    if (bw > 64) return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: blocks of up to 64 columns", name);
    VQ_REQUIRE(ld >= start + bw && ldo >= start + bw && ldh >= start + bw, "%s: the block does not fit the row pitch", name);
    if (rows == 0) return 0;
    VQ_REQUIRE(work && hinv && out && deltas, "%s: null pointer", name);
    VQ_REQUIRE(table && table->lut16, "%s: the value table needs its 65 536-entry form", name);
    VQ_REQUIRE(!shrink || (scale_table && scale_table->lut16 && salience), "%s: the shrink search needs a scale table and the saliences", name);
    VQ_REQUIRE(rows < (1ll << 31) * kGptqThreads, "%s: too many rows", name);
    GptqParams p{};
    p.work = work; p.ld = ld; p.rows = rows; p.start = start; p.bw = bw;
    p.hinv = hinv; p.ldh = ldh; p.salience = salience; p.shrink = shrink ? 1 : 0;
    p.qmax = (float)quant_max;
    p.lut = table->lut16;
    p.slut = scale_table ? scale_table->lut16 : nullptr;
    p.out = out; p.ldo = ldo; p.deltas = deltas; p.scale_out = scale_out;
    cudaStream_t st = (cudaStream_t)stream;
    if (bw <= 16) return launch_gptq<16>(p, st);
    if (bw <= 32) return launch_gptq<32>(p, st);
    return launch_gptq<64>(p, st);
}
