// max |x| per tensor or per channel in one pass over the data: the reduction the observer runs
// before every fake-quantize (`torch.amax(torch.abs(x))`, per-channel `torch.amax(torch.abs(x),
// dim=all but ch_axis)`, quantization/fake_quantize.py:320-325), which upstream computes as an abs
// pass (a full-size temporary) followed by a reduce pass.
//
// The tensor is viewed as [outer, C, inner]; out[c] = max over outer and inner.  |x| is reduced as
// an unsigned bit pattern (finite < inf < NaN, so a NaN wins as in torch.amax) and combined across
// CTAs with atomicMax on the fp32 output, which is zeroed first on the same stream.
//   inner >= 64: a warp per (row = outer * C + c, segment of the row), lanes stride by 16-byte vectors;
//   inner == 1:  columns across threads, rows across the grid, one atomic per column and CTA;
//   otherwise:   flat sweep, every lane keeps the maximum of its current channel and flushes it
//                when the channel changes.
// HBM bound: sizeof(T) read per element.
#include <math_constants.h>

#include "vq_common.cuh"

namespace {

struct AmaxParams {
    const void* in;
    uint32_t* out;          // fp32 bit patterns, [C]
    int64_t outer, C, inner;
    int64_t n;
    int64_t seg_len, segs_per_row, n_items;   // row mode
    FastDiv div_inner, div_C;                 // flat mode (n < 2^31)
    int vec;                                  // 16-byte loads usable
    int smem_cols;                            // column mode: per-CTA maxima staged in shared memory
    // the observer's state update by the CTA that finishes last (history == nullptr: the reduction alone)
    float* history;
    float* scale;
    unsigned int* ticket;                     // zero between launches
    const uint8_t* stay;
    int H, pow2;
    float qmax;
};

// The observer's state update for channel c (quantization/fake_quantize.py:327-341; see observer_update_kernel below).
__device__ __forceinline__ void observer_update_one(int64_t c, float cur, float* __restrict__ history, float* __restrict__ scale, int H,
                                                    int64_t C, float qmax, int pow2, const uint8_t* __restrict__ stay) {
    // torch.amax propagates NaN
    float m = history[c];
    bool nan = m != m;
    for (int h = 1; h < H; ++h) {
        const float v = history[(int64_t)h * C + c];
        nan |= v != v;
        m = fmaxf(m, v);
    }
    if (nan) m = __int_as_float(0x7FC00000);
    // roll by -1 along the history axis, then overwrite slot 0
    const float first = history[c];
    for (int h = 0; h + 1 < H; ++h) history[(int64_t)h * C + c] = history[(int64_t)(h + 1) * C + c];
    history[(int64_t)(H - 1) * C + c] = first;
    history[c] = cur;
    float sf = __fdiv_rn(m, qmax);
    const float prev = scale[c];
    sf = (m > 0.0f) ? sf : prev;
    sf = (fabsf(m) < CUDART_INF_F) ? sf : prev;
    if (pow2) {
        const uint32_t b = __float_as_uint(sf), E = (b >> 23) & 0xFFu, mant = b & 0x7FFFFFu;
        if (stay && (b >> 31) == 0u && E >= 1u && E <= 254u) {
            const int e = (int)E - 127 + (mant < (uint32_t)stay[E] ? 0 : 1);
            sf = e > 127 ? CUDART_INF_F : __uint_as_float((uint32_t)(e + 127) << 23);    // e >= -126 here
        } else {
            sf = exp2f(ceilf(log2f(sf)));
        }
    }
    scale[c] = sf;
}

template <typename T>
__device__ __forceinline__ uint32_t abs16(const T* p);   // max |x| bits of the 16 bytes at p
template <>
__device__ __forceinline__ uint32_t abs16<float>(const float* p) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(p));
    return max(max(a.x & 0x7FFFFFFFu, a.y & 0x7FFFFFFFu), max(a.z & 0x7FFFFFFFu, a.w & 0x7FFFFFFFu));
}
// max(|a|, |b|) per bf16 half; NaN wins; the sign bit of the result is the xor of the input signs
__device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
template <>
__device__ __forceinline__ uint32_t abs16<bf16_t>(const bf16_t* p) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t m2 = absmax2(absmax2(a.x, a.y), absmax2(a.z, a.w));       // two packed maxima
    return max((m2 << 16) & 0x7FFFFFFFu, m2 & 0x7FFF0000u);
}
template <typename T>
__device__ __forceinline__ uint32_t abs1(const T* p, int64_t i);
template <>
__device__ __forceinline__ uint32_t abs1<float>(const float* p, int64_t i) { return __float_as_uint(p[i]) & 0x7FFFFFFFu; }
template <>
__device__ __forceinline__ uint32_t abs1<bf16_t>(const bf16_t* p, int64_t i) { return ((uint32_t)p[i].bits << 16) & 0x7FFFFFFFu; }

// MODE 0: rows, 1: columns (inner == 1), 2: flat
template <typename T, int MODE>
__global__ void __launch_bounds__(MODE == 1 ? 1024 : 256) amax_kernel(const AmaxParams p) {
    constexpr int V = 16 / sizeof(T);
    const T* x = reinterpret_cast<const T*>(p.in);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (MODE == 0) {
        const int64_t n_warps = (int64_t)gridDim.x * 8;
        int64_t cur = -1;                 // channel of the running maximum (one atomic per run of items)
        uint32_t run = 0;
        for (int64_t item = (int64_t)blockIdx.x * 8 + warp; item < p.n_items; item += n_warps) {
            const int64_t row = item / p.segs_per_row;
            const int64_t k0 = (item - row * p.segs_per_row) * p.seg_len;
            const int64_t k1 = k0 + p.seg_len < p.inner ? k0 + p.seg_len : p.inner;
            const T* xr = x + row * p.inner;
            uint32_t m = 0;
            if (p.vec) {
                for (int64_t k = k0 + lane * V; k < k1; k += 32 * V * 4) {
                    uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (k + u * 32 * V < k1) t[u] = abs16<T>(xr + k + u * 32 * V);
                    m = max(m, max(max(t[0], t[1]), max(t[2], t[3])));
                }
            } else {
                for (int64_t k = k0 + lane; k < k1; k += 32) m = max(m, abs1<T>(xr, k));
            }
            const int64_t c = row % p.C;
            if (c != cur) {
                if (cur >= 0) {
                    run = __reduce_max_sync(0xFFFFFFFFu, run);
                    if (lane == 0 && run) atomicMax(p.out + cur, run);
                }
                cur = c;
                run = 0;
            }
            run = max(run, m);
        }
        if (cur >= 0) {
            run = __reduce_max_sync(0xFFFFFFFFu, run);
            if (lane == 0 && run) atomicMax(p.out + cur, run);
        }
    } else if (MODE == 1) {
        // x is [outer, C]: a thread owns V consecutive columns (one 16-byte load per row) of a row
        // lane, or one column; the grid splits the rows.  The row lanes of a CTA meet in shared
        // memory, then one atomic per column and CTA goes to the result (the atomics, not the reads,
        // are what limits this mode, hence few and large CTAs).
        extern __shared__ uint32_t col_max[];
        if (p.vec) {
            const int64_t G = p.C / V;                                   // column groups
            const bool staged = p.smem_cols != 0;
            if (staged) {
                for (int64_t c = threadIdx.x; c < p.C; c += blockDim.x) col_max[c] = 0u;
                __syncthreads();
            }
            const int64_t lanes = G >= blockDim.x ? 1 : blockDim.x / G;   // row lanes of this CTA
            const int64_t lane_id = G >= blockDim.x ? 0 : threadIdx.x / G;
            const int64_t g0 = G >= blockDim.x ? threadIdx.x : threadIdx.x % G;
            if (lane_id < lanes) {
                for (int64_t gcol = g0; gcol < G; gcol += blockDim.x) {
                    const int64_t c = gcol * V;
                    uint32_t m[V];
#pragma unroll
                    for (int j = 0; j < V; ++j) m[j] = 0;
                    constexpr int R = 4;          // rows in flight per thread
                    const int64_t rstep = (int64_t)gridDim.x * lanes;
                    for (int64_t r = (int64_t)blockIdx.x * lanes + lane_id; r < p.outer; r += rstep * R) {
                        uint32_t w[R][4];
#pragma unroll
                        for (int u = 0; u < R; ++u) {
                            uint4 a = make_uint4(0, 0, 0, 0);
                            if (r + u * rstep < p.outer) a = __ldcs(reinterpret_cast<const uint4*>(x + (r + u * rstep) * p.C + c));
                            w[u][0] = a.x; w[u][1] = a.y; w[u][2] = a.z; w[u][3] = a.w;
                        }
#pragma unroll
                        for (int u = 0; u < R; ++u)
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (sizeof(T) == 4) m[j] = max(m[j], w[u][j] & 0x7FFFFFFFu);
                                else {
                                    m[(2 * j) % V] = max(m[(2 * j) % V], (w[u][j] << 16) & 0x7FFFFFFFu);
                                    m[(2 * j + 1) % V] = max(m[(2 * j + 1) % V], w[u][j] & 0x7FFF0000u);
                                }
                            }
                    }
#pragma unroll
                    for (int j = 0; j < V; ++j)
                        if (m[j]) {
                            if (staged) atomicMax(col_max + c + j, m[j]);
                            else atomicMax(p.out + c + j, m[j]);
                        }
                }
            }
            if (staged) {
                __syncthreads();
                for (int64_t c = threadIdx.x; c < p.C; c += blockDim.x)
                    if (col_max[c]) atomicMax(p.out + c, col_max[c]);
            }
        } else {
            for (int64_t c = threadIdx.x; c < p.C; c += blockDim.x) {
                uint32_t m = 0;
                for (int64_t r = blockIdx.x; r < p.outer; r += gridDim.x) m = max(m, abs1<T>(x, r * p.C + c));
                if (m) atomicMax(p.out + c, m);
            }
        }
    } else {
        const uint32_t n = (uint32_t)p.n;
        uint32_t cur = 0xFFFFFFFFu, m = 0;
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
            const uint32_t row = fd_div(i, p.div_inner);
            const uint32_t c = row - fd_div(row, p.div_C) * (uint32_t)p.C;
            if (c != cur) {
                if (cur != 0xFFFFFFFFu && m) atomicMax(p.out + cur, m);
                cur = c;
                m = 0;
            }
            m = max(m, abs1<T>(x, i));
        }
        if (cur != 0xFFFFFFFFu && m) atomicMax(p.out + cur, m);
    }
    if (p.history) {
        // The CTA that draws the last ticket has every CTA's maxima behind it: it runs the observer's update for all
        // channels and leaves the maxima and the ticket at zero for the next step (no memset, no second launch).
        __shared__ int last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) last = atomicAdd(p.ticket, 1u) == gridDim.x - 1u;
        __syncthreads();
        if (last) {
            __threadfence();
            for (int64_t c = threadIdx.x; c < p.C; c += blockDim.x) {
                observer_update_one(c, __uint_as_float(__ldcg(p.out + c)), p.history, p.scale, p.H, p.C, p.qmax, p.pow2, p.stay);
                p.out[c] = 0u;
            }
            if (threadIdx.x == 0) *p.ticket = 0u;
        }
    }
}

// the reduction's launch; with `fused` the last CTA updates the observer's state (p.history etc. set by the caller)
int amax_launch(const char* name, AmaxParams p, const void* in, int dtype, int64_t outer, int64_t C, int64_t inner, cudaStream_t st);

}  // namespace

extern "C" int vq_amax(const void* in, int dtype, int64_t outer, int64_t C, int64_t inner, float* out, void* stream) {
    const char* name = "vq_amax";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(outer >= 0 && C >= 1 && inner >= 0, "%s: bad shape", name);
    VQ_REQUIRE(out != nullptr, "%s: null output", name);
    cudaStream_t st = (cudaStream_t)stream;
    VQ_CUDA(cudaMemsetAsync(out, 0, (size_t)C * sizeof(float), st));
    const int64_t n = outer * C * inner;
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr, "%s: null input", name);
    AmaxParams p{};
    p.out = reinterpret_cast<uint32_t*>(out);
    return amax_launch(name, p, in, dtype, outer, C, inner, st);
}

namespace {
int amax_launch(const char* name, AmaxParams p, const void* in, int dtype, int64_t outer, int64_t C, int64_t inner, cudaStream_t st) {
    const int64_t n = outer * C * inner;
    p.in = in;
    p.outer = outer; p.C = C; p.inner = inner; p.n = n;
    const size_t es = dtype == VQ_F32 ? 4 : 2;
    const int V = (int)(16 / es);
    const int sms = vq_sm_count();
    int mode, blocks, threads = 256;
    size_t smem = 0;
    if (inner >= 64 || (C == 1 && outer == 1)) {
        mode = 0;
        p.vec = (inner % V == 0 && (uintptr_t)in % 16 == 0) ? 1 : 0;
        const int64_t rows = outer * C;
        const int64_t want_items = (int64_t)sms * 8 * 8 * 4;
        int64_t segs = want_items / rows;
        if (segs < 1) segs = 1;
        int64_t seg_len = (inner + segs - 1) / segs;
        const int64_t quantum = 32 * V * 4;
        seg_len = (seg_len + quantum - 1) / quantum * quantum;
        p.seg_len = seg_len;
        p.segs_per_row = (inner + seg_len - 1) / seg_len;
        p.n_items = rows * p.segs_per_row;
        const int64_t want = (p.n_items + 7) / 8;
        blocks = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
    } else if (inner == 1) {
        mode = 1;
        p.vec = (C % V == 0 && (uintptr_t)in % 16 == 0) ? 1 : 0;
        p.smem_cols = (p.vec && C * 4 <= 48 * 1024) ? 1 : 0;
        threads = p.vec ? 1024 : 256;
        smem = p.smem_cols ? (size_t)C * 4 : 0;
        const int64_t cap = p.vec ? sms : (int64_t)sms * 4;
        blocks = (int)(outer < cap ? outer : cap);
    } else {
        VQ_REQUIRE(n < (1ll << 31), "%s: tensors with 1 < inner < 64 must hold fewer than 2^31 elements", name);
        mode = 2;
        p.div_inner = make_fastdiv((uint32_t)inner);
        p.div_C = make_fastdiv((uint32_t)C);
        const int64_t want = (n + 255) / 256;
        blocks = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
    }
    if (dtype == VQ_F32) {
        if (mode == 0) amax_kernel<float, 0><<<blocks, 256, 0, st>>>(p);
        else if (mode == 1) amax_kernel<float, 1><<<blocks, threads, smem, st>>>(p);
        else amax_kernel<float, 2><<<blocks, 256, 0, st>>>(p);
    } else {
        if (mode == 0) amax_kernel<bf16_t, 0><<<blocks, 256, 0, st>>>(p);
        else if (mode == 1) amax_kernel<bf16_t, 1><<<blocks, threads, smem, st>>>(p);
        else amax_kernel<bf16_t, 2><<<blocks, 256, 0, st>>>(p);
    }
    VQ_LAUNCH_CHECK("amax_kernel");
    return 0;
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// The observer's state update, quantization/fake_quantize.py:327-341, as one small kernel:
//   amax = max over the history (BEFORE the current maximum enters it);
//   history <- roll(history, -1, 0); history[0] <- amax_cur;
//   sf = amax / quant_max, keeping the previous scale where amax is 0, NaN or Inf;
//   optionally sf <- 2 ** ceil(log2(sf)).  The CPU's fp32 log2 rounds the logarithm of the first few values above a
//   power of two to the integer itself, so ceil keeps them at that power; how many values that is per exponent
//   comes from the host (`stay`, one count per biased exponent, derived from the CPU arithmetic the observer is
//   defined in), which makes the result equal to upstream's bit for bit.  Without the table (and for subnormal
//   scales) the device's own log2f / exp2f are used.
// Upstream issues about a dozen tiny tensor operations for this.
namespace {
__global__ void observer_update_kernel(const float* __restrict__ amax_cur, float* __restrict__ history, float* __restrict__ scale,
                                       int H, int64_t C, float qmax, int pow2, const uint8_t* __restrict__ stay) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    observer_update_one(c, amax_cur[c], history, scale, H, C, qmax, pow2, stay);
}
}  // namespace

extern "C" int vq_observer_update(const float* amax_cur, float* history, float* scale, int history_len, int64_t channels,
                                  double quant_max, int pow2, const uint8_t* pow2_stay, void* stream) {
    const char* name = "vq_observer_update";
    VQ_REQUIRE(amax_cur && history && scale, "%s: null pointer", name);
    VQ_REQUIRE(history_len >= 1 && channels >= 1, "%s: bad sizes", name);
    observer_update_kernel<<<(unsigned)((channels + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
        amax_cur, history, scale, history_len, channels, (float)quant_max, pow2, pow2_stay);
    VQ_LAUNCH_CHECK("observer_update_kernel");
    return 0;
}

extern "C" int vq_observer_step(const void* in, int dtype, int64_t outer, int64_t channels, int64_t inner, float* amax_scratch,
                                float* history, float* scale, int history_len, double quant_max, int pow2, const uint8_t* pow2_stay,
                                void* stream) {
    const char* name = "vq_observer_step";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(outer >= 0 && channels >= 1 && inner >= 0, "%s: bad shape", name);
    VQ_REQUIRE(amax_scratch && history && scale, "%s: null pointer", name);
    VQ_REQUIRE(history_len >= 1, "%s: bad history length", name);
    cudaStream_t st = (cudaStream_t)stream;
    if (outer * channels * inner == 0) {                  // nothing to reduce: the maxima are the zeros of the scratch
        observer_update_kernel<<<(unsigned)((channels + 127) / 128), 128, 0, st>>>(amax_scratch, history, scale, history_len, channels,
                                                                                 (float)quant_max, pow2, pow2_stay);
        VQ_LAUNCH_CHECK("observer_update_kernel");
        return 0;
    }
    VQ_REQUIRE(in != nullptr, "%s: null input", name);
    AmaxParams p{};
    p.out = reinterpret_cast<uint32_t*>(amax_scratch);
    p.ticket = reinterpret_cast<unsigned int*>(amax_scratch) + channels;
    p.history = history; p.scale = scale; p.H = history_len; p.qmax = (float)quant_max; p.pow2 = pow2; p.stay = pow2_stay;
    return amax_launch(name, p, in, dtype, outer, channels, inner, st);
}
