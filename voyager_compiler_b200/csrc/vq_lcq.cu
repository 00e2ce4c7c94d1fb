// Statistics pass of the learned-codebook fit (upstream: src/voyager_compiler/quantization/lcq.py, unit_scale
// :136-150, Histogram.add :75-105, _accumulate :601-626): every element is divided by its block's scale
// (max(amax, 1e-12) / quant_max), binned between fp32 boundaries and adds its weight, weight * v and weight * v^2
// to three fp64 arrays.  Upstream does this with a dozen full-size tensor passes (abs, amax, divide, bucketize,
// three widenings, three index_add_); here one kernel reads the tensor once from HBM (the second sweep of a
// block comes from L1) and keeps the three arrays of a CTA in shared memory until it is done.
#include "vq_common.cuh"

namespace {

constexpr int kLcqThreads = 512;
constexpr float kLcqEps = 1e-12f;                                // lcq.py:34, as fp32

struct LcqParams {
    const void* x;
    int64_t n;
    int64_t block;               // 0: the values are already normalised
    float qmax;
    const float* weights;
    int64_t n_weights;           // 0: every weight is 1; otherwise element i takes weights[i % n_weights]
    const float* edges;          // bins + 1 ascending boundaries
    int bins;
    double* weight;
    double* total;
    double* square;
};

// Number of boundaries <= v (torch.bucketize(..., right=True)), as a bin index clamped to [0, bins - 1]: a guess
// from the (nearly uniform) spacing, then a walk to the exact place against the boundaries themselves.
__device__ __forceinline__ int bin_of(const float* edges, int n_edges, float v, float inv_step) {
    const int last = n_edges - 2;
    int b = min(max(__float2int_rd((v - edges[0]) * inv_step), 0), last);        // NaN -> 0
    while (b > 0 && edges[b] > v) --b;
    while (b < last && edges[b + 1] <= v) ++b;
    return b;
}

template <typename T>
__global__ void __launch_bounds__(kLcqThreads) lcq_accumulate_kernel(const __grid_constant__ LcqParams p) {
    extern __shared__ double sm_moments[];                       // [3][bins] doubles, then bins + 1 floats
    double* sw = sm_moments;
    double* st = sw + p.bins;
    double* ss = st + p.bins;
    float* edges = reinterpret_cast<float*>(ss + p.bins);
    for (int i = threadIdx.x; i < 3 * p.bins; i += blockDim.x) sm_moments[i] = 0.0;
    for (int i = threadIdx.x; i <= p.bins; i += blockDim.x) edges[i] = p.edges[i];
    __syncthreads();
    const T* x = reinterpret_cast<const T*>(p.x);
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
    const float inv_step = (float)p.bins / (edges[p.bins] - edges[0]);
    auto add = [&](float v, float w) {
        const int b = bin_of(edges, p.bins + 1, v, inv_step);
        const double dv = (double)v, dw = (double)w;
        atomicAdd(&sw[b], dw);
        atomicAdd(&st[b], dw * dv);
        atomicAdd(&ss[b], dw * dv * dv);
    };
    const bool small = p.n < (1ll << 31);
    if (p.block == 0) {
        for (int64_t i = tid; i < p.n; i += nthreads) {
            float w = 1.0f;
            if (p.n_weights == 1) w = p.weights[0];
            else if (p.n_weights) w = p.weights[small ? (int64_t)((uint32_t)i % (uint32_t)p.n_weights) : i % p.n_weights];
            add(load_one<T>(x + i), w);
        }
    } else {
        const int64_t nblk = p.n / p.block;
        for (int64_t b = tid; b < nblk; b += nthreads) {
            const T* xb = x + b * p.block;
            float amax = 0.0f;
            for (int64_t j = 0; j < p.block; ++j) amax = fmaxf(amax, fabsf(load_one<T>(xb + j)));
            const float scale = __fdiv_rn(fmaxf(amax, kLcqEps), p.qmax);
            int64_t c = p.n_weights > 1 ? (b * p.block) % p.n_weights : 0;       // channel of the block's first element
            for (int64_t j = 0; j < p.block; ++j) {
                float w = 1.0f;
                if (p.n_weights) w = p.weights[c];
                if (p.n_weights > 1 && ++c == p.n_weights) c = 0;
                add(__fdiv_rn(load_one<T>(xb + j), scale), w);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.bins; i += blockDim.x) {
        if (sw[i] != 0.0 || st[i] != 0.0 || ss[i] != 0.0) {
            atomicAdd(p.weight + i, sw[i]);
            atomicAdd(p.total + i, st[i]);
            atomicAdd(p.square + i, ss[i]);
        }
    }
}

// Blocks of 4 * G elements (G a power of two up to 32, so blocks of 4 ... 128): G lanes take a block, four
// consecutive elements each (one 16- or 8-byte load, coalesced over the warp), the block's maximum goes round the
// group by shuffles, and every lane bins its own four quotients.  The loads of a warp are whole lines and a lane has
// 4 elements in flight instead of a whole block read one element at a time.
template <typename T>
__device__ __forceinline__ void load4(const T* p, float* v);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* v) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<bf16_t>(const bf16_t* p, float* v) {
    const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xFFFF0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xFFFF0000u);
}

template <typename T>
__global__ void __launch_bounds__(kLcqThreads) lcq_accumulate_group_kernel(const __grid_constant__ LcqParams p, int G) {
    extern __shared__ double sm_moments[];                       // [3][bins] doubles, then bins + 1 floats
    double* sw = sm_moments;
    double* st = sw + p.bins;
    double* ss = st + p.bins;
    float* edges = reinterpret_cast<float*>(ss + p.bins);
    for (int i = threadIdx.x; i < 3 * p.bins; i += blockDim.x) sm_moments[i] = 0.0;
    for (int i = threadIdx.x; i <= p.bins; i += blockDim.x) edges[i] = p.edges[i];
    __syncthreads();
    const T* x = reinterpret_cast<const T*>(p.x);
    const float inv_step = (float)p.bins / (edges[p.bins] - edges[0]);
    const int lane = threadIdx.x & 31, sub = lane & (G - 1);
    const uint32_t gmask = (G == 32) ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int64_t groups = ((int64_t)gridDim.x * blockDim.x) / G, nblk = p.n / p.block;
    const int64_t rounds = (nblk + groups - 1) / groups;
    const int64_t g0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const bool w4 = p.n_weights > 1 && p.n_weights % 4 == 0 && (reinterpret_cast<uintptr_t>(p.weights) & 15) == 0;
    for (int64_t r = 0; r < rounds; ++r) {               // all lanes of a warp stay in the loop together
        const int64_t b = g0 + r * groups;
        const bool live = b < nblk;
        const int64_t e0 = (live ? b : 0) * p.block + sub * 4;
        float v[4], w[4] = {1.0f, 1.0f, 1.0f, 1.0f};
        load4<T>(x + e0, v);
        if (p.n_weights == 1) {
            w[0] = w[1] = w[2] = w[3] = p.weights[0];
        } else if (p.n_weights > 1) {
            const int64_t c = e0 % p.n_weights;
            if (w4) {                                     // e0 and the channel count are multiples of 4: no wrap inside
                const float4 t = __ldg(reinterpret_cast<const float4*>(p.weights + c));
                w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) w[k] = p.weights[(c + k) % p.n_weights];
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        for (int o = G >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
        const float scale = __fdiv_rn(fmaxf(amax, kLcqEps), p.qmax);
        if (live) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float q = __fdiv_rn(v[k], scale);
                const int bin = bin_of(edges, p.bins + 1, q, inv_step);
                const double dv = (double)q, dw = (double)w[k];
                atomicAdd(&sw[bin], dw);
                atomicAdd(&st[bin], dw * dv);
                atomicAdd(&ss[bin], dw * dv * dv);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.bins; i += blockDim.x) {
        if (sw[i] != 0.0 || st[i] != 0.0 || ss[i] != 0.0) {
            atomicAdd(p.weight + i, sw[i]);
            atomicAdd(p.total + i, st[i]);
            atomicAdd(p.square + i, ss[i]);
        }
    }
}

// The table a fitted codebook is used through (lcq.py:270-291): for every bf16 pattern the entry nearest to its value
// clamped to the codebook's range, distances taken in fp32 as upstream's tensor expression does, the first of equal
// distances, entry 0 for a NaN.  One thread per pattern, the entries in shared memory.
constexpr int kQmapThreads = 256;
__global__ void __launch_bounds__(kQmapThreads) codebook_qmap_kernel(const float* __restrict__ entries, int n, uint16_t* __restrict__ table) {
    extern __shared__ float cb[];
    __shared__ float s_lo, s_hi;
    for (int i = threadIdx.x; i < n; i += blockDim.x) cb[i] = entries[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        // minimum and maximum as torch.min / torch.max give them: a NaN entry makes both NaN
        float lo = cb[0], hi = cb[0];
        bool nan = cb[0] != cb[0];
        for (int i = 1; i < n; ++i) {
            nan |= cb[i] != cb[i];
            lo = fminf(lo, cb[i]);
            hi = fmaxf(hi, cb[i]);
        }
        s_lo = nan ? __uint_as_float(0x7FC00000u) : lo;
        s_hi = nan ? __uint_as_float(0x7FC00000u) : hi;
    }
    __syncthreads();
    const uint32_t pat = blockIdx.x * blockDim.x + threadIdx.x;
    if (pat >= 65536u) return;
    const float x = __uint_as_float(pat << 16);
    int best = 0;
    if (x == x) {
        // clamp(x, lo, hi) = min(max(x, lo), hi); a NaN bound passes through as torch.clamp does and ends at entry 0
        float v = (x < s_lo) ? s_lo : x;
        v = (v > s_hi) ? s_hi : v;
        if (s_lo != s_lo) v = s_lo;
        float dmin = fabsf(__fsub_rn(v, cb[0]));
        bool found_nan = dmin != dmin;
        for (int j = 1; j < n && !found_nan; ++j) {
            const float d = fabsf(__fsub_rn(v, cb[j]));
            if (d != d) {                                  // argmin takes the first NaN for the minimum
                best = j;
                found_nan = true;
            } else if (d < dmin) {
                dmin = d;
                best = j;
            }
        }
    }
    table[pat] = (uint16_t)(f32_to_bf16_bits(cb[best]));
}

}  // namespace

extern "C" int vq_codebook_qmap(const float* entries, int n, uint16_t* table, void* stream) {
    const char* name = "vq_codebook_qmap";
    VQ_REQUIRE(n >= 1 && n <= 8192, "%s: between 1 and 8192 entries", name);
    VQ_REQUIRE(entries && table, "%s: null pointer", name);
    codebook_qmap_kernel<<<65536 / kQmapThreads, kQmapThreads, (size_t)n * sizeof(float), (cudaStream_t)stream>>>(entries, n, table);
    VQ_LAUNCH_CHECK("codebook_qmap_kernel");
    return 0;
}

extern "C" int vq_lcq_accumulate(const void* x, int dtype, int64_t n, int64_t block, double quant_max, const float* weights,
                                 int64_t n_weights, const float* edges, int bins, double* weight, double* total,
                                 double* square, void* stream) {
    const char* name = "vq_lcq_accumulate";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(n >= 0 && block >= 0 && bins >= 1 && n_weights >= 0, "%s: bad sizes", name);
    VQ_REQUIRE(block == 0 || n % block == 0, "%s: the element count must be a whole number of blocks", name);
    VQ_REQUIRE(block == 0 || quant_max > 0, "%s: quant_max must be positive", name);
    if (n == 0) return 0;
    VQ_REQUIRE(x && edges && weight && total && square && (n_weights == 0 || weights), "%s: null pointer", name);
    const size_t smem = (size_t)bins * 3 * sizeof(double) + ((size_t)bins + 1) * sizeof(float);
    if ((int)smem > vq_max_smem_optin())
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: %d bins do not fit the shared memory of a CTA", name, bins);
    LcqParams p{};
    p.x = x; p.n = n; p.block = block; p.qmax = (float)quant_max;
    p.weights = weights; p.n_weights = n_weights; p.edges = edges; p.bins = bins;
    p.weight = weight; p.total = total; p.square = square;
    // blocks of 4, 8, ... 128 elements of an aligned tensor: a group of lanes per block
    const int64_t esize = dtype == VQ_F32 ? 4 : 2;
    int G = 0;
    if (block >= 4 && block <= 128 && (block & (block - 1)) == 0 && (uintptr_t)x % (4 * esize) == 0) G = (int)(block / 4);
    const int64_t items = G ? n / 4 : (block ? n / block : n);      // what a thread takes per round
    const int sms = vq_sm_count();
    const int per_sm = smem > 100 * 1024 ? 2 : (smem > 50 * 1024 ? 3 : 4);
    int64_t want = (items + kLcqThreads - 1) / kLcqThreads;
    // a CTA pays for clearing and flushing its arrays: at least some tens of thousands of elements each
    const int64_t by_work = (n + 32767) / 32768;
    if (want > by_work) want = by_work;
    const int blocks = (int)(want < 1 ? 1 : (want > (int64_t)sms * per_sm ? (int64_t)sms * per_sm : want));
    cudaStream_t st = (cudaStream_t)stream;
    if (G) {
        if (dtype == VQ_F32) {
            VQ_CUDA(cudaFuncSetAttribute(lcq_accumulate_group_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            lcq_accumulate_group_kernel<float><<<blocks, kLcqThreads, smem, st>>>(p, G);
        } else {
            VQ_CUDA(cudaFuncSetAttribute(lcq_accumulate_group_kernel<bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            lcq_accumulate_group_kernel<bf16_t><<<blocks, kLcqThreads, smem, st>>>(p, G);
        }
        VQ_LAUNCH_CHECK("lcq_accumulate_group_kernel");
        return 0;
    }
    if (dtype == VQ_F32) {
        VQ_CUDA(cudaFuncSetAttribute(lcq_accumulate_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        lcq_accumulate_kernel<float><<<blocks, kLcqThreads, smem, st>>>(p);
    } else {
        VQ_CUDA(cudaFuncSetAttribute(lcq_accumulate_kernel<bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        lcq_accumulate_kernel<bf16_t><<<blocks, kLcqThreads, smem, st>>>(p);
    }
    VQ_LAUNCH_CHECK("lcq_accumulate_kernel");
    return 0;
}
