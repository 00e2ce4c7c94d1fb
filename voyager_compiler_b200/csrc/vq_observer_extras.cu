// The two optional steps of FusedAmaxObsFakeQuantize.forward around the fake-quantize itself
// (quantization/fake_quantize.py:368-432):
//
//   * record_histogram (:369-371): histogram += histc(floor(log2(|x| as fp32)), 254, min=-126, max=127).
//     The 254 bins over [-126, 127] are 253/254 wide, but every integer k + 126 still lands in bin
//     k + 126 (k/253 * 254 = k + k/253), the maximum 127 in the last one.  Zeros (-inf), subnormals
//     (below -126) and infinities fall outside the range and are not counted; NaNs are not counted
//     here either.  floor(log2(x)) is the exponent field, plus one for the few
//     patterns just below a power of two whose fp32 logarithm rounds up to the next integer: the same
//     per-exponent thresholds the shared-exponent rule uses (vq_exp_tables.bump_at, derived on the host
//     from torch's own log2).
//   * outlier filtering (:388-394, :428-430): skip = |x| >= threshold (threshold rounded to the dtype
//     of x, as torch promotes a scalar or 0-dim tensor); the quantizer sees x with the skipped
//     elements set to zero, and they come back unchanged afterwards.
//
// All three kernels are HBM streams: sizeof(T) read per element for the histogram, sizeof(T) read +
// sizeof(T) written for the split, 2 x sizeof(T) read + sizeof(T) written for the merge.
#include "vq_common.cuh"

namespace {

constexpr int kBins = 254;
constexpr int kHistThreads = 256;

template <typename T>
__device__ __forceinline__ uint32_t abs_f32_bits(T v);
template <>
__device__ __forceinline__ uint32_t abs_f32_bits<float>(float v) { return __float_as_uint(v) & 0x7FFFFFFFu; }
template <>
__device__ __forceinline__ uint32_t abs_f32_bits<bf16_t>(bf16_t v) { return ((uint32_t)v.bits << 16) & 0x7FFFFFFFu; }

// bin of one element, or -1 when it is not counted
__device__ __forceinline__ int exponent_bin(uint32_t b, const uint32_t* bump) {
    if (b == 0u || b >= 0x7F800000u) return -1;
    int e = (b >= 0x00800000u) ? (int)(b >> 23) - 127 : (31 - __clz(b)) - 149;
    e += (b >= bump[e + 149]) ? 1 : 0;
    return (e >= -126 && e <= 127) ? e + 126 : -1;
}

// Lanes with the same bin elect a leader that adds their number to the warp's own histogram: one
// shared-memory update per distinct bin and warp instruction, no atomics (a warp owns its histogram).
__device__ __forceinline__ void warp_count(uint32_t* hist, int bin) {
    const uint32_t peers = __match_any_sync(__activemask(), bin);
    if (bin >= 0 && (threadIdx.x & 31) == (uint32_t)(__ffs(peers) - 1)) hist[bin] += __popc(peers);
    __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(kHistThreads) exp_histogram_kernel(const T* __restrict__ x, int64_t n, const uint32_t* __restrict__ bump_at,
                                                                     unsigned long long* __restrict__ counts, int vec) {
    __shared__ uint32_t bump[277];
    __shared__ uint32_t hist[kHistThreads / 32][256];
    for (int i = threadIdx.x; i < 277; i += blockDim.x) bump[i] = bump_at[i];
    for (int i = threadIdx.x; i < (kHistThreads / 32) * 256; i += blockDim.x) (&hist[0][0])[i] = 0u;
    __syncthreads();
    uint32_t* mine = hist[threadIdx.x >> 5];
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        const int64_t nv = n / V;
        // whole warps run the loop together (the leader election needs converged lanes per call)
        const int64_t nv_round = (nv + 31) / 32 * 32;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv_round; i += stride) {
            __align__(16) T v[V];
            const bool live = i < nv;
            if (live) *reinterpret_cast<uint4*>(v) = __ldcs(reinterpret_cast<const uint4*>(x) + i);
#pragma unroll
            for (int j = 0; j < V; ++j) warp_count(mine, live ? exponent_bin(abs_f32_bits<T>(v[j]), bump) : -1);
        }
        if (blockIdx.x == 0 && threadIdx.x < 32) {
            const int64_t e = nv * V + threadIdx.x;          // fewer than V <= 8 tail elements
            warp_count(mine, (e < n) ? exponent_bin(abs_f32_bits<T>(x[e]), bump) : -1);
        }
    } else {
        const int64_t n_round = (n + 31) / 32 * 32;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_round; i += stride)
            warp_count(mine, (i < n) ? exponent_bin(abs_f32_bits<T>(x[i]), bump) : -1);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < kBins; b += blockDim.x) {
        unsigned long long c = 0;
#pragma unroll
        for (int w = 0; w < kHistThreads / 32; ++w) c += hist[w][b];
        if (c) atomicAdd(counts + b, c);
    }
}

// histogram[b] += float(count[b]): the one fp32 addition per bin and call that `histogram += histc(...)` makes
__global__ void exp_histogram_add_kernel(const unsigned long long* __restrict__ counts, float* __restrict__ histogram) {
    const int b = threadIdx.x;
    if (b < kBins) histogram[b] = __fadd_rn(histogram[b], (float)counts[b]);
}

template <typename T>
__device__ __forceinline__ T zero_of();
template <>
__device__ __forceinline__ float zero_of<float>() { return 0.0f; }
template <>
__device__ __forceinline__ bf16_t zero_of<bf16_t>() { bf16_t z; z.bits = 0; return z; }

// threshold in the dtype of x, as fp32 bits of its magnitude comparison: |x| >= thr  (false for NaN on either side)
template <typename T>
__device__ __forceinline__ float load_threshold(const float* thr) {
    const float t = *thr;
    return sizeof(T) == 4 ? t : bf16_bits_to_f32(f32_to_bf16_bits(t));
}
template <typename T>
__device__ __forceinline__ bool is_outlier(T v, float thr) { return __uint_as_float(abs_f32_bits<T>(v)) >= thr; }

template <typename T>
__global__ void __launch_bounds__(256) outlier_split_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ thr_p,
                                                            T* __restrict__ inliers, unsigned long long* __restrict__ n_outliers, int vec) {
    const float thr = load_threshold<T>(thr_p);
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t found = 0;
    const int64_t nv = vec ? n / V : 0;
    for (int64_t i = tid; i < nv; i += stride) {
        __align__(16) T v[V];
        *reinterpret_cast<uint4*>(v) = __ldcs(reinterpret_cast<const uint4*>(x) + i);
#pragma unroll
        for (int j = 0; j < V; ++j)
            if (is_outlier<T>(v[j], thr)) {
                v[j] = zero_of<T>();
                ++found;
            }
        reinterpret_cast<uint4*>(inliers)[i] = *reinterpret_cast<uint4*>(v);
    }
    for (int64_t e = nv * V + tid; e < n; e += stride) {
        T v = x[e];
        if (is_outlier<T>(v, thr)) {
            v = zero_of<T>();
            ++found;
        }
        inliers[e] = v;
    }
    found = __reduce_add_sync(0xFFFFFFFFu, found);
    if ((threadIdx.x & 31) == 0 && found) atomicAdd(n_outliers, (unsigned long long)found);
}

template <typename T>
__global__ void __launch_bounds__(256) outlier_merge_kernel(const T* __restrict__ x, const T* __restrict__ y, int64_t n,
                                                            const float* __restrict__ thr_p, T* __restrict__ out, int vec) {
    const float thr = load_threshold<T>(thr_p);
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nv = vec ? n / V : 0;
    for (int64_t i = tid; i < nv; i += stride) {
        __align__(16) T a[V];
        __align__(16) T b[V];
        *reinterpret_cast<uint4*>(a) = __ldcs(reinterpret_cast<const uint4*>(x) + i);
        *reinterpret_cast<uint4*>(b) = __ldcs(reinterpret_cast<const uint4*>(y) + i);
#pragma unroll
        for (int j = 0; j < V; ++j)
            if (is_outlier<T>(a[j], thr)) b[j] = a[j];
        __stcs(reinterpret_cast<uint4*>(out) + i, *reinterpret_cast<uint4*>(b));
    }
    for (int64_t e = nv * V + tid; e < n; e += stride) out[e] = is_outlier<T>(x[e], thr) ? x[e] : y[e];
}

inline int stream_blocks(int64_t work_items, int threads) {
    const int64_t cap = (int64_t)vq_sm_count() * 8;
    const int64_t want = (work_items + threads - 1) / threads;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

extern "C" {

int vq_exp_histogram(const void* in, int dtype, int64_t n, const vq_exp_tables* exp, float* histogram, void* workspace,
                     size_t workspace_bytes, void* stream) {
    const char* name = "vq_exp_histogram";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(n >= 0 && histogram != nullptr, "%s: negative size or null histogram", name);
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr && exp != nullptr && exp->bump_at != nullptr, "%s: null input or exponent thresholds (fp32 tables)", name);
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 8 == 0 && workspace_bytes >= kBins * sizeof(unsigned long long),
               "%s: workspace of at least 2032 bytes, 8-byte aligned", name);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned long long* counts = reinterpret_cast<unsigned long long*>(workspace);
    VQ_CUDA(cudaMemsetAsync(counts, 0, kBins * sizeof(unsigned long long), st));
    const int vec = ((uintptr_t)in % 16 == 0) ? 1 : 0;
    const int V = dtype == VQ_F32 ? 4 : 8;
    const int blocks = stream_blocks(vec ? (n + V - 1) / V : n, kHistThreads);
    if (dtype == VQ_F32)
        exp_histogram_kernel<float><<<blocks, kHistThreads, 0, st>>>(reinterpret_cast<const float*>(in), n, exp->bump_at, counts, vec);
    else
        exp_histogram_kernel<bf16_t><<<blocks, kHistThreads, 0, st>>>(reinterpret_cast<const bf16_t*>(in), n, exp->bump_at, counts, vec);
    VQ_LAUNCH_CHECK("exp_histogram_kernel");
    exp_histogram_add_kernel<<<1, 256, 0, st>>>(counts, histogram);
    VQ_LAUNCH_CHECK("exp_histogram_add_kernel");
    return 0;
}

int vq_outlier_split(const void* in, int dtype, int64_t n, const float* threshold, void* inliers, unsigned long long* n_outliers,
                     void* stream) {
    const char* name = "vq_outlier_split";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(n >= 0 && threshold != nullptr && n_outliers != nullptr, "%s: negative size, null threshold or null counter", name);
    cudaStream_t st = (cudaStream_t)stream;
    VQ_CUDA(cudaMemsetAsync(n_outliers, 0, sizeof(unsigned long long), st));
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr && inliers != nullptr, "%s: null tensor", name);
    const int vec = ((uintptr_t)in % 16 == 0 && (uintptr_t)inliers % 16 == 0) ? 1 : 0;
    const int V = dtype == VQ_F32 ? 4 : 8;
    const int blocks = stream_blocks(vec ? (n + V - 1) / V : n, 256);
    if (dtype == VQ_F32)
        outlier_split_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(in), n, threshold,
                                                            reinterpret_cast<float*>(inliers), n_outliers, vec);
    else
        outlier_split_kernel<bf16_t><<<blocks, 256, 0, st>>>(reinterpret_cast<const bf16_t*>(in), n, threshold,
                                                             reinterpret_cast<bf16_t*>(inliers), n_outliers, vec);
    VQ_LAUNCH_CHECK("outlier_split_kernel");
    return 0;
}

int vq_outlier_merge(const void* in, const void* quantized, int dtype, int64_t n, const float* threshold, void* out, void* stream) {
    const char* name = "vq_outlier_merge";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(n >= 0 && threshold != nullptr, "%s: negative size or null threshold", name);
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr && quantized != nullptr && out != nullptr, "%s: null tensor", name);
    const int vec = ((uintptr_t)in % 16 == 0 && (uintptr_t)quantized % 16 == 0 && (uintptr_t)out % 16 == 0) ? 1 : 0;
    const int V = dtype == VQ_F32 ? 4 : 8;
    const int blocks = stream_blocks(vec ? (n + V - 1) / V : n, 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VQ_F32)
        outlier_merge_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(in), reinterpret_cast<const float*>(quantized),
                                                            n, threshold, reinterpret_cast<float*>(out), vec);
    else
        outlier_merge_kernel<bf16_t><<<blocks, 256, 0, st>>>(reinterpret_cast<const bf16_t*>(in), reinterpret_cast<const bf16_t*>(quantized),
                                                             n, threshold, reinterpret_cast<bf16_t*>(out), vec);
    VQ_LAUNCH_CHECK("outlier_merge_kernel");
    return 0;
}

}  // extern "C"
