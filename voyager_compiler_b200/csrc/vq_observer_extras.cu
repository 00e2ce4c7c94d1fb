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
#include <cstdlib>
#include <cstring>

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

// The same histogram for large aligned tensors, without any exchange between lanes: every lane of every warp owns a
// column of 16-bit counters in shared memory, two to a 32-bit word and the words of a warp's 32 lanes in 32 different
// banks, so an element costs a few integer operations for its word and half and one `red.shared.add.u32` of 1 or 65 536:
// no lane ever meets another one's word, nothing is returned and nothing waits.
// A column has 128 rows: row r counts exponent field 64 + r, that is bin 63 + r (2^-62 <= |x| < 2^65 covers what tensors
// hold), row 0 collects the zeros; rows 2j and 2j + 1 share word j.  Everything else takes the exact rule element by element, into the CTA's totals by
// shared-memory atomics: a batch of vectors with an element outside that window, a non-zero subnormal, an infinity or
// NaN, or one of the 256 patterns at the top of a binade, which alone have to look at the thresholds (one running
// maximum and two running minima over the batch tell).  The prologue checks what that relies on (`fast`: every
// threshold of a normal binade lies among those 256 patterns; else every batch takes the exact rule).  A lane counts
// at most 65 528 elements between two flushes of its counters; 24 warps of 8 KB each hide the latency of the updates.
constexpr int kLaneWarps = 24;
constexpr int kLaneThreads = kLaneWarps * 32;
constexpr int kLaneUnroll = 4;                       // 16-byte loads per lane and buffer (two buffers take turns)
constexpr int kLaneRows = 128;
constexpr uint32_t kLaneFirstField = 64;             // row r <-> exponent field 64 + r
constexpr size_t kLaneSmem = 1120 + 1024 + (size_t)kLaneWarps * kLaneRows * 32 * sizeof(uint16_t);

// the exact rule for one element (b: fp32 pattern without the sign), added to the CTA's totals (index: bin + 1)
__device__ __noinline__ void lane_count_exact(uint32_t* totals, uint32_t b, const uint32_t* bump) {
    const int bin = exponent_bin(b, bump);
    if (bin >= 0) atomicAdd(totals + bin + 1, 1u);
}
// One element, given as its word shifted so that the exponent field sits at bits 14..7 (`f`: fp32 >> 16, the high bf16
// half >> 16, the low bf16 half as it is; other bits are ignored).  Fields 2j and 2j + 1 share word j - 32 of the lane's
// column (low and high half); a zero (field 0) is raised to word 0, whose low half no counted field uses (the window
// starts at field 65).  `col32`: shared-memory address of the column minus 32 words.  The addition returns nothing, so
// nothing waits for it.
__device__ __forceinline__ void lane_count_one(uint32_t col32, uint32_t f) {
    const uint32_t addr = col32 + max(f & 0x7F00u, (kLaneFirstField / 2u) << 8) / 2u;  // (field >> 1) * 128 bytes
    const uint32_t inc = 1u << ((f >> 3) & 16u);                                        // the field's lowest bit chooses the half
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(addr), "r"(inc) : "memory");
}

// kLaneUnroll vectors of one lane
template <typename T>
__device__ __forceinline__ void lane_count_batch(uint32_t col_addr, uint32_t* totals, const uint4 (&v)[kLaneUnroll],
                                                 const uint32_t* bump, bool fast, uint32_t top_floor) {
    // t: pattern of |x| with the exponent field at bits 30..23 (fp32) or 14..7 (bf16 halves)
    constexpr uint32_t kOne = sizeof(T) == 4 ? (1u << 23) : (1u << 7);
    constexpr uint32_t kFloor = (kLaneFirstField + 1u) * kOne;             // smallest pattern with a row of its own
    constexpr uint32_t kCeil = (kLaneFirstField + kLaneRows) * kOne;       // first pattern above the window
    uint32_t top = 0u, low = 0xFFFFFFFFu, high = 0u;
#pragma unroll
    for (int u = 0; u < kLaneUnroll; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (sizeof(T) == 4) {
                const uint32_t t = w[k] & 0x7FFFFFFFu;
                top = max(top, w[k] | 0xFF800000u);                  // mantissa field, all ones above it
                low = min(low, t - 1u);                              // a zero wraps to the top
                high = max(high, t);
            } else {
                // a bf16 mantissa ends in 16 zero bits as fp32: never among the top 256 patterns of a binade
                const uint32_t t0 = w[k] & 0x7FFFu, t1 = (w[k] >> 16) & 0x7FFFu;
                low = min(low, min(t0 - 1u, t1 - 1u));
                high = max(high, max(t0, t1));
            }
        }
    }
    if (fast && (sizeof(T) == 2 || top - 0xFF800000u < top_floor) && low >= kFloor - 1u && high < kCeil) {
#pragma unroll
        for (int u = 0; u < kLaneUnroll; ++u) {
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (sizeof(T) != 4) lane_count_one(col_addr, w[k]);
                lane_count_one(col_addr, w[k] >> 16);
            }
        }
    } else {
        // a batch with an element that needs the thresholds: that element takes the exact rule, the others stay plain
        // (a warp with such a batch would otherwise fall far behind the others of its CTA)
        auto one = [&](uint32_t b, uint32_t f) {             // b: fp32 pattern of |x|, f: as for lane_count_one
            const bool plain = fast && (b == 0u || (b >= (kLaneFirstField + 1u) << 23 && b < (kLaneFirstField + kLaneRows) << 23)) &&
                               (b & 0x007FFFFFu) < top_floor;
            if (plain) lane_count_one(col_addr, f);
            else lane_count_exact(totals, b, bump);
        };
#pragma unroll
        for (int u = 0; u < kLaneUnroll; ++u) {                     // registers only: no indexing by a loop variable
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (sizeof(T) == 4) {
                    one(w[k] & 0x7FFFFFFFu, w[k] >> 16);
                } else {
                    one((w[k] << 16) & 0x7FFF0000u, w[k]);
                    one(w[k] & 0x7FFF0000u, w[k] >> 16);
                }
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kLaneThreads, 1) exp_histogram_lanes_kernel(const T* __restrict__ x, int64_t n,
                                                                              const uint32_t* __restrict__ bump_at,
                                                                              unsigned long long* __restrict__ counts, int epoch_vectors,
                                                                              float* __restrict__ histogram) {
    extern __shared__ uint4 lanes_smem[];
    uint32_t* bump = reinterpret_cast<uint32_t*>(lanes_smem);                 // 277 thresholds (1120 bytes reserved)
    uint32_t* totals = bump + 280;                                            // this CTA's counts, index bin + 1
    uint32_t* hist = totals + 256;                                            // [warp][word][lane], two 16-bit rows per word
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kColumn16 = kLaneRows * 32 * 2 / 16;                        // 16-byte pieces of a warp's counters
    uint4* mine4 = reinterpret_cast<uint4*>(hist + (size_t)warp * (kLaneRows / 2) * 32);
    uint32_t* mine = hist + (size_t)warp * (kLaneRows / 2) * 32 + lane;
    const uint32_t col_addr = (uint32_t)__cvta_generic_to_shared(mine) - (kLaneFirstField / 2u) * 128u;   // minus 32 words
    // The smallest mantissa at which any normal binade's threshold lies (binade i - 149 is normal from i = 23 on; its
    // patterns start at (i - 22) << 23): elements below it never look at the thresholds.  `fast` wants it among the
    // top 256 patterns, so that a bf16 value (mantissa ending in 16 zero bits) never reaches it.
    __shared__ uint32_t s_top_floor;
    if (threadIdx.x == 0) s_top_floor = 0x00800000u;
    __syncthreads();
    for (int i = threadIdx.x; i < 277; i += blockDim.x) {
        const uint32_t t = bump_at[i];
        bump[i] = t;
        const uint32_t base = (uint32_t)(i - 22) << 23;
        if (i >= 23) atomicMin(&s_top_floor, t < base ? 0u : (t - base < 0x00800000u ? t - base : 0x00800000u));
    }
    for (int i = threadIdx.x; i < 256; i += blockDim.x) totals[i] = 0u;
    for (int i = lane; i < kColumn16; i += 32) mine4[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const uint32_t top_floor = s_top_floor;
    const bool fast = top_floor >= 0x007FFF00u;
    constexpr int V = 16 / (int)sizeof(T);
    const int64_t nv = n / V, stride = (int64_t)gridDim.x * blockDim.x;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    if (blockIdx.x == 0 && threadIdx.x < (int)(n - nv * V))                   // fewer than V tail elements
        lane_count_exact(totals, abs_f32_bits<T>(x[nv * V + threadIdx.x]), bump);
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool more = true;
    while (more) {
        // two register buffers take turns: the loads of the next kLaneUnroll vectors are under way while this batch is
        // counted (no copy between the buffers: an instruction that reads a loaded register waits for the load)
        if (i < nv) {
            uint4 a[kLaneUnroll], b[kLaneUnroll];
            auto load = [&](uint4(&v)[kLaneUnroll], int64_t at0) {
#pragma unroll
                for (int u = 0; u < kLaneUnroll; ++u) {
                    const int64_t at = at0 + u * stride;
                    v[u] = at < nv ? __ldcs(xv + at) : make_uint4(0u, 0u, 0u, 0u);  // zeros are not counted
                }
            };
            auto count = [&](const uint4(&v)[kLaneUnroll]) { lane_count_batch<T>(col_addr, totals, v, bump, fast, top_floor); };
            const int64_t step = kLaneUnroll * stride;
            int done = 0;
            load(a, i);
            while (true) {
                const bool has_b = i + step < nv && done + kLaneUnroll < epoch_vectors;
                if (has_b) load(b, i + step);
                count(a);
                done += kLaneUnroll;
                i += step;
                if (!has_b) break;
                const bool has_a = i + step < nv && done + kLaneUnroll < epoch_vectors;
                if (has_a) load(a, i + step);
                count(b);
                done += kLaneUnroll;
                i += step;
                if (!has_a) break;
            }
        }
        more = __syncthreads_or(i < nv ? 1 : 0) != 0;        // also: every lane's counters are final for this round
        for (int word = 0; word < kLaneRows / 2; ++word) {
            const uint32_t both = mine[word * 32];
            const uint32_t c0 = __reduce_add_sync(0xFFFFFFFFu, both & 0xFFFFu), c1 = __reduce_add_sync(0xFFFFFFFFu, both >> 16);
            if (lane == (word & 31)) {                       // fields 64 + 2 word and 65 + 2 word; field f is bin f - 1, index f
                if (c0 && word) atomicAdd(totals + kLaneFirstField + 2 * word, c0);         // word 0, low half: the zeros
                if (c1) atomicAdd(totals + kLaneFirstField + 2 * word + 1, c1);
            }
        }
        __syncwarp();
        if (more)
            for (int k = lane; k < kColumn16; k += 32) mine4[k] = make_uint4(0u, 0u, 0u, 0u);
        __syncthreads();
        for (int b = threadIdx.x; b < kBins; b += blockDim.x) {
            if (totals[b + 1]) atomicAdd(counts + b, (unsigned long long)totals[b + 1]);
            totals[b + 1] = 0u;
        }
        __syncthreads();                                     // the exact rule adds to `totals` at any time of the next round
    }
    // `histogram` given: counts[kBins] is a ticket, and the CTA that draws the last one adds the counts to the histogram
    // (the one fp32 addition per bin that `histogram += histc(...)` makes) instead of a launch of its own
    if (histogram) {
        __shared__ int last;
        __threadfence();                                     // this CTA's additions to `counts` before its ticket
        __syncthreads();
        if (threadIdx.x == 0) last = atomicAdd(counts + kBins, 1ull) == (unsigned long long)gridDim.x - 1ull;
        __syncthreads();
        if (last) {
            __threadfence();
            for (int b = threadIdx.x; b < kBins; b += blockDim.x)
                histogram[b] = __fadd_rn(histogram[b], (float)__ldcg(counts + b));
        }
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
    const bool ticket = workspace_bytes >= (kBins + 1) * sizeof(unsigned long long);      // room for the last-CTA ticket
    VQ_CUDA(cudaMemsetAsync(counts, 0, (kBins + (ticket ? 1 : 0)) * sizeof(unsigned long long), st));
    const int vec = ((uintptr_t)in % 16 == 0) ? 1 : 0;
    const int V = dtype == VQ_F32 ? 4 : 8;
    // large aligned tensors: a column of counters per lane (VOYAGER_B200_HISTOGRAM=match keeps the warp-vote kernel)
    const char* form = getenv("VOYAGER_B200_HISTOGRAM");
    if (vec && n >= (1ll << 18) && (int)kLaneSmem <= vq_max_smem_optin() && !(form && !strcmp(form, "match"))) {
        const int64_t want = (n / V + kLaneThreads - 1) / kLaneThreads;
        // a 16-bit counter holds what a lane sees between two flushes (VOYAGER_B200_HISTOGRAM_FLUSH_EVERY, tests: fewer vectors)
        int epoch = 65528 / V / kLaneUnroll * kLaneUnroll;
        if (const char* e = getenv("VOYAGER_B200_HISTOGRAM_FLUSH_EVERY")) {
            const int v = atoi(e) / kLaneUnroll * kLaneUnroll;
            if (v >= kLaneUnroll && v < epoch) epoch = v;
        }
        const int blocks = (int)(want < vq_sm_count() ? want : vq_sm_count());
        if (dtype == VQ_F32) {
            auto kern = exp_histogram_lanes_kernel<float>;
            VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLaneSmem));
            kern<<<blocks, kLaneThreads, kLaneSmem, st>>>(reinterpret_cast<const float*>(in), n, exp->bump_at, counts, epoch, ticket ? histogram : nullptr);
        } else {
            auto kern = exp_histogram_lanes_kernel<bf16_t>;
            VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLaneSmem));
            kern<<<blocks, kLaneThreads, kLaneSmem, st>>>(reinterpret_cast<const bf16_t*>(in), n, exp->bump_at, counts, epoch, ticket ? histogram : nullptr);
        }
        VQ_LAUNCH_CHECK("exp_histogram_lanes_kernel");
        if (!ticket) {
            exp_histogram_add_kernel<<<1, 256, 0, st>>>(counts, histogram);
            VQ_LAUNCH_CHECK("exp_histogram_add_kernel");
        }
        return 0;
    }
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
