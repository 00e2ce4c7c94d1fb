// Per-row codebook quantization: every row of x[rows, K] has its own sorted codebook
// levels[row, 0..n); each element gets the index of its nearest level and, optionally, that level.
//
// The rule is the upstream codebook rule (quantization/lcq.py:270-291: clamp to the codebook range,
// |x - level| in fp32, first minimum wins, NaN -> entry 0) applied per row.  With `round_bf16` the
// element is rounded to bf16 first and the returned level is rounded to bf16, which is what the
// upstream 65 536-entry table + `vmap` (ops/quantized.py:98-121) compute for a per-tensor codebook;
// without it the search runs on the fp32 element and returns the fp32 level.
//
// fp32 rounding of a difference is monotone in the true distance, so the argmin over all levels sits
// at one of the two neighbours of x in the sorted row, and for each adjacent pair (a, b) the set of x
// that prefer b, { x : fl(b - x) < fl(x - a) }, is an up-set: it has a smallest member, the pair's
// THRESHOLD.  The index of the nearest level is therefore the number of thresholds <= x, which also
// covers the clamp (below the first threshold -> 0, above the last -> n - 1) and NaN (no comparison
// holds -> 0).
//   1. row_thresholds_kernel: one thread per pair finds its threshold exactly, by bisection over the
//      ordered fp32 bit patterns between a and b (<= 32 evaluations of the predicate), into a
//      workspace of n floats per row.  Rows whose levels are so close that rounded distances of
//      non-neighbours can coincide (a gap below 2^-20 of the row's range, duplicates included) are
//      flagged instead.
//   2. row_codebook_kernel: one warp per (row, segment); thresholds and levels of the row sit in the
//      warp's slice of shared memory; per element a branchless lower bound over the thresholds (the
//      first two probes from registers, the rest from shared memory) and one read of the level.
//      Flagged rows take the direct form: lower bound over the levels, the two subtractions, and a
//      walk down to the lowest index with the same rounded distance, as argmin does.
// HBM bound: sizeof(T) read + 1 (index) + sizeof(T) (level) written per element.
#include <math_constants.h>

#include "vq_common.cuh"

namespace {

constexpr int kWarps = 8;          // per CTA
constexpr int kMaxLevels = 256;
constexpr int kPasses = 4;       // 16-byte loads in flight per lane

struct RowCbParams {
    const void* x;
    const float* levels;
    float* work;                   // [rows, n_levels]: [0] = 1 when the row is flagged, [k] = threshold of pair (k-1, k)
    uint8_t* idx;
    void* deq;
    int64_t rows, K;
    int64_t seg_len;               // elements per work item, a multiple of 128 * kPasses
    int64_t segs_per_row, n_items;
    int n_levels;
    int round_bf16;
};

// ---------------------------------------------------------------------------------------------
// order-preserving map between fp32 values and unsigned keys
__device__ __forceinline__ uint32_t key_of(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float value_of(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

__global__ void row_thresholds_kernel(const float* __restrict__ levels, float* __restrict__ work, int64_t rows, int n) {
    // one thread per (row, k): k = 0 classifies the row, k >= 1 bisects the threshold of pair (k-1, k)
    const int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= rows * n) return;
    const int64_t row = id / n;
    const int k = (int)(id - row * n);
    const float* lv = levels + row * n;
    if (k == 0) {
        const float lo = lv[0], hi = lv[n - 1];
        float min_gap = CUDART_INF_F;
        for (int i = 1; i < n; ++i) min_gap = fminf(min_gap, lv[i] - lv[i - 1]);
        // a finite, strictly increasing row whose smallest gap is well above the rounding of any distance
        const bool clear = n == 1 || (min_gap > (hi - lo) * 9.5367431640625e-07f && (hi - lo) < CUDART_INF_F);
        work[id] = clear ? 0.0f : 1.0f;
        return;
    }
    const float a = lv[k - 1], b = lv[k];
    float t = CUDART_NAN_F;
    if (a < b) {
        uint32_t klo = key_of(a), khi = key_of(b);       // the predicate is false at a, true at b
        while (khi - klo > 1u) {
            const uint32_t mid = klo + ((khi - klo) >> 1);
            const float x = value_of(mid);
            if ((b - x) < (x - a)) khi = mid; else klo = mid;
        }
        t = value_of(khi);
    }
    work[id] = t;                                       // unused when the row is flagged
}

// ---------------------------------------------------------------------------------------------
// Shared-memory reads by 32-bit address with a compile-time byte offset.  volatile: the slots are
// rewritten for every row, so the reads must stay where they are written (between the warp barriers).
template <int OFF>
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
    return v;
}
__device__ __forceinline__ uint32_t bf16x2_of(float hi, float lo) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// Per-warp slot.  raw: [0] = -inf, [1 .. n] = the row's levels, then +inf.  rounded: the same
// rounded to bf16.  thr: [0 .. n-2] = thresholds of the pairs (0,1) .. (n-2,n-1), then NaN (never
// <= x).  Byte offsets between the arrays are compile-time constants.
template <int LOG2N>
struct Slot {
    static constexpr int NP = 1 << LOG2N;
    float raw[NP + 4];
    float rounded[NP + 4];
    float thr[NP + 4];
    static constexpr int kRoundedFromRaw = (NP + 4) * 4;
    static constexpr int kRawFromThr = -2 * (NP + 4) * 4 + 4;         // thr[i] -> raw[1 + i]
    static constexpr int kRoundedFromThr = -(NP + 4) * 4 + 4;         // thr[i] -> rounded[1 + i]
};

template <int S>
__device__ __forceinline__ float probe(uint32_t addr) { return lds_f32<((1 << S) - 1) * 4>(addr); }

// Fast form: index = number of thresholds <= x.  Four elements in lockstep.
template <int LOG2N, bool ROUNDED_OUT>
__device__ __forceinline__ uint32_t count4(uint32_t tbase, float tm, float tl, float th, const float* x, float* val) {
    uint32_t off[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // probes thr[NP/2 - 1], then thr[NP/4 - 1] or thr[3 NP/4 - 1]: the same for the whole row
        const bool up = tm <= x[j];
        off[j] = up ? (4u << (LOG2N - 1)) : 0u;
        off[j] += ((up ? th : tl) <= x[j]) ? (4u << (LOG2N - 2)) : 0u;
    }
#pragma unroll
    for (int s = LOG2N - 3; s >= 0; --s) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float t;
            switch (s) {                                // the probe offset must be an immediate
                case 5: t = probe<5>(tbase + off[j]); break;
                case 4: t = probe<4>(tbase + off[j]); break;
                case 3: t = probe<3>(tbase + off[j]); break;
                case 2: t = probe<2>(tbase + off[j]); break;
                case 1: t = probe<1>(tbase + off[j]); break;
                default: t = probe<0>(tbase + off[j]); break;
            }
            off[j] += (t <= x[j]) ? (4u << s) : 0u;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        val[j] = ROUNDED_OUT ? lds_f32<Slot<LOG2N>::kRoundedFromThr>(tbase + off[j]) : lds_f32<Slot<LOG2N>::kRawFromThr>(tbase + off[j]);
    return (off[0] >> 2) + off[1] * 64u + off[2] * 16384u + off[3] * 4194304u;
}

// Direct form for flagged rows: lower bound over the levels, two subtractions, walk down over ties.
template <int LOG2N, bool ROUNDED_OUT>
__device__ __forceinline__ uint32_t nearest4(uint32_t base, float lo, float hi, const float* x, float* val) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float xc = fminf(fmaxf(x[j], lo), hi);    // a NaN becomes lo and lands on entry 0
        uint32_t addr = base;                           // ends at the first level that is not below xc
#pragma unroll
        for (int s = LOG2N - 1; s >= 0; --s) {
            float t;
            switch (s) {
                case 7: t = probe<7>(addr); break;
                case 6: t = probe<6>(addr); break;
                case 5: t = probe<5>(addr); break;
                case 4: t = probe<4>(addr); break;
                case 3: t = probe<3>(addr); break;
                case 2: t = probe<2>(addr); break;
                case 1: t = probe<1>(addr); break;
                default: t = probe<0>(addr); break;
            }
            addr += (t < xc) ? (4u << s) : 0u;
        }
        const float r = lds_f32<0>(addr);               // r >= xc > l   (l = -inf left of level 0)
        const float l = lds_f32<-4>(addr);
        const float dr = r - xc, dl = xc - l;
        uint32_t a = addr;
        if (!(dr < dl)) {                               // a tie goes to the lower index
            a -= 4u;
            while (a > base && (xc - lds_f32<-4>(a)) == dl) a -= 4u;
        }
        val[j] = ROUNDED_OUT ? lds_f32<Slot<LOG2N>::kRoundedFromRaw>(a) : lds_f32<0>(a);
        packed |= ((a - base) >> 2) << (8 * j);
    }
    return packed;
}

template <typename T, int LOG2N, bool VEC>
__global__ void __launch_bounds__(kWarps * 32) row_codebook_kernel(const RowCbParams p) {
    constexpr int NP = 1 << LOG2N;
    __shared__ Slot<LOG2N> slots[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    Slot<LOG2N>& slot = slots[warp];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(&slot.raw[1]);
    const uint32_t tbase = (uint32_t)__cvta_generic_to_shared(&slot.thr[0]);
    const T* x = reinterpret_cast<const T*>(p.x);
    T* deq = reinterpret_cast<T*>(p.deq);
    const bool rb = p.round_bf16 != 0;
    const bool rounded_out = rb || sizeof(T) == 2;
    const int n = p.n_levels;
    const int64_t n_warps = (int64_t)gridDim.x * kWarps;
    int64_t cached_row = -1;
    float lo = 0.0f, hi = 0.0f, tm = 0.0f, tl = 0.0f, th = 0.0f;
    bool flagged = true;
    // Rows of up to 16 levels: lane i fetches level i, threshold i and the flag of the NEXT item's row
    // while the current item is processed, so that the row switch costs no trip to memory.
    constexpr bool kPrefetch = LOG2N <= 4;
    float nv = 0.0f, nt = 0.0f, nf = 0.0f;
    auto fetch_row = [&](int64_t row) {
        const float* lv = p.levels + row * n;
        const float* wk = p.work + row * n;
        nv = lane < n ? __ldg(lv + lane) : CUDART_INF_F;
        nt = lane + 1 < n ? __ldg(wk + lane + 1) : CUDART_NAN_F;
        nf = __ldg(wk);
    };
    const int64_t first_item = (int64_t)blockIdx.x * kWarps + warp;
    if (kPrefetch && first_item < p.n_items) fetch_row(first_item / p.segs_per_row);
    for (int64_t item = first_item; item < p.n_items; item += n_warps) {
        const int64_t row = item / p.segs_per_row;
        const uint32_t k_begin = (uint32_t)((item - row * p.segs_per_row) * p.seg_len);
        const uint32_t k_end = (uint32_t)(k_begin + p.seg_len < p.K ? k_begin + p.seg_len : p.K);
        if (row != cached_row) {
            __syncwarp();
            if (kPrefetch) {
                if (lane <= NP) {
                    slot.raw[1 + lane] = nv;
                    slot.rounded[1 + lane] = Arith<bf16_t>::rnd(nv);
                    slot.thr[lane] = nt;
                }
                flagged = nf != 0.0f;
            } else {
                const float* lv = p.levels + row * n;
                const float* wk = p.work + row * n;
                for (int i = lane; i <= NP; i += 32) {
                    const float v = i < n ? __ldg(lv + i) : CUDART_INF_F;
                    slot.raw[1 + i] = v;
                    slot.rounded[1 + i] = Arith<bf16_t>::rnd(v);
                    slot.thr[i] = i + 1 < n ? __ldg(wk + i + 1) : CUDART_NAN_F;
                }
                flagged = __ldg(wk) != 0.0f;
            }
            if (lane == 0) { slot.raw[0] = -CUDART_INF_F; slot.rounded[0] = -CUDART_INF_F; }
            __syncwarp();
            lo = lds_f32<0>(base);
            hi = lds_f32<0>(base + 4u * (uint32_t)(n - 1));
            tm = lds_f32<(NP / 2 - 1) * 4>(tbase);
            tl = lds_f32<(NP / 4 - 1) * 4>(tbase);
            th = lds_f32<(NP / 2 + NP / 4 - 1) * 4>(tbase);
            cached_row = row;
        }
        if (kPrefetch && item + n_warps < p.n_items) {
            const int64_t next_row = (item + n_warps) / p.segs_per_row;
            if (next_row != row) fetch_row(next_row);
        }
        const T* xr = x + row * p.K;
        uint8_t* ir = p.idx ? p.idx + row * p.K : nullptr;
        T* dr_ = deq ? deq + row * p.K : nullptr;
        auto search4 = [&](const float* in, float* out) -> uint32_t {
            if (flagged)
                return rounded_out ? nearest4<LOG2N, true>(base, lo, hi, in, out) : nearest4<LOG2N, false>(base, lo, hi, in, out);
            return rounded_out ? count4<LOG2N, true>(tbase, tm, tl, th, in, out) : count4<LOG2N, false>(tbase, tm, tl, th, in, out);
        };
        if (VEC) {
            // four elements per lane and pass, kPasses passes in flight
            for (uint32_t k = k_begin + lane * 4; k < k_end; k += 128 * kPasses) {
                float v[kPasses][4];
#pragma unroll
                for (int h = 0; h < kPasses; ++h) {
                    const uint32_t kk = k + 128 * h;
                    if (kk >= k_end) break;
                    if (sizeof(T) == 4) {
                        const float4 a = __ldcs(reinterpret_cast<const float4*>(xr + kk));
                        v[h][0] = a.x; v[h][1] = a.y; v[h][2] = a.z; v[h][3] = a.w;
                    } else {
                        const uint2 a = __ldcs(reinterpret_cast<const uint2*>(xr + kk));
                        v[h][0] = __uint_as_float(a.x << 16); v[h][1] = __uint_as_float(a.x & 0xFFFF0000u);
                        v[h][2] = __uint_as_float(a.y << 16); v[h][3] = __uint_as_float(a.y & 0xFFFF0000u);
                    }
                }
#pragma unroll
                for (int h = 0; h < kPasses; ++h) {
                    const uint32_t kk = k + 128 * h;
                    if (kk >= k_end) break;
                    if (rb && sizeof(T) == 4) {
                        // round the elements to bf16 (a NaN stays a NaN)
                        const uint32_t p01 = bf16x2_of(v[h][1], v[h][0]), p23 = bf16x2_of(v[h][3], v[h][2]);
                        v[h][0] = __uint_as_float(p01 << 16); v[h][1] = __uint_as_float(p01 & 0xFFFF0000u);
                        v[h][2] = __uint_as_float(p23 << 16); v[h][3] = __uint_as_float(p23 & 0xFFFF0000u);
                    }
                    float out[4];
                    const uint32_t packed = search4(v[h], out);
                    if (ir) __stcs(reinterpret_cast<uint32_t*>(ir + kk), packed);
                    if (dr_) {
                        if (sizeof(T) == 4) {
                            __stcs(reinterpret_cast<float4*>(dr_ + kk), make_float4(out[0], out[1], out[2], out[3]));
                        } else {
                            __stcs(reinterpret_cast<uint2*>(dr_ + kk), make_uint2(bf16x2_of(out[1], out[0]), bf16x2_of(out[3], out[2])));
                        }
                    }
                }
            }
        } else {
            for (uint32_t k = k_begin + lane; k < k_end; k += 32) {
                float v[4], out[4];
                if (sizeof(T) == 4) v[0] = __ldcs(reinterpret_cast<const float*>(xr) + k);
                else v[0] = bf16_bits_to_f32(__ldcs(reinterpret_cast<const unsigned short*>(xr) + k));
                if (rb) v[0] = Arith<bf16_t>::rnd(v[0]);
                v[1] = v[2] = v[3] = v[0];
                const uint32_t packed = search4(v, out);
                if (ir) ir[k] = (uint8_t)(packed & 0xFFu);
                if (dr_) {
                    if (sizeof(T) == 4) reinterpret_cast<float*>(dr_)[k] = out[0];
                    else reinterpret_cast<unsigned short*>(dr_)[k] = (unsigned short)f32_to_bf16_bits(out[0]);
                }
            }
        }
    }
}

template <typename T, int LOG2N>
void launch_row_codebook(const RowCbParams& p, bool vec, int blocks, cudaStream_t st) {
    if (vec) row_codebook_kernel<T, LOG2N, true><<<blocks, kWarps * 32, 0, st>>>(p);
    else row_codebook_kernel<T, LOG2N, false><<<blocks, kWarps * 32, 0, st>>>(p);
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// The fit of the per-row codebooks: out[row, k] = quantile of the row at q_k = (2k + 1) / (2n),
// linear interpolation, exactly as torch.quantile evaluates it on the CPU in fp32:
//   rank = q * (K - 1) (fp32), lo = floor(rank), w = rank - lo, a = sorted[lo], b = sorted[ceil(rank)],
//   w < 0.5 ? fma(w, b - a, a) : fma(-(b - a), 1 - w, b);  a row holding a NaN gives NaN.
// One CTA per row: the row is sorted in shared memory as order-preserving integer keys (bitonic
// network over the next power of two, padded with the largest key), then n threads interpolate.
namespace {

constexpr int kQuantThreads = 512;

template <typename T>
__device__ __forceinline__ float load_elem(const T* p);
template <>
__device__ __forceinline__ float load_elem<float>(const float* p) { return __ldcs(p); }
template <>
__device__ __forceinline__ float load_elem<bf16_t>(const bf16_t* p) {
    return bf16_bits_to_f32(__ldcs(reinterpret_cast<const unsigned short*>(p)));
}

// Shared-memory position of sort index i: index bits 5..9 are folded onto the bank bits, so that both the
// unit-stride accesses of the wide windows and the stride-8 accesses of the lowest window spread over all banks.
__device__ __forceinline__ int sort_slot(int i) { return i ^ ((i >> 5) & 31); }

// One compare-exchange stage of the bitonic network on the eight keys a thread holds: pairs differ in bit SB of
// the register index; the direction of a pair is ascending where bit `mbit` of its sort index is clear.
template <int SB>
__device__ __forceinline__ void sort_stage(uint32_t (&v)[8], bool base_up, int jm) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j & (1 << SB)) continue;
        const int j2 = j | (1 << SB);
        const bool up = base_up && ((j & jm) == 0);
        const uint32_t lo = min(v[j], v[j2]), hi = max(v[j], v[j2]);
        v[j] = up ? lo : hi;
        v[j2] = up ? hi : lo;
    }
}

// Stages (m, s) for m = m_lo..m_hi, s = min(s_hi, m - 1) down to s_lo of the network over P = 2^p keys, all of
// whose stride bits lie in the window b..b+2: each thread takes the eight keys that differ in those three index
// bits, runs the stages in registers and puts the keys back.  Ends with a CTA barrier.
__device__ __forceinline__ void sort_phase(uint32_t* keys, int P, int p, int b, int m_lo, int m_hi, int s_hi, int s_lo) {
    for (int g = threadIdx.x; g < (P >> 3); g += blockDim.x) {
        int base;
        if (b == 3 && p >= 10) base = (g & 7) | (((g >> 3) & 3) << 8) | (((g >> 5) & 3) << 6) | ((g >> 7) << 10);
        else base = (g & ((1 << b) - 1)) | ((g >> b) << (b + 3));
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = keys[sort_slot(base | (j << b))];
        for (int m = m_lo; m <= m_hi; ++m) {
            const int mbit = 1 << m;
            const bool base_up = (base & mbit) == 0;
            const int jm = (mbit >> b) & 7;                      // the direction bit, when it lies inside the window
            for (int s = min(s_hi, m - 1); s >= s_lo; --s) {
                const int sb = s - b;
                if (sb == 0) sort_stage<0>(v, base_up, jm);
                else if (sb == 1) sort_stage<1>(v, base_up, jm);
                else sort_stage<2>(v, base_up, jm);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) keys[sort_slot(base | (j << b))] = v[j];
    }
    __syncthreads();
}

// Selection without sorting, for the usual case of a few levels over a long row: the row's values are counted
// into kSelBins equal-width bins between its minimum and maximum (a weakly monotone map, so the bins are ordered
// groups), a prefix sum over the counts names the bin and the rank inside it of every wanted order statistic,
// the members of those few bins are collected, and each statistic is picked from its bin by counting.  Rows the
// bins cannot split (an infinite or empty range, more than kSelCap members in a wanted bin) are sorted instead.
constexpr int kSelBins = 4096;
constexpr int kSelSlots = 32;                                    // order statistics per row: 2 per level
constexpr int kSelCap = kSelBins / kSelSlots;                    // members kept per wanted bin (lists reuse the counters)
constexpr int kSelMinK = 1024;
static_assert(kSelBins == 8 * 512, "the prefix sums give every one of the 512 threads eight bins");

__device__ __forceinline__ int sel_bin(float v, float mn, float inv) {
    return min(__float2int_rz(__fmul_rn(__fsub_rn(v, mn), inv)), kSelBins - 1);
}

__device__ __forceinline__ float quantile_rank(int k, int n, int K) {
    const float q = __fdiv_rn((float)(2 * k + 1), (float)(2 * n));
    return __fmul_rn(q, (float)(K - 1));
}

// torch.quantile's linear interpolation between the order statistics a (at floor(rank)) and b (at ceil(rank))
__device__ __forceinline__ float quantile_lerp(float a, float b, float rank) {
    const float w = __fsub_rn(rank, floorf(rank));
    const float d = __fsub_rn(b, a);
    return (w < 0.5f) ? __fmaf_rn(w, d, a) : __fmaf_rn(-d, __fsub_rn(1.0f, w), b);
}

struct SelShared {
    int has_nan, give_up;
    uint32_t kmin, kmax;
    uint32_t warp_tot[kQuantThreads / 32];
    int t_bin[kSelSlots], t_local[kSelSlots], cnt[kSelSlots];
    uint32_t sel[kSelSlots];
};

// The selection for one row whose elements the CTA's kQuantThreads threads hold in registers (element
// j * kQuantThreads + thread in v[j]).  True when out[0..n) was written; false when the row has to be sorted.
// Every thread of the CTA returns the same answer.  hist: kSelBins zeroed counters; slot_of_bin: kSelBins bytes
// of 0xFF (left so); sh.cnt zeroed, sh.kmin / sh.kmax the extreme keys of the row.
template <int EPT>
__device__ __forceinline__ bool select_row(const float (&v)[EPT], int K, int n, float* __restrict__ out, uint32_t* hist,
                                           uint8_t* slot_of_bin, SelShared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kWarpsQ = kQuantThreads / 32, kPerWarp = kSelBins / kWarpsQ;
    const float mn = value_of(sh.kmin), range = __fsub_rn(value_of(sh.kmax), mn);
    const float inv = __fdiv_rn((float)(kSelBins - 1), range);
    if (!(range > 0.0f && range < CUDART_INF_F && inv < CUDART_INF_F)) return false;
#pragma unroll
    for (int j = 0; j < EPT; ++j)
        if (j * kQuantThreads + (int)threadIdx.x < K) atomicAdd(&hist[sel_bin(v[j], mn, inv)], 1u);
    __syncthreads();
    {   // inclusive prefix sums of the counters, restarting at every warp's run of kPerWarp bins; eight bins a thread
        uint4* h4 = reinterpret_cast<uint4*>(hist) + 2 * threadIdx.x;
        uint4 a = h4[0], b = h4[1];
        a.y += a.x; a.z += a.y; a.w += a.z;
        b.x += a.w; b.y += b.x; b.z += b.y; b.w += b.z;
        uint32_t incl = b.w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t excl = incl - b.w;
        a.x += excl; a.y += excl; a.z += excl; a.w += excl;
        b.x += excl; b.y += excl; b.z += excl; b.w += excl;
        h4[0] = a; h4[1] = b;
        if (lane == 31) sh.warp_tot[warp] = incl;
    }
    __syncthreads();
    {   // the bin of every wanted order statistic and its rank there: sixteen lanes search for one statistic,
        // over the warps' totals, then the sixteen 16-bin groups of that warp's run, then the group's bins
        const int t = threadIdx.x >> 4, l = threadIdx.x & 15;
        const unsigned half = 0xFFFFu << (lane & 16);
        const float rank = quantile_rank(t >> 1, n, K);
        uint32_t r = (uint32_t)((t & 1) ? ceilf(rank) : floorf(rank));
        const uint32_t tot = sh.warp_tot[l];
        uint32_t cum = tot;
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, cum, o, 16);
            if (l >= o) cum += up;
        }
        const int w = min(__popc(__ballot_sync(0xFFFFFFFFu, cum <= r) & half), kWarpsQ - 1);
        r -= __shfl_sync(0xFFFFFFFFu, cum - tot, w, 16);         // ranks before the run of warp w
        const int run = w * kPerWarp;
        const int grp = min(__popc(__ballot_sync(0xFFFFFFFFu, hist[run + l * 16 + 15] <= r) & half), 15);
        const uint32_t mine = hist[run + grp * 16 + l];
        const int a = run + grp * 16 + min(__popc(__ballot_sync(0xFFFFFFFFu, mine <= r) & half), 15);
        if (l == 0 && t < 2 * n) {
            const uint32_t before = a == run ? 0u : hist[a - 1];
            if (hist[a] - before > (uint32_t)kSelCap) sh.give_up = 1;
            sh.t_bin[t] = a;
            sh.t_local[t] = (int)(r - before);
            slot_of_bin[a] = (uint8_t)t;                         // statistics sharing a bin share one list: any writer wins
        }
    }
    __syncthreads();
    const bool ok = !sh.give_up;
    if (ok) {
        uint32_t* lists = hist;                                  // the counters are not needed any more
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            if (j * kQuantThreads + (int)threadIdx.x < K) {
                const int s = slot_of_bin[sel_bin(v[j], mn, inv)];
                if (s != 0xFF) lists[s * kSelCap + atomicAdd(&sh.cnt[s], 1)] = key_of(v[j]);
            }
        }
        __syncthreads();
        {   // sixteen lanes per statistic: a lane takes members of the bin and counts the keys below and up to its own
            const int t = threadIdx.x >> 4;
            if (t < 2 * n) {
                const int s = slot_of_bin[sh.t_bin[t]], c = sh.cnt[s], want = sh.t_local[t];
                const uint32_t* list = lists + s * kSelCap;
                for (int e = threadIdx.x & 15; e < c; e += 16) {
                    const uint32_t ke = list[e];
                    int less = 0, leq = 0;
                    for (int f = 0; f < c; ++f) {
                        const uint32_t kf = list[f];
                        less += kf < ke;
                        leq += kf <= ke;
                    }
                    if (less <= want && want < leq) sh.sel[t] = ke;
                }
            }
        }
        __syncthreads();
        if (threadIdx.x < n) {
            const int k = threadIdx.x;
            out[k] = quantile_lerp(value_of(sh.sel[2 * k]), value_of(sh.sel[2 * k + 1]), quantile_rank(k, n, K));
        }
    }
    __syncthreads();
    if (threadIdx.x < 2 * n) slot_of_bin[sh.t_bin[threadIdx.x]] = 0xFF;
    return ok;
}

// EPT > 0: kQuantThreads threads, EPT * kQuantThreads == P, rows selected from registers where that works.
// EPT == 0: every row sorted.
template <typename T, int EPT>
__global__ void __launch_bounds__(kQuantThreads, EPT >= 16 ? 2 : 3)
row_quantile_kernel(const void* __restrict__ xin, float* __restrict__ out, int64_t rows, int K, int P, int p, int n) {
    extern __shared__ uint4 smem_q[];                            // [P] keys | [kSelBins] counters / lists | [kSelBins] bytes
    uint32_t* keys = reinterpret_cast<uint32_t*>(smem_q);
    uint32_t* hist = keys + P;
    uint8_t* slot_of_bin = reinterpret_cast<uint8_t*>(hist + kSelBins);
    __shared__ SelShared sh;
    const T* x = reinterpret_cast<const T*>(xin);
    if (EPT > 0) {
        for (int i = threadIdx.x; i < kSelBins / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(slot_of_bin)[i] = 0xFFFFFFFFu;
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * K;
        if (threadIdx.x == 0) { sh.has_nan = 0; sh.give_up = 0; sh.kmin = 0xFFFFFFFFu; sh.kmax = 0u; }
        bool nan = false;
        if constexpr (EPT > 0) {
            float v[EPT];
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int i = j * kQuantThreads + threadIdx.x;
                v[j] = i < K ? load_elem<T>(xr + i) : CUDART_INF_F;
            }
            reinterpret_cast<uint4*>(hist)[2 * threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4*>(hist)[2 * threadIdx.x + 1] = make_uint4(0u, 0u, 0u, 0u);
            if (threadIdx.x < kSelSlots) sh.cnt[threadIdx.x] = 0;
            float lo_v = CUDART_INF_F, hi_v = -CUDART_INF_F;
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                if (j * kQuantThreads + (int)threadIdx.x < K) {
                    nan |= v[j] != v[j];
                    lo_v = fminf(lo_v, v[j]);
                    hi_v = fmaxf(hi_v, v[j]);
                }
            }
            __syncthreads();                                     // the flags and extremes are reset
            const uint32_t lo_k = __reduce_min_sync(0xFFFFFFFFu, key_of(lo_v));
            const uint32_t hi_k = __reduce_max_sync(0xFFFFFFFFu, key_of(hi_v));
            if ((threadIdx.x & 31) == 0) { atomicMin(&sh.kmin, lo_k); atomicMax(&sh.kmax, hi_k); }
            if (nan) sh.has_nan = 1;
            __syncthreads();
            bool done = false;
            if (sh.has_nan) {                                    // torch.quantile: a NaN anywhere in the row
                for (int k = threadIdx.x; k < n; k += blockDim.x) out[row * n + k] = CUDART_NAN_F;
                done = true;
            } else {
                done = select_row<EPT>(v, K, n, out + row * n, hist, slot_of_bin, sh);
            }
            if (done) {
                __syncthreads();
                continue;
            }
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int i = j * kQuantThreads + threadIdx.x;
                keys[sort_slot(i)] = i < K ? key_of(v[j]) : 0xFFFFFFFFu;
            }
            __syncthreads();
        } else {
            __syncthreads();
            for (int i = threadIdx.x; i < P; i += blockDim.x) {
                uint32_t k = 0xFFFFFFFFu;
                if (i < K) {
                    const float v = load_elem<T>(xr + i);
                    nan |= v != v;
                    k = key_of(v);
                }
                keys[sort_slot(i)] = k;
            }
            if (nan) sh.has_nan = 1;
            __syncthreads();
            if (sh.has_nan) {
                for (int k = threadIdx.x; k < n; k += blockDim.x) out[row * n + k] = CUDART_NAN_F;
                __syncthreads();
                continue;
            }
        }
        // bitonic network, three stride bits per pass over shared memory: merges of 2, 4 and 8 keys in one
        // pass, then every larger merge from its widest strides down
        sort_phase(keys, P, p, 0, 1, 3, 2, 0);
        for (int m = 4; m <= p; ++m) {
            for (int lo = (m - 1) / 3 * 3; lo >= 0; lo -= 3)
                sort_phase(keys, P, p, min(lo, p - 3), m, m, min(lo + 2, m - 1), lo);
        }
        for (int k = threadIdx.x; k < n; k += blockDim.x) {
            const float rank = quantile_rank(k, n, K);
            out[row * n + k] = quantile_lerp(value_of(keys[sort_slot((int)floorf(rank))]),
                                             value_of(keys[sort_slot((int)ceilf(rank))]), rank);
        }
        __syncthreads();
    }
}

template <typename T, int EPT>
int launch_row_quantile(const void* x, float* out, int64_t rows, int K, int P, int p, int n, int threads, cudaStream_t st) {
    const size_t smem = (size_t)P * 4 + (EPT > 0 ? (size_t)kSelBins * 5 : 0);
    const int per_sm = EPT >= 16 ? 2 : (EPT > 0 ? 3 : (2048 / threads < 16 ? 2048 / threads : 16));
    const int64_t cap = (int64_t)vq_sm_count() * per_sm;
    const int blocks = (int)(rows < cap ? rows : cap);
    if (smem > 48 * 1024)
        VQ_CUDA(cudaFuncSetAttribute(row_quantile_kernel<T, EPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    row_quantile_kernel<T, EPT><<<blocks, threads, smem, st>>>(x, out, rows, K, P, p, n);
    VQ_LAUNCH_CHECK("row_quantile_kernel");
    return 0;
}

template <typename T>
int dispatch_row_quantile(const void* x, float* out, int64_t rows, int K, int n, cudaStream_t st) {
    int P = 8, p = 3;                                            // keys padded to a power of two, eight at least
    while (P < K) { P <<= 1; ++p; }
    if (K >= kSelMinK && 2 * n <= kSelSlots) {
        switch (P / kQuantThreads) {
            case 2: return launch_row_quantile<T, 2>(x, out, rows, K, P, p, n, kQuantThreads, st);
            case 4: return launch_row_quantile<T, 4>(x, out, rows, K, P, p, n, kQuantThreads, st);
            case 8: return launch_row_quantile<T, 8>(x, out, rows, K, P, p, n, kQuantThreads, st);
            default: return launch_row_quantile<T, 16>(x, out, rows, K, P, p, n, kQuantThreads, st);
        }
    }
    const int threads = P / 8 < 32 ? 32 : (P / 8 > kQuantThreads ? kQuantThreads : P / 8);
    return launch_row_quantile<T, 0>(x, out, rows, K, P, p, n, threads, st);
}

}  // namespace

extern "C" int vq_row_quantile(const void* x, int dtype, int64_t rows, int64_t K, int n_levels, float* out, void* stream) {
    const char* name = "vq_row_quantile";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(rows >= 0 && n_levels >= 1 && n_levels <= kMaxLevels, "%s: bad sizes", name);
    if (K < 1 || K > 8192) return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: rows of 1 to 8192 elements", name);
    if (rows == 0) return 0;
    VQ_REQUIRE(x && out, "%s: null pointer", name);
    if (dtype == VQ_F32) return dispatch_row_quantile<float>(x, out, rows, (int)K, n_levels, (cudaStream_t)stream);
    return dispatch_row_quantile<bf16_t>(x, out, rows, (int)K, n_levels, (cudaStream_t)stream);
}

extern "C" size_t vq_row_codebook_workspace(int64_t rows, int n_levels) {
    if (rows < 0 || n_levels < 1) return 0;
    return (size_t)rows * (size_t)n_levels * sizeof(float);
}

extern "C" int vq_row_codebook(const void* x, int dtype, int64_t rows, int64_t K, const float* levels, int n_levels,
                               int round_bf16, uint8_t* idx_out, void* deq_out, void* workspace, size_t workspace_bytes,
                               void* stream) {
    const char* name = "vq_row_codebook";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(rows >= 0 && K >= 0 && K < (1ll << 31), "%s: sizes must be non-negative, K below 2^31", name);
    VQ_REQUIRE(n_levels >= 1 && n_levels <= kMaxLevels, "%s: n_levels must be in [1, %d]", name, kMaxLevels);
    if (rows == 0 || K == 0) return 0;
    VQ_REQUIRE(x && levels && (idx_out || deq_out), "%s: null pointer", name);
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 4 == 0 && workspace_bytes >= vq_row_codebook_workspace(rows, n_levels),
               "%s: workspace missing or smaller than vq_row_codebook_workspace(rows, n_levels)", name);
    RowCbParams p{};
    p.x = x; p.levels = levels; p.idx = idx_out; p.deq = deq_out;
    p.work = reinterpret_cast<float*>(workspace);
    p.rows = rows; p.K = K;
    p.n_levels = n_levels;
    p.round_bf16 = round_bf16 ? 1 : 0;
    const size_t es = dtype == VQ_F32 ? 4 : 2;
    const bool vec = K % 4 == 0 && (uintptr_t)x % (4 * es) == 0 && (uintptr_t)idx_out % 4 == 0 && (uintptr_t)deq_out % (4 * es) == 0;
    // work items: enough of them to fill the machine eight times over, never shorter than 256 elements
    const int sms = vq_sm_count();
    const int64_t want_items = (int64_t)sms * 8 * kWarps * 8;
    int64_t segs = want_items / rows;
    if (segs < 1) segs = 1;
    int64_t seg_len = (K + segs - 1) / segs;
    seg_len = (seg_len + 128 * kPasses - 1) / (128 * kPasses) * (128 * kPasses);
    p.seg_len = seg_len;
    p.segs_per_row = (K + seg_len - 1) / seg_len;
    p.n_items = rows * p.segs_per_row;
    int64_t want_blocks = (p.n_items + kWarps - 1) / kWarps;
    const int blocks = (int)(want_blocks < (int64_t)sms * 8 ? want_blocks : (int64_t)sms * 8);
    cudaStream_t st = (cudaStream_t)stream;
    row_thresholds_kernel<<<(unsigned)((rows * n_levels + 255) / 256), 256, 0, st>>>(levels, p.work, rows, n_levels);
    VQ_LAUNCH_CHECK("row_thresholds_kernel");
    const int log2n = n_levels <= 4 ? 2 : (n_levels <= 16 ? 4 : 8);
    if (dtype == VQ_F32) {
        if (log2n == 2) launch_row_codebook<float, 2>(p, vec, blocks, st);
        else if (log2n == 4) launch_row_codebook<float, 4>(p, vec, blocks, st);
        else launch_row_codebook<float, 8>(p, vec, blocks, st);
    } else {
        if (log2n == 2) launch_row_codebook<bf16_t, 2>(p, vec, blocks, st);
        else if (log2n == 4) launch_row_codebook<bf16_t, 4>(p, vec, blocks, st);
        else launch_row_codebook<bf16_t, 8>(p, vec, blocks, st);
    }
    VQ_LAUNCH_CHECK("row_codebook_kernel");
    return 0;
}
