// Outlier side path: split a tensor of [batch, rows, cols] matrices into inliers and a padded CSR of
// outliers (`filter_outlier`, ops/quantized.py:565-621 with `_pad_csr`, :538-562), and the sparse
// correction `spmm_csr` (:786-862) the MX linear adds to its dense product (:335-346).
//
// filter: an element is an outlier when |x| > threshold (threshold rounded to the tensor dtype, as
// torch does for a Python scalar); the inlier tensor keeps x elsewhere and +0 at outliers; the CSR of
// a matrix lists the non-zero outliers row by row in column order (`to_sparse_csr`), values and
// int32 column indices padded to max_nnz with 0 / -1; when a matrix holds more than max_nnz the
// surplus is dropped and the row pointers are clamped to max_nnz, as upstream does.
//   1. count:  one warp per row counts its outliers;
//   2. scan:   one CTA per matrix turns the counts into row pointers (clamped copy for the caller,
//              unclamped copy for step 3) and writes the padding;
//   3. fill:   one warp per row writes inliers and, by ballot + prefix count, its CSR entries.
// Two reads and one write of the tensor; upstream makes ~6 full passes plus a sparse conversion
// per matrix in a Python loop.
#include <cstring>

#include "vq_common.cuh"

namespace {

struct OutlierParams {
    const void* in;
    void* inlier;
    void* data;             // [batch, max_nnz] in the tensor dtype
    int32_t* indices;       // [batch, max_nnz]
    int32_t* indptr;        // [batch, rows + 1], clamped
    int32_t* offs;          // workspace [batch, rows + 1], unclamped
    int64_t batch, rows, cols;
    int64_t max_nnz;
    float thr;              // already rounded to the tensor dtype
    int32_t indptr_offset;
    int vec;                // rows start 16-byte aligned and hold a multiple of 16 bytes
};

// 16 bytes of a row as fp32 values
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* v, uint4& raw) {
        raw = __ldcs(reinterpret_cast<const uint4*>(p));
        v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
    }
    static __device__ __forceinline__ void zero(uint4& raw, int j) { (&raw.x)[j] = 0u; }
};
template <>
struct Vec16<bf16_t> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16_t* p, float* v, uint4& raw) {
        raw = __ldcs(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
    static __device__ __forceinline__ void zero(uint4& raw, int j) { (&raw.x)[j >> 1] &= (j & 1) ? 0x0000FFFFu : 0xFFFF0000u; }
};

template <typename T>
__device__ __forceinline__ float ld(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<bf16_t>(const bf16_t* p, int64_t i) { return bf16_bits_to_f32(p[i].bits); }

__device__ __forceinline__ bool is_outlier(float x, float thr) { return fabsf(x) > thr; }   // false for NaN

template <typename T>
__global__ void __launch_bounds__(256) outlier_count_kernel(const OutlierParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t n_rows = p.batch * p.rows;
    const T* x = reinterpret_cast<const T*>(p.in);
    for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < n_rows; row += (int64_t)gridDim.x * 8) {
        const T* xr = x + row * p.cols;
        int cnt = 0;
        if (p.vec) {
            constexpr int V = Vec16<T>::N;
            for (int64_t c = (int64_t)lane * V; c < p.cols; c += 32 * V) {
                float v[V];
                uint4 raw;
                Vec16<T>::load(xr + c, v, raw);
#pragma unroll
                for (int j = 0; j < V; ++j) cnt += (is_outlier(v[j], p.thr) && v[j] != 0.0f) ? 1 : 0;
            }
        } else
        for (int64_t c = lane; c < p.cols; c += 32) {
            const float v = ld<T>(xr, c);
            cnt += (is_outlier(v, p.thr) && v != 0.0f) ? 1 : 0;
        }
        cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
        const int64_t b = row / p.rows, r = row - b * p.rows;
        if (lane == 0) p.offs[b * (p.rows + 1) + r + 1] = cnt;
    }
}

// one CTA (1024 threads) per matrix: inclusive scan of the row counts
__global__ void __launch_bounds__(1024) outlier_scan_kernel(const OutlierParams p) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int64_t b = blockIdx.x;
    int32_t* offs = p.offs + b * (p.rows + 1);
    int32_t* indptr = p.indptr + b * (p.rows + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry = 0;
        offs[0] = 0;
        indptr[0] = p.indptr_offset;
    }
    __syncthreads();
    const int64_t cap = p.max_nnz;
    for (int64_t r0 = 0; r0 < p.rows; r0 += blockDim.x) {
        const int64_t r = r0 + threadIdx.x;
        int v = r < p.rows ? offs[r + 1] : 0;
        int incl = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int total = incl + (warp ? warp_sums[warp - 1] : 0) + carry;
        if (r < p.rows) {
            offs[r + 1] = total;
            indptr[r + 1] = (int32_t)(total < cap ? total : cap) + p.indptr_offset;
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = total;
        __syncthreads();
    }
    // padding behind the last stored entry
    const int64_t nse = carry < cap ? carry : cap;
    for (int64_t i = nse + threadIdx.x; i < cap; i += blockDim.x) p.indices[b * cap + i] = -1;
}

template <typename T>
__global__ void __launch_bounds__(256) outlier_fill_kernel(const OutlierParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t n_rows = p.batch * p.rows;
    const T* x = reinterpret_cast<const T*>(p.in);
    T* inl = reinterpret_cast<T*>(p.inlier);
    T* data = reinterpret_cast<T*>(p.data);
    for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < n_rows; row += (int64_t)gridDim.x * 8) {
        const int64_t b = row / p.rows, r = row - b * p.rows;
        const T* xr = x + row * p.cols;
        T* ir = inl + row * p.cols;
        int64_t pos = p.offs[b * (p.rows + 1) + r];
        const bool any = p.offs[b * (p.rows + 1) + r + 1] != pos;      // rows without outliers: plain copy
        if (p.vec) {
            // 16 bytes per lane and step: V consecutive elements; CSR order = lane order, then element order
            constexpr int V = Vec16<T>::N;
            for (int64_t c0 = 0; c0 < p.cols; c0 += 32 * V) {
                const int64_t c = c0 + (int64_t)lane * V;
                float v[V];
                uint4 raw = make_uint4(0, 0, 0, 0);
                const bool in = c < p.cols;
                if (in) Vec16<T>::load(xr + c, v, raw);
                uint4 keep_raw = raw;
                int n = 0;
                uint32_t out_mask = 0;
                if (in) {
#pragma unroll
                    for (int j = 0; j < V; ++j)
                        if (is_outlier(v[j], p.thr)) {
                            Vec16<T>::zero(keep_raw, j);
                            if (v[j] != 0.0f) { out_mask |= 1u << j; ++n; }
                        }
                    __stcs(reinterpret_cast<uint4*>(ir + c), keep_raw);
                }
                if (any) {
                    // exclusive prefix of n over the lanes
                    int incl = n;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                        if (lane >= o) incl += t;
                    }
                    int64_t q = pos + incl - n;
                    for (int j = 0; j < V; ++j)
                        if (out_mask & (1u << j)) {
                            if (q < p.max_nnz) {
                                data[b * p.max_nnz + q] = xr[c + j];
                                p.indices[b * p.max_nnz + q] = (int32_t)(c + j);
                            }
                            ++q;
                        }
                    pos += __shfl_sync(0xFFFFFFFFu, incl, 31);
                }
            }
            continue;
        }
        for (int64_t c0 = 0; c0 < p.cols; c0 += 32) {
            const int64_t c = c0 + lane;
            T raw{};
            float v = 0.0f;
            if (c < p.cols) {
                raw = xr[c];
                v = ld<T>(xr, c);
            }
            const bool out = c < p.cols && is_outlier(v, p.thr);
            if (c < p.cols) {
                if (out) store_one<T>(ir + c, 0.0f);
                else ir[c] = raw;
            }
            if (any) {
                const bool keep = out && v != 0.0f;
                const uint32_t mask = __ballot_sync(0xFFFFFFFFu, keep);
                if (keep) {
                    const int64_t q = pos + __popc(mask & ((1u << lane) - 1u));
                    if (q < p.max_nnz) {
                        data[b * p.max_nnz + q] = raw;
                        p.indices[b * p.max_nnz + q] = (int32_t)c;
                    }
                }
                pos += __popc(mask);
            }
        }
    }
}

template <typename T>
__global__ void outlier_pad_data_kernel(const OutlierParams p) {
    // zero the value slots behind the last stored entry of every matrix
    const int64_t b = blockIdx.y;
    const int64_t total = p.offs[b * (p.rows + 1) + p.rows];
    const int64_t nse = total < p.max_nnz ? total : p.max_nnz;
    T* data = reinterpret_cast<T*>(p.data) + b * p.max_nnz;
    for (int64_t i = nse + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.max_nnz; i += (int64_t)gridDim.x * blockDim.x)
        store_one<T>(data + i, 0.0f);
}

// ---------------------------------------------------------------------------------------------
// spmm: Y[b, r, :] = sum over the CSR entries (r, k, v) of v * Bt[b?, k, :], accumulated in fp32 and
// rounded once to the output dtype (upstream: torch.sparse.mm in fp32, then a cast).  Bt is the
// decoded right operand in [K, N] ("ck") order, so every entry reads one contiguous row.
struct SpmmParams {
    const void* data;
    const int32_t* indices;
    const int32_t* indptr;
    const void* Bt;
    const void* addend;           // optional [batch, rows, N]: Y = addend + round(product), the linear's dense part
    void* Y;
    int64_t batch, rows, N, K, max_nnz;
    int64_t bt_batch_stride;      // 0 when Bt is shared by all batches
};

// eight consecutive elements of a row as fp32
template <typename T>
__device__ __forceinline__ void load8(const T* p, float* v);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16_t>(const bf16_t* p, float* v) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* v);     // v already rounded to T
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<bf16_t>(bf16_t* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xFFFF0000u);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// One CTA per output row and 2048-column slab.  VEC: thread t owns the 8 consecutive columns
// slab + 8 t (16- or 32-byte accesses); otherwise columns slab + t, + 256, ...
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) spmm_csr_kernel(const SpmmParams p) {
    const int64_t row = blockIdx.x;
    const int64_t b = row / p.rows, r = row - b * p.rows;
    const int64_t n0 = (int64_t)blockIdx.y * 2048;
    const int32_t* ip = p.indptr + b * (p.rows + 1);
    const int32_t base = ip[0];
    const int64_t e0 = ip[r] - base, e1 = ip[r + 1] - base;
    const T* data = reinterpret_cast<const T*>(p.data) + b * p.max_nnz;
    const int32_t* idx = p.indices + b * p.max_nnz;
    const T* Bt = reinterpret_cast<const T*>(p.Bt) + b * p.bt_batch_stride;
    T* y = reinterpret_cast<T*>(p.Y) + row * p.N;
    const T* add = p.addend ? reinterpret_cast<const T*>(p.addend) + row * p.N : nullptr;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    if (VEC) {
        const int64_t n = n0 + (int64_t)threadIdx.x * 8;
        if (n >= p.N) return;
        for (int64_t e = e0; e < e1; ++e) {
            const float v = ld<T>(data, e);
            float w[8];
            load8<T>(Bt + (int64_t)idx[e] * p.N + n, w);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __fmaf_rn(v, w[j], acc[j]);
        }
        float o[8], a[8];
        if (add) load8<T>(add + n, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j] = Arith<T>::rnd(acc[j]);                              // the product, rounded to the output dtype ...
            if (add) o[j] = Arith<T>::rnd(__fadd_rn(a[j], o[j]));      // ... then added to the dense part in that dtype
        }
        store8<T>(y + n, o);
        return;
    }
    for (int64_t e = e0; e < e1; ++e) {
        const float v = ld<T>(data, e);
        const T* brow = Bt + (int64_t)idx[e] * p.N;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t n = n0 + threadIdx.x + 256 * j;
            if (n < p.N) acc[j] = __fmaf_rn(v, ld<T>(brow, n), acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int64_t n = n0 + threadIdx.x + 256 * j;
        if (n < p.N) {
            float v = Arith<T>::rnd(acc[j]);
            if (add) v = Arith<T>::rnd(__fadd_rn(ld<T>(add, n), v));
            store_one<T>(y + n, v);
        }
    }
}

}  // namespace

extern "C" {

size_t vq_filter_outlier_workspace(int64_t batch, int64_t rows) {
    if (batch < 0 || rows < 0) return 0;
    return (size_t)batch * (size_t)(rows + 1) * sizeof(int32_t);
}

int vq_filter_outlier(const void* in, int dtype, int64_t batch, int64_t rows, int64_t cols, double threshold, int64_t max_nnz,
                      int32_t indptr_offset, void* data, int32_t* indices, int32_t* indptr, void* inlier, void* workspace,
                      size_t workspace_bytes, void* stream) {
    const char* name = "vq_filter_outlier";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0 && max_nnz >= 0, "%s: negative size", name);
    VQ_REQUIRE(rows < (1ll << 31) && cols < (1ll << 31) && rows * cols < (1ll << 31), "%s: matrices must hold fewer than 2^31 elements", name);
    if (batch == 0) return 0;
    VQ_REQUIRE(indptr && inlier && (max_nnz == 0 || (data && indices)), "%s: null output", name);
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 4 == 0 && workspace_bytes >= vq_filter_outlier_workspace(batch, rows),
               "%s: workspace missing or smaller than vq_filter_outlier_workspace(batch, rows)", name);
    VQ_REQUIRE(rows * cols == 0 || in != nullptr, "%s: null input", name);
    OutlierParams p{};
    p.in = in; p.inlier = inlier; p.data = data; p.indices = indices; p.indptr = indptr;
    p.offs = reinterpret_cast<int32_t*>(workspace);
    p.batch = batch; p.rows = rows; p.cols = cols; p.max_nnz = max_nnz;
    p.indptr_offset = indptr_offset;
    float t = (float)threshold;
    if (dtype == VQ_BF16) {        // float -> bf16, round to nearest even, as torch converts the scalar
        uint32_t u;
        memcpy(&u, &t, 4);
        if ((u & 0x7FFFFFFFu) <= 0x7F800000u) u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
        memcpy(&t, &u, 4);
    }
    p.thr = t;
    const size_t es = dtype == VQ_F32 ? 4 : 2;
    p.vec = ((cols * es) % 16 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)inlier % 16 == 0) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int sms = vq_sm_count();
    const int64_t n_rows = batch * rows;
    const int64_t want = (n_rows + 7) / 8;
    const int blocks = (int)(want < 1 ? 1 : (want < (int64_t)sms * 8 ? want : (int64_t)sms * 8));
    if (dtype == VQ_F32) outlier_count_kernel<float><<<blocks, 256, 0, st>>>(p);
    else outlier_count_kernel<bf16_t><<<blocks, 256, 0, st>>>(p);
    VQ_LAUNCH_CHECK("outlier_count_kernel");
    outlier_scan_kernel<<<(unsigned)batch, 1024, 0, st>>>(p);
    VQ_LAUNCH_CHECK("outlier_scan_kernel");
    if (max_nnz > 0) {
        dim3 g((unsigned)((max_nnz + 255) / 256 < 64 ? (max_nnz + 255) / 256 : 64), (unsigned)batch);
        if (dtype == VQ_F32) outlier_pad_data_kernel<float><<<g, 256, 0, st>>>(p);
        else outlier_pad_data_kernel<bf16_t><<<g, 256, 0, st>>>(p);
        VQ_LAUNCH_CHECK("outlier_pad_data_kernel");
    }
    if (n_rows > 0 && cols > 0) {
        if (dtype == VQ_F32) outlier_fill_kernel<float><<<blocks, 256, 0, st>>>(p);
        else outlier_fill_kernel<bf16_t><<<blocks, 256, 0, st>>>(p);
        VQ_LAUNCH_CHECK("outlier_fill_kernel");
    }
    return 0;
}

int vq_spmm_csr(const void* data, const int32_t* indices, const int32_t* indptr, const void* Bt, int dtype, int64_t batch,
                int64_t rows, int64_t K, int64_t N, int64_t max_nnz, int64_t bt_batch_stride, const void* addend, void* Y,
                void* stream) {
    const char* name = "vq_spmm_csr";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(batch >= 0 && rows >= 0 && K >= 0 && N >= 0 && max_nnz >= 0, "%s: negative size", name);
    if (batch * rows * N == 0) return 0;
    VQ_REQUIRE(indptr && Y && (max_nnz == 0 || (data && indices && Bt)), "%s: null pointer", name);
    VQ_REQUIRE(batch * rows < (1ll << 31), "%s: too many rows", name);
    SpmmParams p{};
    p.data = data; p.indices = indices; p.indptr = indptr; p.Bt = Bt; p.Y = Y; p.addend = addend;
    p.batch = batch; p.rows = rows; p.N = N; p.K = K; p.max_nnz = max_nnz; p.bt_batch_stride = bt_batch_stride;
    dim3 grid((unsigned)(batch * rows), (unsigned)((N + 2047) / 2048));
    const size_t es = dtype == VQ_F32 ? 4 : 2;
    const bool vec = N % 8 == 0 && (uintptr_t)Bt % 16 == 0 && (uintptr_t)Y % 16 == 0 && (uintptr_t)addend % 16 == 0 &&
                     (bt_batch_stride * es) % 16 == 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == VQ_F32) {
        if (vec) spmm_csr_kernel<float, true><<<grid, 256, 0, st>>>(p);
        else spmm_csr_kernel<float, false><<<grid, 256, 0, st>>>(p);
    } else {
        if (vec) spmm_csr_kernel<bf16_t, true><<<grid, 256, 0, st>>>(p);
        else spmm_csr_kernel<bf16_t, false><<<grid, 256, 0, st>>>(p);
    }
    VQ_LAUNCH_CHECK("spmm_csr_kernel");
    return 0;
}

}  // extern "C"
