// Row / column slices of a padded CSR tensor on the device, with no host round trip.
//
// Upstream `slice_csr_tensor` (ops/quantized.py:745-788) reads three scalars back to the host
// (`.item()`), builds masks and re-pads with tensor operations.  The outputs have a fixed size
// (capacity = int(max_nnz * size_factor) entries, padded with 0 / -1, row pointers clamped to the
// capacity when more entries survive than fit), so the whole slice can stay on the stream:
//   rows    [start, end): the entries are a contiguous span; one kernel copies, pads and rebases
//           the row pointers;
//   columns [start, end): count per row (a warp per row), scan over the rows (one CTA), ordered
//           compaction (a warp per row, ballot prefix), padding of the tail.
#include "vq_common.cuh"

namespace {

struct SliceParams {
    const uint8_t* data;       // [max_nnz] elements of esize bytes
    const int32_t* indices;    // [max_nnz]
    const int32_t* indptr;     // [rows + 1]
    uint8_t* out_data;         // [cap]
    int32_t* out_indices;      // [cap]
    int32_t* out_indptr;       // rows: [end - start + 1]; columns: [rows + 1]
    int32_t* offs;             // columns: unclamped running counts, [rows + 1] (workspace)
    int64_t rows, max_nnz, cap, start, end;
    int esize;
};

template <typename E>
__global__ void __launch_bounds__(256) csr_slice_rows_kernel(const SliceParams p) {
    const int64_t s0 = p.indptr[p.start], e0 = p.indptr[p.end];
    const int64_t n_out = p.end - p.start + 1;
    const int64_t span = e0 - s0;
    const E* src = reinterpret_cast<const E*>(p.data);
    E* dst = reinterpret_cast<E*>(p.out_data);
    const int64_t total = p.cap > n_out ? p.cap : n_out;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        if (i < n_out) {
            const int64_t v = p.indptr[p.start + i] - s0;
            p.out_indptr[i] = (int32_t)(v < p.cap ? v : p.cap);
        }
        if (i < p.cap) {
            const bool live = i < span && s0 + i < p.max_nnz;
            dst[i] = live ? src[s0 + i] : E(0);
            p.out_indices[i] = live ? p.indices[s0 + i] : -1;
        }
    }
}

__global__ void __launch_bounds__(256) csr_slice_count_kernel(const SliceParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < p.rows; r += nwarps) {
        const int64_t b = p.indptr[r], e = p.indptr[r + 1];
        int cnt = 0;
        for (int64_t i = b + lane; i < e && i < p.max_nnz; i += 32) {
            const int32_t c = p.indices[i];
            cnt += (c >= p.start && c < p.end) ? 1 : 0;
        }
        cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
        if (lane == 0) p.offs[r + 1] = cnt;
    }
}

__global__ void __launch_bounds__(1024) csr_slice_scan_kernel(const SliceParams p) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry = 0;
        p.offs[0] = 0;
        p.out_indptr[0] = 0;
    }
    __syncthreads();
    for (int64_t r0 = 0; r0 < p.rows; r0 += blockDim.x) {
        const int64_t r = r0 + threadIdx.x;
        int incl = r < p.rows ? p.offs[r + 1] : 0;
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
            p.offs[r + 1] = total;
            p.out_indptr[r + 1] = (int32_t)(total < p.cap ? total : p.cap);
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = total;
        __syncthreads();
    }
}

template <typename E>
__global__ void __launch_bounds__(256) csr_slice_fill_kernel(const SliceParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const E* src = reinterpret_cast<const E*>(p.data);
    E* dst = reinterpret_cast<E*>(p.out_data);
    // rows: ordered compaction; the warps past the last row pad the tail [kept entries, cap)
    for (int64_t r = warp; r < p.rows; r += nwarps) {
        const int64_t b = p.indptr[r], e = p.indptr[r + 1];
        int64_t pos = p.offs[r];
        for (int64_t i0 = b; i0 < e && i0 < p.max_nnz; i0 += 32) {
            const int64_t i = i0 + lane;
            int32_t c = -1;
            if (i < e && i < p.max_nnz) c = p.indices[i];
            const bool keep = i < e && i < p.max_nnz && c >= p.start && c < p.end;
            const uint32_t m = __ballot_sync(0xFFFFFFFFu, keep);
            const int64_t at = pos + __popc(m & ((1u << lane) - 1u));
            if (keep && at < p.cap) {
                dst[at] = src[i];
                p.out_indices[at] = c - (int32_t)p.start;
            }
            pos += __popc(m);
        }
    }
    const int64_t kept = p.offs[p.rows];
    for (int64_t i = (kept < p.cap ? kept : p.cap) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.cap;
         i += (int64_t)gridDim.x * blockDim.x) {
        dst[i] = E(0);
        p.out_indices[i] = -1;
    }
}

}  // namespace

extern "C" {

size_t vq_slice_csr_workspace(int64_t rows) { return rows < 0 ? 0 : (size_t)(rows + 1) * sizeof(int32_t); }

int vq_slice_csr(const void* data, const int32_t* indices, const int32_t* indptr, int dtype, int64_t rows, int64_t max_nnz, int dim,
                 int64_t start, int64_t end, int64_t cap, void* out_data, int32_t* out_indices, int32_t* out_indptr, void* workspace,
                 size_t workspace_bytes, void* stream) {
    const char* name = "vq_slice_csr";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(dim == 0 || dim == 1, "%s: Cannot slice sparse CSR matrix along dim %d", name, dim);
    VQ_REQUIRE(rows >= 0 && max_nnz >= 0 && cap >= 0 && cap < (1ll << 31) && max_nnz < (1ll << 31), "%s: sizes out of range", name);
    VQ_REQUIRE(indptr && out_indptr && (max_nnz == 0 || (data && indices)) && (cap == 0 || (out_data && out_indices)), "%s: null pointer", name);
    VQ_REQUIRE(start >= 0 && end >= start, "%s: start / end out of order", name);
    SliceParams p{};
    p.data = reinterpret_cast<const uint8_t*>(data);
    p.indices = indices;
    p.indptr = indptr;
    p.out_data = reinterpret_cast<uint8_t*>(out_data);
    p.out_indices = out_indices;
    p.out_indptr = out_indptr;
    p.rows = rows; p.max_nnz = max_nnz; p.cap = cap; p.start = start; p.end = end;
    p.esize = dtype == VQ_F32 ? 4 : 2;
    cudaStream_t st = (cudaStream_t)stream;
    const int sms = vq_sm_count();
    if (dim == 0) {
        VQ_REQUIRE(end <= rows, "%s: row range [%lld, %lld) outside the %lld rows", name, (long long)start, (long long)end, (long long)rows);
        const int64_t work = (cap > end - start + 1 ? cap : end - start + 1);
        const int blocks = (int)((work + 255) / 256 < (int64_t)sms * 4 ? (work + 255) / 256 : (int64_t)sms * 4);
        if (dtype == VQ_F32) csr_slice_rows_kernel<float><<<blocks > 0 ? blocks : 1, 256, 0, st>>>(p);
        else csr_slice_rows_kernel<uint16_t><<<blocks > 0 ? blocks : 1, 256, 0, st>>>(p);
        VQ_LAUNCH_CHECK("csr_slice_rows_kernel");
        return 0;
    }
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 4 == 0 && workspace_bytes >= vq_slice_csr_workspace(rows),
               "%s: workspace missing or smaller than vq_slice_csr_workspace(rows)", name);
    p.offs = reinterpret_cast<int32_t*>(workspace);
    const int64_t row_blocks = (rows + 7) / 8;
    const int blocks = (int)(row_blocks < (int64_t)sms * 8 ? (row_blocks > 0 ? row_blocks : 1) : (int64_t)sms * 8);
    if (rows > 0) {
        csr_slice_count_kernel<<<blocks, 256, 0, st>>>(p);
        VQ_LAUNCH_CHECK("csr_slice_count_kernel");
    }
    csr_slice_scan_kernel<<<1, 1024, 0, st>>>(p);
    VQ_LAUNCH_CHECK("csr_slice_scan_kernel");
    if (dtype == VQ_F32) csr_slice_fill_kernel<float><<<blocks, 256, 0, st>>>(p);
    else csr_slice_fill_kernel<uint16_t><<<blocks, 256, 0, st>>>(p);
    VQ_LAUNCH_CHECK("csr_slice_fill_kernel");
    return 0;
}

}  // extern "C"
