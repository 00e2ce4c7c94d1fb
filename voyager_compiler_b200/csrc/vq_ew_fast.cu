// Specialised streaming kernels for the common element-wise cases (see vq_mx_fast.cuh for the
// per-chunk body): quantize / table map / dequantize with one scale per 32-byte chunk (scalar
// scale, or [rows, K] tensors whose row length and block are multiples of the chunk), no zero
// point, float output.  Everything else stays on the generic kernel in vq_elementwise.cu.
// HBM bound: 2 x sizeof(T) bytes per element.
#include "vq_mx_fast.cuh"

namespace {

enum { EW_MAP = 0, EW_QUANT = 1, EW_DEQUANT = 2, EW_FAKEQ = 3 };

struct EwFastParams {
    const void* in;
    void* out;
    const void* scale;
    uint32_t nchunk;
    int smode;              // VQ_SCALE_SCALAR or VQ_SCALE_ROWBLOCK
    uint32_t Kc, Bc, nb;    // chunks per row, chunks per block, blocks per row
    FastDiv divK, divB;
    TableDev tab;
};

template <typename T>
__device__ __forceinline__ float load_scale(const void* p, uint32_t i) {
    return load_one<T>(reinterpret_cast<const T*>(p) + i);
}

template <typename T, int OP, int TK, bool SM>
__global__ void __launch_bounds__(1024, 1) ew_fast_kernel(const EwFastParams p) {
    extern __shared__ uint4 smem[];
    FastTab ft;
    ft.lut16 = p.tab.lut16;
    ft.lut8 = nullptr;
    ft.lo = p.tab.lo;
    ft.hi = p.tab.hi;
    ft.lo_is_zero = (p.tab.lo == 0.0f) ? 1 : 0;
    ft.flat_tiny = p.tab.flat_tiny;
    if (SM && TK == TK_LUT && OP != EW_DEQUANT) {
        const uint4* src = reinterpret_cast<const uint4*>(p.tab.lut16);
        for (int i = threadIdx.x; i < 8192; i += blockDim.x) smem[i] = __ldg(src + i);
        __syncthreads();
    }
    constexpr int N = sizeof(T) == 2 ? 16 : 8;
    const T* in = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    float s_all = 1.0f;
    if (OP != EW_MAP && p.smode == VQ_SCALE_SCALAR) s_all = load_scale<T>(p.scale, 0);
    const uint32_t nthreads = gridDim.x * blockDim.x;
    for (uint32_t c0 = blockIdx.x * blockDim.x + threadIdx.x; c0 < p.nchunk; c0 += 2 * nthreads) {
        Chunk x[2];
        const uint32_t c1 = c0 + nthreads;
        x[0].load(in + (size_t)c0 * N);
        if (c1 < p.nchunk) x[1].load(in + (size_t)c1 * N);
        else x[1].zero();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t ci = u ? c1 : c0;
            if (ci >= p.nchunk) continue;
            float s = s_all;
            if (OP != EW_MAP && p.smode == VQ_SCALE_ROWBLOCK) {
                const uint32_t row = fd_div(ci, p.divK);
                s = load_scale<T>(p.scale, row * p.nb + fd_div(ci - row * p.Kc, p.divB));
            }
            if (OP == EW_DEQUANT) {
                uint32_t o[8];
                if (sizeof(T) == 2) {
                    const uint32_t s2 = (__float_as_uint(s) >> 16) * 0x00010001u;
#pragma unroll
                    for (int k = 0; k < 8; ++k) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[k]) : "r"(x[u].w[k]), "r"(s2));
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] = __float_as_uint(__fmul_rn(__uint_as_float(x[u].w[k]), s));
                }
                store32(out + (size_t)ci * N, o);
            } else if (OP == EW_MAP) {
                fast_chunk<T, TK, OUT_FLOAT, SM>(ft, smem, x[u], 1.0f, false, (size_t)ci, out, nullptr);
            } else {
                bool refine = false;
                if (sizeof(T) == 2) {
                    // reciprocal path when the quotients stay normal: always for a table that is flat
                    // over the tiny patterns, otherwise when no non-zero element is tiny
                    refine = true;
                    if (!ft.flat_tiny) chunk_amax<T>(x[u], refine, true);
                }
                fast_chunk<T, TK, OP == EW_FAKEQ ? OUT_FAKEQ : OUT_FLOAT, SM>(ft, smem, x[u], s, refine, (size_t)ci, out, nullptr);
            }
        }
    }
}

template <typename T, int OP, int TK>
int launch3(const EwFastParams& p, bool sm, int threads, int blocks, cudaStream_t st) {
    const size_t smem = sm ? 131072 : 0;
    if (sm) {
        auto k = ew_fast_kernel<T, OP, TK, true>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<blocks, threads, smem, st>>>(p);
    } else {
        ew_fast_kernel<T, OP, TK, false><<<blocks, threads, 0, st>>>(p);
    }
    VQ_LAUNCH_CHECK("ew_fast_kernel");
    return 0;
}

template <typename T>
int launch_op(const EwFastParams& p, int op, int tk, bool sm, int threads, int blocks, cudaStream_t st) {
    if (op == EW_DEQUANT) return launch3<T, EW_DEQUANT, TK_INT>(p, false, threads, blocks, st);
    if (op == EW_MAP)
        return tk == TK_INT ? launch3<T, EW_MAP, TK_INT>(p, false, threads, blocks, st)
                            : launch3<T, EW_MAP, TK_LUT>(p, sm, threads, blocks, st);
    if (op == EW_FAKEQ)
        return tk == TK_INT ? launch3<T, EW_FAKEQ, TK_INT>(p, false, threads, blocks, st)
                            : launch3<T, EW_FAKEQ, TK_LUT>(p, sm, threads, blocks, st);
    return tk == TK_INT ? launch3<T, EW_QUANT, TK_INT>(p, false, threads, blocks, st)
                        : launch3<T, EW_QUANT, TK_LUT>(p, sm, threads, blocks, st);
}

}  // namespace

// op: 0 map, 1 quantize, 2 dequantize (no tables), 3 quantize then multiply by the scale.  Returns 1 when launched, 0 when not eligible.
int vq_ew_fast_try(int op, const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                   const vq_scale_layout* layout, const vq_table* t0, const vq_table* t1, void* out, uint8_t* codes,
                   cudaStream_t st) {
    if (zero_point || codes || !out || n <= 0 || n >= (1ll << 31)) return 0;
    const int N = dtype == VQ_F32 ? 8 : 16;
    if (n % N || (uintptr_t)in % 32 || (uintptr_t)out % 32) return 0;
    int tk = TK_INT;
    if (op == EW_DEQUANT) {
        if ((t0 && t0->kind != VQ_TABLE_NONE) || (t1 && t1->kind != VQ_TABLE_NONE)) return 0;
    } else {
        if (!t0) return 0;
        if (t0->kind == VQ_TABLE_INT) tk = TK_INT;
        else if (t0->kind == VQ_TABLE_LUT16 && t0->nan_uniform && t0->lut16) tk = TK_LUT;
        else return 0;
    }
    EwFastParams p{};
    p.in = in;
    p.out = out;
    p.scale = scale;
    p.nchunk = (uint32_t)(n / N);
    p.tab = to_dev(t0);
    p.smode = VQ_SCALE_SCALAR;
    if (op != EW_MAP) {
        if (!layout || !scale) return 0;
        if (layout->mode == VQ_SCALE_ROWBLOCK) {
            int64_t K = layout->K, bs = layout->block > K ? K : layout->block;
            if (K % N || bs % N) return 0;
            p.smode = VQ_SCALE_ROWBLOCK;
            p.Kc = (uint32_t)(K / N);
            p.Bc = (uint32_t)(bs / N);
            p.nb = (uint32_t)((K + bs - 1) / bs);
            p.divK = make_fastdiv(p.Kc);
            p.divB = make_fastdiv(p.Bc);
        } else if (layout->mode != VQ_SCALE_SCALAR) {
            return 0;
        }
    }
    const int sms = vq_sm_count();
    const bool big = n >= (1ll << 22);
    const bool sm = big && tk == TK_LUT && op != EW_DEQUANT;
    int threads, blocks;
    if (big) {
        threads = sm ? 1024 : 512;
        blocks = sm ? sms : sms * 4;
    } else {
        threads = 128;
        int64_t want = (p.nchunk + 2 * threads - 1) / (2 * threads);
        blocks = (int)(want < 1 ? 1 : (want > (int64_t)sms * 8 ? (int64_t)sms * 8 : want));
    }
    int rc = dtype == VQ_F32 ? launch_op<float>(p, op, tk, sm, threads, blocks, st)
                             : launch_op<bf16_t>(p, op, tk, sm, threads, blocks, st);
    return rc ? rc : 1;
}
