// Patch matrix of a 2-D convolution: out[(n, ho, wo), (kh, kw, c)] = x[n, ho*sh - ph + kh*dh, wo*sw - pw + kw*dw, c],
// zero outside the image and in the padding columns.  With it conv2d_mx becomes the same TN contraction as
// linear_mx (patches [M, K] against the weight stored [O, K] with K ordered (kh, kw, c)), so the convolution runs
// on this library's tensor-core GEMM.  The input is addressed by element strides, which covers NCHW and NHWC.
// With a scale tensor (one value per block of channels at every pixel) the element is multiplied by its scale
// on the way, rounded once in the tensor's dtype, which is `dequantize` of an MX activation fused into the copy.
#include "vq_common.cuh"

namespace {

struct PatchParams {
    const void* x;
    void* out;
    int64_t sn, sh, sw, sc;                                      // element strides of x along n, h, w, c
    int64_t ldk;                                                 // row pitch of out, elements
    int H, W, C, Ho, Wo;
    int kh, kw, str_h, str_w, pad_h, pad_w, dil_h, dil_w;
    int K;                                                       // kh * kw * C
    const void* scale;                                           // nullptr: plain copy
    int64_t ssn, ssh, ssw, ssc;                                  // element strides of scale along n, h, w, channel block
    FastDiv d_blk;                                               // by the block size along the channels
    FastDiv d_wo, d_ho, d_kw;
    FastDiv d_cv;                                                // by C / VEC (vector kernel) or C (scalar kernel)
    FastDiv d_row;                                               // by ldk / VEC or ldk
    int64_t total;                                               // work items of the launch
};

template <typename T>
__device__ __forceinline__ T scaled(T v, T s);
template <>
__device__ __forceinline__ uint16_t scaled<uint16_t>(uint16_t v, uint16_t s) {                  // bf16 bits
    return (uint16_t)f32_to_bf16_bits(__fmul_rn(bf16_bits_to_f32(v), bf16_bits_to_f32(s)));
}
template <>
__device__ __forceinline__ uint32_t scaled<uint32_t>(uint32_t v, uint32_t s) {                  // fp32 bits
    return __float_as_uint(__fmul_rn(__uint_as_float(v), __uint_as_float(s)));
}

// The pieces of a 16-byte vector times one scale: VEC == 8: bf16 pairs; VEC == 4: fp32.
template <int VEC>
__device__ __forceinline__ uint4 scaled_vec(uint4 v, const void* sp) {
    if (VEC == 8) {
        const uint32_t s2 = (uint32_t)(*reinterpret_cast<const uint16_t*>(sp)) * 0x00010001u;
        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.x) : "r"(s2));
        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.y) : "r"(s2));
        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.z) : "r"(s2));
        asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v.w) : "r"(s2));
    } else {
        const uint32_t s = *reinterpret_cast<const uint32_t*>(sp);
        v.x = scaled<uint32_t>(v.x, s); v.y = scaled<uint32_t>(v.y, s);
        v.z = scaled<uint32_t>(v.z, s); v.w = scaled<uint32_t>(v.w, s);
    }
    return v;
}

// One thread per 16-byte piece of a patch row; channels contiguous (sc == 1), C a multiple of the vector width
// (and so is the block of a scale: a piece has one scale).
template <typename V, int VEC>
__global__ void __launch_bounds__(256) patch_rows_vec_kernel(const __grid_constant__ PatchParams p) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; id < p.total; id += stride) {
        // id = m * (ldk / VEC) + piece; both factors stay below 2^31
        const uint32_t pieces = p.d_row.d;
        const int64_t m = p.total < (1ll << 31) ? (int64_t)fd_div((uint32_t)id, p.d_row) : id / pieces;
        const uint32_t piece = (uint32_t)(id - m * pieces);
        const uint32_t k0 = piece * VEC;
        V val;
        memset(&val, 0, sizeof(V));
        if (k0 < (uint32_t)p.K) {
            const uint32_t kk = fd_div(piece, p.d_cv), c = (piece - kk * p.d_cv.d) * VEC;
            const uint32_t ki = fd_div(kk, p.d_kw), kj = kk - ki * p.d_kw.d;
            const uint32_t mm = (uint32_t)m;
            const uint32_t t = fd_div(mm, p.d_wo), wo = mm - t * p.d_wo.d;
            const uint32_t n = fd_div(t, p.d_ho), ho = t - n * p.d_ho.d;
            const int hi = (int)ho * p.str_h - p.pad_h + (int)ki * p.dil_h;
            const int wi = (int)wo * p.str_w - p.pad_w + (int)kj * p.dil_w;
            if (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W) {
                const int64_t off = (int64_t)n * p.sn + (int64_t)hi * p.sh + (int64_t)wi * p.sw + c;
                val = *reinterpret_cast<const V*>(reinterpret_cast<const char*>(p.x) + off * (sizeof(V) / VEC));
                if (p.scale) {
                    const int64_t so = (int64_t)n * p.ssn + (int64_t)hi * p.ssh + (int64_t)wi * p.ssw + (int64_t)fd_div(c, p.d_blk) * p.ssc;
                    val = scaled_vec<VEC>(val, reinterpret_cast<const char*>(p.scale) + so * (sizeof(V) / VEC));
                }
            }
        }
        *reinterpret_cast<V*>(reinterpret_cast<char*>(p.out) + (m * p.ldk + k0) * (sizeof(V) / VEC)) = val;
    }
}

// One thread per G consecutive elements of a patch row (G == 8: one 16-byte store of bf16, ldk a multiple of 8;
// G == 1: any pitch); channels contiguous or not, gathered one by one (reads coalesce when sc == 1).
template <typename T, int G>
__global__ void __launch_bounds__(256) patch_rows_scalar_kernel(const __grid_constant__ PatchParams p) {
    const T* x = reinterpret_cast<const T*>(p.x);
    T* out = reinterpret_cast<T*>(p.out);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t id = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; id < p.total; id += stride) {
        const uint32_t groups = p.d_row.d;                       // ldk / G
        const int64_t m = p.total < (1ll << 31) ? (int64_t)fd_div((uint32_t)id, p.d_row) : id / groups;
        const uint32_t k0 = (uint32_t)(id - m * groups) * G;
        const uint32_t mm = (uint32_t)m;
        const uint32_t t = fd_div(mm, p.d_wo), wo = mm - t * p.d_wo.d;
        const uint32_t n = fd_div(t, p.d_ho), ho = t - n * p.d_ho.d;
        const int h0 = (int)ho * p.str_h - p.pad_h, w0 = (int)wo * p.str_w - p.pad_w;
        const int64_t xn = (int64_t)n * p.sn, sn_ = (int64_t)n * p.ssn;
        T vals[G];
        uint32_t kk = fd_div(k0, p.d_cv), c = k0 - kk * p.d_cv.d;
        uint32_t ki = fd_div(kk, p.d_kw), kj = kk - ki * p.d_kw.d;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            T val;
            memset(&val, 0, sizeof(T));
            if (k0 + g < (uint32_t)p.K) {
                const int hi = h0 + (int)ki * p.dil_h, wi = w0 + (int)kj * p.dil_w;
                if (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W) {
                    val = x[xn + (int64_t)hi * p.sh + (int64_t)wi * p.sw + (int64_t)c * p.sc];
                    if (p.scale)
                        val = scaled<T>(val, reinterpret_cast<const T*>(p.scale)[sn_ + (int64_t)hi * p.ssh + (int64_t)wi * p.ssw +
                                                                                (int64_t)fd_div(c, p.d_blk) * p.ssc]);
                }
            }
            vals[g] = val;
            if (++c == p.d_cv.d) {                               // next kernel tap
                c = 0;
                if (++kj == p.d_kw.d) { kj = 0; ++ki; }
            }
        }
        T* dst = out + m * p.ldk + k0;
        if (G == 8 && sizeof(T) == 2) {
            uint4 v;
            memcpy(&v, vals, 16);
            *reinterpret_cast<uint4*>(dst) = v;
        } else {
#pragma unroll
            for (int g = 0; g < G; ++g) dst[g] = vals[g];
        }
    }
}

// Channels strided, image columns dense (NCHW): a CTA moves a 32 (wo) x 32 (c) tile of one (n, ho, kh, kw)
// through shared memory, reading along the image row and writing along the patch row.
template <typename T>
__global__ void __launch_bounds__(256) patch_rows_tiled_kernel(const __grid_constant__ PatchParams p, int wo_tiles, int c_tiles) {
    __shared__ T tile[32][33];
    const T* x = reinterpret_cast<const T*>(p.x);
    T* out = reinterpret_cast<T*>(p.out);
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    T zero;
    memset(&zero, 0, sizeof(T));
    const T* scale = reinterpret_cast<const T*>(p.scale);
    for (uint32_t item = blockIdx.x; item < (uint32_t)p.total; item += gridDim.x) {
        // item = (((n * Ho + ho) * kh*kw + kk) * c_tiles + ct) * wo_tiles + wt, below 2^31
        uint32_t r = item;
        const int wt = (int)(r % (uint32_t)wo_tiles); r /= (uint32_t)wo_tiles;
        const int ct = (int)(r % (uint32_t)c_tiles); r /= (uint32_t)c_tiles;
        const int kk = (int)(r % (uint32_t)(p.kh * p.kw)); r /= (uint32_t)(p.kh * p.kw);
        const int ho = (int)(r % (uint32_t)p.Ho);
        const int64_t n = r / (uint32_t)p.Ho;
        const int ki = kk / p.kw, kj = kk - ki * p.kw;
        const int hi = ho * p.str_h - p.pad_h + ki * p.dil_h;
        const bool row_in = hi >= 0 && hi < p.H;
        const int wo_r = wt * 32 + tx;
        const int wi = wo_r * p.str_w - p.pad_w + kj * p.dil_w;
        const bool col_in = row_in && wo_r < p.Wo && wi >= 0 && wi < p.W;
#pragma unroll
        for (int cy = ty; cy < 32; cy += 8) {
            const int c = ct * 32 + cy;
            T v = zero;
            if (col_in && c < p.C) {
                v = x[n * p.sn + (int64_t)hi * p.sh + (int64_t)wi * p.sw + (int64_t)c * p.sc];
                if (scale) v = scaled<T>(v, scale[n * p.ssn + (int64_t)hi * p.ssh + (int64_t)wi * p.ssw + (int64_t)fd_div((uint32_t)c, p.d_blk) * p.ssc]);
            }
            tile[cy][tx] = v;
        }
        __syncthreads();
        const int c_w = ct * 32 + tx;
#pragma unroll
        for (int wy = ty; wy < 32; wy += 8) {
            const int wo = wt * 32 + wy;
            if (wo < p.Wo && c_w < p.C) {
                const int64_t m = (n * p.Ho + ho) * p.Wo + wo;
                out[m * p.ldk + (int64_t)kk * p.C + c_w] = tile[tx][wy];
            }
        }
        if (kk == 0 && ct == 0) {                                // the padding columns of these patch rows
            for (int wy = ty; wy < 32; wy += 8) {
                const int wo = wt * 32 + wy;
                if (wo < p.Wo) {
                    const int64_t m = (n * p.Ho + ho) * p.Wo + wo;
                    for (int64_t k = p.K + tx; k < p.ldk; k += 32) out[m * p.ldk + k] = zero;
                }
            }
        }
        __syncthreads();
    }
}

}  // namespace

extern "C" int vq_conv_patches(const void* x, int dtype, int64_t N, int64_t H, int64_t W, int64_t C, int64_t sn, int64_t sh,
                               int64_t sw, int64_t sc, int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w,
                               int dil_h, int dil_w, const void* scale, int64_t block, int64_t ssn, int64_t ssh, int64_t ssw,
                               int64_t ssc, void* out, int64_t ldk, void* stream) {
    const char* name = "vq_conv_patches";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(N >= 0 && H >= 1 && W >= 1 && C >= 1 && kh >= 1 && kw >= 1, "%s: bad sizes", name);
    VQ_REQUIRE(stride_h >= 1 && stride_w >= 1 && dil_h >= 1 && dil_w >= 1 && pad_h >= 0 && pad_w >= 0, "%s: bad stride, padding or dilation", name);
    VQ_REQUIRE(sn >= 0 && sh >= 0 && sw >= 0 && sc >= 0, "%s: negative stride", name);
    const int64_t eh = (int64_t)(kh - 1) * dil_h + 1, ew = (int64_t)(kw - 1) * dil_w + 1;
    const int64_t Ho = (H + 2 * pad_h - eh) / stride_h + 1, Wo = (W + 2 * pad_w - ew) / stride_w + 1;
    VQ_REQUIRE(H + 2 * pad_h >= eh && W + 2 * pad_w >= ew, "%s: the kernel window is larger than the padded image", name);
    const int64_t K = (int64_t)kh * kw * C, M = N * Ho * Wo;
    VQ_REQUIRE(ldk >= K, "%s: ldk is smaller than kh * kw * C", name);
    VQ_REQUIRE(M < (1ll << 31) && ldk < (1ll << 31) && H < (1 << 30) && W < (1 << 30), "%s: sizes must be below 2^31", name);
    if (M == 0) return 0;
    VQ_REQUIRE(x && out, "%s: null pointer", name);
    PatchParams p{};
    p.x = x; p.out = out;
    p.sn = sn; p.sh = sh; p.sw = sw; p.sc = sc; p.ldk = ldk;
    p.H = (int)H; p.W = (int)W; p.C = (int)C; p.Ho = (int)Ho; p.Wo = (int)Wo;
    p.kh = kh; p.kw = kw; p.str_h = stride_h; p.str_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w;
    p.dil_h = dil_h; p.dil_w = dil_w;
    p.K = (int)K;
    if (scale) {
        VQ_REQUIRE(block >= 1 && block < (1ll << 31) && ssn >= 0 && ssh >= 0 && ssw >= 0 && ssc >= 0, "%s: bad scale block or strides", name);
        p.scale = scale; p.ssn = ssn; p.ssh = ssh; p.ssw = ssw; p.ssc = ssc;
        p.d_blk = make_fastdiv((uint32_t)block);
    }
    p.d_wo = make_fastdiv((uint32_t)Wo);
    p.d_ho = make_fastdiv((uint32_t)Ho);
    p.d_kw = make_fastdiv((uint32_t)kw);
    const int sms = vq_sm_count();
    cudaStream_t st = (cudaStream_t)stream;
    const int es = dtype == VQ_F32 ? 4 : 2, vec = 16 / es;
    if (sc == 1) {
        const bool aligned = C % vec == 0 && ldk % vec == 0 && sn % vec == 0 && sh % vec == 0 && sw % vec == 0 &&
                             (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (!scale || block % vec == 0);
        if (aligned) {
            p.d_cv = make_fastdiv((uint32_t)(C / vec));
            p.d_row = make_fastdiv((uint32_t)(ldk / vec));
            p.total = M * (ldk / vec);
            const int64_t want = (p.total + 255) / 256;
            const int blocks = (int)(want < (int64_t)sms * 16 ? want : (int64_t)sms * 16);
            if (dtype == VQ_F32) patch_rows_vec_kernel<uint4, 4><<<blocks, 256, 0, st>>>(p);
            else patch_rows_vec_kernel<uint4, 8><<<blocks, 256, 0, st>>>(p);
            VQ_LAUNCH_CHECK("patch_rows_vec_kernel");
            return 0;
        }
    }
    if (sc == 1 || sw != 1 || C < 8) {
        const bool wide = dtype == VQ_BF16 && ldk % 8 == 0 && (uintptr_t)out % 16 == 0;
        const int G = wide ? 8 : 1;
        p.d_cv = make_fastdiv((uint32_t)C);
        p.d_row = make_fastdiv((uint32_t)(ldk / G));
        p.total = M * (ldk / G);
        const int64_t want = (p.total + 255) / 256;
        const int blocks = (int)(want < (int64_t)sms * 16 ? want : (int64_t)sms * 16);
        if (dtype == VQ_F32) patch_rows_scalar_kernel<uint32_t, 1><<<blocks, 256, 0, st>>>(p);
        else if (wide) patch_rows_scalar_kernel<uint16_t, 8><<<blocks, 256, 0, st>>>(p);
        else patch_rows_scalar_kernel<uint16_t, 1><<<blocks, 256, 0, st>>>(p);
        VQ_LAUNCH_CHECK("patch_rows_scalar_kernel");
        return 0;
    }
    const int wo_tiles = (int)((Wo + 31) / 32), c_tiles = (int)((C + 31) / 32);
    p.total = N * Ho * kh * kw * c_tiles * wo_tiles;
    VQ_REQUIRE(p.total < (1ll << 31), "%s: too many tiles for one launch", name);
    const int blocks = (int)(p.total < (int64_t)sms * 8 ? p.total : (int64_t)sms * 8);
    if (dtype == VQ_F32) patch_rows_tiled_kernel<uint32_t><<<blocks, 256, 0, st>>>(p, wo_tiles, c_tiles);
    else patch_rows_tiled_kernel<uint16_t><<<blocks, 256, 0, st>>>(p, wo_tiles, c_tiles);
    VQ_LAUNCH_CHECK("patch_rows_tiled_kernel");
    return 0;
}
