// Fused MX scale + quantize over MANY tensors in one persistent launch (whole-model weight
// quantization: hundreds of tensors, one table, one block size).
//
// The tensors are cut into tiles of blockDim.x * U 16-byte vectors; a tile never spans two
// tensors.  The descriptors and the running tile counts live in a small device workspace the
// caller provides; each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... and finds the
// tensor of a tile by a binary search over the running counts (uniform across the CTA, served
// from L1).  Per vector the work is the same as the single-tensor fast path: lane-group shuffle
// reduction of |x| bit patterns, scale rule, table lookup from shared memory, packed stores.
// HBM bound; algorithmic bytes per element: sizeof(T) read + the requested outputs.
#include <cstdlib>
#include <new>
#include <vector>

#include "vq_mx_body.cuh"
#include "vq_mx_fast.cuh"

namespace {

struct MultiParams {
    const vq_mx_item* items;     // device
    const int64_t* tile_prefix;  // device, n_items + 1 running tile counts
    int n_items;
    int64_t n_tiles;
    MxParams common;             // rule, table, code_bits, group_shift, smem flags (pointers unused)
};

template <typename T, int U>
__global__ void __launch_bounds__(1024, 1) mx_multi_kernel(const MultiParams mp) {
    extern __shared__ uint4 smem[];
    TableDev tab;
    TableRes res;
    stage_mx(mp.common, smem, tab, res);
    const ScaleRule rule = mp.common.rule;
    constexpr int N = Vec<T>::N;
    const int gs = mp.common.group_shift;
    const uint32_t tile_vecs = blockDim.x * U;

    for (int64_t tile = blockIdx.x; tile < mp.n_tiles; tile += gridDim.x) {
        // largest i with tile_prefix[i] <= tile
        int lo = 0, hi = mp.n_items;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (__ldg(mp.tile_prefix + mid) <= tile) lo = mid; else hi = mid;
        }
        const vq_mx_item* it = mp.items + lo;
        const T* in = reinterpret_cast<const T*>(it->in);
        T* out_scale = reinterpret_cast<T*>(it->out_scale);
        T* out_codes = reinterpret_cast<T*>(it->out_codes);
        float* scale_f32 = it->scale_f32;
        int8_t* exp_e8 = it->exp_e8;
        uint8_t* codes8 = it->codes;
        T* dequant = reinterpret_cast<T*>(it->dequant);
        const uint32_t nvec = (uint32_t)(it->n / N);
        const uint32_t v0 = (uint32_t)(tile - __ldg(mp.tile_prefix + lo)) * tile_vecs + threadIdx.x;

        Vec<T> x[U];
        uint32_t vi[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            vi[u] = v0 + u * blockDim.x;
            if (vi[u] < nvec) x[u].load_stream(in + (size_t)vi[u] * N);
            else {
#pragma unroll
                for (int j = 0; j < N; ++j) x[u].v[j] = 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t m = 0;
#pragma unroll
            for (int j = 0; j < N; ++j) m = max(m, abs_bits(x[u].v[j]));
            for (int o = 1; o < (1 << gs); o <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            if (vi[u] >= nvec) continue;
            const float s = block_scale<T>(rule, m);
            if ((vi[u] & ((1u << gs) - 1u)) == 0) {
                const uint32_t b = vi[u] >> gs;
                if (out_scale) store_one<T>(out_scale + b, s);
                if (scale_f32) scale_f32[b] = s;
                if (exp_e8) exp_e8[b] = (int8_t)scale_exponent(s);
            }
            mx_emit_vector<T>(tab, res, x[u], s, (size_t)vi[u] * N, out_codes, dequant, codes8, mp.common.code_bits);
        }
    }
}


// ---------------------------------------------------------------------------------------------
// Specialised kernel (see vq_mx_fast.cuh).  One descriptor can be passed by value (`single`) so
// that single-tensor ops need no workspace.
struct FastParams {
    const vq_mx_item* items;
    const int64_t* tile_prefix;
    int n_items;
    int64_t n_tiles;
    vq_mx_item single;
    // up to kInlineItems descriptors travel in the kernel parameters (constant bank): no upload
    vq_mx_item inl[32];      // kInlineItems
    int64_t inl_prefix[33];
    int n_inline;
    ScaleRule rule;
    TableDev tab;
    int group_shift;
    int allow_refine;
    int iters;                   // inner iterations per tile (one tensor lookup per tile)
};

// 32-byte chunks a thread has in flight per inner iteration: two when the chunk is quantized (registers), four
// for the scale-only pass, which keeps nothing but the block maxima
__host__ __device__ constexpr int fast_u(int out) { return out == OUT_SCALE ? 4 : 2; }

// GS > 0: the number of lanes per block is 2^GS, known at compile time (the usual block sizes);
// GS == 0: taken from the parameters.
template <typename T, int RULE, int TK, int OUT, bool SM, int U, int GS>
__global__ void __launch_bounds__(1024, 1) mx_fast2_kernel(const __grid_constant__ FastParams p) {
    extern __shared__ uint4 smem[];
    FastTab ft;
    ft.lut16 = p.tab.lut16;
    ft.lut8 = p.tab.lut8;
    ft.lo = p.tab.lo;
    ft.hi = p.tab.hi;
    ft.lo_is_zero = (p.tab.lo == 0.0f) ? 1 : 0;
    ft.flat_tiny = p.tab.flat_tiny;
    if (SM && TK == TK_LUT) {
        // the table (values or packed codes, whichever this output set reads) sits at offset 0
        const bool wide = OUT == OUT_FLOAT || OUT == OUT_FAKEQ;
        const uint4* src = reinterpret_cast<const uint4*>(wide ? (const void*)p.tab.lut16 : (const void*)p.tab.lut8);
        const int n16 = wide ? 8192 : 4096;
        for (int i = threadIdx.x; i < n16; i += blockDim.x) smem[i] = __ldg(src + i);
        __syncthreads();
    }
    constexpr int N = sizeof(T) == 2 ? 16 : 8;   // elements per 32-byte chunk
    const int gs = GS > 0 ? GS : p.group_shift;
    const uint32_t sub_chunks = blockDim.x * U;               // chunks per inner iteration
    const uint32_t tile_chunks = sub_chunks * p.iters;     // chunks per tile (one tensor lookup)
    const bool refine = p.allow_refine != 0;

    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
        const T* in;
        T* out_scale;
        T* out_codes;
        float* scale_f32;
        int8_t* exp_e8;
        uint8_t* codes8;
        uint32_t nchunk, c0;
        if (p.n_items == 1) {
            in = reinterpret_cast<const T*>(p.single.in);
            out_scale = reinterpret_cast<T*>(p.single.out_scale);
            out_codes = reinterpret_cast<T*>(OUT == OUT_FAKEQ ? p.single.dequant : p.single.out_codes);
            scale_f32 = p.single.scale_f32;
            exp_e8 = p.single.exp_e8;
            codes8 = p.single.codes;
            nchunk = (uint32_t)(p.single.n / N);
            c0 = (uint32_t)tile * tile_chunks + threadIdx.x;
        } else if (p.n_inline) {
            int lo = 0, hi = p.n_items;
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (p.inl_prefix[mid] <= tile) lo = mid; else hi = mid;
            }
            const vq_mx_item& it = p.inl[lo];
            in = reinterpret_cast<const T*>(it.in);
            out_scale = reinterpret_cast<T*>(it.out_scale);
            out_codes = reinterpret_cast<T*>(OUT == OUT_FAKEQ ? it.dequant : it.out_codes);
            scale_f32 = it.scale_f32;
            exp_e8 = it.exp_e8;
            codes8 = it.codes;
            nchunk = (uint32_t)(it.n / N);
            c0 = (uint32_t)(tile - p.inl_prefix[lo]) * tile_chunks + threadIdx.x;
        } else {
            int lo = 0, hi = p.n_items;
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (__ldg(p.tile_prefix + mid) <= tile) lo = mid; else hi = mid;
            }
            const vq_mx_item* it = p.items + lo;
            in = reinterpret_cast<const T*>(it->in);
            out_scale = reinterpret_cast<T*>(it->out_scale);
            out_codes = reinterpret_cast<T*>(OUT == OUT_FAKEQ ? it->dequant : it->out_codes);
            scale_f32 = it->scale_f32;
            exp_e8 = it->exp_e8;
            codes8 = it->codes;
            nchunk = (uint32_t)(it->n / N);
            c0 = (uint32_t)(tile - __ldg(p.tile_prefix + lo)) * tile_chunks + threadIdx.x;
        }
        for (int iter = 0; iter < p.iters; ++iter, c0 += sub_chunks) {
        if (c0 - threadIdx.x >= nchunk) break;              // uniform across the CTA
        Chunk x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t ci = c0 + u * blockDim.x;
            if (ci < nchunk) x[u].load(in + (size_t)ci * N);
            else x[u].zero();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t ci = c0 + u * blockDim.x;
            bool safe;
            uint32_t m = chunk_amax<T>(x[u], safe, refine && !ft.flat_tiny);
            if (GS > 0) {
#pragma unroll
                for (int o = 1; o < (1 << GS); o <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            } else {
                for (int o = 1; o < (1 << gs); o <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            }
            if (ci >= nchunk) continue;
            const float s = fast_scale<T, RULE>(p.rule, m);
            if ((ci & ((1u << gs) - 1u)) == 0) {
                const uint32_t b = ci >> gs;
                if (OUT == OUT_FLOAT || OUT == OUT_SCALE || OUT == OUT_FAKEQ) {
                    store_one<T>(out_scale + b, s);
                } else {
                    scale_f32[b] = s;
                    if (RULE == 1 && exp_e8) exp_e8[b] = (int8_t)scale_exponent(s);
                }
            }
            if (OUT != OUT_SCALE)
                fast_chunk<T, TK, OUT == OUT_SCALE ? OUT_FLOAT : OUT, SM>(ft, smem, x[u], s, refine && safe, (size_t)ci, out_codes, codes8);
        }
        }
    }
}

template <typename T, int RULE, int TK, int OUT, bool SM>
int launch_fast2(const FastParams& p, int threads, int blocks, size_t smem, cudaStream_t st) {
    // blocks of 2 or 4 chunks (32 / 64 elements) have the lane-group reduction unrolled
    auto k = p.group_shift == 1   ? mx_fast2_kernel<T, RULE, TK, OUT, SM, fast_u(OUT), 1>
             : p.group_shift == 2 ? mx_fast2_kernel<T, RULE, TK, OUT, SM, fast_u(OUT), 2>
                                  : mx_fast2_kernel<T, RULE, TK, OUT, SM, fast_u(OUT), 0>;
    if (smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<blocks, threads, smem, st>>>(p);
    VQ_LAUNCH_CHECK("mx_fast2_kernel");
    return 0;
}

template <typename T, int RULE, int TK>
int dispatch_out(const FastParams& p, int out, bool sm, int threads, int blocks, size_t smem, cudaStream_t st) {
    if (TK == TK_INT) sm = false;
    switch (out) {
        case OUT_SCALE:
            return launch_fast2<T, RULE, TK_INT, OUT_SCALE, false>(p, threads, blocks, smem, st);
        case OUT_FLOAT:
            return sm ? launch_fast2<T, RULE, TK, OUT_FLOAT, true>(p, threads, blocks, smem, st)
                      : launch_fast2<T, RULE, TK, OUT_FLOAT, false>(p, threads, blocks, smem, st);
        case OUT_FAKEQ:
            return sm ? launch_fast2<T, RULE, TK, OUT_FAKEQ, true>(p, threads, blocks, smem, st)
                      : launch_fast2<T, RULE, TK, OUT_FAKEQ, false>(p, threads, blocks, smem, st);
        case OUT_PACK4:
            return sm ? launch_fast2<T, RULE, TK, OUT_PACK4, true>(p, threads, blocks, smem, st)
                      : launch_fast2<T, RULE, TK, OUT_PACK4, false>(p, threads, blocks, smem, st);
        default:
            return sm ? launch_fast2<T, RULE, TK, OUT_PACK8, true>(p, threads, blocks, smem, st)
                      : launch_fast2<T, RULE, TK, OUT_PACK8, false>(p, threads, blocks, smem, st);
    }
}

template <typename T>
int dispatch_rule(const FastParams& p, int rule, int tk, int out, bool sm, int threads, int blocks, size_t smem,
                  cudaStream_t st) {
    if (rule == 1) {
        return tk == TK_INT ? dispatch_out<T, 1, TK_INT>(p, out, sm, threads, blocks, smem, st)
                            : dispatch_out<T, 1, TK_LUT>(p, out, sm, threads, blocks, smem, st);
    }
    if (p.rule.qmax == 1.0f && p.rule.stab.kind == VQ_TABLE_NONE) {      // the scale is the block maximum itself
        return tk == TK_INT ? dispatch_out<T, 2, TK_INT>(p, out, sm, threads, blocks, smem, st)
                            : dispatch_out<T, 2, TK_LUT>(p, out, sm, threads, blocks, smem, st);
    }
    return tk == TK_INT ? dispatch_out<T, 0, TK_INT>(p, out, sm, threads, blocks, smem, st)
                        : dispatch_out<T, 0, TK_LUT>(p, out, sm, threads, blocks, smem, st);
}

constexpr int kThreads = 1024;
constexpr int kU = 2;
constexpr int kInlineItems = 32;

// Everything a launch of the specialised kernel needs, decided once from the host descriptors.
struct FastLaunch {
    FastParams p;
    int dtype = 0, pow2 = 0, tk = 0, out = 0;
    bool sm = false;
    int threads = 0, blocks = 0;
    size_t smem = 0;
    bool empty = false;             // no element to process: nothing is launched
    bool upload = false;            // descriptors + running tile counts go to the device workspace
    std::vector<int64_t> prefix;    // running tile counts (upload only)
};

// 1: `L` describes the launch; 0: the arguments are outside the specialised kernel's domain.
int fast_prepare(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max, int pow2,
                 const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                 void* workspace, FastLaunch& L) {
    if (n_items < 1 || (pow2 != 0 && pow2 != 1)) return 0;
    int tk;
    const bool no_table = !table || table->kind == VQ_TABLE_NONE;
    if (no_table) tk = TK_INT;                       // scale-only pass: no table is consulted
    else if (table->kind == VQ_TABLE_INT) tk = TK_INT;
    else if (table->kind == VQ_TABLE_LUT16 && table->nan_uniform && table->lut16) tk = TK_LUT;
    else return 0;
    if (scale_table && scale_table->kind == VQ_TABLE_RUNS) return 0;
    const int N = dtype == VQ_F32 ? 8 : 16;   // elements per 32-byte chunk
    if (block % N) return 0;
    const int64_t g = block / N;
    if (g > 32 || (g & (g - 1))) return 0;
    int gs = 0;
    while ((1ll << gs) < g) ++gs;
    // every item must ask for the same output set
    int out = -1;
    int64_t total = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_mx_item& it = items[i];
        int o;
        if (no_table) {
            if (it.out_scale && !it.out_codes && !it.scale_f32 && !it.exp_e8 && !it.codes && !it.dequant) o = OUT_SCALE;
            else return 0;
        } else if (it.out_scale && it.out_codes && !it.scale_f32 && !it.exp_e8 && !it.codes && !it.dequant) o = OUT_FLOAT;
        else if (it.out_scale && it.dequant && !it.out_codes && !it.scale_f32 && !it.exp_e8 && !it.codes) o = OUT_FAKEQ;
        else if (it.codes && it.scale_f32 && !it.out_scale && !it.out_codes && !it.dequant && (code_bits == 4 || code_bits == 8))
            o = code_bits == 4 ? OUT_PACK4 : OUT_PACK8;
        else return 0;
        if (out >= 0 && o != out) return 0;
        if (it.exp_e8 && !pow2) return 0;
        if (it.n % block || it.n >= (1ll << 31) || (uintptr_t)it.in % 32 || (uintptr_t)it.out_codes % 32 || (uintptr_t)it.dequant % 32 ||
            (uintptr_t)it.codes % 16 || (uintptr_t)it.scale_f32 % 4)
            return 0;
        out = o;
        total += it.n;
    }
    const bool packed_out = out == OUT_PACK4 || out == OUT_PACK8;
    if (packed_out && tk == TK_LUT && (!table->lut8 || (uintptr_t)table->lut8 % 16)) return 0;
    if (packed_out && tk == TK_INT && (table->lo < -128.0f || table->hi > 255.0f)) return 0;
    if (n_items > kInlineItems && !workspace) return 0;
    L = FastLaunch{};
    L.dtype = dtype;
    L.pow2 = pow2;
    L.tk = tk;
    L.out = out;
    if (total == 0) {
        L.empty = true;
        return 1;
    }

    FastParams& p = L.p;
    p = FastParams{};
    p.n_items = n_items;
    p.rule.pow2 = pow2;
    p.rule.qmax = (float)quant_max;
    p.rule.bump_at = exp ? exp->bump_at : nullptr;
    p.rule.scale_of = exp ? exp->scale_of : nullptr;
    p.rule.stab = to_dev(pow2 ? nullptr : scale_table);
    p.rule.sres = TableRes{p.rule.stab.lut16, nullptr, nullptr, 0};
    p.tab = to_dev(table);
    p.group_shift = gs;
    p.allow_refine = (p.rule.stab.kind == VQ_TABLE_NONE) ? 1 : 0;

    const bool big = total >= (1ll << 22);
    const int threads = big ? 1024 : 128;
    const int sms = vq_sm_count();
    // tiles large enough to amortise the per-tile tensor lookup, small enough for >= 8 tiles per SM
    const int U = fast_u(out);
    int64_t iters = total / ((int64_t)threads * U * N * sms * 8);
    iters = iters < 1 ? 1 : (iters > 8 ? 8 : iters);
    p.iters = (int)iters;
    const int64_t tile_elems = (int64_t)threads * U * N * iters;
    if (n_items == 1) {
        p.single = items[0];
        p.n_tiles = (items[0].n + tile_elems - 1) / tile_elems;
    } else if (n_items <= kInlineItems) {
        p.n_inline = n_items;
        p.inl_prefix[0] = 0;
        for (int i = 0; i < n_items; ++i) {
            p.inl[i] = items[i];
            p.inl_prefix[i + 1] = p.inl_prefix[i] + (items[i].n + tile_elems - 1) / tile_elems;
        }
        p.n_tiles = p.inl_prefix[n_items];
    } else {
        L.upload = true;
        L.prefix.resize((size_t)n_items + 1);
        L.prefix[0] = 0;
        for (int i = 0; i < n_items; ++i) L.prefix[i + 1] = L.prefix[i] + (items[i].n + tile_elems - 1) / tile_elems;
        p.n_tiles = L.prefix[n_items];
        p.items = reinterpret_cast<const vq_mx_item*>(workspace);
        p.tile_prefix = reinterpret_cast<const int64_t*>((char*)workspace + (size_t)n_items * sizeof(vq_mx_item));
    }
    L.sm = big && tk == TK_LUT;
    L.smem = L.sm ? ((out == OUT_FLOAT || out == OUT_FAKEQ) ? 131072 : 65536) : 0;
    const int64_t cap = big ? sms : (int64_t)sms * 8;
    L.threads = threads;
    L.blocks = (int)(p.n_tiles < cap ? p.n_tiles : cap);
    return 1;
}

// Descriptors and running tile counts -> device workspace (pageable sources are staged before
// cudaMemcpyAsync returns, so the host arrays may be released right after).
int upload_descriptors(const vq_mx_item* items, const int64_t* prefix, int n_items, void* workspace, cudaStream_t st) {
    cudaError_t e1 = cudaMemcpyAsync(workspace, items, (size_t)n_items * sizeof(vq_mx_item), cudaMemcpyHostToDevice, st);
    cudaError_t e2 = cudaMemcpyAsync((char*)workspace + (size_t)n_items * sizeof(vq_mx_item), prefix,
                                     ((size_t)n_items + 1) * sizeof(int64_t), cudaMemcpyHostToDevice, st);
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return vq_set_error(VQ_ERR_CUDA, "descriptor upload failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    return 0;
}

int fast_launch(const FastLaunch& L, cudaStream_t st) {
    if (L.empty) return 0;
    return (L.dtype == VQ_F32) ? dispatch_rule<float>(L.p, L.pow2, L.tk, L.out, L.sm, L.threads, L.blocks, L.smem, st)
                               : dispatch_rule<bf16_t>(L.p, L.pow2, L.tk, L.out, L.sm, L.threads, L.blocks, L.smem, st);
}

// The generic multi-tensor kernel: always reads its descriptors from the workspace.
struct GenericLaunch {
    MultiParams mp;
    int dtype = 0;
    int blocks = 0;
    size_t smem = 0;
    std::vector<int64_t> prefix;
};

int generic_launch(const GenericLaunch& G, cudaStream_t st) {
    if (G.mp.n_tiles == 0) return 0;
    if (G.dtype == VQ_F32) {
        auto k = mx_multi_kernel<float, kU>;
        if (G.smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G.smem));
        k<<<G.blocks, kThreads, G.smem, st>>>(G.mp);
    } else {
        auto k = mx_multi_kernel<bf16_t, kU>;
        if (G.smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G.smem));
        k<<<G.blocks, kThreads, G.smem, st>>>(G.mp);
    }
    VQ_LAUNCH_CHECK("mx_multi_kernel");
    return 0;
}

// A prepared multi-tensor pass: which kernel, its parameters, whether descriptors must be uploaded.
struct MultiLaunch {
    bool fast = false;
    FastLaunch f;
    GenericLaunch g;
    bool needs_upload() const { return fast ? f.upload : true; }
    const int64_t* prefix() const { return fast ? f.prefix.data() : g.prefix.data(); }
    int launch(cudaStream_t st) const { return fast ? fast_launch(f, st) : generic_launch(g, st); }
};

// Argument checks + launch set-up shared by vq_quantize_mx_multi and the plan.  0 on success.
int multi_prepare(const char* name, const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max,
                  int pow2, const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                  void* workspace, size_t workspace_bytes, MultiLaunch& M) {
    VQ_REQUIRE(items != nullptr, "%s: null item array", name);
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(pow2 == 0 || pow2 == 1, "%s: scale rule must be 0 (amax/qmax) or 1 (power of two)", name);
    if (pow2) VQ_REQUIRE(exp && exp->bump_at && exp->scale_of, "%s: power-of-two scales need the exponent tables", name);
    VQ_REQUIRE(table && table->kind != VQ_TABLE_NONE, "%s: a table is required", name);
    VQ_REQUIRE(!scale_table || scale_table->kind == VQ_TABLE_NONE || scale_table->kind == VQ_TABLE_LUT16 ||
                   scale_table->kind == VQ_TABLE_INT, "%s: the scale table must be LUT16 or INT", name);
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 16 == 0 && workspace_bytes >= vq_quantize_mx_multi_workspace(n_items),
               "%s: workspace missing, unaligned or smaller than vq_quantize_mx_multi_workspace(n_items)", name);
    const int N = dtype == VQ_F32 ? 4 : 8;
    VQ_REQUIRE(block > 0 && block % N == 0, "%s: block must be a positive multiple of %d elements", name, N);
    const int64_t g = block / N;
    VQ_REQUIRE(g <= 32 && (g & (g - 1)) == 0, "%s: block / %d must be a power of two <= 32", name, N);
    int gs = 0;
    while ((1ll << gs) < g) ++gs;

    bool any_codes8 = false, any_values = false;
    const int64_t tile_elems = (int64_t)kThreads * kU * N;
    std::vector<int64_t> prefix((size_t)n_items + 1);
    prefix[0] = 0;
    int64_t total = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_mx_item& it = items[i];
        auto al = [](const void* q, size_t a) { return q == nullptr || (uintptr_t)q % a == 0; };
        bool ok = it.in && it.n >= 0 && it.n % block == 0 && it.n < (1ll << 31) && al(it.in, 16) && al(it.out_codes, 16) &&
                  al(it.dequant, 16) && al(it.codes, 8) && al(it.scale_f32, 4) &&
                  (it.out_scale || it.out_codes || it.scale_f32 || it.exp_e8 || it.codes || it.dequant);
        if (!ok)
            return vq_set_error(VQ_ERR_INVALID,
                                "%s: item %d needs a 16-byte aligned input, n a multiple of the block below 2^31, "
                                "aligned outputs and at least one output", name, i);
        if (it.exp_e8 && !pow2) return vq_set_error(VQ_ERR_INVALID, "%s: item %d: exp_e8 needs power-of-two scales", name, i);
        any_codes8 |= it.codes != nullptr;
        any_values |= it.out_codes != nullptr || it.dequant != nullptr;
        prefix[i + 1] = prefix[i] + (it.n + tile_elems - 1) / tile_elems;
        total += it.n;
    }
    if (any_codes8) {
        bool have = table->kind == VQ_TABLE_INT || table->lut8 || (table->kind == VQ_TABLE_RUNS && table->run_codes);
        if (!have || (code_bits != 8 && code_bits != 4))
            return vq_set_error(VQ_ERR_INVALID, "%s: packed codes need code_bits 8 or 4 and a code table", name);
    }

    if (!getenv("VOYAGER_B200_GENERIC_MX") &&
        fast_prepare(items, n_items, dtype, block, quant_max, pow2, exp, scale_table, table, code_bits, workspace, M.f)) {
        M.fast = true;
        return 0;
    }
    M.fast = false;
    GenericLaunch& G = M.g;
    MultiParams& mp = G.mp;
    mp = MultiParams{};
    mp.items = reinterpret_cast<const vq_mx_item*>(workspace);
    mp.tile_prefix = reinterpret_cast<const int64_t*>((char*)workspace + (size_t)n_items * sizeof(vq_mx_item));
    mp.n_items = n_items;
    mp.n_tiles = prefix[n_items];
    mp.common.rule.pow2 = pow2;
    mp.common.rule.qmax = (float)quant_max;
    mp.common.rule.bump_at = exp ? exp->bump_at : nullptr;
    mp.common.rule.scale_of = exp ? exp->scale_of : nullptr;
    mp.common.rule.stab = to_dev(pow2 ? nullptr : scale_table);
    mp.common.rule.sres = TableRes{mp.common.rule.stab.lut16, nullptr, nullptr, 0};
    mp.common.tab = to_dev(table);
    mp.common.code_bits = code_bits;
    mp.common.group_shift = gs;
    const bool big = total >= (1 << 21);
    mp.common.smem_lut16 = (big && table->kind == VQ_TABLE_LUT16 && any_values) ? 1 : 0;
    mp.common.smem_lut8 = (big && table->kind == VQ_TABLE_LUT16 && any_codes8 && table->lut8) ? 1 : 0;
    size_t smem = (mp.common.smem_lut16 ? 131072 : 0) + (mp.common.smem_lut8 ? 65536 : 0) +
                  (table->kind == VQ_TABLE_RUNS ? 5 * VQ_MAX_RUNS : 0);
    if ((int)smem > vq_max_smem_optin()) { mp.common.smem_lut8 = 0; smem -= 65536; }
    G.smem = smem;
    G.dtype = dtype;
    const int sms = vq_sm_count();
    G.blocks = (int)(mp.n_tiles < sms ? mp.n_tiles : sms);
    G.prefix = std::move(prefix);
    return 0;
}

}  // namespace

int vq_mx_fast_try(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max, int pow2,
                   const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                   void* workspace, cudaStream_t st) {
    FastLaunch L;
    if (!fast_prepare(items, n_items, dtype, block, quant_max, pow2, exp, scale_table, table, code_bits, workspace, L)) return 0;
    if (L.upload) {
        int rc = upload_descriptors(items, L.prefix.data(), n_items, workspace, st);
        if (rc) return rc;
    }
    int rc = fast_launch(L, st);
    return rc ? rc : 1;
}

// A prepared pass (see vq_mx_plan_create).
struct vq_mx_plan {
    MultiLaunch m;
    int device = -1;
};

extern "C" {

size_t vq_quantize_mx_multi_workspace(int n_items) {
    if (n_items < 0) return 0;
    return (size_t)n_items * sizeof(vq_mx_item) + ((size_t)n_items + 1) * sizeof(int64_t);
}

int vq_quantize_mx_multi(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max, int pow2,
                         const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                         void* workspace, size_t workspace_bytes, void* stream) {
    const char* name = "vq_quantize_mx_multi";
    VQ_REQUIRE(n_items >= 0, "%s: negative item count", name);
    if (n_items == 0) return 0;
    MultiLaunch M;
    int rc = multi_prepare(name, items, n_items, dtype, block, quant_max, pow2, exp, scale_table, table, code_bits,
                           workspace, workspace_bytes, M);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (M.needs_upload()) {
        rc = upload_descriptors(items, M.prefix(), n_items, workspace, st);
        if (rc) return rc;
    }
    return M.launch(st);
}

int vq_mx_plan_create(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max, int pow2,
                      const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table, int code_bits,
                      void* workspace, size_t workspace_bytes, void* stream, vq_mx_plan** plan_out) {
    const char* name = "vq_mx_plan_create";
    VQ_REQUIRE(plan_out != nullptr, "%s: null plan pointer", name);
    *plan_out = nullptr;
    VQ_REQUIRE(n_items >= 1, "%s: a plan needs at least one tensor", name);
    vq_mx_plan* plan = new (std::nothrow) vq_mx_plan();
    VQ_REQUIRE(plan != nullptr, "%s: out of host memory", name);
    int rc = multi_prepare(name, items, n_items, dtype, block, quant_max, pow2, exp, scale_table, table, code_bits,
                           workspace, workspace_bytes, plan->m);
    cudaStream_t st = (cudaStream_t)stream;
    if (!rc && plan->m.needs_upload()) {
        rc = upload_descriptors(items, plan->m.prefix(), n_items, workspace, st);
        // run() may be queued on any stream afterwards: the descriptors must have landed by then
        if (!rc && cudaStreamSynchronize(st) != cudaSuccess)
            rc = vq_set_error(VQ_ERR_CUDA, "%s: descriptor upload did not complete", name);
    }
    if (!rc && cudaGetDevice(&plan->device) != cudaSuccess) rc = vq_set_error(VQ_ERR_CUDA, "%s: cudaGetDevice failed", name);
    if (rc) {
        delete plan;
        return rc;
    }
    *plan_out = plan;
    return 0;
}

int vq_mx_plan_run(const vq_mx_plan* plan, void* stream) {
    VQ_REQUIRE(plan != nullptr, "vq_mx_plan_run: null plan");
    return plan->m.launch((cudaStream_t)stream);
}

void vq_mx_plan_destroy(vq_mx_plan* plan) { delete plan; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of vq_quantize_mx_multi.
//
// Some callers cannot allocate device memory at the point where they quantize: a plug-in that
// runs inside a host framework's forward pass under a closed memory pool, a serving loop that
// pre-sized everything at start-up, a driver thread that must not take the allocator lock.  For
// them the descriptor workspace the multi-tensor kernel needs lives in a fixed device array inside
// this library instead of a caller-provided buffer.  Every device that loads the library holds
// the array (about 72 KB) until the process exits.
#define VQ_STATIC_MAX_ITEMS 1024
static __device__ __align__(256) unsigned char g_static_workspace[VQ_STATIC_MAX_ITEMS * sizeof(vq_mx_item) +
                                                                  (VQ_STATIC_MAX_ITEMS + 1) * sizeof(int64_t)];

namespace {
// In host code `g_static_workspace` is only a stand-in for the device symbol; the address kernels
// may use is looked up per device, once, with that device current.
void* g_static_ws_ptr[64] = {};
}  // namespace

extern "C" {

int vq_quantize_mx_multi_static_max_items(void) { return VQ_STATIC_MAX_ITEMS; }

int vq_quantize_mx_multi_static(const vq_mx_item* items, int n_items, int dtype, int64_t block, double quant_max,
                                int pow2, const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table,
                                int code_bits, void* stream) {
    const char* name = "vq_quantize_mx_multi_static";
    VQ_REQUIRE(n_items >= 0, "%s: negative item count", name);
    if (n_items > VQ_STATIC_MAX_ITEMS)
        return vq_set_error(VQ_ERR_INVALID, "%s: %d tensors exceed the built-in workspace (at most %d per call); "
                            "split the call or use vq_quantize_mx_multi with your own workspace", name, n_items,
                            VQ_STATIC_MAX_ITEMS);
    int dev = -1;
    VQ_CUDA(cudaGetDevice(&dev));
    VQ_REQUIRE(dev >= 0 && dev < 64, "%s: device ordinal %d is outside the supported range", name, dev);
    if (!g_static_ws_ptr[dev]) {
        // first call on this device: resolve the device address of the array (no allocation)
        void* p = nullptr;
        VQ_CUDA(cudaGetSymbolAddress(&p, g_static_workspace));
        g_static_ws_ptr[dev] = p;
    }
    return vq_quantize_mx_multi(items, n_items, dtype, block, quant_max, pow2, exp, scale_table, table, code_bits,
                                g_static_ws_ptr[dev], sizeof(g_static_workspace), stream);
}

}  // extern "C"
