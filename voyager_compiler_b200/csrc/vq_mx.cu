// MX block scaling: per-block scale, and the fused scale + quantize pass.
//
// Fast path (blocks along the contiguous axis, block = 16 B vector x 2^j): a group of
// block/VEC adjacent lanes owns one block; each lane holds one 16-byte vector, the |x| maximum is
// reduced over the lane group with xor shuffles on the fp32 bit patterns (so NaN propagates like
// torch.max), every lane derives the same scale and quantizes its own vector.  x is read once.
// HBM bound; algorithmic bytes per element: sizeof(T) in + the requested outputs.
//
// General path: tensor viewed as [outer, L, inner] with blocks along L; one warp per block when
// inner == 1 (ragged or unaligned rows), one thread per (outer, block, inner) column otherwise.
#include <cstdlib>

#include "vq_common.cuh"
#include "vq_mx_body.cuh"

namespace {

template <typename T, int U>
__global__ void __launch_bounds__(1024, 1) mx_fast_kernel(const MxParams p) {
    extern __shared__ uint4 smem[];
    TableDev tab;
    TableRes res;
    stage_mx(p, smem, tab, res);
    // scale-table lookups (rare, one per block) always go through global memory
    ScaleRule rule = p.rule;

    constexpr int N = Vec<T>::N;
    const T* in = reinterpret_cast<const T*>(p.in);
    T* out_codes = reinterpret_cast<T*>(p.out_codes);
    T* dequant = reinterpret_cast<T*>(p.dequant);
    const uint32_t nvec = (uint32_t)(p.n / N);
    const uint32_t nthreads = gridDim.x * blockDim.x;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int gs = p.group_shift;
    const bool want_q = tab.kind != VQ_TABLE_NONE;

    // every lane of a warp runs the same number of iterations so the shuffles stay converged
    const uint32_t iters = (nvec + nthreads * U - 1) / (nthreads * U);
    for (uint32_t it = 0; it < iters; ++it) {
        Vec<T> x[U];
        uint32_t vi[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            vi[u] = (it * U + u) * nthreads + tid;
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
            if ((vi[u] & ((1u << gs) - 1u)) == 0) emit_scale<T>(p, vi[u] >> gs, s);
            if (!want_q) continue;
            const Divider dv(s);
            uint32_t codes[N];
            Vec<T> dq;
            const bool want_val = out_codes != nullptr || dequant != nullptr;
            const bool want_code = p.codes != nullptr;
#pragma unroll
            for (int j = 0; j < N; ++j) {
                float q = Arith<T>::rnd(dv(x[u].v[j]));
                Looked lk = table_lookup(tab, res, f32_to_bf16_bits(q), want_val, want_code);
                x[u].v[j] = lk.val;
                codes[j] = lk.code;
                dq.v[j] = Arith<T>::rnd(__fmul_rn(lk.val, s));
            }
            const size_t base = (size_t)vi[u] * N;
            if (out_codes) x[u].store(out_codes + base);
            if (dequant) dq.store(dequant + base);
            if (p.codes) {
                if (p.code_bits == 8) {
                    uint32_t* dst = reinterpret_cast<uint32_t*>(p.codes + base);
#pragma unroll
                    for (int j = 0; j < N / 4; ++j)
                        __stcs(dst + j, codes[4 * j] | (codes[4 * j + 1] << 8) | (codes[4 * j + 2] << 16) | (codes[4 * j + 3] << 24));
                } else {
                    uint32_t w = 0;
#pragma unroll
                    for (int j = 0; j < N; ++j) w |= (codes[j] & 0xFu) << (4 * j);
                    if (N == 8) __stcs(reinterpret_cast<uint32_t*>(p.codes + base / 2), w);
                    else *reinterpret_cast<uint16_t*>(p.codes + base / 2) = (uint16_t)w;
                }
            }
        }
    }
}

// General path.  warp_mode: one warp per (outer, block) with inner == 1; else one thread per
// (outer, block, inner) column.
template <typename T>
__global__ void __launch_bounds__(256) mx_general_kernel(const MxParams p, int warp_mode) {
    extern __shared__ uint4 smem[];
    TableDev tab;
    TableRes res;
    stage_mx(p, smem, tab, res);
    const T* in = reinterpret_cast<const T*>(p.in);
    T* out_codes = reinterpret_cast<T*>(p.out_codes);
    T* dequant = reinterpret_cast<T*>(p.dequant);
    const bool want_q = tab.kind != VQ_TABLE_NONE;
    const int64_t nblocks = p.outer * p.nblk * (warp_mode ? 1 : p.inner);

    if (warp_mode) {
        const int lane = threadIdx.x & 31;
        const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
        for (int64_t b = warp; b < nblocks; b += nwarps) {
            const int64_t o = b / p.nblk, blk = b - o * p.nblk;
            const int64_t l0 = blk * p.block;
            const int64_t len = (p.L - l0 < p.block) ? p.L - l0 : p.block;
            const int64_t base = o * p.L + l0;
            uint32_t m = 0;
            for (int64_t l = lane; l < len; l += 32) m = max(m, abs_bits(load_one<T>(in + base + l)));
            for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
            const float s = block_scale<T>(p.rule, m);
            if (lane == 0) emit_scale<T>(p, b, s);
            if (!want_q) continue;
            const Divider dv(s);
            for (int64_t l = lane; l < len; l += 32) {
                float q = Arith<T>::rnd(dv(load_one<T>(in + base + l)));
                Looked lk = table_lookup(tab, res, f32_to_bf16_bits(q), true, p.codes != nullptr);
                if (out_codes) store_one<T>(out_codes + base + l, lk.val);
                if (dequant) store_one<T>(dequant + base + l, Arith<T>::rnd(__fmul_rn(lk.val, s)));
                if (p.codes) p.codes[base + l] = (uint8_t)lk.code;
            }
        }
        return;
    }
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
    for (int64_t b = tid; b < nblocks; b += nthreads) {
        const int64_t i = b % p.inner;
        const int64_t ob = b / p.inner;
        const int64_t o = ob / p.nblk, blk = ob - o * p.nblk;
        const int64_t l0 = blk * p.block;
        const int64_t len = (p.L - l0 < p.block) ? p.L - l0 : p.block;
        const int64_t base = (o * p.L + l0) * p.inner + i;
        uint32_t m = 0;
        for (int64_t l = 0; l < len; ++l) m = max(m, abs_bits(load_one<T>(in + base + l * p.inner)));
        const float s = block_scale<T>(p.rule, m);
        emit_scale<T>(p, b, s);
        if (!want_q) continue;
        const Divider dv(s);
        for (int64_t l = 0; l < len; ++l) {
            const int64_t e = base + l * p.inner;
            float q = Arith<T>::rnd(dv(load_one<T>(in + e)));
            Looked lk = table_lookup(tab, res, f32_to_bf16_bits(q), true, p.codes != nullptr);
            if (out_codes) store_one<T>(out_codes + e, lk.val);
            if (dequant) store_one<T>(dequant + e, Arith<T>::rnd(__fmul_rn(lk.val, s)));
            if (p.codes) p.codes[e] = (uint8_t)lk.code;
        }
    }
}

int check_mx_table(const vq_table* t, const char* what) {
    if (!t || t->kind == VQ_TABLE_NONE) return 0;
    if (t->kind == VQ_TABLE_LUT16) {
        if (!t->lut16 || (uintptr_t)t->lut16 % 16) return vq_set_error(VQ_ERR_INVALID, "%s: LUT16 table needs a 16-byte aligned lut16", what);
        if (t->lut8 && (uintptr_t)t->lut8 % 16) return vq_set_error(VQ_ERR_INVALID, "%s: lut8 must be 16-byte aligned", what);
    } else if (t->kind == VQ_TABLE_INT) {
        if (!(t->lo <= t->hi)) return vq_set_error(VQ_ERR_INVALID, "%s: INT table needs lo <= hi", what);
    } else if (t->kind == VQ_TABLE_RUNS) {
        if (t->n_runs < 1 || t->n_runs > VQ_MAX_RUNS || !t->run_vals || (t->n_runs > 1 && !t->run_keys))
            return vq_set_error(VQ_ERR_INVALID, "%s: RUNS table needs 1..512 runs with keys and values", what);
    } else {
        return vq_set_error(VQ_ERR_INVALID, "%s: unknown table kind %d", what, t->kind);
    }
    return 0;
}

int run_mx(const char* name, const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, int64_t block,
           double quant_max, int pow2, const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table,
           void* out_scale, void* out_codes, const vq_mx_extras* ex, void* stream) {
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(outer >= 0 && L >= 0 && inner >= 0, "%s: negative size", name);
    VQ_REQUIRE(block > 0, "%s: block_size must be positive", name);
    const int64_t n = outer * L * inner;
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr, "%s: null input", name);
    VQ_REQUIRE(pow2 >= 0 && pow2 <= 2, "%s: scale rule must be 0 (amax/qmax), 1 (power of two) or 2 (raw maximum)", name);
    if (pow2 == 1) VQ_REQUIRE(exp && exp->bump_at && exp->scale_of, "%s: power-of-two scales need the exponent tables", name);
    if (int rc = check_mx_table(scale_table, name)) return rc;
    if (int rc = check_mx_table(table, name)) return rc;
    const bool has_tab = table && table->kind != VQ_TABLE_NONE;
    if (!has_tab) VQ_REQUIRE(!out_codes && (!ex || (!ex->codes && !ex->dequant)), "%s: code outputs need a table", name);

    MxParams p{};
    p.in = in;
    p.outer = outer; p.L = L; p.inner = inner;
    p.block = block > L ? L : block;   // an axis shorter than a block is one block
    p.nblk = (L + p.block - 1) / p.block;
    p.n = n;
    p.rule.pow2 = pow2;
    p.rule.qmax = (float)quant_max;
    p.rule.bump_at = exp ? exp->bump_at : nullptr;
    p.rule.scale_of = exp ? exp->scale_of : nullptr;
    p.rule.stab = to_dev(pow2 ? nullptr : scale_table);
    if (pow2 == 2) VQ_REQUIRE(!table || table->kind == VQ_TABLE_NONE, "%s: the raw-maximum rule produces no codes", name);
    p.rule.sres = TableRes{p.rule.stab.lut16, p.rule.stab.run_keys, p.rule.stab.run_vals, 0};
    if (p.rule.stab.kind == VQ_TABLE_RUNS)
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: RUNS tables are not accepted for the scale table; pass LUT16 or INT", name);
    p.tab = to_dev(table);
    p.out_scale = out_scale;
    p.out_codes = out_codes;
    if (ex) {
        p.scale_f32 = ex->scale_f32;
        p.exp_e8 = ex->exp_e8;
        p.codes = ex->codes;
        p.code_bits = ex->code_bits;
        p.dequant = ex->dequant;
    }
    if (p.codes) {
        VQ_REQUIRE(p.code_bits == 8 || p.code_bits == 4, "%s: code_bits must be 8 or 4", name);
        VQ_REQUIRE(p.tab.kind == VQ_TABLE_INT || p.tab.lut8 || (p.tab.kind == VQ_TABLE_RUNS && p.tab.run_codes),
                   "%s: packed codes need a code table (lut8 / run_codes) or an INT table", name);
    }
    if (p.exp_e8) VQ_REQUIRE(pow2 == 1, "%s: exp_e8 needs power-of-two scales", name);
    VQ_REQUIRE(out_scale || out_codes || p.scale_f32 || p.exp_e8 || p.codes || p.dequant, "%s: no output buffer", name);

    const int N = dtype == VQ_F32 ? 4 : 8;
    const size_t esz = dtype == VQ_F32 ? 4 : 2;
    const int sms = vq_sm_count();
    cudaStream_t st = (cudaStream_t)stream;

    // ---- fast path test
    bool fast = inner == 1 && (L % p.block == 0) && (p.block % N == 0);
    int gs = 0;
    if (fast) {
        int64_t g = p.block / N;
        fast = g <= 32 && (g & (g - 1)) == 0;
        while ((1ll << gs) < g) ++gs;
    }
    auto al16 = [](const void* q) { return q == nullptr || (uintptr_t)q % 16 == 0; };
    fast = fast && al16(in) && al16(out_codes) && al16(p.dequant) && (p.codes == nullptr || (uintptr_t)p.codes % 8 == 0);
    if (p.codes && p.code_bits == 4) {
        if (!fast) return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: 4-bit packed codes need blocks along a contiguous, 16-byte aligned axis with block %% %d == 0", name, N);
    }

    const bool big = n >= (1 << 21);
    const bool need_values = has_tab && (out_codes || p.dequant);
    if (fast && pow2 != 2 && n < (1ll << 31) && !getenv("VOYAGER_B200_GENERIC_MX")) {
        vq_mx_item item{};
        item.in = in; item.out_scale = out_scale; item.out_codes = out_codes; item.scale_f32 = p.scale_f32;
        item.exp_e8 = p.exp_e8; item.codes = p.codes; item.dequant = p.dequant; item.n = n;
        int fr = vq_mx_fast_try(&item, 1, dtype, p.block, quant_max, pow2, exp, scale_table, table, p.code_bits,
                                nullptr, st);
        if (fr != 0) return fr < 0 ? fr : 0;
    }
    if (fast) {
        p.group_shift = gs;
        // pieces of at most 2^30 elements, whole blocks each
        const int64_t max_piece = (1ll << 30) / p.block * p.block;
        for (int64_t off = 0; off < n; off += max_piece) {
            MxParams q = p;
            q.n = (n - off < max_piece) ? n - off : max_piece;
            const int64_t boff = off / p.block;
            q.in = (const char*)in + off * esz;
            if (out_scale) q.out_scale = (char*)out_scale + boff * esz;
            if (out_codes) q.out_codes = (char*)out_codes + off * esz;
            if (p.scale_f32) q.scale_f32 = p.scale_f32 + boff;
            if (p.exp_e8) q.exp_e8 = p.exp_e8 + boff;
            if (p.codes) q.codes = p.codes + (p.code_bits == 4 ? off / 2 : off);
            if (p.dequant) q.dequant = (char*)p.dequant + off * esz;
            size_t smem = 0;
            q.smem_lut16 = (big && q.tab.kind == VQ_TABLE_LUT16 && need_values) ? 1 : 0;
            q.smem_lut8 = (big && q.tab.kind == VQ_TABLE_LUT16 && q.codes && q.tab.lut8) ? 1 : 0;
            smem = (q.smem_lut16 ? 131072 : 0) + (q.smem_lut8 ? 65536 : 0) + (q.tab.kind == VQ_TABLE_RUNS ? 5 * VQ_MAX_RUNS : 0);
            if ((int)smem > vq_max_smem_optin()) { q.smem_lut8 = 0; smem -= 65536; }
            int threads, blocks;
            const int64_t nvec = q.n / N;
            if (smem > 48 * 1024 || big) {
                threads = 1024;
                blocks = sms;
            } else {
                threads = 256;
                int64_t want = (nvec + threads - 1) / threads;
                blocks = (int)(want < 1 ? 1 : (want > (int64_t)sms * 8 ? (int64_t)sms * 8 : want));
            }
            if (dtype == VQ_F32) {
                auto k = mx_fast_kernel<float, 2>;
                if (smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                k<<<blocks, threads, smem, st>>>(q);
            } else {
                auto k = mx_fast_kernel<bf16_t, 2>;
                if (smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                k<<<blocks, threads, smem, st>>>(q);
            }
            VQ_LAUNCH_CHECK("mx_fast_kernel");
        }
        return 0;
    }

    // ---- general path
    const int warp_mode = inner == 1 ? 1 : 0;
    const int64_t units = outer * p.nblk * (warp_mode ? 1 : inner);
    const int threads = 256;
    int64_t want = warp_mode ? (units + 7) / 8 : (units + threads - 1) / threads;
    int blocks = (int)(want < 1 ? 1 : (want > (int64_t)sms * 16 ? (int64_t)sms * 16 : want));
    size_t smem = (p.tab.kind == VQ_TABLE_RUNS) ? 5 * VQ_MAX_RUNS : 0;
    if (dtype == VQ_F32) mx_general_kernel<float><<<blocks, threads, smem, st>>>(p, warp_mode);
    else mx_general_kernel<bf16_t><<<blocks, threads, smem, st>>>(p, warp_mode);
    VQ_LAUNCH_CHECK("mx_general_kernel");
    return 0;
}

}  // namespace

extern "C" {

int vq_mx_scale(const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, int64_t block, double quant_max,
                int pow2, const vq_exp_tables* exp, const vq_table* scale_table, void* out_scale, void* stream) {
    if (!out_scale) return vq_set_error(VQ_ERR_INVALID, "vq_mx_scale: null output");
    return run_mx("vq_mx_scale", in, dtype, outer, L, inner, block, quant_max, pow2, exp, scale_table, nullptr,
                  out_scale, nullptr, nullptr, stream);
}

int vq_quantize_mx(const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, int64_t block, double quant_max,
                   int pow2, const vq_exp_tables* exp, const vq_table* scale_table, const vq_table* table,
                   void* out_scale, void* out_codes, const vq_mx_extras* extras, void* stream) {
    if (!table || table->kind == VQ_TABLE_NONE) return vq_set_error(VQ_ERR_INVALID, "vq_quantize_mx: a table is required");
    return run_mx("vq_quantize_mx", in, dtype, outer, L, inner, block, quant_max, pow2, exp, scale_table, table,
                  out_scale, out_codes, extras, stream);
}

}  // extern "C"
