// Streaming element-wise kernels: table map, quantize, dequantize.
//
// One persistent kernel template serves the three ops.  Each thread moves 16-byte vectors
// (4 fp32 / 8 bf16) with streaming loads and stores; the 65 536-entry table (128 KB) is staged in
// shared memory once per CTA when the tensor is large, read through L1/L2 when it is small, and
// replaced by arithmetic (INT) or by a run-start binary search (RUNS, <= 1 KB of shared memory)
// when the host has proven the table equivalent.  HBM bound: 2 x sizeof(T) bytes per element.
#include <cstdlib>

#include "vq_common.cuh"

namespace {

enum { OP_MAP = 0, OP_QUANT = 1, OP_DEQUANT = 2, OP_FAKEQ = 3 };   // FAKEQ: quantize then multiply by the scale

struct EwParams {
    const void* in;
    void* out;
    uint8_t* codes;
    int code_bits;
    int64_t n;          // elements handled by this launch
    const void* scale;
    const void* zp;
    int smode;
    int vec_ok;         // 16-byte vector path usable
    int vec_uniform;    // every aligned vector lies inside one scale block
    uint32_t K, bs, nb;
    FastDiv divK, divB;
    int ndim;
    int64_t size[6], div[6], stride[6];
    int small;          // STRIDED: n below 2^31, the 32-bit dividers below apply
    FastDiv fsize[6], fdiv[6];
    TableDev t0, t1;
    int smem_lut;       // 0: none, 1: t0's LUT16 staged in shared memory, 2: t1's
};

__device__ __forceinline__ int pow2_steps(int n_runs) {
    int keys = n_runs - 1, p = 1;
    while (p <= keys) p <<= 1;  // smallest power of two > keys
    return p >> 1;
}

// Stage tables in shared memory and resolve the pointers the lookups use.
__device__ __forceinline__ void stage_tables(const EwParams& p, uint4* smem, TableRes& r0, TableRes& r1) {
    r0 = TableRes{p.t0.lut16, p.t0.run_keys, p.t0.run_vals, 0};
    r1 = TableRes{p.t1.lut16, p.t1.run_keys, p.t1.run_vals, 0};
    uint16_t* s16 = reinterpret_cast<uint16_t*>(smem);
    if (p.smem_lut) {
        const TableDev& t = (p.smem_lut == 1) ? p.t0 : p.t1;
        const uint4* src = reinterpret_cast<const uint4*>(t.lut16);
        for (int i = threadIdx.x; i < 8192; i += blockDim.x) smem[i] = __ldg(src + i);
        if (p.smem_lut == 1) r0.lut = s16; else r1.lut = s16;
        s16 += 65536;
    }
    // run tables: VQ_MAX_RUNS keys (padded with 0xFFFF), then VQ_MAX_RUNS values, per table
    const TableDev* ts[2] = {&p.t0, &p.t1};
    TableRes* rs[2] = {&r0, &r1};
    for (int k = 0; k < 2; ++k) {
        if (ts[k]->kind != VQ_TABLE_RUNS) continue;
        int nr = ts[k]->n_runs;
        uint16_t* keys = s16;
        uint16_t* vals = s16 + VQ_MAX_RUNS;
        for (int i = threadIdx.x; i < VQ_MAX_RUNS; i += blockDim.x) {
            keys[i] = (i < nr - 1) ? ts[k]->run_keys[i] : (uint16_t)0xFFFF;
            vals[i] = (i < nr) ? ts[k]->run_vals[i] : (uint16_t)0;
        }
        rs[k]->rk = keys;
        rs[k]->rv = vals;
        rs[k]->steps = pow2_steps(nr);
        s16 += 2 * VQ_MAX_RUNS;
    }
    __syncthreads();
}

template <typename T, int OP>
__device__ __forceinline__ float apply_one(const EwParams& p, const TableRes& r0, const TableRes& r1, float x,
                                           float s, const Divider& dv, float zp, bool has_zp, uint32_t& code) {
    uint32_t pat = 0;
    float val;
    if (OP == OP_MAP) {
        val = table_value(p.t0, r0, x, pat);
    } else if (OP == OP_QUANT) {
        float q = Arith<T>::rnd(dv(x));
        if (has_zp) q = Arith<T>::rnd(__fadd_rn(q, zp));
        Looked lk = table_lookup(p.t0, r0, f32_to_bf16_bits(q), p.out != nullptr, p.codes != nullptr);
        val = lk.val;
        code = lk.code;
    } else if (OP == OP_FAKEQ) {
        const float q = Arith<T>::rnd(dv(x));
        val = Arith<T>::rnd(__fmul_rn(table_value(p.t0, r0, q, pat), s));
    } else {
        float v = x;
        if (p.t0.kind != VQ_TABLE_NONE) v = table_value(p.t0, r0, v, pat);
        if (has_zp) v = Arith<T>::rnd(__fsub_rn(v, zp));
        v = Arith<T>::rnd(__fmul_rn(v, s));
        if (p.t1.kind != VQ_TABLE_NONE) v = table_value(p.t1, r1, v, pat);
        val = v;
    }
    return val;
}

__device__ __forceinline__ int64_t strided_index(const EwParams& p, int64_t i) {
    int64_t idx = 0;
    if (p.small) {
        uint32_t r = (uint32_t)i;
        for (int d = p.ndim - 1; d > 0; --d) {
            const uint32_t q = fd_div(r, p.fsize[d]);
            idx += (int64_t)fd_div(r - q * p.fsize[d].d, p.fdiv[d]) * p.stride[d];
            r = q;
        }
        return idx + (int64_t)fd_div(r, p.fdiv[0]) * p.stride[0];
    }
    for (int d = p.ndim - 1; d >= 0; --d) {
        int64_t c = i % p.size[d];
        i /= p.size[d];
        idx += (c / p.div[d]) * p.stride[d];
    }
    return idx;
}

template <typename T>
__device__ __forceinline__ uint32_t rowblock_index(const EwParams& p, uint32_t i) {
    uint32_t row = fd_div(i, p.divK);
    uint32_t col = i - row * p.K;
    return row * p.nb + fd_div(col, p.divB);
}

template <typename T, int OP>
__global__ void __launch_bounds__(1024, 1) ew_kernel(const EwParams p) {
    extern __shared__ uint4 smem[];
    TableRes r0, r1;
    stage_tables(p, smem, r0, r1);

    const T* in = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    const T* scale = reinterpret_cast<const T*>(p.scale);
    const T* zps = reinterpret_cast<const T*>(p.zp);
    const bool has_zp = zps != nullptr;
    constexpr int N = Vec<T>::N;

    float s_all = 1.0f, z_all = 0.0f;
    if (OP != OP_MAP && p.smode == VQ_SCALE_SCALAR) {
        s_all = load_one<T>(scale);
        if (has_zp) z_all = load_one<T>(zps);
    }

    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;

    if (!p.vec_ok) {
        for (int64_t i = tid; i < p.n; i += nthreads) {
            float s = s_all, z = z_all;
            if (OP != OP_MAP && p.smode != VQ_SCALE_SCALAR) {
                int64_t si = (p.smode == VQ_SCALE_ROWBLOCK) ? (int64_t)rowblock_index<T>(p, (uint32_t)i)
                                                             : strided_index(p, i);
                s = load_one<T>(scale + si);
                if (has_zp) z = load_one<T>(zps + si);
            }
            Divider dv(s);
            uint32_t code = 0;
            float val = apply_one<T, OP>(p, r0, r1, load_one<T>(in + i), s, dv, z, has_zp, code);
            if (out) store_one<T>(out + i, val);
            if (OP == OP_QUANT && p.codes) p.codes[i] = (uint8_t)code;  // code_bits == 8 on this path
        }
        return;
    }

    const int64_t nvec = p.n / N;
    for (int64_t v = tid; v < nvec; v += nthreads) {
        const uint32_t base = (uint32_t)(v * N);
        Vec<T> x;
        x.load_stream(in + base);
        float s = s_all, z = z_all;
        uint32_t si = 0;
        const bool per_elem = (OP != OP_MAP) && p.smode == VQ_SCALE_ROWBLOCK && !p.vec_uniform;
        if (OP != OP_MAP && p.smode == VQ_SCALE_ROWBLOCK && p.vec_uniform) {
            si = rowblock_index<T>(p, base);
            s = load_one<T>(scale + si);
            if (has_zp) z = load_one<T>(zps + si);
        }
        Divider dv(s);
        uint32_t codes[N];
#pragma unroll
        for (int j = 0; j < N; ++j) {
            if (per_elem) {
                si = rowblock_index<T>(p, base + j);
                s = load_one<T>(scale + si);
                if (has_zp) z = load_one<T>(zps + si);
                dv = Divider(s);
            }
            codes[j] = 0;
            x.v[j] = apply_one<T, OP>(p, r0, r1, x.v[j], s, dv, z, has_zp, codes[j]);
        }
        if (out) x.store(out + base);
        if (OP == OP_QUANT && p.codes) {
            if (p.code_bits == 8) {
                uint32_t w[N / 4];
#pragma unroll
                for (int j = 0; j < N / 4; ++j)
                    w[j] = codes[4 * j] | (codes[4 * j + 1] << 8) | (codes[4 * j + 2] << 16) | (codes[4 * j + 3] << 24);
                uint32_t* dst = reinterpret_cast<uint32_t*>(p.codes + base);
#pragma unroll
                for (int j = 0; j < N / 4; ++j) dst[j] = w[j];
            } else {
                uint32_t w = 0;
#pragma unroll
                for (int j = 0; j < N; ++j) w |= (codes[j] & 0xFu) << (4 * j);
                if (N == 8) *reinterpret_cast<uint32_t*>(p.codes + base / 2) = w;
                else *reinterpret_cast<uint16_t*>(p.codes + base / 2) = (uint16_t)w;
            }
        }
    }
    // ragged tail (fewer than N elements): one thread, in order, so nibble pairs stay together
    if (tid == 0 && nvec * N < p.n) {
        uint32_t pending = 0;
        for (int64_t i = nvec * N; i < p.n; ++i) {
            float s = s_all, z = z_all;
            if (OP != OP_MAP && p.smode == VQ_SCALE_ROWBLOCK) {
                uint32_t si = rowblock_index<T>(p, (uint32_t)i);
                s = load_one<T>(scale + si);
                if (has_zp) z = load_one<T>(zps + si);
            }
            Divider dv(s);
            uint32_t code = 0;
            float val = apply_one<T, OP>(p, r0, r1, load_one<T>(in + i), s, dv, z, has_zp, code);
            if (out) store_one<T>(out + i, val);
            if (OP == OP_QUANT && p.codes) {
                if (p.code_bits == 8) p.codes[i] = (uint8_t)code;
                else if (i & 1) p.codes[i >> 1] = (uint8_t)(pending | ((code & 0xFu) << 4));
                else { pending = code & 0xFu; p.codes[i >> 1] = (uint8_t)pending; }
            }
        }
    }
}

int check_table(const vq_table* t, const char* what, bool required) {
    if (!t || t->kind == VQ_TABLE_NONE) {
        if (required) return vq_set_error(VQ_ERR_INVALID, "%s: a table is required", what);
        return 0;
    }
    switch (t->kind) {
        case VQ_TABLE_LUT16:
            if (!t->lut16) return vq_set_error(VQ_ERR_INVALID, "%s: LUT16 table without lut16 pointer", what);
            if ((uintptr_t)t->lut16 % 16) return vq_set_error(VQ_ERR_INVALID, "%s: lut16 must be 16-byte aligned", what);
            return 0;
        case VQ_TABLE_INT:
            if (!(t->lo <= t->hi)) return vq_set_error(VQ_ERR_INVALID, "%s: INT table needs lo <= hi", what);
            return 0;
        case VQ_TABLE_RUNS:
            if (t->n_runs < 1 || t->n_runs > VQ_MAX_RUNS || !t->run_vals || (t->n_runs > 1 && !t->run_keys))
                return vq_set_error(VQ_ERR_INVALID, "%s: RUNS table needs 1..512 runs with keys and values", what);
            return 0;
        default:
            return vq_set_error(VQ_ERR_INVALID, "%s: unknown table kind %d", what, t->kind);
    }
}

template <typename T, int OP>
int launch_ew(EwParams& p, cudaStream_t stream) {
    constexpr int N = Vec<T>::N;
    // Large tensors stage the LUT in shared memory (one 1024-thread CTA per SM, persistent);
    // small ones read the table through the cache hierarchy with a conventional grid.
    size_t smem = 0;
    p.smem_lut = 0;
    const int64_t big = 1 << 21;
    if (p.n >= big) {
        if (OP != OP_DEQUANT || p.t1.kind != VQ_TABLE_LUT16) {
            if (p.t0.kind == VQ_TABLE_LUT16) p.smem_lut = 1;
        } else {
            p.smem_lut = 2;  // the output table sees every element; an input table too, but one must win
        }
    }
    if (p.smem_lut) smem += 65536 * 2;
    if (p.t0.kind == VQ_TABLE_RUNS) smem += 4 * VQ_MAX_RUNS;
    if (p.t1.kind == VQ_TABLE_RUNS) smem += 4 * VQ_MAX_RUNS;
    if ((int)smem > vq_max_smem_optin()) { smem -= 65536 * 2; p.smem_lut = 0; }

    int threads, blocks;
    const int sms = vq_sm_count();
    if (p.smem_lut) {
        threads = 1024;
        blocks = sms;
    } else {
        threads = 256;
        int64_t work = p.vec_ok ? (p.n + N - 1) / N : p.n;
        int64_t want = (work + threads - 1) / threads;
        int64_t cap = (int64_t)sms * 8;
        blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    }
    auto kern = ew_kernel<T, OP>;
    if (smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<blocks, threads, smem, stream>>>(p);
    VQ_LAUNCH_CHECK("ew_kernel");
    return 0;
}

template <int OP>
int run_ew(const void* in, int dtype, int64_t n, const void* scale, const void* zp, const vq_scale_layout* layout,
           const vq_table* t0, const vq_table* t1, void* out, uint8_t* codes, int code_bits, void* stream) {
    const char* name = OP == OP_MAP ? "vq_lut_map" : OP == OP_QUANT ? "vq_quantize" : OP == OP_FAKEQ ? "vq_fake_quantize" : "vq_dequantize";
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(n >= 0, "%s: negative element count", name);
    if (n == 0) return 0;
    VQ_REQUIRE(in != nullptr, "%s: null input", name);
    VQ_REQUIRE(out != nullptr || (OP == OP_QUANT && codes != nullptr), "%s: no output buffer", name);
    if (int rc = check_table(t0, name, OP != OP_DEQUANT)) return rc;
    if (int rc = check_table(t1, name, false)) return rc;
    const size_t esz = dtype == VQ_F32 ? 4 : 2;
    const int N = dtype == VQ_F32 ? 4 : 8;
    if (!getenv("VOYAGER_B200_GENERIC_EW")) {
        int fr = vq_ew_fast_try(OP, in, dtype, n, scale, zp, layout, t0, t1, out, codes, (cudaStream_t)stream);
        if (fr != 0) return fr < 0 ? fr : 0;
    }

    EwParams p{};
    p.t0 = to_dev(t0);
    p.t1 = to_dev(t1);
    p.code_bits = code_bits;
    p.smode = VQ_SCALE_SCALAR;
    p.zp = zp;
    p.scale = scale;
    if (OP != OP_MAP) {
        VQ_REQUIRE(scale != nullptr && layout != nullptr, "%s: scale and layout are required", name);
        p.smode = layout->mode;
        VQ_REQUIRE(p.smode >= VQ_SCALE_SCALAR && p.smode <= VQ_SCALE_STRIDED, "%s: bad scale mode", name);
    }
    if (codes) {
        VQ_REQUIRE(code_bits == 8 || code_bits == 4, "%s: code_bits must be 8 or 4", name);
        VQ_REQUIRE(p.t0.kind == VQ_TABLE_INT || p.t0.lut8 || (p.t0.kind == VQ_TABLE_RUNS && p.t0.run_codes),
                   "%s: packed codes need a code table (lut8 / run_codes) or an INT table", name);
    }

    bool aligned = ((uintptr_t)in % 16 == 0) && (!out || (uintptr_t)out % 16 == 0) && (!codes || (uintptr_t)codes % 8 == 0);
    int64_t rows = 1, K = n;
    if (p.smode == VQ_SCALE_ROWBLOCK) {
        rows = layout->rows; K = layout->K;
        VQ_REQUIRE(rows > 0 && K > 0 && layout->block > 0 && rows * K == n, "%s: ROWBLOCK layout does not match n", name);
        VQ_REQUIRE(K < (1ll << 31), "%s: row length must be below 2^31", name);
        int64_t bs = layout->block > K ? K : layout->block;
        p.K = (uint32_t)K; p.bs = (uint32_t)bs; p.nb = (uint32_t)((K + bs - 1) / bs);
        p.divK = make_fastdiv(p.K); p.divB = make_fastdiv(p.bs);
        p.vec_uniform = (K % N == 0) && (bs % N == 0);
    } else if (p.smode == VQ_SCALE_STRIDED) {
        VQ_REQUIRE(layout->ndim >= 1 && layout->ndim <= 6, "%s: STRIDED layout needs 1..6 dims", name);
        int64_t tot = 1;
        p.ndim = 0;
        for (int d = 0; d < layout->ndim; ++d) {
            VQ_REQUIRE(layout->size[d] > 0 && layout->div[d] > 0, "%s: bad STRIDED dim %d", name, d);
            tot *= layout->size[d];
            const int64_t sz = layout->size[d], dv = layout->div[d] > sz ? sz : layout->div[d];
            const int64_t sd = dv >= sz ? 0 : layout->stride[d];          // one block over the whole dim: a broadcast
            const int last = p.ndim - 1;
            // adjacent dims fold into one when the scale index is linear over the pair: both broadcast, or both
            // undivided with the outer stride equal to the inner extent
            if (last >= 0 && ((p.stride[last] == 0 && sd == 0) ||
                              (p.div[last] == 1 && dv == 1 && sd != 0 && p.stride[last] == sd * sz))) {
                p.size[last] *= sz;
                if (sd == 0) p.div[last] = p.size[last];
                else p.stride[last] = sd;
                continue;
            }
            p.size[p.ndim] = sz; p.div[p.ndim] = sd == 0 ? sz : dv; p.stride[p.ndim] = sd;
            ++p.ndim;
        }
        VQ_REQUIRE(tot == n, "%s: STRIDED sizes do not multiply to n", name);
        p.small = n < (1ll << 31) ? 1 : 0;
        if (p.small) {
            for (int d = 0; d < p.ndim; ++d) {
                p.fsize[d] = make_fastdiv((uint32_t)p.size[d]);
                p.fdiv[d] = make_fastdiv((uint32_t)p.div[d]);
            }
        }
        aligned = false;  // scalar path
    }
    if (codes && code_bits == 4)
        VQ_REQUIRE(aligned && p.smode != VQ_SCALE_STRIDED, "%s: 4-bit codes need 16-byte aligned buffers and a SCALAR/ROWBLOCK layout", name);
    if (!aligned && p.smode == VQ_SCALE_ROWBLOCK) VQ_REQUIRE(n < (1ll << 31), "%s: unaligned ROWBLOCK tensors must be below 2^31 elements", name);
    p.vec_ok = aligned ? 1 : 0;

    // The vector path indexes with 32 bits: split big tensors into row-aligned pieces.
    const int64_t max_piece = 1ll << 30;
    int64_t piece_rows = rows, piece_elems = n;
    if (p.vec_ok && n > max_piece) {
        if (p.smode == VQ_SCALE_ROWBLOCK) {
            piece_rows = max_piece / K; if (piece_rows < 1) piece_rows = 1;
            piece_elems = piece_rows * K;
            VQ_REQUIRE((piece_elems * esz) % 16 == 0 && (code_bits != 4 || piece_elems % 2 == 0),
                       "%s: cannot split this tensor into aligned pieces", name);
        } else {
            piece_elems = max_piece;
        }
    }
    cudaStream_t st = (cudaStream_t)stream;
    for (int64_t off = 0; off < n; off += piece_elems) {
        int64_t cnt = (n - off < piece_elems) ? n - off : piece_elems;
        EwParams q = p;
        q.n = cnt;
        q.in = (const char*)in + off * esz;
        q.out = out ? (char*)out + off * esz : nullptr;
        q.codes = codes ? codes + (code_bits == 4 ? off / 2 : off) : nullptr;
        if (p.smode == VQ_SCALE_ROWBLOCK && p.vec_ok) {
            int64_t soff = (off / K) * p.nb;
            q.scale = (const char*)scale + soff * esz;
            q.zp = zp ? (const char*)zp + soff * esz : nullptr;
        }
        int rc = (dtype == VQ_F32) ? launch_ew<float, OP>(q, st) : launch_ew<bf16_t, OP>(q, st);
        if (rc) return rc;
        if (!p.vec_ok) break;  // scalar path covers everything with 64-bit indices
    }
    return 0;
}

}  // namespace

extern "C" {

int vq_lut_map(const void* in, int dtype, int64_t n, const vq_table* table, void* out, void* stream) {
    return run_ew<OP_MAP>(in, dtype, n, nullptr, nullptr, nullptr, table, nullptr, out, nullptr, 0, stream);
}

int vq_quantize(const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                const vq_scale_layout* layout, const vq_table* table, void* out, uint8_t* out_codes, int code_bits,
                void* stream) {
    return run_ew<OP_QUANT>(in, dtype, n, scale, zero_point, layout, table, nullptr, out, out_codes, code_bits, stream);
}

int vq_fake_quantize(const void* in, int dtype, int64_t n, const void* scale, const vq_scale_layout* layout,
                     const vq_table* table, void* out, void* stream) {
    return run_ew<OP_FAKEQ>(in, dtype, n, scale, nullptr, layout, table, nullptr, out, nullptr, 0, stream);
}

int vq_dequantize(const void* in, int dtype, int64_t n, const void* scale, const void* zero_point,
                  const vq_scale_layout* layout, const vq_table* in_table, const vq_table* out_table, void* out,
                  void* stream) {
    return run_ew<OP_DEQUANT>(in, dtype, n, scale, zero_point, layout, in_table, out_table, out, nullptr, 0, stream);
}

}  // extern "C"
