// Per-channel quantize / fake-quantize over MANY tensors in one launch.
//
// Each tensor is [channels, length] (a conv weight OIHW viewed as [O, I*H*W]).  Pass 1 reduces |x|
// per channel (bit patterns, so NaN wins as in torch.amax), the scale is
// amax / quant_max in the tensor dtype, 1 where amax is 0, NaN or Inf -- what a settled
// FusedAmaxObsFakeQuantize observer hands to `quantize` for a static weight
// (quantization/fake_quantize.py:320-333) -- or a caller-supplied scale; pass 2 re-reads the data
// (L2 resident: a batch is 128 KB) and writes any of: the quantized values
// qmap[bf16(x / scale)] (`quantize`, ops/quantized.py:131-172), packed 8-bit codes, and
// values * scale (`dequantize`, ops/quantized.py:182-227).  Upstream runs amax, divide, expand,
// quantize and dequantize as separate full passes per tensor.
// HBM bound: sizeof(T) read per element + the requested outputs.
#include "vq_mx_body.cuh"
#include "vq_mx_fast.cuh"
#include "vq_divide.cuh"

namespace {


template <typename T>
__device__ __forceinline__ float elem_f32(const T* p, int64_t i);
template <>
__device__ __forceinline__ float elem_f32<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float elem_f32<bf16_t>(const bf16_t* p, int64_t i) { return bf16_bits_to_f32(p[i].bits); }

// four consecutive elements as fp32
template <typename T>
__device__ __forceinline__ void load4(const T* p, float* v, bool streaming);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* v, bool streaming) {
    const float4 a = streaming ? __ldcs(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
__device__ __forceinline__ void load4<bf16_t>(const bf16_t* p, float* v, bool streaming) {
    const uint2 a = streaming ? __ldcs(reinterpret_cast<const uint2*>(p)) : *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
    v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float* v);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float* v) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
}
template <>
__device__ __forceinline__ void store4<bf16_t>(bf16_t* p, const float* v) {
    // the values are bf16-representable already: keep the upper halves
    __stcs(reinterpret_cast<uint2*>(p), make_uint2((__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xFFFF0000u),
                                                   (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xFFFF0000u)));
}

// MODE 1/2: LUT16 table whose NaN patterns all map to one output: hardware bf16 conversion and plain
// table reads (2: tables staged in shared memory).  MODE 0: the generic lookup (INT arithmetic, run
// search, any LUT).
template <typename T, int MODE>
__device__ __forceinline__ void quantize_one(const TableDev& tab, const TableRes& res, float x, const DivPlan& dv,
                                             bool want_val, bool want_code, float& val, uint32_t& code) {
    const float q = divide(dv, x);
    if (MODE != 0) {
        const uint32_t pat = bf16_pattern(q);           // rounds fp32 -> bf16; NaN -> 0x7FFF
        if (want_val) val = __uint_as_float(ld_u16<MODE == 2>(res.lut, pat) << 16);
        if (want_code) code = ld_u8<MODE == 2>(tab.lut8, pat);
    } else {
        const Looked lk = table_lookup(tab, res, f32_to_bf16_bits(q), want_val, want_code);
        val = lk.val;
        code = lk.code;
    }
}

// One CTA per BATCH: a run of consecutive channels of one tensor, about kBatchElems elements, which
// lie contiguously in memory.  Phase 1: all warps sweep the batch as a flat array and reduce |x|
// per channel (shared-memory atomics on bit patterns: finite < inf < NaN, as torch.amax orders
// them).  One thread per channel turns the maximum into the scale and the division plan.  Phase 2:
// the same sweep again (the batch is L2 resident by then) quantizes and writes.  The work of a
// batch is spread over the whole CTA whatever the channel length is.
struct ChanBatch {
    int item, c0, nc;
    FastDiv len;            // flat index -> channel
    int pad[2];
};
constexpr int kBatchElems = 16384;
constexpr int kGroupThreads = 256;
constexpr int kBatchMaxChannels = 256;

struct BatchParams {
    const vq_channel_item* items;     // device
    const ChanBatch* batches;         // device
    int n_batches;
    float qmax;
    MxParams common;                  // table + shared-memory staging flags only
    int table_bytes;                  // shared memory taken by the staged tables
};

struct ChanShared {
    uint32_t amax[kBatchMaxChannels];
    uint32_t minnz[kBatchMaxChannels];      // smallest non-zero |x| bit pattern minus one
    int slow;                               // some channel of the batch needs the checked division
    float s[kBatchMaxChannels];
    float y[kBatchMaxChannels];
    int kind[kBatchMaxChannels];
};

template <typename T, int MODE>
__global__ void __launch_bounds__(1024) channel_quant_kernel(const BatchParams p) {
    extern __shared__ uint4 smem[];
    TableDev tab;
    TableRes res;
    stage_mx(p.common, smem, tab, res);
    // The CTA works as independent groups of kGroupThreads threads that share the staged tables: each
    // group walks its own batches with its own named barrier, so that the phases of different
    // batches overlap on the SM (one group waits for memory while another computes).
    const int group = threadIdx.x / kGroupThreads, tid = threadIdx.x % kGroupThreads;
    const int n_groups = blockDim.x / kGroupThreads;
    ChanShared& sh = reinterpret_cast<ChanShared*>(reinterpret_cast<uint8_t*>(smem) + p.table_bytes)[group];
    const int lane = threadIdx.x & 31;
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(kGroupThreads) : "memory"); };
    for (int b = blockIdx.x * n_groups + group; b < p.n_batches; b += gridDim.x * n_groups) {
        const ChanBatch bt = p.batches[b];
        const vq_channel_item it = p.items[bt.item];
        const uint32_t L = (uint32_t)it.length;
        const uint32_t n = (uint32_t)bt.nc * L;
        const int64_t off = (int64_t)bt.c0 * L;
        const T* x = reinterpret_cast<const T*>(it.input) + off;
        const bool vec = (L & 3) == 0 && ((uintptr_t)it.input & 15) == 0 &&
                         ((uintptr_t)it.values & 15) == 0 && ((uintptr_t)it.dequant & 15) == 0 && ((uintptr_t)it.codes & 3) == 0;
        const uint32_t step = vec ? 4u : 1u;
        const bool need_amax = !it.scale_in || it.amax_out;
        for (int i = tid; i < bt.nc; i += kGroupThreads) {
            sh.amax[i] = 0u;
            sh.minnz[i] = 0xFFFFFFFFu;
        }
        if (tid == 0) sh.slow = need_amax ? 0 : 1;
        group_sync();
        if (need_amax) {
            // phase 1
            constexpr int U1 = 4;                      // loads in flight per thread
            for (uint32_t e0 = tid * step; e0 < n; e0 += kGroupThreads * step * U1) {
                float v[U1][4];
#pragma unroll
                for (int u = 0; u < U1; ++u) {
                    const uint32_t e = e0 + u * kGroupThreads * step;
                    if (e < n) {
                        if (vec) load4<T>(x + e, v[u], false);
                        else v[u][0] = elem_f32<T>(x, e);
                    }
                }
#pragma unroll
                for (int u = 0; u < U1; ++u) {
                    const uint32_t e = e0 + u * kGroupThreads * step;
                    if (e >= n) break;
                    uint32_t m = abs_bits(v[u][0]);
                    uint32_t mn = m - 1u;                      // a zero wraps to the top and drops out
                    if (vec) {
#pragma unroll
                        for (int j = 1; j < 4; ++j) {
                            const uint32_t a = abs_bits(v[u][j]);
                            m = max(m, a);
                            mn = min(mn, a - 1u);
                        }
                    }
                    const uint32_t ch = fd_div(e, bt.len);
                    // the lanes of a warp usually sit in one channel: one atomic for all of them
                    const uint32_t act = __activemask();
                    if (act == 0xFFFFFFFFu && __reduce_min_sync(act, ch) == __reduce_max_sync(act, ch)) {
                        m = __reduce_max_sync(act, m);
                        mn = __reduce_min_sync(act, mn);
                        if (lane == 0) {
                            atomicMax(&sh.amax[ch], m);
                            atomicMin(&sh.minnz[ch], mn);
                        }
                    } else {
                        atomicMax(&sh.amax[ch], m);
                        atomicMin(&sh.minnz[ch], mn);
                    }
                }
            }
            group_sync();
        }
        for (int i = tid; i < bt.nc; i += kGroupThreads) {
            const int64_t c = bt.c0 + i;
            float sc;
            if (need_amax) {
                const uint32_t m = sh.amax[i];
                const float amax = __uint_as_float(m);
                sc = (m != 0u && m < 0x7F800000u) ? Arith<T>::rnd(__fdiv_rn(amax, p.qmax)) : 1.0f;
                if (it.amax_out) store_one<T>(reinterpret_cast<T*>(it.amax_out) + c, amax);
                if (it.scale_out && !it.scale_in) store_one<T>(reinterpret_cast<T*>(it.scale_out) + c, sc);
            }
            if (it.scale_in) sc = elem_f32<T>(reinterpret_cast<const T*>(it.scale_in), c);
            const DivPlan d = plan_division(sc);
            // the corrected reciprocal needs no per-element check when the whole channel lies in
            // 2^-100 <= |x| < 2^61 (zeros aside) and 2^-30 <= scale <= 2^30
            const uint32_t sb = __float_as_uint(sc), ex = (sb >> 23) & 0xFFu;
            const bool in_range = d.kind != 0 && (sb >> 31) == 0u && ex >= 97u && ex <= 157u && need_amax &&
                                  sh.amax[i] < 0x5E000000u && sh.minnz[i] >= 0x0D800000u - 1u;
            if (!in_range) sh.slow = 1;
            sh.s[i] = sc;
            sh.y[i] = d.y;
            sh.kind[i] = d.kind;
        }
        group_sync();
        const bool want_val = it.values != nullptr || it.dequant != nullptr;
        const bool want_code = it.codes != nullptr;
        if (want_val || want_code) {
            // phase 2
            T* values = reinterpret_cast<T*>(it.values) + (it.values ? off : 0);
            T* dequant = reinterpret_cast<T*>(it.dequant) + (it.dequant ? off : 0);
            uint8_t* codes = it.codes + (it.codes ? off : 0);
            const bool fast = MODE != 0 && vec && sh.slow == 0;
            if (fast) {
                // every channel of the batch is in range: x / s = fma(r, y, q0) with q0 = x y and
                // r = fma(-s, q0, x); the sign of x is put back so that -0 stays -0
                for (uint32_t e0 = tid * 4; e0 < n; e0 += kGroupThreads * 8) {
                    float v[2][4];
                    const uint32_t e1 = e0 + kGroupThreads * 4;
                    load4<T>(x + e0, v[0], true);
                    if (e1 < n) load4<T>(x + e1, v[1], true);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const uint32_t e = u ? e1 : e0;
                        if (e >= n) break;
                        const uint32_t ch = fd_div(e, bt.len);
                        const float sc = sh.s[ch], y = sh.y[ch];
                        float q[4], d[4];
                        uint32_t packed = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float xv = v[u][j];
                            const float q0 = __fmul_rn(xv, y);
                            const float qq = __fmaf_rn(__fmaf_rn(-sc, q0, xv), y, q0);
                            const uint32_t pat = bf16_pattern(
                                __uint_as_float((__float_as_uint(qq) & 0x7FFFFFFFu) | (__float_as_uint(xv) & 0x80000000u)));
                            q[j] = want_val ? __uint_as_float(ld_u16<MODE == 2>(res.lut, pat) << 16) : 0.0f;
                            if (want_code) packed |= ld_u8<MODE == 2>(tab.lut8, pat) << (8 * j);
                            d[j] = Arith<T>::rnd(__fmul_rn(q[j], sc));
                        }
                        if (it.values) store4<T>(values + e, q);
                        if (it.dequant) store4<T>(dequant + e, d);
                        if (want_code) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                    }
                }
            } else
            for (uint32_t e0 = tid * step; e0 < n; e0 += kGroupThreads * step * 2) {
                float v[2][4];
                const uint32_t e1 = e0 + kGroupThreads * step;
                if (vec) {
                    load4<T>(x + e0, v[0], true);
                    if (e1 < n) load4<T>(x + e1, v[1], true);
                } else {
                    v[0][0] = elem_f32<T>(x, e0);
                    if (e1 < n) v[1][0] = elem_f32<T>(x, e1);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t e = u ? e1 : e0;
                    if (e >= n) break;
                    const uint32_t ch = fd_div(e, bt.len);
                    DivPlan dv;
                    dv.s = sh.s[ch];
                    dv.y = sh.y[ch];
                    dv.kind = sh.kind[ch];
                    if (vec) {
                        float q[4], d[4];
                        uint32_t packed = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t code = 0;
                            q[j] = 0.0f;
                            quantize_one<T, MODE>(tab, res, v[u][j], dv, want_val, want_code, q[j], code);
                            packed |= code << (8 * j);
                            d[j] = Arith<T>::rnd(__fmul_rn(q[j], dv.s));
                        }
                        if (it.values) store4<T>(values + e, q);
                        if (it.dequant) store4<T>(dequant + e, d);
                        if (want_code) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                    } else {
                        float q = 0.0f;
                        uint32_t code = 0;
                        quantize_one<T, MODE>(tab, res, v[u][0], dv, want_val, want_code, q, code);
                        if (it.values) store_one<T>(values + e, q);
                        if (it.dequant) store_one<T>(dequant + e, Arith<T>::rnd(__fmul_rn(q, dv.s)));
                        if (want_code) codes[e] = (uint8_t)code;
                    }
                }
            }
        }
        group_sync();
    }
}

// batches of one item
inline int64_t batches_of(const vq_channel_item& it) {
    if (it.channels <= 0) return 0;
    int64_t per = kBatchElems / it.length;
    per = per < 1 ? 1 : (per > kBatchMaxChannels ? kBatchMaxChannels : per);
    return (it.channels + per - 1) / per;
}

}  // namespace

extern "C" {

size_t vq_channel_quantize_multi_workspace(const vq_channel_item* items, int n_items) {
    if (n_items < 0 || !items) return 0;
    int64_t nb = 0;
    for (int i = 0; i < n_items; ++i) nb += (items[i].length >= 1) ? batches_of(items[i]) : 0;
    return (size_t)n_items * sizeof(vq_channel_item) + (size_t)nb * sizeof(ChanBatch) + 64;
}

int vq_channel_quantize_multi(const vq_channel_item* items, int n_items, int dtype, double quant_max, const vq_table* table,
                              void* workspace, size_t workspace_bytes, void* stream) {
    const char* name = "vq_channel_quantize_multi";
    VQ_REQUIRE(n_items >= 0, "%s: negative item count", name);
    if (n_items == 0) return 0;
    VQ_REQUIRE(items != nullptr, "%s: null item array", name);
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(quant_max > 0.0, "%s: quant_max must be positive", name);
    bool any_table_out = false, any_codes = false;
    int64_t total = 0, n_batches = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_channel_item& it = items[i];
        const bool ok = it.input && it.channels >= 0 && it.channels < (1ll << 31) && it.length >= 1 &&
                        it.length < (1ll << 22) && (it.amax_out || it.scale_out || it.values || it.codes || it.dequant);
        VQ_REQUIRE(ok, "%s: item %d needs an input, a channel length in [1, 2^22) and at least one output", name, i);
        any_table_out |= it.values || it.codes || it.dequant;
        any_codes |= it.codes != nullptr;
        total += it.channels * it.length;
        n_batches += batches_of(it);
    }
    VQ_REQUIRE(!any_table_out || (table && table->kind != VQ_TABLE_NONE), "%s: quantized outputs need a table", name);
    if (any_codes) {
        const bool have = table->kind == VQ_TABLE_INT || table->lut8 || (table->kind == VQ_TABLE_RUNS && table->run_codes);
        VQ_REQUIRE(have, "%s: packed codes need a code table", name);
    }
    VQ_REQUIRE(n_batches < (1ll << 31), "%s: too many channels", name);
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 16 == 0 && workspace_bytes >= vq_channel_quantize_multi_workspace(items, n_items),
               "%s: workspace missing, unaligned or smaller than vq_channel_quantize_multi_workspace(items, n_items)", name);
    if (n_batches == 0) return 0;

    const size_t items_bytes = ((size_t)n_items * sizeof(vq_channel_item) + 31) / 32 * 32;
    ChanBatch* hb = new ChanBatch[(size_t)n_batches];
    int64_t k = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_channel_item& it = items[i];
        if (it.channels <= 0) continue;
        int64_t per = kBatchElems / it.length;
        per = per < 1 ? 1 : (per > kBatchMaxChannels ? kBatchMaxChannels : per);
        const FastDiv fdv = make_fastdiv((uint32_t)it.length);
        for (int64_t c0 = 0; c0 < it.channels; c0 += per, ++k) {
            hb[k].item = i;
            hb[k].c0 = (int)c0;
            hb[k].nc = (int)(it.channels - c0 < per ? it.channels - c0 : per);
            hb[k].len = fdv;
            hb[k].pad[0] = hb[k].pad[1] = 0;
        }
    }
    BatchParams p{};
    p.items = reinterpret_cast<const vq_channel_item*>(workspace);
    p.batches = reinterpret_cast<const ChanBatch*>((char*)workspace + items_bytes);
    p.n_batches = (int)n_batches;
    p.qmax = (float)quant_max;
    p.common.tab = to_dev(table);
    const bool lut = table && table->kind == VQ_TABLE_LUT16;
    const bool big = total >= (1 << 21);
    p.common.smem_lut16 = (big && lut) ? 1 : 0;
    p.common.smem_lut8 = (big && lut && any_codes && table->lut8) ? 1 : 0;
    p.table_bytes = (p.common.smem_lut16 ? 131072 : 0) + (p.common.smem_lut8 ? 65536 : 0) +
                    ((table && table->kind == VQ_TABLE_RUNS) ? ((5 * VQ_MAX_RUNS + 15) / 16 * 16) : 0);
    const size_t smem = (size_t)p.table_bytes + 4 * sizeof(ChanShared);
    const bool direct = lut && table->nan_uniform && (!any_codes || table->lut8);
    const bool staged = direct && p.common.smem_lut16 && (!any_codes || p.common.smem_lut8);
    const int mode = staged ? 2 : (direct ? 1 : 0);

    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e1 = cudaMemcpyAsync(workspace, items, (size_t)n_items * sizeof(vq_channel_item), cudaMemcpyHostToDevice, st);
    cudaError_t e2 = cudaMemcpyAsync((char*)workspace + items_bytes, hb, (size_t)n_batches * sizeof(ChanBatch),
                                     cudaMemcpyHostToDevice, st);
    delete[] hb;   // pageable copies are staged before cudaMemcpyAsync returns
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return vq_set_error(VQ_ERR_CUDA, "%s: descriptor upload failed: %s", name, cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));

    const int sms = vq_sm_count();
    // tables in shared memory leave room for one CTA per SM: make it a full one
    const int threads = smem > 100 * 1024 ? 1024 : 512;
    const int per_sm = smem > 100 * 1024 ? 1 : 2;
    const int64_t want = (n_batches * kGroupThreads + threads - 1) / threads;
    const int blocks = (int)(want < (int64_t)sms * per_sm ? want : (int64_t)sms * per_sm);
#define VQ_CH_LAUNCH(T, D)                                                                                            \
    do {                                                                                                              \
        auto kern = channel_quant_kernel<T, D>;                                                                       \
        if (smem > 48 * 1024) VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<blocks, threads, smem, st>>>(p);                                                                       \
    } while (0)
    if (dtype == VQ_F32) {
        if (mode == 2) VQ_CH_LAUNCH(float, 2); else if (mode == 1) VQ_CH_LAUNCH(float, 1); else VQ_CH_LAUNCH(float, 0);
    } else {
        if (mode == 2) VQ_CH_LAUNCH(bf16_t, 2); else if (mode == 1) VQ_CH_LAUNCH(bf16_t, 1); else VQ_CH_LAUNCH(bf16_t, 0);
    }
#undef VQ_CH_LAUNCH
    VQ_LAUNCH_CHECK("channel_quant_kernel");
    return 0;
}

}  // extern "C"
