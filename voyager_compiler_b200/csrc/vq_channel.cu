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
#include <algorithm>
#include <type_traits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "vq_mx_body.cuh"
#include "vq_mx_fast.cuh"
#include "vq_divide.cuh"
#include "vq_tc.cuh"

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
    int vec;                // pipelined kernel: the batch starts and ends on 16-byte boundaries of aligned tensors
    int fast;               // pipelined kernel: vec, and the channel length is a multiple of 128 elements
};
constexpr int kBatchElems = 16384;
constexpr int kGroupThreads = 256;
constexpr int kBatchMaxChannels = 256;

struct BatchParams {
    const vq_channel_item* items;     // device
    const ChanBatch* batches;         // device
    int n_batches;
    float qmax;
    float inv_qmax;                   // 1 / qmax when that is exact (qmax a power of two), else 0
    MxParams common;                  // table + shared-memory staging flags only
    int table_bytes;                  // shared memory taken by the staged tables
    long long wait_budget;            // pipelined kernel: clock cycles a wait may take before it gives up
    int skip_batch;                   // pipelined kernel, tests only: the producer leaves this batch out (-1: none)
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

// ---------------------------------------------------------------------------------------------
constexpr int kSmemItems = 96;         // tensor descriptors a CTA of the pipelined kernel keeps in shared memory
constexpr int kSmemBatches = 64;       // batch descriptors it keeps there

// 16 bytes of a batch held in registers between the |x| reduction and the quantization
template <typename T>
struct RawVec;
template <>
struct RawVec<float> {
    float4 r;
    __device__ __forceinline__ void load(const float* p) { r = __ldcs(reinterpret_cast<const float4*>(p)); }
    __device__ __forceinline__ void load_shared(const float* p) { r = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void zero() { r = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void get(float* v) const { v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
    __device__ __forceinline__ void set(int k, float f) { (&r.x)[k] = f; }
};
template <>
struct RawVec<bf16_t> {
    uint2 r;
    __device__ __forceinline__ void load(const bf16_t* p) { r = __ldcs(reinterpret_cast<const uint2*>(p)); }
    __device__ __forceinline__ void load_shared(const bf16_t* p) { r = *reinterpret_cast<const uint2*>(p); }
    __device__ __forceinline__ void zero() { r = make_uint2(0u, 0u); }
    __device__ __forceinline__ void get(float* v) const {
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
    }
    __device__ __forceinline__ void set(int k, float f) {
        uint32_t& w = (k < 2) ? r.x : r.y;
        const uint32_t h = __float_as_uint(f) >> 16;
        w = (k & 1) ? ((w & 0x0000FFFFu) | (h << 16)) : ((w & 0xFFFF0000u) | h);
    }
};

// ---------------------------------------------------------------------------------------------
// Pipelined variant: batches arrive in shared memory by asynchronous bulk copies.
//
// Warp 0 is the producer: one thread walks this CTA's batches and, for each, waits for a free
// stage of a PIPE_STAGES-deep ring and issues ONE cp.async.bulk of the whole batch (up to 28 KB)
// whose completion is counted on the stage's mbarrier.  PIPE_GROUPS consumer groups of PIPE_GT threads
// take the batches in turn: wait for the stage, read it into registers (8 x 16 bytes per thread),
// release the stage at once, reduce |x| per channel, derive the scales, quantize from registers
// and store.  Global loads therefore never stall a compute warp and up to PIPE_STAGES batches
// per SM are in flight whatever the consumers are doing.
//
// The table costs 64 KB + 2 KB of shared memory instead of 192 KB: the packed code comes from the
// code table, the value from `levels2[code + 256 * sign of the input]` (see vq_table), which the
// host only provides when that is the same function as the full value table.  INT tables use
// arithmetic and no table at all.  Batches that bulk copies cannot take (channel length not a
// multiple of 4 elements / 16 bytes, unaligned tensors) are read by the consumers themselves.
// Every wait is bounded; a wait that runs out sets g_channel_status and winds the CTA down.
constexpr int PIPE_GROUPS = 4;
constexpr int PIPE_GT = 192;                                   // threads per consumer group: 4 x 6 + 1 warps leave 80 registers per thread
constexpr int PIPE_STAGES = 4;                                 // a multiple of PIPE_GROUPS: see below
constexpr int PIPE_VECS = 8;                                   // 16-byte vectors per consumer thread
constexpr int PIPE_BATCH = PIPE_GT * PIPE_VECS * 4;            // 6144 elements
constexpr int PIPE_THREADS = 32 + PIPE_GROUPS * PIPE_GT;
constexpr long long PIPE_WAIT = 4000000000ll;                  // ~2 s of SM clocks
// Batch i of a CTA uses stage i % PIPE_STAGES and consumer group i % PIPE_GROUPS.  With the stage count a
// multiple of the group count a stage always belongs to the same group, so that group sees every phase of
// the stage's barriers in order; a parity wait is only meaningful for a waiter that has seen the phase before
// (a group meeting a stage for the first time in its SECOND use would find "parity 1 not pending" and read
// the stage before the first copy into it has landed).
static_assert(PIPE_STAGES % PIPE_GROUPS == 0, "every stage must belong to one consumer group");

__device__ int g_channel_status = 0;

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// value and code of the bf16 pattern `pat` of a quotient: from the code table and the level table in shared
// memory (TK_LUT), or by rounding and clamping (TK_INT)
template <int TK>
__device__ __forceinline__ void pipe_lookup(const uint8_t* s_codes, const float* s_lv2, float lo, float hi, uint32_t pat,
                                            float& val, uint32_t& code) {
    if (TK == TK_LUT) {
        code = s_codes[pat];
        val = s_lv2[code + ((pat >> 15) << 8)];
    } else {
        const float vb = __uint_as_float(pat << 16);
        float q = rintf(vb);
        if (lo == 0.0f) {
            q = (q < lo) ? lo : q;
            q = (q > hi) ? hi : q;
        } else {
            q = fminf(fmaxf(q, lo), hi);
        }
        val = (vb != vb) ? vb : q;
        code = (vb != vb) ? 0u : ((uint32_t)(int)q & 0xFFu);
    }
}
// F(integral constant j) for j = CNT - 1 down to 0, CNT <= PIPE_VECS known at run time: one jump, then straight-line code
#define VQ_PIECES_DOWN(CNT, F)                                   \
    switch (CNT) {                                               \
        case 8: F(std::integral_constant<int, 7>{}); [[fallthrough]]; \
        case 7: F(std::integral_constant<int, 6>{}); [[fallthrough]]; \
        case 6: F(std::integral_constant<int, 5>{}); [[fallthrough]]; \
        case 5: F(std::integral_constant<int, 4>{}); [[fallthrough]]; \
        case 4: F(std::integral_constant<int, 3>{}); [[fallthrough]]; \
        case 3: F(std::integral_constant<int, 2>{}); [[fallthrough]]; \
        case 2: F(std::integral_constant<int, 1>{}); [[fallthrough]]; \
        case 1: F(std::integral_constant<int, 0>{}); [[fallthrough]]; \
        default: break;                                          \
    }
static_assert(PIPE_VECS == 8, "VQ_PIECES_DOWN lists eight pieces");

struct PipeShared {
    ChanShared ch[PIPE_GROUPS][2];
    int ok[PIPE_GROUPS];
    int tables_ok[PIPE_GROUPS];
};

template <typename T, int TK>
__global__ void __launch_bounds__(PIPE_THREADS, 1) channel_pipe_kernel(const BatchParams p, const int n_items) {
    extern __shared__ uint4 smem[];
    // layout: [code table 64 KB (TK_LUT)] [levels2 2 KB (TK_LUT)] [ring] [PipeShared] [items] [barriers]
    constexpr uint32_t TAB_BYTES = TK == TK_LUT ? 65536u + 2048u : 0u;
    constexpr uint32_t STAGE_BYTES = PIPE_BATCH * sizeof(T);
    uint8_t* base = reinterpret_cast<uint8_t*>(smem);
    const uint8_t* s_codes = base;
    const float* s_lv2 = reinterpret_cast<const float*>(base + 65536);
    uint8_t* ring = base + TAB_BYTES;
    PipeShared& ps = *reinterpret_cast<PipeShared*>(ring + PIPE_STAGES * STAGE_BYTES);
    vq_channel_item* sitems = reinterpret_cast<vq_channel_item*>(reinterpret_cast<uint8_t*>(&ps) + ((sizeof(PipeShared) + 15) / 16) * 16);
    ChanBatch* sbatches = reinterpret_cast<ChanBatch*>(sitems + kSmemItems);       // this CTA's first kSmemBatches batches
    const uint32_t bar0 = tc::smem_u32(sbatches + kSmemBatches);
    const uint32_t FULL0 = bar0, EMPTY0 = bar0 + 8u * PIPE_STAGES;
    // Prologue: barriers first, then the tables are fetched by two bulk copies (no thread waits for
    // them until its first lookup) while all threads gather the descriptors; the producer starts
    // loading batches as soon as the descriptors are in place.
    const uint32_t TABLE_BAR = EMPTY0 + 8u * PIPE_STAGES;
    if (threadIdx.x == 0) {
        for (int s = 0; s < PIPE_STAGES; ++s) {
            tc::mbar_init(FULL0 + 8u * s, 1);
            tc::mbar_init(EMPTY0 + 8u * s, PIPE_GT / 32);     // one arrival per consumer warp of the owning group
        }
        tc::mbar_init(TABLE_BAR, 1);
        tc::fence_barrier_init();
        if (TK == TK_LUT) {
            tc::mbar_expect_tx(TABLE_BAR, 65536u + 2048u);
            bulk_load(tc::smem_u32(base), p.common.tab.lut8, 65536u, TABLE_BAR);
            bulk_load(tc::smem_u32(base + 65536), p.common.tab.levels2, 2048u, TABLE_BAR);
        }
    }
    const bool items_staged = n_items <= kSmemItems;
    if (items_staged) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.items);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sitems);
        for (int i = threadIdx.x; i < n_items * (int)(sizeof(vq_channel_item) / 4); i += blockDim.x) dst[i] = src[i];
    }
    {
        // descriptors of the batches this CTA will walk (batch blockIdx.x + i * gridDim.x at slot i)
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.batches);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sbatches);
        constexpr int W = sizeof(ChanBatch) / 4;
        for (int t = threadIdx.x; t < kSmemBatches * W; t += blockDim.x) {
            const int64_t b = blockIdx.x + (int64_t)(t / W) * gridDim.x;
            if (b < p.n_batches) dst[t] = __ldg(src + b * W + t % W);
        }
    }
    __syncthreads();
    const float lo = p.common.tab.lo, hi = p.common.tab.hi;

    if (threadIdx.x < 32) {
        // ------------------------------------------------------------------ producer
        if (threadIdx.x == 0) {
            bool ok = true;
            // Every consumer group has its own sequence of batches (group g: this CTA's batches g, g + G, ...) and
            // its own stage.  The producer serves whichever group has given its stage back, not the groups in turn:
            // a group that is ahead of the others gets its next batch at once.
            int k[PIPE_GROUPS];                               // batches of group g loaded so far
            int left = 0;
#pragma unroll
            for (int g = 0; g < PIPE_GROUPS; ++g) k[g] = 0;
            for (int b = blockIdx.x; b < p.n_batches; b += gridDim.x) ++left;
            long long idle_since = clock64();
            while (left > 0 && ok) {
                bool progress = false;
#pragma unroll
                for (int g = 0; g < PIPE_GROUPS; ++g) {
                    const int i = g + k[g] * PIPE_GROUPS;
                    const int64_t b = blockIdx.x + (int64_t)i * gridDim.x;
                    if (b >= p.n_batches) continue;
                    const int s = i % PIPE_STAGES;
                    const uint32_t ph = (uint32_t)(i / PIPE_STAGES) & 1u;
                    if (i >= PIPE_STAGES && !tc::mbar_try_wait(EMPTY0 + 8u * s, ph ^ 1u)) continue;
                    ++k[g];
                    --left;
                    progress = true;
                    if (b == p.skip_batch) continue;          // test hook: this batch's consumers will see their wait run out
                    const ChanBatch& bt = *(i < kSmemBatches ? static_cast<const ChanBatch*>(sbatches + i) : p.batches + b);
                    const vq_channel_item& it = *(items_staged ? static_cast<const vq_channel_item*>(sitems + bt.item) : p.items + bt.item);
                    const uint32_t L = (uint32_t)it.length;
                    if (bt.vec) {
                        const uint32_t bytes = (uint32_t)bt.nc * L * (uint32_t)sizeof(T);
                        tc::mbar_expect_tx(FULL0 + 8u * s, bytes);
                        bulk_load(tc::smem_u32(ring + s * STAGE_BYTES), reinterpret_cast<const T*>(it.input) + (int64_t)bt.c0 * L,
                                  bytes, FULL0 + 8u * s);
                    } else {
                        tc::mbar_arrive(FULL0 + 8u * s);      // the consumers read this batch themselves
                    }
                }
                if (progress) {
                    idle_since = clock64();
                } else {
                    if (clock64() - idle_since > p.wait_budget) ok = false;
                    __nanosleep(64);
                }
            }
            if (!ok) atomicCAS(&g_channel_status, 0, 21);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    constexpr int GT = PIPE_GT;
    constexpr int GW = GT / 32;
    const int ct = threadIdx.x - 32;
    const int group = ct / GT, tid = ct % GT;
    const int lane = threadIdx.x & 31, warp = tid >> 5;
    const uint32_t warp_e0 = (uint32_t)(tid & ~31) * 4u;
    auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(GT) : "memory"); };
    bool tables_ready = TK != TK_LUT;
    int i = group;
    for (int b = blockIdx.x + group * gridDim.x; b < p.n_batches; b += PIPE_GROUPS * gridDim.x, i += PIPE_GROUPS) {
        const int s = i % PIPE_STAGES;
        const uint32_t ph = (uint32_t)(i / PIPE_STAGES) & 1u;
        // The per-channel scratch alternates between two copies: a thread may enter the next batch (and clear
        // that batch's copy) while slower threads of the group still read this batch's scales; the barriers
        // inside the next batch keep it from going two batches ahead.
        ChanShared& sh = ps.ch[group][(i / PIPE_GROUPS) & 1];
        // descriptors through one pointer each: a select between a shared-memory and a global copy would load both,
        // and the global load would sit at the head of every batch
        const ChanBatch& bt = *(i < kSmemBatches ? static_cast<const ChanBatch*>(sbatches + i) : p.batches + b);
        const vq_channel_item& it = *(items_staged ? static_cast<const vq_channel_item*>(sitems + bt.item) : p.items + bt.item);
        const uint32_t L = (uint32_t)it.length;
        const uint32_t n = (uint32_t)bt.nc * L;
        const int64_t off = (int64_t)bt.c0 * L;
        const T* x = reinterpret_cast<const T*>(it.input) + off;
        const bool vec = bt.vec != 0;
        const bool ragged = (L & 3u) != 0u;                  // a 4-element vector may straddle two channels
        const bool fast = bt.fast != 0;                      // vec and every 128-element run inside one channel
        const bool need_amax = !it.scale_in || it.amax_out;
        for (int c = tid; c < bt.nc; c += GT) {
            sh.amax[c] = 0u;
            sh.minnz[c] = 0xFFFFFFFFu;
        }
        if (tid == 0) {
            sh.slow = need_amax ? 0 : 1;
            ps.ok[group] = tc::mbar_wait_relaxed(FULL0 + 8u * s, ph, p.wait_budget) ? 1 : 0;
        }
        group_sync();
        if (!ps.ok[group]) {
            if (tid == 0) atomicCAS(&g_channel_status, 0, 22);
            break;
        }
        // every consumer warp gives the stage back once per batch (the barrier counts GW arrivals)
        auto release_stage = [&]() {
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(EMPTY0 + 8u * s);
        };
        // Three ways through a batch:
        //   fast     channel length a multiple of 128 elements: every warp takes one contiguous run of the batch in
        //            128-element pieces, each inside one channel, so the channel bookkeeping is one comparison per piece;
        //   in_regs  channel length a multiple of 4: registers too, pieces strided over the group, the channel of a
        //            piece found by division and pieces that straddle channels reduced element-wise;
        //   rolled   anything else (a vector may straddle two channels, e.g. a 7x7x3 stem; unaligned tensors): the
        //            batch stays in the stage (or in global memory) and is walked element by element.
        // The first two copy the batch to registers and give the stage back at once.
        const bool in_regs = vec && !ragged && !fast;
        const T* st = reinterpret_cast<const T*>(ring + s * STAGE_BYTES);
        RawVec<T> raw[PIPE_VECS];
        // fast: this warp's run is pieces [qc, qc + cnt) of the batch
        const uint32_t pieces = n >> 7, per = (pieces + GW - 1) / GW, qc = (uint32_t)warp * per;
        const int cnt = (fast && qc < pieces) ? (int)min(per, pieces - qc) : 0;
        const uint32_t e_w = qc << 7;
        if (fast) {
#pragma unroll
            for (int j = 0; j < PIPE_VECS; ++j)
                if (j < cnt) raw[j].load_shared(st + e_w + (uint32_t)(j << 7) + (uint32_t)lane * 4u);
            release_stage();
        } else if (in_regs) {
#pragma unroll
            for (int j = 0; j < PIPE_VECS; ++j) {
                const uint32_t e = (uint32_t)(j * GT + tid) * 4u;
                if (e < n) raw[j].load_shared(st + e);
                else raw[j].zero();
            }
            release_stage();
        } else if (!vec) {
            release_stage();                                 // nothing was copied: the rolled loops read global memory
        }
        const T* xs = (vec && ragged) ? st : x;              // where the rolled loops read the batch

        if (need_amax && fast) {
            if (cnt > 0) {
                // last piece first: one jump into straight-line code instead of a test per piece
                uint32_t cur = fd_div(e_w + ((uint32_t)(cnt - 1) << 7), bt.len), floor_ = cur * L, m = 0u, mn = 0xFFFFFFFFu;
                auto flush = [&]() {
                    const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, m), wn = __reduce_min_sync(0xFFFFFFFFu, mn);
                    if (lane == 0) {
                        atomicMax(&sh.amax[cur], wm);
                        atomicMin(&sh.minnz[cur], wn);
                    }
                };
                auto piece = [&](auto jc) {
                    constexpr int j = decltype(jc)::value;
                    if (e_w + (uint32_t)(j << 7) < floor_) {  // warp uniform: the run has left the channel
                        flush();
                        --cur;
                        floor_ -= L;
                        m = 0u;
                        mn = 0xFFFFFFFFu;
                    }
                    float v[4];
                    raw[j].get(v);
                    const uint32_t a0 = abs_bits(v[0]), a1 = abs_bits(v[1]), a2 = abs_bits(v[2]), a3 = abs_bits(v[3]);
                    m = max(max(m, a0), max(a1, max(a2, a3)));
                    mn = min(min(mn, a0 - 1u), min(a1 - 1u, min(a2 - 1u, a3 - 1u)));   // a zero wraps to the top and drops out
                };
                VQ_PIECES_DOWN(cnt, piece);
                flush();
            }
        } else if (need_amax && in_regs) {
            uint32_t cur = 0xFFFFFFFFu, m = 0u, mn = 0xFFFFFFFFu;
            auto flush = [&]() {
                if (cur != 0xFFFFFFFFu) {
                    const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, m), wn = __reduce_min_sync(0xFFFFFFFFu, mn);
                    if (lane == 0) {
                        atomicMax(&sh.amax[cur], wm);
                        atomicMin(&sh.minnz[cur], wn);
                    }
                }
                cur = 0xFFFFFFFFu; m = 0u; mn = 0xFFFFFFFFu;
            };
#pragma unroll
            for (int j = 0; j < PIPE_VECS; ++j) {
                const uint32_t first = (uint32_t)(j * GT) * 4u + warp_e0;          // warp uniform
                if (first >= n) continue;
                float v[4];
                raw[j].get(v);
                const uint32_t e = (uint32_t)(j * GT + tid) * 4u;
                const uint32_t a0 = abs_bits(v[0]), a1 = abs_bits(v[1]), a2 = abs_bits(v[2]), a3 = abs_bits(v[3]);
                const uint32_t m4 = max(max(a0, a1), max(a2, a3));
                const uint32_t n4 = min(min(a0 - 1u, a1 - 1u), min(a2 - 1u, a3 - 1u));
                const uint32_t last = min(first + 127u, n - 1u);
                const uint32_t c_first = fd_div(first, bt.len), c_last = fd_div(last, bt.len);
                if (c_first == c_last) {
                    if (c_first != cur) {
                        flush();
                        cur = c_first;
                    }
                    if (e < n) {
                        m = max(m, m4);
                        mn = min(mn, n4);
                    }
                } else {
                    flush();
                    if (e < n) {
                        const uint32_t ch = fd_div(e, bt.len);
                        atomicMax(&sh.amax[ch], m4);
                        atomicMin(&sh.minnz[ch], n4);
                    }
                }
            }
            flush();
        } else if (need_amax) {
            // consecutive lanes take consecutive elements: a warp usually sits in one channel
            for (uint32_t e0 = (uint32_t)(tid & ~31); e0 < n; e0 += GT) {
                const uint32_t e = e0 + lane;
                uint32_t a = 0u, an = 0xFFFFFFFFu, ch = 0u;
                if (e < n) {
                    a = abs_bits(elem_f32<T>(xs, e));
                    an = a - 1u;
                    ch = fd_div(e, bt.len);
                }
                const uint32_t c_first = fd_div(e0, bt.len), c_last = fd_div(min(e0 + 31u, n - 1u), bt.len);
                if (c_first == c_last) {
                    const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, a), wn = __reduce_min_sync(0xFFFFFFFFu, an);
                    if (lane == 0) {
                        atomicMax(&sh.amax[c_first], wm);
                        atomicMin(&sh.minnz[c_first], wn);
                    }
                } else if (e < n) {
                    atomicMax(&sh.amax[ch], a);
                    atomicMin(&sh.minnz[ch], an);
                }
            }
        }
        if (need_amax) group_sync();
        const bool want_val = it.values != nullptr || it.dequant != nullptr;
        const bool want_code = it.codes != nullptr;
        T* values = reinterpret_cast<T*>(it.values) + (it.values ? off : 0);
        T* dequant = reinterpret_cast<T*>(it.dequant) + (it.dequant ? off : 0);
        uint8_t* codes = it.codes + (it.codes ? off : 0);
        const bool st_values = it.values != nullptr, st_dequant = it.dequant != nullptr;
        // value and code of the bf16 pattern `pat` of a quotient whose dividend was `xv`
        auto lookup = [&](uint32_t pat, float& val, uint32_t& code) { pipe_lookup<TK>(s_codes, s_lv2, lo, hi, pat, val, code); };
        // Four elements of one channel whose quotients are in the range of the corrected-reciprocal division
        // (q = x y, q += (x - s q) y: the correctly rounded x / s), two elements per packed fp32 instruction.
        auto quantize4 = [&](const float* v, float sc, float y, float* q, float* d, uint32_t& packed) {
            float t[4], r[4];
            t[0] = v[0]; t[1] = v[1]; t[2] = v[2]; t[3] = v[3];
            mul2(t[0], t[1], y);
            mul2(t[2], t[3], y);
            fma2(r[0], r[1], t[0], t[1], -sc, v[0], v[1]);
            fma2(r[2], r[3], t[2], t[3], -sc, v[2], v[3]);
            fma2(t[0], t[1], r[0], r[1], y, t[0], t[1]);
            fma2(t[2], t[3], r[2], r[3], y, t[2], t[3]);
            packed = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t pat = bf16_pattern(
                    __uint_as_float((__float_as_uint(t[k]) & 0x7FFFFFFFu) | (__float_as_uint(v[k]) & 0x80000000u)));
                uint32_t code;
                lookup(pat, q[k], code);
                packed |= code << (8 * k);
                d[k] = q[k];
            }
            mul2(d[0], d[1], sc);
            mul2(d[2], d[3], sc);
#pragma unroll
            for (int k = 0; k < 4; ++k) d[k] = Arith<T>::rnd(d[k]);
        };
        for (int c = tid; c < bt.nc; c += GT) {
            const int64_t cg = bt.c0 + c;
            float sc;
            if (need_amax) {
                const uint32_t mb = sh.amax[c];
                const float amax = __uint_as_float(mb);
                // amax / qmax; a multiplication gives the same correctly rounded number when qmax is a power of two
                const float ratio = p.inv_qmax != 0.0f ? __fmul_rn(amax, p.inv_qmax) : __fdiv_rn(amax, p.qmax);
                sc = (mb != 0u && mb < 0x7F800000u) ? Arith<T>::rnd(ratio) : 1.0f;
                if (it.amax_out) store_one<T>(reinterpret_cast<T*>(it.amax_out) + cg, amax);
                if (it.scale_out && !it.scale_in) store_one<T>(reinterpret_cast<T*>(it.scale_out) + cg, sc);
            }
            if (it.scale_in) sc = elem_f32<T>(reinterpret_cast<const T*>(it.scale_in), cg);
            const DivPlan d = plan_division(sc);
            const uint32_t sb = __float_as_uint(sc), ex = (sb >> 23) & 0xFFu;
            const bool in_range = d.kind != 0 && (sb >> 31) == 0u && ex >= 97u && ex <= 157u && need_amax &&
                                  sh.amax[c] < 0x5E000000u && sh.minnz[c] >= 0x0D800000u - 1u;
            if (!in_range) sh.slow = 1;
            sh.s[c] = sc;
            sh.y[c] = d.y;
            sh.kind[c] = d.kind;
        }
        // the tables are first needed here: their bulk copies had the first batch's reduction to land
        if (!tables_ready && tid == 0) ps.tables_ok[group] = tc::mbar_wait_relaxed(TABLE_BAR, 0u, p.wait_budget) ? 1 : 0;
        group_sync();
        if (!tables_ready && !ps.tables_ok[group]) {
            if (tid == 0) atomicCAS(&g_channel_status, 0, 23);
            break;
        }
        tables_ready = true;
        if (want_val || want_code) {
            if (fast && sh.slow == 0) {
                if (cnt > 0) {
                    uint32_t cur = fd_div(e_w + ((uint32_t)(cnt - 1) << 7), bt.len), floor_ = cur * L;
                    float sc = sh.s[cur], y = sh.y[cur];
                    auto piece = [&](auto jc) {
                        constexpr int j = decltype(jc)::value;
                        const uint32_t e0 = e_w + (uint32_t)(j << 7);
                        if (e0 < floor_) {                    // warp uniform
                            --cur;
                            floor_ -= L;
                            sc = sh.s[cur];
                            y = sh.y[cur];
                        }
                        const uint32_t e = e0 + (uint32_t)lane * 4u;
                        float v[4], q[4], d[4];
                        uint32_t packed;
                        raw[j].get(v);
                        quantize4(v, sc, y, q, d, packed);
                        if (st_values) store4<T>(values + e, q);
                        if (st_dequant) store4<T>(dequant + e, d);
                        if (want_code) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                    };
                    VQ_PIECES_DOWN(cnt, piece);
                }
            } else if (in_regs && sh.slow == 0) {
#pragma unroll
                for (int j = 0; j < PIPE_VECS; ++j) {
                    const uint32_t e = (uint32_t)(j * GT + tid) * 4u;
                    if (e >= n) continue;
                    const uint32_t ch = fd_div(e, bt.len);
                    float v[4], q[4], d[4];
                    uint32_t packed;
                    raw[j].get(v);
                    quantize4(v, sh.s[ch], sh.y[ch], q, d, packed);
                    if (st_values) store4<T>(values + e, q);
                    if (st_dequant) store4<T>(dequant + e, d);
                    if (want_code) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                }
            } else {
#pragma unroll 1
                for (uint32_t e = tid; e < n; e += GT) {
                    const uint32_t ch = fd_div(e, bt.len);
                    DivPlan dv;
                    dv.s = sh.s[ch];
                    dv.y = sh.y[ch];
                    dv.kind = sh.kind[ch];
                    float q;
                    uint32_t code;
                    lookup(bf16_pattern(divide(dv, elem_f32<T>(xs, e))), q, code);
                    if (it.values) store_one<T>(values + e, q);
                    if (it.dequant) store_one<T>(dequant + e, Arith<T>::rnd(__fmul_rn(q, dv.s)));
                    if (want_code) codes[e] = (uint8_t)code;
                }
            }
        }
        if (vec && ragged) release_stage();                  // the rolled loops read the stage until here
    }
}

// ---------------------------------------------------------------------------------------------
// Streaming variant: warps in ROLES that never meet at a barrier.
//
//   producer warp      bulk-copies batches of whole channels (<= RS_BATCH elements) into an RS_STAGES-deep ring,
//                      serving whichever stage has been returned; before a copy it clears the stage's per-channel
//                      scratch (maximum and smallest non-zero |x|);
//   reduction warps    RS_ATEAMS teams of RS_AW warps; team t takes the batches t, t + RS_ATEAMS, ...: every warp
//                      reads one contiguous run of the batch from the stage (16 bytes per lane and piece), keeps a
//                      running maximum while its run stays inside a channel, and adds it to the scratch with one
//                      warp reduction + one pair of shared-memory atomics per channel it touched; arrives on amax[s];
//   quantization warps RS_QTEAMS teams of RS_QW warps; team t takes the batches t, t + RS_QTEAMS, ...: after amax[s]
//                      lane l of a warp prepares scale and division of channel c_lo + l of the warp's run (at most
//                      RS_MAXCH / ... channels; a run of six pieces touches at most seven), the warp walks its run
//                      from the stage, fetches a channel's numbers by shuffle when the run enters it, quantizes and
//                      stores; the lane whose channel starts inside the run writes the channel's scale and maximum;
//                      arrives on empty[s].
// Nothing is held in registers across phases (64 registers, 31 warps per SM) and no phase waits for a whole
// group: what a warp waits for is data (mbarriers), never a slower neighbour.  Batches that do not qualify for
// the walk in 128-element pieces (channel length no multiple of 128, unaligned tensors) are handled channel by
// channel, the warps of the quantization team taking the channels in turn, with warp reductions; they are rare.
// A stage always belongs to the same reduction team and the same quantization team (RS_STAGES is a multiple of
// both team counts), so every waiter sees every phase of the barriers it waits on.  Every wait is bounded.
constexpr int RS_STAGES = 8, RS_QTEAMS = 4, RS_QW = 6, RS_ATEAMS = 2, RS_AW = 3;
constexpr int RS_PIECES_Q = 6;                                  // 128-element pieces per quantization warp and batch
constexpr int RS_BATCH = RS_QW * RS_PIECES_Q * 128;             // 4608 elements
constexpr int RS_MAXCH = 64;                                    // channels per batch
constexpr int RS_WARPS = 1 + RS_ATEAMS * RS_AW + RS_QTEAMS * RS_QW;
constexpr int RS_THREADS = RS_WARPS * 32;                       // 992
static_assert(RS_STAGES % RS_QTEAMS == 0 && RS_STAGES % RS_ATEAMS == 0, "a stage must belong to one team of each role");
static_assert(RS_PIECES_Q + 1 <= 32 && RS_BATCH / 128 <= RS_MAXCH, "a warp's run touches at most one channel per piece plus one");

// One batch, everything the warps need already worked out on the host (96 bytes): pointers advanced to the
// batch's first element / first channel, so that no warp touches the tensor descriptors or multiplies offsets.
struct StreamBatch {
    const void* x;
    void* values;
    void* dequant;
    uint8_t* codes;
    void* amax_out;
    void* scale_out;            // null when scales are supplied
    const void* scale_in;
    uint32_t L, nc;
    FastDiv len;                // flat index -> channel
    uint32_t flags;             // bit 0: bulk-copied (aligned, whole vectors), bit 1: walked in 128-element pieces
    uint32_t pad[3];
};
static_assert(sizeof(StreamBatch) == 96, "StreamBatch is copied to shared memory in 16-byte pieces");
constexpr int kSmemStream = 48;        // batch records a CTA keeps in shared memory (the rest is read from global memory)

struct StreamScratch {
    uint32_t amax[RS_MAXCH];
    uint32_t minnz[RS_MAXCH];        // smallest non-zero |x| bit pattern minus one
};

// Four elements of one channel whose quotients are in the range of the corrected-reciprocal division
// (q = x y, q += (x - s q) y: the correctly rounded x / s), two elements per packed fp32 instruction.
template <typename T, int TK>
__device__ __forceinline__ void stream_quantize4(const uint8_t* s_codes, const float* s_lv2, float lo, float hi, const float* v,
                                                 float sc, float y, float* q, float* d, uint32_t& packed) {
    float t[4], r[4];
    t[0] = v[0]; t[1] = v[1]; t[2] = v[2]; t[3] = v[3];
    mul2(t[0], t[1], y);
    mul2(t[2], t[3], y);
    fma2(r[0], r[1], t[0], t[1], -sc, v[0], v[1]);
    fma2(r[2], r[3], t[2], t[3], -sc, v[2], v[3]);
    fma2(t[0], t[1], r[0], r[1], y, t[0], t[1]);
    fma2(t[2], t[3], r[2], r[3], y, t[2], t[3]);
    packed = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t pat = bf16_pattern(__uint_as_float((__float_as_uint(t[k]) & 0x7FFFFFFFu) | (__float_as_uint(v[k]) & 0x80000000u)));
        uint32_t code;
        pipe_lookup<TK>(s_codes, s_lv2, lo, hi, pat, q[k], code);
        packed |= code << (8 * k);
        d[k] = q[k];
    }
    mul2(d[0], d[1], sc);
    mul2(d[2], d[3], sc);
#pragma unroll
    for (int k = 0; k < 4; ++k) d[k] = Arith<T>::rnd(d[k]);
}

template <typename T, int TK>
__global__ void __launch_bounds__(RS_THREADS, 1) channel_stream_kernel(const BatchParams p) {
    extern __shared__ uint4 smem[];
    // layout: [code table 64 KB + levels2 2 KB (TK_LUT)] [ring] [scratch per stage] [batch descriptors] [barriers]
    constexpr uint32_t TAB_BYTES = TK == TK_LUT ? 65536u + 2048u : 0u;
    constexpr uint32_t STAGE_BYTES = RS_BATCH * sizeof(T);
    uint8_t* base = reinterpret_cast<uint8_t*>(smem);
    const uint8_t* s_codes = base;
    const float* s_lv2 = reinterpret_cast<const float*>(base + 65536);
    uint8_t* ring = base + TAB_BYTES;
    StreamScratch* scratch = reinterpret_cast<StreamScratch*>(ring + RS_STAGES * STAGE_BYTES);
    StreamBatch* sbatches = reinterpret_cast<StreamBatch*>(scratch + RS_STAGES);    // this CTA's first kSmemStream batches
    const uint32_t bar0 = tc::smem_u32(sbatches + kSmemStream);
    const uint32_t FULL0 = bar0, AMAX0 = bar0 + 8u * RS_STAGES, EMPTY0 = bar0 + 16u * RS_STAGES, TABLE_BAR = bar0 + 24u * RS_STAGES;
    volatile int* team_ok = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(sbatches + kSmemStream) + 8 * (3 * RS_STAGES + 1));
    const StreamBatch* gbatches = reinterpret_cast<const StreamBatch*>(p.batches);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < RS_STAGES; ++s) {
                tc::mbar_init(FULL0 + 8u * s, 1);
                tc::mbar_init(AMAX0 + 8u * s, RS_AW);
                tc::mbar_init(EMPTY0 + 8u * s, RS_QW);
            }
            tc::mbar_init(TABLE_BAR, 1);
            tc::fence_barrier_init();
        }
        __syncwarp();
        if (lane == 0 && TK == TK_LUT) {
            tc::mbar_expect_tx(TABLE_BAR, 65536u + 2048u);
            bulk_load(tc::smem_u32(base), p.common.tab.lut8, 65536u, TABLE_BAR);
            bulk_load(tc::smem_u32(base + 65536), p.common.tab.levels2, 2048u, TABLE_BAR);
        }
    }
    for (int c = threadIdx.x; c < RS_STAGES * RS_MAXCH; c += blockDim.x) {       // every stage's scratch starts empty
        scratch[c / RS_MAXCH].amax[c % RS_MAXCH] = 0u;
        scratch[c / RS_MAXCH].minnz[c % RS_MAXCH] = 0xFFFFFFFFu;
    }
    {
        const uint4* src = reinterpret_cast<const uint4*>(gbatches);
        uint4* dst = reinterpret_cast<uint4*>(sbatches);
        constexpr int W = sizeof(StreamBatch) / 16;
        for (int t = threadIdx.x; t < kSmemStream * W; t += blockDim.x) {
            const int64_t b = blockIdx.x + (int64_t)(t / W) * gridDim.x;
            if (b < p.n_batches) dst[t] = __ldg(src + b * W + t % W);
        }
    }
    __syncthreads();
    const float lo = p.common.tab.lo, hi = p.common.tab.hi;
    auto batch_of = [&](int i, int64_t b) -> const StreamBatch& {
        return *(i < kSmemStream ? static_cast<const StreamBatch*>(sbatches + i) : gbatches + b);
    };
    // A team waits through its first warp: one lane polls, the others sit at the team's named barrier (a waiting warp
    // then issues nothing).  Returns false for the whole team when the wait ran out.
    auto team_wait = [&](int bar_id, int team_threads, bool leader, int slot, uint32_t bar_a, uint32_t bar_b, uint32_t bar_c,
                         uint32_t parity) -> bool {
        if (leader && lane == 0) {
            bool ok = tc::mbar_wait_relaxed(bar_a, parity, p.wait_budget);
            if (ok && bar_b) ok = tc::mbar_wait_relaxed(bar_b, parity, p.wait_budget);
            if (ok && bar_c) ok = tc::mbar_wait_relaxed(bar_c, 0u, p.wait_budget);
            team_ok[slot] = ok ? 1 : 0;
        }
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(team_threads) : "memory");
        return team_ok[slot] != 0;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        int k[RS_STAGES];                                       // batches loaded into stage s so far
#pragma unroll
        for (int s = 0; s < RS_STAGES; ++s) k[s] = 0;
        int left = 0;
        for (int64_t b = blockIdx.x; b < p.n_batches; b += gridDim.x) ++left;
        long long idle_since = clock64();
        bool ok = true;
        while (left > 0 && ok) {
            bool progress = false;
#pragma unroll
            for (int s = 0; s < RS_STAGES; ++s) {
                const int i = s + k[s] * RS_STAGES;
                const int64_t b = blockIdx.x + (int64_t)i * gridDim.x;
                bool go = b < p.n_batches;
                if (go && i >= RS_STAGES) {
                    bool free_ = true;
                    if (lane == 0) free_ = tc::mbar_try_wait(EMPTY0 + 8u * s, ((uint32_t)(i / RS_STAGES) & 1u) ^ 1u);
                    go = __shfl_sync(0xFFFFFFFFu, free_, 0);
                }
                if (!go) continue;                            // warp uniform
                ++k[s];
                --left;
                progress = true;
                // the stage's scratch starts empty: the whole warp clears it, then one lane starts the copy
                for (int c = lane; c < RS_MAXCH; c += 32) {
                    scratch[s].amax[c] = 0u;
                    scratch[s].minnz[c] = 0xFFFFFFFFu;
                }
                __syncwarp();
                if (lane == 0 && b != p.skip_batch) {         // skip_batch, tests only: the waits for this batch run out
                    const StreamBatch& bt = batch_of(i, b);
                    if (bt.flags & 1u) {
                        const uint32_t bytes = bt.nc * bt.L * (uint32_t)sizeof(T);
                        tc::mbar_expect_tx(FULL0 + 8u * s, bytes);
                        bulk_load(tc::smem_u32(ring + s * STAGE_BYTES), bt.x, bytes, FULL0 + 8u * s);
                    } else {
                        tc::mbar_arrive(FULL0 + 8u * s);      // the quantization warp reads this batch itself
                    }
                }
            }
            if (progress) {
                idle_since = clock64();
            } else {
                if (clock64() - idle_since > p.wait_budget) ok = false;
                // nothing was free: sleep on the stage whose batch is the oldest outstanding (woken when it is
                // returned, or after a microsecond to look at the others again)
                int oldest = 0x7FFFFFFF, so = 0;
#pragma unroll
                for (int s = 0; s < RS_STAGES; ++s) {
                    const int i = s + k[s] * RS_STAGES;
                    if (blockIdx.x + (int64_t)i * gridDim.x < p.n_batches && i < oldest) {
                        oldest = i;
                        so = s;
                    }
                }
                if (lane == 0 && oldest >= RS_STAGES && oldest != 0x7FFFFFFF)
                    tc::mbar_try_wait_suspended(EMPTY0 + 8u * so, ((uint32_t)(oldest / RS_STAGES) & 1u) ^ 1u, 1000u);
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            atomicCAS(&g_channel_status, 0, 31);
            // copies already under way get a bounded time to land before the CTA ends
#pragma unroll
            for (int s = 0; s < RS_STAGES; ++s)
                if (k[s] > 0) tc::mbar_wait_relaxed(FULL0 + 8u * s, (uint32_t)(k[s] - 1) & 1u, p.wait_budget >> 4);
        }
        return;
    }

    if (warp <= RS_ATEAMS * RS_AW) {
        // ------------------------------------------------------------------ reduction warps
        const int team = (warp - 1) / RS_AW, idx = (warp - 1) % RS_AW;
        for (int i = team;; i += RS_ATEAMS) {
            const int64_t b = blockIdx.x + (int64_t)i * gridDim.x;
            if (b >= p.n_batches) break;
            const int s = i % RS_STAGES;
            if (!team_wait(1 + team, RS_AW * 32, idx == 0, team * 2 + ((i / RS_ATEAMS) & 1), FULL0 + 8u * s, 0u, 0u,
                           (uint32_t)(i / RS_STAGES) & 1u)) {
                if (lane == 0) atomicCAS(&g_channel_status, 0, 32);
                break;
            }
            const StreamBatch& bt = batch_of(i, b);
            const bool need_amax = !bt.scale_in || bt.amax_out;
            if ((bt.flags & 2u) && need_amax) {
                const uint32_t L = bt.L, n = bt.nc * L;
                const uint32_t pieces = n >> 7, per = (pieces + RS_AW - 1) / RS_AW, q0 = (uint32_t)idx * per;
                const int cnt = q0 < pieces ? (int)min(per, pieces - q0) : 0;
                if (cnt > 0) {
                    const T* st = reinterpret_cast<const T*>(ring + s * STAGE_BYTES) + (q0 << 7) + (uint32_t)lane * 4u;
                    StreamScratch& sc = scratch[s];
                    uint32_t e0 = q0 << 7;
                    uint32_t cur = fd_div(e0, bt.len), next = (cur + 1u) * L, m = 0u, mn = 0xFFFFFFFFu;
                    auto flush = [&]() {
                        const uint32_t wm = __reduce_max_sync(0xFFFFFFFFu, m), wn = __reduce_min_sync(0xFFFFFFFFu, mn);
                        if (lane == 0) {
                            atomicMax(&sc.amax[cur], wm);
                            atomicMin(&sc.minnz[cur], wn);
                        }
                    };
#pragma unroll 4
                    for (int j = 0; j < cnt; ++j, e0 += 128u) {
                        if (e0 >= next) {                     // warp uniform: the run has entered the next channel
                            flush();
                            ++cur;
                            next += L;
                            m = 0u;
                            mn = 0xFFFFFFFFu;
                        }
                        RawVec<T> r;
                        r.load_shared(st + (j << 7));
                        float v[4];
                        r.get(v);
                        const uint32_t a0 = abs_bits(v[0]), a1 = abs_bits(v[1]), a2 = abs_bits(v[2]), a3 = abs_bits(v[3]);
                        m = max(max(m, a0), max(a1, max(a2, a3)));
                        mn = min(min(mn, a0 - 1u), min(a1 - 1u, min(a2 - 1u, a3 - 1u)));   // a zero wraps to the top and drops out
                    }
                    flush();
                }
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(AMAX0 + 8u * s);
        }
        return;
    }

    // ---------------------------------------------------------------------- quantization warps
    const int qw = warp - 1 - RS_ATEAMS * RS_AW;
    const int team = qw / RS_QW, idx = qw % RS_QW;
    bool tables_ready = TK != TK_LUT;
    for (int i = team;; i += RS_QTEAMS) {
        const int64_t b = blockIdx.x + (int64_t)i * gridDim.x;
        if (b >= p.n_batches) break;
        const int s = i % RS_STAGES;
        const uint32_t ph = (uint32_t)(i / RS_STAGES) & 1u;
        // the reductions of this batch are in the scratch, the copy has landed, and (first batch) the tables are in place
        if (!team_wait(1 + RS_ATEAMS + team, RS_QW * 32, idx == 0, 2 * RS_ATEAMS + team * 2 + ((i / RS_QTEAMS) & 1), AMAX0 + 8u * s,
                       FULL0 + 8u * s, tables_ready ? 0u : TABLE_BAR, ph)) {
            if (lane == 0) atomicCAS(&g_channel_status, 0, 33);
            break;
        }
        tables_ready = true;
        const StreamBatch& bt = batch_of(i, b);
        const uint32_t L = bt.L, n = bt.nc * L;
        const bool need_amax = !bt.scale_in || bt.amax_out;
        T* const values = reinterpret_cast<T*>(bt.values);
        T* const dequant = reinterpret_cast<T*>(bt.dequant);
        uint8_t* const codes = bt.codes;
        T* const amax_out = reinterpret_cast<T*>(bt.amax_out);
        T* const scale_out = reinterpret_cast<T*>(bt.scale_out);
        const T* const scale_in = reinterpret_cast<const T*>(bt.scale_in);
        const T* const st = reinterpret_cast<const T*>(ring + s * STAGE_BYTES);
        const StreamScratch& sc_s = scratch[s];
        // scale of a channel from its maximum, as the settled observer derives it
        auto scale_of = [&](uint32_t mb) -> float {
            const float amax = __uint_as_float(mb);
            const float ratio = p.inv_qmax != 0.0f ? __fmul_rn(amax, p.inv_qmax) : __fdiv_rn(amax, p.qmax);
            return (mb != 0u && mb < 0x7F800000u) ? Arith<T>::rnd(ratio) : 1.0f;
        };
        if (bt.flags & 2u) {
            const uint32_t pieces = n >> 7, per = (pieces + RS_QW - 1) / RS_QW, q0 = (uint32_t)idx * per;
            const int cnt = q0 < pieces ? (int)min(per, pieces - q0) : 0;
            if (cnt > 0) {
                const uint32_t e_w = q0 << 7;
                const uint32_t c_lo = fd_div(e_w, bt.len), c_hi = fd_div(e_w + ((uint32_t)cnt << 7) - 1u, bt.len);
                const bool mine = c_lo + (uint32_t)lane <= c_hi;
                const uint32_t c_mine = mine ? c_lo + (uint32_t)lane : c_hi;
                const uint32_t cg = c_mine;                    // the channel pointers start at the batch's first channel
                float sc_l = 1.0f;
                uint32_t mb = 0u;
                if (need_amax) {
                    mb = sc_s.amax[c_mine];
                    sc_l = scale_of(mb);
                    if (mine && c_mine * L >= e_w) {          // the channel starts inside this warp's run
                        if (amax_out) store_one<T>(amax_out + cg, __uint_as_float(mb));
                        if (scale_out) store_one<T>(scale_out + cg, sc_l);
                    }
                }
                if (scale_in) sc_l = elem_f32<T>(scale_in, cg);
                const DivPlan dl = plan_division(sc_l);
                const uint32_t sb = __float_as_uint(sc_l), ex = (sb >> 23) & 0xFFu;
                const bool exact_l = dl.kind != 0 && (sb >> 31) == 0u && ex >= 97u && ex <= 157u && need_amax &&
                                     mb < 0x5E000000u && sc_s.minnz[c_mine] >= 0x0D800000u - 1u;
                const bool all_exact = __all_sync(0xFFFFFFFFu, exact_l);
                if (values || dequant || codes) {
                    const T* src = st + e_w + (uint32_t)lane * 4u;
                    if (all_exact) {
                        // the common case, without a branch per piece (the channel of a piece by division, its numbers
                        // by two shuffles), two pieces per iteration so that their table reads overlap
                        auto piece = [&](int j) {
                            const uint32_t e0 = e_w + ((uint32_t)j << 7);
                            const int from = (int)(fd_div(e0, bt.len) - c_lo);
                            const float sc = __shfl_sync(0xFFFFFFFFu, sc_l, from), y = __shfl_sync(0xFFFFFFFFu, dl.y, from);
                            RawVec<T> r;
                            r.load_shared(src + (j << 7));
                            float v[4], q[4], d[4];
                            uint32_t packed;
                            r.get(v);
                            stream_quantize4<T, TK>(s_codes, s_lv2, lo, hi, v, sc, y, q, d, packed);
                            const uint32_t e = e0 + (uint32_t)lane * 4u;
                            if (values) store4<T>(values + e, q);
                            if (dequant) store4<T>(dequant + e, d);
                            if (codes) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                        };
                        int j = 0;
                        for (; j + 2 <= cnt; j += 2) {
                            piece(j);
                            piece(j + 1);
                        }
                        if (j < cnt) piece(j);
                    } else {
                        // rare: some channel of the run needs the per-element checks of the division
                        uint32_t cur = c_lo, next = (c_lo + 1u) * L, e0 = e_w;
                        float sc = __shfl_sync(0xFFFFFFFFu, sc_l, 0), y = __shfl_sync(0xFFFFFFFFu, dl.y, 0);
                        int kind = __shfl_sync(0xFFFFFFFFu, dl.kind, 0);
#pragma unroll 1
                        for (int j = 0; j < cnt; ++j, e0 += 128u) {
                            if (e0 >= next) {                 // warp uniform
                                ++cur;
                                next += L;
                                const int from = (int)(cur - c_lo);
                                sc = __shfl_sync(0xFFFFFFFFu, sc_l, from);
                                y = __shfl_sync(0xFFFFFFFFu, dl.y, from);
                                kind = __shfl_sync(0xFFFFFFFFu, dl.kind, from);
                            }
                            RawVec<T> r;
                            r.load_shared(src + (j << 7));
                            float v[4], q[4], d[4];
                            uint32_t packed = 0u;
                            r.get(v);
                            DivPlan dv;
                            dv.s = sc;
                            dv.y = y;
                            dv.kind = kind;
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                uint32_t code;
                                pipe_lookup<TK>(s_codes, s_lv2, lo, hi, bf16_pattern(divide(dv, v[kk])), q[kk], code);
                                packed |= code << (8 * kk);
                                d[kk] = Arith<T>::rnd(__fmul_rn(q[kk], sc));
                            }
                            const uint32_t e = e0 + (uint32_t)lane * 4u;
                            if (values) store4<T>(values + e, q);
                            if (dequant) store4<T>(dequant + e, d);
                            if (codes) __stcs(reinterpret_cast<uint32_t*>(codes + e), packed);
                        }
                    }
                }
            }
        } else {
            // channel by channel, the team's warps taking the channels in turn (channel lengths that are no multiple
            // of 128, unaligned tensors); everything stays inside a warp
            const T* xs = (bt.flags & 1u) ? st : reinterpret_cast<const T*>(bt.x);
            for (uint32_t c = (uint32_t)idx; c < bt.nc; c += RS_QW) {
                const uint32_t e_c = c * L;
                const uint32_t cg = c;
                float sc = 1.0f;
                if (need_amax) {
                    uint32_t m = 0u;
                    for (uint32_t e = lane; e < L; e += 32u) m = max(m, abs_bits(elem_f32<T>(xs, e_c + e)));
                    m = __reduce_max_sync(0xFFFFFFFFu, m);
                    sc = scale_of(m);
                    if (lane == 0) {
                        if (amax_out) store_one<T>(amax_out + cg, __uint_as_float(m));
                        if (scale_out) store_one<T>(scale_out + cg, sc);
                    }
                }
                if (scale_in) sc = elem_f32<T>(scale_in, cg);
                if (values || dequant || codes) {
                    const DivPlan dv = plan_division(sc);
                    for (uint32_t e = lane; e < L; e += 32u) {
                        float q;
                        uint32_t code;
                        pipe_lookup<TK>(s_codes, s_lv2, lo, hi, bf16_pattern(divide(dv, elem_f32<T>(xs, e_c + e))), q, code);
                        if (values) store_one<T>(values + e_c + e, q);
                        if (dequant) store_one<T>(dequant + e_c + e, Arith<T>::rnd(__fmul_rn(q, sc)));
                        if (codes) codes[e_c + e] = (uint8_t)code;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(EMPTY0 + 8u * s);
    }
}

// channels per batch / batches of one item, for batches of about `batch_elems` elements
inline int64_t channels_per_batch(const vq_channel_item& it, int64_t batch_elems, int vec_elems = 1, int64_t max_channels = kBatchMaxChannels) {
    int64_t per = batch_elems / it.length;
    per = per < 1 ? 1 : (per > max_channels ? max_channels : per);
    if (vec_elems > 1 && it.length % vec_elems) {
        // channel length no multiple of a 16-byte vector: a multiple of q channels is
        int64_t g = it.length, b = vec_elems;
        while (b) { const int64_t t = g % b; g = b; b = t; }
        const int64_t q = vec_elems / g;
        if (per >= q) per = per / q * q;
    }
    return per;
}
// 1 when the batch [c0, c0 + nc) of `it` can be moved and processed in 16-byte vectors
inline int batch_vec(const vq_channel_item& it, int64_t c0, int64_t nc, int dtype) {
    const int64_t ve = dtype == VQ_F32 ? 4 : 8;
    const bool aligned = ((uintptr_t)it.input & 15) == 0 && ((uintptr_t)it.values & 15) == 0 && ((uintptr_t)it.dequant & 15) == 0 &&
                         ((uintptr_t)it.codes & 3) == 0;
    return aligned && (c0 * it.length) % ve == 0 && (nc * it.length) % ve == 0;
}
inline int64_t batches_of(const vq_channel_item& it, int64_t batch_elems, int vec_elems = 1, int64_t max_channels = kBatchMaxChannels) {
    if (it.channels <= 0) return 0;
    const int64_t per = channels_per_batch(it, batch_elems, vec_elems, max_channels);
    return (it.channels + per - 1) / per;
}
// the workspace is sized for the finest split any kernel uses
constexpr int64_t kSmallestBatch = RS_BATCH < PIPE_BATCH ? RS_BATCH : PIPE_BATCH;
constexpr int64_t kFewestChannels = RS_MAXCH;

}  // namespace
extern "C" size_t vq_channel_quantize_multi_workspace(const vq_channel_item* items, int n_items);
namespace {

inline size_t items_bytes_of(int n_items) { return ((size_t)n_items * sizeof(vq_channel_item) + 31) / 32 * 32; }

// Everything a launch needs, decided once from the host descriptors.
struct ChanLaunch {
    BatchParams p{};
    int kernel = 0;                 // 0 two sweeps, 2 pipelined, 3 streaming roles
    int dtype = 0, mode = 0, n_items = 0;
    bool lut_tab = false;
    int threads = 0, blocks = 0;
    size_t smem = 0, items_bytes = 0;
    std::vector<ChanBatch> batches; // host copy until it has been uploaded
    std::vector<StreamBatch> records;   // streaming kernel: what is uploaded instead of `batches`
};

// Argument checks, kernel choice, batch list.  0 on success; L.p.n_batches == 0: nothing to do.
int channel_prepare(const char* name, const vq_channel_item* items, int n_items, int dtype, double quant_max, const vq_table* table,
                    void* workspace, size_t workspace_bytes, ChanLaunch& L) {
    VQ_REQUIRE(items != nullptr, "%s: null item array", name);
    VQ_REQUIRE(dtype == VQ_F32 || dtype == VQ_BF16, "%s: dtype must be VQ_F32 or VQ_BF16", name);
    VQ_REQUIRE(quant_max > 0.0, "%s: quant_max must be positive", name);
    bool any_table_out = false, any_codes = false;
    int64_t total = 0, longest = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_channel_item& it = items[i];
        const bool ok = it.input && it.channels >= 0 && it.channels < (1ll << 31) && it.length >= 1 &&
                        it.length < (1ll << 22) && (it.amax_out || it.scale_out || it.values || it.codes || it.dequant);
        VQ_REQUIRE(ok, "%s: item %d needs an input, a channel length in [1, 2^22) and at least one output", name, i);
        any_table_out |= it.values || it.codes || it.dequant;
        any_codes |= it.codes != nullptr;
        total += it.channels * it.length;
        if (it.channels > 0 && it.length > longest) longest = it.length;
    }
    VQ_REQUIRE(!any_table_out || (table && table->kind != VQ_TABLE_NONE), "%s: quantized outputs need a table", name);
    if (any_codes) {
        const bool have = table->kind == VQ_TABLE_INT || table->lut8 || (table->kind == VQ_TABLE_RUNS && table->run_codes);
        VQ_REQUIRE(have, "%s: packed codes need a code table", name);
    }
    VQ_REQUIRE(workspace && (uintptr_t)workspace % 16 == 0 && workspace_bytes >= vq_channel_quantize_multi_workspace(items, n_items),
               "%s: workspace missing, unaligned or smaller than vq_channel_quantize_multi_workspace(items, n_items)", name);

    BatchParams& p = L.p;
    p = BatchParams{};
    p.qmax = (float)quant_max;
    {
        int ex = 0;
        const float mant = frexpf(p.qmax, &ex);
        p.inv_qmax = (mant == 0.5f && ex > -100 && ex < 100) ? 1.0f / p.qmax : 0.0f;
    }
    p.wait_budget = PIPE_WAIT;
    p.skip_batch = -1;
    // Test hooks of the bounded waits: VOYAGER_B200_CHANNEL_WAIT_CYCLES shortens the budget and
    // VOYAGER_B200_CHANNEL_SKIP_BATCH makes the producer leave one batch out, so that a wait runs out, the
    // kernel records it (vq_channel_status) and winds down.  Read when a launch is prepared.
    if (const char* e = getenv("VOYAGER_B200_CHANNEL_WAIT_CYCLES")) {
        const long long v = atoll(e);
        if (v > 0) p.wait_budget = v;
    }
    if (const char* e = getenv("VOYAGER_B200_CHANNEL_SKIP_BATCH")) p.skip_batch = atoi(e);
    p.common.tab = to_dev(table);
    const bool lut = table && table->kind == VQ_TABLE_LUT16;
    const bool big = total >= (1 << 21);
    p.common.smem_lut16 = (big && lut) ? 1 : 0;
    p.common.smem_lut8 = (big && lut && any_codes && table->lut8) ? 1 : 0;
    p.table_bytes = (p.common.smem_lut16 ? 131072 : 0) + (p.common.smem_lut8 ? 65536 : 0) +
                    ((table && table->kind == VQ_TABLE_RUNS) ? ((5 * VQ_MAX_RUNS + 15) / 16 * 16) : 0);
    const bool direct = lut && table->nan_uniform && (!any_codes || table->lut8);
    const bool staged = direct && p.common.smem_lut16 && (!any_codes || p.common.smem_lut8);
    const int mode = staged ? 2 : (direct ? 1 : 0);
    // Kernel choice (VOYAGER_B200_CHANNEL_KERNEL=sweep forces the second one, for measurements):
    //   pipe   bulk-copy pipeline; needs every channel to fit a batch and either an INT table or a code
    //          table whose values follow from (code, input sign);
    //   sweep  two sweeps per batch, any table, any channel length.
    const char* want_kernel = getenv("VOYAGER_B200_CHANNEL_KERNEL");
    const bool pipe_table = table && ((table->kind == VQ_TABLE_INT && table->lo >= -128.0f && table->hi <= 255.0f) ||
                                      (table->kind == VQ_TABLE_LUT16 && table->nan_uniform && table->lut8 && table->levels2 &&
                                       (uintptr_t)table->lut8 % 16 == 0 && (uintptr_t)table->levels2 % 16 == 0));
    //   stream the same tables and bulk copies with warps in roles and no barrier; channels up to RS_BATCH elements;
    bool use_pipe = big && (pipe_table || !any_table_out) && longest <= PIPE_BATCH;
    if (want_kernel && !strcmp(want_kernel, "sweep")) use_pipe = false;
    const bool use_stream = use_pipe && longest <= RS_BATCH && !(want_kernel && !strcmp(want_kernel, "pipe"));
    const int64_t batch_elems = use_stream ? RS_BATCH : (use_pipe ? PIPE_BATCH : kBatchElems);
    const int64_t max_channels = use_stream ? RS_MAXCH : kBatchMaxChannels;

    const int vec_elems = use_pipe ? (dtype == VQ_F32 ? 4 : 8) : 1;
    // Batches of the pipelined kernel that cannot go through registers (channel length no multiple of 4
    // elements, unaligned tensors) cost several times more per element: they are cut eight times smaller
    // so that no single one unbalances the CTAs.
    auto item_batch = [&](const vq_channel_item& it) -> int64_t {
        if (!use_pipe) return batch_elems;
        const bool lean = it.length % 4 == 0 && batch_vec(it, 0, 4, dtype);
        if (!lean) return batch_elems / 8;
        // streaming kernel: channels that are not walked in 128-element pieces are taken channel by channel, which
        // costs several times more per element
        if (use_stream && (it.length % 128 != 0 || it.length < 128)) return batch_elems / 4;
        return batch_elems;
    };
    int64_t n_batches = 0;
    for (int i = 0; i < n_items; ++i) n_batches += batches_of(items[i], item_batch(items[i]), vec_elems, max_channels);
    VQ_REQUIRE(n_batches < (1ll << 31), "%s: too many channels", name);
    L.dtype = dtype;
    L.n_items = n_items;
    L.mode = mode;
    if (n_batches == 0) return 0;

    const size_t items_bytes = ((size_t)n_items * sizeof(vq_channel_item) + 31) / 32 * 32;
    L.items_bytes = items_bytes;
    L.batches.resize((size_t)n_batches);
    ChanBatch* hb = L.batches.data();
    int64_t k = 0;
    for (int i = 0; i < n_items; ++i) {
        const vq_channel_item& it = items[i];
        if (it.channels <= 0) continue;
        const int64_t per = channels_per_batch(it, item_batch(it), vec_elems, max_channels);
        const FastDiv fdv = make_fastdiv((uint32_t)it.length);
        for (int64_t c0 = 0; c0 < it.channels; c0 += per, ++k) {
            hb[k].item = i;
            hb[k].c0 = (int)c0;
            hb[k].nc = (int)(it.channels - c0 < per ? it.channels - c0 : per);
            hb[k].len = fdv;
            hb[k].vec = batch_vec(it, hb[k].c0, hb[k].nc, dtype);
            hb[k].fast = (use_pipe && hb[k].vec && it.length % 128 == 0 && it.length >= 128) ? 1 : 0;
        }
    }
    if (use_pipe) {
        // CTA c walks batches c, c + grid, c + 2 grid, ...: with the list ordered by estimated cost every
        // CTA receives one batch of each cost tier
        auto cost = [&](const ChanBatch& b) -> int64_t {
            const vq_channel_item& it = items[b.item];
            const int64_t n = (int64_t)b.nc * it.length;
            const int64_t per_elem = !b.vec ? (use_stream ? 16 : 10) : (it.length % 4 ? (use_stream ? 12 : 6) : ((use_stream && !b.fast) ? 8 : 1));
            return n * per_elem + 64 * (int64_t)b.nc;
        };
        std::stable_sort(hb, hb + n_batches, [&](const ChanBatch& a, const ChanBatch& b) { return cost(a) > cost(b); });
        if (use_stream) {
            // Streaming kernel: instead of dealing the ordered list round robin, every batch goes to the CTA with the
            // least estimated work so far (longest processing time first); CTA c still walks positions c, c + grid, ...
            // of the list, so its batches are written there and the shorter lists end in empty records (no channels).
            const int grid = (int)(n_batches < vq_sm_count() ? n_batches : vq_sm_count());
            std::vector<std::vector<int64_t>> lists((size_t)grid);
            std::vector<std::pair<int64_t, int>> heap;         // (work, cta), smallest work on top
            for (int c = 0; c < grid; ++c) heap.emplace_back(0, c);
            auto cmp = [](const std::pair<int64_t, int>& a, const std::pair<int64_t, int>& b) { return a > b; };
            std::make_heap(heap.begin(), heap.end(), cmp);
            for (int64_t j = 0; j < n_batches; ++j) {
                std::pop_heap(heap.begin(), heap.end(), cmp);
                auto& top = heap.back();
                lists[(size_t)top.second].push_back(j);
                top.first += cost(hb[j]) + 600;                // a fixed share per batch: waits, division plans
                std::push_heap(heap.begin(), heap.end(), cmp);
            }
            size_t longest_list = 0;
            for (auto& l : lists) longest_list = l.size() > longest_list ? l.size() : longest_list;
            const int64_t padded = (int64_t)longest_list * grid;
            const size_t room = (workspace_bytes - items_bytes_of(n_items)) / sizeof(StreamBatch);
            if (padded <= (int64_t)room && padded < (1ll << 31)) {
                std::vector<ChanBatch> dealt((size_t)padded);
                for (auto& b : dealt) b = ChanBatch{-1, 0, 0, make_fastdiv(1u), 0, 0};
                for (int c = 0; c < grid; ++c)
                    for (size_t i = 0; i < lists[(size_t)c].size(); ++i) dealt[i * (size_t)grid + (size_t)c] = hb[lists[(size_t)c][i]];
                L.batches.swap(dealt);
                hb = L.batches.data();
                n_batches = padded;
            }
        }
    }
    p.items = reinterpret_cast<const vq_channel_item*>(workspace);
    p.batches = reinterpret_cast<const ChanBatch*>((char*)workspace + items_bytes);
    p.n_batches = (int)n_batches;
    if (use_stream) {
        const size_t es = dtype == VQ_F32 ? 4 : 2;
        L.records.resize((size_t)n_batches);
        for (int64_t j = 0; j < n_batches; ++j) {
            const ChanBatch& b = hb[j];
            StreamBatch& r = L.records[(size_t)j];
            r = StreamBatch{};
            if (b.item < 0) {                                  // an empty record: every role passes it on at once
                r.L = 1;
                r.len = b.len;
                continue;
            }
            const vq_channel_item& it = items[b.item];
            const size_t off = (size_t)b.c0 * (size_t)it.length;
            r.x = (const char*)it.input + off * es;
            r.values = it.values ? (char*)it.values + off * es : nullptr;
            r.dequant = it.dequant ? (char*)it.dequant + off * es : nullptr;
            r.codes = it.codes ? it.codes + off : nullptr;
            r.amax_out = it.amax_out ? (char*)it.amax_out + (size_t)b.c0 * es : nullptr;
            r.scale_out = (it.scale_out && !it.scale_in) ? (char*)it.scale_out + (size_t)b.c0 * es : nullptr;
            r.scale_in = it.scale_in ? (const char*)it.scale_in + (size_t)b.c0 * es : nullptr;
            r.L = (uint32_t)it.length;
            r.nc = (uint32_t)b.nc;
            r.len = b.len;
            r.flags = (b.vec ? 1u : 0u) | (b.fast ? 2u : 0u);
        }
        L.batches.clear();
    }

    const int sms = vq_sm_count();
    if (use_stream) {
        L.kernel = 3;
        L.lut_tab = any_table_out && table->kind == VQ_TABLE_LUT16;     // no quantized output: no table is staged
        const size_t esize = dtype == VQ_F32 ? 4 : 2;
        L.smem = (L.lut_tab ? 65536 + 2048 : 0) + (size_t)RS_STAGES * RS_BATCH * esize + RS_STAGES * sizeof(StreamScratch) +
                 kSmemStream * sizeof(StreamBatch) + 8 * (3 * RS_STAGES + 1) + 4 * 2 * (RS_ATEAMS + RS_QTEAMS) + 16;
        if ((int)L.smem > vq_max_smem_optin()) return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: device offers too little shared memory", name);
        L.threads = RS_THREADS;
        L.blocks = (int)(n_batches < sms ? n_batches : sms);
    } else if (use_pipe) {
        L.kernel = 2;
        L.lut_tab = any_table_out && table->kind == VQ_TABLE_LUT16;     // no quantized output: no table is staged
        const size_t esize = dtype == VQ_F32 ? 4 : 2;
        L.smem = (L.lut_tab ? 65536 + 2048 : 0) + (size_t)PIPE_STAGES * PIPE_BATCH * esize + ((sizeof(PipeShared) + 15) / 16) * 16 +
                 kSmemItems * sizeof(vq_channel_item) + kSmemBatches * sizeof(ChanBatch) + 16 * PIPE_STAGES + 16;
        if ((int)L.smem > vq_max_smem_optin()) return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: device offers too little shared memory", name);
        L.threads = PIPE_THREADS;
        L.blocks = (int)(n_batches < sms ? n_batches : sms);
    } else {
        L.kernel = 0;
        L.smem = (size_t)p.table_bytes + 4 * sizeof(ChanShared);
        // tables in shared memory leave room for one CTA per SM: make it a full one
        L.threads = L.smem > 100 * 1024 ? 1024 : 512;
        const int per_sm = L.smem > 100 * 1024 ? 1 : 2;
        const int64_t want = (n_batches * kGroupThreads + L.threads - 1) / L.threads;
        L.blocks = (int)(want < (int64_t)sms * per_sm ? want : (int64_t)sms * per_sm);
    }
    return 0;
}

// Descriptors -> device workspace (pageable sources are staged before cudaMemcpyAsync returns).
int channel_upload(const char* name, const ChanLaunch& L, const vq_channel_item* items, int n_items, void* workspace, cudaStream_t st) {
    cudaError_t e1 = cudaMemcpyAsync(workspace, items, (size_t)n_items * sizeof(vq_channel_item), cudaMemcpyHostToDevice, st);
    const void* list = L.kernel == 3 ? (const void*)L.records.data() : (const void*)L.batches.data();
    const size_t list_bytes = L.kernel == 3 ? L.records.size() * sizeof(StreamBatch) : L.batches.size() * sizeof(ChanBatch);
    cudaError_t e2 = cudaMemcpyAsync((char*)workspace + L.items_bytes, list, list_bytes, cudaMemcpyHostToDevice, st);
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return vq_set_error(VQ_ERR_CUDA, "%s: descriptor upload failed: %s", name, cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    return 0;
}

int channel_launch(const ChanLaunch& L, cudaStream_t st) {
    const BatchParams& p = L.p;
    const int dtype = L.dtype, mode = L.mode, blocks = L.blocks, threads = L.threads, n_items = L.n_items;
    const size_t smem = L.smem;
    if (L.kernel == 3) {
#define VQ_CHS_LAUNCH(T, K)                                                                                           \
    do {                                                                                                              \
        auto kern = channel_stream_kernel<T, K>;                                                                      \
        VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                  \
        kern<<<blocks, threads, smem, st>>>(p);                                                                       \
    } while (0)
        if (dtype == VQ_F32) {
            if (L.lut_tab) VQ_CHS_LAUNCH(float, TK_LUT); else VQ_CHS_LAUNCH(float, TK_INT);
        } else {
            if (L.lut_tab) VQ_CHS_LAUNCH(bf16_t, TK_LUT); else VQ_CHS_LAUNCH(bf16_t, TK_INT);
        }
#undef VQ_CHS_LAUNCH
        VQ_LAUNCH_CHECK("channel_stream_kernel");
        return 0;
    }
    if (L.kernel == 2) {
#define VQ_CHP_LAUNCH(T, K)                                                                                           \
    do {                                                                                                              \
        auto kern = channel_pipe_kernel<T, K>;                                                                        \
        VQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                  \
        kern<<<blocks, threads, smem, st>>>(p, n_items);                                                              \
    } while (0)
        if (dtype == VQ_F32) {
            if (L.lut_tab) VQ_CHP_LAUNCH(float, TK_LUT); else VQ_CHP_LAUNCH(float, TK_INT);
        } else {
            if (L.lut_tab) VQ_CHP_LAUNCH(bf16_t, TK_LUT); else VQ_CHP_LAUNCH(bf16_t, TK_INT);
        }
#undef VQ_CHP_LAUNCH
        VQ_LAUNCH_CHECK("channel_pipe_kernel");
        return 0;
    }
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

}  // namespace

// A prepared per-channel pass (see vq_channel_plan_create).
struct vq_channel_plan {
    ChanLaunch l;
};

extern "C" {

int vq_channel_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_channel_status, sizeof(int)) != cudaSuccess) return VQ_ERR_CUDA;
    if (v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_channel_status, &zero, sizeof(int));
    }
    return v;
}

size_t vq_channel_quantize_multi_workspace(const vq_channel_item* items, int n_items) {
    if (n_items < 0 || !items) return 0;
    int64_t nb = 0;
    for (int i = 0; i < n_items; ++i) nb += (items[i].length >= 1) ? batches_of(items[i], kSmallestBatch / 8, 8, kFewestChannels) : 0;
    return (size_t)n_items * sizeof(vq_channel_item) + (size_t)nb * sizeof(StreamBatch) + 64;     // the larger of the two record kinds
}

int vq_channel_quantize_multi(const vq_channel_item* items, int n_items, int dtype, double quant_max, const vq_table* table,
                              void* workspace, size_t workspace_bytes, void* stream) {
    const char* name = "vq_channel_quantize_multi";
    VQ_REQUIRE(n_items >= 0, "%s: negative item count", name);
    if (n_items == 0) return 0;
    ChanLaunch L;
    int rc = channel_prepare(name, items, n_items, dtype, quant_max, table, workspace, workspace_bytes, L);
    if (rc || L.p.n_batches == 0) return rc;
    rc = channel_upload(name, L, items, n_items, workspace, (cudaStream_t)stream);
    if (rc) return rc;
    return channel_launch(L, (cudaStream_t)stream);
}

int vq_channel_plan_create(const vq_channel_item* items, int n_items, int dtype, double quant_max, const vq_table* table,
                           void* workspace, size_t workspace_bytes, void* stream, vq_channel_plan** plan_out) {
    const char* name = "vq_channel_plan_create";
    VQ_REQUIRE(plan_out != nullptr, "%s: null plan pointer", name);
    *plan_out = nullptr;
    VQ_REQUIRE(n_items >= 1, "%s: a plan needs at least one tensor", name);
    vq_channel_plan* plan = new (std::nothrow) vq_channel_plan();
    VQ_REQUIRE(plan != nullptr, "%s: out of host memory", name);
    int rc = channel_prepare(name, items, n_items, dtype, quant_max, table, workspace, workspace_bytes, plan->l);
    cudaStream_t st = (cudaStream_t)stream;
    if (!rc && plan->l.p.n_batches > 0) {
        rc = channel_upload(name, plan->l, items, n_items, workspace, st);
        // run() may be queued on any stream afterwards: the descriptors must have landed by then
        if (!rc && cudaStreamSynchronize(st) != cudaSuccess) rc = vq_set_error(VQ_ERR_CUDA, "%s: descriptor upload did not complete", name);
    }
    if (rc) {
        delete plan;
        return rc;
    }
    plan->l.batches.clear();
    plan->l.batches.shrink_to_fit();
    plan->l.records.clear();
    plan->l.records.shrink_to_fit();
    *plan_out = plan;
    return 0;
}

int vq_channel_plan_run(const vq_channel_plan* plan, void* stream) {
    VQ_REQUIRE(plan != nullptr, "vq_channel_plan_run: null plan");
    if (plan->l.p.n_batches == 0) return 0;
    return channel_launch(plan->l, (cudaStream_t)stream);
}

void vq_channel_plan_destroy(vq_channel_plan* plan) { delete plan; }

}  // extern "C"
