// MX-quantized GEMM on the 5th-generation tensor cores:  Y[M,N] = deq(A)[M,K] * deq(B)[N,K]^T.
//
// Persistent, warp-specialised kernel, one CTA per SM, output tile 128 x 256, K step 64:
//   producer   fills a 4-stage ring of shared-memory operand tiles (K-major, 128-byte swizzle);
//              plain variant: one thread issues TMA tile loads of bf16 operands;
//              fused variant: 8 warps load codes and per-block scales from global memory, form
//              code * scale in bf16 (one rounding, exactly what `codes * expand(scale)` gives in
//              bf16) and store straight into the swizzled layout -- no dequantised copy of the
//              operands ever exists in HBM;
//   MMA        one thread issues tcgen05.mma (bf16 x bf16 -> fp32) into a double-buffered
//              accumulator in tensor memory (2 x 256 columns) and commits to mbarriers;
//   epilogue   4 warps read the finished accumulator with tcgen05.ld, add the bias, round to bf16
//              and store, while the MMA warp already works on the next tile.
// Tensor-core bound: 2*M*N*K flops; operands are re-read from L2 across tiles.
// Every mbarrier wait is bounded; a wait that runs out records a code in `status` and the CTA
// winds down (drains its copies, frees tensor memory) instead of hanging.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "vq_common.cuh"
#include "vq_tc.cuh"

// CTA-pair kernel (vq_gemm2.cu): 256 x 256 tiles on two CTAs; tensor maps with 128-row boxes
int vq_gemm_pair_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, void* const* Ys, int n_outputs, int64_t ldy,
                        int64_t col_offset, const void* bias, int64_t M, int64_t N, int64_t K, int32_t* status,
                        cudaStream_t st, const CUtensorMap* tmSA = nullptr, const CUtensorMap* tmSB = nullptr,
                        const void* a_codes = nullptr, const void* b_codes = nullptr, bool packed_codes = false, int batch = 1,
                        int64_t a_batch_rows = 0, int64_t b_batch_rows = 0, int64_t y_batch_stride = 0,
                        const CUtensorMap* out_maps = nullptr);

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int PRODUCER_WARPS_FUSED = 8;
constexpr long long WAIT_BUDGET = 4000000000ll;   // ~2 s of SM clocks

constexpr int MAX_OUTPUTS = 8;

struct GemmParams {
    uint16_t* Y[MAX_OUTPUTS];   // every output buffer receives the same tile (own memory and peers')
    int n_outputs;
    int64_t ldy;                // elements between rows of the output buffers
    int64_t col_offset;         // first output column this launch owns
    const uint16_t* bias;
    int M, N, K;
    int tiles_m, tiles_n;
    // Batched product (plain variant): `batch` independent M x N x K problems.  A and B are addressed
    // through 2-D maps over the flattened [batch * rows, K] operands, batch b starting a_batch_rows /
    // b_batch_rows rows further down (0: the operand is shared by all batches); a tile that reaches past
    // the end of its batch reads rows of the next one, whose products land in rows / columns the
    // epilogue masks.  Output b starts y_batch_stride elements after output b - 1.
    int batch;
    int a_batch_rows, b_batch_rows;
    int64_t y_batch_stride;
    int32_t* status;
    // fused variant
    const uint16_t* a_codes;
    const uint16_t* a_scale;
    const uint16_t* b_codes;
    const uint16_t* b_scale;
    int blocks_per_row;      // K / 32
};

__device__ __forceinline__ void record_failure(int32_t* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

// code * scale for 8 bf16 values (one 16-byte chunk); product rounded once to bf16
__device__ __forceinline__ uint4 scale_chunk(uint4 c, uint32_t s2) {
    uint4 o;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.x) : "r"(c.x), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.y) : "r"(c.y), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.z) : "r"(c.z), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.w) : "r"(c.w), "r"(s2));
    return o;
}

// TF32: the operands are fp32 matrices read by the tensor cores as tf32 (K step 32 elements = the same 128-byte
// rows), the result and the bias are fp32; plain (TMA-fed) variant only.
template <bool FUSED, bool TF32 = false>
__global__ void __launch_bounds__(FUSED ? (PRODUCER_WARPS_FUSED + 5) * 32 : 192, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle atoms
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
    // barriers (8 bytes each) behind the operand ring: full[STAGES], empty[STAGES], accumulator
    // full[2] / empty[2], then the word the TMEM allocator writes its base address to
    const uint32_t bar_base = base + STAGES * STAGE_BYTES;
    const uint32_t FULL0 = bar_base, EMPTY0 = bar_base + 8u * STAGES, TFULL0 = bar_base + 16u * STAGES,
                   TEMPTY0 = TFULL0 + 16u, SLOT = TEMPTY0 + 16u;

    constexpr int NPROD = FUSED ? PRODUCER_WARPS_FUSED : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mma_warp = NPROD, epi_warp0 = NPROD + 1;
    static_assert(!(FUSED && TF32), "the fused producer stages bf16 codes");
    constexpr int BKE = TF32 ? BK / 2 : BK;                    // elements per k-step: 128 bytes either way
    const int num_k = (p.K + BKE - 1) / BKE;
    const int tiles_per_batch = p.tiles_m * p.tiles_n;
    const int n_tiles = tiles_per_batch * p.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(FULL0 + 8u * s, FUSED ? PRODUCER_WARPS_FUSED : 1);
            tc::mbar_init(EMPTY0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(TFULL0 + 8u * s, 1);
            tc::mbar_init(TEMPTY0 + 8u * s, 4);
        }
        tc::fence_barrier_init();
        if (!FUSED) {
            tc::prefetch_tensormap(&tmA);
            tc::prefetch_tensormap(&tmB);
        }
    }
    if (warp == mma_warp) {
        tc::tmem_alloc(SLOT, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(SLOT));

    if (warp < NPROD) {
        // ------------------------------------------------------------------ producer
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        if (!FUSED) {
            if (lane == 0) {
                for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                    const int bi = tile / tiles_per_batch, rem = tile - bi * tiles_per_batch;
                    const int m0 = bi * p.a_batch_rows + (rem % p.tiles_m) * BM, n0 = bi * p.b_batch_rows + (rem / p.tiles_m) * BN;
                    for (int k = 0; k < num_k; ++k) {
                        if (!tc::mbar_wait(EMPTY0 + 8u * stage, phase ^ 1u, WAIT_BUDGET)) { ok = false; break; }
                        tc::mbar_expect_tx(FULL0 + 8u * stage, STAGE_BYTES);
                        tc::tma_load_2d(base + stage * STAGE_BYTES, &tmA, k * BKE, m0, FULL0 + 8u * stage);
                        tc::tma_load_2d(base + stage * STAGE_BYTES + A_BYTES, &tmB, k * BKE, n0, FULL0 + 8u * stage);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
                if (!ok) {
                    record_failure(p.status, 1);
                    // drain: give the copies already issued a bounded time to land
                    for (int s = 0; s < STAGES; ++s) tc::mbar_wait(FULL0 + 8u * s, 0, WAIT_BUDGET >> 6);
                }
            }
        } else {
            // Fused dequantisation: each producer thread owns fixed (row, 16-byte chunk) slots of
            // the 384-row x 8-chunk stage: rows 0..127 are A rows, 128..383 are B rows.
            const int t = warp * 32 + lane;                       // 0 .. 255
            constexpr int NT = PRODUCER_WARPS_FUSED * 32;
            constexpr int SLOTS = (BM + BN) * 8 / NT;             // 12 chunks per thread per stage
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
                for (int k = 0; k < num_k; ++k) {
                    uint4 c[SLOTS];
                    uint32_t s2[SLOTS];
                    uint32_t outside = 0u;
#pragma unroll
                    for (int j = 0; j < SLOTS; ++j) {
                        const int slot = j * NT + t;
                        const int r = slot >> 3, ch = slot & 7;
                        const bool isA = r < BM;
                        const int grow = isA ? m0 + r : n0 + (r - BM);
                        const int rows = isA ? p.M : p.N;
                        const uint16_t* codes = isA ? p.a_codes : p.b_codes;
                        const uint16_t* scl = isA ? p.a_scale : p.b_scale;
                        // loads only: the SM issues in order, and an instruction that consumes a loaded value here
                        // (a select against zero, the widening of the scale) would hold back the loads behind it;
                        // rows past the end read row 0 and are zeroed when they are stored
                        const size_t srow = grow < rows ? (size_t)grow : 0;
                        c[j] = __ldg(reinterpret_cast<const uint4*>(codes + srow * p.K + k * BK + ch * 8));
                        s2[j] = __ldg(scl + srow * p.blocks_per_row + k * 2 + (ch >> 2));
                        outside |= (grow >= rows ? 1u : 0u) << j;
                    }
                    if (lane == 0) ok = tc::mbar_wait(EMPTY0 + 8u * stage, phase ^ 1u, WAIT_BUDGET);
                    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                    if (!ok) break;
                    uint8_t* st = smem + stage * STAGE_BYTES;
#pragma unroll
                    for (int j = 0; j < SLOTS; ++j) {
                        const int slot = j * NT + t;
                        const int r = slot >> 3, ch = slot & 7;
                        // operand tiles: A rows first, then B; within a tile row r at r*128 bytes,
                        // 16-byte chunk index xor-ed with (r mod 8): the 128-byte swizzle
                        const int rr = r < BM ? r : r - BM;
                        uint8_t* tilep = st + (r < BM ? 0 : A_BYTES);
                        const uint4 v = ((outside >> j) & 1u) ? make_uint4(0, 0, 0, 0) : scale_chunk(c[j], s2[j] * 0x00010001u);
                        *reinterpret_cast<uint4*>(tilep + rr * 128 + ((ch ^ (rr & 7)) << 4)) = v;
                    }
                    tc::fence_proxy_async();      // make the generic-proxy stores visible to the MMA
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(FULL0 + 8u * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && lane == 0) record_failure(p.status, 1);
        }
    } else if (warp == mma_warp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = TF32 ? tc::idesc_tf32_f32(BM, BN) : tc::idesc_bf16_f32(BM, BN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                if (!tc::mbar_wait(TEMPTY0 + 8u * acc, acc_phase ^ 1u, WAIT_BUDGET)) { ok = false; break; }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
                for (int k = 0; k < num_k; ++k) {
                    if (!tc::mbar_wait(FULL0 + 8u * stage, phase, WAIT_BUDGET)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
                    const uint64_t da = tc::smem_desc_k_sw128(sa), db = tc::smem_desc_k_sw128(sb);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {  // 32 bytes of K per instruction: +2 in 16-byte units
                        if (TF32) tc::mma_tf32(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                        else tc::mma_f16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                    }
                    tc::mma_commit(EMPTY0 + 8u * stage);  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc::mma_commit(TFULL0 + 8u * acc);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) record_failure(p.status, 2);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int bi = tile / tiles_per_batch, rem = tile - bi * tiles_per_batch;
            const int m0 = (rem % p.tiles_m) * BM, n0 = (rem / p.tiles_m) * BN;
            if (lane == 0) ok = tc::mbar_wait(TFULL0 + 8u * acc, acc_phase, WAIT_BUDGET);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c * 32, r);
                tc::tmem_ld_wait();
                const int col0 = n0 + c * 32;
                if (TF32) {
                    if (row < p.M && col0 < p.N) {
                        const float* bias = reinterpret_cast<const float*>(p.bias);
                        if (bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __ldg(bias + col0 + j)));
                        }
                        const size_t off = (size_t)bi * p.y_batch_stride + (size_t)row * p.ldy + p.col_offset + col0;
                        for (int d = 0; d < p.n_outputs; ++d) {
                            float* dst = reinterpret_cast<float*>(p.Y[d]) + off;
                            if (col0 + 32 <= p.N && (off & 3) == 0) {
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    *reinterpret_cast<uint4*>(dst + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                            } else {
                                for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __uint_as_float(r[j]);
                            }
                        }
                    }
                    continue;
                }
                if (row < p.M && col0 < p.N) {
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float lo = __uint_as_float(r[2 * j]), hi = __uint_as_float(r[2 * j + 1]);
                        if (p.bias) {
                            const int cc = col0 + 2 * j;
                            if (cc < p.N) lo = __fadd_rn(lo, __uint_as_float((uint32_t)__ldg(p.bias + cc) << 16));
                            if (cc + 1 < p.N) hi = __fadd_rn(hi, __uint_as_float((uint32_t)__ldg(p.bias + cc + 1) << 16));
                        }
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(hi), "f"(lo));
                    }
                    const size_t off = (size_t)bi * p.y_batch_stride + (size_t)row * p.ldy + p.col_offset + col0;
                    for (int d = 0; d < p.n_outputs; ++d) {       // own buffer, then peers over NVLink
                        uint16_t* dst = p.Y[d] + off;
                        if (col0 + 32 <= p.N && (off & 7) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32 && col0 + j < p.N; ++j)
                                dst[j] = (uint16_t)((j & 1) ? (o[j >> 1] >> 16) : (o[j >> 1] & 0xFFFFu));
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(TEMPTY0 + 8u * acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) record_failure(p.status, 3);
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == mma_warp) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [rows, K] bf16 row-major tensor, zero fill outside; operand tiles: box_rows x 64 elements with the
// 128-byte swizzle; scale tiles (box_cols = 16): box_rows x 16 elements, rows of 32 bytes, no swizzle
int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows, int box_cols = BK) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == BK ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// [rows, K] fp32 row-major tensor, zero fill outside; operand tiles of box_rows x 32 elements (128 bytes), 128-byte swizzle
int make_map_f32(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 4};
    cuuint32_t box[2] = {(cuuint32_t)(BK / 2), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

// [rows, K] tensor of bytes (packed int8 codes), zero fill outside; tiles of box_rows x 64 bytes, no swizzle
int make_map_u8(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vq_set_error(VQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

int launch_gemm(bool fused, const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, cudaStream_t st, bool tf32 = false) {
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    if (p.batch < 1) p.batch = 1;
    const int n_tiles = p.tiles_m * p.tiles_n * p.batch;
    const int sms = vq_sm_count();
    const int grid = n_tiles < sms ? n_tiles : sms;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 256 + 1024;
    if ((int)smem > vq_max_smem_optin()) return vq_set_error(VQ_ERR_UNSUPPORTED, "device offers too little shared memory for the GEMM");
    if (tf32) {
        auto k = mx_gemm_kernel<false, true>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<grid, 192, smem, st>>>(tmA, tmB, p);
    } else if (fused) {
        auto k = mx_gemm_kernel<true>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<grid, (PRODUCER_WARPS_FUSED + 5) * 32, smem, st>>>(tmA, tmB, p);
    } else {
        auto k = mx_gemm_kernel<false>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<grid, 192, smem, st>>>(tmA, tmB, p);
    }
    VQ_LAUNCH_CHECK("mx_gemm_kernel");
    return 0;
}

}  // namespace

// for the convolution kernel (vq_conv_gemm.cu): operand map with the 128-byte swizzle over a [rows, K] bf16 matrix
int vq_make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
    return make_map(map, ptr, rows, K, box_rows);
}

extern "C" {

int vq_gemm_bf16_tn(const void* A, const void* B, const void* bias, void* Y, int64_t M, int64_t N, int64_t K,
                    int32_t* status, void* stream) {
    void* ys[1] = {Y};
    return vq_gemm_bf16_tn_scatter(A, B, bias, ys, 1, N, 0, M, N, K, status, stream);
}

int vq_gemm_bf16_tn_batched(const void* A, const void* B, void* Y, int64_t batch, int64_t M, int64_t N, int64_t K,
                            int a_shared, int b_shared, int32_t* status, void* stream) {
    const char* name = "vq_gemm_bf16_tn_batched";
    VQ_REQUIRE(batch >= 0 && M >= 0 && N >= 0 && K >= 0, "%s: negative size", name);
    if (batch == 0 || M == 0 || N == 0) return 0;
    VQ_REQUIRE(A && B && Y, "%s: null pointer", name);
    VQ_REQUIRE(K > 0 && K % 8 == 0, "%s: K must be a positive multiple of 8 (16-byte rows)", name);
    VQ_REQUIRE(batch * M < (1ll << 31) && batch * N < (1ll << 31) && K < (1ll << 31), "%s: batch * rows must be below 2^31", name);
    VQ_REQUIRE((uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0 && (uintptr_t)Y % 2 == 0, "%s: operands must be 16-byte aligned", name);
    const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
    VQ_REQUIRE(tiles * batch < (1ll << 31), "%s: too many output tiles", name);
    const int64_t rowsA = a_shared ? M : batch * M, rowsB = b_shared ? N : batch * N;
    CUtensorMap tmA, tmB;
    if (int rc = make_map(&tmA, A, rowsA, K, BM)) return rc;
    void* ys[1] = {Y};
    const char* tile = getenv("VOYAGER_B200_GEMM_TILE");
    if (M > 128 && !(tile && !strcmp(tile, "1cta"))) {
        if (int rc = make_map(&tmB, B, rowsB, K, 128)) return rc;
        return vq_gemm_pair_launch(tmA, tmB, ys, 1, N, 0, nullptr, M, N, K, status, (cudaStream_t)stream, nullptr, nullptr, nullptr,
                                   nullptr, false, (int)batch, a_shared ? 0 : M, b_shared ? 0 : N, M * N);
    }
    if (int rc = make_map(&tmB, B, rowsB, K, BN)) return rc;
    GemmParams p{};
    p.Y[0] = reinterpret_cast<uint16_t*>(Y);
    p.n_outputs = 1;
    p.ldy = N;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.batch = (int)batch;
    p.a_batch_rows = a_shared ? 0 : (int)M;
    p.b_batch_rows = b_shared ? 0 : (int)N;
    p.y_batch_stride = M * N;
    p.status = status;
    return launch_gemm(false, tmA, tmB, p, (cudaStream_t)stream);
}

int vq_gemm_f32_tn_batched(const void* A, const void* B, const void* bias, void* Y, int64_t batch, int64_t M, int64_t N,
                           int64_t K, int a_shared, int b_shared, int32_t* status, void* stream) {
    const char* name = "vq_gemm_f32_tn_batched";
    VQ_REQUIRE(batch >= 0 && M >= 0 && N >= 0 && K >= 0, "%s: negative size", name);
    if (batch == 0 || M == 0 || N == 0) return 0;
    VQ_REQUIRE(A && B && Y, "%s: null pointer", name);
    VQ_REQUIRE(K > 0 && K % 4 == 0, "%s: K must be a positive multiple of 4 (16-byte rows)", name);
    VQ_REQUIRE(batch * M < (1ll << 31) && batch * N < (1ll << 31) && K < (1ll << 31), "%s: batch * rows must be below 2^31", name);
    VQ_REQUIRE((uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0 && (uintptr_t)Y % 4 == 0, "%s: operands must be 16-byte aligned", name);
    VQ_REQUIRE(bias == nullptr || batch == 1, "%s: a bias goes with one problem only", name);
    const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
    VQ_REQUIRE(tiles * batch < (1ll << 31), "%s: too many output tiles", name);
    CUtensorMap tmA, tmB;
    if (int rc = make_map_f32(&tmA, A, a_shared ? M : batch * M, K, BM)) return rc;
    if (int rc = make_map_f32(&tmB, B, b_shared ? N : batch * N, K, BN)) return rc;
    GemmParams p{};
    p.Y[0] = reinterpret_cast<uint16_t*>(Y);
    p.n_outputs = 1;
    p.ldy = N;
    p.bias = reinterpret_cast<const uint16_t*>(bias);
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.batch = (int)batch;
    p.a_batch_rows = a_shared ? 0 : (int)M;
    p.b_batch_rows = b_shared ? 0 : (int)N;
    p.y_batch_stride = M * N;
    p.status = status;
    return launch_gemm(false, tmA, tmB, p, (cudaStream_t)stream, true);
}

int vq_gemm_bf16_tn_scatter(const void* A, const void* B, const void* bias, void* const* Ys, int n_outputs, int64_t ldy,
                            int64_t col_offset, int64_t M, int64_t N, int64_t K, int32_t* status, void* stream) {
    const char* name = "vq_gemm_bf16_tn_scatter";
    VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, "%s: negative size", name);
    if (M == 0 || N == 0) return 0;
    VQ_REQUIRE(Ys && n_outputs >= 1 && n_outputs <= MAX_OUTPUTS, "%s: 1..%d output buffers", name, MAX_OUTPUTS);
    VQ_REQUIRE(ldy >= col_offset + N && col_offset >= 0, "%s: the column range does not fit the output row", name);
    void* Y = Ys[0];
    for (int d = 0; d < n_outputs; ++d) VQ_REQUIRE(Ys[d] != nullptr, "%s: null output buffer %d", name, d);
    VQ_REQUIRE(A && B && Y, "%s: null pointer", name);
    VQ_REQUIRE(K > 0 && K % 8 == 0, "%s: K must be a positive multiple of 8 (16-byte rows)", name);
    VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: sizes must be below 2^31", name);
    VQ_REQUIRE((uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0 && (uintptr_t)Y % 2 == 0, "%s: operands must be 16-byte aligned", name);
    CUtensorMap tmA, tmB;
    if (int rc = make_map(&tmA, A, M, K, BM)) return rc;
    const char* tile = getenv("VOYAGER_B200_GEMM_TILE");       // "1cta" forces the one-CTA 128x256 tile
    if (M > 128 && !(tile && !strcmp(tile, "1cta"))) {
        if (int rc = make_map(&tmB, B, N, K, 128)) return rc;
        // several output buffers (peers): whole sub-tiles leave by tensor stores; VOYAGER_B200_SCATTER_STORES=rows keeps
        // the one-bulk-copy-per-row form
        CUtensorMap outs[MAX_OUTPUTS];
        const char* how = getenv("VOYAGER_B200_SCATTER_STORES");
        bool tiles = n_outputs > 1 && ldy % 8 == 0 && !(how && !strcmp(how, "rows"));
        for (int d = 0; d < n_outputs && tiles; ++d)
            if ((uintptr_t)Ys[d] % 16 || make_map(&outs[d], Ys[d], M, ldy, 128)) tiles = false;
        return vq_gemm_pair_launch(tmA, tmB, Ys, n_outputs, ldy, col_offset, bias, M, N, K, status, (cudaStream_t)stream, nullptr,
                                   nullptr, nullptr, nullptr, false, 1, 0, 0, 0, tiles ? outs : nullptr);
    }
    if (int rc = make_map(&tmB, B, N, K, BN)) return rc;
    GemmParams p{};
    for (int d = 0; d < n_outputs; ++d) p.Y[d] = reinterpret_cast<uint16_t*>(Ys[d]);
    p.n_outputs = n_outputs;
    p.ldy = ldy;
    p.col_offset = col_offset;
    p.bias = reinterpret_cast<const uint16_t*>(bias);
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.status = status;
    return launch_gemm(false, tmA, tmB, p, (cudaStream_t)stream);
}

int vq_linear_mx(const void* a_codes, const void* a_scale, const void* b_codes, const void* b_scale, const void* bias,
                 void* Y, int64_t M, int64_t N, int64_t K, int64_t block, int32_t* status, void* stream) {
    const char* name = "vq_linear_mx";
    VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, "%s: negative size", name);
    if (M == 0 || N == 0) return 0;
    VQ_REQUIRE(a_codes && a_scale && b_codes && b_scale && Y, "%s: null pointer", name);
    if (block != 32 || K % BK != 0 || K <= 0)
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: the fused kernel needs block 32 along K and K a multiple of %d", name, BK);
    VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: sizes must be below 2^31", name);
    VQ_REQUIRE((uintptr_t)a_codes % 16 == 0 && (uintptr_t)b_codes % 16 == 0, "%s: code tensors must be 16-byte aligned", name);
    CUtensorMap tmA, tmB;
    const char* tile = getenv("VOYAGER_B200_GEMM_TILE");
    if (M > 128 && K % 256 == 0 && (uintptr_t)a_scale % 16 == 0 && (uintptr_t)b_scale % 16 == 0 &&
        !(tile && !strcmp(tile, "1cta"))) {
        // CTA-pair kernel: codes and block scales arrive by TMA, eight warps per CTA dequantise in place
        CUtensorMap tmSA, tmSB;
        if (int rc = make_map(&tmA, a_codes, M, K, 128)) return rc;
        if (int rc = make_map(&tmB, b_codes, N, K, 128)) return rc;
        if (int rc = make_map(&tmSA, a_scale, M, K / 32, 128, 16)) return rc;
        if (int rc = make_map(&tmSB, b_scale, N, K / 32, 128, 16)) return rc;
        void* ys[1] = {Y};
        return vq_gemm_pair_launch(tmA, tmB, ys, 1, N, 0, bias, M, N, K, status, (cudaStream_t)stream, &tmSA, &tmSB, a_codes,
                                   b_codes);
    }
    memset(&tmA, 0, sizeof(tmA));
    memset(&tmB, 0, sizeof(tmB));
    GemmParams p{};
    p.Y[0] = reinterpret_cast<uint16_t*>(Y);
    p.n_outputs = 1;
    p.ldy = N;
    p.col_offset = 0;
    p.bias = reinterpret_cast<const uint16_t*>(bias);
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.status = status;
    p.a_codes = reinterpret_cast<const uint16_t*>(a_codes);
    p.a_scale = reinterpret_cast<const uint16_t*>(a_scale);
    p.b_codes = reinterpret_cast<const uint16_t*>(b_codes);
    p.b_scale = reinterpret_cast<const uint16_t*>(b_scale);
    p.blocks_per_row = (int)(K / 32);
    return launch_gemm(true, tmA, tmB, p, (cudaStream_t)stream);
}

int vq_linear_mx_packed(const int8_t* a_codes, const void* a_scale, const int8_t* b_codes, const void* b_scale,
                        const void* bias, void* Y, int64_t M, int64_t N, int64_t K, int64_t block, int32_t* status,
                        void* stream) {
    const char* name = "vq_linear_mx_packed";
    VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, "%s: negative size", name);
    if (M == 0 || N == 0) return 0;
    VQ_REQUIRE(a_codes && a_scale && b_codes && b_scale && Y, "%s: null pointer", name);
    if (block != 32 || K % 256 != 0 || K <= 0 || M <= 128)
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: needs block 32 along K, K a multiple of 256 and more than 128 rows", name);
    VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "%s: sizes must be below 2^31", name);
    VQ_REQUIRE((uintptr_t)a_codes % 16 == 0 && (uintptr_t)b_codes % 16 == 0 && (uintptr_t)a_scale % 16 == 0 &&
                   (uintptr_t)b_scale % 16 == 0, "%s: code and scale tensors must be 16-byte aligned", name);
    CUtensorMap tmA, tmB, tmSA, tmSB;
    if (int rc = make_map_u8(&tmA, a_codes, M, K, 128)) return rc;
    if (int rc = make_map_u8(&tmB, b_codes, N, K, 128)) return rc;
    if (int rc = make_map(&tmSA, a_scale, M, K / 32, 128, 16)) return rc;
    if (int rc = make_map(&tmSB, b_scale, N, K / 32, 128, 16)) return rc;
    void* ys[1] = {Y};
    return vq_gemm_pair_launch(tmA, tmB, ys, 1, N, 0, bias, M, N, K, status, (cudaStream_t)stream, &tmSA, &tmSB, nullptr, nullptr,
                               true);
}

}  // extern "C"
