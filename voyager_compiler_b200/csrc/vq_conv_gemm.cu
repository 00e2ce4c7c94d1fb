// Convolution as an implicit GEMM on the 5th-generation tensor cores: no patch matrix in HBM.
//
//   Y[m, o] = sum over (i, j, c) of  X[n, ho * sh - ph + i * dh, wo * sw - pw + j * dw, g * Cg + c] * Wm[o, (i, j, c)]
//
// m = (n, ho, wo) runs over the output pixels, o over the output channels of group g.  The activation is
// channels-last (any pixel strides), bf16, optionally still to be multiplied by one scale per block of
// channels at every pixel (the layout `quantize_mx` along the channel axis produces); the weight is the
// decoded [O, kh * kw * Cp] matrix with every tap's channels padded to Cp = 64 * ceil(Cg / 64) (zeros).
//
// One persistent CTA per SM, output tile 128 pixels x BN channels, K step = 64 channels of one tap:
//   16 gather warps  in 4 sets, set s staging the k-steps s, s + 4, ... into stage s of the ring.  Each thread of a
//                    set owns 8 (pixel, 16-byte chunk) slots of the 128 x 64 A tile: it finds the pixels' window
//                    positions once per tile, then per k-step loads its chunks straight from the activation
//                    (zero outside the image or past the last channel), multiplies the block scale in (one bf16
//                    rounding per product, as `codes * scale` in bf16 gives) and stores them in the
//                    128-byte-swizzled K-major layout the MMA reads.  The proxy fence between the stores and
//                    the hand-over waits for the thread's loads, so a set has one step in flight: the four
//                    sets give the pipeline its depth;
//   1 weight warp    one thread issues the TMA tile load of the BN x 64 weight tile of the k-step;
//   1 MMA warp       one thread issues tcgen05.mma (bf16 x bf16 -> fp32) into a double-buffered accumulator
//                    in tensor memory and commits to mbarriers;
//   4 epilogue warps tcgen05.ld, bias, rounding to bf16, stores of [M, O] rows.
// full[s] counts the 4 warps of set s and the weight thread's expect_tx; every wait is bounded and a wait
// that runs out records a code in `status` and winds the CTA down.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "vq_common.cuh"
#include "vq_tc.cuh"

// vq_gemm.cu: tensor map over a [rows, K] bf16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle
int vq_make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows);

namespace {

constexpr int CM = 128, CK = 64;
constexpr int NSETS = 4, SET_WARPS = 4, SET_THREADS = SET_WARPS * 32;   // gather warps: NSETS sets, one per ring stage
constexpr int CSTAGES = NSETS;
constexpr int GATHER_WARPS = NSETS * SET_WARPS;
constexpr int SLOTS = CM * 8 / SET_THREADS;               // 8 chunks per gather thread per k-step
constexpr int CONV_THREADS = (GATHER_WARPS + 2 + 4) * 32;
constexpr long long CWAIT = 4000000000ll;                 // ~2 s of SM clocks

struct ConvParams {
    const uint16_t* x;
    int64_t sn, sh, sw;            // element strides of the NHWC activation (channel stride 1)
    const uint16_t* xs;            // optional block scales [N, H, W, ceil(C / block)] (last stride 1)
    int64_t ssn, ssh, ssw;
    int block_shift;               // log2(block), block >= 8
    int H, W;
    int groups, Cg, Og;            // channels per group, outputs per group
    int kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
    int cblocks;                   // 64-channel steps per tap
    int num_k;                     // kh * kw * cblocks
    int M, O;
    FastDiv div_wo, div_howo;
    int Wo, HoWo;
    uint16_t* y;
    const uint16_t* bias;
    int tiles_m, tiles_n;          // per group
    int32_t* status;
};

__device__ __forceinline__ void conv_fail(int32_t* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint4 mul_chunk(uint4 c, uint32_t s2) {
    uint4 o;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.x) : "r"(c.x), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.y) : "r"(c.y), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.z) : "r"(c.z), "r"(s2));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o.w) : "r"(c.w), "r"(s2));
    return o;
}

template <int BN>
__global__ void __launch_bounds__(CONV_THREADS, 1) conv_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
    constexpr int A_BYTES = CM * CK * 2, B_BYTES = BN * CK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;       // 128-byte swizzle atoms are 1024 bytes
    uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
    const uint32_t bar_base = base + CSTAGES * STAGE_BYTES;
    const uint32_t FULL0 = bar_base, EMPTY0 = bar_base + 8u * CSTAGES, TFULL0 = bar_base + 16u * CSTAGES,
                   TEMPTY0 = TFULL0 + 16u, SLOT = TEMPTY0 + 16u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int W_WARP = GATHER_WARPS, MMA_WARP = GATHER_WARPS + 1;
    const int tiles_per_group = p.tiles_m * p.tiles_n;
    const int n_tiles = tiles_per_group * p.groups;

    if (threadIdx.x == 0) {
        for (int s = 0; s < CSTAGES; ++s) {
            tc::mbar_init(FULL0 + 8u * s, SET_WARPS + 1);
            tc::mbar_init(EMPTY0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(TFULL0 + 8u * s, 1);
            tc::mbar_init(TEMPTY0 + 8u * s, 4);
        }
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmW);
    }
    if (warp == MMA_WARP) {
        tc::tmem_alloc(SLOT, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(SLOT));

    if (warp < GATHER_WARPS) {
        // ------------------------------------------------------------------ activation gather
        // Set s (SET_WARPS warps) stages the k-steps s, s + NSETS, ... of every tile, always into stage s of the
        // ring.  A step is: issue the loads, wait for the stage, store, proxy fence, arrive.  The fence waits for
        // the thread's own loads, so a set has one step in flight; the NSETS sets overlap theirs.
        const int set = warp / SET_WARPS;
        const int t = (warp - set * SET_WARPS) * 32 + lane;    // thread of the set
        const int ch = t & 7;                                  // this thread's 16-byte chunk of the 128-byte rows
        const int stage = set;
        uint32_t phase = 0;
        bool ok = true;
        int kbase = 0;                                         // k-steps of earlier tiles, modulo NSETS
        // the numbers every step uses, in registers
        const uint16_t* const x = p.x;
        const uint16_t* const xs = p.xs;
        const int H = p.H, W = p.W, sh = (int)p.sh, sw = (int)p.sw, ssh = (int)p.ssh, ssw = (int)p.ssw, dil_h = p.dil_h,
                  dil_w = p.dil_w, cblocks = p.cblocks, kw = p.kw, Cg = p.Cg, num_k = p.num_k, block_shift = p.block_shift;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int g = tile / tiles_per_group, rem = tile - g * tiles_per_group;
            const int m0 = (rem % p.tiles_m) * CM;
            // window origin of this thread's pixels (32-bit element offsets: the host checks the sizes)
            int pix_off[SLOTS], sc_off[SLOTS], hw0[SLOTS];
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                const int r = j * (SET_THREADS / 8) + (t >> 3);
                const uint32_t m = (uint32_t)(m0 + r);
                if (m < (uint32_t)p.M) {
                    const uint32_t n = fd_div(m, p.div_howo), hw = m - n * (uint32_t)p.HoWo;
                    const uint32_t ho = fd_div(hw, p.div_wo), wo = hw - ho * (uint32_t)p.Wo;
                    const int hi0 = (int)ho * p.stride_h - p.pad_h, wi0 = (int)wo * p.stride_w - p.pad_w;
                    hw0[j] = (hi0 << 16) | (wi0 & 0xFFFF);
                    pix_off[j] = (int)((int64_t)n * p.sn + (int64_t)hi0 * p.sh + (int64_t)wi0 * p.sw + (int64_t)g * p.Cg);
                    sc_off[j] = (int)((int64_t)n * p.ssn + (int64_t)hi0 * p.ssh + (int64_t)wi0 * p.ssw);
                } else {
                    hw0[j] = (int)0xC0000000;                  // row -16384: no tap brings it inside the image
                    pix_off[j] = 0;
                    sc_off[j] = 0;
                }
            }
            // first k-step of this tile that belongs to the set: global step numbers kbase + k are dealt round robin
            int k = (set - kbase + NSETS) % NSETS;
            kbase = (kbase + num_k) % NSETS;
            int tap = k / cblocks, cb = k - tap * cblocks;     // once per tile; afterwards the counters advance by NSETS steps
            int ti = tap / kw, tj = tap - ti * kw;
            for (; k < num_k; k += NSETS) {
                const int dh = ti * dil_h, dw = tj * dil_w;
                const int cch = cb * CK + ch * 8;              // first channel of this thread's chunk within the group
                const int tap_off = dh * sh + dw * sw + cch;
                const int tap_soff = dh * ssh + dw * ssw + ((g * Cg + cch) >> block_shift);
                const bool c_in = cch < Cg;
                // Loads first, nothing that consumes them: the SM issues in order, so an instruction that needs a
                // loaded value (a select against zero, the widening of a scale) would hold back the loads behind
                // it.  Chunks outside the image are loaded from offset 0 and zeroed when they are stored.
                uint4 c[SLOTS];
                uint32_t sraw[SLOTS];
                uint32_t valid = 0u;
#pragma unroll
                for (int j = 0; j < SLOTS; ++j) {
                    const int hi = (hw0[j] >> 16) + dh, wi = (int)(int16_t)(hw0[j] & 0xFFFF) + dw;
                    const bool in = (uint32_t)hi < (uint32_t)H && (uint32_t)wi < (uint32_t)W && c_in;
                    valid |= (in ? 1u : 0u) << j;
                    c[j] = __ldg(reinterpret_cast<const uint4*>(x + (in ? pix_off[j] + tap_off : 0)));
                    sraw[j] = xs ? (uint32_t)__ldg(xs + (in ? sc_off[j] + tap_soff : 0)) : 0u;
                }
                cb += NSETS;
                while (cb >= cblocks) {
                    cb -= cblocks;
                    if (++tj == kw) {
                        tj = 0;
                        ++ti;
                    }
                }
                if (lane == 0) ok = tc::mbar_wait_relaxed(EMPTY0 + 8u * stage, phase ^ 1u, CWAIT);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                uint8_t* st = smem + stage * STAGE_BYTES;
#pragma unroll
                for (int j = 0; j < SLOTS; ++j) {
                    const int r = j * (SET_THREADS / 8) + (t >> 3);
                    uint4 v = xs ? mul_chunk(c[j], sraw[j] * 0x00010001u) : c[j];
                    if (!((valid >> j) & 1u)) v = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(st + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
                }
                tc::fence_proxy_async();                      // generic-proxy stores -> visible to the MMA
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(FULL0 + 8u * stage);
                phase ^= 1u;
            }
        }
        if (!ok && lane == 0) conv_fail(p.status, 11);
    } else if (warp == W_WARP) {
        // ------------------------------------------------------------------ weight tiles
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int g = tile / tiles_per_group, rem = tile - g * tiles_per_group;
                const int row0 = g * p.Og + (rem / p.tiles_m) * BN;
                for (int k = 0; k < p.num_k; ++k) {
                    if (!tc::mbar_wait_relaxed(EMPTY0 + 8u * stage, phase ^ 1u, CWAIT)) { ok = false; break; }
                    tc::mbar_expect_tx(FULL0 + 8u * stage, B_BYTES);
                    tc::tma_load_2d(base + stage * STAGE_BYTES + A_BYTES, &tmW, k * CK, row0, FULL0 + 8u * stage);
                    if (++stage == CSTAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                conv_fail(p.status, 12);
                for (int s = 0; s < CSTAGES; ++s) tc::mbar_wait(FULL0 + 8u * s, 0, CWAIT >> 6);    // let copies in flight land
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_bf16_f32(CM, BN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                if (!tc::mbar_wait(TEMPTY0 + 8u * acc, acc_phase ^ 1u, CWAIT)) { ok = false; break; }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * 256u;
                for (int k = 0; k < p.num_k; ++k) {
                    if (!tc::mbar_wait(FULL0 + 8u * stage, phase, CWAIT)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
                    const uint64_t da = tc::smem_desc_k_sw128(sa), db = tc::smem_desc_k_sw128(sb);
#pragma unroll
                    for (int kk = 0; kk < CK / 16; ++kk)
                        tc::mma_f16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                    tc::mma_commit(EMPTY0 + 8u * stage);
                    if (++stage == CSTAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc::mma_commit(TFULL0 + 8u * acc);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) conv_fail(p.status, 13);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const int q = warp & 3;                                // the quarter of the tensor-memory lanes this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int g = tile / tiles_per_group, rem = tile - g * tiles_per_group;
            const int m0 = (rem % p.tiles_m) * CM, n0 = (rem / p.tiles_m) * BN;
            if (lane == 0) ok = tc::mbar_wait_relaxed(TFULL0 + 8u * acc, acc_phase, CWAIT);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256u;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c * 32, r);
                tc::tmem_ld_wait();
                const int col0 = n0 + c * 32;                  // within the group
                if (row < p.M && col0 < p.Og) {
                    uint32_t o[16];
                    const int gcol = g * p.Og + col0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float lo = __uint_as_float(r[2 * j]), hi = __uint_as_float(r[2 * j + 1]);
                        if (p.bias) {
                            const int cc = col0 + 2 * j;
                            if (cc < p.Og) lo = __fadd_rn(lo, __uint_as_float((uint32_t)__ldg(p.bias + gcol + 2 * j) << 16));
                            if (cc + 1 < p.Og) hi = __fadd_rn(hi, __uint_as_float((uint32_t)__ldg(p.bias + gcol + 2 * j + 1) << 16));
                        }
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(hi), "f"(lo));
                    }
                    const size_t off = (size_t)row * p.O + gcol;
                    uint16_t* dst = p.y + off;
                    if (col0 + 32 <= p.Og && (off & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.Og; ++j)
                            dst[j] = (uint16_t)((j & 1) ? (o[j >> 1] >> 16) : (o[j >> 1] & 0xFFFFu));
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(TEMPTY0 + 8u * acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) conv_fail(p.status, 14);
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, 512);
    }
}

template <int BN>
int launch_conv(const CUtensorMap& tmW, const ConvParams& p, int grid, cudaStream_t st) {
    const size_t smem = (size_t)CSTAGES * (CM * CK * 2 + BN * CK * 2) + 256 + 1024;
    if ((int)smem > vq_max_smem_optin()) return vq_set_error(VQ_ERR_UNSUPPORTED, "device offers too little shared memory for the convolution");
    auto k = conv_gemm_kernel<BN>;
    VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, CONV_THREADS, smem, st>>>(tmW, p);
    VQ_LAUNCH_CHECK("conv_gemm_kernel");
    return 0;
}

}  // namespace

extern "C" {

int64_t vq_conv2d_weight_columns(int64_t channels_per_group, int kh, int kw) {
    if (channels_per_group <= 0 || kh <= 0 || kw <= 0) return 0;
    return (int64_t)kh * kw * ((channels_per_group + CK - 1) / CK * CK);
}

int vq_conv2d_bf16(const void* x, int64_t N, int64_t H, int64_t W, int64_t C, int64_t sn, int64_t sh, int64_t sw,
                   const void* x_scale, int64_t block, int64_t ssn, int64_t ssh, int64_t ssw, const void* wmat, int64_t O,
                   int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                   const void* bias, void* y, int32_t* status, void* stream) {
    const char* name = "vq_conv2d_bf16";
    VQ_REQUIRE(N >= 0 && H >= 1 && W >= 1 && C >= 1 && O >= 0, "%s: bad tensor sizes", name);
    VQ_REQUIRE(kh >= 1 && kw >= 1 && stride_h >= 1 && stride_w >= 1 && dil_h >= 1 && dil_w >= 1 && pad_h >= 0 && pad_w >= 0,
               "%s: bad window", name);
    VQ_REQUIRE(groups >= 1 && C % groups == 0 && O % groups == 0, "%s: channels must divide into the groups", name);
    const int64_t Cg = C / groups, Og = O / groups;
    const int64_t Ho = (H + 2 * pad_h - (int64_t)dil_h * (kh - 1) - 1) / stride_h + 1;
    const int64_t Wo = (W + 2 * pad_w - (int64_t)dil_w * (kw - 1) - 1) / stride_w + 1;
    VQ_REQUIRE(H + 2 * pad_h >= (int64_t)dil_h * (kh - 1) + 1 && W + 2 * pad_w >= (int64_t)dil_w * (kw - 1) + 1,
               "%s: the window is larger than the padded image", name);
    const int64_t M = N * Ho * Wo;
    if (M == 0 || O == 0) return 0;
    VQ_REQUIRE(x && wmat && y, "%s: null pointer", name);
    if (Cg % 8 != 0 || sn % 8 || sh % 8 || sw % 8 || (uintptr_t)x % 16 || (uintptr_t)wmat % 16 || (uintptr_t)y % 16)
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: channels per group, pixel strides (multiples of 8) and 16-byte alignment", name);
    VQ_REQUIRE(M < (1ll << 31) && O < (1ll << 31) && H < (1 << 24) && W < (1 << 24), "%s: sizes must be below 2^31", name);
    if (H + pad_h + (int64_t)dil_h * kh >= 16384 || W + pad_w + (int64_t)dil_w * kw >= 16384)
        return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: images of up to 16383 pixels a side", name);
    {
        // the gather addresses the activation (and its scales) by 32-bit element offsets
        const int64_t reach = (N - 1) * sn + (H - 1 + pad_h) * sh + (W - 1 + pad_w) * sw + C;
        const int64_t sreach = x_scale ? (N - 1) * ssn + (H - 1 + pad_h) * ssh + (W - 1 + pad_w) * ssw + C : 0;
        if (reach >= (1ll << 31) || sreach >= (1ll << 31) || sn < 0 || sh < 0 || sw < 0 || ssn < 0 || ssh < 0 || ssw < 0)
            return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: the activation must span fewer than 2^31 elements, strides non-negative", name);
    }
    int block_shift = 0;
    if (x_scale) {
        while ((1ll << block_shift) < block) ++block_shift;
        if ((1ll << block_shift) != block || block < 8)
            return vq_set_error(VQ_ERR_UNSUPPORTED, "%s: the activation's blocks must be a power of two of at least 8 channels", name);
    }
    ConvParams p{};
    p.x = reinterpret_cast<const uint16_t*>(x);
    p.sn = sn; p.sh = sh; p.sw = sw;
    p.xs = reinterpret_cast<const uint16_t*>(x_scale);
    p.ssn = ssn; p.ssh = ssh; p.ssw = ssw;
    p.block_shift = block_shift;
    p.H = (int)H; p.W = (int)W;
    p.groups = groups; p.Cg = (int)Cg; p.Og = (int)Og;
    p.kh = kh; p.kw = kw; p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w;
    p.dil_h = dil_h; p.dil_w = dil_w;
    p.cblocks = (int)((Cg + CK - 1) / CK);
    p.num_k = kh * kw * p.cblocks;
    p.M = (int)M; p.O = (int)O;
    p.Wo = (int)Wo; p.HoWo = (int)(Ho * Wo);
    p.div_wo = make_fastdiv((uint32_t)Wo);
    p.div_howo = make_fastdiv((uint32_t)(Ho * Wo));
    p.y = reinterpret_cast<uint16_t*>(y);
    p.bias = reinterpret_cast<const uint16_t*>(bias);
    p.status = status;
    const int64_t Kw = vq_conv2d_weight_columns(Cg, kh, kw);
    // tile width: the narrowest that covers a group's outputs; a wide problem with few tiles is cut finer
    const int sms = vq_sm_count();
    p.tiles_m = (int)((M + CM - 1) / CM);
    int bn = Og <= 64 ? 64 : (Og <= 128 ? 128 : 256);
    if (bn == 256 && (int64_t)p.tiles_m * ((Og + 255) / 256) * groups < sms) bn = 128;
    p.tiles_n = (int)((Og + bn - 1) / bn);
    const int64_t n_tiles = (int64_t)p.tiles_m * p.tiles_n * groups;
    VQ_REQUIRE(n_tiles < (1ll << 31), "%s: too many output tiles", name);
    CUtensorMap tmW;
    if (int rc = vq_make_operand_map(&tmW, wmat, O, Kw, bn)) return rc;
    const int grid = (int)(n_tiles < sms ? n_tiles : sms);
    cudaStream_t st = (cudaStream_t)stream;
    if (bn == 64) return launch_conv<64>(tmW, p, grid, st);
    if (bn == 128) return launch_conv<128>(tmW, p, grid, st);
    return launch_conv<256>(tmW, p, grid, st);
}

}  // extern "C"
