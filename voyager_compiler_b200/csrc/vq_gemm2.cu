// CTA-pair variant of the TMA-fed GEMM: two CTAs of a cluster compute one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128-column half of B
// (32 KB per k-step instead of 48 KB), the pair's leader issues the MMAs for both, every CTA keeps
// 128 rows x 256 columns of the accumulator (double buffered) in its tensor memory and runs its own
// epilogue.  Per SM this writes and reads a third less shared memory per flop than the one-CTA
// 128 x 256 tile, which is bound by the shared-memory data pipe.
//
// Synchronisation (all waits bounded):
//   full[s]    leader's barrier; the leader arms it with the byte count of BOTH CTAs' tile loads,
//              whose completions are all counted on it
//   empty[s]   one per CTA; the leader's tcgen05.commit arrives on both once the MMAs have read stage s
//   tfull[a]   one per CTA; commit arrives on both when accumulator a is complete
//   tempty[a]  leader's barrier, 8 arrivals: the 4 epilogue warps of each CTA
// Epilogue: each thread owns one accumulator row; it stages 128 columns of bf16 in shared memory and
// sends them with one asynchronous bulk copy per output buffer (256 bytes each: own memory and, for
// the column-parallel linear, every peer GPU's copy of Y over NVLink).
#include <cuda.h>

#include <cstring>

#include "vq_common.cuh"
#include "vq_tc.cuh"

namespace {

constexpr int PM = 128;            // rows of A per CTA (pair: 256)
constexpr int PNH = 128;           // columns of B per CTA (pair: 256)
constexpr int PN = 256;
constexpr int PK = 64;
constexpr int PSTAGES = 5;
constexpr int PA_BYTES = PM * PK * 2, PB_BYTES = PNH * PK * 2, PSTAGE_BYTES = PA_BYTES + PB_BYTES;
// epilogue staging: 128 rows x 128 columns of bf16, rows padded by 16 bytes against bank conflicts
constexpr int OUT_COLS = 128, OUT_ROW_BYTES = OUT_COLS * 2 + 16, OUT_BYTES = PM * OUT_ROW_BYTES;
// fused variant: block scales arrive in groups of 8 k-steps: 128 rows x 16 scales (32 bytes per row)
// for A and for B, double buffered
constexpr int SC_GROUP = 8, SC_TILE = 128 * 32, SC_BUF = 2 * SC_TILE, SC_BUFS = 2;
constexpr long long PWAIT = 4000000000ll;
constexpr int P_MAX_OUT = 8;

struct PairParams {
    uint16_t* Y[P_MAX_OUT];
    int n_outputs;
    int64_t ldy, col_offset;
    const uint16_t* bias;
    int M, N, K;
    int tiles_m, tiles_n;      // in units of 256 x 256
    int batch;                 // plain variant: independent problems over flattened [batch * rows, K] operands
    int a_batch_rows, b_batch_rows;   // rows between consecutive batches of A / B (0: shared operand)
    int64_t y_batch_stride;    // elements between consecutive outputs
    int bulk_ok;               // output rows are 16-byte aligned: the epilogue may use bulk stores
    int tma_out;               // tensor maps of the output buffers are given: whole 128 x 64 sub-tiles leave by one TMA store each
    int32_t* status;
    int blocks_per_row;        // fused variant: the operand maps cover the CODES, two more maps the [rows, K/32] scales
    const uint16_t* a_codes;   // register-staged variant: the code tensors themselves, [M, K] and [N, K]
    const uint16_t* b_codes;
};

// tensor maps of up to P_MAX_OUT output buffers ([M, ldy] bf16, boxes of 128 rows x 64 columns, 128-byte swizzle)
struct OutMaps {
    CUtensorMap m[P_MAX_OUT];
};

// shared -> global tile store through a tensor map (rows and columns outside the tensor are dropped)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1), "r"(src_smem)
                 : "memory");
}

// shared -> global asynchronous bulk copy of `bytes` (multiple of 16) issued by one thread
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void record_fail(int32_t* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

// FUSED: the tile loads bring quantized codes; eight extra warps per CTA multiply them by their block
// scales in place (shared memory -> registers -> shared memory, one bf16 rounding per product) before
// the stage is handed to the MMA issuer.  Extra barrier raw[s] (per CTA): completion of the CTA's own
// tile loads; full[s] then counts one arrival per CTA of the pair instead of bytes.
// FUSED == 2: the eight warps fetch the codes themselves with coalesced 16-byte global loads (one
// k-step ahead, in registers), multiply and store straight into the swizzled operand layout: the
// operand ring sees one write and one read per byte, as in the unfused kernel, instead of the
// TMA write + read + write + read of the in-place variant, which is bound by the shared-memory pipe.
// FUSED == 3: the codes are PACKED int8 (one byte per element).  TMA brings 128 x 64-byte tiles into a
// raw ring of 4 stages; the eight warps turn every byte into bf16(code * scale) with a sign-extending
// byte permute, an integer add that plants the value in the significand of 1.5 * 2^23, and one fma
// against the block scale (exact), and write the 128-byte-swizzled operand ring (3 stages).  Per
// k-step and CTA the shared memory sees 16 KB + 16 KB + 32 KB + 32 KB instead of 4 x 32 KB, and HBM /
// L2 half the operand bytes.
template <int FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FUSED ? 448 : 192, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmSA, const __grid_constant__ CUtensorMap tmSB,
                    const __grid_constant__ OutMaps outs, const PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sc_base = base + PSTAGES * PSTAGE_BYTES;       // fused: block-scale tiles, one pair per stage
    const uint32_t out_base = sc_base + (FUSED ? SC_BUFS * SC_BUF : 0);   // epilogue staging buffer
    const uint32_t bar_base = out_base + OUT_BYTES;
    const uint32_t FULL0 = bar_base, EMPTY0 = bar_base + 8u * PSTAGES, TFULL0 = bar_base + 16u * PSTAGES,
                   TEMPTY0 = TFULL0 + 16u, SLOT = TEMPTY0 + 16u, RAW0 = SLOT + 8u,
                   SCF0 = RAW0 + 8u * PSTAGES, SCE0 = SCF0 + 8u * SC_BUFS, ABORT = SCE0 + 8u * SC_BUFS,
                   RAWE0 = ABORT + 8u,       // packed variant: "raw stage free" barriers
                   EPI_OK = RAWE0 + 8u * PSTAGES;   // tensor-store epilogue: outcome of the accumulator wait, shared by its four warps

    constexpr int OST = FUSED == 3 ? 3 : PSTAGES;            // operand ring stages
    constexpr int RST = 4;                                   // packed variant: raw ring stages (16 KB each)
    constexpr uint32_t RAW_TILE = 128u * 64u, RAW_STAGE = 2u * RAW_TILE;
    const uint32_t raw_base = base + OST * PSTAGE_BYTES;     // 3 x 32 KB + 4 x 16 KB = the 5 x 32 KB of the other variants
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int num_k = (p.K + PK - 1) / PK;
    const int tiles_per_batch = p.tiles_m * p.tiles_n;
    const int n_tiles = tiles_per_batch * p.batch;

    if (threadIdx.x == 0) {
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(ABORT), "r"(0u) : "memory");
        for (int s = 0; s < PSTAGES; ++s) {
            tc::mbar_init(FULL0 + 8u * s, FUSED ? 2 : 1);
            tc::mbar_init(EMPTY0 + 8u * s, 1);
            tc::mbar_init(RAW0 + 8u * s, 1);
            tc::mbar_init(RAWE0 + 8u * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(TFULL0 + 8u * s, 1);
            tc::mbar_init(TEMPTY0 + 8u * s, 8);
            tc::mbar_init(SCF0 + 8u * s, 1);
            tc::mbar_init(SCE0 + 8u * s, 8);
        }
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmA);
        tc::prefetch_tensormap(&tmB);
    }
    if (warp == 1) {
        tc::tmem_alloc_pair(SLOT, 512);
        tc::tmem_relinquish_pair();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();          // both CTAs' barriers are initialised before either touches the other's
    tc::tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(SLOT));

    if (warp == 0) {
        // ------------------------------------------------------------------ tile loads (both CTAs)
        if (lane == 0) {
            int stage = 0, rs = 0;
            uint32_t phase = 0, group = 0, rphase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += npairs) {
                const int bi = tile / tiles_per_batch, rem = tile - bi * tiles_per_batch;
                const int m0 = bi * p.a_batch_rows + (rem % p.tiles_m) * 256 + (int)rank * PM;
                const int n0 = bi * p.b_batch_rows + (rem / p.tiles_m) * PN + (int)rank * PNH;
                for (int k = 0; k < num_k; ++k) {
                    if (FUSED && (k % SC_GROUP) == 0) {
                        // block scales of the next 8 k-steps (16 per row) into the free scale buffer
                        const uint32_t b = group & 1u, ph = (group >> 1) & 1u;
                        if (!tc::mbar_wait(SCE0 + 8u * b, ph ^ 1u, PWAIT)) { ok = false; break; }
                        tc::mbar_expect_tx(SCF0 + 8u * b, SC_BUF);
                        tc::tma_load_2d(sc_base + b * SC_BUF, &tmSA, k * 2, m0, SCF0 + 8u * b);
                        tc::tma_load_2d(sc_base + b * SC_BUF + SC_TILE, &tmSB, k * 2, n0, SCF0 + 8u * b);
                        ++group;
                    }
                    if (FUSED == 2) continue;                 // the codes are fetched by the staging warps
                    if (FUSED == 3) {                         // packed codes into the raw ring
                        if (!tc::mbar_wait(RAWE0 + 8u * rs, rphase ^ 1u, PWAIT)) { ok = false; break; }
                        tc::mbar_expect_tx(RAW0 + 8u * rs, RAW_STAGE);
                        tc::tma_load_2d(raw_base + rs * RAW_STAGE, &tmA, k * PK, m0, RAW0 + 8u * rs);
                        tc::tma_load_2d(raw_base + rs * RAW_STAGE + RAW_TILE, &tmB, k * PK, n0, RAW0 + 8u * rs);
                        if (++rs == RST) { rs = 0; rphase ^= 1u; }
                        continue;
                    }
                    if (!tc::mbar_wait_cluster(EMPTY0 + 8u * stage, phase ^ 1u, PWAIT)) { ok = false; break; }
                    if (FUSED == 1) {
                        tc::mbar_expect_tx(RAW0 + 8u * stage, PSTAGE_BYTES);
                        tc::tma_load_2d(base + stage * PSTAGE_BYTES, &tmA, k * PK, m0, RAW0 + 8u * stage);
                        tc::tma_load_2d(base + stage * PSTAGE_BYTES + PA_BYTES, &tmB, k * PK, n0, RAW0 + 8u * stage);
                    } else {
                        const uint32_t leader_full = tc::map_to_cta(FULL0 + 8u * stage, 0);
                        if (rank == 0) tc::mbar_expect_tx(FULL0 + 8u * stage, 2 * PSTAGE_BYTES);
                        tc::tma_load_2d_pair(base + stage * PSTAGE_BYTES, &tmA, k * PK, m0, leader_full);
                        tc::tma_load_2d_pair(base + stage * PSTAGE_BYTES + PA_BYTES, &tmB, k * PK, n0, leader_full);
                    }
                    if (++stage == OST) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) record_fail(p.status, 11);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = tc::idesc_bf16_f32(256, PN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += npairs) {
                if (!tc::mbar_wait_cluster(TEMPTY0 + 8u * acc, acc_phase ^ 1u, PWAIT)) { ok = false; break; }
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * PN;
                for (int k = 0; k < num_k; ++k) {
                    if (!tc::mbar_wait_cluster(FULL0 + 8u * stage, phase, PWAIT)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = base + stage * PSTAGE_BYTES, sb = sa + PA_BYTES;
                    const uint64_t da = tc::smem_desc_k_sw128(sa), db = tc::smem_desc_k_sw128(sb);
#pragma unroll
                    for (int kk = 0; kk < PK / 16; ++kk)
                        tc::mma_f16_pair(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (k | kk) != 0 ? 1u : 0u);
                    tc::mma_commit_pair(EMPTY0 + 8u * stage);
                    if (++stage == OST) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc::mma_commit_pair(TFULL0 + 8u * acc);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) record_fail(p.status, 12);
        }
    } else if (FUSED == 3 && warp >= 6) {
        // ------------------------------------------------------------------ packed int8 codes -> bf16 operands (8 warps per CTA)
        // warps 0..3 convert the 128 A rows, warps 4..7 the 128 B rows; one warp instruction covers
        // 4 rows: lane -> (row lane / 8, 8-element chunk lane % 8): 8 raw bytes in, 16 operand bytes out
        const int t = (warp - 6) * 32 + lane;
        const bool is_b = t >= 128;
        const int wrow0 = ((t >> 5) & 3) * 32 + (lane >> 3);
        const uint32_t c = (uint32_t)lane & 7u;
        const uint32_t leader_full_base = tc::map_to_cta(FULL0, 0);
        int stage = 0, rs = 0;
        uint32_t phase = 0, rphase = 0, group = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles; tile += npairs) {
            for (int k = 0; k < num_k; ++k) {
                bool good = true;
                if (lane == 0) {
                    uint32_t aborted;
                    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(aborted) : "r"(ABORT));
                    good = aborted == 0u;
                    if (good && (k % SC_GROUP) == 0) good = tc::mbar_wait(SCF0 + 8u * (group & 1u), (group >> 1) & 1u, PWAIT);
                    if (good) good = tc::mbar_wait(RAW0 + 8u * rs, rphase, PWAIT);
                    if (good) good = tc::mbar_wait_cluster(EMPTY0 + 8u * stage, phase ^ 1u, PWAIT);
                    if (!good) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(ABORT), "r"(1u) : "memory");
                }
                good = __shfl_sync(0xFFFFFFFFu, good, 0);
                ok &= good;
                const uint32_t sc_addr = sc_base + (group & 1u) * SC_BUF + (is_b ? SC_TILE : 0) + (uint32_t)(k % SC_GROUP) * 4u + (c >> 2) * 2u;
                const uint32_t in_addr = raw_base + rs * RAW_STAGE + (is_b ? RAW_TILE : 0) + c * 8u;
                const uint32_t st_addr = base + stage * PSTAGE_BYTES + (is_b ? PA_BYTES : 0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t r = (uint32_t)(wrow0 + 4 * i);
                    uint32_t w0, w1, sc;
                    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(in_addr + r * 64u));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sc) : "r"(sc_addr + r * 32u));
                    const float sf = __uint_as_float(sc << 16);
                    const float c0 = __fmul_rn(-12582912.0f, sf);          // exact: 1.5 * 2^23 times an 8-bit significand
                    uint32_t o[4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t w = h ? w1 : w0;
                        float f[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // sign-extend byte j, plant it in the significand of 1.5 * 2^23: the float 12582912 + v
                            uint32_t v;
                            asm("prmt.b32 %0, %1, %1, %2;" : "=r"(v) : "r"(w), "r"((uint32_t)(((j | 8) * 0x1110) | j)));
                            f[j] = __fmaf_rn(__uint_as_float(v + 0x4B400000u), sf, c0);     // = v * sf, exact
                        }
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[2 * h]) : "f"(f[1]), "f"(f[0]));
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[2 * h + 1]) : "f"(f[3]), "f"(f[2]));
                    }
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(st_addr + r * 128u + ((c ^ (r & 7u)) << 4)),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                }
                tc::fence_proxy_async();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (t == 0) {
                    tc::mbar_arrive_cluster(leader_full_base + 8u * stage);
                    tc::mbar_arrive(RAWE0 + 8u * rs);
                }
                if ((k % SC_GROUP) == SC_GROUP - 1 || k == num_k - 1) {      // done with this scale buffer
                    if (lane == 0) tc::mbar_arrive(SCE0 + 8u * (group & 1u));
                    ++group;
                }
                if (++stage == OST) { stage = 0; phase ^= 1u; }
                if (++rs == RST) { rs = 0; rphase ^= 1u; }
            }
        }
        if (!ok && lane == 0) record_fail(p.status, 16);
    } else if (FUSED == 2 && warp >= 6) {
        // ------------------------------------------------------------------ register-staged dequantisation (8 warps per CTA)
        // warps 0..3 stage the 128 A rows, warps 4..7 the 128 B rows of this CTA; one warp instruction
        // moves 4 rows x 128 bytes: lane -> (row lane / 8, 16-byte chunk lane % 8)
        const int t = (warp - 6) * 32 + lane;
        const bool is_b = t >= 128;
        const int wrow0 = ((t >> 5) & 3) * 32 + (lane >> 3);
        const uint32_t c = (uint32_t)lane & 7u;
        const uint16_t* gbase = is_b ? p.b_codes : p.a_codes;
        const int nrows = is_b ? p.N : p.M;
        const int my_tiles = pair < n_tiles ? (n_tiles - pair + npairs - 1) / npairs : 0;
        const int total = my_tiles * num_k;                      // num_k is a multiple of 4 here
        const uint32_t leader_full_base = tc::map_to_cta(FULL0, 0);
        int stage = 0;
        uint32_t phase = 0, group = 0;
        bool ok = true;
        auto issue = [&](uint32_t (&buf)[8][4], int step) {
            const int tile = pair + (step / num_k) * npairs, k = step % num_k;
            const int row0 = (is_b ? (tile / p.tiles_m) * PN + (int)rank * PNH : (tile % p.tiles_m) * 256 + (int)rank * PM) + wrow0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int row = row0 + 4 * i;
                if (row < nrows) {
                    const uint16_t* g = gbase + (size_t)row * p.K + (size_t)k * PK + c * 8u;
                    asm volatile("ld.global.nc.v4.b32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(buf[i][0]), "=r"(buf[i][1]), "=r"(buf[i][2]), "=r"(buf[i][3]) : "l"(g));
                } else {
                    buf[i][0] = buf[i][1] = buf[i][2] = buf[i][3] = 0u;     // rows outside the matrix contribute zeros
                }
            }
        };
        // A wait that runs out sets the CTA's abort word; from then on the eight warps skip their waits
        // but keep meeting on the named barrier, so that none of them is left behind at it.
        auto process = [&](uint32_t (&buf)[8][4], int step) -> bool {
            const int k = step % num_k;
            bool good = true;
            if (lane == 0) {
                uint32_t aborted;
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(aborted) : "r"(ABORT));
                good = aborted == 0u;
                if (good && (k % SC_GROUP) == 0) good = tc::mbar_wait(SCF0 + 8u * (group & 1u), (group >> 1) & 1u, PWAIT);
                if (good) good = tc::mbar_wait_cluster(EMPTY0 + 8u * stage, phase ^ 1u, PWAIT);
                if (!good) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(ABORT), "r"(1u) : "memory");
            }
            good = __shfl_sync(0xFFFFFFFFu, good, 0);
            const uint32_t sc_addr = sc_base + (group & 1u) * SC_BUF + (is_b ? SC_TILE : 0) + (uint32_t)(k % SC_GROUP) * 4u + (c >> 2) * 2u;
            const uint32_t st_addr = base + stage * PSTAGE_BYTES + (is_b ? PA_BYTES : 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t r = (uint32_t)(wrow0 + 4 * i);
                uint32_t sc;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sc) : "r"(sc_addr + r * 32u));
                const uint32_t s2 = sc * 0x00010001u;
#pragma unroll
                for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(buf[i][j]) : "r"(s2));
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(st_addr + r * 128u + ((c ^ (r & 7u)) << 4)),
                             "r"(buf[i][0]), "r"(buf[i][1]), "r"(buf[i][2]), "r"(buf[i][3]) : "memory");
            }
            tc::fence_proxy_async();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (t == 0) tc::mbar_arrive_cluster(leader_full_base + 8u * stage);
            if ((k % SC_GROUP) == SC_GROUP - 1 || k == num_k - 1) {      // done with this scale buffer
                if (lane == 0) tc::mbar_arrive(SCE0 + 8u * (group & 1u));
                ++group;
            }
            if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
            return good;
        };
        uint32_t b0[8][4], b1[8][4];
        if (total > 0) issue(b0, 0);
        for (int step = 0; step < total; step += 2) {
            issue(b1, step + 1);
            ok &= process(b0, step);
            if (step + 2 < total) issue(b0, step + 2);
            ok &= process(b1, step + 1);
        }
        if (!ok && lane == 0) record_fail(p.status, 15);
    } else if (FUSED == 1 && warp >= 6) {
        // ------------------------------------------------------------------ in-place dequantisation (8 warps per CTA)
        // Two groups of four warps take alternate k-steps, so that two stages are being rewritten at a
        // time: in group g (the steps with k % 2 == g) thread r owns row r of the A tile and row r of
        // the B tile of this CTA.
        const int t = (warp - 6) * 32 + lane;
        const int g = t >> 7, r = t & 127;
        int stage = 0;
        uint32_t phase = 0, group = 0;
        bool ok = true;
        const uint32_t leader_full_base = tc::map_to_cta(FULL0, 0);
        for (int tile = pair; tile < n_tiles; tile += npairs) {
            for (int k = 0; k < num_k; ++k) {
                const int group_end = ((k / SC_GROUP) + 1) * SC_GROUP < num_k ? ((k / SC_GROUP) + 1) * SC_GROUP : num_k;
                if ((k & 1) == g) {
                    bool good = true;
                    if (lane == 0) {
                        uint32_t aborted;
                        asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(aborted) : "r"(ABORT));
                        good = aborted == 0u;
                        // the first step this group sees of a scale group waits for the scales
                        if (good && (k % SC_GROUP) == g) good = tc::mbar_wait(SCF0 + 8u * (group & 1u), (group >> 1) & 1u, PWAIT);
                        if (good) good = tc::mbar_wait(RAW0 + 8u * stage, phase, PWAIT);
                        if (!good) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(ABORT), "r"(1u) : "memory");
                    }
                    good = __shfl_sync(0xFFFFFFFFu, good, 0);
                    ok &= good;
#pragma unroll
                    for (int op = 0; op < 2; ++op) {                 // this row of the A tile, then of the B tile
                        // the row's two block scales for this k-step (rows outside the matrix were zero filled)
                        uint32_t sc;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc)
                                     : "r"(sc_base + (group & 1u) * SC_BUF + (op ? SC_TILE : 0) + (uint32_t)r * 32u + (uint32_t)(k % SC_GROUP) * 4u));
                        const uint32_t s_lo = (sc & 0xFFFFu) * 0x00010001u, s_hi = (sc >> 16) * 0x00010001u;
                        const uint32_t row_addr = base + stage * PSTAGE_BYTES + (op ? PA_BYTES : 0) + (uint32_t)r * 128u;
                        uint32_t v[8][4];
                        // logical chunk c sits at physical chunk c ^ (r & 7) (128-byte swizzle); walking the
                        // logical index keeps the 8 lanes of a quarter-warp on 8 different bank groups
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(v[c][0]), "=r"(v[c][1]), "=r"(v[c][2]), "=r"(v[c][3])
                                         : "r"(row_addr + (uint32_t)((c ^ (r & 7)) << 4)));
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint32_t s2 = (c >> 2) ? s_hi : s_lo;
#pragma unroll
                            for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v[c][j]) : "r"(s2));
                        }
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(row_addr + (uint32_t)((c ^ (r & 7)) << 4)),
                                         "r"(v[c][0]), "r"(v[c][1]), "r"(v[c][2]), "r"(v[c][3]) : "memory");
                    }
                    tc::fence_proxy_async();
                    // one cluster-scope arrival per CTA and k-step: the group's warps meet on a named barrier first
                    if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                    else asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (r == 0) tc::mbar_arrive_cluster(leader_full_base + 8u * stage);
                    // this warp's last step inside the scale group: release the scale buffer
                    if (k + 2 >= group_end && lane == 0) tc::mbar_arrive(SCE0 + 8u * (group & 1u));
                }
                if (k + 1 == group_end) ++group;
                if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok && lane == 0) record_fail(p.status, 14);
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps per CTA)
        const int q = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += npairs) {
            const int bi = tile / tiles_per_batch, rem = tile - bi * tiles_per_batch;
            const int m0 = (rem % p.tiles_m) * 256 + (int)rank * PM, n0 = (rem / p.tiles_m) * PN;
            const size_t ybase = (size_t)bi * p.y_batch_stride;
            if (p.tma_out) {
                // the four warps meet at a named barrier further down, so they must agree on going on: one thread waits
                // for the accumulator and tells the others
                if (warp == 2 && lane == 0) {
                    const bool good = tc::mbar_wait_cluster(TFULL0 + 8u * acc, acc_phase, PWAIT);
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(EPI_OK), "r"(good ? 1u : 0u) : "memory");
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                uint32_t good;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(good) : "r"(EPI_OK));
                ok = good != 0u;
                asm volatile("bar.sync 2, 128;" ::: "memory");   // everyone has read the word before the next tile rewrites it
            } else {
                if (lane == 0) ok = tc::mbar_wait_cluster(TFULL0 + 8u * acc, acc_phase, PWAIT);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            }
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * PN;
            const int rloc = q * 32 + lane;                                // row inside this CTA's 128 rows
            const uint32_t my_row = out_base + (uint32_t)rloc * OUT_ROW_BYTES;
#pragma unroll 1
            for (int c = 0; c < PN / 32; ++c) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c * 32, r);
                tc::tmem_ld_wait();
                const int col0 = n0 + c * 32;
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
                const int half0 = n0 + (c >> 2) * OUT_COLS;                 // first column of this 128-column half
                const bool bulk = p.bulk_ok && half0 + OUT_COLS <= p.N;      // whole half inside the matrix
                if (bulk && p.tma_out) {
                    // The four epilogue warps stage the half as two sub-tiles of 128 rows x 64 columns in the 128-byte
                    // swizzled layout of the output maps' boxes; one thread then sends each sub-tile to every output
                    // buffer (own memory and the peers') with ONE tensor store: 4 stores per buffer and tile instead of
                    // a 256-byte bulk copy per row and half.  Rows past the end of the matrix are dropped by the store.
                    const bool issuer = warp == 2 && lane == 0;
                    if ((c & 3) == 0) {
                        if (issuer) bulk_wait_read();            // the stores of the previous half have read the buffer
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                    }
                    const uint32_t sub = out_base + ((uint32_t)(c & 3) >> 1) * (128u * 128u) + (uint32_t)rloc * 128u;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t ch = (uint32_t)(c & 1) * 4u + (uint32_t)j;
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(sub + ((ch ^ ((uint32_t)rloc & 7u)) << 4)), "r"(o[4 * j]),
                                     "r"(o[4 * j + 1]), "r"(o[4 * j + 2]), "r"(o[4 * j + 3]) : "memory");
                    }
                    if ((c & 3) == 3) {
                        tc::fence_proxy_async();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (issuer) {
                            const int x0 = (int)p.col_offset + half0, y0 = m0;
                            for (int d = 0; d < p.n_outputs; ++d) {
                                tma_store_2d(&outs.m[d], out_base, x0, y0);
                                tma_store_2d(&outs.m[d], out_base + 128u * 128u, x0 + 64, y0);
                            }
                            bulk_commit();
                        }
                    }
                } else if (bulk) {
                    // every thread stages only its own row and later copies only its own row, so the
                    // only ordering needed is with its own earlier bulk reads of that row
                    if ((c & 3) == 0) bulk_wait_read();
                    const uint32_t dsts = my_row + (uint32_t)(c & 3) * 64u;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dsts + 16u * j), "r"(o[4 * j]), "r"(o[4 * j + 1]),
                                     "r"(o[4 * j + 2]), "r"(o[4 * j + 3]) : "memory");
                    if ((c & 3) == 3) {
                        tc::fence_proxy_async();
                        if (row < p.M) {
                            const size_t off = ybase + (size_t)row * p.ldy + p.col_offset + half0;
                            for (int d = 0; d < p.n_outputs; ++d) bulk_store(p.Y[d] + off, my_row, OUT_COLS * 2);
                        }
                        bulk_commit();
                    }
                } else if (row < p.M && col0 < p.N) {
                    const size_t off = ybase + (size_t)row * p.ldy + p.col_offset + col0;
                    for (int d = 0; d < p.n_outputs; ++d) {
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
            if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_cta(TEMPTY0 + 8u * acc, 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) record_fail(p.status, 13);
        bulk_wait_all();             // this thread's output copies have landed before the CTA may exit
    }

    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();          // neither CTA frees tensor memory or exits while the other may still signal it
    if (warp == 1) {
        tc::tc_fence_after();
        tc::tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace

// Launches the CTA-pair GEMM.  The tensor maps must have 128-row boxes for both operands.  With
// a_scale / b_scale the maps cover code tensors and dequantisation happens inside the kernel.
int vq_gemm_pair_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, void* const* Ys, int n_outputs, int64_t ldy,
                        int64_t col_offset, const void* bias, int64_t M, int64_t N, int64_t K, int32_t* status,
                        cudaStream_t st, const CUtensorMap* tmSA, const CUtensorMap* tmSB, const void* a_codes,
                        const void* b_codes, bool packed_codes, int batch, int64_t a_batch_rows, int64_t b_batch_rows,
                        int64_t y_batch_stride, const CUtensorMap* out_maps) {
    const bool fused = tmSA != nullptr && tmSB != nullptr;
    // VOYAGER_B200_FUSED_STAGING=regs selects the register-staged variant (measured slower: one k-step
    // of global loads in flight per thread does not cover the L2 latency); default: TMA + in-place multiply
    const char* staging = getenv("VOYAGER_B200_FUSED_STAGING");
    const bool regs = fused && a_codes && b_codes && staging && !strcmp(staging, "regs");
    PairParams p{};
    for (int d = 0; d < n_outputs; ++d) p.Y[d] = reinterpret_cast<uint16_t*>(Ys[d]);
    p.n_outputs = n_outputs;
    p.ldy = ldy;
    p.col_offset = col_offset;
    p.bias = reinterpret_cast<const uint16_t*>(bias);
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.tiles_m = (int)((M + 255) / 256);
    p.tiles_n = (int)((N + PN - 1) / PN);
    p.batch = batch;
    p.a_batch_rows = (int)a_batch_rows;
    p.b_batch_rows = (int)b_batch_rows;
    p.y_batch_stride = y_batch_stride;
    p.status = status;
    p.bulk_ok = (ldy % 8 == 0 && col_offset % 8 == 0 && y_batch_stride % 8 == 0) ? 1 : 0;
    for (int d = 0; d < n_outputs; ++d)
        if ((uintptr_t)Ys[d] % 16) p.bulk_ok = 0;
    p.blocks_per_row = (int)(K / 32);
    OutMaps outs;
    memset(&outs, 0, sizeof(outs));
    if (out_maps && p.bulk_ok && batch == 1) {
        for (int d = 0; d < n_outputs; ++d) outs.m[d] = out_maps[d];
        p.tma_out = 1;
    }
    const int n_tiles = p.tiles_m * p.tiles_n * batch;
    const int sms = vq_sm_count();
    int pairs = sms / 2;
    if (n_tiles < pairs) pairs = n_tiles;
    const size_t smem = (size_t)PSTAGES * PSTAGE_BYTES + (fused ? SC_BUFS * SC_BUF : 0) + OUT_BYTES + 256 + 1024;
    if ((int)smem > vq_max_smem_optin()) return vq_set_error(VQ_ERR_UNSUPPORTED, "device offers too little shared memory for the pair GEMM");
    p.a_codes = reinterpret_cast<const uint16_t*>(a_codes);
    p.b_codes = reinterpret_cast<const uint16_t*>(b_codes);
    if (fused && packed_codes) {
        auto k = mx_gemm_pair_kernel<3>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<pairs * 2, 448, smem, st>>>(tmA, tmB, *tmSA, *tmSB, outs, p);
    } else if (regs) {
        auto k = mx_gemm_pair_kernel<2>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<pairs * 2, 448, smem, st>>>(tmA, tmB, *tmSA, *tmSB, outs, p);
    } else if (fused) {
        auto k = mx_gemm_pair_kernel<1>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<pairs * 2, 448, smem, st>>>(tmA, tmB, *tmSA, *tmSB, outs, p);
    } else {
        auto k = mx_gemm_pair_kernel<0>;
        VQ_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k<<<pairs * 2, 192, smem, st>>>(tmA, tmB, tmA, tmB, outs, p);
    }
    VQ_LAUNCH_CHECK("mx_gemm_pair_kernel");
    return 0;
}
