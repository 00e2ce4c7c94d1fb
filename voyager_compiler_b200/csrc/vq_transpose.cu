// Decode + transpose of the right operand of matmul_mx / of a "ck" linear weight.
//
// Upstream hands `aten.matmul` a right operand in [.., K, N] order whose block scales run along K
// (ops/quantized.py:389-406); the tensor-core GEMM of this library wants both operands K-major
// ([rows, K]).  This kernel forms code * scale (one bf16 rounding, what `dequantize` produces) and
// writes it transposed, [batch, N, K], in the same pass, so putting the operand into GEMM order
// costs no traffic beyond the decode that has to happen anyway.
//
// 64 x 64 tiles through shared memory; every thread owns 2 x 2 elements: it reads two 32-bit
// words (rows k, k+1; columns n, n+1), multiplies by the two scales of its columns and regroups
// the four values into two words that are contiguous along K.  Loads and stores are 128-byte
// segments per warp.  HBM bound: 2 B read + 2 B written per element (+ scales).
#include "vq_common.cuh"

namespace {

constexpr int TT = 64;          // tile edge in elements

struct TransposeParams {
    const uint16_t* in;         // [batch, K, N]
    const uint16_t* scale;      // [batch, scale_rows, N] or null
    uint16_t* out;              // [batch, N, K]
    int K, N, block, scale_rows;
    int tiles_k, tiles_n;
    int64_t n_tiles;            // batch * tiles_k * tiles_n
};

__global__ void __launch_bounds__(256) dequant_transpose_kernel(const TransposeParams p) {
    __shared__ uint32_t tile[TT][TT / 2 + 1];        // [n][k pair], padded
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_batch = p.tiles_k * p.tiles_n;
    for (int64_t t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
        const int b = (int)(t / per_batch), rem = (int)(t - (int64_t)b * per_batch);
        const int k0 = (rem / p.tiles_n) * TT, n0 = (rem % p.tiles_n) * TT;
        const uint16_t* in = p.in + (size_t)b * p.K * p.N;
        const uint16_t* sc = p.scale ? p.scale + (size_t)b * p.scale_rows * p.N : nullptr;
        uint16_t* out = p.out + (size_t)b * p.N * p.K;
        const int n = n0 + 2 * lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kp = warp + 8 * i;             // k pair inside the tile
            const int k = k0 + 2 * kp;
            uint32_t w0 = 0u, w1 = 0u;
            if (n < p.N) {
                if (k < p.K) w0 = __ldcs(reinterpret_cast<const uint32_t*>(in + (size_t)k * p.N + n));
                if (k + 1 < p.K) w1 = __ldcs(reinterpret_cast<const uint32_t*>(in + (size_t)(k + 1) * p.N + n));
                if (sc) {
                    // rows k and k + 1 share a block (k even, block even)
                    const uint32_t s2 = __ldg(reinterpret_cast<const uint32_t*>(sc + (size_t)(k / p.block) * p.N + n));
                    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(w0) : "r"(s2));
                    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(w1) : "r"(s2));
                }
            }
            // {in[k][n], in[k+1][n]} and {in[k][n+1], in[k+1][n+1]}
            tile[2 * lane][kp] = __byte_perm(w0, w1, 0x5410);
            tile[2 * lane + 1][kp] = __byte_perm(w0, w1, 0x7632);
        }
        __syncthreads();
        const int k = k0 + 2 * lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int nn = warp + 8 * i;
            if (n0 + nn < p.N && k < p.K)            // K is even: a pair never straddles the end
                __stcs(reinterpret_cast<uint32_t*>(out + (size_t)(n0 + nn) * p.K + k), tile[nn][lane]);
        }
        __syncthreads();
    }
}

}  // namespace

extern "C" int vq_dequantize_transpose(const void* in, const void* scale, int64_t batch, int64_t K, int64_t N, int64_t block,
                                       int64_t scale_rows, void* out, void* stream) {
    const char* name = "vq_dequantize_transpose";
    VQ_REQUIRE(batch >= 0 && K >= 0 && N >= 0, "%s: negative size", name);
    if (batch == 0 || K == 0 || N == 0) return 0;
    VQ_REQUIRE(in && out, "%s: null pointer", name);
    VQ_REQUIRE(K % 2 == 0 && N % 2 == 0, "%s: K and N must be even (32-bit accesses)", name);
    VQ_REQUIRE((uintptr_t)in % 4 == 0 && (uintptr_t)out % 4 == 0 && (uintptr_t)scale % 4 == 0, "%s: tensors must be 4-byte aligned", name);
    VQ_REQUIRE(K < (1ll << 31) && N < (1ll << 31), "%s: sizes must be below 2^31", name);
    if (scale) {
        VQ_REQUIRE(block > 0 && block % 2 == 0, "%s: the block size must be even", name);
        VQ_REQUIRE(scale_rows >= (K + block - 1) / block, "%s: the scale has too few rows for K / block", name);
    }
    TransposeParams p{};
    p.in = reinterpret_cast<const uint16_t*>(in);
    p.scale = reinterpret_cast<const uint16_t*>(scale);
    p.out = reinterpret_cast<uint16_t*>(out);
    p.K = (int)K; p.N = (int)N; p.block = (int)(scale ? block : 2); p.scale_rows = (int)scale_rows;
    p.tiles_k = (int)((K + TT - 1) / TT);
    p.tiles_n = (int)((N + TT - 1) / TT);
    p.n_tiles = batch * p.tiles_k * p.tiles_n;
    const int64_t cap = (int64_t)vq_sm_count() * 8;
    const int blocks = (int)(p.n_tiles < cap ? p.n_tiles : cap);
    dequant_transpose_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p);
    VQ_LAUNCH_CHECK("dequant_transpose_kernel");
    return 0;
}
