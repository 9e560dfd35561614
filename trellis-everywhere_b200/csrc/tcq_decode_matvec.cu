// Decode-matvec: y = Zq x straight from packed trellis codes, Zq never materialised.
//
// The consumer side of the packed format: what the reference's runtime does in its
// DECODE_MATMUL shader (web/kernels.js:105-128), where one thread walks a whole output
// row and decodes every weight with wz() (window at stream bit (255-t)*K of tile
// (row/16)*tiles_in + col/16, t = (row%16)*16 + col%16).  The incoherence-processing
// fold around it (web/packed.js:163-182) stays with the caller.
//
// Work split here: one CTA per tile row (16 output rows), eight warps striding over the
// column tiles.  A half-warp owns one tile per iteration, lane i its row i: the 16
// weights of that row sit in 15K+16 consecutive stream bits, fetched as two or three
// words, and every window is a compile-time shift of those.  The 16 x values a tile
// needs are the same for the 16 lanes of the half-warp (broadcast loads, L1 resident).
// Partial sums stay in registers; the two half-warps meet in one shuffle and the eight
// warps in shared memory, in a fixed order, so results are reproducible run to run.
//
// Bound: instruction issue, not HBM.  A weight costs about seven instructions to decode
// (funnel shift, mask, multiply, and/xor, two conversions/adds) plus one FMA per
// right-hand side, three of them on the half-rate integer pipe, i.e. about 20 weights per
// clock per SM; the K/8 bytes per weight that this pulls from HBM is a third of what the
// memory system delivers.  Up to four right-hand sides share one decode.
#include "tcq_traceback.cuh"

namespace tcq {

namespace {

constexpr int kMvWarps = 8;

template <int K, int CB, int M>
__global__ void __launch_bounds__(kMvWarps * 32)
tcq_decode_matvec_kernel(const uint32_t* __restrict__ packed, int tiles_in, const float* __restrict__ x, long long ldx,
                         int m, float* __restrict__ y, long long ldy) {
    constexpr int NW = Geo<K>::NWORDS;
    constexpr int WN = (K == 2) ? 2 : 3;                    // words that hold one tile row's 15K+16 bits
    __shared__ float red[kMvWarps][M][16];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = lane & 15, half = lane >> 4;
    const uint32_t sb = uint32_t(240 - 16 * i) * K;          // stream bit of this row's last weight (t = 16i + 15)
    const uint32_t word0 = sb >> 5, sh = sb & 31;            // sh is 0, or 16 for even rows at K = 3
    const uint32_t* const row_base = packed + (long long)blockIdx.x * tiles_in * NW;

    float acc[M];
#pragma unroll
    for (int j = 0; j < M; ++j) acc[j] = 0.0f;

    for (int c = 2 * warp + half; c < tiles_in; c += 2 * kMvWarps) {
        const uint32_t* const p = row_base + (long long)c * NW;
        uint32_t v[WN];
#pragma unroll
        for (int j = 0; j < WN; ++j) {
            const uint32_t wi = word0 + j;
            v[j] = __ldg(p + (wi >= uint32_t(NW) ? wi - NW : wi));       // the first row's window wraps to word 0
        }
        if constexpr (K == 3) {
#pragma unroll
            for (int j = 0; j + 1 < WN; ++j) v[j] = __funnelshift_r(v[j], v[j + 1], sh);
            v[WN - 1] >>= sh;
        }
        float4 xr[M][4];
#pragma unroll
        for (int j = 0; j < M; ++j) {
            const float4* const xp = reinterpret_cast<const float4*>(x + (long long)(j < m ? j : 0) * ldx + 16 * c);
#pragma unroll
            for (int q = 0; q < 4; ++q) xr[j][q] = __ldg(xp + q);
        }
#pragma unroll
        for (int col = 0; col < 16; ++col) {
            const int off = (15 - col) * K;
            const int wd = off >> 5, s = off & 31;
            const uint32_t win = (s + 16 <= 32) ? (v[wd] >> s) : __funnelshift_r(v[wd], v[wd + 1 < WN ? wd + 1 : wd], s);
            const float val = cb_value<CB>(win & 0xFFFFu);
#pragma unroll
            for (int j = 0; j < M; ++j) {
                const float4 q4 = xr[j][col >> 2];
                const float xv = (col & 3) == 0 ? q4.x : (col & 3) == 1 ? q4.y : (col & 3) == 2 ? q4.z : q4.w;
                acc[j] = __fmaf_rn(val, xv, acc[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < M; ++j) {
        acc[j] += __shfl_xor_sync(0xFFFFFFFFu, acc[j], 16);
        if (half == 0) red[warp][j][i] = acc[j];
    }
    __syncthreads();
    if (threadIdx.x < 16 * M) {
        const int j = threadIdx.x >> 4, r = threadIdx.x & 15;
        float s = red[0][j][r];
#pragma unroll
        for (int w = 1; w < kMvWarps; ++w) s += red[w][j][r];
        if (j < m) y[(long long)j * ldy + 16ll * blockIdx.x + r] = s;
    }
}

template <int K, int CB>
cudaError_t launch_m(const uint32_t* packed, int tiles_out, int tiles_in, const float* x, long long ldx, int m, float* y,
                     long long ldy, cudaStream_t stream) {
    const dim3 grid(tiles_out), block(kMvWarps * 32);
    if (m == 1)      tcq_decode_matvec_kernel<K, CB, 1><<<grid, block, 0, stream>>>(packed, tiles_in, x, ldx, m, y, ldy);
    else if (m == 2) tcq_decode_matvec_kernel<K, CB, 2><<<grid, block, 0, stream>>>(packed, tiles_in, x, ldx, m, y, ldy);
    else             tcq_decode_matvec_kernel<K, CB, 4><<<grid, block, 0, stream>>>(packed, tiles_in, x, ldx, m, y, ldy);
    return cudaGetLastError();
}

template <int K>
cudaError_t launch_cb(int codebook, const uint32_t* packed, int tiles_out, int tiles_in, const float* x, long long ldx, int m,
                      float* y, long long ldy, cudaStream_t stream) {
    switch (codebook) {
        case kCb1Mad:  return launch_m<K, kCb1Mad>(packed, tiles_out, tiles_in, x, ldx, m, y, ldy, stream);
        case kCb3Inst: return launch_m<K, kCb3Inst>(packed, tiles_out, tiles_in, x, ldx, m, y, ldy, stream);
        case kCbMcg:   return launch_m<K, kCbMcg>(packed, tiles_out, tiles_in, x, ldx, m, y, ldy, stream);
        default:       return cudaErrorInvalidValue;
    }
}

}  // namespace

// y[j][row] = sum_col Zq[row][col] * x[j][col] for j < m; right-hand sides go four at a time.
cudaError_t launch_decode_matvec(const uint32_t* packed, long long n_out, long long k_in, int K, int codebook, const float* x,
                                 long long ldx, int m, float* y, long long ldy, cudaStream_t stream) {
    if (n_out <= 0 || k_in <= 0 || m <= 0) return cudaSuccess;
    const int tiles_out = int(n_out / 16), tiles_in = int(k_in / 16);
    for (int j0 = 0; j0 < m; j0 += 4) {
        const int mj = m - j0 < 4 ? m - j0 : 4;
        cudaError_t err;
        switch (K) {
            case 2: err = launch_cb<2>(codebook, packed, tiles_out, tiles_in, x + j0 * ldx, ldx, mj, y + j0 * ldy, ldy, stream); break;
            case 3: err = launch_cb<3>(codebook, packed, tiles_out, tiles_in, x + j0 * ldx, ldx, mj, y + j0 * ldy, ldy, stream); break;
            case 4: err = launch_cb<4>(codebook, packed, tiles_out, tiles_in, x + j0 * ldx, ldx, mj, y + j0 * ldy, ldy, stream); break;
            default: return cudaErrorInvalidValue;
        }
        if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
}

}  // namespace tcq
