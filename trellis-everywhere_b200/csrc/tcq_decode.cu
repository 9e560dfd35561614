// Decode kernels: packed code words or symbol streams -> reconstructed weights,
// plus symbol packing and codebook tabulation.  All are streaming kernels bounded
// by HBM bandwidth (4 bytes written per weight, K/8 or 8 bytes read).
//
// The state at step t is the 16-bit sliding window of the symbol stream
// (src/trellis/qtip.py:4-7), so every weight is decoded independently.
#include "tcq_traceback.cuh"

namespace tcq {

namespace {

// Packed decode.  Replaces lut[states2] (qtip.py:144), the wrapped decode of
// tests/test_qtip.py:55-67 and WGSL wz() (web/kernels.js:115-122): weight t is the
// codebook value of the window that starts at stream bit (255-t)*K; the window of
// the first few weights runs past the last word and continues at word 0.
// One thread decodes four consecutive weights and stores them as one float4.
template <int K>
__global__ void __launch_bounds__(256) tcq_decode_packed_kernel(const uint32_t* __restrict__ packed, long long n,
                                                               int codebook, float* __restrict__ dq) {
    constexpr uint32_t NW = Geo<K>::NWORDS;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one per 4 weights
    const long long tile = gid >> 6;
    if (tile >= n) return;
    const uint32_t t0 = uint32_t(gid & 63) * 4;
    const uint32_t* const p = packed + tile * NW;
    float o[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t bit = (kT - 1 - (t0 + i)) * K;
        const uint32_t j = bit >> 5, sh = bit & 31;
        const uint32_t w0 = __ldg(p + j);
        const uint32_t w1 = __ldg(p + (j + 1 == NW ? 0 : j + 1));
        const uint32_t win = __funnelshift_r(w0, w1, sh);      // (w1:w0) >> sh, low 32 bits
        o[i] = cb_value_rt(codebook, win & 0xFFFFu);
    }
    *reinterpret_cast<float4*>(dq + tile * kT + t0) = make_float4(o[0], o[1], o[2], o[3]);
}

// Symbol-stream decode (decode_recursive == decode_window, qtip.py:70-110).
// Thread per output; the window is rebuilt from the ceil(16/K) latest symbols and,
// near the start, from the surviving bits of the start state s0.
__global__ void __launch_bounds__(256) tcq_decode_symbols_kernel(const long long* __restrict__ bits, long long n,
                                                                long long T, int K, int codebook,
                                                                const long long* __restrict__ s0,
                                                                float* __restrict__ out) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n * T) return;
    const long long row = gid / T, t = gid - row * T;
    const int need = (kL + K - 1) / K;
    uint32_t s = 0;
    for (int j = need - 1; j >= 0; --j) {
        const long long idx = t - j;
        const uint32_t sym = idx >= 0 ? uint32_t(bits[row * T + idx]) : 0u;
        s = (s << K) | sym;
    }
    if (s0 != nullptr && (t + 1) * K < kL) s |= uint32_t(s0[row]) << ((t + 1) * K);
    out[gid] = cb_value_rt(codebook, s & 0xFFFFu);
}

// pack_bits_np (scripts/export_packed_8b.py:52-62): thread per output word.
__global__ void __launch_bounds__(256) tcq_pack_symbols_kernel(const long long* __restrict__ bits, long long n, int K,
                                                              uint32_t* __restrict__ packed) {
    const uint32_t NW = kT * K / 32;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n * NW) return;
    const long long tile = gid / NW;
    const uint32_t j = uint32_t(gid - tile * NW);
    uint32_t word = 0;
    for (uint32_t b = 0; b < 32; ++b) {
        const uint32_t p = 32 * j + b;
        const uint32_t t = (kT - 1) - p / K;
        word |= ((uint32_t(bits[tile * kT + t]) >> (p % K)) & 1u) << b;
    }
    packed[gid] = word;
}

__global__ void __launch_bounds__(256) tcq_codebook_lut_kernel(int codebook, float* __restrict__ lut) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < uint32_t(kStates)) lut[s] = cb_value_rt(codebook, s);
}

}  // namespace

cudaError_t launch_decode_packed(const uint32_t* packed, long long n, int K, int codebook, float* dq, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const unsigned grid = unsigned((n * 64 + 255) / 256);
    switch (K) {
        case 2: tcq_decode_packed_kernel<2><<<grid, 256, 0, stream>>>(packed, n, codebook, dq); break;
        case 3: tcq_decode_packed_kernel<3><<<grid, 256, 0, stream>>>(packed, n, codebook, dq); break;
        case 4: tcq_decode_packed_kernel<4><<<grid, 256, 0, stream>>>(packed, n, codebook, dq); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_decode_symbols(const long long* bits, long long n, long long T, int K, int codebook,
                                  const long long* s0, float* out, cudaStream_t stream) {
    if (n <= 0 || T <= 0) return cudaSuccess;
    const unsigned grid = unsigned((n * T + 255) / 256);
    tcq_decode_symbols_kernel<<<grid, 256, 0, stream>>>(bits, n, T, K, codebook, s0, out);
    return cudaGetLastError();
}

cudaError_t launch_pack_symbols(const long long* bits, long long n, int K, uint32_t* packed, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const unsigned grid = unsigned((n * (kT * K / 32) + 255) / 256);
    tcq_pack_symbols_kernel<<<grid, 256, 0, stream>>>(bits, n, K, packed);
    return cudaGetLastError();
}

cudaError_t launch_codebook_lut(int codebook, float* lut, cudaStream_t stream) {
    tcq_codebook_lut_kernel<<<kStates / 256, 256, 0, stream>>>(codebook, lut);
    return cudaGetLastError();
}

}  // namespace tcq
