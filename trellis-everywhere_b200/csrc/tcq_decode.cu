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
// One warp decodes one tile: lane l takes the eight weights t = 8l .. 8l+7, whose windows lie in
// 7K+16 consecutive stream bits (three words at most, loaded once), and stores them as two float4;
// the warp reads the tile's 32K bytes and writes its 1 KiB contiguously.
template <int K, int CB>
__global__ void __launch_bounds__(256) tcq_decode_packed_kernel(const uint32_t* __restrict__ packed, long long n,
                                                               float* __restrict__ dq) {
    constexpr uint32_t NW = Geo<K>::NWORDS;
    const long long tile = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (tile >= n) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t sb = (kT - 8 - 8 * lane) * K;            // stream bit of the lane's last weight (t = 8l + 7)
    const uint32_t word0 = sb >> 5, sh = sb & 31;
    const uint32_t* const p = packed + tile * NW;
    uint32_t v[3];
#pragma unroll
    for (uint32_t j = 0; j < 3; ++j) {
        const uint32_t wi = word0 + j;
        v[j] = __ldg(p + (wi >= NW ? wi - NW : wi));         // lane 0's windows wrap to word 0
    }
    const uint32_t u0 = __funnelshift_r(v[0], v[1], sh), u1 = __funnelshift_r(v[1], v[2], sh);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        constexpr int kMaxOff = 7 * K;                       // 28 at most: the window starts inside u0
        const int s = (7 - i) * K;
        static_assert(kMaxOff < 32, "window offsets must start in the first normalised word");
        const uint32_t win = (s + 16 <= 32) ? (u0 >> s) : __funnelshift_r(u0, u1, s);
        o[i] = cb_value<CB>(win & 0xFFFFu);
    }
    float4* const out = reinterpret_cast<float4*>(dq + tile * kT + 8 * lane);
    out[0] = make_float4(o[0], o[1], o[2], o[3]);
    out[1] = make_float4(o[4], o[5], o[6], o[7]);
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

namespace {
template <int K>
cudaError_t launch_decode_packed_k(const uint32_t* packed, long long n, int codebook, float* dq, cudaStream_t stream) {
    const unsigned grid = unsigned((n + 7) / 8);
    switch (codebook) {
        case kCb1Mad:  tcq_decode_packed_kernel<K, kCb1Mad><<<grid, 256, 0, stream>>>(packed, n, dq); break;
        case kCb3Inst: tcq_decode_packed_kernel<K, kCb3Inst><<<grid, 256, 0, stream>>>(packed, n, dq); break;
        case kCbMcg:   tcq_decode_packed_kernel<K, kCbMcg><<<grid, 256, 0, stream>>>(packed, n, dq); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_decode_packed(const uint32_t* packed, long long n, int K, int codebook, float* dq, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    switch (K) {
        case 2: return launch_decode_packed_k<2>(packed, n, codebook, dq, stream);
        case 3: return launch_decode_packed_k<3>(packed, n, codebook, dq, stream);
        case 4: return launch_decode_packed_k<4>(packed, n, codebook, dq, stream);
        default: return cudaErrorInvalidValue;
    }
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
