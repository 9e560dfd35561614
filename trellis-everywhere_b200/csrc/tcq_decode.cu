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
// One warp decodes one tile.  Lane l takes two runs of four weights, t = 4l .. 4l+3 and t = 128+4l .. 128+4l+3:
// a run's windows lie in 3K+16 <= 28 consecutive stream bits (two words, normalised to one by a funnel
// shift), and each of the warp's two store instructions then writes 512 contiguous bytes (whole sectors),
// where eight consecutive weights per lane would make every store cover half of each sector it touches
// (measured on 262 144 tiles: 4.45 -> 5.69 TB/s).  The stores are cache-streaming: the output is written
// once and not read back by this kernel, and keeping it out of the way of L2's resident set was worth
// another 20 % (6.6-7.2 TB/s, at the measured copy peak).
template <int K, int CB>
__global__ void __launch_bounds__(256) tcq_decode_packed_kernel(const uint32_t* __restrict__ packed, long long n,
                                                               float* __restrict__ dq) {
    constexpr uint32_t NW = Geo<K>::NWORDS;
    const long long tile = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (tile >= n) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t* const p = packed + tile * NW;
    float4* const out = reinterpret_cast<float4*>(dq + tile * kT);
#pragma unroll
    for (uint32_t run = 0; run < 2; ++run) {
        const uint32_t t_last = 128 * run + 4 * lane + 3;
        const uint32_t sb = (kT - 1 - t_last) * K;          // stream bit of the run's last weight
        const uint32_t word0 = sb >> 5, sh = sb & 31;
        const uint32_t w1 = word0 + 1 >= NW ? word0 + 1 - NW : word0 + 1;   // weight 0..3's windows wrap to word 0
        const uint32_t u = __funnelshift_r(__ldg(p + word0), __ldg(p + w1), sh);
        static_assert(3 * K + 16 <= 32, "a run of four windows fits one normalised word");
        float4 o;
        o.x = cb_value<CB>((u >> (3 * K)) & 0xFFFFu);
        o.y = cb_value<CB>((u >> (2 * K)) & 0xFFFFu);
        o.z = cb_value<CB>((u >> K) & 0xFFFFu);
        o.w = cb_value<CB>(u & 0xFFFFu);
        __stcs(out + 32 * run + lane, o);
    }
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
