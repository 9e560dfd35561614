// Shared definitions of the B200 trellis codec kernels: trellis geometry, the
// computed codebooks as device functions, and small helpers.
//
// Numerics contract (what makes the encoder bit-identical to the fp32 PyTorch
// dynamic programme of the reference, src/trellis/qtip.py:147-196):
//   * every fp32 operation of the path metric is an explicit round-to-nearest
//     intrinsic (__fsub_rn, __fmul_rn, __fadd_rn), so nothing is contracted into
//     a fused multiply-add, and the file is compiled with -fmad=false as well;
//   * "infinity" is FLT_MAX / 4 (bit pattern 0x7E7FFFFF), as in qtip.py:159;
//   * the minimum over the 2^K predecessors keeps the lowest index on ties.
#pragma once

#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace tcq {

constexpr int kL = 16;          // state bits
constexpr int kT = 256;         // weights per tile
constexpr int kStates = 1 << kL;
constexpr uint32_t kInfBits = 0x7E7FFFFFu;  // FLT_MAX / 4

enum : int { kCb1Mad = 0, kCb3Inst = 1, kCbMcg = 2 };

// Trellis geometry for K bits per weight.
template <int K>
struct Geo {
    static constexpr int Q = 1 << K;              // candidates per edge
    static constexpr int E = 1 << (kL - K);       // edges = length of the path-metric vector
    static constexpr int HN = E >> K;             // butterflies: Q predecessors -> Q successors
    static constexpr int ROWB = E * K / 8;        // bytes of packed backpointers per step
    static constexpr int NWORDS = kT * K / 32;    // packed code words per tile
};

// x(state) = state * MUL + ADD (mod 2^32) is the linear-congruential scramble that
// each codebook starts with; it is affine in the state, so kernels form it once
// per butterfly and add compile-time multiples of MUL for the other states.
template <int CB> struct CbLcg;
template <> struct CbLcg<kCb1Mad>  { static constexpr uint32_t MUL = 34038481u,   ADD = 76625530u; };  // qtip.py:35
template <> struct CbLcg<kCb3Inst> { static constexpr uint32_t MUL = 89226354u,   ADD = 64248484u; };  // qtip.py:43
template <> struct CbLcg<kCbMcg>   { static constexpr uint32_t MUL = 0xCBAC1FEDu, ADD = 0u; };         // qtip.py:51

// Codebook value from the scrambled word x.
//  1MAD  (qtip.py:36-37): y = sum of the four bytes; (y - 510) / 147.800537109375.
//        y < 1021, so y - 510 is formed exactly with the 2^23 magic-number trick, and
//        the division is a reciprocal multiply followed by one exact-residual
//        correction; that sequence equals IEEE division for all 1021 numerators
//        (checked exhaustively by the codebook tests).
//  3INST / MCG (qtip.py:44-45, 52-53): (x & 0x8FFF8FFF) ^ 0x3B603B60 read as two
//        binary16 values whose sum is taken in fp32 (it is exact there).
template <int CB>
__device__ __forceinline__ float cb_from_x(uint32_t x) {
    if constexpr (CB == kCb1Mad) {
        const uint32_t y = __dp4a(x, 0x01010101u, 0u);
        const float n = __fsub_rn(__uint_as_float(0x4B000000u | y), 8389118.0f);  // (2^23 + y) - (2^23 + 510)
        const float d = 147.800537109375f;
        const float r = 1.0f / 147.800537109375f;  // folded at compile time, correctly rounded
        const float a = __fmul_rn(n, r);
        const float res = __fmaf_rn(-a, d, n);
        return __fmaf_rn(res, r, a);
    } else {
        const uint32_t v = (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
        const __half2 h = *reinterpret_cast<const __half2*>(&v);
        const float2 f = __half22float2(h);
        return __fadd_rn(f.y, f.x);
    }
}

template <int CB>
__device__ __forceinline__ float cb_value(uint32_t state) {
    return cb_from_x<CB>(state * CbLcg<CB>::MUL + CbLcg<CB>::ADD);
}

__device__ __forceinline__ float cb_value_rt(int cb, uint32_t state) {
    switch (cb) {
        case kCb1Mad:  return cb_value<kCb1Mad>(state);
        case kCb3Inst: return cb_value<kCb3Inst>(state);
        default:       return cb_value<kCbMcg>(state);
    }
}

// Squared emission error plus predecessor metric, rounded after every operation.
__device__ __forceinline__ float cand_cost(float w, float v, float c) {
    const float d = __fsub_rn(w, v);
    return __fadd_rn(__fmul_rn(d, d), c);
}

}  // namespace tcq
