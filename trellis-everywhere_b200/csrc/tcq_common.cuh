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
        // fp32(hi) + lo with the mixed-precision add of sm_100 (fp16 operand widened in the adder):
        // one instruction less than two conversions and an add; the sum is exact either way.
        float r;
        asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 fh;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.f32.f16 fh, hi;\n\tadd.rn.f32.f16 %0, lo, fh;\n\t}" : "=f"(r) : "r"(v));
        return r;
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

// ---- Blackwell packed-fp32 arithmetic -------------------------------------------------
// sm_100 executes add/sub/mul on two fp32 values held in a 64-bit register pair as ONE
// instruction (each half is an ordinary IEEE round-to-nearest operation, no flush to
// zero).  The fp32 lanes are not wider for it, but it costs one issue slot instead of
// two, and issue slots are what bounds the Viterbi step kernel.
using f32x2 = unsigned long long;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// Candidates of two predecessors at once: fl(fl(fl(w - v) * fl(w - v)) + c) per half.
// The final addition is written as fma(product, one2, c) with one2 = {1.0f, 1.0f} passed in
// at run time.  ptxas contracts a packed multiply that feeds a packed add into one fused
// multiply-add (single rounding) even when both carry .rn and -fmad=false is given, which
// changes path metrics by an ulp; a product that enters an fma as the MULTIPLICAND cannot
// be contracted, and x * 1 + c rounds exactly like x + c.
__device__ __forceinline__ f32x2 cand_cost2(f32x2 w2, f32x2 v2, f32x2 c2, f32x2 one2) {
    const f32x2 d = sub2(w2, v2);
    return fma2(mul2(d, d), one2, c2);
}

// Three-input minimum (one instruction on sm_100).
__device__ __forceinline__ float min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
template <int N> __device__ __forceinline__ float min_of(const float (&c)[N]);
template <> __device__ __forceinline__ float min_of<4>(const float (&c)[4]) { return fminf(min3(c[0], c[1], c[2]), c[3]); }
template <> __device__ __forceinline__ float min_of<8>(const float (&c)[8]) {
    return min3(min3(c[0], c[1], c[2]), min3(c[3], c[4], c[5]), fminf(c[6], c[7]));
}
template <> __device__ __forceinline__ float min_of<16>(const float (&c)[16]) {
    const float a = min3(min3(c[0], c[1], c[2]), min3(c[3], c[4], c[5]), min3(c[6], c[7], c[8]));
    const float b = min3(min3(c[9], c[10], c[11]), min3(c[12], c[13], c[14]), c[15]);
    return fminf(a, b);
}

// Conditional move "if (c == best) tag = value", the argmin scan's inner operation.
// Compare/select instructions issue at half the rate of fp32 arithmetic on sm_100, and the
// scan has one compare per candidate already, so the moves alternate between the two pipes:
//   * odd q: an ordinary select (compare/select pipe);
//   * even q: tag = c * zero + value as a predicated fma on the candidate itself, with
//     zero = 0.0f passed in at run time, which executes on the fp32 multiply-add pipe.  (It
//     must depend on a loop-varying register: one * value would be hoisted as a constant and
//     leave a predicated register move on the compare/select pipe.)  c is finite, so
//     c * 0 + value == value exactly.
__device__ __forceinline__ void take_if_equal_fma(float& tag, float c, float best, float zero, float value) {
    asm("{\n\t.reg .pred p;\n\tsetp.eq.f32 p, %1, %2;\n\t@p fma.rn.f32 %0, %1, %3, %4;\n\t}" : "+f"(tag) : "f"(c), "f"(best), "f"(zero), "f"(value));
}
// Q = candidates per successor.  With 8 or fewer, every other move is a select; with 16 the compare/select
// pipe is the busier one and only every fourth move stays there (measured: +1.4 % at K = 4, -0.5 % at K = 3).
// (At Q = 8, other splits were measured against 3 selects + 4 fmas: 2 + 5 -0.3 %, 1 + 6 -1.6 %, 0 + 7 -2.1 %, 5 + 2 -3.0 %.)
template <int Q>
__device__ __forceinline__ void take_if_equal_balanced(int q, float& tag, float c, float best, float zero, float value) {
    const bool on_select_pipe = Q >= 16 ? (q & 3) == 1 : (q & 1) != 0;
    if (on_select_pipe) tag = (c == best) ? value : tag;
    else take_if_equal_fma(tag, c, best, zero, value);
}

}  // namespace tcq
