// Viterbi step kernel: the forward (add-compare-select) sweep of one pass of the
// tail-biting encoder over a batch of independent 256-weight tiles.
//
// It replaces the 256-iteration PyTorch loop of src/trellis/qtip.py:177-182 and the
// Triton program src/trellis/viterbi_triton.py:24-78.
//
// Work decomposition (K bits per weight, Q = 2^K, E = 2^(16-K) edges):
//   new[h*Q + l] = min_q  old[q*HN + h] + (w_t - codebook[q*E + h*Q + l])^2 ,  HN = E/Q
// so the step is HN independent "butterflies", each reading Q path metrics (stride
// HN) and writing Q contiguous ones.  All 65536 codebook values are used exactly
// once per step and do not depend on the tile or on t, so one CTA advances G tiles
// in lock step and computes each codebook value once for all G of them, in
// registers, from the state number (no table).
//
//   * one persistent CTA per SM; a CTA owns groups of G consecutive tiles;
//   * path metrics live in shared memory, double buffered: [2][G][E] fp32;
//   * a work item is (butterfly h, chunk of LU successors); thread i takes items
//     i, i+NT, ... so that a warp reads 32 consecutive h (conflict-free LDS);
//   * the argmin q (K bits) of every edge is packed into a shared-memory row of
//     E*K/8 bytes per tile (edge e at bit e*K), double buffered, and the row of
//     step t-1 is streamed to HBM with coalesced 128-bit stores while step t
//     computes;
//   * one __syncthreads per step.
//
// Inner loop, per (successor, tile): the Q candidates are formed two at a time with
// packed fp32 sub/mul/add (f32x2), their minimum with three-input min, and the argmin
// as "lowest q whose candidate equals the minimum" with conditional moves, split between
// the compare/select pipe and the fp32 pipe, that build argmin * 2^(l*K) as an exact float;
// the tags of an item's successors are summed and converted to the packed backpointer bits once.  Per candidate that is about 1.5
// (arithmetic) + 0.5 (min) + 2 (compare, conditional move) issue slots, plus the
// shared codebook evaluation.
//
// Shared memory: 2*G*E*4 + 2*G*E*K/8 + G*1024 bytes (K=3, G=3: 217 KiB of the
// 227 KiB a CTA may use).
#pragma once

#include "tcq_common.cuh"

namespace tcq {

// ForwardArgs::flags
constexpr int kFwdResetStatus = 1;   // clear the status word at kernel start (the first launch of a call only)
constexpr int kFwdCheckFinite = 2;   // flag NaN / infinite weights in the status word

struct ForwardArgs {
    const float* w;          // [n,256] tiles, or (ld > 0) a 16-row block of a row-major matrix
    const float* w_add;      // nullptr, or a second operand of the same layout: the kernel encodes fl(w + w_add)
    long long ld;            // 0: tiles.  > 0: weight t of tile i is w[(t & 15) * ld + 16 * i + (t >> 4)], the LDLQ
                             //    row-block layout of src/trellis/ldlq.py:138-140 (16 input channels x n_out)
    long long n;             // tiles in this launch
    const int* overlap;      // [n] forced first/last edge, or nullptr (unconstrained, metrics start at 0)
    int roll;                // step t consumes w[(t + roll) & 255]   (roll = 128: torch.roll(w,128))
    int bp_steps;            // backpointer rows kept per tile: the LAST bp_steps steps (256 or 128)
    unsigned char* bp;       // [n][bp_steps][E*K/8] packed backpointers
    int* e_final;            // [n] out: argmin edge of the final metrics (lowest index on ties), or nullptr
    float* final_cost;       // [n] out: final metric at overlap[tile] (constrained) / its minimum, or nullptr
    float one;               // must be 1.0f: run-time constant of the fused arithmetic tricks (see tcq_common.cuh)
    int inject_extra_bytes;  // 0; the wait self-test sets 16 so that the cluster kernel's byte counts can never be met
    unsigned int* status;    // device word or nullptr: bit 0 = a bounded wait gave up, bit 1 = a weight was NaN or infinite
    int flags;               // kFwdResetStatus | kFwdCheckFinite
};

// Weight j of the staging order for tile `tile`: returns the value and the step index t it belongs to.
// Tiles: t = j.  Row block: consecutive j walk along a matrix row (coalesced), t = (j & 15) * 16 + (j >> 4).
__device__ __forceinline__ float load_weight(const ForwardArgs& a, long long tile, int j, int& t) {
    long long off;
    if (a.ld == 0) {
        t = j;
        off = tile * kT + j;
    } else {
        t = ((j & 15) << 4) | (j >> 4);
        off = (long long)(j >> 4) * a.ld + tile * 16 + (j & 15);
    }
    const float x = a.w[off];
    return a.w_add != nullptr ? __fadd_rn(x, a.w_add[off]) : x;
}

template <int K, int G>
constexpr size_t forward_smem_bytes() {
    return size_t(2) * G * Geo<K>::E * 4 + size_t(2) * G * Geo<K>::ROWB + size_t(G) * kT * 4 + 64 * 8;
}

template <int K, int CB, int G, int NT, int LU>
__global__ void __launch_bounds__(NT, 1) tcq_forward_kernel(const ForwardArgs a) {
    using GE = Geo<K>;
    constexpr int Q = GE::Q, E = GE::E, HN = GE::HN, ROWB = GE::ROWB;
    constexpr int NCHUNK = Q / LU;                 // successor chunks per butterfly
    constexpr int NITEMS = HN * NCHUNK;
    constexpr int ITEM_BITS = LU * K;
    static_assert(LU % 4 == 0 && Q % LU == 0, "successor chunk must be whole float4s");
    static_assert(ITEM_BITS % 8 == 0 && ITEM_BITS <= 32, "an item's backpointers must be whole bytes in one word");
    static_assert(NITEMS % NT == 0, "items must divide evenly over the threads");
    constexpr uint32_t MUL = CbLcg<CB>::MUL, ADD = CbLcg<CB>::ADD;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* const cost = reinterpret_cast<float*>(smem_raw);                       // [2][G][E]
    unsigned char* const stage = smem_raw + size_t(2) * G * E * 4;                // [2][G][ROWB]
    float* const wv = reinterpret_cast<float*>(stage + size_t(2) * G * ROWB);     // [G][256]
    unsigned long long* const red = reinterpret_cast<unsigned long long*>(wv + G * kT);  // [NT/32] reduction scratch

    const int tid = threadIdx.x;
    const long long ngroups = (a.n + G - 1) / G;
    const bool constrained = a.overlap != nullptr;
    const int t_store0 = kT - a.bp_steps;
    const float kInf = __uint_as_float(kInfBits);
    const f32x2 one2 = pack2(a.one, a.one);
    const float zero = a.one - 1.0f;
    if ((a.flags & kFwdResetStatus) && blockIdx.x == 0 && tid == 0 && a.status != nullptr) atomicExch(a.status, 0u);

    for (long long grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
        const long long tile0 = grp * G;

        // ---- load the group's weights, initialise the metrics (qtip.py:161-165) ----
        for (int i = tid; i < G * kT; i += NT) {
            const long long tile = tile0 + (i >> 8);
            int t = i & 255;
            const float x = tile < a.n ? load_weight(a, tile, i & 255, t) : 0.0f;
            wv[(i & ~255) | t] = x;
            if ((a.flags & kFwdCheckFinite) && !isfinite(x) && a.status != nullptr) atomicOr(a.status, 2u);   // reported, never trapped on
        }
        {
            const float init = constrained ? kInf : 0.0f;
            for (int i = tid; i < G * E; i += NT) cost[i] = init;
        }
        __syncthreads();
        if (constrained && tid < G) {
            const long long tile = tile0 + tid;
            const int ov = tile < a.n ? a.overlap[tile] : 0;
            cost[tid * E + (ov & (E - 1))] = 0.0f;
        }
        __syncthreads();

        int cur = 0;
        for (int t = 0; t < kT; ++t) {
            f32x2 w2[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float wt = wv[g * kT + ((t + a.roll) & (kT - 1))];
                w2[g] = pack2(wt, wt);
            }

            // ---- stream the previous step's backpointer rows to HBM (128-bit, coalesced) ----
            if (t > t_store0) {
                const uint4* src = reinterpret_cast<const uint4*>(stage + size_t((t - 1) & 1) * G * ROWB);
                constexpr int V = ROWB / 16;
                for (int i = tid; i < G * V; i += NT) {
                    const int g = i / V, c = i - g * V;
                    const long long tile = tile0 + g;
                    if (tile < a.n) {
                        uint4* dst = reinterpret_cast<uint4*>(a.bp + (size_t(tile) * a.bp_steps + (t - 1 - t_store0)) * ROWB);
                        dst[c] = src[i];
                    }
                }
            }

            const float* const cin_base = cost + size_t(cur) * G * E;
            float* const cout_base = cost + size_t(cur ^ 1) * G * E;
            unsigned char* const st = stage + size_t(t & 1) * G * ROWB;

#pragma unroll 1
            for (int it = tid; it < NITEMS; it += NT) {
                const int h = it & (HN - 1);
                const int lc = it / HN;
                const int e0 = h * Q + lc * LU;                 // first successor edge of the item

                // predecessor metrics, paired (q, q+1) for the packed arithmetic
                f32x2 cin2[G][Q / 2];
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int j = 0; j < Q / 2; ++j)
                        cin2[g][j] = pack2(cin_base[g * E + (2 * j) * HN + h], cin_base[g * E + (2 * j + 1) * HN + h]);

                const uint32_t xb = uint32_t(e0) * MUL + ADD;   // scrambled word of state (q=0, e0)
                float outv[G][LU];
                float tags[G];                                  // sum_l argmin_l * 2^(l*K), exact in fp32 (< 2^24)
#pragma unroll
                for (int g = 0; g < G; ++g) tags[g] = 0.0f;

#pragma unroll
                for (int lu = 0; lu < LU; ++lu) {
                    // codebook values of the Q predecessors' states, once for all G tiles
                    f32x2 v2[Q / 2];
#pragma unroll
                    for (int j = 0; j < Q / 2; ++j)
                        v2[j] = pack2(cb_from_x<CB>(xb + uint32_t((2 * j) * E + lu) * MUL),
                                      cb_from_x<CB>(xb + uint32_t((2 * j + 1) * E + lu) * MUL));
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        float c[Q];
#pragma unroll
                        for (int j = 0; j < Q / 2; ++j) unpack2(cand_cost2(w2[g], v2[j], cin2[g][j], one2), c[2 * j], c[2 * j + 1]);
                        const float best = min_of<Q>(c);
                        // lowest q whose candidate equals the minimum (== first minimum, as torch.min)
                        float tag = float((Q - 1) << (lu * K));
#pragma unroll
                        for (int q = Q - 2; q >= 0; --q) take_if_equal_balanced<Q>(q, tag, c[q], best, zero, float(q << (lu * K)));
                        outv[g][lu] = best;
                        tags[g] = __fadd_rn(tags[g], tag);
                    }
                }
                uint32_t args[G];
#pragma unroll
                for (int g = 0; g < G; ++g) args[g] = __float2uint_rz(tags[g]);

#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float4* dst = reinterpret_cast<float4*>(cout_base + g * E + e0);
#pragma unroll
                    for (int j = 0; j < LU / 4; ++j)
                        dst[j] = make_float4(outv[g][4 * j], outv[g][4 * j + 1], outv[g][4 * j + 2], outv[g][4 * j + 3]);
                    unsigned char* sb = st + g * ROWB + (e0 * K) / 8;
                    if constexpr (ITEM_BITS == 32) {
                        *reinterpret_cast<uint32_t*>(sb) = args[g];
                    } else if constexpr (ITEM_BITS == 16) {
                        *reinterpret_cast<uint16_t*>(sb) = uint16_t(args[g]);
                    } else {
#pragma unroll
                        for (int b = 0; b < ITEM_BITS / 8; ++b) sb[b] = (unsigned char)(args[g] >> (8 * b));
                    }
                }
            }
            __syncthreads();
            cur ^= 1;
        }

        // ---- last backpointer row ----
        {
            const uint4* src = reinterpret_cast<const uint4*>(stage + size_t((kT - 1) & 1) * G * ROWB);
            constexpr int V = ROWB / 16;
            for (int i = tid; i < G * V; i += NT) {
                const int g = i / V, c = i - g * V;
                const long long tile = tile0 + g;
                if (tile < a.n) {
                    uint4* dst = reinterpret_cast<uint4*>(a.bp + (size_t(tile) * a.bp_steps + (a.bp_steps - 1)) * ROWB);
                    dst[c] = src[i];
                }
            }
        }

        // ---- final metrics: argmin edge (qtip.py:185-186) and/or the path cost ----
        const float* const fin = cost + size_t(cur) * G * E;
        if (a.e_final != nullptr || (a.final_cost != nullptr && !constrained)) {
            for (int g = 0; g < G; ++g) {
                // key = (metric bits << 32) | index: metrics are non-negative floats, so the
                // unsigned order of the key is (metric, index) and min() keeps the lowest index.
                unsigned long long key = ~0ull;
                for (int i = tid; i < E; i += NT) {
                    const unsigned long long k2 = (static_cast<unsigned long long>(__float_as_uint(fin[g * E + i])) << 32) | unsigned(i);
                    key = k2 < key ? k2 : key;
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const unsigned long long o = __shfl_xor_sync(0xffffffffu, key, off);
                    key = o < key ? o : key;
                }
                if ((tid & 31) == 0) red[tid >> 5] = key;
                __syncthreads();
                if (tid < 32) {
                    unsigned long long k2 = tid < NT / 32 ? red[tid] : ~0ull;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
                        const unsigned long long o = __shfl_xor_sync(0xffffffffu, k2, off);
                        k2 = o < k2 ? o : k2;
                    }
                    const long long tile = tile0 + g;
                    if (tid == 0 && tile < a.n) {
                        if (a.e_final) a.e_final[tile] = int(k2 & 0xffffffffu);
                        if (a.final_cost && !constrained) a.final_cost[tile] = __uint_as_float(unsigned(k2 >> 32));
                    }
                }
                __syncthreads();
            }
        }
        if (a.final_cost != nullptr && constrained && tid < G) {
            const long long tile = tile0 + tid;
            if (tile < a.n) a.final_cost[tile] = fin[tid * E + (a.overlap[tile] & (E - 1))];
        }
        __syncthreads();   // the next group's initialisation overwrites the metrics
    }
}

// Host-side launcher for one (K, codebook): picks the tiles-per-CTA variant.
// Implemented once per K in tcq_forward_k{2,3,4}.cu.
// `keys` ([n][4] 64-bit scratch) enables the cluster kernel; *nkeys is then the number of
// per-CTA partial minima written per tile (0: the single-CTA kernel ran and wrote e_final).
template <int K>
cudaError_t launch_forward(int codebook, const ForwardArgs& args, unsigned long long* keys, int num_sms,
                           cudaStream_t stream, int* nkeys);

}  // namespace tcq
