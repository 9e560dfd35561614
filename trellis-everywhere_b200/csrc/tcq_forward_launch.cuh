// Host-side dispatch of the Viterbi step kernel for one K; included by
// tcq_forward_k2.cu / _k3.cu / _k4.cu, which are separate translation units only
// so that the large kernels compile in parallel.
#pragma once

#include "tcq_forward.cuh"

namespace tcq {

template <int K, int CB, int G, int NT, int LU>
static cudaError_t launch_variant(const ForwardArgs& a, int num_sms, cudaStream_t stream) {
    auto kern = tcq_forward_kernel<K, CB, G, NT, LU>;
    constexpr size_t smem = forward_smem_bytes<K, G>();
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (err != cudaSuccess) return err;
    const long long ngroups = (a.n + G - 1) / G;
    const int grid = int(ngroups < num_sms ? ngroups : num_sms);
    kern<<<grid, NT, smem, stream>>>(a);
    return cudaGetLastError();
}

// Relative time of one group of G tiles: G tiles of add-compare-select work plus
// one set of codebook evaluations shared by the group (about 0.85 of a tile's work).
static inline double group_cost(int G) { return double(G) + 0.85; }

// Picks the group size that finishes n tiles soonest on num_sms persistent CTAs.
template <int GMAX>
static int pick_group(long long n, int num_sms) {
    int best = 1;
    double best_t = 1e300;
    for (int G = 1; G <= GMAX; ++G) {
        const long long groups = (n + G - 1) / G;
        const long long rounds = (groups + num_sms - 1) / num_sms;
        const double t = double(rounds) * group_cost(G);
        if (t < best_t - 1e-9) { best_t = t; best = G; }
    }
    return best;
}

}  // namespace tcq
