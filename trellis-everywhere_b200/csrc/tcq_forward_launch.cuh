// Host-side dispatch of the Viterbi step kernel for one K; included by
// tcq_forward_k2.cu / _k3.cu / _k4.cu, which are separate translation units only
// so that the large kernels compile in parallel.
#pragma once

#include <cstdlib>
#include <cstring>

#include "tcq_forward_cluster.cuh"

namespace tcq {

constexpr int kMaxDeviceOrdinals = 64;

// Current device ordinal, or -1 if it does not fit the per-device caches below (then nothing is cached).
static inline cudaError_t device_slot(int* slot) {
    int dev = 0;
    const cudaError_t err = cudaGetDevice(&dev);
    *slot = (err == cudaSuccess && dev >= 0 && dev < kMaxDeviceOrdinals) ? dev : -1;
    return err;
}

// Per kernel instantiation and device, once: opt in to the kernel's dynamic shared memory.  Small
// encoder calls (an LDLQ block is a few hundred tiles) would otherwise pay for the attribute call
// on every launch.  (Racing first calls from two host threads both set the same value.)
template <typename Kern>
static cudaError_t ensure_smem_optin(Kern kern, size_t smem, bool (&done)[kMaxDeviceOrdinals], int slot) {
    if (slot >= 0 && done[slot]) return cudaSuccess;
    const cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (err == cudaSuccess && slot >= 0) done[slot] = true;
    return err;
}

template <int K, int CB, int G, int NT, int LU>
static cudaError_t launch_variant(const ForwardArgs& a, int num_sms, cudaStream_t stream) {
    auto kern = tcq_forward_kernel<K, CB, G, NT, LU>;
    constexpr size_t smem = forward_smem_bytes<K, G>();
    static bool optin[kMaxDeviceOrdinals] = {false};
    int slot = -1;
    cudaError_t err = device_slot(&slot);
    if (err != cudaSuccess) return err;
    if ((err = ensure_smem_optin(kern, smem, optin, slot)) != cudaSuccess) return err;
    const long long ngroups = (a.n + G - 1) / G;
    const int grid = int(ngroups < num_sms ? ngroups : num_sms);
    kern<<<grid, NT, smem, stream>>>(a);
    return cudaGetLastError();
}

// Cluster form.  Returns cudaErrorNotSupported (and launches nothing) if this device cannot
// co-schedule a cluster of C CTAs with the kernel's shared-memory footprint.
template <int K, int CB, int C, int GS, int NT, int LU>
static cudaError_t launch_cluster_variant(const ForwardArgs& a, unsigned long long* keys, cudaStream_t stream) {
    auto kern = tcq_forward_cluster_kernel<K, CB, C, GS, NT, LU>;
    constexpr size_t smem = cluster_smem_bytes<K, C, GS>();
    static bool optin[kMaxDeviceOrdinals] = {false};
    int dev = -1;
    cudaError_t err = device_slot(&dev);
    if (err != cudaSuccess) return err;
    if ((err = ensure_smem_optin(kern, smem, optin, dev)) != cudaSuccess) return err;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = C;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NT);
    cfg.gridDim = dim3(C);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    static int max_clusters[kMaxDeviceOrdinals] = {0};   // per device ordinal; 0 = not known yet, -1 = cannot schedule this cluster
    int maxc = dev >= 0 ? max_clusters[dev] : 0;
    if (maxc == 0) {
        int q = 0;
        err = cudaOccupancyMaxActiveClusters(&q, kern, &cfg);
        if (err != cudaSuccess) {
            (void)cudaGetLastError();              // a failed query says nothing about the device: ask again next time
            return cudaErrorNotSupported;
        }
        maxc = q > 0 ? q : -1;
        if (dev >= 0) max_clusters[dev] = maxc;    // cached only when the query itself succeeded
    }
    if (maxc < 0) return cudaErrorNotSupported;
    constexpr int G = 2 * GS;
    const long long ngroups = (a.n + G - 1) / G;
    const long long ncl = ngroups < maxc ? ngroups : maxc;
    cfg.gridDim = dim3(unsigned(ncl * C));
    ClusterArgs ca{a, keys};
    return cudaLaunchKernelEx(&cfg, kern, ca);
}

// Tiles per set (a cluster advances two sets): the size that finishes n tiles soonest on the
// device's clusters, counting whole rounds of groups and a fixed cost per round.  Measured on a
// B200 at K = 3, one round of 2 / 4 / 6 tiles per cluster takes 1.12 / 1.91 / 2.74 ms, i.e.
// 0.406 ms x (tiles + 0.75).
static inline int pick_cluster_set(long long n, int num_sms, int C, int gs_max) {
    const long long clusters = num_sms / C > 0 ? num_sms / C : 1;
    int best = 1;
    double best_t = 1e300;
    for (int gs = 1; gs <= gs_max; ++gs) {
        const long long groups = (n + 2 * gs - 1) / (2 * gs);
        const long long rounds = (groups + clusters - 1) / clusters;
        const double t = double(rounds) * (2.0 * gs + 0.75);
        if (t < best_t - 1e-9) { best_t = t; best = gs; }
    }
    return best;
}

// Which step kernel runs.  Returns the cluster size (2 or 4) or 0 for the single-CTA kernel.
// Default: 2-CTA clusters (all 148 SMs of a B200 pair up; clusters of 4 leave 16 SMs idle).
// TCQ_FORWARD_KERNEL = cta | cluster2 | cluster4 overrides it for comparison runs; the single-CTA
// kernel is also the fallback on a device that cannot co-schedule clusters.
static inline int cluster_size_choice() {
    const char* v = std::getenv("TCQ_FORWARD_KERNEL");
    if (v != nullptr) {
        if (std::strcmp(v, "cta") == 0) return 0;
        if (std::strcmp(v, "cluster4") == 0) return 4;
    }
    return 2;
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
