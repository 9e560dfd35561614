// Viterbi step kernel instantiations for K = 3 bits per weight.
#include "tcq_forward_launch.cuh"

namespace tcq {

namespace {
constexpr int kNT = 512;     // threads per CTA
constexpr int kLU = 8;       // successors per work item, single-CTA kernel
constexpr int kGMax = 3;     // most tiles one CTA advances together (shared-memory bound)
constexpr int kCLU4 = 4;     // successors per work item with 4 CTAs per cluster (32 codebook values per thread)
constexpr int kCLU2 = 4;     // ... with 2 CTAs per cluster (64 codebook values per thread, two items of four successors; one item of
                             //     eight was measured 8 % slower: it spills at the 128-register limit; 256 threads
                             //     with 128 values each, 226-231 registers, 11-21 % slower: too few warps to hide latencies)

template <int CB>
cudaError_t launch_cb(const ForwardArgs& a, unsigned long long* keys, int num_sms, cudaStream_t stream, int* nkeys) {
    *nkeys = 0;
    const int csize = cluster_size_choice();
    if (keys != nullptr && csize != 0) {
        cudaError_t err;
        if (csize == 2) {
            switch (pick_cluster_set(a.n, num_sms, 2, 3)) {
                case 1: err = launch_cluster_variant<3, CB, 2, 1, kNT, kCLU2>(a, keys, stream); break;
                case 2: err = launch_cluster_variant<3, CB, 2, 2, kNT, kCLU2>(a, keys, stream); break;
                default: err = launch_cluster_variant<3, CB, 2, 3, kNT, kCLU2>(a, keys, stream); break;
            }
        } else {
            err = pick_cluster_set(a.n, num_sms, 4, 2) == 2 ? launch_cluster_variant<3, CB, 4, 2, kNT, kCLU4>(a, keys, stream)
                                                           : launch_cluster_variant<3, CB, 4, 1, kNT, kCLU4>(a, keys, stream);
        }
        if (err != cudaErrorNotSupported) {
            *nkeys = csize;
            return err;
        }
    }
    switch (pick_group<kGMax>(a.n, num_sms)) {
        case 1: return launch_variant<3, CB, 1, kNT, kLU>(a, num_sms, stream);
        case 2: return launch_variant<3, CB, 2, kNT, kLU>(a, num_sms, stream);
        case 3: return launch_variant<3, CB, 3, kNT, kLU>(a, num_sms, stream);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

template <>
cudaError_t launch_forward<3>(int codebook, const ForwardArgs& a, unsigned long long* keys, int num_sms,
                               cudaStream_t stream, int* nkeys) {
    switch (codebook) {
        case kCb1Mad:  return launch_cb<kCb1Mad>(a, keys, num_sms, stream, nkeys);
        case kCb3Inst: return launch_cb<kCb3Inst>(a, keys, num_sms, stream, nkeys);
        case kCbMcg:   return launch_cb<kCbMcg>(a, keys, num_sms, stream, nkeys);
        default:       return cudaErrorInvalidValue;
    }
}

}  // namespace tcq
