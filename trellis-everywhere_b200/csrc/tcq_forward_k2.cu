// Viterbi step kernel instantiations for K = 2 bits per weight.
#include "tcq_forward_launch.cuh"

namespace tcq {

namespace {
constexpr int kNT = 256;   // threads per CTA
constexpr int kLU = 4;     // successors per work item
constexpr int kGMax = 1;   // most tiles one CTA advances together (shared-memory bound)

template <int CB>
cudaError_t launch_cb(const ForwardArgs& a, int num_sms, cudaStream_t stream) {
    switch (pick_group<kGMax>(a.n, num_sms)) {
        case 1: return launch_variant<2, CB, 1, kNT, kLU>(a, num_sms, stream);


        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

template <>
cudaError_t launch_forward<2>(int codebook, const ForwardArgs& a, int num_sms, cudaStream_t stream) {
    switch (codebook) {
        case kCb1Mad:  return launch_cb<kCb1Mad>(a, num_sms, stream);
        case kCb3Inst: return launch_cb<kCb3Inst>(a, num_sms, stream);
        case kCbMcg:   return launch_cb<kCbMcg>(a, num_sms, stream);
        default:       return cudaErrorInvalidValue;
    }
}

}  // namespace tcq
