// Arguments of the traceback kernel (see tcq_traceback.cu).
#pragma once

#include "tcq_common.cuh"

namespace tcq {

struct TracebackArgs {
    const unsigned char* bp;   // [n][bp_steps][E*K/8] packed backpointers of the LAST bp_steps steps
    long long n;               // tiles
    int bp_steps;              // 256 (whole pass) or 128 (second half only)
    int codebook;              // used for dq
    const int* e_start;        // [n] edge after the last step (argmin edge, or the forced overlap); or nullptr with `keys`
    const unsigned long long* keys;  // [n][nkeys] partial minima (metric bits << 32 | edge) whose smallest gives the start edge
    int nkeys;
    int* e_out;                // [n] out: edge BEFORE the first walked step (the overlap when bp_steps = 128), or nullptr
    long long* states;         // [n,256] out (only the walked steps are written), or nullptr
    long long* bits;           // [n,256] out: state & (2^K - 1), or nullptr
    float* dq;                 // [n,256] out: codebook value of each state, or nullptr
    uint32_t* packed;          // [n][packed_stride] out: exporter word layout, 8K words per tile (needs bp_steps = 256), or nullptr
    long long packed_stride;   // words from one tile's packed codes to the next tile's (>= 8K)
    // LDLQ row-block outputs (need bp_steps = 256); all three share the layout [16][ld], tile i = columns 16i..16i+15
    float* wq;                 // out: reconstruction, or nullptr
    float* err;                // out: src - reconstruction, or nullptr
    const float* src;          // in: the uncompensated block (read only when err != nullptr)
    long long ld;
};

cudaError_t launch_traceback(int K, const TracebackArgs& args, cudaStream_t stream);

// Decode / packing kernels (tcq_decode.cu).
cudaError_t launch_decode_packed(const uint32_t* packed, long long n, int K, int codebook, float* dq, cudaStream_t stream);
cudaError_t launch_decode_matvec(const uint32_t* packed, long long n_out, long long k_in, int K, int codebook, const float* x,
                                 long long ldx, int m, float* y, long long ldy, cudaStream_t stream);
cudaError_t launch_decode_symbols(const long long* bits, long long n, long long T, int K, int codebook,
                                  const long long* s0, float* out, cudaStream_t stream);
cudaError_t launch_pack_symbols(const long long* bits, long long n, int K, uint32_t* packed, cudaStream_t stream);
cudaError_t launch_codebook_lut(int codebook, float* lut, cudaStream_t stream);

// Incoherence processing (tcq_ip.cu).
size_t ip_workspace_bytes(long long n, long long k);
cudaError_t launch_ip_forward(const float* w, long long n, long long k, const float* sv, const float* su, float cb_rms,
                              int tiled, float* z_out, float* out_s, float* in_s, float* scale, void* ws, cudaStream_t stream);
cudaError_t launch_ip_restore(const float* zq, int tiled, long long n, long long k, const float* sv, const float* su,
                              const float* out_s, const float* in_s, const float* scale, float* w_hat, void* ws,
                              cudaStream_t stream);

}  // namespace tcq
