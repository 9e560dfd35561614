// tcq_encode_tb_static: the tail-biting encoder for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they need the encoder:
// a plugin running inside another framework's memory budget, a service that fixed its device
// footprint at start-up.  tcq_encode_tb asks such a
// caller for a workspace it has no way to obtain.  This entry point needs none: the backpointer
// scratch is a fixed array in the library's own device image.
//
//   * The array is TCQ_STATIC_SCRATCH_BYTES (32 MiB) and is part of every GPU context that loads
//     the library, used or not, until the process exits.
//   * That bounds the batch: tcq_encode_tb_static_max_tiles(K) tiles per call (31 / 42 / 63 for
//     K = 2 / 3 / 4).  Larger batches are refused with TCQ_E_TOO_MANY_TILES and nothing is launched.
//   * The first call on each device looks up the array's device address (with that device
//     current) and remembers it.  Make that first call outside any stream capture.
//   * All calls share the one array and it keeps whatever the previous call left in it.  The
//     encoder never reads a byte it has not written earlier in the same call (every backpointer
//     row, argmin edge and overlap word is produced before it is consumed), so nothing has to be
//     cleared; but two calls whose kernels overlap on the GPU (different streams, no dependency)
//     overwrite each other's backpointers.  Serialise them.
//   * tcq_encode_tb_static_status(stream) is tcq_workspace_status for this path: the status word
//     (a bounded in-kernel wait gave up / a weight was NaN or infinite) lives inside the array, where a
//     caller without the array's address could not otherwise read it.  It reports on the LAST call made
//     on the current device and synchronises the stream.
//
// The name of a __device__ array is, in host code, only a handle for the runtime: it is not a
// device address, and handing it to a kernel would make the kernel fault or scribble over
// unrelated memory.  The address comes from cudaGetSymbolAddress below.
#include "../../include/tcq_b200.h"

#include <cuda_runtime.h>

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[TCQ_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};     // written once per device with the same value by whoever comes first

// Batch size and K of the last call on each device: the status word's place inside the array depends on them.
struct LastCall { long long n; int K; };
LastCall g_last_call[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(void** out, int* dev_out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return TCQ_E_CUDA;
    }
    if (dev < 0 || dev >= kMaxDevices) return TCQ_E_CUDA;
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (err != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return TCQ_E_CUDA;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    if (dev_out != nullptr) *dev_out = dev;
    return TCQ_OK;
}

}  // namespace

extern "C" {

int64_t tcq_encode_tb_static_max_tiles(int K) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    // Worked out once per K.  Batches this small are far below one full-speed chunk, where the workspace
    // size depends on the tile count and K only, not on the device.
    static int64_t cached[5] = {0, 0, 0, 0, 0};
    if (cached[K] == 0) {
        int64_t n = 0;
        while (tcq_workspace_bytes(n + 1, K) <= size_t(TCQ_STATIC_SCRATCH_BYTES)) ++n;
        cached[K] = n;
    }
    return cached[K];
}

int tcq_encode_tb_static(const float* w, int64_t n_tiles, int K, int codebook, uint32_t* packed, int64_t* bits,
                         float* dq, float* sse, void* stream) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    if (n_tiles < 0) return TCQ_E_BAD_COUNT;
    if (n_tiles > tcq_encode_tb_static_max_tiles(K)) return TCQ_E_TOO_MANY_TILES;
    if (n_tiles == 0) return TCQ_OK;
    void* scratch = nullptr;
    int dev = 0;
    const int rc = scratch_for_current_device(&scratch, &dev);
    if (rc != TCQ_OK) return rc;
    g_last_call[dev] = LastCall{n_tiles, K};
    // From here on this is the ordinary encoder with the static array as its workspace.
    return tcq_encode_tb(w, n_tiles, K, codebook, packed, bits, dq, sse, scratch, size_t(TCQ_STATIC_SCRATCH_BYTES), stream);
}

int tcq_encode_tb_static_status(void* stream) {
    void* scratch = nullptr;
    int dev = 0;
    const int rc = scratch_for_current_device(&scratch, &dev);
    if (rc != TCQ_OK) return rc;
    const LastCall last = g_last_call[dev];
    if (last.n <= 0) return TCQ_OK;                 // nothing has run on this device yet
    return tcq_workspace_status(scratch, size_t(TCQ_STATIC_SCRATCH_BYTES), last.n, last.K, stream);
}

}  // extern "C"
