// C ABI of the B200 trellis codec (declared in include/tcq_b200.h): argument
// checking, workspace carving, chunking and the launch sequence.  No device
// memory is allocated or freed here and nothing synchronises with the host.
#include "../../include/tcq_b200.h"

#include <cstdio>
#include <cstring>

#include "tcq_forward.cuh"
#include "tcq_traceback.cuh"

namespace {

using namespace tcq;

thread_local char g_last_cuda_error[256] = "";

int cuda_fail(cudaError_t err, const char* where) {
    std::snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", where, cudaGetErrorString(err));
    return TCQ_E_CUDA;
}

// SM count of the current device (cached per device ordinal).
int current_num_sms(int* out) {
    static int cache[64] = {0};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaGetDevice");
    if (dev >= 0 && dev < 64 && cache[dev] > 0) { *out = cache[dev]; return TCQ_OK; }
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return cuda_fail(err, "cudaDeviceGetAttribute");
    if (dev >= 0 && dev < 64) cache[dev] = sms;
    *out = sms;
    return TCQ_OK;
}

size_t rowb(int K) { return (size_t(1) << (kL - K)) * size_t(K) / 8; }
size_t bp_bytes_per_tile(int K) { return size_t(kT) * rowb(K); }
constexpr size_t kAlign = 256;
size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

constexpr int kMaxKeys = 4;   // partial minima per tile left by the cluster kernel (one per CTA of a cluster)

// Workspace for `chunk` tiles: backpointers of one whole pass, two int32 hand-off arrays and the
// per-CTA partial minima of the final metrics.
size_t ws_bytes_for_chunk(long long chunk, int K) {
    return align_up(size_t(chunk) * bp_bytes_per_tile(K)) + 2 * align_up(size_t(chunk) * sizeof(int)) +
           align_up(size_t(chunk) * kMaxKeys * sizeof(unsigned long long)) + kAlign /* status word */;
}

// Tiles per chunk at full speed: eight rounds of the largest tile group on every SM.
long long default_chunk(int num_sms) { return 8LL * 3 * num_sms; }

struct Workspace {
    unsigned char* bp;
    int* e_final;
    int* overlap;
    unsigned long long* keys;
    unsigned int* status;
    long long chunk;
};

int carve(void* ws, size_t ws_bytes, long long n, int K, int num_sms, Workspace* out) {
    if (ws == nullptr) return TCQ_E_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(ws) % kAlign) return TCQ_E_MISALIGNED;
    long long chunk = n < default_chunk(num_sms) ? n : default_chunk(num_sms);
    if (ws_bytes_for_chunk(chunk, K) > ws_bytes) {
        // largest chunk that fits: solve conservatively, then step down
        chunk = (long long)((ws_bytes > 5 * kAlign ? ws_bytes - 5 * kAlign : 0) / (bp_bytes_per_tile(K) + 2 * sizeof(int) + kMaxKeys * sizeof(unsigned long long)));
        while (chunk > 0 && ws_bytes_for_chunk(chunk, K) > ws_bytes) --chunk;
        if (chunk < 1) return TCQ_E_WORKSPACE;
        // whole rounds of full groups avoid a ragged last wave inside every chunk
        const long long wave = 3LL * num_sms;
        if (chunk > wave) chunk = chunk / wave * wave;
    }
    unsigned char* base = static_cast<unsigned char*>(ws);
    out->bp = base;
    base += align_up(size_t(chunk) * bp_bytes_per_tile(K));
    out->e_final = reinterpret_cast<int*>(base);
    base += align_up(size_t(chunk) * sizeof(int));
    out->overlap = reinterpret_cast<int*>(base);
    base += align_up(size_t(chunk) * sizeof(int));
    out->keys = reinterpret_cast<unsigned long long*>(base);
    base += align_up(size_t(chunk) * kMaxKeys * sizeof(unsigned long long));
    out->status = reinterpret_cast<unsigned int*>(base);
    out->chunk = chunk;
    return TCQ_OK;
}

cudaError_t forward(int K, int codebook, const ForwardArgs& a, const Workspace& wk, int num_sms, cudaStream_t s, int* nkeys) {
    switch (K) {
        case 2: return launch_forward<2>(codebook, a, wk.keys, num_sms, s, nkeys);
        case 3: return launch_forward<3>(codebook, a, wk.keys, num_sms, s, nkeys);
        case 4: return launch_forward<4>(codebook, a, wk.keys, num_sms, s, nkeys);
        default: return cudaErrorInvalidValue;
    }
}

int check_common(int K, int codebook, long long n) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    if (codebook < 0 || codebook > 2) return TCQ_E_BAD_CODEBOOK;
    if (n < 0) return TCQ_E_BAD_COUNT;
    return TCQ_OK;
}

bool misaligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a != 0; }

// What one tail-biting encode reads and writes; tiles (ld == 0) or an LDLQ row block (ld > 0).
struct EncodeIO {
    const float* w;
    const float* w_add;
    long long ld;
    long long n;               // tiles
    uint32_t* packed;
    long long packed_stride;
    int64_t* bits;
    float* dq;
    float* sse;
    float* wq;
    float* err;
};

// The launch sequence of the tail-biting encoder (src/trellis/qtip.py:135-144) per workspace chunk:
// step kernel on the rotated tile -> traceback to the overlap -> step kernel tied to the overlap -> traceback.
// The first step kernel of the call clears the workspace's status word itself (no separate memset node).
int encode_core(const EncodeIO& io, int K, int codebook, void* ws, size_t ws_bytes, cudaStream_t s) {
    int rc, num_sms = 0;
    if ((rc = current_num_sms(&num_sms)) != TCQ_OK) return rc;
    Workspace wk;
    if ((rc = carve(ws, ws_bytes, io.n, K, num_sms, &wk)) != TCQ_OK) return rc;
    // start of chunk c0 inside w / w_add / wq / err: whole tiles (1 KiB each) or 16 columns of the row block per tile
    const long long tile_step = io.ld > 0 ? 16 : kT;
    for (long long c0 = 0; c0 < io.n; c0 += wk.chunk) {
        const long long cn = io.n - c0 < wk.chunk ? io.n - c0 : wk.chunk;
        const float* w = io.w + c0 * tile_step;
        const float* w_add = io.w_add ? io.w_add + c0 * tile_step : nullptr;
        cudaError_t err;
        // pass 1: tile rotated by half its length, free start; only the second half of the
        // backpointers is needed to reach the state at rotated position 128 (qtip.py:138-141)
        ForwardArgs f1{w, w_add, io.ld, cn, nullptr, kT / 2, kT / 2, wk.bp, wk.e_final, nullptr, 1.0f, 0, wk.status,
                       c0 == 0 ? kFwdResetStatus : 0};
        int nkeys = 0;
        if ((err = forward(K, codebook, f1, wk, num_sms, s, &nkeys)) != cudaSuccess) return cuda_fail(err, "forward pass 1");
        TracebackArgs t1{};
        t1.bp = wk.bp;
        t1.n = cn;
        t1.bp_steps = kT / 2;
        t1.codebook = codebook;
        t1.e_start = wk.e_final;
        t1.keys = nkeys ? wk.keys : nullptr;
        t1.nkeys = nkeys;
        t1.e_out = wk.overlap;
        if ((err = launch_traceback(K, t1, s)) != cudaSuccess) return cuda_fail(err, "traceback pass 1");
        // pass 2: true order, start and end tied to the overlap (qtip.py:142)
        ForwardArgs f2{w, w_add, io.ld, cn, wk.overlap, 0, kT, wk.bp, nullptr, io.sse ? io.sse + c0 : nullptr, 1.0f, 0,
                       wk.status, kFwdCheckFinite};
        if ((err = forward(K, codebook, f2, wk, num_sms, s, &nkeys)) != cudaSuccess) return cuda_fail(err, "forward pass 2");
        TracebackArgs t2{};
        t2.bp = wk.bp;
        t2.n = cn;
        t2.bp_steps = kT;
        t2.codebook = codebook;
        t2.e_start = wk.overlap;
        t2.bits = io.bits ? reinterpret_cast<long long*>(io.bits) + c0 * kT : nullptr;
        t2.dq = io.dq ? io.dq + c0 * kT : nullptr;
        t2.packed = io.packed ? io.packed + c0 * io.packed_stride : nullptr;
        t2.packed_stride = io.packed_stride;
        t2.wq = io.wq ? io.wq + c0 * tile_step : nullptr;
        t2.err = io.err ? io.err + c0 * tile_step : nullptr;
        t2.src = io.w + c0 * tile_step;
        t2.ld = io.ld;
        if ((err = launch_traceback(K, t2, s)) != cudaSuccess) return cuda_fail(err, "traceback pass 2");
    }
    return TCQ_OK;
}

}  // namespace

extern "C" {

int tcq_abi_version(void) { return 4; }

const char* tcq_strerror(int code) {
    switch (code) {
        case TCQ_OK: return "ok";
        case TCQ_E_BAD_K: return "K must be 2, 3 or 4";
        case TCQ_E_BAD_CODEBOOK: return "unknown codebook id (0 = 1mad, 1 = 3inst, 2 = mcg)";
        case TCQ_E_BAD_COUNT: return "negative tile or element count";
        case TCQ_E_NULL_POINTER: return "a required pointer is NULL";
        case TCQ_E_MISALIGNED: return "pointer is not aligned as the interface requires";
        case TCQ_E_WORKSPACE: return "workspace is smaller than tcq_workspace_min_bytes(K)";
        case TCQ_E_CUDA: return "CUDA runtime error (see tcq_last_cuda_error)";
        case TCQ_E_BAD_ARGUMENT: return "invalid argument";
        case TCQ_E_NONFINITE_INPUT: return "a weight was NaN or infinite; the codes of its tile are meaningless";
        case TCQ_E_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up; the outputs of that call are invalid";
        case TCQ_E_TOO_MANY_TILES: return "more tiles than the static scratch holds (see tcq_encode_tb_static_max_tiles)";
        default: return "unknown error code";
    }
}

const char* tcq_last_cuda_error(void) { return g_last_cuda_error; }

size_t tcq_workspace_min_bytes(int K) {
    if (K < 2 || K > 4) return 0;
    return ws_bytes_for_chunk(1, K);
}

size_t tcq_workspace_bytes(int64_t n_tiles, int K) {
    if (K < 2 || K > 4 || n_tiles < 0) return 0;
    int num_sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) num_sms = sms;
    } else {
        (void)cudaGetLastError();
    }
    long long chunk = n_tiles < default_chunk(num_sms) ? n_tiles : default_chunk(num_sms);
    if (chunk < 1) chunk = 1;
    return ws_bytes_for_chunk(chunk, K);
}

int tcq_encode_tb(const float* w, int64_t n_tiles, int K, int codebook, uint32_t* packed, int64_t* bits, float* dq,
                  float* sse, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_common(K, codebook, n_tiles);
    if (rc != TCQ_OK) return rc;
    if (n_tiles == 0) return TCQ_OK;
    if (w == nullptr || packed == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(w, 16) || misaligned(packed, 4) || (dq && misaligned(dq, 4)) || (bits && misaligned(bits, 8)) ||
        (sse && misaligned(sse, 4)))
        return TCQ_E_MISALIGNED;
    EncodeIO io{};
    io.w = w;
    io.n = n_tiles;
    io.packed = packed;
    io.packed_stride = kT * K / 32;
    io.bits = bits;
    io.dq = dq;
    io.sse = sse;
    return encode_core(io, K, codebook, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int tcq_encode_tb_rows(const float* src, const float* comp, int64_t ld, int64_t n_out, int K, int codebook,
                       uint32_t* packed, int64_t packed_stride, float* wq, float* err, float* sse, void* ws,
                       size_t ws_bytes, void* stream) {
    int rc = check_common(K, codebook, n_out);
    if (rc != TCQ_OK) return rc;
    if (n_out % 16 || ld < n_out) return TCQ_E_BAD_ARGUMENT;
    if (packed != nullptr && packed_stride < kT * K / 32) return TCQ_E_BAD_ARGUMENT;
    if (n_out == 0) return TCQ_OK;
    if (src == nullptr || wq == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(src, 4) || (comp && misaligned(comp, 4)) || misaligned(wq, 4) || (err && misaligned(err, 4)) ||
        (packed && misaligned(packed, 4)) || (sse && misaligned(sse, 4)))
        return TCQ_E_MISALIGNED;
    EncodeIO io{};
    io.w = src;
    io.w_add = comp;
    io.ld = ld;
    io.n = n_out / 16;
    io.packed = packed;
    io.packed_stride = packed_stride;
    io.sse = sse;
    io.wq = wq;
    io.err = err;
    return encode_core(io, K, codebook, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int tcq_viterbi_pass(const float* w, int64_t n_tiles, int K, int codebook, const int32_t* overlap, int roll,
                     int64_t* states, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_common(K, codebook, n_tiles);
    if (rc != TCQ_OK) return rc;
    if (roll != 0 && roll != kT / 2) return TCQ_E_BAD_ARGUMENT;
    if (n_tiles == 0) return TCQ_OK;
    if (w == nullptr || states == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(w, 16) || misaligned(states, 8) || (overlap && misaligned(overlap, 4))) return TCQ_E_MISALIGNED;
    int num_sms = 0;
    if ((rc = current_num_sms(&num_sms)) != TCQ_OK) return rc;
    Workspace wk;
    if ((rc = carve(ws, ws_bytes, n_tiles, K, num_sms, &wk)) != TCQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(wk.status, 0, sizeof(unsigned int), s) != cudaSuccess) return cuda_fail(cudaGetLastError(), "status reset");

    for (long long c0 = 0; c0 < n_tiles; c0 += wk.chunk) {
        const long long cn = n_tiles - c0 < wk.chunk ? n_tiles - c0 : wk.chunk;
        cudaError_t err;
        ForwardArgs f{w + c0 * kT, nullptr, 0, cn, overlap ? overlap + c0 : nullptr, roll, kT, wk.bp,
                      overlap ? nullptr : wk.e_final, nullptr, 1.0f, 0, wk.status, kFwdCheckFinite};
        int nkeys = 0;
        if ((err = forward(K, codebook, f, wk, num_sms, s, &nkeys)) != cudaSuccess) return cuda_fail(err, "forward");
        const bool use_keys = overlap == nullptr && nkeys > 0;
        TracebackArgs t{};
        t.bp = wk.bp;
        t.n = cn;
        t.bp_steps = kT;
        t.codebook = codebook;
        t.e_start = overlap ? overlap + c0 : wk.e_final;
        t.keys = use_keys ? wk.keys : nullptr;
        t.nkeys = nkeys;
        t.states = reinterpret_cast<long long*>(states) + c0 * kT;
        if ((err = launch_traceback(K, t, s)) != cudaSuccess) return cuda_fail(err, "traceback");
    }
    return TCQ_OK;
}

int tcq_forward_pass(const float* w, int64_t n_tiles, int K, int codebook, const int32_t* overlap, int roll,
                     int bp_steps, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_common(K, codebook, n_tiles);
    if (rc != TCQ_OK) return rc;
    if ((roll != 0 && roll != kT / 2) || (bp_steps != kT && bp_steps != kT / 2)) return TCQ_E_BAD_ARGUMENT;
    if (n_tiles == 0) return TCQ_OK;
    if (w == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(w, 16) || (overlap && misaligned(overlap, 4))) return TCQ_E_MISALIGNED;
    int num_sms = 0;
    if ((rc = current_num_sms(&num_sms)) != TCQ_OK) return rc;
    Workspace wk;
    if ((rc = carve(ws, ws_bytes, n_tiles, K, num_sms, &wk)) != TCQ_OK) return rc;
    if (wk.chunk < n_tiles) return TCQ_E_WORKSPACE;
    if (cudaMemsetAsync(wk.status, 0, sizeof(unsigned int), static_cast<cudaStream_t>(stream)) != cudaSuccess)
        return cuda_fail(cudaGetLastError(), "status reset");
    ForwardArgs f{w, nullptr, 0, n_tiles, overlap, roll, bp_steps, wk.bp, overlap ? nullptr : wk.e_final, nullptr, 1.0f, 0,
                  wk.status, kFwdCheckFinite};
    int nkeys = 0;
    cudaError_t err = forward(K, codebook, f, wk, num_sms, static_cast<cudaStream_t>(stream), &nkeys);
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "forward");
}

int tcq_workspace_status(const void* ws, size_t ws_bytes, int64_t n_tiles, int K, void* stream) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    if (n_tiles <= 0) return n_tiles == 0 ? TCQ_OK : TCQ_E_BAD_COUNT;
    int num_sms = 0;
    int rc = current_num_sms(&num_sms);
    if (rc != TCQ_OK) return rc;
    Workspace wk;
    if ((rc = carve(const_cast<void*>(ws), ws_bytes, n_tiles, K, num_sms, &wk)) != TCQ_OK) return rc;
    unsigned int host = 0;
    cudaError_t err = cudaMemcpyAsync(&host, wk.status, sizeof(host), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return cuda_fail(err, "status read");
    if (host & 1u) return TCQ_E_DEVICE_TIMEOUT;
    return (host & 2u) ? TCQ_E_NONFINITE_INPUT : TCQ_OK;
}

int tcq_selftest_wait_timeout(const float* w, int64_t n_tiles, int K, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_common(K, 0, n_tiles);
    if (rc != TCQ_OK) return rc;
    if (n_tiles < 1 || n_tiles > 8) return TCQ_E_BAD_COUNT;
    if (w == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(w, 16)) return TCQ_E_MISALIGNED;
    int num_sms = 0;
    if ((rc = current_num_sms(&num_sms)) != TCQ_OK) return rc;
    Workspace wk;
    if ((rc = carve(ws, ws_bytes, n_tiles, K, num_sms, &wk)) != TCQ_OK) return rc;
    if (wk.chunk < n_tiles) return TCQ_E_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(wk.status, 0, sizeof(unsigned int), s) != cudaSuccess) return cuda_fail(cudaGetLastError(), "status reset");
    // the buffers of the final metrics are told to expect 16 bytes more than the cluster will ever send
    ForwardArgs f{w, nullptr, 0, n_tiles, nullptr, 0, kT, wk.bp, wk.e_final, nullptr, 1.0f, 16, wk.status, 0};
    int nkeys = 0;
    cudaError_t err = forward(K, kCbMcg, f, wk, num_sms, s, &nkeys);
    if (err != cudaSuccess) return cuda_fail(err, "forward (self-test)");
    return nkeys > 0 ? TCQ_OK : TCQ_E_BAD_ARGUMENT;   // the single-CTA kernel has no bounded waits to test
}

int64_t tcq_encode_launches(int64_t n_tiles, int K, size_t ws_bytes) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    if (n_tiles < 0) return TCQ_E_BAD_COUNT;
    if (n_tiles == 0) return 0;
    int num_sms = 0;
    int rc = current_num_sms(&num_sms);
    if (rc != TCQ_OK) return rc;
    Workspace wk;
    alignas(256) static unsigned char dummy[256];          // carve() only does pointer arithmetic on it
    if ((rc = carve(dummy, ws_bytes, n_tiles, K, num_sms, &wk)) != TCQ_OK) return rc;
    return 4 * ((n_tiles + wk.chunk - 1) / wk.chunk);
}

int tcq_decode_packed(const uint32_t* packed, int64_t n_tiles, int K, int codebook, float* dq, void* stream) {
    int rc = check_common(K, codebook, n_tiles);
    if (rc != TCQ_OK) return rc;
    if (n_tiles == 0) return TCQ_OK;
    if (packed == nullptr || dq == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(packed, 4) || misaligned(dq, 16)) return TCQ_E_MISALIGNED;
    cudaError_t err = launch_decode_packed(packed, n_tiles, K, codebook, dq, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "decode_packed");
}

int tcq_decode_matvec(const uint32_t* packed, int64_t n_out, int64_t k_in, int K, int codebook, const float* x, int64_t ldx,
                      int m, float* y, int64_t ldy, void* stream) {
    int rc = check_common(K, codebook, n_out);
    if (rc != TCQ_OK) return rc;
    if (k_in < 0 || m < 0) return TCQ_E_BAD_COUNT;
    if (n_out % 16 || k_in % 16 || n_out / 16 > 0x7FFFFFFF || k_in / 16 > 0x7FFFFFFF) return TCQ_E_BAD_ARGUMENT;
    if (n_out == 0 || k_in == 0 || m == 0) return TCQ_OK;
    if (ldx < k_in || ldx % 4 || ldy < n_out) return TCQ_E_BAD_ARGUMENT;
    if (packed == nullptr || x == nullptr || y == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(packed, 4) || misaligned(x, 16) || misaligned(y, 4)) return TCQ_E_MISALIGNED;
    cudaError_t err = launch_decode_matvec(packed, n_out, k_in, K, codebook, x, ldx, m, y, ldy,
                                           static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "decode_matvec");
}

int tcq_decode_symbols(const int64_t* bits, int64_t n, int64_t T, int K, int codebook, const int64_t* s0, float* out,
                       void* stream) {
    int rc = check_common(K, codebook, n);
    if (rc != TCQ_OK) return rc;
    if (T < 0) return TCQ_E_BAD_COUNT;
    if (n == 0 || T == 0) return TCQ_OK;
    if (bits == nullptr || out == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(bits, 8) || misaligned(out, 4) || (s0 && misaligned(s0, 8))) return TCQ_E_MISALIGNED;
    cudaError_t err = launch_decode_symbols(reinterpret_cast<const long long*>(bits), n, T, K, codebook,
                                            reinterpret_cast<const long long*>(s0), out,
                                            static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "decode_symbols");
}

int tcq_pack_symbols(const int64_t* bits, int64_t n_tiles, int K, uint32_t* packed, void* stream) {
    if (K < 2 || K > 4) return TCQ_E_BAD_K;
    if (n_tiles < 0) return TCQ_E_BAD_COUNT;
    if (n_tiles == 0) return TCQ_OK;
    if (bits == nullptr || packed == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(bits, 8) || misaligned(packed, 4)) return TCQ_E_MISALIGNED;
    cudaError_t err = launch_pack_symbols(reinterpret_cast<const long long*>(bits), n_tiles, K, packed,
                                          static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "pack_symbols");
}

namespace {
int check_ip_shape(int64_t n, int64_t k) {
    if (n < 0 || k < 0) return TCQ_E_BAD_COUNT;
    if (n % 16 || k % 16 || n / 16 > 65535) return TCQ_E_BAD_ARGUMENT;
    return TCQ_OK;
}
}  // namespace

size_t tcq_ip_workspace_bytes(int64_t n, int64_t k) {
    if (check_ip_shape(n, k) != TCQ_OK || n == 0 || k == 0) return 0;
    return ip_workspace_bytes(n, k);
}

int tcq_ip_forward(const float* w, int64_t n, int64_t k, const float* sv, const float* su, float cb_rms, int tiled,
                   float* z, float* out_s, float* in_s, float* scale, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_ip_shape(n, k);
    if (rc != TCQ_OK) return rc;
    if (!(cb_rms > 0.0f)) return TCQ_E_BAD_ARGUMENT;
    if (n == 0 || k == 0) return TCQ_OK;
    if (!w || !sv || !su || !z || !out_s || !in_s || !scale || !ws) return TCQ_E_NULL_POINTER;
    if (misaligned(w, 4) || misaligned(z, 16) || misaligned(sv, 4) || misaligned(su, 4) || misaligned(out_s, 4) ||
        misaligned(in_s, 16) || misaligned(scale, 4) || misaligned(ws, 256))
        return TCQ_E_MISALIGNED;
    if (ws_bytes < ip_workspace_bytes(n, k)) return TCQ_E_WORKSPACE;
    cudaError_t err = launch_ip_forward(w, n, k, sv, su, cb_rms, tiled != 0, z, out_s, in_s, scale, ws,
                                        static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "ip_forward");
}

int tcq_ip_restore(const float* zq, int tiled, int64_t n, int64_t k, const float* sv, const float* su, const float* out_s,
                   const float* in_s, const float* scale, float* w_hat, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_ip_shape(n, k);
    if (rc != TCQ_OK) return rc;
    if (n == 0 || k == 0) return TCQ_OK;
    if (!zq || !sv || !su || !out_s || !in_s || !scale || !w_hat || !ws) return TCQ_E_NULL_POINTER;
    if (misaligned(zq, 16) || misaligned(w_hat, 4) || misaligned(sv, 4) || misaligned(su, 4) || misaligned(out_s, 4) ||
        misaligned(in_s, 16) || misaligned(scale, 4) || misaligned(ws, 256))
        return TCQ_E_MISALIGNED;
    if (ws_bytes < ip_workspace_bytes(n, k)) return TCQ_E_WORKSPACE;
    cudaError_t err = launch_ip_restore(zq, tiled != 0, n, k, sv, su, out_s, in_s, scale, w_hat, ws,
                                        static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "ip_restore");
}

int tcq_codebook_lut(int codebook, float* lut, void* stream) {
    if (codebook < 0 || codebook > 2) return TCQ_E_BAD_CODEBOOK;
    if (lut == nullptr) return TCQ_E_NULL_POINTER;
    if (misaligned(lut, 4)) return TCQ_E_MISALIGNED;
    cudaError_t err = launch_codebook_lut(codebook, lut, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? TCQ_OK : cuda_fail(err, "codebook_lut");
}

}  // extern "C"
