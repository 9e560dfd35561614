// Incoherence processing around the codec on the device (src/trellis/qtip.py:199-268).
//
// Forward (IPContext.__init__, qtip.py:238-260):
//   z = w * sv[:,None] * su[None,:]
//   out_s = rms over each row, clamped at 1e-8, divided by its mean;   z = Hb_rows(z / out_s[:,None])
//   in_s  = rms over each column, same treatment;                      z = Hb_cols(z / in_s[None,:])
//   scale = rms(z) / cb_rms;                                           z = z / scale
// Restore (qtip.py:262-268) undoes the steps in reverse order.  Hb is the block-diagonal
// orthonormal Sylvester-Hadamard transform with blocks of the largest power of two, at most
// 128, that divides the axis (qtip.py:208-223).  The reference multiplies by the dense
// [128,128] matrix; here each block is a fast Walsh-Hadamard transform (log2(B) butterfly
// stages) held in registers: along the row axis a thread owns one column of the block, along
// the column axis a warp owns 128 columns of one row and exchanges through shuffles.  The
// second forward pass writes straight into the encoder's tile order
// (tile = (row/16)*(k/16) + col/16, t = (row%16)*16 + col%16, qtip.py:288).
//
// All kernels stream: 4 bytes read + 4 bytes written per weight and pass, bound by HBM.
// Every reduction runs in a fixed order (no atomics), so results are reproducible run to run.
// scale = rms(z) is taken before the last transform instead of after it: the transform is
// orthonormal, so the two are equal up to rounding.  Forward divisions by the scale vectors are
// multiplications by their reciprocals (one rounding more than the reference's division).
#include <cmath>

#include "tcq_traceback.cuh"

namespace tcq {

namespace {

constexpr int kIpThreads = 256;
constexpr int kRowThreads = 128;    // columns per CTA of the row-axis transform

__host__ __device__ inline int pow2_block(long long d, int cap) {
    int b = 1;
    while (b < cap && d % (2 * b) == 0) b *= 2;
    return b;
}

// sum of squares of each row; one CTA per row, fixed-order tree.
__global__ void __launch_bounds__(kIpThreads) ip_row_sumsq_kernel(const float* __restrict__ w, long long k,
                                                                 float* __restrict__ rowsq) {
    __shared__ float part[kIpThreads];
    const float* const row = w + (long long)blockIdx.x * k;
    float s = 0.0f;
    for (long long c = threadIdx.x; c < k; c += kIpThreads) {
        const float v = row[c];
        s = __fmaf_rn(v, v, s);
    }
    part[threadIdx.x] = s;
    __syncthreads();
    for (int h = kIpThreads / 2; h > 0; h >>= 1) {
        if (threadIdx.x < h) part[threadIdx.x] += part[threadIdx.x + h];
        __syncthreads();
    }
    if (threadIdx.x == 0) rowsq[blockIdx.x] = part[0];
}

// s[i] = max(sqrt(sum_b sumsq[b][i] / count), 1e-8) / mean(those), inv_s[i] = 1 / s[i];  optionally
// *scale_out = sqrt(sum_i (sum_b sumsq[b][i]) / s[i]^2 / total_count) / cb_rms.  One CTA.
__global__ void __launch_bounds__(1024) ip_finish_scales_kernel(const float* __restrict__ sumsq, int parts, long long d,
                                                               float count, float* __restrict__ s, float* __restrict__ inv_s,
                                                               float total_count, float cb_rms, float* __restrict__ scale_out) {
    __shared__ float red[1024];
    __shared__ float mean_sh;
    float acc = 0.0f;
    for (long long i = threadIdx.x; i < d; i += 1024) {
        float t = 0.0f;
        for (int b = 0; b < parts; ++b) t += sumsq[(long long)b * d + i];
        const float r = fmaxf(sqrtf(t / count), 1e-8f);
        s[i] = r;
        acc += r;
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int h = 512; h > 0; h >>= 1) {
        if (threadIdx.x < h) red[threadIdx.x] += red[threadIdx.x + h];
        __syncthreads();
    }
    if (threadIdx.x == 0) mean_sh = red[0] / float(d);
    __syncthreads();
    const float mean = mean_sh;
    float tot = 0.0f;
    for (long long i = threadIdx.x; i < d; i += 1024) {
        const float r = s[i] / mean;
        s[i] = r;
        inv_s[i] = 1.0f / r;
        if (scale_out != nullptr) {
            float t = 0.0f;
            for (int b = 0; b < parts; ++b) t += sumsq[(long long)b * d + i];
            tot += t / (r * r);
        }
    }
    if (scale_out != nullptr) {
        __syncthreads();
        red[threadIdx.x] = tot;
        __syncthreads();
        for (int h = 512; h > 0; h >>= 1) {
            if (threadIdx.x < h) red[threadIdx.x] += red[threadIdx.x + h];
            __syncthreads();
        }
        if (threadIdx.x == 0) *scale_out = sqrtf(red[0] / total_count) / cb_rms;
    }
}

// column[i] = sum over the `parts` row blocks of sumsq[b][i], in block order (coalesced across threads).
__global__ void __launch_bounds__(kIpThreads) ip_sum_parts_kernel(const float* __restrict__ sumsq, int parts, long long d,
                                                                 float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * kIpThreads + threadIdx.x;
    if (i >= d) return;
    float t = 0.0f;
    for (int b = 0; b < parts; ++b) t += sumsq[(long long)b * d + i];
    out[i] = t;
}

// Transform along the row axis (blocks of B rows): one thread per column keeps the block's B values of
// its column in registers and runs all log2(B) butterfly stages there (natural Sylvester order); a warp
// reads and writes 128 contiguous bytes of each row.  No shared memory, no barriers.
//   forward: in = w,  v = w * (sv[r] / out_s[r]) * su[c] with the reciprocal of out_s taken once per row (rs = 1/out_s;
//            a division per element would sit between the loads and serialise them);  out = z1;
//            colpart[block][c] = sum over the block's rows of z1^2
//   inverse: in = y1, out = ((v * out_s[r]) * sv[r]) * su[c]  (rs = out_s)
template <int B, bool INV>
__global__ void __launch_bounds__(kRowThreads) ip_had_rows_kernel(const float* __restrict__ in, long long k, float norm,
                                                                 const float* __restrict__ sv, const float* __restrict__ su,
                                                                 const float* __restrict__ out_s /* rs */, float* __restrict__ out,
                                                                 float* __restrict__ colpart) {
    const long long r0 = (long long)blockIdx.y * B, c = (long long)blockIdx.x * kRowThreads + threadIdx.x;
    if (c >= k) return;
    const float suc = su[c];
    float v[B];
#pragma unroll
    for (int r = 0; r < B; ++r) {
        v[r] = in[(r0 + r) * k + c];
        if (!INV) v[r] = __fmul_rn(__fmul_rn(v[r], __fmul_rn(sv[r0 + r], out_s[r0 + r])), suc);
    }
#pragma unroll
    for (int h = 1; h < B; h <<= 1) {
#pragma unroll
        for (int b = 0; b < B / 2; ++b) {
            const int i = ((b / h) * 2 * h) + (b % h);
            const float a = v[i], d = v[i + h];
            v[i] = a + d;
            v[i + h] = a - d;
        }
    }
    float sq = 0.0f;
#pragma unroll
    for (int r = 0; r < B; ++r) {
        float o = __fmul_rn(v[r], norm);
        if (INV) o = __fmul_rn(__fmul_rn(__fmul_rn(o, out_s[r0 + r]), sv[r0 + r]), suc);
        else sq = __fmaf_rn(o, o, sq);
        out[(r0 + r) * k + c] = o;
    }
    if (!INV) colpart[(long long)blockIdx.y * k + c] = sq;
}

// Transform along the column axis (blocks of 2^logB columns): one warp per row and 128-column chunk,
// four consecutive columns per lane (one 16-byte load and store); the first two stages run inside the
// lane, the others through warp shuffles.  No shared memory, no barriers.
//   forward: in = z1 (row-major), v = z1 * cs[c] with cs = 1/in_s;  out = v * (1/scale), in tile order or row-major
//   inverse: in = zq (tile order or row-major), v = zq * scale;  out = v * cs[c] with cs = in_s, row-major
// Forward: a CTA of 16 warps takes 16 consecutive rows (n is a multiple of 16) and one 128-column chunk, so that in
// tile order it writes eight whole tiles, 8 KiB contiguous (3 % faster than rows spread over CTAs).  Inverse: eight
// warps per CTA walk the (row, chunk) pairs in row-major order (the 16-row form was 1 % slower there).
constexpr int kColThreadsFwd = 512;

template <bool INV>
__global__ void __launch_bounds__(INV ? kIpThreads : kColThreadsFwd)
ip_had_cols_kernel(const float* __restrict__ in, long long n, long long k, int logB, float norm, const float* __restrict__ in_s,
                   const float* __restrict__ scale, int tiled, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    long long r, c;
    if constexpr (INV) {
        const long long chunks = (k + 127) / 128;
        const long long gw = (long long)blockIdx.x * (kIpThreads / 32) + (threadIdx.x >> 5);
        r = gw / chunks;
        c = (gw - r * chunks) * 128 + lane * 4;
    } else {
        r = (long long)blockIdx.y * 16 + (threadIdx.x >> 5);
        c = (long long)blockIdx.x * 128 + lane * 4;
    }
    if (r >= n) return;                                       // whole warps leave together
    const bool live = c < k;                                  // k is a multiple of 16: a lane's four columns are all in or all out
    const long long rowmajor = r * k + c;
    const long long tile_addr = ((r >> 4) * (k >> 4) + (c >> 4)) * 256 + ((r & 15) << 4) + (c & 15);
    const float sc = INV ? *scale : 1.0f / *scale;
    float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f), s4 = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if (live) {
        x = *reinterpret_cast<const float4*>(in + ((INV && tiled) ? tile_addr : rowmajor));
        s4 = *reinterpret_cast<const float4*>(in_s + c);
    }
    float v[4] = {x.x, x.y, x.z, x.w};
    const float s[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(v[j], INV ? sc : s[j]);
    {   // strides 1 and 2 (logB >= 4 always)
        const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
        v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
    }
    for (int lh = 2; lh < logB; ++lh) {                        // stride 2^lh elements = lane distance 2^(lh-2)
        const int m = 1 << (lh - 2);
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v[j], m);
            v[j] = upper ? o - v[j] : v[j] + o;
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = __fmul_rn(v[j], norm);
        v[j] = __fmul_rn(v[j], INV ? s[j] : sc);
    }
    if (live)
        *reinterpret_cast<float4*>(out + ((!INV && tiled) ? tile_addr : rowmajor)) = make_float4(v[0], v[1], v[2], v[3]);
}

template <bool INV>
cudaError_t launch_rows(int B, dim3 grid, cudaStream_t stream, const float* in, long long k, const float* sv, const float* su,
                        const float* out_s, float* out, float* colpart) {
    const float norm = float(1.0 / sqrt(double(B)));
    switch (B) {
        case 16:  ip_had_rows_kernel<16, INV><<<grid, kRowThreads, 0, stream>>>(in, k, norm, sv, su, out_s, out, colpart); break;
        case 32:  ip_had_rows_kernel<32, INV><<<grid, kRowThreads, 0, stream>>>(in, k, norm, sv, su, out_s, out, colpart); break;
        case 64:  ip_had_rows_kernel<64, INV><<<grid, kRowThreads, 0, stream>>>(in, k, norm, sv, su, out_s, out, colpart); break;
        case 128: ip_had_rows_kernel<128, INV><<<grid, kRowThreads, 0, stream>>>(in, k, norm, sv, su, out_s, out, colpart); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

int ilog2(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }

}  // namespace

size_t ip_workspace_bytes(long long n, long long k) {
    const int B0 = pow2_block(n, 128);
    const size_t z1 = size_t(n) * size_t(k) * 4;
    const size_t colpart = size_t(n / B0) * size_t(k) * 4;
    const size_t rowsq = size_t(n) * 4, colsum = size_t(k) * 4;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    return up(z1) + up(colpart) + 2 * up(rowsq) + 2 * up(colsum);
}

namespace {
struct IpWs { float* z1; float* colpart; float* rowsq; float* colsum; float* inv_out_s; float* inv_in_s; };
IpWs carve_ip(void* ws, long long n, long long k) {
    const int B0 = pow2_block(n, 128);
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    unsigned char* p = static_cast<unsigned char*>(ws);
    IpWs o;
    o.z1 = reinterpret_cast<float*>(p);        p += up(size_t(n) * size_t(k) * 4);
    o.colpart = reinterpret_cast<float*>(p);   p += up(size_t(n / B0) * size_t(k) * 4);
    o.rowsq = reinterpret_cast<float*>(p);     p += up(size_t(n) * 4);
    o.colsum = reinterpret_cast<float*>(p);    p += up(size_t(k) * 4);
    o.inv_out_s = reinterpret_cast<float*>(p); p += up(size_t(n) * 4);
    o.inv_in_s = reinterpret_cast<float*>(p);
    return o;
}
}  // namespace

cudaError_t launch_ip_forward(const float* w, long long n, long long k, const float* sv, const float* su, float cb_rms,
                              int tiled, float* z_out, float* out_s, float* in_s, float* scale, void* ws, cudaStream_t stream) {
    const int B0 = pow2_block(n, 128), B1 = pow2_block(k, 128);
    const IpWs wk = carve_ip(ws, n, k);
    ip_row_sumsq_kernel<<<unsigned(n), kIpThreads, 0, stream>>>(w, k, wk.rowsq);
    ip_finish_scales_kernel<<<1, 1024, 0, stream>>>(wk.rowsq, 1, n, float(k), out_s, wk.inv_out_s, 0.0f, 1.0f, nullptr);
    const dim3 g0(unsigned((k + kRowThreads - 1) / kRowThreads), unsigned(n / B0));
    cudaError_t err = launch_rows<false>(B0, g0, stream, w, k, sv, su, wk.inv_out_s, wk.z1, wk.colpart);
    if (err != cudaSuccess) return err;
    ip_sum_parts_kernel<<<unsigned((k + kIpThreads - 1) / kIpThreads), kIpThreads, 0, stream>>>(wk.colpart, int(n / B0), k, wk.colsum);
    ip_finish_scales_kernel<<<1, 1024, 0, stream>>>(wk.colsum, 1, k, float(n), in_s, wk.inv_in_s, float(n) * float(k), cb_rms, scale);
    const dim3 g1(unsigned((k + 127) / 128), unsigned(n / 16));
    ip_had_cols_kernel<false><<<g1, kColThreadsFwd, 0, stream>>>(wk.z1, n, k, ilog2(B1), float(1.0 / sqrt(double(B1))), wk.inv_in_s, scale, tiled, z_out);
    return cudaGetLastError();
}

cudaError_t launch_ip_restore(const float* zq, int tiled, long long n, long long k, const float* sv, const float* su,
                              const float* out_s, const float* in_s, const float* scale, float* w_hat, void* ws,
                              cudaStream_t stream) {
    const int B0 = pow2_block(n, 128), B1 = pow2_block(k, 128);
    const IpWs wk = carve_ip(ws, n, k);
    const long long warps = n * ((k + 127) / 128);
    const unsigned g1 = unsigned((warps + kIpThreads / 32 - 1) / (kIpThreads / 32));
    ip_had_cols_kernel<true><<<g1, kIpThreads, 0, stream>>>(zq, n, k, ilog2(B1), float(1.0 / sqrt(double(B1))), in_s, scale, tiled, wk.z1);
    const dim3 g0(unsigned((k + kRowThreads - 1) / kRowThreads), unsigned(n / B0));
    return launch_rows<true>(B0, g0, stream, wk.z1, k, sv, su, out_s, w_hat, nullptr);
}

}  // namespace tcq
