// Traceback kernel: walks the packed backpointers written by the Viterbi step
// kernel from the last step to the first and emits, per tile, the state path and
// everything derived from it (symbols, packed code words, reconstruction).
//
// Replaces the host loops of src/trellis/qtip.py:189-196 and
// src/trellis/viterbi_triton.py:112-116 (256 tiny launches per pass) and fuses the
// exporter's bit packing (scripts/export_packed_8b.py:52-62).
//
// One warp per tile.  The walk itself is a chain of dependent loads:
//   q_t = bp[t][e_t],  s_t = (q_t << (16-K)) | e_t,  e_{t-1} = s_t >> K .
// Whatever q_t turns out to be, e_{t-1} is one of only Q edges that share the low
// bits e_t >> K, so lane j < Q fetches row t-1's entry for candidate q = j while
// the row-t load is still in flight, and the pick is a shuffle; one row further
// back there are Q*Q possible edges, which can be fetched the same way.  The
// dependent chain is thus one memory round trip per two (or three) steps.
// Afterwards the 32 lanes turn the 256 states held in shared memory into coalesced
// outputs.
#include "tcq_traceback.cuh"

namespace tcq {

namespace {

constexpr int kWarpsPerCta = 4;

template <int K>
__device__ __forceinline__ uint32_t bp_entry(const unsigned char* row, uint32_t e) {
    // Edge e's K-bit argmin sits at bit e*K of the row (little endian).  Two byte
    // loads cover a field that straddles a byte; the second index is clamped so the
    // last entry of a row never reads past it.
    constexpr uint32_t Q = Geo<K>::Q, ROWB = Geo<K>::ROWB;
    const uint32_t bit = e * K;
    const uint32_t b0 = bit >> 3;
    const uint32_t b1 = b0 + 1 < ROWB ? b0 + 1 : b0;
    const uint32_t v = uint32_t(row[b0]) | (uint32_t(row[b1]) << 8);
    return (v >> (bit & 7)) & (Q - 1);
}

template <int K, int DEPTH>
__global__ void __launch_bounds__(kWarpsPerCta * 32) tcq_traceback_kernel(const TracebackArgs a) {
    using GE = Geo<K>;
    constexpr uint32_t Q = GE::Q, E = GE::E, ROWB = GE::ROWB, NW = GE::NWORDS;
    constexpr int SH = kL - K;                     // q sits above the edge bits
    constexpr int HB = kL - 2 * K;                 // predecessor edge = (q << HB) | (e >> K)

    __shared__ uint16_t st_all[kWarpsPerCta][kT];
    const int lane = threadIdx.x & 31;
    const int wrp = threadIdx.x >> 5;
    uint16_t* const st = st_all[wrp];
    const long long tile = (long long)blockIdx.x * kWarpsPerCta + wrp;
    if (tile >= a.n) return;                       // whole warp leaves together; no block-wide barrier below

    const unsigned char* const bp = a.bp + size_t(tile) * a.bp_steps * ROWB;
    uint32_t e;
    if (a.keys != nullptr) {            // argmin of the final metrics, left as per-CTA partial minima by the cluster kernel
        unsigned long long k = a.keys[tile * a.nkeys];
        for (int i = 1; i < a.nkeys; ++i) {
            const unsigned long long o = a.keys[tile * a.nkeys + i];
            k = o < k ? o : k;
        }
        e = uint32_t(k) & (E - 1);
    } else {
        e = uint32_t(a.e_start[tile]) & (E - 1);
    }
    const int t_off = kT - a.bp_steps;             // row r holds step t = r + t_off

    // ---- the walk: DEPTH rows per memory round trip ----
    // Row r's entry is one broadcast load.  Row r-1's entry can only sit at one of Q edges ((j1 << HB) | (e >> K)),
    // row r-2's at one of Q*Q ((j2 << HB) | (j1 << (HB-K)) | (e >> 2K)); lanes fetch all of them at once and the
    // picks are shuffles.  DEPTH = 3 shortens the dependent chain by a third but every trip then waits for the
    // slowest of 1 + Q + Q*Q scattered sectors instead of 1 + Q; measured, it pays only at K = 2 (16 candidates)
    // and only for small batches, where the walk is bound by latency rather than by sector traffic.
    static_assert(DEPTH == 2 || DEPTH == 3, "two or three rows per trip");
    constexpr int PER = 32 / int(Q) > 0 ? 32 / int(Q) : 1;      // level-2 candidates j2 covered by one load per lane
    constexpr int NL2 = (int(Q) + PER - 1) / PER;              // level-2 loads per lane
    int r = a.bp_steps - 1;
    for (; r >= DEPTH - 1; r -= DEPTH) {
        const uint32_t q1 = bp_entry<K>(bp + size_t(r) * ROWB, e);
        const uint32_t j1 = uint32_t(lane) & (Q - 1);
        const uint32_t e1c = (j1 << HB) | (e >> K);
        const uint32_t c1 = bp_entry<K>(bp + size_t(r - 1) * ROWB, e1c);          // lanes >= Q repeat lanes < Q
        uint32_t c2[NL2];
        if constexpr (DEPTH == 3) {
#pragma unroll
            for (int i = 0; i < NL2; ++i) {
                const uint32_t j2 = (uint32_t(lane) / Q + uint32_t(i * PER)) & (Q - 1);
                c2[i] = bp_entry<K>(bp + size_t(r - 2) * ROWB, (j2 << HB) | (e1c >> K));
            }
        }
        const uint32_t s1 = (q1 << SH) | e;
        const uint32_t e1 = s1 >> K;                                              // == candidate edge of lane q1
        const uint32_t q0 = __shfl_sync(0xffffffffu, c1, int(q1));
        const uint32_t s0 = (q0 << SH) | e1;
        e = s0 >> K;
        if (lane == 0) {
            st[r + t_off] = uint16_t(s1);
            st[r - 1 + t_off] = uint16_t(s0);
        }
        if constexpr (DEPTH == 3) {
            uint32_t pick = c2[0];                                                // q0 is the same in every lane
#pragma unroll
            for (int i = 1; i < NL2; ++i) pick = (q0 / PER == uint32_t(i)) ? c2[i] : pick;
            const uint32_t qm = __shfl_sync(0xffffffffu, pick, int(q1 + Q * (q0 % PER)));
            const uint32_t sm = (qm << SH) | e;
            if (lane == 0) st[r - 2 + t_off] = uint16_t(sm);
            e = sm >> K;
        }
    }
    for (; r >= 0; --r) {                          // the rows left over: one round trip each
        const uint32_t q = bp_entry<K>(bp + size_t(r) * ROWB, e);
        const uint32_t s = (q << SH) | e;
        if (lane == 0) st[r + t_off] = uint16_t(s);
        e = s >> K;
    }
    if (lane == 0 && a.e_out != nullptr) a.e_out[tile] = int(e);
    __syncwarp();

    // ---- outputs over the steps that were walked ----
    if (a.states != nullptr)
        for (int t = t_off + lane; t < kT; t += 32) a.states[tile * kT + t] = (long long)st[t];
    if (a.bits != nullptr)
        for (int t = t_off + lane; t < kT; t += 32) a.bits[tile * kT + t] = (long long)(st[t] & (Q - 1));
    if (a.dq != nullptr)
        for (int t = t_off + lane; t < kT; t += 32) a.dq[tile * kT + t] = cb_value_rt(a.codebook, st[t]);
    if (a.wq != nullptr && t_off == 0) {
        // LDLQ row-block layout (src/trellis/ldlq.py:142-143): weight t of this tile is element
        // [t & 15][16 * tile + (t >> 4)] of a 16-row block; j walks along the matrix rows so that a
        // half-warp writes 64 contiguous bytes.  err = src - reconstruction is the block error the
        // recursion feeds back (ldlq.py:90,97), formed here instead of by a separate pass over the block.
        for (int j = lane; j < kT; j += 32) {
            const int t = ((j & 15) << 4) | (j >> 4);
            const float v = cb_value_rt(a.codebook, st[t]);
            const long long off = (long long)(j >> 4) * a.ld + tile * 16 + (j & 15);
            a.wq[off] = v;
            if (a.err != nullptr) a.err[off] = __fsub_rn(a.src[off], v);
        }
    }
    if (a.packed != nullptr && t_off == 0) {
        // word j holds stream bits 32j .. 32j+31; stream bit p is bit (p % K) of symbol 255 - p / K
        for (uint32_t j = lane; j < NW; j += 32) {
            uint32_t word = 0;
#pragma unroll 8
            for (uint32_t b = 0; b < 32; ++b) {
                const uint32_t p = 32 * j + b;
                const uint32_t t = (kT - 1) - p / K;
                word |= ((uint32_t(st[t]) >> (p % K)) & 1u) << b;
            }
            a.packed[tile * a.packed_stride + j] = word;
        }
    }
}

}  // namespace

cudaError_t launch_traceback(int K, const TracebackArgs& a, cudaStream_t stream) {
    if (a.n <= 0) return cudaSuccess;
    const unsigned grid = unsigned((a.n + kWarpsPerCta - 1) / kWarpsPerCta);
    switch (K) {
        case 2:
            if (a.n <= 1024) tcq_traceback_kernel<2, 3><<<grid, kWarpsPerCta * 32, 0, stream>>>(a);
            else tcq_traceback_kernel<2, 2><<<grid, kWarpsPerCta * 32, 0, stream>>>(a);
            break;
        case 3: tcq_traceback_kernel<3, 2><<<grid, kWarpsPerCta * 32, 0, stream>>>(a); break;
        case 4: tcq_traceback_kernel<4, 2><<<grid, kWarpsPerCta * 32, 0, stream>>>(a); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace tcq
