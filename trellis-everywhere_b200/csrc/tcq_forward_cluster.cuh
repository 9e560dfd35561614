// Viterbi step kernel, thread-block-cluster form: the whole codebook lives in registers.
//
// The plain step kernel (tcq_forward.cuh) re-evaluates each of the 65536 codebook values on
// every step and shares it between the few tiles one SM's shared memory can hold; that
// evaluation is a quarter of its instructions.  Here a cluster of C CTAs (C SMs) owns a group
// of tiles together and the 65536 states are divided among its C * NT threads, so each thread
// keeps its 65536 / (C * NT) codebook values in registers for the whole launch:
//
//   * CTA r owns the butterflies h in [r * HN/C, (r+1) * HN/C): it needs the path metrics
//     old[q * HN + h] for all q (E/C values per tile, in ITS shared memory, layout [Q][HN/C])
//     and produces new[h * Q + l], a contiguous E/C slice of the next metric vector;
//   * every produced metric is consumed, one step later, by exactly one CTA of the cluster
//     (the owner of h' = (h * Q + l) mod HN), so each result is stored once, straight into the
//     consumer's shared memory: a local store or a distributed-shared-memory store
//     (cluster.map_shared_rank), never both;
//   * steps are separated by the hardware cluster barrier.  The group's tiles are split into
//     two sets that alternate; the phase that publishes one set's step is opened (arrive) in
//     the middle of the other set's step and closed (wait) at its end, so neither the release
//     fence nor the barrier latency is exposed;
//   * backpointers: each CTA packs the argmins of its slice into shared memory and streams
//     the previous step's row slice to HBM with 128-bit stores, as the plain kernel does.
//
// A work item is (butterfly, LU successors); with LU * K not a multiple of 8 (K = 3, LU = 4)
// the two items of a butterfly sit in neighbouring lanes and merge their 12 argmin bits with
// one shuffle.  Nothing in this kernel waits on memory written by another CTA except through
// the cluster barrier, and every CTA of a cluster executes the same number of barrier phases.
#pragma once

#include <cooperative_groups.h>

#include "tcq_forward.cuh"

namespace tcq {

namespace cg = cooperative_groups;

template <int K, int C, int GS>
constexpr size_t cluster_smem_bytes() {
    // per CTA: metrics [2 sets][GS][2 buffers][E/C] fp32, staging [2][2*GS][ROWB/C], weights [2*GS][256], reduction scratch
    return size_t(2) * GS * 2 * (Geo<K>::E / C) * 4 + size_t(2) * 2 * GS * (Geo<K>::ROWB / C) + size_t(2) * GS * kT * 4 + 64 * 8;
}

// Split-phase hardware cluster barrier (all threads of all CTAs of the cluster take part).
#ifdef TCQ_X_RELAXED
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
#else
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
#endif
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

struct ClusterArgs {
    ForwardArgs f;
    unsigned long long* keys;   // [n][C] out: per-CTA (metric bits << 32 | edge) minima of the final metrics, or nullptr
};

template <int K, int CB, int C, int GS, int NT, int LU>
__global__ void __launch_bounds__(NT, 1) tcq_forward_cluster_kernel(const ClusterArgs ca) {
    using GE = Geo<K>;
    constexpr int Q = GE::Q, E = GE::E, HN = GE::HN, ROWB = GE::ROWB;
    constexpr int G = 2 * GS;                      // tiles per cluster group (two alternating sets)
    constexpr int HNC = HN / C;                    // butterflies per CTA
    constexpr int EC = E / C;                      // metrics per tile held by a CTA
    constexpr int ROWBC = ROWB / C;                // backpointer bytes per step produced by a CTA
    constexpr int NCHUNK = Q / LU;
    constexpr int NITEMS = HNC * NCHUNK;           // items per CTA
    constexpr int NI = NITEMS / NT;                // items per thread
    constexpr int ITEM_BITS = LU * K;
    constexpr bool PAIRED = (ITEM_BITS % 8) != 0;  // two neighbouring lanes merge their bits
    static_assert(NITEMS % NT == 0 && NI >= 1, "items must divide evenly over the threads");
    static_assert(LU == 2 || LU % 4 == 0, "successor chunk is a float2 or whole float4s");
    static_assert(!PAIRED || (NCHUNK == 2 && 2 * ITEM_BITS % 8 == 0 && 2 * ITEM_BITS <= 24), "paired items must complete whole bytes");
    static_assert(PAIRED || (ITEM_BITS % 8 == 0 && ITEM_BITS <= 24), "an item's backpointers must be whole bytes and exact in fp32");
    static_assert(ROWBC % 16 == 0, "row slices are streamed as 128-bit words");
    constexpr uint32_t MUL = CbLcg<CB>::MUL, ADD = CbLcg<CB>::ADD;
    const ForwardArgs& a = ca.f;

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = int(cluster.block_rank());

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* const cost = reinterpret_cast<float*>(smem_raw);                          // [G][2][EC]
    unsigned char* const stage = smem_raw + size_t(G) * 2 * EC * 4;                   // [2][G][ROWBC]
    float* const wv = reinterpret_cast<float*>(stage + size_t(2) * G * ROWBC);        // [G][256]
    unsigned long long* const red = reinterpret_cast<unsigned long long*>(wv + G * kT);

    const int tid = threadIdx.x;
    const bool constrained = a.overlap != nullptr;
    const int t_store0 = kT - a.bp_steps;
    const float kInf = __uint_as_float(kInfBits);
    const f32x2 one2 = pack2(a.one, a.one);
    const float zero = a.one - 1.0f;

    // ---- this thread's items: codebook values and destinations, fixed for the whole launch ----
    int h_loc[NI];               // butterfly index inside this CTA
    int e_out[NI];               // first successor edge (global numbering)
    float* dst[NI];              // where its LU results go: consumer CTA's metric buffer (tile 0, buffer 0)
    f32x2 cbv[NI][LU][Q / 2];    // codebook values of (q = 2j, 2j+1; successor lu)
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int it = tid + i * NT;
        const int hl = it / NCHUNK, lc = it % NCHUNK;     // chunk index fastest: a butterfly's items are neighbours
        const int h = rank * HNC + hl;
        const int e0 = h * Q + lc * LU;
        h_loc[i] = hl;
        e_out[i] = e0;
        const int qn = e0 / HN, hn = e0 % HN;              // role of e0 in the next step: predecessor qn of butterfly hn
        const int owner = hn / HNC;
        float* local = cost + qn * HNC + (hn % HNC);
#ifdef TCQ_X_LOCAL
        dst[i] = local;
#else
        dst[i] = owner == rank ? local : cluster.map_shared_rank(local, owner);
#endif
        const uint32_t xb = uint32_t(e0) * MUL + ADD;
#pragma unroll
        for (int lu = 0; lu < LU; ++lu)
#pragma unroll
            for (int j = 0; j < Q / 2; ++j)
                cbv[i][lu][j] = pack2(cb_from_x<CB>(xb + uint32_t((2 * j) * E + lu) * MUL),
                                      cb_from_x<CB>(xb + uint32_t((2 * j + 1) * E + lu) * MUL));
    }

    const long long ngroups = (a.n + G - 1) / G;
    const long long nclusters = gridDim.x / C;
    const long long cluster_id = blockIdx.x / C;

    long long tile0 = 0;                           // first tile of the group being processed

    // stream one step's row slices of tile set `s` (written during step t) to HBM (coalesced 128-bit stores)
    auto flush_set = [&](int s, int t, long long tile0) {
        if (t < t_store0) return;
#ifdef TCQ_X_NOFLUSH
        if (t >= 0) return;
#endif
        const uint4* src = reinterpret_cast<const uint4*>(stage + size_t(t & 1) * G * ROWBC + size_t(s) * GS * ROWBC);
        constexpr int V = ROWBC / 16;
        for (int i = tid; i < GS * V; i += NT) {
            const int gg = i / V, cc = i - gg * V;
            const long long tile = tile0 + s * GS + gg;
            if (tile < a.n) {
                uint4* d = reinterpret_cast<uint4*>(a.bp + (size_t(tile) * a.bp_steps + (t - t_store0)) * ROWB + size_t(rank) * ROWBC);
                d[cc] = src[i];
            }
        }
    };

    // one add-compare-select step of tile set `s` (tiles s*GS .. s*GS+GS-1), reading buffer `cur`
    // (`arrive_mid`: half way through, open the pending barrier phase and then stream the set's
    // previous rows to HBM; see the main loop)
    auto step_set = [&](int s, int t, int cur, bool arrive_mid) {
        f32x2 w2[GS];
#pragma unroll
        for (int gg = 0; gg < GS; ++gg) {
            const float wt = wv[(s * GS + gg) * kT + ((t + a.roll) & (kT - 1))];
            w2[gg] = pack2(wt, wt);
        }
        unsigned char* const st = stage + size_t(t & 1) * G * ROWBC;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            f32x2 cin2[GS][Q / 2];
#pragma unroll
            for (int gg = 0; gg < GS; ++gg) {
                const float* cin = cost + (size_t(s * GS + gg) * 2 + cur) * EC + h_loc[i];
#pragma unroll
                for (int j = 0; j < Q / 2; ++j) cin2[gg][j] = pack2(cin[(2 * j) * HNC], cin[(2 * j + 1) * HNC]);
            }
            float outv[GS][LU];
            float tags[GS];
#pragma unroll
            for (int gg = 0; gg < GS; ++gg) tags[gg] = 0.0f;
#pragma unroll
            for (int lu = 0; lu < LU; ++lu) {
                if (i == NI / 2 && lu == (NI > 1 ? 0 : LU / 2) && arrive_mid) {
                    cluster_arrive();
                    if (t > 0) flush_set(s, t - 1, tile0);
                }
#pragma unroll
                for (int gg = 0; gg < GS; ++gg) {
                    float c[Q];
#pragma unroll
                    for (int j = 0; j < Q / 2; ++j)
                        unpack2(cand_cost2(w2[gg], cbv[i][lu][j], cin2[gg][j], one2), c[2 * j], c[2 * j + 1]);
                    const float best = min_of<Q>(c);
                    float tag = float((Q - 1) << (lu * K));
#pragma unroll
                    for (int q = Q - 2; q >= 0; --q) take_if_equal_balanced(q, tag, c[q], best, zero, float(q << (lu * K)));
                    outv[gg][lu] = best;
                    tags[gg] = __fadd_rn(tags[gg], tag);
                }
            }
#pragma unroll
            for (int gg = 0; gg < GS; ++gg) {
                float* d = dst[i] + (size_t(s * GS + gg) * 2 + (cur ^ 1)) * EC;
                if constexpr (LU == 2) {
                    *reinterpret_cast<float2*>(d) = make_float2(outv[gg][0], outv[gg][1]);
                } else {
#pragma unroll
                    for (int j = 0; j < LU / 4; ++j)
                        reinterpret_cast<float4*>(d)[j] = make_float4(outv[gg][4 * j], outv[gg][4 * j + 1], outv[gg][4 * j + 2], outv[gg][4 * j + 3]);
                }
                unsigned char* sb = st + (s * GS + gg) * ROWBC + ((e_out[i] - rank * EC) * K) / 8;
                if constexpr (PAIRED) {
                    // lanes 2m (chunk 0) and 2m+1 (chunk 1) hold the two halves of one butterfly's bits
                    const float other = __shfl_xor_sync(0xffffffffu, tags[gg], 1);
                    if ((tid & 1) == 0) {
                        const uint32_t bits = __float2uint_rz(tags[gg]) | (__float2uint_rz(other) << ITEM_BITS);
#pragma unroll
                        for (int b = 0; b < 2 * ITEM_BITS / 8; ++b) sb[b] = (unsigned char)(bits >> (8 * b));
                    }
                } else {
                    const uint32_t bits = __float2uint_rz(tags[gg]);
#pragma unroll
                    for (int b = 0; b < ITEM_BITS / 8; ++b) sb[b] = (unsigned char)(bits >> (8 * b));
                }
            }
        }
    };

    for (long long grp = cluster_id; grp < ngroups; grp += nclusters) {
        tile0 = grp * G;
        // ---- weights and initial metrics (src/trellis/qtip.py:161-165) ----
        for (int i = tid; i < G * kT; i += NT) {
            const long long tile = tile0 + (i >> 8);
            wv[i] = tile < a.n ? a.w[tile * kT + (i & 255)] : 0.0f;
        }
        {
            const float init = constrained ? kInf : 0.0f;
            for (int i = tid; i < G * EC; i += NT) cost[(size_t(i / EC) * 2) * EC + (i % EC)] = init;
        }
        __syncthreads();
        if (constrained && tid < G) {
            const long long tile = tile0 + tid;
            const int ov = (tile < a.n ? a.overlap[tile] : 0) & (E - 1);
            const int qn = ov / HN, hn = ov % HN;                 // metric of edge ov is predecessor qn of butterfly hn
            if (hn / HNC == rank) cost[(size_t(tid) * 2) * EC + qn * HNC + (hn % HNC)] = 0.0f;
        }
        cluster.sync();   // every CTA's buffers are initialised before anyone stores into them

        // Two tile sets alternate, and the barrier phase that publishes one set's step is opened
        // (arrive) HALF WAY THROUGH the other set's next step and closed (wait) at its end:
        //   * the arrive carries release semantics, i.e. it waits for this thread's earlier
        //     stores (remote shared memory, backpointer rows) to be performed.  The rows of the
        //     set's previous step are therefore streamed to HBM right AFTER the arrive, a whole
        //     step before the next one, so that no fence ever finds them in flight;
        //   * the second half of the step covers the barrier's own latency.
        // Staging rows of set s, step t-1 are read in the middle of its step t: after the phase
        // that published them closed, and before the arrive (middle of the other set's next step)
        // of the phase that lets step t+1 overwrite them.
        step_set(0, 0, 0, false);
        for (int t = 0; t < kT; ++t) {
            const int cur = t & 1;
            step_set(1, t, cur, true);       // middle: arrive for "set 0, step t", then stream set 1's step t-1
            cluster_wait();                  // set 0, step t: complete in every CTA
            if (t + 1 < kT) step_set(0, t + 1, cur ^ 1, true);   // middle: arrive for "set 1, step t", stream set 0's step t
            else { cluster_arrive(); }
            cluster_wait();                  // set 1, step t: complete in every CTA
        }
        flush_set(0, kT - 1, tile0);
        flush_set(1, kT - 1, tile0);

        // ---- final metrics live in buffer 0 (256 steps), layout [Q][HNC] = edges q*HN + rank*HNC + hl ----
        const int fin = 0;
        if (ca.keys != nullptr) {
            for (int g = 0; g < G; ++g) {
                const float* fv = cost + (size_t(g) * 2 + fin) * EC;
                unsigned long long key = ~0ull;
                for (int i = tid; i < EC; i += NT) {
                    const unsigned edge = unsigned(i / HNC) * HN + rank * HNC + (i % HNC);
                    const unsigned long long k2 = (static_cast<unsigned long long>(__float_as_uint(fv[i])) << 32) | edge;
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
                    if (tid == 0 && tile < a.n) ca.keys[tile * C + rank] = k2;
                }
                __syncthreads();
            }
        }
        if (a.final_cost != nullptr && constrained && tid < G) {
            const long long tile = tile0 + tid;
            if (tile < a.n) {
                const int ov = a.overlap[tile] & (E - 1);
                const int qn = ov / HN, hn = ov % HN;
                if (hn / HNC == rank) a.final_cost[tile] = cost[(size_t(tid) * 2 + fin) * EC + qn * HNC + (hn % HNC)];
            }
        }
        cluster.sync();   // nobody may start re-initialising while a neighbour still reads or is written to
    }
}

}  // namespace tcq
