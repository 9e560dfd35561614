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
//   * the stores are asynchronous (st.async) and each one reports its 16 bytes to an mbarrier
//     in the consumer CTA; a CTA starts a step when the mbarrier of its input buffer has
//     counted the whole buffer.  No thread ever executes a memory fence, which matters because
//     a release fence on this chip waits for every outstanding store of the SM, including the
//     backpointer rows on their way to HBM;
//   * the only other synchronisation is write-after-read: nobody may store into a buffer that
//     a neighbour is still reading.  The hardware cluster barrier handles that with relaxed
//     arrives at the end of every step and a wait just before the next step's first store;
//   * the group's tiles form two sets that alternate, so both kinds of wait normally find
//     their condition already true: the other set's step has run in between;
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

// Hardware cluster barrier, split phase, no memory ordering: used only to keep stores away from
// buffers that are still being read.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_relaxed() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }

// ---- mbarrier + asynchronous distributed-shared-memory stores ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
// shared::cta address -> the same location in CTA `rank` of the cluster (shared::cluster address)
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// one arrival that also announces `bytes` of asynchronous stores for the phase in progress
__device__ __forceinline__ void mbar_expect(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// One poll (the hardware may park the thread briefly before answering).
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(mbar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: polls until the phase completes or kMbarWaitCycles SM clocks (about a quarter of a
// second) have passed, where a healthy wait takes microseconds.  The caller records the failure
// and stops exchanging metrics, so a counting bug shows up as an error status and invalid codes,
// never as a hang.  (No suspend-time hint on the poll: a hint makes every unsatisfied poll sleep
// for about that long, which cost 7 % of the kernel's throughput.)
//
// `gave_up` is a word in this CTA's shared memory, zero at launch.  The first wait that runs out
// sets it, and from then on no wait of this CTA spins: each polls twice and reports failure, so a
// launch whose protocol broke ends after about one time limit, not one per remaining wait.  The
// flag is looked at on the slow path only and lives in shared memory on purpose: the step loop sits
// at the register limit, and any extra state carried through its fast path (tried: a predicate, a
// second return value) cost 6-7 % of the kernel's throughput.
constexpr long long kMbarWaitCycles = 500000000LL;
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity, volatile unsigned int* gave_up) {
    if (mbar_try_wait(mbar, parity)) return true;
    const long long t0 = clock64();
    const long long limit = *gave_up ? 0 : kMbarWaitCycles;
    while (clock64() - t0 < limit)
        if (mbar_try_wait(mbar, parity)) return true;
    // One more poll after the deadline: a thread that was descheduled across it (time slicing, an attached
    // profiler) must not report a phase that completed meanwhile as lost.
    if (mbar_try_wait(mbar, parity)) return true;
    *gave_up = 1u;
    return false;
}
__device__ __forceinline__ void st_async_v4(uint32_t dst, float x, float y, float z, float w, uint32_t mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(dst), "f"(x), "f"(y), "f"(z), "f"(w), "r"(mbar) : "memory");
}
__device__ __forceinline__ void st_async_v2(uint32_t dst, float x, float y, uint32_t mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                 ::"r"(dst), "f"(x), "f"(y), "r"(mbar) : "memory");
}

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
    unsigned long long* const red = reinterpret_cast<unsigned long long*>(wv + G * kT);   // [32] reduction scratch
    unsigned long long* const mbar = red + 32;     // [2 sets][2 buffers] mbarriers counting the bytes of each metric buffer
    volatile unsigned int* const gave_up = reinterpret_cast<volatile unsigned int*>(red + 40);   // set by the first wait that runs out

    const int tid = threadIdx.x;
    const bool constrained = a.overlap != nullptr;
    const int t_store0 = kT - a.bp_steps;
    const float kInf = __uint_as_float(kInfBits);
    const f32x2 one2 = pack2(a.one, a.one);
    const float zero = a.one - 1.0f;

    // ---- this thread's items: codebook values and destinations, fixed for the whole launch ----
    int h_loc[NI];               // butterfly index inside this CTA
    int e_out[NI];               // first successor edge (global numbering)
    uint32_t dst[NI];            // where its LU results go: shared::cluster address in the consumer CTA (tile 0, buffer 0)
    uint32_t dst_bar[NI];        // the consumer CTA's mbarrier array (shared::cluster address)
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
        dst[i] = map_to_rank(smem_u32(cost + qn * HNC + (hn % HNC)), owner);
        dst_bar[i] = map_to_rank(smem_u32(mbar), owner);
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

    // stream one step's row slices of tile set `s` (written during step t into staging buffer `buf` = t & 1) to HBM
    // (coalesced 128-bit stores).  A set's slices are GS * ROWBC / 16 <= NT words, one per thread; which word, which
    // tile of the set and the byte offset from the set's first row are fixed for the launch.
    constexpr int V = ROWBC / 16;
    constexpr int FW = (GS * V + NT - 1) / NT;     // 128-bit words of a set's row slices per thread
    int fl_src[FW];
    size_t fl_off[FW];
    int fl_gg[FW];
#pragma unroll
    for (int k = 0; k < FW; ++k) {
        const int wd = tid + k * NT;
        fl_src[k] = wd;
        fl_gg[k] = wd < GS * V ? wd / V : -1;
        fl_off[k] = size_t(wd / V) * a.bp_steps * ROWB + size_t(rank) * ROWBC + size_t(wd % V) * 16;
    }
    auto flush_set = [&](int s, int t, int buf, long long tile0) {
        if (t < t_store0) return;
        const uint4* src = reinterpret_cast<const uint4*>(stage + size_t(buf) * G * ROWBC + size_t(s) * GS * ROWBC);
        unsigned char* row0 = a.bp + (size_t(tile0 + s * GS) * a.bp_steps + (t - t_store0)) * ROWB;     // uniform
#pragma unroll
        for (int k = 0; k < FW; ++k)
            if (fl_gg[k] >= 0 && tile0 + s * GS + fl_gg[k] < a.n) *reinterpret_cast<uint4*>(row0 + fl_off[k]) = src[fl_src[k]];
    };

    constexpr uint32_t kBufBytes = uint32_t(GS) * EC * 4;     // bytes every (set, buffer) receives per step
    uint32_t parity = 0;          // bit (2*s + b): parity of the phase the next wait on mbarrier (s, b) is for
    bool timed_out = false;
    bool wait_pending = false;    // the barrier phase entered during the PREVIOUS step_set has not been closed yet
    auto war_wait = [&]() {
        if (wait_pending) {
            cluster_wait_relaxed();
            wait_pending = false;
        }
    };

    // All bytes of buffer b of set s have landed; then re-arm its mbarrier for the next use.
    // A wait that runs out is recorded (the launch's results are then invalid) and the thread
    // carries on; it never re-arms an mbarrier again, because an arrive on an mbarrier whose phase
    // cannot complete would underflow its arrival count, which is a hardware error.  The byte
    // counts do not depend on the data, so a wait can only run out through a programming error,
    // which the tests would show on every run; the limit exists so that even then nothing hangs.
    // (`last`: the re-arm for the phase that the end-of-group wait checks; the wait self-test
    // inflates exactly that one, so that its timeouts happen after the last store has landed.)
    auto wait_buffer = [&](int s, int b, bool last) {
        const uint32_t m = smem_u32(mbar + (2 * s + b));
        if (!mbar_wait(m, (parity >> (2 * s + b)) & 1u, gave_up)) timed_out = true;
        parity ^= 1u << (2 * s + b);
        if (tid == 0 && !timed_out) mbar_expect(m, kBufBytes + (last ? uint32_t(a.inject_extra_bytes) : 0u));
    };

    // One add-compare-select step of tile set `s` (tiles s*GS .. s*GS+GS-1), reading buffer `cur`.
    // Half way through, the set's previous backpointer rows are streamed to HBM.
    auto step_set = [&](int s, int t, int cur) {
        if (t > 0) wait_buffer(s, cur, t == kT - 2);
        f32x2 w2[GS];
#pragma unroll
        for (int gg = 0; gg < GS; ++gg) {
            const float wt = wv[(s * GS + gg) * kT + ((t + a.roll) & (kT - 1))];
            w2[gg] = pack2(wt, wt);
        }
        unsigned char* const st = stage + size_t(cur) * G * ROWBC;        // cur == t & 1
#pragma unroll
        for (int i = 0; i < NI; ++i) {
#pragma unroll
            for (int gg = 0; gg < GS; ++gg) {
                // The codebook is in registers, so tiles need not share anything: one tile at a time
                // keeps only Q predecessor metrics live and lets the next tile's loads fly under
                // this tile's arithmetic.
                f32x2 cin2[Q / 2];
                const float* cin = cost + (size_t(s * GS + gg) * 2 + cur) * EC + h_loc[i];
#pragma unroll
                for (int j = 0; j < Q / 2; ++j) cin2[j] = pack2(cin[(2 * j) * HNC], cin[(2 * j + 1) * HNC]);
                constexpr int SV = LU < 4 ? LU : 4;            // successors per store (float2 or float4)
                float outv[SV];
                float tags = 0.0f;
                const uint32_t d0 = dst[i] + uint32_t((size_t(s * GS + gg) * 2 + (cur ^ 1)) * EC * 4);
                const uint32_t m = dst_bar[i] + uint32_t(2 * s + (cur ^ 1)) * 8u;
#pragma unroll
                for (int lu = 0; lu < LU; ++lu) {
                    if (i == NI / 2 && gg == GS / 2 && lu == ((NI > 1 || GS > 1) ? 0 : LU / 2) && t > 0) flush_set(s, t - 1, cur ^ 1, tile0);
                    float c[Q];
#pragma unroll
                    for (int j = 0; j < Q / 2; ++j)
                        unpack2(cand_cost2(w2[gg], cbv[i][lu][j], cin2[j], one2), c[2 * j], c[2 * j + 1]);
                    const float best = min_of<Q>(c);
                    float tag = float((Q - 1) << (lu * K));
#pragma unroll
                    for (int q = Q - 2; q >= 0; --q) take_if_equal_balanced<Q>(q, tag, c[q], best, zero, float(q << (lu * K)));
                    outv[lu % SV] = best;
                    tags = __fadd_rn(tags, tag);
                    if (i == NI - 1 && gg == GS - 1 && lu == 0) {
                        // Every input of this step has been loaded AND used (the first successor of the
                        // last tile of the last item consumed all of its predecessors' metrics), so this
                        // thread no longer reads the input buffers: tell the cluster, well before anyone
                        // needs to know.  (The barrier's phases are sequential: close the previous one first.)
                        war_wait();
                        cluster_arrive_relaxed();
                    }
                    if (lu % SV == SV - 1) {
                        // Results leave as soon as a store's worth is ready (fewer live registers).
                        // Write-after-read: the buffer written now was read by every CTA one step of this
                        // set ago; the barrier phase that every thread entered during the previous
                        // step_set (of the other set) proves it, and it is closed before the first store.
                        war_wait();
                        const uint32_t d = d0 + uint32_t(lu + 1 - SV) * 4u;
                        if constexpr (SV == 2) st_async_v2(d, outv[0], outv[1], m);
                        else st_async_v4(d, outv[0], outv[1], outv[2], outv[3], m);
                    }
                }
                unsigned char* sb = st + (s * GS + gg) * ROWBC + ((e_out[i] - rank * EC) * K) / 8;
                if constexpr (PAIRED) {
                    // lanes 2m (chunk 0) and 2m+1 (chunk 1) hold the two halves of one butterfly's bits
                    const float other = __shfl_xor_sync(0xffffffffu, tags, 1);
                    if ((tid & 1) == 0) {
                        const uint32_t bits = __float2uint_rz(tags) | (__float2uint_rz(other) << ITEM_BITS);
#pragma unroll
                        for (int b = 0; b < 2 * ITEM_BITS / 8; ++b) sb[b] = (unsigned char)(bits >> (8 * b));
                    }
                } else {
                    const uint32_t bits = __float2uint_rz(tags);
#pragma unroll
                    for (int b = 0; b < ITEM_BITS / 8; ++b) sb[b] = (unsigned char)(bits >> (8 * b));
                }
            }
        }
        wait_pending = true;          // the phase entered above is closed during the next step_set
    };

    if ((a.flags & kFwdResetStatus) && blockIdx.x == 0 && tid == 0 && a.status != nullptr) atomicExch(a.status, 0u);

    // ---- mbarriers: one arrival (the re-arming thread) plus kBufBytes of stores per phase ----
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(mbar + i), 1);
        mbar_fence_init();
        *gave_up = 0u;
    }
    cluster.sync();                      // every CTA's mbarriers exist before anyone can signal them
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mbar_expect(smem_u32(mbar + i), kBufBytes);
    }

    for (long long grp = cluster_id; grp < ngroups; grp += nclusters) {
        tile0 = grp * G;
        // ---- weights and initial metrics (src/trellis/qtip.py:161-165) ----
        for (int i = tid; i < G * kT; i += NT) {
            const long long tile = tile0 + (i >> 8);
            int t = i & 255;
            const float x = tile < a.n ? load_weight(a, tile, i & 255, t) : 0.0f;
            wv[(i & ~255) | t] = x;
            if ((a.flags & kFwdCheckFinite) && !isfinite(x) && rank == 0 && a.status != nullptr) atomicOr(a.status, 2u);   // reported, never trapped on
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

        // The two tile sets alternate; every step_set waits for its input buffer's bytes, computes,
        // waits for the previous step_set's barrier phase before its first store, stores, arrives.
        // (two steps per trip, so that the buffer index is a constant in every instance of step_set)
        step_set(0, 0, 0);
        for (int t = 0; t < kT; t += 2) {
            step_set(1, t, 0);
            step_set(0, t + 1, 1);
            step_set(1, t + 1, 1);
            if (t + 2 < kT) step_set(0, t + 2, 0);
        }
        cluster_wait_relaxed();          // closes the phase opened by the last step_set
        wait_pending = false;
        wait_buffer(0, 0, false);        // step 255 wrote the final metrics into buffer 0
        wait_buffer(1, 0, false);
        // The barrier phase above was entered at the START of the last step_set, so it says nothing
        // about that step's backpointer bytes; the rows are CTA-local, a CTA barrier orders them.
        __syncthreads();
        flush_set(0, kT - 1, (kT - 1) & 1, tile0);
        flush_set(1, kT - 1, (kT - 1) & 1, tile0);

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
    if (timed_out && a.status != nullptr) atomicOr(a.status, 1u);
}

}  // namespace tcq
