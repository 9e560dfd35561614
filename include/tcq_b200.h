/*
 * C ABI of the B200 trellis codec (tail-biting bitshift-trellis Viterbi encoder
 * and decoder, L = 16-bit state, T = 256 weights per tile, K = 2, 3 or 4 bits per
 * weight, computed codebooks).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless its name ends
 *     in _host.  The library never allocates or frees device memory; scratch is
 *     passed in as `ws` (size from tcq_workspace_bytes()).
 *   - `stream` is a cudaStream_t passed as void*.  All work is queued on it and
 *     the call returns without synchronising.  Calls on different streams may
 *     overlap if they use different workspaces.
 *   - Return value: TCQ_OK (0) or a negative TCQ_E_* code; tcq_strerror() gives
 *     the text.  Nothing is launched when an argument is rejected.
 *   - Tiles are rows of 256 consecutive fp32 values; tile i starts at w + 256*i.
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     returns TCQ_E_CUDA.
 *
 * Each entry point names the reference interface (file:line inside
 * Azimml/trellis-everywhere) that it replaces.
 */
#ifndef TCQ_B200_H
#define TCQ_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TCQ_API __attribute__((visibility("default")))
#else
#define TCQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define TCQ_T 256      /* weights per tile (src/trellis/qtip.py:23 T_SEQ) */
#define TCQ_L 16       /* trellis state bits (src/trellis/qtip.py:21 L) */

/* Codebook ids: the keys of CODEBOOKS, src/trellis/qtip.py:56. */
#define TCQ_CB_1MAD 0  /* src/trellis/qtip.py:32-37 cb_1mad  */
#define TCQ_CB_3INST 1 /* src/trellis/qtip.py:40-45 cb_3inst */
#define TCQ_CB_MCG 2   /* src/trellis/qtip.py:48-53 cb_mcg   */

#define TCQ_OK 0
#define TCQ_E_BAD_K (-1)         /* K not in {2,3,4} */
#define TCQ_E_BAD_CODEBOOK (-2)  /* codebook id unknown */
#define TCQ_E_BAD_COUNT (-3)     /* negative tile / element count */
#define TCQ_E_NULL_POINTER (-4)  /* a required pointer is NULL */
#define TCQ_E_MISALIGNED (-5)    /* pointer not aligned as documented */
#define TCQ_E_WORKSPACE (-6)     /* workspace smaller than tcq_workspace_min_bytes() */
#define TCQ_E_CUDA (-7)          /* CUDA runtime error (no device, launch failure) */
#define TCQ_E_BAD_ARGUMENT (-8)  /* other invalid argument (roll, T, ...) */
#define TCQ_E_NONFINITE_INPUT (-11) /* tcq_workspace_status: a weight of the last call was NaN or infinite */
#define TCQ_E_DEVICE_TIMEOUT (-10) /* a bounded in-kernel wait gave up (tcq_workspace_status) */
#define TCQ_E_TOO_MANY_TILES (-9) /* batch larger than tcq_encode_tb_static_max_tiles(K) */

/* Version of this ABI (bumped on any signature change). */
TCQ_API int tcq_abi_version(void);

/* Text for a return code.  Never NULL. */
TCQ_API const char *tcq_strerror(int code);

/* Text of the last CUDA error seen by this library on the calling thread. */
TCQ_API const char *tcq_last_cuda_error(void);

/*
 * Scratch sizing.  tcq_workspace_bytes(): the size with which tcq_encode_tb /
 * tcq_viterbi_pass process n_tiles at full speed (backpointers of up to one
 * chunk of tiles, K bits per trellis edge per step, plus per-tile hand-off
 * words).  tcq_workspace_min_bytes(): the smallest accepted size (one tile per
 * SM-resident group); anything in between just means smaller chunks.
 * Replaces the per-batch torch.empty scratch of
 * src/trellis/viterbi_triton.py:96-102.  Returns 0 for invalid K.
 */
TCQ_API size_t tcq_workspace_bytes(int64_t n_tiles, int K);
TCQ_API size_t tcq_workspace_min_bytes(int K);

/*
 * Tail-biting encode of n_tiles tiles.
 * Replaces viterbi_tb (src/trellis/qtip.py:124-144) and viterbi_tb_triton
 * (src/trellis/viterbi_triton.py:121-129), with pack_bits_np
 * (scripts/export_packed_8b.py:52-62) fused into the traceback.
 *   w       [n_tiles,256] fp32, 16-byte aligned, never written
 *   packed  [n_tiles, 8*K] u32: bit kb of symbol t at bit (255-t)*K+kb   (required)
 *   bits    [n_tiles,256] int64 symbols (< 2^K), or NULL
 *   dq      [n_tiles,256] fp32 reconstruction codebook[state_t], or NULL
 *   sse     [n_tiles] fp32 sum_t (w_t-dq_t)^2 accumulated in time order, or NULL
 *   ws      scratch, 256-byte aligned, ws_bytes >= tcq_workspace_min_bytes(K)
 */
TCQ_API int tcq_encode_tb(const float *w, int64_t n_tiles, int K, int codebook, uint32_t *packed, int64_t *bits,
                  float *dq, float *sse, void *ws, size_t ws_bytes, void *stream);

/*
 * Tail-biting encode of one LDLQ row block, in place in the recursion's own matrices.
 * Replaces the enc closure of src/trellis/ldlq.py:136-143 (and its bits-capturing twin,
 * scripts/export_packed_8b.py:117-125): the two transposing copies around the encoder, the
 * "rows = bW + comp" addition before it (ldlq.py:94) and the "bW - bWq" error after it
 * (ldlq.py:90,97) are done by the kernels' own loads and stores.
 *   src     [16][ld] fp32: 16 consecutive input-channel rows of the transposed matrix (k_in x n_out,
 *           row-major, leading dimension ld >= n_out); n_out a multiple of 16
 *   comp    [16][ld] fp32 feedback owed to these rows, or NULL; the block encoded is fl(src + comp)
 *   tile i  = columns 16i .. 16i+15, weight t = (column % 16) * 16 + row   (ldlq.py:138-140)
 *   packed  code words of tile i at packed + i * packed_stride (u32 units, packed_stride >= 8*K), or NULL;
 *           with packed_stride = (k_in/16) * 8K and packed pointing at the block's column of the
 *           [n_out/16][k_in/16][8K] array, the calls of one matrix fill the exporter's tile order directly
 *   wq      [16][ld] fp32 out: reconstruction in the same layout (required)
 *   err     [16][ld] fp32 out: src - wq (the uncompensated error the recursion feeds back), or NULL
 *   sse     [n_out/16] fp32 out: squared error of each tile against src + comp, or NULL
 *   ws      as tcq_encode_tb, sized for n_out/16 tiles
 * src and comp are only read; wq and err must not overlap them or each other.
 * Codes and reconstruction are bit-identical to tcq_encode_tb on the transposed copy.
 */
TCQ_API int tcq_encode_tb_rows(const float *src, const float *comp, int64_t ld, int64_t n_out, int K, int codebook,
                               uint32_t *packed, int64_t packed_stride, float *wq, float *err, float *sse, void *ws,
                               size_t ws_bytes, void *stream);

/*
 * One Viterbi pass: the optimal state path of each tile.
 * Replaces _viterbi_pass (src/trellis/qtip.py:147-196) and viterbi_pass_triton
 * (src/trellis/viterbi_triton.py:81-118).
 *   overlap [n_tiles] int32 edge (< 2^(16-K)) that the path must start from and
 *           end at, or NULL for the unconstrained pass
 *   roll    0, or 128 to run on the tile rotated by half its length
 *           (torch.roll(w, 128, dims=1), src/trellis/qtip.py:138) without a copy
 *   states  [n_tiles,256] int64 out
 */
TCQ_API int tcq_viterbi_pass(const float *w, int64_t n_tiles, int K, int codebook, const int32_t *overlap, int roll,
                     int64_t *states, void *ws, size_t ws_bytes, void *stream);

/*
 * tcq_encode_tb for callers that cannot allocate device memory (no counterpart in the
 * reference, which allocates its scratch with torch.empty on every call).
 * Same inputs, outputs and results as tcq_encode_tb, but no workspace argument: the
 * backpointer scratch is a fixed TCQ_STATIC_SCRATCH_BYTES array inside the library's device
 * image, so the call performs no cudaMalloc / cudaFree and uses no allocating library.
 *   - at most tcq_encode_tb_static_max_tiles(K) tiles per call (31 / 42 / 63 for K = 2 / 3 / 4);
 *     more returns TCQ_E_TOO_MANY_TILES and launches nothing;
 *   - every GPU context that loads the library holds the array until the process exits;
 *   - the first call on a device resolves the array's address (cudaGetSymbolAddress, with
 *     that device current); make it before any stream capture begins;
 *   - all calls share the array: calls that may overlap on the GPU must be serialised by
 *     the caller.  Nothing needs clearing between calls.
 */
#define TCQ_STATIC_SCRATCH_BYTES (32u << 20)
TCQ_API int64_t tcq_encode_tb_static_max_tiles(int K);
TCQ_API int tcq_encode_tb_static(const float *w, int64_t n_tiles, int K, int codebook, uint32_t *packed, int64_t *bits,
                                 float *dq, float *sse, void *stream);
/*
 * tcq_workspace_status for the static-scratch path: health of the LAST tcq_encode_tb_static call on the
 * current device (TCQ_OK, TCQ_E_DEVICE_TIMEOUT or TCQ_E_NONFINITE_INPUT).  Synchronises the stream and
 * copies one word to the host; allocates nothing.  No reference counterpart.
 */
TCQ_API int tcq_encode_tb_static_status(void *stream);

/*
 * The forward sweep of one pass alone (no traceback): runs the Viterbi step kernel
 * exactly as tcq_encode_tb does for one chunk and leaves the packed backpointers of
 * the last bp_steps steps (256, or 128 as in the encoder's first pass) in `ws`.
 * For profiling and roofline measurements of the step kernel; it replaces the
 * same reference code as tcq_viterbi_pass (src/trellis/qtip.py:177-182,
 * src/trellis/viterbi_triton.py:24-78).  n_tiles must fit one chunk of the
 * workspace (otherwise TCQ_E_WORKSPACE).
 */
TCQ_API int tcq_forward_pass(const float *w, int64_t n_tiles, int K, int codebook, const int32_t *overlap, int roll,
                             int bp_steps, void *ws, size_t ws_bytes, void *stream);

/*
 * Health check of the last tcq_encode_tb / tcq_viterbi_pass / tcq_forward_pass call that used
 * this workspace with the same n_tiles and K.  The step kernel's CTAs exchange path metrics
 * through shared memory of neighbouring SMs and wait for them with a bounded number of polls;
 * a wait that runs out sets a flag in the workspace instead of hanging.  This call copies the
 * flag to the host and SYNCHRONISES the stream (the only entry point that does): TCQ_OK,
 * TCQ_E_DEVICE_TIMEOUT if the outputs of that call must not be used, or TCQ_E_NONFINITE_INPUT if
 * some weight was NaN or infinite (the kernels never trap on such input; they encode it to
 * meaningless codes and flag it here).  No reference counterpart.
 */
TCQ_API int tcq_workspace_status(const void *ws, size_t ws_bytes, int64_t n_tiles, int K, void *stream);

/*
 * Self-test of the bounded waits: runs one pass of the step kernel on 1..8 tiles while telling
 * the buffers of the final path metrics to expect 16 bytes more than will ever arrive.  The last
 * wait of every thread then runs out after its time limit (about a quarter of a second), the kernel
 * finishes normally, and tcq_workspace_status afterwards must report TCQ_E_DEVICE_TIMEOUT.  Nothing faults, traps or spins without limit.  Returns TCQ_E_BAD_ARGUMENT
 * if the device runs the single-CTA step kernel (which has no such waits).  No reference counterpart.
 */
TCQ_API int tcq_selftest_wait_timeout(const float *w, int64_t n_tiles, int K, void *ws, size_t ws_bytes, void *stream);

/*
 * Number of kernel launches tcq_encode_tb issues for n_tiles with a workspace of
 * ws_bytes (four per chunk: step kernel and traceback for each of the two passes),
 * or a negative TCQ_E_* code.  No reference counterpart; used for accounting.
 */
TCQ_API int64_t tcq_encode_launches(int64_t n_tiles, int K, size_t ws_bytes);

/*
 * Decode packed tiles: dq[i,t] = codebook(16-bit window at bit (255-t)*K of tile
 * i's words, wrapping past the last word).  Replaces lut[states2]
 * (src/trellis/qtip.py:144), the wrapped-stream decode of tests/test_qtip.py:55-67
 * and the WGSL window decode wz() (web/kernels.js:115-122).
 *   packed [n_tiles, 8*K] u32, 4-byte aligned;  dq [n_tiles,256] fp32, 16-byte aligned
 */
TCQ_API int tcq_decode_packed(const uint32_t *packed, int64_t n_tiles, int K, int codebook, float *dq, void *stream);

/*
 * Matrix-vector products straight from packed codes: y[j][row] = sum_col Zq[row][col] * x[j][col],
 * Zq[row][col] = codebook(window at bit (255-t)*K of tile (row/16)*(k_in/16) + col/16,
 * t = (row%16)*16 + col%16), never materialised.  Replaces the DECODE_MATMUL shader
 * (web/kernels.js:105-128), which does the same for one vector with one thread per
 * output row; the incoherence-processing fold around it (web/packed.js:163-182)
 * stays with the caller.  fp32 accumulation in a fixed order (reproducible run to run).
 *   packed [n_out/16 * k_in/16, 8*K] u32;  n_out, k_in multiples of 16
 *   x [m][ldx] fp32 right-hand sides, 16-byte aligned, ldx >= k_in and a multiple of 4
 *   y [m][ldy] fp32 results, ldy >= n_out;  m >= 0 (decoded once per four right-hand sides)
 */
TCQ_API int tcq_decode_matvec(const uint32_t *packed, int64_t n_out, int64_t k_in, int K, int codebook, const float *x,
                      int64_t ldx, int m, float *y, int64_t ldy, void *stream);

/*
 * Incoherence processing on the device.  Replaces IPContext.__init__ / IPContext.restore
 * (src/trellis/qtip.py:238-268): row signs sv and column signs su (+-1, drawn by the
 * caller so that the reference's seeded CPU generator stays the source), per-row RMS
 * scales out_s and block-Hadamard over the row axis, per-column RMS scales in_s and
 * block-Hadamard over the column axis (blocks: largest power of two <= 128 dividing the
 * axis, qtip.py:208-223; fast Walsh-Hadamard transform instead of the dense matrix of
 * qtip.py:216-223), then one global scale so that z has RMS cb_rms.
 *   tcq_ip_forward:  w [n,k] fp32 -> z (tiled != 0: [n/16*k/16, 256] in the encoder's tile
 *                    order, qtip.py:288; tiled == 0: [n,k]), out_s [n], in_s [k], scale [1]
 *                    (all device memory; scale stays on the device so nothing synchronises)
 *   tcq_ip_restore:  zq (same two layouts) -> w_hat [n,k]
 *   n, k multiples of 16, n <= 16 * 65535;  z, zq and in_s 16-byte aligned;
 *   ws: tcq_ip_workspace_bytes(n,k) bytes, 256-byte aligned
 * Floating point: equal to the reference's matmul form up to fp32 summation order.
 */
TCQ_API size_t tcq_ip_workspace_bytes(int64_t n, int64_t k);
TCQ_API int tcq_ip_forward(const float *w, int64_t n, int64_t k, const float *sv, const float *su, float cb_rms, int tiled,
                   float *z, float *out_s, float *in_s, float *scale, void *ws, size_t ws_bytes, void *stream);
TCQ_API int tcq_ip_restore(const float *zq, int tiled, int64_t n, int64_t k, const float *sv, const float *su,
                   const float *out_s, const float *in_s, const float *scale, float *w_hat, void *ws, size_t ws_bytes,
                   void *stream);

/*
 * Decode unpacked symbol streams of any length T (no wrap): state_t is the last
 * 16 bits of s0 followed by symbols 0..t.  Replaces decode_recursive and
 * decode_window (src/trellis/qtip.py:70-110), which are equal by construction.
 *   bits [n,T] int64;  s0 [n] int64 start states or NULL (zeros);  out [n,T] fp32
 */
TCQ_API int tcq_decode_symbols(const int64_t *bits, int64_t n, int64_t T, int K, int codebook, const int64_t *s0,
                       float *out, void *stream);

/*
 * Pack symbols into the exporter's word layout.  Replaces pack_bits_np
 * (scripts/export_packed_8b.py:52-62) for callers that already hold symbols.
 *   bits [n_tiles,256] int64;  packed [n_tiles,8*K] u32
 */
TCQ_API int tcq_pack_symbols(const int64_t *bits, int64_t n_tiles, int K, uint32_t *packed, void *stream);

/*
 * Evaluate a computed codebook on all 65536 states.  Replaces codebook_lut
 * (src/trellis/qtip.py:59-66).   lut [65536] fp32
 */
TCQ_API int tcq_codebook_lut(int codebook, float *lut, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TCQ_B200_H */
