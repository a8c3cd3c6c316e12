/*
 * nanoquant_b200 — C ABI of the sm_100a kernels for the NanoQuant binary
 * low-rank quantised linear
 *
 *     y = s_out * (U_b . (s_mid * (V_b . (s_in * x))))
 *
 * with V_b [R, N] and U_b [M, R] packed ±1 matrices (bit 1 = -1, bit 0 = +1),
 * N = in_features, R = rank, M = out_features, T = tokens.
 *
 * Every pointer is a DEVICE pointer unless its name ends in `_host`.  No torch
 * types cross this boundary.  All functions are asynchronous on `stream`
 * (a `cudaStream_t`), never synchronise the device, never allocate unless the
 * comment says so, and return 0 (NQ_OK) or a negative nq_status.  They do not
 * throw.  The library is built for sm_100a only and has no CPU fallback.
 *
 * The citations name the reference interface (SamsungLabs/NanoQuant, paths
 * relative to that project) that each entry point replaces.
 */
#ifndef NANOQUANT_B200_H
#define NANOQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* nq_stream_t; /* == cudaStream_t */

typedef enum {
    NQ_OK = 0,
    NQ_ERR_NULL = -1,        /* a required pointer is NULL */
    NQ_ERR_SHAPE = -2,       /* a dimension is <= 0 or violates a divisibility rule */
    NQ_ERR_DTYPE = -3,       /* dtype is not NQ_F16 / NQ_BF16, or method id unknown */
    NQ_ERR_ALIGN = -4,       /* a pointer is not aligned as required (16 bytes) */
    NQ_ERR_SCRATCH = -5,     /* scratch / workspace buffer too small */
    NQ_ERR_CUDA = -6,        /* a CUDA runtime call failed; see nq_last_cuda_error() */
    NQ_ERR_TIMEOUT = -7,     /* a bounded device-side wait gave up (read from a status word) */
    NQ_ERR_UNSUPPORTED = -8, /* shape outside what the kernels implement */
    NQ_ERR_TOO_LARGE = -9    /* size beyond a stated fixed maximum */
} nq_status;

typedef enum { NQ_F16 = 0, NQ_BF16 = 1 } nq_dtype;

/* Bit order inside a 32-column word.
 * reference: src/nanoquant/kernel/utils.py:99-104 */
typedef enum {
    NQ_LSB_FIRST = 0, /* element k -> bit k (checkpoint layout) */
    NQ_HALF2 = 1      /* element 2j -> bit 15-j, element 2j+1 -> bit 31-j (GEMV runtime layout) */
} nq_bit_order;

/* Library / ABI identification. */
int nq_abi_version(void);
const char* nq_strerror(int status);
/* Text of the last CUDA runtime error seen by this thread inside the library. */
const char* nq_last_cuda_error(void);

/* ------------------------------------------------------------------------ *
 * Pack / layout kernels (bit-exact with the reference's PyTorch packers)
 * ------------------------------------------------------------------------ */

/* ±1 int8 [rows, cols] -> int32 [rows, ceil(cols/32)], padding columns +1.
 * replaces: pack_binary_gemv, src/nanoquant/kernel/utils.py:51-113 */
int nq_pack_rows(const int8_t* w, int32_t* packed, int64_t rows, int64_t cols,
                 int bit_order, nq_stream_t stream);

/* inverse of nq_pack_rows.
 * replaces: unpack_binary_gemv, src/nanoquant/kernel/utils.py:116-183 */
int nq_unpack_rows(const int32_t* packed, int8_t* w, int64_t rows, int64_t cols,
                   int bit_order, nq_stream_t stream);

/* Re-order the bits of every word from one nq_bit_order to another without
 * materialising the dense ±1 matrix (checkpoint layout -> GEMV runtime layout).
 * replaces: the unpack-to-bf16 + re-pack detour of
 * src/nanoquant/utils/load_utils.py:279-287 and src/nanoquant/modules/linear.py:171-172 */
int nq_reorder_words(const int32_t* in, int32_t* out, int64_t n_words,
                     int order_in, int order_out, nq_stream_t stream);

/* ±1 int8 weight [out_f, in_f] (out_f % 64 == 0, in_f % 16 == 0) ->
 * int32 B [in_f/16, out_f/2] in the Marlin mma-fragment order.
 * replaces: the bit part of pack_binary_marlin, src/nanoquant/kernel/utils.py:191-205 */
int nq_pack_marlin(const int8_t* w, int32_t* B, int64_t out_f, int64_t in_f,
                   nq_stream_t stream);

/* inverse of nq_pack_marlin: B [in_f/16, out_f/2] -> row-packed words
 * [out_f, in_f/32] in `bit_order` (in_f % 32 == 0).  Lets operands prepared
 * with the reference's Marlin packer be consumed by the kernels here. */
int nq_marlin_to_rows(const int32_t* B, int32_t* packed, int64_t out_f, int64_t in_f,
                      int bit_order, nq_stream_t stream);

/* Scale permutations of the Marlin packer on 16-bit elements.
 * kind 0: per group of 16, new[4b+2a+c] = old[8a+2b+c]  (utils.py:206-207)
 * kind 1: per group of 32, new[8b+2a+c] = old[8a+2b+c]  (utils.py:208-209)
 * inverse != 0 applies the inverse permutation. */
int nq_permute_scale16(const void* s, void* out, int64_t n, int kind, int inverse,
                       nq_stream_t stream);

/* ------------------------------------------------------------------------ *
 * Runtime tile layout of the GEMV kernel
 * ------------------------------------------------------------------------ */

/* Bytes of the tile layout of a packed [rows, cols] matrix:
 * ceil(rows/16) * ceil(cols/256) tiles of 512 bytes. */
size_t nq_tiles_bytes(int64_t rows, int64_t cols);

/* rows layout (int32 [rows, ceil(cols/32)] in `bit_order`) -> tile layout.
 * A tile covers 16 rows x 256 columns, stored as 32 lanes x 16 bytes, tiles
 * ordered [row_group][chunk]; lane 4g+q holds the words {row g cols h=0, row g+8
 * h=0, row g h=1, row g+8 h=1} and the weight of chunk column 32j + 16h + 4q + b
 * sits at bit 8b + j of its word.  Rows / columns beyond the matrix are +1.
 * replaces: the `binary_packer(..., method="half2")` re-pack of
 * src/nanoquant/modules/linear.py:171-172 (runtime layout of the reference GEMV) */
int nq_rows_to_tiles(const int32_t* packed, void* tiles, int64_t rows, int64_t cols,
                     int bit_order, nq_stream_t stream);

/* inverse of nq_rows_to_tiles. */
int nq_tiles_to_rows(const void* tiles, int32_t* packed, int64_t rows, int64_t cols,
                     int bit_order, nq_stream_t stream);

/* ------------------------------------------------------------------------ *
 * Decode GEMV (small T)
 * ------------------------------------------------------------------------ */

/* One quantised linear y[T, M] = s_out * (U . (s_mid * (V . (s_in * x[T, N])))) + bias + residual.
 * v_tiles / u_tiles are V [R, N] and U [M, R] in the tile layout, s_mid may be
 * NULL; x, y, the scales, bias and residual share one dtype; ldx / ldy / ldr are row strides in
 * elements.  bias [M] and residual [T, ldr] may be NULL (zero the struct before filling it); they are
 * added in fp32 after the output scale and before the saturation, i.e. y = sat(s_out * (...) + bias + residual).
 * bias matches the add of src/nanoquant/modules/linear.py:148-149, which the reference's kernel branches
 * (linear.py:121-141) leave out; the residual is the decoder layer's skip connection.
 * residual may alias y (each output element is read, then written, by one thread). */
typedef struct {
    const void* x;
    const void* s_in;
    const void* v_tiles;
    const void* s_mid;
    const void* u_tiles;
    const void* s_out;
    void* y;
    int N, R, M;
    int64_t ldx, ldy;
    const void* bias;
    const void* residual;
    int64_t ldr;
} nq_linear_desc;

/* Bytes of scratch nq_gemv_fwd / nq_gemv_group_fwd need (0 on invalid sizes). */
size_t nq_gemv_scratch_bytes(int T, int N, int R, int M);
size_t nq_gemv_group_scratch_bytes(const nq_linear_desc* linears_host, int n_linears, int T);

/* The decode GEMV.  Accumulation is exact integer arithmetic on a 16-bit
 * fixed-point image of (s_in * x) and of the rank-R intermediate (per-token
 * scale), results are converted once per output in fp32.  `scratch` holds a
 * 256-byte header (a free-running launch counter + status word) followed by
 * the fp32 intermediate, each element stored with the tag of the launch that
 * wrote it (8 bytes per element); it must be 16-byte aligned, at least
 * nq_gemv_scratch_bytes() long and ZEROED ONCE, AS A WHOLE, by the caller after
 * allocation (never the header alone: the tags of the elements refer to the
 * counter).  Calls that share a scratch buffer must be ordered on one stream.
 * T > 4 is processed as several launches.
 * fp16 outputs saturate at +-64504, bf16 at +-3.3895e38 like the reference.
 * replaces: nanoquant_dyn_forward, src/nanoquant/kernel/cuda/gemv_kernel.cu:308-429
 * (schema src/nanoquant/kernel/pybind.cpp:85-90) */
int nq_gemv_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                const void* u_tiles, const void* s_out, void* y,
                void* scratch, size_t scratch_bytes,
                int T, int N, int R, int M, int dtype, nq_stream_t stream);

/* Up to 4 linears whose two phases run together in ONE launch (q/k/v or
 * gate/up of a decoder layer).  `linears_host` is a HOST array; its pointers are
 * device pointers.  Same scratch contract as nq_gemv_fwd with
 * nq_gemv_group_scratch_bytes().
 * replaces: consecutive nanoquant_dyn_forward calls issued by
 * src/nanoquant/modules/linear.py:121-130 for projections that share a layer input */
int nq_gemv_group_fwd(const nq_linear_desc* linears_host, int n_linears, int T, int dtype,
                      void* scratch, size_t scratch_bytes, nq_stream_t stream);

/* nq_gemv_fwd for callers that cannot hand the library any device memory of their own
 * beyond inputs and outputs: code running where allocation is forbidden or already frozen
 * (inside a serving loop whose memory plan is fixed, a plugin host that owns the allocator,
 * a capture-only phase).  It has NO counterpart in the reference.  The intermediate and the
 * launch counter live in a fixed array inside the library image (about 256 KB, present on
 * every GPU that loads the library until the process exits); nothing is allocated or freed,
 * here or in any library it calls.  Limits: rank R <= nq_gemv_static_max_rank() (8192),
 * otherwise NQ_ERR_TOO_LARGE; T > 4 runs as several launches like nq_gemv_fwd.
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress)
 * and keeps it for the life of the process: make that first call outside any stream
 * capture, and do not reset the device's primary context afterwards (the kept address
 * would be stale).  Nothing has to start at zero between
 * calls (the array is zero when the library is loaded; every launch tags its intermediate
 * with a fresh value of the counter), but every call reuses the same array, so two calls
 * that can overlap on the GPU (different streams, or threads, without ordering) race on
 * it: order them. */
int nq_gemv_fwd_static(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                       const void* u_tiles, const void* s_out, void* y,
                       int T, int N, int R, int M, int dtype, nq_stream_t stream);
size_t nq_gemv_static_max_rank(void);

/* Synchronises `stream` and returns the status word of a scratch buffer:
 * NQ_OK, or NQ_ERR_TIMEOUT when a device-wide wait of an earlier launch gave up
 * (the scratch must then be zeroed again before reuse; until then launches on it do
 * not spin at all and their results are void).  scratch == NULL reports the array of
 * nq_gemv_fwd_static on the current device. */
int nq_scratch_status(const void* scratch, nq_stream_t stream);

/* Number of polls a wait for the tagged intermediate may spend before it gives up
 * (per thread and launch: after its first expiry a thread does not spin again).
 * 0 restores the default (4e6, seconds).  Host-side setting read at launch time;
 * returns the previous value.  For failure-path tests and for callers that want a
 * tighter bound. */
unsigned nq_gemv_set_wait_limit(unsigned polls);

/* ------------------------------------------------------------------------ *
 * Prefill GEMM (many tokens) on tcgen05 / tensor memory
 * ------------------------------------------------------------------------ */

/* Bytes of scratch nq_gemm_fwd needs: a 256-byte header (status word at byte 8,
 * the same place as in the GEMV scratch; tile counters of the split-K path in
 * bytes 32..255) followed by the rank-R intermediate t[T, R] in the I/O dtype
 * and, for up to 24 tokens, the fp32 partial sums of the k splits (above that
 * a k split runs over the CTAs of a thread-block cluster and needs no scratch). */
size_t nq_gemm_scratch_bytes(int T, int N, int R, int M);

/* Precision of the rank-R intermediate of bf16 linears in the GEMM path (process-wide; returns the old setting).
 * 0 (default): t is rounded to bf16 between the stages, as the reference's Marlin path keeps it in the I/O type;
 * that rounding alone is up to 1.6e-3 of the output's maximum (inside the parity bar, by a narrow margin).
 * 1: t is kept as fp16 times a per-token power of two found by one more small kernel per launch group (a bound
 * on |t| from sum_k |s_in[k] x[k]| and max|s_mid|); the error beyond the output's own rounding drops to the fp16
 * path's level (0.5e-3 of the maximum) at 12-21 % more time (least at 2048 tokens, most at 16).
 * fp16 linears are not affected. */
int nq_gemm_set_precise_intermediate(int on);

/* y[T, M] = s_out * (U . (s_mid * (V . (s_in * x[T, N])))) as two tensor-core
 * GEMMs.  v_tiles / u_tiles are the same tile layout the GEMV reads.  The
 * intermediate is rounded to the I/O dtype between the stages, accumulation is
 * fp32, the products x * (+-s_in) are exact.  Requires N % 8 == 0, R % 8 == 0,
 * 16-byte aligned x, y, scales and scratch.  The scratch header must be zeroed
 * once by the caller (the tile counters return to zero by themselves); a
 * device-side wait that gives up sets its status word (nq_scratch_status).
 * Consecutive launches overlap through programmatic dependent launch: a
 * kernel loads activations and stores results only after the previous kernel
 * of the stream has completed.
 * replaces: marlin_nanoquant_cuda, src/nanoquant/kernel/cuda/gemm.cpp:112-122
 * (schema src/nanoquant/kernel/pybind.cpp:99-104) */
int nq_gemm_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                const void* u_tiles, const void* s_out, void* y,
                void* scratch, size_t scratch_bytes,
                int T, int N, int R, int M, int dtype, nq_stream_t stream);

/* The same for up to four linears that share the token count (q/k/v, gate/up; the
 * descriptors of nq_gemv_group_fwd, with ldx / ldy honoured): one launch per
 * stage for the whole group, which matters for few tokens, where a single linear
 * leaves most SMs idle.  No counterpart in the reference (its callers run one
 * linear per call).  Scratch: nq_gemm_group_scratch_bytes(), zeroed once. */
size_t nq_gemm_group_scratch_bytes(const nq_linear_desc* linears_host, int n_linears, int T);
int nq_gemm_group_fwd(const nq_linear_desc* linears_host, int n_linears, int T, int dtype,
                      void* scratch, size_t scratch_bytes, nq_stream_t stream);

/* One stage: y[T, Nout] = s_out * (W . (s_in * x[T, K])) with W [Nout, K] in the
 * tile layout; s_in and s_out may be NULL.  `status_word` points at a zeroed
 * 16-byte device area (a scratch header works) whose third word receives a
 * timeout status.
 * replaces: marlin_onebit_cuda, src/nanoquant/kernel/cuda/gemm.cpp:59-98
 * (schema src/nanoquant/kernel/pybind.cpp:93-98) */
int nq_onebit_gemm_fwd(const void* x, const void* tiles, const void* s_in, const void* s_out,
                       void* y, void* status_word, int T, int K, int Nout, int dtype,
                       nq_stream_t stream);

/* ------------------------------------------------------------------------ *
 * Tensor parallelism: all-gather of the output shards over peer memory
 * ------------------------------------------------------------------------ */

/* All-gather of [T, M/G] output shards as ONE small kernel per call (plain peer stores over NVLink, a
 * flag word per rank, a bounded wait), so that a tensor-parallel step can be captured in a CUDA graph
 * together with the GEMV / GEMM launches.  The reference has no distributed code; the portable
 * alternative is an NCCL all-gather (nanoquant_b200/tp.py uses either).
 * Every rank owns a buffer of the same layout whose base pointers (peer-accessible, 16-byte aligned,
 * e.g. from symmetric memory) are passed by every rank in rank order: nq_allgather_flags_bytes() of
 * flag words, zeroed once, at `flags_offset`, and gathered regions.  The call copies `shard`
 * (shard_bytes, a multiple of 16) into slot `rank` of the region at `region_offset` in EVERY rank's
 * buffer, signals the peers and waits until all ranks' shards have arrived in this rank's region;
 * kernels launched afterwards on `stream` see the gathered [G][shard] data.  `local_state`:
 * nq_allgather_state_bytes() of local device memory, zeroed once, one per communicator.  All ranks
 * must issue the same sequence of calls; consecutive calls must use different regions (a rank may be
 * one call ahead of a peer).  nq_allgather_status() synchronises and reports an expired wait (NQ_ERR_TIMEOUT). */
size_t nq_allgather_state_bytes(void);
size_t nq_allgather_flags_bytes(int world);
int nq_allgather_push(const void* shard, size_t shard_bytes, void* const* rank_bases_host,
                      size_t flags_offset, size_t region_offset, void* local_state,
                      int world, int rank, nq_stream_t stream);
int nq_allgather_status(const void* local_state, nq_stream_t stream);
/* Polls (64 ns apart) the wait for a peer's shard may spend before it gives up; 0 restores the default (4e6).
 * After an expiry the status word of `local_state` stays set and later launches on it poll once and go on
 * (zero the state to re-arm it).  Returns the previous value. */
unsigned nq_allgather_set_wait_limit(unsigned polls);

/* Token-count dispatch the reference leaves to the caller's `kernel_type`:
 * the GEMV for T <= nq_gemv_max_tokens(), the GEMM above.  Scratch must satisfy
 * nq_linear_scratch_bytes(). */
int nq_gemv_max_tokens(void);
size_t nq_linear_scratch_bytes(int T, int N, int R, int M);
int nq_linear_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                  const void* u_tiles, const void* s_out, void* y,
                  void* scratch, size_t scratch_bytes,
                  int T, int N, int R, int M, int dtype, nq_stream_t stream);

/* Dense 16-bit GEMV for the layers the reference leaves un-quantised in a decode step, above all
 * `lm_head`: y[t, v] = sum_k x[t, k] * w[v, k] (+ bias[v]), w [V, N] row-major with `ldw` elements
 * between rows (N % 8 == 0, ldw % 8 == 0, w and x 16-byte aligned), x [T, N] contiguous, y [T, V] with
 * `ldy` elements between tokens, bias nullable, fp32 accumulation, 1 <= T <= nq_dense_gemv_max_tokens()
 * (NQ_ERR_UNSUPPORTED above: use a GEMM).  HBM bound: w is streamed once per launch; all tokens of a
 * launch sit in shared memory, and where 9-16 tokens of a very wide row do not fit they go in two launches.
 * replaces: the nn.Linear `lm_head` call of the HF model forward that the reference's decode loop
 * runs per token (src/nanoquant/kernel/test_decode.py:385-417); lm_head is excluded from quantisation
 * (src/nanoquant/utils/load_utils.py:322). */
int nq_dense_gemv_max_tokens(void);
int nq_dense_gemv_fwd(const void* x, const void* w, const void* bias, void* y, int T, int N, int V,
                      int64_t ldw, int64_t ldy, int dtype, nq_stream_t stream);

/* ------------------------------------------------------------------------ *
 * Measurement probes (no counterpart in the reference; nothing on the hot path calls them)
 * ------------------------------------------------------------------------ */

/* SYNCHRONOUS, allocate and free their own device memory, run on streams of their own: call them from a benchmark,
 * not from serving code.
 * nq_probe_chain: microseconds per launch of the dependent chain of a decode launch with the arithmetic taken out
 * (dependency wait, broadcast load of an 8 KB input by every CTA, tagged hand-over of a rank-R vector between all
 * CTAs, barriers, output store; 100 cooperative launches with programmatic stream serialization in a CUDA graph,
 * replayed 10 times) for `ctas` CTAs; `pause_ns` > 0 sleeps that long before the first poll.
 * nq_probe_loop: GB/s of packed factors through the GEMV's item loop fed from shared memory only (mode 0: the
 * arithmetic ceiling), through a cp.async ring (mode 1) or through registers (mode 2); one CTA per SM,
 * `items_per_warp` KB per warp (a multiple of 4, at most 1024). */
int nq_probe_chain(int ctas, int R, int pause_ns, float* us_per_launch_host);
int nq_probe_loop(int mode, int items_per_warp, float* gbs_host);

#ifdef __cplusplus
}
#endif
#endif /* NANOQUANT_B200_H */
