/*
 * C ABI of the B200 (sm_100a) W4A16 matmul path.
 *
 * This is the drop-in boundary for the AWQ int4 / group-128 / bf16-activation
 * linear layers of the reference server: the functions below are what its C++
 * launchers in src/kernels/gemv_w4a16.{cuh,cu} and src/kernels/gemm_w4a16.{cuh,cu}
 * bind to (the inline C++ shims with the reference's exact signatures live in
 * dropin/kernels/ of the package). Every pointer that names tensor data is a
 * DEVICE pointer; `stream` is a cudaStream_t passed as void*. Every function
 * returns 0 on success or a negative W4A16_E* code, never aborts, and leaves a
 * message for w4a16_last_error(). Nothing here synchronises the device or
 * allocates inside a launch, so all launchers can be captured into a CUDA graph
 * after one eager warm-up call.
 *
 * "file:line" below cites the reference interface each entry replaces, by the
 * file's path inside the reference project.
 */
#ifndef W4A16_B200_H_
#define W4A16_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define W4A16_OK 0
#define W4A16_EINVAL (-1)   /* bad argument: null/misaligned pointer, unsupported shape */
#define W4A16_ECUDA (-2)    /* a CUDA runtime call failed */
#define W4A16_ESCRATCH (-3) /* scratch / workspace too small for this call */
#define W4A16_ETIMEOUT (-4) /* a bounded device-side wait expired */
#define W4A16_ECOMM (-5)    /* shard descriptor inconsistent */

/* Kernel-private weight container; field-for-field the reference's
 * qwen::W4A16Weights (src/kernels/gemv_w4a16.cuh:50-60). The three buffers are
 * independent allocations, so callers may cudaFree them one by one as the
 * reference's callers do. Private layout (group_size 128): all weight data lives
 * in ONE stream behind `qweight`, so that a CTA fetches a whole 128-row x
 * 128-k group with one bulk copy; `scale` and `zp` are small placeholder
 * allocations kept only so that the reference's free-one-by-one pattern works.
 *   qweight [ceil(out_f/128)][G] blocks of 8576 B, block (t, g) =
 *             [4 chunks of 32 k][128 slots] uint4   row r of the tile, chunk c sits in
 *                                                  slot (r + 4*(c&1)) & 127 (bank rotation);
 *                                                  inside a word k-offset o is nibble
 *                                                  (o>>1) + 4*(o&1), stored value + 8
 *             [128] bf16 scales, [128] u8 zero-points (raw stored nibble, value + 8)
 *           rows past out_f in the last tile are zero. */
typedef struct w4a16_weights {
  uint32_t* qweight;
  uint16_t* scale; /* bf16 bits */
  uint8_t* zp;
  int out_f, in_f, group_size, num_groups;
} w4a16_weights_t;

/* Caller-owned scratch; field-for-field qwen::GemvScratch
 * (src/kernels/gemv_w4a16.cuh:94-110). Here: `partial` holds split-K partial
 * tiles, `xgsum` the per-(tile, warp) arrival counters (zero between calls),
 * `xf` the per-CTA (max, index) pairs of the fused argmax. One call in flight
 * per scratch, as in the reference. */
typedef struct w4a16_scratch {
  float* xf;
  float* xgsum;
  float* partial;
  int max_in, max_groups, max_out, max_splits, max_m;
  size_t partial_elems;
} w4a16_scratch_t;

/* Prefill workspace; mirrors qwen::GemmWorkspace (src/kernels/gemm_w4a16.cuh:30-38).
 * The fused prefill GEMM needs no dequantised tile and no library handle: `wbuf` is a
 * small placeholder allocation (the reference's callers free it themselves) and
 * `cublas` stays NULL. The activation tensor map travels as a kernel parameter. */
typedef struct w4a16_workspace {
  uint16_t* wbuf;
  size_t bytes;
  int max_rows;
  void* cublas;
} w4a16_workspace_t;

/* INT8 weight container of the lm_head variant; field-for-field qwen::W8A16Weights
 * (src/kernels/gemv_w4a16.cuh:148-155). Symmetric int8 codes in [-127,127], one bf16 scale
 * per (row, group of 128). Both buffers are independent allocations (the reference's
 * caller frees them one by one, src/model/model.cu:384-385); the whole stream - blocks of
 * 16640 B per (128-row tile, group): [8 chunks of 16 k][128 rows] 16 B of int8, then 128
 * bf16 scales - lives behind `qweight`, `scale` is a placeholder. */
typedef struct w4a16_w8_weights {
  int8_t* qweight;
  uint16_t* scale; /* bf16 bits */
  int out_f, in_f, group_size, num_groups;
} w4a16_w8_weights_t;

const char* w4a16_last_error(void);
/* Sticky device-side status of the last kernels on the current device (0 = ok,
 * W4A16_ETIMEOUT if a bounded wait expired). Synchronises the device. */
int w4a16_device_status(void);
/* Clears the status word of the current device (synchronises it first). After a
 * W4A16_ETIMEOUT: w4a16_device_status_clear(), then w4a16_scratch_reset() on every scratch
 * that was in use (and w4a16_gemv_static_reset() if that entry point was), then carry on. */
int w4a16_device_status_clear(void);
/* Launches one tiny kernel whose only wait is on a barrier nobody arrives at, with a limit
 * of `polls` tests: the wait gives up, the kernel sets W4A16_ETIMEOUT in the status word and
 * returns normally. Lets a caller (or a test) exercise the detection path end to end without
 * any fault or hang. polls in [1, 4096]. */
int w4a16_selftest_wait_timeout(int polls, void* stream);

/* awq_alloc_fused (gemv_w4a16.cuh:85, gemv_w4a16.cu:308-315): allocate the three buffers. */
int w4a16_weights_alloc(w4a16_weights_t* w, int out_f, int in_f, int group_size, void* stream);
/* awq_repack_into (gemv_w4a16.cuh:87-89, gemv_w4a16.cu:317-323): on-disk tensors
 * packed [out_f][in_f/8] u32, scale [out_f][G] bf16, zp [out_f/8][G] u32 -> private
 * layout, rows written at dst_row_offset (a multiple of 16). Asynchronous on `stream`; the next matmul call
 * on the same stream is ordered behind it by the library. A matmul on ANOTHER stream, or weight buffers
 * written by other means, need the caller's own event or synchronisation before the first launch that
 * reads them (the kernels fetch weights before they wait for the kernel in front of them). */
int w4a16_repack_into(const w4a16_weights_t* w, int dst_row_offset, const uint32_t* packed,
                      const uint16_t* scale, const uint32_t* zp, int out_f, void* stream);
/* awq_free (gemv_w4a16.cuh:90). */
int w4a16_weights_free(w4a16_weights_t* w);

/* gemv_scratch_alloc / gemv_scratch_free (gemv_w4a16.cuh:106-107, gemv_w4a16.cu:344-371). */
int w4a16_scratch_alloc(w4a16_scratch_t* s, int max_in, int max_out, int min_group, int max_m);
int w4a16_scratch_free(w4a16_scratch_t* s);
/* Zeroes the counters and the published split-tile pieces of a scratch on `stream`. Only needed
 * after a bounded wait expired (a launch that gave up may leave some behind); launches that
 * complete leave them at zero themselves. */
int w4a16_scratch_reset(w4a16_scratch_t* s, void* stream);
/* gemv_partial_check (gemv_w4a16.cuh:109): W4A16_ESCRATCH instead of abort. */
int w4a16_scratch_check(const w4a16_scratch_t* s, int out_f, int M);
/* gemv_choose_splits (gemv_w4a16.cuh:135): the number of CTAs that share one
 * output tile's K range under the persistent schedule (>= 1). */
int w4a16_choose_splits(int out_f, int num_groups);

/* gemv_w4a16 / gemv_w4a16_f32 (gemv_w4a16.cuh:129-132): y[out_f] = W x, x bf16 [in_f];
 * y is bf16 when y_is_f32 == 0, fp32 otherwise. */
int w4a16_gemv(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x,
               w4a16_scratch_t* s, void* stream);
/* No counterpart in the reference. The same GEMV for callers that must not allocate device
 * memory and so cannot own a w4a16_scratch_t: for example code that runs after the serving
 * process has given all remaining HBM to its KV cache, or that cannot afford the device-wide
 * synchronisation an allocation implies. The scratch is a fixed device array inside the library
 * (about 5.3 MB per GPU, held until exit); layers wider than 65536 rows, or devices with more
 * than 160 SMs, are refused with W4A16_EINVAL. The first call on a device looks the array up
 * and clears its counters, so make that call before capturing a stream. All calls share the
 * array: calls that overlap on the GPU race; calls in stream order are fine. */
int w4a16_gemv_static(void* y, int y_is_f32, const w4a16_weights_t* w, const uint16_t* x, void* stream);
/* Zeroes the counters and published pieces inside the built-in array of w4a16_gemv_static on `stream`
 * (recovery after W4A16_ETIMEOUT; allocates nothing). */
int w4a16_gemv_static_reset(void* stream);
/* gemm_small_w4a16 and gemm_mma_w4a16 (gemv_w4a16.cuh:124-125,187-188):
 * Y[M][out_f] = X[M][in_f] W^T, 1 <= M <= 16, row-major bf16, weights read once. */
int w4a16_gemm_skinny(uint16_t* y, const w4a16_weights_t* w, const uint16_t* x, int M,
                      w4a16_scratch_t* s, void* stream);
/* lm_head with the argmax fused. Replaces gemv_w4a16 / gemm_mma_w4a16 on lm_head
 * followed by argmax / argmax_rows (src/model/model.cu:796-815,1009-1051;
 * src/kernels/elementwise.cu:96-194): ids[m] = index of the largest bf16-rounded
 * logit of row m, lowest index on ties. `logits` (bf16 [M][out_f]) may be NULL.
 * `pairs` may be NULL; otherwise it receives M x {float best, int32 index} with
 * index = row + row_offset, for the cross-rank reduction of a vocab-sharded head. */
int w4a16_lm_head_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset,
                         const w4a16_weights_t* w, const uint16_t* x, int M,
                         w4a16_scratch_t* s, void* stream);
/* Reduce nranks x M gathered {float,int32} pairs (rank-major) to ids[M]:
 * larger value wins, then lower index. The cross-rank step of the sharded lm_head. */
int w4a16_argmax_pairs_reduce(int32_t* ids, const void* pairs, int nranks, int M, void* stream);

/* quantize_w8a16 (gemv_w4a16.cuh:157-158, gemv_w4a16.cu:479-499,610-617): allocate `dst` and
 * quantise src bf16 [out_f][in_f] (device) per (row, group): s = max|v|/127 stored as bf16,
 * q = clamp(rn(v * (127/max|v|)), -127, 127). group_size must be 128, out_f a multiple of 16. */
int w4a16_w8_quantize(w4a16_w8_weights_t* dst, const uint16_t* src, int out_f, int in_f,
                      int group_size, void* stream);
/* w8a16_free (gemv_w4a16.cuh:166). */
int w4a16_w8_free(w4a16_w8_weights_t* w);
/* Rows [row0,row0+nrows) back as plain tensors: q int8 [nrows][in_f], scale bf16 [nrows][G]
 * (either may be NULL). The check that anchors the INT8 path bit for bit; no reference
 * counterpart (its layout is never read back). */
int w4a16_w8_unpack_rows(int8_t* q, uint16_t* scale, const w4a16_w8_weights_t* w, int row0,
                         int nrows, void* stream);
/* gemv_w8a16 (gemv_w4a16.cuh:159-160, gemv_w4a16.cu:619-632): y bf16 [out_f] = W x. */
int w4a16_w8_gemv(uint16_t* y, const w4a16_w8_weights_t* w, const uint16_t* x,
                  w4a16_scratch_t* s, void* stream);
/* gemm_small_w8a16 (gemv_w4a16.cuh:164-165, gemv_w4a16.cu:570-608): Y[M][out_f], 1 <= M <= 16. */
int w4a16_w8_gemm_skinny(uint16_t* y, const w4a16_w8_weights_t* w, const uint16_t* x, int M,
                         w4a16_scratch_t* s, void* stream);
/* INT8 lm_head with the argmax fused; same contract as w4a16_lm_head_argmax. Replaces
 * gemv_w8a16 / gemm_small_w8a16 followed by argmax / argmax_rows
 * (src/model/model.cu:805-806,1049; src/kernels/elementwise.cu:96-194). */
int w4a16_w8_lm_head_argmax(int32_t* ids, uint16_t* logits, void* pairs, int row_offset,
                            const w4a16_w8_weights_t* w, const uint16_t* x, int M,
                            w4a16_scratch_t* s, void* stream);

/* A linear layer (M <= 16 tokens) with its elementwise neighbours fused in; every part is optional:
 *   ln_weight != NULL  RMSNorm in front (src/kernels/elementwise.cu:8-33, called at src/model/model.cu:681,774):
 *                      xn = bf16(x * rsqrt(mean(x^2) + ln_eps) * (1 + ln_weight)), the layer multiplies xn;
 *                      xn_out (may be NULL) receives xn [M][in_f] for callers that need it elsewhere.
 *   W4A16_EPILOGUE_SWIGLU    swiglu (elementwise.cu:40-49, model.cu:781): the weights hold gate and up rows
 *                      INTERLEAVED (w4a16_repack_into_swiglu), y is [M][out_f / 2]:
 *                      y = bf16(g / (1 + exp(-g)) * u) with g, u the bf16-rounded gate and up outputs.
 *   W4A16_EPILOGUE_RESIDUAL  residual_add (elementwise.cu:35-38, model.cu:777,785): y [M][out_f] is the running
 *                      hidden state, updated in place: y = bf16(float(y) + float(bf16(W x))).
 * The scratch must have been allocated with max_m >= 2 whenever ln_weight is given (the norm runs in the
 * pre-pass kernel that otherwise only serves M >= 2). */
#define W4A16_EPILOGUE_NONE 0
#define W4A16_EPILOGUE_SWIGLU 1
#define W4A16_EPILOGUE_RESIDUAL 2
int w4a16_linear_fused(uint16_t* y, const w4a16_weights_t* w, const uint16_t* x, int M,
                       const uint16_t* ln_weight, float ln_eps, uint16_t* xn_out, int epilogue,
                       w4a16_scratch_t* s, void* stream);
/* awq_repack_into for a fused gate|up layer that will run with W4A16_EPILOGUE_SWIGLU: logical row o of the
 * [gate (inter rows) | up (inter rows)] layer lands in physical row 2 o (gate) or 2 (o - inter) + 1 (up), so
 * that a gate row and its up row are neighbours. dst_row_offset and out_f are in logical rows, as for
 * w4a16_repack_into; `inter` is the logical number of gate rows of the container (out_f_total / 2). */
int w4a16_repack_into_swiglu(const w4a16_weights_t* w, int dst_row_offset, const uint32_t* packed,
                             const uint16_t* scale, const uint32_t* zp, int out_f, int inter, void* stream);

/* w4a16_dequant_rows (gemm_w4a16.cuh:45-48, gemm_w4a16.cu:15-38,56-61): rows
 * [row0,row0+nrows) -> row-major bf16 [nrows][in_f], bf16(float(q-zp)*float(s)). */
int w4a16_dequant_rows(uint16_t* dst, const w4a16_weights_t* w, int row0, int nrows, void* stream);

/* gemm_workspace_alloc / free (gemm_w4a16.cuh:37-38). */
int w4a16_workspace_alloc(w4a16_workspace_t* ws, size_t bytes);
int w4a16_workspace_free(w4a16_workspace_t* ws);
/* gemm_w4a16 (gemm_w4a16.cuh:42-43, gemm_w4a16.cu:63-88): C[M][out_f] = A[M][in_f] W^T,
 * any M >= 1, bf16 in/out, fp32 accumulate, dequantisation fused into the tensor-core tiles. */
int w4a16_gemm_prefill(uint16_t* C, const w4a16_weights_t* w, const uint16_t* A, int M,
                       w4a16_workspace_t* ws, void* stream);

/* Column (output-row) sharding over the GPUs of one node. No reference
 * counterpart (the reference is single-GPU; README.md:123). Rank r of nranks owns
 * rows [row_begin,row_end) of an out_f-row layer; both are multiples of 16. */
int w4a16_shard_rows(int out_f, int nranks, int rank, int* row_begin, int* row_end);
/* Completion flags of the fused exchanges. Every rank owns one 256-byte block of zero-initialised,
 * peer-mapped device memory (a symmetric-memory allocation, an IPC mapping ...): words [0, nranks) are
 * counters written by the ranks (word r by rank r: every signalling launch adds 65536 in total, each CTA
 * its share right after its own last store: one system-scope fence, then one add per rank over NVLink),
 * word 16 is the rank's own count of signalling launches. blocks[r] is rank r's block as mapped here;
 * blocks[rank] is the local one. All ranks must issue
 * the same sequence of signalling launches on a communicator (every w4a16_*_gather / *_sharded call below
 * signals once). Zero the blocks and make that visible on every rank (a host barrier) before the first
 * call. Every wait is bounded (about a second): on expiry the waiting kernel records W4A16_ETIMEOUT in
 * the device status word and carries on. No reference counterpart (the reference is single-GPU). */
typedef struct w4a16_comm {
  uint32_t* blocks[8];
  int nranks, rank;
} w4a16_comm_t;
/* w4a16_gemm_skinny_sharded with the completion signal: when the grid's last CTA has stored its slice,
 * this rank's flag is raised on every rank. wait_prev != 0: before x is read, the kernel waits until
 * every rank has signalled its PREVIOUS launch on this communicator, i.e. x may be the gathered output
 * of that launch (layer i+1 consuming layer i without a host barrier or a collective in between). */
int w4a16_gemm_skinny_gather(uint16_t* const* y_peers, const w4a16_comm_t* comm, int wait_prev,
                             int out_f_total, int row_begin, const w4a16_weights_t* w_shard,
                             const uint16_t* x, int M, w4a16_scratch_t* s, void* stream);
/* The gather-free sharded MLP (no reference counterpart; the single-GPU chain it replaces is
 * src/model/model.cu:779-785): gate|up stays ROW-sharded and runs with the SwiGLU epilogue on the shard
 * (w4a16_linear_fused, no exchange at all), its [M][inter / nranks] output is exactly the input slice of the
 * K-sharded down projection, and only the [M][hidden] partial sums cross the link:
 *   w4a16_gemm_skinny_partial  this rank's fp32 partial of Y = X W^T over its K range (w_kshard: all out_f rows,
 *                              in_f = the shard's share of K) is stored into slot `rank` of EVERY rank's buffer
 *                              (partial_peers[r]: rank r's buffer of nranks x M x out_f floats, peer-mapped), then
 *                              the completion flag is raised;
 *   w4a16_reduce_partials      waits (bounded) for every rank's flag, adds the nranks slots of the local buffer in
 *                              rank order (the same bits on every rank), rounds to bf16 once and writes y [M][out_f],
 *                              or, with residual != 0, adds it to y in place as residual_add does. */
int w4a16_gemm_skinny_partial(float* const* partial_peers, const w4a16_comm_t* comm,
                              const w4a16_weights_t* w_kshard, const uint16_t* x_slice, int M,
                              w4a16_scratch_t* s, void* stream);
int w4a16_reduce_partials(uint16_t* y, const float* partials_local, const w4a16_comm_t* comm, int M,
                          int out_f, int residual, void* stream);
/* For consumers that are not kernels of this library: one tiny kernel on `stream` that returns once every
 * rank has signalled the last launch of this communicator (bounded; W4A16_ETIMEOUT in the status word
 * when the wait runs out). */
int w4a16_wait_gather(const w4a16_comm_t* comm, void* stream);
/* Vocab-sharded lm_head in ONE launch: the fused per-shard argmax, then this rank's M (max, global index)
 * pairs are stored into every rank's pair table (pairs_peers[r]: rank r's table of nranks x 16 pairs of
 * {float, int32}, peer-mapped, 8-byte aligned), the flag is raised, the other ranks' pairs are awaited
 * and reduced: larger value, else lower index. ids[M] is complete on every rank when the kernel ends;
 * 8 M bytes per peer cross the link, no logits. row_offset = first vocabulary row of this shard. */
int w4a16_lm_head_argmax_sharded(int32_t* ids, void* const* pairs_peers, const w4a16_comm_t* comm,
                                 int wait_prev, int row_offset, const w4a16_weights_t* w_shard,
                                 const uint16_t* x, int M, w4a16_scratch_t* s, void* stream);
int w4a16_w8_lm_head_argmax_sharded(int32_t* ids, void* const* pairs_peers, const w4a16_comm_t* comm,
                                    int wait_prev, int row_offset, const w4a16_w8_weights_t* w_shard,
                                    const uint16_t* x, int M, w4a16_scratch_t* s, void* stream);

/* gemm_w4a16 on this rank's shard of a column-sharded layer: the epilogue stores every finished tile into
 * every rank's full C[M][out_f_total] at column row_begin (plain peer stores over NVLink, overlapped with
 * the tensor-core work on the next tiles), then raises this rank's flag; a consumer waits with
 * w4a16_wait_gather. Each rank receives (nranks - 1) / nranks of M x out_f_total x 2 bytes, which bounds
 * the call at large M (285 MB for M = 4096 on the gate|up layer). No reference counterpart. */
int w4a16_gemm_prefill_sharded(uint16_t* const* C_peers, const w4a16_comm_t* comm, int out_f_total,
                               int row_begin, const w4a16_weights_t* w_shard, const uint16_t* A, int M,
                               w4a16_workspace_t* ws, void* stream);

/* Skinny GEMM on this rank's shard whose epilogue stores the [M][shard rows] slice
 * straight into every rank's full Y[M][out_f_total] at column row_begin: the
 * all-gather fused into the kernel over NVLink peer stores. y_peers[nranks] are
 * device pointers to each rank's Y (peer-mapped); y_peers[rank] is the local one.
 * Completion on the peers is ordered by the caller's next cross-rank barrier. */
int w4a16_gemm_skinny_sharded(uint16_t* const* y_peers, int nranks, int rank, int out_f_total,
                              int row_begin, const w4a16_weights_t* w_shard, const uint16_t* x,
                              int M, w4a16_scratch_t* s, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* W4A16_B200_H_ */
