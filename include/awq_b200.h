/*
 * awq_b200.h — C ABI of the B200 (sm_100a) AWQ W4A16 quantized-linear kernels.
 *
 * Every entry point takes raw DEVICE pointers, plain sizes and a CUDA stream,
 * returns an int status (0 = ok) and never throws, exits or allocates: the
 * caller owns all memory, including repacked weights and workspaces.  The
 * library keeps no state between calls apart from a per-device cache of
 * immutable device properties.
 *
 * Tensor formats (the reference's on-disk AWQ tensors, group size G):
 *   qweight int32 [K, N/8]   bits 4i..4i+3 of word c hold channel 8c+ORDER[i],
 *                            ORDER = {0,2,4,6,1,3,5,7}
 *   qzeros  int32 [K/G, N/8] same nibble rule
 *   scales  fp16  [K/G, N]
 *   bias    fp16  [N] or NULL
 *   W[k,n]  = fp16_rn( fp16(q[k,n] - z[k/G,n]) * scales[k/G,n] )
 *   y[m,n]  = fp16( sum_k x[m,k] * W[k,n] )  then  y = fp16(y + bias[n])
 *
 * Kernel-side weight layout ("packed", produced once at load by
 * awq_b200_repack, same byte count as qweight): [K/128][N][16] uint32, where
 * word j of (block b, column n) holds q[128b + 8j + e, n] for e = 0..7 at
 * nibble position (e >> 1) + 4 * (e & 1).  qzeros and scales are used as they
 * are on disk.
 *
 * Shape rules for every compute entry point: K % 128 == 0, N % 8 == 0, K % G == 0 and G a multiple of
 * 128, or 32 / 64 for the entry points that build the exact fp16 weight per element (awq_b200_gemm*,
 * awq_b200_skinny, awq_b200_dequant*, and awq_b200_linear*, which routes such groups to those two kernels);
 * all pointers 16-byte aligned.
 */
#ifndef AWQ_B200_H_
#define AWQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AWQ_B200_API __attribute__((visibility("default")))
#else
#define AWQ_B200_API
#endif

/* A cudaStream_t, spelled without the CUDA headers. */
typedef void* awq_b200_stream_t;

enum awq_b200_status {
  AWQ_B200_OK = 0,
  AWQ_B200_ERR_NULL = 1,      /* a required pointer is NULL                       */
  AWQ_B200_ERR_SHAPE = 2,     /* M/K/N violate the shape rules above              */
  AWQ_B200_ERR_ALIGN = 3,     /* a pointer is not 16-byte aligned                 */
  AWQ_B200_ERR_GROUP = 4,     /* unsupported group size                           */
  AWQ_B200_ERR_WORKSPACE = 5, /* workspace missing or smaller than *_workspace_bytes */
  AWQ_B200_ERR_CUDA = 6,      /* a CUDA call failed; see awq_b200_last_cuda_error  */
  AWQ_B200_ERR_ARCH = 7,      /* current device is not compute capability 10.x    */
  AWQ_B200_ERR_TOO_LARGE = 8  /* size beyond what an entry point supports         */
};

/* Library version, major * 1000 + minor.  No reference counterpart (the
 * reference extension is unversioned, LLMQRT/runtime_refact/csrc/bindings.cpp:9-47). */
AWQ_B200_API int awq_b200_version(void);

/* Static, human-readable name of a status code. */
AWQ_B200_API const char* awq_b200_status_string(int status);

/* cudaError_t value of the last failed CUDA call on the calling thread (0 if none). */
AWQ_B200_API int awq_b200_last_cuda_error(void);

/* Make `device` current for the calling thread inside this library's CUDA
 * runtime instance.  Replaces the `at::cuda::OptionalCUDAGuard` the reference
 * installs in its GEMM entry points (LLMQRT/runtime_refact/csrc/awq/gemm_db.cu:683). */
AWQ_B200_API int awq_b200_set_device(int device);

/* ---- load-time repack --------------------------------------------------- */

/* Bytes of the packed weight for a K x N linear (= K * N / 2). */
AWQ_B200_API size_t awq_b200_packed_bytes(int K, int N);

/* qweight [K, N/8] -> packed.  Load-time step with no reference counterpart:
 * the reference kernels read the on-disk layout directly
 * (LLMQRT/runtime_refact/csrc/awq/gemv.cu:132-135). */
AWQ_B200_API int awq_b200_repack(const int32_t* qweight, void* packed, int K, int N,
                    awq_b200_stream_t stream);

/* packed -> qweight [K, N/8]; exact inverse of awq_b200_repack, so a module's
 * state_dict can always be produced in the on-disk format. */
AWQ_B200_API int awq_b200_unpack(const void* packed, int32_t* qweight, int K, int N,
                    awq_b200_stream_t stream);

/* ---- dequantisation (parity aid and fp16 fallback for callers) ---------- */

/* On-disk tensors -> W fp16 [K, N], bit-for-bit the reference's
 * dequantize_gemm (LLMQRT/runtime_refact/utils/packing_utils.py:65-80). */
AWQ_B200_API int awq_b200_dequant(const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     void* W, int K, int N, int group_size, awq_b200_stream_t stream);

/* Packed weight -> W fp16 [K, N] through the very device function the GEMV and
 * GEMM kernels dequantise with; must equal awq_b200_dequant bit-for-bit. */
AWQ_B200_API int awq_b200_dequant_packed(const void* packed, const int32_t* qzeros, const void* scales,
                            void* W, int K, int N, int group_size, awq_b200_stream_t stream);

/* ---- decode: split-K GEMV, M <= 64 (8 rows per CTA) ---------------------- */

/* Bytes of scratch awq_b200_gemv needs for (M, K, N).  The first
 * awq_b200_gemv_counter_bytes(N) bytes (a constant, 16 KiB) hold arrival
 * counters that must be zero before the first call and are left zero by every
 * completed call; the rest holds fp32 partial sums and needs no initialisation.
 * One workspace may serve linears of any shape, but awq_b200_gemv and
 * awq_b200_linear lay it out differently: do not hand the same buffer to both. */
AWQ_B200_API size_t awq_b200_gemv_workspace_bytes(int M, int K, int N);
AWQ_B200_API size_t awq_b200_gemv_counter_bytes(int N);

/* y[M, N] = x[M, K] . W (+ bias), 1 <= M <= 64 (awq_b200_gemv_static: 16), one pass over the weights per 8
 * rows.  Replaces awq_gemv / awq_gemv_coalesced
 * (LLMQRT/runtime_refact/csrc/awq/gemv.cu:171-208, gemv_coalesced.cu:263-303).
 * A row's result does not depend on M or on the other rows, and repeated calls
 * give identical bits.  Calls sharing one workspace must not overlap on the GPU. */
AWQ_B200_API int awq_b200_gemv(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const void* bias, void* y, int M, int K, int N, int group_size,
                  void* workspace, size_t workspace_bytes, awq_b200_stream_t stream);

/* Call flags for the *_ex entry points. */
enum awq_b200_flags {
  /* The packed weights, scales and zeros are not being written by work still pending on the
   * stream.  The kernel may then be launched with programmatic dependent launch: it fetches
   * those constants while the previous kernel of the stream drains, and waits for that kernel
   * before it reads x or writes y / the workspace. */
  AWQ_B200_OVERLAP_PREVIOUS = 1,
  /* Decode kernel: add the split-k partial sums through the global workspace even where the
   * splits could form a thread-block cluster (2..8 splits) and add them over distributed shared
   * memory.  Both ways add in the same order and give identical bits; this flag exists for tests. */
  AWQ_B200_NO_CLUSTER = 2,
  /* Decode kernel: which way the (column group, k range) work reaches the CTAs.  By default a
   * shape that needs more than one wave of CTAs runs as a persistent stream (every resident CTA
   * walks an equal share of the work through one copy pipeline) and smaller shapes as one CTA per
   * (column group, k split).  These two flags force one or the other; they exist for tests and
   * tuning.  The two decompositions add a column's k blocks in different (fixed) groupings, so
   * their results agree to fp32 rounding, not bit for bit. */
  AWQ_B200_GEMV_STREAM = 4,
  AWQ_B200_GEMV_PER_SPLIT = 8,
  /* awq_b200_linear_fused only: where the call takes the GEMM route, use the kernel that stages the
   * dequantised weights in shared memory (as awq_b200_gemm_smem does).  For tests. */
  AWQ_B200_GEMM_SMEM = 16,
  /* awq_b200_linear_ex / awq_b200_linear_fused: serve every call of fewer than 8 rows with ONE kernel (the GEMV)
   * whatever the weight's size, as the reference does so that decode (1 row) and speculative verification
   * (2..7 rows) add in the same order and cannot flip an argmax near a tie
   * (LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:161-166).  Without the flag rows 1..4 share a
   * kernel and rows 5..8 share a kernel, and large weights take faster kernels that differ between those classes. */
  AWQ_B200_ONE_KERNEL_BELOW_8 = 32
};

/* awq_b200_gemv with call flags.  No reference counterpart (the reference launches on the
 * legacy default stream with no overlap, LLMQRT/runtime_refact/csrc/awq/gemv.cu:196-201). */
AWQ_B200_API int awq_b200_gemv_ex(const void* x, const void* packed, const void* scales,
                     const int32_t* qzeros, const void* bias, void* y, int M, int K, int N,
                     int group_size, void* workspace, size_t workspace_bytes,
                     awq_b200_stream_t stream, unsigned flags);

/* awq_b200_gemv for hosts that must not allocate device memory while serving: runtimes that size
 * every device buffer at start-up and then forbid cudaMalloc (fixed-arena inference servers, plugin
 * hosts that give the plugin no allocator), where there is nobody to hand this call a workspace.
 * It has no counterpart in the reference.  The split-k scratch lives in a fixed 8 MiB array inside
 * the library's device image (awq_b200_gemv_static_scratch_bytes()), present on every GPU that
 * loads the library until the process exits; the caller passes only inputs and the output.
 *   - Shapes whose planned scratch (awq_b200_gemv_workspace_bytes) exceeds the array return
 *     AWQ_B200_ERR_TOO_LARGE and launch nothing.
 *   - The first call on a device resolves the array's device address and zeroes its counters on
 *     `stream`; make that first call, with the device current, before starting any stream capture.
 *   - No cudaMalloc / cudaFree or allocating library routine is called, on any call.
 *   - All calls share the one array and it keeps the previous call's partial sums: calls that can
 *     overlap on the GPU (different streams) race.  Serialise them, or use awq_b200_gemv with one
 *     workspace per stream.
 * Results are bit-identical to awq_b200_gemv.
 * awq_b200_gemv_static_status copies the array's status word (0, or the code of a device-side wait that
 * expired in some earlier call on the current device) to *status_out on the host; it synchronises with
 * `stream` and allocates nothing either. */
AWQ_B200_API size_t awq_b200_gemv_static_scratch_bytes(void);
AWQ_B200_API int awq_b200_gemv_static_status(unsigned* status_out, awq_b200_stream_t stream);
AWQ_B200_API int awq_b200_gemv_static(const void* x, const void* packed, const void* scales,
                         const int32_t* qzeros, const void* bias, void* y, int M, int K, int N,
                         int group_size, awq_b200_stream_t stream);

/* Tuning hook: awq_b200_gemv with the decomposition forced: ntw in {2,4} column
 * tiles per warp, kw warps that split k inside a CTA (1,2,4,8 with 8 compute warps per CTA;
 * 104, 108, 116 select 16 compute warps with kw = 4, 8, 16), bps k-blocks of 128 per
 * grid-level split; 0 = planner's choice.
 * Its workspace must hold awq_b200_gemv_workspace_bytes_max(M, K, N).  No
 * reference counterpart. */
AWQ_B200_API size_t awq_b200_gemv_workspace_bytes_max(int M, int K, int N);
AWQ_B200_API int awq_b200_gemv_plan(const void* x, const void* packed, const void* scales,
                       const int32_t* qzeros, const void* bias, void* y, int M, int K, int N,
                       int group_size, void* workspace, size_t workspace_bytes,
                       awq_b200_stream_t stream, int ntw, int kw, int bps, unsigned flags);

/* ---- prefill: TMA + tcgen05/TMEM GEMM, any M >= 1 ----------------------- */

/* Workspace of the GEMM entry points.  Its first 256 bytes (status word) must be zero before the first
 * call; 256 bytes are enough for a correct result.  With the full size returned here the tensor-memory
 * kernel may cut the tiles of a partial last wave along k, share them between all SMs and finish them
 * through fp32 partial tiles that a small second kernel adds in k order (deterministic; equal to the
 * one-CTA-per-tile result to fp32 rounding). */
AWQ_B200_API size_t awq_b200_gemm_workspace_bytes(int M, int K, int N);

/* Y[M, N] = X[M, K] . W (+ bias) with fp32 accumulation in tensor memory.
 * Two tcgen05 kernels stand behind it (dequantised weights staged in shared memory as the B operand,
 * or written to tensor memory as the A operand); the faster tile shape is picked per (M, N).
 * Replaces awq_gemm / awq_gemm_db / awq_gemm_cutlass
 * (LLMQRT/runtime_refact/csrc/awq/gemm.cu:407-467, gemm_db.cu:670-732,
 * gemm_cutlass.cu:314-374); the reference's split_k_iters argument has no
 * equivalent because partial sums never leave tensor memory. */
AWQ_B200_API int awq_b200_gemm(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                  const void* bias, void* y, int M, int K, int N, int group_size,
                  void* workspace, size_t workspace_bytes, awq_b200_stream_t stream);

/* Tuning hook: awq_b200_gemm restricted to the kernel that stages the dequantised weights in
 * shared memory (awq_b200_gemm itself picks per shape between that kernel and awq_b200_gemm_wtm;
 * both produce identical bits as long as every tile is finished by one CTA). */
AWQ_B200_API int awq_b200_gemm_smem(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size,
                       void* workspace, size_t workspace_bytes, awq_b200_stream_t stream);

/* Same contract as awq_b200_gemm; the dequantised weights go to tensor memory (the MMA's A operand)
 * instead of shared memory.  No reference counterpart beyond awq_gemm's. */
AWQ_B200_API int awq_b200_gemm_wtm(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                      const void* bias, void* y, int M, int K, int N, int group_size,
                      void* workspace, size_t workspace_bytes, awq_b200_stream_t stream);

/* Few activation rows (1 <= M <= 64) on the tensor-memory path with split-K: the packed weights are
 * cut into units of 256 columns x 128 k, every SM streams an equal share of the units through one
 * copy pipeline, dequantises them into tensor memory as the tcgen05.mma A operand and accumulates in
 * fp32; column tiles shared by several SMs are completed through fp32 partials added in k order.
 * Same arguments and output contract as awq_b200_gemv_ex (bit-exact reference fp16 weights, fp32
 * accumulation, one fp16 rounding, then the bias); a row's bits do not depend on M.  The workspace
 * must hold awq_b200_skinny_workspace_bytes(M, K, N) bytes, start zero-initialised and is left
 * clean.  Replaces the same reference calls as awq_b200_gemv
 * (LLMQRT/runtime_refact/csrc/awq/gemv.cu:168-206 for one row, awq/gemm.cu:195-229 for several). */
AWQ_B200_API size_t awq_b200_skinny_workspace_bytes(int M, int K, int N);
AWQ_B200_API int awq_b200_skinny(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                    const void* bias, void* y, int M, int K, int N, int group_size,
                    void* workspace, size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags);

/* Decode rows (1 <= M <= 8) of a large matrix on the INTEGER tensor-core path (tcgen05.mma kind::i8): the packed
 * bytes (16 q_hi + q_lo) are a tensor-core operand as they arrive, next to one masked copy (word & 0xf0f0f0f0: one
 * logic operation per word), and are multiplied as unsigned bytes with the activations in block-fixed-point form
 * (per row and 128-k block: x ~ sx * t, t a 15-bit integer held as two signed-byte planes); all sums are exact
 * int32 and the kernel applies s * sx * (sum - z * sum t) in fp32 once per 128-k unit.  From 3 rows the planes of
 * the call are written once by a small kernel launched in front (two launches per call; up to 2 rows every CTA
 * builds the planes of its own units).  Weights are applied un-rounded, as in the reference's
 * GEMV (LLMQRT/runtime_refact/csrc/awq/gemv.cu:138); the activations carry a relative error below the fp16
 * spacing of the largest activation of their block.  Results are within the 2e-3 layer bound of the fp16-weight
 * path, not bit-equal to it.  Deterministic; a row's bits do not depend on M within 1..4 and within 5..8 rows.  Same split-K stream of 256-column
 * x 128-k units, arguments and flags as awq_b200_skinny; the workspace must hold
 * awq_b200_decode_workspace_bytes(M, K, N) bytes, start zero-initialised and is left clean.  Replaces the same
 * reference calls as awq_b200_gemv. */
AWQ_B200_API size_t awq_b200_decode_workspace_bytes(int M, int K, int N);
AWQ_B200_API int awq_b200_decode_i8(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                       const void* bias, void* y, int M, int K, int N, int group_size,
                       void* workspace, size_t workspace_bytes, awq_b200_stream_t stream, unsigned flags);

/* Tuning hook: awq_b200_gemm_wtm with the activation-row tile forced (64, 128, 192; 0 = by M). */
AWQ_B200_API int awq_b200_gemm_wtm_tile(const void* x, const void* packed, const void* scales,
                           const int32_t* qzeros, const void* bias, void* y, int M, int K, int N,
                           int group_size, void* workspace, size_t workspace_bytes,
                           awq_b200_stream_t stream, int m_tile);

/* ---- row-parallel shards: one-shot sum over peer memory ------------------- */

/* Bytes of the per-rank flag array of awq_b200_peer_allreduce (zero before the first call).  Two of its
 * 32-bit words are the caller's to read and write (with no call in flight):
 *   AWQ_B200_PEER_STATUS_WORD      0, or 1 / 2 / 3 after a wait on a peer expired (pull form: the peers'
 *                                  partials / the peers' reads; push form: the peers' pushes).  Sticky.
 *   AWQ_B200_PEER_WAIT_LIMIT_WORD  how long one call may wait for its peers, in units of 1024 SM clock
 *                                  cycles; 0 selects the default of about 2 s.
 * After an expiry the ranks' call counters no longer agree and later calls expire as well.  Recover with
 * a collective reset: with no call in flight on any rank, every rank zeroes its flag array (the limit word
 * may be kept) and its receive area, and all ranks meet at a barrier before the next call. */
#define AWQ_B200_PEER_STATUS_WORD 34
#define AWQ_B200_PEER_WAIT_LIMIT_WORD 37
AWQ_B200_API size_t awq_b200_peer_allreduce_flag_bytes(void);

/* out[i] = fp16( sum over ranks r of bufs[r][i] ) (+ bias[i % ncols]), i < count, on every rank of one node.
 * bufs / flags are DEVICE arrays of `world` pointers into memory every rank can load and store (peer-mapped
 * or symmetric allocations, exchanged by the caller): bufs[r] is rank r's fp16 partial, written by earlier
 * work on this stream; flags[r] is rank r's flag array.  Every rank reads all partials with plain peer loads
 * and adds them in rank order in fp32, so all ranks get identical bits; the call returns (stream-wise) only
 * after every peer has read this rank's partial, so the partial may be rewritten by the next kernel.
 * All ranks must make matching calls in the same order.  count % 8 == 0, buffers 16-byte aligned,
 * world <= 16.  Waits on peers are bounded (see AWQ_B200_PEER_WAIT_LIMIT_WORD): on expiry the status word
 * of the flag array becomes non-zero and the output is invalid.  The reference has no counterpart (it is single-GPU,
 * LLMQRT/runtime_refact/core/base.py:44); this replaces the all-reduce of a row-parallel linear
 * (spec-decoding-src-code/eagle_ssd/ssd/layers/linear.py:186-199) at decode sizes. */
AWQ_B200_API int awq_b200_peer_allreduce(const void* const* bufs, void* const* flags, void* out, const void* bias,
                            size_t count, int ncols, int rank, int world, awq_b200_stream_t stream);

/* The same sum with the data pushed instead of pulled: every rank stores its partial into a receive slot on
 * each peer in a self-validating wire format (8-byte words of 4 payload bytes + the call's counter), so a
 * rank waits for one one-way trip over NVLink, polling its own memory, and needs neither fences nor flags.
 * `partial` is this rank's [count] fp16 partial (any memory of this GPU); recv[r] points to rank r's receive
 * area of 2 * world * slot_elems * 4 bytes (peer-mapped like the flag arrays, zero before the first call;
 * slot_elems >= count, a multiple of 8); its two halves alternate on the parity of the call counter kept in
 * the flag array, which makes a closing hand-shake unnecessary.  Same flag arrays, ordering rules,
 * bit-identical results on all ranks, bounded waits (the status word becomes 3; one limit covers the
 * whole call) and graph-capture behaviour as awq_b200_peer_allreduce. */
AWQ_B200_API int awq_b200_peer_allreduce_push(const void* partial, void* const* recv, void* const* flags, void* out,
                                 const void* bias, size_t count, int ncols, size_t slot_elems, int rank,
                                 int world, awq_b200_stream_t stream);

/* awq_b200_decode_i8 for this rank's ROW shard of a row-parallel linear, with the push form of the exchange done by
 * the kernel's own epilogue: each finished pair of results is stored, in the wire format of
 * awq_b200_peer_allreduce_push, into this rank's slot on every peer; the same threads then collect the peers' words
 * for that position out of this rank's receive area, add all ranks' values in rank order in fp32 and write the SUM to
 * y[M, N] - the bits awq_b200_decode_i8 followed by awq_b200_peer_allreduce_push give, in one launch less.
 * recv / flags / slot_elems / rank / world (2..8) as for awq_b200_peer_allreduce_push, and the calls of the two entry
 * points may be mixed freely (they share the call counter), as long as every rank makes the same sequence of calls.
 * bias (this rank's, normally rank 0 only) is added to the partial before the exchange.  Waits on peers are bounded
 * (AWQ_B200_PEER_WAIT_LIMIT_WORD); on expiry the status word (AWQ_B200_PEER_STATUS_WORD) becomes 3.
 * Plays the part of the all-reduce that follows a row-parallel linear in the reference's tensor-parallel layers
 * (spec-decoding-src-code/eagle_ssd/ssd/layers/linear.py:195-199). */
AWQ_B200_API int awq_b200_decode_i8_push(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                            const void* bias, void* y, int M, int K, int N, int group_size, void* workspace,
                            size_t workspace_bytes, void* const* recv, void* const* flags, size_t slot_elems,
                            int rank, int world, awq_b200_stream_t stream, unsigned call_flags);

/* ---- dispatch ------------------------------------------------------------ */

/* Largest M the GEMV entry points accept (64). */
AWQ_B200_API int awq_b200_gemv_max_rows(void);

AWQ_B200_API size_t awq_b200_linear_workspace_bytes(int M, int K, int N);

/* Picks the kernel from the row count and the shape.  M <= 16 -> awq_b200_gemv, except for large weights:
 * awq_b200_decode_i8 for M <= 4 from 24 MiB of packed weights and for 5 <= M <= 8 from 48 MiB; awq_b200_skinny for
 * 9 <= M <= 16 from 16 MiB (beyond 8 rows the GEMV does its unpacking twice).  The thresholds depend on K and N
 * only, so within a row-count class (1..4, 5..8, 9..16, 17..64) a row's bits do not change with the number of rows
 * decoded together; AWQ_B200_ONE_KERNEL_BELOW_8 (awq_b200_linear_ex) makes 1..7 rows one class.
 * 17 <= M <= 64 -> awq_b200_gemv for small matrices (packed MiB x ceil(M / 8) <= 32), else awq_b200_skinny where the
 * GEMM would leave most SMs idle (N <= 18944 and K >= 4096);
 * awq_b200_gemm otherwise.  Group sizes 32 and 64 always take awq_b200_skinny (M <= 64) or awq_b200_gemm.
 * Mirrors the row-count switch in AWQLinearMMFunction.forward
 * (LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:167-185), which also changes kernel
 * (and with it the order of additions) between row counts. */
AWQ_B200_API int awq_b200_linear(const void* x, const void* packed, const void* scales, const int32_t* qzeros,
                    const void* bias, void* y, int M, int K, int N, int group_size,
                    void* workspace, size_t workspace_bytes, awq_b200_stream_t stream);

/* awq_b200_linear with call flags (the flags only affect the few-row kernels). */
AWQ_B200_API int awq_b200_linear_ex(const void* x, const void* packed, const void* scales,
                       const int32_t* qzeros, const void* bias, void* y, int M, int K, int N,
                       int group_size, void* workspace, size_t workspace_bytes,
                       awq_b200_stream_t stream, unsigned flags);

/* Elementwise work that follows the linear in a decoder layer, done in the kernel's epilogue.  Every
 * step rounds to fp16 where the unfused sequence of fp16 tensor operations does (the reference's
 * modules run exactly that sequence: `out + bias`, linear_awq.py:205; Hugging Face's gated MLP
 * `down_proj(act_fn(gate_proj(x)) * up_proj(x))` and the decoder layer's `residual + hidden_states`
 * around the reference's quantized linears, nn_models/modules/nonlinear/transformer_layer.py:139-151):
 *   h = fp16(acc);  h = fp16(h + bias[n])                                (bias != NULL)
 *   gated = 1: the columns are (gate, up) pairs (2j, 2j+1) - build such a weight with
 *              awq_b200_interleave_columns - and y has N / 2 columns:
 *              h = fp16(fp16(silu(h_gate)) * h_up), silu(v) = v / (1 + exp(-v)) in fp32
 *   h = fp16(h + residual[m][column of y])                                (residual != NULL)
 * y is [M, N] fp16, or [M, N / 2] with gated = 1 (which needs N % 16 == 0); bias is in the column order
 * of the packed weight; residual has the shape of y and may be y itself. */
typedef struct awq_b200_epilogue {
  const void* bias;
  const void* residual;
  int gated;
} awq_b200_epilogue;

/* awq_b200_linear_ex with an epilogue (NULL = none).  Same routing, workspace and flags. */
AWQ_B200_API int awq_b200_linear_fused(const void* x, const void* packed, const void* scales,
                          const int32_t* qzeros, const awq_b200_epilogue* epilogue, void* y, int M, int K,
                          int N, int group_size, void* workspace, size_t workspace_bytes,
                          awq_b200_stream_t stream, unsigned flags);

/* Column-interleaves two AWQ int4 tensors of equal shape (qweight [K, n/8] or qzeros [K/G, n/8], int32
 * words in the on-disk nibble order): column 2j of `out` [rows, 2 * words_per_row] is column j of `a`,
 * column 2j+1 is column j of `b`.  With the scales interleaved the same way this turns the separate gate
 * and up projections of a gated MLP (which the reference keeps as two AWQ linears) into the one weight
 * a gated epilogue expects.  Load-time utility. */
AWQ_B200_API int awq_b200_interleave_columns(const int32_t* a, const int32_t* b, int32_t* out, int rows,
                                int words_per_row, awq_b200_stream_t stream);

/* ---- decode-time plumbing between the linears of a decoder layer -------------- */

/* One token's fused qkv row [(H + 2 KV) * D] fp16 -> per-head RMSNorm of the q and k heads (q_weight / k_weight
 * [D] fp16, both NULL for models without q/k norms), rotary embedding of q and k with row `*pos` of cos_tab /
 * sin_tab [max_len, D] (the layout of Hugging Face's rotary module: both halves of a row hold the same D/2
 * angles), q to q_out [H, D], k and v into row `*pos` of k_cache / v_cache [KV, max_len, D].  `pos` points to an
 * int64 in DEVICE memory, so the launch is the same for every token (CUDA-graph friendly).  D is 64 or 128.
 * Each fp16 step rounds where the reference's separate tensor operations round
 * (LLMQRT/runtime_refact/nn_models/modules/nonlinear/attention.py:299-330: q_norm / k_norm, rope, cache
 * update).  A position outside [0, max_len) writes nothing. */
AWQ_B200_API int awq_b200_qk_norm_rope_cache(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                                const void* cos_tab, const void* sin_tab, const int64_t* pos, void* q_out,
                                void* k_cache, void* v_cache, int H, int KV, int D, int max_len,
                                awq_b200_stream_t stream);

/* out [H * D] fp16 = softmax(scale * q . K[0..*pos]^T) . V[0..*pos] for one query token of H heads against a cache
 * of KV heads (grouped-query attention, H % KV == 0); fp32 online softmax.  Stands in, at decode time, for the
 * attention call of the reference's attention block (attention.py:331-380), which is outside the quantized-linear
 * path; it exists so that a whole decode step is a fixed sequence of launches.
 * workspace (optional, 16-byte aligned, awq_b200_attn_workspace_bytes(H, D) bytes, its first 256 * ceil(H / 64)
 * bytes zero before the first use and left zero): with it, contexts beyond 256 positions are cut into chunks of
 * about 128 positions (at most min(8, 148 / H) per head), one CTA per (head, chunk), whose partial results the
 * last CTA of a head to finish adds in chunk order (deterministic); without it, or up to 256 positions, one CTA
 * per head. */
AWQ_B200_API size_t awq_b200_attn_workspace_bytes(int H, int D);
AWQ_B200_API int awq_b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos,
                         void* out, int H, int KV, int D, int max_len, float scale, void* workspace,
                         size_t workspace_bytes, awq_b200_stream_t stream);

/* y[M, D] fp16 = RMSNorm(x[M, D]) * weight[D]: fp32 arithmetic, one rounding (torch.nn.functional.rms_norm's); D even.
 * The norms between the linears of a decoder layer (LLMQRT/runtime_refact/nn_models/modules/nonlinear/
 * transformer_layer.py:139-151) as one launch that may overlap its predecessor's tail. */
AWQ_B200_API int awq_b200_rmsnorm(const void* x, const void* weight, float eps, void* y, int M, int D,
                     awq_b200_stream_t stream);

/* awq_b200_qk_norm_rope_cache followed by awq_b200_attn_decode as ONE launch (one CTA per query head): qkv
 * [(H + 2 KV) * D] fp16 is the fused qkv linear's output row; every CTA normalises / rotates its query head and its
 * group's key head itself, attends over cache rows 0 .. *pos - 1 plus the fresh key / value, and the first CTA of a
 * group appends the fresh key / value to row *pos of the caches.  out [H * D] fp16; same bits as the two calls
 * (given the same workspace choice; workspace as for awq_b200_attn_decode). */
AWQ_B200_API int awq_b200_attn_step(const void* qkv, const void* q_weight, const void* k_weight, float eps,
                       const void* cos_tab, const void* sin_tab, const int64_t* pos, void* k_cache, void* v_cache,
                       void* out, int H, int KV, int D, int max_len, float scale, void* workspace,
                       size_t workspace_bytes, awq_b200_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------------
 * The reference extension's other quantized linears: FP8 (e4m3) and SmoothQuant INT8, 8-bit x 8-bit GEMMs with a
 * scaling epilogue.  Operands arrive quantised, as they do in the reference: activations xq [M, K] row-major with
 * a row pitch of ldx bytes; weights wq [N, K] row-major with a row pitch of ldw bytes (the memory behind the
 * `[K, N]`, stride `[1, K]` view the reference passes).  Pitches are multiples of 16 bytes and >= K; xq and wq
 * are 16-byte aligned.  bias_kind: 0 none (bias NULL), 1 bf16, 2 fp16, 3 fp32.  `status` (optional, device word)
 * receives a non-zero code if a bounded wait inside the kernel ran out.
 * Problems of few rows split K over the CTAs of a thread-block cluster, which add their partial sums over
 * distributed shared memory in a fixed order: results do not depend on timing, and for INT8 not on the split
 * either.  `flags`: AWQ_B200_Q8_NO_SPLIT forbids the split (tests, tuning).
 * --------------------------------------------------------------------------------------------------------------- */
#define AWQ_B200_Q8_NO_SPLIT 1u
/* Number of K splits (1..8) the GEMMs below use for this problem on the current device. */
AWQ_B200_API int awq_b200_q8_splits(int M, int N, int K);

/* y[M, N] = alpha' * (xq . wq^T) + beta * bias, fp32 accumulation, y bf16 (out_bf16 != 0) or fp16.
 * alpha' = alpha * (*alpha_dev) * (*alpha_dev2); either pointer may be NULL.  They let a dynamic activation scale
 * and a weight-scale parameter stay on the device: the reference multiplies the two on the device and reads the
 * product back to pass it as a float (linear_fp8.py:216-225).
 * Replaces cutlass_f8f8bf16_tensorwise_sm89(XQ, WQ, bias, alpha, beta, dtype_str)
 * (LLMQRT/runtime_refact/csrc/bindings.cpp:15-17; csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:30-160, :316-328). */
AWQ_B200_API int awq_b200_fp8_gemm_tensorwise(const void* xq, int ldx, const void* wq, int ldw, const void* bias,
                                 int bias_kind, void* y, int M, int N, int K, float alpha, const float* alpha_dev,
                                 const float* alpha_dev2, float beta, int out_bf16, unsigned flags,
                                 unsigned* status, awq_b200_stream_t stream);

/* y[M, N] bf16 = ((xq . wq^T) * x_scale[m]) * w_scale[n] + bias[n]; xq e4m3 or e5m2 (x_is_e5m2), wq e4m3.
 * Replaces cutlass_f8f8bf16_rowwise_sm89(XQ, WQ, bias, x_scale, w_scale, use_fast_accum)
 * (csrc/bindings.cpp:18-20; csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:425-2248).  The accumulator is always fp32 in
 * tensor memory, so use_fast_accum has nothing to select. */
AWQ_B200_API int awq_b200_fp8_gemm_rowwise(const void* xq, int ldx, int x_is_e5m2, const void* wq, int ldw,
                              const void* bias, int bias_kind, const float* x_scale, const float* w_scale, void* y,
                              int M, int N, int K, unsigned flags, unsigned* status, awq_b200_stream_t stream);

/* y[M, N] = alpha' * float(int32(xq . wq^T)) + beta * bias; xq, wq int8; exact int32 accumulation.
 * Replaces w8a8_int8_linear_bbf16_obf16_per_tensor(input, weight, bias, alpha, beta)
 * (csrc/bindings.cpp:12-14; csrc/smoothquant/sq_gemm.cu:30-190), whose output element type is fp16. */
AWQ_B200_API int awq_b200_int8_gemm_tensorwise(const void* xq, int ldx, const void* wq, int ldw, const void* bias,
                                  int bias_kind, void* y, int M, int N, int K, float alpha, const float* alpha_dev,
                                  const float* alpha_dev2, float beta, int out_bf16, unsigned flags,
                                  unsigned* status, awq_b200_stream_t stream);

/* Activation quantisation in front of those GEMMs, with the roundings of the reference's torch expressions run on
 * a GPU.  x [M, K] fp16 or bf16 (x_is_bf16), contiguous, 16-byte aligned, K % 8 == 0; xq [M, K] bytes.
 *   mode 0  e4m3, one dynamic scale:  per_tensor_quantize        (linear_fp8.py:11-33)     scale_out[0] = scale
 *   mode 1  e4m3, one scale per row:  per_token_quantize         (linear_fp8.py:41-64)     scale_out[m] = scale
 *   mode 2  e4m3, given fp32 scale *static_scale: static_per_tensor_quantize (linear_fp8.py:35-38)
 *   mode 3  int8, one dynamic scale:  quantize_activation_per_tensor_absmax (linear_sq.py:19-28)
 *           scale_out[0] = scale, scale_out[1] = scale * weight_scale rounded to x's type (linear_sq.py:97)
 * amax_ws: one device word of scratch (modes 0 and 3).  An all-zero fp16 tensor, which the reference turns into
 * NaNs (its scale underflows to 0), quantises to zeros here. */
AWQ_B200_API int awq_b200_q8_quantize(const void* x, int x_is_bf16, int M, int K, int mode, const float* static_scale,
                         float weight_scale, void* xq, float* scale_out, unsigned* amax_ws,
                         awq_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AWQ_B200_H_ */
