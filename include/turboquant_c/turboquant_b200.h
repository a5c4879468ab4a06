/*
 * turboquant_b200.h — tensor-level C entry points of the B200 TurboQuant core.
 *
 * turboquant_c.h (next to this file) carries the reference project's C symbols
 * unchanged in meaning.  That API passes tensors as opaque `void*` and has no
 * tensor-level "linear forward / quantise / dequantise / rotate" calls: those live in
 * the reference's C++ layer.  This header exposes exactly that layer over a plain C
 * ABI — pointers and sizes only — so that a cgo / JNI / N-API / ctypes / Swift binding
 * can reach the CUDA kernels.  Each declaration names the reference interface it stands
 * in for (paths relative to the reference project root).
 *
 * Conventions
 *   - Every data pointer may be a HOST pointer or a CUDA DEVICE pointer; the library
 *     looks the pointer up and copies when needed.  Device pointers are used in place.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Work is
 *     enqueued asynchronously; when an OUTPUT pointer is host memory the call waits
 *     for the stream before returning so the bytes are valid.
 *   - Functions returning int return 0 on success, non-zero on error; functions
 *     returning a handle return NULL on error.  tq_last_error() then gives the reason
 *     (thread-local string).  No C++ exception crosses this boundary.
 *   - There is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef TURBOQUANT_B200_H
#define TURBOQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype tags for activation / result buffers */
enum { TQ_F32 = 0, TQ_F16 = 1, TQ_U8 = 2, TQ_U32 = 3 };

/* ---- library / device -------------------------------------------------------- */

/** Message of the last failed call on this thread ("" if none). */
const char* tq_last_error(void);
/** Number of CUDA devices visible; <= 0 means the library cannot run. */
int tq_device_count(void);
/** Select the device used by this thread for subsequent calls and new handles. */
int tq_set_device(int device);

/* ---- opaque tensor handle for the void* slots of turboquant_c.h ------------------
 * The reference passes `mlx::core::array*` through those slots
 * (src/turboquant_c.cpp:115-116, 127, 149).  Here the slot carries a tq_array: a
 * device buffer with dtype and shape. */
typedef struct tq_array_s* tq_array_t;

/** Copy `data` (host or device) into a new device-resident array. */
tq_array_t tq_array_create(const void* data, int dtype, int ndim, const int* shape);
/** Wrap an existing device buffer without copying or taking ownership. */
tq_array_t tq_array_wrap_device(void* device_ptr, int dtype, int ndim, const int* shape);
int tq_array_ndim(tq_array_t a);
int tq_array_dim(tq_array_t a, int axis);
int tq_array_dtype(tq_array_t a);
size_t tq_array_nbytes(tq_array_t a);
/** Device pointer of the payload. */
void* tq_array_data(tq_array_t a);
/** Copy the payload to host memory (waits for pending work on the array). */
int tq_array_to_host(tq_array_t a, void* dst, size_t dst_bytes);
/* tq_array_free(void*) is declared in turboquant_c.h. */

/* ---- codebooks: include/turboquant/codebook.h:25-46 ------------------------------ */

/** generate_codebook (src/codebook.cpp:71-85): 2^bits centroids, 2^bits-1 boundaries. */
int tq_codebook_generate(int bits, float* centroids, float* boundaries);

/** generate_codebook_from_data (include/turboquant/codebook.h:42, src/codebook.cpp:99-143, 269-282):
 *  Lloyd-Max fit of 2^bits centroids to data[n] (fp32, host or device), started from the analytic
 *  codebook, at most `iterations` rounds, stopping when no centroid moves by 1e-6 or more.  Runs on the
 *  device for every n; bins by lower_bound and sums in double like the reference's CPU path.  n = 0
 *  returns the analytic codebook.  centroids[2^bits], boundaries[2^bits - 1] (may be NULL) and
 *  iterations_run (may be NULL) are host memory. */
int tq_codebook_fit(const float* data, long n, int bits, int iterations, float* centroids, float* boundaries,
                    int* iterations_run, void* stream);

/** The converter's per-layer codebook fit (src/converter.cpp:291-368) for one weight matrix
 *  [out_features, in_features] (fp32, host or device): the primary codebook is fitted to
 *  sqrt(in) * WHT(row / |row|) with the seed the quantiser derives from the weight, the residual
 *  codebook (residual_bits > 0) to what the shared analytic primary codebook leaves of those samples.
 *  Outputs are host arrays: 2^bits centroids, 2^bits - 1 boundaries (boundaries may be NULL). */
int tq_fit_layer_codebooks(const float* weight, int out_features, int in_features, uint32_t block, int primary_bits,
                           int residual_bits, int iterations, float* primary_centroids, float* primary_boundaries,
                           float* residual_centroids, float* residual_boundaries, void* stream);

/** metal/turboquant_qjl.metal:52-137 (tq_qjl_compress): the shader's 1-bit residual compression with a dense
 *  +-1 projection.  residual fp32 [num_tokens, num_heads, head_dim]; proj_dim a power of two <= 1024;
 *  signs_out uint32 [num_tokens * num_heads * ceil(proj_dim / 32)] (bit i of word w = sign of projection
 *  32 w + i, 1 for >= 0); norms_out fp32 [num_tokens * num_heads] (the shader's tree sum over the first
 *  min(head_dim, proj_dim) squares).  Host or device pointers.  At most 65535 tokens per call. */
int tq_qjl_compress(const float* residual, int num_tokens, int num_heads, int head_dim, int proj_dim, uint32_t proj_seed,
                    uint32_t* signs_out, float* norms_out, void* stream);
/** metal/turboquant_qjl.metal:163-216 (tq_qjl_dot_correction) for head head_idx:
 *  corrections[q * num_keys + k] = sqrt(pi/2) / proj_dim * (2 * popcount(~(signs_q ^ signs_k)) - proj_dim) * norms_k
 *  (the shader's index expression `query_idx * gid.x + key_idx` equals this one for query 0, the decode case). */
int tq_qjl_dot_correction(const uint32_t* signs_q, const uint32_t* signs_k, const float* norms_k, int num_queries,
                          int num_keys, int num_heads, int head_idx, int proj_dim, float* corrections, void* stream);

/** Largest power of two <= max_block dividing in_features (src/converter.cpp:228-240). */
uint32_t tq_adaptive_block_size(int in_features, uint32_t max_block);
/** N of the first ".layers.N." in a tensor name, -1 if none (src/converter.cpp:52-59). */
int tq_layer_index(const char* name);
/** 1 when a layer is kept at fp16: index < sensitive_start or > max_layer_index - sensitive_end
 *  (src/converter.cpp:81-93); never for index < 0. */
int tq_is_sensitive_layer(int layer_index, int max_layer_index, int sensitive_start, int sensitive_end);

/* ---- rotation: apply_wht_rotation / apply_inverse_wht_rotation
 *      (include/turboquant/quantizer.h:29-39, src/rotation.cpp:364-403) --------------- */

/** fp32 [rows, cols] -> fp32 [rows, cols]; cols % block == 0, block a power of two in
 *  [32, 1024].  Bit-identical to the reference's CPU route. */
int tq_wht_rotate(const float* in, float* out, int rows, int cols, uint32_t seed, uint32_t block, int inverse,
                  void* stream);

/* ---- weight quantiser: quantize_weight
 *      (include/turboquant/quantizer.h:54-60, src/quantizer.cpp:41-261) -------------- */

/** weight fp32 [out, in].  packed_primary u8 [out, in/2] (primary_bits <= 4) or
 *  [out, in] (5); packed_residual u8 [out, in/2]; norms fp32 [out]; seeds u32[3] =
 *  {seed_primary, seed_residual or 0, block}.  Codes, norms and seeds are bit-identical
 *  to the reference's CPU path. */
int tq_quantize_weight(const float* weight, int out_features, int in_features, const float* primary_centroids,
                       int n_primary, const float* residual_centroids, int n_residual, int primary_bits,
                       int residual_bits, uint32_t block, int shared_rotation, uint8_t* packed_primary,
                       uint8_t* packed_residual, float* norms, uint32_t* seeds, void* stream);

/** The same with the two rotation seeds given by the caller instead of derived from the weight's
 *  bytes (derive_seed, src/quantizer.cpp:12-28): for callers that fix the seeds per layer, e.g. to
 *  quantise shards of one matrix consistently.  seeds[] still receives {seed_primary, seed_residual
 *  or 0 under shared rotation, block}. */
int tq_quantize_weight_seeded(const float* weight, int out_features, int in_features, const float* primary_centroids,
                              int n_primary, const float* residual_centroids, int n_residual, int primary_bits,
                              int residual_bits, uint32_t block, int shared_rotation, uint32_t seed_primary,
                              uint32_t seed_residual, uint8_t* packed_primary, uint8_t* packed_residual, float* norms,
                              uint32_t* seeds, void* stream);

/* ---- TurboQuantLinear (include/turboquant/linear.h:11-35) and the dequantiser
 *      (include/turboquant/dequantizer.h:11-39) ------------------------------------- */

typedef struct tq_linear_s* tq_linear_t;

/* ---- layers of a model loaded by tq_model_load (turboquant_c.h) ----
 * tq_model_load(dir) reads every TurboQuant safetensors shard of a converted model directory
 * (tensor names and metadata of src/serialization.cpp:19-97, loading rules of
 * src/turboquant_c_dequant.cpp:68-150) and uploads each quantised weight as a linear handle; a
 * directory without such shards gives a model with no layers, as the reference's handle has.  The
 * handles below stay owned by the model (tq_model_free frees them). */
#ifndef TURBOQUANT_C_H
typedef struct tq_model_s* tq_model_t;   /* as in turboquant_c.h */
#endif
int tq_model_layer_count(tq_model_t model);
/** Name of layer `index` (the tensor-name prefix, e.g. "model.layers.0.mlp.down_proj"), NULL if out of range. */
const char* tq_model_layer_name(tq_model_t model, int index);
/** The linear handle of the layer called `name`, NULL (see tq_last_error) if there is none. */
tq_linear_t tq_model_layer(tq_model_t model, const char* name);

/** Build a device-resident linear layer from a QuantizedWeight
 *  (include/turboquant/quantizer.h:22-27) plus its two codebooks.
 *  primary_cols is in/2 (4-bit primary) or in (5-bit primary); the residual plane is
 *  always [out, in/2].  The packing mode, "residual present" and shared-vs-dual
 *  rotation are detected exactly as src/dequantizer.cpp:72-74, 118-133 do — once, here,
 *  not on every forward. */
tq_linear_t tq_linear_create(int in_features, int out_features, const uint8_t* packed_primary, int primary_cols,
                             const uint8_t* packed_residual, const float* norms, const uint32_t* seeds,
                             const float* primary_centroids, int n_primary, const float* residual_centroids,
                             int n_residual, uint32_t block);

/** TurboQuantLinear::forward / fused_dequant_matmul (src/linear.cpp:20-26,
 *  src/dequantizer.cpp:606-721): x [batch, in] of x_dtype (TQ_F32 or TQ_F16; cast to
 *  fp16 first) -> y fp16 [batch, out], fp32 accumulation.  Up to 32 rows run through the
 *  decode kernel (passes of 8); more rows run through the tensor-core GEMM when in_features
 *  is a multiple of 64 (its working memory, batch * in * 2 bytes per rotation plane, is
 *  allocated on first use and kept). */
int tq_linear_forward(tq_linear_t lin, const void* x, int x_dtype, int batch, void* y_fp16, void* stream);

/** Forward pass that performs no device or host allocation of any kind.
 *  (No counterpart in the reference: its forward allocates its output and temporaries
 *  through MLX on every call.)
 *
 *  Who needs it: a serving process that, once its models are loaded, gives all remaining
 *  device memory to its own pool — after that a cudaMalloc from inside a library can fail
 *  or stall the whole device while the driver synchronises — and any caller that runs the
 *  layer while a CUDA stream capture is open on the thread, where allocating calls are
 *  rejected.  tq_linear_forward is unsuitable for both when it has to grow a staging
 *  buffer; this entry never does.
 *
 *  x: DEVICE pointer, fp16 [batch, in]; y: DEVICE pointer, fp16 [batch, out]; batch 1..8.
 *  Host pointers are refused (copying them would need staging memory).  Results are the
 *  same as tq_linear_forward's.
 *
 *  The working memory the kernels need (rotated activation, partial sums of layers wider
 *  than 4096 inputs, arrival counters) comes from one fixed array of
 *  tq_linear_noalloc_scratch_limit() bytes (2 MiB) compiled into the library; each GPU
 *  that loads the library holds that array until the process ends.  A layer whose need
 *  8*4*in*planes + 8*4*ceil(in/4096)*planes*out (+ counters) exceeds the limit is refused
 *  with an error; nothing is truncated.
 *
 *  All calls on a device share that array and it keeps the previous call's contents (the
 *  part that must start at zero is cleared in stream order by each call).  Calls that can
 *  run at the same time on one GPU — different streams, or different threads — would
 *  overwrite each other's working memory: keep such calls on one stream or order them
 *  with events.
 *
 *  The first call on each device looks up the array's device address; make that first
 *  call before any stream capture begins. */
int tq_linear_forward_noalloc(tq_linear_t lin, const void* x_fp16_device, int batch, void* y_fp16_device, void* stream);
/** Size in bytes of the built-in working array used by tq_linear_forward_noalloc. */
size_t tq_linear_noalloc_scratch_limit(void);

/** dequantize_weight_cpu / dequantize_weight_gpu (src/dequantizer.cpp:52-256, 347-451):
 *  result [out, in] as TQ_F32 (bit-identical to the reference's CPU result) or TQ_F16
 *  (the same values rounded to nearest even, src/turboquant_c_dequant.cpp:156-167). */
int tq_linear_dequantize(tq_linear_t lin, void* result, int result_dtype, void* stream);

/** Decode forward (x: DEVICE fp16 [batch, in], batch 1..8) whose result is written to n_dst
 *  (1..8) buffers at once: destination d receives output row r of activation row n at
 *  dst[d][n * dst_row_stride + row_offset + r] (fp16).  For a layer whose rows are sharded over
 *  GPUs (an LM head), dst holds the same logits buffer of every rank (the local one and the
 *  peers' mapped with tq_shared_open), dst_row_stride = vocabulary size, row_offset = this rank's
 *  first row: the kernel's epilogue stores each value into every rank's buffer over NVLink and no
 *  all-gather follows, only a barrier among the ranks before the logits are read.  Plain peer
 *  stores: no multicast, and the kernel waits on nobody.  No counterpart in the reference. */
int tq_linear_forward_scatter(tq_linear_t lin, const void* x_fp16_device, int batch, void* const* dst, int n_dst,
                              long dst_row_stride, long row_offset, void* stream);

/** Several layers that multiply the same activation (q / k / v, gate / up: 1..4 handles with the same
 *  in_features, WHT block and rotation mode; x and every y[i] device fp16) in ONE launch of each kernel
 *  of the path: y[i] = [batch, out_features of layer i], each bit-equal to tq_linear_forward on that
 *  layer alone.  Up to 8 rows the SMs of the decode kernel are divided among the layers in proportion to
 *  their sizes; from 9 rows on the group shares one rotation launch, one tensor-memory GEMM launch and
 *  one split-K finish.  A decode step's small projections pay the launches and the set-up once.  Stands in for consecutive calls of the
 *  reference's forward (src/linear.cpp:19-28) on the same input. */
int tq_linear_forward_group(const tq_linear_t* lins, int n, const void* x_fp16_device, int batch, void* const* y_fp16_device,
                            void* stream);

/** Forward whose fp16 result is this layer's rows inside a wider buffer: activation row n goes to
 *  y_fp16_device[n * y_row_stride ...] (y_row_stride >= out_features, in elements).  x and y are
 *  device pointers; any batch size (decode kernel up to 8 rows, tensor-memory kernel above).  A
 *  rank of a row-sharded layer passes its first row's address inside the full [batch, total_rows]
 *  buffer and total_rows as the stride.  Stands in for the reference's forward
 *  (src/linear.cpp:19-28) followed by a copy into place. */
int tq_linear_forward_strided(tq_linear_t lin, const void* x_fp16_device, int batch, void* y_fp16_device, long y_row_stride,
                              void* stream);

/** The same, followed by a completion signal: signal[d] points to an array of 32-bit flags in
 *  destination d's memory (e.g. at the end of its shared buffer); when every result of this
 *  call has been stored, flag signal_slot (0..31, normally this rank) of every destination is
 *  set to signal_value (release, system scope).  tq_linear_wait_peers enqueues one small kernel
 *  on this GPU that waits until flags [0, n_flags) of the LOCAL array have all reached `value`
 *  (callers pass a value that grows with every step): after it, on that stream, the results of
 *  all ranks are visible here — a rank-to-rank barrier costing one flag store and one kernel
 *  launch, fused into the GEMV's tail instead of a separate collective.  The wait gives up after
 *  one second and records it in the handle's status (tq_linear_status).  A buffer must not be
 *  scattered into again before every rank has read the previous results (alternate two buffers).
 *  No counterpart in the reference. */
int tq_linear_forward_scatter_signal(tq_linear_t lin, const void* x_fp16_device, int batch, void* const* dst, int n_dst,
                                     long dst_row_stride, long row_offset, void* const* signal, int signal_slot,
                                     unsigned int signal_value, void* stream);
int tq_linear_wait_peers(tq_linear_t lin, const void* local_flags, int n_flags, unsigned int value, void* stream);

/** Device memory that other processes on the same machine can map: tq_shared_alloc (cudaMalloc,
 *  zero-filled) on the owner, tq_shared_export writes a 64-byte handle to send to the peers
 *  (any channel), tq_shared_open maps it there (CUDA IPC with lazy peer access; the pointer is
 *  valid on the opener's current device), tq_shared_close unmaps, tq_shared_free releases. */
void* tq_shared_alloc(size_t bytes);
void tq_shared_free(void* ptr);
int tq_shared_export(void* ptr, void* handle_out, size_t handle_bytes);
void* tq_shared_open(const void* handle, size_t handle_bytes);
int tq_shared_close(void* peer_ptr);

/* ---- rank-to-rank exchange for the sharded paths ---------------------------------------
 * One process per GPU; every rank allocates a buffer with tq_shared_alloc, the handles travel by
 * the caller's own channel, and each rank maps the others' buffers with tq_shared_open.  The
 * reference plans a layer split and ships no data plane between devices
 * (src/distributed.cpp:201-253, benchmarks/bench_distributed.cpp:9-12): no counterpart there.
 *
 * tq_exchange_broadcast copies a block of this rank's device memory (rows x row_bytes, row_bytes
 * a multiple of 16) to dst[0..n_dst): the same block's place in the other ranks' buffers (and in
 * the local one, if the block was computed elsewhere) - plain 16-byte stores over NVLink, no
 * multicast, no collective library - and then stores this exchange's broadcast count into flag
 * `rank` of every flags[0..n_flags) (arrays of 32 words, one in every rank's memory, the local
 * one included), release at system scope.  tq_exchange_wait enqueues a
 * one-warp kernel that waits until flags [0, n_flags) of the LOCAL array have reached this
 * exchange's wait count; it gives up after one second (tq_exchange_status then fails).  Both counts
 * live in device memory and advance by one per call, so every rank must issue the same sequence of
 * broadcasts and waits - and a captured CUDA graph of that sequence can be replayed.  A block must
 * not be broadcast into again before every rank has read the previous one: alternate two buffers.
 *   all-gather of row shards  = broadcast(own shard)               ; wait
 *   all-reduce of partial sums = broadcast(partial into slot rank) ; wait ; tq_exchange_sum_f16
 *   merge of attention parts  = broadcast(out, lse into slot part) ; wait ; tq_exchange_merge_attention */
typedef struct tq_exchange_s* tq_exchange_t;
tq_exchange_t tq_exchange_create(int rank, int world);
int tq_exchange_broadcast(tq_exchange_t ex, const void* src, void* const* dst, int n_dst, int rows, long row_bytes,
                          long src_stride_bytes, long dst_stride_bytes, void* const* flags, int n_flags, void* stream);
int tq_exchange_wait(tq_exchange_t ex, const void* local_flags, int n_flags, void* stream);
/** out[i] = fp16( residual[i] + sum over s = 0..n_slots-1, in that order, of slots[s * slot_stride + i] ),
 *  fp32 accumulate (residual_fp16 may be NULL): every rank adds the same values in the same order
 *  and gets the same bits. */
int tq_exchange_sum_f16(const void* slots_fp16, int n_slots, long slot_stride, long count, const void* residual_fp16,
                        void* out_fp16, void* stream);
/** tq_exchange_sum_f16 over whole rows ([rows, cols]) followed in the same kernel by the RMSNorm of the summed rows
 *  (see tq_exchange_sum_packets_rmsnorm). */
int tq_exchange_sum_f16_rmsnorm(const void* slots_fp16, int n_slots, long slot_stride, long rows, int cols, const void* residual_fp16,
                                void* out_fp16, const void* norm_weight_fp16, void* normed_fp16, float eps, void* stream);
/** Attention over the union of disjoint token ranges from each range's output and log-sum-exp
 *  (tq_kv_attention_lse): outs [parts][rows][head_dim] fp16, lses [parts][rows] fp32, parts
 *  part_stride_out / part_stride_lse elements apart. */
int tq_exchange_merge_attention(const void* outs_fp16, const void* lses_fp32, int parts, long rows, int head_dim,
                                long part_stride_out, long part_stride_lse, void* out_fp16, void* stream);
/** A row-sharded layer's forward fused with the all-gather of its result, for 1..8 activation rows:
 *  ONE kernel computes this rank's rows into dst[0] (its own buffer; row r of activation row n at
 *  dst[d][n * dst_row_stride + row_offset + r]), the CTA that finishes last copies the block to
 *  dst[1..n_dst) with 16-byte peer stores and raises this rank's flag in flags[0..n_flags) (counts as
 *  one tq_exchange_broadcast of `ex`).  With wait_local_flags != NULL every CTA first waits - for
 *  at most a second - until the n_wait local flags have reached the exchange's next wait count
 *  (counts as one tq_exchange_wait): the activation x may then be the result of the previous
 *  exchange, and a chain of sharded layers runs without any separate exchange kernel.  The first
 *  fused call of a chain must find an earlier broadcast to wait for, or pass NULL.  Replaces the
 *  reference's forward (src/linear.cpp:19-28) plus the collective the reference does not have. */
int tq_linear_forward_allgather(tq_linear_t lin, tq_exchange_t ex, const void* x_fp16_device, int batch, void* const* dst,
                                int n_dst, long dst_row_stride, long row_offset, void* const* flags, int n_flags,
                                const void* wait_local_flags, int n_wait, void* stream);

/** The same all-gather with the flag inside the data ("packets"): the kernel stores this rank's rows to
 *  y_fp16_device (plain fp16, rows y_row_stride apart) and its last CTA writes them to every OTHER rank as
 *  16-byte packets {2 halves, epoch, 2 halves, epoch} - each 8-byte half lands atomically, so a reader that
 *  sees the epoch in both halves has the data, and no fence or separate flag is on the path.
 *  packet_buffers[r] is rank r's packet buffer (its own for r = this rank; peers' mapped with
 *  tq_shared_open), each 2 * world * batch * (out / 4) * 16 bytes, zero-filled before the first use:
 *  [epoch parity][source rank][packet].  wait_previous != 0: every CTA first polls (bounded, 1 s) the
 *  packets the other ranks wrote in the previous call of this sequence - the dependency a decoder layer has
 *  on the gathered output of the layer before.  Every rank issues the same sequence of calls on `ex`
 *  (and none of tq_exchange_broadcast / _wait in between: they share the epochs).  out % 4 == 0, batch <= 8.
 *  tq_exchange_unpack_packets turns a source rank's packets back into contiguous fp16.
 *  No counterpart in the reference. */
int tq_linear_forward_allgather_packets(tq_linear_t lin, tq_exchange_t ex, const void* x_fp16_device, int batch,
                                        void* y_fp16_device, long y_row_stride, void* const* packet_buffers,
                                        int wait_previous, void* stream);
/** After a tq_linear_forward_allgather_packets call on this rank (same stream): waits - bounded, 1 s - for the
 *  packets the other ranks wrote in that exchange and writes their rows into the gathered result
 *  out[n * out_row_stride + source * rows_per_rank + row] (this rank's own block is not touched: let the forward
 *  write it there).  local_packets = this rank's packet buffer.  A peer that never sends shows up in
 *  tq_exchange_status.  This is the wait of that exchange: use it (or tq_exchange_sum_packets) after calls made with
 *  wait_previous = 0, and not for an exchange that the next call's wait_previous = 1 already waits for. */
int tq_exchange_wait_packets(tq_exchange_t ex, const void* local_packets, long rows_per_rank, int batch, void* out_fp16,
                             long out_row_stride, void* stream);
/** The all-reduce of a column-sharded layer over packets: after tq_linear_forward_allgather_packets wrote this
 *  rank's partial output to local_partial_fp16 ([batch][rows] contiguous, count = batch * rows elements) and sent it
 *  to the other ranks, this waits - bounded - for their packets and writes
 *  out = fp16(residual + sum over ranks in rank order, fp32): the arithmetic of tq_exchange_sum_f16, so every rank
 *  gets the same bits.  residual_fp16 may be NULL.  Counts as this exchange's wait. */
int tq_exchange_sum_packets(tq_exchange_t ex, const void* local_packets, const void* local_partial_fp16, long count,
                            const void* residual_fp16, void* out_fp16, void* stream);
/** tq_exchange_sum_packets over whole rows ([rows, cols], cols a multiple of 4) followed, in the same kernel (one CTA per
 *  row), by the RMSNorm of the summed rows: normed = out * rsqrt(mean(out^2) + eps) * norm_weight, the bits
 *  tq_rmsnorm_f16 gives on out.  The residual stream (out) and the next projection's input (normed) in one launch. */
int tq_exchange_sum_packets_rmsnorm(tq_exchange_t ex, const void* local_packets, const void* local_partial_fp16, long rows, int cols,
                                    const void* residual_fp16, void* out_fp16, const void* norm_weight_fp16, void* normed_fp16, float eps,
                                    void* stream);
int tq_exchange_unpack_packets(const void* packets, long n_packets, void* out_fp16, void* stream);
/* Element-wise glue of a decoder layer, device fp16 in and out, fp32 arithmetic.  The reference
 * leaves these to MLX in the host application (no file of its own computes them); they are here so
 * that a whole tensor-parallel decode step runs on this library's stream without a framework.
 *   tq_rmsnorm_f16: y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * weight
 *   tq_rope_f16   : in place on x [rows, heads, head_dim]; element i pairs with i + head_dim/2,
 *                   angle = positions[row] * theta^(-2i/head_dim)
 *   tq_swiglu_f16 : act[r,j] = silu(gate_up[r,j]) * gate_up[r, intermediate + j] */
int tq_rmsnorm_f16(const void* x_fp16, const void* weight_fp16, void* y_fp16, long rows, int cols, float eps, void* stream);
int tq_rope_f16(void* x_fp16, const int* positions, long rows, int heads, int head_dim, float theta, void* stream);
/** tq_rope_f16 on the queries [rows, q_heads, head_dim] and the keys [rows, kv_heads, head_dim] of a step in one launch. */
int tq_rope_qk_f16(void* q_fp16, void* k_fp16, const int* positions, long rows, int q_heads, int kv_heads, int head_dim, float theta,
                   void* stream);
int tq_swiglu_f16(const void* gate_up_fp16, void* act_fp16, long rows, int intermediate, void* stream);

/** Waits for the device; non-zero if a wait of this exchange gave up. */
int tq_exchange_status(tq_exchange_t ex);
void tq_exchange_free(tq_exchange_t ex);

/** Waits for the device, then returns 0 if every kernel launched through this handle ran to
 *  completion, non-zero (see tq_last_error) if one refused to run or gave up on a bounded wait.
 *  Calls with host output check this themselves; callers that pass device pointers and
 *  synchronise on their own can ask here.  No counterpart in the reference. */
int tq_linear_status(tq_linear_t lin);

int tq_linear_in_features(tq_linear_t lin);
int tq_linear_out_features(tq_linear_t lin);
/** Safe to call with NULL. */
void tq_linear_free(tq_linear_t lin);

/* ---- compressed KV cache, pointer-level (handle type from turboquant_c.h) ------------
 * The reference's tq_kv_cache_* calls take opaque arrays; these take plain pointers
 * (host or device) and a stream, and add what a decode loop needs: a batched attention
 * over several caches (one cache = one sequence, as in the reference) and an export of
 * the raw compressed storage in the reference's layout. */
#ifndef TURBOQUANT_C_H
typedef struct tq_kv_cache_s* tq_kv_cache_t;
#endif

/** TQKVCache::append (src/kv_cache.cpp:16-61): keys/values [tokens, heads, head_dim] of
 *  dtype TQ_F32 or TQ_F16.  3-bit codes, norms, QJL sign words and QJL norms are
 *  bit-identical to the reference's encoder. */
int tq_kv_append(tq_kv_cache_t cache, int layer, const void* keys, const void* values, int dtype, int tokens,
                 void* stream);

/** TQKVCache::get_keys_fp16 / get_values_fp16 (src/kv_cache.cpp:260-365): tokens
 *  [start, end) as fp16 [end-start, heads, head_dim]; values != 0 selects V. */
int tq_kv_get_fp16(tq_kv_cache_t cache, int layer, int values, int start, int end, void* out_fp16, void* stream);

/** Raw storage of one layer, token-major as in include/turboquant/kv_cache.h:25-36:
 *  code words [tokens*heads, ceil(d/10)], norms [tokens*heads], QJL words
 *  [tokens*heads, ceil(d/32)], QJL norms [tokens*heads].  Any pointer may be NULL.
 *  Returns the layer's token count, or -1. */
int tq_kv_export(tq_kv_cache_t cache, int layer, uint32_t* k_words, uint32_t* v_words, float* k_norms,
                 float* v_norms, uint32_t* qjl_words, float* qjl_norms);

/** TQKVCache::snapshot + snapshot_serialize (src/kv_cache.cpp:509-524, src/cache_snapshot.cpp:62-83):
 *  the cache's transferable byte stream ("TQCS" header, then one length-prefixed blob per layer
 *  holding the token count and the six storage arrays), byte-identical to the reference's for the
 *  same appended data.  Returns the stream's size in bytes (or -1); the stream is written to the
 *  HOST buffer `out` only when capacity is large enough, so a first call with out = NULL sizes it. */
long tq_kv_snapshot(tq_kv_cache_t cache, void* out, size_t capacity, uint32_t model_hash, uint32_t codebook_hash);
/** snapshot_deserialize + TQKVCache::restore (src/cache_snapshot.cpp:85-110, src/kv_cache.cpp:526-545):
 *  replaces the cache's contents with a stream from tq_kv_snapshot or from the reference.  The
 *  stream's layer count, head count and head_dim must match the cache; malformed input is refused
 *  (non-zero) before anything changes. */
int tq_kv_restore(tq_kv_cache_t cache, const void* data, size_t size);

/** TQKVCache::delta + delta_serialize (src/kv_cache.cpp:566-581, src/cache_snapshot.cpp:110-123):
 *  positions [from, to) of every layer (clamped to each layer's length) as the reference's "TQCD"
 *  byte stream.  Returns the size needed (negative on error) and writes the stream when `out`
 *  (HOST memory) has `capacity` >= that size; call with out = NULL to size the buffer. */
long tq_kv_delta(tq_kv_cache_t cache, void* out, size_t capacity, uint32_t from, uint32_t to);
/** delta_deserialize + TQKVCache::apply_delta (src/cache_snapshot.cpp:125-140, src/kv_cache.cpp:583-594):
 *  appends a stream from tq_kv_delta or from the reference to every layer.  The layer count must
 *  match; malformed input is refused (non-zero) before anything changes. */
int tq_kv_apply_delta(tq_kv_cache_t cache, const void* data, size_t size);

/** Which decode-attention kernel calls that name this cache FIRST use for head_dim 128:
 *  0 chooses by job size (default), 1 the load-based kernel, 2 the bulk-copy pipeline (cp.async.bulk
 *  + mbarrier ring; applies to 1, 2 or a multiple of 4 KV heads, otherwise 1 is used).  Results of
 *  the two agree to rounding (different split of the context); the knob exists for tuning and tests. */
int tq_kv_set_attention_kernel(tq_kv_cache_t cache, int kernel);
/** Non-zero (message via tq_last_error) if an attention call on this cache that has finished
 *  reported a device-side failure (a bounded wait of the pipeline kernel ran out); clears the
 *  report.  Calls with host outputs check this themselves; callers with device outputs call it
 *  after synchronising their stream. */
int tq_kv_attention_status(tq_kv_cache_t cache);

/** Room for `tokens` tokens of `layer` without further allocation (storage otherwise grows by
 *  doubling, which copies and synchronises): call once with the expected context length. */
int tq_kv_reserve(tq_kv_cache_t cache, int layer, int tokens, void* stream);

/** One decode step of a batch: keys / values [n_seqs, heads, head_dim] (DEVICE memory, TQ_F32 or
 *  TQ_F16), row i appended as one token to caches[i] (same results as n_seqs calls of
 *  tq_kv_append with one token each, in two kernel launches per 32 sequences).  No counterpart in
 *  the reference, whose cache holds one sequence. */
int tq_kv_append_batch(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* keys, const void* values,
                       int dtype, void* stream);

/** Decode attention for a batch of sequences: hybrid_attention's long-context branch
 *  (src/attention_dispatch.cpp:58-73) computed directly on the compressed cache.
 *  queries [n_seqs, q_heads, head_dim] (TQ_F32 / TQ_F16, rounded to fp16 first) ->
 *  out fp16 [n_seqs, q_heads, head_dim]; tokens [start, end) of every cache, end < 0
 *  meaning "all tokens of that cache"; q_heads a multiple of the cache's heads
 *  (grouped-query attention).  use_qjl != 0 adds the 1-bit residual correction to the
 *  key scores (an extension: the reference stores those bits but never reads them).
 *  The call keeps a table of per-sequence descriptors and its staging buffers in caches[0]: issue
 *  the calls that share a first cache on one stream.  The table is uploaded (from pageable host
 *  memory) only when it changed - another set of caches, ranges or token counts; a call that
 *  repeats the previous descriptors enqueues kernels only and can be captured in a CUDA graph
 *  (run the same call once before the capture; do not capture a call whose descriptors change). */
int tq_kv_attention(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* queries, int q_dtype,
                    int q_heads, void* out_fp16, int start, int end, int use_qjl, void* stream);

/** The same, and additionally lse_out[n_seqs, q_heads] (fp32, host or device; may be NULL): the
 *  natural log of each row's softmax denominator over the scaled scores of tokens
 *  [start, end).  Two results (out_a, lse_a), (out_b, lse_b) over disjoint token ranges of one
 *  sequence merge exactly as  out = (out_a e^{lse_a - m} + out_b e^{lse_b - m}) /
 *  (e^{lse_a - m} + e^{lse_b - m}),  m = max(lse_a, lse_b) — which is how a sequence's context is
 *  split across GPUs.  No counterpart in the reference. */
int tq_kv_attention_lse(const tq_kv_cache_t* caches, int n_seqs, int layer, const void* queries, int q_dtype,
                        int q_heads, void* out_fp16, float* lse_out, int start, int end, int use_qjl, void* stream);

/* ---- fp16 decode window and hybrid attention -------------------------------------------------
 * The reference keeps these in its C++ layer only (no C symbol): turboquant::DecodeBuffer
 * (include/turboquant/decode_buffer.h:11-47, src/decode_buffer.cpp) and hybrid_attention
 * (src/attention_dispatch.cpp:21-74).  Here the window lives in device memory as fp16
 * [slot][head][dim]; slot = absolute token index % window_size. */
typedef struct tq_decode_buffer_s* tq_decode_buffer_t;

/** DecodeBuffer(window_size, num_heads, head_dim), zero-filled (src/decode_buffer.cpp:9-14). */
tq_decode_buffer_t tq_decode_buffer_create(int window_size, int num_heads, int head_dim);
void tq_decode_buffer_free(tq_decode_buffer_t buf);
int tq_decode_buffer_window_size(tq_decode_buffer_t buf);
int tq_decode_buffer_current_length(tq_decode_buffer_t buf);
/** rebuild (src/decode_buffer.cpp:16-47): keys / values [num_tokens, heads, head_dim] (TQ_F32 or
 *  TQ_F16, host or device); the first min(num_tokens, window) tokens go to slots 0.., the length
 *  becomes num_tokens and the slide position 0. */
int tq_decode_buffer_rebuild(tq_decode_buffer_t buf, const void* keys, const void* values, int dtype, int num_tokens,
                             void* stream);
/** append_token (src/decode_buffer.cpp:49-70): one token [heads, head_dim] into slot length % window. */
int tq_decode_buffer_append_token(tq_decode_buffer_t buf, const void* key, const void* value, int dtype, void* stream);
/** slide_window (src/decode_buffer.cpp:72-103): num_tokens tokens over the oldest slots, from the
 *  slide position, which then advances by num_tokens (mod window). */
int tq_decode_buffer_slide_window(tq_decode_buffer_t buf, const void* new_keys, const void* new_values, int dtype,
                                  int num_tokens, void* stream);
/** keys(start, end) / values(start, end) (src/decode_buffer.cpp:128-142): fp16 [end - start, heads,
 *  head_dim] to host or device memory; fails unless 0 <= start < end <= current_length. */
int tq_decode_buffer_keys(tq_decode_buffer_t buf, int start, int end, void* out_fp16, void* stream);
int tq_decode_buffer_values(tq_decode_buffer_t buf, int start, int end, void* out_fp16, void* stream);

/** hybrid_attention (src/attention_dispatch.cpp:21-74) for one query position: queries
 *  [q_heads, head_dim] (TQ_F32 / TQ_F16, rounded to fp16) -> out fp16 [q_heads, head_dim].  An empty
 *  cache gives zeros; a context of at most window_size tokens is attended in the window (plain
 *  scaled-dot-product attention over its fp16 keys and values, scale 1/sqrt(head_dim)); a longer
 *  one over the compressed cache (the reference decompresses it first; residual bits not used). */
int tq_hybrid_attention(tq_kv_cache_t cache, tq_decode_buffer_t buf, int layer, const void* queries, int q_dtype,
                        int q_heads, void* out_fp16, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_B200_H */
