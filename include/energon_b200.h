/*
 * energon_b200 — C ABI of the B200 (sm_100a) implementation of EnergonAI's tensor-parallel
 * transformer layer forward.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every tensor is allocated by the caller and must be
 *     device memory of the current CUDA device, contiguous in the stated layout;
 *   - `dtype` is one of EB_F32 / EB_F16 / EB_BF16;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); all work
 *     is enqueued on it, nothing synchronises the device;
 *   - the return value is EB_OK or a negative EB_E* code; on failure eb_last_error() returns
 *     a thread-local human-readable message.  Nothing throws, exits or prints.
 *
 * Each declaration cites the reference interface it replaces (path inside the EnergonAI
 * repository : line).
 */
#ifndef ENERGON_B200_H
#define ENERGON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EB_API __attribute__((visibility("default")))
#else
#define EB_API
#endif

#define EB_OK 0
#define EB_EINVAL (-1)       /* bad argument (null pointer, size, alignment, dtype)          */
#define EB_ECUDA (-2)        /* the CUDA runtime / driver reported an error at launch        */
#define EB_EUNSUPPORTED (-3) /* valid request outside what the kernels implement            */
#define EB_ETIMEDOUT (-4)    /* a bounded device-side wait expired (see eb_device_status)    */
#define EB_ELIMIT (-5)       /* request exceeds a documented fixed capacity                 */

#define EB_F32 0
#define EB_F16 1
#define EB_BF16 2

/* activation codes for eb_gemm */
#define EB_ACT_NONE 0
#define EB_ACT_RELU 1
#define EB_ACT_GELU_TANH 2 /* energonai/model/model_factory.py:32-35 (gelu_impl)            */
#define EB_ACT_GELU_ERF 3  /* torch.nn.functional.gelu                                      */

/* flags for eb_gemm */
#define EB_GEMM_STATIC_W 1 /* W is constant (model weights): the kernel may start reading it while
                              earlier work of the stream is still running */

/* flags for eb_scale_mask_softmax */
#define EB_SM_CAUSAL 1  /* keys j > query i are masked to exactly 0 (reference behaviour)    */
#define EB_SM_KEYLEN 2  /* keys j >= real_seq_len[b] are masked to exactly 0                 */
#define EB_SM_ALLROWS 4 /* also rewrite query rows i >= real_seq_len[b] (reference skips them) */

EB_API int eb_version(void);
EB_API const char *eb_last_error(void);

/* ---- padding offsets and (un)padding copies ------------------------------------------ */

/* Replaces ft_build_padding_offsets_wrapper
 * (energonai/kernel/cuda_native/csrc/transpose_pad_fusion_wrapper.cpp:93-104, kernel
 * transpose_pad_fusion_kernel.cu:112-131).  seq_lens[batch] (each 0..max_seq_len);
 * valid_word_num[0] = sum of lengths; tmp_mask_offset[k], k < sum, = number of padding slots
 * before valid token k in the [batch, max_seq_len] layout.  tmp_mask_offset must hold at
 * least sum(seq_lens) entries (batch*max_seq_len always suffices).  Entries beyond the sum
 * are not written. */
EB_API int eb_build_padding_offsets(const int32_t *seq_lens, int batch, int max_seq_len, int32_t *valid_word_num,
                             int32_t *tmp_mask_offset, void *stream);

/* Replaces ft_remove_padding_wrapper (transpose_pad_fusion_wrapper.cpp:113-140, kernel
 * transpose_pad_fusion_kernel.cu:142-155): tgt[k,:] = src[k + off[k],:] for k < valid, and
 * mask_offset[k] = tmp_mask_offset[k].  src [batch*max_seq_len, n], tgt [valid, n]. */
EB_API int eb_remove_padding(const void *src, void *tgt, const int32_t *tmp_mask_offset, int32_t *mask_offset, int valid,
                      int n, int dtype, void *stream);

/* Replaces ft_rebuild_padding_wrapper (transpose_pad_fusion_wrapper.cpp:147-172, kernel
 * transpose_pad_fusion_kernel.cu:178-190): tgt[k + off[k],:] = src[k,:].  The reference
 * scatters into a freshly zeroed tensor; here the same kernel writes the zero rows
 * (zero_fill != 0), so tgt [batch*max_seq_len, n] may be uninitialised memory. */
EB_API int eb_rebuild_padding(const void *src, void *tgt, const int32_t *mask_offset, int valid, int n, int batch,
                       int max_seq_len, int dtype, int zero_fill, void *stream);

/* Replaces ft_transpose_rebuild_padding_wrapper (transpose_pad_fusion_wrapper.cpp:181-209,
 * kernel transpose_pad_fusion_kernel.cu:213-236): packed Q,K,V [valid, head_num,
 * size_per_head] -> q_buf,k_buf,v_buf [batch, head_num, seq_len, size_per_head].  With
 * zero_fill == 0 rows of padding tokens are left untouched, as in the reference (whose
 * callers pre-zero the buffers); with zero_fill != 0 they are written as zeros. */
EB_API int eb_transpose_rebuild_padding(const void *Q, const void *K, const void *V, void *q_buf, void *k_buf, void *v_buf,
                                 int batch, int seq_len, int head_num, int size_per_head, int valid,
                                 const int32_t *mask_offset, int dtype, int zero_fill, void *stream);

/* Replaces ft_transpose_remove_padding_wrapper (transpose_pad_fusion_wrapper.cpp:218-244,
 * kernel transpose_pad_fusion_kernel.cu:268-289): src [batch, head_num, seq_len,
 * size_per_head] -> dst [valid, head_num*size_per_head]. */
EB_API int eb_transpose_remove_padding(const void *src, void *dst, int valid, int batch, int seq_len, int head_num,
                                int size_per_head, const int32_t *mask_offset, int dtype, void *stream);

/* Replaces transpose_pad_wrapper (transpose_pad_fusion_wrapper.cpp:33-57, kernel
 * transpose_pad_fusion_kernel.cu:58-84): packed src [sum_len, head_num, size_per_head] ->
 * dst [batch, head_num, max_seq_len, size_per_head], zeros where position >= seq_lens[b]. */
EB_API int eb_transpose_pad(const void *src, void *dst, int batch, int max_seq_len, const int32_t *seq_lens, int head_num,
                     int size_per_head, int dtype, void *stream);

/* Replaces transpose_depad_wrapper (transpose_pad_fusion_wrapper.cpp:59-83, kernel
 * transpose_pad_fusion_kernel.cu:8-35): src [batch, head_num, max_seq_len, size_per_head] ->
 * dst [sum_seq, head_num, size_per_head]; rows of dst beyond sum(seq_lens) are zeroed. */
EB_API int eb_transpose_depad(const void *src, void *dst, int batch, int sum_seq, int max_seq_len, const int32_t *seq_lens,
                       int head_num, int size_per_head, int dtype, void *stream);

/* ---- scale-mask-softmax ----------------------------------------------------------------- */

/* Replaces scale_mask_softmax_wrapper (csrc/scale_mask_softmax_wrapper.cpp:25-44, kernel
 * scale_mask_softmax_kernel.cu:12-42).  In place over scores [batch, head_num, seq_len,
 * seq_len].  Reference behaviour = flags EB_SM_CAUSAL, scale 1.0f: rows i < real_seq_len[b]
 * become softmax over keys j <= i with keys j > i set to 0, other rows are untouched.  The
 * scores are multiplied by `scale` before the softmax.  No limit on seq_len (the reference
 * stops at 1024).  dtype F32, F16 or BF16. */
EB_API int eb_scale_mask_softmax(void *scores, const int32_t *real_seq_len, int batch, int seq_len, int head_num, int dtype,
                          int flags, float scale, void *stream);

/* ---- LayerNorm forward -------------------------------------------------------------------- */

/* Replaces forward_affine (csrc/layer_norm_cuda.cpp:82-103, kernel
 * layer_norm_cuda_kernel.cu:243-279) and the LayerNorm1D modules of the block
 * (energonai/model/endecoder.py:28,39).  Rows n1, row length n2.
 *   t   = x (+ residual) (+ bias[n2])            (optional operands may be NULL)
 *   with residual or bias, t is rounded to in_dtype first (what a residual stream stores);
 *   sum_out = t (in in_dtype), if sum_out != NULL
 *   y   = gamma * (t - mean) * invvar + beta     (gamma/beta NULL: no affine)
 *   mean[n1], invvar[n1] fp32, if non-NULL.
 * Statistics in fp32 over a register-resident row (one pass over the row shifted by its first
 * element), biased variance. */
EB_API int eb_layer_norm_fwd(void *y, float *mean, float *invvar, const void *x, const void *residual, const void *bias,
                      void *sum_out, const void *gamma, const void *beta, int64_t n1, int n2, double eps, int in_dtype,
                      int out_dtype, void *stream);

/* ---- tensor-parallel exchange context --------------------------------------------------------
 *
 * One eb_comm per rank of a tensor-parallel group (one process per GPU).  It takes the place of
 * what the reference obtains from colossalai.launch (energonai/worker.py:27-28: the NCCL
 * process groups) and of its unbuilt NCCL-id helper
 * (energonai/kernel/cuda_native/csrc/get_ncclid.cpp:104-127), for the exchanges this library
 * performs itself: the all-reduce of the row-parallel layers (colossalai's Linear1D_Row,
 * constructed at energonai/model/attention.py:37 and energonai/model/mlp.py:22).
 *
 * Each rank owns a receive area its peers write into over NVLink with plain stores.  Set-up:
 *   eb_comm_create(rank, world, line_bytes, bulk_bytes, NULL, &c)   allocates and zeroes the local area
 *   eb_comm_export_handle(c, blob, n)                        n = eb_comm_handle_bytes()
 *   ... the caller gathers every rank's blob with its own process group, in rank order ...
 *   eb_comm_connect(c, all_blobs, world * n)                 maps the peers' areas (CUDA IPC)
 *   ... a barrier of the caller's: nobody exchanges before everybody is connected ...
 * A caller that maps peer memory itself (one process driving several GPUs, or another symmetric
 * allocator) passes its own area (eb_comm_area_bytes(line_bytes, bulk_bytes) bytes, zero-filled)
 * as recv_local and the peers' addresses to eb_comm_connect_pointers instead.  An area has two
 * regions.  The flagged-line region (line_bytes) carries generation-step exchanges:
 * eb_comm_exchange_bytes(world, rows, cols) bytes per HALF of it for a [rows, cols] 16-bit
 * matrix (data travels with a sequence number beside every 4 bytes, so it takes twice its size).
 * The bulk region (bulk_bytes, may be 0) carries prompt-sized tensors as plain data: the staging
 * and gather areas of eb_gemm_reduce_scatter / eb_reduce_broadcast, at offsets the caller
 * chooses; eb_comm_local_area returns its local address so that results can be read in place.
 * All ranks must issue the same exchanges in the same order.  A wait on a peer that lasts longer
 * than the budget (5 s unless changed) is abandoned: the kernel records EB_ETIMEDOUT in the
 * context (eb_comm_status) or in the device status word (eb_device_status), its result is then
 * unspecified and the ranks' sequence numbers no longer agree: tear the group down.  One host
 * thread at a time per context; exchanges sharing a context must not overlap on the device. */
typedef struct eb_comm eb_comm;
EB_API size_t eb_comm_handle_bytes(void);
EB_API size_t eb_comm_exchange_bytes(int world, int rows, int cols);
EB_API int eb_comm_create(int rank, int world, size_t line_bytes, size_t bulk_bytes, void *recv_local, eb_comm **out);
EB_API size_t eb_comm_area_bytes(size_t line_bytes, size_t bulk_bytes);
EB_API int eb_comm_local_area(eb_comm *comm, void **bulk_ptr, size_t *bulk_bytes);
EB_API int eb_comm_export_handle(const eb_comm *comm, void *blob, size_t blob_bytes);
EB_API int eb_comm_connect(eb_comm *comm, const void *all_blobs, size_t all_blobs_bytes);
EB_API int eb_comm_connect_pointers(eb_comm *comm, void *const *peer_recv);
EB_API int eb_comm_set_wait_budget(eb_comm *comm, double seconds);
EB_API int eb_comm_status(eb_comm *comm, int *out4, int clear);
EB_API int eb_comm_destroy(eb_comm *comm);

/* All-reduce of a prompt-sized row-parallel product in two launches, replacing "F.linear, then
 * dist.all_reduce, then + bias" of colossalai's Linear1D_Row for M > 128 rows (the layers
 * constructed at energonai/model/attention.py:37 and energonai/model/mlp.py:22, called with the
 * whole prompt at attention.py:127-128 and mlp.py:35).
 *   eb_gemm_reduce_scatter: A [M,K] . W [N,K]^T (this rank's column shard of the weight) on the
 *     tensor cores; every finished 128-row tile is stored, in the operand type, straight into
 *     the staging area of the rank that owns those rows (bulk region + stage_offset of that
 *     rank, over NVLink, 128-byte row segments), so the reduce-scatter half of the all-reduce
 *     travels while the product is still being computed.  Rows are dealt out in `world`
 *     contiguous blocks of whole 128-row tiles.
 *   eb_reduce_broadcast: after a barrier over the ranks, each rank adds the `world` partials of
 *     its own rows in fp32, in rank order, + bias + residual (rows ldr apart, may be NULL),
 *     rounds to the operand type and stores the finished rows into the gather area (bulk region
 *     + gather_offset, [M][N]) of every rank; a second barrier ends the kernel, after which
 *     every rank reads the complete [M, N] sum at its own eb_comm_local_area + gather_offset.
 * The staging area takes eb_reduce_broadcast_stage_bytes(world, M, N) bytes, the gather area
 * M*N*2; offsets are multiples of 256 and the two must not overlap, nor be reused while a peer
 * may still read them (alternate two gather areas between consecutive calls).  Waits are
 * bounded (eb_comm_status).  N a multiple of 8, fp16 / bf16. */
EB_API int eb_gemm_reduce_scatter(const void *A, long long lda, const void *W, long long ldw, int M, int N, int K, int dtype,
                           int flags, eb_comm *comm, size_t stage_offset, void *stream);
EB_API int eb_reduce_broadcast(eb_comm *comm, long long M, int N, int dtype, size_t stage_offset, size_t gather_offset,
                        const void *bias, const void *residual, long long ldr, void *stream);
EB_API size_t eb_reduce_broadcast_stage_bytes(int world, long long M, int N);

/* In-place SUM of buf[count] (dtype fp32 / fp16 / bf16, sums formed in fp32 in rank order, so
 * every rank holds the bit-identical result) over the ranks of `comm`: each rank stores its
 * buffer into every rank's receive area and adds up what it received ("one-shot": one NVLink
 * crossing, meant for the kilobyte-to-megabyte messages of generation steps; NCCL remains the
 * tool for prompt-sized tensors).  buf 8-byte aligned, count * size a multiple of 8 bytes,
 * world * count * size * 2 <= line_bytes / 2.  Replaces dist.all_reduce inside Linear1D_Row. */
EB_API int eb_allreduce(eb_comm *comm, void *buf, size_t count, int dtype, void *stream);

/* ---- dense layers (tcgen05 tensor-core GEMM) --------------------------------------------- */

/* C = act(A . W^T + bias) + residual, fp32 accumulation in tensor memory.
 * Replaces the F.linear inside the column-parallel and row-parallel layers the reference
 * builds from colossalai (Linear1D_Col / Linear1D_Row, constructed at
 * energonai/model/attention.py:29-37 and energonai/model/mlp.py:20-22) and mlp_gemm
 * (energonai/kernel/cuda_native/csrc/linear_wrapper.cpp:82-111).
 *   A [M,K] rows lda apart, W [N,K] rows ldw apart (both fp16 or both bf16, `dtype`);
 *   C [M,N] in `out_dtype` (= dtype, or EB_F32); bias [N] (dtype) or NULL; residual [M,N]
 *   rows ldr apart (dtype) or NULL; act one of EB_ACT_*.
 *   Row m of C starts at element m*ldc, or, when c_rows_per_batch > 0, at
 *   (m / c_rows_per_batch)*c_batch_stride + (m % c_rows_per_batch)*ldc  (this lets a
 *   projection write straight into a [batch, max_len, width] cache at a position offset).
 *   c_row_offset_device, if non-NULL, is a device int32 read by the kernel: that many further
 *   rows (of ldc elements) are added to every row's offset, so a captured launch can append
 *   at a position that advances between replays.  c_row_offset_limit > 0 bounds it: a device
 *   value outside [0, limit) stores nothing and records EB_ELIMIT in the device status word
 *   (the caller's buffer was not sized for that position).
 *   K must be a multiple of 8 and pointers 16-byte aligned; for M > 128 also N, all leading
 *   dimensions and c_batch_stride (for M <= 128 the output is written element by element).
 * The kernel is launched so that it may begin before the preceding kernel of the stream has
 * finished; it reads A, bias and residual only after that kernel completed, and W too unless
 * flags has EB_GEMM_STATIC_W.
 * For M <= 128 (generation steps) the kernel streams W exactly once, split evenly over all SMs
 * (stream-K over 128-row tiles; a K of at most 1280 is not cut, one CTA per tile), and combines
 * the partial sums of tiles shared by several CTAs
 * through `workspace`: at least eb_gemm_workspace_bytes(M,N,K) bytes, 16-byte aligned,
 * zero-filled once before first use (the kernel leaves it reusable; summation order is fixed,
 * results are deterministic).  Calls that share a workspace must not overlap on the device.
 * workspace may be NULL for M > 128. */
EB_API int eb_gemm(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc, const void *bias,
            const void *residual, long long ldr, int M, int N, int K, int dtype, int out_dtype, int act,
            int c_rows_per_batch, long long c_batch_stride, const int32_t *c_row_offset_device,
            int c_row_offset_limit, int flags, void *workspace, size_t workspace_bytes, void *stream);
EB_API size_t eb_gemm_workspace_bytes(int M, int N, int K);

/* Row-parallel GEMM with the tensor-parallel all-reduce fused into its epilogue, for the
 * generation orientation (M <= 128).  Replaces "F.linear, then dist.all_reduce, then + bias" of
 * colossalai's Linear1D_Row (the row-parallel layers constructed at
 * energonai/model/attention.py:37 and energonai/model/mlp.py:22).  Arguments as eb_gemm, plus the
 * exchange context.  The thread that completes the batch values of an output column stores them
 * (rounded to the operand type, as an all-reduce of the product would see them) into every
 * rank's receive area over NVLink, then adds up what all ranks sent it, in rank order, so every
 * rank obtains the bit-identical result; bias, activation and residual are applied after the
 * sum on every rank.  One launch = one exchange of the context (see eb_comm above):
 * eb_comm_exchange_bytes(world, M rounded up to 16 / 32 / 64 / 128, N) must fit half of the
 * receive area, N must be a multiple of 4.  A context of one rank exchanges with itself (same result
 * as eb_gemm up to the rounding of the product to the operand type). */
EB_API int eb_gemm_allreduce(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
                      const void *bias, const void *residual, long long ldr, int M, int N, int K, int dtype,
                      int out_dtype, int act, int c_rows_per_batch, long long c_batch_stride,
                      const int32_t *c_row_offset_device, int c_row_offset_limit, int flags, void *workspace,
                      size_t workspace_bytes, eb_comm *comm, void *stream);

/* eb_gemm for M <= 32 rows with a LayerNorm folded in (generation steps): A holds the
 * UN-normalised rows x [M, K] and W the weights already multiplied by the LayerNorm scale,
 * W'[n][k] = W[n][k] * gamma[k], rounded to the operand type.  The kernel computes each row's
 * mean and 1/sqrt(var + eps) over the K columns (fp32, as eb_layer_norm_fwd does) and evaluates
 *   C[m][n] = act( rstd[m] * (sum_k x[m][k] W'[n][k] - mean[m] * ln_colsum[n]) + ln_bias[n] ) + residual[m][n]
 * with ln_colsum[n] = sum_k W'[n][k] and ln_bias[n] = bias[n] + sum_k W[n][k] * beta[k], both fp32
 * device vectors prepared once by the caller.  This is LayerNorm (energonai/model/endecoder.py:52,
 * 63) followed by the column-parallel projection (attention.py:73-80, mlp.py:38) in one launch,
 * without rounding the normalised activations to the operand type in between; K must be the
 * whole normalised width.  Other arguments, workspace and errors as eb_gemm. */
EB_API int eb_gemm_ln(const void *A, long long lda, const void *W, long long ldw, void *C, long long ldc,
               const float *ln_colsum, const float *ln_bias, double eps, const void *residual, long long ldr,
               int M, int N, int K, int dtype, int out_dtype, int act, int c_rows_per_batch,
               long long c_batch_stride, const int32_t *c_row_offset_device, int c_row_offset_limit, int flags,
               void *workspace, size_t workspace_bytes, void *stream);

/* ---- a chain of generation-step operations in one launch ----------------------------------- */

#define EB_OP_GEMM 0
#define EB_OP_LAYERNORM 1
#define EB_OP_REDUCE_LAYERNORM 2

/* One operation of eb_decode_chain.
 * EB_OP_GEMM: C = act(A . W^T + bias) + residual with the fields of eb_gemm (A [M,K], W [N,K],
 *   static weights).  With `exchange` != 0 the product is this rank's part of a row-parallel
 *   layer: it is not stored but sent to every rank of the chain's context (bias, residual and
 *   act must be unset, C is unused), and the next operation must be EB_OP_REDUCE_LAYERNORM.
 * EB_OP_LAYERNORM: y = gamma * norm(x) + beta over M rows of n2 elements (x, y, gamma, beta in
 *   the chain's dtype).
 * EB_OP_REDUCE_LAYERNORM: t = (sum over ranks of the preceding exchanged product) + bias +
 *   residual, rounded to the chain's dtype and written to C (rows ldc apart); then
 *   y = gamma * norm(t) + beta (gamma NULL: no normalisation).  This is the all-reduce, bias and
 *   skip connection of Linear1D_Row followed by the LayerNorm of the next sub-layer
 *   (energonai/model/endecoder.py:56-63).  n2 = the product's N. */
typedef struct eb_chain_op {
  int type;
  const void *A; long long lda; const void *W; long long ldw; void *C; long long ldc;
  const void *bias; const void *residual; long long ldr;
  int N, K, out_dtype, act, c_rows_per_batch;
  long long c_batch_stride;
  const int32_t *c_row_offset_device;
  int c_row_offset_limit;
  int exchange;
  const void *x; void *y; const void *gamma; const void *beta;
  int n2;
  double eps;
} eb_chain_op;

/* Runs up to 8 dependent operations (each consumes the previous one's complete output) of a
 * generation step, M <= 128 rows, as ONE persistent kernel: e.g. the tail of a decoder layer
 * (energonai/model/endecoder.py:48-70) out-proj -> norm2 -> FC1 -> FC2 -> next layer's norm1 ->
 * next layer's QKV projection.  Between operations the grid synchronises through arrival
 * counters in `workspace`, while the weights of the following GEMM keep streaming into shared
 * memory (weights must be static: nobody may be writing them).  Results are identical to
 * running eb_gemm / eb_layer_norm_fwd one after the other.  Buffers written by an operation
 * must not alias anything an earlier operation of the same chain reads.  `workspace`:
 * eb_decode_chain_workspace_bytes(...) bytes, 16-byte aligned, zero-filled once before first
 * use; launches sharing it must not overlap on the device.  All grid-wide waits are bounded
 * (1 s, eb_device_status).  The kernel needs every SM to host one of its CTAs at the same time:
 * do not run it concurrently with other work that pins shared memory on the device.
 * `comm` (NULL unless an operation exchanges): the tensor-parallel context; a launch performs
 * as many exchanges of it as it has exchanged products, and while the grid waits for the other
 * ranks' parts the weights of the following GEMM keep arriving, so the NVLink flight and the
 * ranks' skew hide under the weight stream. */
EB_API int eb_decode_chain(const eb_chain_op *ops, int n_ops, int M, int dtype, void *workspace,
                    size_t workspace_bytes, eb_comm *comm, void *stream);
EB_API size_t eb_decode_chain_workspace_bytes(const eb_chain_op *ops, int n_ops, int M);

/* ---- the tail of a greedy generation step ----------------------------------------------------- */

/* Replaces, per step, the arg-max / concatenate / embed sequence of the reference's generation
 * loop (energonai/model/model_factory.py:124-131, energonai/model/embedding.py:44-57) by one launch:
 *   token[b]   = argmax_v logits[b][v]                      (lowest index among equal maxima)
 *   tok[b]     = token[b]  (if tok != NULL);  out_ids[b][kv_state[1]] = token[b]  (if that column < out_cols)
 *   hidden_out[b][:] = word_emb[token[b] - vocab_start][:] (zero if the token belongs to another
 *                      rank's slice of the vocabulary) + pos_emb[kv_state[0] + 1][:] (if add_pos)
 *   kv_state[0] += 1; kv_state[1] += 1                      (after every sequence has read them)
 * kv_state = {position of the token the step just processed, column of out_ids for the new token},
 * device int32[2]; counter: one device int32, zero between launches.  `dtype` is the logits' type,
 * `emb_dtype` that of the embedding tables and of hidden_out; word_emb == NULL skips the embedding.  With the vocabulary split over a
 * tensor-parallel group every rank passes its own slice and exactly one rank passes add_pos = 1;
 * the all-reduce of hidden_out that follows completes the sum. */
EB_API int eb_greedy_step(const void *logits, long long ld_logits, int batch, int vocab, int dtype, int64_t *out_ids,
                   long long ld_out, int out_cols, int64_t *tok, int32_t *kv_state, const void *word_emb,
                   long long vocab_start, int vocab_rows, const void *pos_emb, int pos_rows, int add_pos, int hidden,
                   int emb_dtype, void *hidden_out, long long ld_hidden, int32_t *counter, void *stream);

/* ---- fused attention ----------------------------------------------------------------------- */

/* Replaces the score / mask / softmax / value products of MultiHeadAttention1D.forward
 * (energonai/model/attention.py:105-124) for a whole prompt, without materialising the
 * [batch, heads, q_len, kv_len] score tensor:
 *   out[b,i,h,:] = softmax_j( scale * q[b,i,h,:].k[b,j,h,:] + mask[b,j] ; causal ) . v[b,j,h,:]
 * q, k, v, out are addressed as base + b*batch_stride + row*row_stride + h*head_dim + d
 * (elements), so they may be column slices of one fused projection buffer.  mask is an
 * additive per-key row [batch][kv_len] in the tensor dtype (the reference's 0 / -10000
 * padding mask) or NULL.  causal != 0 hides keys j > i + (kv_len - q_len).  head_dim 64 or
 * 128, dtype fp16 or bf16, strides multiples of 8.  Softmax statistics are fp32. */
EB_API int eb_attention_prefill(const void *q, const void *k, const void *v, void *out, const void *mask,
                         long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                         long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                         long long o_batch_stride, long long o_row_stride, long long mask_batch_stride, int batch,
                         int heads, int q_len, int kv_len, int head_dim, int causal, float scale, int dtype,
                         void *stream);

/* The same product on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
 * memory, Q / K / V tiles by TMA): the kernel for prompts.  Same arguments and result as
 * eb_attention_prefill (the probabilities are rounded to the tensor dtype before the value
 * product, as the reference's softmax output is); scale must be positive.  One CTA per 256
 * query rows of a (sequence, head): for q_len well under 128 prefer eb_attention_prefill.  A
 * wait that runs out is reported by eb_device_status ("where" codes 100 and up). */
EB_API int eb_attention_prefill_tc(const void *q, const void *k, const void *v, void *out, const void *mask,
                            long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                            long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                            long long o_batch_stride, long long o_row_stride, long long mask_batch_stride, int batch,
                            int heads, int q_len, int kv_len, int head_dim, int causal, float scale, int dtype,
                            void *stream);

/* The same product for one new query row per sequence against the cached keys/values (the
 * generation step; replaces the torch.cat past_cache reads of attention.py:86-98 followed by
 * attention.py:105-124).  q[b] is the row at base + b*q_batch_stride + (kv_len-1)*q_row_stride +
 * h*head_dim: q_row_stride 0 for a plain [batch, heads*head_dim] tensor, or the cache row
 * stride when the query projection sits in the cache row of the new token.  All kv_len cached
 * keys are visible.  kv_len_device, if non-NULL, is a device int32 that overrides
 * kv_len at run time (so a captured launch can be replayed while the cache grows); kv_len, when
 * positive, is then the capacity the device value is clamped to.  The key
 * range is split over `nsplit` CTAs per (sequence, head); for nsplit > 1 `scratch` must hold
 * eb_attention_decode_scratch_bytes(...) bytes, 16-byte aligned, zero-filled once before
 * first use.  Calls sharing a scratch must not overlap on the device. */
EB_API int eb_attention_decode(const void *q, const void *k, const void *v, void *out, const void *mask,
                        long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                        long long k_row_stride, long long v_batch_stride, long long v_row_stride, long long o_batch_stride,
                        long long mask_batch_stride, int batch, int heads, int kv_len, const int32_t *kv_len_device,
                        int head_dim, float scale, int dtype, int nsplit, void *scratch, size_t scratch_bytes,
                        void *stream);
EB_API size_t eb_attention_decode_scratch_bytes(int batch, int heads, int head_dim, int nsplit);

/* The same computation as eb_attention_decode for callers that cannot allocate device memory
 * (a serving worker whose pool was carved up at start-up, code running while the allocator is
 * locked, a host that only receives raw pointers): the split-KV scratch is an 8 MiB array built
 * into the library, resident on every GPU that loads it until the process exits.  The caller
 * passes inputs and outputs only.  Requests whose scratch (see
 * eb_attention_decode_scratch_bytes) exceeds 8 MiB are refused with EB_ELIMIT.  The first call on
 * each device looks the array's address up and clears its counters on `stream`; make that
 * first call outside any stream capture.  All calls on a device share the one array and it
 * keeps the previous call's contents, so calls that overlap on the GPU (two streams, two
 * threads) race: serialise them, the first call per device included (the address look-up is
 * guarded against concurrent host threads, but the clearing of the counters is ordered only
 * on the stream of the call that does it).  A request with nsplit 1 uses no scratch and skips
 * all of this.  Nothing is allocated or freed.  No counterpart in the reference. */
EB_API int eb_attention_decode_noalloc(const void *q, const void *k, const void *v, void *out, const void *mask,
                                long long q_batch_stride, long long q_row_stride, long long k_batch_stride,
                                long long k_row_stride, long long v_batch_stride, long long v_row_stride,
                                long long o_batch_stride, long long mask_batch_stride, int batch, int heads,
                                int kv_len, const int32_t *kv_len_device, int head_dim, float scale, int dtype,
                                int nsplit, void *stream);

/* Device-side waits are bounded; when one expires the kernel records it and returns.  This
 * reads (synchronously) the status word of the current device: out4[0] = 0 or EB_ETIMEDOUT,
 * out4[1] = which wait, out4[2] = block, out4[3] = detail.  clear != 0 resets it.  No
 * counterpart in the reference, whose kernels have no waits. */
EB_API int eb_device_status(int *out4, int clear);

#ifdef __cplusplus
}
#endif
#endif /* ENERGON_B200_H */
