/*
 * flashloop_b200 -- C ABI of the B200 (sm_100a) kernels for FlashLoop's late-loop decode path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches on that
 * stream without synchronising, allocates nothing, and returns FL_OK or a negative status
 * (fl_last_error() holds the message of the calling thread's last failure).  Outputs and the
 * scratch workspace are caller-provided, so a decode step built from these calls can be
 * captured in a CUDA graph.
 *
 * Each declaration cites the interface of the reference project (paths relative to its root)
 * that it replaces.  Where the reference is batch-one with scalar lengths, the replacement is
 * batched: per-sequence lengths live in device memory (fl_layer.seq_state).
 *
 * Fixed by the reference and by these kernels: head_dim 128, quantisation group 64
 * (flashloop/config.py:40-43, flashloop/kivi_backend.py:174-175).
 */
#ifndef FLASHLOOP_B200_H
#define FLASHLOOP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FL_HEAD_DIM 128
#define FL_GROUP 64
#define FL_STREAMS 4
/* bytes of one V record in the cache: codes, 8 bytes of metadata, 8 bytes of padding */
#define FL_V_RECORD_BYTES(bits) (16 * (bits) + 16)
#define FL_STATE_WORDS 8

/* status codes */
#define FL_OK 0
#define FL_ERR_ARGUMENT (-1)
#define FL_ERR_CUDA (-2)
#define FL_ERR_WORKSPACE (-3)
#define FL_ERR_UNSUPPORTED (-4)

/* element types of floating-point inputs */
#define FL_DTYPE_BF16 0
#define FL_DTYPE_F16 1
#define FL_DTYPE_F32 2

/* words of fl_layer.seq_state[b] */
#define FL_STATE_QUANT_TOKENS 0 /* tokens held in the packed streams (multiple of 64)          */
#define FL_STATE_TAIL_LEN 1     /* tokens held in the BF16 tail                                */
#define FL_STATE_TAIL_START 2   /* ring slot of the oldest tail token                           */
#define FL_STATE_ROWS2 3        /* rows in use in stream 2 (multiple of 64 between rollovers)   */
#define FL_STATE_ROWS3 4        /* rows in use in stream 3                                      */

typedef void* fl_cuda_stream; /* a cudaStream_t */

/*
 * One physical cache layer: the anchor stream and three delta streams of K and of V for every
 * (sequence, head), the four BF16 tails and the per-sequence state.  Replaces the tensors held
 * by CrossLoopKVLayer (flashloop/cache.py:628-657): _packed_keys/_packed_values, rank_maps,
 * _tail_keys/_tail_values, _tail_active, quantized_tokens, _tail_length.
 *
 * Streams use the row layout of flashloop/packing.py:49-54, 71-99 (one token per row, even
 * channel in the low nibble; 2-bit rows hold four channels per byte).  K metadata is one
 * float16 minimum and scale per channel per 64-row group (packing.py:146-170); V metadata is
 * one minimum and scale per token per 64-channel group (packing.py:173-197), stored in the
 * same record as the token's V codes: a V record is 16*bits bytes of codes, then float16
 * min0 min1 scale0 scale1, then 8 bytes of padding (FL_V_RECORD_BYTES(bits) in all), so that a
 * gathered read of one token's V is one contiguous request.
 *
 * Rows of (b, h) in stream s start at row_base[s][b*heads + h]; their K metadata groups start
 * at group_base[s][b*heads + h]; row r belongs to group r / 64.  Streams 2 and 3 hold only
 * the rows retained by loops 3 and 4: rank[s-2][rank_base[b] + t] is the row of logical token
 * t, or -1.  A rollover appends one 64-row block to every stream, so a compact stream's rows
 * of one metadata group are contiguous and never share a group with another block
 * (the row layout's append rule, flashloop/cache.py:202-242).
 *
 * The struct itself lives in host memory; all pointers in it are device pointers.
 */
typedef struct fl_layer {
  int32_t batch;
  int32_t heads;
  int32_t bits;          /* 4 or 2 */
  int32_t tail_capacity; /* ring size in tokens, >= 128 */
  void* k_codes[FL_STREAMS];           /* uint8 [rows][16*bits]            */
  void* k_min[FL_STREAMS];             /* float16 [groups][128]            */
  void* k_scale[FL_STREAMS];           /* float16 [groups][128]            */
  void* v_rows[FL_STREAMS];            /* uint8 [rows][FL_V_RECORD_BYTES(bits)]: codes, metadata */
  const int64_t* row_base[FL_STREAMS]; /* [batch*heads]                    */
  const int64_t* group_base[FL_STREAMS];
  int32_t* rank[2];                    /* streams 2 and 3                  */
  const int64_t* rank_base;            /* [batch]                          */
  void* tail_k[FL_STREAMS];            /* bfloat16 [batch*heads][tail_capacity][128], per loop */
  void* tail_v[FL_STREAMS];
  uint8_t* tail_active[2];             /* [batch][tail_capacity] loop-3 / loop-4 retention   */
  int32_t* seq_state;                  /* [batch][FL_STATE_WORDS]          */
} fl_layer;

const char* fl_last_error(void);
int fl_version(void);

/* ---------------------------------------------------------------------------------------
 * Quantise + pack.  Bit-exact with the reference's CPU codecs on the same input.
 * ------------------------------------------------------------------------------------- */

/* flashloop/packing.py:146-170 pack_k_per_channel.  values [bh][tokens][128] of `dtype`;
 * codes [bh][tokens][16*bits]; minimum/scale float16 [bh][ceil(tokens/64)][128]. */
int fl_pack_k_rows(const void* values, int32_t dtype, int64_t batch_heads, int64_t tokens,
                   int32_t bits, void* codes, void* minimum, void* scale, fl_cuda_stream stream);

/* flashloop/packing.py:173-197 pack_v_per_token.  minimum/scale float16, element (bh, t, g) at
 * [(bh*tokens + t)*meta_stride + g]; meta_stride 2 gives the reference's [bh][tokens][2]. */
int fl_pack_v_rows(const void* values, int32_t dtype, int64_t batch_heads, int64_t tokens,
                   int32_t bits, void* codes, void* minimum, void* scale, int64_t meta_stride,
                   fl_cuda_stream stream);

/* flashloop/kivi_backend.py:404-438 pack_kivi_k_per_channel (and its GPU twin
 * _triton_pack_kivi, :162-256).  payload int32 [bh][ceil(tokens/8)][128]. */
int fl_pack_kivi_k(const void* values, int32_t dtype, int64_t batch_heads, int64_t tokens,
                   void* payload, void* minimum, void* scale, fl_cuda_stream stream);

/* flashloop/kivi_backend.py:441-475 pack_kivi_v_per_token.  payload int32 [bh][16][tokens];
 * minimum/scale float16 [bh][2][tokens]. */
int fl_pack_kivi_v(const void* values, int32_t dtype, int64_t batch_heads, int64_t tokens,
                   void* payload, void* minimum, void* scale, fl_cuda_stream stream);

/* Packed4Bit.decode (flashloop/packing.py:108-132): code*scale + minimum in float32, rounded
 * to bfloat16.  per_channel != 0 selects K metadata ([bh][groups][128]); otherwise V metadata
 * with meta_stride as in fl_pack_v_rows.  out bfloat16 [bh][tokens][128]. */
int fl_decode_rows(const void* codes, const void* minimum, const void* scale, int32_t per_channel,
                   int64_t meta_stride, int64_t batch_heads, int64_t tokens, int32_t bits,
                   void* out, fl_cuda_stream stream);

/* Re-arrange a KIVI word stream (flashloop/kivi_backend.py:286-322) into the row layout; the
 * codes and metadata values are unchanged.  K: payload int32 [bh][ceil(tokens/8)][128] ->
 * codes [bh][tokens][64].  V: payload [bh][16][tokens] -> codes; metadata [bh][2][tokens] ->
 * [bh][tokens][meta_stride]. */
int fl_kivi_to_rows_k(const void* payload, int64_t batch_heads, int64_t tokens, void* codes,
                      fl_cuda_stream stream);
int fl_kivi_to_rows_v(const void* payload, const void* minimum, const void* scale,
                      int64_t batch_heads, int64_t tokens, void* codes, void* out_minimum,
                      void* out_scale, int64_t meta_stride, fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Readers.
 * ------------------------------------------------------------------------------------- */

/* The reference allocates its logits / probability scratch inside every call with torch::empty
 * (flashloop/csrc/kivi_outer_gemv_cuda.cu:2016-2020); here the caller owns it.  Bytes of scratch
 * needed by the readers for `batch_heads` (b,h) pairs and contexts of at most
 * `max_context_tokens`.  The workspace must be zero-filled once before its first use
 * (fl_workspace_init); the readers leave it ready for the next call.  Calls that share one
 * workspace must not overlap on the GPU. */
size_t fl_reader_workspace_bytes(int64_t batch_heads, int64_t max_context_tokens);
int fl_workspace_init(void* workspace, size_t bytes, fl_cuda_stream stream);

/* Synchronises `stream` and copies the workspace's status word (its first word, whatever
 * batch_heads is) to *status (host memory): 0, or 1 when a reader launched with this workspace
 * gave up waiting for one of its own asynchronous copies (its output is then undefined).  The
 * reference has no counterpart: its kernels never wait on anything. */
int fl_workspace_status(const void* workspace, int64_t batch_heads, int32_t* status,
                        fl_cuda_stream stream);

/* CrossLoopKVLayer.dense_source_attention (flashloop/cache.py:1644-1756) ->
 * dense_source_attention_cuda (flashloop/csrc/kivi_outer_gemv_cuda.cu:1914-2076, kernels :722,
 * :813, :870) as ONE launch: softmax(scaling * q [K_loop; K_tail; k_cur]^T) [V_loop; V_tail;
 * v_cur], K_loop = sum of dequantised streams 0..loop (loop 0..3; the reference stops at 1).
 * query/current_key/current_value bfloat16 [bh][128]; output float32 [bh][128]; logits
 * (nullable) float32 [bh][logits_stride] receives the scaled logits of the quant+tail+1 keys
 * of each sequence, as the reference returns for loop 1.  max_context_tokens bounds
 * quant+tail over the batch (host-known; sizes the grid). */
int fl_dense_source_attention(const fl_layer* layer, int32_t loop, const void* query,
                              const void* current_key, const void* current_value, float scaling,
                              float* output, float* logits, int64_t logits_stride,
                              int64_t max_context_tokens, void* workspace, size_t workspace_bytes,
                              fl_cuda_stream stream);

/* fl_dense_source_attention without a workspace argument.  It has no counterpart in the
 * reference.  It is for callers that cannot allocate device memory where they call the reader:
 * code inside a stream capture, a plugin inside a server whose device memory belongs to a
 * fixed pool, a language binding with no device allocator at hand.  The scratch is a static
 * device array of about 0.3 MB that every GPU loading this library keeps until exit; nothing
 * is allocated or freed by the call.  Limits: batch*heads <= 128 and max_context_tokens <=
 * 16384 (FL_ERR_UNSUPPORTED beyond them).  The first call on each device looks up the array's
 * device address and clears its header, so make that call outside any stream capture.  All
 * calls on a device share the array: calls that may overlap on the GPU (different streams)
 * race and must be serialised by the caller.  The first call on a device is not thread-safe:
 * make it from one host thread.  Results are identical to fl_dense_source_attention. */
int fl_dense_source_attention_static(const fl_layer* layer, int32_t loop, const void* query,
                                     const void* current_key, const void* current_value,
                                     float scaling, float* output, float* logits,
                                     int64_t logits_stride, int64_t max_context_tokens,
                                     fl_cuda_stream stream);

/* The status word of the built-in scratch of fl_dense_source_attention_static on the current
 * device, read like fl_workspace_status reads a workspace's (synchronises `stream`): 0, or 1
 * when a launch through that entry point gave up waiting for one of its own copies.  Allocates
 * nothing.  No counterpart in the reference. */
int fl_static_status(int32_t* status, fl_cuda_stream stream);

/* CrossLoopKVLayer.cached_mass_sparse_attention_delta (flashloop/cache.py:1517-1642) ->
 * sparse_attention_delta_cuda (kivi_outer_gemv_cuda.cu:1711-1912, kernels :1015, :813, :1146)
 * as ONE launch: over the valid selected logical indices (prefix rows through the rank maps,
 * tail rows, or the current token at index quant+tail) compute the subset softmax target and
 * return global_mass * (target - source_output).  indices int32 / valid uint8 [bh][capacity];
 * source_output float32 [bh][128]; global_mass float32 [bh]; output float32 [bh][128];
 * current_logits (nullable) float32 [bh] receives the scaled logit of the current token.
 * source_output and output must be 16-byte aligned.  The selected readers (this entry,
 * fl_selected_pv, fl_selected_qk) hold a row's number within its (b,h) in 31 bits.  Indices
 * may come in any order; an ascending list (what fl_select_decode_keys emits) is the fast
 * case, because consecutive slots then share K metadata groups. */
int fl_sparse_attention_delta(const fl_layer* layer, int32_t loop, const void* query,
                              const void* current_key, const void* current_value,
                              const int32_t* indices, const uint8_t* valid, int64_t capacity,
                              const float* source_output, const float* global_mass, float scaling,
                              float* output, float* current_logits, void* workspace,
                              size_t workspace_bytes, fl_cuda_stream stream);

/* CrossLoopKVLayer.pv (flashloop/cache.py:1358-1515) -> pv_cross_loop_cuda
 * (kivi_outer_gemv_cuda.cu:1625-1709) fused with the current-token term of
 * FlashLoopEngine._selected_value_aggregate (flashloop/engine.py:346-371):
 * output = sum_j weights[j] * V_loop[indices[j]], the row of index quant+tail being
 * current_value (nullable: then that index contributes nothing).  weights float32
 * [bh][capacity]; valid nullable. */
int fl_selected_pv(const fl_layer* layer, int32_t loop, const float* weights,
                   const int32_t* indices, const uint8_t* valid, int64_t capacity,
                   const void* current_value, float* output, void* workspace,
                   size_t workspace_bytes, fl_cuda_stream stream);

/* CrossLoopKVLayer.qk (flashloop/cache.py:1202-1356) -> qk_cross_loop_cuda
 * (kivi_outer_gemv_cuda.cu:1541-1623): unscaled logits of the selected logical rows;
 * index quant+tail reads current_key (nullable).  logits float32 [bh][capacity]; slots that
 * are invalid or out of range receive 0. */
int fl_selected_qk(const fl_layer* layer, int32_t loop, const void* query, const int32_t* indices,
                   const uint8_t* valid, int64_t capacity, const void* current_key, float* logits,
                   fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Append.
 * ------------------------------------------------------------------------------------- */

/* CrossLoopKVLayer.append_decode_token + _roll_one_group (flashloop/cache.py:1758-1838) and the
 * block re-encode they trigger (from_prefill / _encode_initial_prefix, cache.py:752-817,
 * 1008-1074), for every sequence at once and with no host round trip: the four loops' K and V
 * rows of one decoded token per sequence (keys[r], values[r]: bfloat16 [batch*heads][128],
 * r = 0..3; the two tables are host arrays of device pointers) go into the BF16 tail rings;
 * every sequence whose tail thereby reaches 128 tokens has its oldest 64 tail tokens turned into
 * one new 64-row block of all eight streams (anchor, delta-2, delta-3/4 of the retained rows,
 * bfloat16 residual arithmetic and codes bit-exact with the reference), its rank maps extended
 * and its seq_state advanced.  The caller guarantees room for the new block in every stream. */
int fl_append_decode_token(const fl_layer* layer, const void* const* keys, const void* const* values,
                           fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Selection.
 * ------------------------------------------------------------------------------------- */

/* select_decode_keys (flashloop/selection.py:72-88) and the inline selection of
 * FlashLoopEngine.decode (flashloop/engine.py:438-481: softmax, topk, sort, gather, pad,
 * mass, renormalise) as ONE launch per call: per (b,h) pick the budget = min(N, max(1,
 * ceil(N*fraction))) largest of N float32 values (ties: lower index first), emit their indices
 * in ascending order padded with zeros to `capacity`, the validity mask, the selected global
 * softmax mass and (nullable) the selected weights divided by that mass.
 * values [bh][values_stride]; if values_are_logits != 0 they are scaled logits and the weights
 * are their softmax over the N keys, else they are the weights themselves.
 * N = n_keys when seq_state is NULL, else quant+tail+1 of each sequence.
 * capacity must be >= (budget/64 + 1)*64 for the largest N (engine.py:100). */
int fl_select_decode_keys(const float* values, int64_t values_stride, int32_t batch, int32_t heads,
                          int32_t n_keys, const int32_t* seq_state, double fraction,
                          int32_t values_are_logits, int32_t* indices, uint8_t* valid,
                          int64_t capacity, int32_t* counts, float* global_mass,
                          float* selected_weights, fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Token retention (sparse late loops of the prefill).
 * ------------------------------------------------------------------------------------- */

/* _hidden_delta_score (flashloop/engine.py:78-81): ||h_r - h_{r-1}|| / max(||h_r||, 1e-12) per
 * token row, float32.  current/previous bfloat16 [rows][hidden], hidden a multiple of 8. */
int fl_hidden_delta_score(const void* current, const void* previous, int64_t rows, int32_t hidden,
                          float* scores, fl_cuda_stream stream);

/* select_prefill_tokens (flashloop/selection.py:26-69) fused with the position list and rank
 * map built around it (flashloop/engine.py:276-277, flashloop/cache.py:281-289): per sequence
 * keep min(max(1, ceil(tokens*fraction)), eligible) tokens, the last token first when forced,
 * then the highest scores among the other eligible tokens (ties: lower index).  scores float32
 * [batch][tokens]; eligible uint8 [batch][tokens] or NULL; mask uint8 [batch][tokens];
 * positions int32 [batch][tokens] = kept positions ascending then -1; rank int32
 * [batch][tokens] = index into positions or -1; count int32 [batch]. */
int fl_select_prefill_tokens(const float* scores, const uint8_t* eligible, int32_t batch,
                             int32_t tokens, double fraction, int32_t force_last_token,
                             uint8_t* mask, int32_t* positions, int32_t* rank, int32_t* count,
                             fl_cuda_stream stream);

/* The row movement of the sparse prefill loops (flashloop/prefill.py:144, 154-158, 193-194,
 * 237, 252-254: index_select of active rows, index_copy_ of their results).  full is
 * [outer][full_rows][row_bytes], compact is [outer][compact_rows][row_bytes]; sequence
 * outer / per_sequence owns positions[seq*positions_stride + r], r < count[seq].
 * fl_gather_rows: compact[r] = full[positions[r]]; fl_scatter_rows: full[positions[r]] = compact[r].
 * row_bytes must be a multiple of 16. */
int fl_gather_rows(const void* full, void* compact, const int32_t* positions, const int32_t* count,
                   int64_t positions_stride, int64_t outer, int32_t per_sequence, int64_t full_rows,
                   int64_t compact_rows, int32_t row_bytes, fl_cuda_stream stream);
int fl_scatter_rows(void* full, const void* compact, const int32_t* positions, const int32_t* count,
                    int64_t positions_stride, int64_t outer, int32_t per_sequence, int64_t full_rows,
                    int64_t compact_rows, int32_t row_bytes, fl_cuda_stream stream);

/* The prefill-time residual encoder: CrossLoopKVLayerBuilder.from_loop1 / add_loop2 /
 * _install_sparse_streams / finalize and _encode_initial_prefix (flashloop/cache.py:343-397,
 * 415-439, 469-508, 510-625, 1008-1074) in three launches.  keys / values: four pointers (loops
 * 1-4) to bfloat16 [sequence_count][heads][tokens][128] of sequences sequence_begin .. of the
 * layer.  The first seq_state[b][FL_STATE_QUANT_TOKENS] tokens of every sequence are encoded:
 * stream 0 = loop 1, stream 1 = loop 2 - decode(stream 0), streams 2 / 3 = loops 3 / 4 minus the
 * running reconstruction at the retained positions, 64 compact rows per K metadata group; every
 * subtraction and add-back rounded to bfloat16 as the reference's tensor ops round.  positions3 /
 * positions4: int32 [sequence_count][positions_stride], retained positions ascending then -1
 * (both NULL: no compact streams).  recon_k / recon_v: scratch of the size of one K / V input.
 * Rank maps, tails and state words are the caller's to fill. */
int fl_encode_prefill(const fl_layer* layer, int32_t sequence_begin, int32_t sequence_count, int64_t tokens,
                      const void* const* keys, const void* const* values, const int32_t* positions3,
                      const int32_t* positions4, int64_t positions_stride, void* recon_k, void* recon_v,
                      fl_cuda_stream stream);

/* The same encoder one loop at a time, for a prefill that frees every loop's K/V as soon as it
 * is packed: CrossLoopKVLayerBuilder.from_loop1 (stage 0, flashloop/cache.py:343-397), add_loop2
 * (stage 1, :415-439) and the two halves of _install_sparse_streams / finalize (stages 2 and 3,
 * :469-508, 510-625).  Every stage reads the base it subtracts back from the streams already
 * packed in the layer (decode(anchor); decode(anchor) + decode(delta-2); + decode(delta-3) at the
 * position's loop-3 row), as the reference's builder does, so no reconstruction scratch is kept
 * between the stages and the codes are the same bits as fl_encode_prefill's.  keys / values:
 * bfloat16 [sequence_count][heads][rows][128] of the stage's loop.  Stages 0 and 1: rows = prompt
 * tokens.  Stages 2 and 3: positions int32 [sequence_count][positions_stride] (retained positions
 * ascending, then -1); with compact_input != 0 input row i of a sequence is its i-th retained row
 * (rows = rows per sequence of that compact tensor), otherwise the row of its logical position.
 * Stage 3 needs the layer's loop-3 rank map filled. */
int fl_encode_prefill_stage(const fl_layer* layer, int32_t sequence_begin, int32_t sequence_count, int64_t rows,
                            int32_t stage, const void* keys, const void* values, const int32_t* positions,
                            int64_t positions_stride, int32_t compact_input, fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Elementwise glue of one decode step around the readers (bfloat16 rows, one token per row).
 * Each restates module arithmetic of the reference's decode loop with the roundings of
 * bfloat16 tensor ops and replaces five to eight framework launches by one.
 * ------------------------------------------------------------------------------------- */

/* The RMSNorm modules of flashloop/engine.py:396 (input_layernorm) and :533-537 (the sandwich
 * norms around attention and MLP):  out = [residual +] weight * bf16(s * rsqrt(mean(s^2) + eps))
 * with s = x, or s = bf16(addend + x) when addend is given (the `projected0 + o_proj(delta)` of the
 * late loops, flashloop/engine.py:529-531, folded in); with weight2/out2 also out2 = weight2 *
 * bf16(out * rsqrt(mean(out^2) + eps2)), i.e. the next norm of the residual stream in the same
 * launch.  x, addend, residual, out, out2: [rows][width]. */
int fl_rmsnorm(const void* x, const void* addend, const void* residual, const void* weight, float eps,
               const void* weight2, float eps2, int64_t rows, int32_t width, void* out, void* out2,
               fl_cuda_stream stream);

/* ---------------------------------------------------------------------------------------
 * Tensor-parallel decode.  No counterpart in the reference, which runs on one GPU
 * (flashloop/engine.py:112-150): with the heads and FFN columns of a layer split over the
 * ranks, the o_proj and down_proj outputs of flashloop/engine.py:531-537 are partial sums, and
 * these entry points sum them over the ranks inside the norm launch that consumes them.
 *
 * A communicator is one device allocation per rank (receive slots for two calls in flight,
 * arrival flags, a sequence counter, a status word), mapped into the other ranks' processes
 * through CUDA IPC.  One process per GPU; every rank makes the same sequence of calls.
 * ------------------------------------------------------------------------------------- */

/* Size of the opaque handle fl_comm_create writes (a cudaIpcMemHandle_t).  No counterpart in the
 * reference. */
size_t fl_comm_handle_bytes(void);

/* Allocate this rank's part on the current device for rows of `width` bfloat16 values
 * (a multiple of 8, at most 8192), up to rows_max rows per call, world <= 8 ranks.
 * *comm_out receives the communicator, handle_out (fl_comm_handle_bytes() bytes) the handle
 * the other ranks need.  The caller carries the handles between the processes.  No counterpart
 * in the reference. */
int fl_comm_create(int32_t rank, int32_t world, int32_t rows_max, int32_t width, void** comm_out,
                   void* handle_out);

/* handles: world handles in rank order (this rank's own is not opened).  All ranks must have
 * returned from fl_comm_connect before any of them calls fl_allreduce_rmsnorm.  No counterpart
 * in the reference. */
int fl_comm_connect(void* comm, const void* handles);

/* Unmaps the peers' parts and frees this rank's.  No counterpart in the reference. */
int fl_comm_destroy(void* comm);

/* *status = 0, or 1 after a wait for a peer's rows ran out in some call since the last reset
 * (that call summed what had arrived).  Synchronises `stream`; with reset != 0 clears it.
 * No counterpart in the reference. */
int fl_comm_status(void* comm, int32_t* status, int32_t reset, fl_cuda_stream stream);

/* One launch per rank:  s = [addend +] sum over ranks of x  (float32 in rank order, rounded to
 * bfloat16); then as fl_rmsnorm on s:  out = [residual +] weight * bf16(s * rsqrt(mean(s^2) +
 * eps)), and with weight2/out2 the next norm of `out`.  weight == NULL: out = s and nothing
 * else.  sum_out (or NULL) receives s.  x, addend, residual, sum_out, out, out2:
 * [rows][width] bfloat16 of this rank, rows <= rows_max, 16-byte aligned.
 * Each rank stores its rows into every rank's receive slots with plain peer stores, then waits
 * for the others' rows; a wait gives up after wait_limit polls (0 = the default, a few seconds)
 * and raises the status word instead of blocking.  skip_store != 0 makes this rank publish
 * nothing in this call (the way a test lets the other ranks' waits run out).
 * Allocation-free and recordable in a CUDA graph: the sequence number lives on the device.
 * The arithmetic after the sum is that of the reference's norm modules
 * (flashloop/engine.py:533-537), as fl_rmsnorm. */
int fl_allreduce_rmsnorm(void* comm, const void* x, const void* addend, const void* residual,
                         const void* weight, float eps, const void* weight2, float eps2, int64_t rows,
                         void* sum_out, void* out, void* out2, int32_t skip_store, int32_t wait_limit,
                         fl_cuda_stream stream);

/* The bias-free nn.Linear modules of a decode step -- q/k/v_proj and o_proj (flashloop/engine.py:410-419,
 * 531), gate/up/down_proj (flashloop/weights.py:108-117), lm_head (flashloop/engine.py:342) -- for at
 * most 16 rows (one token per sequence):  out[m][n] = bf16(sum_k x[m][k] * weight[n][k]), float32
 * accumulation, the weight streamed once.  x [rows][in_features] of x_dtype FL_DTYPE_BF16 or
 * FL_DTYPE_F32 (rounded to bfloat16 as it is read: the `.to(dtype)` the reference applies to the
 * readers' float32 output before o_proj); weight [out_features][in_features] bfloat16; 16-byte
 * aligned; in_features a multiple of 32, out_features of 16.  With swiglu != 0 the weight is the gate
 * rows followed by the up rows (out_features = 2F, a multiple of 32) and out [rows][F] receives
 * bf16(silu(bf16 gate)) * bf16 up, i.e. fl_swiglu of the product in the same launch. */
int fl_linear_rows(const void* x, int32_t x_dtype, const void* weight, int64_t rows, int32_t out_features,
                   int32_t in_features, int32_t swiglu, void* out, fl_cuda_stream stream);

/* The fused Q/K/V projection of flashloop/weights.py:74-105 (project_qkv) followed by the
 * view/transpose and _apply_rope of flashloop/engine.py:59-75, 410-419, for at most 16 rows: weight
 * [3 * heads * 128][in_features] = q rows, k rows, v rows; cos/sin [rows][128]; q_out, k_out (rotated)
 * and v_out [rows][heads * 128].  The same arithmetic as fl_linear_rows followed by fl_rope_split. */
int fl_qkv_rope_rows(const void* x, const void* weight, int64_t rows, int32_t heads, int32_t in_features,
                     const void* cosv, const void* sinv, void* q_out, void* k_out, void* v_out,
                     fl_cuda_stream stream);

/* fl_linear_rows for a weight with few output rows (o_proj, down_proj:
 * flashloop/engine.py:531, flashloop/weights.py:108-117 fused_mlp's down projection) on one GPU,
 * split over `splits` (1..4) slices of in_features: partial [splits][rows][out_features] float32
 * receives every slice's sums; their sum in slice order, rounded once to bfloat16, is what
 * fl_linear_rows would have written.  fl_rmsnorm_partial takes them as they are.  in_features a
 * multiple of 32 * splits with at most 1536 values per slice, out_features a multiple of 8. */
int fl_linear_rows_partial(const void* x, int32_t x_dtype, const void* weight, int64_t rows,
                           int32_t out_features, int32_t in_features, int32_t splits, float* partial,
                           fl_cuda_stream stream);

/* fl_rmsnorm whose input is bf16(sum of `splits` float32 slices [splits][rows][width]) as left by
 * fl_linear_rows_partial (no counterpart in the reference: the sum belongs to the projection);
 * sum_out (nullable) receives that bfloat16 input. */
int fl_rmsnorm_partial(const float* partial, int32_t splits, const void* addend, const void* residual,
                       const void* weight, float eps, const void* weight2, float eps2, int64_t rows,
                       int32_t width, void* sum_out, void* out, void* out2, fl_cuda_stream stream);

/* The view/transpose of the Q/K/V projections and _apply_rope (flashloop/engine.py:59-75,
 * 410-419) for one token per row: q_out/k_out = x * cos + rotate_half(x) * sin, v_out = v.
 * q_in/k_in/v_in: rows of heads*128 values, in_stride elements apart (three slices of one
 * fused projection or three separate tensors); cos/sin [rows][128]; outputs [rows][heads*128]. */
int fl_rope_split(const void* q_in, const void* k_in, const void* v_in, int64_t in_stride, const void* cosv,
                  const void* sinv, int64_t rows, int32_t heads, void* q_out, void* k_out, void* v_out,
                  fl_cuda_stream stream);

/* fused_mlp's activation (flashloop/weights.py:108-117): out = bf16(silu(gate)) * up with
 * gate_up = [rows][2*width] (gate then up), out [rows][width]. */
int fl_swiglu(const void* gate_up, int64_t rows, int32_t width, void* out, fl_cuda_stream stream);

#ifdef __cplusplus
}
#endif

#endif /* FLASHLOOP_B200_H */
