/*
 * frwkv_b200 -- C ABI of the B200 (sm_100a) WKV7 time-mix kernels.
 *
 * Every entry point takes raw device pointers and sizes, launches on the given
 * stream and returns immediately (no synchronisation, no allocation, no
 * exceptions).  Return value: FRWKV_OK, or a negative FRWKV_ERR_* code with a
 * message available from frwkv_last_error() on the calling thread.  All tensors
 * are contiguous.  "io16" tensors are fp16 or bf16 according to io_dtype.
 * Tensor pointers are expected on 32-byte boundaries (a device allocation, or an
 * offset of whole token rows or state tiles into one): the kernels move rows as
 * 16- and 32-byte vectors.  The chunked entries (fused forward, adjoint scan,
 * chunk backward) check this and return FRWKV_ERR_INVALID_ARGUMENT otherwise.
 *
 * Each declaration names the interface of the FlashRWKV2 reference it replaces
 * (paths inside the reference project).
 */
#ifndef FRWKV_B200_H_
#define FRWKV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* frwkv_stream_t; /* == cudaStream_t */

enum {
  FRWKV_DTYPE_FP16 = 0,
  FRWKV_DTYPE_BF16 = 1,
};

enum {
  FRWKV_OK = 0,
  FRWKV_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive size, size over a limit */
  FRWKV_ERR_UNSUPPORTED = -2,      /* shape or dtype this build has no kernel for */
  FRWKV_ERR_CUDA = -3,             /* the CUDA runtime rejected the launch */
};

/* Bits written to the metadata status word (0 = valid).  Same values as the
 * reference's MetadataError (csrc/validation/recurrent_metadata.cu:15-20). */
enum {
  FRWKV_META_INVALID_ENDPOINT = 1,
  FRWKV_META_INVALID_RANGE = 2,
  FRWKV_META_INVALID_SLOT = 4,
  FRWKV_META_DUPLICATE_SLOT = 8,
  /* Not in the reference: set by a decode kernel of this library whose bounded wait on a copy ran out.  The
   * sequences it could not finish read as NaN and their state tiles keep their old value; because the bit stays in
   * the status word, every later call that is given the same word fails closed like a call with bad metadata. */
  FRWKV_META_WAIT_TIMEOUT = 16,
};

/* ABI version of this header (bumped on any signature change). */
int frwkv_abi_version(void);

/* Message of the last error returned on this thread ("" if none). */
const char* frwkv_last_error(void);

/* *flag (device int32) = 1 when cu_seqlens[i] == i for i = 0..B and state_indices[i] == i for i = 0..B-1, else 0:
 * every sequence is one token and owns the state slot of its own number.  See FRWKV_RECURRENT_DIRECT_SLOTS. */
int frwkv_recurrent_metadata_is_direct(const int32_t* cu_seqlens, const int32_t* state_indices, int num_sequences,
                                       int32_t* flag, frwkv_stream_t stream);

/*
 * Validate packed-sequence metadata on the device and snapshot it.
 * Replaces prepare_recurrent_metadata_cuda / validate_recurrent_metadata_kernel
 * (csrc/validation/recurrent_metadata.cu:22-128).
 *   cu_seqlens [B+1], state_indices [B] int32; 1 <= B <= 65535.
 *   status [2] int32: status[0] = OR of FRWKV_META_* bits, status[1] = longest
 *   sequence length found.  cu_snapshot [B+1], idx_snapshot [B] receive copies
 *   taken before validation (the values later kernels must use).
 */
int frwkv_validate_recurrent_metadata(const int32_t* cu_seqlens, const int32_t* state_indices,
                                      int num_sequences, int total_tokens, int state_pool_size,
                                      int32_t* status, int32_t* cu_snapshot, int32_t* idx_snapshot,
                                      frwkv_stream_t stream);

/*
 * Validate the chunk tables of the training operators on the device: status[0] (int32, cleared first) receives
 * FRWKV_META_INVALID_RANGE if a chunk lies outside [0, total_tokens], holds more than max_chunk tokens or does not
 * start where its predecessor in the same sequence ends, FRWKV_META_INVALID_ENDPOINT if the offsets do not rise from 0
 * to num_chunks.  Kernels given this word as metadata_status fail closed (NaN outputs, states untouched), so a bad
 * caller-built table cannot drive out-of-range accesses.  The reference validates its RL chunk tables on the host
 * (csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_forward.cpp:100-133).
 */
int frwkv_validate_chunk_tables(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                const int32_t* chunk_ends, int num_sequences, int num_chunks, int total_tokens,
                                int max_chunk, int32_t* status, frwkv_stream_t stream);

/*
 * WKV7 recurrence over packed sequences with an fp32 state pool updated in place.
 * Replaces recurrent_fp32_from_decay_logits_cuda
 * (csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:448-508).
 *   per token:  w = exp(-exp(-0.5) * sigmoid(decay_logits + decay_bias))
 *               sa = S^T a ; S = diag(w) S + b sa^T + k v^T ; y = scale * S^T r
 *   r, decay_logits, k, v, a, b, y : io16 [total_tokens, H, D]
 *   state_pool : fp32 [slots, H, D, D] (key row, value column)
 *   decay_bias : io16 [H, D] or NULL;  y_fp32 : fp32 [total_tokens, H, D] or NULL
 *     (the unrounded outputs, for precision checks)
 *   metadata_status : int32 device word; when *metadata_status != 0 the kernel
 *     fills y with NaN and leaves the state pool untouched.  The kernels only read it, except that a decode
 *     kernel whose bounded wait runs out ORs FRWKV_META_WAIT_TIMEOUT into it (hence the cast from const).
 *   head_size 64 (tuned kernels), 128 or 256 (general kernel).
 */
int frwkv_wkv7_recurrent_fp32io16_forward_varlen(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    float* state_pool, const void* r, const void* decay_logits, const void* k, const void* v,
    const void* a, const void* b, const void* decay_bias, void* y, float* y_fp32,
    int total_tokens, int num_sequences, int num_heads, int head_size, int max_seqlen,
    int io_dtype, float scale, frwkv_stream_t stream);

/* Same, with flags: bit 0 = FRWKV_RECURRENT_REVERSE_ORDER, walk the (sequence, head) tiles from the far end of the
 * batch.  The result does not depend on it.  A decode loop that alternates the bit between consecutive steps finds
 * the state tiles it wrote last still in L2 (126 MB on B200) when the next step starts with them.
 * bit 1 = FRWKV_RECURRENT_DIRECT_SLOTS: the caller has established (frwkv_recurrent_metadata_is_direct) that
 * cu_seqlens[i] == i and state_indices[i] == i; with max_seqlen == 1 and total_tokens == num_sequences the register
 * kernel (batches below the ring kernel's threshold) then reads neither table and is one dependent round trip
 * shorter per launch.  The status word is still honoured.  Ignored where it does not apply. */
enum { FRWKV_RECURRENT_REVERSE_ORDER = 1, FRWKV_RECURRENT_DIRECT_SLOTS = 2 };
int frwkv_wkv7_recurrent_fp32io16_forward_varlen_ex(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    float* state_pool, const void* r, const void* decay_logits, const void* k, const void* v,
    const void* a, const void* b, const void* decay_bias, void* y, float* y_fp32,
    int total_tokens, int num_sequences, int num_heads, int head_size, int max_seqlen,
    int io_dtype, float scale, int flags, frwkv_stream_t stream);

/*
 * WKV7 recurrence with an fp16 state pool updated in place (the "Albatross" contract).
 * Replaces recurrent_fp16_from_decay_logits of the reference
 * (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu; Python wrapper
 * flashrwkv2/tmix/wkv7/__init__.py:280-339; contract restated in tests/tmix/wkv7/test.py:216-277).
 *   per token:  delta = half(exp(-exp(-0.5) * sigmoid(decay_logits + decay_bias)) - 1 + dither)
 *               sa = S^T a ; S = half(S + S delta + b sa^T + k v^T) ; y = scale * S^T r  (rounded new state)
 *               dither = int32(uint32(phase) * 2654435769) * 2^-41,
 *               phase = head * D + key channel + elapsed_state_pool[slot] + index of the token in its sequence
 *   state_pool : fp16 [slots, H, D, D];  elapsed_state_pool : int32 [slots], read only;
 *   the other arguments as in frwkv_wkv7_recurrent_fp32io16_forward_varlen_ex.  head_size 64 (tuned kernels), 128 or 256 (general kernel).
 */
int frwkv_wkv7_recurrent_fp16_forward_varlen(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    const int32_t* elapsed_state_pool, void* state_pool, const void* r, const void* decay_logits, const void* k,
    const void* v, const void* a, const void* b, const void* decay_bias, void* y, int total_tokens, int num_sequences,
    int num_heads, int head_size, int max_seqlen, int io_dtype, float scale, int flags, frwkv_stream_t stream);

/* elapsed_state[i] += amount for all `count` counters (32-bit wrap-around).
 * Replaces recurrent_fp16_advance_i32 (flashrwkv2/tmix/wkv7/__init__.py:65-80). */
int frwkv_recurrent_fp16_advance_i32(int32_t* elapsed_state, long long count, int amount, frwkv_stream_t stream);

/* elapsed_state_pool[state_indices[i]] += cu_seqlens[i+1] - cu_seqlens[i]; nothing is touched when
 * *metadata_status != 0.  Replaces recurrent_fp16_advance_i32_varlen (flashrwkv2/tmix/wkv7/__init__.py:83-140). */
int frwkv_recurrent_fp16_advance_i32_varlen(int32_t* elapsed_state_pool, const int32_t* cu_seqlens,
                                            const int32_t* state_indices, const int32_t* metadata_status,
                                            int num_sequences, frwkv_stream_t stream);

/*
 * Chunked WKV7 forward on the tensor cores: same recurrence and tensors as
 * frwkv_wkv7_recurrent_fp32io16_forward_varlen, evaluated chunk by chunk (chunk length <= 64).
 * Replaces the reference's chunk families: infer_chunk_bf16_forward_varlen_cuda
 * (csrc/sm120/tmix/wkv7/infer_chunk_bf16_forward_varlen.cu:268-334), rl_infctx_chunk_fp32io16_forward
 * (csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_forward.cpp:157-229) and the forward of
 * statetune_recurrent_fp32io16 (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu:32-130).
 *   seq_chunk_offsets [B+1], chunk_starts [Cn], chunk_ends [Cn] int32: sequence s owns chunks
 *     [seq_chunk_offsets[s], seq_chunk_offsets[s+1]); chunk c covers tokens [chunk_starts[c], chunk_ends[c]),
 *     at most 64 of them, consecutive chunks of a sequence being adjacent token ranges.
 *   state_pool fp32 [slots,H,64,64]: initial state in, final state out (in place); sequence s uses slot
 *     state_indices[s], or slot s when state_indices is NULL.
 *   boundary fp32 [Cn,H,64,64] or NULL: receives the state at the start of every chunk.
 *   workspace: frwkv_wkv7_chunk_workspace_bytes(Cn, H) bytes of device memory, 128-byte aligned.
 *   error_flag: device int32 or NULL; set non-zero if a tensor-core completion wait ran out (outputs invalid).
 *   metadata_status / y_fp32 / decay_bias / scale: as in the recurrent entry point.
 */
size_t frwkv_wkv7_chunk_workspace_bytes(int num_chunks, int num_heads);
int frwkv_wkv7_chunk_fp32io16_forward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, void* workspace, size_t workspace_bytes, int32_t* error_flag,
    int total_tokens, int num_sequences, int num_chunks, int num_heads, int head_size, int io_dtype, float scale,
    frwkv_stream_t stream);

/*
 * The same chunked forward as ONE kernel without a workspace: a CTA owns a (sequence, head) pair, keeps the
 * fp32 state on chip and walks that sequence's chunks in order, so only token rows, outputs and the optional
 * boundary / state_dot_a tensors cross HBM.  It needs enough (sequence, head) pairs to fill the GPU (two per
 * SM); frwkv_wkv7_chunk_prefers_fused() says which of the two forms is expected to be faster for a batch.
 * Replaces the same reference kernels as frwkv_wkv7_chunk_fp32io16_forward, and for training the forward of
 * statetune_recurrent_fp32io16 (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu:32-130), whose
 * state_dot_a output it produces directly:
 *   state_dot_a fp32 [N,H,64] or NULL: sa_t = S_{t-1}^T a_t for every token.
 * On a failed wait the rows of the affected (sequence, head) pairs are NaN, their state slots untouched, and
 * *error_flag is non-zero.  Other arguments as in frwkv_wkv7_chunk_fp32io16_forward.
 */
int frwkv_wkv7_chunk_prefers_fused(int num_sequences, int num_heads);
int frwkv_wkv7_chunk_fused_fp32io16_forward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, float* state_dot_a, int32_t* error_flag, int total_tokens,
    int num_sequences, int num_chunks, int num_heads, int head_size, int io_dtype, float scale,
    frwkv_stream_t stream);

/*
 * First stage of the chunked backward: the adjoint of the state at every chunk boundary, and the gradient of the
 * initial state.  The adjoint obeys a recurrence of the forward's own form (a and b exchanged, a modified key, the
 * upstream gradient in place of v, time reversed), so it is computed by the fused forward kernel walking every
 * sequence backwards.  Replaces the state-adjoint part of the reference's serial backward kernels
 * (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:139-254,
 * csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:222-282).
 *   grad_output io16 [N,H,64]; grad_state fp32 [B,H,64,64]: in = gradient of the final state (zeros if none), out =
 *   gradient of the initial state;  boundary_adjoint fp32 [Cn,H,64,64]: receives dL/dS at the END of every chunk;
 *   the modified keys scale * (w * r + (b . r) a) are made inside the kernel: no scratch tensor;
 *   metadata_status (may be NULL): the word of frwkv_validate_chunk_tables; non-zero = the scan does nothing.
 */
int frwkv_wkv7_adjoint_scan(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
                            const void* r, const void* decay_logits, const void* a, const void* b,
                            const void* decay_bias, const void* grad_output, float* grad_state,
                            float* boundary_adjoint, int32_t* error_flag,
                            const int32_t* metadata_status, int total_tokens, int num_sequences, int num_chunks,
                            int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream);

/*
 * Second stage of the chunked backward: the six token gradients of every (chunk, head), chunk-parallel on the tensor
 * cores, from the forward's boundary states and state_dot_a rows and the first stage's boundary adjoints.
 * Replaces the token-gradient part of the reference's serial backward kernels
 * (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:49-255; cuda_backward_v3 of
 * csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:163-291).
 *   final_state fp32 [B,H,64,64], boundary fp32 [Cn,H,64,64], state_dot_a fp32 [N,H,64]: outputs of the forward;
 *   boundary_adjoint fp32 [Cn,H,64,64]: output of frwkv_wkv7_adjoint_scan; grad_output io16 [N,H,64];
 *   grad_r .. grad_b io16 [N,H,64] (grad_decay_logits is with respect to the raw decay logits).
 * On a failed wait the gradients of the affected chunks are NaN and *error_flag is non-zero.  metadata_status (may be
 * NULL): the word of frwkv_validate_chunk_tables; non-zero = all gradients NaN, nothing else touched.
 */
int frwkv_wkv7_chunk_backward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends, const float* final_state,
    const float* boundary, const float* boundary_adjoint, const float* state_dot_a, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    const void* grad_output, void* grad_r, void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b,
    int32_t* error_flag, const int32_t* metadata_status, int total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream);

/*
 * The same chunked forward for hosts that may not allocate device memory (servers that gave the whole GPU to
 * fixed pools at start-up, real-time loops, plain C callers without a caching allocator).  It has no
 * counterpart in the reference, whose chunk operators allocate their workspaces through Torch on every call.
 * The workspace is a 16 MiB array built into the library (resident on every GPU that loads it), which limits a
 * call to num_chunks * num_heads <= frwkv_wkv7_chunk_noalloc_max_items() = 256; larger calls are refused with
 * FRWKV_ERR_INVALID_ARGUMENT and a message.  No cudaMalloc / cudaFree or allocating library call is made.
 * The first call on each device looks up the array's device address and, if nothing of this library ran there
 * before, makes the CUDA runtime load the library's module onto that device (a one-time, driver-side set-up that
 * may itself allocate): make that call at start-up, outside stream capture, before the no-allocation phase begins.
 * All calls share the one array: calls whose kernels could overlap on the GPU must be ordered by the caller.
 * Arguments are those of frwkv_wkv7_chunk_fp32io16_forward without workspace / workspace_bytes.
 */
size_t frwkv_wkv7_chunk_noalloc_max_items(void);
int frwkv_wkv7_chunk_fp32io16_forward_noalloc(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, int32_t* error_flag, int total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream);

/*
 * Training-side replay: per chunk, run the recurrence from the chunk-start state boundary[c] and store
 *   state_dot_a fp32 [N,H,64]      sa_t = S_{t-1}^T a_t for every token, and
 *   checkpoints fp32 [Cn,3,H,64,64] the state after tokens 16, 32 and 48 of each chunk (where the chunk is longer);
 *                                   may be NULL.
 * Replaces the state_dot_a / checkpoint outputs of forward_kernel_preload
 * (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:32-97) and statetune_recurrent_fp32io16_forward_kernel
 * (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu:32-130), and emit_outputs_kernel
 * (csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_backward.cu:45-127).
 */
int frwkv_wkv7_chunk_replay(const int32_t* chunk_starts, const int32_t* chunk_ends, const float* boundary,
                            const void* r, const void* decay_logits, const void* k, const void* v, const void* a,
                            const void* b, const void* decay_bias, float* state_dot_a, float* checkpoints,
                            int num_chunks, int num_heads, int head_size, int io_dtype, frwkv_stream_t stream);

/*
 * Dense training layout [B,T,H,64]: fills checkpoints fp32 [B,H,T/16,64,64] with the state (key row, value column)
 * after every 16 tokens, from the state at the start of every 64-token chunk (boundary fp32 [B*ceil(T/64),H,64,64],
 * chunks of one sequence consecutive) and the rows state_dot_a fp32 [B,T,H,64] that the chunk forward wrote.
 * T must be a multiple of 16.  Replaces the `s_` checkpoint stores of forward_kernel_preload
 * (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:85-92).
 */
int frwkv_wkv7_dense_checkpoints(const float* boundary, const float* state_dot_a, const void* decay_logits,
                                 const void* k, const void* v, const void* b, float* checkpoints, int batch,
                                 int tokens, int num_heads, int head_size, int io_dtype, frwkv_stream_t stream);

/*
 * WKV7 backward over packed sequences with chunk tables (see frwkv_wkv7_chunk_fp32io16_forward for their meaning).
 * Inputs: the forward's final_state [B,H,64,64], boundary [Cn,H,64,64], and the replay's checkpoints / state_dot_a;
 * grad_output io16 [N,H,64] (NULL = zero) and grad_final_state fp32 [B,H,64,64] (NULL = zero).
 * Outputs (each may be NULL): grad_r .. grad_b io16 [N,H,64] (grad_decay_logits is with respect to the raw decay
 * logits), grad_initial_state fp32 [B,H,64,64].
 * Replaces cuda_backward_v3 (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:163-291) and
 * statetune_recurrent_fp32io16_backward (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:49-255).
 */
int frwkv_wkv7_backward(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
                        const float* final_state, const float* boundary, const float* checkpoints,
                        const float* state_dot_a, const void* r, const void* decay_logits, const void* k, const void* v,
                        const void* a, const void* b, const void* grad_output, const float* grad_final_state,
                        void* grad_r, void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b,
                        float* grad_initial_state, int num_sequences, int num_heads, int head_size, int io_dtype,
                        float scale, frwkv_stream_t stream);

/*
 * WKV7 training at head sizes 128 and 256 (the plain recurrence; head size 64 has the chunked tensor-core entries
 * above).  Chunk tables as in frwkv_wkv7_chunk_fp32io16_forward, chunks of at most 64 tokens; tensors [N,H,D] 16-bit,
 * states [B,H,D,D] fp32 (key row, value column).
 *   forward: `state` holds the initial states and receives the final ones; y io16 [N,H,D]; boundary fp32
 *     [Cn,H,D,D] (state at the start of every chunk, may be NULL); state_dot_a fp32 [N,H,D] (may be NULL);
 *     dense_checkpoints fp32 [B,H,dense_groups,D,D] or NULL: the state after every 16 tokens of each sequence
 *     (dense_groups = tokens per sequence / 16), the `s` tensor of the reference's dense pretraining operator.
 *   backward: gradients of r, decay logits (raw), k, v, a, b (io16 [N,H,D], each may be NULL) and of the initial
 *     state (fp32 [B,H,D,D], may be NULL) from the forward's final_state, boundary and state_dot_a; grad_output
 *     io16 [N,H,D] (NULL = zero), grad_final_state fp32 [B,H,D,D] (NULL = zero); workspace of
 *     frwkv_wkv7_train_wide_workspace_floats(...) floats (16-token checkpoints and per-column-block partial sums).
 *   metadata_status (may be NULL): the word of frwkv_validate_chunk_tables; when it is non-zero the kernels return
 *     without reading or writing anything (outputs stay as they were: the caller poisons them).
 * Replace forward_kernel_split64 / backward_kernel_split64 / the tiled D = 256 backward
 * (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:110-150,293-478) and the D = 128 / 256 instantiations of
 * the StateTune kernels (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:317-502).
 */
int frwkv_wkv7_train_wide_forward(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                  const int32_t* chunk_ends, float* state, const void* r, const void* decay_logits,
                                  const void* k, const void* v, const void* a, const void* b, void* y, float* boundary,
                                  float* state_dot_a, float* dense_checkpoints, int dense_groups,
                                  const int32_t* metadata_status, int num_sequences, int num_heads, int head_size,
                                  int io_dtype, float scale, frwkv_stream_t stream);
size_t frwkv_wkv7_train_wide_workspace_floats(long long total_tokens, int num_chunks, int num_heads, int head_size);
int frwkv_wkv7_train_wide_backward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends, const float* final_state,
    const float* boundary, const float* state_dot_a, const void* r, const void* decay_logits, const void* k,
    const void* v, const void* a, const void* b, const void* grad_output, const float* grad_final_state, void* grad_r,
    void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b, float* grad_initial_state,
    float* workspace, const int32_t* metadata_status, long long total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream);

/*
 * TMix token shift: out[j] = x + (prev - x) * mix_j for the six mix vectors (r, w, k, v, a, g); prev is the previous
 * packed row, or shift_state_pool[state_indices[s]] at the first row of sequence s; afterwards that slot holds the
 * sequence's last row.  Replaces tmix_mix6_forward_varlen_cuda (csrc/sm120/tmix/mix6/infer_fp16_forward_varlen.cu:190-303).
 *   x io16 [rows, C]; shift_state_pool io16 [slots, C]; x_r..x_g io16 [C]; out io16 [6, rows, C]; C % 8 == 0.
 *   max_seqlen: longest sequence if known (1 lets the kernel skip the separate slot-update launch), else <= 0.
 */
int frwkv_tmix_mix6_forward_varlen(const void* x, void* shift_state_pool, const void* x_r, const void* x_w,
                                   const void* x_k, const void* x_v, const void* x_a, const void* x_g,
                                   const int32_t* cu_seqlens, const int32_t* state_indices,
                                   const int32_t* metadata_status, void* out, int total_rows, int num_sequences,
                                   int channels, int max_seqlen, int io_dtype, frwkv_stream_t stream);

/* (k', -kk, kk*a) with kk = normalize_head(k * k_k), a = sigmoid(a0 + a12), k' = k * (1 + (a - 1) * k_a).
 * Replaces tmix_kk_a_gate_forward_varlen_cuda (csrc/sm120/tmix/kk_a_gate/infer_fp16_forward_varlen.cu:116-210).
 * k, a12, outputs io16 [rows, C]; k_k, a0, k_a io16 [C]; head_size must be 64. */
int frwkv_tmix_kk_a_gate_forward_varlen(const void* k, const void* k_k, const void* a0, const void* a12,
                                        const void* k_a, void* new_k, void* neg_kk, void* kka, long long total_rows,
                                        int channels, int head_size, int io_dtype, frwkv_stream_t stream);

/* (GroupNorm per head of x (biased variance, eps) * weight + bias + (sum_d r k r_k) * v) * g.
 * Replaces tmix_lnx_rkvres_xg_forward_varlen_cuda (csrc/sm120/tmix/lnx_rkvres_xg/infer_fp16_forward_varlen.cu:133-244). */
int frwkv_tmix_lnx_rkvres_xg_forward_varlen(const void* x, const void* r, const void* k, const void* v, const void* r_k,
                                            const void* weight, const void* bias, const void* g, void* out,
                                            long long total_rows, int channels, int head_size, float eps, int io_dtype,
                                            frwkv_stream_t stream);

/* v + (v_first - v) * sigmoid(v0 + v12).  Replaces tmix_vres_gate_forward_varlen_cuda
 * (csrc/sm120/tmix/vres_gate/infer_fp16_forward_varlen.cu:47-93). */
int frwkv_tmix_vres_gate_forward_varlen(const void* v, const void* v_first, const void* v0, const void* v12, void* out,
                                        long long total_rows, int channels, int io_dtype, frwkv_stream_t stream);

/*
 * Add + LayerNorm over rows of `channels` 16-bit values (fp32 statistics, biased variance, of the ROUNDED sum):
 *   sum_out = x + residual ;  norm_out = (sum - mean) * rsqrt(var + eps) * weight + bias
 *   residual == NULL : LayerNorm of x                       (tmix_layer_norm_forward_varlen)
 *   weight == bias == NULL : plain add into sum_out         (tmix_add_forward_varlen)
 *   sum_out == NULL : only the normalised rows              (tmix_add_last_layer_norm_forward_varlen)
 *   all given : both outputs                                (tmix_add_layer_norm_forward_varlen)
 * Replaces the normalization family of the reference (flashrwkv2/tmix/normalization/__init__.py:31-90).
 */
int frwkv_tmix_add_layer_norm_forward(const void* x, const void* residual, const void* weight, const void* bias,
                                      void* sum_out, void* norm_out, long long rows, int channels, float eps,
                                      int io_dtype, frwkv_stream_t stream);

/*
 * The same followed by the six-way token shift, for batches of one-token sequences (row i is sequence i):
 *   sum_out = x + residual ; n = LayerNorm(sum) rounded ; mix_out[j] = n + (shift[slot_i] - n) * x_j ; shift[slot_i] = n
 * mix_out is [6][rows][channels].  When *metadata_status != 0 the outputs are NaN and the shift states untouched.
 * Replaces tmix_mix6_add_layer_norm_forward_varlen (flashrwkv2/tmix/mix6/__init__.py:103-199), which the reference
 * restricts to one row of 4096 channels.
 */
int frwkv_tmix_mix6_add_layer_norm_forward(const void* x, const void* residual, const void* weight, const void* bias,
                                           const void* x_r, const void* x_w, const void* x_k, const void* x_v,
                                           const void* x_a, const void* x_g, void* shift_state_pool,
                                           const int32_t* state_indices, const int32_t* metadata_status, void* sum_out,
                                           void* mix_out, int rows, int channels, float eps, int io_dtype,
                                           frwkv_stream_t stream);

/*
 * Token shift fused into up to eight projections of the same rows (decode, 1..8 rows):
 *   y_j[m][n] = sum_c (x[m][c] + (prev[m][c] - x[m][c]) * mix_j[c]) * weight_j[n][c]
 * with prev the previous row of the same sequence or, for its first row, shift_state_pool[state_indices[s]]; afterwards
 * the last row of every sequence is stored in its shift-state slot.  One launch does what tmix_mix6_forward_varlen
 * (csrc/sm120/tmix/mix6/infer_fp16_forward_varlen.cu:75-303) followed by tmix_lowrank_wagv_in_forward_varlen and
 * three tmix_linear_forward_varlen calls (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:2229-2521,2685-2952) do
 * in the reference; the interpolated rows stay in fp32 instead of being rounded to 16 bits in between.  There is no
 * single reference entry point with this signature.  `projections` is a host array.  When *metadata_status != 0 the
 * outputs are NaN and the shift states untouched.
 */
typedef struct {
  const void* mix;     /* io16 [channels] */
  const void* weight;  /* io16 [n][channels] */
  void* y;             /* io16 [total_rows][n] */
  int n;               /* multiple of 8 */
} frwkv_shift_projection;
int frwkv_tmix_shift_project_varlen(const void* x, void* shift_state_pool, const int32_t* cu_seqlens,
                                    const int32_t* state_indices, const int32_t* metadata_status,
                                    const frwkv_shift_projection* projections, int count, int total_rows,
                                    int num_sequences, int channels, int io_dtype, frwkv_stream_t stream);

/*
 * The same operator for more than 8 rows: the token shift happens inside the tensor-core GEMM.  Per pipeline stage TMA
 * brings the x tile and the tile of the rows before it (the same tensor map, one row up); four warps turn the x tile
 * into x + (prev - x) * mix in shared memory (for a sequence's first row prev comes from its shift state) before the
 * tcgen05 products read it.  Projections go out four per launch; afterwards every sequence's last row becomes its shift
 * state.  row_workspace: int32 [total_rows].  error_flag (may be NULL) is set if a bounded wait ran out.  Replaces
 * tmix_mix6_forward_varlen followed by the projections' GEMMs
 * (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:3058-3099 of the reference).
 */
int frwkv_tmix_shift_project_gemm(const void* x, void* shift_state_pool, const int32_t* cu_seqlens,
                                  const int32_t* state_indices, const int32_t* metadata_status,
                                  const frwkv_shift_projection* projections, int count, int total_rows,
                                  int num_sequences, int channels, int io_dtype, int32_t* row_workspace,
                                  int32_t* error_flag, frwkv_stream_t stream);

/* Elementwise tanh (act = 1) or sigmoid (act = 2) of a 16-bit tensor with `elements` (multiple of 8) values.
 * Replaces linear_act_tanh / linear_act_sigmoid (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:1235-1373). */
int frwkv_tmix_act_forward(const void* x, void* out, long long elements, int act, int io_dtype, frwkv_stream_t stream);

/*
 * Grouped TMix projections: for each of 1..4 problems, y[m][n] = act(x)[m][k] * weight[n][k]^T, optionally followed by
 * the value-residual epilogue  y = v + (v_first - v) * sigmoid(v0 + y).  All problems share the row count m.
 * Replaces tmix_lowrank_{in,wagv_in,out,vres}_forward_varlen, tmix_linear_forward_varlen and the rank_in/rank_out/
 * linear_t family (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:2229-3100).  m <= 8 runs the bandwidth-bound
 * small-row kernel, larger m the tcgen05 GEMM.  `problems` is a host array.  n and k must be multiples of 8.
 */
typedef struct {
  const void* x;       /* io16 [m][k] */
  const void* weight;  /* io16 [n][k]  (the reference's original layout) */
  void* y;             /* io16 [m][n] */
  int n, k;
  int act;             /* applied to x: 0 none, 1 tanh, 2 sigmoid */
  int epilogue;        /* 0 none, 1 value residual */
  const void* v;       /* epilogue 1: io16 [m][n] */
  const void* v_first; /* epilogue 1: io16 [m][n] */
  const void* v0;      /* epilogue 1: io16 [n] */
} frwkv_linear_problem;
int frwkv_tmix_linear_grouped(const frwkv_linear_problem* problems, int count, int m, int io_dtype,
                              int32_t* error_flag, frwkv_stream_t stream);
/* One projection whose `weight` is in the reference's RUNTIME layout [k][n] (weight_is_transposed=True, the `w1` /
 * `w2` arguments of the low-rank operators: flashrwkv2/tmix/linear/__init__.py:25-56,279-320 and
 * csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cpp:289-308), read in place.  With m > 8 `act` must be 0. */
int frwkv_tmix_linear_runtime_layout(const frwkv_linear_problem* problem, int m, int io_dtype, int32_t* error_flag,
                                     frwkv_stream_t stream);

/*
 * One RWKV-7 TMix layer for a decode batch (one token per sequence; rows = sequences <= 8; head size 64) as one
 * persistent, cooperatively launched kernel: token shift, r / k / v and the four rank-in projections, rank-out
 * projections with the value-residual gate, kk_a_gate, the WKV7 step on state_pool, lnx_rkvres_xg and the output
 * projection, separated by grid-wide barriers (bounded waits; on a time-out error_flag is set and out is NaN).
 * Row m belongs to sequence m: its shift state is shift_state_pool[state_indices[m]] (updated to x[m]) and its WKV7
 * state state_pool[state_indices[m]] (fp32 [slots,H,64,64], updated in place).  mix = x_r, x_w, x_k, x_v, x_a, x_g;
 * w1 / w2 / rank = decay, a, gate, value-residual low-rank pairs ([R,C] and [C,R]); all weights in the original
 * layout.  workspace: frwkv_tmix_decode_layer_workspace_bytes bytes for the 16-bit intermediates; barrier: four
 * 32-bit words that are zero before the first launch (the kernel leaves them zero; launches that may overlap on
 * the GPU need words of their own).  metadata_status may be NULL.
 * No single counterpart in the reference: equals the operator sequence of csrc/sm120/tmix/{mix6,linear,kk_a_gate,
 * wkv7,lnx_rkvres_xg} up to summation order.
 */
typedef struct {
  const void* x;
  const void* v_first;
  void* shift_state_pool;
  float* state_pool;
  const void* mix[6];
  const void* w_r;
  const void* w_k;
  const void* w_v;
  const void* w_o;
  const void* w1[4];
  const void* w2[4];
  int rank[4];
  const void* k_k;
  const void* a0;
  const void* k_a;
  const void* r_k;
  const void* ln_w;
  const void* ln_b;
  const void* v0;
  void* out;
  void* workspace;
  uint32_t* barrier;
} frwkv_tmix_decode_layer_args;
size_t frwkv_tmix_decode_layer_workspace_bytes(int rows, int channels, const int* rank);
int frwkv_tmix_decode_layer_forward(const frwkv_tmix_decode_layer_args* args, const int32_t* state_indices,
                                    const int32_t* metadata_status, int rows, int channels, int num_heads, float ln_eps,
                                    int io_dtype, int32_t* error_flag, frwkv_stream_t stream);

/* out = x + vec; x, out io16 [total_rows][channels], vec io16 [channels], channels even.  Replaces
 * recurrent_add_vec_forward_varlen_cuda (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:1247-1290). */
int frwkv_recurrent_add_vec_forward(const void* x, const void* vec, void* out, long long total_rows, int channels,
                                    int io_dtype, frwkv_stream_t stream);

/*
 * ---- Training-side TMix glue on dense [B, T, C] tensors (rows = B * T), forward and backward ----------------------
 * io16 tensors are bf16 in the reference (io_dtype FRWKV_DTYPE_BF16); fp16 is accepted too.  channels must be a
 * multiple of 8.  A backward that also returns the gradient of a [C] parameter sums it over the rows in two steps
 * (per-slab fp32 partials in `workspace`, then a fixed-order sum), so the result is the same on every run;
 * `workspace` holds at least frwkv_pretrain_workspace_floats(rows, channels, vectors) floats, `vectors` = the
 * number of parameter gradients of that call (a_gate 1, vres_gate 1, mix6 6, kk_pre 2, lnx_rkvres_xg 3).
 */
long long frwkv_pretrain_workspace_floats(long long rows, int channels, int vectors);

/* out = sigmoid(a0 + a12); a0 [C], a12 [rows][C].  Replaces tmix_a_gate forward / backward
 * (csrc/sm90/tmix/a_gate/pretrain_bf16_forward.cu, pretrain_bf16_backward.cu). */
int frwkv_pretrain_a_gate_forward(const void* a0, const void* a12, void* out, long long rows, int channels,
                                  int io_dtype, frwkv_stream_t stream);
int frwkv_pretrain_a_gate_backward(const void* grad_out, const void* a0, const void* a12, void* grad_a0,
                                   void* grad_a12, float* workspace, long long workspace_floats, long long rows,
                                   int channels, int io_dtype, frwkv_stream_t stream);

/* Backward of v + (v_first - v) * sigmoid(v0 + v12); the forward is frwkv_tmix_vres_gate_forward_varlen with
 * total_rows = rows.  Replaces csrc/sm90/tmix/vres_gate/pretrain_bf16_backward.cu. */
int frwkv_pretrain_vres_gate_backward(const void* grad_out, const void* v, const void* v_first, const void* v0,
                                      const void* v12, void* grad_v, void* grad_v_first, void* grad_v0,
                                      void* grad_v12, float* workspace, long long workspace_floats, long long rows,
                                      int channels, int io_dtype, frwkv_stream_t stream);

/* out[j] = x + (x[t-1] - x) * mix[j], j = r, w, k, v, a, g; x [batch][seq_len][C], x[-1] = 0; mix, out, grad_out and
 * grad_mix are arrays of six pointers.  Replaces csrc/sm90/tmix/mix6/pretrain_bf16_{forward,backward}.cu. */
int frwkv_pretrain_mix6_forward(const void* x, const void* const* mix, void* const* out, long long batch, int seq_len,
                                int channels, int io_dtype, frwkv_stream_t stream);
int frwkv_pretrain_mix6_backward(const void* const* grad_out, const void* x, const void* const* mix, void* grad_x,
                                 void* const* grad_mix, float* workspace, long long workspace_floats, long long batch,
                                 int seq_len, int channels, int io_dtype, frwkv_stream_t stream);

/* StateTune form of mix6: the row before t = 0 is initial_shift[b] ([batch][C]) and the last row of every sequence
 * is also returned as final_shift[b]; the backward takes the gradient of final_shift and returns that of
 * initial_shift.  Replaces statetune_tmix_mix6_forward / backward (flashrwkv2/tmix/mix6/__init__.py:244-262). */
int frwkv_statetune_mix6_forward(const void* x, const void* initial_shift, const void* const* mix, void* const* out,
                                 void* final_shift, long long batch, int seq_len, int channels, int io_dtype,
                                 frwkv_stream_t stream);
int frwkv_statetune_mix6_backward(const void* const* grad_out, const void* grad_final_shift, const void* x,
                                  const void* initial_shift, const void* const* mix, void* grad_x,
                                  void* grad_initial_shift, void* const* grad_mix, float* workspace,
                                  long long workspace_floats, long long batch, int seq_len, int channels, int io_dtype,
                                  frwkv_stream_t stream);

/* kk = normalize(k * k_k) per head (eps 1e-12); new_k = k * (1 + (a - 1) * k_a), neg_kk = -kk, kka = kk * a;
 * inv_norm fp32 [rows][C / head_size] is saved for the backward.  head_size 64, 128 or 256.
 * Replaces csrc/sm90/tmix/kk_pre/pretrain_bf16_{forward,backward}.cu. */
int frwkv_pretrain_kk_pre_forward(const void* k, const void* k_k, const void* a, const void* k_a, void* new_k,
                                  void* neg_kk, void* kka, float* inv_norm, long long rows, int channels,
                                  int head_size, int io_dtype, frwkv_stream_t stream);
int frwkv_pretrain_kk_pre_backward(const void* grad_new_k, const void* grad_neg_kk, const void* grad_kka,
                                   const void* k, const void* k_k, const void* a, const void* k_a,
                                   const float* inv_norm, void* grad_k, void* grad_k_k, void* grad_a, void* grad_k_a,
                                   float* workspace, long long workspace_floats, long long rows, int channels,
                                   int head_size, int io_dtype, frwkv_stream_t stream);

/* out = (LayerNorm per head of x (biased variance, eps 64e-5) * weight + bias + (sum_head r k r_k) * v) * g; mean and
 * rstd fp32 [rows][C / head_size] are saved for the backward.
 * Replaces csrc/sm90/tmix/lnx_rkvres_xg/pretrain_bf16_{forward,backward}.cu. */
int frwkv_pretrain_lnx_rkvres_xg_forward(const void* x, const void* r, const void* k, const void* v, const void* r_k,
                                         const void* weight, const void* bias, const void* g, void* out, float* mean,
                                         float* rstd, long long rows, int channels, int head_size, int io_dtype,
                                         frwkv_stream_t stream);
int frwkv_pretrain_lnx_rkvres_xg_backward(const void* grad_out, const void* x, const void* r, const void* k,
                                          const void* v, const void* r_k, const void* weight, const void* bias,
                                          const void* g, const float* mean, const float* rstd, void* grad_x,
                                          void* grad_r, void* grad_k, void* grad_v, void* grad_r_k, void* grad_weight,
                                          void* grad_bias, void* grad_g, float* workspace, long long workspace_floats,
                                          long long rows, int channels, int head_size, int io_dtype,
                                          frwkv_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FRWKV_B200_H_ */
