/*
 * megaqwen_b200 — C ABI of the sm_100a Qwen3-0.6B greedy prefill + decode path.
 *
 * This is the boundary a non-Python caller links against.  It replaces the
 * reference's `extern "C" launch_*` functions (csrc/megakernel/
 * fused_decode_ldg_launch.inl, fused_prefill_launch.inl) and keeps their
 * conventions: the caller owns every buffer (weights, KV cache, scratch, token
 * and position scalars are device pointers), token in/out and the position are
 * DEVICE scalars so that steps can be chained without a host round trip and
 * captured in a CUDA graph, and every call is asynchronous on the given
 * stream.  Unlike the reference (which returns void and drops errors) every
 * entry point returns an int: 0 on success, a negative MQ_ERR_* code for a
 * rejected argument, or a positive cudaError_t value.  Device-side waits are
 * bounded; one that expires sets a bit in the caller's `status` word instead
 * of hanging.
 *
 * Plain C types only: no torch, no C++ in the signatures.
 */
#ifndef MEGAQWEN_B200_H
#define MEGAQWEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Fixed block geometry the kernels are compiled for
 * (reference: csrc/megakernel/config.cuh:64-73). */
#define MQ_HIDDEN 1024
#define MQ_INTERMEDIATE 3072
#define MQ_NUM_Q_HEADS 16
#define MQ_NUM_KV_HEADS 8
#define MQ_HEAD_DIM 128
#define MQ_Q_SIZE 2048
#define MQ_KV_SIZE 1024

#define MQ_OK 0
#define MQ_ERR_BAD_ARG (-1)       /* null pointer, non-positive size */
#define MQ_ERR_TOO_LONG (-2)      /* sequence / position exceeds max_seq_len or scratch capacity */
#define MQ_ERR_UNSUPPORTED (-3)   /* device is not sm_100, or geometry not supported */
#define MQ_ERR_ALIGNMENT (-4)     /* a pointer is not 16-byte aligned */

/* Bits of the device status word (MqDecodeBuffers.status). */
#define MQ_STATUS_WAIT_TIMEOUT 1u /* a bounded shared-memory barrier wait expired */
#define MQ_STATUS_BAD_POSITION 2u /* position >= max_seq_len seen on the device; the step was skipped */
#define MQ_STATUS_BAD_TOKEN 4u    /* token id outside [0, vocab) seen on the device; clamped */

/* Launch flags. */
#define MQ_FLAG_CHAINED 1   /* this step directly follows another decode step of the same
                               buffers on the same stream (lets its first kernel overlap
                               the previous step's LM head) */
#define MQ_FLAG_NO_PDL 2    /* launch every kernel with full stream serialisation
                               (no programmatic dependent launch); for A/B measurements */

/* Per-layer weight table, bf16 row-major [out, in] exactly as HF nn.Linear.weight.
 * Same member order as the reference's LDGLayerWeights
 * (csrc/megakernel/fused_decode_ldg_common.inl:97-109, bindings_decode.cpp:32-44). */
typedef struct MqLayerWeights {
    const void* input_layernorm;     /* [1024]        */
    const void* q_proj;              /* [2048, 1024]  */
    const void* k_proj;              /* [1024, 1024]  */
    const void* v_proj;              /* [1024, 1024]  */
    const void* q_norm;              /* [128]         */
    const void* k_norm;              /* [128]         */
    const void* o_proj;              /* [1024, 2048]  */
    const void* post_attn_layernorm; /* [1024]        */
    const void* gate_proj;           /* [3072, 1024]  */
    const void* up_proj;             /* [3072, 1024]  */
    const void* down_proj;           /* [1024, 3072]  */
} MqLayerWeights;

/* Model description.  `layers` is a HOST array of num_layers entries holding
 * device pointers (the reference passes a host table to launch_prefill_float,
 * bindings_prefill.cpp:798, and a device table to launch_ldg_decode). */
typedef struct MqModel {
    const void* embed;        /* [vocab, 1024] bf16 */
    const MqLayerWeights* layers;
    const void* final_norm;   /* [1024] bf16 */
    const void* lm_head;      /* [vocab, 1024] bf16 (tied: same pointer as embed) */
    const void* cos_table;    /* [max_seq_len, 128] bf16 */
    const void* sin_table;    /* [max_seq_len, 128] bf16 */
    int num_layers;
    int vocab_size;
    int max_seq_len;
} MqModel;

/* Caller-owned state and scratch of one batch-1 decoder.  KV cache layout is
 * the reference's: [num_layers, 8, max_seq_len, 128] bf16, K stored after
 * QK-norm and RoPE, V raw (bindings_decode.cpp:127-130). */
typedef struct MqDecodeBuffers {
    void* k_cache;
    void* v_cache;
    void* hidden;             /* bf16 [1024]  residual stream                     */
    void* qkv;                /* bf16 [4096]  raw q|k|v of the current layer      */
    void* attn_out;           /* bf16 [2048]                                      */
    void* mlp_act;            /* bf16 [3072]  silu(gate)*up                       */
    float* attn_partials;     /* fp32 [16 * nsplit * 130] split-KV partials       */
    unsigned int* counters;   /* u32 [16], zero-initialised by the caller once    */
    unsigned long long* argmax_slot; /* u64 [1], zero-initialised by the caller once */
    unsigned int* status;     /* u32 [1], sticky MQ_STATUS_* bits                 */
    int attn_nsplit;          /* from mq_decode_attn_nsplit(max_seq_len)          */
} MqDecodeBuffers;

/* Number of KV splits the decode attention kernel uses for a cache of
 * max_seq_len positions; sizes MqDecodeBuffers.attn_partials. */
int mq_decode_attn_nsplit(int max_seq_len);

/* Bytes of MqDecodeBuffers.attn_partials for a given max_seq_len. */
size_t mq_decode_partials_bytes(int max_seq_len);

/* Number of kernels one mq_launch_decode call launches (for launch counting). */
int mq_decode_launch_count(int num_layers);

/* One greedy decode step: reads *in_token and *position (device), writes K/V of
 * that position, attends over position+1 entries and writes the arg-max token
 * (lowest index among equal bf16 logits) to *out_token.  If logits != NULL the
 * bf16-rounded logits are also written there as fp32 [vocab].
 * Replaces launch_ldg_decode / launch_ldg_decode_with_logits
 * (csrc/megakernel/fused_decode_ldg_launch.inl:55-212, 215-364). */
int mq_launch_decode(const MqModel* model, const MqDecodeBuffers* buf,
                     const int* in_token, int* out_token, const int* position,
                     float* logits, int flags, void* stream);

/* ---- FP8 (e4m3) shadow KV cache, opt-in (reference: MEGAQWEN_SPLIT_KV_FP8,
 * csrc/megakernel/bindings_prefill.cpp:513, 1371-1400; kernels split_decode_gemm.cu:74-78,
 * 223-300, 429-493, 950-1310).  The bf16 caches stay authoritative and are still written by
 * every step; the attention kernels read K and V from the shadow cache instead: half the
 * bytes per cached position.  One scale per (layer, kv head): x ~ e4m3 * scale.
 *   k_fp8 / v_fp8     u8  [num_layers, 8, max_seq_len, 128]  (batched: one such block per sequence)
 *   k_scale / v_scale f32 [num_layers, 8]                    (batched: [batch, num_layers, 8]);
 *                     a stored scale below 1e-8 reads as 1, so zero-filled scales are valid
 *                     before the first mq_launch_kv_quantize_fp8. */
typedef struct MqKvFp8 {
    void* k_fp8;
    void* v_fp8;
    float* k_scale;
    float* v_scale;
} MqKvFp8;

/* Quantises positions [start_pos, end_pos) of ONE sequence's bf16 caches into its shadow
 * caches and SETS the scales from that span: scale = max|x| / 448 (1 if the span is all zero),
 * value = e4m3_rn_satfinite(x / scale).  k_cache / v_cache: bf16 [num_layers, 8, max_seq_len,
 * 128].  An empty span is a no-op.  Replaces launch_split_quantize_kv_cache_fp8
 * (split_decode_gemm.cu:302-345); rows appended later by decode steps are quantised with the
 * scales found here (split_decode_gemm.cu:487-493). */
int mq_launch_kv_quantize_fp8(const void* k_cache, const void* v_cache, const MqKvFp8* kv8, int num_layers,
                              int max_seq_len, int start_pos, int end_pos, void* stream);

/* mq_launch_decode with the attention reading the shadow cache (the step also quantises its
 * own new K/V row into it). */
int mq_launch_decode_kv8(const MqModel* model, const MqDecodeBuffers* buf, const MqKvFp8* kv8,
                         const int* in_token, int* out_token, const int* position,
                         float* logits, int flags, void* stream);

/* ---- Persistent decode: n_steps greedy steps in ONE cooperative launch (one CTA per SM).
 * The device-resident equivalent of the reference's cooperative megakernel and of its
 * decode_steps_cuda / decode_greedy_cuda chains (csrc/megakernel/fused_decode_ldg_kernel.inl:
 * 43-258, bindings_prefill.cpp:1045-1349), which launch one cooperative kernel plus two LM-head
 * kernels per token.  The weights are first repacked ONCE into per-CTA byte streams in
 * consumption order (the reference repacks q|k|v and gate|up for its split backend in the same
 * spirit, bindings_prefill.cpp:604-621); the HF-layout tensors remain the ones the constructor
 * takes and the prefill reads.
 *
 *   mq_stream_packed_bytes   bytes of the packed copy for this model on the current device
 *                            (0 if the device is unsupported)
 *   mq_stream_pack           fills `packed` (256-byte aligned, device memory) from the model
 *   mq_stream_scratch_bytes  bytes of `scratch`: 256-byte aligned, zeroed ONCE by the caller
 *                            and never touched afterwards (it carries a phase counter from
 *                            launch to launch)
 *   mq_stream_max_context    largest position0 + n_steps a launch accepts (2304 on 148 SMs);
 *                            longer contexts go through mq_launch_decode
 *   mq_stream_grid           CTAs per launch (= SMs); mq_stream_stage_count stage slots each
 *
 * mq_launch_decode_stream: step i consumes forced_tokens[i] if forced_tokens != NULL, else the
 * token produced by step i-1 (step 0: *first_token), at position *position0 + i, and writes
 * its arg-max token to tokens_out[i].  logits: optional fp32, [n_steps][vocab] if logits_all
 * else [vocab] of the last step (bf16-rounded values).  stage_cycles: optional device array
 * u64 [grid][num_layers + 1][stages] to which thread 0 of every CTA ADDS the SM cycles it spent
 * per layer in: 0 wait for the hidden vector, 1 RMSNorm + q|k|v rows, 2 wait for q|k|v,
 * 3 attention, 4 split merge, 5 wait for the attention output, 6 Wo rows, 7 wait for the
 * post-attention hidden vector, 8 RMSNorm + gate/up rows, 9 wait for the MLP activation,
 * 10 Wd rows; in row [num_layers]: 11 wait for the last hidden vector, 12 LM head, 13 wait for
 * the arg-max keys; slots 14 and 15 are unused (the counterpart of the reference's per-stage
 * clock64 counters, fused_decode_ldg_common.inl:24-69).
 * Results agree with n_steps calls of mq_launch_decode up to fp32 summation order. */
size_t mq_stream_packed_bytes(const MqModel* model);
int mq_stream_pack(const MqModel* model, void* packed, size_t packed_bytes, void* stream);
size_t mq_stream_scratch_bytes(void);
int mq_stream_max_context(void);
int mq_stream_grid(void);
int mq_stream_stage_count(void);
int mq_launch_decode_stream(const MqModel* model, const void* packed, void* k_cache, void* v_cache,
                            void* scratch, unsigned int* status, const int* first_token,
                            const int* position0, const int* forced_tokens, int* tokens_out,
                            int n_steps, float* logits, int logits_all,
                            unsigned long long* stage_cycles, void* stream);

/* The same decode step for callers that must not allocate device memory.
 * It has no counterpart in the reference.  Who needs it: a host process that
 * receives one fixed arena at start-up and may never call cudaMalloc again
 * (plug-ins of a serving runtime, real-time loops where cudaMalloc's implicit
 * device-wide synchronisation is not acceptable, processes whose pool belongs
 * to another component).  Such a caller passes only inputs and outputs - the
 * model, its KV cache (state, read and written), the token / position scalars,
 * the optional logits and the status word, all device pointers it already
 * owns.  The step's scratch (residual stream, q|k|v, attention output, MLP
 * activation, split-KV partials, tickets, arg-max slot) lives in a static
 * device array of MQ_NOALLOC_SCRATCH_BYTES inside the library; every GPU that
 * loads the library holds it until the process exits.
 *
 * - model->max_seq_len must not exceed MQ_NOALLOC_MAX_SEQ_LEN, else
 *   MQ_ERR_TOO_LONG is returned and nothing is launched.
 * - The call allocates nothing: no cudaMalloc / cudaFree and no allocating
 *   library routine.  Its first call on each device resolves the array's
 *   device address (cudaGetSymbolAddress); make that first call, and
 *   mq_init_device(), before any stream capture.
 * - All calls on a device share the one array, which keeps the previous call's
 *   contents; the entry point clears the words that must start at zero on the
 *   given stream.  Two calls that overlap on the GPU (different streams, or two
 *   decoders driven concurrently) race on it: serialise them.
 * - MQ_FLAG_CHAINED is ignored (each step is fully stream-ordered after the
 *   previous one).  Results are identical to mq_launch_decode. */
#define MQ_NOALLOC_MAX_SEQ_LEN 8192
#define MQ_NOALLOC_SCRATCH_BYTES (576 * 1024)
int mq_launch_decode_noalloc(const MqModel* model, void* k_cache, void* v_cache,
                             const int* in_token, int* out_token, const int* position,
                             float* logits, unsigned int* status, int flags, void* stream);

/* Caller-owned activation buffers of the prefill path, all bf16, max_tokens rows. */
typedef struct MqPrefillBuffers {
    void* h;      /* [max_tokens, 1024] residual stream                    */
    void* x;      /* [max_tokens, 1024] normalised input of the linears    */
    void* qkv;    /* [max_tokens, 4096] q | k | v                          */
    void* attn;   /* [max_tokens, 2048] attention output                   */
    void* act;    /* [max_tokens, 3072] silu(gate) * up                    */
    int max_tokens;
} MqPrefillBuffers;

/* Full-sequence forward of seq_len tokens (device ids) placed at positions
 * pos0 .. pos0 + seq_len - 1: writes their K/V into dbuf's cache, attends
 * causally over everything cached so far, and writes the arg-max token that
 * follows the last one to *out_token (logits: optional fp32 [vocab] of that
 * row).  bf16 tensors between all ops; the seven linears per layer run on
 * tcgen05 tensor cores.  Replaces launch_prefill_float
 * (csrc/megakernel/fused_prefill_launch.inl:71-731). */
int mq_launch_prefill(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pbuf,
                      const int* ids, int seq_len, int pos0, int* out_token, float* logits, void* stream);

/* The same forward with rows audio_start .. audio_start + audio_len - 1 of the embedded prompt
 * replaced by externally computed embeddings audio_embeds [audio_len, 1024] bf16 (device,
 * 16-byte aligned) before the first layer: the hook the reference's speech front-end uses
 * (prefill_asr, csrc/megakernel/bindings_prefill.cpp:835-955; patch kernel
 * fused_prefill_kernels.inl:28-45).  The token ids of the replaced rows are ignored. */
int mq_launch_prefill_asr(const MqModel* model, const MqDecodeBuffers* dbuf, const MqPrefillBuffers* pbuf,
                          const int* ids, int seq_len, int pos0, const void* audio_embeds, int audio_start,
                          int audio_len, int* out_token, float* logits, void* stream);

/* State and scratch of a batch of independent sequences (no counterpart in the
 * reference, which is batch-1 only).  Sequence b owns the cache slice
 * [b][num_layers, 8, max_seq_len, 128]; a prefill of sequence b is an
 * mq_launch_prefill call whose MqDecodeBuffers point at that slice. */
typedef struct MqBatchBuffers {
    void* k_cache;            /* bf16 [batch, num_layers, 8, max_seq_len, 128] */
    void* v_cache;
    int* positions;           /* device int32 [batch]: tokens consumed per sequence */
    void* logits;             /* bf16 [batch, vocab] scratch                    */
    MqPrefillBuffers act;     /* activation buffers, max_tokens >= batch        */
    unsigned int* status;
    int batch;
    float* partials;          /* optional fp32 scratch of the split-K path (batch <= 64):        */
    size_t partials_bytes;    /* at least 4 * batch * 6144 * 4 bytes; NULL = 128-row tile GEMMs  */
    float* attn_parts;        /* optional fp32 scratch that lets several CTAs share the keys of  */
    size_t attn_parts_bytes;  /* one (sequence, kv head): at least batch * 8 * 4 * 2 * 130 * 4   */
    unsigned int* attn_tickets; /* bytes, with u32 [batch * 8] counters zeroed ONCE by the caller; */
                              /* NULL = one CTA per (sequence, kv head)                          */
} MqBatchBuffers;

/* One greedy decode step for every sequence of the batch: sequence b consumes
 * in_tokens[b] at position positions[b] (its K/V are written there), attends
 * over its own positions[b] + 1 cached entries and out_tokens[b] receives the
 * arg-max token; positions[b] is incremented on the device, so steps chain
 * without host work.  The linears run as M = batch GEMMs on tcgen05 (weights
 * are read once per step for the whole batch).  logits_f32: optional fp32
 * [batch, vocab].  vocab must be a multiple of 128. */
int mq_launch_decode_batch(const MqModel* model, const MqBatchBuffers* bb, const int* in_tokens,
                           int* out_tokens, float* logits_f32, void* stream);
/* Prefill of several sequences in one pass (no reference counterpart: the reference prefills one
 * sequence at a time).  The prompts are packed row after row: ids[total_rows]; row_seq[r] /
 * row_pos[r] give the sequence (0..bb->batch-1) and position of packed row r; the causal
 * attention runs per 64-row query tile: tile t covers rows tile_q0[t]..+63 of sequence
 * tile_seq[t] (callers list long tiles first); seq_len[b] and seq_row0[b] are the length and
 * the first packed row of sequence b.  All tables are device int32 arrays.  bb->positions[b]
 * must hold seq_len[b] - 1 on entry and holds seq_len[b] afterwards; out_tokens[b] is the
 * token that follows prompt b.  total_rows must not exceed bb->act.max_tokens. */
int mq_launch_prefill_packed(const MqModel* model, const MqBatchBuffers* bb, const int* ids, const int* row_seq,
                             const int* row_pos, const int* tile_seq, const int* tile_q0, const int* seq_len,
                             const int* seq_row0, int total_rows, int num_tiles, int* out_tokens, void* stream);

/* mq_launch_decode_batch with the attention reading the shadow caches (kv8 holds one block and
 * one scale row per sequence, see MqKvFp8). */
int mq_launch_decode_batch_kv8(const MqModel* model, const MqBatchBuffers* bb, const MqKvFp8* kv8,
                               const int* in_tokens, int* out_tokens, float* logits_f32, void* stream);

/* Kernels one step launches on the tile-GEMM path (batch > 64); two fewer per layer on the split-K path. */
int mq_decode_batch_launch_count(int num_layers);

/* Number of kernels one mq_launch_prefill call launches. */
int mq_prefill_launch_count(int num_layers);

/* C[M,N] = A[M,K] * B[N,K]^T (+ R), bf16 row-major, fp32 accumulation, on the
 * tcgen05 path; N a multiple of 128, K a multiple of 64, lda/ldc multiples of
 * 8.  R (optional) has C's shape and leading dimension and may alias C.  The
 * building block of mq_launch_prefill, exposed for unit tests; the reference
 * calls cublasGemmEx here (fused_prefill_launch.inl:290-323). */
int mq_launch_gemm_bf16(const void* A, int lda, const void* B, void* C, const void* R,
                        int M, int N, int K, int ldc, unsigned int* status, void* stream);

/* Test hook for the error path that every bounded device wait shares: the same GEMM (no residual),
 * but the TMA producer never requests k-block drop_kb (0 <= drop_kb < K / 64), so one wait of every
 * CTA runs out after about 0.2 s.  The kernel must then return, set MQ_STATUS_WAIT_TIMEOUT in
 * *status, store nothing to C, drain the copies and MMAs it has in flight, free its tensor memory,
 * and leave the device usable (clear *status before the next call).  No production path uses it. */
int mq_debug_gemm_drop_load(const void* A, int lda, const void* B, void* C, int M, int N, int K, int ldc,
                            unsigned int* status, void* stream, int drop_kb);

/* Standalone bf16 ops with the rounding points of the fused kernels.  They
 * replace the reference's csrc/kernels launchers (declared in
 * csrc/kernels/__init__.py:40-95): launch_rms_norm (rms_norm.cu:60-170),
 * launch_silu_mul (silu_mul.cu:22-111), launch_rope / launch_rope_single
 * (rope.cu:31-188; q/k laid out [seq_len, heads, head_dim], cos/sin
 * [positions, head_dim]) and launch_attention_decode (attention_decode.cu:
 * 110-357; q/out [batch, n_q_heads, head_dim], caches [batch, n_kv_heads,
 * max_seq_len, head_dim]). */
int mq_launch_rms_norm(const void* x, const void* weight, void* out, int n_rows, int n_cols, float eps, void* stream);
int mq_launch_silu_mul(const void* gate, const void* up, void* out, long long n_elements, void* stream);
int mq_launch_rope(const void* q, const void* k, const void* cos, const void* sin, void* q_out, void* k_out,
                   int seq_len, int n_q_heads, int n_kv_heads, int head_dim, void* stream);
int mq_launch_rope_single(const void* x, const void* cos, const void* sin, void* out, int n_heads, int head_dim,
                          int position, void* stream);
int mq_launch_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, int batch_size,
                               int cache_len, int n_q_heads, int n_kv_heads, int head_dim, int max_seq_len,
                               float scale, void* stream);

/* dst[i] = start + i.  Replaces launch_ldg_fill_iota
 * (csrc/megakernel/fused_decode_ldg_launch.inl:5-17). */
int mq_launch_fill_iota(int* dst, int start, int n, void* stream);

/* *out_index = min(*out_index, first i in [0,n) with tokens[i] in eos_ids[0..n_eos)).
 * The caller initialises *out_index (e.g. to n).  Replaces
 * launch_ldg_find_first_eos (csrc/megakernel/fused_decode_ldg_launch.inl:19-53). */
int mq_launch_find_first_eos(const int* tokens, int n, const int* eos_ids, int n_eos,
                             int* out_index, void* stream);

/* Library / device facts: returns 0 and fills the outputs (any may be NULL). */
int mq_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* One-time set-up of the current device (shared-memory opt-in of the kernels).
 * Every launch entry point does this lazily on its first call; call it
 * explicitly before capturing launches into a CUDA graph.  Returns
 * MQ_ERR_UNSUPPORTED on anything but an sm_100 device. */
int mq_init_device(void);

/* ABI version of this header. */
int mq_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MEGAQWEN_B200_H */
