/*
 * qmm_decoder.h — C ABI of the decode engine of libqmm.
 *
 * The engine plays the role examples/gemma4.rs plays in nm-z/nates-recipe-rs (model held in VRAM,
 * every activation buffer allocated once, one projection after another per layer, greedy
 * sampling: examples/gemma4.rs:231-271, 638-742, 758-783, 1021-1057) for a Llama/Gemma-style
 * decoder whose weights are random-init GGUF blocks.  All allocation happens in
 * qmm_decoder_create; qmm_decoder_step only launches kernels on the given stream.
 */
#ifndef QMM_DECODER_H
#define QMM_DECODER_H
#include "qmm.h"
#include "qmm_gguf.h"
#ifdef __cplusplus
extern "C" {
#endif

#define QMM_DECODER_MAX_TP 8
#define QMM_ACT_GELU_TANH 0
#define QMM_ACT_SILU 1

/* tensor ids for qmm_decoder_get_tensor (layer = -1 for the last three) */
#define QMM_T_ATTN_NORM 0
#define QMM_T_WQ 1     /* returned as the fused [Wq ; Wk] block of this rank */
#define QMM_T_WK 2     /* not a separate tensor: use QMM_T_WQ */
#define QMM_T_WV 3
#define QMM_T_WO 4
#define QMM_T_FFN_NORM 5
#define QMM_T_WGATE 6  /* returned as the fused [Wgate ; Wup] block of this rank */
#define QMM_T_WUP 7    /* not a separate tensor: use QMM_T_WGATE */
#define QMM_T_WDOWN 8
#define QMM_T_FINAL_NORM 9
#define QMM_T_HEAD 10
#define QMM_T_EMBED 11

typedef struct {
    int n_layers, hidden, n_q_heads, n_kv_heads, head_dim, ffn, vocab, ctx_len;
    float rope_theta, rms_eps;
    int act;                                  /* QMM_ACT_* */
    int type_attn_qk, type_attn_v, type_attn_o, type_ffn_gate_up, type_ffn_down, type_head; /* QMM_TYPE_* */
    int max_batch;
    int tp_rank, tp_size;                     /* tensor-parallel rank / world (1 = single GPU) */
    unsigned long long seed;
} qmm_decoder_config;

/* Builds the model on the current device: allocates and fills weights (seeded closed-form normal,
 * sigma 0.02, quantized on the device), KV cache (fp16, zeroed) and every activation buffer. */
int qmm_decoder_create(const qmm_decoder_config* cfg, void** handle);
/* The same engine with its weights read from a GGUF file (include/qmm_gguf.h): hyper-parameters from the
 * "<architecture>." metadata keys of the format's naming convention, matrices from blk.<i>.attn_q /
 * attn_k / attn_v / attn_output / ffn_gate / ffn_up / ffn_down .weight, token_embd.weight, output.weight
 * (absent: tied to token_embd) and the f32 norm gains; every rank reads only its shard (row ranges of the
 * column-parallel matrices, whole-block column ranges of O and down).  ctx_len 0 = the file's context
 * length.  One block type per role across the layers.  This is the place where the upstream would plug a
 * quantized dense into its forward (recipe-infer/src/forward.rs:372-384). */
int qmm_decoder_create_from_gguf(const char* path, int max_batch, int ctx_len, int tp_rank, int tp_size, void** handle);
/* Writes the model of a single-GPU decoder as a GGUF file (architecture NULL = "llama"). */
int qmm_decoder_export_gguf(void* handle, const char* path, const char* architecture);
int qmm_decoder_destroy(void* handle);
/* packed weight bytes this rank streams per decoded token (all layers + head) */
long qmm_decoder_weight_bytes(void* handle);
/* device pointer and packed byte size of a tensor (norm weights are f32, matrices packed blocks).  On a
 * tensor-parallel rank the rows of a Q6_K O or down shard may lie further apart on the device than their
 * packed length (padded to 16-byte boundaries for the tensor-core matvec): read such a tensor with
 * qmm_decoder_read_tensor, which packs the rows. */
int qmm_decoder_get_tensor(void* handle, int layer, int which, void** ptr, long* bytes);
/* copies a tensor to host memory (synchronises the device); capacity in bytes */
int qmm_decoder_read_tensor(void* handle, int layer, int which, void* host_dst, long capacity);
/* fills the whole KV cache with seeded N(0,1) values (emulates a full context for benchmarks) */
int qmm_decoder_fill_cache(void* handle, unsigned long long seed, void* stream);

/* Tensor-parallel wiring.  Each rank exports the handle of its exchange area (64 bytes, a
 * cudaIpcMemHandle_t), the host program gathers them, and every rank imports its peers'.
 * Rules for a tensor-parallel host:
 *   - all ranks pass a host-side barrier after qmm_decoder_tp_ready and before the first step, and
 *     enter every step within the wait bound (about two seconds of SM clock) of each other: a rank
 *     that waits longer for a peer gives up, leaves its activations unwritten for that step and
 *     stores -1 in next_tokens;
 *   - after a step (or a batch of steps) call qmm_device_status before trusting next_tokens: a
 *     non-zero status (5 = a peer did not arrive) means the step's results are not valid. */
int qmm_decoder_ipc_export(void* handle, void* out_handle_64_bytes);
int qmm_decoder_ipc_import(void* handle, int peer_rank, const void* handle_64_bytes);
int qmm_decoder_tp_ready(void* handle); /* call once after all imports (uploads the pointer tables) */

/* The prompt path: all n_tokens positions of a prompt through every layer at once, the way the upstream's layer
 * function runs a sequence (examples/gemma4.rs:638-742: every projection one gpu_gemm_bt_f64_into over the t rows,
 * the attention one gpu_gqa_attn_into).  Projections are launch_qdense without bias or activation (the tcgen05
 * GEMM on bf16(x) for Q4_K weights from 64 rows on, the Q8_1 matvec otherwise), the attention launch_attn_prefill
 * (causal), the small operators the decode path's kernels with one row per position.  Fills the KV cache of
 * sequence `seq` for positions 0..n_tokens-1 and writes the greedy token after the last position to next_token[0]
 * (device), its logits to logits_out (device, vocab floats; may be NULL); decoding continues with
 * qmm_decoder_step at pos = n_tokens.  tokens: device pointer.  Its activation buffers are allocated on first use
 * for the longest prompt so far (freed with the decoder).  One GPU only (QMM_ERR_UNSUPPORTED with tp_size > 1).
 * The logits differ from feeding the prompt token by token through qmm_decoder_step by the rounding of the
 * activations (bf16 / f16 here, Q8_1 blocks there). */
int qmm_decoder_prefill(void* handle, const int* tokens, int n_tokens, int seq, int* next_token, float* logits_out, void* stream);
/* The same for tokens that CONTINUE sequence `seq`: tokens[0] is position pos0 and the cache already holds positions
 * 0..pos0-1 (from an earlier prompt call or from decode steps).  A long prompt can be fed in pieces, a conversation
 * extended turn by turn; every query attends to the cached positions and causally to its own piece.  pos0 = 0 is
 * qmm_decoder_prefill.  pos0 + n_tokens <= ctx_len. */
int qmm_decoder_prefill_at(void* handle, const int* tokens, int n_tokens, int seq, int pos0, int* next_token, float* logits_out,
                           void* stream);

/* One decode step: tokens (device, batch ints) at position pos -> next_tokens (device, batch ints,
 * greedy).  logits (optional, device, batch x vocab_local f32) receives this rank's slice of the
 * logits.  With tensor parallelism the ranks exchange their slice's best candidate inside the
 * step, so next_tokens holds the same global token on every rank; best (optional, device, batch
 * f32) receives this rank's own best logit.  batch <= 1024. */
int qmm_decoder_step(void* handle, const int* tokens, int batch, int pos, int* next_tokens, float* logits, float* best, void* stream);

#ifdef __cplusplus
}
#endif
#endif
