/* b200_gguf.h -- C ABI of the B200-native GGUF inference engine (libb200gguf.so).
 *
 * This is the boundary the Python host (`llama_cpp.Llama`, the drop-in for the object that
 * /root/reference/api.py:7,24-28,55-63 drives) sits on, through ctypes. The reference reaches
 * its engine through llama-cpp-python 0.2.77's ctypes binding of libllama (un-vendored
 * upstream, pinned at /root/reference/docker/Dockerfile.base:30); each entry point below names
 * the libllama call(s) of that binding it stands in for. Plain pointers and sizes only; no
 * torch or C++ types cross this line.
 *
 * Conventions: every function returns 0 on success and a negative code on failure;
 * b2_last_error() returns a thread-local message for the most recent failure on the calling
 * thread. Functions may be called from any host thread (each call selects the engine's device);
 * calls on ONE engine must not overlap in time (the Python host serialises them).
 * "host" pointers are ordinary CPU memory, "dev" pointers are CUDA device memory.
 */
#ifndef B200_GGUF_H
#define B200_GGUF_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_ERR_ARG -1
#define B2_ERR_CUDA -2
#define B2_ERR_UNSUPPORTED -3
#define B2_ERR_STATE -4

/* ggml tensor type ids accepted for weights (gguf/constants.py:4059-4094) */
#define B2_TYPE_F32 0
#define B2_TYPE_F16 1
#define B2_TYPE_Q4_0 2
#define B2_TYPE_Q8_0 8
#define B2_TYPE_Q4_K 12
#define B2_TYPE_Q5_K 13
#define B2_TYPE_Q6_K 14
#define B2_TYPE_I32 26    /* integer tables of layer-list models */
#define B2_TYPE_BF16 30   /* dense tensors of layer-list models (safetensors BF16) */

typedef struct b2_engine b2_engine;

typedef struct b2_config {
    int32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab;
    float rms_eps;
    float rope_freq_base;
    int32_t n_ctx;            /* max tokens per sequence (api.py:17,27 passes 1024) */
    int32_t max_seqs;         /* sequence slots that can be live at once */
    int32_t kv_block_tokens;  /* tokens per KV page */
    int32_t kv_num_blocks;    /* pages in the pool shared by all slots */
    int32_t device;           /* CUDA device ordinal */
    int32_t flags;            /* B2_FLAG_* */
} b2_config;

#define B2_FLAG_NO_GRAPH 1      /* launch kernels directly instead of replaying CUDA graphs */
#define B2_FLAG_NO_PDL 2        /* no programmatic dependent launch between kernels */
#define B2_FLAG_ACT8 4          /* single int8 activation plane (faster, ~0.5% noise) */
#define B2_FLAG_F32 8           /* layer-list models: every product in true 32-bit (no tensor cores), f32 cache pages */

typedef struct b2_sampling {
    float temperature;        /* <= 0: greedy */
    float top_p;
    float min_p;
    float repeat_penalty;
    float frequency_penalty;
    float presence_penalty;
    int32_t top_k;            /* 1..1024 */
    int32_t penalty_last_n;   /* <= 64 */
} b2_sampling;

/* ---- library ------------------------------------------------------------------------- */
const char* b2_last_error(void);
int b2_version(void);
int b2_device_count(int* n);

/* ---- engine lifecycle: replaces llama_load_model_from_file + llama_new_context_with_model
 *      behind Llama.__init__ (api.py:24-28) and llama_free / llama_free_model. ------------ */
int b2_engine_create(const b2_config* cfg, b2_engine** out);
int b2_engine_destroy(b2_engine* e);
/* Copy one GGUF tensor's raw blocks, unchanged, into HBM (the upload half of llama.cpp's
 * llama_model_loader::load_all_data). ne0 = contiguous length K, ne1 = rows (1 for vectors). */
int b2_upload_tensor(b2_engine* e, const char* name, int ggml_type, int64_t ne0, int64_t ne1,
                     const void* host_data, int64_t nbytes);
/* Tensor parallelism for models that do not fit (or should not occupy) one GPU: one process per GPU, each creating an
 * engine whose b2_config carries the LOCAL head counts and n_ff (1 / world of the model's) and the FULL n_embd and n_vocab,
 * and uploading its shard of every matrix (llama_cpp/tp_shard.py: whole rows of attn_q/k/v, ffn_gate/up and output, K
 * ranges of attn_output and ffn_down cut at 256-element block boundaries). The engine then all-reduces (sum, NCCL) the
 * hidden vector after attn_output and ffn_down and all-gathers the logits. No counterpart in the reference, which only
 * runs independent replicas (/root/reference/helm/values.yaml:17). b2_tp_unique_id: rank 0 makes the 128-byte NCCL id,
 * the host distributes it; b2_engine_tp_init: collective over all ranks, after b2_engine_create and before
 * b2_engine_finalize. In this mode prompts and multi-slot steps run through the mat-vec path. */
int b2_tp_unique_id(void* host_out_128_bytes);
int b2_engine_tp_init(b2_engine* e, int rank, int world, const void* host_id_128_bytes);
/* All tensors uploaded: validate the set, build the per-layer launch plans. */
int b2_engine_finalize(b2_engine* e);
int b2_engine_device_bytes(b2_engine* e, int64_t* weight_bytes, int64_t* kv_bytes);

/* ---- sequences (paged KV): replaces llama_kv_cache_* bookkeeping (llama.cpp llama_kv_cache).
 *      The page allocator lives in the host (llama_cpp/kv_pages.py); the engine only holds
 *      each slot's page table. -------------------------------------------------------------- */
int b2_seq_set_blocks(b2_engine* e, int slot, const int32_t* host_blocks, int n_blocks);
/* Start (or restart) a slot: n_past tokens are already in its KV pages; `host_history` are the
 * last <= 64 tokens of the sequence so far (for the penalties); `host_uniforms` are n_uniform
 * (<= 8192) doubles in [0,1) for the multinomial draws of this sequence. */
int b2_seq_begin(b2_engine* e, int slot, int n_past, const int32_t* host_history, int n_history,
                 const b2_sampling* sampling, const double* host_uniforms, int n_uniform);

/* ---- forward: replaces llama_decode (llama.cpp llama_decode_internal) + llama_get_logits +
 *      llama_sample_* under Llama.eval / Llama.sample (api.py:55-63). ------------------------ */
/* Append n_tokens prompt tokens at positions n_past.. to the slot, filling its KV pages; the
 * logits of the LAST token are left in the slot's logit buffer. */
int b2_prefill(b2_engine* e, int slot, const int32_t* host_tokens, int n_tokens);
/* Sample from the slot's logit buffer with the slot's sampling settings; the sampled token
 * becomes the slot's next input. */
int b2_sample(b2_engine* e, int slot, int32_t* host_token_out);
/* One decode step for each listed slot: forward the slot's pending token, sample the next.
 * Writes n sampled tokens. */
int b2_decode(b2_engine* e, const int32_t* host_slots, int n, int32_t* host_tokens_out);
/* n decode steps of ONE slot queued back to back (the sampled token never leaves the device
 * between steps); the n sampled tokens come back in one copy at the end. Used for run-ahead
 * decoding: the host checks stop conditions afterwards and rewinds with b2_seq_rewind. */
int b2_decode_n(b2_engine* e, int slot, int n, int32_t* host_tokens_out);
/* Forget everything after the first n_keep tokens of the slot (KV pages beyond are simply
 * overwritten later); the token at position n_keep becomes the pending input. Needs the
 * recent-token history as it stood at that point (for the penalties). */
int b2_seq_rewind(b2_engine* e, int slot, int n_keep, int32_t pending_token,
                  const int32_t* host_history, int n_history);
/* Teacher forcing / tests: overwrite the slot's pending input token. */
int b2_seq_set_token(b2_engine* e, int slot, int32_t token);
/* Forward the slot's pending token without sampling (logits left in the slot's buffer). */
int b2_forward_pending(b2_engine* e, int slot);
/* Copy the slot's current logits [n_vocab] to the host (llama_get_logits). */
int b2_get_logits(b2_engine* e, int slot, float* host_out);
int b2_synchronize(b2_engine* e);

/* ---- layer-list models: decoders given as a list of layers over dense bf16 / f32 tensors (no counterpart in the
 *      reference, whose libllama only builds the graphs compiled into it). Each layer = one token mixer + an optional
 *      feed-forward block, both followed by a layer norm AFTER the residual sum: x <- LN(residual_scale * x + f(x)).
 *      Tensor names follow the Goponex files: embed, final.norm, head, l<i>.norm1/2, l<i>.mix.*, l<i>.mlp.*. ------------ */
#define B2_MIX_WINDOW_SCAN 1     /* sliding-window attention with a kept prefix (values = raw keys) beside a selective
                                    scan (Mamba); the two outputs are RMS-normed over the width and averaged */
#define B2_MIX_MATRIX_MEMORY 2   /* mLSTM: per-head matrix memory with capped exponential gating */
#define B2_MIX_LATENT_ATTN 3     /* sliding-window attention over one cached low-rank latent + one shared rotated key part
                                    per token, per-head softmax sink, sigmoid output gate */
#define B2_MIX_DELTA_RULE 4      /* gated delta rule: per-head matrix memory with per-row input-dependent decays, short
                                    causal convolutions on q / k / v */
#define B2_MIX_SSD 5             /* Mamba-2 state-space recurrence: scalar decay per head, grouped B / C, gated group norm */
#define B2_MIX_CHUNK_LINEAR 6    /* chunk-local attention with sigmoid key weights (whole-projection query / key norm, capped
                                    scores, per-head bias, no rotation) beside a linear attention with one fixed decay per head
                                    (SiLU feature maps, gated RMS norm over all heads); the outputs are added with fixed weights */
#define B2_MIX_SINK_DELTA 7      /* softmax attention (sliding window, a learned sink term in each head's denominator, partial
                                    rotate-half rotation, the heads' weights mixed across heads, one sigmoid gate per head) beside a
                                    gated delta rule with ONE input-dependent decay per head; the two outputs are RMS-normed over the
                                    width and averaged */
#define B2_MIX_SINK_ATTN 8       /* the same softmax attention alone; what differs is chosen by attn_flags */
#define B2_FF_RELU2 0            /* squared-ReLU block with biases (when n_ff > 0) */
#define B2_FF_MOE 1              /* routed mixture of gated (SiLU) experts, n_ff = width of one expert */
#define B2_FF_GLU 2              /* gated SiLU unit without biases: down(silu(gate x) * (up x)) */
#define B2_FF_PIECEWISE 3        /* down(act(up x)) without biases; act(z) = a z^2 + z / 2 for z > 0, b (exp(z) - 1 - z) + z / 2 otherwise,
                                    a = softplus(p), b = 1/2 + softplus(q) with (p, q) in tensor mlp.act */
#define B2_EXPERT_SILU 0         /* expert: down(silu(gate x) * (up x)) */
#define B2_EXPERT_CLAMPED 1      /* expert: g = min(gate x, limit), u = clamp(up x, -limit, limit); down(g * sigmoid(alpha g) * (u + 1)) */
#define B2_ATTN_BIAS 1           /* attn_flags: q, k, v projections carry biases (tensors q.b, k.b, v.b) */
#define B2_ATTN_UNIT_QK 2        /* after the rotation every head's q and k are divided by their RMS (no weight) */
#define B2_ATTN_TALK 4           /* weight_h(i, j) <- sum_g talk[h][g] weight_g(i, j) after the softmax (tensor talk [H][H]) */
#define B2_ATTN_HEAD_GATE 8      /* the sigmoid output gate is one number per head (tensor g [H][W]); else one per output entry */
#define B2_ROUTE_SOFTMAX_ALL 0   /* scores = softmax over all slots; an additive correction steers the choice only */
#define B2_ROUTE_TOPK_SOFTMAX 1  /* biased logits choose; weights = softmax over the chosen logits */
#define B2_BLOCK_POSTSUM_LN 0    /* x <- LayerNorm(alpha * x + f(x)) */
#define B2_BLOCK_PRENORM_RMS 1   /* x <- x + m * f(RMSNorm(x) * (1 + w)); the embedding and the output are normed the same way */
#define B2_BLOCK_OUTNORM_RMS 2   /* x <- x + RMSNorm_parts(f(x)) * w: the branch OUTPUT is normed, over norm_groups equal parts;
                                    the output norm has the same form */
#define B2_BLOCK_HYPER_RMS 3     /* n_streams copies x_1..x_S of the stream (all the embedding at first). A sublayer reads
                                    h = RMSNorm(sum_s in[s] x_s) * w, passed through a causal convolution with a skip when canon_taps > 0
                                    (h + conv(h), tensors l<i>.canon1/2 [W][taps]); its output y goes back as
                                    x_t <- sum_s mix[s][t] x_s + out[t] y (tensors l<i>.hc1/2.in, .mix, .out; absent: plain residual).
                                    The output norm reads the sum of the copies. */
typedef struct b2_layer_desc {
    int32_t mixer;            /* B2_MIX_* */
    int32_t n_ff;             /* width of the feed-forward block (of one expert for B2_FF_MOE); 0 = the layer has none */
    /* window attention */
    int32_t n_head, n_head_kv, head_dim, rot_dims, window, keep_first, rope_orig_ctx, pad0_;
    double attn_scale, rope_base, rope_factor /* <= 0: no frequency blending */, rope_fast, rope_slow;
    /* selective scan */
    int32_t conv_taps, dt_rank, d_inner, d_state;
    /* matrix memory */
    int32_t mm_heads, mm_dim, mm_vdim, pad_;
    double gate_cap;
    /* latent attention: n_head, head_dim (unrotated part), window (<= 0: none), attn_scale, rope_base, rot_dims as above */
    int32_t la_rot_dim, la_vdim, la_rank, ff_kind /* B2_FF_* */;
    /* delta rule: mm_heads, mm_dim, mm_vdim, conv_taps as above; state-space: mm_heads, mm_vdim, d_state, conv_taps */
    int32_t key_heads;        /* delta rule: q / k heads; state-space: groups sharing B and C */
    int32_t rank_a, rank_g;   /* delta rule: inner sizes of the two-step decay and gate projections */
    int32_t norm_groups;      /* state-space: parts of the gated output norm */
    /* mixture of experts */
    int32_t moe_experts, moe_identity, moe_top, moe_groups, moe_keep, pad1_;
    double moe_scale;
    int32_t moe_route;        /* B2_ROUTE_* */
    int32_t moe_shared_ff;    /* width of a gated expert every token also runs (0: none) */
    /* chunk-local sigmoid attention (n_head, n_head_kv, head_dim, attn_scale as above; window = chunk size, <= 0: causal over
     * the whole sequence) beside fixed-decay linear attention (mm_heads, mm_dim, mm_vdim; decays in tensor mix.right.decay) */
    int32_t attn_vdim, pad2_;
    double softcap;           /* score <- softcap * tanh(score / softcap); <= 0: scores are not capped */
    double branch_scale[2];   /* weights of the two branches in the sum */
    /* softmax attention with a sink (n_head, n_head_kv, head_dim, attn_vdim, rot_dims, rope_base, window (<= 0: none), attn_scale as
     * above) and the head-decay delta rule (mm_heads, key_heads, mm_dim, mm_vdim, conv_taps) */
    int32_t attn_flags;       /* B2_ATTN_* */
    int32_t weights_of;       /* 1 + index of the layer whose tensors this entry uses (a repeated run of layers shares weights; every
                                 entry keeps cache and state of its own); 0: its own */
    int32_t moe_expert;       /* B2_EXPERT_* */
    int32_t moe_renorm;       /* != 0: the chosen scores are divided by their sum (+ 1e-20) */
    double moe_limit;         /* B2_EXPERT_CLAMPED */
    double moe_alpha;         /* B2_EXPERT_CLAMPED: slope inside the sigmoid */
} b2_layer_desc;
typedef struct b2_layered_config {
    int32_t n_layer, n_embd, n_vocab;
    float norm_eps, residual_scale;
    int32_t n_ctx;            /* max tokens per sequence */
    int32_t max_seqs;         /* sequence slots = recurrent-state slots */
    int32_t kv_block_tokens, kv_num_blocks;
    int32_t max_step_tokens;  /* most tokens one b2_step call may bring */
    int32_t device, flags;    /* B2_FLAG_F32 */
    int32_t block_style;      /* B2_BLOCK_* */
    float logit_scale;        /* logits = head x * logit_scale (0 is read as 1) */
    float embed_scale;        /* the embedding row times this (0 is read as 1) */
    int32_t norm_groups;      /* B2_BLOCK_OUTNORM_RMS: equal consecutive parts of the width, each normed by itself (0 is read as 1) */
    int32_t tie_head;         /* != 0: the output map is the embedding table (no tensor "head") */
    int32_t n_streams;        /* B2_BLOCK_HYPER_RMS: copies of the residual stream (0 is read as 1) */
    int32_t canon_taps;       /* B2_BLOCK_HYPER_RMS: taps of the convolution on every sublayer's input (0: none) */
} b2_layered_config;
/* Then b2_upload_tensor for every tensor (BF16 / F32), b2_engine_finalize, b2_seq_set_blocks / b2_seq_begin (n_past must be
 * 0: recurrent state cannot be rewound; it zeroes the slot's state) as for any engine. */
int b2_engine_create_layered(const b2_layered_config* cfg, const b2_layer_desc* layers, b2_engine** out);

/* One step over a ragged batch: entry i brings n_tokens[i] consecutive tokens (a prompt portion or one decoded token) of
 * the sequence in slots[i], continuing from what earlier steps left in its pages and state; `host_tokens` holds all
 * entries' tokens one after another. `want_rows` (indices into host_tokens) are the rows whose logits are copied to
 * host_logits [n_want][n_vocab]. sample[i] != 0: sample from the logits of entry i's last token with the slot's sampler
 * and return the token in host_sampled[i] (-1 elsewhere); those logits also stay in the slot's logit buffer. Any of
 * want_rows / sample / host_sampled may be NULL. */
#define B2_STEP_MAX_ENTRIES 64
int b2_step(b2_engine* e, int n_entries, const int32_t* slots, const int32_t* n_tokens, const int32_t* host_tokens,
            const int32_t* want_rows, int n_want, float* host_logits, const int32_t* sample, int32_t* host_sampled);
/* Debugging / parity: keep the residual stream after every layer of the next steps (on != 0), and read it back:
 * host_out [n_layer][T][n_embd] for the T tokens of the last step. */
int b2_step_trace(b2_engine* e, int on);
int b2_step_trace_read(b2_engine* e, float* host_out, int n_layer, int T);
/* Device time of the last `b2_step` by kernel kind (events around every launch when on != 0; slows the step down).
 * kinds: 0 embed, 1 dense products, 2 attention, 3 scan / state-space, 4 matrix memories, 5 norms, 6 head, 7 expert routing.
 * ms_out[8], launches_out[8]. */
int b2_step_profile(b2_engine* e, int on);
int b2_step_profile_read(b2_engine* e, float* ms_out, int32_t* launches_out);

/* ---- measurement hooks (bench.py): CUDA events on the engine's own stream --------------- */
int b2_timer_start(b2_engine* e);
int b2_timer_stop(b2_engine* e, float* ms_out);          /* synchronises */
int b2_kernel_launch_count(b2_engine* e, int64_t* n);   /* kernels launched since create */
/* How the engine is running: CUDA graphs on/off, PDL on/off, int8 activation planes (1|2),
 * CTAs per mat-vec launch, attention split count. Any pointer may be NULL. */
int b2_engine_mode(b2_engine* e, int* graph, int* pdl, int* act_planes, int* n_ctas, int* n_splits);
/* Tensor-parallel state: rank, world size (1 = not tensor parallel) and whether the hidden-vector all-reduce runs over
 * mapped peer memory (1) or through NCCL (0). Any pointer may be NULL. */
int b2_engine_tp_mode(b2_engine* e, int* rank, int* world, int* peer_memory);
/* Per-kernel-kind device time of ONE un-graphed, un-overlapped decode step of `slot`
 * (events around every launch). kinds: 0 embed, 1 qkv, 2 attention, 3 attn_out, 4 gate_up,
 * 5 ffn_down, 6 lm_head, 7 sampler. ms_out[8], launches_out[8], bytes_out[8] (algorithmic). */
int b2_profile_decode_step(b2_engine* e, int slot, float* ms_out, int32_t* launches_out,
                           int64_t* bytes_out);

/* Streaming rate of the decode mat-vec kernel alone (scripts/mv_micro.py): synthetic weight bytes made on the
 * device, `iters` launches back to back on one stream cycling through n_copies weight sets (size them past the
 * L2), chained by programmatic dependent launch when pdl != 0. mode: 0 store, 1 residual add, 3 fused gate|up
 * (two matrices of n_rows). us_per_launch_out = mean device time per launch (CUDA events). */
int b2_bench_matvec(int device, int mode, int ggml_type, int n_rows, int K, int n_copies, int iters, int n_ctas,
                    int act_planes, int pdl, float* us_per_launch_out);

/* ---- single-operator entry points (parity tests call the kernels through these).
 *      All pointers are HOST memory; the call stages data through device scratch. ---------- */
/* ggml dequantize_row_* / gguf.quants.dequantize */
int b2_op_dequantize(int device, int ggml_type, const void* host_blocks, int64_t n_elems, float* host_out);
/* y[n_rows] = W[n_rows, K] . x  (+ optional fused RMSNorm of x, + optional residual);
 * ggml-cuda quantize_q8_1 + mul_mat_vec_q (+ rms_norm_f32, add). act_planes = 1 or 2. */
int b2_op_matvec(int device, int ggml_type, const void* host_w, int n_rows, int K, const float* host_x,
                 const float* host_norm_w, float eps, const float* host_resid, float* host_y,
                 int act_planes, int n_ctas);
/* fused gate/up: y[n_rows] = silu(Wg . x) * (Wu . x), x optionally RMS-normed first */
int b2_op_gate_up(int device, int type_gate, const void* host_wg, int type_up, const void* host_wu,
                  int n_rows, int K, const float* host_x, const float* host_norm_w, float eps,
                  float* host_y, int n_ctas);
/* Prefill / batched GEMM on the tensor cores (tcgen05, in-shared-memory dequantisation):
 * y[t][n] = (y_in ? y_in[t][n] : 0) + sum_k f16(x[t][k]) * W[n][k]; x [T][K] f32 (rounded to f16 on the device),
 * W [n_rows][K] raw GGUF blocks, T <= 512, K % 256 == 0. Replaces ggml-cuda's dequantise-to-f16 + cublasGemmEx
 * prompt path that create_chat_completion reaches (/root/reference/api.py:55-63).
 * n_splits: K ranges computed by separate CTAs and added in order (0 = the engine's own choice, else 1..16). */
int b2_op_gemm(int device, int type, const void* host_w, int n_rows, int K, const float* host_x, int T,
               const float* host_y_in, float* host_y, int n_splits);
/* ggml rms_norm_f32 * weight */
int b2_op_rmsnorm(int device, const float* host_x, const float* host_w, float eps, int K, int rows, float* host_y);
/* Decode attention for one sequence: q [n_head*head_dim] f32 (already rotated), K/V as f16
 * [n_ctx_tokens][n_kv][head_dim] (token-major; the op scatters them into pages in the order
 * host_blocks gives), attends to all n_ctx_tokens. out [n_head*head_dim] f32. * n_splits < 0 selects the tensor-core kernel (attention_mma.cu, q rounded to f16) with -n_splits splits. */
int b2_op_attention_decode(int device, const float* host_q, const uint16_t* host_k, const uint16_t* host_v,
                           int n_ctx_tokens, int n_head, int n_kv, int head_dim, int block_tokens,
                           const int32_t* host_blocks, int n_blocks_total, int n_splits, float* host_out);
/* penalties + greedy/top-k/top-p/min-p/temperature draw over logits[n_vocab] with the given
 * recent-token history and uniform u in [0,1). */
int b2_op_sample(int device, const float* host_logits, int n_vocab, const b2_sampling* sampling,
                 const int32_t* host_history, int n_history, double u, int32_t* host_token_out);

/* ---- decode attention that allocates nothing (no counterpart in the reference: llama.cpp
 *      allocates its compute buffers itself; this exists for hosts of THIS library).
 *
 * Same kernel and same result as the split path of b2_op_attention_decode, for callers that
 * cannot ask the driver for memory at call time: a host that has already committed all of its
 * HBM to weights and KV pages, or one whose token loop must not hit the allocator (an
 * allocation serialises the device and can fail under memory pressure). The split-merge
 * scratch is a fixed 1 MiB array (plus 256 B of tickets) built into the library; every GPU that
 * loads the library carries it until the process exits.
 *
 * All pointers are DEVICE pointers owned by the caller: q [n_head*head_dim] f32, the paged K and
 * V pools [page][n_kv][block_tokens][head_dim] f16, the page table (max_pages entries), *dev_pos
 * = index of the newest token (attends to 0..pos), out [n_head*head_dim] f32. `stream` is a
 * cudaStream_t (NULL = default stream); the call only enqueues work.
 * Limits: n_splits >= 2, (n_head / n_kv) * n_splits <= 512, n_head * n_splits * (head_dim + 2) <= 262144 floats,
 * n_kv <= 64, max_pages <= 512; anything larger is rejected with B2_ERR_ARG and a message naming the limit.
 * The K and V pools must be 16-byte aligned (the kernel reads them with bulk copies), the other pointers 4-byte
 * aligned; misaligned pointers are rejected. *dev_pos must be < max_pages * block_tokens: the kernel reads the
 * position on the device and attends to at most max_pages * block_tokens positions whatever it says.
 * The caller's current CUDA device is left as it was.
 * The first call on each device also looks up the array's device address (cudaGetSymbolAddress)
 * and sets a kernel attribute; make that first call before starting any stream capture.
 * Every call uses the same array: it clears the tickets, the partials are overwritten before they
 * are read, and two calls that overlap on the GPU (different streams) race with each other.
 * No cudaMalloc, cudaFree or allocating library routine is called, also when this is the very first call
 * into the library. The engine paths report a kernel that timed out on a barrier through a pinned host word;
 * creating that word allocates, so this entry point does without it and cannot report such a time-out. */
int b2_attention_decode_static(int device, const float* dev_q, const uint16_t* dev_k_pool,
                               const uint16_t* dev_v_pool, const int32_t* dev_block_table, int max_pages,
                               const int32_t* dev_pos, int n_head, int n_kv, int head_dim, int block_tokens,
                               int n_splits, float* dev_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_GGUF_H */
