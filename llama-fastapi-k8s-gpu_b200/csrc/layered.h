// Layer-list models: a decoder described by a list of layers, each a token mixer (of several kinds) and an optional
// feed-forward block, over dense bf16 / f32 tensors. Internal launch interfaces between the graph (layered.cu), the
// dense products (dense.cu) and the mixer kernels (mixers.cu). The llama graph over GGUF blocks is engine.cu.
//
// A step is a RAGGED batch: `n_seg` segments (one per sequence taking part), segment s brings seg_len[s] consecutive
// tokens of the sequence in slot seg_slot[s] starting at position seg_pos0[s]; all T tokens are concatenated. Prompt
// portions and single decoded tokens are the same thing. Every kernel below reads this description from device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct b2_engine;

namespace b2 {

struct RaggedDev {             // device pointers, valid for one step
    const int* tok_id;         // [T] token ids
    const int* tok_seg;        // [T] segment of each token
    const int* tok_pos;        // [T] position inside its sequence
    const int* seg_slot;       // [n_seg]
    const int* seg_start;      // [n_seg] first row of the segment
    const int* seg_len;        // [n_seg]
    const int* seg_pos0;       // [n_seg] position of the segment's first token
    const int* tile_seg;       // [n_tiles] tiles of up to 64 consecutive rows of one segment: its segment ...
    const int* tile_row0;      // ... and its first row
    int T, n_seg, n_tiles;
};

// ---------------------------------------------------------------- dense products (dense.cu)
// Y[t][n] = epi(sum_k X[t][k] * W[n][k] (+ bias[n])), X f32 [T][ldx], W [N][K] (bf16 or f32), Y f32 [T][ldy].
// Each output element is one fixed-order sum over k: a row's result does not depend on what else is in the batch.
// EPI_GLU_SILU: weight rows come in pairs (2i = gate, 2i + 1 = up); output column i = silu(gate) * up, N counts weight rows.
// EPI_MUL_SIGMOID: the product times sigmoid(aux[t][n]).
// EPI_GLU_CLAMP: pairs as above; g = min(gate, p0), u = clamp(up, -p0, p0); output = g * sigmoid(p1 * g) * (u + 1).
// EPI_PIECEWISE: z > 0: p0 z^2 + z / 2; else p1 (exp(z) - 1 - z) + z / 2.
enum DenseEpi { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_RELU2 = 2, EPI_GLU_SILU = 3, EPI_MUL_SIGMOID = 4, EPI_GLU_CLAMP = 5, EPI_PIECEWISE = 6 };
// Grouped products (mixture of experts): the rows of a step's (token, choice) pairs, each against the matrix of its group.
//   tiles == nullptr: row p of the product is pair p itself, blockIdx.y walks the pairs one by one (few-token steps);
//   else: pairs sorted by group, tile i = rows [tile_row0[i], + tile_rows[i]) of group tile_group[i]; *n_tiles of them.
// The input row of pair row p is x_rows ? x_rows[p] : p; pairs whose group is >= n_groups (or < 0) are skipped.
struct DenseGroups {
    const int* group = nullptr;        // untiled: [rows] group of each row
    const int* x_rows = nullptr;       // [rows] input row of each product row, or null
    const int* tile_group = nullptr;   // tiled: per tile
    const int* tile_row0 = nullptr;
    const int* tile_rows = nullptr;
    const int* n_tiles = nullptr;      // device scalar
    int n_groups = 0;
    long w_stride = 0;                 // elements between the matrices of two groups
    int max_tiles = 0;                 // grid size of a tiled launch
    int tile_max = 64;                 // most rows of a tile: 64, or 128 (large tensor-core tiles; bf16 serving mode only)
    int x_total_rows = 0;              // rows of the input matrix (128-row tiles: it is rounded to bf16 as a whole first)
};
struct DenseArgs {
    const float* x; int ldx;
    const void* w; int w_type;      // T_BF16 or T_F32 (quant_blocks.cuh ids)
    const float* bias;              // f32 [N] or null
    float* y; int ldy;
    int T, N, K;
    int epi;
    bool exact;                     // true: 32-bit multiply-adds (no tensor cores, inputs not rounded)
    __nv_bfloat16* xb;              // scratch [T][K] for X rounded to bf16 (large tensor-core steps); null: not available
    float scale = 1.f;              // the product (after the epilogue) times this
    float p0 = 0.f, p1 = 0.f;       // constants of EPI_GLU_CLAMP / EPI_PIECEWISE
    const float* aux = nullptr; int ldaux = 0;      // EPI_MUL_SIGMOID
    // batch > 1: `batch` independent products, operand b at x + b * x_bs, w + b * w_bs (elements), y + b * y_bs, aux + b * aux_bs
    int batch = 1; long x_bs = 0, w_bs = 0, y_bs = 0, aux_bs = 0;
    int x_span = 0;                 // batch > 1: columns of x that hold all batches' inputs (for the rounded copy), or 0
    const DenseGroups* groups = nullptr;            // grouped product (T = number of pair rows)
};
cudaError_t dense_launch(const DenseArgs& a, cudaStream_t s);

// ---------------------------------------------------------------- mixers and norms (mixers.cu)
// x[t] = table[tok_id[t]] * scale
cudaError_t embed_ragged_launch(const void* table, int w_type, int W, const int* tok_id, int T, float* x, float scale, cudaStream_t s);
// gather rows: y[i] = x[rows[i]]
cudaError_t gather_rows_launch(const float* x, int W, const int* rows, int n, float* y, cudaStream_t s);

// Post-sum layer norm: x[t] = LN(alpha * x[t] + y[t]) * w with
//   y = a                      (b == nullptr)
//   y = (rms(a) * wa + rms(b) * wb) / 2   (two branches, each RMS-normed over the width first)
cudaError_t postsum_norm_launch(float* x, const float* a, const float* wa, const float* b, const float* wb, const float* w,
                                float alpha, float eps, int W, int T, cudaStream_t s);
// Pre-norm blocks: if (add) x[t] += mult * add[t]; if (y) y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * (w_offset + w) * out_scale.
// y may be x itself.
cudaError_t resid_rms_norm_launch(float* x, const float* add, float mult, const float* w, float w_offset, float out_scale,
                                  float eps, int W, int T, float* y, cudaStream_t s);
// plain layer norm without bias: y[t] = LN(x[t]) * w
cudaError_t layer_norm_launch(const float* x, const float* w, float eps, int W, int T, float* y, cudaStream_t s);

struct RotaryTable {           // cos and sin of position * frequency (frequencies already blended, magnitude factor folded
    const float* cos;          // in), [n_ctx][rot_dims / 2] each, built on the host in double precision
    const float* sin;
    int rot_dims;
};
struct WindowAttnArgs {
    const float* proj; int ldp; int q_off, k_off;     // projection rows: q at q_off [H*d], k at k_off [G*d]
    const float* q_norm_w; const float* k_norm_w;     // [d]
    RotaryTable rot;
    void* k_pool; void* v_pool; int cache_f32;        // pages [page][G][block_tokens][d]; bf16 or f32
    int* const* block_tables;                         // [slot] -> page table
    int block_tokens;
    int H, G, d;
    int window, keep_first;
    float scale, eps;
    float* q_rot;              // scratch [T][H*d]
    float* out;                // [T][H*d]
    float* split_scratch;      // few-token steps: partial (max, sum, output) per key range, [T][H][splits][d + 2]
    int split_capacity;        // floats in split_scratch
};
// norm + rotate q and k, store k (rotated) and v (= k as projected) into the pages
cudaError_t window_attn_store_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s);
// softmax attention of every step token over the visible cached keys of its sequence
cudaError_t window_attn_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s);

struct ScanArgs {              // selective scan (Mamba)
    const float* proj; int ldp; int x_off, z_off;     // W_in output rows: x at x_off [inner], z at z_off [inner]
    const float* conv_w; const float* conv_b; int taps;   // [inner][taps], [inner]
    float* conv_state;         // [slot][inner][taps-1] last inputs, newest last
    float* xc;                 // [T][inner] convolved + SiLU
    const float* xproj; int ldx; int R, N;            // W_x output rows: dt [R] | B [N] | C [N]
    const float* dt_raw;       // [T][inner] W_dt dt (bias not yet added)
    const float* dt_bias; const float* A_log; const float* D;
    float* ssm_state;          // [slot][inner][N]
    float* y;                  // [T][inner] gated output
    int inner;
};
cudaError_t scan_conv_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s);
cudaError_t scan_recurrence_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s);

struct MatrixMemArgs {         // mLSTM
    const float* proj; int ldp; int q_off, k_off, v_off, g_off, i_off, f_off;
    const float* i_bias; const float* f_bias; const float* norm_w;
    int H, d, dv;
    float cap, eps;
    float* S; float* n; float* m;      // per slot: [H][d][dv], [H][d], [H]
    float* o_raw;              // [T][H*dv] scratch: memory read-out before the head norm
    float* out;                // [T][H*dv]
};
cudaError_t matrix_mem_launch(const MatrixMemArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- short causal convolution (state_mixers.cu)
// out[t][c] = silu(bias[c] + sum_j w[c][j] * in[t - (taps-1) + j][c]) over C neighbouring columns of `in`; inputs before the
// step come from the slot's state (the last taps-1 inputs, [slot][taps-1][C]), zeros before the sequence.
struct ConvArgs {
    const float* in; int ld_in;
    int C, taps;
    const float* w; const float* bias;      // [C][taps]; [C] or null
    float* state;
    float* out; int ld_out;
    int skip = 0;                            // 1: out = in + conv(in) without bias or activation (a convolution around a skip path)
};
cudaError_t causal_conv_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s);
// the state moves on to the last taps-1 inputs of every segment (after causal_conv_launch has read the old one)
cudaError_t causal_conv_advance_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- matrix-state recurrences (state_mixers.cu)
// Per head a memory S [R rows][P columns], 32-bit, one per sequence slot. For every token of a segment, in order:
//   S[r][:] *= row_decay[r] * head_decay          (either may be absent)
//   u = val_scale * (val - (delta ? S^T wk : 0))  (delta rule: write only what the memory does not return yet)
//   S += wk u^T ;  y = S^T rk + skip * val        (the read-out sees the current token's write)
// Covers the gated delta rule (row decays, delta = 1), the Mamba-2 state-space recurrence (head decay, skip) and linear
// attention with one fixed decay per head (head_const, no value scale).
struct ColStateArgs {
    const float* wk; int ld_wk;            // [T][G * R] write keys
    const float* rk; int ld_rk;            // [T][G * R] read keys
    const float* row_decay; int ld_rd;     // [T][H * R] or null
    const float* head_decay; int ld_hd;    // [T][H] or null
    const float* head_const = nullptr;     // [H] or null: a decay that does not depend on the token (used when head_decay is null)
    const float* val; int ld_v;            // [T][H * P]
    const float* val_scale; int ld_vs;     // [T][H], or null for 1
    const float* skip;                     // [H] or null
    int H, G, R, P, delta;
    float* state;                          // [slot][H][P][Rp], Rp = R rounded up to 4 (column-major, pads stay zero)
    float* y; int ld_y;                    // [T][H * P]
};
inline size_t col_state_floats(int H, int R, int P) { return (size_t)H * P * ((R + 3) / 4 * 4); }
cudaError_t col_state_launch(const ColStateArgs& a, const RaggedDev& r, cudaStream_t s);

// Delta-rule inputs, in place: q and k [T][G*d] to unit length per head (q also times d^-1/2), the decay columns
// a [T][H*d] <- exp(-exp(A_log[h]) * softplus(a + dt_bias)), beta [T][H] <- sigmoid(beta).
struct DeltaPrepArgs {
    float* q; float* k; int ld_qk; int G, d;
    float* a; int ld_a; const float* A_log; const float* dt_bias; int H;
    float* beta; int ld_b;
    float unit_eps;
    int a_cols = 0;                          // decay columns per head: 0 = d (one per key channel), 1 = one decay per head
};
cudaError_t delta_prepare_launch(const DeltaPrepArgs& a, int T, cudaStream_t s);
// Mamba-2 step sizes, in place: dt [T][H] <- softplus(dt + dt_bias[h]); decay [T][H] = exp(-exp(A_log[h]) * dt)
cudaError_t ssd_prepare_launch(float* dt, int ld_dt, const float* dt_bias, const float* A_log, int H, float* decay, int T, cudaStream_t s);

// RMS norm over groups of n neighbouring columns with a gate. gate_first = 0: y = x / rms(x) * w * sigmoid(gate);
// gate_first = 1: v = x * silu(gate), y = v / rms(v) * w. w index: group * w_gstride + i.
struct GroupNormArgs {
    const float* x; int ld_x; const float* gate; int ld_g; const float* w; int w_gstride;
    int groups, n; float eps; int gate_first;
    float out_scale = 1.f;
    int gate_silu = 0;                       // gate_first = 0 only: times silu(gate) instead of sigmoid(gate)
    float* y; int ld_y;
};
cudaError_t group_norm_gate_launch(const GroupNormArgs& a, int T, cudaStream_t s);

// ---------------------------------------------------------------- latent attention (latent_attn.cu)
// Every token caches one row [c (rank) | rotated shared key part (dr)]; all heads read the same rows. With the per-head
// key expansion folded into the query (qv[t][h] = [W_uk,h^T q_h | rotated q part]) a head's score is one dot product with
// the cached row, and the attention output is a weighted sum of the c parts, expanded to values afterwards.
// Sliding window; the softmax denominator also holds exp(sink[h]).
struct LatentAttnArgs {
    const float* proj; int ldp; int q_off, dkv_off;   // q [H][d + dr], dkv [rank + dr]
    const float* c_norm_w;                            // [rank]
    RotaryTable rot;                                  // pairs (i, i + rot_dims / 2)
    void* pool; int cache_f32;                        // pages [page][block_tokens][rank + dr]
    int* const* block_tables; int block_tokens;
    int H, d, dr, rank, window;
    float scale, eps;
    const float* sink;                                // [H]
    float* qv;                                        // [T][H][rank + dr]; the first `rank` of each head are filled by the caller
    float* o_lat;                                     // [T][H][rank]
    float* split_scratch;      // few-token steps: partial (max, sum, output) per key range, [T][H][splits][rank + 2]
    int split_capacity;        // floats in split_scratch
};
// norm of c, rotation of the shared key part, both into the pages; rotated query parts into qv
cudaError_t latent_store_launch(const LatentAttnArgs& a, const RaggedDev& r, cudaStream_t s);
cudaError_t latent_attn_launch(const LatentAttnArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- mixture of experts (moe.cu)
struct MoeRouteArgs {
    const float* logits; int ld;           // [T][n_slots] router outputs (32-bit products)
    const float* correction;               // [n_slots]
    int n_slots, n_experts, top, n_groups, keep_groups;
    float scale;
    int mode = 0;                          // 0: weight = softmax over all slots (times scale), `correction` added for the choice only;
                                           // 1: logits + correction choose, weight = softmax over the chosen biased logits
    int renorm = 0;                        // mode 0: the chosen scores are divided by their sum (+ 1e-20) before the scale
    int* sel; float* weight;               // [T][top]
    int* pair_token;                       // [T][top]: t (the input row of each pair)
};
cudaError_t moe_route_launch(const MoeRouteArgs& a, int T, cudaStream_t s);
// pairs sorted by expert into tiles of `tile` rows: pos[p] = row of pair p in the sorted order (-1: identity slot), x_rows[row] =
// token of that row, and the tile table; all in device memory (meta: [0] = number of tiles)
struct MoeSortArgs {
    const int* sel; int n_pairs, top, n_experts, tile;      // tile: rows per tile
    int* pos; int* x_rows; int* tile_group; int* tile_row0; int* tile_rows; int* n_tiles; int max_tiles;
};
cudaError_t moe_sort_launch(const MoeSortArgs& a, cudaStream_t s);
// out[t] = sum over the token's choices, in choice order, of weight * (expert output row | h[t] for identity slots)
cudaError_t moe_combine_launch(const int* sel, const float* weight, const int* pos, const float* rows, const float* h, int n_experts,
                               int top, int W, int T, float* out, cudaStream_t s);

// the same sum joined to the residual stream in one pass (pre-norm blocks): x[t] += mult * sum; if (y) y[t] = RMS norm of the
// new x[t] times (w_offset + w). y may be the buffer h points to (a token's h is read before its y is written).
struct MoeJoinArgs {
    const int* sel; const float* weight; const int* pos; const float* rows; const float* h;
    int n_experts, top;
};
cudaError_t moe_join_launch(const MoeJoinArgs& j, float* x, float mult, const float* w, float w_offset, float eps, int W, int T, float* y,
                            cudaStream_t s);

// Blocks that norm what a branch RETURNS: v[t] = a[t] (if given) + the mixture's weighted sum (if given); each of `groups` equal
// consecutive parts of v is brought to unit RMS, the whole is multiplied by w; then x[t] += that (x given) or y[t] = that.
// y may be a.
cudaError_t outnorm_join_launch(float* x, const float* a, const MoeJoinArgs* moe, const float* w, int groups, float eps, int W, int T,
                                float* y, cudaStream_t s);

// ---------------------------------------------------------------- sigmoid attention (sigmoid_attn.cu)
// Attention without a softmax: the weight of a visible key is sigmoid(cap(q . k * scale) + bias[h]), cap(z) = softcap *
// tanh(z / softcap); nothing is normalised over the keys and no position is rotated in. Visible keys: those of the query's own
// chunk of `chunk` positions (chunks counted from position 0 of the sequence) up to the query; chunk <= 0: all earlier keys.
// Queries and keys are RMS-normed over the WHOLE projection (all heads at once) with a weight of that size. Grouped query
// heads; the value size may differ from the key size.
struct SigmoidAttnArgs {
    const float* proj; int ldp; int q_off, k_off, v_off;      // projection rows: q [H*d], k [G*d], v [G*dv]
    const float* q_norm_w; const float* k_norm_w;              // [H*d], [G*d]
    void* k_pool; void* v_pool; int cache_f32;                 // pages [page][G][block_tokens][d] and [page][G][block_tokens][dv]
    int* const* block_tables; int block_tokens;
    int H, G, d, dv, chunk;
    float scale, softcap, eps;                                 // softcap <= 0: none
    const float* bias;                                         // [H] or null
    float* q_out;                                              // scratch [T][H*d]: normed queries
    float* out; int ld_out; float out_scale;                   // out[t][h*dv + i], times out_scale
    float* act; int act_n;                                     // act_n > 0: columns [0, act_n) of act (row stride ldp) get SiLU in place
};
// norm of q and k, keys and values into the pages (and the SiLU columns)
cudaError_t sigmoid_attn_store_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s);
cudaError_t sigmoid_attn_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- softmax attention with a sink (sink_attn.cu)
// Grouped-query softmax attention over the paged cache: sliding window (position i sees j with 0 <= i - j < window; window
// <= 0: all earlier keys), rotate-half rotation of the first rot_dims entries of every head of q and k, optionally unit-RMS q
// and k after the rotation, and one extra term exp(sink[h]) in every head's denominator (no key, no value). With `talk` the
// normalised weights of the heads are mixed, weight_h <- sum_g talk[h][g] weight_g, before head h applies them to the values
// of ITS key/value head: the kernels then compute A[g][c] = sum_j weight_g(j) v_c(j) for every (query head g, value head c)
// and a small pass forms out_h = gate_h * sum_g talk[h][g] A[g][c(h)]. The value size may differ from the key size.
struct SinkAttnArgs {
    const float* proj; int ldp; int q_off, k_off, v_off;      // projection rows: q [H*d], k [G*d], v [G*dv]
    RotaryTable rot;                                           // pairs (i, i + rot_dims / 2)
    int unit_qk;
    void* k_pool; void* v_pool; int cache_f32;                 // pages [page][G][block_tokens][d] and [page][G][block_tokens][dv]
    int* const* block_tables; int block_tokens;
    int H, G, d, dv, window;
    float scale, eps;
    const float* sink;                                         // [H] or null
    const float* talk;                                         // [H][H] or null
    const float* gate; int ld_gate; int gate_per_head;         // sigmoid output gate read at gate[t * ld_gate + (h | h * dv + i)], or null
    float* q_rot;                                              // scratch [T][H*d]
    float* cross;                                              // scratch [T][H][G][dv] (talk only)
    float* part; int part_capacity;                            // few-token steps: (max, sum, output) per key range, floats available
    int max_keys;                                              // most keys a query can see (the window, or the context size)
    float* pbuf; size_t pbuf_floats;                           // prompts with mixed heads: the normalised weights of a group of query tiles
    float* out; int ld_out;                                    // out[t][h*dv + i]
};
// rotation (and unit RMS) of q and k, keys and values into the pages
cudaError_t sink_attn_store_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s);
cudaError_t sink_attn_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s);

// ---------------------------------------------------------------- several copies of the residual stream (hyper.cu)
// The stream exists in S copies xs[s] (copy s of token t at xs + s * stream_stride + t * W). One pass per sublayer boundary:
//   1. the pending sublayer output y[t] -- a dense row `a`, or (rms(a) wa + rms(b) wb) / 2 for a two-branch mixer, plus a
//      mixture's weighted sum of expert rows -- is written back: x_t <- sum_s mix[s][t] x_s + out[t] y   (mix == null: x_t += y)
//   2. the next sublayer's input is read: hn[t] = RMSNorm(sum_s in[s] x_s) * norm_w                        (in == null: x_0)
//   3. sum_out[t] = sum_s x_s (for the output norm and for tracing)
// Any of the three may be absent. bcast != 0: only copy 0 holds data yet; the others are read as equal to it and all are written
// (the state right after the embedding).
struct HyperJoinArgs {
    float* xs; long stream_stride; int S;
    const float* a; const float* wa; const float* b; const float* wb;      // pending output (a == null and no moe: nothing pending)
    const MoeJoinArgs* moe;
    const float* mix; const float* out;                                     // [S][S] indexed [from][to], [S]
    const float* in; const float* norm_w; float* hn;                        // next read (hn == null: none)
    float* sum_out;
    int bcast;
    float eps;
};
cudaError_t hyper_join_launch(const HyperJoinArgs& a, int W, int T, cudaStream_t s);
// Few-token steps (hyper_join_conv_fits): the same pass, the convolution around a skip on the input it reads (cv.in is not used:
// the normed input never leaves the chip; cv.out gets in + conv(in)) and the hand-over of the convolution's state, in ONE launch
// with one CTA per segment. Same numbers as hyper_join_launch + causal_conv_launch + causal_conv_advance_launch.
bool hyper_join_conv_fits(int W, int taps, int T, int S);
cudaError_t hyper_join_conv_launch(const HyperJoinArgs& a, const ConvArgs& cv, const RaggedDev& r, int W, cudaStream_t s);

// ---------------------------------------------------------------- graph (layered.cu)
struct LayeredModel;
int layered_finalize(b2_engine* e);
void layered_destroy(b2_engine* e);
int layered_seq_reset(b2_engine* e, int slot);

}  // namespace b2
