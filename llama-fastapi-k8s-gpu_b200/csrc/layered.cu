// Layer-list models (include/b200_gguf.h: b2_engine_create_layered, b2_step): the graph of a decoder given as a list of
// layers over dense bf16 / f32 tensors, stepped over ragged batches. Token mixers: window attention beside a selective
// scan, an mLSTM matrix memory, latent attention, the gated delta rule, a Mamba-2 state-space layer, chunk-local sigmoid
// attention beside fixed-decay linear attention, softmax attention with a sink alone or beside a head-decay delta rule.
// Feed-forward blocks: squared ReLU with biases, a gated SiLU unit, a block with a piecewise activation, or a routed mixture of
// gated experts (SiLU or clamped; with an optional shared expert). Four block styles: layer norm AFTER each residual sum,
// pre-norm (zero-centred RMS weights) with a scaled branch, an RMS norm in parts on each branch's OUTPUT, or pre-norm over
// several copies of the stream with mixing matrices and a convolution on every sublayer's input. A layer entry may name another
// layer's tensors (a repeated run of layers: shared weights, cache and state of its own). Shares the engine object with the
// llama graph (engine.cu): tensors, sequence slots and their page tables, sampler state, stream, error reporting. Owns: fused
// projection matrices, per-layer cache pages, per-slot recurrent state, the step workspace.
#include "engine_state.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <math.h>
#include <string.h>

#include <algorithm>

namespace b2 {

struct DenseW { const void* w = nullptr; int type = 0, N = 0, K = 0; };

struct LyLayer {
    b2_layer_desc d = {};
    float *norm1 = nullptr, *norm2 = nullptr;
    // window attention + selective scan
    DenseW in_proj, attn_o, scan_x, scan_dt, scan_o;      // in_proj rows: q | k | x | z
    int q_off = 0, k_off = 0, x_off = 0, z_off = 0;
    float *q_norm = nullptr, *k_norm = nullptr, *left_w = nullptr, *right_w = nullptr;
    float *rot_cos = nullptr, *rot_sin = nullptr;
    float *conv_w = nullptr, *conv_b = nullptr, *dt_b = nullptr, *A_log = nullptr, *Dskip = nullptr;
    void *k_pool = nullptr, *v_pool = nullptr;
    float *conv_state = nullptr, *ssm_state = nullptr;
    // matrix memory
    DenseW mm_proj, mm_o;                                  // mm_proj rows: q | k | v | g | i | f
    int mq = 0, mk = 0, mv = 0, mg = 0, mi = 0, mf = 0;
    float *i_b = nullptr, *f_b = nullptr, *mm_norm = nullptr;
    float *S = nullptr, *nvec = nullptr, *mmax = nullptr;
    // feed-forward
    DenseW up, down;
    float *up_b = nullptr, *down_b = nullptr;
    // latent attention: la_proj rows q | dkv | g; uk_t = W_uk transposed per head [H][rank][d]
    DenseW la_proj, uk_t, uv;
    int g_off = 0, dkv_off = 0;
    float *c_norm = nullptr, *sink = nullptr;
    void* la_pool = nullptr;
    // delta rule (st_proj rows q | k | v | b | a1 | g1) and state-space layer (st_proj rows z | x | B | C | dt)
    DenseW st_proj, a2, g2, ag, st_o;                      // ag: a2 and g2 as one block-diagonal matrix over the input a1 | g1
    int v_off = 0, b_off = 0, a1_off = 0, g1_off = 0, dt_off = 0, conv_off = 0, conv_C = 0;
    float *st_conv_w = nullptr, *st_conv_b = nullptr, *st_conv_state = nullptr, *st_A_log = nullptr, *st_dt_bias = nullptr,
          *st_D = nullptr, *st_norm = nullptr, *st_state = nullptr;
    // mixture of experts: gate_up = [E][2 ff][W] with rows 2i = gate i, 2i + 1 = up i; e_down = [E][W][ff]
    DenseW router, gate_up, e_down;
    float* correction = nullptr;
    // gated unit (alone, or the mixture's shared expert): gate and up rows interleaved [2 ff][W], down [W][ff]
    DenseW glu_gate_up, glu_down;
    // chunk-local sigmoid attention + fixed-decay linear attention: cl_proj rows left q | k | v | right q | k | v | g;
    // cl_o = [W][H * vdim + heads * vdim'] the two output maps side by side (one product forms the weighted sum)
    DenseW cl_proj, cl_o;
    int rq_off = 0;
    float *pb = nullptr, *decay = nullptr, *la_state = nullptr;
    // softmax attention with a sink (alone, or beside the head-decay delta rule): sk_proj rows left q | k | v | g (| right q | k | v
    // | b | a | g); reuses attn_o, sink, left_w, right_w, rot_*, k_pool, v_pool and the delta rule's st_* fields
    DenseW sk_proj;
    int gl_off = 0, ra_off = 0, rg_off = 0;
    float *sk_bias = nullptr, *talk = nullptr;
    // several copies of the stream: per sublayer (0 mixer, 1 feed-forward) read weights, mixing matrix, write weights; the
    // convolution on the sublayer's input and the last taps-1 inputs per slot
    float *hc_in[2] = {}, *hc_mix[2] = {}, *hc_out[2] = {}, *canon_w[2] = {}, *canon_state[2] = {};
    float act_p0 = 0.f, act_p1 = 0.f;          // piecewise activation: softplus(p), 1/2 + softplus(q)
};

struct StepGraph { cudaGraphExec_t exec = nullptr; int n_launch = 0; bool failed = false; };

struct LayeredModel {
    b2_layered_config c = {};
    std::vector<LyLayer> layers;
    std::vector<void*> owned;          // device allocations freed at destroy
    DenseW embed, head;
    float *final_norm = nullptr, *embed_norm = nullptr;
    bool exact = false;                // B2_FLAG_F32
    int** block_tables = nullptr;      // device [max_seqs] -> page table
    // step workspace (max_step_tokens rows)
    float *xs = nullptr, *hc = nullptr, *cross = nullptr;     // copies of the stream [S][max_step_tokens][W]; convolved sublayer input; per-(query head, value head) attention sums
    float *x = nullptr, *proj = nullptr, *buf[4] = {}, *oL = nullptr, *oR = nullptr, *hn = nullptr, *ff = nullptr, *rows = nullptr, *logits = nullptr;
    __nv_bfloat16* xb = nullptr;       // a product's input rounded to bf16 [max_step_tokens][widest input]
    std::unordered_map<std::string, StepGraph> graphs;     // replayable small steps, by shape (b2_step)
    bool graphs_on = true;
    // mixture of experts: router outputs, choices, the sorted pair table, expert activations and outputs
    float *moe_logits = nullptr, *moe_weight = nullptr, *moe_h = nullptr, *moe_y = nullptr;
    int *moe_sel = nullptr, *moe_tok = nullptr, *moe_pos = nullptr, *moe_rows = nullptr, *moe_tiles = nullptr;
    int moe_max_tiles = 0;
    float* attn_pbuf = nullptr;        // prompts with mixed heads: normalised attention weights of a group of query tiles
    size_t attn_pbuf_floats = 0;
    float* attn_split = nullptr;       // few-token steps: partial attention results per key range
    int attn_split_floats = 0;
    int* meta = nullptr;               // device ints: ragged description + wanted rows
    int* meta_host = nullptr;          // pinned
    float* logits_host = nullptr;      // pinned [LOGIT_ROWS][n_vocab]
    float* trace = nullptr;            // [n_layer][max_step_tokens][n_embd] when tracing
    int last_T = 0;
    bool profile = false;
    std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> prof_ev;
    float prof_ms[8] = {};
    int prof_n[8] = {};
};

constexpr int LOGIT_ROWS = 256;

__global__ void to_f32_kernel(int type, const void* src, long n, float* dst) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    dst[i] = type == T_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i])
           : type == T_F16 ? __half2float(reinterpret_cast<const __half*>(src)[i])
                           : reinterpret_cast<const float*>(src)[i];
}

static int dev_alloc(LayeredModel* m, void** p, size_t bytes, bool zero = false) {
    CK(cudaMalloc(p, bytes ? bytes : 16));
    m->owned.push_back(*p);
    if (zero) CK(cudaMemset(*p, 0, bytes ? bytes : 16));
    return B2_OK;
}

static int find(b2_engine* e, const std::string& name, int64_t ne0, int64_t ne1, DevTensor& out) {
    auto it = e->tensors.find(name);
    if (it == e->tensors.end()) return b2_fail(B2_ERR_STATE, "missing tensor " + name);
    const DevTensor& t = it->second;
    if (t.ne0 != ne0 || t.ne1 != ne1)
        return b2_fail(B2_ERR_ARG, "tensor " + name + " has shape [" + std::to_string(t.ne1) + "," + std::to_string(t.ne0) +
                                       "], expected [" + std::to_string(ne1) + "," + std::to_string(ne0) + "]");
    if (t.type != T_BF16 && t.type != T_F32) return b2_fail(B2_ERR_UNSUPPORTED, "tensor " + name + " must be BF16 or F32");
    out = t;
    return B2_OK;
}

// a vector (or small table) as f32 on the device, whatever the file holds
static int vec_f32(b2_engine* e, LayeredModel* m, const std::string& name, int64_t n0, int64_t n1, float** out) {
    DevTensor t;
    int rc = find(e, name, n0, n1, t); if (rc) return rc;
    const long n = (long)(n0 * n1);
    if ((rc = dev_alloc(m, (void**)out, (size_t)n * 4))) return rc;
    to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(t.type, t.ptr, n, *out);
    CK(cudaGetLastError());
    return B2_OK;
}

static int matrix(b2_engine* e, const std::string& name, int N, int K, DenseW& out) {
    DevTensor t;
    int rc = find(e, name, K, N, t); if (rc) return rc;
    out.w = t.ptr; out.type = t.type; out.N = N; out.K = K;
    return B2_OK;
}

// several matrices over the same input stacked into one [sum N][K] matrix: one product instead of several
static int fuse(b2_engine* e, LayeredModel* m, const std::vector<std::pair<std::string, int>>& parts, int K, DenseW& out,
                std::vector<int>& offs) {
    int total = 0, type = -1;
    std::vector<DevTensor> ts(parts.size());
    for (size_t i = 0; i < parts.size(); i++) {
        int rc = find(e, parts[i].first, K, parts[i].second, ts[i]); if (rc) return rc;
        if (type < 0) type = ts[i].type;
        if (ts[i].type != type) return b2_fail(B2_ERR_UNSUPPORTED, "tensor " + parts[i].first + ": projections of one input must share a dtype");
        offs.push_back(total);
        total += parts[i].second;
    }
    const size_t esz = type == T_BF16 ? 2 : 4;
    void* p = nullptr;
    int rc = dev_alloc(m, &p, (size_t)total * K * esz + 64); if (rc) return rc;
    for (size_t i = 0; i < parts.size(); i++)
        CK(cudaMemcpyAsync((char*)p + (size_t)offs[i] * K * esz, ts[i].ptr, (size_t)parts[i].second * K * esz, cudaMemcpyDeviceToDevice, e->stream));
    out.w = p; out.type = type; out.N = total; out.K = K;
    return B2_OK;
}

// W [H * d][rank] -> [H][rank][d] (elements of esz bytes): the per-head key expansion as a map applied to the query
__global__ void transpose_heads_kernel(const unsigned char* src, unsigned char* dst, int H, int d, int rank, int esz) {
    const long n = (long)H * d * rank, i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % rank), j = (int)((i / rank) % d), h = (int)(i / ((long)rank * d));
    const long o = ((long)h * rank + c) * d + j;
    for (int b = 0; b < esz; b++) dst[o * esz + b] = src[i * esz + b];
}

// several f32 tables of rows of `cols` entries one after another in one allocation
static int concat_f32(b2_engine* e, LayeredModel* m, const std::vector<std::pair<std::string, int>>& parts, int cols, float** out) {
    long rows = 0;
    for (auto& p : parts) rows += p.second;
    int rc = dev_alloc(m, (void**)out, (size_t)rows * cols * 4); if (rc) return rc;
    long at = 0;
    for (auto& p : parts) {
        DevTensor t;
        if ((rc = find(e, p.first, cols, p.second, t))) return rc;
        const long n = (long)p.second * cols;
        to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(t.type, t.ptr, n, *out + at);
        CK(cudaGetLastError());
        at += n;
    }
    return B2_OK;
}

// the experts of a layer stacked: [E][2 ff][W] with gate and up rows interleaved, and [E][W][ff]
// (names p + "<index>."); n_experts == 0: the single unit named p + "."
static int stack_experts(b2_engine* e, LayeredModel* m, const std::string& p, int n_experts, int ff, int W, DenseW& gate_up, DenseW& down) {
    int type = -1;
    void *gu = nullptr, *dn = nullptr;
    const int E = std::max(1, n_experts);
    for (int x = 0; x < E; x++) {
        DevTensor tg, tu, td;
        const std::string q = n_experts > 0 ? p + std::to_string(x) + "." : p + ".";
        int rc;
        if ((rc = find(e, q + "gate", W, ff, tg)) || (rc = find(e, q + "up", W, ff, tu)) || (rc = find(e, q + "down", ff, W, td))) return rc;
        if (type < 0) {
            type = tg.type;
            const size_t esz = type == T_BF16 ? 2 : 4;
            if ((rc = dev_alloc(m, &gu, (size_t)E * 2 * ff * W * esz + 64)) || (rc = dev_alloc(m, &dn, (size_t)E * W * ff * esz + 64))) return rc;
        }
        if (tg.type != type || tu.type != type || td.type != type) return b2_fail(B2_ERR_UNSUPPORTED, q + ": the experts of a layer must share a dtype");
        const size_t esz = type == T_BF16 ? 2 : 4, rowb = (size_t)W * esz;
        char* base = (char*)gu + (size_t)x * 2 * ff * rowb;
        CK(cudaMemcpy2DAsync(base, 2 * rowb, tg.ptr, rowb, rowb, ff, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpy2DAsync(base + rowb, 2 * rowb, tu.ptr, rowb, rowb, ff, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpyAsync((char*)dn + (size_t)x * W * ff * esz, td.ptr, (size_t)W * ff * esz, cudaMemcpyDeviceToDevice, e->stream));
    }
    gate_up.w = gu; gate_up.type = type; gate_up.N = 2 * ff; gate_up.K = W;
    down.w = dn; down.type = type; down.N = W; down.K = ff;
    return B2_OK;
}

// blended rotary frequencies (interpolated below the slow boundary, original above the fast one, linear ramp between)
// and the magnitude factor; cos / sin per position in double precision
static int build_rotary(b2_engine* e, LayeredModel* m, LyLayer& L) {
    const b2_layer_desc& d = L.d;
    const int half = d.rot_dims / 2;
    if (half <= 0) return B2_OK;
    std::vector<double> f(half);
    double mag = 1.0;
    for (int i = 0; i < half; i++) f[i] = pow((double)d.rope_base, -2.0 * i / (double)d.rot_dims);
    if (d.rope_factor > 0.0) {
        auto corr = [&](double turns) { return d.rot_dims * log((double)d.rope_orig_ctx / (2.0 * M_PI * turns)) / (2.0 * log((double)d.rope_base)); };
        const double lo = std::max(floor(corr(d.rope_fast)), 0.0), hi = std::min(ceil(corr(d.rope_slow)), (double)d.rot_dims - 1.0);
        for (int i = 0; i < half; i++) {
            double ramp = (i - lo) / std::max(hi - lo, 0.001);
            ramp = std::min(1.0, std::max(0.0, ramp));
            f[i] = f[i] / d.rope_factor * ramp + f[i] * (1.0 - ramp);
        }
        mag = 0.1 * log((double)d.rope_factor) + 1.0;
    }
    const int n_ctx = m->c.n_ctx;
    std::vector<float> cs((size_t)n_ctx * half), sn((size_t)n_ctx * half);
    for (int p = 0; p < n_ctx; p++)
        for (int i = 0; i < half; i++) {
            const double a = (double)p * f[i];
            cs[(size_t)p * half + i] = (float)(cos(a) * mag);
            sn[(size_t)p * half + i] = (float)(sin(a) * mag);
        }
    int rc;
    if ((rc = dev_alloc(m, (void**)&L.rot_cos, cs.size() * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&L.rot_sin, sn.size() * 4))) return rc;
    CK(cudaMemcpy(L.rot_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.rot_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    return B2_OK;
}

int layered_finalize(b2_engine* e) {
    LayeredModel* m = e->layered;
    const b2_layered_config& c = m->c;
    const int W = c.n_embd, V = c.n_vocab, S = c.max_seqs, Tm = c.max_step_tokens;
    CK(cudaSetDevice(c.device));
    int rc;
    if ((rc = matrix(e, "embed", V, W, m->embed))) return rc;
    if (c.tie_head) m->head = m->embed;
    else if ((rc = matrix(e, "head", V, W, m->head))) return rc;
    if ((rc = vec_f32(e, m, "final.norm", W, 1, &m->final_norm))) return rc;
    if (c.block_style == B2_BLOCK_PRENORM_RMS && (rc = vec_f32(e, m, "embed.norm", W, 1, &m->embed_norm))) return rc;
    const size_t cache_esz = m->exact ? 4 : 2;
    size_t max_proj = 1, max_buf = 1, max_ff = 1, max_attn = 0, max_attn_d = 0, max_glu = 0;
    size_t moe_pairs = 0, moe_slots = 0, moe_ff = 0, moe_experts = 0, moe_xb = 0;     // moe_xb: expert activations per step token
    const bool hyper = c.block_style == B2_BLOCK_HYPER_RMS;
    const int n_streams = std::max(1, c.n_streams);
    size_t max_cross = 0, max_pbuf = 0, max_part = 0;      // max_part: floats of one token's partial attention results with one key range
    // cache pages and recurrent state of a sink-attention layer (every run of a repeated layer has its own)
    auto sink_state = [&](LyLayer& L) -> int {
        const b2_layer_desc& d = L.d;
        int rc2;
        const size_t kpool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.head_dim * cache_esz;
        const size_t vpool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.attn_vdim * cache_esz;
        if ((rc2 = dev_alloc(m, &L.k_pool, kpool, true))) return rc2;
        if ((rc2 = dev_alloc(m, &L.v_pool, vpool, true))) return rc2;
        e->kv_bytes += (int64_t)(kpool + vpool);
        if (d.mixer == B2_MIX_SINK_DELTA) {
            if ((rc2 = dev_alloc(m, (void**)&L.st_conv_state, (size_t)S * std::max(1, d.conv_taps - 1) * L.conv_C * 4, true))) return rc2;
            if ((rc2 = dev_alloc(m, (void**)&L.st_state, (size_t)S * col_state_floats(d.mm_heads, d.mm_dim, d.mm_vdim) * 4, true))) return rc2;
        }
        return B2_OK;
    };
    auto canon_state = [&](LyLayer& L) -> int {
        for (int q = 0; q < 2; q++) {
            L.canon_state[q] = nullptr;
            if (!L.canon_w[q]) continue;
            const int rc2 = dev_alloc(m, (void**)&L.canon_state[q], (size_t)S * std::max(1, c.canon_taps - 1) * W * 4, true);
            if (rc2) return rc2;
        }
        return B2_OK;
    };
    for (int li = 0; li < c.n_layer; li++) {
        LyLayer& L = m->layers[li];
        const b2_layer_desc& d = L.d;
        const int wl = d.weights_of > 0 ? d.weights_of - 1 : li;
        const std::string p = "l" + std::to_string(wl) + ".";
        const bool sink_kind = d.mixer == B2_MIX_SINK_DELTA || d.mixer == B2_MIX_SINK_ATTN;
        if (sink_kind) {
            // a repeated run shares the weights of the first run of the same layer and gets a cache and state of its own
            int earlier = -1;
            for (int j = 0; j < li && earlier < 0; j++) if (m->layers[j].d.weights_of > 0 && m->layers[j].d.weights_of == d.weights_of) earlier = j;
            if (earlier >= 0) {
                const b2_layer_desc mine = L.d;
                L = m->layers[earlier];
                L.d = mine;
                if ((rc = sink_state(L)) || (rc = canon_state(L))) return rc;
                continue;
            }
        }
        if ((rc = vec_f32(e, m, p + "norm1", W, 1, &L.norm1))) return rc;
        if (hyper) {
            for (int q = 0; q < (d.n_ff > 0 ? 2 : 1); q++) {
                const std::string hc = p + "hc" + std::to_string(q + 1) + ".";
                if (e->tensors.count(hc + "mix")) {
                    if ((rc = vec_f32(e, m, hc + "in", n_streams, 1, &L.hc_in[q]))) return rc;
                    if ((rc = vec_f32(e, m, hc + "mix", n_streams, n_streams, &L.hc_mix[q]))) return rc;
                    if ((rc = vec_f32(e, m, hc + "out", n_streams, 1, &L.hc_out[q]))) return rc;
                } else if (n_streams > 1) return b2_fail(B2_ERR_STATE, "missing tensor " + hc + "mix");
                if (c.canon_taps > 0 && (rc = vec_f32(e, m, p + "canon" + std::to_string(q + 1), c.canon_taps, W, &L.canon_w[q]))) return rc;
            }
            if ((rc = canon_state(L))) return rc;
        }
        if (sink_kind) {
            const bool two = d.mixer == B2_MIX_SINK_DELTA;
            const std::string a = two ? p + "mix.left." : p + "mix.", b = p + "mix.right.";
            const int H = d.n_head, G = d.n_head_kv, qd = H * d.head_dim, kd = G * d.head_dim, vd = G * d.attn_vdim, od = H * d.attn_vdim;
            const int gd = (d.attn_flags & B2_ATTN_HEAD_GATE) ? H : od;
            const int Hr = d.mm_heads, rkd = d.key_heads * d.mm_dim, rvd = Hr * d.mm_vdim;
            std::vector<std::pair<std::string, int>> parts = {{a + "q", qd}, {a + "k", kd}, {a + "v", vd}, {a + "g", gd}};
            if (two) for (auto& pr : std::vector<std::pair<std::string, int>>{{b + "q", rkd}, {b + "k", rkd}, {b + "v", rvd}, {b + "b", Hr}, {b + "a", Hr}, {b + "g", rvd}}) parts.push_back(pr);
            std::vector<int> offs;
            if ((rc = fuse(e, m, parts, W, L.sk_proj, offs))) return rc;
            L.q_off = offs[0]; L.k_off = offs[1]; L.v_off = offs[2]; L.gl_off = offs[3];
            if (d.attn_flags & B2_ATTN_BIAS) {       // one bias row for the fused product; the gate has none
                if ((rc = dev_alloc(m, (void**)&L.sk_bias, (size_t)L.sk_proj.N * 4, true))) return rc;
                const std::pair<std::string, int> bs[3] = {{a + "q.b", qd}, {a + "k.b", kd}, {a + "v.b", vd}};
                for (int k = 0; k < 3; k++) {
                    DevTensor t;
                    if ((rc = find(e, bs[k].first, bs[k].second, 1, t))) return rc;
                    to_f32_kernel<<<(unsigned)((bs[k].second + 255) / 256), 256, 0, e->stream>>>(t.type, t.ptr, bs[k].second, L.sk_bias + offs[k]);
                    CK(cudaGetLastError());
                }
            }
            if (e->tensors.count(a + "sink") && (rc = vec_f32(e, m, a + "sink", H, 1, &L.sink))) return rc;
            if ((d.attn_flags & B2_ATTN_TALK) && (rc = vec_f32(e, m, a + "talk", H, H, &L.talk))) return rc;
            if ((rc = matrix(e, a + "o", W, od, L.attn_o))) return rc;
            if ((rc = build_rotary(e, m, L))) return rc;
            if (two) {
                L.conv_off = offs[4]; L.conv_C = 2 * rkd + rvd; L.b_off = offs[7]; L.ra_off = offs[8]; L.rg_off = offs[9];
                if ((rc = concat_f32(e, m, {{b + "q.conv", rkd}, {b + "k.conv", rkd}, {b + "v.conv", rvd}}, d.conv_taps, &L.st_conv_w))) return rc;
                if ((rc = vec_f32(e, m, b + "A_log", Hr, 1, &L.st_A_log))) return rc;
                if ((rc = vec_f32(e, m, b + "dt_bias", Hr, 1, &L.st_dt_bias))) return rc;
                if ((rc = vec_f32(e, m, b + "norm", d.mm_vdim, 1, &L.st_norm))) return rc;
                if ((rc = matrix(e, b + "o", W, rvd, L.st_o))) return rc;
                if ((rc = vec_f32(e, m, a + "out", W, 1, &L.left_w))) return rc;
                if ((rc = vec_f32(e, m, b + "out", W, 1, &L.right_w))) return rc;
            }
            if ((rc = sink_state(L))) return rc;
            max_proj = std::max<size_t>(max_proj, L.sk_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)qd, (size_t)od, two ? (size_t)L.conv_C : 1, two ? (size_t)rvd : 1});
            if (d.attn_flags & B2_ATTN_TALK) max_cross = std::max<size_t>(max_cross, (size_t)H * G * d.attn_vdim);
            max_part = std::max<size_t>(max_part, (size_t)H * ((d.attn_flags & B2_ATTN_TALK) ? G : 1) * (d.attn_vdim + 2));
            if ((d.attn_flags & B2_ATTN_TALK) && !m->exact) {       // all tiles of the largest step, up to 512 MB
                const size_t keys = d.window > 0 ? std::min(d.window, c.n_ctx) : c.n_ctx;
                max_pbuf = std::max<size_t>(max_pbuf, (size_t)H * 64 * ((keys + 62) / 64 + 2) * 64 * (Tm / 64 + 2));
            }
        } else if (d.mixer == B2_MIX_WINDOW_SCAN) {
            const std::string a = p + "mix.left.", b = p + "mix.right.";
            const int qd = d.n_head * d.head_dim, kd = d.n_head_kv * d.head_dim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", qd}, {a + "k", kd}, {b + "in", 2 * d.d_inner}}, W, L.in_proj, offs))) return rc;
            L.q_off = offs[0]; L.k_off = offs[1]; L.x_off = offs[2]; L.z_off = offs[2] + d.d_inner;
            if ((rc = vec_f32(e, m, a + "q.norm", d.head_dim, 1, &L.q_norm))) return rc;
            if ((rc = vec_f32(e, m, a + "k.norm", d.head_dim, 1, &L.k_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, qd, L.attn_o))) return rc;
            if ((rc = vec_f32(e, m, a + "out", W, 1, &L.left_w))) return rc;
            if ((rc = vec_f32(e, m, b + "out", W, 1, &L.right_w))) return rc;
            if ((rc = vec_f32(e, m, b + "conv", d.conv_taps, d.d_inner, &L.conv_w))) return rc;
            if ((rc = vec_f32(e, m, b + "conv.b", d.d_inner, 1, &L.conv_b))) return rc;
            if ((rc = matrix(e, b + "x", d.dt_rank + 2 * d.d_state, d.d_inner, L.scan_x))) return rc;
            if ((rc = matrix(e, b + "dt", d.d_inner, d.dt_rank, L.scan_dt))) return rc;
            if ((rc = vec_f32(e, m, b + "dt.b", d.d_inner, 1, &L.dt_b))) return rc;
            if ((rc = vec_f32(e, m, b + "A_log", d.d_state, d.d_inner, &L.A_log))) return rc;
            if ((rc = vec_f32(e, m, b + "D", d.d_inner, 1, &L.Dskip))) return rc;
            if ((rc = matrix(e, b + "o", W, d.d_inner, L.scan_o))) return rc;
            if ((rc = build_rotary(e, m, L))) return rc;
            const size_t pool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.head_dim * cache_esz;
            if ((rc = dev_alloc(m, &L.k_pool, pool, true))) return rc;
            if ((rc = dev_alloc(m, &L.v_pool, pool, true))) return rc;
            e->kv_bytes += 2 * (int64_t)pool;
            if ((rc = dev_alloc(m, (void**)&L.conv_state, (size_t)S * d.d_inner * std::max(1, d.conv_taps - 1) * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.ssm_state, (size_t)S * d.d_inner * d.d_state * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.in_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)qd, (size_t)d.d_inner, (size_t)d.dt_rank + 2 * d.d_state});
            max_attn = 1; max_attn_d = std::max<size_t>(max_attn_d, d.head_dim);
        } else if (d.mixer == B2_MIX_LATENT_ATTN) {
            const std::string a = p + "mix.";
            const int H = d.n_head, dq = d.head_dim + d.la_rot_dim, Dk = d.la_rank + d.la_rot_dim, vd = H * d.la_vdim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", H * dq}, {a + "dkv", Dk}, {a + "g", vd}}, W, L.la_proj, offs))) return rc;
            L.q_off = offs[0]; L.dkv_off = offs[1]; L.g_off = offs[2];
            if ((rc = vec_f32(e, m, a + "dkv.norm", d.la_rank, 1, &L.c_norm))) return rc;
            if ((rc = vec_f32(e, m, a + "sink", H, 1, &L.sink))) return rc;
            DenseW uk;
            if ((rc = matrix(e, a + "uk", H * d.head_dim, d.la_rank, uk))) return rc;
            {
                const size_t esz = uk.type == T_BF16 ? 2 : 4;
                void* tp = nullptr;
                if ((rc = dev_alloc(m, &tp, (size_t)H * d.head_dim * d.la_rank * esz + 64))) return rc;
                const long n = (long)H * d.head_dim * d.la_rank;
                transpose_heads_kernel<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>((const unsigned char*)uk.w, (unsigned char*)tp, H, d.head_dim, d.la_rank, (int)esz);
                CK(cudaGetLastError());
                L.uk_t.w = tp; L.uk_t.type = uk.type; L.uk_t.N = d.la_rank; L.uk_t.K = d.head_dim;
            }
            if ((rc = matrix(e, a + "uv", H * d.la_vdim, d.la_rank, L.uv))) return rc;
            L.uv.N = d.la_vdim;                       // applied head by head
            if ((rc = matrix(e, a + "o", W, vd, L.attn_o))) return rc;
            if ((rc = build_rotary(e, m, L))) return rc;
            const size_t pool = (size_t)c.kv_num_blocks * c.kv_block_tokens * Dk * cache_esz;
            if ((rc = dev_alloc(m, &L.la_pool, pool, true))) return rc;
            e->kv_bytes += (int64_t)pool;
            max_proj = std::max<size_t>(max_proj, L.la_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)H * Dk, (size_t)H * dq, (size_t)vd});
            max_attn = 1; max_attn_d = std::max<size_t>(max_attn_d, d.la_rank);
        } else if (d.mixer == B2_MIX_CHUNK_LINEAR) {
            const std::string a = p + "mix.left.", b = p + "mix.right.";
            const int qd = d.n_head * d.head_dim, kd = d.n_head_kv * d.head_dim, vd = d.n_head_kv * d.attn_vdim, od = d.n_head * d.attn_vdim;
            const int rqd = d.mm_heads * d.mm_dim, rvd = d.mm_heads * d.mm_vdim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", qd}, {a + "k", kd}, {a + "v", vd}, {b + "q", rqd}, {b + "k", rqd}, {b + "v", rvd}, {b + "g", rvd}}, W,
                           L.cl_proj, offs))) return rc;
            L.q_off = offs[0]; L.k_off = offs[1]; L.v_off = offs[2]; L.rq_off = offs[3]; L.g_off = offs[6];
            if ((rc = vec_f32(e, m, a + "q.norm", qd, 1, &L.q_norm))) return rc;
            if ((rc = vec_f32(e, m, a + "k.norm", kd, 1, &L.k_norm))) return rc;
            if ((rc = vec_f32(e, m, a + "pb", d.n_head, 1, &L.pb))) return rc;
            if ((rc = vec_f32(e, m, b + "norm", rvd, 1, &L.mm_norm))) return rc;
            if ((rc = vec_f32(e, m, b + "decay", d.mm_heads, 1, &L.decay))) return rc;
            {   // the two output maps side by side: [W][od + rvd]
                DevTensor tl, tr;
                if ((rc = find(e, a + "o", od, W, tl)) || (rc = find(e, b + "o", rvd, W, tr))) return rc;
                if (tl.type != tr.type) return b2_fail(B2_ERR_UNSUPPORTED, a + "o: the two output maps must share a dtype");
                const size_t esz = tl.type == T_BF16 ? 2 : 4, Kt = (size_t)od + rvd;
                void* cat = nullptr;
                if ((rc = dev_alloc(m, &cat, (size_t)W * Kt * esz + 64))) return rc;
                CK(cudaMemcpy2DAsync(cat, Kt * esz, tl.ptr, od * esz, od * esz, W, cudaMemcpyDeviceToDevice, e->stream));
                CK(cudaMemcpy2DAsync((char*)cat + od * esz, Kt * esz, tr.ptr, rvd * esz, rvd * esz, W, cudaMemcpyDeviceToDevice, e->stream));
                L.cl_o.w = cat; L.cl_o.type = tl.type; L.cl_o.N = W; L.cl_o.K = (int)Kt;
            }
            const size_t kpool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.head_dim * cache_esz;
            const size_t vpool = (size_t)c.kv_num_blocks * d.n_head_kv * c.kv_block_tokens * d.attn_vdim * cache_esz;
            if ((rc = dev_alloc(m, &L.k_pool, kpool, true))) return rc;
            if ((rc = dev_alloc(m, &L.v_pool, vpool, true))) return rc;
            e->kv_bytes += (int64_t)(kpool + vpool);
            if ((rc = dev_alloc(m, (void**)&L.la_state, (size_t)S * col_state_floats(d.mm_heads, d.mm_dim, d.mm_vdim) * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.cl_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)qd, (size_t)od + rvd});
        } else if (d.mixer == B2_MIX_DELTA_RULE) {
            const std::string a = p + "mix.";
            const int H = d.mm_heads, G = d.key_heads, kd = G * d.mm_dim, vd = H * d.mm_vdim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", kd}, {a + "k", kd}, {a + "v", vd}, {a + "b", H}, {a + "a1", d.rank_a}, {a + "g1", d.rank_g}}, W, L.st_proj, offs))) return rc;
            L.q_off = offs[0]; L.k_off = offs[1]; L.v_off = offs[2]; L.b_off = offs[3]; L.a1_off = offs[4]; L.g1_off = offs[5];
            L.conv_off = 0; L.conv_C = 2 * kd + vd;
            if ((rc = concat_f32(e, m, {{a + "q.conv", kd}, {a + "k.conv", kd}, {a + "v.conv", vd}}, d.conv_taps, &L.st_conv_w))) return rc;
            if ((rc = matrix(e, a + "a2", H * d.mm_dim, d.rank_a, L.a2))) return rc;
            if ((rc = matrix(e, a + "g2", vd, d.rank_g, L.g2))) return rc;
            if (L.a2.type == L.g2.type) {      // one product for both second steps: zeros off the diagonal blocks add nothing
                const size_t esz = L.a2.type == T_BF16 ? 2 : 4;
                const int Ka = d.rank_a, Kg = d.rank_g, Kt = Ka + Kg, Na = H * d.mm_dim;
                void* bd = nullptr;
                if ((rc = dev_alloc(m, &bd, (size_t)(Na + vd) * Kt * esz + 64, true))) return rc;
                CK(cudaMemcpy2DAsync(bd, Kt * esz, L.a2.w, Ka * esz, Ka * esz, Na, cudaMemcpyDeviceToDevice, e->stream));
                CK(cudaMemcpy2DAsync((char*)bd + ((size_t)Na * Kt + Ka) * esz, Kt * esz, L.g2.w, Kg * esz, Kg * esz, vd, cudaMemcpyDeviceToDevice, e->stream));
                L.ag.w = bd; L.ag.type = L.a2.type; L.ag.N = Na + vd; L.ag.K = Kt;
            }
            if ((rc = vec_f32(e, m, a + "A_log", H, 1, &L.st_A_log))) return rc;
            if ((rc = vec_f32(e, m, a + "dt_bias", H * d.mm_dim, 1, &L.st_dt_bias))) return rc;
            if ((rc = vec_f32(e, m, a + "norm", d.mm_vdim, 1, &L.st_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, vd, L.st_o))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.st_conv_state, (size_t)S * std::max(1, d.conv_taps - 1) * L.conv_C * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.st_state, (size_t)S * col_state_floats(H, d.mm_dim, d.mm_vdim) * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.st_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)L.conv_C, (size_t)H * d.mm_dim + vd});
        } else if (d.mixer == B2_MIX_SSD) {
            const std::string a = p + "mix.";
            const int H = d.mm_heads, inner = H * d.mm_vdim, gn = d.key_heads * d.d_state;
            if ((rc = matrix(e, a + "in", 2 * inner + 2 * gn + H, W, L.st_proj))) return rc;
            L.conv_off = inner; L.conv_C = inner + 2 * gn; L.dt_off = 2 * inner + 2 * gn;
            if ((rc = vec_f32(e, m, a + "conv", d.conv_taps, L.conv_C, &L.st_conv_w))) return rc;
            if ((rc = vec_f32(e, m, a + "conv.b", L.conv_C, 1, &L.st_conv_b))) return rc;
            if ((rc = vec_f32(e, m, a + "dt_bias", H, 1, &L.st_dt_bias))) return rc;
            if ((rc = vec_f32(e, m, a + "A_log", H, 1, &L.st_A_log))) return rc;
            if ((rc = vec_f32(e, m, a + "D", H, 1, &L.st_D))) return rc;
            if ((rc = vec_f32(e, m, a + "norm", inner, 1, &L.st_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, inner, L.st_o))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.st_conv_state, (size_t)S * std::max(1, d.conv_taps - 1) * L.conv_C * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.st_state, (size_t)S * col_state_floats(H, d.d_state, d.mm_vdim) * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.st_proj.N);
            max_buf = std::max<size_t>({max_buf, (size_t)L.conv_C, (size_t)inner, (size_t)H});
        } else {
            const std::string a = p + "mix.";
            const int qd = d.mm_heads * d.mm_dim, vd = d.mm_heads * d.mm_vdim;
            std::vector<int> offs;
            if ((rc = fuse(e, m, {{a + "q", qd}, {a + "k", qd}, {a + "v", vd}, {a + "g", vd}, {a + "i", d.mm_heads}, {a + "f", d.mm_heads}}, W, L.mm_proj, offs))) return rc;
            L.mq = offs[0]; L.mk = offs[1]; L.mv = offs[2]; L.mg = offs[3]; L.mi = offs[4]; L.mf = offs[5];
            if ((rc = vec_f32(e, m, a + "i.b", d.mm_heads, 1, &L.i_b))) return rc;
            if ((rc = vec_f32(e, m, a + "f.b", d.mm_heads, 1, &L.f_b))) return rc;
            if ((rc = vec_f32(e, m, a + "norm", vd, 1, &L.mm_norm))) return rc;
            if ((rc = matrix(e, a + "o", W, vd, L.mm_o))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.S, (size_t)S * d.mm_heads * d.mm_dim * d.mm_vdim * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.nvec, (size_t)S * d.mm_heads * d.mm_dim * 4, true))) return rc;
            if ((rc = dev_alloc(m, (void**)&L.mmax, (size_t)S * d.mm_heads * 4, true))) return rc;
            max_proj = std::max<size_t>(max_proj, L.mm_proj.N);
            max_buf = std::max<size_t>(max_buf, (size_t)vd);
        }
        if (d.n_ff > 0 && d.ff_kind == B2_FF_MOE) {
            const int slots = d.moe_experts + d.moe_identity;
            if ((rc = vec_f32(e, m, p + "norm2", W, 1, &L.norm2))) return rc;
            if ((rc = matrix(e, p + "mlp.router", slots, W, L.router))) return rc;
            const std::string cn = p + (d.moe_route == B2_ROUTE_TOPK_SOFTMAX ? "mlp.router.b" : "mlp.correction");
            if ((!hyper || e->tensors.count(cn)) && (rc = vec_f32(e, m, cn, slots, 1, &L.correction))) return rc;
            if ((rc = stack_experts(e, m, p + "mlp.e", d.moe_experts, d.n_ff, W, L.gate_up, L.e_down))) return rc;
            if (d.moe_shared_ff > 0) {
                if ((rc = stack_experts(e, m, p + "mlp.shared", 0, d.moe_shared_ff, W, L.glu_gate_up, L.glu_down))) return rc;
                max_glu = std::max<size_t>(max_glu, d.moe_shared_ff);
            }
            moe_pairs = std::max<size_t>(moe_pairs, (size_t)Tm * d.moe_top);
            moe_slots = std::max<size_t>(moe_slots, slots);
            moe_ff = std::max<size_t>(moe_ff, d.n_ff);
            moe_xb = std::max<size_t>(moe_xb, (size_t)d.moe_top * d.n_ff);
            moe_experts = std::max<size_t>(moe_experts, d.moe_experts);
        } else if (d.n_ff > 0 && d.ff_kind == B2_FF_PIECEWISE) {
            float* act = nullptr;
            float host[2] = {0.f, 0.f};
            if ((rc = vec_f32(e, m, p + "norm2", W, 1, &L.norm2))) return rc;
            if ((rc = matrix(e, p + "mlp.up", d.n_ff, W, L.up))) return rc;
            if ((rc = matrix(e, p + "mlp.down", W, d.n_ff, L.down))) return rc;
            if ((rc = vec_f32(e, m, p + "mlp.act", 2, 1, &act))) return rc;
            CK(cudaStreamSynchronize(e->stream));
            CK(cudaMemcpy(host, act, 8, cudaMemcpyDeviceToHost));
            auto softplus = [](double z) { return z > 0.0 ? z + log1p(exp(-z)) : log1p(exp(z)); };
            L.act_p0 = (float)softplus(host[0]); L.act_p1 = (float)(0.5 + softplus(host[1]));
            max_ff = std::max<size_t>(max_ff, d.n_ff);
        } else if (d.n_ff > 0 && d.ff_kind == B2_FF_GLU) {
            if ((rc = vec_f32(e, m, p + "norm2", W, 1, &L.norm2))) return rc;
            if ((rc = stack_experts(e, m, p + "mlp", 0, d.n_ff, W, L.glu_gate_up, L.glu_down))) return rc;
            max_glu = std::max<size_t>(max_glu, d.n_ff);
        } else if (d.n_ff > 0) {
            if ((rc = vec_f32(e, m, p + "norm2", W, 1, &L.norm2))) return rc;
            if ((rc = matrix(e, p + "mlp.up", d.n_ff, W, L.up))) return rc;
            if ((rc = vec_f32(e, m, p + "mlp.up.b", d.n_ff, 1, &L.up_b))) return rc;
            if ((rc = matrix(e, p + "mlp.down", W, d.n_ff, L.down))) return rc;
            if ((rc = vec_f32(e, m, p + "mlp.down.b", W, 1, &L.down_b))) return rc;
            max_ff = std::max<size_t>(max_ff, d.n_ff);
        }
    }
    if ((rc = dev_alloc(m, (void**)&m->x, (size_t)Tm * W * 4))) return rc;
    if (hyper) {
        if ((rc = dev_alloc(m, (void**)&m->xs, (size_t)n_streams * Tm * W * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->hc, (size_t)Tm * W * 4))) return rc;
        if (max_cross > 0 && (rc = dev_alloc(m, (void**)&m->cross, (size_t)Tm * max_cross * 4))) return rc;
        if (max_pbuf > 0) {
            m->attn_pbuf_floats = std::min<size_t>(max_pbuf, (size_t)128 << 20);
            if ((rc = dev_alloc(m, (void**)&m->attn_pbuf, m->attn_pbuf_floats * 4))) return rc;
        }
    }
    if ((rc = dev_alloc(m, (void**)&m->proj, (size_t)Tm * max_proj * 4))) return rc;
    for (int i = 0; i < 4; i++) if ((rc = dev_alloc(m, (void**)&m->buf[i], (size_t)Tm * max_buf * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->oL, (size_t)Tm * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->oR, (size_t)Tm * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->hn, (size_t)Tm * W * 4))) return rc;
    max_ff = std::max(max_ff, max_glu);
    if ((rc = dev_alloc(m, (void**)&m->ff, (size_t)Tm * max_ff * 4))) return rc;
    if (!m->exact && (rc = dev_alloc(m, (void**)&m->xb, (size_t)(Tm + B2_STEP_MAX_ENTRIES) * std::max<size_t>({max_buf, max_ff, (size_t)W, moe_xb}) * 2 + 64))) return rc;
    if (max_part > 0) {                      // sink attention: up to 8 tokens x 16 key ranges
        m->attn_split_floats = (int)std::min<size_t>(max_part * 8 * 16, (size_t)1 << 28);
        if ((rc = dev_alloc(m, (void**)&m->attn_split, (size_t)m->attn_split_floats * 4))) return rc;
    } else if (max_attn > 0) {
        m->attn_split_floats = (int)(148 * 2 * (max_attn_d + 2));       // T * H * splits <= 2 * 148 on the split path
        if ((rc = dev_alloc(m, (void**)&m->attn_split, (size_t)m->attn_split_floats * 4))) return rc;
    }
    if (moe_pairs > 0) {
        m->moe_max_tiles = (int)(moe_pairs / 64 + moe_experts + 1);
        if ((rc = dev_alloc(m, (void**)&m->moe_logits, (size_t)Tm * moe_slots * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_weight, moe_pairs * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_sel, moe_pairs * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_tok, moe_pairs * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_pos, moe_pairs * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_rows, moe_pairs * 4, true))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_tiles, (size_t)(3 * m->moe_max_tiles + 1) * 4, true))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_h, moe_pairs * moe_ff * 4))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->moe_y, moe_pairs * W * 4))) return rc;
    }
    if ((rc = dev_alloc(m, (void**)&m->rows, (size_t)LOGIT_ROWS * W * 4))) return rc;
    if ((rc = dev_alloc(m, (void**)&m->logits, (size_t)LOGIT_ROWS * V * 4))) return rc;
    const size_t n_meta = (size_t)4 * Tm + 2 * (Tm / 64 + B2_STEP_MAX_ENTRIES) + 5 * B2_STEP_MAX_ENTRIES + 64;
    if ((rc = dev_alloc(m, (void**)&m->meta, n_meta * 4))) return rc;
    CK(cudaMallocHost(&m->meta_host, n_meta * 4));
    CK(cudaMallocHost(&m->logits_host, (size_t)LOGIT_ROWS * V * 4));
    {
        std::vector<int*> tabs(S);
        for (int i = 0; i < S; i++) tabs[i] = e->slots[i].block_table;
        if ((rc = dev_alloc(m, (void**)&m->block_tables, sizeof(int*) * S))) return rc;
        CK(cudaMemcpy(m->block_tables, tabs.data(), sizeof(int*) * S, cudaMemcpyHostToDevice));
    }
    CK(cudaStreamSynchronize(e->stream));
    e->finalized = true;
    return B2_OK;
}

void layered_destroy(b2_engine* e) {
    LayeredModel* m = e->layered;
    if (!m) return;
    for (void* p : m->owned) cudaFree(p);
    if (m->meta_host) cudaFreeHost(m->meta_host);
    if (m->logits_host) cudaFreeHost(m->logits_host);
    for (auto& pe : m->prof_ev) { cudaEventDestroy(pe.second.first); cudaEventDestroy(pe.second.second); }
    for (auto& kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    delete m;
    e->layered = nullptr;
}

// a slot starts a new sequence: its recurrent state goes back to zero (cache pages are simply overwritten)
int layered_seq_reset(b2_engine* e, int slot) {
    LayeredModel* m = e->layered;
    for (auto& L : m->layers) {
        const b2_layer_desc& d = L.d;
        for (int q = 0; q < 2; q++)
            if (L.canon_state[q]) {
                const size_t cs = (size_t)std::max(1, m->c.canon_taps - 1) * m->c.n_embd;
                CK(cudaMemsetAsync(L.canon_state[q] + slot * cs, 0, cs * 4, e->stream));
            }
        if (d.mixer == B2_MIX_SINK_ATTN) {
            // nothing but cache pages, which are overwritten
        } else if (d.mixer == B2_MIX_SINK_DELTA) {
            const size_t cs = (size_t)std::max(1, d.conv_taps - 1) * L.conv_C, ss = col_state_floats(d.mm_heads, d.mm_dim, d.mm_vdim);
            CK(cudaMemsetAsync(L.st_conv_state + slot * cs, 0, cs * 4, e->stream));
            CK(cudaMemsetAsync(L.st_state + slot * ss, 0, ss * 4, e->stream));
        } else if (d.mixer == B2_MIX_WINDOW_SCAN) {
            const size_t cs = (size_t)d.d_inner * std::max(1, d.conv_taps - 1), ss = (size_t)d.d_inner * d.d_state;
            CK(cudaMemsetAsync(L.conv_state + slot * cs, 0, cs * 4, e->stream));
            CK(cudaMemsetAsync(L.ssm_state + slot * ss, 0, ss * 4, e->stream));
        } else if (d.mixer == B2_MIX_LATENT_ATTN) {
            // nothing but cache pages, which are overwritten
        } else if (d.mixer == B2_MIX_CHUNK_LINEAR) {
            const size_t ss = col_state_floats(d.mm_heads, d.mm_dim, d.mm_vdim);
            CK(cudaMemsetAsync(L.la_state + slot * ss, 0, ss * 4, e->stream));
        } else if (d.mixer == B2_MIX_DELTA_RULE || d.mixer == B2_MIX_SSD) {
            const size_t cs = (size_t)std::max(1, d.conv_taps - 1) * L.conv_C;
            const size_t ss = col_state_floats(d.mm_heads, d.mixer == B2_MIX_SSD ? d.d_state : d.mm_dim, d.mm_vdim);
            CK(cudaMemsetAsync(L.st_conv_state + slot * cs, 0, cs * 4, e->stream));
            CK(cudaMemsetAsync(L.st_state + slot * ss, 0, ss * 4, e->stream));
        } else {
            const size_t s1 = (size_t)d.mm_heads * d.mm_dim * d.mm_vdim, s2 = (size_t)d.mm_heads * d.mm_dim;
            CK(cudaMemsetAsync(L.S + slot * s1, 0, s1 * 4, e->stream));
            CK(cudaMemsetAsync(L.nvec + slot * s2, 0, s2 * 4, e->stream));
            CK(cudaMemsetAsync(L.mmax + slot * d.mm_heads, 0, (size_t)d.mm_heads * 4, e->stream));
        }
    }
    return B2_OK;
}

}  // namespace b2

// ------------------------------------------------------------------------------------------ C ABI
extern "C" int b2_engine_create_layered(const b2_layered_config* c, const b2_layer_desc* layers, b2_engine** out) {
    if (!c || !layers || !out) return b2_fail(B2_ERR_ARG, "null argument");
    if (c->n_layer <= 0 || c->n_embd <= 0 || c->n_vocab <= 0 || c->n_ctx <= 0 || c->max_seqs <= 0 || c->kv_block_tokens <= 0 ||
        c->kv_num_blocks <= 0 || c->max_step_tokens <= 0)
        return b2_fail(B2_ERR_ARG, "bad model/config dimensions");
    if (c->max_seqs > B2_STEP_MAX_ENTRIES) return b2_fail(B2_ERR_ARG, "at most 64 sequence slots");
    for (int i = 0; i < c->n_layer; i++) {
        const b2_layer_desc& d = layers[i];
        const std::string li = "layer " + std::to_string(i) + ": ";
        if (d.n_ff < 0) return b2_fail(B2_ERR_ARG, li + "negative feed-forward width");
        if (d.mixer == B2_MIX_WINDOW_SCAN) {
            if (d.n_head <= 0 || d.n_head_kv <= 0 || d.n_head % d.n_head_kv || d.head_dim <= 0) return b2_fail(B2_ERR_ARG, li + "bad head counts");
            if (d.head_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "head size above 256");
            if (d.rot_dims < 0 || d.rot_dims > d.head_dim || d.rot_dims % 2) return b2_fail(B2_ERR_ARG, li + "rotary dims must be even and <= the head size");
            if (d.window <= 0 || d.keep_first < 0) return b2_fail(B2_ERR_ARG, li + "bad window");
            if (d.conv_taps <= 0 || d.conv_taps > 64 || d.dt_rank <= 0 || d.d_inner <= 0 || d.d_state <= 0) return b2_fail(B2_ERR_ARG, li + "bad scan sizes");
            if (d.d_state > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "scan state above 256");
        } else if (d.mixer == B2_MIX_MATRIX_MEMORY) {
            if (d.mm_heads <= 0 || d.mm_dim <= 0 || d.mm_vdim <= 0 || !(d.gate_cap > 0.0)) return b2_fail(B2_ERR_ARG, li + "bad matrix-memory sizes");
            if (d.mm_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "matrix-memory key size above 256");
        } else if (d.mixer == B2_MIX_LATENT_ATTN) {
            if (d.n_head <= 0 || d.head_dim <= 0 || d.la_rot_dim < 0 || d.la_vdim <= 0 || d.la_rank <= 0) return b2_fail(B2_ERR_ARG, li + "bad latent-attention sizes");
            if (d.rot_dims < 0 || d.rot_dims > d.la_rot_dim || d.rot_dims % 2) return b2_fail(B2_ERR_ARG, li + "rotary dims must be even and <= the rotated part");
            if (d.la_rank + d.la_rot_dim > 640) return b2_fail(B2_ERR_UNSUPPORTED, li + "latent + rotated key part above 640");
        } else if (d.mixer == B2_MIX_DELTA_RULE) {
            if (d.mm_heads <= 0 || d.key_heads <= 0 || d.mm_heads % d.key_heads || d.mm_dim <= 0 || d.mm_vdim <= 0 || d.rank_a <= 0 || d.rank_g <= 0 ||
                d.conv_taps <= 0 || d.conv_taps > 64)
                return b2_fail(B2_ERR_ARG, li + "bad delta-rule sizes");
            if (d.mm_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "delta-rule key size above 256");
        } else if (d.mixer == B2_MIX_SSD) {
            if (d.mm_heads <= 0 || d.key_heads <= 0 || d.mm_heads % d.key_heads || d.d_state <= 0 || d.mm_vdim <= 0 || d.conv_taps <= 0 || d.conv_taps > 64 ||
                d.norm_groups <= 0 || (d.mm_heads * d.mm_vdim) % d.norm_groups)
                return b2_fail(B2_ERR_ARG, li + "bad state-space sizes");
            if (d.d_state > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "state size above 256");
        } else if (d.mixer == B2_MIX_CHUNK_LINEAR) {
            if (d.n_head <= 0 || d.n_head_kv <= 0 || d.n_head % d.n_head_kv || d.head_dim <= 0 || d.attn_vdim <= 0) return b2_fail(B2_ERR_ARG, li + "bad head counts");
            if (d.head_dim > 256 || d.attn_vdim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "key or value size above 256");
            if (d.mm_heads <= 0 || d.mm_dim <= 0 || d.mm_vdim <= 0) return b2_fail(B2_ERR_ARG, li + "bad linear-attention sizes");
            if (d.mm_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "linear-attention key size above 256");
        } else if (d.mixer == B2_MIX_SINK_DELTA || d.mixer == B2_MIX_SINK_ATTN) {
            if (d.n_head <= 0 || d.n_head_kv <= 0 || d.n_head % d.n_head_kv || d.head_dim <= 0 || d.attn_vdim <= 0) return b2_fail(B2_ERR_ARG, li + "bad head counts");
            if (d.head_dim > 256 || d.attn_vdim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "key or value size above 256");
            if (d.rot_dims < 0 || d.rot_dims > d.head_dim || d.rot_dims % 2) return b2_fail(B2_ERR_ARG, li + "rotary dims must be even and <= the head size");
            if (d.mixer == B2_MIX_SINK_DELTA) {
                if (d.mm_heads <= 0 || d.key_heads <= 0 || d.mm_heads % d.key_heads || d.mm_dim <= 0 || d.mm_vdim <= 0 || d.conv_taps <= 0 || d.conv_taps > 64)
                    return b2_fail(B2_ERR_ARG, li + "bad delta-rule sizes");
                if (d.mm_dim > 256) return b2_fail(B2_ERR_UNSUPPORTED, li + "delta-rule key size above 256");
            }
            if (c->block_style != B2_BLOCK_HYPER_RMS) return b2_fail(B2_ERR_UNSUPPORTED, li + "this mixer belongs to blocks with stream copies");
        } else return b2_fail(B2_ERR_UNSUPPORTED, li + "unknown mixer kind");
        if (d.weights_of < 0 || d.weights_of > c->n_layer) return b2_fail(B2_ERR_ARG, li + "weights_of out of range");
        if (d.n_ff > 0 && d.ff_kind == B2_FF_MOE) {
            const int slots = d.moe_experts + d.moe_identity;
            if (d.moe_experts <= 0 || d.moe_identity < 0 || d.moe_top <= 0 || d.moe_top > slots || d.moe_groups <= 0 || slots % d.moe_groups ||
                d.moe_keep <= 0 || d.moe_keep > d.moe_groups || d.moe_top > d.moe_keep * (slots / d.moe_groups))
                return b2_fail(B2_ERR_ARG, li + "bad mixture-of-experts sizes");
            if (slots > 4096) return b2_fail(B2_ERR_UNSUPPORTED, li + "more than 4096 expert slots");
            if (d.moe_route != B2_ROUTE_SOFTMAX_ALL && d.moe_route != B2_ROUTE_TOPK_SOFTMAX) return b2_fail(B2_ERR_ARG, li + "unknown routing rule");
            if (d.moe_route == B2_ROUTE_TOPK_SOFTMAX && (d.moe_identity > 0 || d.moe_groups > 1)) return b2_fail(B2_ERR_UNSUPPORTED, li + "top-k softmax routing has no identity slots or groups");
            if (d.moe_shared_ff < 0) return b2_fail(B2_ERR_ARG, li + "negative shared-expert width");
            if (d.moe_expert != B2_EXPERT_SILU && d.moe_expert != B2_EXPERT_CLAMPED) return b2_fail(B2_ERR_ARG, li + "unknown expert kind");
            if (d.moe_expert == B2_EXPERT_CLAMPED && !(d.moe_limit > 0.0)) return b2_fail(B2_ERR_ARG, li + "a clamped expert needs a positive limit");
        } else if (d.ff_kind != B2_FF_RELU2 && d.ff_kind != B2_FF_GLU && d.ff_kind != B2_FF_PIECEWISE) return b2_fail(B2_ERR_UNSUPPORTED, li + "unknown feed-forward kind");
        if (c->block_style == B2_BLOCK_PRENORM_RMS ? (d.mixer == B2_MIX_WINDOW_SCAN) : false)
            return b2_fail(B2_ERR_UNSUPPORTED, li + "the two-branch mixer belongs to post-sum blocks");
    }
    if (c->block_style != B2_BLOCK_POSTSUM_LN && c->block_style != B2_BLOCK_PRENORM_RMS && c->block_style != B2_BLOCK_OUTNORM_RMS &&
        c->block_style != B2_BLOCK_HYPER_RMS)
        return b2_fail(B2_ERR_ARG, "unknown block style");
    if (c->block_style == B2_BLOCK_HYPER_RMS) {
        if (c->n_streams < 0 || c->n_streams > 16) return b2_fail(B2_ERR_UNSUPPORTED, "at most 16 copies of the stream");
        if (c->canon_taps < 0 || c->canon_taps > 64) return b2_fail(B2_ERR_ARG, "bad number of taps");
        for (int i = 0; i < c->n_layer; i++)
            if (layers[i].mixer != B2_MIX_SINK_DELTA && layers[i].mixer != B2_MIX_SINK_ATTN)
                return b2_fail(B2_ERR_UNSUPPORTED, "layer " + std::to_string(i) + ": blocks with stream copies take the sink-attention mixers");
    }
    if (c->block_style == B2_BLOCK_OUTNORM_RMS && (c->norm_groups < 0 || (c->norm_groups > 0 && c->n_embd % c->norm_groups)))
        return b2_fail(B2_ERR_ARG, "the norm's parts must divide the width");
    b2_engine* e = new b2_engine();
    b2_config& b = e->cfg;
    memset(&b, 0, sizeof(b));
    b.n_layer = c->n_layer; b.n_embd = c->n_embd; b.n_vocab = c->n_vocab; b.rms_eps = c->norm_eps; b.n_ctx = c->n_ctx;
    b.max_seqs = c->max_seqs; b.kv_block_tokens = c->kv_block_tokens; b.kv_num_blocks = c->kv_num_blocks; b.device = c->device;
    b.flags = c->flags;
    LayeredModel* m = new LayeredModel();
    m->c = *c;
    m->exact = (c->flags & B2_FLAG_F32) != 0;
    m->layers.resize(c->n_layer);
    for (int i = 0; i < c->n_layer; i++) m->layers[i].d = layers[i];
    e->layered = m;
    e->use_graph = !(c->flags & B2_FLAG_NO_GRAPH) && !getenv("B2_NO_GRAPH");
    m->graphs_on = e->use_graph;
    e->use_pdl = e->chain_pdl = !(c->flags & B2_FLAG_NO_PDL) && !getenv("B2_NO_CHAIN_PDL");
    auto init = [&]() -> int {
        CK(cudaSetDevice(c->device));
        cudaDeviceGetAttribute(&e->n_sms, cudaDevAttrMultiProcessorCount, c->device);
        CK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
        CK(cudaEventCreate(&e->ev0));
        CK(cudaEventCreate(&e->ev1));
        CK(cudaMallocHost(&e->pinned, sizeof(int32_t) * (size_t)(c->max_seqs + B2_STEP_MAX_ENTRIES + 16)));
        e->max_blocks = (c->n_ctx + c->kv_block_tokens - 1) / c->kv_block_tokens;
        e->slots.resize(c->max_seqs);
        for (auto& s : e->slots) {
            CK(cudaMalloc(&s.logits, sizeof(float) * c->n_vocab));
            CK(cudaMalloc(&s.ints, sizeof(int) * 8));
            CK(cudaMemset(s.ints, 0, sizeof(int) * 8));
            CK(cudaMalloc(&s.block_table, sizeof(int) * e->max_blocks));
            CK(cudaMemset(s.block_table, 0, sizeof(int) * e->max_blocks));
            CK(cudaMalloc(&s.ring, sizeof(int) * (c->n_ctx + 1)));
            CK(cudaMemset(s.ring, 0, sizeof(int) * (c->n_ctx + 1)));
            CK(cudaMalloc(&s.sst, sizeof(SamplerState)));
            CK(cudaMemset(s.sst, 0, sizeof(SamplerState)));
            CK(cudaMalloc(&s.sp, sizeof(SampleParams)));
            CK(cudaMemset(s.sp, 0, sizeof(SampleParams)));
            CK(cudaMalloc(&s.uniforms, sizeof(double) * 8192));
            CK(cudaMemset(s.uniforms, 0, sizeof(double) * 8192));
        }
        return B2_OK;
    };
    const int rc = init();
    if (rc) { b2_engine_destroy(e); return rc; }
    *out = e;
    return B2_OK;
}

namespace {
struct StepProfiler {                 // events around launches of one kind, only when profiling is on
    LayeredModel* m; cudaStream_t st; cudaEvent_t b = nullptr;
    int kind;
    StepProfiler(LayeredModel* m_, cudaStream_t s, int k) : m(m_), st(s), kind(k) {
        if (!m->profile) return;
        cudaEvent_t a; cudaEventCreate(&a); cudaEventCreate(&b);
        cudaEventRecord(a, st);
        m->prof_ev.push_back({kind, {a, b}});
    }
    ~StepProfiler() { if (b) cudaEventRecord(b, st); }
};
}  // namespace

static int dense(b2_engine* e, LayeredModel* m, const DenseW& w, const float* x, int ldx, float* y, int ldy, int T,
                 const float* bias = nullptr, int epi = EPI_NONE, int kind = 1, DenseArgs* more = nullptr) {
    StepProfiler sp(m, e->stream, kind);
    DenseArgs a = more ? *more : DenseArgs{};
    a.x = x; a.ldx = ldx; a.w = w.w; a.w_type = w.type; a.bias = bias; a.y = y; a.ldy = ldy; a.T = T; a.N = w.N; a.K = w.K;
    a.epi = epi; a.exact = m->exact || (more && more->exact); a.xb = m->xb;
    CK(dense_launch(a, e->stream));
    e->launches++;
    return B2_OK;
}

// ---- token mixers: each reads the sublayer input `in` [T][W] and leaves its output in m->oL (the two-branch mixer also m->oR)
static int mix_window_scan(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd;
    int rc;
    const int Np = L.in_proj.N, qd = d.n_head * d.head_dim;
    if ((rc = dense(e, m, L.in_proj, in, W, m->proj, Np, T))) return rc;
    WindowAttnArgs a = {};
    a.proj = m->proj; a.ldp = Np; a.q_off = L.q_off; a.k_off = L.k_off; a.q_norm_w = L.q_norm; a.k_norm_w = L.k_norm;
    a.rot.cos = L.rot_cos; a.rot.sin = L.rot_sin; a.rot.rot_dims = d.rot_dims;
    a.k_pool = L.k_pool; a.v_pool = L.v_pool; a.cache_f32 = m->exact ? 1 : 0; a.block_tables = m->block_tables;
    a.block_tokens = c.kv_block_tokens; a.H = d.n_head; a.G = d.n_head_kv; a.d = d.head_dim; a.window = d.window;
    a.keep_first = d.keep_first; a.scale = (float)d.attn_scale; a.eps = c.norm_eps; a.q_rot = m->buf[0]; a.out = m->buf[1];
    a.split_scratch = m->attn_split; a.split_capacity = m->attn_split_floats;
    {
        StepProfiler sp(m, st, 2);
        CK(window_attn_store_launch(a, r, st));
        CK(window_attn_launch(a, r, st));
        e->launches += 2;
    }
    if ((rc = dense(e, m, L.attn_o, m->buf[1], qd, m->oL, W, T))) return rc;
    ScanArgs s = {};
    s.proj = m->proj; s.ldp = Np; s.x_off = L.x_off; s.z_off = L.z_off; s.conv_w = L.conv_w; s.conv_b = L.conv_b;
    s.taps = d.conv_taps; s.conv_state = L.conv_state; s.xc = m->buf[0]; s.xproj = m->buf[2];
    s.ldx = d.dt_rank + 2 * d.d_state; s.R = d.dt_rank; s.N = d.d_state; s.dt_raw = m->buf[3]; s.dt_bias = L.dt_b;
    s.A_log = L.A_log; s.D = L.Dskip; s.ssm_state = L.ssm_state; s.y = m->buf[1]; s.inner = d.d_inner;
    {
        StepProfiler sp(m, st, 3);
        CK(scan_conv_launch(s, r, st));
        e->launches++;
    }
    if ((rc = dense(e, m, L.scan_x, m->buf[0], d.d_inner, m->buf[2], s.ldx, T))) return rc;
    if ((rc = dense(e, m, L.scan_dt, m->buf[2], s.ldx, m->buf[3], d.d_inner, T))) return rc;
    {
        StepProfiler sp(m, st, 3);
        CK(scan_recurrence_launch(s, r, st));
        e->launches += d.d_state <= 32 ? 2 : 1;      // states up to a warp wide: a preparation pass goes first
    }
    return dense(e, m, L.scan_o, m->buf[1], d.d_inner, m->oR, W, T);
}

static int mix_matrix_memory(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    const int T = r.T, W = c.n_embd;
    int rc;
    const int Np = L.mm_proj.N, vd = d.mm_heads * d.mm_vdim;
    if ((rc = dense(e, m, L.mm_proj, in, W, m->proj, Np, T))) return rc;
    MatrixMemArgs a = {};
    a.proj = m->proj; a.ldp = Np; a.q_off = L.mq; a.k_off = L.mk; a.v_off = L.mv; a.g_off = L.mg; a.i_off = L.mi; a.f_off = L.mf;
    a.i_bias = L.i_b; a.f_bias = L.f_b; a.norm_w = L.mm_norm; a.H = d.mm_heads; a.d = d.mm_dim; a.dv = d.mm_vdim;
    a.cap = (float)d.gate_cap; a.eps = c.norm_eps; a.S = L.S; a.n = L.nvec; a.m = L.mmax; a.o_raw = m->buf[0]; a.out = m->buf[1];
    {
        StepProfiler sp(m, e->stream, 4);
        CK(matrix_mem_launch(a, r, e->stream));
        e->launches += 3;
    }
    return dense(e, m, L.mm_o, m->buf[1], vd, m->oL, W, T);
}

static int mix_latent_attn(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd, H = d.n_head, dq = d.head_dim + d.la_rot_dim, Dk = d.la_rank + d.la_rot_dim, Np = L.la_proj.N;
    int rc;
    if ((rc = dense(e, m, L.la_proj, in, W, m->proj, Np, T))) return rc;
    LatentAttnArgs a = {};
    a.proj = m->proj; a.ldp = Np; a.q_off = L.q_off; a.dkv_off = L.dkv_off; a.c_norm_w = L.c_norm;
    a.rot.cos = L.rot_cos; a.rot.sin = L.rot_sin; a.rot.rot_dims = d.rot_dims;
    a.pool = L.la_pool; a.cache_f32 = m->exact ? 1 : 0; a.block_tables = m->block_tables; a.block_tokens = c.kv_block_tokens;
    a.H = H; a.d = d.head_dim; a.dr = d.la_rot_dim; a.rank = d.la_rank; a.window = d.window > 0 ? d.window : c.n_ctx;
    a.scale = (float)d.attn_scale; a.eps = c.norm_eps; a.sink = L.sink; a.qv = m->buf[0]; a.o_lat = m->buf[1];
    a.split_scratch = m->attn_split; a.split_capacity = m->attn_split_floats;
    {
        StepProfiler sp(m, st, 2);
        CK(latent_store_launch(a, r, st));
        e->launches++;
    }
    // every head's unrotated query through its transposed key map: the head's query in the latent's coordinates
    DenseArgs b = {};
    b.batch = H; b.x_bs = dq; b.w_bs = (long)d.la_rank * d.head_dim; b.y_bs = Dk; b.x_span = H * dq;
    if ((rc = dense(e, m, L.uk_t, m->proj + L.q_off, Np, m->buf[0], H * Dk, T, nullptr, EPI_NONE, 1, &b))) return rc;
    {
        StepProfiler sp(m, st, 2);
        CK(latent_attn_launch(a, r, st));
        e->launches += 2;
    }
    // values of the weighted latent sums, head by head, times the sigmoid output gate
    DenseArgs v = {};
    v.batch = H; v.x_bs = d.la_rank; v.w_bs = (long)d.la_vdim * d.la_rank; v.y_bs = d.la_vdim; v.x_span = H * d.la_rank;
    v.aux = m->proj + L.g_off; v.ldaux = Np; v.aux_bs = d.la_vdim;
    if ((rc = dense(e, m, L.uv, m->buf[1], H * d.la_rank, m->buf[2], H * d.la_vdim, T, nullptr, EPI_MUL_SIGMOID, 1, &v))) return rc;
    return dense(e, m, L.attn_o, m->buf[2], H * d.la_vdim, m->oL, W, T);
}

static int mix_delta_rule(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd, H = d.mm_heads, G = d.key_heads, kd = G * d.mm_dim, vd = H * d.mm_vdim, Np = L.st_proj.N;
    int rc;
    if ((rc = dense(e, m, L.st_proj, in, W, m->proj, Np, T))) return rc;
    ConvArgs cv = {};
    cv.in = m->proj + L.conv_off; cv.ld_in = Np; cv.C = L.conv_C; cv.taps = d.conv_taps; cv.w = L.st_conv_w; cv.bias = nullptr;
    cv.state = L.st_conv_state; cv.out = m->buf[0]; cv.ld_out = L.conv_C;
    {
        StepProfiler sp(m, st, 3);
        CK(causal_conv_launch(cv, r, st));
        CK(causal_conv_advance_launch(cv, r, st));
        e->launches += d.conv_taps > 1 ? 2 : 1;
    }
    // decays [T][H*dim] and gate inputs [T][H*vdim]: side by side in buf[1] (one product), or in buf[1] and buf[2]
    float *a_out = m->buf[1], *g_out = m->buf[2];
    int ld_a = H * d.mm_dim, ld_g = vd;
    if (L.ag.w && L.g1_off == L.a1_off + d.rank_a) {
        g_out = m->buf[1] + H * d.mm_dim;
        ld_a = ld_g = H * d.mm_dim + vd;
        if ((rc = dense(e, m, L.ag, m->proj + L.a1_off, Np, m->buf[1], ld_a, T))) return rc;
    } else {
        if ((rc = dense(e, m, L.a2, m->proj + L.a1_off, Np, a_out, ld_a, T))) return rc;
        if ((rc = dense(e, m, L.g2, m->proj + L.g1_off, Np, g_out, ld_g, T))) return rc;
    }
    DeltaPrepArgs pa = {};
    pa.q = m->buf[0]; pa.k = m->buf[0] + kd; pa.ld_qk = L.conv_C; pa.G = G; pa.d = d.mm_dim;
    pa.a = a_out; pa.ld_a = ld_a; pa.A_log = L.st_A_log; pa.dt_bias = L.st_dt_bias; pa.H = H;
    pa.beta = m->proj + L.b_off; pa.ld_b = Np; pa.unit_eps = 1e-6f;
    ColStateArgs cs = {};
    cs.wk = m->buf[0] + kd; cs.ld_wk = L.conv_C; cs.rk = m->buf[0]; cs.ld_rk = L.conv_C;
    cs.row_decay = a_out; cs.ld_rd = ld_a; cs.val = m->buf[0] + 2 * kd; cs.ld_v = L.conv_C;
    cs.val_scale = m->proj + L.b_off; cs.ld_vs = Np; cs.H = H; cs.G = G; cs.R = d.mm_dim; cs.P = d.mm_vdim; cs.delta = 1;
    cs.state = L.st_state; cs.y = m->buf[3]; cs.ld_y = vd;
    GroupNormArgs gn = {};
    gn.x = m->buf[3]; gn.ld_x = vd; gn.gate = g_out; gn.ld_g = ld_g; gn.w = L.st_norm; gn.w_gstride = 0; gn.groups = H; gn.n = d.mm_vdim;
    gn.eps = c.norm_eps; gn.gate_first = 0; gn.y = m->buf[3]; gn.ld_y = vd;
    {
        StepProfiler sp(m, st, 4);
        CK(delta_prepare_launch(pa, T, st));
        CK(col_state_launch(cs, r, st));
        CK(group_norm_gate_launch(gn, T, st));
        e->launches += 3;
    }
    return dense(e, m, L.st_o, m->buf[3], vd, m->oL, W, T);
}

static int mix_ssd(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd, H = d.mm_heads, G = d.key_heads, N = d.d_state, inner = H * d.mm_vdim, Np = L.st_proj.N;
    int rc;
    if ((rc = dense(e, m, L.st_proj, in, W, m->proj, Np, T))) return rc;
    ConvArgs cv = {};
    cv.in = m->proj + L.conv_off; cv.ld_in = Np; cv.C = L.conv_C; cv.taps = d.conv_taps; cv.w = L.st_conv_w; cv.bias = L.st_conv_b;
    cv.state = L.st_conv_state; cv.out = m->buf[0]; cv.ld_out = L.conv_C;
    ColStateArgs cs = {};
    cs.wk = m->buf[0] + inner; cs.ld_wk = L.conv_C; cs.rk = m->buf[0] + inner + G * N; cs.ld_rk = L.conv_C;
    cs.head_decay = m->buf[1]; cs.ld_hd = H; cs.val = m->buf[0]; cs.ld_v = L.conv_C;
    cs.val_scale = m->proj + L.dt_off; cs.ld_vs = Np; cs.skip = L.st_D; cs.H = H; cs.G = G; cs.R = N; cs.P = d.mm_vdim; cs.delta = 0;
    cs.state = L.st_state; cs.y = m->buf[2]; cs.ld_y = inner;
    GroupNormArgs gn = {};
    gn.x = m->buf[2]; gn.ld_x = inner; gn.gate = m->proj; gn.ld_g = Np; gn.w = L.st_norm; gn.w_gstride = inner / d.norm_groups;
    gn.groups = d.norm_groups; gn.n = inner / d.norm_groups; gn.eps = c.norm_eps; gn.gate_first = 1; gn.y = m->buf[2]; gn.ld_y = inner;
    {
        StepProfiler sp(m, st, 3);
        CK(causal_conv_launch(cv, r, st));
        CK(causal_conv_advance_launch(cv, r, st));
        CK(ssd_prepare_launch(m->proj + L.dt_off, Np, L.st_dt_bias, L.st_A_log, H, m->buf[1], T, st));
        CK(col_state_launch(cs, r, st));
        CK(group_norm_gate_launch(gn, T, st));
        e->launches += d.conv_taps > 1 ? 5 : 4;
    }
    return dense(e, m, L.st_o, m->buf[2], inner, m->oL, W, T);
}

// both branches read `in`; the weighted sum of their outputs is formed by ONE product over [left heads | right heads]
static int mix_chunk_linear(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd, Np = L.cl_proj.N;
    const int od = d.n_head * d.attn_vdim, rqd = d.mm_heads * d.mm_dim, rvd = d.mm_heads * d.mm_vdim, Kt = od + rvd;
    int rc;
    if ((rc = dense(e, m, L.cl_proj, in, W, m->proj, Np, T))) return rc;
    SigmoidAttnArgs a = {};
    a.proj = m->proj; a.ldp = Np; a.q_off = L.q_off; a.k_off = L.k_off; a.v_off = L.v_off; a.q_norm_w = L.q_norm; a.k_norm_w = L.k_norm;
    a.k_pool = L.k_pool; a.v_pool = L.v_pool; a.cache_f32 = m->exact ? 1 : 0; a.block_tables = m->block_tables; a.block_tokens = c.kv_block_tokens;
    a.H = d.n_head; a.G = d.n_head_kv; a.d = d.head_dim; a.dv = d.attn_vdim; a.chunk = d.window;
    a.scale = (float)d.attn_scale; a.softcap = (float)d.softcap; a.eps = c.norm_eps; a.bias = L.pb;
    a.q_out = m->buf[0]; a.out = m->buf[1]; a.ld_out = Kt; a.out_scale = (float)d.branch_scale[0];
    a.act = m->proj + L.rq_off; a.act_n = 2 * rqd + rvd;          // the linear branch's q | k | v get their SiLU in the same pass
    {
        StepProfiler sp(m, st, 2);
        CK(sigmoid_attn_store_launch(a, r, st));
        CK(sigmoid_attn_launch(a, r, st));
        e->launches += 2;
    }
    ColStateArgs cs = {};
    cs.wk = m->proj + L.rq_off + rqd; cs.ld_wk = Np; cs.rk = m->proj + L.rq_off; cs.ld_rk = Np;
    cs.head_const = L.decay; cs.val = m->proj + L.rq_off + 2 * rqd; cs.ld_v = Np;
    cs.H = d.mm_heads; cs.G = d.mm_heads; cs.R = d.mm_dim; cs.P = d.mm_vdim; cs.delta = 0;
    cs.state = L.la_state; cs.y = m->buf[2]; cs.ld_y = rvd;
    GroupNormArgs gn = {};
    gn.x = m->buf[2]; gn.ld_x = rvd; gn.gate = m->proj + L.g_off; gn.ld_g = Np; gn.w = L.mm_norm; gn.w_gstride = 0; gn.groups = 1; gn.n = rvd;
    gn.eps = c.norm_eps; gn.gate_first = 0; gn.y = m->buf[1] + od; gn.ld_y = Kt; gn.out_scale = (float)d.branch_scale[1];
    {
        StepProfiler sp(m, st, 4);
        CK(col_state_launch(cs, r, st));
        CK(group_norm_gate_launch(gn, T, st));
        e->launches += 2;
    }
    return dense(e, m, L.cl_o, m->buf[1], Kt, m->oL, W, T);
}

// softmax attention with a sink, alone (output in m->oL) or beside the head-decay delta rule (attention in m->oL, delta rule in
// m->oR; the caller norms and averages them)
static int mix_sink(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const b2_layered_config& c = m->c;
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd, Np = L.sk_proj.N, H = d.n_head, od = H * d.attn_vdim;
    int rc;
    if ((rc = dense(e, m, L.sk_proj, in, W, m->proj, Np, T, L.sk_bias, L.sk_bias ? EPI_BIAS : EPI_NONE))) return rc;
    SinkAttnArgs a = {};
    a.proj = m->proj; a.ldp = Np; a.q_off = L.q_off; a.k_off = L.k_off; a.v_off = L.v_off;
    a.rot.cos = L.rot_cos; a.rot.sin = L.rot_sin; a.rot.rot_dims = d.rot_dims; a.unit_qk = (d.attn_flags & B2_ATTN_UNIT_QK) ? 1 : 0;
    a.k_pool = L.k_pool; a.v_pool = L.v_pool; a.cache_f32 = m->exact ? 1 : 0; a.block_tables = m->block_tables; a.block_tokens = c.kv_block_tokens;
    a.H = H; a.G = d.n_head_kv; a.d = d.head_dim; a.dv = d.attn_vdim; a.window = d.window; a.scale = (float)d.attn_scale; a.eps = c.norm_eps;
    a.sink = L.sink; a.talk = L.talk; a.gate = m->proj + L.gl_off; a.ld_gate = Np; a.gate_per_head = (d.attn_flags & B2_ATTN_HEAD_GATE) ? 1 : 0;
    a.q_rot = m->buf[0]; a.cross = m->cross; a.out = m->buf[1]; a.ld_out = od;
    a.pbuf = m->attn_pbuf; a.pbuf_floats = m->attn_pbuf_floats;
    a.part = m->attn_split; a.part_capacity = m->attn_split_floats; a.max_keys = d.window > 0 ? std::min(d.window, c.n_ctx) : c.n_ctx;
    {
        StepProfiler sp(m, st, 2);
        CK(sink_attn_store_launch(a, r, st));
        CK(sink_attn_launch(a, r, st));
        e->launches += L.talk ? 3 : 2;
    }
    if ((rc = dense(e, m, L.attn_o, m->buf[1], od, m->oL, W, T))) return rc;
    if (d.mixer != B2_MIX_SINK_DELTA) return B2_OK;
    const int Hr = d.mm_heads, G = d.key_heads, kd = G * d.mm_dim, vd = Hr * d.mm_vdim;
    ConvArgs cv = {};
    cv.in = m->proj + L.conv_off; cv.ld_in = Np; cv.C = L.conv_C; cv.taps = d.conv_taps; cv.w = L.st_conv_w; cv.bias = nullptr;
    cv.state = L.st_conv_state; cv.out = m->buf[0]; cv.ld_out = L.conv_C;
    {
        StepProfiler sp(m, st, 3);
        CK(causal_conv_launch(cv, r, st));
        CK(causal_conv_advance_launch(cv, r, st));
        e->launches += d.conv_taps > 1 ? 2 : 1;
    }
    DeltaPrepArgs pa = {};
    pa.q = m->buf[0]; pa.k = m->buf[0] + kd; pa.ld_qk = L.conv_C; pa.G = G; pa.d = d.mm_dim;
    pa.a = m->proj + L.ra_off; pa.ld_a = Np; pa.A_log = L.st_A_log; pa.dt_bias = L.st_dt_bias; pa.H = Hr; pa.a_cols = 1;
    pa.beta = m->proj + L.b_off; pa.ld_b = Np; pa.unit_eps = 1e-6f;
    ColStateArgs cs = {};
    cs.wk = m->buf[0] + kd; cs.ld_wk = L.conv_C; cs.rk = m->buf[0]; cs.ld_rk = L.conv_C;
    cs.head_decay = m->proj + L.ra_off; cs.ld_hd = Np; cs.val = m->buf[0] + 2 * kd; cs.ld_v = L.conv_C;
    cs.val_scale = m->proj + L.b_off; cs.ld_vs = Np; cs.H = Hr; cs.G = G; cs.R = d.mm_dim; cs.P = d.mm_vdim; cs.delta = 1;
    cs.state = L.st_state; cs.y = m->buf[2]; cs.ld_y = vd;
    GroupNormArgs gn = {};
    gn.x = m->buf[2]; gn.ld_x = vd; gn.gate = m->proj + L.rg_off; gn.ld_g = Np; gn.w = L.st_norm; gn.w_gstride = 0; gn.groups = Hr; gn.n = d.mm_vdim;
    gn.eps = c.norm_eps; gn.gate_first = 0; gn.gate_silu = 1; gn.y = m->buf[2]; gn.ld_y = vd;
    {
        StepProfiler sp(m, st, 4);
        CK(delta_prepare_launch(pa, T, st));
        CK(col_state_launch(cs, r, st));
        CK(group_norm_gate_launch(gn, T, st));
        e->launches += 3;
    }
    return dense(e, m, L.st_o, m->buf[2], vd, m->oR, W, T);
}

// ---- feed-forward blocks: input `in` [T][W], output in m->oL
static int ff_piecewise(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const int T = r.T, W = m->c.n_embd;
    DenseArgs up = {};
    up.p0 = L.act_p0; up.p1 = L.act_p1;
    int rc;
    if ((rc = dense(e, m, L.up, in, W, m->ff, L.d.n_ff, T, nullptr, EPI_PIECEWISE, 1, &up))) return rc;
    return dense(e, m, L.down, m->ff, L.d.n_ff, m->oL, W, T);
}

static int ff_relu2(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const int T = r.T, W = m->c.n_embd;
    int rc;
    if ((rc = dense(e, m, L.up, in, W, m->ff, L.d.n_ff, T, L.up_b, EPI_BIAS_RELU2))) return rc;
    return dense(e, m, L.down, m->ff, L.d.n_ff, m->oL, W, T, L.down_b, EPI_BIAS);
}

static int ff_glu(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    const int T = r.T, W = m->c.n_embd, ff = L.glu_down.K;
    int rc;
    if ((rc = dense(e, m, L.glu_gate_up, in, W, m->ff, ff, T, nullptr, EPI_GLU_SILU))) return rc;
    return dense(e, m, L.glu_down, m->ff, ff, m->oL, W, T);
}

// defer != nullptr: the weighted sum of the expert outputs is left to the caller's residual kernel (described in *defer)
static int ff_moe(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in, MoeJoinArgs* defer) {
    const b2_layer_desc& d = L.d;
    cudaStream_t st = e->stream;
    const int T = r.T, W = m->c.n_embd, slots = d.moe_experts + d.moe_identity, pairs = T * d.moe_top, ff = d.n_ff;
    int rc;
    DenseArgs ex = {};
    ex.exact = true;                               // router scores are 32-bit products in both modes
    if ((rc = dense(e, m, L.router, in, W, m->moe_logits, slots, T, nullptr, EPI_NONE, 7, &ex))) return rc;
    MoeRouteArgs ra = {};
    ra.logits = m->moe_logits; ra.ld = slots; ra.correction = L.correction; ra.n_slots = slots; ra.n_experts = d.moe_experts;
    ra.top = d.moe_top; ra.n_groups = d.moe_groups; ra.keep_groups = d.moe_keep; ra.scale = (float)d.moe_scale;
    ra.mode = d.moe_route == B2_ROUTE_TOPK_SOFTMAX ? 1 : 0; ra.renorm = d.moe_renorm;
    ra.sel = m->moe_sel; ra.weight = m->moe_weight; ra.pair_token = m->moe_tok;
    DenseGroups g = {};
    g.n_groups = d.moe_experts;
    const bool tiled = T > 8;
    // long prompts in the serving mode: 128-row tiles through the large tensor-core kernel
    const bool big = tiled && !m->exact && L.gate_up.type == T_BF16 && pairs >= 1024 && W % 8 == 0 && ff % 8 == 0 && m->xb;
    g.tile_max = big ? 128 : 64;
    {
        StepProfiler sp(m, st, 7);
        CK(moe_route_launch(ra, T, st));
        e->launches++;
        if (tiled) {
            MoeSortArgs sa = {};
            sa.sel = m->moe_sel; sa.n_pairs = pairs; sa.top = d.moe_top; sa.n_experts = d.moe_experts; sa.tile = g.tile_max; sa.pos = m->moe_pos; sa.x_rows = m->moe_rows;
            sa.n_tiles = m->moe_tiles; sa.tile_group = m->moe_tiles + 1; sa.tile_row0 = sa.tile_group + m->moe_max_tiles;
            sa.tile_rows = sa.tile_row0 + m->moe_max_tiles; sa.max_tiles = m->moe_max_tiles;
            CK(moe_sort_launch(sa, st));
            e->launches++;
            g.tile_group = sa.tile_group; g.tile_row0 = sa.tile_row0; g.tile_rows = sa.tile_rows; g.n_tiles = sa.n_tiles;
            g.max_tiles = std::min(m->moe_max_tiles, pairs / g.tile_max + d.moe_experts + 1);
        } else g.group = m->moe_sel;
    }
    DenseArgs up = {};
    g.x_rows = tiled ? m->moe_rows : m->moe_tok; g.w_stride = (long)2 * ff * W; g.x_total_rows = T;
    up.groups = &g;
    up.p0 = (float)d.moe_limit; up.p1 = (float)d.moe_alpha;
    if ((rc = dense(e, m, L.gate_up, in, W, m->moe_h, ff, pairs, nullptr, d.moe_expert == B2_EXPERT_CLAMPED ? EPI_GLU_CLAMP : EPI_GLU_SILU, 1, &up))) return rc;
    DenseGroups g2 = g;
    g2.x_rows = nullptr; g2.w_stride = (long)W * ff; g2.x_total_rows = pairs;
    DenseArgs dn = {};
    dn.groups = &g2;
    if ((rc = dense(e, m, L.e_down, m->moe_h, ff, m->moe_y, W, pairs, nullptr, EPI_NONE, 1, &dn))) return rc;
    if (defer) {
        defer->sel = m->moe_sel; defer->weight = m->moe_weight; defer->pos = tiled ? m->moe_pos : nullptr; defer->rows = m->moe_y; defer->h = in;
        defer->n_experts = d.moe_experts; defer->top = d.moe_top;
        return B2_OK;
    }
    StepProfiler sp(m, st, 7);
    CK(moe_combine_launch(m->moe_sel, m->moe_weight, tiled ? m->moe_pos : nullptr, m->moe_y, in, d.moe_experts, d.moe_top, W, T, m->oL, st));
    e->launches++;
    return B2_OK;
}

static int run_mixer(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in) {
    switch (L.d.mixer) {
        case B2_MIX_WINDOW_SCAN: return mix_window_scan(e, m, L, r, in);
        case B2_MIX_MATRIX_MEMORY: return mix_matrix_memory(e, m, L, r, in);
        case B2_MIX_LATENT_ATTN: return mix_latent_attn(e, m, L, r, in);
        case B2_MIX_DELTA_RULE: return mix_delta_rule(e, m, L, r, in);
        case B2_MIX_SSD: return mix_ssd(e, m, L, r, in);
        case B2_MIX_CHUNK_LINEAR: return mix_chunk_linear(e, m, L, r, in);
        case B2_MIX_SINK_DELTA: case B2_MIX_SINK_ATTN: return mix_sink(e, m, L, r, in);
    }
    return b2_fail(B2_ERR_UNSUPPORTED, "unknown mixer kind");
}
static int run_ff(b2_engine* e, LayeredModel* m, LyLayer& L, const RaggedDev& r, const float* in, MoeJoinArgs* defer = nullptr) {
    if (L.d.ff_kind == B2_FF_MOE) return ff_moe(e, m, L, r, in, defer);
    if (L.d.ff_kind == B2_FF_PIECEWISE) return ff_piecewise(e, m, L, r, in);
    return L.d.ff_kind == B2_FF_GLU ? ff_glu(e, m, L, r, in) : ff_relu2(e, m, L, r, in);
}

static int run_layers(b2_engine* e, LayeredModel* m, const RaggedDev& r) {
    const b2_layered_config& c = m->c;
    cudaStream_t st = e->stream;
    const int T = r.T, W = c.n_embd;
    const bool prenorm = c.block_style == B2_BLOCK_PRENORM_RMS;
    int rc;
    {
        StepProfiler sp(m, st, 0);
        CK(embed_ragged_launch(m->embed.w, m->embed.type, W, r.tok_id, T, m->x, c.embed_scale != 0.f ? c.embed_scale : 1.f, st));
        e->launches++;
        if (prenorm) {
            CK(resid_rms_norm_launch(m->x, nullptr, 0.f, m->embed_norm, 1.f, 1.f, c.norm_eps, W, T, m->x, st));
            e->launches++;
        }
    }
    // pre-norm blocks: a branch output waits in m->oL until the next norm (or the end of the layer) adds it to the stream
    // (a mixture's weighted sum is not even formed before: the same kernel adds it up)
    const float* pending = nullptr;
    MoeJoinArgs pending_moe = {};
    auto join = [&](const float* norm_w, float* y) -> int {
        StepProfiler sp(m, st, 5);
        if (pending_moe.sel) CK(moe_join_launch(pending_moe, m->x, c.residual_scale, norm_w, 1.f, c.norm_eps, W, T, y, st));
        else CK(resid_rms_norm_launch(m->x, pending, c.residual_scale, norm_w, 1.f, 1.f, c.norm_eps, W, T, y, st));
        e->launches++;
        pending = nullptr;
        pending_moe = MoeJoinArgs{};
        return B2_OK;
    };
    if (c.block_style == B2_BLOCK_HYPER_RMS) {
        // The embedding sits in copy 0. A sublayer's output waits (in m->oL / m->oR / the mixture's rows) until the next boundary:
        // one kernel writes it back into all copies, reads the next sublayer's input and norms it.
        HyperJoinArgs hj = {};
        MoeJoinArgs hj_moe = {};
        bool first = true;
        // cw / cstate: the convolution around a skip on the input that is read (null: none). Returns what the sublayer reads.
        auto boundary = [&](const float* in_w, const float* norm_w, float* hn, float* sum_out, const float* cw, float* cstate, const float** in_out) -> int {
            StepProfiler sp(m, st, 5);
            hj.xs = m->xs; hj.stream_stride = (long)c.max_step_tokens * W; hj.S = std::max(1, c.n_streams); hj.eps = c.norm_eps;
            hj.in = in_w; hj.norm_w = norm_w; hj.hn = hn; hj.sum_out = sum_out; hj.bcast = first ? 1 : 0;
            hj.moe = hj_moe.sel ? &hj_moe : nullptr;
            ConvArgs cv = {};
            cv.in = m->hn; cv.ld_in = W; cv.C = W; cv.taps = c.canon_taps; cv.w = cw; cv.state = cstate; cv.out = m->hc; cv.ld_out = W; cv.skip = 1;
            if (hn && cw && hyper_join_conv_fits(W, c.canon_taps, T, hj.S)) {
                CK(hyper_join_conv_launch(hj, cv, r, W, st));
                e->launches++;
            } else {
                CK(hyper_join_launch(hj, W, T, st));
                e->launches++;
                if (hn && cw) {
                    CK(causal_conv_launch(cv, r, st));
                    CK(causal_conv_advance_launch(cv, r, st));
                    e->launches += c.canon_taps > 1 ? 2 : 1;
                }
            }
            if (in_out) *in_out = hn && cw ? m->hc : m->hn;
            hj = HyperJoinArgs{}; hj_moe = MoeJoinArgs{};
            first = false;
            return B2_OK;
        };
        CK(cudaMemcpyAsync(m->xs, m->x, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st));
        for (int li = 0; li < c.n_layer; li++) {
            LyLayer& L = m->layers[li];
            const b2_layer_desc& d = L.d;
            const float* in = nullptr;
            if ((rc = boundary(L.hc_in[0], L.norm1, m->hn, nullptr, L.canon_w[0], L.canon_state[0], &in))) return rc;
            if ((rc = run_mixer(e, m, L, r, in))) return rc;
            hj.a = m->oL; hj.mix = L.hc_mix[0]; hj.out = L.hc_out[0];
            if (d.mixer == B2_MIX_SINK_DELTA) { hj.wa = L.left_w; hj.b = m->oR; hj.wb = L.right_w; }
            if (d.n_ff > 0) {
                if ((rc = boundary(L.hc_in[1], L.norm2, m->hn, nullptr, L.canon_w[1], L.canon_state[1], &in))) return rc;
                const bool moe = d.ff_kind == B2_FF_MOE;
                if ((rc = run_ff(e, m, L, r, in, moe ? &hj_moe : nullptr))) return rc;
                hj.a = moe ? nullptr : m->oL; hj.mix = L.hc_mix[1]; hj.out = L.hc_out[1];
            }
            if (m->trace || li == c.n_layer - 1) {
                if ((rc = boundary(nullptr, nullptr, nullptr, m->x, nullptr, nullptr, nullptr))) return rc;
                if (m->trace) CK(cudaMemcpyAsync(m->trace + ((size_t)li * c.max_step_tokens) * W, m->x, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st));
            }
        }
        return B2_OK;
    }
    for (int li = 0; li < c.n_layer; li++) {
        LyLayer& L = m->layers[li];
        const b2_layer_desc& d = L.d;
        if (c.block_style == B2_BLOCK_OUTNORM_RMS) {
            // both sublayers read the stream itself; what they return is normed in parts and added
            const int ng = std::max(1, c.norm_groups);
            if ((rc = run_mixer(e, m, L, r, m->x))) return rc;
            {
                StepProfiler sp(m, st, 5);
                CK(outnorm_join_launch(m->x, m->oL, nullptr, L.norm1, ng, c.norm_eps, W, T, nullptr, st));
                e->launches++;
            }
            if (d.n_ff > 0) {
                const bool moe = d.ff_kind == B2_FF_MOE;
                MoeJoinArgs mj = {};
                if ((rc = run_ff(e, m, L, r, m->x, moe ? &mj : nullptr))) return rc;
                const float* dense_part = moe ? nullptr : m->oL;
                if (moe && d.moe_shared_ff > 0) {          // the shared expert runs for every token; the join adds it to the weighted sum
                    if ((rc = ff_glu(e, m, L, r, m->x))) return rc;
                    dense_part = m->oL;
                }
                StepProfiler sp(m, st, 5);
                CK(outnorm_join_launch(m->x, dense_part, moe ? &mj : nullptr, L.norm2, ng, c.norm_eps, W, T, nullptr, st));
                e->launches++;
            }
        } else if (prenorm) {
            if ((rc = join(L.norm1, m->hn))) return rc;
            if ((rc = run_mixer(e, m, L, r, m->hn))) return rc;
            pending = m->oL;
            if (d.n_ff > 0) {
                if ((rc = join(L.norm2, m->hn))) return rc;
                const bool moe = d.ff_kind == B2_FF_MOE;
                if ((rc = run_ff(e, m, L, r, m->hn, moe ? &pending_moe : nullptr))) return rc;
                pending = moe ? nullptr : m->oL;
            }
            if (m->trace || li == c.n_layer - 1) { if ((rc = join(nullptr, nullptr))) return rc; }
        } else {
            if ((rc = run_mixer(e, m, L, r, m->x))) return rc;
            {
                const bool two = d.mixer == B2_MIX_WINDOW_SCAN;
                StepProfiler sp(m, st, 5);
                CK(postsum_norm_launch(m->x, m->oL, two ? L.left_w : nullptr, two ? m->oR : nullptr, two ? L.right_w : nullptr, L.norm1,
                                       c.residual_scale, c.norm_eps, W, T, st));
                e->launches++;
            }
            if (d.n_ff > 0) {
                if ((rc = run_ff(e, m, L, r, m->x))) return rc;
                StepProfiler sp(m, st, 5);
                CK(postsum_norm_launch(m->x, m->oL, nullptr, nullptr, nullptr, L.norm2, c.residual_scale, c.norm_eps, W, T, st));
                e->launches++;
            }
        }
        if (m->trace)
            CK(cudaMemcpyAsync(m->trace + ((size_t)li * c.max_step_tokens) * W, m->x, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st));
    }
    return B2_OK;
}

struct StepChainPdl {
    bool prev;
    explicit StepChainPdl(bool on) : prev(g_chain_pdl) { g_chain_pdl = on; }
    ~StepChainPdl() { g_chain_pdl = prev; }
};

int b2_sample_enqueue(b2_engine* e, Slot& s, int pinned_index);

extern "C" int b2_step(b2_engine* e, int n_entries, const int32_t* slots, const int32_t* n_tokens, const int32_t* tokens,
                       const int32_t* want_rows, int n_want, float* host_logits, const int32_t* sample, int32_t* host_sampled) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "b2_step needs an engine made by b2_engine_create_layered");
    if (!e->finalized) return b2_fail(B2_ERR_STATE, "engine not finalized");
    if (n_entries <= 0 || n_entries > B2_STEP_MAX_ENTRIES || !slots || !n_tokens || !tokens) return b2_fail(B2_ERR_ARG, "bad arguments");
    if (n_want < 0 || (n_want > 0 && (!want_rows || !host_logits))) return b2_fail(B2_ERR_ARG, "bad wanted rows");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    const b2_layered_config& c = m->c;
    int T = 0;
    for (int i = 0; i < n_entries; i++) {
        if (slots[i] < 0 || slots[i] >= c.max_seqs) return b2_fail(B2_ERR_ARG, "slot out of range");
        for (int j = 0; j < i; j++) if (slots[j] == slots[i]) return b2_fail(B2_ERR_ARG, "slot listed twice");
        if (n_tokens[i] <= 0) return b2_fail(B2_ERR_ARG, "empty entry");
        if (e->slots[slots[i]].n_past + n_tokens[i] > c.n_ctx) return b2_fail(B2_ERR_ARG, "context window full");
        T += n_tokens[i];
        if (T > c.max_step_tokens) return b2_fail(B2_ERR_ARG, "more tokens than max_step_tokens in one step");
    }
    for (int i = 0; i < T; i++) if (tokens[i] < 0 || tokens[i] >= c.n_vocab) return b2_fail(B2_ERR_ARG, "token id out of range");
    for (int i = 0; i < n_want; i++) if (want_rows[i] < 0 || want_rows[i] >= T) return b2_fail(B2_ERR_ARG, "wanted row out of range");
    CK(cudaSetDevice(c.device));
    cudaStream_t st = e->stream;
    StepChainPdl chain(e->chain_pdl);
    // ragged description: [tok_id T][tok_seg T][tok_pos T][seg_slot n][seg_start n][seg_len n][seg_pos0 n][tile_seg][tile_row0][rows ...]
    int* h = m->meta_host;
    const int n = n_entries;
    int *h_id = h, *h_seg = h + T, *h_pos = h + 2 * T, *h_slot = h + 3 * T, *h_start = h_slot + n, *h_len = h_start + n, *h_p0 = h_len + n;
    int n_tiles = 0;
    for (int i = 0; i < n; i++) n_tiles += (n_tokens[i] + 63) / 64;
    int *h_tseg = h_p0 + n, *h_trow = h_tseg + n_tiles;
    int* h_rows = h_trow + n_tiles;
    int row = 0, tile = 0;
    for (int i = 0; i < n; i++) {
        const int p0 = e->slots[slots[i]].n_past;
        h_slot[i] = slots[i]; h_start[i] = row; h_len[i] = n_tokens[i]; h_p0[i] = p0;
        for (int k = 0; k < n_tokens[i]; k += 64) { h_tseg[tile] = i; h_trow[tile++] = row + k; }
        for (int k = 0; k < n_tokens[i]; k++, row++) { h_id[row] = tokens[row]; h_seg[row] = i; h_pos[row] = p0 + k; }
    }
    // rows whose logits are needed: the wanted ones, then the last token of every sampled entry
    int n_rows = 0;
    for (int i = 0; i < n_want; i++) h_rows[n_rows++] = want_rows[i];
    std::vector<int> samp_row(n, -1);
    for (int i = 0; i < n; i++)
        if (sample && sample[i]) { samp_row[i] = n_rows; h_rows[n_rows++] = h_start[i] + h_len[i] - 1; }
    const size_t n_meta = (size_t)3 * T + 4 * n + 2 * n_tiles + n_rows;
    RaggedDev r = {};
    r.tok_id = m->meta; r.tok_seg = m->meta + T; r.tok_pos = m->meta + 2 * T; r.seg_slot = m->meta + 3 * T;
    r.seg_start = r.seg_slot + n; r.seg_len = r.seg_start + n; r.seg_pos0 = r.seg_len + n; r.T = T; r.n_seg = n;
    r.tile_seg = r.seg_pos0 + n; r.tile_row0 = r.tile_seg + n_tiles; r.n_tiles = n_tiles;
    const int* d_rows = r.tile_row0 + n_tiles;
    if (m->profile) {
        for (auto& pe : m->prof_ev) { cudaEventDestroy(pe.second.first); cudaEventDestroy(pe.second.second); }
        m->prof_ev.clear();
    }
    const int W = c.n_embd, V = c.n_vocab;
    int rc;
    // logits of rows [r0, r0 + nr): final norm, head, wanted rows to the pinned buffer, sampled rows to their slots
    auto head_chunk = [&](int r0, int nr) -> int {
        {
            StepProfiler sp(m, st, 5);
            CK(gather_rows_launch(m->x, W, d_rows + r0, nr, m->rows, st));
            if (c.block_style == B2_BLOCK_OUTNORM_RMS) CK(outnorm_join_launch(nullptr, m->rows, nullptr, m->final_norm, std::max(1, c.norm_groups), c.norm_eps, W, nr, m->rows, st));
            else if (c.block_style == B2_BLOCK_PRENORM_RMS) CK(resid_rms_norm_launch(m->rows, nullptr, 0.f, m->final_norm, 1.f, 1.f, c.norm_eps, W, nr, m->rows, st));
            else if (c.block_style == B2_BLOCK_HYPER_RMS) CK(resid_rms_norm_launch(m->rows, nullptr, 0.f, m->final_norm, 0.f, 1.f, c.norm_eps, W, nr, m->rows, st));
            else CK(layer_norm_launch(m->rows, m->final_norm, c.norm_eps, W, nr, m->rows, st));
            e->launches += 2;
        }
        DenseArgs hs = {};
        hs.scale = c.logit_scale != 0.f ? c.logit_scale : 1.f;
        int rc2 = dense(e, m, m->head, m->rows, W, m->logits, V, nr, nullptr, EPI_NONE, 6, &hs);
        if (rc2) return rc2;
        const int n_w = std::max(0, std::min(n_want - r0, nr));
        if (n_w > 0) CK(cudaMemcpyAsync(m->logits_host, m->logits, (size_t)n_w * V * 4, cudaMemcpyDeviceToHost, st));
        for (int i = 0; i < n; i++)
            if (samp_row[i] >= r0 && samp_row[i] < r0 + nr)
                CK(cudaMemcpyAsync(e->slots[slots[i]].logits, m->logits + (size_t)(samp_row[i] - r0) * V, (size_t)V * 4, cudaMemcpyDeviceToDevice, st));
        return B2_OK;
    };
    // everything the step enqueues up to the logits, for steps whose rows fit one head chunk
    auto forward_once = [&]() -> int {
        CK(cudaMemcpyAsync(m->meta, h, n_meta * 4, cudaMemcpyHostToDevice, st));
        int rc2 = run_layers(e, m, r);
        if (rc2) return rc2;
        return n_rows > 0 ? head_chunk(0, n_rows) : B2_OK;
    };
    // Small steps that repeat (the same slots decoding token after token) are replayed as a CUDA graph: the batch description
    // is read from device memory, so nothing in the launches changes from one such step to the next. A shape is captured the
    // second time it is seen.
    bool done = false;
    if (m->graphs_on && !m->trace && !m->profile && T <= 64 && n_rows <= LOGIT_ROWS) {
        std::string key;
        key.reserve(16 + 12 * n);
        auto put = [&](int v) { key.append(reinterpret_cast<const char*>(&v), sizeof(v)); };
        put(n); put(n_want);
        for (int i = 0; i < n; i++) { put(slots[i]); put(n_tokens[i]); put(samp_row[i]); }
        auto it = m->graphs.find(key);
        if (it == m->graphs.end()) {
            if (m->graphs.size() >= 256) {
                for (auto& kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
                m->graphs.clear();
            }
            m->graphs[key] = StepGraph();
        } else {
            StepGraph& sg = it->second;
            if (!sg.exec && !sg.failed) {
                const int64_t before = e->launches;
                cudaGraph_t g = nullptr;
                CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                const int crc = forward_once();
                const cudaError_t ce = cudaStreamEndCapture(st, &g);
                sg.n_launch = (int)(e->launches - before);
                e->launches = before;
                if (crc == B2_OK && ce == cudaSuccess && g && cudaGraphInstantiate(&sg.exec, g, 0) != cudaSuccess) sg.exec = nullptr;
                if (g) cudaGraphDestroy(g);
                if (!sg.exec) { sg.failed = true; cudaGetLastError(); }
            }
            if (sg.exec) {
                CK(cudaGraphLaunch(sg.exec, st));
                e->launches += sg.n_launch;
                done = true;
            }
        }
    }
    if (!done) {
        if (n_rows <= LOGIT_ROWS) {
            if ((rc = forward_once())) return rc;
        } else {
            CK(cudaMemcpyAsync(m->meta, h, n_meta * 4, cudaMemcpyHostToDevice, st));
            if ((rc = run_layers(e, m, r))) return rc;
        }
    }
    m->last_T = T;
    for (int i = 0; i < n; i++) if (samp_row[i] >= 0) e->slots[slots[i]].logits_view = e->slots[slots[i]].logits;
    if (n_rows <= LOGIT_ROWS) {
        if (n_want > 0) {
            CK(cudaStreamSynchronize(st));
            memcpy(host_logits, m->logits_host, (size_t)n_want * V * 4);
        }
    } else {
        for (int r0 = 0; r0 < n_rows; r0 += LOGIT_ROWS) {
            const int nr = std::min(LOGIT_ROWS, n_rows - r0);
            if ((rc = head_chunk(r0, nr))) return rc;
            const int n_w = std::max(0, std::min(n_want - r0, nr));
            if (n_w > 0) {
                CK(cudaStreamSynchronize(st));
                memcpy(host_logits + (size_t)r0 * V, m->logits_host, (size_t)n_w * V * 4);
            }
        }
    }
    for (int i = 0; i < n; i++) e->slots[slots[i]].n_past += n_tokens[i];
    for (int i = 0; i < n; i++) {
        if (host_sampled) host_sampled[i] = -1;
        if (samp_row[i] >= 0) { if ((rc = b2_sample_enqueue(e, e->slots[slots[i]], i))) return rc; }
    }
    CK(cudaStreamSynchronize(st));
    if ((rc = b2_check_kernel_error())) return rc;
    if (host_sampled) for (int i = 0; i < n; i++) if (samp_row[i] >= 0) host_sampled[i] = e->pinned[i];
    if (m->profile) {
        for (int k = 0; k < 8; k++) { m->prof_ms[k] = 0.f; m->prof_n[k] = 0; }
        for (auto& pe : m->prof_ev) {
            float t = 0.f;
            cudaEventElapsedTime(&t, pe.second.first, pe.second.second);
            m->prof_ms[pe.first] += t; m->prof_n[pe.first]++;
        }
    }
    return B2_OK;
}

extern "C" int b2_step_trace(b2_engine* e, int on) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    CK(cudaSetDevice(m->c.device));
    if (on && !m->trace) {
        int rc = dev_alloc(m, (void**)&m->trace, (size_t)m->c.n_layer * m->c.max_step_tokens * m->c.n_embd * 4);
        if (rc) return rc;
    }
    if (!on) m->trace = nullptr;       // the buffer stays owned and is freed with the engine
    return B2_OK;
}

extern "C" int b2_step_trace_read(b2_engine* e, float* out, int n_layer, int T) {
    if (!e || !e->layered || !out) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    LayeredModel* m = e->layered;
    if (!m->trace) return b2_fail(B2_ERR_STATE, "tracing is off");
    if (n_layer != m->c.n_layer || T != m->last_T) return b2_fail(B2_ERR_ARG, "shape does not match the last step");
    CK(cudaSetDevice(m->c.device));
    const size_t W = m->c.n_embd;
    for (int l = 0; l < n_layer; l++)
        CK(cudaMemcpy(out + (size_t)l * T * W, m->trace + (size_t)l * m->c.max_step_tokens * W, (size_t)T * W * 4, cudaMemcpyDeviceToHost));
    return B2_OK;
}

extern "C" int b2_step_profile(b2_engine* e, int on) {
    if (!e || !e->layered) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    e->layered->profile = on != 0;
    return B2_OK;
}

extern "C" int b2_step_profile_read(b2_engine* e, float* ms, int32_t* nl) {
    if (!e || !e->layered || !ms || !nl) return b2_fail(B2_ERR_UNSUPPORTED, "not a layer-list engine");
    std::lock_guard<std::mutex> lk(e->mu);
    for (int k = 0; k < 8; k++) { ms[k] = e->layered->prof_ms[k]; nl[k] = e->layered->prof_n[k]; }
    return B2_OK;
}
