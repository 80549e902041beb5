// Softmax attention with a sink over the paged cache (layered.h: SinkAttnArgs): grouped query heads, sliding window, rotate-half
// rotation of the leading entries, optional unit-RMS queries and keys, one extra term exp(sink[h]) in every head's denominator,
// optional mixing of the heads' normalised weights across heads, sigmoid output gate. Scores, softmax, mixing and the weighted
// sums are 32-bit; only the cache pages may be bf16.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <stdlib.h>

#include <algorithm>

namespace b2 {

namespace {
__device__ __forceinline__ float sk_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ void sk_store(void* pool, int f32, size_t i, float v) {
    if (f32) reinterpret_cast<float*>(pool)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(pool)[i] = __float2bfloat16(v);
}
template <bool F32>
__device__ __forceinline__ float sk_load(const void* pool, size_t i) {
    if constexpr (F32) return reinterpret_cast<const float*>(pool)[i];
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(pool)[i]);
}
__device__ __forceinline__ float sk_gate(const SinkAttnArgs& a, int t, int h, int i) {
    if (!a.gate) return 1.f;
    return sk_sigmoid(a.gate[(size_t)t * a.ld_gate + (a.gate_per_head ? h : h * a.dv + i)]);
}
}  // namespace

constexpr int SK_MAXE = 8;       // key and value sizes <= 256

// grid (T), 8 warps: a warp per head vector of q (H of them) and of k (G): rotation, optional unit RMS, q into scratch and k into
// its page; then the values into theirs.
__global__ void __launch_bounds__(256) sink_attn_store_kernel(SinkAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float* row = a.proj + (size_t)t * a.ldp;
    const int pos = r.tok_pos[t], d = a.d, half = a.rot.rot_dims / 2;
    const size_t page = a.block_tables[r.seg_slot[r.tok_seg[t]]][pos / a.block_tokens];
    const int in_page = pos % a.block_tokens;
    const float* cs = a.rot.cos + (size_t)pos * half;
    const float* sn = a.rot.sin + (size_t)pos * half;
    for (int hv = warp; hv < a.H + a.G; hv += nw) {
        const bool is_q = hv < a.H;
        const int head = is_q ? hv : hv - a.H;
        const float* x = row + (is_q ? a.q_off : a.k_off) + (size_t)head * d;
        float v[SK_MAXE];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < SK_MAXE; e++) {
            const int i = lane + 32 * e;
            float o = 0.f;
            if (i < d) {
                o = x[i];
                if (i < half) o = o * cs[i] - x[i + half] * sn[i];
                else if (i < 2 * half) o = o * cs[i - half] + x[i - half] * sn[i - half];
            }
            v[e] = o;
            ss = fmaf(o, o, ss);
        }
        const float mul = a.unit_qk ? 1.f / sqrtf(warp_sum(ss) / (float)d + a.eps) : 1.f;
#pragma unroll
        for (int e = 0; e < SK_MAXE; e++) {
            const int i = lane + 32 * e;
            if (i >= d) continue;
            if (is_q) a.q_rot[((size_t)t * a.H + head) * d + i] = v[e] * mul;
            else sk_store(a.k_pool, a.cache_f32, ((page * a.G + head) * a.block_tokens + in_page) * d + i, v[e] * mul);
        }
    }
    const int nv = a.G * a.dv;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / a.dv, c = i - g * a.dv;
        sk_store(a.v_pool, a.cache_f32, ((page * a.G + g) * a.block_tokens + in_page) * a.dv + c, row[a.v_off + i]);
    }
}
cudaError_t sink_attn_store_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > SK_MAXE * 32 || a.rot.rot_dims > a.d || a.rot.rot_dims % 2) return cudaErrorInvalidValue;
    return launch_chain(sink_attn_store_kernel, dim3(r.T), dim3(256), 0, s, a, r);
}

// grid (T, H, Gv), 8 warps. Query head h of token t against the keys of its own key head; the weights are applied to the values
// of value head c = blockIdx.z when the heads' weights are mixed afterwards (Gv = G), else of the head's own (Gv = 1). A warp
// takes 4 visible keys per round and keeps a running maximum, sum and output of its own; the warps are merged once, in warp
// order, together with the sink term.
constexpr int SK_WARPS = 8, SK_KEYS = 4;
template <bool F32>
__global__ void __launch_bounds__(SK_WARPS * 32) sink_attn_kernel(SinkAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_o[SK_WARPS][SK_MAXE * 32];
    __shared__ float sm_m[SK_WARPS], sm_l[SK_WARPS];
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int* table = a.block_tables[r.seg_slot[r.tok_seg[t]]];
    const int g = h / (a.H / a.G), d = a.d, dv = a.dv;
    const int vg = a.talk ? (int)blockIdx.z : g;
    const float* q = a.q_rot + ((size_t)t * a.H + h) * d;
    float qr[SK_MAXE], acc[SK_MAXE];
#pragma unroll
    for (int e = 0; e < SK_MAXE; e++) { const int i = lane + 32 * e; qr[e] = i < d ? q[i] * a.scale : 0.f; acc[e] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    for (int j0 = lo + warp * SK_KEYS; j0 <= pos; j0 += SK_WARPS * SK_KEYS) {
        size_t kb[SK_KEYS], vb[SK_KEYS];
        float sc[SK_KEYS];
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) {
            const int j = min(j0 + u, pos);                   // past the end: the last key again, its weight is dropped below
            const size_t page = table[j / a.block_tokens];
            kb[u] = ((page * a.G + g) * a.block_tokens + j % a.block_tokens) * d;
            vb[u] = ((page * a.G + vg) * a.block_tokens + j % a.block_tokens) * dv;
        }
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < SK_MAXE; e++) { const int i = lane + 32 * e; if (i < d) dot = fmaf(qr[e], sk_load<F32>(a.k_pool, kb[u] + i), dot); }
            sc[u] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < SK_KEYS; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
        float mx = m_run;
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) if (j0 + u <= pos) mx = fmaxf(mx, sc[u]);
        const float corr = expf(m_run - mx);                  // 0 at the first round (m_run = -inf, mx finite)
        l_run *= corr;
#pragma unroll
        for (int e = 0; e < SK_MAXE; e++) acc[e] *= corr;
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) {
            const float p = j0 + u <= pos ? expf(sc[u] - mx) : 0.f;
            l_run += p;
#pragma unroll
            for (int e = 0; e < SK_MAXE; e++) { const int i = lane + 32 * e; if (i < dv) acc[e] = fmaf(p, sk_load<F32>(a.v_pool, vb[u] + i), acc[e]); }
        }
        m_run = mx;
    }
#pragma unroll
    for (int e = 0; e < SK_MAXE; e++) sm_o[warp][lane + 32 * e] = acc[e];
    if (lane == 0) { sm_m[warp] = m_run; sm_l[warp] = l_run; }
    __syncthreads();
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float m = sink;
#pragma unroll
    for (int w2 = 0; w2 < SK_WARPS; w2++) m = fmaxf(m, sm_m[w2]);
    float l = a.sink ? expf(sink - m) : 0.f;
    float f[SK_WARPS];
#pragma unroll
    for (int w2 = 0; w2 < SK_WARPS; w2++) { f[w2] = sm_m[w2] > -INFINITY ? expf(sm_m[w2] - m) : 0.f; l = fmaf(sm_l[w2], f[w2], l); }
    const float inv = 1.f / l;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < SK_WARPS; w2++) o = fmaf(sm_o[w2][i], f[w2], o);
        o *= inv;
        if (a.talk) a.cross[(((size_t)t * a.H + h) * a.G + vg) * dv + i] = o;
        else a.out[(size_t)t * a.ld_out + (size_t)h * dv + i] = o * sk_gate(a, t, h, i);
    }
}

// grid (T): out_h = gate_h * sum_g talk[h][g] A[g][c(h)], the sum in head order
__global__ void __launch_bounds__(256) sink_attn_talk_kernel(SinkAttnArgs a, int T) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, H = a.H, G = a.G, dv = a.dv;
    for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
        const int h = e / dv, i = e - h * dv, c = h / (H / G);
        float o = 0.f;
        for (int g = 0; g < H; g++) o = fmaf(a.talk[h * H + g], a.cross[(((size_t)t * H + g) * G + c) * dv + i], o);
        a.out[(size_t)t * a.ld_out + e] = o * sk_gate(a, t, h, i);
    }
}

cudaError_t sink_attn_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > SK_MAXE * 32 || a.dv > SK_MAXE * 32 || a.H % a.G) return cudaErrorInvalidValue;
    const dim3 grid(r.T, a.H, a.talk ? a.G : 1);
    cudaError_t e = a.cache_f32 ? launch_chain(sink_attn_kernel<true>, grid, dim3(SK_WARPS * 32), 0, s, a, r)
                                : launch_chain(sink_attn_kernel<false>, grid, dim3(SK_WARPS * 32), 0, s, a, r);
    if (e != cudaSuccess || !a.talk) return e;
    return launch_chain(sink_attn_talk_kernel, dim3(r.T), dim3(256), 0, s, a, r.T);
}

}  // namespace b2
