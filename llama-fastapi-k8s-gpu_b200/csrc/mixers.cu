// Token mixers and norms of the layer-list models, over a ragged step (layered.h): post-sum layer norm with RMS-normed
// branches, sliding-window attention with a kept prefix over the paged cache (query/key norm, partial interleaved
// rotary with blended frequencies, values = un-normalised keys), selective scan (causal depthwise convolution +
// diagonal state recurrence), and the mLSTM matrix memory. Softmax, norms, gates, decays and all recurrent state are
// 32-bit; only the cache pages may be bf16. Every recurrence walks a segment's tokens in order from the state its
// slot holds, so a sequence cut into portions gives the same numbers as the whole.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <stdlib.h>

#include <algorithm>

namespace b2 {

__device__ __forceinline__ float block_sum(float v, float* red) {      // all threads get the sum; red: >= 33 floats
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ void cp_async_4(float* smem_dst, const float* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return -softplus_f(-z); }

// ---------------------------------------------------------------- embedding, gather
template <typename TW>
__global__ void embed_ragged_kernel(const TW* __restrict__ table, int W, const int* __restrict__ tok, float* __restrict__ x, float scale) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const TW* row = table + (size_t)tok[t] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        if constexpr (sizeof(TW) == 2) x[(size_t)t * W + i] = __bfloat162float(row[i]) * scale;
        else x[(size_t)t * W + i] = row[i] * scale;
    }
}
cudaError_t embed_ragged_launch(const void* table, int w_type, int W, const int* tok_id, int T, float* x, float scale, cudaStream_t s) {
    if (w_type == T_BF16) return launch_chain(embed_ragged_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, s, (const __nv_bfloat16*)table, W, tok_id, x, scale);
    if (w_type == T_F32) return launch_chain(embed_ragged_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)table, W, tok_id, x, scale);
    return cudaErrorInvalidValue;
}

__global__ void gather_rows_kernel(const float* __restrict__ x, int W, const int* __restrict__ rows, float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    const float* src = x + (size_t)rows[blockIdx.x] * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[(size_t)blockIdx.x * W + i] = src[i];
}
cudaError_t gather_rows_launch(const float* x, int W, const int* rows, int n, float* y, cudaStream_t s) {
    return launch_chain(gather_rows_kernel, dim3(n), dim3(128), 0, s, x, W, rows, y);
}

// ---------------------------------------------------------------- norms
// one CTA per token; the row lives in shared memory between the passes (mean, then squared deviations)
__global__ void __launch_bounds__(256) postsum_norm_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ wa,
                                                           const float* __restrict__ b, const float* __restrict__ wb,
                                                           const float* __restrict__ w, float alpha, float eps, int W) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * W;
    float ra = 1.f, rb = 1.f;
    if (b) {
        float sa = 0.f, sb = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) { const float u = a[base + i], v = b[base + i]; sa += u * u; sb += v * v; }
        sa = block_sum(sa, red); sb = block_sum(sb, red);
        ra = 1.f / sqrtf(sa / (float)W + eps); rb = 1.f / sqrtf(sb / (float)W + eps);
    }
    float sum = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float yv = b ? 0.5f * (a[base + i] * ra * wa[i] + b[base + i] * rb * wb[i]) : (a ? a[base + i] : 0.f);
        const float v = alpha * x[base + i] + yv;
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, red) / (float)W;
    float sq = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float dlt = row[i] - mean; sq += dlt * dlt; }
    const float rstd = 1.f / sqrtf(block_sum(sq, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) x[base + i] = (row[i] - mean) * rstd * w[i];
}
cudaError_t postsum_norm_launch(float* x, const float* a, const float* wa, const float* b, const float* wb, const float* w,
                                float alpha, float eps, int W, int T, cudaStream_t s) {
    return launch_chain(postsum_norm_kernel, dim3(T), dim3(256), (size_t)W * 4, s, x, a, wa, b, wb, w, alpha, eps, W);
}

// pre-norm blocks: the pending branch output joins the 32-bit residual stream, and the next sublayer's input is made in the same pass
__global__ void __launch_bounds__(256) resid_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ add, float mult,
                                                             const float* __restrict__ w, float w_offset, float out_scale, float eps, int W,
                                                             float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = x[base + i];
        if (add) { v = fmaf(mult, add[base + i], v); x[base + i] = v; }
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!y) return;
    const float rinv = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[base + i] = row[i] * rinv * (w_offset + w[i]) * out_scale;
}
cudaError_t resid_rms_norm_launch(float* x, const float* add, float mult, const float* w, float w_offset, float out_scale,
                                  float eps, int W, int T, float* y, cudaStream_t s) {
    return launch_chain(resid_rms_norm_kernel, dim3(T), dim3(256), (size_t)W * 4, s, x, add, mult, w, w_offset, out_scale, eps, W, y);
}

__global__ void __launch_bounds__(256) layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int W,
                                                         float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * W;
    float sum = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) sum += x[base + i];
    const float mean = block_sum(sum, red) / (float)W;
    float sq = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float dlt = x[base + i] - mean; sq += dlt * dlt; }
    const float rstd = 1.f / sqrtf(block_sum(sq, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[base + i] = (x[base + i] - mean) * rstd * w[i];
}
cudaError_t layer_norm_launch(const float* x, const float* w, float eps, int W, int T, float* y, cudaStream_t s) {
    return launch_chain(layer_norm_kernel, dim3(T), dim3(256), 0, s, x, w, eps, W, y);
}

// ---------------------------------------------------------------- window attention
__device__ __forceinline__ void cache_store(void* pool, int f32, size_t i, float v) {
    if (f32) reinterpret_cast<float*>(pool)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(pool)[i] = __float2bfloat16(v);
}
__device__ __forceinline__ float cache_load(const void* pool, int f32, size_t i) {
    return f32 ? reinterpret_cast<const float*>(pool)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(pool)[i]);
}

// grid (T, H + G), one warp: head slots [0, H) are queries, [H, H + G) are key/value heads
__global__ void __launch_bounds__(32) window_attn_store_kernel(WindowAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, hs = blockIdx.y, lane = threadIdx.x;
    const bool is_q = hs < a.H;
    const int head = is_q ? hs : hs - a.H;
    const float* src = a.proj + (size_t)t * a.ldp + (is_q ? a.q_off : a.k_off) + head * a.d;
    const float* nw = is_q ? a.q_norm_w : a.k_norm_w;
    const int pos = r.tok_pos[t];
    float ss = 0.f;
    for (int i = lane; i < a.d; i += 32) { const float v = src[i]; ss += v * v; }
    const float rinv = 1.f / sqrtf(warp_sum(ss) / (float)a.d + a.eps);
    size_t dst = 0;
    if (!is_q) {
        const int slot = r.seg_slot[r.tok_seg[t]];
        const int page = a.block_tables[slot][pos / a.block_tokens];
        dst = (((size_t)page * a.G + head) * a.block_tokens + pos % a.block_tokens) * a.d;
    }
    float* qdst = a.q_rot + (size_t)t * a.H * a.d + (size_t)head * a.d;
    // pairs (2i, 2i+1): rotated inside the first rot_dims entries, passed through after them
    for (int p = lane; 2 * p < a.d; p += 32) {
        const int i0 = 2 * p, i1 = 2 * p + 1;
        const float r0 = src[i0], r1 = i1 < a.d ? src[i1] : 0.f;
        float u = r0 * rinv * nw[i0], v = i1 < a.d ? r1 * rinv * nw[i1] : 0.f;
        if (i1 < a.rot.rot_dims) {
            const size_t ti = (size_t)pos * (a.rot.rot_dims / 2) + p;
            const float sn = a.rot.sin[ti], cs = a.rot.cos[ti];
            const float u2 = u * cs - v * sn, v2 = v * cs + u * sn;
            u = u2; v = v2;
        }
        if (is_q) {
            qdst[i0] = u;
            if (i1 < a.d) qdst[i1] = v;
        } else {
            cache_store(a.k_pool, a.cache_f32, dst + i0, u);
            cache_store(a.v_pool, a.cache_f32, dst + i0, r0);
            if (i1 < a.d) { cache_store(a.k_pool, a.cache_f32, dst + i1, v); cache_store(a.v_pool, a.cache_f32, dst + i1, r1); }
        }
    }
}
cudaError_t window_attn_store_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(window_attn_store_kernel, dim3(r.T, a.H + a.G), dim3(32), 0, s, a, r);
}

// grid (T, H), 4 warps: warp w takes visible keys w, w + 4, ...; a lane holds entries lane, lane + 32, ... of the head
constexpr int ATT_WARPS = 4, ATT_MAXE = 8;     // head size <= 256
__global__ void __launch_bounds__(ATT_WARPS * 32) window_attn_kernel(WindowAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_m[ATT_WARPS], sm_l[ATT_WARPS];
    __shared__ float sm_o[ATT_WARPS][ATT_MAXE * 32];
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int slot = r.seg_slot[r.tok_seg[t]];
    const int* table = a.block_tables[slot];
    const int g = h / (a.H / a.G);
    const float* q = a.q_rot + (size_t)t * a.H * a.d + (size_t)h * a.d;
    float qr[ATT_MAXE], acc[ATT_MAXE];
#pragma unroll
    for (int e = 0; e < ATT_MAXE; e++) { const int i = lane + 32 * e; qr[e] = i < a.d ? q[i] * a.scale : 0.f; acc[e] = 0.f; }
    // visible: the kept prefix [0, n_keep) and the window [lo, pos]
    const int lo = max(0, pos - a.window + 1);
    const int n_keep = min(a.keep_first, lo);
    const int n_vis = n_keep + (pos - lo + 1);
    float m = -INFINITY, l = 0.f;
    for (int i = warp; i < n_vis; i += ATT_WARPS) {
        const int j = i < n_keep ? i : lo + (i - n_keep);
        const size_t base = (((size_t)table[j / a.block_tokens] * a.G + g) * a.block_tokens + j % a.block_tokens) * a.d;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < ATT_MAXE; e++) { const int d = lane + 32 * e; if (d < a.d) dot = fmaf(qr[e], cache_load(a.k_pool, a.cache_f32, base + d), dot); }
        const float sc = warp_sum(dot);
        const float m_new = fmaxf(m, sc);
        const float corr = expf(m - m_new), p = expf(sc - m_new);
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < ATT_MAXE; e++) { const int d = lane + 32 * e; if (d < a.d) acc[e] = fmaf(p, cache_load(a.v_pool, a.cache_f32, base + d), acc[e] * corr); }
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < ATT_MAXE; e++) sm_o[warp][lane + 32 * e] = acc[e];
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < ATT_WARPS; w2++) M = fmaxf(M, sm_m[w2]);
    float L = 0.f;
    for (int w2 = 0; w2 < ATT_WARPS; w2++) if (sm_m[w2] > -INFINITY) L += sm_l[w2] * expf(sm_m[w2] - M);
    for (int d = threadIdx.x; d < a.d; d += blockDim.x) {
        float o = 0.f;
        for (int w2 = 0; w2 < ATT_WARPS; w2++) if (sm_m[w2] > -INFINITY) o += sm_o[w2][d] * expf(sm_m[w2] - M);
        a.out[(size_t)t * a.H * a.d + (size_t)h * a.d + d] = o / L;
    }
}
// Even head sizes: 8 warps, a warp takes 4 visible keys per round (their loads and the four dot-product reductions overlap),
// a lane holds pairs of neighbouring entries (one 4- or 8-byte load per key and 64 entries of the head).
constexpr int ATT2_WARPS = 8, ATT2_KEYS = 4, ATT2_PASS = 4;       // head size <= 256
template <bool F32>
__device__ __forceinline__ float2 cache_load2(const void* pool, size_t i) {
    if constexpr (F32) return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(pool) + i);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(pool) + i);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <bool F32>
__global__ void __launch_bounds__(ATT2_WARPS * 32) window_attn_pairs_kernel(WindowAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_m[ATT2_WARPS], sm_l[ATT2_WARPS];
    __shared__ float sm_o[ATT2_WARPS][ATT2_PASS * 64];
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int slot = r.seg_slot[r.tok_seg[t]];
    const int* table = a.block_tables[slot];
    const int g = h / (a.H / a.G), d = a.d;
    const float* q = a.q_rot + (size_t)t * a.H * d + (size_t)h * d;
    float2 qr[ATT2_PASS], acc[ATT2_PASS];
#pragma unroll
    for (int e = 0; e < ATT2_PASS; e++) {
        const int i = 64 * e + 2 * lane;
        qr[e] = i < d ? make_float2(q[i] * a.scale, q[i + 1] * a.scale) : make_float2(0.f, 0.f);
        acc[e] = make_float2(0.f, 0.f);
    }
    const int lo = max(0, pos - a.window + 1);
    const int n_keep = min(a.keep_first, lo);
    const int n_all = n_keep + (pos - lo + 1);
    // several CTAs per (token, head) when the step is small: CTA z takes the z-th range of the visible keys
    const int n_splits = gridDim.z, chunk = (n_all + n_splits - 1) / n_splits;
    const int i_begin = blockIdx.z * chunk, n_vis = min(n_all, i_begin + chunk);
    float m = -INFINITY, l = 0.f;
    for (int i0 = i_begin + warp * ATT2_KEYS; i0 < n_vis; i0 += ATT2_WARPS * ATT2_KEYS) {
        size_t base[ATT2_KEYS];
        float2 kv[ATT2_KEYS][ATT2_PASS], vv[ATT2_KEYS][ATT2_PASS];
        float sc[ATT2_KEYS];
#pragma unroll
        for (int u = 0; u < ATT2_KEYS; u++) {
            const int i = min(i0 + u, n_vis - 1);         // past the end: the last key again, its weight is dropped below
            const int j = i < n_keep ? i : lo + (i - n_keep);
            base[u] = (((size_t)table[j / a.block_tokens] * a.G + g) * a.block_tokens + j % a.block_tokens) * d;
        }
#pragma unroll
        for (int u = 0; u < ATT2_KEYS; u++)
#pragma unroll
            for (int e = 0; e < ATT2_PASS; e++) {
                const int i = 64 * e + 2 * lane;
                kv[u][e] = i < d ? cache_load2<F32>(a.k_pool, base[u] + i) : make_float2(0.f, 0.f);
                vv[u][e] = i < d ? cache_load2<F32>(a.v_pool, base[u] + i) : make_float2(0.f, 0.f);
            }
#pragma unroll
        for (int u = 0; u < ATT2_KEYS; u++) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < ATT2_PASS; e++) dot = fmaf(qr[e].x, kv[u][e].x, fmaf(qr[e].y, kv[u][e].y, dot));
            sc[u] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < ATT2_KEYS; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
        float m_new = m;
#pragma unroll
        for (int u = 0; u < ATT2_KEYS; u++) if (i0 + u < n_vis) m_new = fmaxf(m_new, sc[u]);
        const float corr = expf(m - m_new);
        float p[ATT2_KEYS], ps = 0.f;
#pragma unroll
        for (int u = 0; u < ATT2_KEYS; u++) { p[u] = i0 + u < n_vis ? expf(sc[u] - m_new) : 0.f; ps += p[u]; }
        l = l * corr + ps;
#pragma unroll
        for (int e = 0; e < ATT2_PASS; e++) {
            float ax = acc[e].x * corr, ay = acc[e].y * corr;
#pragma unroll
            for (int u = 0; u < ATT2_KEYS; u++) { ax = fmaf(p[u], vv[u][e].x, ax); ay = fmaf(p[u], vv[u][e].y, ay); }
            acc[e] = make_float2(ax, ay);
        }
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < ATT2_PASS; e++) { sm_o[warp][64 * e + 2 * lane] = acc[e].x; sm_o[warp][64 * e + 2 * lane + 1] = acc[e].y; }
    __syncthreads();
    float M = -INFINITY;
    for (int w2 = 0; w2 < ATT2_WARPS; w2++) M = fmaxf(M, sm_m[w2]);
    float L = 0.f;
    for (int w2 = 0; w2 < ATT2_WARPS; w2++) if (sm_m[w2] > -INFINITY) L += sm_l[w2] * expf(sm_m[w2] - M);
    float* part = n_splits > 1 ? a.split_scratch + (((size_t)t * a.H + h) * n_splits + blockIdx.z) * (d + 2) : nullptr;
    if (part && threadIdx.x == 0) { part[0] = M; part[1] = L; }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float o = 0.f;
        for (int w2 = 0; w2 < ATT2_WARPS; w2++) if (sm_m[w2] > -INFINITY) o += sm_o[w2][i] * expf(sm_m[w2] - M);
        if (part) part[2 + i] = o;                         // unnormalised: window_attn_merge_kernel finishes
        else a.out[(size_t)t * a.H * d + (size_t)h * d + i] = o / L;
    }
}

// sum of the key ranges of one (token, head) in range order
__global__ void __launch_bounds__(128) window_attn_merge_kernel(WindowAttnArgs a, int n_splits) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, h = blockIdx.y, d = a.d;
    const float* part = a.split_scratch + ((size_t)t * a.H + h) * n_splits * (d + 2);
    float M = -INFINITY;
    for (int s2 = 0; s2 < n_splits; s2++) M = fmaxf(M, part[(size_t)s2 * (d + 2)]);
    float L = 0.f;
    for (int s2 = 0; s2 < n_splits; s2++) { const float ms = part[(size_t)s2 * (d + 2)]; if (ms > -INFINITY) L += part[(size_t)s2 * (d + 2) + 1] * expf(ms - M); }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float o = 0.f;
        for (int s2 = 0; s2 < n_splits; s2++) { const float ms = part[(size_t)s2 * (d + 2)]; if (ms > -INFINITY) o += part[(size_t)s2 * (d + 2) + 2 + i] * expf(ms - M); }
        a.out[(size_t)t * a.H * d + (size_t)h * d + i] = o / L;
    }
}

// Tensor-core prompt attention (bf16 pages, head size a multiple of 16 up to 128): a CTA takes one tile of up to 64 consecutive
// queries of a segment and one head; 4 warps x 16 query rows; keys in blocks of 64 -- first the blocks that hold kept-prefix
// keys, then the blocks the tile's windows reach -- staged in shared memory once for all 64 queries. S = Q K^T and O += P V
// with mma.sync m16n8k16 (bf16 in, f32 accumulate); mask, running maximum, exponentials and the sum are 32-bit. Queries and
// probabilities enter the products as TWO bf16 each (value = leading part + remainder), so the only 16-bit rounding on this
// path is that of the cached keys and values -- the same as on the decode path.
constexpr int FA_Q = 64, FA_K = 64;
__device__ __forceinline__ void cp_async_16z(void* smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_bf16(a - __low2float(h), b - __high2float(h));
}

template <int DMAX>
__global__ void __launch_bounds__(128) window_attn_mma_kernel(WindowAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char fa_smem[];
    const int d = a.d, LD = d + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(fa_smem);     // [64][LD] leading bf16 of the scaled query
    __nv_bfloat16* Ql = Qs + FA_Q * LD;                                 // [64][LD] what the first bf16 leaves over
    __nv_bfloat16* Ks = Ql + FA_Q * LD;
    __nv_bfloat16* Vs = Ks + FA_K * LD;
    const int tile = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(FA_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const int g = h / (a.H / a.G);
    const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(a.k_pool);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(a.v_pool);
    // queries: scaled, rounded to bf16; rows past the tile are zero
    for (int i = threadIdx.x; i < FA_Q * (d / 2); i += blockDim.x) {
        const int rr = i / (d / 2), c = (i % (d / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (rr < nq) {
            const float* q = a.q_rot + (size_t)(row0 + rr) * a.H * d + (size_t)h * d + c;
            v = make_float2(q[0] * a.scale, q[1] * a.scale);
        }
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(Qs + rr * LD + c) = hi;
        *reinterpret_cast<__nv_bfloat162*>(Ql + rr * LD + c) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
    }
    const int lo_first = max(0, p0 - a.window + 1);
    const int n_kept_blocks = lo_first > 0 ? (min(a.keep_first, lo_first) + FA_K - 1) / FA_K : 0;
    const int win_b0 = max(lo_first / FA_K, n_kept_blocks), win_b1 = p_last / FA_K;
    const int n_blocks = n_kept_blocks + (win_b1 - win_b0 + 1);
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    for (int bi = 0; bi < n_blocks; bi++) {
        const int kb = bi < n_kept_blocks ? bi : win_b0 + (bi - n_kept_blocks);
        const int j0 = kb * FA_K;
        __syncthreads();                      // everybody is done with the previous block's K and V (and Q is written)
        for (int i = threadIdx.x; i < FA_K * (d / 8); i += blockDim.x) {
            const int rr = i / (d / 8), c = (i % (d / 8)) * 8;
            const int j = j0 + rr;
            const int jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + g) * a.block_tokens + jj % a.block_tokens) * d + c;
            cp_async_16z(Ks + rr * LD + c, kp + base, j <= p_last ? 16 : 0);
            cp_async_16z(Vs + rr * LD + c, vp + base, j <= p_last ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();
        // S = Q K^T for this warp's 16 rows
        float sacc[FA_K / 8][4];
#pragma unroll
        for (int ni = 0; ni < FA_K / 8; ni++) sacc[ni][0] = sacc[ni][1] = sacc[ni][2] = sacc[ni][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DMAX; ks += 16) {
            if (ks < d) {
                uint32_t af[4], al[4];
                ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
                ldsm_x4(al, Ql + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
#pragma unroll
                for (int nj = 0; nj < FA_K / 16; nj++) {
                    uint32_t bf[4];
                    ldsm_x4(bf, Ks + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks + ((lane >> 3) & 1) * 8);
                    mma_16816(sacc[2 * nj], al, bf[0], bf[1]);
                    mma_16816(sacc[2 * nj + 1], al, bf[2], bf[3]);
                    mma_16816(sacc[2 * nj], af, bf[0], bf[1]);
                    mma_16816(sacc[2 * nj + 1], af, bf[2], bf[3]);
                }
            }
        }
        // mask, running maximum, exponentials
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int ni = 0; ni < FA_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int rr = qrow[e >> 1], i = p0 + rr, j = j0 + ni * 8 + 2 * tq + (e & 1);
                const bool vis = rr < nq && j <= i && (i - j < a.window || j < a.keep_first);
                const float v = vis ? sacc[ni][e] : -INFINITY;
                sacc[ni][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float corr[2], msafe[2];
#pragma unroll
        for (int q2 = 0; q2 < 2; q2++) {
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 1));
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 2));
            const float m_new = fmaxf(m_run[q2], mx[q2]);
            msafe[q2] = m_new == -INFINITY ? 0.f : m_new;
            corr[q2] = expf(m_run[q2] - msafe[q2]);
            m_run[q2] = m_new;
            l_run[q2] *= corr[q2];
        }
#pragma unroll
        for (int ni = 0; ni < FA_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pv = expf(sacc[ni][e] - msafe[e >> 1]);
                sacc[ni][e] = pv;
                l_run[e >> 1] += pv;
            }
#pragma unroll
        for (int i = 0; i < DMAX / 8; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // O += P V
#pragma unroll
        for (int kc = 0; kc < FA_K / 16; kc++) {
            uint32_t pf[4], pl[4];         // probabilities as two bf16 each (leading part + remainder): ~16 bits reach the product
            split_bf16(sacc[2 * kc][0], sacc[2 * kc][1], pf[0], pl[0]);
            split_bf16(sacc[2 * kc][2], sacc[2 * kc][3], pf[1], pl[1]);
            split_bf16(sacc[2 * kc + 1][0], sacc[2 * kc + 1][1], pf[2], pl[2]);
            split_bf16(sacc[2 * kc + 1][2], sacc[2 * kc + 1][3], pf[3], pl[3]);
#pragma unroll
            for (int nd = 0; nd < DMAX / 16; nd++) {
                if (nd * 16 < d) {
                    uint32_t vf[4];
                    ldsm_x4_t(vf, Vs + (kc * 16 + (lane & 15)) * LD + nd * 16 + (lane >> 4) * 8);
                    mma_16816(o[2 * nd], pl, vf[0], vf[1]);
                    mma_16816(o[2 * nd + 1], pl, vf[2], vf[3]);
                    mma_16816(o[2 * nd], pf, vf[0], vf[1]);
                    mma_16816(o[2 * nd + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        l_run[q2] += __shfl_xor_sync(0xffffffffu, l_run[q2], 1);
        l_run[q2] += __shfl_xor_sync(0xffffffffu, l_run[q2], 2);
    }
#pragma unroll
    for (int i = 0; i < DMAX / 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int rr = qrow[e >> 1], c = i * 8 + 2 * tq + (e & 1);
            if (rr < nq && c < d) a.out[(size_t)(row0 + rr) * a.H * d + (size_t)h * d + c] = o[i][e] / l_run[e >> 1];
        }
}

cudaError_t window_attn_launch(const WindowAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > ATT_MAXE * 32) return cudaErrorInvalidValue;
    static const bool no_mma = getenv("B2_NO_ATTN_MMA") != nullptr;        // tuning aid: scalar attention for prompts too
    if (!no_mma && !a.cache_f32 && r.T > 8 && a.d % 16 == 0 && a.d <= 128) {
        static bool attr_done = false;
        if (!attr_done) {
            cudaFuncSetAttribute(window_attn_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * (64 + 8) * 2);
            cudaFuncSetAttribute(window_attn_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * (128 + 8) * 2);
            attr_done = true;
        }
        const size_t smem = (size_t)4 * 64 * (a.d + 8) * 2;
        if (a.d <= 64) return launch_chain(window_attn_mma_kernel<64>, dim3(r.n_tiles, a.H), dim3(128), smem, s, a, r);
        return launch_chain(window_attn_mma_kernel<128>, dim3(r.n_tiles, a.H), dim3(128), smem, s, a, r);
    }
    if (a.d % 2 == 0) {
        // a step of a few tokens does not fill the GPU with one CTA per (token, head): split the keys (up to 16 ranges)
        int splits = 1;
        if (a.split_scratch && r.T * a.H < 148) {
            splits = std::min(16, (2 * 148) / (r.T * a.H));
            while (splits > 1 && (size_t)r.T * a.H * splits * (a.d + 2) > (size_t)a.split_capacity) splits--;
        }
        const dim3 grid(r.T, a.H, splits);
        cudaError_t ce = a.cache_f32 ? launch_chain(window_attn_pairs_kernel<true>, grid, dim3(ATT2_WARPS * 32), 0, s, a, r)
                                     : launch_chain(window_attn_pairs_kernel<false>, grid, dim3(ATT2_WARPS * 32), 0, s, a, r);
        if (ce != cudaSuccess || splits == 1) return ce;
        return launch_chain(window_attn_merge_kernel, dim3(r.T, a.H), dim3(128), 0, s, a, splits);
    }
    return launch_chain(window_attn_kernel, dim3(r.T, a.H), dim3(ATT_WARPS * 32), 0, s, a, r);
}

// ---------------------------------------------------------------- selective scan
// xc[t][c] = silu(bias[c] + sum_j w[c][j] * in[t - (taps-1) + j][c]); inputs before the segment come from the slot's state
__global__ void __launch_bounds__(256) scan_conv_kernel(ScanArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int seg = r.tok_seg[t], slot = r.seg_slot[seg], i = t - r.seg_start[seg];
    const int hist = a.taps - 1;
    for (int c = threadIdx.x; c < a.inner; c += blockDim.x) {
        float acc = a.conv_b[c];
        for (int j = 0; j < a.taps; j++) {
            const int srci = i - hist + j;
            const float v = srci >= 0 ? a.proj[(size_t)(t - i + srci) * a.ldp + a.x_off + c]
                                      : a.conv_state[((size_t)slot * a.inner + c) * hist + (hist + srci)];
            acc = fmaf(a.conv_w[(size_t)c * a.taps + j], v, acc);
        }
        a.xc[(size_t)t * a.inner + c] = silu_f(acc);
    }
}
cudaError_t scan_conv_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(scan_conv_kernel, dim3(r.T), dim3(256), 0, s, a, r);
}

// grid (n_seg, inner / 8): a warp per channel, lanes over the states (SCAN_MAXS per lane)
constexpr int SCAN_MAXS = 8;       // state size <= 256
__global__ void __launch_bounds__(256) scan_recurrence_kernel(ScanArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int seg = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.y * 8 + warp;
    if (c >= a.inner) return;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int hist = a.taps - 1;
    // the convolution's memory moves on: the last taps-1 inputs of the sequence (read before written: index k + len > k)
    if (lane == 0) {
        float* st = a.conv_state + ((size_t)slot * a.inner + c) * hist;
        for (int k = 0; k < hist; k++) {
            const int srci = len + k - hist;
            st[k] = srci >= 0 ? a.proj[(size_t)(start + srci) * a.ldp + a.x_off + c] : st[k + len];
        }
    }
    float A[SCAN_MAXS], S[SCAN_MAXS];
    float* sst = a.ssm_state + ((size_t)slot * a.inner + c) * a.N;
#pragma unroll
    for (int e = 0; e < SCAN_MAXS; e++) {
        const int n = lane + 32 * e;
        A[e] = n < a.N ? -expf(a.A_log[(size_t)c * a.N + n]) : 0.f;
        S[e] = n < a.N ? sst[n] : 0.f;
    }
    const float Dc = a.D[c], dtb = a.dt_bias[c];
    for (int i = 0; i < len; i++) {
        const int t = start + i;
        const float dt = softplus_f(a.dt_raw[(size_t)t * a.inner + c] + dtb);
        const float xv = a.xc[(size_t)t * a.inner + c];
        const float* Bp = a.xproj + (size_t)t * a.ldx + a.R;
        const float* Cp = Bp + a.N;
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < SCAN_MAXS; e++) {
            const int n = lane + 32 * e;
            if (n < a.N) {
                S[e] = expf(dt * A[e]) * S[e] + dt * xv * Bp[n];
                part = fmaf(S[e], Cp[n], part);
            }
        }
        const float yv = warp_sum(part) + Dc * xv;
        if (lane == 0) a.y[(size_t)t * a.inner + c] = yv * silu_f(a.proj[(size_t)t * a.ldp + a.z_off + c]);
    }
#pragma unroll
    for (int e = 0; e < SCAN_MAXS; e++) { const int n = lane + 32 * e; if (n < a.N) sst[n] = S[e]; }
}
// Small states (N <= NMAX <= 64): a thread per channel keeps its N states in registers, the step's B and C rows are staged in
// shared memory for a block of tokens, and the next token's inputs are fetched while the current one is computed. No
// shuffles, every global access is coalesced over the channels. grid (n_seg, inner / SCAN_CH).
constexpr int SCAN_CH = 64, SCAN_TB = 16;
template <int NMAX>
__global__ void __launch_bounds__(SCAN_CH) scan_recurrence_chan_kernel(ScanArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float bc[];          // [SCAN_TB][2 N]
    const int seg = blockIdx.x, c = blockIdx.y * SCAN_CH + threadIdx.x;
    const bool ok = c < a.inner;
    const int cc = ok ? c : a.inner - 1;    // idle threads shadow the last channel (they still take part in the barriers)
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int hist = a.taps - 1, N = a.N;
    if (ok) {
        float* st = a.conv_state + ((size_t)slot * a.inner + c) * hist;
        for (int k = 0; k < hist; k++) {
            const int srci = len + k - hist;
            st[k] = srci >= 0 ? a.proj[(size_t)(start + srci) * a.ldp + a.x_off + c] : st[k + len];
        }
    }
    float A[NMAX], S[NMAX];
    float* sst = a.ssm_state + ((size_t)slot * a.inner + cc) * N;
#pragma unroll
    for (int n = 0; n < NMAX; n++) {
        A[n] = n < N ? -expf(a.A_log[(size_t)cc * N + n]) : 0.f;
        S[n] = n < N ? sst[n] : 0.f;
    }
    const float Dc = a.D[cc], dtb = a.dt_bias[cc];
    float n_dt = a.dt_raw[(size_t)start * a.inner + cc], n_x = a.xc[(size_t)start * a.inner + cc];
    float n_z = a.proj[(size_t)start * a.ldp + a.z_off + cc];
    for (int i0 = 0; i0 < len; i0 += SCAN_TB) {
        const int nb = min(SCAN_TB, len - i0);
        __syncthreads();
        for (int j = threadIdx.x; j < nb * 2 * N; j += SCAN_CH) {
            const int tt = j / (2 * N), e = j % (2 * N);
            bc[j] = a.xproj[(size_t)(start + i0 + tt) * a.ldx + a.R + e];
        }
        __syncthreads();
        for (int ii = 0; ii < nb; ii++) {
            const int t = start + i0 + ii;
            const float dt = softplus_f(n_dt + dtb), xv = n_x, zv = n_z;
            if (i0 + ii + 1 < len) {
                n_dt = a.dt_raw[(size_t)(t + 1) * a.inner + cc];
                n_x = a.xc[(size_t)(t + 1) * a.inner + cc];
                n_z = a.proj[(size_t)(t + 1) * a.ldp + a.z_off + cc];
            }
            const float* Bp = bc + ii * 2 * N;
            const float* Cp = Bp + N;
            const float dx = dt * xv;
            float yv = 0.f;
#pragma unroll
            for (int n = 0; n < NMAX; n++)
                if (n < N) {
                    S[n] = expf(dt * A[n]) * S[n] + dx * Bp[n];
                    yv = fmaf(S[n], Cp[n], yv);
                }
            if (ok) a.y[(size_t)t * a.inner + c] = (yv + Dc * xv) * silu_f(zv);
        }
    }
    if (ok) {
#pragma unroll
        for (int n = 0; n < NMAX; n++) if (n < N) sst[n] = S[n];
    }
}

// States up to a warp wide (N <= LPC <= 32): LPC lanes per channel, one state each, so a step keeps 16-32 times more warps in
// flight than a thread per channel; the read-out is a shuffle reduction over the LPC lanes. Step sizes and output gates are
// made beforehand, in place, by scan_prepare_kernel (softplus(dt + bias) over dt_raw, silu over the z columns); inputs are
// fetched four tokens ahead.
__global__ void scan_prepare_kernel(ScanArgs a, int T) {
    griddep_launch();
    griddep_wait();
    const long n = (long)T * a.inner;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long t = i / a.inner;
        const int c = (int)(i % a.inner);
        float* dtp = const_cast<float*>(a.dt_raw) + i;
        *dtp = softplus_f(*dtp + a.dt_bias[c]);
        float* zp = const_cast<float*>(a.proj) + t * a.ldp + a.z_off + c;
        *zp = silu_f(*zp);
    }
}

template <int LPC>
__global__ void __launch_bounds__(256) scan_recurrence_lanes_kernel(ScanArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    constexpr int CPB = 256 / LPC, AHEAD = 4;
    const int seg = blockIdx.x, n = threadIdx.x % LPC, c = blockIdx.y * CPB + threadIdx.x / LPC;
    const int N = a.N;
    const bool c_ok = c < a.inner, ok = c_ok && n < N;
    const int cc = c_ok ? c : a.inner - 1, nn = n < N ? n : 0;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int hist = a.taps - 1;
    if (c_ok && n == 0) {
        float* st = a.conv_state + ((size_t)slot * a.inner + c) * hist;
        for (int k = 0; k < hist; k++) {
            const int srci = len + k - hist;
            st[k] = srci >= 0 ? a.proj[(size_t)(start + srci) * a.ldp + a.x_off + c] : st[k + len];
        }
    }
    float* sst = a.ssm_state + ((size_t)slot * a.inner + cc) * N + nn;
    const float A = -expf(a.A_log[(size_t)cc * N + nn]);
    float S = ok ? *sst : 0.f;
    const float Dc = a.D[cc];
    struct In { float dt, x, B, C, gate; };
    auto fetch = [&](int i) {
        In v;
        const int t = start + min(i, len - 1);
        v.dt = a.dt_raw[(size_t)t * a.inner + cc];
        v.x = a.xc[(size_t)t * a.inner + cc];
        v.B = ok ? a.xproj[(size_t)t * a.ldx + a.R + nn] : 0.f;
        v.C = ok ? a.xproj[(size_t)t * a.ldx + a.R + N + nn] : 0.f;
        v.gate = a.proj[(size_t)t * a.ldp + a.z_off + cc];
        return v;
    };
    In cur[AHEAD], nxt[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; u++) cur[u] = fetch(u);
    for (int i0 = 0; i0 < len; i0 += AHEAD) {
        if (i0 + AHEAD < len) {
#pragma unroll
            for (int u = 0; u < AHEAD; u++) nxt[u] = fetch(i0 + AHEAD + u);
        }
#pragma unroll
        for (int u = 0; u < AHEAD; u++) {
            if (i0 + u < len) {
                const In v = cur[u];
                S = expf(v.dt * A) * S + v.dt * v.x * v.B;
                float part = S * v.C;
#pragma unroll
                for (int o = LPC / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if (n == 0 && c_ok) a.y[(size_t)(start + i0 + u) * a.inner + c] = (part + Dc * v.x) * v.gate;
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; u++) cur[u] = nxt[u];
    }
    if (ok) *sst = S;
}

cudaError_t scan_recurrence_launch(const ScanArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.N > SCAN_MAXS * 32) return cudaErrorInvalidValue;
    PlainLaunch pl;        // latency-bound over the prompt: CTAs spread over all SMs (see kernels.h)
    if (a.N <= 32) {
        const long n = (long)r.T * a.inner;
        cudaError_t ce = launch_chain(scan_prepare_kernel, dim3((unsigned)std::min<long>((n + 255) / 256, 148 * 8)), dim3(256), 0, s, a, r.T);
        if (ce != cudaSuccess) return ce;
        const int lpc = a.N <= 4 ? 4 : a.N <= 8 ? 8 : a.N <= 16 ? 16 : 32;
        const dim3 grid(r.n_seg, (a.inner + 256 / lpc - 1) / (256 / lpc));
        if (lpc == 4) return launch_chain(scan_recurrence_lanes_kernel<4>, grid, dim3(256), 0, s, a, r);
        if (lpc == 8) return launch_chain(scan_recurrence_lanes_kernel<8>, grid, dim3(256), 0, s, a, r);
        if (lpc == 16) return launch_chain(scan_recurrence_lanes_kernel<16>, grid, dim3(256), 0, s, a, r);
        return launch_chain(scan_recurrence_lanes_kernel<32>, grid, dim3(256), 0, s, a, r);
    }
    if (a.N <= 64) {
        const dim3 grid(r.n_seg, (a.inner + SCAN_CH - 1) / SCAN_CH), block(SCAN_CH);
        const size_t smem = (size_t)SCAN_TB * 2 * a.N * 4;
        if (a.N <= 16) return launch_chain(scan_recurrence_chan_kernel<16>, grid, block, smem, s, a, r);
        if (a.N <= 32) return launch_chain(scan_recurrence_chan_kernel<32>, grid, block, smem, s, a, r);
        return launch_chain(scan_recurrence_chan_kernel<64>, grid, block, smem, s, a, r);
    }
    return launch_chain(scan_recurrence_kernel, dim3(r.n_seg, (a.inner + 7) / 8), dim3(256), 0, s, a, r);
}

// ---------------------------------------------------------------- matrix memory (mLSTM)
// Gate activations for every (token, head), in place over the projection's i and f columns: i <- cap tanh((i + b_i) / cap),
// f <- logsigmoid(cap tanh((f + b_f) / cap)). Parallel over the step, so the recurrence below only carries the maximum.
__global__ void matrix_mem_gates_kernel(MatrixMemArgs a, int T) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * a.H) return;
    const int t = i / a.H, h = i % a.H;
    float* p = const_cast<float*>(a.proj) + (size_t)t * a.ldp;
    p[a.i_off + h] = a.cap * tanhf((p[a.i_off + h] + a.i_bias[h]) / a.cap);
    p[a.f_off + h] = log_sigmoid_f(a.cap * tanhf((p[a.f_off + h] + a.f_bias[h]) / a.cap));
}

// grid (n_seg, H, ceil(dv / 32)): a CTA owns 32 columns of one head's d x dv memory. Thread (col, grp) keeps rows grp * MM_ROWS ..
// of its column in registers; a warp is one row group, and its lanes each carry one row of the normaliser n. Tokens go in blocks of MM_TB: a thread's state update for token t + 1 needs
// only its own registers after token t, so the block barrier is paid once per block -- for the inputs (q, k, v and the two gate
// values of the next block arrive in shared memory as asynchronous copies while this block is computed) and for the partial
// read-outs per row group, which all threads then sum in a fixed order, one (token, column) each. The normaliser n and the
// running maximum m are carried by every CTA of the head (same arithmetic, same values); the first one writes them back.
constexpr int MM_ROWS = 16, MM_COLS = 32, MM_TB = 8;      // key size <= 16 * 16 = 256 (512 threads)
__global__ void __launch_bounds__(512) matrix_mem_kernel(MatrixMemArgs a, RaggedDev r, int RG) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float sm[];
    const int d = a.d, dv = a.dv;
    float* qs = sm;                                // [2][MM_TB][d]
    float* ks = qs + 2 * MM_TB * d;                // [2][MM_TB][d]
    float* vs = ks + 2 * MM_TB * d;                // [2][MM_TB][MM_COLS]
    float* gs = vs + 2 * MM_TB * MM_COLS;          // [2][MM_TB][2]: log input gate, log forget gate
    float* ms = gs + 2 * MM_TB * 2;                // [2][MM_TB]: running maximum after each token
    float* red = ms + 2 * MM_TB;                   // [2][MM_TB][RG][MM_COLS + 1]: partial read-outs, last column = partial n.q
    const int red_tok = RG * (MM_COLS + 1);
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * MM_COLS;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int lc = threadIdx.x % MM_COLS, grp = threadIdx.x / MM_COLS, col = c0 + lc;
    const bool col_ok = col < dv, act = grp < RG;       // threads past the last row group only help with copies and sums
    float* Sg = a.S + (((size_t)slot * a.H + h) * d) * dv;
    float* ng = a.n + ((size_t)slot * a.H + h) * d;
    float S[MM_ROWS];
#pragma unroll
    for (int i = 0; i < MM_ROWS; i++) {
        const int row = grp * MM_ROWS + i;
        S[i] = (act && col_ok && row < d) ? Sg[(size_t)row * dv + col] : 0.f;
    }
    const int nrow = grp * MM_ROWS + lc;                      // lanes 0 .. MM_ROWS-1 of a warp: one row of n each
    const bool n_ok = act && lc < MM_ROWS && nrow < d;
    float nr = n_ok ? ng[nrow] : 0.f;
    const bool vec4 = (d % 4) == 0;
    float m = a.m[(size_t)slot * a.H + h];
    const float qscale = 1.f / sqrtf((float)d);
    auto stage = [&](int i0, int buf) {                  // tokens i0 .. of the segment into buffer `buf`
        const int nb = min(MM_TB, len - i0);
        for (int j = threadIdx.x; j < nb * d; j += blockDim.x) {
            const int u = j / d, e = j % d;
            const float* p = a.proj + (size_t)(start + i0 + u) * a.ldp;
            cp_async_4(&qs[(buf * MM_TB + u) * d + e], p + a.q_off + h * d + e);
            cp_async_4(&ks[(buf * MM_TB + u) * d + e], p + a.k_off + h * d + e);
        }
        for (int j = threadIdx.x; j < nb * MM_COLS; j += blockDim.x) {
            const int u = j / MM_COLS, e = j % MM_COLS;
            const float* p = a.proj + (size_t)(start + i0 + u) * a.ldp;
            if (c0 + e < dv) cp_async_4(&vs[(buf * MM_TB + u) * MM_COLS + e], p + a.v_off + h * dv + c0 + e);
            if (e < 2) cp_async_4(&gs[(buf * MM_TB + u) * 2 + e], p + (e == 0 ? a.i_off : a.f_off) + h);
        }
    };
    auto finish = [&](int i0, int buf) {                 // sum of the row groups in a fixed order, then the read-out
        const int nb = min(MM_TB, len - i0);
        for (int j = threadIdx.x; j < nb * MM_COLS; j += blockDim.x) {
            const int u = j / MM_COLS, e = j % MM_COLS;
            if (c0 + e >= dv) continue;
            const float* rd = red + (size_t)(buf * MM_TB + u) * red_tok;
            float num = 0.f, nq = 0.f;
            for (int g2 = 0; g2 < RG; g2++) { num += rd[g2 * (MM_COLS + 1) + e]; nq += rd[g2 * (MM_COLS + 1) + MM_COLS]; }
            const float den = fmaxf(fabsf(nq), expf(-ms[buf * MM_TB + u])) + 1e-6f;
            a.o_raw[(size_t)(start + i0 + u) * a.H * dv + (size_t)h * dv + c0 + e] = num / den;
        }
    };
    for (int j = threadIdx.x; j < 2 * MM_TB * MM_COLS; j += blockDim.x) vs[j] = 0.f;
    __syncthreads();
    if (len > 0) stage(0, 0);
    cp_async_commit();
    for (int i0 = 0; i0 < len; i0 += MM_TB) {
        const int nb = min(MM_TB, len - i0), buf = (i0 / MM_TB) & 1;
        cp_async_wait_all();
        __syncthreads();
        if (i0 + MM_TB < len) stage(i0 + MM_TB, buf ^ 1);
        cp_async_commit();
        if (i0 > 0) finish(i0 - MM_TB, buf ^ 1);
        for (int u = 0; u < nb; u++) {
            const int bu = buf * MM_TB + u;
            const float ig = gs[bu * 2], fg = gs[bu * 2 + 1];
            const float m_new = fmaxf(fg + m, ig);
            const float da = expf(fg + m - m_new), ib = expf(ig - m_new);
            m = m_new;
            if (threadIdx.x == 0) ms[bu] = m;
            const float vb = ib * vs[bu * MM_COLS + lc];
            float part = 0.f;
            if (act) {
                const float* kr = ks + bu * d + grp * MM_ROWS;
                const float* qr = qs + bu * d + grp * MM_ROWS;
                if (vec4 && grp * MM_ROWS + MM_ROWS <= d) {
#pragma unroll
                    for (int k4 = 0; k4 < MM_ROWS; k4 += 4) {
                        const float4 k4v = *reinterpret_cast<const float4*>(kr + k4), q4v = *reinterpret_cast<const float4*>(qr + k4);
                        S[k4 + 0] = fmaf(da, S[k4 + 0], k4v.x * vb); part = fmaf(S[k4 + 0], q4v.x, part);
                        S[k4 + 1] = fmaf(da, S[k4 + 1], k4v.y * vb); part = fmaf(S[k4 + 1], q4v.y, part);
                        S[k4 + 2] = fmaf(da, S[k4 + 2], k4v.z * vb); part = fmaf(S[k4 + 2], q4v.z, part);
                        S[k4 + 3] = fmaf(da, S[k4 + 3], k4v.w * vb); part = fmaf(S[k4 + 3], q4v.w, part);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < MM_ROWS; k++)
                        if (grp * MM_ROWS + k < d) { S[k] = fmaf(da, S[k], kr[k] * vb); part = fmaf(S[k], qr[k], part); }
                }
            }
            part *= qscale;
            // normaliser: lane l of the warp has row l of this group; n . q summed over the group's lanes
            float npart = 0.f;
            if (n_ok) { nr = fmaf(da, nr, ib * ks[bu * d + nrow]); npart = nr * qs[bu * d + nrow]; }
#pragma unroll
            for (int o = MM_ROWS / 2; o > 0; o >>= 1) npart += __shfl_xor_sync(0xffffffffu, npart, o);
            npart *= qscale;
            if (act) {
                float* rd = red + (size_t)bu * red_tok;
                rd[grp * (MM_COLS + 1) + lc] = part;
                if (lc == 0) rd[grp * (MM_COLS + 1) + MM_COLS] = npart;
            }
        }
    }
    __syncthreads();
    if (len > 0) { const int last0 = (len - 1) / MM_TB * MM_TB; finish(last0, (last0 / MM_TB) & 1); }
#pragma unroll
    for (int i = 0; i < MM_ROWS; i++) {
        const int row = grp * MM_ROWS + i;
        if (act && col_ok && row < d) Sg[(size_t)row * dv + col] = S[i];
    }
    if (n_ok && blockIdx.z == 0) ng[nrow] = nr;
    if (threadIdx.x == 0 && blockIdx.z == 0) a.m[(size_t)slot * a.H + h] = m;
}

// per (token, head): out = o / rms(o) * norm_w * sigmoid(gate)
__global__ void __launch_bounds__(128) matrix_mem_out_kernel(MatrixMemArgs a) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t base = (size_t)t * a.H * a.dv + (size_t)h * a.dv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.dv; i += blockDim.x) { const float v = a.o_raw[base + i]; ss += v * v; }
    const float rinv = 1.f / sqrtf(block_sum(ss, red) / (float)a.dv + a.eps);
    for (int i = threadIdx.x; i < a.dv; i += blockDim.x) {
        const float gate = sigmoid_f(a.proj[(size_t)t * a.ldp + a.g_off + h * a.dv + i]);
        a.out[base + i] = a.o_raw[base + i] * rinv * a.norm_w[h * a.dv + i] * gate;
    }
}

cudaError_t matrix_mem_launch(const MatrixMemArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.dv <= 0 || a.d <= 0 || a.d > MM_ROWS * 16) return cudaErrorInvalidValue;
    const int RG = (a.d + MM_ROWS - 1) / MM_ROWS;
    const size_t smem = (size_t)(2 * MM_TB * (2 * a.d + MM_COLS + 2 + 1 + RG * (MM_COLS + 1))) * 4;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(matrix_mem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); attr_done = true; }
    cudaError_t ce = launch_chain(matrix_mem_gates_kernel, dim3((r.T * a.H + 127) / 128), dim3(128), 0, s, a, r.T);
    if (ce != cudaSuccess) return ce;
    {
        PlainLaunch pl;    // latency-bound over the prompt: CTAs spread over all SMs (see kernels.h)
        ce = launch_chain(matrix_mem_kernel, dim3(r.n_seg, a.H, (a.dv + MM_COLS - 1) / MM_COLS), dim3(std::max(RG * MM_COLS, 64)), smem, s, a, r, RG);
    }
    if (ce != cudaSuccess) return ce;
    return launch_chain(matrix_mem_out_kernel, dim3(r.T, a.H), dim3(128), 0, s, a);
}

}  // namespace b2
