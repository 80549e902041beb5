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

// grid (T, H * Gc, splits), 8 warps. Query head h of token t against the keys of its own key head; the weights are applied to the
// values of the head's own key/value head (VH = 1, Gc = 1) or, when the heads' weights are mixed afterwards, to the values of VH
// value heads at once (Gc = ceil(G / VH) chunks of value heads): the scores are computed once for all of them. A warp takes 4
// visible keys per round and keeps a running maximum, sum and outputs of its own; the warps are merged once, in warp order. With
// one split the sink term joins there and the normalised result is written; with several (few-token steps: the visible keys are
// cut into `splits` equal ranges so that a single decoded token still fills the GPU) every CTA leaves (maximum, sum, output) of
// its range in `part` and sink_attn_merge_kernel adds them in range order.
constexpr int SK_WARPS = 8, SK_KEYS = 4, SK_MAX_SPLITS = 16, SK_FEW_TOKENS = 8, SK_VH = 4;
template <bool F32, int VH>
__global__ void __launch_bounds__(SK_WARPS * 32) sink_attn_kernel(SinkAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float sk_sm_o[];                        // [SK_WARPS][VH][SK_MAXE * 32]
    __shared__ float sm_m[SK_WARPS], sm_l[SK_WARPS];
    const int Gv = a.talk ? a.G : 1, Gc = (Gv + VH - 1) / VH;
    const int t = blockIdx.x, h = blockIdx.y / Gc, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_splits = gridDim.z, split = blockIdx.z;
    const int pos = r.tok_pos[t];
    const int* table = a.block_tables[r.seg_slot[r.tok_seg[t]]];
    const int g = h / (a.H / a.G), d = a.d, dv = a.dv;
    const int vg0 = a.talk ? (int)(blockIdx.y % Gc) * VH : g;            // first of this CTA's value heads
    const float* q = a.q_rot + ((size_t)t * a.H + h) * d;
    float qr[SK_MAXE], acc[VH][SK_MAXE];
#pragma unroll
    for (int e = 0; e < SK_MAXE; e++) {
        const int i = lane + 32 * e;
        qr[e] = i < d ? q[i] * a.scale : 0.f;
#pragma unroll
        for (int v = 0; v < VH; v++) acc[v][e] = 0.f;
    }
    float m_run = -INFINITY, l_run = 0.f;
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0, hi = pos;
    if (n_splits > 1) {                                       // this CTA's share of the visible keys, whole warp rounds
        const int per = ((pos - lo + n_splits) / n_splits + SK_WARPS * SK_KEYS - 1) / (SK_WARPS * SK_KEYS) * (SK_WARPS * SK_KEYS);
        lo += split * per;
        hi = min(pos, lo + per - 1);
    }
    for (int j0 = lo + warp * SK_KEYS; j0 <= hi; j0 += SK_WARPS * SK_KEYS) {
        size_t kb[SK_KEYS], vb[SK_KEYS];
        float sc[SK_KEYS];
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) {
            const int j = min(j0 + u, hi);                    // past the end: the last key again, its weight is dropped below
            const size_t page = table[j / a.block_tokens];
            kb[u] = ((page * a.G + g) * a.block_tokens + j % a.block_tokens) * d;
            vb[u] = (page * a.G * a.block_tokens + j % a.block_tokens) * dv;       // value head v adds v * block_tokens * dv
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
        for (int u = 0; u < SK_KEYS; u++) if (j0 + u <= hi) mx = fmaxf(mx, sc[u]);
        const float corr = expf(m_run - mx);                  // 0 at the first round (m_run = -inf, mx finite)
        l_run *= corr;
#pragma unroll
        for (int v = 0; v < VH; v++)
#pragma unroll
            for (int e = 0; e < SK_MAXE; e++) acc[v][e] *= corr;
#pragma unroll
        for (int u = 0; u < SK_KEYS; u++) {
            const float p = j0 + u <= hi ? expf(sc[u] - mx) : 0.f;
            l_run += p;
#pragma unroll
            for (int v = 0; v < VH; v++) {
                const size_t vbase = vb[u] + (size_t)min(vg0 + v, a.G - 1) * a.block_tokens * dv;       // past the last head: its last one again, not stored
#pragma unroll
                for (int e = 0; e < SK_MAXE; e++) { const int i = lane + 32 * e; if (i < dv) acc[v][e] = fmaf(p, sk_load<F32>(a.v_pool, vbase + i), acc[v][e]); }
            }
        }
        m_run = mx;
    }
#pragma unroll
    for (int v = 0; v < VH; v++)
#pragma unroll
        for (int e = 0; e < SK_MAXE; e++) sk_sm_o[(warp * VH + v) * (SK_MAXE * 32) + lane + 32 * e] = acc[v][e];
    if (lane == 0) { sm_m[warp] = m_run; sm_l[warp] = l_run; }
    __syncthreads();
    const float sink = a.sink && n_splits == 1 ? a.sink[h] : -INFINITY;
    float m = sink;
#pragma unroll
    for (int w2 = 0; w2 < SK_WARPS; w2++) m = fmaxf(m, sm_m[w2]);
    float l = sink > -INFINITY ? expf(sink - m) : 0.f;
    float f[SK_WARPS];
#pragma unroll
    for (int w2 = 0; w2 < SK_WARPS; w2++) { f[w2] = sm_m[w2] > -INFINITY ? expf(sm_m[w2] - m) : 0.f; l = fmaf(sm_l[w2], f[w2], l); }
    const float inv = n_splits > 1 ? 1.f : 1.f / l;
    for (int e = threadIdx.x; e < VH * dv; e += blockDim.x) {
        const int v = e / dv, i = e - v * dv, vg = vg0 + v;
        if (a.talk && vg >= a.G) continue;
        float o = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < SK_WARPS; w2++) o = fmaf(sk_sm_o[(w2 * VH + v) * (SK_MAXE * 32) + i], f[w2], o);
        o *= inv;
        if (n_splits > 1) {
            float* part = a.part + ((((size_t)t * a.H + h) * Gv + (a.talk ? vg : 0)) * n_splits + split) * (dv + 2);
            if (i == 0) { part[0] = m; part[1] = l; }
            part[2 + i] = o;
        } else if (a.talk) a.cross[(((size_t)t * a.H + h) * a.G + vg) * dv + i] = o;
        else a.out[(size_t)t * a.ld_out + (size_t)h * dv + i] = o * sk_gate(a, t, h, i);
    }
}

// grid (T, H * Gv), 128 threads: the ranges' (maximum, sum, output) and the sink term, in range order
__global__ void __launch_bounds__(128) sink_attn_merge_kernel(SinkAttnArgs a, int n_splits) {
    griddep_launch();
    griddep_wait();
    const int Gv = a.talk ? a.G : 1;
    const int t = blockIdx.x, h = blockIdx.y / Gv, vg = blockIdx.y % Gv, dv = a.dv;
    const float* part = a.part + (((size_t)t * a.H + h) * Gv + vg) * n_splits * (dv + 2);
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float m = sink;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, part[(size_t)s * (dv + 2)]);
    float l = a.sink ? expf(sink - m) : 0.f;
    float f[SK_MAX_SPLITS];
#pragma unroll
    for (int s = 0; s < SK_MAX_SPLITS; s++) {
        f[s] = 0.f;
        if (s < n_splits) {
            const float ms = part[(size_t)s * (dv + 2)];
            f[s] = ms > -INFINITY ? expf(ms - m) : 0.f;
            l = fmaf(part[(size_t)s * (dv + 2) + 1], f[s], l);
        }
    }
    const float inv = 1.f / l;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int s = 0; s < SK_MAX_SPLITS; s++) if (s < n_splits) o = fmaf(part[(size_t)s * (dv + 2) + 2 + i], f[s], o);
        o *= inv;
        if (a.talk) a.cross[(((size_t)t * a.H + h) * a.G + vg) * dv + i] = o;
        else a.out[(size_t)t * a.ld_out + (size_t)h * dv + i] = o * sk_gate(a, t, h, i);
    }
}

// grid (T, H), 128 threads: out_h = gate_h * sum_g talk[h][g] A[g][c(h)], the sum in head order
__global__ void __launch_bounds__(128) sink_attn_talk_kernel(SinkAttnArgs a, int T) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, h = blockIdx.y, H = a.H, G = a.G, dv = a.dv, c = h / (H / G);
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.f;
        for (int g = 0; g < H; g++) o = fmaf(a.talk[h * H + g], a.cross[(((size_t)t * H + g) * G + c) * dv + i], o);
        a.out[(size_t)t * a.ld_out + (size_t)h * dv + i] = o * sk_gate(a, t, h, i);
    }
}

// Tensor-core prompt attention (bf16 pages, key and value sizes multiples of 16 up to 128): a CTA takes one tile of up to 64
// consecutive queries of a segment, one query head and one value head; 4 warps x 16 query rows; keys in blocks of 64 from the block
// that holds the oldest key of the tile's first query to the block of its last query, staged in shared memory once for all 64
// queries. S = Q K^T and O += P V with mma.sync m16n8k16 (bf16 in, f32 accumulate); scale, mask, running maximum, sums and the
// sink term are 32-bit. Queries and probabilities enter the products as TWO bf16 each (value = leading part + remainder), so the
// only 16-bit rounding on this path is that of the cached keys and values -- the same as on the few-token path.
constexpr int SKM_Q = 64, SKM_K = 64;
namespace {
__device__ __forceinline__ void sk_cp_async_16z(void* smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void sk_ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void sk_ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void sk_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sk_split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
}  // namespace

template <int DMAX, int DVMAX>
__global__ void __launch_bounds__(128) sink_attn_mma_kernel(SinkAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int d = a.d, dv = a.dv, LD = d + 8, LDV = dv + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sk_smem);     // [64][LD] leading bf16 of the query
    __nv_bfloat16* Ql = Qs + SKM_Q * LD;                                // [64][LD] what the first bf16 leaves over
    __nv_bfloat16* Ks = Ql + SKM_Q * LD;                                // [64][LD]
    __nv_bfloat16* Vs = Ks + SKM_K * LD;                                // [64][LDV]
    const int Gv = a.talk ? a.G : 1;
    // late tiles of a segment have the most key blocks: they start first
    const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y / Gv, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(SKM_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const int g = h / (a.H / a.G);
    const int vg = a.talk ? (int)(blockIdx.y % Gv) : g;
    const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(a.k_pool);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(a.v_pool);
    for (int i = threadIdx.x; i < SKM_Q * (d / 2); i += blockDim.x) {
        const int rr = i / (d / 2), c = (i % (d / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (rr < nq) v = *reinterpret_cast<const float2*>(a.q_rot + ((size_t)(row0 + rr) * a.H + h) * d + c);
        v.x *= a.scale; v.y *= a.scale;
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(Qs + rr * LD + c) = hi;
        *reinterpret_cast<__nv_bfloat162*>(Ql + rr * LD + c) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
    }
    const int lo_first = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int b0 = lo_first / SKM_K, b1 = p_last / SKM_K;
    float o[DVMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    int qlo[2];                                    // oldest visible key of the lane's two query rows
    float m_run[2], l_run[2];
    const float sink = a.sink ? a.sink[h] : -INFINITY;
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        const int i = p0 + qrow[q2];
        qlo[q2] = a.window > 0 ? max(0, i - a.window + 1) : 0;
        m_run[q2] = sink; l_run[q2] = 0.f;         // the running maximum starts at the sink; its term joins the sum at the end
    }
    for (int kb = b0; kb <= b1; kb++) {
        const int j0 = kb * SKM_K;
        __syncthreads();                      // everybody is done with the previous block's K and V (and Q is written)
        for (int i = threadIdx.x; i < SKM_K * (d / 8); i += blockDim.x) {
            const int rr = i / (d / 8), c = (i % (d / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + g) * a.block_tokens + jj % a.block_tokens) * d + c;
            sk_cp_async_16z(Ks + rr * LD + c, kp + base, j <= p_last ? 16 : 0);
        }
        for (int i = threadIdx.x; i < SKM_K * (dv / 8); i += blockDim.x) {
            const int rr = i / (dv / 8), c = (i % (dv / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + vg) * a.block_tokens + jj % a.block_tokens) * dv + c;
            sk_cp_async_16z(Vs + rr * LDV + c, vp + base, j <= p_last ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        float sacc[SKM_K / 8][4];
#pragma unroll
        for (int ni = 0; ni < SKM_K / 8; ni++) sacc[ni][0] = sacc[ni][1] = sacc[ni][2] = sacc[ni][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DMAX; ks += 16) {
            if (ks < d) {
                uint32_t af[4], al[4];
                sk_ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
                sk_ldsm_x4(al, Ql + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
#pragma unroll
                for (int nj = 0; nj < SKM_K / 16; nj++) {
                    uint32_t bf[4];
                    sk_ldsm_x4(bf, Ks + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks + ((lane >> 3) & 1) * 8);
                    sk_mma_16816(sacc[2 * nj], al, bf[0], bf[1]);
                    sk_mma_16816(sacc[2 * nj + 1], al, bf[2], bf[3]);
                    sk_mma_16816(sacc[2 * nj], af, bf[0], bf[1]);
                    sk_mma_16816(sacc[2 * nj + 1], af, bf[2], bf[3]);
                }
            }
        }
        // mask, running maximum per query row (a row lives in the four lanes of a quad), probabilities
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int rr = qrow[e >> 1], i = p0 + rr, j = j0 + ni * 8 + 2 * tq + (e & 1);
                const bool vis = rr < nq && j <= i && j >= qlo[e >> 1];
                sacc[ni][e] = vis ? sacc[ni][e] : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sacc[ni][e]);
            }
        float corr[2], msafe[2], rs[2] = {0.f, 0.f};
#pragma unroll
        for (int q2 = 0; q2 < 2; q2++) {
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 1));
            mx[q2] = fmaxf(mx[q2], __shfl_xor_sync(0xffffffffu, mx[q2], 2));
            msafe[q2] = mx[q2] > -INFINITY ? mx[q2] : 0.f;             // nothing visible yet and no sink: every term is exp(-inf) = 0
            corr[q2] = __expf(m_run[q2] - msafe[q2]);
            m_run[q2] = mx[q2];
        }
#pragma unroll
        for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = __expf(sacc[ni][e] - msafe[e >> 1]);
                sacc[ni][e] = p;
                rs[e >> 1] += p;
            }
#pragma unroll
        for (int q2 = 0; q2 < 2; q2++) {
            rs[q2] += __shfl_xor_sync(0xffffffffu, rs[q2], 1);
            rs[q2] += __shfl_xor_sync(0xffffffffu, rs[q2], 2);
            l_run[q2] = fmaf(l_run[q2], corr[q2], rs[q2]);
        }
#pragma unroll
        for (int i = 0; i < DVMAX / 8; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
        for (int kc = 0; kc < SKM_K / 16; kc++) {
            uint32_t pf[4], pl[4];
            sk_split_bf16(sacc[2 * kc][0], sacc[2 * kc][1], pf[0], pl[0]);
            sk_split_bf16(sacc[2 * kc][2], sacc[2 * kc][3], pf[1], pl[1]);
            sk_split_bf16(sacc[2 * kc + 1][0], sacc[2 * kc + 1][1], pf[2], pl[2]);
            sk_split_bf16(sacc[2 * kc + 1][2], sacc[2 * kc + 1][3], pf[3], pl[3]);
#pragma unroll
            for (int nd = 0; nd < DVMAX / 16; nd++) {
                if (nd * 16 < dv) {
                    uint32_t vf[4];
                    sk_ldsm_x4_t(vf, Vs + (kc * 16 + (lane & 15)) * LDV + nd * 16 + (lane >> 4) * 8);
                    sk_mma_16816(o[2 * nd], pl, vf[0], vf[1]);
                    sk_mma_16816(o[2 * nd + 1], pl, vf[2], vf[3]);
                    sk_mma_16816(o[2 * nd], pf, vf[0], vf[1]);
                    sk_mma_16816(o[2 * nd + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
    float inv[2];
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        const float l = l_run[q2] + (a.sink ? __expf(sink - m_run[q2]) : 0.f);
        inv[q2] = l > 0.f ? 1.f / l : 0.f;
    }
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int rr = qrow[e >> 1], c = i * 8 + 2 * tq + (e & 1);
            if (rr >= nq || c >= dv) continue;
            const float v = o[i][e] * inv[e >> 1];
            const int t = row0 + rr;
            if (a.talk) a.cross[(((size_t)t * a.H + h) * a.G + vg) * dv + c] = v;
            else a.out[(size_t)t * a.ld_out + (size_t)h * dv + c] = v * sk_gate(a, t, h, c);
        }
}

// ---- prompts with mixed heads (bf16 pages): the weights are mixed BEFORE they meet the values, in three passes over a group of
// query tiles whose normalised weights fit the scratch `pbuf` ([tile][head][64 rows][span] f32, span = the most key blocks a tile
// can touch x 64):
//   1. sink_attn_probs_kernel  per (tile, head): scores twice -- first the running maximum and the sum (with the sink), then the
//                              normalised weights exp(s - m) / l into pbuf (zeros where the mask hides a key)
//   2. sink_attn_mix_kernel    per (tile, row): w_h <- sum_g talk[h][g] w_g in place, a chunk of columns at a time through shared memory
//   3. sink_attn_pv_kernel     per (tile, head): O = W_h V with the values of the head's own key/value head, gate, store
// Against the form that keeps a separate weighted sum per (query head, value head) pair this does the score products twice and
// the value products once instead of G times each; the scratch costs two passes over HBM.
struct SinkMix { int tile0, span; };

template <int DMAX>
__global__ void __launch_bounds__(128) sink_attn_probs_kernel(SinkAttnArgs a, RaggedDev r, SinkMix mx) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int d = a.d, LD = d + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sk_smem);     // [64][LD] leading bf16 of the (scaled) query
    __nv_bfloat16* Ql = Qs + SKM_Q * LD;                                // [64][LD] remainder
    __nv_bfloat16* Ks = Ql + SKM_Q * LD;                                // [64][LD]
    const int tile = mx.tile0 + blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(SKM_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const int g = h / (a.H / a.G);
    const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(a.k_pool);
    for (int i = threadIdx.x; i < SKM_Q * (d / 2); i += blockDim.x) {
        const int rr = i / (d / 2), c = (i % (d / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (rr < nq) v = *reinterpret_cast<const float2*>(a.q_rot + ((size_t)(row0 + rr) * a.H + h) * d + c);
        v.x *= a.scale; v.y *= a.scale;
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(Qs + rr * LD + c) = hi;
        *reinterpret_cast<__nv_bfloat162*>(Ql + rr * LD + c) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
    }
    const int lo_first = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int b0 = lo_first / SKM_K, b1 = min(p_last / SKM_K, b0 + mx.span / SKM_K - 1);
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    int qlo[2];
    float m_run[2], l_run[2], inv[2] = {0.f, 0.f};
    const float sink = a.sink ? a.sink[h] : -INFINITY;
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        const int i = p0 + qrow[q2];
        qlo[q2] = a.window > 0 ? max(0, i - a.window + 1) : 0;
        m_run[q2] = sink; l_run[q2] = 0.f;
    }
    float* prow[2];
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) prow[q2] = a.pbuf + (((size_t)blockIdx.x * a.H + h) * SKM_Q + qrow[q2]) * mx.span;
    for (int pass = 0; pass < 2; pass++) {
        for (int kb = b0; kb <= b1; kb++) {
            const int j0 = kb * SKM_K;
            __syncthreads();                      // everybody is done with the previous block's K (and Q is written)
            for (int i = threadIdx.x; i < SKM_K * (d / 8); i += blockDim.x) {
                const int rr = i / (d / 8), c = (i % (d / 8)) * 8;
                const int j = j0 + rr, jj = min(j, p_last);
                const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + g) * a.block_tokens + jj % a.block_tokens) * d + c;
                sk_cp_async_16z(Ks + rr * LD + c, kp + base, j <= p_last ? 16 : 0);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            float sacc[SKM_K / 8][4];
#pragma unroll
            for (int ni = 0; ni < SKM_K / 8; ni++) sacc[ni][0] = sacc[ni][1] = sacc[ni][2] = sacc[ni][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DMAX; ks += 16) {
                if (ks < d) {
                    uint32_t af[4], al[4];
                    sk_ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
                    sk_ldsm_x4(al, Ql + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
#pragma unroll
                    for (int nj = 0; nj < SKM_K / 16; nj++) {
                        uint32_t bf[4];
                        sk_ldsm_x4(bf, Ks + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks + ((lane >> 3) & 1) * 8);
                        sk_mma_16816(sacc[2 * nj], al, bf[0], bf[1]);
                        sk_mma_16816(sacc[2 * nj + 1], al, bf[2], bf[3]);
                        sk_mma_16816(sacc[2 * nj], af, bf[0], bf[1]);
                        sk_mma_16816(sacc[2 * nj + 1], af, bf[2], bf[3]);
                    }
                }
            }
#pragma unroll
            for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int rr = qrow[e >> 1], i = p0 + rr, j = j0 + ni * 8 + 2 * tq + (e & 1);
                    const bool vis = rr < nq && j <= i && j >= qlo[e >> 1];
                    sacc[ni][e] = vis ? sacc[ni][e] : -INFINITY;
                }
            if (pass == 0) {
                float mxr[2] = {m_run[0], m_run[1]}, rs[2] = {0.f, 0.f}, msafe[2];
#pragma unroll
                for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
                    for (int e = 0; e < 4; e++) mxr[e >> 1] = fmaxf(mxr[e >> 1], sacc[ni][e]);
#pragma unroll
                for (int q2 = 0; q2 < 2; q2++) {
                    mxr[q2] = fmaxf(mxr[q2], __shfl_xor_sync(0xffffffffu, mxr[q2], 1));
                    mxr[q2] = fmaxf(mxr[q2], __shfl_xor_sync(0xffffffffu, mxr[q2], 2));
                    msafe[q2] = mxr[q2] > -INFINITY ? mxr[q2] : 0.f;
                }
#pragma unroll
                for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
                    for (int e = 0; e < 4; e++) rs[e >> 1] += __expf(sacc[ni][e] - msafe[e >> 1]);
#pragma unroll
                for (int q2 = 0; q2 < 2; q2++) {
                    rs[q2] += __shfl_xor_sync(0xffffffffu, rs[q2], 1);
                    rs[q2] += __shfl_xor_sync(0xffffffffu, rs[q2], 2);
                    l_run[q2] = fmaf(l_run[q2], __expf(m_run[q2] - msafe[q2]), rs[q2]);
                    m_run[q2] = mxr[q2];
                }
            } else {
#pragma unroll
                for (int ni = 0; ni < SKM_K / 8; ni++)
#pragma unroll
                    for (int q2 = 0; q2 < 2; q2++) {
                        const float2 w = make_float2(__expf(sacc[ni][2 * q2] - m_run[q2]) * inv[q2], __expf(sacc[ni][2 * q2 + 1] - m_run[q2]) * inv[q2]);
                        *reinterpret_cast<float2*>(prow[q2] + (kb - b0) * SKM_K + ni * 8 + 2 * tq) = w;
                    }
            }
        }
        if (pass == 0) {
#pragma unroll
            for (int q2 = 0; q2 < 2; q2++) {
                const float msafe = m_run[q2] > -INFINITY ? m_run[q2] : 0.f;
                const float l = l_run[q2] + (a.sink ? __expf(sink - msafe) : 0.f);
                inv[q2] = l > 0.f ? 1.f / l : 0.f;
                m_run[q2] = msafe;
            }
        }
    }
}

// grid (tiles of the group * 64 rows), 256 threads; shared: talk [H][H], then [H][256] weights of a chunk of columns
__global__ void __launch_bounds__(256) sink_attn_mix_kernel(SinkAttnArgs a, RaggedDev r, SinkMix mx) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float mix_sm[];
    const int H = a.H;
    float* tk = mix_sm;
    float* vals = mix_sm + H * H;
    const int tl = blockIdx.x / SKM_Q, row = blockIdx.x % SKM_Q, tile = mx.tile0 + tl;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(SKM_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    if (row >= nq) return;
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int lo_first = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int b0 = lo_first / SKM_K, b1 = min(p_last / SKM_K, b0 + mx.span / SKM_K - 1);
    const int ncol = (b1 - b0 + 1) * SKM_K;
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = a.talk[i];
    float* base = a.pbuf + ((size_t)tl * H * SKM_Q + row) * mx.span;          // head g adds g * 64 * span
    const size_t hs = (size_t)SKM_Q * mx.span;
    for (int c0 = 0; c0 < ncol; c0 += 256) {
        const int c = c0 + threadIdx.x;
        __syncthreads();
        if (c < ncol) for (int g = 0; g < H; g++) vals[g * 256 + threadIdx.x] = base[g * hs + c];
        __syncthreads();                           // also: talk is in place
        if (c < ncol)
            for (int h = 0; h < H; h++) {
                float o = 0.f;
                for (int g = 0; g < H; g++) o = fmaf(tk[h * H + g], vals[g * 256 + threadIdx.x], o);
                base[h * hs + c] = o;
            }
    }
}

template <int DVMAX>
__global__ void __launch_bounds__(128) sink_attn_pv_kernel(SinkAttnArgs a, RaggedDev r, SinkMix mx) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int dv = a.dv, LDV = dv + 8;
    __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(sk_smem);     // [64][LDV]
    const int tile = mx.tile0 + blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(SKM_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const int vg = h / (a.H / a.G);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(a.v_pool);
    const int lo_first = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int b0 = lo_first / SKM_K, b1 = min(p_last / SKM_K, b0 + mx.span / SKM_K - 1);
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    const float* prow[2];
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) prow[q2] = a.pbuf + (((size_t)blockIdx.x * a.H + h) * SKM_Q + qrow[q2]) * mx.span;
    float o[DVMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    for (int kb = b0; kb <= b1; kb++) {
        const int j0 = kb * SKM_K;
        __syncthreads();
        for (int i = threadIdx.x; i < SKM_K * (dv / 8); i += blockDim.x) {
            const int rr = i / (dv / 8), c = (i % (dv / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + vg) * a.block_tokens + jj % a.block_tokens) * dv + c;
            sk_cp_async_16z(Vs + rr * LDV + c, vp + base, j <= p_last ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        // this block's mixed weights straight from the scratch in the MMA's row layout, while the values arrive
        float2 w[SKM_K / 16][4];
#pragma unroll
        for (int kc = 0; kc < SKM_K / 16; kc++)
#pragma unroll
            for (int f = 0; f < 4; f++) {
                const int rr = qrow[f & 1];
                w[kc][f] = rr < nq ? *reinterpret_cast<const float2*>(prow[f & 1] + (kb - b0) * SKM_K + kc * 16 + (f >> 1) * 8 + 2 * tq) : make_float2(0.f, 0.f);
            }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
#pragma unroll
        for (int kc = 0; kc < SKM_K / 16; kc++) {
            uint32_t pf[4], pl[4];
#pragma unroll
            for (int f = 0; f < 4; f++) sk_split_bf16(w[kc][f].x, w[kc][f].y, pf[f], pl[f]);
#pragma unroll
            for (int nd = 0; nd < DVMAX / 16; nd++) {
                if (nd * 16 < dv) {
                    uint32_t vf[4];
                    sk_ldsm_x4_t(vf, Vs + (kc * 16 + (lane & 15)) * LDV + nd * 16 + (lane >> 4) * 8);
                    sk_mma_16816(o[2 * nd], pl, vf[0], vf[1]);
                    sk_mma_16816(o[2 * nd + 1], pl, vf[2], vf[3]);
                    sk_mma_16816(o[2 * nd], pf, vf[0], vf[1]);
                    sk_mma_16816(o[2 * nd + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int rr = qrow[e >> 1], c = i * 8 + 2 * tq + (e & 1);
            if (rr >= nq || c >= dv) continue;
            const int t = row0 + rr;
            a.out[(size_t)t * a.ld_out + (size_t)h * dv + c] = o[i][e] * sk_gate(a, t, h, c);
        }
}

template <int DMAX>
static cudaError_t sink_attn_probs_pick(const SinkAttnArgs& a, const RaggedDev& r, const SinkMix& mx, int nt, cudaStream_t s) {
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(sink_attn_probs_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 64 * (DMAX + 8) * 2); attr_done = true; }
    return launch_chain(sink_attn_probs_kernel<DMAX>, dim3(nt, a.H), dim3(128), (size_t)3 * 64 * (a.d + 8) * 2, s, a, r, mx);
}
template <int DVMAX>
static cudaError_t sink_attn_pv_pick(const SinkAttnArgs& a, const RaggedDev& r, const SinkMix& mx, int nt, cudaStream_t s) {
    return launch_chain(sink_attn_pv_kernel<DVMAX>, dim3(nt, a.H), dim3(128), (size_t)64 * (a.dv + 8) * 2, s, a, r, mx);
}
// false: the scratch cannot hold even one tile (or too many heads for the mixing pass's shared memory)
static bool sink_attn_mixed_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s, cudaError_t& e) {
    const int span = ((a.max_keys + 62) / 64 + 2) * 64;
    const size_t per_tile = (size_t)a.H * SKM_Q * span;
    const size_t mix_smem = (size_t)(a.H * a.H + a.H * 256) * 4;
    if (!a.pbuf || per_tile > a.pbuf_floats || mix_smem > 96 * 1024) return false;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(sink_attn_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); attr_done = true; }
    const int group = (int)std::min<size_t>(a.pbuf_floats / per_tile, (size_t)r.n_tiles);
    e = cudaSuccess;
    for (int t0 = 0; t0 < r.n_tiles && e == cudaSuccess; t0 += group) {
        const int nt = std::min(group, r.n_tiles - t0);
        SinkMix mx = {t0, span};
        e = a.d <= 64 ? sink_attn_probs_pick<64>(a, r, mx, nt, s) : sink_attn_probs_pick<128>(a, r, mx, nt, s);
        if (e == cudaSuccess) e = launch_chain(sink_attn_mix_kernel, dim3(nt * SKM_Q), dim3(256), mix_smem, s, a, r, mx);
        if (e == cudaSuccess) e = a.dv <= 64 ? sink_attn_pv_pick<64>(a, r, mx, nt, s) : sink_attn_pv_pick<128>(a, r, mx, nt, s);
    }
    return true;
}

template <int DMAX, int DVMAX>
static cudaError_t sink_attn_mma_pick(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    const size_t smem = (size_t)(3 * 64 * (a.d + 8) + 64 * (a.dv + 8)) * 2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(sink_attn_mma_kernel<DMAX, DVMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (3 * 64 * (DMAX + 8) + 64 * (DVMAX + 8)) * 2);
        attr_done = true;
    }
    return launch_chain(sink_attn_mma_kernel<DMAX, DVMAX>, dim3(r.n_tiles, a.H * (a.talk ? a.G : 1)), dim3(128), smem, s, a, r);
}

cudaError_t sink_attn_launch(const SinkAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > SK_MAXE * 32 || a.dv > SK_MAXE * 32 || a.H % a.G) return cudaErrorInvalidValue;
    static const bool no_mma = getenv("B2_NO_ATTN_MMA") != nullptr;        // tuning aid: scalar attention for prompts too
    const int Gv = a.talk ? a.G : 1;
    cudaError_t e;
    if (!no_mma && !a.cache_f32 && r.T > SK_FEW_TOKENS && a.d % 16 == 0 && a.dv % 16 == 0 && a.d <= 128 && a.dv <= 128) {
        static const bool no_mixed = getenv("B2_NO_ATTN_MIXED") != nullptr;    // tuning aid: one weighted sum per (query head, value head) pair
        // with one or two key/value heads the separate sums cost no more than the second score pass and the scratch traffic
        // (measured at 8 heads over 2: 0.84 against 1.08 ms for four layers and 2048 tokens)
        if (a.talk && a.G >= 3 && !no_mixed && sink_attn_mixed_launch(a, r, s, e)) return e;
        if (a.d <= 64) e = a.dv <= 64 ? sink_attn_mma_pick<64, 64>(a, r, s) : sink_attn_mma_pick<64, 128>(a, r, s);
        else e = a.dv <= 64 ? sink_attn_mma_pick<128, 64>(a, r, s) : sink_attn_mma_pick<128, 128>(a, r, s);
    } else {
        // few tokens: enough key ranges to fill the GPU; the count depends on the step's shape and the window only, never on the
        // positions, so that a captured step can be replayed
        int splits = 1;
        if (r.T <= SK_FEW_TOKENS && a.part) {
            const int ctas = r.T * a.H * (a.talk ? (a.G + SK_VH - 1) / SK_VH : 1);
            splits = std::min({SK_MAX_SPLITS, std::max(1, (a.max_keys + 127) / 128), std::max(1, 592 / ctas)});
            while (splits > 1 && (size_t)r.T * a.H * Gv * splits * (a.dv + 2) > (size_t)a.part_capacity) splits--;
        }
        if (a.talk) {
            const dim3 grid(r.T, a.H * ((a.G + SK_VH - 1) / SK_VH), splits);
            const size_t smem = (size_t)SK_WARPS * SK_VH * SK_MAXE * 32 * 4;
            e = a.cache_f32 ? launch_chain(sink_attn_kernel<true, SK_VH>, grid, dim3(SK_WARPS * 32), smem, s, a, r)
                            : launch_chain(sink_attn_kernel<false, SK_VH>, grid, dim3(SK_WARPS * 32), smem, s, a, r);
        } else {
            const dim3 grid(r.T, a.H, splits);
            const size_t smem = (size_t)SK_WARPS * SK_MAXE * 32 * 4;
            e = a.cache_f32 ? launch_chain(sink_attn_kernel<true, 1>, grid, dim3(SK_WARPS * 32), smem, s, a, r)
                            : launch_chain(sink_attn_kernel<false, 1>, grid, dim3(SK_WARPS * 32), smem, s, a, r);
        }
        if (e == cudaSuccess && splits > 1) e = launch_chain(sink_attn_merge_kernel, dim3(r.T, a.H * Gv), dim3(128), 0, s, a, splits);
    }
    if (e != cudaSuccess || !a.talk) return e;
    return launch_chain(sink_attn_talk_kernel, dim3(r.T, a.H), dim3(128), 0, s, a, r.T);
}

}  // namespace b2
