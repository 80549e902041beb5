// Chunk-local attention with sigmoid key weights over the paged cache (layered.h: SigmoidAttnArgs). The weight of a key is
// sigmoid(cap(q . k * scale) + bias[h]) and nothing is normalised over the keys, so partial sums over key ranges simply add;
// scores, caps, sigmoids and the weighted sums are 32-bit, only the cache pages may be bf16.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <stdlib.h>

#include <algorithm>

namespace b2 {

namespace {
__device__ __forceinline__ float sa_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float sa_silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ void sa_store(void* pool, int f32, size_t i, float v) {
    if (f32) reinterpret_cast<float*>(pool)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(pool)[i] = __float2bfloat16(v);
}
template <bool F32>
__device__ __forceinline__ float sa_load(const void* pool, size_t i) {
    if constexpr (F32) return reinterpret_cast<const float*>(pool)[i];
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(pool)[i]);
}
__device__ __forceinline__ float sa_block_sum(float v, float* red) {      // all threads get the sum; red: >= 33 floats
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
// the weight of one key from its raw dot product
__device__ __forceinline__ float sa_weight(float dot, float scale, float softcap, float bias) {
    float z = dot * scale;
    if (softcap > 0.f) z = softcap * tanhf(z / softcap);
    return sa_sigmoid(z + bias);
}
}  // namespace

// grid (T), 256 threads: one token's q and k rows are normed over all their heads at once
__global__ void __launch_bounds__(256) sigmoid_attn_store_kernel(SigmoidAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, nq = a.H * a.d, nk = a.G * a.d, nv = a.G * a.dv;
    const float* row = a.proj + (size_t)t * a.ldp;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = row[a.q_off + i]; sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = row[a.k_off + i]; sk = fmaf(v, v, sk); }
    const float rq = 1.f / sqrtf(sa_block_sum(sq, red) / (float)nq + a.eps);
    const float rk = 1.f / sqrtf(sa_block_sum(sk, red) / (float)nk + a.eps);
    const int pos = r.tok_pos[t];
    const int page = a.block_tables[r.seg_slot[r.tok_seg[t]]][pos / a.block_tokens], in_page = pos % a.block_tokens;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) a.q_out[(size_t)t * nq + i] = row[a.q_off + i] * rq * a.q_norm_w[i];
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int g = i / a.d, c = i % a.d;
        sa_store(a.k_pool, a.cache_f32, (((size_t)page * a.G + g) * a.block_tokens + in_page) * a.d + c, row[a.k_off + i] * rk * a.k_norm_w[i]);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / a.dv, c = i % a.dv;
        sa_store(a.v_pool, a.cache_f32, (((size_t)page * a.G + g) * a.block_tokens + in_page) * a.dv + c, row[a.v_off + i]);
    }
    if (a.act_n > 0) {
        float* act = a.act + (size_t)t * a.ldp;
        for (int i = threadIdx.x; i < a.act_n; i += blockDim.x) act[i] = sa_silu(act[i]);
    }
}
cudaError_t sigmoid_attn_store_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(sigmoid_attn_store_kernel, dim3(r.T), dim3(256), 0, s, a, r);
}

// grid (T, H), 8 warps: a warp takes 4 visible keys per round (their loads and the four dot-product reductions overlap); a lane
// holds entries lane, lane + 32, ... of the key and of the value. The warps' partial sums are added in warp order.
constexpr int SA_WARPS = 8, SA_KEYS = 4, SA_MAXE = 8;       // key and value sizes <= 256
template <bool F32>
__global__ void __launch_bounds__(SA_WARPS * 32) sigmoid_attn_kernel(SigmoidAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float sm_o[SA_WARPS][SA_MAXE * 32];
    const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = r.tok_pos[t];
    const int* table = a.block_tables[r.seg_slot[r.tok_seg[t]]];
    const int g = h / (a.H / a.G), d = a.d, dv = a.dv;
    const float* q = a.q_out + (size_t)t * a.H * d + (size_t)h * d;
    const float bias = a.bias ? a.bias[h] : 0.f;
    float qr[SA_MAXE], acc[SA_MAXE];
#pragma unroll
    for (int e = 0; e < SA_MAXE; e++) { const int i = lane + 32 * e; qr[e] = i < d ? q[i] : 0.f; acc[e] = 0.f; }
    const int lo = a.chunk > 0 ? pos / a.chunk * a.chunk : 0;
    for (int j0 = lo + warp * SA_KEYS; j0 <= pos; j0 += SA_WARPS * SA_KEYS) {
        size_t kb[SA_KEYS], vb[SA_KEYS];
        float sc[SA_KEYS];
#pragma unroll
        for (int u = 0; u < SA_KEYS; u++) {
            const int j = min(j0 + u, pos);                   // past the end: the last key again, its weight is dropped below
            const size_t pr = ((size_t)table[j / a.block_tokens] * a.G + g) * a.block_tokens + j % a.block_tokens;
            kb[u] = pr * d; vb[u] = pr * dv;
        }
#pragma unroll
        for (int u = 0; u < SA_KEYS; u++) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < SA_MAXE; e++) { const int i = lane + 32 * e; if (i < d) dot = fmaf(qr[e], sa_load<F32>(a.k_pool, kb[u] + i), dot); }
            sc[u] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < SA_KEYS; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
#pragma unroll
        for (int u = 0; u < SA_KEYS; u++) {
            const float p = j0 + u <= pos ? sa_weight(sc[u], a.scale, a.softcap, bias) : 0.f;
#pragma unroll
            for (int e = 0; e < SA_MAXE; e++) { const int i = lane + 32 * e; if (i < dv) acc[e] = fmaf(p, sa_load<F32>(a.v_pool, vb[u] + i), acc[e]); }
        }
    }
#pragma unroll
    for (int e = 0; e < SA_MAXE; e++) sm_o[warp][lane + 32 * e] = acc[e];
    __syncthreads();
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < SA_WARPS; w2++) o += sm_o[w2][i];
        a.out[(size_t)t * a.ld_out + (size_t)h * dv + i] = o * a.out_scale;
    }
}

cudaError_t sigmoid_attn_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > SA_MAXE * 32 || a.dv > SA_MAXE * 32 || a.H % a.G) return cudaErrorInvalidValue;
    const dim3 grid(r.T, a.H);
    return a.cache_f32 ? launch_chain(sigmoid_attn_kernel<true>, grid, dim3(SA_WARPS * 32), 0, s, a, r)
                       : launch_chain(sigmoid_attn_kernel<false>, grid, dim3(SA_WARPS * 32), 0, s, a, r);
}

}  // namespace b2
