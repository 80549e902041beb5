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

// grid (T, 3), 256 threads. A token's q and k rows are normed over all their heads at once; the three parts of the work are
// independent, so three CTAs share a token: y = 0 the query (norm into q_out), 1 the key (norm) and the value into their pages,
// 2 the SiLU columns. A decoded token's row is then ready after one third of the single-CTA latency.
__global__ void __launch_bounds__(256) sigmoid_attn_store_kernel(SigmoidAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[33];
    const int t = blockIdx.x, part = blockIdx.y, nq = a.H * a.d, nk = a.G * a.d, nv = a.G * a.dv;
    const float* row = a.proj + (size_t)t * a.ldp;
    if (part == 0) {
        float sq = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = row[a.q_off + i]; sq = fmaf(v, v, sq); }
        const float rq = 1.f / sqrtf(sa_block_sum(sq, red) / (float)nq + a.eps);
        for (int i = threadIdx.x; i < nq; i += blockDim.x) a.q_out[(size_t)t * nq + i] = row[a.q_off + i] * rq * a.q_norm_w[i];
    } else if (part == 1) {
        float sk = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = row[a.k_off + i]; sk = fmaf(v, v, sk); }
        const float rk = 1.f / sqrtf(sa_block_sum(sk, red) / (float)nk + a.eps);
        const int pos = r.tok_pos[t];
        const size_t page = a.block_tables[r.seg_slot[r.tok_seg[t]]][pos / a.block_tokens];
        const int in_page = pos % a.block_tokens;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const int g = i / a.d, c = i - g * a.d;
            sa_store(a.k_pool, a.cache_f32, ((page * a.G + g) * a.block_tokens + in_page) * a.d + c, row[a.k_off + i] * rk * a.k_norm_w[i]);
        }
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            const int g = i / a.dv, c = i - g * a.dv;
            sa_store(a.v_pool, a.cache_f32, ((page * a.G + g) * a.block_tokens + in_page) * a.dv + c, row[a.v_off + i]);
        }
    } else {
        float* act = a.act + (size_t)t * a.ldp;
        for (int i = threadIdx.x; i < a.act_n; i += blockDim.x) act[i] = sa_silu(act[i]);
    }
}
cudaError_t sigmoid_attn_store_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(sigmoid_attn_store_kernel, dim3(r.T, a.act_n > 0 ? 3 : 2), dim3(256), 0, s, a, r);
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

// Tensor-core prompt attention (bf16 pages, key and value sizes multiples of 16 up to 128): a CTA takes one tile of up to 64
// consecutive queries of a segment and one head; 4 warps x 16 query rows; keys in blocks of 64, from the block that holds the
// chunk start of the tile's first query to the block of its last query, staged in shared memory once for all 64 queries.
// S = Q K^T and O += P V with mma.sync m16n8k16 (bf16 in, f32 accumulate); scale, cap, bias, sigmoid and mask are 32-bit.
// Queries and weights enter the products as TWO bf16 each (value = leading part + remainder), so the only 16-bit rounding on
// this path is that of the cached keys and values -- the same as on the few-token path. Nothing is rescaled between blocks:
// the weights are not normalised, so the output is a plain running sum.
constexpr int SM_Q = 64, SM_K = 64;
__device__ __forceinline__ void sa_cp_async_16z(void* smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void sa_ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void sa_ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void sa_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sa_split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int DMAX, int DVMAX>
__global__ void __launch_bounds__(128) sigmoid_attn_mma_kernel(SigmoidAttnArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char sa_smem[];
    const int d = a.d, dv = a.dv, LD = d + 8, LDV = dv + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sa_smem);     // [64][LD] leading bf16 of the query
    __nv_bfloat16* Ql = Qs + SM_Q * LD;                                 // [64][LD] what the first bf16 leaves over
    __nv_bfloat16* Ks = Ql + SM_Q * LD;                                 // [64][LD]
    __nv_bfloat16* Vs = Ks + SM_K * LD;                                 // [64][LDV]
    // late tiles of a chunk have the most key blocks: they start first
    const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = r.tile_seg[tile], row0 = r.tile_row0[tile];
    const int nq = min(SM_Q, r.seg_start[seg] + r.seg_len[seg] - row0);
    const int p0 = r.tok_pos[row0], p_last = p0 + nq - 1;
    const int* table = a.block_tables[r.seg_slot[seg]];
    const int g = h / (a.H / a.G);
    const float bias = a.bias ? a.bias[h] : 0.f;
    const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(a.k_pool);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(a.v_pool);
    for (int i = threadIdx.x; i < SM_Q * (d / 2); i += blockDim.x) {
        const int rr = i / (d / 2), c = (i % (d / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (rr < nq) v = *reinterpret_cast<const float2*>(a.q_out + (size_t)(row0 + rr) * a.H * d + (size_t)h * d + c);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(Qs + rr * LD + c) = hi;
        *reinterpret_cast<__nv_bfloat162*>(Ql + rr * LD + c) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
    }
    const int lo_first = a.chunk > 0 ? p0 / a.chunk * a.chunk : 0;
    const int b0 = lo_first / SM_K, b1 = p_last / SM_K;
    float o[DVMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int gq = lane >> 2, tq = lane & 3;
    const int qrow[2] = {warp * 16 + gq, warp * 16 + gq + 8};
    int qlo[2];                                    // first visible key of the lane's two query rows
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) { const int i = p0 + qrow[q2]; qlo[q2] = a.chunk > 0 ? i / a.chunk * a.chunk : 0; }
    for (int kb = b0; kb <= b1; kb++) {
        const int j0 = kb * SM_K;
        __syncthreads();                      // everybody is done with the previous block's K and V (and Q is written)
        for (int i = threadIdx.x; i < SM_K * (d / 8); i += blockDim.x) {
            const int rr = i / (d / 8), c = (i % (d / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + g) * a.block_tokens + jj % a.block_tokens) * d + c;
            sa_cp_async_16z(Ks + rr * LD + c, kp + base, j <= p_last ? 16 : 0);
        }
        for (int i = threadIdx.x; i < SM_K * (dv / 8); i += blockDim.x) {
            const int rr = i / (dv / 8), c = (i % (dv / 8)) * 8;
            const int j = j0 + rr, jj = min(j, p_last);
            const size_t base = (((size_t)table[jj / a.block_tokens] * a.G + g) * a.block_tokens + jj % a.block_tokens) * dv + c;
            sa_cp_async_16z(Vs + rr * LDV + c, vp + base, j <= p_last ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        float sacc[SM_K / 8][4];
#pragma unroll
        for (int ni = 0; ni < SM_K / 8; ni++) sacc[ni][0] = sacc[ni][1] = sacc[ni][2] = sacc[ni][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DMAX; ks += 16) {
            if (ks < d) {
                uint32_t af[4], al[4];
                sa_ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
                sa_ldsm_x4(al, Ql + (warp * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8);
#pragma unroll
                for (int nj = 0; nj < SM_K / 16; nj++) {
                    uint32_t bf[4];
                    sa_ldsm_x4(bf, Ks + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + ks + ((lane >> 3) & 1) * 8);
                    sa_mma_16816(sacc[2 * nj], al, bf[0], bf[1]);
                    sa_mma_16816(sacc[2 * nj + 1], al, bf[2], bf[3]);
                    sa_mma_16816(sacc[2 * nj], af, bf[0], bf[1]);
                    sa_mma_16816(sacc[2 * nj + 1], af, bf[2], bf[3]);
                }
            }
        }
        // weights: capped score + bias through the sigmoid; keys outside the query's chunk or after it weigh nothing
#pragma unroll
        for (int ni = 0; ni < SM_K / 8; ni++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int rr = qrow[e >> 1], i = p0 + rr, j = j0 + ni * 8 + 2 * tq + (e & 1);
                const bool vis = rr < nq && j <= i && j >= qlo[e >> 1];
                sacc[ni][e] = vis ? sa_weight(sacc[ni][e], a.scale, a.softcap, bias) : 0.f;
            }
#pragma unroll
        for (int kc = 0; kc < SM_K / 16; kc++) {
            uint32_t pf[4], pl[4];
            sa_split_bf16(sacc[2 * kc][0], sacc[2 * kc][1], pf[0], pl[0]);
            sa_split_bf16(sacc[2 * kc][2], sacc[2 * kc][3], pf[1], pl[1]);
            sa_split_bf16(sacc[2 * kc + 1][0], sacc[2 * kc + 1][1], pf[2], pl[2]);
            sa_split_bf16(sacc[2 * kc + 1][2], sacc[2 * kc + 1][3], pf[3], pl[3]);
#pragma unroll
            for (int nd = 0; nd < DVMAX / 16; nd++) {
                if (nd * 16 < dv) {
                    uint32_t vf[4];
                    sa_ldsm_x4_t(vf, Vs + (kc * 16 + (lane & 15)) * LDV + nd * 16 + (lane >> 4) * 8);
                    sa_mma_16816(o[2 * nd], pl, vf[0], vf[1]);
                    sa_mma_16816(o[2 * nd + 1], pl, vf[2], vf[3]);
                    sa_mma_16816(o[2 * nd], pf, vf[0], vf[1]);
                    sa_mma_16816(o[2 * nd + 1], pf, vf[2], vf[3]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < DVMAX / 8; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int rr = qrow[e >> 1], c = i * 8 + 2 * tq + (e & 1);
            if (rr < nq && c < dv) a.out[(size_t)(row0 + rr) * a.ld_out + (size_t)h * dv + c] = o[i][e] * a.out_scale;
        }
}

template <int DMAX, int DVMAX>
static cudaError_t sigmoid_attn_mma_pick(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    const size_t smem = (size_t)(3 * 64 * (a.d + 8) + 64 * (a.dv + 8)) * 2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(sigmoid_attn_mma_kernel<DMAX, DVMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (3 * 64 * (DMAX + 8) + 64 * (DVMAX + 8)) * 2);
        attr_done = true;
    }
    return launch_chain(sigmoid_attn_mma_kernel<DMAX, DVMAX>, dim3(r.n_tiles, a.H), dim3(128), smem, s, a, r);
}

cudaError_t sigmoid_attn_launch(const SigmoidAttnArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.d > SA_MAXE * 32 || a.dv > SA_MAXE * 32 || a.H % a.G) return cudaErrorInvalidValue;
    static const bool no_mma = getenv("B2_NO_ATTN_MMA") != nullptr;        // tuning aid: scalar attention for prompts too
    if (!no_mma && !a.cache_f32 && r.T > 8 && a.d % 16 == 0 && a.dv % 16 == 0 && a.d <= 128 && a.dv <= 128) {
        if (a.d <= 64) return a.dv <= 64 ? sigmoid_attn_mma_pick<64, 64>(a, r, s) : sigmoid_attn_mma_pick<64, 128>(a, r, s);
        return a.dv <= 64 ? sigmoid_attn_mma_pick<128, 64>(a, r, s) : sigmoid_attn_mma_pick<128, 128>(a, r, s);
    }
    const dim3 grid(r.T, a.H);
    return a.cache_f32 ? launch_chain(sigmoid_attn_kernel<true>, grid, dim3(SA_WARPS * 32), 0, s, a, r)
                       : launch_chain(sigmoid_attn_kernel<false>, grid, dim3(SA_WARPS * 32), 0, s, a, r);
}

}  // namespace b2
