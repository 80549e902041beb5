// Dense products for the layer-list models: Y[T][N] = epi(X[T][K] . W[N][K]^T + bias), weights bf16 or f32 as stored
// in the file, activations f32 in memory. Three kernels:
//   dense_rows_kernel   T <= 8 (decode steps): one warp per weight row, the row is streamed once for all tokens
//   dense_mma_kernel    T > 8, bf16 weights: tensor cores (mma.sync m16n8k16 bf16, f32 accumulate), X rounded to bf16
//   dense_fma_kernel    T > 8, exact mode (or f32 weights): 32-bit multiply-adds, nothing rounded
// Every output element is one sum over k in a fixed order that depends only on (K, kernel), never on T or on the
// other rows, so a token's result is the same whatever else shares the step. Arbitrary T, N, K (edges are guarded).
// The llama graph's counterpart (quantised blocks, tcgen05) is gemm.cu / matvec.cu.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"
#include "quant_blocks.cuh"

#include <algorithm>

namespace b2 {

__device__ __forceinline__ float ld_w(const __nv_bfloat16* w, size_t i) { return __bfloat162float(w[i]); }
__device__ __forceinline__ float ld_w(const float* w, size_t i) { return w[i]; }

// what a kernel needs beyond its operands: epilogue, batch strides, grouping (DenseArgs, by value)
struct DenseDev {
    const float* x; int ldx;
    const void* w;
    const float* bias;
    float* y; int ldy;
    int T, N, K, epi;
    float scale, p0, p1;
    const float* aux; int ldaux;
    long x_bs, w_bs, y_bs, aux_bs;
    int grouped;                   // 0 plain, 1 one pair per blockIdx.y, 2 tiles
    DenseGroups g;
};

// The rows [t0, t1) this CTA computes and the operands they use. false: nothing to do.
template <typename TW>
__device__ __forceinline__ bool dense_tile(const DenseDev& a, int rows_per_cta, const float*& x, const TW*& w, float*& y, const float*& aux,
                                           int& t0, int& t1) {
    x = a.x; w = reinterpret_cast<const TW*>(a.w); y = a.y; aux = a.aux;
    if (a.grouped == 0) {
        const long b = blockIdx.z;
        x += b * a.x_bs; w += b * a.w_bs; y += b * a.y_bs;
        if (aux) aux += b * a.aux_bs;
        t0 = blockIdx.y * rows_per_cta; t1 = a.T;
        return t0 < t1;
    }
    if (a.grouped == 1) {
        const int p = blockIdx.y, g = a.g.group[p];
        if (g < 0 || g >= a.g.n_groups) return false;
        w += (long)g * a.g.w_stride;
        t0 = p; t1 = p + 1;
        return true;
    }
    const int tile = blockIdx.y;
    if (tile >= *a.g.n_tiles) return false;
    w += (long)a.g.tile_group[tile] * a.g.w_stride;
    t0 = a.g.tile_row0[tile]; t1 = t0 + a.g.tile_rows[tile];
    return true;
}
__device__ __forceinline__ int x_row(const DenseDev& a, int t) { return (a.grouped && a.g.x_rows) ? a.g.x_rows[t] : t; }

__device__ __forceinline__ float silu_act(float z) { return z / (1.f + expf(-z)); }
// one output column
__device__ __forceinline__ void epi_store(const DenseDev& a, float* y, const float* aux, int t, int n, float v) {
    if (a.epi == EPI_BIAS || a.epi == EPI_BIAS_RELU2) { if (a.bias) v += a.bias[n]; }
    if (a.epi == EPI_BIAS_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
    if (a.epi == EPI_MUL_SIGMOID) v *= 1.f / (1.f + expf(-aux[(size_t)t * a.ldaux + n]));
    if (a.epi == EPI_PIECEWISE) v = v > 0.f ? fmaf(a.p0 * v, v, 0.5f * v) : fmaf(a.p1, expm1f(v) - v, 0.5f * v);
    y[(size_t)t * a.ldy + n] = v * a.scale;
}
// two neighbouring columns n (even) and n + 1
__device__ __forceinline__ void epi_store2(const DenseDev& a, float* y, const float* aux, int t, int n, float v0, float v1) {
    if (a.epi == EPI_GLU_SILU) {
        if (n + 1 < a.N) y[(size_t)t * a.ldy + (n >> 1)] = silu_act(v0) * v1 * a.scale;
        return;
    }
    if (a.epi == EPI_GLU_CLAMP) {
        const float g = fminf(v0, a.p0), u = fminf(fmaxf(v1, -a.p0), a.p0);
        if (n + 1 < a.N) y[(size_t)t * a.ldy + (n >> 1)] = g / (1.f + expf(-a.p1 * g)) * (u + 1.f) * a.scale;
        return;
    }
    if (n < a.N) epi_store(a, y, aux, t, n, v0);
    if (n + 1 < a.N) epi_store(a, y, aux, t, n + 1, v1);
}

// ---------------------------------------------------------------- few tokens: a warp per R weight rows
// TT = compiled token count (1, 2, 4 or 8 >= T), R = rows per warp (the activations a lane loads serve R rows: with several
// tokens the activation loads, not the weights, fill the load pipe). Fast path (K % 8 == 0, 16-byte aligned rows): a lane takes
// 8 consecutive weights per load and keeps R x U = 4 loads in flight, 2 KB per warp on the wire. Each output is still one sum
// over k in an order that depends on K alone.
constexpr int ROWS_MAX_T = 8;
template <typename TW, int TT, int R>
__global__ void __launch_bounds__(256) dense_rows_kernel(DenseDev a) {
    griddep_launch();
    griddep_wait();
    constexpr int U = 4 / R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = a.N, K = a.K, ldx = a.ldx;
    const int n0 = (blockIdx.x * 8 + warp) * R;
    if (n0 >= N) return;
    const float* x; const TW* w; float* y; const float* aux; int t0, t1;
    if (!dense_tile<TW>(a, ROWS_MAX_T, x, w, y, aux, t0, t1)) return;
    const int T = a.grouped ? 1 : a.T;
    if (a.grouped) { x += (size_t)x_row(a, t0) * ldx; y += (size_t)t0 * a.ldy; if (aux) aux += (size_t)t0 * a.ldaux; }
    const TW* rows[R];
#pragma unroll
    for (int r = 0; r < R; r++) rows[r] = w + (size_t)min(n0 + r, N - 1) * K;      // past the end: the last row again, not stored
    float acc[TT][R];
#pragma unroll
    for (int t = 0; t < TT; t++)
#pragma unroll
        for (int r = 0; r < R; r++) acc[t][r] = 0.f;
    const bool vec = (K % 8 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    if (vec) {
        auto load8 = [&](const TW* row, int k, float (&wv)[8]) {
            if constexpr (sizeof(TW) == 2) {
                const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(row + k));       // streamed once: do not keep in L1
                const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; i++) { wv[2 * i] = __uint_as_float(u[i] << 16); wv[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
            } else {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(row + k)), b = __ldcs(reinterpret_cast<const float4*>(row + k + 4));
                wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
            }
        };
        auto fma8 = [&](const float (&wv)[R][8], int k) {
#pragma unroll
            for (int t = 0; t < TT; t++)
                if (t < T) {
                    const float4 a = *reinterpret_cast<const float4*>(x + (size_t)t * ldx + k);
                    const float4 b = *reinterpret_cast<const float4*>(x + (size_t)t * ldx + k + 4);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        float v = acc[t][r];
                        v = fmaf(a.x, wv[r][0], v); v = fmaf(a.y, wv[r][1], v); v = fmaf(a.z, wv[r][2], v); v = fmaf(a.w, wv[r][3], v);
                        v = fmaf(b.x, wv[r][4], v); v = fmaf(b.y, wv[r][5], v); v = fmaf(b.z, wv[r][6], v); v = fmaf(b.w, wv[r][7], v);
                        acc[t][r] = v;
                    }
                }
        };
        int k = lane * 8;
        for (; k + (U - 1) * 256 < K; k += U * 256) {
            float wv[U][R][8];
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < R; r++) load8(rows[r], k + u * 256, wv[u][r]);
#pragma unroll
            for (int u = 0; u < U; u++) fma8(wv[u], k + u * 256);
        }
        for (; k < K; k += 256) {
            float wv[R][8];
#pragma unroll
            for (int r = 0; r < R; r++) load8(rows[r], k, wv[r]);
            fma8(wv, k);
        }
    } else {
        // lanes take k = lane, lane + 32, ...: neighbouring lanes read neighbouring weights
        for (int k = lane; k < K; k += 32) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float wv = ld_w(rows[r], k);
#pragma unroll
                for (int t = 0; t < TT; t++)
                    if (t < T) acc[t][r] = fmaf(x[(size_t)t * ldx + k], wv, acc[t][r]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        if (t >= T) continue;
        float v[R];
#pragma unroll
        for (int r = 0; r < R; r++) v[r] = warp_sum(acc[t][r]);
        if (lane != 0) continue;
        if constexpr (R % 2 == 0) {
#pragma unroll
            for (int r = 0; r < R; r += 2) epi_store2(a, y, aux, t, n0 + r, v[r], v[r + 1]);
        } else {
            epi_store(a, y, aux, t, n0, v[0]);
        }
    }
}

template <typename TW>
static cudaError_t launch_rows(const DenseDev& d, int batch, cudaStream_t s) {
    dim3 block(256);
    const unsigned gy = d.grouped ? d.T : 1, gz = d.grouped ? 1 : batch;       // grouped: one pair row per blockIdx.y
    const int N = d.N;
    if (d.grouped || d.T == 1) {
        if (d.epi == EPI_GLU_SILU || d.epi == EPI_GLU_CLAMP) return launch_chain(dense_rows_kernel<TW, 1, 2>, dim3((N + 15) / 16, gy, gz), block, 0, s, d);
        return launch_chain(dense_rows_kernel<TW, 1, 1>, dim3((N + 7) / 8, gy, gz), block, 0, s, d);
    }
    if (d.T == 2) return launch_chain(dense_rows_kernel<TW, 2, 2>, dim3((N + 15) / 16, gy, gz), block, 0, s, d);
    if (d.T <= 4) return launch_chain(dense_rows_kernel<TW, 4, 4>, dim3((N + 31) / 32, gy, gz), block, 0, s, d);
    return launch_chain(dense_rows_kernel<TW, 8, 4>, dim3((N + 31) / 32, gy, gz), block, 0, s, d);
}

// ---------------------------------------------------------------- exact: 64 x 64 tile, 16-deep, 4 x 4 per thread
template <typename TW>
__global__ void __launch_bounds__(256) dense_fma_kernel(DenseDev a) {
    griddep_launch();
    griddep_wait();
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const float* x; const TW* w; float* y; const float* aux; int t0, T;
    if (!dense_tile<TW>(a, BM, x, w, y, aux, t0, T)) return;
    const int N = a.N, K = a.K, ldx = a.ldx;
    const int n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // thread tile: rows ty*4.., cols tx*4..
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, kk = i % BK;
            const int t = t0 + r, k = k0 + kk;
            xs[kk][r] = (t < T && k < K) ? x[(size_t)x_row(a, t) * ldx + k] : 0.f;
            const int n = n0 + r;
            ws[kk][r] = (n < N && k < K) ? ld_w(w, (size_t)n * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = xs[kk][ty * 4 + i]; b[i] = ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j += 2) epi_store2(a, y, aux, t, n0 + tx * 4 + j, acc[i][j], acc[i][j + 1]);
    }
}

// ---------------------------------------------------------------- tensor cores: 64 x 64 tile, 32-deep, 4 warps of 32 x 32
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128) dense_mma_kernel(DenseDev a) {
    griddep_launch();
    griddep_wait();
    constexpr int BM = 64, BN = 64, BK = 32, LD = BK + 8;      // rows padded by 16 bytes: fragment reads hit 32 banks
    __shared__ __align__(16) __nv_bfloat16 xs[BM][LD];
    __shared__ __align__(16) __nv_bfloat16 ws[BN][LD];
    const float* x; const __nv_bfloat16* w; float* y; const float* aux; int t0, T;
    if (!dense_tile<__nv_bfloat16>(a, BM, x, w, y, aux, t0, T)) return;
    const int N = a.N, K = a.K, ldx = a.ldx;
    const int n0 = blockIdx.x * BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int g = lane >> 2, tq = lane & 3;
    float acc[2][4][4] = {};
    const bool w_vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    for (int k0 = 0; k0 < K; k0 += BK) {
        // X tile: f32 -> bf16 (round to nearest even), 64 x 32
        for (int i = threadIdx.x; i < BM * BK / 2; i += 128) {
            const int r = i / (BK / 2), kk = (i % (BK / 2)) * 2;
            const int t = t0 + r, k = k0 + kk;
            float v0 = 0.f, v1 = 0.f;
            if (t < T) {
                const float* xr = x + (size_t)x_row(a, t) * ldx;
                if (k < K) v0 = xr[k];
                if (k + 1 < K) v1 = xr[k + 1];
            }
            *reinterpret_cast<__nv_bfloat162*>(&xs[r][kk]) = __floats2bfloat162_rn(v0, v1);
        }
        // W tile: 64 rows x 32 bf16
        if (w_vec) {
            for (int i = threadIdx.x; i < BN * BK / 8; i += 128) {
                const int r = i / (BK / 8), kk = (i % (BK / 8)) * 8;
                const int n = n0 + r, k = k0 + kk;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (n < N && k < K) v = *reinterpret_cast<const uint4*>(w + (size_t)n * K + k);
                *reinterpret_cast<uint4*>(&ws[r][kk]) = v;
            }
        } else {
            for (int i = threadIdx.x; i < BN * BK; i += 128) {
                const int r = i / BK, kk = i % BK;
                const int n = n0 + r, k = k0 + kk;
                ws[r][kk] = (n < N && k < K) ? w[(size_t)n * K + k] : __float2bfloat16(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < BK; ks += 16) {
            uint32_t af[2][4], bf[4][2];
#pragma unroll
            for (int mi = 0; mi < 2; mi++) {
                const int r = wm + mi * 16 + g;
                af[mi][0] = *reinterpret_cast<const uint32_t*>(&xs[r][ks + 2 * tq]);
                af[mi][1] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][ks + 2 * tq]);
                af[mi][2] = *reinterpret_cast<const uint32_t*>(&xs[r][ks + 2 * tq + 8]);
                af[mi][3] = *reinterpret_cast<const uint32_t*>(&xs[r + 8][ks + 2 * tq + 8]);
            }
#pragma unroll
            for (int ni = 0; ni < 4; ni++) {
                const int c = wn + ni * 8 + g;
                bf[ni][0] = *reinterpret_cast<const uint32_t*>(&ws[c][ks + 2 * tq]);
                bf[ni][1] = *reinterpret_cast<const uint32_t*>(&ws[c][ks + 2 * tq + 8]);
            }
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
#pragma unroll
                for (int ni = 0; ni < 4; ni++) mma_bf16_16816(acc[mi][ni], af[mi], bf[ni]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const int t = t0 + wm + mi * 16 + g + (e >> 1) * 8;
                if (t < T) epi_store2(a, y, aux, t, n0 + wn + ni * 8 + 2 * tq, acc[mi][ni][e], acc[mi][ni][e + 1]);
            }
}

// ---------------------------------------------------------------- tensor cores, large steps: 128 x 128 x 64 tiles, 8 warps of
// 64 x 32, three stages of 16-byte asynchronous copies, ldmatrix fragments. X is rounded to bf16 ONCE per product by
// rows_to_bf16_kernel (the 64 x 64 kernel above converts every tile it loads, N / 64 times per element). Needs K % 8 == 0.
__global__ void rows_to_bf16_kernel(const float* __restrict__ x, int ldx, int T, int K, __nv_bfloat16* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    const long n = (long)T * (K / 2);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long t = i / (K / 2);
        const int k = (int)(i % (K / 2)) * 2;
        const float* p = x + t * ldx + k;
        *reinterpret_cast<__nv_bfloat162*>(y + t * K + k) = __floats2bfloat162_rn(p[0], p[1]);
    }
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_src) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_src)));
}

constexpr int BIG_BM = 128, BIG_BN = 128, BIG_BK = 64, BIG_LD = BIG_BK + 8, BIG_STAGES = 3;
constexpr int BIG_SMEM = BIG_STAGES * (BIG_BM + BIG_BN) * BIG_LD * 2;
__global__ void __launch_bounds__(256, 2) dense_mma_big_kernel(const __nv_bfloat16* __restrict__ xb, int ldxb, DenseDev a) {
    griddep_launch();
    griddep_wait();
    extern __shared__ __align__(16) unsigned char big_smem[];
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(big_smem);                       // [stage][BM][LD]
    __nv_bfloat16* Bs = As + BIG_STAGES * BIG_BM * BIG_LD;                                  // [stage][BN][LD]
    const float* x; const __nv_bfloat16* w; float* y; const float* aux; int t0, T;
    if (!dense_tile<__nv_bfloat16>(a, BIG_BM, x, w, y, aux, t0, T)) return;
    const int N = a.N, K = a.K;
    const int n0 = blockIdx.x * BIG_BN;
    // the rounded copy holds the input rows as [row][ldxb] (grouped: gathered here; batched: batch b starts at column b * x_bs)
    if (!a.grouped) xb += (long)blockIdx.z * a.x_bs;
    int my_rows[BIG_BK / 16];
#pragma unroll
    for (int it = 0; it < BIG_BK / 16; it++) {
        const int row = (threadIdx.x + it * 256) / (BIG_BK / 8);
        my_rows[it] = x_row(a, min(t0 + row, T - 1));
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
    const int KT = (K + BIG_BK - 1) / BIG_BK;
    auto load_stage = [&](int stage, int kt) {
        const int k0 = kt * BIG_BK;
#pragma unroll
        for (int it = 0; it < BIG_BK / 16; it++) {
            const int c = threadIdx.x + it * 256;          // 128 rows x BK / 8 chunks of 16 bytes per operand tile
            const int row = c / (BIG_BK / 8), kk = (c % (BIG_BK / 8)) * 8;
            const int k = k0 + kk;
            const int t = t0 + row, n = n0 + row;
            const bool ka = k < K;
            cp_async_16(As + ((size_t)stage * BIG_BM + row) * BIG_LD + kk, xb + (size_t)my_rows[it] * ldxb + (ka ? k : 0), (ka && t < T) ? 16 : 0);
            cp_async_16(Bs + ((size_t)stage * BIG_BN + row) * BIG_LD + kk, w + (size_t)min(n, N - 1) * K + (ka ? k : 0), (ka && n < N) ? 16 : 0);
        }
    };
    float acc[4][4][4] = {};
    for (int s = 0; s < BIG_STAGES - 1; s++) {
        if (s < KT) load_stage(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < KT; kt++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(BIG_STAGES - 2) : "memory");
        __syncthreads();
        const int nxt = kt + BIG_STAGES - 1;
        if (nxt < KT) load_stage(nxt % BIG_STAGES, nxt);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* A = As + (size_t)(kt % BIG_STAGES) * BIG_BM * BIG_LD;
        const __nv_bfloat16* B = Bs + (size_t)(kt % BIG_STAGES) * BIG_BN * BIG_LD;
#pragma unroll
        for (int ks = 0; ks < BIG_BK; ks += 16) {
            uint32_t af[4][4], bf[2][4];
#pragma unroll
            for (int mi = 0; mi < 4; mi++) ldmatrix_x4(af[mi], A + (size_t)(wm + mi * 16 + (lane & 15)) * BIG_LD + ks + (lane >> 4) * 8);
#pragma unroll
            for (int nj = 0; nj < 2; nj++)
                ldmatrix_x4(bf[nj], B + (size_t)(wn + nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * BIG_LD + ks + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int mi = 0; mi < 4; mi++)
#pragma unroll
                for (int ni = 0; ni < 4; ni++) {
                    const uint32_t b2[2] = {bf[ni >> 1][(ni & 1) * 2], bf[ni >> 1][(ni & 1) * 2 + 1]};
                    mma_bf16_16816(acc[mi][ni], af[mi], b2);
                }
        }
    }
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 4; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const int t = t0 + wm + mi * 16 + g + (e >> 1) * 8;
                if (t < T) epi_store2(a, y, aux, t, n0 + wn + ni * 8 + 2 * tq, acc[mi][ni][e], acc[mi][ni][e + 1]);
            }
}

cudaError_t dense_launch(const DenseArgs& a, cudaStream_t s) {
    if (a.T <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return cudaErrorInvalidValue;
    if (a.w_type != T_BF16 && a.w_type != T_F32) return cudaErrorInvalidValue;
    if ((a.epi == EPI_GLU_SILU || a.epi == EPI_GLU_CLAMP) && a.N % 2) return cudaErrorInvalidValue;
    if (a.groups && a.batch != 1) return cudaErrorInvalidValue;
    const bool wb = a.w_type == T_BF16;
    DenseDev d = {};
    d.x = a.x; d.ldx = a.ldx; d.w = a.w; d.bias = a.bias; d.y = a.y; d.ldy = a.ldy; d.T = a.T; d.N = a.N; d.K = a.K; d.epi = a.epi;
    d.scale = a.scale; d.p0 = a.p0; d.p1 = a.p1; d.aux = a.aux; d.ldaux = a.ldaux; d.x_bs = a.x_bs; d.w_bs = a.w_bs; d.y_bs = a.y_bs; d.aux_bs = a.aux_bs;
    if (a.groups) { d.g = *a.groups; d.grouped = a.groups->tile_group ? 2 : 1; }
    if (d.grouped == 1 || (!d.grouped && a.T <= ROWS_MAX_T)) return wb ? launch_rows<__nv_bfloat16>(d, a.batch, s) : launch_rows<float>(d, a.batch, s);
    // few output columns in 32-bit (router scores): the tiled kernel would run a handful of CTAs over the whole K; the
    // few-token kernel over chunks of 8 rows keeps every SM busy and streams the small matrix from L2
    if (a.exact && !d.grouped && a.batch == 1 && a.N <= 64) {
        const int chunks = a.T / ROWS_MAX_T, rem = a.T % ROWS_MAX_T;
        DenseDev c = d;
        c.T = ROWS_MAX_T; c.x_bs = (long)ROWS_MAX_T * a.ldx; c.y_bs = (long)ROWS_MAX_T * a.ldy; c.aux_bs = (long)ROWS_MAX_T * a.ldaux; c.w_bs = 0;
        cudaError_t ce = wb ? launch_rows<__nv_bfloat16>(c, chunks, s) : launch_rows<float>(c, chunks, s);
        if (ce != cudaSuccess || rem == 0) return ce;
        c = d;
        c.T = rem; c.x += (size_t)chunks * ROWS_MAX_T * a.ldx; c.y += (size_t)chunks * ROWS_MAX_T * a.ldy;
        if (c.aux) c.aux += (size_t)chunks * ROWS_MAX_T * a.ldaux;
        return wb ? launch_rows<__nv_bfloat16>(c, 1, s) : launch_rows<float>(c, 1, s);
    }
    const unsigned gz = d.grouped ? 1 : a.batch;
    // The large-tile kernel reads a rounded copy of the input: [T][K]; batched: [T][x_span] with batch b at column b * x_bs;
    // grouped (128-row tiles): [x_total_rows][K], gathered by the kernel.
    const int x_rows_total = d.grouped ? a.groups->x_total_rows : a.T;
    const int span = a.batch > 1 ? a.x_span : a.K;
    const bool big_ok = wb && !a.exact && a.xb && a.K % 8 == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && span % 8 == 0 &&
                        (a.batch == 1 || (a.x_span > 0 && a.x_bs % 8 == 0 && a.w_bs % 8 == 0));
    if (d.grouped == 2 && a.groups->tile_max == BIG_BM && !big_ok) return cudaErrorInvalidValue;
    if (big_ok && (d.grouped ? a.groups->tile_max == BIG_BM : a.T >= 64)) {
        static bool attr_done = false;
        if (!attr_done) { cudaFuncSetAttribute(dense_mma_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BIG_SMEM); attr_done = true; }
        const long pairs = (long)x_rows_total * (span / 2);
        cudaError_t ce = launch_chain(rows_to_bf16_kernel, dim3((unsigned)std::min<long>((pairs + 255) / 256, 148 * 8)), dim3(256), 0, s,
                                      a.x, a.ldx, x_rows_total, span, a.xb);
        if (ce != cudaSuccess) return ce;
        const unsigned gy = d.grouped ? (unsigned)a.groups->max_tiles : (unsigned)((a.T + BIG_BM - 1) / BIG_BM);
        return launch_chain(dense_mma_big_kernel, dim3((a.N + BIG_BN - 1) / BIG_BN, gy, gz), dim3(256), (size_t)BIG_SMEM, s,
                            (const __nv_bfloat16*)a.xb, span, d);
    }
    dim3 grid((a.N + 63) / 64, d.grouped ? (unsigned)a.groups->max_tiles : (unsigned)((a.T + 63) / 64), gz);
    if (wb && !a.exact) return launch_chain(dense_mma_kernel, grid, dim3(128), 0, s, d);
    if (wb) return launch_chain(dense_fma_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, d);
    return launch_chain(dense_fma_kernel<float>, grid, dim3(256), 0, s, d);
}

}  // namespace b2
