// Several copies of the residual stream (layered.h: HyperJoinArgs). One pass per sublayer boundary writes the pending sublayer
// output back into every copy through the layer's mixing matrix, reads the next sublayer's input as the RMS-normed weighted
// sum of the copies, and / or leaves the plain sum of the copies for the output norm. Everything is 32-bit.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

namespace b2 {

constexpr int HY_MAX_S = 8;

namespace {
struct HyperDev {
    HyperJoinArgs a;
    MoeJoinArgs moe; int moe_on;
    int W;
};
__device__ __forceinline__ float hy_block_sum(float v, float* red) {      // all threads get the sum; red: >= 33 floats
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
}  // namespace

// grid (T), 256 threads; shared: [W] the next sublayer's input before its norm
__global__ void __launch_bounds__(256) hyper_join_kernel(HyperDev p) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float hy_row[];
    __shared__ float red[33];
    __shared__ float s_mix[HY_MAX_S * HY_MAX_S], s_out[HY_MAX_S], s_in[HY_MAX_S];
    const HyperJoinArgs& a = p.a;
    const int t = blockIdx.x, W = p.W, S = a.S;
    const size_t base = (size_t)t * W;
    const bool pending = a.a != nullptr || p.moe_on;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = a.mix ? a.mix[i] : (i / S == i % S ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) { s_out[i] = a.out ? a.out[i] : 1.f; s_in[i] = a.in ? a.in[i] : (i == 0 ? 1.f : 0.f); }
    // a two-branch output: both branches are normed over the width first
    float ra = 1.f, rb = 1.f;
    if (a.b) {
        float sa = 0.f, sb = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) { const float u = a.a[base + i], v = a.b[base + i]; sa = fmaf(u, u, sa); sb = fmaf(v, v, sb); }
        ra = 1.f / sqrtf(hy_block_sum(sa, red) / (float)W + a.eps);
        rb = 1.f / sqrtf(hy_block_sum(sb, red) / (float)W + a.eps);
    }
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float x[HY_MAX_S];
#pragma unroll
        for (int s = 0; s < HY_MAX_S; s++) if (s < S) x[s] = a.xs[(a.bcast ? 0 : s) * a.stream_stride + base + i];
        if (pending) {
            float y = 0.f;
            if (a.b) y = 0.5f * (a.a[base + i] * ra * a.wa[i] + a.b[base + i] * rb * a.wb[i]);
            else if (a.a) y = a.a[base + i];
            if (p.moe_on) {
                const MoeJoinArgs& j = p.moe;
                for (int c = 0; c < j.top; c++) {
                    const int q = t * j.top + c, e = j.sel[q];
                    const float v = e < j.n_experts ? j.rows[(size_t)(j.pos ? j.pos[q] : q) * W + i] : j.h[base + i];
                    y = fmaf(j.weight[q], v, y);
                }
            }
            float nx[HY_MAX_S];
#pragma unroll
            for (int to = 0; to < HY_MAX_S; to++) {
                if (to >= S) continue;
                float v = s_out[to] * y;
#pragma unroll
                for (int s = 0; s < HY_MAX_S; s++) if (s < S) v = fmaf(s_mix[s * S + to], x[s], v);
                nx[to] = v;
            }
#pragma unroll
            for (int s = 0; s < HY_MAX_S; s++) if (s < S) x[s] = nx[s];
        }
        if (pending || a.bcast) {
#pragma unroll
            for (int s = 0; s < HY_MAX_S; s++) if (s < S && (pending || s > 0)) a.xs[s * a.stream_stride + base + i] = x[s];
        }
        if (a.sum_out) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < HY_MAX_S; s++) if (s < S) v += x[s];
            a.sum_out[base + i] = v;
        }
        if (a.hn) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HY_MAX_S; s++) if (s < S) u = fmaf(s_in[s], x[s], u);
            hy_row[i] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!a.hn) return;
    const float rinv = 1.f / sqrtf(hy_block_sum(ss, red) / (float)W + a.eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) a.hn[base + i] = hy_row[i] * rinv * a.norm_w[i];
}

cudaError_t hyper_join_launch(const HyperJoinArgs& a, int W, int T, cudaStream_t s) {
    if (a.S <= 0 || a.S > HY_MAX_S) return cudaErrorInvalidValue;
    HyperDev p = {};
    p.a = a; p.W = W;
    if (a.moe) { p.moe = *a.moe; p.moe_on = 1; }
    p.a.moe = nullptr;
    const size_t smem = (size_t)W * 4;
    if (smem > 48 * 1024) {
        static bool attr_done = false;
        if (!attr_done) { cudaFuncSetAttribute(hyper_join_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); attr_done = true; }
    }
    return launch_chain(hyper_join_kernel, dim3(T), dim3(256), smem, s, p);
}

}  // namespace b2
