// Several copies of the residual stream (layered.h: HyperJoinArgs). One pass per sublayer boundary writes the pending sublayer
// output back into every copy through the layer's mixing matrix, reads the next sublayer's input as the RMS-normed weighted
// sum of the copies, and / or leaves the plain sum of the copies for the output norm. Everything is 32-bit.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

namespace b2 {

constexpr int HY_MAX_S = 16;       // copies of the stream; the kernels are compiled for up to 4, 8 and 16

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

// one token: write the pending output back, sum the copies, read the next sublayer's input. With `row` (shared, [W]) the normed
// input is left there for the caller (all threads have passed a barrier after the last write); else it goes to a.hn.
template <int SM>
__device__ __forceinline__ void hyper_token(const HyperDev& p, int t, float* hy_row, float* red, const float* s_mix, const float* s_out,
                                            const float* s_in, bool keep_in_row) {
    const HyperJoinArgs& a = p.a;
    const int W = p.W, S = a.S;
    const size_t base = (size_t)t * W;
    const bool pending = a.a != nullptr || p.moe_on;
    // a two-branch output: both branches are normed over the width first
    float ra = 1.f, rb = 1.f;
    if (a.b) {
        float sa = 0.f, sb = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) { const float u = a.a[base + i], v = a.b[base + i]; sa = fmaf(u, u, sa); sb = fmaf(v, v, sb); }
        ra = 1.f / sqrtf(hy_block_sum(sa, red) / (float)W + a.eps);
        rb = 1.f / sqrtf(hy_block_sum(sb, red) / (float)W + a.eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float x[SM];
#pragma unroll
        for (int s = 0; s < SM; s++) if (s < S) x[s] = a.xs[(a.bcast ? 0 : s) * a.stream_stride + base + i];
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
            float nx[SM];
#pragma unroll
            for (int to = 0; to < SM; to++) {
                if (to >= S) continue;
                float v = s_out[to] * y;
#pragma unroll
                for (int s = 0; s < SM; s++) if (s < S) v = fmaf(s_mix[s * S + to], x[s], v);
                nx[to] = v;
            }
#pragma unroll
            for (int s = 0; s < SM; s++) if (s < S) x[s] = nx[s];
        }
        if (pending || a.bcast) {
#pragma unroll
            for (int s = 0; s < SM; s++) if (s < S && (pending || s > 0)) a.xs[s * a.stream_stride + base + i] = x[s];
        }
        if (a.sum_out) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < SM; s++) if (s < S) v += x[s];
            a.sum_out[base + i] = v;
        }
        if (a.hn) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < SM; s++) if (s < S) u = fmaf(s_in[s], x[s], u);
            hy_row[i] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!a.hn) return;
    const float rinv = 1.f / sqrtf(hy_block_sum(ss, red) / (float)W + a.eps);
    if (keep_in_row) {
        for (int i = threadIdx.x; i < W; i += blockDim.x) hy_row[i] = hy_row[i] * rinv * a.norm_w[i];
        __syncthreads();
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) a.hn[base + i] = hy_row[i] * rinv * a.norm_w[i];
    }
}

__device__ __forceinline__ void hyper_tables(const HyperJoinArgs& a, float* s_mix, float* s_out, float* s_in) {
    const int S = a.S;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = a.mix ? a.mix[i] : (i / S == i % S ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) { s_out[i] = a.out ? a.out[i] : 1.f; s_in[i] = a.in ? a.in[i] : (i == 0 ? 1.f : 0.f); }
    __syncthreads();
}

// grid (T), NT threads (256 when the step has many tokens, 1024 when it has few: a decoded token's row is then walked in a quarter
// of the rounds, and the kernel is bound by the latency of those rounds); shared: [W] the next sublayer's input before its norm
template <int NT, int SM>
__global__ void __launch_bounds__(NT) hyper_join_kernel(HyperDev p) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float hy_row[];
    __shared__ float red[33];
    __shared__ float s_mix[HY_MAX_S * HY_MAX_S], s_out[HY_MAX_S], s_in[HY_MAX_S];
    hyper_tables(p.a, s_mix, s_out, s_in);
    hyper_token<SM>(p, blockIdx.x, hy_row, red, s_mix, s_out, s_in, false);
}

// Few-token steps: the same pass joined to the convolution around a skip on the sublayer's input and to the hand-over of its
// state. grid (n_seg), 1024 threads: a CTA walks its segment's tokens in order; the normed inputs of the last `taps` tokens live
// in a ring in shared memory ([taps][W]); older ones come from the slot's state, which is rewritten at the end. The sums run in
// the order of causal_conv_kernel, so both paths give the same numbers.
template <int SM>
__global__ void __launch_bounds__(1024) hyper_join_conv_kernel(HyperDev p, ConvArgs cv, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float hy_ring[];
    __shared__ float red[33];
    __shared__ float s_mix[HY_MAX_S * HY_MAX_S], s_out[HY_MAX_S], s_in[HY_MAX_S];
    hyper_tables(p.a, s_mix, s_out, s_in);
    const int seg = blockIdx.x, slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int W = p.W, taps = cv.taps, hist = taps - 1;
    float* state = cv.state + (size_t)slot * hist * W;
    for (int k = 0; k < len; k++) {
        float* row = hy_ring + (size_t)(k % taps) * W;
        hyper_token<SM>(p, start + k, row, red, s_mix, s_out, s_in, true);
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            float acc = 0.f;
            for (int j = 0; j < taps; j++) {
                const int srci = k - hist + j;
                const float v = srci >= 0 ? hy_ring[(size_t)(srci % taps) * W + c] : state[(size_t)(hist + srci) * W + c];
                acc = fmaf(cv.w[(size_t)c * taps + j], v, acc);
            }
            cv.out[(size_t)(start + k) * cv.ld_out + c] = row[c] + acc;
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        for (int k = 0; k < hist; k++) {               // entry k of the new state is read at k + len > k of the old one before it is written
            const int srci = len + k - hist;
            state[(size_t)k * W + c] = srci >= 0 ? hy_ring[(size_t)(srci % taps) * W + c] : state[(size_t)(k + len) * W + c];
        }
}

template <int SM>
static cudaError_t hyper_join_pick(const HyperDev& p, bool few, int T, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) {
        static bool attr_done = false;
        if (!attr_done) {
            cudaFuncSetAttribute(hyper_join_kernel<256, SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(hyper_join_kernel<1024, SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            attr_done = true;
        }
    }
    if (few && SM <= 8) return launch_chain(hyper_join_kernel<1024, SM>, dim3(T), dim3(1024), smem, s, p);
    return launch_chain(hyper_join_kernel<256, SM>, dim3(T), dim3(256), smem, s, p);
}
template <int SM>
static cudaError_t hyper_join_conv_pick(const HyperDev& p, const ConvArgs& cv, const RaggedDev& r, int W, size_t smem, cudaStream_t s) {
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(hyper_join_conv_kernel<SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); attr_done = true; }
    return launch_chain(hyper_join_conv_kernel<SM>, dim3(r.n_seg), dim3(W >= 1024 ? 1024 : 256), smem, s, p, cv, r);
}

cudaError_t hyper_join_launch(const HyperJoinArgs& a, int W, int T, cudaStream_t s) {
    if (a.S <= 0 || a.S > HY_MAX_S) return cudaErrorInvalidValue;
    HyperDev p = {};
    p.a = a; p.W = W;
    if (a.moe) { p.moe = *a.moe; p.moe_on = 1; }
    p.a.moe = nullptr;
    const size_t smem = (size_t)W * 4;
    const bool few = T <= 16 && W >= 1024;
    return a.S <= 4 ? hyper_join_pick<4>(p, few, T, smem, s) : a.S <= 8 ? hyper_join_pick<8>(p, few, T, smem, s) : hyper_join_pick<16>(p, few, T, smem, s);
}

bool hyper_join_conv_fits(int W, int taps, int T, int S) { return T <= 8 && S <= 8 && taps >= 1 && (size_t)taps * W * 4 <= 160 * 1024; }

cudaError_t hyper_join_conv_launch(const HyperJoinArgs& a, const ConvArgs& cv, const RaggedDev& r, int W, cudaStream_t s) {
    if (a.S <= 0 || a.S > HY_MAX_S || !a.hn || !cv.skip || cv.C != W || cv.ld_in != W) return cudaErrorInvalidValue;
    HyperDev p = {};
    p.a = a; p.W = W;
    if (a.moe) { p.moe = *a.moe; p.moe_on = 1; }
    p.a.moe = nullptr;
    const size_t smem = (size_t)cv.taps * W * 4;
    if (a.S > 8) return cudaErrorInvalidValue;          // more copies take the separate kernels (hyper_join_conv_fits)
    return a.S <= 4 ? hyper_join_conv_pick<4>(p, cv, r, W, smem, s) : hyper_join_conv_pick<8>(p, cv, r, W, smem, s);
}

}  // namespace b2
