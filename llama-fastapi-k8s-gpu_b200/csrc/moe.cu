// Mixture of experts for the layer-list models: routing (softmax scores, additive choice correction, group-limited
// top-k with identity slots; or biased logits with a softmax over the chosen ones), the bookkeeping that sorts a step's (token, choice) pairs by expert into row tiles for the
// grouped products of dense.cu, and the weighted combination. Routing arithmetic is 32-bit.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

#include <algorithm>

namespace b2 {

namespace {
// (value, index) maximum over a warp; ties go to the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
    }
}
}  // namespace

// grid (T), one warp. shared: scores [n_slots], choice scores [n_slots], group maxima [n_groups]
__global__ void __launch_bounds__(32) moe_route_kernel(MoeRouteArgs a) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float rs[];
    float* score = rs;
    float* choice = rs + a.n_slots;
    float* gbest = choice + a.n_slots;
    const int t = blockIdx.x, lane = threadIdx.x, n = a.n_slots;
    const float* z = a.logits + (size_t)t * a.ld;
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, z[i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) { const float e = expf(z[i] - mx); score[i] = e; sum += e; }
    sum = warp_sum(sum);
    for (int i = lane; i < n; i += 32) { const float s = score[i] / sum; score[i] = s; choice[i] = s + (a.correction ? a.correction[i] : 0.f); }
    __syncwarp();
    if (a.n_groups > 1 && a.keep_groups < a.n_groups) {
        const int per = n / a.n_groups;
        for (int g = lane; g < a.n_groups; g += 32) {
            float b = -INFINITY;
            for (int i = 0; i < per; i++) b = fmaxf(b, choice[g * per + i]);
            gbest[g] = b;
        }
        __syncwarp();
        // the groups that are NOT among the best keep_groups lose their slots: pick the best ones one by one
        for (int k = 0; k < a.keep_groups; k++) {
            float v = -INFINITY; int idx = 0x7fffffff;
            for (int g = lane; g < a.n_groups; g += 32) { const float b = gbest[g]; if (b > v || (b == v && g < idx)) { v = b; idx = g; } }
            warp_argmax(v, idx);
            __syncwarp();
            if (lane == 0 && idx < a.n_groups) gbest[idx] = NAN;       // marks a kept group
            __syncwarp();
        }
        for (int i = lane; i < n; i += 32) if (gbest[i / per] == gbest[i / per]) choice[i] = -INFINITY;   // not NaN: dropped
        __syncwarp();
    }
    for (int k = 0; k < a.top; k++) {
        float v = -INFINITY; int idx = 0x7fffffff;
        for (int i = lane; i < n; i += 32) { const float c = choice[i]; if (c > v || (c == v && i < idx)) { v = c; idx = i; } }
        warp_argmax(v, idx);
        if (idx >= n) idx = 0;                     // fewer allowed slots than `top` (a config error): stay in range
        __syncwarp();
        if (lane == 0) {
            a.sel[(size_t)t * a.top + k] = idx;
            a.weight[(size_t)t * a.top + k] = score[idx] * a.scale;
            a.pair_token[(size_t)t * a.top + k] = t;
            choice[idx] = NAN;                     // taken: NaN never wins a comparison
        }
        __syncwarp();
    }
    if (a.renorm) {                                // every lane the same sum, in pick order
        float tot = 0.f;
        for (int k = 0; k < a.top; k++) tot += a.weight[(size_t)t * a.top + k];
        __syncwarp();
        for (int k = lane; k < a.top; k += 32) a.weight[(size_t)t * a.top + k] /= tot / a.scale + 1e-20f;
    }
}
// grid (T), one warp: the `top` largest of logit + bias (ties to the lower index); weights = softmax over those alone.
// shared: biased logits [n_slots], chosen values [top]
__global__ void __launch_bounds__(32) moe_route_topk_kernel(MoeRouteArgs a) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float rs[];
    float* choice = rs;
    float* picked = rs + a.n_slots;
    const int t = blockIdx.x, lane = threadIdx.x, n = a.n_slots;
    const float* z = a.logits + (size_t)t * a.ld;
    for (int i = lane; i < n; i += 32) choice[i] = z[i] + (a.correction ? a.correction[i] : 0.f);
    __syncwarp();
    for (int k = 0; k < a.top; k++) {
        float v = -INFINITY; int idx = 0x7fffffff;
        for (int i = lane; i < n; i += 32) { const float c = choice[i]; if (c > v || (c == v && i < idx)) { v = c; idx = i; } }
        warp_argmax(v, idx);
        if (idx >= n) { idx = 0; v = -INFINITY; }
        __syncwarp();
        if (lane == 0) {
            a.sel[(size_t)t * a.top + k] = idx;
            a.pair_token[(size_t)t * a.top + k] = t;
            picked[k] = v;
            choice[idx] = NAN;                     // taken: NaN never wins a comparison
        }
        __syncwarp();
    }
    const float mx = picked[0];                    // the first pick is the largest
    float sum = 0.f;
    for (int k = 0; k < a.top; k++) sum += expf(picked[k] - mx);       // every lane the same sum, in pick order
    for (int k = lane; k < a.top; k += 32) a.weight[(size_t)t * a.top + k] = expf(picked[k] - mx) / sum * a.scale;
}
cudaError_t moe_route_launch(const MoeRouteArgs& a, int T, cudaStream_t s) {
    if (a.mode == 1) {
        const size_t smem = (size_t)(a.n_slots + a.top) * 4;
        if (smem > 48 * 1024) return cudaErrorInvalidValue;
        return launch_chain(moe_route_topk_kernel, dim3(T), dim3(32), smem, s, a);
    }
    const size_t smem = (size_t)(2 * a.n_slots + a.n_groups + 1) * 4;
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    return launch_chain(moe_route_kernel, dim3(T), dim3(32), smem, s, a);
}

// One CTA: histogram of the pairs by expert, tile table, placement. Which row of an expert's range a pair
// gets depends on the order of the atomics, but every output row is computed from its own input row alone, so the
// order changes no number.
__global__ void __launch_bounds__(1024) moe_sort_kernel(MoeSortArgs a) {
    griddep_launch();
    griddep_wait();
    extern __shared__ int ms[];
    int* count = ms;                       // [n_experts]
    int* offset = count + a.n_experts;     // [n_experts + 1]
    int* cursor = offset + a.n_experts + 1;
    for (int e = threadIdx.x; e < a.n_experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < a.n_pairs; p += blockDim.x) {
        const int e = a.sel[p];
        if (e >= 0 && e < a.n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < a.n_experts; e++) {
            offset[e] = rows;
            for (int r0 = 0; r0 < count[e] && tiles < a.max_tiles; r0 += a.tile, tiles++) {
                a.tile_group[tiles] = e; a.tile_row0[tiles] = rows + r0; a.tile_rows[tiles] = min(a.tile, count[e] - r0);
            }
            rows += count[e];
        }
        offset[a.n_experts] = rows;
        *a.n_tiles = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < a.n_pairs; p += blockDim.x) {
        const int e = a.sel[p];
        int row = -1;
        if (e >= 0 && e < a.n_experts) {
            row = offset[e] + atomicAdd(&cursor[e], 1);
            a.x_rows[row] = p / a.top;
        }
        a.pos[p] = row;
    }
}
cudaError_t moe_sort_launch(const MoeSortArgs& a, cudaStream_t s) {
    const size_t smem = (size_t)(3 * a.n_experts + 1) * 4;
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    return launch_chain(moe_sort_kernel, dim3(1), dim3(1024), smem, s, a);
}

// grid (T)
__global__ void __launch_bounds__(256) moe_combine_kernel(const int* __restrict__ sel, const float* __restrict__ weight, const int* __restrict__ pos,
                                                          const float* __restrict__ rows, const float* __restrict__ h, int n_experts, int top,
                                                          int W, float* __restrict__ out) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; c++) {
            const int p = t * top + c, e = sel[p];
            const float wv = weight[p];
            const float v = e < n_experts ? rows[(size_t)(pos ? pos[p] : p) * W + i] : h[(size_t)t * W + i];
            acc = fmaf(wv, v, acc);
        }
        out[(size_t)t * W + i] = acc;
    }
}
cudaError_t moe_combine_launch(const int* sel, const float* weight, const int* pos, const float* rows, const float* h, int n_experts,
                               int top, int W, int T, float* out, cudaStream_t s) {
    return launch_chain(moe_combine_kernel, dim3(T), dim3(256), 0, s, sel, weight, pos, rows, h, n_experts, top, W, out);
}

// grid (T): the row lives in shared memory between the sum and the normalisation
__global__ void __launch_bounds__(256) moe_join_kernel(MoeJoinArgs j, float* __restrict__ x, float mult, const float* __restrict__ w,
                                                       float w_offset, float eps, int W, float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float row[];
    __shared__ float red[8];
    const int t = blockIdx.x;
    const size_t base = (size_t)t * W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < j.top; c++) {
            const int p = t * j.top + c, e = j.sel[p];
            const float v = e < j.n_experts ? j.rows[(size_t)(j.pos ? j.pos[p] : p) * W + i] : j.h[base + i];
            acc = fmaf(j.weight[p], v, acc);
        }
        const float v = fmaf(mult, acc, x[base + i]);
        x[base + i] = v;
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!y) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < 8; k++) tot += red[k];
    const float rinv = 1.f / sqrtf(tot / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[base + i] = row[i] * rinv * (w_offset + w[i]);
}
cudaError_t moe_join_launch(const MoeJoinArgs& j, float* x, float mult, const float* w, float w_offset, float eps, int W, int T, float* y,
                            cudaStream_t s) {
    return launch_chain(moe_join_kernel, dim3(T), dim3(256), (size_t)W * 4, s, j, x, mult, w, w_offset, eps, W, y);
}

// grid (T): the branch output (a dense branch and / or a mixture's weighted sum) lives in shared memory between the sums of
// squares of its parts and the scaling
struct OutNormMoe { MoeJoinArgs j; int on; };
__global__ void __launch_bounds__(256) outnorm_join_kernel(float* __restrict__ x, const float* __restrict__ a, OutNormMoe mo,
                                                          const float* __restrict__ w, int groups, float eps, int W, float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    extern __shared__ float row[];             // [W] values, then [groups] 1 / rms
    float* rinv = row + W;
    const int t = blockIdx.x, n = W / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const size_t base = (size_t)t * W;
    const MoeJoinArgs& j = mo.j;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = a ? a[base + i] : 0.f;
        if (mo.on)
            for (int c = 0; c < j.top; c++) {
                const int p = t * j.top + c, e = j.sel[p];
                const float v = e < j.n_experts ? j.rows[(size_t)(j.pos ? j.pos[p] : p) * W + i] : j.h[base + i];
                acc = fmaf(j.weight[p], v, acc);
            }
        row[i] = acc;
    }
    __syncthreads();
    for (int g = warp; g < groups; g += nw) {
        float ss = 0.f;
        for (int i = lane; i < n; i += 32) { const float v = row[g * n + i]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) rinv[g] = 1.f / sqrtf(ss / (float)n + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float v = row[i] * rinv[i / n] * w[i];
        if (x) x[base + i] += v;
        else y[base + i] = v;
    }
}
cudaError_t outnorm_join_launch(float* x, const float* a, const MoeJoinArgs* moe, const float* w, int groups, float eps, int W, int T,
                                float* y, cudaStream_t s) {
    if (groups <= 0 || W % groups) return cudaErrorInvalidValue;
    OutNormMoe mo = {};
    if (moe) { mo.j = *moe; mo.on = 1; }
    return launch_chain(outnorm_join_kernel, dim3(T), dim3(256), (size_t)(W + groups) * 4, s, x, a, mo, w, groups, eps, W, y);
}

}  // namespace b2
