// Recurrent token mixers of the layer-list models that keep a MATRIX per head: the gated delta rule (rows of the memory
// decay each at their own input-dependent rate; the write is the part of the value the memory does not return yet) and
// the Mamba-2 state-space recurrence (one scalar decay per head, input and output maps shared by the heads of a group).
// Both run through one kernel (col_state_kernel). Also here: the short causal convolution in front of them, their
// 32-bit input preparation (unit norms, softplus, exponentials, sigmoid) and the gated group norm behind them.
// State, decays, step sizes and norms are 32-bit; a segment's tokens are walked in order from the state its slot holds,
// so a sequence cut into portions gives the same numbers as the whole.
#include "kernels.h"
#include "layered.h"
#include "ptx.cuh"

#include <stdlib.h>

#include <algorithm>

namespace b2 {

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 0.f ? z + log1pf(expf(-z)) : log1pf(expf(z)); }
__device__ __forceinline__ void cp_async_4(float* smem_dst, const float* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
}  // namespace

// ---------------------------------------------------------------- short causal convolution
// grid (T, ceil(C / 256)): a thread per (token, channel)
__global__ void __launch_bounds__(256) causal_conv_kernel(ConvArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.C) return;
    const int seg = r.tok_seg[t], slot = r.seg_slot[seg], i = t - r.seg_start[seg];
    const int hist = a.taps - 1;
    float acc = a.bias && !a.skip ? a.bias[c] : 0.f;
    for (int j = 0; j < a.taps; j++) {
        const int srci = i - hist + j;
        const float v = srci >= 0 ? a.in[(size_t)(t - i + srci) * a.ld_in + c]
                                  : a.state[((size_t)slot * hist + (hist + srci)) * a.C + c];
        acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
    }
    a.out[(size_t)t * a.ld_out + c] = a.skip ? a.in[(size_t)t * a.ld_in + c] + acc : silu_f(acc);
}
cudaError_t causal_conv_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s) {
    return launch_chain(causal_conv_kernel, dim3(r.T, (a.C + 255) / 256), dim3(256), 0, s, a, r);
}
// grid (n_seg, ceil(C / 256)); entry k of the new state is read at k + len > k of the old one before it is written
__global__ void __launch_bounds__(256) causal_conv_advance_kernel(ConvArgs a, RaggedDev r) {
    griddep_launch();
    griddep_wait();
    const int seg = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= a.C) return;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int hist = a.taps - 1;
    float* st = a.state + (size_t)slot * hist * a.C + c;
    for (int k = 0; k < hist; k++) {
        const int srci = len + k - hist;
        st[(size_t)k * a.C] = srci >= 0 ? a.in[(size_t)(start + srci) * a.ld_in + c] : st[(size_t)(k + len) * a.C];
    }
}
cudaError_t causal_conv_advance_launch(const ConvArgs& a, const RaggedDev& r, cudaStream_t s) {
    if (a.taps <= 1) return cudaSuccess;
    return launch_chain(causal_conv_advance_kernel, dim3(r.n_seg, (a.C + 255) / 256), dim3(256), 0, s, a, r);
}

// ---------------------------------------------------------------- inputs of the recurrences
// grid (T): unit vectors, decays, write strengths
__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepArgs a) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float qmul = 1.f / sqrtf((float)a.d);
    for (int hv = warp; hv < 2 * a.G; hv += nw) {          // a warp per (q | k, head)
        const bool is_q = hv < a.G;
        float* v = (is_q ? a.q : a.k) + (size_t)t * a.ld_qk + (size_t)(is_q ? hv : hv - a.G) * a.d;
        float ss = 0.f;
        for (int i = lane; i < a.d; i += 32) ss = fmaf(v[i], v[i], ss);
        const float rinv = (is_q ? qmul : 1.f) / sqrtf(warp_sum(ss) + a.unit_eps);
        for (int i = lane; i < a.d; i += 32) v[i] *= rinv;
    }
    const int ac = a.a_cols > 0 ? a.a_cols : a.d;
    for (int i = threadIdx.x; i < a.H * ac; i += blockDim.x) {
        float* p = a.a + (size_t)t * a.ld_a + i;
        *p = expf(-expf(a.A_log[i / ac]) * softplus_f(*p + a.dt_bias[i]));
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        float* p = a.beta + (size_t)t * a.ld_b + h;
        *p = sigmoid_f(*p);
    }
}
cudaError_t delta_prepare_launch(const DeltaPrepArgs& a, int T, cudaStream_t s) {
    return launch_chain(delta_prepare_kernel, dim3(T), dim3(256), 0, s, a);
}

__global__ void ssd_prepare_kernel(float* dt, int ld_dt, const float* dt_bias, const float* A_log, int H, float* decay, int T) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * H) return;
    const int t = i / H, h = i % H;
    const float v = softplus_f(dt[(size_t)t * ld_dt + h] + dt_bias[h]);
    dt[(size_t)t * ld_dt + h] = v;
    decay[i] = expf(-expf(A_log[h]) * v);
}
cudaError_t ssd_prepare_launch(float* dt, int ld_dt, const float* dt_bias, const float* A_log, int H, float* decay, int T, cudaStream_t s) {
    return launch_chain(ssd_prepare_kernel, dim3((T * H + 127) / 128), dim3(128), 0, s, dt, ld_dt, dt_bias, A_log, H, decay, T);
}

// ---------------------------------------------------------------- the recurrence
// grid (n_seg, H, ceil(P / CS_COLS)), 4 warps: a warp is 4 column groups x 8 row lanes; a lane keeps NCH chunks of four rows
// (chunk index = row lane + 8 i, so the 8 row lanes of a group read 32 neighbouring floats) of CS_CPL neighbouring columns
// in registers. The row vectors of a token (write key, read key, row decays) are loaded from shared memory once per lane
// and serve its CS_CPL columns, whose dependency chains interleave; the two sums over the rows -- what the memory
// returns for the write key, and the read-out -- are shuffle reductions over the 8 row lanes. The row vectors are the
// same for every column of the head: they come into shared memory as asynchronous copies, CS_TB tokens at a time, the
// next block while this one is computed.
// Columns per lane (CS_CPL = 1, 2 or 4) are chosen so that the grid fills the GPU: few heads -> narrow CTAs on many SMs.
// The kernel is bound by the latency of one token's chain and runs one CTA per SM at most. It is launched WITHOUT the
// dependent-launch attribute: as a dependent its CTAs become resident while the previous kernel still fills most SMs, so
// several land on the same few SMs and share their schedulers for the whole prompt (measured: 3.0 -> 0.9 ms).
constexpr int CS_LANES = 8, CS_WARPS = 4, CS_TB = 8;
template <int NCH, int CS_CPL, bool DELTA, bool ROWDEC>
__global__ void __launch_bounds__(CS_WARPS * 32) col_state_kernel(ColStateArgs a, RaggedDev r) {
    constexpr int CS_COLS = CS_WARPS * 4 * CS_CPL;
    griddep_wait();
    extern __shared__ __align__(16) float cs_sm[];
    const int R = a.R, P = a.P, Rp = (R + 3) / 4 * 4, n_chunks = Rp / 4;
    float* wks = cs_sm;                              // [2][CS_TB][Rp]
    float* rks = wks + 2 * CS_TB * Rp;               // [2][CS_TB][Rp]
    float* rds = rks + 2 * CS_TB * Rp;               // [2][CS_TB][Rp] (only with row decays)
    float* vs = rds + (ROWDEC ? 2 * CS_TB * Rp : 0); // [2][CS_TB][CS_COLS]
    float* sc = vs + 2 * CS_TB * CS_COLS;            // [2][CS_TB][2]: value scale, head decay
    const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CS_COLS;
    const int slot = r.seg_slot[seg], start = r.seg_start[seg], len = r.seg_len[seg];
    const int rl = threadIdx.x % CS_LANES, lc = (threadIdx.x / CS_LANES) * CS_CPL, col = c0 + lc;     // first of the lane's columns
    const int g = h / (a.H / a.G);
    float* Sg = a.state + (((size_t)slot * a.H + h) * P) * Rp;
    float4 S[CS_CPL][NCH];
#pragma unroll
    for (int j = 0; j < CS_CPL; j++)
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            const int ch = rl + CS_LANES * i;
            S[j][i] = (col + j < P && ch < n_chunks) ? *reinterpret_cast<const float4*>(Sg + (size_t)(col + j) * Rp + 4 * ch) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    for (int j = threadIdx.x; j < (ROWDEC ? 6 : 4) * CS_TB * Rp + 2 * CS_TB * (CS_COLS + 2); j += blockDim.x) cs_sm[j] = 0.f;
    __syncthreads();
    auto stage = [&](int i0, int buf) {
        const int nb = min(CS_TB, len - i0);
        for (int u = 0; u < nb; u++) {
            const size_t t = start + i0 + u;
            const int d = (buf * CS_TB + u) * Rp;
            for (int e = threadIdx.x; e < R; e += blockDim.x) {
                cp_async_4(wks + d + e, a.wk + t * a.ld_wk + (size_t)g * R + e);
                cp_async_4(rks + d + e, a.rk + t * a.ld_rk + (size_t)g * R + e);
                if (ROWDEC) cp_async_4(rds + d + e, a.row_decay + t * a.ld_rd + (size_t)h * R + e);
            }
        }
        for (int j = threadIdx.x; j < nb * CS_COLS; j += blockDim.x) {
            const int u = j / CS_COLS, e = j % CS_COLS;
            const size_t t = start + i0 + u;
            if (c0 + e < P) cp_async_4(vs + (buf * CS_TB + u) * CS_COLS + e, a.val + t * a.ld_v + (size_t)h * P + c0 + e);
            if (e == 0 && a.val_scale) cp_async_4(sc + (buf * CS_TB + u) * 2, a.val_scale + t * a.ld_vs + h);
            if (e == 1 && a.head_decay) cp_async_4(sc + (buf * CS_TB + u) * 2 + 1, a.head_decay + t * a.ld_hd + h);
        }
    };
    const float skip = a.skip ? a.skip[h] : 0.f;
    const float hconst = a.head_const ? a.head_const[h] : 1.f;
    if (len > 0) stage(0, 0);
    cp_async_commit();
    for (int i0 = 0; i0 < len; i0 += CS_TB) {
        const int nb = min(CS_TB, len - i0), buf = (i0 / CS_TB) & 1;
        cp_async_wait_all();
        __syncthreads();                 // this block's inputs have landed; everybody is done with the other buffer
        if (i0 + CS_TB < len) stage(i0 + CS_TB, buf ^ 1);
        cp_async_commit();
        for (int u = 0; u < nb; u++) {
            const int bu = buf * CS_TB + u;
            const float4* wk4 = reinterpret_cast<const float4*>(wks + bu * Rp);
            const float4* rk4 = reinterpret_cast<const float4*>(rks + bu * Rp);
            const float4* rd4 = reinterpret_cast<const float4*>(rds + bu * Rp);
            float v[CS_CPL];
#pragma unroll
            for (int j = 0; j < CS_CPL; j++) v[j] = vs[bu * CS_COLS + lc + j];
            const float vscale = a.val_scale ? sc[bu * 2] : 1.f;
            const float hd = a.head_decay ? sc[bu * 2 + 1] : hconst;
            float4 kw[NCH];
            float pred[CS_CPL];
#pragma unroll
            for (int j = 0; j < CS_CPL; j++) pred[j] = 0.f;
#pragma unroll
            for (int i = 0; i < NCH; i++) {
                const int ch = min(rl + CS_LANES * i, n_chunks - 1);      // past the end: a valid address; the state there stays zero
                kw[i] = rl + CS_LANES * i < n_chunks ? wk4[ch] : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 dc = make_float4(hd, hd, hd, hd);
                if (ROWDEC) { const float4 q = rd4[ch]; dc = make_float4(q.x * hd, q.y * hd, q.z * hd, q.w * hd); }
#pragma unroll
                for (int j = 0; j < CS_CPL; j++) {
                    float4& s4 = S[j][i];
                    s4.x *= dc.x; s4.y *= dc.y; s4.z *= dc.z; s4.w *= dc.w;
                    if (DELTA) pred[j] += fmaf(s4.x, kw[i].x, s4.y * kw[i].y) + fmaf(s4.z, kw[i].z, s4.w * kw[i].w);
                }
            }
            float uval[CS_CPL];
            if (DELTA) {
#pragma unroll
                for (int o = CS_LANES / 2; o > 0; o >>= 1)
#pragma unroll
                    for (int j = 0; j < CS_CPL; j++) pred[j] += __shfl_xor_sync(0xffffffffu, pred[j], o);
            }
#pragma unroll
            for (int j = 0; j < CS_CPL; j++) uval[j] = vscale * (v[j] - pred[j]);
            float out[CS_CPL];
#pragma unroll
            for (int j = 0; j < CS_CPL; j++) out[j] = 0.f;
#pragma unroll
            for (int i = 0; i < NCH; i++) {
                const int ch = min(rl + CS_LANES * i, n_chunks - 1);
                const float4 q = rl + CS_LANES * i < n_chunks ? rk4[ch] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < CS_CPL; j++) {
                    float4& s4 = S[j][i];
                    s4.x = fmaf(kw[i].x, uval[j], s4.x); s4.y = fmaf(kw[i].y, uval[j], s4.y);
                    s4.z = fmaf(kw[i].z, uval[j], s4.z); s4.w = fmaf(kw[i].w, uval[j], s4.w);
                    out[j] += fmaf(s4.x, q.x, s4.y * q.y) + fmaf(s4.z, q.z, s4.w * q.w);
                }
            }
#pragma unroll
            for (int o = CS_LANES / 2; o > 0; o >>= 1)
#pragma unroll
                for (int j = 0; j < CS_CPL; j++) out[j] += __shfl_xor_sync(0xffffffffu, out[j], o);
            if (rl == 0) {
                float* yp = a.y + (size_t)(start + i0 + u) * a.ld_y + (size_t)h * P + col;
#pragma unroll
                for (int j = 0; j < CS_CPL; j++) if (col + j < P) yp[j] = fmaf(skip, v[j], out[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CS_CPL; j++)
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            const int ch = rl + CS_LANES * i;
            if (col + j < P && ch < n_chunks) *reinterpret_cast<float4*>(Sg + (size_t)(col + j) * Rp + 4 * ch) = S[j][i];
        }
    griddep_launch();
}

template <int NCH, int CPL>
static cudaError_t col_state_pick(const ColStateArgs& a, const RaggedDev& r, cudaStream_t s) {
    constexpr int COLS = CS_WARPS * 4 * CPL;
    const int Rp = (a.R + 3) / 4 * 4;
    const size_t smem = (size_t)((a.row_decay ? 6 : 4) * CS_TB * Rp + 2 * CS_TB * (COLS + 2)) * 4;
    const dim3 grid(r.n_seg, a.H, (a.P + COLS - 1) / COLS), block(CS_WARPS * 32);
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(col_state_kernel<NCH, CPL, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        cudaFuncSetAttribute(col_state_kernel<NCH, CPL, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    }
    if (a.delta && a.row_decay) return launch_chain(col_state_kernel<NCH, CPL, true, true>, grid, block, smem, s, a, r);
    if (a.delta) return launch_chain(col_state_kernel<NCH, CPL, true, false>, grid, block, smem, s, a, r);
    if (a.row_decay) return launch_chain(col_state_kernel<NCH, CPL, false, true>, grid, block, smem, s, a, r);
    return launch_chain(col_state_kernel<NCH, CPL, false, false>, grid, block, smem, s, a, r);
}
template <int NCH>
static cudaError_t col_state_width(const ColStateArgs& a, const RaggedDev& r, cudaStream_t s) {
    const int per16 = r.n_seg * a.H * ((a.P + 15) / 16);       // CTAs with one column per lane
    if (per16 <= 160) return col_state_pick<NCH, 1>(a, r, s);
    if (per16 <= 320) return col_state_pick<NCH, 2>(a, r, s);
    return col_state_pick<NCH, 4>(a, r, s);
}

cudaError_t col_state_launch(const ColStateArgs& a, const RaggedDev& r, cudaStream_t s) {
    PlainLaunch pl;
    if (a.R <= 0 || a.R > 256 || a.P <= 0 || a.H <= 0 || a.G <= 0 || a.H % a.G) return cudaErrorInvalidValue;
    const int n_chunks = (a.R + 3) / 4;
    if (n_chunks <= 8) return col_state_width<1>(a, r, s);
    if (n_chunks <= 16) return col_state_width<2>(a, r, s);
    if (n_chunks <= 32) return col_state_width<4>(a, r, s);
    return col_state_width<8>(a, r, s);
}

// ---------------------------------------------------------------- gated group norm
// grid (T, groups)
__global__ void __launch_bounds__(128) group_norm_gate_kernel(GroupNormArgs a) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[4];
    const int t = blockIdx.x, g = blockIdx.y, n = a.n;
    const float* x = a.x + (size_t)t * a.ld_x + (size_t)g * n;
    const float* gate = a.gate + (size_t)t * a.ld_g + (size_t)g * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = a.gate_first ? x[i] * silu_f(gate[i]) : x[i];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float rinv = 1.f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)n + a.eps);
    const float* w = a.w + (size_t)g * a.w_gstride;
    float* y = a.y + (size_t)t * a.ld_y + (size_t)g * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        y[i] = (a.gate_first ? x[i] * silu_f(gate[i]) * rinv * w[i] : x[i] * rinv * w[i] * (a.gate_silu ? silu_f(gate[i]) : sigmoid_f(gate[i]))) * a.out_scale;
}
cudaError_t group_norm_gate_launch(const GroupNormArgs& a, int T, cudaStream_t s) {
    return launch_chain(group_norm_gate_kernel, dim3(T, a.groups), dim3(128), 0, s, a);
}

}  // namespace b2
