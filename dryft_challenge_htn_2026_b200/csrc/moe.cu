// Mixture of experts: the router and the routed experts' feed-forward.
//
// Router (float32 throughout): z = W_r x, s = sigmoid(z); the choice is made on s + correction, among the
// experts of the `keep` best of `groups` equal groups of neighbouring experts (a group's score is the sum of
// its two largest choice scores; the others' choice scores count as minus infinity), the `top` largest;
// the weights are the chosen experts' s (without the correction) over their sum, times a constant. The same
// kernel works out the gate of a shared expert, sigmoid(w_sg . x), one number a token.
//
// Experts, row form (this file): every (token, chosen expert) pair is a row of its own,
//   mid[pair] = act(W_gate[e] x) * (W_up[e] x),   out[token] = sum_j weight_j W_down[e_j] mid[pair_j]
//                                                              + gate * shared[token],
// a warp per output column, float32 sums. It serves single-token steps, where a pair reads its expert's
// matrices once, and every float32 step; prompts in bfloat16 go through the tiled form (moe_tiles.cu).
#include "common.cuh"

#define MOE_MAX_EXPERTS 256
#define ROUTE_WARPS 4

// (value, index) with the larger value, the lower index among equal values, over the warp
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
moe_route_kernel(const T* x, int W, const float* __restrict__ wr, const float* __restrict__ corr,
                 const float* __restrict__ wsg, int E, int top, int groups, int keep, float scale, int* idx, float* wt,
                 float* sgate, int n_tok) {
    __shared__ float s_all[ROUTE_WARPS][MOE_MAX_EXPERTS];
    __shared__ float c_all[ROUTE_WARPS][MOE_MAX_EXPERTS];
    __shared__ float g_all[ROUTE_WARPS][MOE_MAX_EXPERTS];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + w;
    if (t >= n_tok) return;
    float* s = s_all[w];
    float* c = c_all[w];
    float* gs = g_all[w];
    const T* xr = x + (size_t)t * W;
    for (int e = 0; e < E; e++) {
        float acc = 0.f;
        for (int k = lane; k < W; k += 32) acc = fmaf(wr[(size_t)e * W + k], to_f(xr[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            s[e] = 1.f / (1.f + expf(-acc));
            c[e] = s[e] + (corr ? corr[e] : 0.f);
        }
    }
    if (wsg != nullptr) {
        float acc = 0.f;
        for (int k = lane; k < W; k += 32) acc = fmaf(wsg[k], to_f(xr[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) sgate[t] = 1.f / (1.f + expf(-acc));
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {       // a group's score: its two largest choice scores
            float a = -INFINITY, b = -INFINITY;
            for (int i = 0; i < per; i++) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // the keep best groups are marked by +inf; all others' experts then leave the choice
        for (int it = 0; it < keep; it++) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] != INFINITY && (gs[g] > bv || bi == 0x7fffffff)) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < groups) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int j = 0; j < top; j++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (c[e] > bv) { bv = c[e]; bi = e; }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;                             // nothing left to choose from (more picks than allowed experts)
        wsum += s[bi];
        if (lane == 0) {
            idx[(size_t)t * top + j] = bi;
            c[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane < top) {
        const int e = idx[(size_t)t * top + lane];
        wt[(size_t)t * top + lane] = s[e] / (wsum + 1e-20f) * scale;
    }
}

__device__ __forceinline__ float moe_act(float z, int act) {
    if (act == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

// Block (pair, slice of ff): mid[pair][f] = act(W_gu[e][f] . x) * (W_gu[e][ff + f] . x), W_gu [E, 2 ff, W].
template <typename T>
__global__ void __launch_bounds__(128)
moe_up_rows_kernel(const T* x, int W, const T* __restrict__ wgu, const int* idx, T* mid, int ff, int top, int rows_per_block,
                   int act) {
    extern __shared__ float xs[];
    pdl_wait();
    pdl_launch_dependents();
    const int pair = blockIdx.x, t = pair / top;
    const int e = idx[pair];
    for (int k = threadIdx.x; k < W; k += blockDim.x) xs[k] = to_f(x[(size_t)t * W + k]);
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int f_end = min(ff, (int)(blockIdx.y + 1) * rows_per_block);
    const T* base = wgu + (size_t)e * 2 * ff * W;
    for (int f = blockIdx.y * rows_per_block + w; f < f_end; f += 4) {
        const T* g = base + (size_t)f * W;
        const T* u = base + (size_t)(ff + f) * W;
        float ag = 0.f, au = 0.f;
        for (int k = lane; k < W; k += 32) {
            ag = fmaf(to_f(g[k]), xs[k], ag);
            au = fmaf(to_f(u[k]), xs[k], au);
        }
        ag = warp_sum(ag);
        au = warp_sum(au);
        if (lane == 0) mid[(size_t)pair * ff + f] = from_f<T>(moe_act(ag, act) * au);
    }
}

// Block (token, slice of the width): out[t][c] = sum_j wt[t][j] (W_d[e_j][c] . mid[t*top + j]) + sgate[t] * shared[t][c].
template <typename T>
__global__ void __launch_bounds__(128)
moe_down_rows_kernel(const T* mid, const T* __restrict__ wd, const int* idx, const float* wt, const T* shared,
                     const float* sgate, T* out, int W, int ff, int top, int rows_per_block) {
    extern __shared__ float ms[];        // [top][ff], already times the pair's weight
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x)
        ms[i] = to_f(mid[(size_t)t * top * ff + i]) * wt[(size_t)t * top + i / ff];
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c_end = min(W, (int)(blockIdx.y + 1) * rows_per_block);
    for (int c = blockIdx.y * rows_per_block + w; c < c_end; c += 4) {
        float acc = 0.f;
        for (int j = 0; j < top; j++) {
            const T* row = wd + ((size_t)idx[(size_t)t * top + j] * W + c) * ff;
            float a = 0.f;
            for (int k = lane; k < ff; k += 32) a = fmaf(to_f(row[k]), ms[j * ff + k], a);
            acc += a;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (shared != nullptr) acc = fmaf(sgate ? sgate[t] : 1.f, to_f(shared[(size_t)t * W + c]), acc);
            out[(size_t)t * W + c] = from_f<T>(acc);
        }
    }
}

DK_EXPORT int dk_moe_route(int dtype, const void* x, int W, const float* wr, const float* corr, const float* wsg, int E,
                           int top, int groups, int keep, float scale, int* idx, float* wt, float* sgate, int n_tok,
                           cudaStream_t st) {
    if (E < 1 || E > MOE_MAX_EXPERTS || top < 1 || top > 32 || top > E || groups < 1 || E % groups || keep < 1 || keep > groups)
        return (int)cudaErrorInvalidValue;
    const dim3 grid((n_tok + ROUTE_WARPS - 1) / ROUTE_WARPS), block(32 * ROUTE_WARPS);
    if (dtype == 0)
        return dk_launch(moe_route_kernel<float>, grid, block, 0, st, (const float*)x, W, wr, corr, wsg, E, top, groups,
                         keep, scale, idx, wt, sgate, n_tok);
    return dk_launch(moe_route_kernel<bf16>, grid, block, 0, st, (const bf16*)x, W, wr, corr, wsg, E, top, groups, keep,
                     scale, idx, wt, sgate, n_tok);
}

DK_EXPORT int dk_moe_up_rows(int dtype, const void* x, int W, const void* wgu, const int* idx, void* mid, int ff, int top,
                             int n_tok, int act, cudaStream_t st) {
    const int rpb = 32;
    const dim3 grid(n_tok * top, (ff + rpb - 1) / rpb), block(128);
    const size_t smem = sizeof(float) * (size_t)W;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return dk_launch(moe_up_rows_kernel<float>, grid, block, smem, st, (const float*)x, W, (const float*)wgu, idx,
                         (float*)mid, ff, top, rpb, act);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_rows_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(moe_up_rows_kernel<bf16>, grid, block, smem, st, (const bf16*)x, W, (const bf16*)wgu, idx, (bf16*)mid,
                     ff, top, rpb, act);
}

DK_EXPORT int dk_moe_down_rows(int dtype, const void* mid, const void* wd, const int* idx, const float* wt,
                               const void* shared, const float* sgate, void* out, int W, int ff, int top, int n_tok,
                               cudaStream_t st) {
    const int rpb = 32;
    const dim3 grid(n_tok, (W + rpb - 1) / rpb), block(128);
    const size_t smem = sizeof(float) * (size_t)top * ff;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return dk_launch(moe_down_rows_kernel<float>, grid, block, smem, st, (const float*)mid, (const float*)wd, idx, wt,
                         (const float*)shared, sgate, (float*)out, W, ff, top, rpb);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_rows_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return dk_launch(moe_down_rows_kernel<bf16>, grid, block, smem, st, (const bf16*)mid, (const bf16*)wd, idx, wt,
                     (const bf16*)shared, sgate, (bf16*)out, W, ff, top, rpb);
}
