// Linear attention with a constant decay per head ("lightning attention"):
//   S_t = d_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   q, k, v = act(projection rows)
// with the state S [hd, hdv] of every (sequence, head) kept in float32 between steps, and the
// norm-and-gate step that follows it: all heads of a token together through a weighted RMS norm, times
// sigmoid(gate), times a constant. State, decay powers, scores and sums are float32; the projections
// come in the model's storage type and their activation is worked out in float32.
//
// This file: the recurrence token by token, one block per (sequence, head), the state in registers; it
// serves single-token steps, short portions and every float32 step. Portions of many tokens in bfloat16
// run in blocks of 64 tokens on the tensor cores (linear_attention_bf16.cu).
#include "common.cuh"

#define LA_THREADS 256
#define LA_TB 8   // tokens staged at a time by the step kernel

__device__ __forceinline__ float act_silu(float x) { return x / (1.f + expf(-x)); }

// Block (sequence s, head h, slice of up to cslice value columns: the columns of a state evolve independently,
// and a slice of 32 keeps a thread's share of the state at hd / 8 registers, so that several blocks fit an
// SM). Thread (rg, c): column c of the slice, rows rg, rg + R, ... (R row groups).
// cu_q == nullptr: one token per sequence (row s is sequence s). seq_pos0[s] < 0: a padding row.
template <typename T, int EPT>
__global__ void __launch_bounds__(LA_THREADS)
linear_attention_step_kernel(const T* q, const T* k, const T* v, long long ld, float* out, float* state,
                             const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* __restrict__ decay,
                             int nh, int hd, int hdv, int cols_pad, int cslice) {
    extern __shared__ float sm[];
    const int R = LA_THREADS / cols_pad;
    float* sq = sm;                              // [LA_TB][hd]
    float* sk = sq + LA_TB * hd;                 // [LA_TB][hd]
    float* sv = sk + LA_TB * hd;                 // [LA_TB][cslice]
    float* part = sv + LA_TB * cslice;           // [LA_TB][R][cols_pad]
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cslice;
    const int cols = min(cslice, hdv - col0);            // value columns of this block: [col0, col0 + cols)
    const int r0 = cu_q ? cu_q[s] : s, r1 = cu_q ? cu_q[s + 1] : s + 1;
    const int tid = threadIdx.x, c = tid % cols_pad, rg = tid / cols_pad;
    const size_t ow = (size_t)nh * hdv;
    if (seq_pos0[s] < 0) {
        for (int t = r0; t < r1; t++)
            for (int i = tid; i < cols; i += LA_THREADS) out[(size_t)t * ow + (size_t)h * hdv + col0 + i] = 0.f;
        return;
    }
    const float d = decay[h];
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)hd * hdv + col0;
    float st[EPT];
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int row = rg + R * i;
        st[i] = (row < hd && c < cols) ? S[(size_t)row * hdv + c] : 0.f;
    }
    for (int t0 = r0; t0 < r1; t0 += LA_TB) {
        const int nt = min(LA_TB, r1 - t0);
        __syncthreads();
        for (int i = tid; i < nt * hd; i += LA_THREADS) {
            const size_t at = (size_t)(t0 + i / hd) * ld + (size_t)h * hd + i % hd;
            sq[i] = act_silu(to_f(q[at]));
            sk[i] = act_silu(to_f(k[at]));
        }
        for (int i = tid; i < nt * cols; i += LA_THREADS)
            sv[i] = act_silu(to_f(v[(size_t)(t0 + i / cols) * ld + (size_t)h * hdv + col0 + i % cols]));
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float vc = c < cols ? sv[tt * cols + c] : 0.f;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                const int row = rg + R * i;
                if (row < hd) {
                    st[i] = fmaf(d, st[i], sk[tt * hd + row] * vc);
                    o = fmaf(st[i], sq[tt * hd + row], o);
                }
            }
            part[(tt * R + rg) * cols_pad + c] = o;
        }
        __syncthreads();
        for (int i = tid; i < nt * cols; i += LA_THREADS) {
            const int tt = i / cols, cc = i % cols;
            float o = 0.f;
            for (int g = 0; g < R; g++) o += part[(tt * R + g) * cols_pad + cc];
            out[(size_t)(t0 + tt) * ow + (size_t)h * hdv + col0 + cc] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int row = rg + R * i;
        if (row < hd && c < cols) S[(size_t)row * hdv + c] = st[i];
    }
}

// out[t] = rmsnorm(o[t]) * w * sigmoid(gate[t]) * out_scale over the whole row of all heads (width n).
template <typename T>
__global__ void norm_gate_kernel(const float* o, const float* __restrict__ w, float eps, const T* gate, long long ldg,
                                 float out_scale, T* out, long long ldo, int n) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    const float* orow = o + t * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += orow[i] * orow[i];
    ss = block_sum(ss, red);
    const float rs = out_scale / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = orow[i] * rs * w[i];
        if (gate) v *= 1.f / (1.f + expf(-to_f(gate[t * ldg + i])));
        out[t * ldo + i] = from_f<T>(v);
    }
}

template <typename T>
static int launch_step(const void* q, const void* k, const void* v, long long ld, float* out, float* state,
                       const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* decay, int n_seq, int nh,
                       int hd, int hdv, cudaStream_t st) {
    const int cslice = hdv < 32 ? hdv : 32;
    int cols_pad = 1;
    while (cols_pad < cslice) cols_pad <<= 1;
    const int R = LA_THREADS / cols_pad;
    const int ept = (hd + R - 1) / R;
    const size_t smem = sizeof(float) * (size_t)(LA_TB * (2 * hd + cslice) + LA_TB * LA_THREADS);
    const dim3 grid(n_seq, nh, (hdv + cslice - 1) / cslice), block(LA_THREADS);
#define LA_STEP(E)                                                                                                       \
    if (ept <= E) {                                                                                                      \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(linear_attention_step_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return dk_launch(linear_attention_step_kernel<T, E>, grid, block, smem, st, (const T*)q, (const T*)k, (const T*)v, \
                         ld, out, state, cu_q, seq_pos0, seq_slot, decay, nh, hd, hdv, cols_pad, cslice);                 \
    }
    LA_STEP(4) LA_STEP(8) LA_STEP(16) LA_STEP(32) LA_STEP(64) LA_STEP(128) LA_STEP(256)
#undef LA_STEP
    return (int)cudaErrorInvalidValue;
}

DK_EXPORT int dk_linear_attention_step(int dtype, const void* q, const void* k, const void* v, long long ld, float* out,
                                       float* state, const int* cu_q, const int* seq_pos0, const int* seq_slot,
                                       const float* decay, int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    if (hd > 256 || hdv > 256 || hd < 1 || hdv < 1) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return launch_step<float>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
    return launch_step<bf16>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
}

DK_EXPORT int dk_norm_gate(int dtype, const float* o, const float* w, float eps, const void* gate, long long ldg,
                           float out_scale, void* out, long long ldo, int n_tok, int n, cudaStream_t st) {
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    if (dtype == 0)
        return dk_launch(norm_gate_kernel<float>, dim3(n_tok), dim3(threads), 0, st, o, w, eps, (const float*)gate, ldg,
                         out_scale, (float*)out, ldo, n);
    return dk_launch(norm_gate_kernel<bf16>, dim3(n_tok), dim3(threads), 0, st, o, w, eps, (const bf16*)gate, ldg,
                     out_scale, (bf16*)out, ldo, n);
}
