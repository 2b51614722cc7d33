// Linear attention with a constant decay per head ("lightning attention"):
//   S_t = d_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   q, k, v = act(projection rows)
// with the state S [hd, hdv] of every (sequence, head) kept in float32 between steps, and the
// norm-and-gate step that follows it: all heads of a token together through a weighted RMS norm, times
// sigmoid(gate), times a constant. State, decay powers, scores and sums are float32; the projections
// come in the model's storage type and their activation is worked out in float32.
//
// The same kernel also runs gated linear attention: a decay per key channel and token instead of one per
// head, alpha_t = sigmoid(z_t + b)^(1/tau) from rows z of a low-rank projection, acting on the rows of
// the state, S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, with q times a constant and no activation. The
// decay is worked out in float32 as exp(log sigmoid(z) / tau).
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
// GATED: ``zrows`` [tokens, nh * hd] float32 and ``zbias`` [nh * hd] give the decay of every state row and token,
// exp(log sigmoid(z + b) * inv_tau); q is multiplied by q_scale and nothing goes through SiLU.
template <typename T, int EPT, bool GATED>
__global__ void __launch_bounds__(LA_THREADS)
linear_attention_step_kernel(const T* q, const T* k, const T* v, long long ld, float* out, float* state,
                             const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* __restrict__ decay,
                             int nh, int hd, int hdv, int cols_pad, int cslice, const float* zrows,
                             const float* __restrict__ zbias, float inv_tau, float q_scale) {
    extern __shared__ float sm[];
    const int R = LA_THREADS / cols_pad;
    float* sq = sm;                              // [LA_TB][hd]
    float* sk = sq + LA_TB * hd;                 // [LA_TB][hd]
    float* sv = sk + LA_TB * hd;                 // [LA_TB][cslice]
    float* part = sv + LA_TB * cslice;           // [LA_TB][R][cols_pad]
    float* sd = part + LA_TB * LA_THREADS;       // [LA_TB][hd], GATED only
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
    const float d = GATED ? 0.f : decay[h];
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
            if (GATED) {
                sq[i] = to_f(q[at]) * q_scale;
                sk[i] = to_f(k[at]);
                const float z = zrows[(size_t)(t0 + i / hd) * nh * hd + (size_t)h * hd + i % hd] + zbias[h * hd + i % hd];
                sd[i] = expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);   // sigmoid(z)^(1/tau)
            } else {
                sq[i] = act_silu(to_f(q[at]));
                sk[i] = act_silu(to_f(k[at]));
            }
        }
        for (int i = tid; i < nt * cols; i += LA_THREADS) {
            const float x = to_f(v[(size_t)(t0 + i / cols) * ld + (size_t)h * hdv + col0 + i % cols]);
            sv[i] = GATED ? x : act_silu(x);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float vc = c < cols ? sv[tt * cols + c] : 0.f;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                const int row = rg + R * i;
                if (row < hd) {
                    st[i] = fmaf(GATED ? sd[tt * hd + row] : d, st[i], sk[tt * hd + row] * vc);
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

// out[t] = rmsnorm(o[t]) * w * sigmoid(gate[t]) * out_scale, the norm over each group of ``group`` columns of
// the row (the whole row of all heads, width n, or one head at a time with a weight of the head's size,
// shared by the heads); gate_act 1: SiLU of the gate instead of its sigmoid. Block (token, group).
template <typename T>
__global__ void norm_gate_kernel(const float* o, const float* __restrict__ w, float eps, const T* gate, long long ldg,
                                 float out_scale, T* out, long long ldo, int n, int group, int gate_act) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * group;
    const float* orow = o + t * n + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) ss += orow[i] * orow[i];
    ss = block_sum(ss, red);
    const float rs = out_scale / sqrtf(ss / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = orow[i] * rs * w[i];
        if (gate) {
            const float g = to_f(gate[t * ldg + c0 + i]);
            v *= (gate_act == 1 ? g : 1.f) / (1.f + expf(-g));
        }
        out[t * ldo + c0 + i] = from_f<T>(v);
    }
}

template <typename T, bool GATED>
static int launch_step(const void* q, const void* k, const void* v, long long ld, float* out, float* state,
                       const int* cu_q, const int* seq_pos0, const int* seq_slot, const float* decay, int n_seq, int nh,
                       int hd, int hdv, cudaStream_t st, const float* zrows = nullptr, const float* zbias = nullptr,
                       float inv_tau = 0.f, float q_scale = 1.f) {
    const int cslice = hdv < 32 ? hdv : 32;
    int cols_pad = 1;
    while (cols_pad < cslice) cols_pad <<= 1;
    const int R = LA_THREADS / cols_pad;
    const int ept = (hd + R - 1) / R;
    const size_t smem = sizeof(float) * (size_t)(LA_TB * ((GATED ? 3 : 2) * hd + cslice) + LA_TB * LA_THREADS);
    const dim3 grid(n_seq, nh, (hdv + cslice - 1) / cslice), block(LA_THREADS);
#define LA_STEP(E)                                                                                                       \
    if (ept <= E) {                                                                                                      \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(linear_attention_step_kernel<T, E, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return dk_launch(linear_attention_step_kernel<T, E, GATED>, grid, block, smem, st, (const T*)q, (const T*)k, (const T*)v, \
                         ld, out, state, cu_q, seq_pos0, seq_slot, decay, nh, hd, hdv, cols_pad, cslice, zrows, zbias,    \
                         inv_tau, q_scale);                                                                              \
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
        return launch_step<float, false>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
    return launch_step<bf16, false>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, decay, n_seq, nh, hd, hdv, st);
}

DK_EXPORT int dk_gated_linear_attention_step(int dtype, const void* q, const void* k, const void* v, long long ld,
                                             float* out, float* state, const int* cu_q, const int* seq_pos0,
                                             const int* seq_slot, const float* zrows, const float* zbias, float inv_tau,
                                             float q_scale, int n_seq, int nh, int hd, int hdv, cudaStream_t st) {
    if (hd > 256 || hdv > 256 || hd < 1 || hdv < 1) return (int)cudaErrorInvalidValue;
    if (dtype == 0)
        return launch_step<float, true>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, nullptr, n_seq, nh, hd, hdv,
                                        st, zrows, zbias, inv_tau, q_scale);
    return launch_step<bf16, true>(q, k, v, ld, out, state, cu_q, seq_pos0, seq_slot, nullptr, n_seq, nh, hd, hdv, st,
                                   zrows, zbias, inv_tau, q_scale);
}

DK_EXPORT int dk_norm_gate(int dtype, const float* o, const float* w, float eps, const void* gate, long long ldg,
                           float out_scale, void* out, long long ldo, int n_tok, int n, int group, int gate_act,
                           cudaStream_t st) {
    if (group < 1 || n % group) return (int)cudaErrorInvalidValue;
    const int threads = group >= 2048 ? 512 : (group >= 512 ? 256 : (group >= 128 ? 128 : (group > 32 ? 64 : 32)));
    const dim3 grid(n_tok, n / group);
    if (dtype == 0)
        return dk_launch(norm_gate_kernel<float>, grid, dim3(threads), 0, st, o, w, eps, (const float*)gate, ldg,
                         out_scale, (float*)out, ldo, n, group, gate_act);
    return dk_launch(norm_gate_kernel<bf16>, grid, dim3(threads), 0, st, o, w, eps, (const bf16*)gate, ldg,
                     out_scale, (bf16*)out, ldo, n, group, gate_act);
}
