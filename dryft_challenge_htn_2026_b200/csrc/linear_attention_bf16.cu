// Linear attention with a constant decay per head for portions of many tokens (bfloat16 storage), in
// blocks of 64 tokens (see linear_attention.cu for the recurrence and its token-by-token form):
//   inside a block   o_i  = sum_{j <= i} d^(i-j) (q_i . k_j) v_j           ((Q K^T) * D) V
//   across blocks    o_i += d^(i+1) q_i . S,   S <- d^n S + sum_j d^(n-1-j) k_j v_j^T   (n tokens in the block)
// Built once per key head size with -DHD=<multiple of 16 up to 256>. grid (sequence, head, slice of DVB
// value columns): the columns of a state evolve independently, so a head's state is split over blocks.
// Four warps, 16 rows of the block each. The products Q K^T, P V and Q S run on the tensor cores
// (mma.sync m16n8k16, bfloat16 operands, float32 sums): q, k, v = silu(projection) are rounded to bfloat16
// once, as operands; the decay weights multiply the float32 scores; the state enters Q S as a high and a
// low bfloat16 half (two products), so it counts with 16 bits of mantissa. The state itself stays in
// float32 registers of the threads that own it and is updated there on the CUDA cores (fused multiply-add
// in float32 with the float32 decay weights), then stored back.
#include "attention_mma.cuh"

constexpr int LB = 64;    // tokens a block of the sequence

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ void stage_rows(bf16* dst, int dstride, const bf16* src, long long ld, int n, int width) {
    const int cpr = width / 8;
    for (int idx = threadIdx.x; idx < LB * cpr; idx += blockDim.x) {
        const int row = idx / cpr, col = (idx % cpr) * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (row < n) {
            raw = *reinterpret_cast<const uint4*>(src + (size_t)row * ld + col);
            bf16* e = reinterpret_cast<bf16*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; i++) e[i] = __float2bfloat16_rn(silu_f(__bfloat162float(e[i])));
        }
        *reinterpret_cast<uint4*>(dst + row * dstride + col) = raw;
    }
}

template <int DVB>
__global__ void __launch_bounds__(128)
linear_attention_chunk_kernel(const bf16* q, const bf16* k, const bf16* v, long long ld, float* out, float* state,
                              const int* cu_q, const int* seq_slot, const float* __restrict__ decay, int nh, int hdv) {
    constexpr int VS = DVB + 8;
    constexpr int CG = DVB / 4, RG = 128 / CG, RPT = (HD + RG - 1) / RG;
    extern __shared__ __align__(16) unsigned char raw_smem[];
    bf16* Qs = reinterpret_cast<bf16*>(raw_smem);
    bf16* Ks = Qs + LB * KSTR;
    bf16* Vs = Ks + LB * KSTR;
    bf16* Sh = Vs + LB * VS;
    bf16* Sl = Sh + HD * VS;
    float* pw = reinterpret_cast<float*>(Sl + HD * VS);    // pw[n] = d^n, n = 0..64
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DVB;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int r0 = cu_q[s], r1 = cu_q[s + 1];
    const float d = decay[h];
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)HD * hdv;
    const int cg = tid % CG, rg = tid / CG;
    if (tid <= LB) pw[tid] = (float)pow((double)d, (double)tid);
    float st[RPT][4];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int row = rg + RG * i;
#pragma unroll
        for (int e = 0; e < 4; e++) st[i][e] = row < HD ? S[(size_t)row * hdv + c0 + 4 * cg + e] : 0.f;
    }
    const size_t ow = (size_t)nh * hdv;
    for (int t0 = r0; t0 < r1; t0 += LB) {
        const int n = min(LB, r1 - t0);
        // the state as two bfloat16 halves for this block's Q S, and the block's operands
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            const int row = rg + RG * i;
            if (row < HD) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const bf16 hi = __float2bfloat16_rn(st[i][e]);
                    Sh[row * VS + 4 * cg + e] = hi;
                    Sl[row * VS + 4 * cg + e] = __float2bfloat16_rn(st[i][e] - __bfloat162float(hi));
                }
            }
        }
        stage_rows(Qs, KSTR, q + (size_t)t0 * ld + (size_t)h * HD, ld, n, HD);
        stage_rows(Ks, KSTR, k + (size_t)t0 * ld + (size_t)h * HD, ld, n, HD);
        stage_rows(Vs, VS, v + (size_t)t0 * ld + (size_t)h * hdv + c0, ld, n, DVB);
        __syncthreads();
        if (warp * 16 < n) {
            uint32_t qf[HD / 16][4];
            load_q_frags(qf, Qs + (warp * 16 + g) * KSTR, Qs + (warp * 16 + g + 8) * KSTR);
            float sc[LB / 8][4];
#pragma unroll
            for (int i = 0; i < LB / 8; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
            const int j4 = lane >> 3;
#pragma unroll
            for (int np = 0; np < LB / 16; np++) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    uint32_t b[4];
                    ldsm_x4(b, Ks + (np * 16 + (lane & 7) + 8 * (j4 >> 1)) * KSTR + ks * 16 + 8 * (j4 & 1));
                    mma16816(sc[2 * np], qf[ks], b[0], b[1]);
                    mma16816(sc[2 * np + 1], qf[ks], b[2], b[3]);
                }
            }
            // decay weights: score_ij * d^(i-j) for j <= i, nothing beyond the diagonal
#pragma unroll
            for (int nt = 0; nt < LB / 8; nt++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int i = warp * 16 + g + 8 * (c >> 1), j = nt * 8 + 2 * t + (c & 1);
                    sc[nt][c] = j <= i ? sc[nt][c] * pw[i - j] : 0.f;
                }
            }
            float acc[DVB / 8][4], acs[DVB / 8][4];
#pragma unroll
            for (int i = 0; i < DVB / 8; i++) {
                acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
                acs[i][0] = acs[i][1] = acs[i][2] = acs[i][3] = 0.f;
            }
#pragma unroll
            for (int kk = 0; kk < LB / 16; kk++) {
                uint32_t a[4];
                a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DVB / 16; dp++) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 15)) * VS + dp * 16 + 8 * (lane >> 4));
                    mma16816(acc[2 * dp], a, b[0], b[1]);
                    mma16816(acc[2 * dp + 1], a, b[2], b[3]);
                }
            }
            // across blocks: q . S with the state's two halves
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
#pragma unroll
                for (int dp = 0; dp < DVB / 16; dp++) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, Sh + (ks * 16 + (lane & 15)) * VS + dp * 16 + 8 * (lane >> 4));
                    mma16816(acs[2 * dp], qf[ks], b[0], b[1]);
                    mma16816(acs[2 * dp + 1], qf[ks], b[2], b[3]);
                    ldsm_x4_trans(b, Sl + (ks * 16 + (lane & 15)) * VS + dp * 16 + 8 * (lane >> 4));
                    mma16816(acs[2 * dp], qf[ks], b[0], b[1]);
                    mma16816(acs[2 * dp + 1], qf[ks], b[2], b[3]);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int i = warp * 16 + g + 8 * r;
                if (i < n) {
                    const float w = pw[i + 1];
                    float* orow = out + (size_t)(t0 + i) * ow + (size_t)h * hdv + c0;
#pragma unroll
                    for (int nt = 0; nt < DVB / 8; nt++)
                        *reinterpret_cast<float2*>(orow + nt * 8 + 2 * t) =
                            make_float2(fmaf(w, acs[nt][2 * r], acc[nt][2 * r]), fmaf(w, acs[nt][2 * r + 1], acc[nt][2 * r + 1]));
                }
            }
        }
        // the state moves on by the block's n tokens, in float32 in its owners' registers
        const float dn = pw[n];
#pragma unroll
        for (int i = 0; i < RPT; i++) {
#pragma unroll
            for (int e = 0; e < 4; e++) st[i][e] *= dn;
        }
        for (int j = 0; j < n; j++) {
            const float w = pw[n - 1 - j];
            float vv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) vv[e] = __bfloat162float(Vs[j * VS + 4 * cg + e]);
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                const int row = rg + RG * i;
                if (row < HD) {
                    const float kw = __bfloat162float(Ks[j * KSTR + row]) * w;
#pragma unroll
                    for (int e = 0; e < 4; e++) st[i][e] = fmaf(kw, vv[e], st[i][e]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        const int row = rg + RG * i;
        if (row < HD) {
#pragma unroll
            for (int e = 0; e < 4; e++) S[(size_t)row * hdv + c0 + 4 * cg + e] = st[i][e];
        }
    }
}

template <int DVB>
static int launch_chunk(const void* q, const void* k, const void* v, long long ld, float* out, float* state,
                        const int* cu_q, const int* seq_slot, const float* decay, int n_seq, int nh, int hdv,
                        cudaStream_t st) {
    constexpr int VS = DVB + 8;
    const size_t smem = sizeof(bf16) * (size_t)(2 * LB * KSTR + LB * VS + 2 * HD * VS) + sizeof(float) * 72;
    static bool attr = false;
    if (!attr && smem > 48 * 1024) {
        cudaFuncSetAttribute(linear_attention_chunk_kernel<DVB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr = true;
    }
    return dk_launch(linear_attention_chunk_kernel<DVB>, dim3(n_seq, nh, hdv / DVB), dim3(128), smem, st, (const bf16*)q,
                     (const bf16*)k, (const bf16*)v, ld, out, state, cu_q, seq_slot, decay, nh, hdv);
}

DK_EXPORT int dk_linear_attention_chunk_bf16(const void* q, const void* k, const void* v, long long ld, float* out,
                                             float* state, const int* cu_q, const int* seq_slot, const float* decay,
                                             int n_seq, int nh, int hdv, cudaStream_t st) {
    if (hdv % 16 != 0 || ld % 8 != 0) return (int)cudaErrorInvalidValue;
    if (hdv % 32 == 0) return launch_chunk<32>(q, k, v, ld, out, state, cu_q, seq_slot, decay, n_seq, nh, hdv, st);
    return launch_chunk<16>(q, k, v, ld, out, state, cu_q, seq_slot, decay, n_seq, nh, hdv, st);
}
