// Linear attention with a constant decay per head for portions of many tokens (bfloat16 storage), in
// blocks of 64 tokens (see linear_attention.cu for the recurrence and its token-by-token form):
//   inside a block   o_i  = sum_{j <= i} d^(i-j) (q_i . k_j) v_j           ((Q K^T) * D) V
//   across blocks    o_i += d^(i+1) q_i . S,   S <- d^n S + sum_j d^(n-1-j) k_j v_j^T   (n tokens in the block)
// Built once per key head size with -DHD=<multiple of 16 up to 256>. grid (sequence, head, slice of DVB
// value columns): the columns of a state evolve independently, so a head's state is split over blocks.
// Eight warps: four work out the block's outputs, 16 rows each, while the other four hold the state and move
// it on. The products Q K^T, P V and Q S run on the tensor cores
// (mma.sync m16n8k16, bfloat16 operands, float32 sums): q, k, v = silu(projection) are rounded to bfloat16
// once, as operands (in place, by a kernel of its own before this one); the decay weights multiply the float32 scores; the state enters Q S as a high and a
// low bfloat16 half (two products), so it counts with 16 bits of mantissa. The state itself stays in
// float32, in the accumulator registers of its own update S <- d^n S + (K w)^T V, also a tensor-core
// product: the decay weights w_j are float32 and k_j w_j enters as a high and a low half like the state.
// Key head sizes up to 128 (four staged key tiles must fit the shared memory).
#include "attention_mma.cuh"

constexpr int LB = 64;    // tokens a block of the sequence

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.f + __expf(-x)); }   // 2 ulp, then rounded to bfloat16

// The rows of a block are requested a block ahead (cp.async, 16 bytes a piece) straight into the tile the
// products read them from: their activation was applied in place by silu_rows_kernel before this kernel
// ran. Rows beyond the block's n tokens are zeros.
__device__ __forceinline__ void fetch_rows(bf16* dst, int dstride, const bf16* src, long long ld, int n, int width) {
    const int cpr = width / 8;
    for (int idx = threadIdx.x; idx < LB * cpr; idx += blockDim.x) {
        const int row = idx / cpr, col = (idx % cpr) * 8;
        if (row < n) cp_async16(dst + row * dstride + col, src + (size_t)row * ld + col);
        else *reinterpret_cast<uint4*>(dst + row * dstride + col) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// x <- silu(x) in place on the rows [rows, width] of up to three matrices that share a row stride
// (q, k and v of a fused projection): grid.y picks the matrix. Once per token and head, not once per block
// of the recurrence that reads it.
__global__ void silu_rows_kernel(bf16* a, int wa, bf16* b, int wb, bf16* c, int wc, long long ld, long long rows) {
    pdl_wait();
    pdl_launch_dependents();
    bf16* x = blockIdx.y == 0 ? a : (blockIdx.y == 1 ? b : c);
    const int width = blockIdx.y == 0 ? wa : (blockIdx.y == 1 ? wb : wc);
    const int cpr = width / 8;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * cpr) return;
    bf16* p = x + (idx / cpr) * ld + (idx % cpr) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    bf16* e = reinterpret_cast<bf16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; i++) e[i] = __float2bfloat16_rn(silu_f(__bfloat162float(e[i])));
    *reinterpret_cast<uint4*>(p) = raw;
}

// k * w_j (w_j = d^(n-1-j), float32) as a high and a low bfloat16 half, for the state's update on the tensor cores
__device__ __forceinline__ void stage_weighted_keys(bf16* hi, bf16* lo, const bf16* Ks, const float* pw, int n) {
    constexpr int cpr = HD / 8;
    for (int idx = threadIdx.x; idx < LB * cpr; idx += blockDim.x) {
        const int row = idx / cpr, col = (idx % cpr) * 8;
        uint4 rk = *reinterpret_cast<const uint4*>(Ks + row * KSTR + col), rh, rl;
        const bf16* e = reinterpret_cast<const bf16*>(&rk);
        bf16* eh = reinterpret_cast<bf16*>(&rh);
        bf16* el = reinterpret_cast<bf16*>(&rl);
        const float w = row < n ? pw[n - 1 - row] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float x = __bfloat162float(e[i]) * w;
            eh[i] = __float2bfloat16_rn(x);
            el[i] = __float2bfloat16_rn(x - __bfloat162float(eh[i]));
        }
        *reinterpret_cast<uint4*>(hi + row * KSTR + col) = rh;
        *reinterpret_cast<uint4*>(lo + row * KSTR + col) = rl;
    }
}

// A fragment (16 rows m0.., 16 columns k0..) of the transpose of a matrix stored [k][m] with row stride KSTR:
// the four 8x8 blocks (m0,k0), (m0+8,k0), (m0,k0+8), (m0+8,k0+8) come from the stored blocks with rows and
// columns exchanged, each loaded transposed.
__device__ __forceinline__ void ldsm_a_transposed(uint32_t (&a)[4], const bf16* base, int k0, int m0) {
    const int lane = threadIdx.x & 31, i = lane & 7, blk = lane >> 3;
    ldsm_x4_trans(a, base + (k0 + i + 8 * (blk >> 1)) * KSTR + m0 + 8 * (blk & 1));
}

constexpr int LC_THREADS = 256;   // warps 0-3: the block's outputs, 16 rows each; warps 4-7: the state and its update

template <int DVB>
__global__ void __launch_bounds__(LC_THREADS)
linear_attention_chunk_kernel(const bf16* q, const bf16* k, const bf16* v, long long ld, float* out, float* state,
                              const int* cu_q, const int* seq_slot, const float* __restrict__ decay, int nh, int hdv) {
    constexpr int VS = DVB + 8;
    constexpr int MT = HD / 16, MTW = (MT + 3) / 4;      // 16-row tiles of the state; those a warp owns (w, w+4, ..)
    extern __shared__ __align__(16) unsigned char raw_smem[];
    constexpr int IN_TILE = 2 * LB * KSTR + LB * VS;        // q, k and v of one block of tokens; two of them, in turn
    bf16* in0 = reinterpret_cast<bf16*>(raw_smem);
    bf16* Kh = in0 + 2 * IN_TILE;
    bf16* Kl = Kh + LB * KSTR;
    bf16* Sh = Kl + LB * KSTR;
    bf16* Sl = Sh + HD * VS;
    float* pw = reinterpret_cast<float*>(Sl + HD * VS);    // pw[n] = d^n, n = 0..64
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DVB;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int warp = (tid >> 5) & 3;
    const bool owns_state = (tid >> 7) == 1;
    const int r0 = cu_q[s], r1 = cu_q[s + 1];
    const float d = decay[h];
    float* S = state + ((size_t)seq_slot[s] * nh + h) * (size_t)HD * hdv + c0;
    if (tid <= LB) pw[tid] = (float)pow((double)d, (double)tid);
    // the state in the accumulator layout of its update: tile mt = warp + 4 i, rows 16 mt + g (+8), columns 8 nt + 2t (+1)
    float st[MTW][DVB / 8][4];
#pragma unroll
    for (int i = 0; i < MTW; i++) {
        const int mt = warp + 4 * i;
#pragma unroll
        for (int nt = 0; nt < DVB / 8; nt++) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                float2 x = make_float2(0.f, 0.f);
                if (mt < MT && owns_state) x = *reinterpret_cast<const float2*>(S + (size_t)(mt * 16 + g + 8 * r) * hdv + nt * 8 + 2 * t);
                st[i][nt][2 * r] = x.x;
                st[i][nt][2 * r + 1] = x.y;
            }
        }
    }
    const size_t ow = (size_t)nh * hdv;
    auto fetch = [&](int t0, int buf) {
        const int n = min(LB, r1 - t0);
        bf16* base = in0 + buf * IN_TILE;
        fetch_rows(base, KSTR, q + (size_t)t0 * ld + (size_t)h * HD, ld, n, HD);
        fetch_rows(base + LB * KSTR, KSTR, k + (size_t)t0 * ld + (size_t)h * HD, ld, n, HD);
        fetch_rows(base + 2 * LB * KSTR, VS, v + (size_t)t0 * ld + (size_t)h * hdv + c0, ld, n, DVB);
        cp_async_commit();
    };
    if (r0 < r1) fetch(r0, 0);
    for (int t0 = r0, it = 0; t0 < r1; t0 += LB, it++) {
        const int n = min(LB, r1 - t0);
        bf16* Qs = in0 + (it & 1) * IN_TILE;
        bf16* Ks = Qs + LB * KSTR;
        bf16* Vs = Ks + LB * KSTR;
        // the state as two bfloat16 halves for this block's Q S, and the block's operands
#pragma unroll
        for (int i = 0; i < MTW; i++) {
            const int mt = warp + 4 * i;
            if (mt < MT && owns_state) {
#pragma unroll
                for (int nt = 0; nt < DVB / 8; nt++) {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const float x0 = st[i][nt][2 * r], x1 = st[i][nt][2 * r + 1];
                        const __nv_bfloat162 hi = __floats2bfloat162_rn(x0, x1);
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(x0 - __bfloat162float(hi.x), x1 - __bfloat162float(hi.y));
                        const int at = (mt * 16 + g + 8 * r) * VS + nt * 8 + 2 * t;
                        *reinterpret_cast<__nv_bfloat162*>(Sh + at) = hi;
                        *reinterpret_cast<__nv_bfloat162*>(Sl + at) = lo;
                    }
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                       // this block's rows have landed, for every thread
        if (t0 + LB < r1) fetch(t0 + LB, (it + 1) & 1);        // the next block's, into the tiles the last block is done with
        stage_weighted_keys(Kh, Kl, Ks, pw, n);
        __syncthreads();
        if (!owns_state && warp * 16 < n) {
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
        // the state moves on by the block's n tokens: S <- d^n S + (K w)^T V, float32 sums in the registers that hold
        // it, by the other four warps while the first four work out the outputs
        const float dn = pw[n];
#pragma unroll
        for (int i = 0; i < MTW; i++) {
            const int mt = warp + 4 * i;
            if (mt < MT && owns_state) {
#pragma unroll
                for (int nt = 0; nt < DVB / 8; nt++) {
#pragma unroll
                    for (int c = 0; c < 4; c++) st[i][nt][c] *= dn;
                }
#pragma unroll
                for (int kk = 0; kk < LB / 16; kk++) {
                    uint32_t ah[4], al[4];
                    ldsm_a_transposed(ah, Kh, kk * 16, mt * 16);
                    ldsm_a_transposed(al, Kl, kk * 16, mt * 16);
#pragma unroll
                    for (int dp = 0; dp < DVB / 16; dp++) {
                        uint32_t b[4];
                        ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 15)) * VS + dp * 16 + 8 * (lane >> 4));
                        mma16816(st[i][2 * dp], ah, b[0], b[1]);
                        mma16816(st[i][2 * dp + 1], ah, b[2], b[3]);
                        mma16816(st[i][2 * dp], al, b[0], b[1]);
                        mma16816(st[i][2 * dp + 1], al, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < MTW; i++) {
        const int mt = warp + 4 * i;
        if (mt < MT && owns_state) {
#pragma unroll
            for (int nt = 0; nt < DVB / 8; nt++) {
#pragma unroll
                for (int r = 0; r < 2; r++)
                    *reinterpret_cast<float2*>(S + (size_t)(mt * 16 + g + 8 * r) * hdv + nt * 8 + 2 * t) =
                        make_float2(st[i][nt][2 * r], st[i][nt][2 * r + 1]);
            }
        }
    }
}

template <int DVB>
static int launch_chunk(const void* q, const void* k, const void* v, long long ld, float* out, float* state,
                        const int* cu_q, const int* seq_slot, const float* decay, int n_seq, int nh, int hdv,
                        cudaStream_t st) {
    constexpr int VS = DVB + 8;
    const size_t smem = sizeof(bf16) * (size_t)(6 * LB * KSTR + 2 * LB * VS + 2 * HD * VS) + sizeof(float) * 72;
    static bool attr = false;
    if (!attr && smem > 48 * 1024) {
        cudaFuncSetAttribute(linear_attention_chunk_kernel<DVB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr = true;
    }
    return dk_launch(linear_attention_chunk_kernel<DVB>, dim3(n_seq, nh, hdv / DVB), dim3(LC_THREADS), smem, st, (const bf16*)q,
                     (const bf16*)k, (const bf16*)v, ld, out, state, cu_q, seq_slot, decay, nh, hdv);
}

// q, k and v are overwritten by their activation (nothing else reads them after this call).
DK_EXPORT int dk_linear_attention_chunk_bf16(void* q, void* k, void* v, long long ld, long long n_rows, float* out,
                                             float* state, const int* cu_q, const int* seq_slot, const float* decay,
                                             int n_seq, int nh, int hdv, cudaStream_t st) {
    if (hdv % 16 != 0 || ld % 8 != 0) return (int)cudaErrorInvalidValue;
    const int widest = nh * (HD > hdv ? HD : hdv);
    const long long items = n_rows * (widest / 8);
    int e = dk_launch(silu_rows_kernel, dim3((unsigned)((items + 255) / 256), 3), dim3(256), 0, st, (bf16*)q, nh * HD, (bf16*)k,
                      nh * HD, (bf16*)v, nh * hdv, ld, n_rows);
    if (e != 0) return e;
    // 32 value columns a block; 16 while that leaves SMs without a block (a block of 16 repeats Q K^T for half the
    // columns, but the chain of a sequence's blocks is what the kernel's time is made of)
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (hdv % 32 == 0 && (long long)n_seq * nh * (hdv / 32) >= sms)
        return launch_chunk<32>(q, k, v, ld, out, state, cu_q, seq_slot, decay, n_seq, nh, hdv, st);
    return launch_chunk<16>(q, k, v, ld, out, state, cu_q, seq_slot, decay, n_seq, nh, hdv, st);
}
