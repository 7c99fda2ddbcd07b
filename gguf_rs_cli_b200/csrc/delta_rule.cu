// The pieces of a gated delta-rule mixer with one decay per head and key channel:
//   1. a short causal convolution over time per channel, followed by SiLU, whose last inputs
//      are carried from step to step per sequence;
//   2. the recurrence itself, state in 32-bit;
//   3. the per-head RMS norm of what the recurrence reads out, times a weight and a sigmoid gate.
// Everything that enters the recurrence is computed in 32-bit from the projections' outputs:
// unit vectors, decays (exponentials, softplus), the write strength, the state.
#include <math.h>

#include "common.cuh"

// ------------------------------------------------- short convolution + SiLU
// out[t, c] = silu(sum_j taps[c, j] * in[t - (K-1-j), c]); rows before the step's first token come from
// the sequence's carried inputs state[slot, 0..K-2, c] (oldest first; zero for a sequence that starts).
// blockIdx.x is the token, blockIdx.y a slice of blockDim.x channels.  Padding tokens (seq_of < 0) give zeros.
__global__ void short_conv_silu_kernel(const void* __restrict__ xin, int dtype, long long ldx, int C, int K,
                                       const void* __restrict__ taps, int taps_dtype, const float* __restrict__ state,
                                       const int* __restrict__ seq_of, const int* __restrict__ cu,
                                       const int* __restrict__ slots, void* __restrict__ out, long long ldo) {
    const int t = blockIdx.x;
    const int b = seq_of[t];
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    if (b < 0) {
        gb_store(out, dtype, size_t(t) * ldo + c, 0.f);
        return;
    }
    const int first = cu[b], i = t - first, slot = slots[b];
    const float* st = state + size_t(slot) * (K - 1) * C;
    {
        float acc = 0.f;
        for (int j = 0; j < K; ++j) {
            const int src = i - (K - 1 - j);
            const float xv = src >= 0 ? gb_load(xin, dtype, size_t(first + src) * ldx + c)
                                      : st[size_t(K - 1 + src) * C + c];
            acc = fmaf(xv, gb_load(taps, taps_dtype, size_t(c) * K + j), acc);
        }
        gb_store(out, dtype, size_t(t) * ldo + c, acc / (1.f + expf(-acc)));
    }
}

// After the convolution: the sequence's carried inputs become the last K-1 inputs including this step's.
// blockIdx.x is the sequence, blockIdx.y a slice of channels; a thread owns a channel, reads all it needs and
// then writes.
constexpr int CONV_MAX_TAPS = 16;

__global__ void short_conv_carry_kernel(const void* __restrict__ xin, int dtype, long long ldx, int C, int K,
                                        float* __restrict__ state, const int* __restrict__ cu,
                                        const int* __restrict__ slots, const int* __restrict__ qlens) {
    const int b = blockIdx.x;
    const int slot = slots[b], n = qlens[b];
    if (slot < 0 || n <= 0) return;
    const int first = cu[b];
    float* st = state + size_t(slot) * (K - 1) * C;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < C) {
        float keep[CONV_MAX_TAPS - 1];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
            if (j < K - 1) {
                const int src = n - (K - 1) + j;
                keep[j] = src >= 0 ? gb_load(xin, dtype, size_t(first + src) * ldx + c) : st[size_t(j + n) * C + c];
            }
        }
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) st[size_t(j) * C + c] = keep[j];
    }
}

// xin: [T, C] with pitch ldx (the projections' outputs); taps [C, K], last column on the current token;
// state f32 [slots, K-1, C]; out [T, C] with pitch ldo, same dtype as xin.  The carried inputs are renewed.
GB_API int gb_short_conv_silu(const void* xin, int dtype, long long ldx, int T, int B, int C, int K, const void* taps,
                              int taps_dtype, float* state, const int* seq_of, const int* cu, const int* slots,
                              const int* qlens, void* out, long long ldo, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(taps_dtype), "gb_short_conv_silu: bad dtype");
    GB_REQUIRE(C > 0 && K >= 1 && K <= CONV_MAX_TAPS && ldx >= C && ldo >= C, "gb_short_conv_silu: bad sizes C=%d taps=%d (1..%d)",
               C, K, CONV_MAX_TAPS);
    GB_REQUIRE(K == 1 || state, "gb_short_conv_silu: a convolution of %d taps needs the carried inputs", K);
    if (T == 0) return 0;
    const int threads = 128, slices = (C + threads - 1) / threads;
    GB_REQUIRE(slices <= 65535, "gb_short_conv_silu: too many channels (%d)", C);
    short_conv_silu_kernel<<<dim3(T, slices), threads, 0, stream>>>(xin, dtype, ldx, C, K, taps, taps_dtype, state, seq_of, cu, slots, out, ldo);
    GB_LAUNCH_OK("gb_short_conv_silu");
    if (K > 1 && B > 0) {
        short_conv_carry_kernel<<<dim3(B, slices), threads, 0, stream>>>(xin, dtype, ldx, C, K, state, cu, slots, qlens);
        GB_LAUNCH_OK("gb_short_conv_silu (carry)");
    }
    return 0;
}

// ------------------------------------------------------------ the recurrence
// Per sequence and head, with S [D, Dv] (key channel i, value column j), for every token in order:
//   qn = q / sqrt(sum q^2 + 1e-6) * q_scale,  kn = k / sqrt(sum k^2 + 1e-6)
//   decay_i = exp(-exp(A_log_h) * softplus(a_i + dt_bias_i)),  beta = sigmoid(b)
//   S_ij <- decay_i S_ij;  u_j = beta (v_j - sum_i S_ij kn_i);  S_ij <- S_ij + kn_i u_j;  o_j = sum_i S_ij qn_i
// Columns of S do not interact, so a block takes a slice of columns of one (sequence, head): a column is
// shared by R lanes of a warp (R a power of two), lane r holding rows r, r + R, ...: NR of them in
// registers; the sums over i end with shuffles over those lanes.  The token's q, k, decay, v and beta are
// prepared for a few tokens at a time in shared memory by the whole block (rows padded to R*NR entries with
// zeros, so the inner loops carry no bounds).  The state is read once at the start and written once at the end.
struct DeltaRuleParams {
    const void *q, *k, *v;          // after convolution and SiLU: q, k [T, G*D], v [T, H*Dv], rows `ld` apart
    const void* beta;               // [T, H] before the sigmoid, rows ld_beta apart
    const void* a;                  // [T, H*D] before bias and softplus, rows ld_a apart
    const void *dt_bias, *A_log;    // [H*D], [H]
    float* state;                   // [slots, H, D, Dv]
    float* out;                     // [T, H*Dv], rows ldo apart
    const int *cu, *slots, *qlens;
    long long ld, ld_beta, ld_a, ldo;
    int dtype, w_dtype, H, G, D, Dv, R, TC;
    float q_scale;
};

template <int NR>
__global__ void __launch_bounds__(128) delta_rule_kernel(const DeltaRuleParams p) {
    extern __shared__ float sm[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int slot = p.slots[b], n = p.qlens[b];
    if (slot < 0 || n <= 0) return;
    const int R = p.R, CW = 32 / R, CB = 4 * CW, DP = R * NR, D = p.D, Dv = p.Dv, TC = p.TC;
    float* qs = sm;
    float* ks = qs + TC * DP;
    float* gs = ks + TC * DP;
    float* vs = gs + TC * DP;
    float* bs = vs + TC * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane / CW, jj = lane - r * CW;
    const int j = blockIdx.z * CB + warp * CW + jj;
    const bool col_ok = j < Dv;
    const int g = h / (p.H / p.G);
    float* sp = p.state + (size_t(slot) * p.H + h) * size_t(D) * Dv;
    float S[NR];
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r + R * m;
        S[m] = (i < D && col_ok) ? sp[size_t(i) * Dv + j] : 0.f;
    }
    const int t0 = p.cu[b];
    const float rate = expf(gb_load(p.A_log, p.w_dtype, h));
    for (int c0 = 0; c0 < n; c0 += TC) {
        const int nt = min(TC, n - c0);
        __syncthreads();                                   // the chunk before has been consumed
        for (int tt = warp; tt < nt; tt += 4) {
            const size_t t = size_t(t0 + c0 + tt);
            const size_t row = t * p.ld + size_t(g) * D;
            float sq = 0.f, sk = 0.f;
            for (int d = lane; d < DP; d += 32) {
                float qv = 0.f, kv = 0.f, gv = 0.f;
                if (d < D) {
                    qv = gb_load(p.q, p.dtype, row + d);
                    kv = gb_load(p.k, p.dtype, row + d);
                    const float z = gb_load(p.a, p.dtype, t * p.ld_a + size_t(h) * D + d) +
                                    gb_load(p.dt_bias, p.w_dtype, size_t(h) * D + d);
                    const float soft = z > 20.f ? z : log1pf(expf(z));
                    gv = expf(-rate * soft);
                }
                qs[tt * DP + d] = qv;
                ks[tt * DP + d] = kv;
                gs[tt * DP + d] = gv;
                sq = fmaf(qv, qv, sq);
                sk = fmaf(kv, kv, sk);
            }
            sq = gb_warp_sum(sq);
            sk = gb_warp_sum(sk);
            const float qn = p.q_scale / sqrtf(sq + 1e-6f), kn = 1.f / sqrtf(sk + 1e-6f);
            for (int d = lane; d < DP; d += 32) {          // each lane rescales what it wrote itself
                qs[tt * DP + d] *= qn;
                ks[tt * DP + d] *= kn;
            }
            if (lane == 0) bs[tt] = 1.f / (1.f + expf(-gb_load(p.beta, p.dtype, t * p.ld_beta + h)));
        }
        for (int idx = threadIdx.x; idx < nt * CB; idx += 128) {
            const int tt = idx / CB, cj = idx - tt * CB;
            const int col = blockIdx.z * CB + cj;
            vs[idx] = col < Dv ? gb_load(p.v, p.dtype, size_t(t0 + c0 + tt) * p.ld + size_t(h) * Dv + col) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* qq = qs + tt * DP + r;
            const float* kk = ks + tt * DP + r;
            const float* gg = gs + tt * DP + r;
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int m = 0; m < NR; m += 2) {
                S[m] *= gg[R * m];
                d0 = fmaf(S[m], kk[R * m], d0);
                S[m + 1] *= gg[R * (m + 1)];
                d1 = fmaf(S[m + 1], kk[R * (m + 1)], d1);
            }
            float dot = d0 + d1;
            for (int off = CW; off < 32; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            const float u = bs[tt] * (vs[tt * CB + warp * CW + jj] - dot);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int m = 0; m < NR; m += 2) {
                S[m] = fmaf(kk[R * m], u, S[m]);
                o0 = fmaf(S[m], qq[R * m], o0);
                S[m + 1] = fmaf(kk[R * (m + 1)], u, S[m + 1]);
                o1 = fmaf(S[m + 1], qq[R * (m + 1)], o1);
            }
            float o = o0 + o1;
            for (int off = CW; off < 32; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (r == 0 && col_ok) p.out[size_t(t0 + c0 + tt) * p.ldo + size_t(h) * Dv + j] = o;
        }
    }
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r + R * m;
        if (i < D && col_ok) sp[size_t(i) * Dv + j] = S[m];
    }
}

// Rows per lane and lanes per column for key size D: 32 rows a lane up to D = 1024, 64 beyond.
static void delta_rule_shape(int D, int* nr, int* r) {
    int NR = D > 1024 ? 64 : 32, R = 1;
    while (R * NR < D) R <<= 1;
    *nr = NR;
    *r = R;
}

GB_API int gb_delta_rule(const void* q, const void* k, const void* v, int dtype, long long ld, const void* beta,
                         long long ld_beta, const void* a, long long ld_a, const void* dt_bias, const void* A_log,
                         int w_dtype, float* state, float* out, long long ldo, const int* cu, const int* slots,
                         const int* qlens, int B, int H, int G, int D, int Dv, float q_scale, cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(dtype) && gb_is_dtype(w_dtype), "gb_delta_rule: bad dtype");
    GB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0, "gb_delta_rule: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d", H, G, D, Dv);
    GB_REQUIRE(D <= 2048, "gb_delta_rule: key size %d exceeds 2048", D);
    GB_REQUIRE(H <= 65535, "gb_delta_rule: too many heads (%d)", H);
    if (B == 0) return 0;
    DeltaRuleParams p;
    p.q = q; p.k = k; p.v = v; p.beta = beta; p.a = a; p.dt_bias = dt_bias; p.A_log = A_log; p.state = state; p.out = out;
    p.cu = cu; p.slots = slots; p.qlens = qlens; p.ld = ld; p.ld_beta = ld_beta; p.ld_a = ld_a; p.ldo = ldo;
    p.dtype = dtype; p.w_dtype = w_dtype; p.H = H; p.G = G; p.D = D; p.Dv = Dv; p.q_scale = q_scale;
    int NR, R;
    delta_rule_shape(D, &NR, &R);
    const int CB = 4 * (32 / R), DP = R * NR;
    const int per_token = 4 * (3 * DP + CB + 1);
    int TC = (40 * 1024) / per_token;
    TC = TC < 1 ? 1 : (TC > 16 ? 16 : TC);
    p.R = R; p.TC = TC;
    const size_t smem = size_t(TC) * per_token;
    GB_REQUIRE(smem <= 48 * 1024, "gb_delta_rule: key size %d needs %zu bytes of shared memory", D, smem);
    dim3 grid(B, H, (Dv + CB - 1) / CB);
    GB_REQUIRE(grid.z <= 65535, "gb_delta_rule: value size %d is too large", Dv);
    if (NR == 32) delta_rule_kernel<32><<<grid, 128, smem, stream>>>(p);
    else delta_rule_kernel<64><<<grid, 128, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_delta_rule");
    return 0;
}

// --------------------------------------------- per-head RMS norm, weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w[:] * sigmoid(gate[t, h, :]); one warp per
// (token, head); w [Dv] is shared by the heads.
__global__ void gated_head_norm_kernel(const float* __restrict__ o, long long ldo, const void* __restrict__ gate,
                                       int gate_dtype, long long ldg, const void* __restrict__ w, int w_dtype, float eps,
                                       void* __restrict__ out, int out_dtype, long long ld_out, long long items, int H, int Dv) {
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long long t = item / H;
    const int h = int(item - t * H);
    const float* orow = o + t * ldo + size_t(h) * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss = fmaf(orow[d], orow[d], ss);
    const float rms = sqrtf(gb_warp_sum(ss) / float(Dv) + eps);
    for (int d = lane; d < Dv; d += 32) {
        const float gt = gb_load(gate, gate_dtype, size_t(t) * ldg + size_t(h) * Dv + d);
        gb_store(out, out_dtype, size_t(t) * ld_out + size_t(h) * Dv + d,
                 orow[d] / rms * gb_load(w, w_dtype, d) * (1.f / (1.f + expf(-gt))));
    }
}

GB_API int gb_gated_head_norm(const float* o, long long ldo, const void* gate, int gate_dtype, long long ldg, const void* w,
                              int w_dtype, float eps, void* out, int out_dtype, long long ld_out, int T, int H, int Dv,
                              cudaStream_t stream) {
    GB_REQUIRE(gb_is_dtype(gate_dtype) && gb_is_dtype(w_dtype) && gb_is_dtype(out_dtype), "gb_gated_head_norm: bad dtype");
    GB_REQUIRE(H > 0 && Dv > 0 && eps > 0.f, "gb_gated_head_norm: bad sizes heads=%d vdim=%d eps=%g", H, Dv, eps);
    if (T == 0) return 0;
    const long long items = (long long)T * H;
    gated_head_norm_kernel<<<unsigned((items + 3) / 4), 128, 0, stream>>>(o, ldo, gate, gate_dtype, ldg, w, w_dtype, eps, out,
                                                                          out_dtype, ld_out, items, H, Dv);
    GB_LAUNCH_OK("gb_gated_head_norm");
    return 0;
}
