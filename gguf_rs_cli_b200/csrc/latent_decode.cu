// Latent attention for steps in which every sequence brings one token: all heads of a token share one key/value
// head, the cached rows [c (C entries), rotated part (R entries)], and each head's query has already been
// brought into that space (q' = W_uk^T q, then the rotated part).  score_h(j) = q_h . row_j * scale over the
// C + R entries; the mix of values is the mix of the rows' first C entries.
//
// One block per (token, split of the token's keys) serves ALL heads from one pass over its keys: 32 rows at a
// time are copied into shared memory once (16-byte pieces, rows padded by 16 bytes so that lanes reading
// different rows fall into different banks) and every warp takes its heads (warp, warp + 8, ...) over them:
// lane = key for the scores, lane = pair of entries for the values.  The general kernel, with a block per
// (token, head), reads every row once per head.  Scores, softmax and mix are 32-bit.  A split leaves its
// maximum, its sum and its unnormalised mix in scratch memory; a second kernel merges the splits in split
// order, so the result does not depend on timing.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LD_WARPS = 8;
constexpr int LD_THREADS = LD_WARPS * 32;
constexpr int LD_MAX_HEADS = 16;                    // heads per token: at most 2 per warp (with 32 heads the general
                                                    // kernel's block per head was measured faster: 0.774 against 0.799 ms a step)
constexpr int LD_HW = LD_MAX_HEADS / LD_WARPS;
constexpr int LD_MAX_C = 512;                       // entries of the value: at most 8 pairs per lane
constexpr int LD_PAIRS = LD_MAX_C / 64;

// Entries between two rows of the tile in shared memory: 16 bytes of padding, 32 where 16 would put all rows
// on the same banks.
__host__ __device__ inline int ld_row_stride(int hdk) { return (hdk + 8) % 64 ? hdk + 8 : hdk + 16; }

struct LdParams {
    const __nv_bfloat16* q;       // [T, H*(C+R)] rows ldq apart
    const __nv_bfloat16* cache;   // [pages, 1, 64, C+R]
    const int *seq_of, *pos, *table;
    float* scratch;               // [T, H, splits, C + 2]: unnormalised mix, maximum, sum
    long long ldq;
    int H, C, R, splits, table_width, ring_pages;
    float scale;
};

__global__ void __launch_bounds__(LD_THREADS) latent_decode_kernel(const LdParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, split = blockIdx.y;
    const int b = p.seq_of[t];
    if (b < 0) return;                                       // padding: the merge writes zeros
    const int H = p.H, C = p.C, HDK = p.C + p.R, KS = ld_row_stride(HDK);   // KS: entries of a padded row in shared memory
    float* qs = reinterpret_cast<float*>(smem_raw);                                   // [H][HDK]
    __nv_bfloat16* kt = reinterpret_cast<__nv_bfloat16*>(qs + size_t(H) * HDK);       // [32][KS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.pos[t];
    const int nkb = (pos >> 5) + 1;                          // blocks of 32 keys up to the token's own
    const int per = (nkb + p.splits - 1) / p.splits;
    const int kb0 = split * per, kb1 = min(nkb, kb0 + per);
    const int* trow = p.table + size_t(b) * p.table_width;

    for (int i = threadIdx.x; i < H * HDK; i += LD_THREADS)
        qs[i] = __bfloat162float(p.q[size_t(t) * p.ldq + i]);

    float m[LD_HW], l[LD_HW], acc[LD_HW][2 * LD_PAIRS];
#pragma unroll
    for (int hi = 0; hi < LD_HW; ++hi) {
        m[hi] = -INFINITY;
        l[hi] = 0.f;
#pragma unroll
        for (int c = 0; c < 2 * LD_PAIRS; ++c) acc[hi][c] = 0.f;
    }
    const int pieces = HDK / 8;
    for (int kb = kb0; kb < kb1; ++kb) {
        __syncthreads();                                     // the tile before has been used (and qs is written)
        for (int i = threadIdx.x; i < 32 * pieces; i += LD_THREADS) {
            const int r = i / pieces, c8 = i - r * pieces, j = kb * 32 + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (j <= pos) v = *reinterpret_cast<const uint4*>(p.cache + gb_kv_offset(trow, p.ring_pages, j, 0, 1, HDK) + 8 * c8);
            *reinterpret_cast<uint4*>(kt + r * KS + 8 * c8) = v;
        }
        __syncthreads();
        const bool valid = kb * 32 + lane <= pos;
#pragma unroll
        for (int hi = 0; hi < LD_HW; ++hi) {
            const int h = warp + LD_WARPS * hi;
            if (h >= H) break;
            const float* qh = qs + size_t(h) * HDK;
            const __nv_bfloat16* kr = kt + lane * KS;
            float d0 = 0.f, d1 = 0.f;
            for (int c8 = 0; c8 < pieces; ++c8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(kr + 8 * c8);
                const float4 qa = *reinterpret_cast<const float4*>(qh + 8 * c8), qb = *reinterpret_cast<const float4*>(qh + 8 * c8 + 4);
                const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 k0 = __bfloat1622float2(k2[0]), k1 = __bfloat1622float2(k2[1]);
                const float2 k2f = __bfloat1622float2(k2[2]), k3 = __bfloat1622float2(k2[3]);
                d0 = fmaf(qa.x, k0.x, d0); d1 = fmaf(qa.y, k0.y, d1);
                d0 = fmaf(qa.z, k1.x, d0); d1 = fmaf(qa.w, k1.y, d1);
                d0 = fmaf(qb.x, k2f.x, d0); d1 = fmaf(qb.y, k2f.y, d1);
                d0 = fmaf(qb.z, k3.x, d0); d1 = fmaf(qb.w, k3.y, d1);
            }
            const float s = valid ? (d0 + d1) * p.scale : -INFINITY;
            const float m_new = fmaxf(m[hi], gb_warp_max(s));
            const float alpha = m[hi] == -INFINITY ? 0.f : expf(m[hi] - m_new);
            const float pj = valid ? expf(s - m_new) : 0.f;
            l[hi] = l[hi] * alpha + gb_warp_sum(pj);
            m[hi] = m_new;
#pragma unroll
            for (int c = 0; c < 2 * LD_PAIRS; ++c) acc[hi][c] *= alpha;
            for (int r = 0; r < 32; ++r) {
                const float pr = __shfl_sync(0xffffffffu, pj, r);
                if (pr == 0.f) continue;                     // uniform over the warp
                const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(kt + r * KS);
#pragma unroll
                for (int cp = 0; cp < LD_PAIRS; ++cp) {
                    if (64 * cp + 2 * lane < C) {
                        const float2 vv = __bfloat1622float2(vr[32 * cp + lane]);
                        acc[hi][2 * cp] = fmaf(pr, vv.x, acc[hi][2 * cp]);
                        acc[hi][2 * cp + 1] = fmaf(pr, vv.y, acc[hi][2 * cp + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int hi = 0; hi < LD_HW; ++hi) {
        const int h = warp + LD_WARPS * hi;
        if (h >= H) break;
        float* o = p.scratch + ((size_t(t) * H + h) * p.splits + split) * (C + 2);
#pragma unroll
        for (int cp = 0; cp < LD_PAIRS; ++cp) {
            const int c = 64 * cp + 2 * lane;
            if (c < C) {
                o[c] = acc[hi][2 * cp];
                o[c + 1] = acc[hi][2 * cp + 1];
            }
        }
        if (lane == 0) {
            o[C] = m[hi];
            o[C + 1] = l[hi];
        }
    }
}

// out[t, h, :] = sum_s mix_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in order; padding tokens give zeros.
__global__ void latent_decode_merge_kernel(const float* __restrict__ scratch, const int* __restrict__ seq_of,
                                           __nv_bfloat16* __restrict__ out, long long ldo, int H, int C, int splits) {
    const int t = blockIdx.x, h = blockIdx.y;
    __nv_bfloat16* o = out + size_t(t) * ldo + size_t(h) * C;
    if (seq_of[t] < 0) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* base = scratch + (size_t(t) * H + h) * splits * (C + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, base[size_t(s) * (C + 2) + C]);
    float L = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = base[size_t(s) * (C + 2) + C];
        if (ms != -INFINITY) L += base[size_t(s) * (C + 2) + C + 1] * expf(ms - M);
    }
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = base[size_t(s) * (C + 2) + C];
            if (ms != -INFINITY) v += base[size_t(s) * (C + 2) + c] * expf(ms - M);
        }
        o[c] = __float2bfloat16_rn(v / L);
    }
}

}  // namespace

GB_API int gb_latent_decode_supported(int H, int C, int R, int q_dtype, int cache_dtype) {
    const size_t smem = size_t(H) * (C + R) * 4 + size_t(32) * ld_row_stride(C + R) * 2;
    return q_dtype == GB_BF16 && cache_dtype == GB_BF16 && H >= 1 && H <= LD_MAX_HEADS && C >= 2 && C <= LD_MAX_C && C % 2 == 0 &&
           (C + R) % 8 == 0 && smem <= 160 * 1024;
}

GB_API long long gb_latent_decode_scratch_floats(int T, int H, int C, int splits) {
    return (long long)T * H * splits * (C + 2);
}

// q: [T, H*(C+R)] bf16 (each head: q' of C entries, then the rotated part); out: [T, H*C] bf16; cache: the latent
// rows, [pages, 1, 64, C+R] bf16.  splits: parts of each token's keys (blocks of 32 keys are shared out evenly).
GB_API int gb_latent_decode(const void* q, long long ldq, void* out, long long ldo, int T, int H, int C, int R,
                            const int* seq_of, const int* pos, const int* table, int table_width, int ring_pages,
                            const void* cache, float scale, int splits, float* scratch, cudaStream_t stream) {
    GB_REQUIRE(gb_latent_decode_supported(H, C, R, GB_BF16, GB_BF16), "gb_latent_decode: sizes heads=%d kv_rank=%d rot_dim=%d are not supported", H, C, R);
    GB_REQUIRE(splits >= 1 && splits <= 65535 && scratch && table_width > 0 && ring_pages > 0, "gb_latent_decode: bad arguments");
    GB_REQUIRE((ldq % 2) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(scratch) & 7) == 0,
               "gb_latent_decode: misaligned operands");
    if (T == 0) return 0;
    LdParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.seq_of = seq_of; p.pos = pos; p.table = table;
    p.scratch = scratch; p.ldq = ldq; p.H = H; p.C = C; p.R = R; p.splits = splits; p.table_width = table_width;
    p.ring_pages = ring_pages; p.scale = scale;
    const size_t smem = size_t(H) * (C + R) * 4 + size_t(32) * ld_row_stride(C + R) * 2;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        if (cudaFuncSetAttribute(latent_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
            return gb_fail("gb_latent_decode: cannot get %zu bytes of shared memory", smem);
        configured = 160 * 1024;
    }
    latent_decode_kernel<<<dim3(T, splits), LD_THREADS, smem, stream>>>(p);
    GB_LAUNCH_OK("gb_latent_decode");
    latent_decode_merge_kernel<<<dim3(T, H), 128, 0, stream>>>(scratch, seq_of, (__nv_bfloat16*)out, ldo, H, C, splits);
    GB_LAUNCH_OK("gb_latent_decode (merge)");
    return 0;
}
