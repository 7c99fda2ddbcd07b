// The norm of a sublayer's result on its way into the residual stream, for layers that norm what a sublayer
// gives and not what it reads:
//   x[t,:] += y[t,:] / sqrt(mean(y[t,:]^2) + eps) * w        (32-bit; x is the residual stream)
//   xb[t,:] = bfloat16(x[t,:])                               (optional: the rows that the next sublayer's products read)
// y null: only the copy is made.  One block per token; the row of y is read twice (the second time from cache).
#include "common.cuh"

__global__ void __launch_bounds__(256) norm_residual_add_kernel(float* __restrict__ x, const void* __restrict__ y, int y_dtype,
                                                                long long ldy, int E, const void* __restrict__ w, int w_dtype,
                                                                float eps, __nv_bfloat16* __restrict__ xb) {
    __shared__ float red[8];
    const int t = blockIdx.x;
    float* xr = x + size_t(t) * E;
    float f = 0.f;
    if (y) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float v = gb_load(y, y_dtype, size_t(t) * ldy + i);
            ss = fmaf(v, v, ss);
        }
        ss = gb_warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int k = 0; k < (blockDim.x >> 5); ++k) tot += red[k];
        f = 1.f / sqrtf(tot / float(E) + eps);
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float v = xr[i];
        if (y) {
            v += gb_load(y, y_dtype, size_t(t) * ldy + i) * f * gb_load(w, w_dtype, i);
            xr[i] = v;
        }
        if (xb) xb[size_t(t) * E + i] = __float2bfloat16_rn(v);
    }
}

// x float32 [T, E] contiguous; y [T, E] with rows ldy apart (or null); w [E]; xb bfloat16 [T, E] contiguous (or null).
GB_API int gb_norm_residual_add(float* x, const void* y, int y_dtype, long long ldy, int T, int E, const void* w, int w_dtype,
                                float eps, void* xb, cudaStream_t stream) {
    GB_REQUIRE(!y || (gb_is_dtype(y_dtype) && gb_is_dtype(w_dtype) && w && eps > 0.f), "gb_norm_residual_add: bad arguments");
    GB_REQUIRE(T >= 0 && E > 0 && (y || xb), "gb_norm_residual_add: bad sizes T=%d E=%d", T, E);
    if (T == 0) return 0;
    norm_residual_add_kernel<<<T, 256, 0, stream>>>(x, y, y_dtype, ldy, E, w, w_dtype, eps, (__nv_bfloat16*)xb);
    GB_LAUNCH_OK("gb_norm_residual_add");
    return 0;
}
