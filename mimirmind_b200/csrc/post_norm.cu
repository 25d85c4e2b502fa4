// The norm after the sum, the gated activation of a two-matrix feed-forward as a pass of its own, and the rounding of
// the residual stream to the activation dtype.
//
//   post norm:   y = alpha x + ca a + cb b;   x <- y / sqrt(mean(y^2) + eps) * w      (x: the fp32 residual stream, in place)
//
// a and b are a layer's branch outputs (either may be absent); the new stream is also written in the activation dtype,
// which is what the next sublayer's products read.
#include "common.cuh"

template <typename TB, typename TO>
__global__ void __launch_bounds__(256) post_norm_kernel(float* __restrict__ x, const TB* __restrict__ a, const TB* __restrict__ b,
                                                        const float* __restrict__ w, TO* __restrict__ out, int D, float alpha, float ca, float cb,
                                                        float eps) {
    extern __shared__ float pn_row[];
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    float* xr = x + t * D;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float y = alpha * xr[i];
        if (a) y = fmaf(ca, to_f32<TB>(a[t * D + i]), y);
        if (b) y = fmaf(cb, to_f32<TB>(b[t * D + i]), y);
        pn_row[i] = y;
        ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float y = pn_row[i] * r * w[i];
        xr[i] = y;
        if (out) out[t * D + i] = from_f32<TO>(y);
    }
}

// Eight numbers at a time (16-byte words of bfloat16, two of fp32): the same arithmetic in the same order per element.
__device__ __forceinline__ void pn_load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void pn_load8(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void pn_store8(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void pn_store8(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

template <typename TB, typename TO>
__global__ void __launch_bounds__(256) post_norm8_kernel(float* __restrict__ x, const TB* __restrict__ a, const TB* __restrict__ b,
                                                         const float* __restrict__ w, TO* __restrict__ out, int D, float alpha, float ca, float cb,
                                                         float eps) {
    extern __shared__ __align__(16) float pn_row[];
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    float* xr = x + t * D;
    float ss = 0.0f;
    for (int i = threadIdx.x * 8; i < D; i += blockDim.x * 8) {
        float y[8], u[8];
        pn_load8(xr + i, y);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] *= alpha;
        if (a) {
            pn_load8(a + t * D + i, u);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = fmaf(ca, u[e], y[e]);
        }
        if (b) {
            pn_load8(b + t * D + i, u);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = fmaf(cb, u[e], y[e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(y[e], y[e], ss);
        pn_store8(pn_row + i, y);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x * 8; i < D; i += blockDim.x * 8) {
        float y[8], wv[8];
        pn_load8(pn_row + i, y);
        pn_load8(w + i, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = y[e] * r * wv[e];
        pn_store8(xr + i, y);
        if (out) pn_store8(out + t * D + i, y);
    }
}

// x [n, D] fp32 residual (in place); a, b [n, D] of dtype `b_dtype` or null; w fp32 [D]; out [n, D] of `out_dtype` or null.
MM_EXPORT int mm_post_norm(void* x, const void* a, const void* b, int b_dtype, const void* w, void* out, int out_dtype, int n, int D, float alpha,
                           float ca, float cb, float eps, void* stream) {
    MM_REQUIRE(n >= 0 && D > 0 && D <= 51200, "post norm: widths above 51200 are not supported");
    MM_REQUIRE(x != nullptr && w != nullptr, "post norm: the stream and the weight are needed");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)D * sizeof(float);
    typedef __nv_bfloat16 bf;
    const bool by8 = D % 8 == 0 && (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
#define PN_LAUNCH(TB, TO)                                                                                                         \
    do {                                                                                                                          \
        auto kernel = by8 ? post_norm8_kernel<TB, TO> : post_norm_kernel<TB, TO>;                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
        mm_launch(kernel, dim3(n), dim3(256), smem, s, (float*)x, (const TB*)a, (const TB*)b, (const float*)w, (TO*)out, D, alpha, ca, cb, eps); \
    } while (0)
    if (b_dtype == MM_F32 && out_dtype == MM_F32) PN_LAUNCH(float, float);
    else if (b_dtype == MM_BF16 && out_dtype == MM_BF16) PN_LAUNCH(bf, bf);
    else if (b_dtype == MM_F32 && out_dtype == MM_BF16) PN_LAUNCH(float, bf);
    else MM_REQUIRE(false, "post norm: this combination of dtypes is not built");
#undef PN_LAUNCH
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// out [n, F] = glu_act(gu[:, :F] * s, gu[:, F:] * s): the gate's columns, then the up columns; row_scale fp32 [n] or null.
template <typename TI, typename TO>
__global__ void glu_rows_kernel(const TI* __restrict__ gu, long long ld, TO* __restrict__ out, long long total, int F, int act, float limit,
                                const float* __restrict__ row_scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / F;
    const int c = (int)(i - t * F);
    const TI* row = gu + t * ld;
    out[i] = from_f32<TO>(glu_act<false>(to_f32<TI>(row[c]), to_f32<TI>(row[F + c]), act, limit, row_scale ? row_scale[t] : 1.0f));
}

MM_EXPORT int mm_glu_rows(const void* gu, int in_dtype, long long ld, void* out, int out_dtype, int n, int F, int act, float limit,
                          const void* row_scale, void* stream) {
    MM_REQUIRE(n >= 0 && F > 0 && ld >= 2 * (long long)F, "gated activation: bad sizes");
    MM_REQUIRE(act == MM_GLU_SILU || act == MM_GLU_CLAMPED, "gated activation: unknown kind");
    if (n == 0) return MM_OK;
    const long long total = (long long)n * F;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const dim3 grid(ceil_div(total, 256));
    if (in_dtype == MM_F32 && out_dtype == MM_F32)
        mm_launch(glu_rows_kernel<float, float>, grid, dim3(256), 0, s, (const float*)gu, ld, (float*)out, total, F, act, limit, (const float*)row_scale);
    else if (in_dtype == MM_BF16 && out_dtype == MM_BF16)
        mm_launch(glu_rows_kernel<bf, bf>, grid, dim3(256), 0, s, (const bf*)gu, ld, (bf*)out, total, F, act, limit, (const float*)row_scale);
    else if (in_dtype == MM_F32 && out_dtype == MM_BF16)
        mm_launch(glu_rows_kernel<float, bf>, grid, dim3(256), 0, s, (const float*)gu, ld, (bf*)out, total, F, act, limit, (const float*)row_scale);
    else
        MM_REQUIRE(false, "gated activation: this combination of dtypes is not built");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// fp32 rows to the activation dtype
template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_f32<TO>(x[i]);
}

MM_EXPORT int mm_cast_rows(const void* x, void* out, int out_dtype, long long total, void* stream) {
    MM_REQUIRE(total >= 0, "cast: bad size");
    if (total == 0) return MM_OK;
    const dim3 grid(ceil_div(total, 256));
    if (out_dtype == MM_F32)
        mm_launch(cast_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, (const float*)x, (float*)out, total);
    else if (out_dtype == MM_BF16)
        mm_launch(cast_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, (const float*)x, (__nv_bfloat16*)out, total);
    else
        MM_REQUIRE(false, "cast: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// out = ca a + cb b, element by element (two branches as one where nothing downstream adds them itself)
template <typename T>
__global__ void scaled_sum2_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long total, float ca, float cb) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_f32<T>(fmaf(cb, to_f32<T>(b[i]), ca * to_f32<T>(a[i])));
}

MM_EXPORT int mm_scaled_sum2(const void* a, const void* b, void* out, int dtype, long long total, float ca, float cb, void* stream) {
    MM_REQUIRE(total >= 0, "scaled sum: bad size");
    if (total == 0) return MM_OK;
    const dim3 grid(ceil_div(total, 256));
    if (dtype == MM_F32)
        mm_launch(scaled_sum2_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, (const float*)a, (const float*)b, (float*)out, total, ca, cb);
    else if (dtype == MM_BF16)
        mm_launch(scaled_sum2_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                  (__nv_bfloat16*)out, total, ca, cb);
    else
        MM_REQUIRE(false, "scaled sum: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
