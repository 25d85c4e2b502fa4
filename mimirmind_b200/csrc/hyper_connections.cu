// Residual connections over several copies of the residual stream ("hyper-connections").
//
// Instead of one residual x a model keeps S streams x_1 .. x_S per token, fp32 [n, S, D].  A sublayer reads
//     u = sum_s a[s] x_s,          h = u / sqrt(mean(u^2) + eps) * w            (hc_read)
// and its result y (scaled per channel by an optional "layer scale" g) is written back to all streams at once,
//     x_t <- sum_s M[s][t] x_s + b[t] (g . y)                                   (hc_write)
// where every new stream is made from the old ones.  hc_write can also produce the next sublayer's h from the new
// streams in the same pass (its own a', w'), so a sublayer boundary is one launch: the streams are read and written once.
// S = 1 with a = M = b = 1 is the ordinary residual sum (with or without layer scale); summing the streams for the
// model's last norm is hc_read with a = 1 and a gather of the wanted rows.
//
// All arithmetic is fp32; a row's sums are taken in a fixed order (a thread over its own elements, then the block's
// tree), so a token's result never depends on what else is in the batch.
#include "common.cuh"

#define HC_MAX_STREAMS 8

__device__ __forceinline__ float hc_load(const void* p, int dtype, size_t i) {
    return dtype == MM_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void hc_store(void* p, int dtype, size_t i, float v) {
    if (dtype == MM_F32)
        reinterpret_cast<float*>(p)[i] = v;
    else
        reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// V consecutive numbers (V = 1 or 4; with 4 the index is a multiple of 4 and the row 16-byte aligned)
template <int V>
__device__ __forceinline__ void hc_load_v(const void* p, int dtype, size_t i, float* v) {
    if (V == 4) {
        if (dtype == MM_F32) {
            const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
            v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
        }
    } else {
        v[0] = hc_load(p, dtype, i);
    }
}
template <int V>
__device__ __forceinline__ void hc_store_v(void* p, int dtype, size_t i, const float* v) {
    if (V == 4) {
        if (dtype == MM_F32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
            uint2 raw;
            raw.x = *reinterpret_cast<uint32_t*>(&lo);
            raw.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
        }
    } else {
        hc_store(p, dtype, i, v[0]);
    }
}

// out[t, s, :] = src[t, :] for every stream s
__global__ void stream_copies_kernel(const float* __restrict__ src, float* __restrict__ out, int S, int D, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / D;
    const int d = (int)(i - t * D);
    const float v = src[i];
    for (int s = 0; s < S; ++s) out[(t * S + s) * D + d] = v;
}

MM_EXPORT int mm_stream_copies(const void* src, void* out, int n_tokens, int S, int D, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && S >= 1 && D >= 1, "stream copies: bad sizes");
    if (n_tokens == 0) return MM_OK;
    const long long total = (long long)n_tokens * D;
    mm_launch(stream_copies_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream, (const float*)src, (float*)out, S, D, total);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// One block per output row.  rows: the source row of output row i (null: i).  norm_w null: no norm, out = u.
// V: numbers per thread and turn (4 where the width is a multiple of 4).
template <int V>
__global__ void hc_read_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ a,
                               const void* __restrict__ norm_w, int w_dtype, float eps, void* __restrict__ out, int out_dtype, int S, int D) {
    extern __shared__ __align__(16) float u_row[];      // [D]
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const float* xr = x + r * S * D;
    float w_in[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) w_in[s] = s < S ? a[s] : 0.0f;
    float sq = 0.0f;
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float u[V];
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = 0.0f;
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) {
            if (s < S) {
                float v[V];
                hc_load_v<V>(xr, MM_F32, (size_t)s * D + d, v);
#pragma unroll
                for (int e = 0; e < V; ++e) u[e] = fmaf(w_in[s], v[e], u[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            u_row[d + e] = u[e];
            sq = fmaf(u[e], u[e], sq);
        }
    }
    float inv = 1.0f;
    if (norm_w != nullptr) inv = rsqrtf(block_sum(sq, scratch) / (float)D + eps);
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float u[V], w[V];                               // u_row[d ..] was written by this thread
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = u_row[d + e];
        if (norm_w != nullptr) {
            hc_load_v<V>(norm_w, w_dtype, d, w);
#pragma unroll
            for (int e = 0; e < V; ++e) u[e] = u[e] * inv * w[e];
        }
        hc_store_v<V>(out, out_dtype, (size_t)i * D + d, u);
    }
}

// One block per token: the streams in place, and (a2 not null) the next sublayer's input from the new streams.
template <int V>
__global__ void hc_write_kernel(float* __restrict__ x, const void* __restrict__ y, int y_dtype, const float* __restrict__ g,
                                const float* __restrict__ M, const float* __restrict__ b, const float* __restrict__ a2,
                                const void* __restrict__ norm_w, int w_dtype, float eps, void* __restrict__ out, int out_dtype, int S, int D) {
    extern __shared__ __align__(16) float u_row[];      // [D]
    __shared__ float scratch[32];
    __shared__ float sM[HC_MAX_STREAMS * HC_MAX_STREAMS], sb[HC_MAX_STREAMS], sa[HC_MAX_STREAMS];
    const int t = blockIdx.x;
    if (threadIdx.x < S * S) sM[threadIdx.x] = M[threadIdx.x];
    if (threadIdx.x < S) {
        sb[threadIdx.x] = b[threadIdx.x];
        sa[threadIdx.x] = a2 ? a2[threadIdx.x] : 0.0f;
    }
    __syncthreads();
    float* xr = x + (size_t)t * S * D;
    float sq = 0.0f;
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float old[HC_MAX_STREAMS][V];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) hc_load_v<V>(xr, MM_F32, (size_t)s * D + d, old[s]);
        float branch[V];
        hc_load_v<V>(y, y_dtype, (size_t)t * D + d, branch);
        if (g != nullptr) {
            float gv[V];
            hc_load_v<V>(g, MM_F32, d, gv);
#pragma unroll
            for (int e = 0; e < V; ++e) branch[e] *= gv[e];
        }
        float u[V];
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = 0.0f;
#pragma unroll
        for (int to = 0; to < HC_MAX_STREAMS; ++to) {
            if (to < S) {
                float v[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float acc = 0.0f;
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; ++s)
                        if (s < S) acc = fmaf(sM[s * S + to], old[s][e], acc);
                    v[e] = fmaf(sb[to], branch[e], acc);
                    u[e] = fmaf(sa[to], v[e], u[e]);
                }
                hc_store_v<V>(xr, MM_F32, (size_t)to * D + d, v);
            }
        }
        if (a2 != nullptr) {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                u_row[d + e] = u[e];
                sq = fmaf(u[e], u[e], sq);
            }
        }
    }
    if (a2 == nullptr) return;
    float inv = 1.0f;
    if (norm_w != nullptr) inv = rsqrtf(block_sum(sq, scratch) / (float)D + eps);
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float u[V], w[V];
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = u_row[d + e];
        if (norm_w != nullptr) {
            hc_load_v<V>(norm_w, w_dtype, d, w);
#pragma unroll
            for (int e = 0; e < V; ++e) u[e] = u[e] * inv * w[e];
        }
        hc_store_v<V>(out, out_dtype, (size_t)t * D + d, u);
    }
}

static inline int hc_threads(int D) { return D >= 4096 ? 512 : (D >= 1024 ? 256 : 128); }
// four numbers per thread where every row starts on a 16-byte boundary
static inline bool hc_vec(int D, const void* p0, const void* p1, const void* p2, const void* p3) {
    return D % 4 == 0 && (((uintptr_t)p0 | (uintptr_t)p1 | (uintptr_t)p2 | (uintptr_t)p3) & 15) == 0;
}

MM_EXPORT int mm_hc_read(const void* x, const void* rows, const void* a, const void* norm_w, int w_dtype, float eps, void* out, int out_dtype,
                         int n_out, int S, int D, void* stream) {
    MM_REQUIRE(n_out >= 0 && S >= 1 && S <= HC_MAX_STREAMS && D >= 1, "stream read: 1 to 8 streams");
    MM_REQUIRE((size_t)D * sizeof(float) <= 160 * 1024, "stream read: the width does not fit a block's shared memory");
    if (n_out == 0) return MM_OK;
    const size_t smem = (size_t)D * sizeof(float);
    const bool vec = hc_vec(D, x, norm_w, out, nullptr);
    auto kernel = vec ? hc_read_kernel<4> : hc_read_kernel<1>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        mm_set_last_error("stream read: shared memory for a row could not be set");
        return MM_ERR_UNSUPPORTED;
    }
    mm_launch(kernel, dim3(n_out), dim3(hc_threads(D)), smem, (cudaStream_t)stream, (const float*)x, (const int32_t*)rows, (const float*)a,
              norm_w, w_dtype, eps, out, out_dtype, S, D);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_hc_write(void* x, const void* y, int y_dtype, const void* g, const void* M, const void* b, const void* a2, const void* norm_w,
                          int w_dtype, float eps, void* out, int out_dtype, int n_tokens, int S, int D, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && S >= 1 && S <= HC_MAX_STREAMS && D >= 1, "stream write: 1 to 8 streams");
    MM_REQUIRE((size_t)D * sizeof(float) <= 160 * 1024, "stream write: the width does not fit a block's shared memory");
    MM_REQUIRE(a2 == nullptr || out != nullptr, "stream write: the next input needs a place");
    if (n_tokens == 0) return MM_OK;
    const size_t smem = a2 ? (size_t)D * sizeof(float) : 0;
    const bool vec = hc_vec(D, x, y, g, norm_w) && hc_vec(D, out, nullptr, nullptr, nullptr);
    auto kernel = vec ? hc_write_kernel<4> : hc_write_kernel<1>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        mm_set_last_error("stream write: shared memory for a row could not be set");
        return MM_ERR_UNSUPPORTED;
    }
    mm_launch(kernel, dim3(n_tokens), dim3(hc_threads(D)), smem, (cudaStream_t)stream, (float*)x, y, y_dtype, (const float*)g,
              (const float*)M, (const float*)b, (const float*)a2, norm_w, w_dtype, eps, out, out_dtype, S, D);
    MM_CHECK_LAUNCH();
    return MM_OK;
}
