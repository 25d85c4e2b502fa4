// Steps around an attention kernel that several kinds of attention share, all fp32 arithmetic:
//
//   * rope_half_table: (cos, sin) per (token, frequency) of position * frequency, the frequency given as the sum of two
//     floats (made in float64 on the host) and the product's rounding error carried into the result, so that the angle
//     is as good as a float64 product although every operation is a 32-bit one;
//   * qkv_split_post: fp32 rows of a projection (after their convolution, if any) cut into queries, keys and values; the
//     queries go to a dense buffer, keys and values into their pages, in the run's dtype;
//   * latent_prep: the step between the projections of a latent attention and its kernel: the latent vector is RMS-normed,
//     the shared rotated key part and every head's rotated query part are turned (pairs i, i + dims/2), and latent and
//     rotated key are written side by side into one per-token cache array;
//   * head_matmul: out[t, h, :] = in[t, h, :] . M[h] with a matrix per head (absorbing the key or value up-projection
//     of a latent attention into the query or the output), fp32 FMAs over eight runs of k, summed in order;
//   * head_finish: what happens to each head's attention output before the output projection: the difference of two
//     maps (a1 - lambda a2), a division by the head's root mean square, a constant factor, a sigmoid gate per (token, head).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------------------
__global__ void rope_half_table_kernel(const int32_t* __restrict__ positions, const float* __restrict__ f_hi, const float* __restrict__ f_lo,
                                       float2* __restrict__ table, int n_tokens, int half) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * half) return;
    const int t = (int)(i / half), p = (int)(i - (long long)t * half);
    const float pos = (float)positions[t];
    const float a = pos * f_hi[p];
    const float rest = fmaf(pos, f_lo[p], fmaf(pos, f_hi[p], -a));     // what the rounded product left out, and the low word's share
    float sn, cs;
    sincosf(a, &sn, &cs);
    table[i] = make_float2(fmaf(-rest, sn, cs), fmaf(rest, cs, sn));
}

MM_EXPORT int mm_rope_half_table(const void* positions, const void* f_hi, const void* f_lo, void* table, int n_tokens, int half, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && half > 0, "rotation table: bad sizes");
    if (n_tokens == 0) return MM_OK;
    const long long total = (long long)n_tokens * half;
    mm_launch(rope_half_table_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream, (const int32_t*)positions,
              (const float*)f_hi, (const float*)f_lo, (float2*)table, n_tokens, half);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// rows [n, ld] fp32: Hq * dk query numbers at q_off, Gk * dk key numbers at k_off, Gv * dv value numbers at v_off.
// slots[t] = page * page_size + place (negative: nothing to cache); pools [pages, heads, page_size, size].
template <typename T>
__global__ void qkv_split_post_kernel(const float* __restrict__ rows, int ld, int q_off, int k_off, int v_off, T* __restrict__ q_out,
                                      T* __restrict__ k_pages, T* __restrict__ v_pages, const int32_t* __restrict__ slots, int page_size,
                                      int Hq, int Gk, int dk, int Gv, int dv) {
    const int t = blockIdx.x;
    const float* row = rows + (size_t)t * ld;
    const int nq = Hq * dk;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[(size_t)t * nq + i] = from_f32<T>(row[q_off + i]);
    if (k_pages == nullptr) return;
    const long long slot = slots[t];
    if (slot < 0) return;
    const long long page = slot / page_size;
    const int place = (int)(slot - page * page_size);
    for (int i = threadIdx.x; i < Gk * dk; i += blockDim.x) {
        const int g = i / dk, e = i - g * dk;
        k_pages[(((size_t)page * Gk + g) * page_size + place) * dk + e] = from_f32<T>(row[k_off + i]);
    }
    for (int i = threadIdx.x; i < Gv * dv; i += blockDim.x) {
        const int g = i / dv, e = i - g * dv;
        v_pages[(((size_t)page * Gv + g) * page_size + place) * dv + e] = from_f32<T>(row[v_off + i]);
    }
}

MM_EXPORT int mm_qkv_split_post(const void* rows, int ld, int q_off, int k_off, int v_off, void* q_out, void* k_pages, void* v_pages, int dtype,
                                const void* slots, int page_size, int n_tokens, int Hq, int Gk, int dk, int Gv, int dv, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && Hq > 0 && Gk > 0 && Gv > 0 && dk > 0 && dv > 0, "qkv split: bad sizes");
    MM_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && ld >= q_off + Hq * dk && ld >= k_off + Gk * dk && ld >= v_off + Gv * dv,
               "qkv split: the rows are narrower than what is cut out of them");
    MM_REQUIRE(k_pages == nullptr || (v_pages != nullptr && slots != nullptr && page_size > 0), "qkv split: bad page geometry");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MM_F32)
        mm_launch(qkv_split_post_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (const float*)rows, ld, q_off, k_off, v_off, (float*)q_out,
                  (float*)k_pages, (float*)v_pages, (const int32_t*)slots, page_size, Hq, Gk, dk, Gv, dv);
    else if (dtype == MM_BF16)
        mm_launch(qkv_split_post_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (const float*)rows, ld, q_off, k_off, v_off,
                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (const int32_t*)slots, page_size, Hq, Gk, dk, Gv, dv);
    else
        MM_REQUIRE(false, "qkv split: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// rows [n, ld] fp32: H heads of (dk plain, dr rotated) query numbers at q_off; the latent's `rank` numbers and the shared
// key part's dr numbers at c_off.  rot [n, rot_dims / 2] (cos, sin); dimensions from rot_dims on of a rotated part pass.
// q_plain [n, H, dk]; q_full [n, H, rank + dr] gets each head's rotated part at [rank, rank + dr); pages
// [pages, 1, page_size, rank + dr] get (normed latent, rotated key part).
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ rows, int ld, int q_off, int c_off, const void* __restrict__ norm_w, int w_dtype,
                                   float eps, const float2* __restrict__ rot, int rot_dims, T* __restrict__ q_plain, T* __restrict__ q_full,
                                   T* __restrict__ pages, const int32_t* __restrict__ slots, int page_size, int H, int dk, int dr, int rank) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = rows + (size_t)t * ld;
    const int half = rot_dims / 2;
    const float2* rt = rot + (size_t)t * half;
    const int wide = rank + dr;
    // queries: plain parts to their buffer, rotated parts into the joined query
    for (int i = threadIdx.x; i < H * dk; i += blockDim.x) {
        const int h = i / dk, e = i - h * dk;
        q_plain[(size_t)t * H * dk + i] = from_f32<T>(row[q_off + h * (dk + dr) + e]);
    }
    for (int i = threadIdx.x; i < H * dr; i += blockDim.x) {
        const int h = i / dr, e = i - h * dr;
        const float* part = row + q_off + h * (dk + dr) + dk;
        float v = part[e];
        if (e < half) {
            v = part[e] * rt[e].x - part[e + half] * rt[e].y;
        } else if (e < rot_dims) {
            v = part[e] * rt[e - half].x + part[e - half] * rt[e - half].y;
        }
        q_full[((size_t)t * H + h) * wide + rank + e] = from_f32<T>(v);
    }
    // the latent: divided by its root mean square, times its weight
    float sq = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) sq = fmaf(row[c_off + i], row[c_off + i], sq);
    const float inv = rsqrtf(block_sum(sq, scratch) / (float)rank + eps);
    if (pages == nullptr) return;
    const long long slot = slots[t];
    if (slot < 0) return;
    T* dst = pages + (size_t)slot * wide;          // one head: [page][place] is [slot]
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float w = w_dtype == MM_F32 ? reinterpret_cast<const float*>(norm_w)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(norm_w)[i]);
        dst[i] = from_f32<T>(row[c_off + i] * inv * w);
    }
    const float* part = row + c_off + rank;
    for (int e = threadIdx.x; e < dr; e += blockDim.x) {
        float v = part[e];
        if (e < half) {
            v = part[e] * rt[e].x - part[e + half] * rt[e].y;
        } else if (e < rot_dims) {
            v = part[e] * rt[e - half].x + part[e - half] * rt[e - half].y;
        }
        dst[rank + e] = from_f32<T>(v);
    }
}

MM_EXPORT int mm_latent_prep(const void* rows, int ld, int q_off, int c_off, const void* norm_w, int w_dtype, float eps, const void* rot,
                             int rot_dims, void* q_plain, void* q_full, void* pages, int dtype, const void* slots, int page_size, int n_tokens,
                             int H, int dk, int dr, int rank, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && dk > 0 && dr >= 0 && rank > 0, "latent prep: bad sizes");
    MM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr && (rot_dims == 0 || rot != nullptr), "latent prep: the rotated dimensions are even and at most the rotated part");
    MM_REQUIRE(q_off >= 0 && c_off >= 0 && ld >= q_off + H * (dk + dr) && ld >= c_off + rank + dr, "latent prep: the rows are narrower than what is cut out of them");
    MM_REQUIRE(pages == nullptr || (slots != nullptr && page_size > 0), "latent prep: bad page geometry");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MM_F32)
        mm_launch(latent_prep_kernel<float>, dim3(n_tokens), dim3(256), 0, s, (const float*)rows, ld, q_off, c_off, norm_w, w_dtype, eps,
                  (const float2*)rot, rot_dims, (float*)q_plain, (float*)q_full, (float*)pages, (const int32_t*)slots, page_size, H, dk, dr, rank);
    else if (dtype == MM_BF16)
        mm_launch(latent_prep_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, s, (const float*)rows, ld, q_off, c_off, norm_w, w_dtype, eps,
                  (const float2*)rot, rot_dims, (__nv_bfloat16*)q_plain, (__nv_bfloat16*)q_full, (__nv_bfloat16*)pages, (const int32_t*)slots,
                  page_size, H, dk, dr, rank);
    else
        MM_REQUIRE(false, "latent prep: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// out[t, h, j] = sum_k in[t, h, k] M[h, k, j]; in: token stride in_ld, head stride in_hs; out likewise.  Eight tokens
// of one head per block share each matrix element; a thread owns one output column.
#define HM_TOKENS 8
#define HM_COLS 64
#define HM_SLICES 8
// A block of HM_COLS x HM_SLICES threads makes HM_TOKENS tokens x HM_COLS columns of one head: slice y sums its run of k
// (ascending), then thread (x, y) adds the slices' sums of token y in slice order.  The cut of k depends on K alone, so
// a token's result never depends on the batch.
template <typename T>
__global__ void __launch_bounds__(HM_COLS * HM_SLICES) head_matmul_kernel(
    const T* __restrict__ in, long long in_ld, int in_hs, const T* __restrict__ M, T* __restrict__ out, long long out_ld, int out_hs,
    int n_tokens, int K, int N) {
    extern __shared__ float in_s[];   // [HM_TOKENS][K]
    __shared__ float part[HM_SLICES][HM_TOKENS][HM_COLS];
    const int h = blockIdx.y, t0 = blockIdx.z * HM_TOKENS;
    const int x = threadIdx.x, y = threadIdx.y, tid = y * HM_COLS + x;
    const int j = blockIdx.x * HM_COLS + x;
    for (int i = tid; i < HM_TOKENS * K; i += HM_COLS * HM_SLICES) {
        const int tt = i / K, k = i - tt * K;
        in_s[i] = (t0 + tt < n_tokens) ? to_f32<T>(in[(size_t)(t0 + tt) * in_ld + (size_t)h * in_hs + k]) : 0.0f;
    }
    __syncthreads();
    float acc[HM_TOKENS];
#pragma unroll
    for (int tt = 0; tt < HM_TOKENS; ++tt) acc[tt] = 0.0f;
    const int per = (K + HM_SLICES - 1) / HM_SLICES;
    const int k_lo = y * per, k_hi = min(K, k_lo + per);
    if (j < N) {
        const T* Mh = M + (size_t)h * K * N + j;
#pragma unroll 4
        for (int k = k_lo; k < k_hi; ++k) {
            const float w = to_f32<T>(Mh[(size_t)k * N]);
#pragma unroll
            for (int tt = 0; tt < HM_TOKENS; ++tt) acc[tt] = fmaf(in_s[tt * K + k], w, acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < HM_TOKENS; ++tt) part[y][tt][x] = acc[tt];
    __syncthreads();
    if (j >= N || t0 + y >= n_tokens) return;
    float sum = 0.0f;
#pragma unroll
    for (int sl = 0; sl < HM_SLICES; ++sl) sum += part[sl][y][x];
    out[(size_t)(t0 + y) * out_ld + (size_t)h * out_hs + j] = from_f32<T>(sum);
}

MM_EXPORT int mm_head_matmul(const void* in, long long in_ld, int in_hs, const void* M, void* out, long long out_ld, int out_hs, int dtype,
                             int n_tokens, int H, int K, int N, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && K > 0 && N > 0 && H <= 65535, "head product: bad sizes");
    MM_REQUIRE((size_t)HM_TOKENS * K * sizeof(float) <= 96 * 1024, "head product: the depth does not fit a block's shared memory");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)HM_TOKENS * K * sizeof(float);
    const dim3 grid(ceil_div(N, HM_COLS), H, ceil_div(n_tokens, HM_TOKENS)), block(HM_COLS, HM_SLICES);
    if (grid.z > 65535) {
        mm_set_last_error("head product: too many tokens for one launch");
        return MM_ERR_BAD_ARG;
    }
    if (dtype == MM_F32) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(head_matmul_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mm_launch(head_matmul_kernel<float>, grid, block, smem, s, (const float*)in, in_ld, in_hs, (const float*)M, (float*)out, out_ld, out_hs,
                  n_tokens, K, N);
    } else if (dtype == MM_BF16) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(head_matmul_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mm_launch(head_matmul_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)in, in_ld, in_hs, (const __nv_bfloat16*)M,
                  (__nv_bfloat16*)out, out_ld, out_hs, n_tokens, K, N);
    } else {
        MM_REQUIRE(false, "head product: dtype must be float32 or bfloat16");
    }
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// att [n, heads_in, dv]; with pair > 0 head h's second map is head h + pair of the same token.  One warp per (token, head):
//   o = a1 - lambda a2;  normalize: o <- o / sqrt(mean(o^2) + eps);  o <- o * post * sigmoid(gate[t * ldg + h])
template <typename T, typename TO = T>
__global__ void head_finish_kernel(const T* __restrict__ att, int heads_in, int pair, float lambda, int normalize, float eps, float post,
                                   const float* __restrict__ gate, int ldg, TO* __restrict__ out, int n_tokens, int H, int dv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const T* a1 = att + ((size_t)t * heads_in + h) * dv;
    const T* a2 = a1 + (size_t)pair * dv;
    float factor = post;
    if (normalize) {
        float sq = 0.0f;
        for (int d = lane; d < dv; d += 32) {
            const float o = pair ? fmaf(-lambda, to_f32<T>(a2[d]), to_f32<T>(a1[d])) : to_f32<T>(a1[d]);
            sq = fmaf(o, o, sq);
        }
        factor *= rsqrtf(warp_sum(sq) / (float)dv + eps);
    }
    if (gate != nullptr) factor *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
    TO* o_row = out + ((size_t)t * H + h) * dv;
    for (int d = lane; d < dv; d += 32) {
        const float o = pair ? fmaf(-lambda, to_f32<T>(a2[d]), to_f32<T>(a1[d])) : to_f32<T>(a1[d]);
        o_row[d] = from_f32<TO>(o * factor);
    }
}

MM_EXPORT int mm_head_finish(const void* att, int heads_in, int pair, float lambda, int normalize, float eps, float post, const void* gate, int ldg,
                             void* out, int dtype, int out_dtype, int n_tokens, int H, int dv, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && dv > 0 && pair >= 0 && heads_in >= H + pair, "head finish: bad sizes");
    MM_REQUIRE(gate == nullptr || ldg >= H, "head finish: one gate per head");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)n_tokens * H;
    const int blocks = ceil_div(items, 4);
    MM_REQUIRE(out_dtype == dtype || dtype == MM_F32, "head finish: only an fp32 input can be given out in another type");
    if (dtype == MM_F32 && out_dtype == MM_BF16)
        mm_launch(head_finish_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(128), 0, s, (const float*)att, heads_in, pair, lambda, normalize,
                  eps, post, (const float*)gate, ldg, (__nv_bfloat16*)out, n_tokens, H, dv);
    else if (dtype == MM_F32)
        mm_launch(head_finish_kernel<float>, dim3(blocks), dim3(128), 0, s, (const float*)att, heads_in, pair, lambda, normalize, eps, post,
                  (const float*)gate, ldg, (float*)out, n_tokens, H, dv);
    else if (dtype == MM_BF16)
        mm_launch(head_finish_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, s, (const __nv_bfloat16*)att, heads_in, pair, lambda, normalize,
                  eps, post, (const float*)gate, ldg, (__nv_bfloat16*)out, n_tokens, H, dv);
    else
        MM_REQUIRE(false, "head finish: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
