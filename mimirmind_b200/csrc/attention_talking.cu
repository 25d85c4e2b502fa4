// Attention whose heads talk to one another before the softmax, with a learned sink per head.
//
//   q [n, H, dk], keys [.., G, dk], values [.., G, dv]; query head g reads kv head g / (H / G);
//   r_g(i, j) = (q_g(i) . k(j)) * scale for every head g;   s_h(i, j) = sum_g T[h][g] r_g(i, j)   (T [H, H], row h
//   makes head h's score);   a query at absolute position a sees keys max(0, a + 1 - W) .. a (W = 0: all);
//   p_h(j) = exp(s_h(j)) / (exp(sink_h) + sum_i exp(s_h(i)))  (sink null: plain softmax);   o_h = sum_j p_h(j) v(j).
//
// Because every head's score needs the raw scores of all heads at the same (query, key) pair, the unit of work is a
// query token with all its heads, not a (token, head) pair.
//
// This file holds (1) the step between the q/k/v projection (and its short convolution) and attention: RMS norm per
// head of q and k with one weight for all heads, rotation of the half-split pairs (i, i + dims/2) of the first `dims`
// numbers of every q and k head, values divided by their root mean square per head, and the write of keys and values
// into their pages; (2) the fp32-arithmetic attention kernel for any sizes, one block per query token (and key split),
// its keys in chunks of 32 aligned to absolute position so that a token's result depends on its own position and keys
// only.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------------------
// norm per head + rotation + unit values + cache write
// ---------------------------------------------------------------------------------------------------------------
// rows [n, ld] fp32: q at q_off (H heads of dk), k at k_off (G heads of dk), v at v_off (G heads of dv).  One warp
// per head vector.  q_norm, k_norm: fp32 [dk] or null (no norm); rot [n, rot_dims / 2] (cos, sin) or null; v_unit:
// values are divided by sqrt(mean(v^2) + eps).  slots[t] = page * page_size + place (negative: nothing to write).
template <typename T>
__global__ void __launch_bounds__(256) talking_prep_kernel(const float* __restrict__ rows, int ld, int q_off, int k_off, int v_off,
                                                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                                           const float2* __restrict__ rot, int rot_dims, int v_unit, T* __restrict__ q_out,
                                                           T* __restrict__ k_pages, T* __restrict__ v_pages, const int32_t* __restrict__ slots,
                                                           int page_size, int H, int G, int dk, int dv) {
    extern __shared__ float prep_vec[];          // one vector of max(dk, dv) per warp
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float* row = rows + (size_t)t * ld;
    const long long slot = (k_pages != nullptr) ? (long long)slots[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int place = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const int half = rot_dims / 2;
    const int wide = dk > dv ? dk : dv;
    float* sv = prep_vec + (size_t)warp * wide;
    for (int vec = warp; vec < H + 2 * G; vec += warps) {
        const bool is_q = vec < H, is_k = !is_q && vec < H + G;
        const int head = is_q ? vec : (is_k ? vec - H : vec - H - G);
        const int d = (is_q || is_k) ? dk : dv;
        const float* p = row + (is_q ? q_off + head * dk : (is_k ? k_off + head * dk : v_off + head * dv));
        const float* w = is_q ? q_norm : (is_k ? k_norm : nullptr);
        const bool normed = (is_q || is_k) ? (w != nullptr) : (v_unit != 0);
        float ss = 0.0f;
        for (int i = lane; i < d; i += 32) {
            const float x = p[i];
            sv[i] = x;
            ss = fmaf(x, x, ss);
        }
        ss = warp_sum(ss);
        __syncwarp();
        if (normed) {
            const float r = 1.0f / sqrtf(ss / (float)d + eps);
            for (int i = lane; i < d; i += 32) sv[i] = sv[i] * r * (w ? w[i] : 1.0f);
            __syncwarp();
        }
        if ((is_q || is_k) && rot_dims) {
            const float2* cs = rot + (size_t)t * half;
            for (int i = lane; i < half; i += 32) {
                const float a = sv[i], b = sv[i + half];
                sv[i] = a * cs[i].x - b * cs[i].y;
                sv[i + half] = b * cs[i].x + a * cs[i].y;
            }
            __syncwarp();
        }
        T* dst = nullptr;
        if (is_q) dst = q_out + ((size_t)t * H + head) * dk;
        else if (page >= 0) dst = is_k ? k_pages + (((size_t)page * G + head) * page_size + place) * dk
                                       : v_pages + (((size_t)page * G + head) * page_size + place) * dv;
        if (dst != nullptr)
            for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(sv[i]);
        __syncwarp();
    }
}

MM_EXPORT int mm_talking_prep(const void* rows, int ld, int q_off, int k_off, int v_off, const void* q_norm, const void* k_norm, float eps,
                              const void* rot, int rot_dims, int v_unit, void* q_out, void* k_pages, void* v_pages, int dtype, const void* slots,
                              int page_size, int n_tokens, int H, int G, int dk, int dv, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0 && ld > 0, "attention prep: bad sizes");
    MM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || rot != nullptr),
               "attention prep: the rotated dimensions must be even, at most the key size, and have their table");
    MM_REQUIRE(k_pages == nullptr || (page_size > 0 && slots != nullptr && v_pages != nullptr), "attention prep: bad page geometry");
    MM_REQUIRE(dk <= 1024 && dv <= 1024, "attention prep: head sizes above 1024 are not supported");
    if (n_tokens == 0) return MM_OK;
    const size_t smem = (size_t)8 * (dk > dv ? dk : dv) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MM_F32)
        mm_launch(talking_prep_kernel<float>, dim3(n_tokens), dim3(256), smem, s, (const float*)rows, ld, q_off, k_off, v_off, (const float*)q_norm,
                  (const float*)k_norm, eps, (const float2*)rot, rot_dims, v_unit, (float*)q_out, (float*)k_pages, (float*)v_pages,
                  (const int32_t*)slots, page_size, H, G, dk, dv);
    else if (dtype == MM_BF16)
        mm_launch(talking_prep_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), smem, s, (const float*)rows, ld, q_off, k_off, v_off,
                  (const float*)q_norm, (const float*)k_norm, eps, (const float2*)rot, rot_dims, v_unit, (__nv_bfloat16*)q_out,
                  (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (const int32_t*)slots, page_size, H, G, dk, dv);
    else
        MM_REQUIRE(false, "attention prep: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// attention with mixed heads, fp32 arithmetic, any sizes
// ---------------------------------------------------------------------------------------------------------------
#define TALK_THREADS 256
#define TALK_MAX_ACC 32          // H * dv <= 32 * 256

// One block per (query token, key split).  Per chunk of 32 keys: (1) every (head, key) pair's raw score by one thread;
// (2) every (head, key) pair's mixed score; a warp per head then moves that head's running maximum and mass and leaves
// the chunk's weights; (3) every thread adds the chunk's weighted values to its own (head, value channel) sums.
// splits == 1: the result is written; otherwise unnormalised sums go to part_o [n, H, splits, dv] and (maximum, mass)
// to part_ml [n, H, splits, 2], and a merge kernel finishes the rows (the sink enters there).
template <typename T, typename TO>
__global__ void __launch_bounds__(TALK_THREADS) attention_talking_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, TO* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, int splits, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
    const int32_t* __restrict__ block_table, int table_width, int page_size, int H, int G, int dk, int dv, int window, float scale,
    const float* __restrict__ talk, const float* __restrict__ sink) {
    extern __shared__ __align__(16) float talk_smem[];
    long long* kb = reinterpret_cast<long long*>(talk_smem);      // [32] page of each key of the chunk (-1: not seen)
    float* qs = talk_smem + 64;                  // [H][dk], scaled
    float* Ts = qs + (size_t)H * dk;             // [H][H] (identity when talk is null)
    float* raw = Ts + (size_t)H * H;             // [H][32]
    float* ps = raw + (size_t)H * 32;            // [H][32]
    float* ms = ps + (size_t)H * 32;             // [H] running maximum
    float* ls = ms + H;                          // [H] running mass
    float* al = ls + H;                          // [H] the chunk's rescale factor

    const int t = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int rep = H / G;

    for (int i = tid; i < H * dk; i += TALK_THREADS) qs[i] = to_f32<T>(q[(size_t)t * H * dk + i]) * scale;
    for (int i = tid; i < H * H; i += TALK_THREADS) Ts[i] = talk ? talk[i] : ((i / H == i % H) ? 1.0f : 0.0f);
    // without splits the sink starts the running softmax: a maximum of the head's logit and a mass of 1
    for (int h = tid; h < H; h += TALK_THREADS) {
        const bool start = sink != nullptr && splits == 1;
        ms[h] = start ? sink[h] : -INFINITY;
        ls[h] = start ? 1.0f : 0.0f;
    }
    float acc[TALK_MAX_ACC];
#pragma unroll
    for (int a = 0; a < TALK_MAX_ACC; ++a) acc[a] = 0.0f;
    const int n_out = H * dv;
    const size_t k_stride = (size_t)G * page_size * dk, v_stride = (size_t)G * page_size * dv;

    // the chunks of this split: aligned to absolute position, shared out evenly
    const int c_first = lo / 32, c_end = (hi + 31) / 32;
    const int per = (c_end - c_first + splits - 1) / splits;
    const int c0 = c_first + split * per, c1 = min(c_end, c0 + per);
    __syncthreads();

    for (int cc = c0; cc < c1; ++cc) {
        const int c = cc * 32;
        if (tid < 32) {
            const int j = c + tid;
            kb[tid] = (j >= lo && j < hi) ? (long long)table[j / page_size] : -1;
        }
        __syncthreads();
        for (int pair = tid; pair < H * 32; pair += TALK_THREADS) {
            const int g = pair >> 5, jj = pair & 31;
            float dot = 0.0f;
            if (kb[jj] >= 0) {
                const T* kr = k_pages + (size_t)kb[jj] * k_stride + ((size_t)(g / rep) * page_size + (size_t)((c + jj) % page_size)) * dk;
                const float* qg = qs + (size_t)g * dk;
                for (int d = 0; d < dk; ++d) dot = fmaf(qg[d], to_f32<T>(kr[d]), dot);
            }
            raw[pair] = dot;
        }
        __syncthreads();
        for (int h = warp; h < H; h += TALK_THREADS / 32) {
            float s = -INFINITY;
            if (kb[lane] >= 0) {
                s = 0.0f;
                for (int g = 0; g < H; ++g) s = fmaf(Ts[h * H + g], raw[g * 32 + lane], s);
            }
            const float m_old = ms[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float p = (kb[lane] >= 0) ? expf(s - m_new) : 0.0f;
            const float a = (m_new == -INFINITY) ? 1.0f : expf(m_old - m_new);     // m_old = -inf on the first chunk gives 0
            const float sum = warp_sum(p);
            ps[h * 32 + lane] = p;
            if (lane == 0) {
                ms[h] = m_new;
                ls[h] = ls[h] * a + sum;
                al[h] = a;
            }
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < TALK_MAX_ACC; ++a) {
            const int item = a * TALK_THREADS + tid;
            if (item < n_out) {
                const int h = item / dv, d = item - h * dv;
                const size_t v_head = (size_t)(h / rep) * page_size * dv;
                float x = acc[a] * al[h];
                for (int jj = 0; jj < 32; ++jj) {
                    if (kb[jj] < 0) continue;
                    const T* vr = v_pages + (size_t)kb[jj] * v_stride + v_head + (size_t)((c + jj) % page_size) * dv;
                    x = fmaf(ps[h * 32 + jj], to_f32<T>(vr[d]), x);
                }
                acc[a] = x;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < TALK_MAX_ACC; ++a) {
        const int item = a * TALK_THREADS + tid;
        if (item < n_out) {
            const int h = item / dv, d = item - h * dv;
            if (splits == 1) {
                const float l = ls[h];
                out[(size_t)t * n_out + item] = from_f32<TO>(l > 0.0f ? acc[a] / l : 0.0f);
            } else {
                part_o[(((size_t)t * H + h) * splits + split) * dv + d] = acc[a];
            }
        }
    }
    if (splits > 1)
        for (int h = tid; h < H; h += TALK_THREADS) {
            part_ml[(((size_t)t * H + h) * splits + split) * 2] = ms[h];
            part_ml[(((size_t)t * H + h) * splits + split) * 2 + 1] = ls[h];
        }
}

// The splits of a (token, head) row put together in the order of the splits; the sink's exp(logit) joins the mass.
template <typename TO>
__global__ void attention_talking_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, TO* __restrict__ out,
                                               int splits, int H, int dv, const float* __restrict__ sink) {
    const size_t row = blockIdx.x;              // token * H + head
    const int h = (int)(row % H);
    float m = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row * splits + s) * 2]);
    float l = sink ? expf(sink[h] - m) : 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(row * splits + s) * 2];
        if (ms != -INFINITY) l += part_ml[(row * splits + s) * 2 + 1] * expf(ms - m);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(row * splits + s) * 2];
            if (ms != -INFINITY) o = fmaf(part_o[(row * splits + s) * dv + d], expf(ms - m), o);
        }
        out[row * dv + d] = from_f32<TO>(o * inv);
    }
}

MM_EXPORT int mm_attention_talking(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype, void* part_o, void* part_ml,
                                   int splits, const void* positions, const void* token_req, const void* block_table, int table_width,
                                   int page_size, int n_tokens, int H, int G, int dk, int dv, int window, float scale, const void* talk,
                                   const void* sink, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0 && H % G == 0, "attention: heads must be a positive multiple of kv heads");
    MM_REQUIRE(H * dv <= TALK_MAX_ACC * TALK_THREADS, "attention with mixed heads: heads * value size above 8192 is not supported");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention: bad page geometry or window");
    MM_REQUIRE(splits >= 1 && (splits == 1 || (part_o != nullptr && part_ml != nullptr)), "attention: key splits need their scratch");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = sizeof(float) * ((size_t)H * dk + (size_t)H * H + 64 * (size_t)H + 3 * (size_t)H) + 32 * sizeof(long long);
    MM_REQUIRE(smem <= 200 * 1024, "attention with mixed heads: heads * key size is too large for the kernel's shared memory");
    const dim3 grid(n_tokens, splits);
    typedef __nv_bfloat16 bf;
#define TALK_LAUNCH(T)                                                                                                                       \
    do {                                                                                                                                     \
        auto kernel = attention_talking_kernel<T, T>;                                                                                        \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                          \
        mm_launch(kernel, grid, dim3(TALK_THREADS), smem, s, (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, (float*)part_o,     \
                  (float*)part_ml, splits, (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)block_table, table_width,   \
                  page_size, H, G, dk, dv, window, scale, (const float*)talk, (const float*)sink);                                           \
        MM_CHECK_LAUNCH();                                                                                                                   \
        if (splits > 1) {                                                                                                                    \
            mm_launch(attention_talking_merge_kernel<T>, dim3(n_tokens * H), dim3(128), 0, s, (const float*)part_o, (const float*)part_ml,   \
                      (T*)out, splits, H, dv, (const float*)sink);                                                                           \
            MM_CHECK_LAUNCH();                                                                                                               \
        }                                                                                                                                    \
    } while (0)
    if (dtype == MM_F32) TALK_LAUNCH(float);
    else if (dtype == MM_BF16) TALK_LAUNCH(bf);
    else MM_REQUIRE(false, "attention: dtype must be float32 or bfloat16");
#undef TALK_LAUNCH
    return MM_OK;
}
