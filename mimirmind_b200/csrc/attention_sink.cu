// Windowed attention with a softmax sink, and keys and values of different sizes.
//
//   q [n, H, dk], keys [.., G, dk], values [.., G, dv]; query head h reads kv head h / (H / G);
//   a query at absolute position a sees keys max(0, a + 1 - W) .. a (W = 0: all);
//   s_j = (q . k_j) * scale;  p_j = exp(s_j) / (sink + sum_i exp(s_i)),  sink = 1 or 0;  o = sum_j p_j v_j.
//
// The sink is a key of score 0 that has no value: it only takes its share of the weights.  The fp32-arithmetic
// kernel also takes a learned sink, exp(logit of the head) in its place, and a learned bias per (distance, head)
// that is added to the scaled score: bias[h][min(a - j, rows - 1)] (a table by distance per head, clamped at its last
// entry); the bfloat16 tensor-core kernels (attention_sink_mma.cu) take both as well.
//
// This file holds (1) the step between the q/k/v projection and attention: rotation of adjacent pairs
// (2i, 2i+1) of q and k by position (angles from a per-step table), the mixing of this layer's values with those of
// an earlier layer, and the write of keys and values into their pages; (2) the fp32-arithmetic attention kernel for any sizes, one warp per
// (token, head), its keys in chunks of 32 aligned to absolute position so that a token's result depends on its own
// position and keys only.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------------------
// rotation of pairs + value mixing + cache write
// ---------------------------------------------------------------------------------------------------------------
// The step's rotation table: (cos, sin) of position * inv_freq[i] for every token and pair, fp32, made once per step
// and read by every layer with the same frequencies.
__global__ void rope_pairs_table_kernel(const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                        float2* __restrict__ table, int n_tokens, int half) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * half) return;
    const int t = (int)(i / half), p = (int)(i - (long long)t * half);
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[p], &sn, &cs);
    table[i] = make_float2(cs, sn);
}

MM_EXPORT int mm_rope_pairs_table(const void* positions, const void* inv_freq, void* table, int n_tokens, int half, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && half > 0, "rope pairs table: bad sizes");
    if (n_tokens == 0) return MM_OK;
    const long long total = (long long)n_tokens * half;
    mm_launch(rope_pairs_table_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream, (const int32_t*)positions,
              (const float*)inv_freq, (float2*)table, n_tokens, half);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// qkv [n, H*dk + G*dk + G*dv] (bias already added).  Pair i < rot_dims/2 of every q and k head turns by the angle of
// rot[t][i]; dimensions from rot_dims on pass unchanged.  slots[t] = page * page_size + place of the token in its
// cache group (negative: nothing to write).
// mix_mode 0: values as they are; 1: also copy them to v_first (this layer is the source); 2: v = (1-lambda) v +
// lambda v_first.  What is cached is the mixed value.
template <typename T>
__global__ void qkv_pairs_post_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                      T* __restrict__ v_pages, T* __restrict__ v_first, const float2* __restrict__ rot,
                                      const int32_t* __restrict__ slots, int page_size, int H, int G,
                                      int dk, int dv, int rot_dims, int mix_mode, float lambda) {
    const int t = blockIdx.x;
    const int width = (H + G) * dk + G * dv;
    const T* row = qkv + (size_t)t * width;
    const long long slot = (k_pages != nullptr) ? (long long)slots[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int place = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const int half = (dk + 1) / 2;
    const float2* rt = rot + (size_t)t * (rot_dims / 2);
    for (int item = threadIdx.x; item < (H + G) * half; item += blockDim.x) {
        const int head = item / half, p = item - head * half;
        const int e0 = 2 * p, e1 = e0 + 1;
        float a = to_f32<T>(row[head * dk + e0]);
        float b = e1 < dk ? to_f32<T>(row[head * dk + e1]) : 0.0f;
        if (e1 < rot_dims) {
            const float2 cs = rt[p];
            const float ra = a * cs.x - b * cs.y, rb = b * cs.x + a * cs.y;
            a = ra;
            b = rb;
        }
        T* dst;
        if (head < H) {
            dst = q_out + ((size_t)t * H + head) * dk;
        } else {
            if (page < 0) continue;
            dst = k_pages + (((size_t)page * G + (head - H)) * page_size + place) * dk;
        }
        dst[e0] = from_f32<T>(a);
        if (e1 < dk) dst[e1] = from_f32<T>(b);
    }
    const T* vrow = row + (H + G) * dk;
    for (int item = threadIdx.x; item < G * dv; item += blockDim.x) {
        float v = to_f32<T>(vrow[item]);
        if (mix_mode == 1) v_first[(size_t)t * G * dv + item] = vrow[item];
        if (mix_mode == 2) v = (1.0f - lambda) * v + lambda * to_f32<T>(v_first[(size_t)t * G * dv + item]);
        if (page >= 0) {
            const int g = item / dv, e = item - g * dv;
            v_pages[(((size_t)page * G + g) * page_size + place) * dv + e] = from_f32<T>(v);
        }
    }
}

// bfloat16 with key, value and rotated sizes that are multiples of 8: one 16-byte chunk (four pairs) per thread
__global__ void qkv_pairs_post_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                             __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                             __nv_bfloat16* __restrict__ v_first, const float2* __restrict__ rot,
                                             const int32_t* __restrict__ slots, int page_size, int n_tokens, int H, int G,
                                             int dk, int dv, int rot_dims, int mix_mode, float lambda) {
    const int kc = dk / 8, vc = dv / 8;
    const int per_token = (H + G) * kc + G * vc;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * per_token) return;
    const int t = (int)(i / per_token), c = (int)(i - (long long)t * per_token);
    const long long slot = (k_pages != nullptr) ? (long long)slots[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int place = slot >= 0 ? (int)(slot - page * page_size) : 0;
    const __nv_bfloat16* row = qkv + (size_t)t * ((H + G) * dk + G * dv);
    if (c < (H + G) * kc) {
        const int head = c / kc, part = c - head * kc;
        uint4 raw = *reinterpret_cast<const uint4*>(row + head * dk + part * 8);
        if (part * 8 < rot_dims) {
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
            const float4 cs01 = *reinterpret_cast<const float4*>(rot + (size_t)t * (rot_dims / 2) + part * 4);
            const float4 cs23 = *reinterpret_cast<const float4*>(rot + (size_t)t * (rot_dims / 2) + part * 4 + 2);
            const float cs[8] = {cs01.x, cs01.y, cs01.z, cs01.w, cs23.x, cs23.y, cs23.z, cs23.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 ab = __bfloat1622float2(p2[k]);
                p2[k] = __floats2bfloat162_rn(ab.x * cs[2 * k] - ab.y * cs[2 * k + 1], ab.y * cs[2 * k] + ab.x * cs[2 * k + 1]);
            }
        }
        if (head < H)
            *reinterpret_cast<uint4*>(q_out + ((size_t)t * H + head) * dk + part * 8) = raw;
        else if (page >= 0)
            *reinterpret_cast<uint4*>(k_pages + (((size_t)page * G + (head - H)) * page_size + place) * dk + part * 8) = raw;
        return;
    }
    const int vcid = c - (H + G) * kc;
    const int g = vcid / vc, part = vcid - g * vc;
    uint4 raw = *reinterpret_cast<const uint4*>(row + (H + G) * dk + g * dv + part * 8);
    __nv_bfloat16* vf = v_first + (size_t)t * G * dv + g * dv + part * 8;
    if (mix_mode == 1) *reinterpret_cast<uint4*>(vf) = raw;
    if (mix_mode == 2) {
        const uint4 first = *reinterpret_cast<const uint4*>(vf);
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
        const __nv_bfloat162* f2 = reinterpret_cast<const __nv_bfloat162*>(&first);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 a = __bfloat1622float2(p2[k]), f = __bfloat1622float2(f2[k]);
            p2[k] = __floats2bfloat162_rn((1.0f - lambda) * a.x + lambda * f.x, (1.0f - lambda) * a.y + lambda * f.y);
        }
    }
    if (page >= 0) *reinterpret_cast<uint4*>(v_pages + (((size_t)page * G + g) * page_size + place) * dv + part * 8) = raw;
}

MM_EXPORT int mm_qkv_pairs_post(const void* qkv, void* q_out, void* k_pages, void* v_pages, void* v_first, int dtype,
                                const void* rot, const void* slots, int page_size, int n_tokens, int H, int G, int dk, int dv,
                                int rot_dims, int mix_mode, float lambda, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0, "qkv post: bad sizes");
    MM_REQUIRE(rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0, "qkv post: the rotated dimensions must be even and at most the head size");
    MM_REQUIRE(rot_dims == 0 || rot != nullptr, "qkv post: a rotation needs its table");
    MM_REQUIRE(mix_mode == 0 || v_first != nullptr, "qkv post: value mixing needs the first values");
    MM_REQUIRE(k_pages == nullptr || (page_size > 0 && slots != nullptr && v_pages != nullptr), "qkv post: bad page geometry");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)v_first | (uintptr_t)rot) & 15) == 0;
    if (dtype == MM_BF16 && dk % 8 == 0 && dv % 8 == 0 && rot_dims % 8 == 0 && aligned) {
        const long long total = (long long)n_tokens * ((H + G) * (dk / 8) + G * (dv / 8));
        mm_launch(qkv_pairs_post_bf16x8_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, s, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out,
                  (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)v_first, (const float2*)rot, (const int32_t*)slots,
                  page_size, n_tokens, H, G, dk, dv, rot_dims, mix_mode, lambda);
    } else if (dtype == MM_F32)
        mm_launch(qkv_pairs_post_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)qkv, (float*)q_out, (float*)k_pages,
                  (float*)v_pages, (float*)v_first, (const float2*)rot, (const int32_t*)slots, page_size, H, G, dk, dv, rot_dims, mix_mode, lambda);
    else if (dtype == MM_BF16)
        mm_launch(qkv_pairs_post_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)v_first,
                  (const float2*)rot, (const int32_t*)slots, page_size, H, G, dk, dv, rot_dims, mix_mode, lambda);
    else
        MM_REQUIRE(false, "qkv post: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// attention, fp32 arithmetic, any sizes
// ---------------------------------------------------------------------------------------------------------------
#define SINK_MAX_ACC 16  // dv <= 512

template <typename T, typename TO = T>
__global__ void attention_sink_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                              const T* __restrict__ v_pages, TO* __restrict__ out,
                                              const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                              const int32_t* __restrict__ block_table, int table_width, int page_size,
                                              int n_tokens, int H, int G, int dk, int dv, int window, float scale, int sink,
                                              const float* __restrict__ sink_logit, const float* __restrict__ dist_bias, int dist_max,
                                              float softcap, int Gv, int v_row) {
    extern __shared__ float q_smem[];  // [warps][dk]
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps_per_block + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int g = h / (H / G);
    const int pos = positions[t];
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;

    float* qs = q_smem + warp * dk;
    const T* qrow = q + ((size_t)t * H + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[d] = to_f32<T>(qrow[d]) * scale;
    __syncwarp();

    // the sink starts the running softmax: a maximum of 0 (or of the head's learned logit) and a mass of 1 with
    // nothing accumulated
    float m = sink_logit ? sink_logit[h] : (sink ? 0.0f : -INFINITY), l = (sink_logit || sink) ? 1.0f : 0.0f;
    float acc[SINK_MAX_ACC];
#pragma unroll
    for (int a = 0; a < SINK_MAX_ACC; ++a) acc[a] = 0.0f;
    const size_t k_head = (size_t)g * page_size * dk, k_stride = (size_t)G * page_size * dk;
    // values: Gv heads of which key head g reads g mod Gv, consecutive tokens v_row numbers apart (a pool of its own: dv)
    const size_t v_head = (size_t)(g % Gv) * page_size * v_row, v_stride = (size_t)Gv * page_size * v_row;
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;

    for (int c = (lo / 32) * 32; c < hi; c += 32) {
        const int j = c + lane;
        const bool valid = (j >= lo) && (j < hi);
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            const T* kr = k_pages + (size_t)page * k_stride + k_head + (size_t)(j % page_size) * dk;
            float dot = 0.0f;
            for (int d = 0; d < dk; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            if (softcap > 0.0f) dot = softcap * tanhf(dot * inv_cap);      // the scaled score, bent into (-cap, cap)
            // a learned bias per (distance, head), not scaled: the table's last row stands for every larger distance
            s = dist_bias ? dot + dist_bias[(size_t)h * (dist_max + 1) + min(pos - j, dist_max)] : dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);  // m = -inf on the first chunk gives 0
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int a = 0; a < SINK_MAX_ACC; ++a) acc[a] *= alpha;
        for (int jj = 0; jj < 32; ++jj) {
            const int key = c + jj;
            if (key < lo || key >= hi) continue;  // uniform over the warp
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int page = table[key / page_size];
            const T* vr = v_pages + (size_t)page * v_stride + v_head + (size_t)(key % page_size) * v_row;
#pragma unroll
            for (int a = 0; a < SINK_MAX_ACC; ++a) {
                const int d = a * 32 + lane;
                if (d < dv) acc[a] = fmaf(pj, to_f32<T>(vr[d]), acc[a]);
            }
        }
        m = m_new;
    }
    const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
    TO* orow = out + ((size_t)t * H + h) * dv;
#pragma unroll
    for (int a = 0; a < SINK_MAX_ACC; ++a) {
        const int d = a * 32 + lane;
        if (d < dv) orow[d] = from_f32<TO>(acc[a] * inv_l);
    }
}

MM_EXPORT int mm_attention_sink_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                        const void* positions, const void* token_req, const void* block_table,
                                        int table_width, int page_size, int n_tokens, int H, int G, int dk, int dv, int window,
                                        float scale, int sink, const void* sink_logit, const void* dist_bias, int dist_max, float softcap,
                                        int Gv, int v_row, int out_f32, void* stream) {
    MM_REQUIRE(dist_bias == nullptr || dist_max >= 0, "attention: the distance table needs at least one row");
    MM_REQUIRE(Gv >= 1 && G % Gv == 0 && v_row >= dv && softcap >= 0.0f, "attention: value heads must divide the key heads, a value row holds at least dv numbers");
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0 && H % G == 0, "attention: heads must be a positive multiple of kv heads");
    MM_REQUIRE(dv <= 32 * SINK_MAX_ACC && dk <= 2048, "attention: value size above 512 or key size above 2048 is not supported");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention: bad page geometry or window");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const size_t smem = (size_t)warps * dk * sizeof(float);
    const long long items = (long long)n_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (dtype == MM_F32)
        mm_launch(attention_sink_generic_kernel<float>, dim3(blocks), dim3(warps * 32), smem, s, (const float*)q, (const float*)k_pages,
                  (const float*)v_pages, (float*)out, (const int32_t*)positions, (const int32_t*)token_req,
                  (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, dk, dv, window, scale, sink,
                  (const float*)sink_logit, (const float*)dist_bias, dist_max, softcap, Gv, v_row);
    else if (dtype == MM_BF16 && out_f32)      // the result is not rounded: what follows takes a difference of heads
        mm_launch(attention_sink_generic_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(warps * 32), smem, s, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (float*)out, (const int32_t*)positions,
                  (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, dk, dv, window,
                  scale, sink, (const float*)sink_logit, (const float*)dist_bias, dist_max, softcap, Gv, v_row);
    else if (dtype == MM_BF16)
        mm_launch(attention_sink_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, s, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, (const int32_t*)positions,
                  (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, dk, dv, window,
                  scale, sink, (const float*)sink_logit, (const float*)dist_bias, dist_max, softcap, Gv, v_row);
    else
        MM_REQUIRE(false, "attention: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
