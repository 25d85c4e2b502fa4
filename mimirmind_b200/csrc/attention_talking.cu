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
// only; (3) the tensor-core kernel for bfloat16 (mma.sync m16n8k16, fp32 scores): a CTA owns 16 query tokens of one
// request with all their heads; per key tile the warps share out the heads' raw score products, leave them in shared
// memory, and every warp then mixes, masks and softmaxes the scores of its own heads and multiplies them with the values.
#include "common.cuh"
#include "mma_sync.cuh"

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

// ---------------------------------------------------------------------------------------------------------------
// attention with mixed heads on the tensor cores (bfloat16 operands, fp32 scores, mixing, softmax and sums)
// ---------------------------------------------------------------------------------------------------------------
// A tile: 16 consecutive tokens (or fewer) of one request, tiles[i] = (first token, tokens); positions and the request are
// read from the device, so a captured decode step replays the same list.  grid = (tiles, head groups, key splits).
// A CTA of NW warps: all H heads' raw scores of a key tile are made by the warps in turn (head g by warp g mod NW, at most
// two per warp) and written, scaled, to shared memory over the key tile they were made from; warp w then owns HPW heads of
// the CTA's head group: it mixes their scores from all raw heads (fp32), masks, keeps the running maximum and mass per
// row, and adds P V to its accumulators.  Shared memory: Q [H][16][dk + 8], K [G][TK][dk + 8] (then raw [H][16][TK + 8]
// fp32 in the same place), V [G][TK][dv + 8], the head group's rows of the mixing matrix.
#define TALK_LOG2E 1.4426950408889634f

template <int DV, int HPW, int TK>
__global__ void __launch_bounds__(512) attention_talking_mma_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table, int table_width,
    int page_size, int H, int G, int dk, int Hc, int window, float scale, const float* __restrict__ talk, const float* __restrict__ sink) {
    constexpr int NT_S = TK / 8, NT_O = DV / 8, RS = TK + 8, VS = DV + 8;
    extern __shared__ __align__(16) unsigned char tm_smem[];
    const int KS = dk + 8;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(tm_smem);
    const size_t q_bytes = (size_t)H * 16 * KS * 2;
    const size_t k_bytes = (size_t)G * TK * KS * 2, raw_bytes = (size_t)H * 16 * RS * 4;
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(tm_smem + q_bytes);
    float* sRaw = reinterpret_cast<float*>(tm_smem + q_bytes);
    const size_t kr_bytes = ((k_bytes > raw_bytes ? k_bytes : raw_bytes) + 15) & ~(size_t)15;
    __nv_bfloat16* sV = reinterpret_cast<__nv_bfloat16*>(tm_smem + q_bytes + kr_bytes);
    float* sT = reinterpret_cast<float*>(tm_smem + q_bytes + kr_bytes + (size_t)G * TK * VS * 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, NW = blockDim.x >> 5, threads = blockDim.x;
    const int t0 = tiles[2 * blockIdx.x], nq = tiles[2 * blockIdx.x + 1];
    const int hg = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
    const int pos0 = positions[t0];
    const int32_t* table = block_table + (size_t)token_req[t0] * table_width;
    const int rep = H / G;
    const int hi_all = pos0 + nq;                                                   // keys below this position
    const int lo_all = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    // key tiles of this split, aligned to TK
    const int kt_first = lo_all / TK, kt_end = (hi_all + TK - 1) / TK;
    const int per = (kt_end - kt_first + splits - 1) / splits;
    const int kt0 = kt_first + split * per, kt1 = min(kt_end, kt0 + per);

    // Q of all heads, rows beyond the tile's tokens zero
    const int qparts = dk / 8;
    for (int i = tid; i < H * 16 * qparts; i += threads) {
        const int part = i % qparts, r = (i / qparts) % 16, h = i / (qparts * 16);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r) * H + h) * dk + part * 8);
        *reinterpret_cast<uint4*>(sQ + ((size_t)h * 16 + r) * KS + part * 8) = v;
    }
    const int h_first = hg * Hc;
    for (int i = tid; i < Hc * H; i += threads) {
        const int hl = i / H, g = i - hl * H;
        const int h = h_first + hl;
        sT[i] = h < H ? (talk ? talk[(size_t)h * H + g] : (h == g ? 1.0f : 0.0f)) : 0.0f;
    }

    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const int pos_lo = pos0 + r_lo, pos_hi = pos0 + r_hi;
    const int wlo_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int wlo_hi = (window > 0 && pos_hi + 1 > window) ? pos_hi + 1 - window : 0;
    const bool valid_lo = r_lo < nq, valid_hi = r_hi < nq;

    float o[HPW][NT_O][4], m_lo[HPW], m_hi[HPW], l_lo[HPW], l_hi[HPW];
#pragma unroll
    for (int x = 0; x < HPW; ++x) {
        const int h = h_first + warp * HPW + x;
        // without key splits the sink starts the running softmax: its logit as the maximum, a mass of 1
        const bool start = sink != nullptr && splits == 1 && h < H;
        m_lo[x] = m_hi[x] = start ? sink[h] * TALK_LOG2E : -INFINITY;
        l_lo[x] = l_hi[x] = (start && (lane & 3) == 0) ? 1.0f : 0.0f;       // a row's mass is summed over its quad at the end
#pragma unroll
        for (int j = 0; j < NT_O; ++j) o[x][j][0] = o[x][j][1] = o[x][j][2] = o[x][j][3] = 0.0f;
    }
    const int ksteps = dk / 16;
    const int id = lane >> 3, rr = lane & 7;
    const int kparts = dk / 8, vparts = DV / 8;
    const int most = kparts > vparts ? kparts : vparts;
    const int row_shift = most <= 4 ? 2 : (most <= 8 ? 3 : (most <= 16 ? 4 : 5));      // dk <= 256: at most 32 copies a row
    const int row_threads = 1 << row_shift;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    for (int kt = kt0; kt < kt1; ++kt) {
        const int key0 = kt * TK;
        __syncthreads();                        // the tile before is used up (and, the first time, Q and T are written)
        // a row of the tile (kv head, key) is copied by `row_threads` neighbouring threads, 16 bytes each: no division per copy
        for (int row = tid >> row_shift; row < G * TK; row += threads >> row_shift) {
            const int g = row / TK, key = row % TK;          // TK is a power of two
            const int j = key0 + key;
            const int part = tid & (row_threads - 1);
            const bool seen = j >= lo_all && j < hi_all;
            size_t at = 0;
            if (seen) {
                const int pg = page_shift >= 0 ? j >> page_shift : j / page_size;
                at = ((size_t)table[pg] * G + g) * page_size + (size_t)(j - pg * page_size);
            }
            if (part < kparts) {
                __nv_bfloat16* dst = sK + ((size_t)g * TK + key) * KS + part * 8;
                if (seen) cp_async16(dst, k_pages + at * dk + part * 8);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
            if (part < vparts) {
                __nv_bfloat16* dst = sV + ((size_t)g * TK + key) * VS + part * 8;
                if (seen) cp_async16(dst, v_pages + at * DV + part * 8);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        // a tile whose keys all lie at or before the first row's position and inside the last row's window needs no masks
        const bool interior = key0 + TK - 1 <= pos0 && (window == 0 || key0 >= pos0 + 15 + 1 - window);
        // raw scores of the heads this warp takes in this phase
        float s[2][NT_S][4];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int g = warp + NW * x;
#pragma unroll
            for (int j = 0; j < NT_S; ++j) s[x][j][0] = s[x][j][1] = s[x][j][2] = s[x][j][3] = 0.0f;
            if (g < H) {
                const __nv_bfloat16* tQ = sQ + (size_t)g * 16 * KS;
                const __nv_bfloat16* tK = sK + (size_t)(g / rep) * TK * KS;
#pragma unroll 2
                for (int ks = 0; ks < ksteps; ++ks) {
                    uint32_t qf[4];
                    ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], tQ + ((id & 1) * 8 + rr) * KS + ks * 16 + (id >> 1) * 8);
#pragma unroll
                    for (int jp = 0; jp < NT_S / 2; ++jp) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(b0, b1, b2, b3, tK + (jp * 16 + (id >> 1) * 8 + rr) * KS + ks * 16 + (id & 1) * 8);
                        mma_bf16(s[x][jp * 2], qf, b0, b1);
                        mma_bf16(s[x][jp * 2 + 1], qf, b2, b3);
                    }
                }
            }
        }
        __syncthreads();                        // every warp is done with the keys: the raw scores take their place
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int g = warp + NW * x;
            if (g < H) {
                float* rg = sRaw + (size_t)g * 16 * RS;
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    const int c = j * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2*>(rg + r_lo * RS + c) = make_float2(s[x][j][0] * scale, s[x][j][1] * scale);
                    *reinterpret_cast<float2*>(rg + r_hi * RS + c) = make_float2(s[x][j][2] * scale, s[x][j][3] * scale);
                }
            }
        }
        __syncthreads();

        // the mixed scores of the warp's heads: every raw head's tile is read once for all of them
        float mxs[HPW][NT_S][4];
#pragma unroll
        for (int x = 0; x < HPW; ++x)
#pragma unroll
            for (int j = 0; j < NT_S; ++j) mxs[x][j][0] = mxs[x][j][1] = mxs[x][j][2] = mxs[x][j][3] = 0.0f;
        if (warp * HPW < Hc) {
            const float* th = sT + (size_t)warp * HPW * H;
#pragma unroll 4
            for (int g = 0; g < H; ++g) {
                float t[HPW];
#pragma unroll
                for (int x = 0; x < HPW; ++x) t[x] = (warp * HPW + x < Hc) ? th[x * H + g] : 0.0f;
                const float* rg = sRaw + (size_t)g * 16 * RS + (lane & 3) * 2;
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    const float2 a = *reinterpret_cast<const float2*>(rg + r_lo * RS + j * 8);
#pragma unroll
                    for (int x = 0; x < HPW; ++x) {
                        mxs[x][j][0] = fmaf(t[x], a.x, mxs[x][j][0]); mxs[x][j][1] = fmaf(t[x], a.y, mxs[x][j][1]);
                    }
                    if (nq > 8) {           // a tile of at most eight tokens (a decode step's) has no second half of rows
                        const float2 b = *reinterpret_cast<const float2*>(rg + r_hi * RS + j * 8);
#pragma unroll
                        for (int x = 0; x < HPW; ++x) {
                            mxs[x][j][2] = fmaf(t[x], b.x, mxs[x][j][2]); mxs[x][j][3] = fmaf(t[x], b.y, mxs[x][j][3]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int x = 0; x < HPW; ++x) {
            const int hl = warp * HPW + x, h = h_first + hl;
            if (hl >= Hc || h >= H) continue;
            float (&mx)[NT_S][4] = mxs[x];
            float new_lo = m_lo[x], new_hi = m_hi[x];
            if (interior) {
                // every key of the tile is seen by every row: no masks (rows beyond the tile's tokens hold zeros and are never stored)
#pragma unroll
                for (int j = 0; j < NT_S; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        mx[j][c] *= TALK_LOG2E;
                        if (c < 2) new_lo = fmaxf(new_lo, mx[j][c]);
                        else new_hi = fmaxf(new_hi, mx[j][c]);
                    }
            } else {
#pragma unroll
                for (int j = 0; j < NT_S; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int key = key0 + j * 8 + (lane & 3) * 2 + c;
                        const bool ok_lo = valid_lo && key <= pos_lo && key >= wlo_lo;
                        const bool ok_hi = valid_hi && key <= pos_hi && key >= wlo_hi;
                        mx[j][c] = ok_lo ? mx[j][c] * TALK_LOG2E : -INFINITY;
                        mx[j][2 + c] = ok_hi ? mx[j][2 + c] * TALK_LOG2E : -INFINITY;
                        new_lo = fmaxf(new_lo, mx[j][c]);
                        new_hi = fmaxf(new_hi, mx[j][2 + c]);
                    }
            }
            new_lo = fmaxf(new_lo, __shfl_xor_sync(0xffffffffu, new_lo, 1));
            new_lo = fmaxf(new_lo, __shfl_xor_sync(0xffffffffu, new_lo, 2));
            new_hi = fmaxf(new_hi, __shfl_xor_sync(0xffffffffu, new_hi, 1));
            new_hi = fmaxf(new_hi, __shfl_xor_sync(0xffffffffu, new_hi, 2));
            const float ref_lo = new_lo == -INFINITY ? 0.0f : new_lo, ref_hi = new_hi == -INFINITY ? 0.0f : new_hi;
            const float a_lo = exp2f(m_lo[x] - ref_lo), a_hi = exp2f(m_hi[x] - ref_hi);       // a maximum of -inf gives 0
            m_lo[x] = new_lo;
            m_hi[x] = new_hi;
            uint32_t pf[TK / 16][4];
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int j = 0; j < NT_S; ++j) {
                const float p0 = exp2f(mx[j][0] - ref_lo), p1 = exp2f(mx[j][1] - ref_lo);
                const float p2 = exp2f(mx[j][2] - ref_hi), p3 = exp2f(mx[j][3] - ref_hi);
                sum_lo += p0 + p1;
                sum_hi += p2 + p3;
                pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_lo[x] = l_lo[x] * a_lo + sum_lo;
            l_hi[x] = l_hi[x] * a_hi + sum_hi;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[x][j][0] *= a_lo; o[x][j][1] *= a_lo; o[x][j][2] *= a_hi; o[x][j][3] *= a_hi;
            }
            const __nv_bfloat16* tV = sV + (size_t)(h / rep) * TK * VS;
#pragma unroll
            for (int ks = 0; ks < TK / 16; ++ks)
#pragma unroll
                for (int jp = 0; jp < NT_O / 2; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, tV + (ks * 16 + (id & 1) * 8 + rr) * VS + (jp * 2 + (id >> 1)) * 8);
                    mma_bf16(o[x][jp * 2], pf[ks], b0, b1);
                    mma_bf16(o[x][jp * 2 + 1], pf[ks], b2, b3);
                }
        }
    }
#pragma unroll
    for (int x = 0; x < HPW; ++x) {
        const int hl = warp * HPW + x, h = h_first + hl;
        if (hl >= Hc || h >= H) continue;
        float ll = l_lo[x], lh = l_hi[x];
        ll += __shfl_xor_sync(0xffffffffu, ll, 1);
        ll += __shfl_xor_sync(0xffffffffu, ll, 2);
        lh += __shfl_xor_sync(0xffffffffu, lh, 1);
        lh += __shfl_xor_sync(0xffffffffu, lh, 2);
        if (splits == 1) {
            const float i_lo = ll > 0.0f ? 1.0f / ll : 0.0f, i_hi = lh > 0.0f ? 1.0f / lh : 0.0f;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                const int c = j * 8 + (lane & 3) * 2;
                if (valid_lo) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + r_lo) * H + h) * DV + c) = pack_bf16(o[x][j][0] * i_lo, o[x][j][1] * i_lo);
                if (valid_hi) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + r_hi) * H + h) * DV + c) = pack_bf16(o[x][j][2] * i_hi, o[x][j][3] * i_hi);
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                const int c = j * 8 + (lane & 3) * 2;
                if (valid_lo) *reinterpret_cast<float2*>(part_o + ((((size_t)(t0 + r_lo) * H + h) * splits + split) * DV + c)) = make_float2(o[x][j][0], o[x][j][1]);
                if (valid_hi) *reinterpret_cast<float2*>(part_o + ((((size_t)(t0 + r_hi) * H + h) * splits + split) * DV + c)) = make_float2(o[x][j][2], o[x][j][3]);
            }
            if ((lane & 3) == 0) {
                // the merge works with natural exponents
                if (valid_lo) {
                    float* ml = part_ml + (((size_t)(t0 + r_lo) * H + h) * splits + split) * 2;
                    ml[0] = m_lo[x] / TALK_LOG2E;
                    ml[1] = ll;
                }
                if (valid_hi) {
                    float* ml = part_ml + (((size_t)(t0 + r_hi) * H + h) * splits + split) * 2;
                    ml[0] = m_hi[x] / TALK_LOG2E;
                    ml[1] = lh;
                }
            }
        }
    }
}

// How the tensor-core kernel would run these sizes: heads per warp, head groups (grid.y), warps, keys per tile and shared
// memory; false when it does not take them.
static int g_talk_prefer16 = 1;
MM_EXPORT void mm_attention_talking_prefer16(int on) { g_talk_prefer16 = on; }

struct TalkPlan {
    int hpw, groups, hc, warps, tk;
    size_t smem;
};
static bool talk_plan(int H, int G, int dk, int dv, TalkPlan& p) {
    if (H < 1 || G < 1 || H % G || dk % 16 || dk < 16 || dk > 256 || !(dv == 32 || dv == 64 || dv == 96 || dv == 128) || H > 32) return false;
    p.hpw = dv <= 64 ? 2 : 1;
    p.groups = (p.hpw == 1 && H > 16) ? 2 : 1;
    p.hc = (H + p.groups - 1) / p.groups;
    p.warps = (p.hc + p.hpw - 1) / p.hpw;
    if (p.warps > 16 || (H + p.warps - 1) / p.warps > 2) return false;
    // 32 keys per tile where two CTAs of them share an SM or nothing smaller does either; else 16 keys if that gets two CTAs
    // onto an SM (a CTA of few warps waits on every barrier and copy: a second one fills those gaps) or is all that fits
    size_t need[2];
    for (int i = 0; i < 2; ++i) {
        const int tk = i == 0 ? 32 : 16;
        const size_t q = (size_t)H * 16 * (dk + 8) * 2, k = (size_t)G * tk * (dk + 8) * 2, raw = (size_t)H * 16 * (tk + 8) * 4;
        const size_t kr = ((k > raw ? k : raw) + 15) & ~(size_t)15;
        need[i] = q + kr + (size_t)G * tk * (dv + 8) * 2 + (size_t)p.hc * H * 4;
    }
    const size_t whole = 227 * 1024, half = 113 * 1024;
    if (need[1] > whole) return false;
    const bool two_of_16 = need[1] <= half && need[0] > half && p.warps <= 16;
    const bool use16 = need[0] > whole || (two_of_16 && g_talk_prefer16);
    p.tk = use16 ? 16 : 32;
    p.smem = use16 ? need[1] : need[0];
    return true;
}

MM_EXPORT int mm_attention_talking_mma_supported(int H, int G, int dk, int dv) {
    TalkPlan p;
    return talk_plan(H, G, dk, dv, p) ? 1 : 0;
}

template <int DV, int HPW, int TK>
static void talk_mma_launch(const TalkPlan& p, dim3 grid, cudaStream_t s, const void* q, const void* k_pages, const void* v_pages, void* out,
                            void* part_o, void* part_ml, const void* tiles, const void* positions, const void* token_req, const void* block_table,
                            int table_width, int page_size, int H, int G, int dk, int window, float scale, const void* talk, const void* sink) {
    auto kernel = attention_talking_mma_kernel<DV, HPW, TK>;
    if (p.smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    mm_launch(kernel, grid, dim3(p.warps * 32), p.smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
              (__nv_bfloat16*)out, (float*)part_o, (float*)part_ml, (const int32_t*)tiles, (const int32_t*)positions, (const int32_t*)token_req,
              (const int32_t*)block_table, table_width, page_size, H, G, dk, p.hc, window, scale, (const float*)talk, (const float*)sink);
}

// tiles [n_tiles, 2] int32 = (first token, tokens <= 16) of one request each; out [n, H * dv] bfloat16.  splits > 1: the
// key tiles of a tile of tokens are shared out over that many CTAs (part_o fp32 [n, H, splits, dv], part_ml fp32
// [n, H, splits, 2]) and the merge kernel finishes every row.
MM_EXPORT int mm_attention_talking_mma(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o, void* part_ml, int splits,
                                       const void* tiles, int n_tiles, int n_tokens, const void* positions, const void* token_req,
                                       const void* block_table, int table_width, int page_size, int H, int G, int dk, int dv, int window,
                                       float scale, const void* talk, const void* sink, void* stream) {
    TalkPlan p;
    MM_REQUIRE(talk_plan(H, G, dk, dv, p), "attention with mixed heads: the tensor-core kernel does not take these sizes");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0 && n_tiles >= 0, "attention: bad page geometry or window");
    MM_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || (part_o != nullptr && part_ml != nullptr)), "attention: key splits need their scratch");
    if (n_tiles == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tiles, p.groups, splits);
#define TALK_MMA(DV, HPW)                                                                                                                          \
    do {                                                                                                                                           \
        if (p.tk == 32)                                                                                                                            \
            talk_mma_launch<DV, HPW, 32>(p, grid, s, q, k_pages, v_pages, out, part_o, part_ml, tiles, positions, token_req, block_table, table_width, \
                                         page_size, H, G, dk, window, scale, talk, sink);                                                         \
        else                                                                                                                                       \
            talk_mma_launch<DV, HPW, 16>(p, grid, s, q, k_pages, v_pages, out, part_o, part_ml, tiles, positions, token_req, block_table, table_width, \
                                         page_size, H, G, dk, window, scale, talk, sink);                                                         \
    } while (0)
    if (dv == 32) TALK_MMA(32, 2);
    else if (dv == 64) TALK_MMA(64, 2);
    else if (dv == 96) TALK_MMA(96, 1);
    else TALK_MMA(128, 1);
#undef TALK_MMA
    MM_CHECK_LAUNCH();
    if (splits > 1) {
        mm_launch(attention_talking_merge_kernel<__nv_bfloat16>, dim3(n_tokens * H), dim3(128), 0, s, (const float*)part_o, (const float*)part_ml,
                  (__nv_bfloat16*)out, splits, H, dv, (const float*)sink);
        MM_CHECK_LAUNCH();
    }
    return MM_OK;
}
