// Mixers that keep a matrix per head instead of keys and values: per head, with S a [dk, dv] matrix in fp32,
//
//   S <- g_t S;   u_t = v_t                      (plain)      or   u_t = beta_t (v_t - S^T k_t)   (delta rule);
//   S <- S + k_t u_t^T;   o_t = S^T q_t.
//
// g_t is a constant of the head (`head_decay`) or one number per token and head (`gate`).  Retention and lightning
// attention are the plain form with a constant decay, the gated delta rule is the second form with a decay per token.
// The state is carried per request in a state slot; a request at position 0 starts from zero whatever its slot holds.
//
// This file holds (1) the short causal convolution per channel whose last inputs are state too, (2) what happens to
// q, k and v between their projection and the recurrence (activation, rotation of half-split pairs, unit length,
// scale, and the decay per token and the write strength of the delta rule), all in fp32 and in place, and (3) the recurrence as a
// walk over each request's tokens.  Columns of S are independent of one another: a thread owns an eighth of one
// column, eight lanes add up the dot products of a token, and a block of 128 threads walks 16 columns of one head.  The layout of the state in a slot is [H, dv, dk]: what a warp reads is one run.
#include "common.cuh"

#define LS_MAX_TAPS 8
#define LS_AHEAD 16      // tokens staged in shared memory at a time
#define LS_COLS 16       // columns of S per block

__device__ __forceinline__ float ls_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ls_silu(float x) { return x * ls_sigmoid(x); }
__device__ __forceinline__ float ls_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------------------------
// short causal convolution over time, per channel, in place: y_t = act(sum_j taps[c][K-1-j] x_(t-j))
// ---------------------------------------------------------------------------------------------------------------
// x [n, ld] fp32 (the first C columns are convolved), taps [C, K] fp32 (last column: the current token), tail
// [slots, tail_stride] fp32 with the request's last K-1 inputs at [j * C + c], j = 0 the most recent.  One thread
// per (request, channel) walks the request's tokens with the last inputs in registers.
__global__ void causal_conv_walk_kernel(float* __restrict__ x, int ld, int C, const float* __restrict__ taps, int K,
                                        float* __restrict__ tail, long long tail_stride, const int32_t* __restrict__ req_meta,
                                        const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int act) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int t0 = req_meta ? req_meta[4 * r] : r;
    const int n = req_meta ? req_meta[4 * r + 1] : 1;
    float* tl = tail + (size_t)slots[r] * tail_stride;
    const bool fresh = positions[t0] == 0;
    float w[LS_MAX_TAPS], win[LS_MAX_TAPS];      // win[j]: the input j+1 tokens back
#pragma unroll
    for (int j = 0; j < LS_MAX_TAPS; ++j) {
        w[j] = j < K ? taps[(size_t)c * K + (K - 1 - j)] : 0.0f;      // w[j] multiplies the input j tokens back
        win[j] = (j < K - 1 && !fresh) ? tl[(size_t)j * C + c] : 0.0f;
    }
    for (int t = t0; t < t0 + n; ++t) {
        float* p = x + (size_t)t * ld + c;
        const float cur = *p;
        float y = w[0] * cur;
#pragma unroll
        for (int j = 1; j < LS_MAX_TAPS; ++j) y = fmaf(w[j], win[j - 1], y);
#pragma unroll
        for (int j = LS_MAX_TAPS - 1; j > 0; --j) win[j] = win[j - 1];
        win[0] = cur;
        *p = act ? ls_silu(y) : y;
    }
#pragma unroll
    for (int j = 0; j < LS_MAX_TAPS; ++j)
        if (j < K - 1) tl[(size_t)j * C + c] = win[j];
}

MM_EXPORT int mm_causal_conv_walk(void* x, int ld, int C, const void* taps, int K, void* tail, long long tail_stride,
                                  const void* req_meta, const void* slots, const void* positions, int n_requests, int act, void* stream) {
    MM_REQUIRE(C > 0 && ld >= C && K >= 1 && K <= LS_MAX_TAPS, "causal conv: 1 to 8 taps, and at least as many columns as channels");
    MM_REQUIRE((tail != nullptr || K == 1) && slots != nullptr && positions != nullptr, "causal conv: the state and the positions are needed");
    if (n_requests <= 0) return MM_OK;
    mm_launch(causal_conv_walk_kernel, dim3(ceil_div(C, 128), n_requests), dim3(128), 0, (cudaStream_t)stream, (float*)x, ld, C,
              (const float*)taps, K, (float*)tail, tail_stride, (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions, act);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// The same convolution for long portions, one thread per (token, channel): y (another buffer, [n, ldy]) gets the
// result, x stays as it is, and the state is read only; a second launch then leaves the request's last K-1 inputs in
// the state (one thread per (request, channel), which reads what it needs of the old state before it writes).
__global__ void causal_conv_tokens_kernel(const float* __restrict__ x, int ld, int C, const float* __restrict__ taps, int K,
                                          const float* __restrict__ tail, long long tail_stride, float* __restrict__ y, int ldy,
                                          const int32_t* __restrict__ token_req, const int32_t* __restrict__ req_meta,
                                          const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int act, int n_tokens) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * C) return;
    const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
    const int r = token_req[t];
    const int o = t - (req_meta ? req_meta[4 * r] : t);       // the token's place in its portion
    const int pos = positions[t];
    const float* tl = tail + (size_t)slots[r] * tail_stride;
    float acc = 0.0f;
    for (int j = 0; j < K; ++j) {
        if (pos - j < 0) break;                                // before the sequence's start: zeros
        const float in = (o - j >= 0) ? x[(size_t)(t - j) * ld + c] : tl[(size_t)(j - o - 1) * C + c];
        acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], in, acc);
    }
    y[(size_t)t * ldy + c] = act ? ls_silu(acc) : acc;
}

// The same per (token, 4 consecutive channels): a block owns 8 consecutive tokens x 128 channels, so the rows that
// neighbouring tokens share are read from DRAM once and from L1 after that; 16-byte loads and stores.  A channel's
// products are summed in the same order as above, so both forms give the same bits.
template <int K>
__global__ void __launch_bounds__(256) causal_conv_tokens4_kernel(
    const float* __restrict__ x, int ld, int C, const float* __restrict__ taps, const float* __restrict__ tail,
    long long tail_stride, float* __restrict__ y, int ldy, const int32_t* __restrict__ token_req, const int32_t* __restrict__ req_meta,
    const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int act, int n_tokens) {
    const int c = (blockIdx.x * 32 + (threadIdx.x & 31)) * 4;
    const int t = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (c >= C || t >= n_tokens) return;
    const int r = token_req[t];
    const int o = t - (req_meta ? req_meta[4 * r] : t);       // the token's place in its portion
    const int pos = positions[t];
    const float* tl = tail + (size_t)slots[r] * tail_stride;
    float4 in[K];                                              // every load is issued before the first product
#pragma unroll
    for (int j = 0; j < K; ++j) {
        in[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);           // before the sequence's start: zeros (a product with zero adds nothing)
        if (pos - j >= 0)
            in[j] = (o - j >= 0) ? *reinterpret_cast<const float4*>(x + (size_t)(t - j) * ld + c)
                                 : *reinterpret_cast<const float4*>(tl + (size_t)(j - o - 1) * C + c);
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < K; ++j) {
        const float* w = taps + (size_t)c * K + (K - 1 - j);
        acc[0] = fmaf(w[0], in[j].x, acc[0]);
        acc[1] = fmaf(w[K], in[j].y, acc[1]);
        acc[2] = fmaf(w[2 * K], in[j].z, acc[2]);
        acc[3] = fmaf(w[3 * K], in[j].w, acc[3]);
    }
    if (act) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = ls_silu(acc[e]);
    }
    *reinterpret_cast<float4*>(y + (size_t)t * ldy + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

__global__ void causal_conv_tail_kernel(const float* __restrict__ x, int ld, int C, int K, float* __restrict__ tail, long long tail_stride,
                                        const int32_t* __restrict__ req_meta, const int32_t* __restrict__ slots,
                                        const int32_t* __restrict__ positions) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int t0 = req_meta ? req_meta[4 * r] : r;
    const int n = req_meta ? req_meta[4 * r + 1] : 1;
    float* tl = tail + (size_t)slots[r] * tail_stride;
    const bool fresh = positions[t0] == 0;
    float keep[LS_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < LS_MAX_TAPS; ++j) {
        keep[j] = 0.0f;
        if (j < K - 1) keep[j] = j < n ? x[(size_t)(t0 + n - 1 - j) * ld + c] : (fresh ? 0.0f : tl[(size_t)(j - n) * C + c]);
    }
#pragma unroll
    for (int j = 0; j < LS_MAX_TAPS; ++j)
        if (j < K - 1) tl[(size_t)j * C + c] = keep[j];
}

MM_EXPORT int mm_causal_conv_tokens(const void* x, int ld, int C, const void* taps, int K, void* tail, long long tail_stride, void* y, int ldy,
                                    const void* token_req, const void* req_meta, const void* slots, const void* positions, int n_tokens,
                                    int n_requests, int act, void* stream) {
    MM_REQUIRE(C > 0 && ld >= C && ldy >= C && K >= 1 && K <= LS_MAX_TAPS, "causal conv: 1 to 8 taps, and at least as many columns as channels");
    MM_REQUIRE((tail != nullptr || K == 1) && slots != nullptr && positions != nullptr && token_req != nullptr && y != nullptr && y != x,
               "causal conv: the state, the positions, the tokens' requests and a result buffer of its own are needed");
    if (n_tokens <= 0 || n_requests <= 0) return MM_OK;
    const bool by4 = C % 4 == 0 && ld % 4 == 0 && ldy % 4 == 0 && tail_stride % 4 == 0 && ceil_div(n_tokens, 8) <= 65535 &&
                     (((uintptr_t)x | (uintptr_t)y | (uintptr_t)tail) & 15) == 0;
    if (by4) {
#define CONV4_CASE(KK)                                                                                                                  \
    case KK:                                                                                                                            \
        mm_launch(causal_conv_tokens4_kernel<KK>, dim3(ceil_div(C, 128), ceil_div(n_tokens, 8)), dim3(256), 0, (cudaStream_t)stream,     \
                  (const float*)x, ld, C, (const float*)taps, (const float*)tail, tail_stride, (float*)y, ldy, (const int32_t*)token_req, \
                  (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions, act, n_tokens);                            \
        break;
        switch (K) {
            CONV4_CASE(1) CONV4_CASE(2) CONV4_CASE(3) CONV4_CASE(4) CONV4_CASE(5) CONV4_CASE(6) CONV4_CASE(7) CONV4_CASE(8)
            default: break;
        }
#undef CONV4_CASE
    } else {
        mm_launch(causal_conv_tokens_kernel, dim3(ceil_div((long long)n_tokens * C, 256)), dim3(256), 0, (cudaStream_t)stream, (const float*)x, ld, C,
                  (const float*)taps, K, (const float*)tail, tail_stride, (float*)y, ldy, (const int32_t*)token_req, (const int32_t*)req_meta,
                  (const int32_t*)slots, (const int32_t*)positions, act, n_tokens);
    }
    MM_CHECK_LAUNCH();
    if (K > 1) {
        mm_launch(causal_conv_tail_kernel, dim3(ceil_div(C, 128), n_requests), dim3(128), 0, (cudaStream_t)stream, (const float*)x, ld, C, K,
                  (float*)tail, tail_stride, (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions);
        MM_CHECK_LAUNCH();
    }
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// between projection and recurrence, in place on the fp32 rows of the projection
// ---------------------------------------------------------------------------------------------------------------
// Row t of x holds q at q_off (Gq heads of dk), k at k_off (Gq heads of dk) and v at v_off (n_v numbers).  In this
// order: act (1: silu on q, k and v); rotation of the pairs (i, i + rot_dims/2) of every q and k head by the angles
// of rot[t] (cos, sin per pair; made from the positions once per step); unit length (x / sqrt(sum x^2 + unit_eps))
// when `unit`; q *= q_scale, k *= k_scale.  With a_off >= 0 also a decay per token and head,
// gate = exp(-exp(A_log) softplus(a + dt_bias)), and with b_off >= 0 the delta rule's write strength, beta = sigmoid(b),
// from the columns a_off.. and b_off.. of the row of gx (row stride gld; null: of x itself).
__global__ void linear_state_prep_kernel(float* __restrict__ x, int ld, int q_off, int k_off, int v_off, int Gq, int dk, int n_v,
                                         int act, const float2* __restrict__ rot, int rot_dims, int unit, float unit_eps,
                                         float q_scale, float k_scale, const float* __restrict__ gx, int gld, int a_off, int b_off, int H,
                                         const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ gate,
                                         float* __restrict__ beta) {
    extern __shared__ float prep_smem[];             // one vector of dk per warp: a head is read once and written once
    const int t = blockIdx.x;
    float* row = x + (size_t)t * ld;
    const float* grow = gx + (size_t)t * gld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int half = rot_dims / 2;
    float* sv = prep_smem + warp * dk;
    for (int vec = warp; vec < 2 * Gq; vec += warps) {
        const bool is_q = vec < Gq;
        float* p = row + (is_q ? q_off + vec * dk : k_off + (vec - Gq) * dk);
        for (int d = lane; d < dk; d += 32) sv[d] = act ? ls_silu(p[d]) : p[d];
        __syncwarp();
        if (rot_dims) {
            const float2* cs = rot + (size_t)t * half;
            for (int i = lane; i < half; i += 32) {
                const float a = sv[i], b = sv[i + half];
                sv[i] = a * cs[i].x - b * cs[i].y;
                sv[i + half] = b * cs[i].x + a * cs[i].y;
            }
            __syncwarp();
        }
        float f = is_q ? q_scale : k_scale;
        if (unit) {
            float ss = 0.0f;
            for (int d = lane; d < dk; d += 32) ss = fmaf(sv[d], sv[d], ss);
            ss = warp_sum(ss);
            f *= 1.0f / sqrtf(ss + unit_eps);
        }
        for (int d = lane; d < dk; d += 32) p[d] = f != 1.0f ? sv[d] * f : sv[d];
        __syncwarp();
    }
    if (act)
        for (int d = threadIdx.x; d < n_v; d += blockDim.x) row[v_off + d] = ls_silu(row[v_off + d]);
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        if (a_off >= 0) gate[(size_t)t * H + h] = expf(-expf(A_log[h]) * ls_softplus(grow[a_off + h] + dt_bias[h]));
        if (b_off >= 0) beta[(size_t)t * H + h] = ls_sigmoid(grow[b_off + h]);
    }
}

MM_EXPORT int mm_linear_state_prep(void* x, int ld, int n_tokens, int q_off, int k_off, int v_off, int Gq, int dk, int n_v, int act,
                                   const void* rot, int rot_dims, int unit, float unit_eps, float q_scale, float k_scale, const void* gx,
                                   int gld, int a_off, int b_off, int H, const void* A_log, const void* dt_bias, void* gate, void* beta,
                                   void* stream) {
    if (gx == nullptr) {
        gx = x;
        gld = ld;
    }
    MM_REQUIRE(n_tokens >= 0 && Gq > 0 && dk > 0 && n_v >= 0 && ld > 0, "linear state prep: bad sizes");
    MM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || rot != nullptr), "linear state prep: the rotated dimensions must be even, at most the head size, and have their table");
    MM_REQUIRE(a_off < 0 || (H > 0 && A_log && dt_bias && gate), "linear state prep: the decay per token needs its inputs and its output");
    MM_REQUIRE(b_off < 0 || (H > 0 && beta), "linear state prep: the write strength needs its output");
    if (a_off < 0 && b_off < 0) H = 0;
    if (n_tokens == 0) return MM_OK;
    MM_REQUIRE(dk <= 1024, "linear state prep: key sizes above 1024 are not supported");
    mm_launch(linear_state_prep_kernel, dim3(n_tokens), dim3(256), (size_t)8 * dk * sizeof(float), (cudaStream_t)stream, (float*)x, ld, q_off, k_off, v_off, Gq, dk, n_v, act,
              (const float2*)rot, rot_dims, unit, unit_eps, q_scale, k_scale, (const float*)gx, gld, a_off, b_off, H, (const float*)A_log,
              (const float*)dt_bias,
              (float*)gate, (float*)beta);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// (cos, sin) of position * freq[i] for every token and pair, fp32
__global__ void angle_table_kernel(const int32_t* __restrict__ positions, const float* __restrict__ freq, float2* __restrict__ table,
                                   int n_tokens, int half) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * half) return;
    const int t = (int)(i / half), p = (int)(i - (long long)t * half);
    float sn, cs;
    sincosf((float)positions[t] * freq[p], &sn, &cs);
    table[i] = make_float2(cs, sn);
}

MM_EXPORT int mm_angle_table(const void* positions, const void* freq, void* table, int n_tokens, int half, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && half > 0, "angle table: bad sizes");
    if (n_tokens == 0) return MM_OK;
    mm_launch(angle_table_kernel, dim3(ceil_div((long long)n_tokens * half, 256)), dim3(256), 0, (cudaStream_t)stream,
              (const int32_t*)positions, (const float*)freq, (float2*)table, n_tokens, half);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// the recurrence, token by token
// ---------------------------------------------------------------------------------------------------------------
// q, k: fp32 rows with Gq heads of dk (row strides ldq, ldk); v: fp32 rows with H heads of dv (ldv); head h reads
// q/k head h / (H / Gq).  gate, beta: [n, H] fp32 or null; head_decay [H] fp32 (used when gate is null).
// out [n, H*dv] fp32.  state: the slot's S as [H, dv, dk] at `state`, slots `state_stride` floats apart.
//
// A thread's entries of its column are i = 32 (e / 4) + 4 (lane % 8) + e % 4, e < PER: the eight lanes of a column
// read q and k of a token as 16-byte words without bank conflicts.  The tokens of a request come in batches of
// LS_AHEAD through two shared-memory buffers filled by asynchronous copies, so a batch's loads run under the batch
// before it; within a batch nothing but the eight-lane sums synchronises, and the loop over tokens is unrolled so
// that the sums of neighbouring tokens overlap (without the delta rule only S itself is carried from token to token).
__device__ __forceinline__ void ls_cp_async4(void* smem, const void* gmem) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem));
}
__device__ __forceinline__ void ls_cp_async16(void* smem, const void* gmem) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem));
}
__device__ __forceinline__ void ls_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void ls_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

//
// MODE 0: a request's tokens from its slot's state, which is left updated.  Long portions without the delta rule are cut
// into chunks that are walked side by side (the state's update is linear: S_end = (product of the decays) S_start + what
// the chunk adds): MODE 1 walks chunk blockIdx.z from zero and leaves what it adds, and the product of its decays, in
// scratch; a carry kernel then walks each request's chunks in order, leaves every chunk's starting state in scratch and
// the last state in the slot; MODE 2 walks every chunk again from its starting state and writes the outputs.
// CPT: columns per thread (a thread of the chunk passes owns two columns, 16 apart, and reads q and k once for both: those
// passes are bound by the shared-memory reads)
template <int PER, bool DELTA, int MODE, int CPT>
__global__ void __launch_bounds__(128) linear_state_walk_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ldq, int ldk, int ldv,
    const float* __restrict__ gate, const float* __restrict__ beta, const float* __restrict__ head_decay, float* __restrict__ out,
    float* __restrict__ state, long long state_stride, const int32_t* __restrict__ req_meta, const int32_t* __restrict__ slots,
    const int32_t* __restrict__ positions, int H, int Gq, int dk, int dv, int vec_ok, float* __restrict__ chunk_gain) {
    constexpr int DKP = 8 * PER;
    constexpr int COLS = LS_COLS * CPT;
    constexpr int STAGE = LS_AHEAD * (2 * DKP + COLS + 2);      // floats of one buffer: q, k, v, decay, write strength
    extern __shared__ __align__(16) float ls_smem[];
    float* so = ls_smem + 2 * STAGE;                               // [AHEAD][COLS]
    float* skq = so + LS_AHEAD * COLS;                          // [AHEAD] k . q of the batch's tokens

    const int h = blockIdx.y, r = blockIdx.z;
    const int col0 = blockIdx.x * COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ks = lane & 7, cl = warp * 4 + (lane >> 3);
    bool col_ok[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) col_ok[c] = col0 + cl + 16 * c < dv;
    const int gq = h / (H / Gq);
    // MODE 1, 2: r is a chunk, req_meta the chunk list (first token, tokens, ., .), state the scratch with one matrix set per chunk
    const int t0 = req_meta ? req_meta[4 * r] : r;
    const int n = req_meta ? req_meta[4 * r + 1] : 1;
    float* st[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
        st[c] = state + (size_t)(MODE == 0 ? slots[r] : r) * state_stride + ((size_t)h * dv + (col_ok[c] ? col0 + cl + 16 * c : 0)) * dk;
    const bool fresh = MODE == 1 || (MODE == 0 && positions[t0] == 0);
    const float hd = head_decay ? head_decay[h] : 1.0f;
    float gain = 1.0f;

    float S[CPT][PER];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int i = (e >> 2) * 32 + ks * 4 + (e & 3);
            S[c][e] = (col_ok[c] && i < dk && !fresh) ? st[c][i] : 0.0f;
        }
    // what no copy writes (entries beyond dk, columns beyond dv) stays zero in both buffers
    for (int i = threadIdx.x; i < 2 * STAGE; i += 128) ls_smem[i] = 0.0f;
    __syncthreads();

    auto fill = [&](int buf, int base) {
        float* sq = ls_smem + buf * STAGE;
        float* sk = sq + LS_AHEAD * DKP;
        float* sv = sk + LS_AHEAD * DKP;
        float* sg = sv + LS_AHEAD * COLS;
        float* sb = sg + LS_AHEAD;
        const int cnt = min(LS_AHEAD, n - base);
        if (vec_ok) {
            const int per_row = dk >> 2;
            for (int idx = threadIdx.x; idx < cnt * per_row; idx += 128) {
                const int tt = idx / per_row, i = (idx - tt * per_row) * 4;
                const size_t t = (size_t)(t0 + base + tt);
                ls_cp_async16(sq + tt * DKP + i, q + t * ldq + gq * dk + i);
                ls_cp_async16(sk + tt * DKP + i, k + t * ldk + gq * dk + i);
            }
            const int vcols = min(COLS, dv - col0) >> 2;
            for (int idx = threadIdx.x; idx < cnt * vcols; idx += 128) {
                const int tt = idx / vcols, c = (idx - tt * vcols) * 4;
                ls_cp_async16(sv + tt * COLS + c, v + (size_t)(t0 + base + tt) * ldv + h * dv + col0 + c);
            }
        } else {
            for (int idx = threadIdx.x; idx < cnt * dk; idx += 128) {
                const int tt = idx / dk, i = idx - tt * dk;
                const size_t t = (size_t)(t0 + base + tt);
                ls_cp_async4(sq + tt * DKP + i, q + t * ldq + gq * dk + i);
                ls_cp_async4(sk + tt * DKP + i, k + t * ldk + gq * dk + i);
            }
            const int vcols = min(COLS, dv - col0);
            for (int idx = threadIdx.x; idx < cnt * vcols; idx += 128) {
                const int tt = idx / vcols, c = idx - tt * vcols;
                ls_cp_async4(sv + tt * COLS + c, v + (size_t)(t0 + base + tt) * ldv + h * dv + col0 + c);
            }
        }
        if (threadIdx.x < cnt) {
            const size_t t = (size_t)(t0 + base + threadIdx.x);
            if (gate) ls_cp_async4(sg + threadIdx.x, gate + t * H + h);
            else sg[threadIdx.x] = hd;
            if (DELTA) ls_cp_async4(sb + threadIdx.x, beta + t * H + h);
        }
        ls_cp_commit();
    };

    fill(0, 0);
    int buf = 0;
    for (int base = 0; base < n; base += LS_AHEAD, buf ^= 1) {
        const int cnt = min(LS_AHEAD, n - base);
        if (base + LS_AHEAD < n) {
            fill(buf ^ 1, base + LS_AHEAD);
            ls_cp_wait<1>();
        } else {
            ls_cp_wait<0>();
        }
        __syncthreads();
        const float* sq = ls_smem + buf * STAGE;
        const float* sk = sq + LS_AHEAD * DKP;
        const float* sv = sk + LS_AHEAD * DKP;
        const float* sg = sv + LS_AHEAD * COLS;
        const float* sb = sg + LS_AHEAD;
        if (MODE != 1) {
            // k . q of every token of the batch, once for all columns: a warp takes every fourth token
            for (int tt = warp; tt < cnt; tt += 4) {
                float d = 0.0f;
                for (int i = lane; i < DKP; i += 32) d = fmaf(sk[tt * DKP + i], sq[tt * DKP + i], d);
                d = warp_sum(d);
                if (lane == 0) skq[tt] = d;
            }
            __syncthreads();
        }
#pragma unroll 4
        for (int tt = 0; tt < cnt; ++tt) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DKP) + ks;
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * DKP) + ks;
            float kk[PER];
            float dq[CPT][4], dkk[CPT][4];
#pragma unroll
            for (int c = 0; c < CPT; ++c)
#pragma unroll
                for (int x = 0; x < 4; ++x) dq[c][x] = dkk[c][x] = 0.0f;
#pragma unroll
            for (int j = 0; j < PER / 4; ++j) {
                const float4 qv = q4[j * 8], kv = k4[j * 8];
                kk[4 * j] = kv.x; kk[4 * j + 1] = kv.y; kk[4 * j + 2] = kv.z; kk[4 * j + 3] = kv.w;
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    dq[c][0] = fmaf(S[c][4 * j], qv.x, dq[c][0]); dq[c][1] = fmaf(S[c][4 * j + 1], qv.y, dq[c][1]);
                    dq[c][2] = fmaf(S[c][4 * j + 2], qv.z, dq[c][2]); dq[c][3] = fmaf(S[c][4 * j + 3], qv.w, dq[c][3]);
                    if (DELTA) {
                        dkk[c][0] = fmaf(S[c][4 * j], kv.x, dkk[c][0]); dkk[c][1] = fmaf(S[c][4 * j + 1], kv.y, dkk[c][1]);
                        dkk[c][2] = fmaf(S[c][4 * j + 2], kv.z, dkk[c][2]); dkk[c][3] = fmaf(S[c][4 * j + 3], kv.w, dkk[c][3]);
                    }
                }
            }
            const float g = sg[tt];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float sdq = (dq[c][0] + dq[c][1]) + (dq[c][2] + dq[c][3]);
                float sdk = DELTA ? (dkk[c][0] + dkk[c][1]) + (dkk[c][2] + dkk[c][3]) : 0.0f;
                if (MODE != 1) {
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) {
                        if (DELTA) sdk += __shfl_xor_sync(0xffffffffu, sdk, o);
                        sdq += __shfl_xor_sync(0xffffffffu, sdq, o);
                    }
                }
                const float vv = sv[tt * COLS + cl + 16 * c];
                const float u = DELTA ? sb[tt] * (vv - g * sdk) : vv;
#pragma unroll
                for (int e = 0; e < PER; ++e) S[c][e] = fmaf(kk[e], u, g * S[c][e]);
                if (MODE != 1 && ks == 0) so[tt * COLS + cl + 16 * c] = fmaf(u, skq[tt], g * sdq);     // S_new^T q = g S_old^T q + u (k . q)
            }
            if (MODE == 1) gain *= g;
        }
        __syncthreads();
        if (MODE != 1)
            for (int idx = threadIdx.x; idx < cnt * COLS; idx += 128) {
                const int tt = idx / COLS, c = idx - tt * COLS;
                if (col0 + c < dv) out[(size_t)(t0 + base + tt) * H * dv + h * dv + col0 + c] = so[idx];
            }
    }
    if (MODE == 1 && blockIdx.x == 0 && threadIdx.x == 0) chunk_gain[(size_t)r * H + h] = gain;
    if (MODE == 2) return;
#pragma unroll
    for (int c = 0; c < CPT; ++c)
        if (col_ok[c]) {
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int i = (e >> 2) * 32 + ks * 4 + (e & 3);
                if (i < dk) st[c][i] = S[c][e];
            }
        }
}

template <int PER, bool DELTA, int MODE, int CPT>
static void ls_walk_launch_one(dim3 grid, cudaStream_t s, const float* q, const float* k, const float* v, int ldq, int ldk, int ldv,
                               const float* gate, const float* beta, const float* head_decay, float* out, float* state, long long state_stride,
                               const int32_t* req_meta, const int32_t* slots, const int32_t* positions, int H, int Gq, int dk, int dv, int vec_ok,
                               float* chunk_gain) {
    auto kernel = linear_state_walk_kernel<PER, DELTA, MODE, CPT>;
    const size_t smem = sizeof(float) * (2 * LS_AHEAD * (2 * 8 * PER + LS_COLS * CPT + 2) + LS_AHEAD * LS_COLS * CPT + LS_AHEAD);
    grid.x = (dv + LS_COLS * CPT - 1) / (LS_COLS * CPT);
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mm_launch(kernel, grid, dim3(128), smem, s, q, k, v, ldq, ldk, ldv, gate, beta, head_decay, out, state, state_stride, req_meta, slots,
              positions, H, Gq, dk, dv, vec_ok, chunk_gain);
}

// mode 0 with or without the delta rule; modes 1 and 2 (chunks) without it
template <int PER>
static void ls_walk_launch(bool delta, int mode, dim3 grid, cudaStream_t s, const float* q, const float* k, const float* v, int ldq, int ldk, int ldv,
                           const float* gate, const float* beta, const float* head_decay, float* out, float* state, long long state_stride,
                           const int32_t* req_meta, const int32_t* slots, const int32_t* positions, int H, int Gq, int dk, int dv,
                           float* chunk_gain) {
    // 16-byte copies where every row and head of q, k and v starts on a 16-byte boundary, 4-byte copies otherwise
    const int vec_ok = dk % 4 == 0 && dv % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ldv % 4 == 0 &&
                       (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0;
#define LS_ONE(D, M, C) ls_walk_launch_one<PER, D, M, C>(grid, s, q, k, v, ldq, ldk, ldv, gate, beta, head_decay, out, state, state_stride, req_meta, \
                                                   slots, positions, H, Gq, dk, dv, vec_ok, chunk_gain)
    if (mode == 1) LS_ONE(false, 1, 2);
    else if (mode == 2) LS_ONE(false, 2, 2);
    else if (delta) LS_ONE(true, 0, 1);
    else LS_ONE(false, 0, 1);
#undef LS_ONE
}

MM_EXPORT int mm_linear_state_walk(const void* q, const void* k, const void* v, int ldq, int ldk, int ldv, const void* gate,
                                   const void* beta, const void* head_decay, void* out, void* state, long long state_stride,
                                   const void* req_meta, const void* slots, const void* positions, int n_requests, int H, int Gq,
                                   int dk, int dv, void* stream) {
    MM_REQUIRE(H > 0 && Gq > 0 && H % Gq == 0 && dk > 0 && dv > 0, "linear state: heads must be a positive multiple of the q/k heads");
    MM_REQUIRE(dk <= 256, "linear state: key sizes above 256 are not supported");
    MM_REQUIRE(gate != nullptr || head_decay != nullptr, "linear state: a decay per token or per head is needed");
    MM_REQUIRE(state != nullptr && slots != nullptr && positions != nullptr, "linear state: the state and the positions are needed");
    if (n_requests <= 0) return MM_OK;
    const bool delta = beta != nullptr;
    const dim3 grid(ceil_div(dv, LS_COLS), H, n_requests);
    cudaStream_t s = (cudaStream_t)stream;
#define LS_ARGS delta, 0, grid, s, (const float*)q, (const float*)k, (const float*)v, ldq, ldk, ldv, (const float*)gate, (const float*)beta, \
                (const float*)head_decay, (float*)out, (float*)state, state_stride, (const int32_t*)req_meta, (const int32_t*)slots,       \
                (const int32_t*)positions, H, Gq, dk, dv, (float*)nullptr
    if (dk <= 32) ls_walk_launch<4>(LS_ARGS);
    else if (dk <= 64) ls_walk_launch<8>(LS_ARGS);
    else if (dk <= 96) ls_walk_launch<12>(LS_ARGS);
    else if (dk <= 128) ls_walk_launch<16>(LS_ARGS);
    else ls_walk_launch<32>(LS_ARGS);
#undef LS_ARGS
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// The carry between the two chunk passes: thread per number of the state.  chunk_meta [chunks, 4] = (first token, tokens,
// request, .), req_chunks [requests, 2] = (first chunk, chunks); scratch [chunks, H * dv * dk] holds what every chunk adds
// and gets what every chunk starts from; gain [chunks, H].
__global__ void linear_state_carry_kernel(float* __restrict__ scratch, const float* __restrict__ gain, float* __restrict__ state,
                                          long long state_stride, const int32_t* __restrict__ chunk_meta, const int32_t* __restrict__ req_chunks,
                                          const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int H, int per_head, long long size) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (i >= size) return;
    const int h = (int)(i / per_head);
    const int first = req_chunks[2 * r], count = req_chunks[2 * r + 1];
    float* st = state + (size_t)slots[r] * state_stride + i;
    float S = positions[chunk_meta[4 * first]] == 0 ? 0.0f : *st;
    // eight chunks' loads in flight at a time: they do not depend on the carried value
    for (int c0 = first; c0 < first + count; c0 += 8) {
        float add[8], gn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool in = c0 + j < first + count;
            add[j] = in ? scratch[(size_t)(c0 + j) * size + i] : 0.0f;
            gn[j] = in ? gain[(size_t)(c0 + j) * H + h] : 1.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (c0 + j < first + count) {
                scratch[(size_t)(c0 + j) * size + i] = S;
                S = fmaf(gn[j], S, add[j]);
            }
        }
    }
    *st = S;
}

// Long portions without the delta rule, chunk by chunk (three launches).  scratch: fp32 [chunks, H * dv * dk], gain: fp32 [chunks, H].
MM_EXPORT int mm_linear_state_chunked(const void* q, const void* k, const void* v, int ldq, int ldk, int ldv, const void* gate,
                                      const void* head_decay, void* out, void* state, long long state_stride, const void* chunk_meta,
                                      const void* req_chunks, const void* slots, const void* positions, int n_requests, int n_chunks, int H,
                                      int Gq, int dk, int dv, void* scratch, void* gain, void* stream) {
    MM_REQUIRE(H > 0 && Gq > 0 && H % Gq == 0 && dk > 0 && dv > 0 && dk <= 256, "linear state: heads must be a positive multiple of the q/k heads, keys at most 256");
    MM_REQUIRE(gate != nullptr || head_decay != nullptr, "linear state: a decay per token or per head is needed");
    MM_REQUIRE(state && slots && positions && chunk_meta && req_chunks && scratch && gain, "linear state: the chunked walk needs its lists and its scratch");
    if (n_requests <= 0 || n_chunks <= 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long size = (long long)H * dv * dk;
    const dim3 grid(ceil_div(dv, LS_COLS), H, n_chunks);
    for (int mode = 1; mode <= 2; ++mode) {
#define LS_ARGS false, mode, grid, s, (const float*)q, (const float*)k, (const float*)v, ldq, ldk, ldv, (const float*)gate, (const float*)nullptr, \
                (const float*)head_decay, (float*)out, (float*)scratch, size, (const int32_t*)chunk_meta, (const int32_t*)slots,               \
                (const int32_t*)positions, H, Gq, dk, dv, (float*)gain
        if (dk <= 32) ls_walk_launch<4>(LS_ARGS);
        else if (dk <= 64) ls_walk_launch<8>(LS_ARGS);
        else if (dk <= 96) ls_walk_launch<12>(LS_ARGS);
        else if (dk <= 128) ls_walk_launch<16>(LS_ARGS);
        else ls_walk_launch<32>(LS_ARGS);
#undef LS_ARGS
        MM_CHECK_LAUNCH();
        if (mode == 1) {
            mm_launch(linear_state_carry_kernel, dim3(ceil_div(size, 256), n_requests), dim3(256), 0, s, (float*)scratch, (const float*)gain,
                      (float*)state, state_stride, (const int32_t*)chunk_meta, (const int32_t*)req_chunks, (const int32_t*)slots,
                      (const int32_t*)positions, H, dv * dk, size);
            MM_CHECK_LAUNCH();
        }
    }
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// a forget gate per key channel whose complement is the write strength (HGRN2)
// ---------------------------------------------------------------------------------------------------------------
//   f_t = l + (1 - l) sigmoid(z_t + b)    per head and key channel, with a lower bound l per channel;
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;    o_t = S_t^T q_t.
// The key of the general recurrence is tied to the decay, which is a vector over the rows of S instead of one number.
//
// Between the projection and the recurrence, in place on the fp32 rows x [n, ld]: act_q (1: silu) on the n_qf numbers at
// q_off, and the n_qf numbers at f_off become the forget gate from the bias and the lower bound (fp32 [n_qf], bias null: 0).
__global__ void forget_gate_prep_kernel(float* __restrict__ x, int ld, long long total, int q_off, int f_off, int n_qf, int act_q,
                                        const float* __restrict__ bias, const float* __restrict__ lower) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / n_qf;
    const int c = (int)(i - t * n_qf);
    float* row = x + (size_t)t * ld;
    if (act_q) row[q_off + c] = ls_silu(row[q_off + c]);
    const float l = lower ? lower[c] : 0.0f;
    row[f_off + c] = l + (1.0f - l) * ls_sigmoid(row[f_off + c] + (bias ? bias[c] : 0.0f));
}

MM_EXPORT int mm_forget_gate_prep(void* x, int ld, int n_tokens, int q_off, int f_off, int n_qf, int act_q, const void* bias, const void* lower,
                                  void* stream) {
    MM_REQUIRE(n_tokens >= 0 && n_qf > 0 && q_off >= 0 && f_off >= 0 && q_off + n_qf <= ld && f_off + n_qf <= ld, "forget gate: columns outside the row");
    if (n_tokens == 0) return MM_OK;
    const long long total = (long long)n_tokens * n_qf;
    mm_launch(forget_gate_prep_kernel, dim3(ceil_div(total, 256)), dim3(256), 0, (cudaStream_t)stream, (float*)x, ld, total, q_off, f_off, n_qf, act_q,
              (const float*)bias, (const float*)lower);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// The walk: q, f fp32 rows with H heads of dk (row strides ldq, ldf), v with H heads of dv.  A block of 8 warps owns 32
// columns of one head's S for one request (or chunk); eight lanes share a column, lane `ks` of them the entries
// i = 32 (e / 4) + 4 ks + e % 4, e < PER, so that q and f of a token are read as 16-byte words without bank conflicts and
// a token's read-out is a sum over eight lanes.  q, f and v of FG_AHEAD tokens at a time are staged in shared memory (rows
// padded to 8 PER numbers; q is zero beyond dk, so the padding adds nothing).  The state's layout in a slot is [H, dv, dk],
// as in the walk above; a request at position 0 starts from zero whatever its slot holds.
#define FG_AHEAD 16
#define FG_COLS 32
// MODE 0: a request's tokens from its slot's state, which is left updated.  Long portions are cut into chunks that are walked
// side by side, because the update is linear in S with a diagonal transition (S_end = diag(product of the f) S_start + what
// the chunk adds): MODE 1 walks chunk blockIdx.z from zero and leaves what it adds in scratch (the products of the gates per
// key channel are made by a kernel of their own); a carry kernel walks each request's chunks in order, leaves every chunk's
// starting state in scratch and the last state in the slot; MODE 2 walks every chunk again from its starting state and
// writes the outputs.
template <int PER, int MODE>
__global__ void __launch_bounds__(256) forget_gate_walk_kernel(const float* __restrict__ q, const float* __restrict__ f, const float* __restrict__ v,
                                                               int ldq, int ldf, int ldv, float* __restrict__ out, float* __restrict__ state,
                                                               long long state_stride, const int32_t* __restrict__ req_meta,
                                                               const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int H,
                                                               int dk, int dv) {
    constexpr int DKP = 8 * PER;
    extern __shared__ __align__(16) float fg_smem[];
    float* sq = fg_smem;                          // [AHEAD][DKP]
    float* sf = sq + FG_AHEAD * DKP;              // [AHEAD][DKP]
    float* sv = sf + FG_AHEAD * DKP;              // [AHEAD][COLS]
    float* so = sv + FG_AHEAD * FG_COLS;          // [AHEAD][COLS]
    const int h = blockIdx.y, r = blockIdx.z, col0 = blockIdx.x * FG_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ks = lane & 7, cl = warp * 4 + (lane >> 3);
    const int col = col0 + cl;
    const bool col_ok = col < dv;
    const int t0 = req_meta ? req_meta[4 * r] : r;
    const int n = req_meta ? req_meta[4 * r + 1] : 1;
    const bool fresh = MODE == 1 || (MODE == 0 && positions[t0] == 0);
    // MODE 1, 2: r is a chunk, req_meta the chunk list, state the scratch with one set of matrices per chunk
    float* st = state + (size_t)(MODE == 0 ? slots[r] : r) * state_stride + ((size_t)h * dv + (col_ok ? col : 0)) * dk;
    float S[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int i = (e >> 2) * 32 + ks * 4 + (e & 3);
        S[e] = (!fresh && col_ok && i < dk) ? st[i] : 0.0f;
    }
    for (int i = threadIdx.x; i < 2 * FG_AHEAD * DKP; i += 256) fg_smem[i] = 0.0f;      // what no copy writes stays zero
    for (int base = 0; base < n; base += FG_AHEAD) {
        const int cnt = min(FG_AHEAD, n - base);
        __syncthreads();
        for (int idx = threadIdx.x; idx < cnt * dk; idx += 256) {
            const int tt = idx / dk, i = idx - tt * dk;
            const size_t t = (size_t)(t0 + base + tt);
            sq[tt * DKP + i] = q[t * ldq + h * dk + i];
            sf[tt * DKP + i] = f[t * ldf + h * dk + i];
        }
        for (int idx = threadIdx.x; idx < cnt * FG_COLS; idx += 256) {
            const int tt = idx / FG_COLS, c = idx - tt * FG_COLS;
            sv[idx] = col0 + c < dv ? v[(size_t)(t0 + base + tt) * ldv + h * dv + col0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < cnt; ++tt) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DKP) + ks;
            const float4* f4 = reinterpret_cast<const float4*>(sf + tt * DKP) + ks;
            const float vv = sv[tt * FG_COLS + cl];
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
            for (int j = 0; j < PER / 4; ++j) {
                const float4 fv = f4[j * 8];
                S[4 * j] = fmaf(fv.x, S[4 * j], (1.0f - fv.x) * vv);
                S[4 * j + 1] = fmaf(fv.y, S[4 * j + 1], (1.0f - fv.y) * vv);
                S[4 * j + 2] = fmaf(fv.z, S[4 * j + 2], (1.0f - fv.z) * vv);
                S[4 * j + 3] = fmaf(fv.w, S[4 * j + 3], (1.0f - fv.w) * vv);
                if (MODE != 1) {
                    const float4 qv = q4[j * 8];
                    d0 = fmaf(S[4 * j], qv.x, d0);
                    d1 = fmaf(S[4 * j + 1], qv.y, d1);
                    d2 = fmaf(S[4 * j + 2], qv.z, d2);
                    d3 = fmaf(S[4 * j + 3], qv.w, d3);
                }
            }
            if (MODE != 1) {
                float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (ks == 0) so[tt * FG_COLS + cl] = dot;
            }
        }
        __syncthreads();
        if (MODE != 1)
            for (int idx = threadIdx.x; idx < cnt * FG_COLS; idx += 256) {
                const int tt = idx / FG_COLS, c = idx - tt * FG_COLS;
                if (col0 + c < dv) out[(size_t)(t0 + base + tt) * H * dv + h * dv + col0 + c] = so[idx];
            }
    }
    if (MODE == 2 || !col_ok) return;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int i = (e >> 2) * 32 + ks * 4 + (e & 3);
        if (i < dk) st[i] = S[e];
    }
}

// The product of a chunk's gates per head and key channel: gain [chunks, H * dk]; f fp32 rows with row stride ldf.
__global__ void forget_gate_gain_kernel(const float* __restrict__ f, int ldf, const int32_t* __restrict__ chunk_meta, float* __restrict__ gain, int width) {
    const int c = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= width) return;
    const int t0 = chunk_meta[4 * c], n = chunk_meta[4 * c + 1];
    float p = 1.0f;
    for (int t = 0; t < n; ++t) p *= f[(size_t)(t0 + t) * ldf + i];
    gain[(size_t)c * width + i] = p;
}

template <int MODE>
static void fg_walk_launch(dim3 grid, cudaStream_t s, const float* q, const float* f, const float* v, int ldq, int ldf, int ldv, float* out, float* state,
                           long long state_stride, const int32_t* req_meta, const int32_t* slots, const int32_t* positions, int H, int dk, int dv) {
#define FG_LAUNCH(PER)                                                                                                                         \
    do {                                                                                                                                       \
        const size_t smem = sizeof(float) * FG_AHEAD * (2 * 8 * PER + 2 * FG_COLS);                                                             \
        mm_launch(forget_gate_walk_kernel<PER, MODE>, grid, dim3(256), smem, s, q, f, v, ldq, ldf, ldv, out, state, state_stride, req_meta, slots, \
                  positions, H, dk, dv);                                                                                                       \
    } while (0)
    if (dk <= 32) FG_LAUNCH(4);
    else if (dk <= 64) FG_LAUNCH(8);
    else if (dk <= 128) FG_LAUNCH(16);
    else FG_LAUNCH(32);
#undef FG_LAUNCH
}

MM_EXPORT int mm_forget_gate_walk(const void* q, const void* f, const void* v, int ldq, int ldf, int ldv, void* out, void* state,
                                  long long state_stride, const void* req_meta, const void* slots, const void* positions, int n_requests, int H,
                                  int dk, int dv, void* stream) {
    MM_REQUIRE(H > 0 && dk > 0 && dv > 0, "forget gate walk: bad sizes");
    MM_REQUIRE(dk <= 256, "forget gate walk: key sizes above 256 are not supported");
    MM_REQUIRE(state != nullptr && slots != nullptr && positions != nullptr, "forget gate walk: the state and the positions are needed");
    if (n_requests <= 0) return MM_OK;
    fg_walk_launch<0>(dim3(ceil_div(dv, FG_COLS), H, n_requests), (cudaStream_t)stream, (const float*)q, (const float*)f, (const float*)v, ldq, ldf, ldv,
                      (float*)out, (float*)state, state_stride, (const int32_t*)req_meta, (const int32_t*)slots, (const int32_t*)positions, H, dk, dv);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// The carry between the two chunk passes: a thread per number of the state.  scratch [chunks, H * dv * dk] holds what every
// chunk adds and gets what every chunk starts from; gain [chunks, H * dk] the product of the chunk's gates per key channel.
__global__ void forget_gate_carry_kernel(float* __restrict__ scratch, const float* __restrict__ gain, float* __restrict__ state, long long state_stride,
                                         const int32_t* __restrict__ chunk_meta, const int32_t* __restrict__ req_chunks,
                                         const int32_t* __restrict__ slots, const int32_t* __restrict__ positions, int H, int dk, int dv, long long size) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (i >= size) return;
    const int first = req_chunks[2 * r], count = req_chunks[2 * r + 1];
    if (count <= 0) return;
    const int h = (int)(i / ((long long)dv * dk)), ch = (int)(i % dk);
    float* st = state + (size_t)slots[r] * state_stride + i;
    float S = positions[chunk_meta[4 * first]] == 0 ? 0.0f : *st;
    // eight chunks at a time: their loads are issued together, then the chain of eight multiply-adds runs
    for (int c0 = first; c0 < first + count; c0 += 8) {
        float add[8], gn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool in = c0 + j < first + count;
            add[j] = in ? scratch[(size_t)(c0 + j) * size + i] : 0.0f;
            gn[j] = in ? gain[((size_t)(c0 + j) * H + h) * dk + ch] : 1.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (c0 + j < first + count) {
                scratch[(size_t)(c0 + j) * size + i] = S;
                S = fmaf(gn[j], S, add[j]);
            }
        }
    }
    *st = S;
}

// Long portions chunk by chunk (three launches).  chunk_meta [chunks, 4] = (first token, tokens, request, .), req_chunks
// [requests, 2] = (first chunk, chunks); scratch fp32 [chunks, H * dv * dk], gain fp32 [chunks, H * dk].
MM_EXPORT int mm_forget_gate_chunked(const void* q, const void* f, const void* v, int ldq, int ldf, int ldv, void* out, void* state,
                                     long long state_stride, const void* chunk_meta, const void* req_chunks, const void* slots, const void* positions,
                                     int n_requests, int n_chunks, int H, int dk, int dv, void* scratch, void* gain, void* stream) {
    MM_REQUIRE(H > 0 && dk > 0 && dv > 0 && dk <= 256, "forget gate walk: bad sizes, or a key size above 256");
    MM_REQUIRE(state && slots && positions && chunk_meta && req_chunks && scratch && gain, "forget gate walk: the chunked walk needs its lists and its scratch");
    if (n_requests <= 0 || n_chunks <= 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long long size = (long long)H * dv * dk;
    const dim3 grid(ceil_div(dv, FG_COLS), H, n_chunks);
    fg_walk_launch<1>(grid, s, (const float*)q, (const float*)f, (const float*)v, ldq, ldf, ldv, (float*)out, (float*)scratch, size,
                      (const int32_t*)chunk_meta, (const int32_t*)slots, (const int32_t*)positions, H, dk, dv);
    MM_CHECK_LAUNCH();
    mm_launch(forget_gate_gain_kernel, dim3(ceil_div((long long)H * dk, 128), n_chunks), dim3(128), 0, s, (const float*)f, ldf, (const int32_t*)chunk_meta,
              (float*)gain, H * dk);
    MM_CHECK_LAUNCH();
    mm_launch(forget_gate_carry_kernel, dim3(ceil_div(size, 256), n_requests), dim3(256), 0, s, (float*)scratch, (const float*)gain, (float*)state,
              state_stride, (const int32_t*)chunk_meta, (const int32_t*)req_chunks, (const int32_t*)slots, (const int32_t*)positions, H, dk, dv, size);
    MM_CHECK_LAUNCH();
    fg_walk_launch<2>(grid, s, (const float*)q, (const float*)f, (const float*)v, ldq, ldf, ldv, (float*)out, (float*)scratch, size,
                      (const int32_t*)chunk_meta, (const int32_t*)slots, (const int32_t*)positions, H, dk, dv);
    MM_CHECK_LAUNCH();
    return MM_OK;
}
