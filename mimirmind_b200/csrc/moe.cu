// Mixture of experts: the router's choice, the rows of every expert put side by side, the experts' products over
// those rows, and the weighted sum.
//
//   s = softmax(z) over all E experts (z: the router's fp32 logits);
//   the experts stand in `groups` equal runs of neighbours; a run's score is its best expert's; only the experts of
//   the `keep` best runs can be chosen; of those the `top` with the largest s are taken (ties: the lower index);
//   weights: the chosen s divided by their sum (+ 1e-20);
//   y = sum over the chosen e of weight_e * W_down[e] (act(W_gate[e] x) * (W_up[e] x)).
//
// Nothing here waits for the host: the lists are made on the device (route -> sort), the products run over a grid
// that is large enough for any split of the step's rows between experts (CTAs without a tile return), and the sum
// over a token's experts is taken in the order of its choice, so a token's output does not depend on its neighbours.
#include "common.cuh"
#include "mma_sync.cuh"

// ---------------------------------------------------------------------------------------------------------------
// the router's choice: one warp per token
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void warp_argmax(float& v, int& i) {      // the largest value, the lowest index among equals
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
        }
    }
}

// One warp: the choice for one token from its E logits `zr`; s, gs: the warp's scratch (E and `groups` floats).
// scoring 0: s = softmax(z), the chosen weights divided by their sum; 1: s = sigmoid(z), the chosen weights as they are.
__device__ __forceinline__ void moe_route_warp(const float* zr, float* s, float* gs, int lane, int E, int top, int groups, int keep,
                                               int32_t* __restrict__ idx, float* __restrict__ wts, size_t t, int scoring = 0) {
    if (scoring == 1) {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-zr[e]));
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
        m = warp_max(m);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(zr[e] - m);
            s[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) s[e] *= inv;
    }
    __syncwarp();
    const int size = E / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float b = 0.0f;
            for (int e = 0; e < size; ++e) b = fmaxf(b, s[g * size + e]);
            gs[g] = b;
        }
        __syncwarp();
        // the keep best runs get their score replaced by -1: what stays non-negative is dropped
        for (int kk = 0; kk < keep; ++kk) {
            float bv = -1.0f;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] >= 0.0f && (gs[g] > bv)) {
                    bv = gs[g];
                    bi = g;
                }
            warp_argmax(bv, bi);
            if (lane == 0 && bi != 0x7fffffff) gs[bi] = -1.0f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / size] >= 0.0f) s[e] = -1.0f - s[e];      // not eligible
        __syncwarp();
    }
    float total = 0.0f;
    for (int kk = 0; kk < top; ++kk) {
        float bv = -1.0f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (s[e] >= 0.0f && s[e] > bv) {
                bv = s[e];
                bi = e;
            }
        warp_argmax(bv, bi);
        if (bi == 0x7fffffff) {     // fewer eligible experts than `top`: the rest of the choice carries no weight
            bi = 0;
            bv = 0.0f;
        } else if (lane == 0) {
            s[bi] = -3.0f;
        }
        __syncwarp();
        total += bv;
        if (lane == 0) {
            idx[t * top + kk] = bi;
            wts[t * top + kk] = bv;
        }
    }
    __syncwarp();
    if (lane == 0 && scoring == 0) {
        const float d = total + 1e-20f;
        for (int kk = 0; kk < top; ++kk) wts[t * top + kk] /= d;
    }
}

__global__ void moe_route_kernel(const float* __restrict__ z, int ldz, int n_tokens, int E, int top, int groups, int keep,
                                 int32_t* __restrict__ idx, float* __restrict__ wts, int scoring) {
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x * warps + warp;
    if (t >= n_tokens) return;
    float* s = route_smem + (size_t)warp * (E + groups);
    moe_route_warp(z + (size_t)t * ldz, s, s + E, lane, E, top, groups, keep, idx, wts, (size_t)t, scoring);
}

// The router's product and its choice in one launch, one block per token: every warp takes experts in turn and sums
// x . w_e over lanes in fp32 (a fixed order, whatever else is in the batch); then the first warp chooses.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float* v);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_router_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, int D, int E, int top,
                                                         int groups, int keep, int vec, int32_t* __restrict__ idx, float* __restrict__ wts, int scoring) {
    extern __shared__ float route_smem[];      // logits [E], scores [E], runs [groups]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t t = blockIdx.x;
    const T* xr = x + t * ldx;
    for (int e = warp; e < E; e += 8) {
        const float* we = w + (size_t)e * D;
        float acc = 0.0f;
        if (vec) {        // rows that start on 16-byte boundaries: eight numbers per lane and step, several steps in flight
            float a2 = 0.0f;
#pragma unroll 4
            for (int d = lane * 8; d < D; d += 256) {
                float xv[8], wv[8];
                load8<T>(xr + d, xv);
                load8<float>(we + d, wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc = fmaf(xv[i], wv[i], acc);
                    a2 = fmaf(xv[4 + i], wv[4 + i], a2);
                }
            }
            acc += a2;
        } else {
            for (int d = lane; d < D; d += 32) acc = fmaf(to_f32<T>(xr[d]), we[d], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) route_smem[e] = acc;
    }
    __syncthreads();
    if (warp == 0) moe_route_warp(route_smem, route_smem + E, route_smem + 2 * E, lane, E, top, groups, keep, idx, wts, t, scoring);
}

MM_EXPORT int mm_moe_router_scored(const void* x, int x_dtype, int ldx, const void* w, int n_tokens, int D, int E, int top, int groups, int keep,
                                   int scoring, void* idx, void* wts, void* stream) {
    MM_REQUIRE(scoring == 0 || scoring == 1, "moe router: the scoring is 0 (softmax, renormed) or 1 (sigmoid, as it is)");
    MM_REQUIRE(n_tokens >= 0 && D > 0 && ldx >= D && E > 0 && top > 0 && top <= E && groups > 0 && E % groups == 0 && keep > 0 && keep <= groups,
               "moe router: experts must split into equal runs, and 0 < top <= experts, 0 < keep <= runs");
    MM_REQUIRE((size_t)(2 * E + groups) * sizeof(float) <= 48 * 1024, "moe router: too many experts for the router's shared memory");
    if (n_tokens == 0) return MM_OK;
    const size_t smem = (size_t)(2 * E + groups) * sizeof(float);
    const int vec = D % 8 == 0 && ldx % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
    if (x_dtype == MM_F32)
        mm_launch(moe_router_kernel<float>, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (const float*)x, ldx, (const float*)w, D, E, top,
                  groups, keep, vec, (int32_t*)idx, (float*)wts, scoring);
    else if (x_dtype == MM_BF16)
        mm_launch(moe_router_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx,
                  (const float*)w, D, E, top, groups, keep, vec, (int32_t*)idx, (float*)wts, scoring);
    else
        MM_REQUIRE(false, "moe router: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_moe_router(const void* x, int x_dtype, int ldx, const void* w, int n_tokens, int D, int E, int top, int groups, int keep,
                            void* idx, void* wts, void* stream) {
    return mm_moe_router_scored(x, x_dtype, ldx, w, n_tokens, D, E, top, groups, keep, 0, idx, wts, stream);
}

MM_EXPORT int mm_moe_route(const void* z, int ldz, int n_tokens, int E, int top, int groups, int keep, void* idx, void* wts, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && E > 0 && top > 0 && top <= E && groups > 0 && E % groups == 0 && keep > 0 && keep <= groups && ldz >= E,
               "moe route: experts must split into equal runs, and 0 < top <= experts, 0 < keep <= runs");
    MM_REQUIRE((size_t)(E + groups) * 4 * sizeof(float) <= 48 * 1024, "moe route: too many experts for the router's shared memory");
    if (n_tokens == 0) return MM_OK;
    const int warps = 4;
    mm_launch(moe_route_kernel, dim3(ceil_div(n_tokens, warps)), dim3(warps * 32), (size_t)warps * (E + groups) * sizeof(float),
              (cudaStream_t)stream, (const float*)z, ldz, n_tokens, E, top, groups, keep, (int32_t*)idx, (float*)wts, 0);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// rows by expert: offsets [E + 1] and, for every place in the sorted order, the row (token * top + choice) it holds
// ---------------------------------------------------------------------------------------------------------------
// One block.  Rows keep their order inside an expert (a row's place is the number of rows of its expert before it), so the
// lists are the same on every run.
// Also made here, for the grouped tensor-core products: the list of row tiles (first row, end row, expert; at most
// `tile_rows` rows, none across an expert's border) with their number, each row's token (order / top), and each
// (token, choice)'s place in the sorted order.
#define SORT_FAST_EXPERTS 256

__global__ void moe_sort_kernel(const int32_t* __restrict__ idx, int n_rows, int E, int32_t* __restrict__ offsets, int32_t* __restrict__ order,
                                int top, int tile_rows, int32_t* __restrict__ tiles, int32_t* __restrict__ n_tiles,
                                int32_t* __restrict__ row_token, int32_t* __restrict__ place) {
    extern __shared__ int32_t sort_smem[];     // counts [E], then the running cursors [E]
    int32_t* counts = sort_smem;
    int32_t* cursor = counts + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < n_rows; r += blockDim.x) atomicAdd(&counts[idx[r]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = acc;
            cursor[e] = acc;
            acc += counts[e];
        }
        offsets[E] = acc;
        if (tiles != nullptr) {
            int nt = 0;
            for (int e = 0; e < E; ++e)
                for (int lo = offsets[e]; lo < offsets[e + 1]; lo += tile_rows, ++nt) {
                    tiles[3 * nt] = lo;
                    tiles[3 * nt + 1] = min(lo + tile_rows, offsets[e + 1]);
                    tiles[3 * nt + 2] = e;
                }
            *n_tiles = nt;
        }
    }
    __syncthreads();
    // stable placement
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    auto put = [&](int r, int at) {
        order[at] = r;
        if (row_token != nullptr) row_token[at] = r / top;
        if (place != nullptr) place[r] = at;
    };
    if (E <= SORT_FAST_EXPERTS) {
        // every warp owns a run of consecutive rows: it counts its rows per expert, the counts of the warps before it give
        // its first place in every expert's list, and it then places its rows 32 at a time (a row's rank among the rows
        // of its expert inside the 32 comes from a match over the warp)
        int32_t* wcount = cursor + E;                              // [warps][E]
        const int per_warp = (n_rows + warps - 1) / warps;
        const int lo = min(n_rows, warp * per_warp), hi = min(n_rows, lo + per_warp);
        for (int e = lane; e < E; e += 32) wcount[warp * E + e] = 0;
        __syncwarp();
        for (int r = lo + lane; r < hi; r += 32) atomicAdd(&wcount[warp * E + idx[r]], 1);
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            int at = offsets[e];
            for (int w = 0; w < warps; ++w) {
                const int c = wcount[w * E + e];
                wcount[w * E + e] = at;
                at += c;
            }
        }
        __syncthreads();
        for (int base = lo; base < hi; base += 32) {
            const int r = base + lane;
            const int e = r < hi ? idx[r] : -1;
            if (e >= 0) {
                const unsigned peers = __match_any_sync(__activemask(), e);
                const int rank = __popc(peers & ((1u << lane) - 1));
                const int first = __ffs(peers) - 1;
                int start = 0;
                if (lane == first) {
                    start = wcount[warp * E + e];
                    wcount[warp * E + e] = start + __popc(peers);
                }
                start = __shfl_sync(peers, start, first);
                put(r, start + rank);
            }
            __syncwarp();
        }
        return;
    }
    // many experts: the rows are taken blockDim.x at a time, and the warps take their turn
    for (int base = 0; base < n_rows; base += blockDim.x) {
        const int r = base + threadIdx.x;
        const int e = r < n_rows ? idx[r] : -1;
        for (int w = 0; w < warps; ++w) {
            if (w == warp && e >= 0) {
                const unsigned peers = __match_any_sync(__activemask(), e);
                const int rank = __popc(peers & ((1u << lane) - 1));
                const int first = __ffs(peers) - 1;
                int start = 0;
                if (lane == first) start = atomicAdd(&cursor[e], __popc(peers));
                start = __shfl_sync(peers, start, first);
                put(r, start + rank);
            }
            __syncthreads();
        }
    }
}

MM_EXPORT int mm_moe_sort(const void* idx, int n_rows, int E, void* offsets, void* order, int top, int tile_rows, void* tiles, void* n_tiles,
                          void* row_token, void* place, void* stream) {
    MM_REQUIRE(n_rows >= 0 && E > 0 && E <= 4096 && top > 0, "moe sort: bad sizes");
    MM_REQUIRE(tiles == nullptr || (tile_rows > 0 && n_tiles != nullptr), "moe sort: the tile list needs its tile size and its count");
    const int threads = n_rows > 256 ? 1024 : 256;
    const size_t sort_smem = (size_t)(2 + (E <= SORT_FAST_EXPERTS ? threads / 32 : 0)) * E * sizeof(int32_t);
    mm_launch(moe_sort_kernel, dim3(1), dim3(threads), sort_smem, (cudaStream_t)stream,
              (const int32_t*)idx, n_rows, E, (int32_t*)offsets, (int32_t*)order, top, tile_rows, (int32_t*)tiles, (int32_t*)n_tiles,
              (int32_t*)row_token, (int32_t*)place);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// the experts' products over their rows
// ---------------------------------------------------------------------------------------------------------------
// A CTA's tile: expert e and rows [lo, hi) of the sorted order, found from the offsets (every expert's rows start a
// tile of their own).  Returns false when the CTA has no tile.
template <int TM>
__device__ __forceinline__ bool moe_tile(const int32_t* __restrict__ offsets, int E, int tile, int& e, int& lo, int& hi) {
    int seen = 0;
    for (int x = 0; x < E; ++x) {
        const int a = offsets[x], b = offsets[x + 1];
        const int tiles = (b - a + TM - 1) / TM;
        if (tile < seen + tiles) {
            e = x;
            lo = a + (tile - seen) * TM;
            hi = min(lo + TM, b);
            return true;
        }
        seen += tiles;
    }
    return false;
}

#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MMA_BK 64
#define MOE_STAGES 3

// fp32 FMA units, every output summed over k in ascending order.  GATED: W is [E, 2F, K], the gate's rows then the
// up rows, and the output is act(gate) * up over F columns, the input rows gathered through order / top; otherwise
// W is [E, N, K], the input rows are the sorted ones and output row order[i] is written.
template <typename TA, typename TW, typename TC, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, TC* __restrict__ C, int ldc,
                                                            const int32_t* __restrict__ offsets, const int32_t* __restrict__ order, int E, int top,
                                                            int N, int K, int act, float limit, const float* __restrict__ row_scale) {
    __shared__ float As[MOE_BK][MOE_BM + 4];
    __shared__ float Ws[MOE_BK][MOE_BN + 4];
    __shared__ float Us[GATED ? MOE_BK : 1][MOE_BN + 4];
    __shared__ int32_t rows[MOE_BM];
    __shared__ int tile_info[3];
    const int tid = threadIdx.x;
    if (tid == 0) {
        int e = -1, lo = 0, hi = 0;
        if (!moe_tile<MOE_BM>(offsets, E, blockIdx.y, e, lo, hi)) e = -1;
        tile_info[0] = e;
        tile_info[1] = lo;
        tile_info[2] = hi;
    }
    __syncthreads();
    const int e = tile_info[0], lo = tile_info[1], hi = tile_info[2];
    if (e < 0) return;
    const int M = hi - lo;
    if (tid < MOE_BM) rows[tid] = tid < M ? (GATED ? order[lo + tid] / top : lo + tid) : 0;
    __syncthreads();
    const int tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * MOE_BN;
    const TW* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[4][4], up[GATED ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
            if (GATED) up[i][j] = 0.0f;
        }
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = tid + x * 256;
            const int r = i >> 4, kk = i & 15;
            const int k = k0 + kk;
            float a = 0.0f, w = 0.0f, u = 0.0f;
            if (k < K) {
                if (r < M) a = to_f32<TA>(A[(size_t)rows[r] * lda + k]);
                if (n0 + r < N) {
                    w = to_f32<TW>(We[(size_t)(n0 + r) * K + k]);
                    if (GATED) u = to_f32<TW>(We[(size_t)(N + n0 + r) * K + k]);
                }
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
            if (GATED) Us[kk][r] = u;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float a[4], w[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = Ws[kk][tx * 4 + j];
                u[j] = GATED ? Us[kk][tx * 4 + j] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (GATED) up[i][j] = fmaf(a[i], u[j], up[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = ty * 4 + i;
        if (m >= M) continue;
        const size_t out_row = GATED ? (size_t)(lo + m) : (size_t)order[lo + m];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = glu_act<false>(v, up[i][j], act, limit, row_scale ? row_scale[order[lo + m]] : 1.0f);
            C[out_row * ldc + n] = from_f32<TC>(v);
        }
    }
}

// bfloat16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation): the same tiles, 64 rows x 64 columns, four
// warps of 32 x 32 (gated: gate and up accumulators side by side), K in steps of 64 through a ring of shared-memory stages.
template <bool GATED, typename TC>
__global__ void __launch_bounds__(128) moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W,
                                                           TC* __restrict__ C, int ldc, const int32_t* __restrict__ offsets,
                                                           const int32_t* __restrict__ order, int E, int top, int N, int K, int interleaved, int act, float limit,
                                                           const float* __restrict__ row_scale) {
    // K in steps of 64 through a ring of MOE_STAGES stages: a decode step's tiles hold a handful of rows and stream a
    // whole expert, so what counts is how many bytes of weights a CTA keeps in flight (rows of 144 bytes: ldmatrix
    // reads without bank conflicts)
    constexpr int BK = MOE_MMA_BK, LD = BK + 8;
    constexpr int WROWS_ = GATED ? 2 * MOE_BN : MOE_BN;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    typedef __nv_bfloat16 (*ATile)[MOE_BM][LD];
    typedef __nv_bfloat16 (*WTile)[WROWS_][LD];
    ATile As = reinterpret_cast<ATile>(moe_smem);
    WTile Ws = reinterpret_cast<WTile>(moe_smem + sizeof(__nv_bfloat16) * MOE_STAGES * MOE_BM * LD);
    __shared__ int32_t rows[MOE_BM];
    __shared__ int tile_info[3];
    const int tid = threadIdx.x;
    if (tid == 0) {
        int e = -1, lo = 0, hi = 0;
        if (!moe_tile<MOE_BM>(offsets, E, blockIdx.y, e, lo, hi)) e = -1;
        tile_info[0] = e;
        tile_info[1] = lo;
        tile_info[2] = hi;
    }
    __syncthreads();
    const int e = tile_info[0], lo = tile_info[1], hi = tile_info[2];
    if (e < 0) return;
    const int M = hi - lo;
    if (tid < MOE_BM) rows[tid] = tid < M ? (GATED ? order[lo + tid] / top : lo + tid) : -1;
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int n0 = blockIdx.x * MOE_BN;
    const __nv_bfloat16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    constexpr int WROWS = GATED ? 2 * MOE_BN : MOE_BN;
    float acc[2][4][4], up[GATED ? 2 : 1][4][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[a][b][c] = 0.0f;
                if (GATED) up[a][b][c] = 0.0f;
            }
    auto load = [&](int stage, int k0) {
        // 16-byte chunks: 8 per row of 64 k
        for (int i = tid; i < MOE_BM * 8; i += 128) {
            const int r = i >> 3, c = (i & 7) * 8;
            __nv_bfloat16* dst = &As[stage][r][c];
            if (rows[r] >= 0 && k0 + c < K) cp_async16(dst, A + (size_t)rows[r] * lda + k0 + c);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < WROWS * 8; i += 128) {
            const int r = i >> 3, c = (i & 7) * 8;
            // gated: column j of the gate is row j of the expert's matrix and the up column row N + j, or, interleaved in
            // blocks of 8 (the layout the tensor-memory product's epilogue wants), rows 16 (j / 8) + j % 8 and + 8
            const int j = GATED ? (r < MOE_BN ? n0 + r : n0 + r - MOE_BN) : n0 + r;
            const int n = !GATED ? j : (interleaved ? 16 * (j >> 3) + (j & 7) + (r < MOE_BN ? 0 : 8) : (r < MOE_BN ? j : N + j));
            const bool ok = j < N;
            __nv_bfloat16* dst = &Ws[stage][r][c];
            if (ok && k0 + c < K) cp_async16(dst, We + (size_t)n * K + k0 + c);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };
    const int steps = (K + BK - 1) / BK;
#pragma unroll
    for (int p = 0; p < MOE_STAGES - 1; ++p) {
        if (p < steps) load(p, p * BK);
        else cp_async_commit();              // an empty group keeps the count of groups in step
    }
    for (int s = 0; s < steps; ++s) {
        cp_async_wait<MOE_STAGES - 2>();     // the copies of step s have landed
        __syncthreads();                     // ... for every thread, and the stage of step s - 1 is free
        if (s + MOE_STAGES - 1 < steps) load((s + MOE_STAGES - 1) % MOE_STAGES, (s + MOE_STAGES - 1) * BK);
        else cp_async_commit();
        const int st = s % MOE_STAGES;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                ldmatrix_x4(af[mi][0], af[mi][1], af[mi][2], af[mi][3], &As[st][wm + mi * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int nj = 0; nj < 2; ++nj) {
                uint32_t b0, b1, b2, b3;
                // rows wn + nj*16 .. +15 of W: matrices (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                ldmatrix_x4(b0, b1, b2, b3, &Ws[st][wn + nj * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    mma_bf16(acc[mi][nj * 2], af[mi], b0, b1);
                    mma_bf16(acc[mi][nj * 2 + 1], af[mi], b2, b3);
                }
                if (GATED) {
                    ldmatrix_x4(b0, b1, b2, b3, &Ws[st][MOE_BN + wn + nj * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        mma_bf16(up[mi][nj * 2], af[mi], b0, b1);
                        mma_bf16(up[mi][nj * 2 + 1], af[mi], b2, b3);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = wm + mi * 16 + (lane >> 2) + half * 8;
            if (m >= M) continue;
            const size_t out_row = GATED ? (size_t)(lo + m) : (size_t)order[lo + m];
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int n = n0 + wn + ni * 8 + (lane & 3) * 2 + c;
                    if (n >= N) continue;
                    float v = acc[mi][ni][half * 2 + c];
                    if (GATED) v = glu_act<true>(v, up[mi][ni][half * 2 + c], act, limit, row_scale ? row_scale[order[lo + m]] : 1.0f);
                    C[out_row * ldc + n] = from_f32<TC>(v);
                }
        }
}

// A [rows, lda] (gated: the step's tokens; else the sorted hidden rows), W the experts' stacked matrices, C: gated
// [n_rows, N] in sorted order, else [n_rows, N] with row order[i] written.  n_rows = tokens * top.
// act: what a gated product does with its two halves (glu_act in common.cuh: 0 silu(g) u; 1 the clamped form with
// `limit`); row_scale [tokens * top] fp32 or null: row (token * top + choice) of a gated product is multiplied by it
// before the activation (a weight on the expert's input: W (s x) = s (W x)).
MM_EXPORT int mm_moe_gemm_act(const void* A, int a_dtype, int lda, const void* W, int w_dtype, void* C, int c_dtype, int ldc, const void* offsets,
                              const void* order, int n_rows, int E, int top, int N, int K, int gated, int tensor_cores, int interleaved,
                              int act, float limit, const void* row_scale_, void* stream) {
    const float* row_scale = (const float*)row_scale_;
    MM_REQUIRE(act == 0 || act == 1, "moe gemm: the activation is 0 (silu) or 1 (clamped)");
    MM_REQUIRE(gated || (act == 0 && row_scale == nullptr), "moe gemm: activation and row scale belong to the gated product");
    MM_REQUIRE(n_rows >= 0 && E > 0 && top > 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "moe gemm: bad sizes");
    MM_REQUIRE(!interleaved || (gated && N % 8 == 0), "moe gemm: interleaved gate and up rows need a gated product of a multiple of 8 columns");
    if (n_rows == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(ceil_div(N, MOE_BN), ceil_div(n_rows, MOE_BM) + E);
    typedef __nv_bfloat16 bf;
    const int32_t* off = (const int32_t*)offsets;
    const int32_t* ord = (const int32_t*)order;
    if (tensor_cores && a_dtype == MM_BF16 && w_dtype == MM_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
        const size_t tile_smem = sizeof(bf) * MOE_STAGES * (MOE_BM + (gated ? 2 : 1) * MOE_BN) * (MOE_MMA_BK + 8);
        static bool configured = false;
        if (!configured) {
            cudaFuncSetAttribute(moe_gemm_mma_kernel<true, bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(bf) * MOE_STAGES * (MOE_BM + 2 * MOE_BN) * (MOE_MMA_BK + 8)));
            cudaFuncSetAttribute(moe_gemm_mma_kernel<false, bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(bf) * MOE_STAGES * (MOE_BM + MOE_BN) * (MOE_MMA_BK + 8)));
            cudaFuncSetAttribute(moe_gemm_mma_kernel<false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(bf) * MOE_STAGES * (MOE_BM + MOE_BN) * (MOE_MMA_BK + 8)));
            configured = true;
        }
        if (gated && c_dtype == MM_BF16)
            mm_launch(moe_gemm_mma_kernel<true, bf>, grid, dim3(128), tile_smem, s, (const bf*)A, lda, (const bf*)W, (bf*)C, ldc, off, ord, E, top, N, K, interleaved, act, limit, row_scale);
        else if (!gated && c_dtype == MM_BF16)
            mm_launch(moe_gemm_mma_kernel<false, bf>, grid, dim3(128), tile_smem, s, (const bf*)A, lda, (const bf*)W, (bf*)C, ldc, off, ord, E, top, N, K, 0, 0, 0.0f, (const float*)nullptr);
        else if (!gated && c_dtype == MM_F32)
            mm_launch(moe_gemm_mma_kernel<false, float>, grid, dim3(128), tile_smem, s, (const bf*)A, lda, (const bf*)W, (float*)C, ldc, off, ord, E, top, N, K, 0, 0, 0.0f, (const float*)nullptr);
        else
            MM_REQUIRE(false, "moe gemm: this combination of dtypes is not built");
        MM_CHECK_LAUNCH();
        return MM_OK;
    }
    MM_REQUIRE(!interleaved, "moe gemm: interleaved gate and up rows are read by the tensor-core kernels only");
#define MOE_SIMT(TA, TW, TC)                                                                                                                  \
    do {                                                                                                                                      \
        if (gated)                                                                                                                            \
            mm_launch(moe_gemm_simt_kernel<TA, TW, TC, true>, grid, dim3(256), 0, s, (const TA*)A, lda, (const TW*)W, (TC*)C, ldc, off, ord, E, top, N, K, act, limit, row_scale); \
        else                                                                                                                                  \
            mm_launch(moe_gemm_simt_kernel<TA, TW, TC, false>, grid, dim3(256), 0, s, (const TA*)A, lda, (const TW*)W, (TC*)C, ldc, off, ord, E, top, N, K, 0, 0.0f, (const float*)nullptr); \
    } while (0)
    if (a_dtype == MM_F32 && w_dtype == MM_F32 && c_dtype == MM_F32) MOE_SIMT(float, float, float);
    else if (a_dtype == MM_BF16 && w_dtype == MM_BF16 && c_dtype == MM_BF16) MOE_SIMT(bf, bf, bf);
    else if (a_dtype == MM_BF16 && w_dtype == MM_BF16 && c_dtype == MM_F32) MOE_SIMT(bf, bf, float);
    else MM_REQUIRE(false, "moe gemm: this combination of dtypes is not built");
#undef MOE_SIMT
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_moe_gemm(const void* A, int a_dtype, int lda, const void* W, int w_dtype, void* C, int c_dtype, int ldc, const void* offsets,
                          const void* order, int n_rows, int E, int top, int N, int K, int gated, int tensor_cores, int interleaved,
                          void* stream) {
    return mm_moe_gemm_act(A, a_dtype, lda, W, w_dtype, C, c_dtype, ldc, offsets, order, n_rows, E, top, N, K, gated, tensor_cores, interleaved,
                           0, 0.0f, nullptr, stream);
}

// The step's rows copied into sorted order, each multiplied by its (token, choice)'s weight and rounded to the rows'
// dtype: out[i] = x[row_token[i]] * wts[order[i]] (wts null: a plain copy).
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ x, const int32_t* __restrict__ row_token, const int32_t* __restrict__ order,
                                         const float* __restrict__ wts, T* __restrict__ out, int d) {
    const size_t i = blockIdx.x;
    const T* src = x + (size_t)row_token[i] * d;
    const float s = wts ? wts[order[i]] : 1.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[i * d + c] = from_f32<T>(to_f32<T>(src[c]) * s);
}

MM_EXPORT int mm_moe_gather_scaled(const void* x, int dtype, const void* row_token, const void* order, const void* wts, void* out, int n_rows, int d,
                                   void* stream) {
    MM_REQUIRE(n_rows >= 0 && d > 0 && row_token != nullptr && order != nullptr, "moe gather: bad sizes");
    if (n_rows == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MM_BF16)
        mm_launch(moe_gather_scaled_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, s, (const __nv_bfloat16*)x, (const int32_t*)row_token,
                  (const int32_t*)order, (const float*)wts, (__nv_bfloat16*)out, d);
    else if (dtype == MM_F32)
        mm_launch(moe_gather_scaled_kernel<float>, dim3(n_rows), dim3(256), 0, s, (const float*)x, (const int32_t*)row_token, (const int32_t*)order,
                  (const float*)wts, (float*)out, d);
    else
        MM_REQUIRE(false, "moe gather: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// out[t, :] = sum over the token's choices c, in order, of wts[t, c] * y[row(t, c), :], row(t, c) = t * top + c or, when
// y stands in sorted order, place[t * top + c]
template <typename TY, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const float* __restrict__ wts, const int32_t* __restrict__ place, TO* __restrict__ out,
                                   int top, int d) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int c = 0; c < top; ++c) {
            const size_t row = place ? (size_t)place[t * top + c] : t * top + c;
            acc = fmaf(wts ? wts[t * top + c] : 1.0f, to_f32<TY>(y[row * d + i]), acc);      // no weights: the plain sum
        }
        out[t * d + i] = from_f32<TO>(acc);
    }
}

MM_EXPORT int mm_moe_combine(const void* y, int y_dtype, const void* wts, const void* place, void* out, int out_dtype, int n_tokens, int top, int d,
                             void* stream) {
    MM_REQUIRE(n_tokens >= 0 && top > 0 && d > 0, "moe combine: bad sizes");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const dim3 grid(n_tokens), block(d >= 1024 ? 256 : 128);
    if (y_dtype == MM_F32 && out_dtype == MM_F32)
        mm_launch(moe_combine_kernel<float, float>, grid, block, 0, s, (const float*)y, (const float*)wts, (const int32_t*)place, (float*)out, top, d);
    else if (y_dtype == MM_F32 && out_dtype == MM_BF16)
        mm_launch(moe_combine_kernel<float, bf>, grid, block, 0, s, (const float*)y, (const float*)wts, (const int32_t*)place, (bf*)out, top, d);
    else if (y_dtype == MM_BF16 && out_dtype == MM_BF16)
        mm_launch(moe_combine_kernel<bf, bf>, grid, block, 0, s, (const bf*)y, (const float*)wts, (const int32_t*)place, (bf*)out, top, d);
    else
        MM_REQUIRE(false, "moe combine: this combination of dtypes is not built");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
