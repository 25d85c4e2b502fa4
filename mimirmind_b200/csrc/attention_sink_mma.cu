// bfloat16 paged attention on the tensor cores (mma.sync m16n8k16, fp32 accumulate and fp32 softmax) for keys of
// size DK and values of size DV (each one of 32, 64, 96, 128), a sliding window and a softmax sink:
//
//   s_j = (q . k_j) * scale;  p_j = exp(s_j) / (sink + sum_i exp(s_i));  o = sum_j p_j v_j
//
// The sink is a key of score 0 without a value: the running softmax starts from (maximum 0, mass 1, nothing
// accumulated) instead of (-inf, 0, 0).
//
//   * prefill: one CTA per (tile of 64 query tokens of one request, query head); keys and values stream through
//     shared memory in tiles of 64 keys gathered page by page with cp.async, two stages deep; online softmax.  Only
//     the key tiles between the first row's window edge and the last row's position are visited.
//   * decode: one CTA per (token, KV head, split of the token's key tiles).  The rows of the tile are the query heads
//     that share the KV head, so a key or value is read once for all of them; the four warps take 16 keys each of every
//     64-key tile and are merged through shared memory; with more than one split the partial results go through scratch
//     memory and a merge launch, which also adds the sink.  Positions come from the device, so a captured step replays
//     with new positions.
//
// Same tiling as csrc/attention_mma.cu (equal key and value sizes, no sink), which this file generalises.
#include "common.cuh"
#include "mma_sync.cuh"

#define SKT 64            // keys per tile
#define SATT_THREADS 128  // 4 warps
#define SDEC_STAGES 3

// 64 key rows [64][DK + 8] and the same 64 value rows [64][DV + 8] of one KV head; rows outside [lo, hi) are zero.
// Warp w fetches rows 16 w .. 16 w + 15: its first sixteen lanes look up one row's page and place each, and every lane
// takes those from the row's lane for the 16-byte pieces it copies (one table read per row, not per piece).  Every
// thread of the CTA must call this together.
template <int DK, int DV>
__device__ __forceinline__ void load_kv_tile2(__nv_bfloat16* dK, __nv_bfloat16* dV, const __nv_bfloat16* __restrict__ kpool,
                                              const __nv_bfloat16* __restrict__ vpool, const int32_t* __restrict__ table,
                                              int key0, int lo, int hi, int G, int g, int page_size, int page_shift, int Gv) {
    constexpr int KS = DK + 8, VS = DV + 8, KC = DK / 8, VC = DV / 8;
    static_assert(SATT_THREADS == 128 && SKT == 64 && (16 * KC) % 32 == 0 && (16 * VC) % 32 == 0, "a warp per 16 rows");
    const int gv = g % Gv;      // the value pool has Gv heads; key head g reads value head g mod Gv
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int page = -1, slot = 0;
    {
        const int key = key0 + warp * 16 + (lane & 15);
        if (key >= lo && key < hi) {
            const int pidx = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
            slot = key - pidx * page_size;
            page = table[pidx];
        }
    }
#pragma unroll
    for (int i = 0; i < 16 * KC / 32; ++i) {
        const int c = i * 32 + lane, r = c / KC, part = c - r * KC;
        const int p = __shfl_sync(0xffffffffu, page, r), sl = __shfl_sync(0xffffffffu, slot, r);
        __nv_bfloat16* d = dK + (warp * 16 + r) * KS + part * 8;
        if (p >= 0) cp_async16(d, kpool + (((size_t)p * G + g) * page_size + sl) * DK + part * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 16 * VC / 32; ++i) {
        const int c = i * 32 + lane, r = c / VC, part = c - r * VC;
        const int p = __shfl_sync(0xffffffffu, page, r), sl = __shfl_sync(0xffffffffu, slot, r);
        __nv_bfloat16* d = dV + (warp * 16 + r) * VS + part * 8;
        if (p >= 0) cp_async16(d, vpool + (((size_t)p * Gv + gv) * page_size + sl) * DV + part * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
}

// ---------------------------------------------------------------------------
// prefill
//   tiles: int32 [n_tiles, 4] = (request index, first token row, rows in the tile, position of the first row)
// ---------------------------------------------------------------------------
#define SINK_LOG2E_F 1.4426950408889634f

template <int DK, int DV>
__global__ void __launch_bounds__(SATT_THREADS) attention_sink_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, float* __restrict__ out32,
    const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ block_table, int table_width, int page_size, int H, int G, int window, float scale_log2,
    int sink, const float* __restrict__ sink_logit, const float* __restrict__ dist_bias, int dist_max, float softcap, int Gv) {
    constexpr int KS = DK + 8, VS = DV + 8;
    constexpr int KSTEPS = DK / 16;
    constexpr int NT_O = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [64][KS]
    __nv_bfloat16* sK = sQ + 64 * KS;                                // [2][64][KS]
    __nv_bfloat16* sV = sK + 2 * SKT * KS;                           // [2][64][VS]

    // heads fastest, later (longer) tiles first
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
    const int g = h / (H / G);
    const int req = tiles[tile * 4 + 0], row0 = tiles[tile * 4 + 1], n_rows = tiles[tile * 4 + 2], pos0 = tiles[tile * 4 + 3];
    const int32_t* table = block_table + (size_t)req * table_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int hi_all = pos0 + n_rows;                                     // exclusive
    const int lo_all = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int kt_begin = lo_all / SKT, kt_end = (hi_all + SKT - 1) / SKT;

    for (int c = threadIdx.x; c < 64 * (DK / 8); c += SATT_THREADS) {
        const int r = c / (DK / 8), part = c - r * (DK / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + r) * H + h) * DK + part * 8);
        *reinterpret_cast<uint4*>(sQ + r * KS + part * 8) = v;
    }
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    load_kv_tile2<DK, DV>(sK, sV, k_pages, v_pages, table, kt_begin * SKT, lo_all, hi_all, G, g, page_size, page_shift, Gv);
    cp_async_commit();
    __syncthreads();

    uint32_t qf[KSTEPS][4];
    {
        const int id = lane >> 3, rr = lane & 7;
        const int r = warp * 16 + (id & 1) * 8 + rr;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + r * KS + ks * 16 + (id >> 1) * 8);
    }
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = pos0 + r_lo, pos_hi = pos0 + r_hi;
    const int wlo_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int wlo_hi = (window > 0 && pos_hi + 1 > window) ? pos_hi + 1 - window : 0;
    const bool valid_lo = r_lo < n_rows, valid_hi = r_hi < n_rows;

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    // the sink: maximum 0 (raw score), mass 1 held by the first thread of the quad that shares a row.  With a learned
    // sink or a distance bias the scores are brought to their final form (scaled, bias added, in units of log2 e) right
    // after the product, and from there on the scale is 1; the learned sink then starts the maximum at its logit.
    // A soft cap bends the scaled score into (-cap, cap): s <- cap tanh(s / cap), before any bias.
    const bool ext = sink_logit != nullptr || dist_bias != nullptr || softcap > 0.0f;
    const float sl2 = ext ? 1.0f : scale_log2;
    const float cap_in = softcap > 0.0f ? scale_log2 / (SINK_LOG2E_F * softcap) : 0.0f, cap_out = softcap * SINK_LOG2E_F;
    const float* bias_h = dist_bias ? dist_bias + (size_t)h * (dist_max + 1) : nullptr;
    const float l0 = ((sink || sink_logit) && (lane & 3) == 0) ? 1.0f : 0.0f;
    float m_lo = sink_logit ? sink_logit[h] * SINK_LOG2E_F : (sink ? 0.0f : -INFINITY), m_hi = m_lo, l_lo = l0, l_hi = l0;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) {
            load_kv_tile2<DK, DV>(sK + (buf ^ 1) * SKT * KS, sV + (buf ^ 1) * SKT * VS, k_pages, v_pages, table, (kt + 1) * SKT,
                                  lo_all, hi_all, G, g, page_size, page_shift, Gv);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* tK = sK + buf * SKT * KS;
        const __nv_bfloat16* tV = sV + buf * SKT * VS;
        const int key0 = kt * SKT;
        // a warp whose rows all lie before this tile, or whose windows all begin after it, has nothing to do in it
        const bool warp_active = (pos0 + warp * 16 + 15 >= key0) && (warp * 16 < n_rows) &&
                                 (window == 0 || key0 + SKT - 1 >= pos0 + warp * 16 + 1 - window);
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    const int id = lane >> 3, rr = lane & 7;
                    const int n = jp * 16 + (id >> 1) * 8 + rr;
                    ldmatrix_x4(b0, b1, b2, b3, tK + n * KS + ks * 16 + (id & 1) * 8);
                    mma_bf16(s[jp * 2], qf[ks], b0, b1);
                    mma_bf16(s[jp * 2 + 1], qf[ks], b2, b3);
                }
            }
            const bool interior = (key0 + SKT - 1 <= pos0 + warp * 16) && (warp * 16 + 15 < n_rows) &&
                                  (window == 0 || key0 >= pos0 + warp * 16 + 16 - window);
            float mx_lo = m_lo, mx_hi = m_hi;
            if (ext) {
                // every key of the tile at least dist_max behind every row of the warp: one bias for all
                const bool all_far = bias_h != nullptr && pos0 + warp * 16 - (key0 + SKT - 1) >= dist_max;
                const float far_bias = bias_h ? bias_h[dist_max] * SINK_LOG2E_F : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float b = far_bias;
                        if (bias_h != nullptr && !all_far) {
                            const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                            const int dist = (e >= 2 ? pos_hi : pos_lo) - key;
                            b = bias_h[min(max(dist, 0), dist_max)] * SINK_LOG2E_F;
                        }
                        s[j][e] = softcap > 0.0f ? fmaf(tanhf(s[j][e] * cap_in), cap_out, b) : fmaf(s[j][e], scale_log2, b);
                    }
                }
            }
            if (!interior) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                        const bool hi_row = e >= 2;
                        const bool ok = hi_row ? (valid_hi && key <= pos_hi && key >= wlo_hi) : (valid_lo && key <= pos_lo && key >= wlo_lo);
                        if (!ok) s[j][e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float use_lo = (mx_lo == -INFINITY) ? 0.0f : mx_lo * sl2;
            const float use_hi = (mx_hi == -INFINITY) ? 0.0f : mx_hi * sl2;
            const float a_lo = exp2f(m_lo * sl2 - use_lo), a_hi = exp2f(m_hi * sl2 - use_hi);
            m_lo = mx_lo;
            m_hi = mx_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
            uint32_t pf[4][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = exp2f(fmaf(s[j][0], sl2, -use_lo)), p1 = exp2f(fmaf(s[j][1], sl2, -use_lo));
                const float p2 = exp2f(fmaf(s[j][2], sl2, -use_hi)), p3 = exp2f(fmaf(s[j][3], sl2, -use_hi));
                sum_lo += p0 + p1;
                sum_hi += p2 + p3;
                pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_lo = l_lo * a_lo + sum_lo;
            l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int jp = 0; jp < NT_O / 2; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    const int id = lane >> 3, rr = lane & 7;
                    const int key = ks * 16 + (id & 1) * 8 + rr;
                    ldmatrix_x4_trans(b0, b1, b2, b3, tV + key * VS + (jp * 2 + (id >> 1)) * 8);
                    mma_bf16(o[jp * 2], pf[ks], b0, b1);
                    mma_bf16(o[jp * 2 + 1], pf[ks], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inv_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        const int col = j * 8 + (lane & 3) * 2;
        const size_t at_lo = ((size_t)(row0 + r_lo) * H + h) * DV + col, at_hi = ((size_t)(row0 + r_hi) * H + h) * DV + col;
        if (out32 != nullptr) {
            if (valid_lo) *reinterpret_cast<float2*>(out32 + at_lo) = make_float2(o[j][0] * inv_lo, o[j][1] * inv_lo);
            if (valid_hi) *reinterpret_cast<float2*>(out32 + at_hi) = make_float2(o[j][2] * inv_hi, o[j][3] * inv_hi);
        } else {
            if (valid_lo) *reinterpret_cast<uint32_t*>(out + at_lo) = pack_bf16(o[j][0] * inv_lo, o[j][1] * inv_lo);
            if (valid_hi) *reinterpret_cast<uint32_t*>(out + at_hi) = pack_bf16(o[j][2] * inv_hi, o[j][3] * inv_hi);
        }
    }
}

// ---------------------------------------------------------------------------
// decode: items int32 [n_items] token rows (null: item i is token i)
// ---------------------------------------------------------------------------
template <int DK, int DV>
__global__ void __launch_bounds__(SATT_THREADS) attention_sink_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, float* __restrict__ out32, float* __restrict__ part_o,
    float* __restrict__ part_ml, const int32_t* __restrict__ items,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table,
    int table_width, int page_size, int H, int G, int window, float scale_log2, int sink, const float* __restrict__ sink_logit,
    const float* __restrict__ dist_bias, int dist_max, float softcap, int Gv) {
    constexpr int KS = DK + 8, VS = DV + 8;
    constexpr int KSTEPS = DK / 16;
    constexpr int NT_O = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [STAGES][64][KS]
    const float cap_in = softcap > 0.0f ? scale_log2 / (SINK_LOG2E_F * softcap) : 0.0f, cap_out = softcap * SINK_LOG2E_F;
    __nv_bfloat16* sV = sK + SDEC_STAGES * SKT * KS;                 // [STAGES][64][VS]

    const int item = blockIdx.x, g = blockIdx.y;
    const int t = items ? items[item] : item;
    const int pos = positions[t];
    const int k_end = pos + 1;
    const int k_begin = (window > 0 && k_end > window) ? k_end - window : 0;
    // gridDim.z CTAs share the token's key tiles evenly (a CTA may get none: it posts an empty partial result)
    const int n_splits = gridDim.z, split = blockIdx.z;
    const int kt_first = k_begin / SKT, kt_last = (k_end + SKT - 1) / SKT;
    const int per_split = (kt_last - kt_first + n_splits - 1) / n_splits;
    const int kt_begin = min(kt_last, kt_first + split * per_split), kt_end = min(kt_last, kt_begin + per_split);
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int qpg = H / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

#pragma unroll
    for (int st = 0; st < SDEC_STAGES - 1; ++st) {
        if (kt_begin + st < kt_end)
            load_kv_tile2<DK, DV>(sK + st * SKT * KS, sV + st * SKT * VS, k_pages, v_pages, table, (kt_begin + st) * SKT, k_begin, k_end,
                                  G, g, page_size, page_shift, Gv);
        cp_async_commit();
    }
    uint32_t qf[KSTEPS][4];
    {
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
        const __nv_bfloat16* q_lo = q + ((size_t)t * H + g * qpg + r_lo) * DK;
        const __nv_bfloat16* q_hi = q + ((size_t)t * H + g * qpg + r_hi) * DK;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int c = ks * 16 + (lane & 3) * 2;
            qf[ks][0] = r_lo < qpg ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
            qf[ks][1] = r_hi < qpg ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
            qf[ks][2] = r_lo < qpg ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
            qf[ks][3] = r_hi < qpg ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
        }
    }
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) % SDEC_STAGES;
        {
            const int nxt = kt + SDEC_STAGES - 1;
            if (nxt < kt_end) {
                const int nb = (nxt - kt_begin) % SDEC_STAGES;
                load_kv_tile2<DK, DV>(sK + nb * SKT * KS, sV + nb * SKT * VS, k_pages, v_pages, table, nxt * SKT, k_begin, k_end, G, g,
                                      page_size, page_shift, Gv);
            }
            cp_async_commit();
            cp_async_wait<SDEC_STAGES - 1>();
        }
        __syncthreads();
        const __nv_bfloat16* tK = sK + buf * SKT * KS + warp * 16 * KS;   // this warp's 16 keys
        const __nv_bfloat16* tV = sV + buf * SKT * VS + warp * 16 * VS;
        const int key0 = kt * SKT + warp * 16;
        if (key0 < k_end && key0 + 16 > k_begin) {
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
            s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t b0, b1, b2, b3;
                const int id = lane >> 3, rr = lane & 7;
                ldmatrix_x4(b0, b1, b2, b3, tK + ((id >> 1) * 8 + rr) * KS + ks * 16 + (id & 1) * 8);
                mma_bf16(s[0], qf[ks], b0, b1);
                mma_bf16(s[1], qf[ks], b2, b3);
            }
            float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    float v = -INFINITY;
                    if (key >= k_begin && key < k_end) {
                        // rows of the tile are the query heads of this kv head; the rows beyond them hold zero queries and
                        // scores, whose capped form is zero as well
                        const bool real_row = (lane >> 2) + (e >= 2 ? 8 : 0) < qpg;
                        v = softcap > 0.0f ? (real_row ? tanhf(s[j][e] * cap_in) * cap_out : 0.0f) : s[j][e] * scale_log2;
                        // the bias of (distance, head)
                        const int hq = g * qpg + (lane >> 2) + (e >= 2 ? 8 : 0);
                        if (dist_bias != nullptr && hq < H) v += dist_bias[(size_t)hq * (dist_max + 1) + min(pos - key, dist_max)] * SINK_LOG2E_F;
                    }
                    s[j][e] = v;
                    if (e >= 2) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float use_lo = (mx_lo == -INFINITY) ? 0.0f : mx_lo;
            const float use_hi = (mx_hi == -INFINITY) ? 0.0f : mx_hi;
            const float a_lo = exp2f(m_lo - use_lo), a_hi = exp2f(m_hi - use_hi);
            m_lo = mx_lo;
            m_hi = mx_hi;
            uint32_t pf[4];
            const float p00 = exp2f(s[0][0] - use_lo), p01 = exp2f(s[0][1] - use_lo);
            const float p02 = exp2f(s[0][2] - use_hi), p03 = exp2f(s[0][3] - use_hi);
            const float p10 = exp2f(s[1][0] - use_lo), p11 = exp2f(s[1][1] - use_lo);
            const float p12 = exp2f(s[1][2] - use_hi), p13 = exp2f(s[1][3] - use_hi);
            pf[0] = pack_bf16(p00, p01);
            pf[1] = pack_bf16(p02, p03);
            pf[2] = pack_bf16(p10, p11);
            pf[3] = pack_bf16(p12, p13);
            l_lo = l_lo * a_lo + (p00 + p01 + p10 + p11);
            l_hi = l_hi * a_hi + (p02 + p03 + p12 + p13);
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int id = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(b0, b1, b2, b3, tV + ((id & 1) * 8 + rr) * VS + (jp * 2 + (id >> 1)) * 8);
                mma_bf16(o[jp * 2], pf, b0, b1);
                mma_bf16(o[jp * 2 + 1], pf, b2, b3);
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    cp_async_wait<0>();
    __syncthreads();
    // merge the four warps (and the sink) through shared memory: the K/V buffers are free now
    float* mo = reinterpret_cast<float*>(smem_raw);         // [4][16][DV]
    float* mml = mo + 4 * 16 * DV;                          // [4][16][2]
    {
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            const int col = j * 8 + (lane & 3) * 2;
            float* base = mo + (size_t)warp * 16 * DV;
            base[r_lo * DV + col] = o[j][0];
            base[r_lo * DV + col + 1] = o[j][1];
            base[r_hi * DV + col] = o[j][2];
            base[r_hi * DV + col + 1] = o[j][3];
        }
        if ((lane & 3) == 0) {
            mml[(warp * 16 + r_lo) * 2] = m_lo;
            mml[(warp * 16 + r_lo) * 2 + 1] = l_lo;
            mml[(warp * 16 + r_hi) * 2] = m_hi;
            mml[(warp * 16 + r_hi) * 2 + 1] = l_hi;
        }
    }
    __syncthreads();
    const bool single = n_splits == 1;
    for (int idx = threadIdx.x; idx < qpg * DV; idx += SATT_THREADS) {
        const int r = idx / DV, col = idx - r * DV;
        const bool with_sink = (sink || sink_logit) && single;
        const float sink_m = sink_logit ? sink_logit[g * qpg + r] * SINK_LOG2E_F : 0.0f;
        float m = with_sink ? sink_m : -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, mml[(w * 16 + r) * 2]);
        const float mu = (m == -INFINITY) ? 0.0f : m;
        float l = with_sink ? exp2f(sink_m - mu) : 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(mml[(w * 16 + r) * 2] - mu);
            l += mml[(w * 16 + r) * 2 + 1] * f;
            acc += mo[((size_t)w * 16 + r) * DV + col] * f;
        }
        const int h = g * qpg + r;
        if (single) {
            const float res = l > 0.0f ? acc / l : 0.0f;
            if (out32 != nullptr) out32[((size_t)t * H + h) * DV + col] = res;
            else out[((size_t)t * H + h) * DV + col] = __float2bfloat16_rn(res);
        } else {
            const size_t p = ((size_t)item * H + h) * n_splits + split;
            part_o[p * DV + col] = acc;
            if (col == 0) {
                part_ml[p * 2] = m;
                part_ml[p * 2 + 1] = l;
            }
        }
    }
}

// The splits of every (item, head) put together in split order, with the sink's share: one block per (item, head).
__global__ void attention_sink_merge_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ out32, const float* __restrict__ part_o,
                                            const float* __restrict__ part_ml, const int32_t* __restrict__ items, int H, int dv,
                                            int n_splits, int sink, const float* __restrict__ sink_logit) {
    const int item = blockIdx.x, h = blockIdx.y;
    const int t = items ? items[item] : item;
    const size_t p0 = ((size_t)item * H + h) * n_splits;
    const bool with_sink = sink || sink_logit;
    const float sink_m = sink_logit ? sink_logit[h] * SINK_LOG2E_F : 0.0f;
    float m = with_sink ? sink_m : -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(p0 + s) * 2]);
    const float mu = (m == -INFINITY) ? 0.0f : m;
    float l = with_sink ? exp2f(sink_m - mu) : 0.0f;
    for (int s = 0; s < n_splits; ++s) l += part_ml[(p0 + s) * 2 + 1] * exp2f(part_ml[(p0 + s) * 2] - mu);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int col = threadIdx.x; col < dv; col += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) acc += part_o[(p0 + s) * dv + col] * exp2f(part_ml[(p0 + s) * 2] - mu);
        if (out32 != nullptr) out32[((size_t)t * H + h) * dv + col] = acc * inv;
        else out[((size_t)t * H + h) * dv + col] = __float2bfloat16_rn(acc * inv);
    }
}

static const float SINK_LOG2E = 1.4426950408889634f;

template <int DK, int DV>
static int launch_sink_prefill(const void* q, const void* k, const void* v, void* out, const void* tiles, int n_tiles,
                               const void* table, int table_width, int page_size, int H, int G, int window, float scale, int sink,
                               const void* sink_logit, const void* dist_bias, int dist_max, float softcap, int Gv, int out_f32,
                               cudaStream_t s) {
    const size_t smem = (size_t)(3 * 64 * (DK + 8) + 2 * 64 * (DV + 8)) * sizeof(__nv_bfloat16);
    auto kernel = attention_sink_prefill_kernel<DK, DV>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        mm_set_last_error("sink attention: shared memory for the prefill tile could not be set");
        return MM_ERR_UNSUPPORTED;
    }
    mm_launch(kernel, dim3(H, n_tiles), dim3(SATT_THREADS), smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
              (const __nv_bfloat16*)v, out_f32 ? nullptr : (__nv_bfloat16*)out, out_f32 ? (float*)out : nullptr, (const int32_t*)tiles,
              (const int32_t*)table, table_width, page_size, H, G,
              window, scale * SINK_LOG2E, sink, (const float*)sink_logit, (const float*)dist_bias, dist_max, softcap, Gv);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

template <int DK, int DV>
static int launch_sink_decode(const void* q, const void* k, const void* v, void* out, void* part_o, void* part_ml, int n_splits,
                              const void* items, int n_items,
                              const void* positions, const void* token_req, const void* table, int table_width, int page_size,
                              int H, int G, int window, float scale, int sink, const void* sink_logit, const void* dist_bias, int dist_max,
                              float softcap, int Gv, int out_f32, cudaStream_t s) {
    const size_t kv = (size_t)SDEC_STAGES * 64 * (DK + 8 + DV + 8) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(4 * 16 * DV + 4 * 16 * 2) * sizeof(float);
    const size_t smem = kv > merge ? kv : merge;
    auto kernel = attention_sink_decode_kernel<DK, DV>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        mm_set_last_error("sink attention: shared memory for the decode tiles could not be set");
        return MM_ERR_UNSUPPORTED;
    }
    mm_launch(kernel, dim3(n_items, G, n_splits), dim3(SATT_THREADS), smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
              (const __nv_bfloat16*)v, out_f32 ? nullptr : (__nv_bfloat16*)out, out_f32 ? (float*)out : nullptr, (float*)part_o,
              (float*)part_ml, (const int32_t*)items,
              (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)table, table_width, page_size, H, G, window,
              scale * SINK_LOG2E, sink, (const float*)sink_logit, (const float*)dist_bias, dist_max, softcap, Gv);
    MM_CHECK_LAUNCH();
    if (n_splits > 1) {
        mm_launch(attention_sink_merge_kernel, dim3(n_items, H), dim3(DV >= 64 ? 64 : 32), 0, s, out_f32 ? nullptr : (__nv_bfloat16*)out,
                  out_f32 ? (float*)out : nullptr, (const float*)part_o,
                  (const float*)part_ml, (const int32_t*)items, H, DV, n_splits, sink, (const float*)sink_logit);
        MM_CHECK_LAUNCH();
    }
    return MM_OK;
}

// the sizes the kernels are built for: keys and values of 32, 64, 96 or 128
#define SINK_DISPATCH(FN, ...)                                                         \
    switch (dk * 1000 + dv) {                                                          \
        case 32032: return FN<32, 32>(__VA_ARGS__);                                    \
        case 32064: return FN<32, 64>(__VA_ARGS__);                                    \
        case 32096: return FN<32, 96>(__VA_ARGS__);                                    \
        case 32128: return FN<32, 128>(__VA_ARGS__);                                   \
        case 64032: return FN<64, 32>(__VA_ARGS__);                                    \
        case 64064: return FN<64, 64>(__VA_ARGS__);                                    \
        case 64096: return FN<64, 96>(__VA_ARGS__);                                    \
        case 64128: return FN<64, 128>(__VA_ARGS__);                                   \
        case 96032: return FN<96, 32>(__VA_ARGS__);                                    \
        case 96064: return FN<96, 64>(__VA_ARGS__);                                    \
        case 96096: return FN<96, 96>(__VA_ARGS__);                                    \
        case 96128: return FN<96, 128>(__VA_ARGS__);                                   \
        case 128032: return FN<128, 32>(__VA_ARGS__);                                  \
        case 128064: return FN<128, 64>(__VA_ARGS__);                                  \
        case 128096: return FN<128, 96>(__VA_ARGS__);                                  \
        case 128128: return FN<128, 128>(__VA_ARGS__);                                 \
        default: break;                                                                \
    }

MM_EXPORT int mm_attention_sink_supported(int dk, int dv) {
    return (dk == 32 || dk == 64 || dk == 96 || dk == 128) && (dv == 32 || dv == 64 || dv == 96 || dv == 128);
}

MM_EXPORT int mm_attention_sink_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const void* tiles,
                                             int n_tiles, const void* block_table, int table_width, int page_size, int H, int G,
                                             int dk, int dv, int window, float scale, int sink, const void* sink_logit, const void* dist_bias,
                                             int dist_max, float softcap, int Gv, int out_f32, void* stream) {
    MM_REQUIRE(Gv >= 1 && G % Gv == 0 && softcap >= 0.0f, "sink attention: the value heads must divide the key heads");
    MM_REQUIRE(n_tiles >= 0 && H > 0 && G > 0 && H % G == 0, "sink attention: heads must be a positive multiple of kv heads");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0 && scale > 0.0f, "sink attention: bad page geometry, window or scale");
    if (n_tiles == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    SINK_DISPATCH(launch_sink_prefill, q, k_pages, v_pages, out, tiles, n_tiles, block_table, table_width, page_size, H, G, window, scale,
                  sink, sink_logit, dist_bias, dist_max, softcap, Gv, out_f32, s);
    mm_set_last_error("sink attention: key and value sizes must each be one of 32, 64, 96, 128");
    return MM_ERR_UNSUPPORTED;
}

// n_splits > 1: the key tiles of every token are shared out over that many CTAs, whose partial results go through
// part_o [n_items, H, n_splits, dv] and part_ml [n_items, H, n_splits, 2] (fp32) and a merge launch.
MM_EXPORT int mm_attention_sink_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o,
                                            void* part_ml, int n_splits, const void* items,
                                            int n_items, const void* positions, const void* token_req, const void* block_table,
                                            int table_width, int page_size, int H, int G, int dk, int dv, int window, float scale,
                                            int sink, const void* sink_logit, const void* dist_bias, int dist_max, float softcap, int Gv,
                                            int out_f32, void* stream) {
    MM_REQUIRE(Gv >= 1 && G % Gv == 0 && softcap >= 0.0f, "sink attention: the value heads must divide the key heads");
    MM_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)),
               "sink attention: 1..64 splits, with scratch for more than one");
    MM_REQUIRE(n_items >= 0 && H > 0 && G > 0 && H % G == 0 && H / G <= 16, "sink attention: at most 16 query heads per kv head");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "sink attention: bad page geometry or window");
    if (n_items == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    SINK_DISPATCH(launch_sink_decode, q, k_pages, v_pages, out, part_o, part_ml, n_splits, items, n_items, positions, token_req, block_table,
                  table_width, page_size, H, G, window, scale, sink, sink_logit, dist_bias, dist_max, softcap, Gv, out_f32, s);
    mm_set_last_error("sink attention: key and value sizes must each be one of 32, 64, 96, 128");
    return MM_ERR_UNSUPPORTED;
}
