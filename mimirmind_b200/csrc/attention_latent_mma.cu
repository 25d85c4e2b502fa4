// bfloat16 attention of many query heads over ONE shared key head whose leading `rank` numbers are also the value
// (latent attention with absorbed up-projections), on the tensor cores: mma.sync m16n8k16, fp32 accumulation, fp32
// softmax.  A token's cache row holds `wide = rank + extra` numbers; a query row holds the same `wide` numbers.
//
//   s_j = (q . row_j) * scale;  p = softmax_j over the keys j <= position (and inside the window, if one is given);
//   o = sum_j p_j row_j[0 : rank]
//
// One CTA (8 or 16 warps: 2 or 4 row groups of 4 warps) owns a tile of 32 or 64 query rows, each row one (token, head)
// pair of one request; because every head reads the same keys, a key tile is fetched once for all of them.  Keys stream through shared memory in tiles of 32,
// gathered page by page with cp.async, two stages deep.  Per key tile:
//
//   1. scores: warp (rg, cg) multiplies the 16 query rows of row group rg with the 32 keys over every fourth 16-wide
//      slice of `wide` (slices cg, cg + 4, ...) and leaves its partial sums in shared memory;
//   2. softmax: eight threads per row add the four partial sums, scale and mask them, keep the running maximum and
//      mass of the row in registers, and leave the weights (bfloat16) and the row's rescale factor in shared memory;
//   3. values: warp (rg, cg) multiplies the weights of its 16 rows with the columns [cg * 8 NT, (cg + 1) * 8 NT) of the
//      same key tile (read transposed with ldmatrix) into its fp32 accumulators, NT n-tiles of 8 columns per warp
//      (rank <= 32 NT).
// Stages 1 to 3 exchange data inside a row group only, so they are separated by a barrier of the group's four warps.
//
// The key tiles of a query tile may be shared out over several CTAs (blockIdx.y); their partial results then go
// through scratch memory and a merge launch.  Positions come from the device, so a captured step replays with new ones.
#include "common.cuh"
#include "mma_sync.cuh"

#define LAT_KEYS 32        // keys per tile
#define LAT_SS 33          // stride of a row of partial scores (floats)
#define LAT_PS 40          // stride of a row of weights (bfloat16)
#define LAT_LOG2E 1.4426950408889634f

// 32 cache rows [32][WS] (WS = wide rounded up to 16, + 8); rows outside [lo, hi) and the padding are zero
template <int THREADS>
__device__ __forceinline__ void latent_load_keys(__nv_bfloat16* dst, const __nv_bfloat16* __restrict__ pool,
                                                 const int32_t* __restrict__ table, int key0, int lo, int hi, int page_size,
                                                 int page_shift, int wide, int WS) {
    // a warp per row (one page lookup per row), a lane per 16-byte piece
    const int chunks = (WS - 8) / 8, real = wide / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < LAT_KEYS; r += THREADS / 32) {
        const int key = key0 + r;
        const bool ok = key >= lo && key < hi;
        const __nv_bfloat16* src = pool;
        if (ok) {
            const int pidx = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
            const int slot = key - pidx * page_size;
            src = pool + ((size_t)table[pidx] * page_size + slot) * wide;
        }
        __nv_bfloat16* d = dst + r * WS;
        for (int part = lane; part < chunks; part += 32) {
            if (ok && part < real) cp_async16(d + part * 8, src + part * 8);
            else *reinterpret_cast<uint4*>(d + part * 8) = make_uint4(0, 0, 0, 0);
        }
    }
}

// A barrier of the four warps of one row group (named barrier 1 + group): the partial scores, the weights and the
// rescale factors of a row are written and read inside its group only (the softmax threads of a group's rows are the
// group's own 128 threads), so the groups need not wait for one another between the stages of a key tile and one
// group's products overlap another's softmax.
__device__ __forceinline__ void group_sync(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

// tiles: int32 [n_tiles, 5] = (request, first token row, tokens, first head, heads); row r of the tile is token
// first + r / heads, head first_head + r % heads; tokens * heads <= 32 MT.  MT: 16-row tiles per warp (a CTA owns 32 MT rows).
template <int NT, int MT, int RG>
__global__ void __launch_bounds__(RG * 128) attention_latent_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool, __nv_bfloat16* __restrict__ out,
    float* __restrict__ out32, float* __restrict__ part_o, float* __restrict__ part_ml, const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ block_table, int table_width, int page_size, int H,
    int wide, int rank, int window, float scale_log2) {
    constexpr int THREADS = RG * 128;             // RG row groups x 4 column groups of one warp each
    constexpr int ROWS = 16 * MT * RG;            // query rows of the CTA
    constexpr int TPR = THREADS / ROWS;           // threads per row in the softmax stage
    constexpr int KPT = LAT_KEYS / TPR;           // keys per thread there
    const int WP = (wide + 15) & ~15, WS = WP + 8, KSTEPS = WP / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [ROWS][WS]
    __nv_bfloat16* sK = sQ + ROWS * WS;                                       // [2][32][WS]
    float* sS = reinterpret_cast<float*>(sK + 2 * LAT_KEYS * WS);             // [4][ROWS][LAT_SS]
    float* sAlpha = sS + 4 * ROWS * LAT_SS;                                   // [ROWS]
    int* sPos = reinterpret_cast<int*>(sAlpha + ROWS);                        // [ROWS]
    __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sPos + ROWS);        // [ROWS][LAT_PS]

    const int tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int req = tiles[tile * 5 + 0], tok0 = tiles[tile * 5 + 1], n_tok = tiles[tile * 5 + 2];
    const int head0 = tiles[tile * 5 + 3], n_heads = tiles[tile * 5 + 4];
    const int n_rows = n_tok * n_heads;
    const int32_t* table = block_table + (size_t)req * table_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = warp >> 2, cg = warp & 3;
    const int row_base = rg * 16 * MT;            // this warp's first row

    const int pos_first = positions[tok0], pos_last = positions[tok0 + n_tok - 1];
    const int hi_all = pos_last + 1;
    const int lo_all = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;
    int kt_begin = lo_all / LAT_KEYS, kt_end = (hi_all + LAT_KEYS - 1) / LAT_KEYS;
    if (n_splits > 1) {
        const int per = (kt_end - kt_begin + n_splits - 1) / n_splits;
        kt_begin = kt_begin + split * per;
        kt_end = min(kt_end, kt_begin + per);
    }

    if (threadIdx.x < ROWS) sPos[threadIdx.x] = threadIdx.x < n_rows ? positions[tok0 + threadIdx.x / n_heads] : -1;
    {
        const int chunks = WP / 8, real = wide / 8;
        for (int c = threadIdx.x; c < ROWS * chunks; c += THREADS) {
            const int r = c / chunks, part = c - r * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rows && part < real) {
                const int tok = tok0 + r / n_heads, h = head0 + r % n_heads;
                v = *reinterpret_cast<const uint4*>(q + ((size_t)tok * H + h) * wide + part * 8);
            }
            *reinterpret_cast<uint4*>(sQ + r * WS + part * 8) = v;
        }
    }
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    if (kt_begin < kt_end)
        latent_load_keys<THREADS>(sK, pool, table, kt_begin * LAT_KEYS, lo_all, hi_all, page_size, page_shift, wide, WS);
    cp_async_commit();

    float o[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j) o[mt][j][0] = o[mt][j][1] = o[mt][j][2] = o[mt][j][3] = 0.0f;
    // the softmax stage: thread t holds row t / TPR and the keys (t % TPR) * KPT .. + KPT - 1 of a tile
    const int srow = threadIdx.x / TPR, skey = (threadIdx.x % TPR) * KPT;
    float m_run = -INFINITY, l_run = 0.0f;
    const int col0 = cg * NT * 8;                    // this warp's first value column
    const int id = lane >> 3, rr = lane & 7;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();                             // tile kt has landed; everyone is done with tile kt - 1
        if (kt + 1 < kt_end) {
            latent_load_keys<THREADS>(sK + (buf ^ 1) * LAT_KEYS * WS, pool, table, (kt + 1) * LAT_KEYS, lo_all, hi_all, page_size,
                             page_shift, wide, WS);
            cp_async_commit();
        }
        const __nv_bfloat16* tK = sK + buf * LAT_KEYS * WS;
        const int key0 = kt * LAT_KEYS;
        // 1. partial scores of 16 MT rows x 32 keys over this warp's slices
        {
            float s[MT][4][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.0f;
            for (int ks = cg; ks < KSTEPS; ks += 4) {
                uint32_t a[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3],
                                sQ + (row_base + mt * 16 + (id & 1) * 8 + rr) * WS + ks * 16 + (id >> 1) * 8);
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, tK + (jp * 16 + (id >> 1) * 8 + rr) * WS + ks * 16 + (id & 1) * 8);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_bf16(s[mt][jp * 2], a[mt], b0, b1);
                        mma_bf16(s[mt][jp * 2 + 1], a[mt], b2, b3);
                    }
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                float* dst = sS + (cg * ROWS + row_base + mt * 16 + (lane >> 2)) * LAT_SS + (lane & 3) * 2;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dst[j * 8] = s[mt][j][0];
                    dst[j * 8 + 1] = s[mt][j][1];
                    dst[8 * LAT_SS + j * 8] = s[mt][j][2];
                    dst[8 * LAT_SS + j * 8 + 1] = s[mt][j][3];
                }
            }
        }
        group_sync(rg);
        // 2. softmax of the tile's scores, row by row
        {
            const int pos = sPos[srow];
            const int wlo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            float sc[KPT];
            float mx = m_run;
#pragma unroll
            for (int e = 0; e < KPT; ++e) {
                const float* src = sS + srow * LAT_SS + skey + e;
                const float v = (src[0] + src[ROWS * LAT_SS]) + (src[2 * ROWS * LAT_SS] + src[3 * ROWS * LAT_SS]);
                const int key = key0 + skey + e;
                sc[e] = (key <= pos && key >= wlo) ? v * scale_log2 : -INFINITY;
                mx = fmaxf(mx, sc[e]);
            }
#pragma unroll
            for (int d = 1; d < TPR; d <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            const float use = mx == -INFINITY ? 0.0f : mx;
            const float alpha = exp2f(m_run - use);        // m_run = -inf: 0
            float sum = 0.0f;
#pragma unroll
            for (int e = 0; e < KPT; ++e) {
                sc[e] = exp2f(sc[e] - use);
                sum += sc[e];
            }
#pragma unroll
            for (int d = 1; d < TPR; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
            l_run = l_run * alpha + sum;
            m_run = mx;
#pragma unroll
            for (int e = 0; e < KPT; e += 4)
                *reinterpret_cast<uint2*>(sP + srow * LAT_PS + skey + e) = make_uint2(pack_bf16(sc[e], sc[e + 1]), pack_bf16(sc[e + 2], sc[e + 3]));
            if (threadIdx.x % TPR == 0) sAlpha[srow] = alpha;
        }
        group_sync(rg);
        // 3. the weights times the leading `rank` numbers of the same rows
        {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float a_lo = sAlpha[row_base + mt * 16 + (lane >> 2)], a_hi = sAlpha[row_base + mt * 16 + 8 + (lane >> 2)];
                // a factor of 1 (no row of the warp met a new maximum in this tile) changes nothing
                if (__any_sync(0xffffffffu, a_lo != 1.0f || a_hi != 1.0f)) {
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        o[mt][j][0] *= a_lo; o[mt][j][1] *= a_lo; o[mt][j][2] *= a_hi; o[mt][j][3] *= a_hi;
                    }
                }
            }
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                uint32_t a[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3],
                                sP + (row_base + mt * 16 + (id & 1) * 8 + rr) * LAT_PS + ks * 16 + (id >> 1) * 8);
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    if (col0 + jp * 16 < rank) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(b0, b1, b2, b3, tK + (ks * 16 + (id & 1) * 8 + rr) * WS + col0 + (jp * 2 + (id >> 1)) * 8);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_bf16(o[mt][jp * 2], a[mt], b0, b1);
                            mma_bf16(o[mt][jp * 2 + 1], a[mt], b2, b3);
                        }
                    }
                }
            }
        }
    }
    // every row's mass and maximum, for the warps that hold its accumulators
    __syncthreads();
    if (threadIdx.x % TPR == 0) {
        sAlpha[srow] = l_run;
        sS[srow] = m_run;
    }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = row_base + mt * 16 + half * 8 + (lane >> 2);
            if (r >= n_rows) continue;
            const int tok = tok0 + r / n_heads, h = head0 + r % n_heads;
            const size_t row = (size_t)tok * H + h;
            const float l = sAlpha[r];
            if (n_splits > 1) {
                float* dst = part_o + (row * n_splits + split) * rank;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int col = col0 + j * 8 + (lane & 3) * 2;
                    if (col < rank) *reinterpret_cast<float2*>(dst + col) = make_float2(o[mt][j][half * 2], o[mt][j][half * 2 + 1]);
                }
                if (cg == 0 && (lane & 3) == 0) {
                    part_ml[(row * n_splits + split) * 2] = sS[r];
                    part_ml[(row * n_splits + split) * 2 + 1] = l;
                }
            } else {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int col = col0 + j * 8 + (lane & 3) * 2;
                    if (col >= rank) continue;
                    const float x = o[mt][j][half * 2] * inv, y = o[mt][j][half * 2 + 1] * inv;
                    if (out32 != nullptr) *reinterpret_cast<float2*>(out32 + row * rank + col) = make_float2(x, y);
                    else *reinterpret_cast<uint32_t*>(out + row * rank + col) = pack_bf16(x, y);
                }
            }
        }
    }
}

// out[row] = sum_s w_s o_s / sum_s w_s l_s with w_s = 2^(m_s - max m): the partial results of a row's splits
__global__ void attention_latent_merge_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ out32, const float* __restrict__ part_o,
                                              const float* __restrict__ part_ml, int rank, int n_splits) {
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, ml[s * 2]);
    float mass = 0.0f;
    for (int s = 0; s < n_splits; ++s) mass += ml[s * 2] == -INFINITY ? 0.0f : exp2f(ml[s * 2] - mx) * ml[s * 2 + 1];
    const float inv = mass > 0.0f ? 1.0f / mass : 0.0f;
    for (int col = threadIdx.x; col < rank; col += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float m = ml[s * 2];
            if (m != -INFINITY) acc = fmaf(exp2f(m - mx), part_o[(row * n_splits + s) * rank + col], acc);
        }
        if (out32 != nullptr) out32[row * rank + col] = acc * inv;
        else out[row * rank + col] = __float2bfloat16(acc * inv);
    }
}


static size_t latent_smem(int wide, int rows) {
    const int WS = ((wide + 15) & ~15) + 8;
    return (size_t)(rows + 2 * LAT_KEYS) * WS * 2 + (size_t)4 * rows * LAT_SS * 4 + rows * 8 + (size_t)rows * LAT_PS * 2;
}

#define LAT_ARGS const void* q, const void* pool, void* out, void* part_o, void* part_ml, int n_splits, const void* tiles, \
                 int n_tiles, int n_rows, const void* positions, const void* table, int table_width, int page_size, int H, \
                 int wide, int rank, int window, float scale, int out_f32, cudaStream_t s
#define LAT_PASS q, pool, out, part_o, part_ml, n_splits, tiles, n_tiles, n_rows, positions, table, table_width, page_size, H, \
                 wide, rank, window, scale, out_f32, s

template <int NT, int MT, int RG>
static int launch_latent(LAT_ARGS) {
    const size_t smem = latent_smem(wide, 16 * MT * RG);
    auto kernel = attention_latent_kernel<NT, MT, RG>;
    static size_t allowed = 0;                     // per instantiation
    if (smem > allowed) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            mm_set_last_error("latent attention: the key tiles do not fit the shared memory");
            return MM_ERR_UNSUPPORTED;
        }
        allowed = smem;
    }
    mm_launch(kernel, dim3(n_tiles, n_splits), dim3(RG * 128), smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool,
              out_f32 ? nullptr : (__nv_bfloat16*)out, out_f32 ? (float*)out : nullptr, (float*)part_o, (float*)part_ml,
              (const int32_t*)tiles, (const int32_t*)positions, (const int32_t*)table, table_width, page_size, H, wide, rank, window,
              scale * LAT_LOG2E);
    MM_CHECK_LAUNCH();
    if (n_splits > 1) {
        mm_launch(attention_latent_merge_kernel, dim3(n_rows), dim3(rank >= 256 ? 128 : 64), 0, s, out_f32 ? nullptr : (__nv_bfloat16*)out,
                  out_f32 ? (float*)out : nullptr, (const float*)part_o, (const float*)part_ml, rank, n_splits);
        MM_CHECK_LAUNCH();
    }
    return MM_OK;
}

#define LAT_SMEM_MAX (220 * 1024)

// sizes the kernel takes: rank a multiple of 16 up to 512, wide = rank + extra a multiple of 8 whose tiles fit
MM_EXPORT int mm_attention_latent_supported(int wide, int rank) {
    return rank >= 16 && rank <= 512 && rank % 16 == 0 && wide >= rank && wide % 8 == 0 && latent_smem(wide, 32) <= LAT_SMEM_MAX;
}

// the rows of a tile the kernel may be given for this width: 64 (sixteen warps) where that many query rows fit, else 32
MM_EXPORT int mm_attention_latent_tile_rows(int wide) { return latent_smem(wide, 64) <= LAT_SMEM_MAX ? 64 : 32; }

// q [n, H, wide] and pool [pages, page, wide] bfloat16; out [n, H, rank] bfloat16 or fp32.  tiles int32 [n_tiles, 5] of at
// most tile_rows (32 or 64) rows each; n_rows = n * H.  n_splits > 1: part_o [n_rows, n_splits, rank] and part_ml
// [n_rows, n_splits, 2] (fp32).
MM_EXPORT int mm_attention_latent_bf16(const void* q, const void* pool, void* out, void* part_o, void* part_ml, int n_splits,
                                       const void* tiles, int n_tiles, int tile_rows, int n_rows, const void* positions,
                                       const void* table, int table_width, int page_size, int H, int wide, int rank, int window,
                                       float scale, int out_f32, void* stream) {
    MM_REQUIRE(mm_attention_latent_supported(wide, rank), "latent attention: rank a multiple of 16 up to 512, row width a multiple of 8");
    MM_REQUIRE(tile_rows == 32 || (tile_rows == 64 && mm_attention_latent_tile_rows(wide) == 64), "latent attention: tiles of 32 or 64 rows");
    MM_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)),
               "latent attention: 1..64 splits, with scratch for more than one");
    MM_REQUIRE(n_tiles >= 0 && H > 0 && page_size > 0 && table_width > 0 && window >= 0 && scale > 0.0f,
               "latent attention: bad heads, page geometry, window or scale");
    if (n_tiles == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (tile_rows == 64) {
        if (rank <= 64) return launch_latent<2, 1, 4>(LAT_PASS);
        if (rank <= 128) return launch_latent<4, 1, 4>(LAT_PASS);
        if (rank <= 256) return launch_latent<8, 1, 4>(LAT_PASS);
        return launch_latent<16, 1, 4>(LAT_PASS);
    }
    if (rank <= 64) return launch_latent<2, 1, 2>(LAT_PASS);
    if (rank <= 128) return launch_latent<4, 1, 2>(LAT_PASS);
    if (rank <= 256) return launch_latent<8, 1, 2>(LAT_PASS);
    return launch_latent<16, 1, 2>(LAT_PASS);
}
