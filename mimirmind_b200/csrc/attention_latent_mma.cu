// bfloat16 attention of many query heads over ONE shared key head whose leading `rank` numbers are also the value
// (latent attention with absorbed up-projections), on the tensor cores: mma.sync m16n8k16, fp32 accumulation, fp32
// softmax.  A token's cache row holds `wide = rank + extra` numbers; a query row holds the same `wide` numbers.
//
//   s_j = (q . row_j) * scale;  p = softmax_j over the keys j <= position (and inside the window, if one is given);
//   o = sum_j p_j row_j[0 : rank]
//
// One CTA (8 warps) owns a tile of 32 query rows, each row one (token, head) pair of one request; because every head
// reads the same keys, a key tile is fetched once for all of them.  Keys stream through shared memory in tiles of 32,
// gathered page by page with cp.async, two stages deep.  Per key tile:
//
//   1. scores: warp (rg, cg) multiplies the 16 query rows of row group rg with the 32 keys over every fourth 16-wide
//      slice of `wide` (slices cg, cg + 4, ...) and leaves its partial sums in shared memory;
//   2. softmax: eight threads per row add the four partial sums, scale and mask them, keep the running maximum and
//      mass of the row in registers, and leave the weights (bfloat16) and the row's rescale factor in shared memory;
//   3. values: warp (rg, cg) multiplies the weights of its 16 rows with columns [cg * 8 NT * ..) of the same key tile
//      (read transposed with ldmatrix) into its fp32 accumulators, NT n-tiles of 8 columns per warp (rank <= 32 NT).
//
// The key tiles of a query tile may be shared out over several CTAs (blockIdx.y); their partial results then go
// through scratch memory and a merge launch.  Positions come from the device, so a captured step replays with new ones.
#include "common.cuh"
#include "mma_sync.cuh"

#define LAT_ROWS 32        // query rows per CTA
#define LAT_KEYS 32        // keys per tile
#define LAT_THREADS 256    // 8 warps: 2 row groups x 4 column groups
#define LAT_SS 33          // stride of a row of partial scores (floats)
#define LAT_PS 40          // stride of a row of weights (bfloat16)
#define LAT_LOG2E 1.4426950408889634f

// 32 cache rows [32][WS] (WS = wide rounded up to 16, + 8); rows outside [lo, hi) and the padding are zero
__device__ __forceinline__ void latent_load_keys(__nv_bfloat16* dst, const __nv_bfloat16* __restrict__ pool,
                                                 const int32_t* __restrict__ table, int key0, int lo, int hi, int page_size,
                                                 int page_shift, int wide, int WS) {
    const int chunks = (WS - 8) / 8, real = wide / 8;
    for (int c = threadIdx.x; c < LAT_KEYS * chunks; c += LAT_THREADS) {
        const int r = c / chunks, part = c - r * chunks;
        const int key = key0 + r;
        __nv_bfloat16* d = dst + r * WS + part * 8;
        if (key >= lo && key < hi && part < real) {
            const int pidx = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
            const int slot = key - pidx * page_size;
            cp_async16(d, pool + ((size_t)table[pidx] * page_size + slot) * wide + part * 8);
        } else {
            *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
    }
}

// tiles: int32 [n_tiles, 5] = (request, first token row, tokens, first head, heads); row r of the tile is token
// first + r / heads, head first_head + r % heads; tokens * heads <= 32.
template <int NT>
__global__ void __launch_bounds__(LAT_THREADS) attention_latent_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool, __nv_bfloat16* __restrict__ out,
    float* __restrict__ out32, float* __restrict__ part_o, float* __restrict__ part_ml, const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ block_table, int table_width, int page_size, int H,
    int wide, int rank, int window, float scale_log2) {
    const int WP = (wide + 15) & ~15, WS = WP + 8, KSTEPS = WP / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [32][WS]
    __nv_bfloat16* sK = sQ + LAT_ROWS * WS;                                   // [2][32][WS]
    float* sS = reinterpret_cast<float*>(sK + 2 * LAT_KEYS * WS);             // [4][32][LAT_SS]
    float* sAlpha = sS + 4 * LAT_ROWS * LAT_SS;                               // [32]
    int* sPos = reinterpret_cast<int*>(sAlpha + LAT_ROWS);                    // [32]
    __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sPos + LAT_ROWS);    // [32][LAT_PS]

    const int tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int req = tiles[tile * 5 + 0], tok0 = tiles[tile * 5 + 1], n_tok = tiles[tile * 5 + 2];
    const int head0 = tiles[tile * 5 + 3], n_heads = tiles[tile * 5 + 4];
    const int n_rows = n_tok * n_heads;
    const int32_t* table = block_table + (size_t)req * table_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = warp >> 2, cg = warp & 3;

    const int pos_first = positions[tok0], pos_last = positions[tok0 + n_tok - 1];
    const int hi_all = pos_last + 1;
    const int lo_all = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;
    int kt_begin = lo_all / LAT_KEYS, kt_end = (hi_all + LAT_KEYS - 1) / LAT_KEYS;
    if (n_splits > 1) {
        const int per = (kt_end - kt_begin + n_splits - 1) / n_splits;
        kt_begin = kt_begin + split * per;
        kt_end = min(kt_end, kt_begin + per);
    }

    if (threadIdx.x < LAT_ROWS) sPos[threadIdx.x] = threadIdx.x < n_rows ? positions[tok0 + threadIdx.x / n_heads] : -1;
    {
        const int chunks = WP / 8, real = wide / 8;
        for (int c = threadIdx.x; c < LAT_ROWS * chunks; c += LAT_THREADS) {
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
        latent_load_keys(sK, pool, table, kt_begin * LAT_KEYS, lo_all, hi_all, page_size, page_shift, wide, WS);
    cp_async_commit();

    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    // the softmax stage: thread t holds row t / 8 and the keys (t % 8) * 4 .. + 3 of a tile
    const int srow = threadIdx.x >> 3, skey = (threadIdx.x & 7) * 4;
    float m_run = -INFINITY, l_run = 0.0f;
    const int col0 = cg * NT * 8;                    // this warp's first value column
    const int id = lane >> 3, rr = lane & 7;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        cp_async_wait<0>();
        __syncthreads();                             // tile kt has landed; everyone is done with tile kt - 1
        if (kt + 1 < kt_end) {
            latent_load_keys(sK + (buf ^ 1) * LAT_KEYS * WS, pool, table, (kt + 1) * LAT_KEYS, lo_all, hi_all, page_size,
                             page_shift, wide, WS);
            cp_async_commit();
        }
        const __nv_bfloat16* tK = sK + buf * LAT_KEYS * WS;
        const int key0 = kt * LAT_KEYS;
        // 1. partial scores of 16 rows x 32 keys over this warp's slices
        {
            float s[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
            for (int ks = cg; ks < KSTEPS; ks += 4) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], sQ + (rg * 16 + (id & 1) * 8 + rr) * WS + ks * 16 + (id >> 1) * 8);
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, tK + (jp * 16 + (id >> 1) * 8 + rr) * WS + ks * 16 + (id & 1) * 8);
                    mma_bf16(s[jp * 2], a, b0, b1);
                    mma_bf16(s[jp * 2 + 1], a, b2, b3);
                }
            }
            float* dst = sS + (cg * LAT_ROWS + rg * 16 + (lane >> 2)) * LAT_SS + (lane & 3) * 2;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dst[j * 8] = s[j][0];
                dst[j * 8 + 1] = s[j][1];
                dst[8 * LAT_SS + j * 8] = s[j][2];
                dst[8 * LAT_SS + j * 8 + 1] = s[j][3];
            }
        }
        __syncthreads();
        // 2. softmax of the tile's scores, row by row
        {
            const int pos = sPos[srow];
            const int wlo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            float sc[4];
            float mx = m_run;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float* src = sS + srow * LAT_SS + skey + e;
                const float v = (src[0] + src[LAT_ROWS * LAT_SS]) + (src[2 * LAT_ROWS * LAT_SS] + src[3 * LAT_ROWS * LAT_SS]);
                const int key = key0 + skey + e;
                sc[e] = (key <= pos && key >= wlo) ? v * scale_log2 : -INFINITY;
                mx = fmaxf(mx, sc[e]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float use = mx == -INFINITY ? 0.0f : mx;
            const float alpha = exp2f(m_run - use);        // m_run = -inf: 0
            float p[4], sum = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(sc[e] - use);
                sum += p[e];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            l_run = l_run * alpha + sum;
            m_run = mx;
            uint2 packed = make_uint2(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]));
            *reinterpret_cast<uint2*>(sP + srow * LAT_PS + skey) = packed;
            if ((threadIdx.x & 7) == 0) sAlpha[srow] = alpha;
        }
        __syncthreads();
        // 3. the weights times the leading `rank` numbers of the same rows
        {
            const float a_lo = sAlpha[rg * 16 + (lane >> 2)], a_hi = sAlpha[rg * 16 + 8 + (lane >> 2)];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], sP + (rg * 16 + (id & 1) * 8 + rr) * LAT_PS + ks * 16 + (id >> 1) * 8);
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    if (col0 + jp * 16 < rank) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(b0, b1, b2, b3, tK + (ks * 16 + (id & 1) * 8 + rr) * WS + col0 + (jp * 2 + (id >> 1)) * 8);
                        mma_bf16(o[jp * 2], a, b0, b1);
                        mma_bf16(o[jp * 2 + 1], a, b2, b3);
                    }
                }
            }
        }
    }
    // every row's mass and maximum, for the warps that hold its accumulators
    __syncthreads();
    if ((threadIdx.x & 7) == 0) {
        sAlpha[srow] = l_run;
        sS[srow] = m_run;
    }
    __syncthreads();
    const int r_lo = rg * 16 + (lane >> 2), r_hi = r_lo + 8;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r_hi : r_lo;
        if (r >= n_rows) continue;
        const int tok = tok0 + r / n_heads, h = head0 + r % n_heads;
        const size_t row = (size_t)tok * H + h;
        const float l = sAlpha[r];
        if (n_splits > 1) {
            float* dst = part_o + (row * n_splits + split) * rank;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int col = col0 + j * 8 + (lane & 3) * 2;
                if (col < rank) *reinterpret_cast<float2*>(dst + col) = make_float2(o[j][half * 2], o[j][half * 2 + 1]);
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
                const float x = o[j][half * 2] * inv, y = o[j][half * 2 + 1] * inv;
                if (out32 != nullptr) *reinterpret_cast<float2*>(out32 + row * rank + col) = make_float2(x, y);
                else *reinterpret_cast<uint32_t*>(out + row * rank + col) = pack_bf16(x, y);
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

static size_t latent_smem(int wide) {
    const int WS = ((wide + 15) & ~15) + 8;
    return (size_t)3 * LAT_ROWS * WS * 2 + (size_t)4 * LAT_ROWS * LAT_SS * 4 + LAT_ROWS * 8 + (size_t)LAT_ROWS * LAT_PS * 2;
}

template <int NT>
static int launch_latent(const void* q, const void* pool, void* out, void* part_o, void* part_ml, int n_splits, const void* tiles,
                         int n_tiles, int n_rows, const void* positions, const void* table, int table_width, int page_size, int H,
                         int wide, int rank, int window, float scale, int out_f32, cudaStream_t s) {
    const size_t smem = latent_smem(wide);
    auto kernel = attention_latent_kernel<NT>;
    static size_t allowed = 0;                     // per instantiation
    if (smem > allowed) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            mm_set_last_error("latent attention: the key tiles do not fit the shared memory");
            return MM_ERR_UNSUPPORTED;
        }
        allowed = smem;
    }
    mm_launch(kernel, dim3(n_tiles, n_splits), dim3(LAT_THREADS), smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool,
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

// sizes the kernel takes: rank a multiple of 16 up to 512, wide = rank + extra a multiple of 8 whose tiles fit
MM_EXPORT int mm_attention_latent_supported(int wide, int rank) {
    return rank >= 16 && rank <= 512 && rank % 16 == 0 && wide >= rank && wide % 8 == 0 && latent_smem(wide) <= 200 * 1024;
}

// q [n, H, wide] and pool [pages, page, wide] bfloat16; out [n, H, rank] bfloat16 or fp32.  tiles int32 [n_tiles, 5];
// n_rows = n * H.  n_splits > 1: part_o [n_rows, n_splits, rank] and part_ml [n_rows, n_splits, 2] (fp32).
MM_EXPORT int mm_attention_latent_bf16(const void* q, const void* pool, void* out, void* part_o, void* part_ml, int n_splits,
                                       const void* tiles, int n_tiles, int n_rows, const void* positions, const void* block_table,
                                       int table_width, int page_size, int H, int wide, int rank, int window, float scale, int out_f32,
                                       void* stream) {
    MM_REQUIRE(mm_attention_latent_supported(wide, rank), "latent attention: rank a multiple of 16 up to 512, row width a multiple of 8");
    MM_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o != nullptr && part_ml != nullptr)),
               "latent attention: 1..64 splits, with scratch for more than one");
    MM_REQUIRE(n_tiles >= 0 && H > 0 && page_size > 0 && table_width > 0 && window >= 0 && scale > 0.0f,
               "latent attention: bad heads, page geometry, window or scale");
    if (n_tiles == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (rank <= 64) return launch_latent<2>(q, pool, out, part_o, part_ml, n_splits, tiles, n_tiles, n_rows, positions, block_table, table_width, page_size, H, wide, rank, window, scale, out_f32, s);
    if (rank <= 128) return launch_latent<4>(q, pool, out, part_o, part_ml, n_splits, tiles, n_tiles, n_rows, positions, block_table, table_width, page_size, H, wide, rank, window, scale, out_f32, s);
    if (rank <= 256) return launch_latent<8>(q, pool, out, part_o, part_ml, n_splits, tiles, n_tiles, n_rows, positions, block_table, table_width, page_size, H, wide, rank, window, scale, out_f32, s);
    return launch_latent<16>(q, pool, out, part_o, part_ml, n_splits, tiles, n_tiles, n_rows, positions, block_table, table_width, page_size, H, wide, rank, window, scale, out_f32, s);
}
