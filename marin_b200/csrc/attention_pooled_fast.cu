// bf16 attention over a window of single positions and pooled blocks before it, with capped scores and the sums that mixing
// the heads' weights needs, on the tensor cores (mma.sync), compiled for one head layout:
//   -DHEAD_DIM (keys and queries), -DV_DIM (values), -DGROUP (query heads per kv head), -DVALUE_HEADS (kv heads whose values a
//   CTA sums at a time); both sizes multiples of 16 up to 128.
// Position i sees the positions j with max(0, i - window + 1) <= j <= i (window 0: from 0) and the pooled rows of the blocks
// b < nb(i) = max(0, (i - window + 1) / pool): one key and one value per block of `pool` positions, kept in the page of the
// block's last position at row (its offset) / pool (see attention_pooled.cu).  s = q . k * scale, capped: cap tanh(s / cap).
// Prompt portions: a CTA takes 64 queries of one query head g and walks 64-row blocks, first of pooled rows, then of
// positions; the scores use the keys of g's kv head, the weights (one running softmax per row) multiply the values of
// `VALUE_HEADS` kv heads at a time: with mixing (`all_heads`) every query head needs its weighted sum over every kv head's
// values, A[g][c] (float32 [tokens][H][K][V_DIM]), which a second kernel mixes, out_h = sum_g talk[h][g] A[g][kv(h)]; a CTA
// then takes the kv heads c0 .. c0 + VALUE_HEADS - 1 (blockIdx.y counts (g, c0 / VALUE_HEADS)) and repeats the scores for
// each such slice.  Without mixing a CTA sums the values of g's own kv head and writes bf16 [tokens][H][V_DIM].
// Single tokens (`single`: every request of the step brings one token): the tile's rows are the GROUP query heads of one kv
// head instead of 64 queries of one head (blockIdx.y counts (kv head, slice)), so the heads that share keys share their loads.
// `single` = 2 (mixing, at most four slices): a CTA takes a kv head's query heads with *all* slices, warp w working out the
// sums of slice w over the one copy of the keys (the scores are cheap enough to repeat per warp); the value buffer then holds
// every kv head's block.
// Scores, maxima and sums are float32 (in the exp2 domain); the weights are rounded to bf16 for the product with V.
#define MB_LIB "attention_pooled_fast"
#define MB_LIB_ID 19
#include "common.cuh"
#include "launch.cuh"
#include "mma_helpers.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#ifndef V_DIM
#define V_DIM HEAD_DIM
#endif
#ifndef GROUP
#define GROUP 4
#endif
#ifndef VALUE_HEADS
#define VALUE_HEADS 1
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "key heads: a multiple of 16 up to 128");
static_assert(V_DIM % 16 == 0 && V_DIM >= 16 && V_DIM <= 128, "value heads: a multiple of 16 up to 128");
static_assert(VALUE_HEADS >= 1 && VALUE_HEADS * V_DIM <= 256, "a thread keeps 16 rows x VALUE_HEADS * V_DIM sums in registers");

#define D HEAD_DIM
#define DV V_DIM
#define VH VALUE_HEADS
#define LDK (D + 8)                   // padded rows in shared memory (elements): ldmatrix without bank conflicts
#define LDV (DV + 8)
#define BM 64
#define BN 64
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tanh(x) = 1 - 2 / (1 + e^(2x)) from the fast exponential: its absolute error is a few 1e-7, which times the cap stays far below
// a score's rounding (the hardware's own tanh approximation is good to 2^-11 only, times a cap of 50 a visible 0.01 in a score)
__device__ __forceinline__ float tanh_approx(float x) {
    return 1.0f - __fdividef(2.0f, 1.0f + ex2_approx(x * (2.0f * LOG2E)));
}

// One 64-row block of keys (kv head kh) and of the values of `nvh` kv heads from c0 on (cp.async), two threads a row.  Rows
// [row_first, row_last] of the numbering are there, the others are zero.  pooled: row n is block n's pooled row; else position n.
__device__ __forceinline__ void load_block(bf16* dst_k, bf16* dst_v, const bf16* __restrict__ keys, const bf16* __restrict__ values,
                                           const int* __restrict__ table, int K, int kh, int c0, int nvh, int page_shift, int row0,
                                           int row_first, int row_last, bool pooled, int pool, int pool_rows, int which) {
    // which: 1 the keys, 2 the values, 3 both
    constexpr int CK = D / 8, CV = DV / 8;
    const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int n = row0 + row;
    bf16* dk = dst_k + row * LDK;
    if (n <= row_last && n >= row_first) {
        const int page_mask = (1 << page_shift) - 1;
        const int p = pooled ? n * pool + pool - 1 : n;                 // the position whose page holds the row
        const size_t page = (size_t)table[p >> page_shift];
        const size_t per_head = pooled ? (size_t)pool_rows : ((size_t)1 << page_shift);
        const size_t at = pooled ? (size_t)((p & page_mask) / pool) : (size_t)(p & page_mask);
        const bf16* sk = keys + ((page * K + kh) * per_head + at) * D;
        if (which & 1) {
#pragma unroll
            for (int c = half; c < CK; c += 2) cp_async16(dk + c * 8, sk + c * 8);
        }
#pragma unroll
        for (int v = 0; v < VH; ++v) {
            if (v < nvh && (which & 2)) {
                const bf16* sv = values + ((page * K + c0 + v) * per_head + at) * DV;
                bf16* dv = dst_v + (v * BN + row) * LDV;
#pragma unroll
                for (int c = half; c < CV; c += 2) cp_async16(dv + c * 8, sv + c * 8);
            }
        }
        for (int v = VH; v < nvh; ++v) {                  // (a CTA that holds every kv head's block: the heads beyond a slice)
            if (which & 2) {
                const bf16* sv = values + ((page * K + c0 + v) * per_head + at) * DV;
                bf16* dv = dst_v + (v * BN + row) * LDV;
#pragma unroll
                for (int c = half; c < CV; c += 2) cp_async16(dv + c * 8, sv + c * 8);
            }
        }
    } else {
        if (which & 1) {
#pragma unroll
            for (int c = half; c < CK; c += 2) *reinterpret_cast<uint4*>(dk + c * 8) = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int v = 0; v < VH; ++v) {
            if (v < nvh && (which & 2)) {
                bf16* dv = dst_v + (v * BN + row) * LDV;
#pragma unroll
                for (int c = half; c < CV; c += 2) *reinterpret_cast<uint4*>(dv + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        for (int v = VH; v < nvh; ++v) {
            if (which & 2) {
                bf16* dv = dst_v + (v * BN + row) * LDV;
#pragma unroll
                for (int c = half; c < CV; c += 2) *reinterpret_cast<uint4*>(dv + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    }
}
static_assert(BN == 64, "load_block: two of the 128 threads a row");

#define PF_SMEM ((BM * LDK + 2 * BN * LDK + VH * BN * LDV) * 2)       // queries, two key blocks in turn, one block of values

__global__ void __launch_bounds__(128) attn_pooled_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const bf16* __restrict__ k_pool,
    const bf16* __restrict__ v_pool, float* __restrict__ parts, bf16* __restrict__ out, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_tokens, const int* __restrict__ seq_lens, int first_req, int K, int page_shift, float scale, float cap,
    int window, int pool, int pool_rows, int all_heads, int single) {
    PDL_ENTER_EARLY();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache); k_pool = pdl_fresh(k_pool); v_pool = pdl_fresh(v_pool);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK0 = sQ + BM * LDK;
    bf16* sV = sK0 + 2 * BN * LDK;
    const int H = K * GROUP;
    const int slices = all_heads ? (K + VH - 1) / VH : 1;
    // (single: `h` is the first query head of the kv head, and row i of the tile is head h + i at the one position)
    const bool by_warp = single == 2;                        // every slice in this CTA, a warp each
    const int per_y = by_warp ? 1 : slices;
    const int r = first_req + blockIdx.z, h = single ? (blockIdx.y / per_y) * GROUP : blockIdx.y / per_y, qt = gridDim.x - 1 - blockIdx.x;
    const int tok0 = cu_tokens[r], n = cu_tokens[r + 1] - tok0;
    if (qt * BM >= n) return;
    const int len = seq_lens[r], pos0 = len - n;
    const int rows = single ? GROUP : min(BM, n - qt * BM);
    const int q_first = pos0 + qt * BM, q_last = single ? q_first : q_first + rows - 1;
    const int kh = h / GROUP;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // c0, nvh: the kv heads whose values this warp sums; load_c0, load_n: those the CTA's value buffer holds
    const int c0 = by_warp ? min(warp, slices - 1) * VH : all_heads ? (blockIdx.y % slices) * VH : kh;
    const int nvh = all_heads ? min(VH, K - c0) : 1;
    const int load_c0 = by_warp ? 0 : c0, load_n = by_warp ? K : nvh;
    const int* table = block_table + (size_t)r * max_pages;
    const int k_first = window > 0 ? max(0, q_first - window + 1) : 0;
    const int kb_first = k_first / BN, kb_last = q_last / BN;
    const bool pools = pool > 0 && window > 0;
    const int nb_most = pools ? max(0, (q_last - window + 1) / pool) : 0;      // pooled rows the tile's last query sees
    const int pooled_blocks = (nb_most + BN - 1) / BN;
    const int steps = pooled_blocks + (kb_last - kb_first + 1);
    {
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < BM * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * LDK + c * 8;
            if (row < rows) cp_async16(d, q + (single ? (size_t)tok0 * H + h + row : (size_t)(tok0 + qt * BM + row) * H + h) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    }
    const int tile_row = by_warp ? 0 : warp * 16;            // (by warp: every warp works on the one tile of GROUP heads)
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + (tile_row + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
    float o[VH][DV / 8][4];
#pragma unroll
    for (int v = 0; v < VH; ++v)
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[v][i][0] = o[v][i][1] = o[v][i][2] = o[v][i][3] = 0.0f; }
    const int row0 = tile_row + (lane >> 2);                  // this thread's rows: row0 and row0 + 8
    const int qp[2] = {single ? q_first : q_first + row0, single ? q_first : q_first + row0 + 8};
    const int lo[2] = {window > 0 ? max(0, qp[0] - window + 1) : 0, window > 0 ? max(0, qp[1] - window + 1) : 0};
    const int nb[2] = {pools ? max(0, (qp[0] - window + 1) / pool) : 0, pools ? max(0, (qp[1] - window + 1) / pool) : 0};
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f, cap_l2 = cap * LOG2E, sl2 = scale * LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    // The loads run ahead of the products: while block i is worked on, the keys of block i + 1 arrive in the other key buffer
    // (asked for at the top of step i), and the values of block i + 1 are asked for as soon as step i is done with the one
    // value buffer, so they arrive during the next step's scores.  cp.async groups complete in order: keys(i) | values(i) |
    // keys(i + 1) | ...; "all but the newest group" is what a step waits for, twice.
    auto fetch = [&](int step, int which) {
        const bool pooled = step < pooled_blocks;
        const int key0 = pooled ? step * BN : (kb_first + step - pooled_blocks) * BN;
        bf16* dk = sK0 + (step & 1) * BN * LDK;
        if (pooled) load_block(dk, sV, k_pool, v_pool, table, K, kh, load_c0, load_n, page_shift, key0, 0, nb_most - 1, true, pool, pool_rows, which);
        else load_block(dk, sV, k_cache, v_cache, table, K, kh, load_c0, load_n, page_shift, key0, k_first, q_last, false, pool, pool_rows, which);
        cp_async_commit();
    };
    fetch(0, 1);                                               // (the queries ride in this group's wait)
    fetch(0, 2);
    // a warp whose rows hold no head (or, by warp, that has no slice) only helps with the loads
    const bool idle = by_warp ? warp >= slices : (single && warp * 16 >= GROUP);
    for (int step = 0; step < steps; ++step) {
        const bool pooled = step < pooled_blocks;
        const int key0 = pooled ? step * BN : (kb_first + step - pooled_blocks) * BN;
        const bf16* sK = sK0 + (step & 1) * BN * LDK;
        cp_async_wait<1>();                                    // this block's keys are there (its values may still be on their way)
        __syncthreads();
        if (step + 1 < steps) fetch(step + 1, 1);
        else cp_async_commit();                                // (an empty group keeps the count of groups in step)
        if (idle) {
            cp_async_wait<1>();
            __syncthreads();
            __syncthreads();
            if (step + 1 < steps) fetch(step + 1, 2);
            else cp_async_commit();
            continue;
        }
        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t qa[4];
            ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
            for (int j = 0; j < BN / 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(k_addr + (uint32_t)(j * 8 * LDK * 2 + kk * 32), b0, b1, b2, b3);
                mma_bf16_16816(s[j], qa, b0, b1);
                mma_bf16_16816(s[j + 1], qa, b2, b3);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            const int key = key0 + j * 8 + 2 * (lane & 3);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1, kj = key + (e & 1);
                const bool seen = pooled ? kj < nb[rr] : (kj <= qp[rr] && kj >= lo[rr]);
                float v = cap > 0.0f ? cap_l2 * tanh_approx(s[j][e] * scale * inv_cap) : s[j][e] * sl2;
                s[j][e] = seen ? v : -INFINITY;
                mx[rr] = fmaxf(mx[rr], s[j][e]);
            }
        }
        float corr[2], base[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m_run[rr], mx[rr]);
            base[rr] = m_new == -INFINITY ? 0.0f : m_new;
            corr[rr] = ex2_approx(m_run[rr] - base[rr]);
            m_run[rr] = m_new;
        }
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[j][e] = ex2_approx(s[j][e] - base[e >> 1]);
                sum[e >> 1] += s[j][e];
            }
        }
        l_run[0] = l_run[0] * corr[0] + sum[0];
        l_run[1] = l_run[1] * corr[1] + sum[1];
        uint32_t pa[BN / 16][4];
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            pa[ks][0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pa[ks][1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pa[ks][2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[ks][3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
        }
        cp_async_wait<1>();                                    // this block's values are there
        __syncthreads();
        // O_c += P V_c for every kv head of the slice
#pragma unroll
        for (int v = 0; v < VH; ++v) {
            if (v < nvh) {
#pragma unroll
                for (int i = 0; i < DV / 8; ++i) { o[v][i][0] *= corr[0]; o[v][i][1] *= corr[0]; o[v][i][2] *= corr[1]; o[v][i][3] *= corr[1]; }
                const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + ((c0 - load_c0 + v) * BN + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
                    for (int dt = 0; dt < DV / 8; dt += 2) {
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4_trans(v_addr + (uint32_t)(ks * 16 * LDV * 2 + dt * 16), b0, b1, b2, b3);
                        mma_bf16_16816(o[v][dt], pa[ks], b0, b1);
                        mma_bf16_16816(o[v][dt + 1], pa[ks], b2, b3);
                    }
                }
            }
        }
        __syncthreads();                                       // everyone is done with the value buffer
        if (step + 1 < steps) fetch(step + 1, 2);
        else cp_async_commit();
    }
    cp_async_wait<0>();
    const int col = 2 * (lane & 3);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        float l = l_run[rr];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = row0 + 8 * rr;
        if (row < rows && !idle) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const size_t t = single ? (size_t)tok0 : (size_t)(tok0 + qt * BM + row);
            const int hh = single ? h + row : h;
            if (all_heads) {
#pragma unroll
                for (int v = 0; v < VH; ++v) {
                    if (v < nvh) {
                        float* dst = parts + ((t * H + hh) * K + c0 + v) * DV;
#pragma unroll
                        for (int i = 0; i < DV / 8; ++i)
                            *reinterpret_cast<float2*>(dst + i * 8 + col) = make_float2(o[v][i][2 * rr] * inv, o[v][i][2 * rr + 1] * inv);
                    }
                }
            } else {
                bf16* dst = out + (t * H + hh) * DV;
#pragma unroll
                for (int i = 0; i < DV / 8; ++i)
                    *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[0][i][2 * rr] * inv, o[0][i][2 * rr + 1] * inv);
            }
        }
    }
}

static int page_shift_of(int page_size) {
    for (int s = 0; s <= 6; ++s)
        if ((1 << s) == page_size) return s;
    return -1;
}

MB_API int mb_attn_pooled_layout(int* d, int* dv, int* group, int* value_heads) { *d = D; *dv = DV; *group = GROUP; *value_heads = VH; return 0; }

// Prompt portions: requests first_req .. first_req + count - 1 of the step.  all_heads: parts float32 [tokens][H][K][V_DIM] is
// written (every query head's weighted sum over every kv head's values); else out bf16 [tokens][H][V_DIM].
MB_API int mb_attn_pooled_prefill(const void* q, const void* k_cache, const void* v_cache, const void* k_pool, const void* v_pool, float* parts,
                                  void* out, const int* block_table, int max_pages, const int* cu_tokens, const int* seq_lens, int first_req,
                                  int count, int max_query_len, int K, int page_size, float scale, float cap, int window, int pool,
                                  int pool_rows, int all_heads, int single, int by_warp_from, cudaStream_t s) {
    if (count <= 0 || max_query_len <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || window < 0 || pool < 0 || (pool > 0 && (k_pool == nullptr || v_pool == nullptr))) return MB_ERR_BAD_SIZE;
    if (pool > 0 && pool_rows != (page_size + pool - 1) / pool) return MB_ERR_BAD_SIZE;
    const int slices = all_heads ? (K + VH - 1) / VH : 1;
    if (single && (max_query_len != 1 || GROUP > 16)) single = 0;
    size_t smem = PF_SMEM;
    if (single && all_heads && slices > 1 && slices <= 4 && count * K >= by_warp_from) {
        // every slice in one CTA: the value buffer holds all K heads' blocks, if that fits beside queries and keys.  Only where
        // requests x kv heads still fill the device (`by_warp_from` CTAs, twice the SMs by default): a CTA then walks its blocks
        // with loads four times as large, and with
        // few requests that latency counts for more than the keys read once instead of four times (measured at 4B sizes: batch
        // 64, 526 -> 425 us a call; batch 8, 73 -> 107 us)
        const size_t wide = (size_t)(BM * LDK + 2 * BN * LDK + K * BN * LDV) * 2;
        if (wide <= 200 * 1024) { single = 2; smem = wide > smem ? wide : smem; }
    }
    cudaFuncSetAttribute(attn_pooled_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid((max_query_len + BM - 1) / BM, single == 2 ? K : (single ? K : K * GROUP) * slices, count);
    return launch_kernel(attn_pooled_prefill_kernel, grid, 128, smem, s, 0, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         (const bf16*)k_pool, (const bf16*)v_pool, parts, (bf16*)out, block_table, max_pages, cu_tokens, seq_lens, first_req, K,
                         shift, scale, cap, window, pool, pool_rows, all_heads, single);
}
