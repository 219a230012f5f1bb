// bf16 softmax attention with a sink, a chunked mask or a window, value heads of their own width and an output gate, on the
// tensor cores (mma.sync), compiled for one head layout:
//   -DHEAD_DIM (keys and queries), -DV_DIM (values), -DGROUP (query heads per kv head); both sizes multiples of 16 up to 128.
// A position i sees the keys j <= i with j >= lo(i) = max(i - window + 1 (window > 0), floor(i / chunk) chunk (chunk > 0), 0).
//   p_j = exp(s_j) / (sink + sum_j exp(s_j)), s_j = q_i . k_j * scale, sink = exp(b_h) (a key without a value whose score b_h is
//   0 or a learned number per query head, not scaled) or 0;
//   out_i = (sum_j p_j v_j) * sigmoid(gate_i) where a gate is given.
// Scores, maxima and sums are float32 (in the exp2 domain); the weights are rounded to bf16 for the product with V.
// Prompt portions: 64 queries x 64-key blocks per CTA, only the blocks between lo(first query) and the last query.
// Single tokens: the visible keys of a sequence split over CTAs, partial (max, sum, accumulator) merged by a second kernel
// in chunk order, which also adds the sink and applies the gate.
// K pages [page][kv_head][offset][HEAD_DIM], V pages [page][kv_head][offset][V_DIM].
// -DV_IN_K: there are no value pages; a position's values are the first V_DIM elements of its key row (a latent that keys and
// values share), so a key block in shared memory serves both products and nothing is fetched twice.  The pages then hold one
// kv head that every query head reads: the launchers' `K` only counts groups of GROUP query heads (a CTA's rows), so any
// number of query heads that is a multiple of GROUP can share the rows.
#define MB_LIB "attention_sink_fast"
#define MB_LIB_ID 15
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
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "key heads: a multiple of 16 up to 256");
static_assert(V_DIM % 16 == 0 && V_DIM >= 16 && V_DIM <= 128, "value heads: a multiple of 16 up to 128");
static_assert(GROUP >= 1 && GROUP <= 16, "1 to 16 query heads per kv head");

#define D HEAD_DIM
#define DV V_DIM
#define LDK (D + 8)                   // padded rows in shared memory (elements): ldmatrix without bank conflicts
#ifdef V_IN_K
static_assert(V_DIM <= HEAD_DIM, "values inside the key rows cannot be wider than the rows");
#define LDV LDK
#define V_ROWS 0                      // rows of shared memory a value block takes beside its key block
#else
#define LDV (DV + 8)
#define V_ROWS BN
#endif
#define BM 64
#define BN 64
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sigmoid_of(float s) { return __fdividef(1.0f, 1.0f + ex2_approx(s * -LOG2E)); }

__device__ __forceinline__ int first_seen(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    return lo;
}

// The rows of one 64-key block of K and V (cp.async); keys outside [k_first, k_last] are zero (their pages may not exist).
// Two threads a row (128 threads, 64 rows), each taking every other 16-byte piece: the page look-up and the row's address
// are worked out once a thread and block, and the copies that follow differ by constants.  (With one piece a thread and
// turn, index arithmetic and look-ups were most of the kernel's instructions: 800 a warp and block, against 36 MMAs.)
__device__ __forceinline__ void load_kv_block(bf16* dst_k, bf16* dst_v, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                              const int* __restrict__ table, int K, int kh, int page_shift, int key0, int k_first, int k_last) {
#ifdef V_IN_K
    constexpr int CK = D / 8, CV = 0;
#else
    constexpr int CK = D / 8, CV = DV / 8;
#endif
    const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int key = key0 + row;
    bf16* dk = dst_k + row * LDK;
    bf16* dv = dst_v + row * LDV;
    if (key <= k_last && key >= k_first) {
        const int page_mask = (1 << page_shift) - 1;
#ifdef V_IN_K
        const size_t slot = ((size_t)table[key >> page_shift] << page_shift) + (size_t)(key & page_mask);       // one kv head
#else
        const size_t slot = (((size_t)table[key >> page_shift] * K + kh) << page_shift) + (size_t)(key & page_mask);
#endif
        const bf16* sk = k_cache + slot * D;
#pragma unroll
        for (int c = half; c < CK; c += 2) cp_async16(dk + c * 8, sk + c * 8);
        if (CV > 0) {
            const bf16* sv = v_cache + slot * DV;
#pragma unroll
            for (int c = half; c < CV; c += 2) cp_async16(dv + c * 8, sv + c * 8);
        }
    } else {
#pragma unroll
        for (int c = half; c < CK; c += 2) *reinterpret_cast<uint4*>(dk + c * 8) = make_uint4(0, 0, 0, 0);
        if (CV > 0) {
#pragma unroll
            for (int c = half; c < CV; c += 2) *reinterpret_cast<uint4*>(dv + c * 8) = make_uint4(0, 0, 0, 0);
        }
    }
}
static_assert(BN == 64, "load_kv_block: two of the 128 threads a row");

#define PF_SMEM ((BM * LDK + BN * LDK + V_ROWS * LDV) * 2)

__global__ void __launch_bounds__(128, 2) attn_sink_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, bf16* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_tokens, const int* __restrict__ seq_lens,
    int first_req, int K, int page_shift, float scale, int window, int chunk, int sink, const float* __restrict__ sink_logit,
    const bf16* __restrict__ gate, int gate_stride) {
    PDL_ENTER_EARLY();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache); gate = pdl_fresh(gate);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + BM * LDK;
#ifdef V_IN_K
    bf16* sV = sK;
#else
    bf16* sV = sK + BN * LDK;
#endif
    const int H = K * GROUP;
    const int r = first_req + blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;   // long tiles first
    const int tok0 = cu_tokens[r], n = cu_tokens[r + 1] - tok0;
    if (qt * BM >= n) return;
    const int len = seq_lens[r], pos0 = len - n;
    const int rows = min(BM, n - qt * BM);
    const int q_first = pos0 + qt * BM, q_last = q_first + rows - 1;
    const int kh = h / GROUP;
    const int* table = block_table + (size_t)r * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_first = first_seen(q_first, window, chunk);       // lo() never decreases with the position
    const int kb_first = k_first / BN, kb_last = q_last / BN;
    {
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < BM * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * LDK + c * 8;
            if (row < rows) cp_async16(d, q + ((size_t)(tok0 + qt * BM + row) * H + h) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
        load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, kb_first * BN, k_first, q_last);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int row0 = warp * 16 + (lane >> 2);                 // this thread's rows: row0 and row0 + 8
    const int qp[2] = {q_first + row0, q_first + row0 + 8};
    const int lo[2] = {first_seen(qp[0], window, chunk), first_seen(qp[1], window, chunk)};
    const float sl2 = scale * LOG2E;
    // running maximum (log2 units) and this thread's share of the running sum, per row; the sink is a score (0 or the head's
    // learned number, not scaled) and a 1 in the sum
    float m_run[2], l_run[2];
    m_run[0] = m_run[1] = sink ? (sink_logit != nullptr ? sink_logit[h] * LOG2E : 0.0f) : -INFINITY;
    l_run[0] = l_run[1] = (sink && (lane & 3) == 0) ? 1.0f : 0.0f;

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int key0 = kb * BN;
        if (kb > kb_first) {                                   // the barrier at the end of the last block freed the buffers
            load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, key0, k_first, q_last);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
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
        // a block that lies wholly between the last row's first seen key and the first row's position needs no mask
        const bool interior = key0 + BN - 1 <= q_first && key0 >= first_seen(q_last, window, chunk);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            const int key = key0 + j * 8 + 2 * (lane & 3);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1, kj = key + (e & 1);
                const float v = s[j][e] * sl2;
                s[j][e] = (interior || (kj <= qp[rr] && kj >= lo[rr])) ? v : -INFINITY;
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
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // O += P V
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int dt = 0; dt < DV / 8; dt += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(v_addr + (uint32_t)(ks * 16 * LDV * 2 + dt * 16), b0, b1, b2, b3);
                mma_bf16_16816(o[dt], pa, b0, b1);
                mma_bf16_16816(o[dt + 1], pa, b2, b3);
            }
        }
        __syncthreads();                                       // everyone is done with this block's buffers
    }
    const int col = 2 * (lane & 3);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        float l = l_run[rr];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = row0 + 8 * rr;
        if (row < rows) {
            const float inv = 1.0f / l;
            const size_t t = (size_t)(tok0 + qt * BM + row);
            bf16* dst = out + (t * H + h) * DV;
            const bf16* grow = gate != nullptr ? gate + t * gate_stride + (size_t)h * DV : nullptr;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                float a = o[i][2 * rr] * inv, b = o[i][2 * rr + 1] * inv;
                if (grow != nullptr) {
                    const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(grow + i * 8 + col));
                    a *= sigmoid_of(gg.x);
                    b *= sigmoid_of(gg.y);
                }
                *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(a, b);
            }
        }
    }
}

// ---- single tokens: the visible keys of a sequence split over CTAs -------------------------------------------------------
// CTA (chunk, kv head, request): keys [start + chunk * split, + split) where start = lo(pos) rounded down to a block of 64; the
// GROUP query heads of the kv head are rows 0..GROUP-1 of a 16-row tile (a thread holds row g of the tile's upper half and,
// with more than 8 heads, row g + 8 of the lower: two running maxima and sums); warp w takes keys 16 w .. 16 w + 15 of every
// block with a running (max, sum) of its own.  The four warps are merged in shared memory in warp order and written as the chunk's
// part: acc[chunk][request][head][DV] and ml[chunk][request][head][2] (max in log2 units, sum), float32.
// Rows that are keys and values both are fetched a block ahead, into the other of two buffers: a block of many heads over
// one row takes about as long to compute as to fetch, and two buffers of rows still leave room for four CTAs an SM.  Keys
// and values of their own keep one buffer (two halved the CTAs per SM and were slower: 36.8 -> 45.0 us a call at batch 8).
#ifdef V_IN_K
#define DEC_STAGES 2
#else
#define DEC_STAGES 1
#endif
#define DEC_STAGE_ELEMS (BN * LDK + V_ROWS * LDV)
#define DEC_KV_BYTES (DEC_STAGES * DEC_STAGE_ELEMS * 2)
#define DEC_SUM_BYTES (4 * GROUP * DV * 4)                 // the warps' sums are written over the key and value block
#define DEC_SMEM (16 * LDK * 2 + (DEC_KV_BYTES > DEC_SUM_BYTES ? DEC_KV_BYTES : DEC_SUM_BYTES))
#define DEC_LOWER (GROUP > 8)                              // the tile's rows 8..15 hold query heads too

__global__ void __launch_bounds__(128, 4) attn_sink_decode_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, float* __restrict__ part_acc,
    float* __restrict__ part_ml, const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_lens, int K,
    int page_shift, float scale, int window, int chunk_size, int split) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ float s_m[4][16], s_l[4][16];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK0 = sQ + 16 * LDK;
    const int chunk = blockIdx.x, kh = blockIdx.y, r = blockIdx.z, R = gridDim.z;
    const int H = K * GROUP;
    const int len = seq_lens[r], pos = len - 1;
    if (len <= 0) return;
    const int lo = first_seen(pos, window, chunk_size);
    const int c_begin = (lo / BN) * BN + chunk * split, c_end = min(len, c_begin + split);
    if (c_begin >= len) return;
    const int* table = block_table + (size_t)r * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < 16 * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * LDK + c * 8;
            if (row < GROUP) cp_async16(d, q + ((size_t)r * H + kh * GROUP + row) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
    }
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int g = lane >> 2;                                   // this thread's row of the tile: a query head if g < GROUP
    const float sl2 = scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.0f;
    float m_low = -INFINITY, l_low = 0.0f;                    // row g + 8 (used with more than 8 heads)
#ifdef V_IN_K
    load_kv_block(sK0, sK0, k_cache, v_cache, table, K, kh, page_shift, c_begin, lo, pos);
    cp_async_commit();
    int stage = 0;
#endif
    for (int key0 = c_begin; key0 < c_end; key0 += BN) {
#ifdef V_IN_K
        bf16* sK = sK0 + stage * DEC_STAGE_ELEMS;
        bf16* sV = sK;
        if (key0 + BN < c_end) {                               // the next block, into the buffer the last block's products have left
            bf16* next = sK0 + (stage ^ 1) * DEC_STAGE_ELEMS;
            load_kv_block(next, next, k_cache, v_cache, table, K, kh, page_shift, key0 + BN, lo, pos);
        }
        cp_async_commit();
        cp_async_wait<1>();                                    // all but the newest group: this block (and the queries) are here
        stage ^= 1;
#else
        bf16* sK = sK0;
        bf16* sV = sK + BN * LDK;
        load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, key0, lo, pos);
        cp_async_commit();
        cp_async_wait<0>();
#endif
        __syncthreads();
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t qa[4], b0, b1, b2, b3;
            ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
            ldsm_x4(k_addr + (uint32_t)(kk * 32), b0, b1, b2, b3);
            mma_bf16_16816(s[0], qa, b0, b1);
            mma_bf16_16816(s[1], qa, b2, b3);
        }
        float mx = -INFINITY, mx_low = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {                      // elements 2 and 3 belong to rows 8..15
                const int key = key0 + warp * 16 + j * 8 + 2 * (lane & 3) + e;
                const bool seen = key <= pos && key >= lo;
                s[j][e] = seen ? s[j][e] * sl2 : -INFINITY;
                mx = fmaxf(mx, s[j][e]);
                if (DEC_LOWER) {
                    s[j][2 + e] = seen ? s[j][2 + e] * sl2 : -INFINITY;
                    mx_low = fmaxf(mx_low, s[j][2 + e]);
                }
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float base = m_new == -INFINITY ? 0.0f : m_new;
        const float corr = ex2_approx(m_run - base);
        m_run = m_new;
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = ex2_approx(s[j][0] - base);
            s[j][1] = ex2_approx(s[j][1] - base);
            sum += s[j][0] + s[j][1];
        }
        l_run = l_run * corr + sum;
        float corr_low = 1.0f;
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = 0u;
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = 0u;
        if (DEC_LOWER) {
            mx_low = fmaxf(mx_low, __shfl_xor_sync(0xffffffffu, mx_low, 1));
            mx_low = fmaxf(mx_low, __shfl_xor_sync(0xffffffffu, mx_low, 2));
            const float m_new_low = fmaxf(m_low, mx_low);
            const float base_low = m_new_low == -INFINITY ? 0.0f : m_new_low;
            corr_low = ex2_approx(m_low - base_low);
            m_low = m_new_low;
            float sum_low = 0.0f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][2] = ex2_approx(s[j][2] - base_low);
                s[j][3] = ex2_approx(s[j][3] - base_low);
                sum_low += s[j][2] + s[j][3];
            }
            l_low = l_low * corr_low + sum_low;
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
        }
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
#pragma unroll
        for (int dt = 0; dt < DV / 8; dt += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(v_addr + (uint32_t)(dt * 16), b0, b1, b2, b3);
            o[dt][0] *= corr; o[dt][1] *= corr; o[dt + 1][0] *= corr; o[dt + 1][1] *= corr;
            if (DEC_LOWER) { o[dt][2] *= corr_low; o[dt][3] *= corr_low; o[dt + 1][2] *= corr_low; o[dt + 1][3] *= corr_low; }
            mma_bf16_16816(o[dt], pa, b0, b1);
            mma_bf16_16816(o[dt + 1], pa, b2, b3);
        }
        __syncthreads();
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (DEC_LOWER) {
        l_low += __shfl_xor_sync(0xffffffffu, l_low, 1);
        l_low += __shfl_xor_sync(0xffffffffu, l_low, 2);
    }
    cp_async_wait<0>();
    float* sums = reinterpret_cast<float*>(sK0);              // [4 warps][GROUP][DV]
    if (g < GROUP) {
        const int col = 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            sums[(warp * GROUP + g) * DV + i * 8 + col] = o[i][0];
            sums[(warp * GROUP + g) * DV + i * 8 + col + 1] = o[i][1];
        }
        if ((lane & 3) == 0) { s_m[warp][g] = m_run; s_l[warp][g] = l_run; }
    }
    if (DEC_LOWER && g + 8 < GROUP) {
        const int col = 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            sums[(warp * GROUP + g + 8) * DV + i * 8 + col] = o[i][2];
            sums[(warp * GROUP + g + 8) * DV + i * 8 + col + 1] = o[i][3];
        }
        if ((lane & 3) == 0) { s_m[warp][g + 8] = m_low; s_l[warp][g + 8] = l_low; }
    }
    __syncthreads();
    const size_t at = ((size_t)chunk * R + r) * H + (size_t)kh * GROUP;
    for (int idx = threadIdx.x; idx < GROUP * DV; idx += 128) {
        const int gg = idx / DV;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][gg]);
        float a = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = s_m[w][gg] == -INFINITY ? 0.0f : exp2f(s_m[w][gg] - mm);
            a = fmaf(sums[w * GROUP * DV + idx], f, a);
            ll = fmaf(s_l[w][gg], f, ll);
        }
        part_acc[at * DV + idx] = a;
        if (idx % DV == 0) { part_ml[(at + gg) * 2] = mm; part_ml[(at + gg) * 2 + 1] = ll; }
    }
}

// out[r][h][:] = (sum_c acc_c 2^(m_c - M)) / (sink 2^(b_h - M) + sum_c l_c 2^(m_c - M)) * sigmoid(gate), chunks in increasing order.
// A block per (request, head): the chunks' weights 2^(m_c - M) are made side by side, then every output is one sum over the chunks.
#define MG_THREADS 128
#define MG_MAX_CHUNKS 1024
__global__ void __launch_bounds__(MG_THREADS) attn_sink_merge_kernel(
    const float* __restrict__ part_acc, const float* __restrict__ part_ml, const int* __restrict__ seq_lens, int split, int window,
    int chunk_size, int sink, const float* __restrict__ sink_logit, int R, int H, const bf16* __restrict__ gate, int gate_stride,
    bf16* __restrict__ out) {
    PDL_ENTER();
    part_acc = pdl_fresh(part_acc); part_ml = pdl_fresh(part_ml); gate = pdl_fresh(gate);
    __shared__ float wgt[MG_MAX_CHUNKS], scratch[32];
    const int r = blockIdx.x / H, h = blockIdx.x % H;
    const int len = seq_lens[r];
    if (len <= 0) return;
    const int pos = len - 1;
    const int start = (first_seen(pos, window, chunk_size) / BN) * BN;
    const int chunks = min((len - start + split - 1) / split, MG_MAX_CHUNKS);
    const float s0 = sink_logit != nullptr ? sink_logit[h] * LOG2E : 0.0f;        // the sink's score in log2 units
    float mx = sink ? s0 : -INFINITY;
    for (int c = threadIdx.x; c < chunks; c += MG_THREADS) {
        const float mc = part_ml[(((size_t)c * R + r) * H + h) * 2];
        wgt[c] = mc;
        mx = fmaxf(mx, mc);
    }
    const float M = block_max(mx, scratch);
    float part = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += MG_THREADS) {
        const float mc = wgt[c];
        const float f = mc == -INFINITY ? 0.0f : exp2f(mc - M);
        wgt[c] = f;
        part = fmaf(part_ml[(((size_t)c * R + r) * H + h) * 2 + 1], f, part);
    }
    const float total = block_sum(part, scratch) + (sink ? exp2f(s0 - M) : 0.0f);       // (its barriers publish wgt)
    const float inv = 1.0f / total;
    for (int i = threadIdx.x; i < DV; i += MG_THREADS) {
        float a = 0.0f;
        int c = 0;
        for (; c + 8 <= chunks; c += 8) {                      // eight loads in flight, added in chunk order
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = part_acc[(((size_t)(c + u) * R + r) * H + h) * DV + i];
#pragma unroll
            for (int u = 0; u < 8; ++u) a = fmaf(x[u], wgt[c + u], a);
        }
        for (; c < chunks; ++c) a = fmaf(part_acc[(((size_t)c * R + r) * H + h) * DV + i], wgt[c], a);
        a *= inv;
        if (gate != nullptr) a *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_stride + (size_t)h * DV + i])));
        out[((size_t)r * H + h) * DV + i] = __float2bfloat16_rn(a);
    }
}

static int page_shift_of(int page_size) {
    int s = 0;
    while ((1 << s) < page_size) ++s;
    return (1 << s) == page_size ? s : -1;
}

MB_API int mb_attn_sink_layout(int* d, int* dv, int* group) { *d = D; *dv = DV; *group = GROUP; return 0; }

// Single tokens: requests 0 .. requests - 1 bring one token each (token t belongs to request t).  part_acc: float32
// [chunks][requests][K * GROUP][V_DIM], part_ml: [chunks][requests][K * GROUP][2]; split: keys per chunk, a multiple of 64;
// chunks * split covers the most keys a token sees plus one block.
MB_API int mb_attn_sink_decode(const void* q, const void* k_cache, const void* v_cache, float* part_acc, float* part_ml,
                               const int* block_table, int max_pages, const int* seq_lens, int requests, int K, int page_size,
                               float scale, int window, int chunk, int split, int chunks, cudaStream_t s) {
    if (requests <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || split <= 0 || split % BN != 0 || chunks <= 0 || chunks > MG_MAX_CHUNKS || window < 0 || chunk < 0) return MB_ERR_BAD_SIZE;
    cudaFuncSetAttribute(attn_sink_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    return launch_kernel(attn_sink_decode_kernel, dim3(chunks, K, requests), 128, DEC_SMEM, s, 0, (const bf16*)q, (const bf16*)k_cache,
                         (const bf16*)v_cache, part_acc, part_ml, block_table, max_pages, seq_lens, K, shift, scale, window, chunk, split);
}

// The parts of every request merged in chunk order, with the sink and the gate: out bf16 [requests][K * GROUP][V_DIM].
MB_API int mb_attn_sink_merge(const float* part_acc, const float* part_ml, void* out, const int* seq_lens, int requests, int K, int window,
                              int chunk, int sink, const void* gate, int gate_stride, int split, const float* sink_logit, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (split <= 0) return MB_ERR_BAD_SIZE;
    return launch_kernel(attn_sink_merge_kernel, requests * K * GROUP, MG_THREADS, 0, s, 0, (const float*)part_acc,
                         (const float*)part_ml, seq_lens, split, window, chunk, sink, sink_logit, requests, K * GROUP, (const bf16*)gate, gate_stride,
                         (bf16*)out);
}

// Prompt portions: requests first_req .. first_req + count - 1 of the step.
MB_API int mb_attn_sink_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                                int max_pages, const int* cu_tokens, const int* seq_lens, int first_req, int count, int max_query_len,
                                int K, int page_size, float scale, int window, int chunk, int sink, const void* gate, int gate_stride,
                                const float* sink_logit, cudaStream_t s) {
    if (count <= 0 || max_query_len <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || window < 0 || chunk < 0) return MB_ERR_BAD_SIZE;
    cudaFuncSetAttribute(attn_sink_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    dim3 grid((max_query_len + BM - 1) / BM, K * GROUP, count);
    return launch_kernel(attn_sink_prefill_kernel, grid, 128, PF_SMEM, s, 0, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         (bf16*)out, block_table, max_pages, cu_tokens, seq_lens, first_req, K, shift, scale, window, chunk, sink, sink_logit,
                         (const bf16*)gate, gate_stride);
}
