// Grouped-query softmax attention over a window of single positions plus pooled blocks before it, with the heads' softmax
// weights mixed by a matrix.
//
// Position i sees the positions j with 0 <= i - j < window (window 0: every earlier one) and, where `pool` = P > 0, one key
// and value for every block b of P positions that lies wholly before the window: b P + P - 1 <= i - window, so the first
// nb(i) = max(0, (i - window + 1) / P) blocks.  A block's key is the mean of its P keys as the pages hold them, its value
// the mean of its values; they are made once, when the block's last position has been written (`pool_blocks_kernel`), and
// kept in the page of that position at row (offset of that position) / P (K pool pages [page][kv_head][rows][d]).  Single
// positions and blocks share one softmax.  Scores may be capped: s <- cap tanh(s / cap).
//
// Mixing (`talk`, [H][H]): w'_h(i, j) = sum_g talk[h][g] w_g(i, j), and head h applies w'_h to the values of its own kv head.
// Since sum_j w'_h(i, j) v_c(j) = sum_g talk[h][g] (sum_j w_g(i, j) v_c(j)), every query head g keeps one running softmax and
// one weighted sum per kv head c, A[g][c]; a second kernel mixes them: out_h = sum_g talk[h][g] A[g][kv(h)].  Without mixing a
// head keeps the sum over its own kv head only and writes its output itself.
//
// This file holds the plain kernels, which serve any size in both dtypes; sums, scores and weights are float32.
#define MB_LIB "attention_pooled"
#define MB_LIB_ID 17
#include "common.cuh"
#include "launch.cuh"

#define PB_THREADS 128

// ---- pooled rows: a block per (token, kv head); only a token that ends a block of `pool` positions does anything ---------
template <typename T>
__global__ void __launch_bounds__(PB_THREADS) pool_blocks_kernel(
    const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_index, const int* __restrict__ positions,
    const int* __restrict__ slot_mapping, int K, int d, int dv, int page_size, int pool, int pool_rows) {
    PDL_ENTER();
    k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    const int t = blockIdx.x, kh = blockIdx.y;
    const int pos = positions[t];
    if (slot_mapping[t] < 0 || (pos + 1) % pool != 0) return;
    const int* table = block_table + (size_t)req_index[t] * max_pages;
    const int first = pos + 1 - pool;
    const size_t dst_page = (size_t)table[pos / page_size];
    const size_t dst_row = (dst_page * K + kh) * pool_rows + (size_t)((pos % page_size) / pool);
    const float inv = 1.0f / (float)pool;
    for (int i = threadIdx.x; i < d + dv; i += PB_THREADS) {
        const bool key = i < d;
        const int e = key ? i : i - d;
        const int width = key ? d : dv;
        const T* src = key ? k_cache : v_cache;
        float sum = 0.0f;
        for (int j = 0; j < pool; ++j) {
            const int p = first + j;
            const size_t page = (size_t)table[p / page_size];
            sum += to_f32(src[((page * K + kh) * page_size + (size_t)(p % page_size)) * width + e]);
        }
        (key ? k_pool : v_pool)[dst_row * width + e] = from_f32<T>(sum * inv);
    }
}

MB_API int mb_pool_blocks(const void* k_cache, const void* v_cache, void* k_pool, void* v_pool, int dtype, const int* block_table,
                          int max_pages, const int* req_index, const int* positions, const int* slot_mapping, int tokens, int K, int d,
                          int dv, int page_size, int pool, int pool_rows, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (K <= 0 || d <= 0 || dv <= 0 || pool <= 0 || pool_rows != (page_size + pool - 1) / pool) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, K);
    if (dtype == MB_F32)
        return launch_kernel(pool_blocks_kernel<float>, grid, PB_THREADS, 0, s, 0, (const float*)k_cache, (const float*)v_cache,
                             (float*)k_pool, (float*)v_pool, block_table, max_pages, req_index, positions, slot_mapping, K, d, dv, page_size,
                             pool, pool_rows);
    if (dtype == MB_BF16)
        return launch_kernel(pool_blocks_kernel<bf16>, grid, PB_THREADS, 0, s, 0, (const bf16*)k_cache, (const bf16*)v_cache,
                             (bf16*)k_pool, (bf16*)v_pool, block_table, max_pages, req_index, positions, slot_mapping, K, d, dv, page_size,
                             pool, pool_rows);
    return MB_ERR_BAD_DTYPE;
}

// ---- attention: a block per (token, query head) walking the visible keys in runs of PA_THREADS --------------------------
#define PA_THREADS 128
#define PA_MAX_PER_THREAD 16      // value elements a thread sums: all kv heads' values, kv_heads * dv <= 2,048

// Key number n of a token's visible keys: the pooled blocks 0 .. blocks - 1 first, then the positions lo .. pos.
template <typename T>
__device__ __forceinline__ const T* visible_row(const T* pages, const T* pool_pages, const int* table, int n, int blocks, int lo, int K,
                                                int kh, int page_size, int pool, int pool_rows, int width) {
    if (n < blocks) {
        const int last = n * pool + pool - 1;
        const size_t page = (size_t)table[last / page_size];
        return pool_pages + ((page * K + kh) * pool_rows + (size_t)((last % page_size) / pool)) * width;
    }
    const int p = lo + (n - blocks);
    const size_t page = (size_t)table[p / page_size];
    return pages + ((page * K + kh) * page_size + (size_t)(p % page_size)) * width;
}

// parts: float32 [tokens][H][K][dv] (talk != null) ; out: [tokens][H][dv] (talk == null).
template <typename T>
__global__ void __launch_bounds__(PA_THREADS) attention_pooled_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, const T* __restrict__ k_pool,
    const T* __restrict__ v_pool, float* __restrict__ parts, T* __restrict__ out, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ req_index, const int* __restrict__ positions, const int* __restrict__ seq_lens, int H, int K, int d, int dv,
    int page_size, float scale, float cap, int window, int pool, int pool_rows, int all_heads) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache); k_pool = pdl_fresh(k_pool); v_pool = pdl_fresh(v_pool);
    extern __shared__ float smem[];
    float* qs = smem;                 // [d]
    float* ps = smem + d;             // [PA_THREADS]
    float* scratch = ps + PA_THREADS; // [32]
    const int t = blockIdx.x, head = blockIdx.y;
    const int own = head / (H / K);
    const int req = req_index[t];
    const int pos = positions[t];
    const bool live = seq_lens[req] > 0;          // a row that pads a captured batch sees nothing and gives zeros
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int blocks = (pool > 0 && window > 0) ? max(0, (pos - window + 1) / pool) : 0;
    const int total = live ? blocks + (pos - lo + 1) : 0;
    const int* table = block_table + (size_t)req * max_pages;
    const T* qrow = q + ((size_t)t * H + head) * d;
    for (int i = threadIdx.x; i < d; i += PA_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();
    const int c_lo = all_heads ? 0 : own, c_n = all_heads ? K : 1;
    const int elems = c_n * dv;

    float m = -INFINITY, l = 0.0f;
    float acc[PA_MAX_PER_THREAD];
#pragma unroll
    for (int r = 0; r < PA_MAX_PER_THREAD; ++r) acc[r] = 0.0f;

    for (int base = 0; base < total; base += PA_THREADS) {
        const int n = base + threadIdx.x;
        float s = -INFINITY;
        if (n < total) {
            const T* krow = visible_row(k_cache, k_pool, table, n, blocks, lo, K, own, page_size, pool, pool_rows, d);
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
            if (cap > 0.0f) s = cap * tanhf(s / cap);
        }
        const float block_top = block_max(s, scratch);
        const float m_new = fmaxf(m, block_top);
        const float corr = expf(m - m_new);       // exp(-inf) = 0 on the first run
        const float p = n < total ? expf(s - m_new) : 0.0f;
        __syncthreads();
        ps[threadIdx.x] = p;
        const float block_total = block_sum(p, scratch);      // has the barriers that publish ps
        l = l * corr + block_total;
        m = m_new;
        const int count = min(PA_THREADS, total - base);
#pragma unroll
        for (int r = 0; r < PA_MAX_PER_THREAD; ++r) {
            const int e = threadIdx.x + r * PA_THREADS;
            if (e < elems) {
                const int c = c_lo + e / dv, dd = e % dv;
                float a = acc[r] * corr;
                for (int j = 0; j < count; ++j) {
                    const T* vrow = visible_row(v_cache, v_pool, table, base + j, blocks, lo, K, c, page_size, pool, pool_rows, dv);
                    a = fmaf(ps[j], to_f32(vrow[dd]), a);
                }
                acc[r] = a;
            }
        }
        __syncthreads();
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int r = 0; r < PA_MAX_PER_THREAD; ++r) {
        const int e = threadIdx.x + r * PA_THREADS;
        if (e < elems) {
            if (all_heads) parts[((size_t)t * H + head) * K * dv + e] = acc[r] * inv;
            else out[((size_t)t * H + head) * dv + e] = from_f32<T>(acc[r] * inv);
        }
    }
}

MB_API int mb_attention_pooled(const void* q, const void* k_cache, const void* v_cache, const void* k_pool, const void* v_pool, float* parts,
                               void* out, int dtype, const int* block_table, int max_pages, const int* req_index, const int* positions,
                               const int* seq_lens, int tokens, int H, int K, int d, int dv, int page_size, float scale, float cap, int window,
                               int pool, int pool_rows, int all_heads, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || K <= 0 || H % K != 0 || window < 0 || pool < 0) return MB_ERR_BAD_SIZE;
    if ((all_heads ? K : 1) * dv > PA_THREADS * PA_MAX_PER_THREAD) return MB_ERR_BAD_SIZE;
    if (pool > 0 && (k_pool == nullptr || v_pool == nullptr)) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, H);
    const size_t smem = (size_t)(d + PA_THREADS + 32) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(attention_pooled_kernel<float>, grid, PA_THREADS, smem, s, 0, (const float*)q, (const float*)k_cache,
                             (const float*)v_cache, (const float*)k_pool, (const float*)v_pool, parts, (float*)out, block_table, max_pages,
                             req_index, positions, seq_lens, H, K, d, dv, page_size, scale, cap, window, pool, pool_rows, all_heads);
    if (dtype == MB_BF16)
        return launch_kernel(attention_pooled_kernel<bf16>, grid, PA_THREADS, smem, s, 0, (const bf16*)q, (const bf16*)k_cache,
                             (const bf16*)v_cache, (const bf16*)k_pool, (const bf16*)v_pool, parts, (bf16*)out, block_table, max_pages,
                             req_index, positions, seq_lens, H, K, d, dv, page_size, scale, cap, window, pool, pool_rows, all_heads);
    return MB_ERR_BAD_DTYPE;
}

// ---- the heads' sums mixed: out[t][h][:] = sum_g talk[h][g] parts[t][g][kv(h)][:], a block per (token, kv head) -------------
// The H rows parts[t][:][c][:] go through shared memory once (each is read by all query heads of kv head c).
template <typename T>
__global__ void __launch_bounds__(256) talk_mix_kernel(const float* __restrict__ parts, const float* __restrict__ talk, T* __restrict__ out,
                                                       int H, int K, int dv) {
    PDL_ENTER();
    parts = pdl_fresh(parts);
    extern __shared__ float rows[];            // [H][dv]
    const int t = blockIdx.x, c = blockIdx.y, group = H / K;
    for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
        const int g = e / dv, dd = e - g * dv;
        rows[e] = parts[(((size_t)t * H + g) * K + c) * dv + dd];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < group * dv; e += blockDim.x) {
        const int h = c * group + e / dv, dd = e % dv;
        float sum = 0.0f;
        for (int g = 0; g < H; ++g) sum = fmaf(talk[h * H + g], rows[g * dv + dd], sum);
        out[((size_t)t * H + h) * dv + dd] = from_f32<T>(sum);
    }
}

MB_API int mb_talk_mix(const float* parts, const float* talk, void* out, int dtype, int tokens, int H, int K, int dv, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (H <= 0 || K <= 0 || H % K != 0 || dv <= 0) return MB_ERR_BAD_SIZE;
    const size_t smem = (size_t)H * dv * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, K);
    if (dtype == MB_F32) return launch_kernel(talk_mix_kernel<float>, grid, 256, smem, s, 0, parts, talk, (float*)out, H, K, dv);
    if (dtype == MB_BF16) return launch_kernel(talk_mix_kernel<bf16>, grid, 256, smem, s, 0, parts, talk, (bf16*)out, H, K, dv);
    return MB_ERR_BAD_DTYPE;
}
