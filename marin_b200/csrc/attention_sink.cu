// Causal grouped-query softmax attention over the paged cache with the options several designs combine:
//   * keys of `d` elements, values of `dv` (they may differ): K pages [page][kv_head][offset][d], V pages [..][dv];
//   * which keys a position sees: all before it, the last `window`, or those of its own chunk of `chunk` positions
//     (chunks counted from position 0 of the sequence, wherever a prompt was cut);
//   * a sink: one more term in the softmax's denominator, a key without a value whose score is 0 or a learned number per
//     query head (not scaled),  p_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j));
//   * values that are the leading `dv` elements of the key rows (a latent shared by keys and values): the value pointer is
//     the key pointer and `v_stride`, the distance between two positions' values, is the key rows' width;
//   * an output gate: the result is multiplied element by element with sigmoid(g), g a column block of the fused
//     projection.
// This file holds the head preparation (biases, RMS norm of q and k per head or over the whole projection, partial
// rotation with scaled sines and cosines, value mixing with the values an earlier layer left for the same tokens, cache
// write) and the plain attention kernel that serves any size in both dtypes.  Sums, norms, angles, scores and weights
// are float32.
#define MB_LIB "attention_sink"
#define MB_LIB_ID 13
#include "common.cuh"
#include "launch.cuh"

#define QF_THREADS 256            // at least; 1024 where a token's q and k have 4,096 elements and more

// ---- heads of the fused q|k|v(|g) projection, a token per block ---------------------------------------------------------
// A row of `row` holds q (H heads of d), k (K heads of d), v (K heads of dv), then whatever follows (the gate's columns).
// norm_mode 0: none; 1: per head over d, weight [d] shared by the heads; 2: over all of q (and all of k) at once, before
// the split into heads, weight [H d] (and [K d]).  The first rot_dim elements of a head are rotated in pairs
// (i, i + rot_dim/2), or (2i, 2i + 1) if `interleaved`, by the angle pos * inv_freq[i]; sines and cosines are multiplied by
// rot_mag.
// v_mode 0: values as they are; 1: they are also left in v_shared (activation dtype [tokens][K dv]) for later layers;
// 2: v <- (1 - lam) v + lam v_shared, lam = *v_lambda, and the mixed values go to the cache.
template <typename T>
__global__ void __launch_bounds__(1024) qkv_finish_kernel(
    const T* __restrict__ row, int row_stride, T* __restrict__ q_out, const float* __restrict__ q_b, const float* __restrict__ k_b,
    const float* __restrict__ v_b, int norm_mode, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim, float rot_mag,
    const int* __restrict__ slot_mapping, T* __restrict__ k_cache, T* __restrict__ v_cache, int v_mode, T* __restrict__ v_shared,
    const float* __restrict__ v_lambda, int H, int K, int d, int dv, int page_size, int write_kv, int interleaved) {
    PDL_ENTER();
    row = pdl_fresh(row); v_shared = pdl_fresh(v_shared);
    extern __shared__ float smem[];
    const int heads = write_kv ? H + K : H;
    const int half = rot_dim >> 1;
    float* vals = smem;                        // [heads * d]: q then k, float32
    float* cs_tab = vals + (size_t)heads * d;  // [half] cosines, [half] sines
    float* head_ss = cs_tab + 2 * half;        // [heads]
    __shared__ float s_factor[2];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x / 32, threads = blockDim.x;
    const T* src = row + (size_t)t * row_stride;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += threads) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = cs * rot_mag;
            cs_tab[half + i] = sn * rot_mag;
        }
    }
    // every element of q and k (+ bias) into shared memory as float32, all threads side by side
    const int qk = heads * d, q_len = H * d;
    for (int idx = threadIdx.x; idx < qk; idx += threads) {
        float v = to_f32(src[idx]);
        if (idx < q_len) { if (q_b != nullptr) v += q_b[idx]; }
        else if (k_b != nullptr) v += k_b[idx - q_len];
        vals[idx] = v;
    }
    __syncthreads();
    // sums of squares per head: a warp per head, lanes in a fixed order
    for (int head = warp; head < heads; head += warps) {
        float ss = 0.0f;
        for (int i = lane; i < d; i += 32) { const float v = vals[head * d + i]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) head_ss[head] = ss;
    }
    __syncthreads();
    if (norm_mode == 2 && threadIdx.x < 2) {
        const int first = threadIdx.x == 0 ? 0 : H, count = threadIdx.x == 0 ? H : heads - H;
        float total = 0.0f;
        for (int j = 0; j < count; ++j) total += head_ss[first + j];
        s_factor[threadIdx.x] = count > 0 ? 1.0f / sqrtf(total / (float)(count * d) + eps) : 0.0f;
    }
    __syncthreads();
    const int slot = write_kv ? slot_mapping[t] : -1;
    T* k_dst = slot >= 0 ? k_cache + (((size_t)(slot / page_size)) * K * page_size + (size_t)(slot % page_size)) * d : nullptr;
    // a warp per head, lanes along the head: no division per element, 64-byte runs per store
    for (int head = warp; head < heads; head += warps) {
        const bool is_q = head < H;
        const int kh = head - H;
        if (!is_q && k_dst == nullptr) continue;
        float factor = 1.0f;
        const float* w = nullptr;
        if (norm_mode == 1) {
            factor = 1.0f / sqrtf(head_ss[head] / (float)d + eps);
            w = is_q ? q_w : k_w;
        } else if (norm_mode == 2) {
            factor = s_factor[is_q ? 0 : 1];
            w = is_q ? q_w + (size_t)head * d : k_w + (size_t)kh * d;
        }
        const float* hv = vals + (size_t)head * d;
        T* dst = is_q ? q_out + (size_t)t * q_len + (size_t)head * d : k_dst + (size_t)kh * page_size * d;
        for (int i = lane; i < d; i += 32) {
            float a = hv[i] * factor * (w != nullptr ? w[i] : 1.0f);
            if (i < rot_dim) {                                 // (rot_dim is 0 without a rotation)
                const bool low = interleaved ? (i & 1) == 0 : i < half;
                const int j = interleaved ? i >> 1 : low ? i : i - half;
                const int other = interleaved ? i ^ 1 : low ? i + half : i - half;
                const float b = hv[other] * factor * (w != nullptr ? w[other] : 1.0f);
                const float cs = cs_tab[j], sn = cs_tab[half + j];
                a = low ? a * cs - b * sn : a * cs + b * sn;
            }
            dst[i] = from_f32<T>(a);
        }
    }
    if (!write_kv) return;
    const float lam = v_mode == 2 ? *v_lambda : 0.0f;
    const int vcol0 = (H + K) * d;
    for (int kh = warp; kh < K; kh += warps) {
        T* dst = slot >= 0 ? v_cache + ((((size_t)(slot / page_size)) * K + kh) * page_size + (size_t)(slot % page_size)) * dv : nullptr;
        for (int e = lane; e < dv; e += 32) {
            const int i = kh * dv + e;
            float v = to_f32(src[vcol0 + i]);
            if (v_b != nullptr) v += v_b[i];
            if (v_mode == 1) v_shared[(size_t)t * K * dv + i] = from_f32<T>(v);
            else if (v_mode == 2) v = (1.0f - lam) * v + lam * to_f32(v_shared[(size_t)t * K * dv + i]);
            if (dst != nullptr) dst[e] = from_f32<T>(v);
        }
    }
}

// The same for bf16 rows whose sizes are multiples of 8 (heads, value heads, half the rotated width, the row's stride):
// a thread owns runs of 8 elements (one 16-byte load, one 16-byte store), keeps them in registers between the two phases
// and fetches only its rotation partners from shared memory.  Sums of squares: a thread's 8 elements in order, then the
// block's (norm over the whole projection) or a warp per head over shared memory (per-head norm): fixed orders.
// RUNS runs per thread: one or two with few tokens (every load of a token in flight at once), four with many (smaller
// blocks, several of them on an SM at different stages: a block's life is a chain of waits on memory and barriers).
__device__ __forceinline__ void unpack8(const uint4& raw, float* x) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 pack8(const float* x) {
    uint4 out;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    return out;
}
__device__ __forceinline__ void load8(const float* p, float* x) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

template <int RUNS>
__global__ void __launch_bounds__(RUNS <= 2 ? 1024 : 256) qkv_finish_vec_kernel(
    const bf16* __restrict__ row, int row_stride, bf16* __restrict__ q_out, const float* __restrict__ q_b, const float* __restrict__ k_b,
    const float* __restrict__ v_b, int norm_mode, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim, float rot_mag,
    const int* __restrict__ slot_mapping, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int v_mode, bf16* __restrict__ v_shared,
    const float* __restrict__ v_lambda, int H, int K, int d, int dv, int page_size, int write_kv, int interleaved) {
    PDL_ENTER();
    row = pdl_fresh(row); v_shared = pdl_fresh(v_shared);
    extern __shared__ __align__(16) float smem[];
    __shared__ float scratch[32];
    const int heads = write_kv ? H + K : H;
    const int half = rot_dim >> 1;
    float* vals = smem;                        // [heads * d]
    float* cs_tab = vals + (size_t)heads * d;  // [half] cosines, [half] sines
    float* head_ss = cs_tab + 2 * half;        // [heads]
    const int t = blockIdx.x, threads = blockDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = threads >> 5;
    const bf16* src = row + (size_t)t * row_stride;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += threads) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = cs * rot_mag;
            cs_tab[half + i] = sn * rot_mag;
        }
    }
    const int runs = heads * d / 8, q_runs = H * d / 8;
    float x[RUNS][8];
    float ss_q = 0.0f, ss_k = 0.0f;
#pragma unroll
    for (int u = 0; u < RUNS; ++u) {
        const int v = threadIdx.x + u * threads;
        if (v < runs) {
            unpack8(*reinterpret_cast<const uint4*>(src + v * 8), x[u]);
            const float* bias = v < q_runs ? q_b : k_b;
            if (bias != nullptr) {
                float b[8];
                load8(bias + (v < q_runs ? v : v - q_runs) * 8, b);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[u][e] += b[e];
            }
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[u][e] * x[u][e];
            if (v < q_runs) ss_q += ss; else ss_k += ss;
            *reinterpret_cast<float4*>(vals + v * 8) = make_float4(x[u][0], x[u][1], x[u][2], x[u][3]);
            *reinterpret_cast<float4*>(vals + v * 8 + 4) = make_float4(x[u][4], x[u][5], x[u][6], x[u][7]);
        }
    }
    float f_q = 1.0f, f_k = 1.0f;
    if (norm_mode == 2) {
        ss_q = block_sum(ss_q, scratch);
        ss_k = block_sum(ss_k, scratch);
        f_q = 1.0f / sqrtf(ss_q / (float)(H * d) + eps);
        f_k = heads > H ? 1.0f / sqrtf(ss_k / (float)((heads - H) * d) + eps) : 0.0f;
        __syncthreads();
    } else {
        __syncthreads();
        if (norm_mode == 1) {
            for (int head = warp; head < heads; head += warps) {
                float ss = 0.0f;
                for (int i = lane; i < d; i += 32) { const float v = vals[head * d + i]; ss += v * v; }
                ss = warp_sum(ss);
                if (lane == 0) head_ss[head] = ss;
            }
            __syncthreads();
        }
    }
    const int slot = write_kv ? slot_mapping[t] : -1;
    bf16* k_dst = slot >= 0 ? k_cache + (((size_t)(slot / page_size)) * K * page_size + (size_t)(slot % page_size)) * d : nullptr;
#pragma unroll
    for (int u = 0; u < RUNS; ++u) {
        const int v = threadIdx.x + u * threads;
        if (v >= runs) continue;
        const int head = (v * 8) / d, i0 = v * 8 - head * d;
        const bool is_q = head < H;
        const int kh = head - H;
        if (!is_q && k_dst == nullptr) continue;
        float factor = 1.0f;
        const float* w = nullptr;
        if (norm_mode == 1) {
            factor = 1.0f / sqrtf(head_ss[head] / (float)d + eps);
            w = is_q ? q_w : k_w;
        } else if (norm_mode == 2) {
            factor = is_q ? f_q : f_k;
            w = is_q ? q_w + (size_t)head * d : k_w + (size_t)kh * d;
        }
        float a[8];
        if (w != nullptr) {
            float ww[8];
            load8(w + i0, ww);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = x[u][e] * factor * ww[e];
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = x[u][e] * factor;
        }
        if (i0 < rot_dim && interleaved) {                     // partners are neighbours inside the run
            const float4 c4 = *reinterpret_cast<const float4*>(cs_tab + (i0 >> 1)), s4 = *reinterpret_cast<const float4*>(cs_tab + half + (i0 >> 1));
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float u = a[2 * e], v = a[2 * e + 1];
                a[2 * e] = u * cs[e] - v * sn[e];
                a[2 * e + 1] = v * cs[e] + u * sn[e];
            }
        } else if (i0 < rot_dim) {
            const bool low = i0 < half;
            const int j0 = low ? i0 : i0 - half, other = low ? i0 + half : i0 - half;
            float b[8], cs[8], sn[8];
            load8(vals + head * d + other, b);
            if (w != nullptr) {
                float ww[8];
                load8(w + other, ww);
#pragma unroll
                for (int e = 0; e < 8; ++e) b[e] *= factor * ww[e];
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) b[e] *= factor;
            }
            load8(cs_tab + j0, cs);
            load8(cs_tab + half + j0, sn);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = low ? a[e] * cs[e] - b[e] * sn[e] : a[e] * cs[e] + b[e] * sn[e];
        }
        bf16* dst = is_q ? q_out + (size_t)t * H * d + (size_t)v * 8 : k_dst + (size_t)kh * page_size * d + i0;
        *reinterpret_cast<uint4*>(dst) = pack8(a);
    }
    if (!write_kv) return;
    const float lam = v_mode == 2 ? *v_lambda : 0.0f;
    const int vcol0 = (H + K) * d;
    for (int v = threadIdx.x; v < K * dv / 8; v += threads) {
        float val[8];
        unpack8(*reinterpret_cast<const uint4*>(src + vcol0 + v * 8), val);
        if (v_b != nullptr) {
            float b[8];
            load8(v_b + v * 8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) val[e] += b[e];
        }
        bf16* shared_at = v_shared + (size_t)t * K * dv + v * 8;
        if (v_mode == 1) {
            *reinterpret_cast<uint4*>(shared_at) = pack8(val);
        } else if (v_mode == 2) {
            float first[8];
            unpack8(*reinterpret_cast<const uint4*>(shared_at), first);
#pragma unroll
            for (int e = 0; e < 8; ++e) val[e] = (1.0f - lam) * val[e] + lam * first[e];
        }
        if (slot >= 0) {
            const int kh = (v * 8) / dv, e0 = v * 8 - kh * dv;
            *reinterpret_cast<uint4*>(v_cache + ((((size_t)(slot / page_size)) * K + kh) * page_size + (size_t)(slot % page_size)) * dv + e0) = pack8(val);
        }
    }
}

static bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

MB_API int mb_qkv_finish(const void* row, int row_stride, int dtype, void* q_out, const float* q_b, const float* k_b, const float* v_b,
                         int norm_mode, const float* q_w, const float* k_w, float eps, const int* positions, const float* inv_freq,
                         int rot_dim, float rot_mag, const int* slot_mapping, void* k_cache, void* v_cache, int v_mode, void* v_shared,
                         const float* v_lambda, int tokens, int H, int K, int d, int dv, int page_size, int write_kv, int interleaved,
                         cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || H <= 0 || K <= 0 || rot_dim > d || (rot_dim & 1) || norm_mode < 0 || norm_mode > 2) return MB_ERR_BAD_SIZE;
    if ((v_mode == 1 || v_mode == 2) && v_shared == nullptr) return MB_ERR_BAD_SIZE;
    if (v_mode == 2 && v_lambda == nullptr) return MB_ERR_BAD_SIZE;
    if (inv_freq == nullptr) rot_dim = 0;
    const size_t smem = ((size_t)(H + K) * d + rot_dim + H + K) * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_BAD_SIZE;
    const int runs8 = (H + K) * d / 8;
    if (dtype == MB_BF16 && d % 8 == 0 && dv % 8 == 0 && (interleaved ? rot_dim % 8 == 0 : (rot_dim / 2) % 8 == 0) && row_stride % 8 == 0 && runs8 <= 1024 * 2 &&
        aligned16(row) && aligned16(q_out) && aligned16(q_b) && aligned16(k_b) && aligned16(v_b) && aligned16(q_w) && aligned16(k_w) &&
        aligned16(k_cache) && aligned16(v_cache) && aligned16(v_shared)) {
#define QV_LAUNCH(RUNS, threads)                                                                                                        \
    do {                                                                                                                                \
        if (smem > 48 * 1024) {                                                                                                         \
            const int rc = (int)cudaFuncSetAttribute(qkv_finish_vec_kernel<RUNS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc != 0) return rc;                                                                                                     \
        }                                                                                                                               \
        return launch_kernel(qkv_finish_vec_kernel<RUNS>, tokens, threads, smem, s, 0, (const bf16*)row, row_stride, (bf16*)q_out, q_b, k_b, \
                             v_b, norm_mode, q_w, k_w, eps, positions, inv_freq, rot_dim, rot_mag, slot_mapping, (bf16*)k_cache,         \
                             (bf16*)v_cache, v_mode, (bf16*)v_shared, v_lambda, H, K, d, dv, page_size, write_kv, interleaved);          \
    } while (0)
        const int quarter = (((runs8 + 3) / 4 + 31) / 32) * 32;
        if (tokens >= 512 && quarter <= 256) QV_LAUNCH(4, quarter < 64 ? 64 : quarter);
        const int whole = ((runs8 + 31) / 32) * 32;
        if (whole <= 1024) QV_LAUNCH(1, whole < 128 ? 128 : whole);
        QV_LAUNCH(2, (((runs8 + 1) / 2 + 31) / 32) * 32);
#undef QV_LAUNCH
    }
#define QF_LAUNCH(TT)                                                                                                                \
    do {                                                                                                                             \
        if (smem > 48 * 1024) {                                                                                                      \
            const int rc = (int)cudaFuncSetAttribute(qkv_finish_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc != 0) return rc;                                                                                                  \
        }                                                                                                                            \
        return launch_kernel(qkv_finish_kernel<TT>, tokens, (H + K) * d < 4096 ? QF_THREADS : tokens <= 64 ? 1024 : 512, smem, s, 0, (const TT*)row, row_stride, (TT*)q_out, q_b, k_b, \
                             v_b, norm_mode, q_w, k_w, eps, positions, inv_freq, rot_dim, rot_mag, slot_mapping, (TT*)k_cache,      \
                             (TT*)v_cache, v_mode, (TT*)v_shared, v_lambda, H, K, d, dv, page_size, write_kv, interleaved);          \
    } while (0)
    if (dtype == MB_F32) QF_LAUNCH(float);
    if (dtype == MB_BF16) QF_LAUNCH(bf16);
#undef QF_LAUNCH
    return MB_ERR_BAD_DTYPE;
}

// ---- the plain kernel: one block per (token, query head), keys in blocks of 128 in increasing order ----------------------
#define SK_THREADS 128
#define SK_MAX_PER_THREAD 4

template <typename T>
__global__ void __launch_bounds__(SK_THREADS) attention_sink_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_index, const int* __restrict__ positions,
    int H, int K, int d, int dv, int page_size, float scale, int window, int chunk, int sink, const float* __restrict__ sink_logit,
    int v_stride, const T* __restrict__ gate, int gate_stride) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache); gate = pdl_fresh(gate);
    extern __shared__ float smem[];
    float* qs = smem;                 // [d]
    float* ps = smem + d;             // [SK_THREADS]
    float* scratch = ps + SK_THREADS; // [32]
    const int t = blockIdx.x, head = blockIdx.y;
    const int kh = head / (H / K);
    const int req = req_index[t];
    const int pos = positions[t];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int* table = block_table + (size_t)req * max_pages;
    const T* qrow = q + ((size_t)t * H + head) * d;
    for (int i = threadIdx.x; i < d; i += SK_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    // the sink is a key whose value is zero: the running maximum starts at its score (0 or the head's learned number) and
    // the sum at 1
    float m = sink ? (sink_logit != nullptr ? sink_logit[head] : 0.0f) : -INFINITY, l = sink ? 1.0f : 0.0f;
    float acc[SK_MAX_PER_THREAD];
#pragma unroll
    for (int r = 0; r < SK_MAX_PER_THREAD; ++r) acc[r] = 0.0f;

    for (int base = lo; base <= pos; base += SK_THREADS) {
        const int key = base + threadIdx.x;
        float s = -INFINITY;
        if (key <= pos) {
            const size_t page = (size_t)table[key / page_size];
            const T* krow = k_cache + ((page * K + kh) * page_size + (size_t)(key % page_size)) * d;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
        }
        const float block_top = block_max(s, scratch);
        const float m_new = fmaxf(m, block_top);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first block without a sink
        const float p = key <= pos ? expf(s - m_new) : 0.0f;
        __syncthreads();
        ps[threadIdx.x] = p;
        const float block_total = block_sum(p, scratch);  // has the barriers that publish ps
        l = l * corr + block_total;
        m = m_new;
        const int count = min(SK_THREADS, pos - base + 1);
#pragma unroll
        for (int r = 0; r < SK_MAX_PER_THREAD; ++r) {
            const int dd = threadIdx.x + r * SK_THREADS;
            if (dd < dv) {
                float a = acc[r] * corr;
                for (int j = 0; j < count; ++j) {
                    const int kj = base + j;
                    const size_t page = (size_t)table[kj / page_size];
                    const T* vrow = v_cache + ((page * K + kh) * page_size + (size_t)(kj % page_size)) * v_stride;
                    a = fmaf(ps[j], to_f32(vrow[dd]), a);
                }
                acc[r] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * H + head) * dv;
    const T* grow = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)head * dv : nullptr;
#pragma unroll
    for (int r = 0; r < SK_MAX_PER_THREAD; ++r) {
        const int dd = threadIdx.x + r * SK_THREADS;
        if (dd < dv) {
            float o = acc[r] / l;
            if (grow != nullptr) o *= 1.0f / (1.0f + expf(-to_f32(grow[dd])));
            orow[dd] = from_f32<T>(o);
        }
    }
}

// gate: null, or the first gate column of token 0 (rows `gate_stride` elements apart, H heads of dv side by side).
// sink_logit: null (a sink of score 0, if `sink`) or a float32 score per query head.  v_stride: elements between the values of
// two positions of a page (dv for value pages of their own; the key rows' width where values are the start of the key rows).
MB_API int mb_attention_sink(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype, const int* block_table,
                             int max_pages, const int* req_index, const int* positions, int tokens, int H, int K, int d, int dv,
                             int page_size, float scale, int window, int chunk, int sink, const float* sink_logit, int v_stride,
                             const void* gate, int gate_stride, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (v_stride < dv) return MB_ERR_BAD_SIZE;
    if (d <= 0 || dv <= 0 || dv > SK_THREADS * SK_MAX_PER_THREAD || K <= 0 || H % K != 0 || window < 0 || chunk < 0) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, H);
    const size_t smem = (size_t)(d + SK_THREADS + 32) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(attention_sink_kernel<float>, grid, SK_THREADS, smem, s, 0, (const float*)q, (const float*)k_cache,
                             (const float*)v_cache, (float*)out, block_table, max_pages, req_index, positions, H, K, d, dv, page_size,
                             scale, window, chunk, sink, sink_logit, v_stride, (const float*)gate, gate_stride);
    if (dtype == MB_BF16)
        return launch_kernel(attention_sink_kernel<bf16>, grid, SK_THREADS, smem, s, 0, (const bf16*)q, (const bf16*)k_cache,
                             (const bf16*)v_cache, (bf16*)out, block_table, max_pages, req_index, positions, H, K, d, dv, page_size,
                             scale, window, chunk, sink, sink_logit, v_stride, (const bf16*)gate, gate_stride);
    return MB_ERR_BAD_DTYPE;
}
