// Attention over a latent that keys and values share (one row of `r` numbers per position, plus `dr` rotated numbers that
// serve as a key part for every head).  Per head a the key is [W_uk_a c | k_rot] and the value W_uv_a c, so with
//     q'_a = [W_uk_a^T q_a(unrotated) | q_a(rotated)],   score = q'_a . [c | k_rot],   out_a = W_uv_a (sum_j p_j c_j)
// every head reads the same cached row: grouped-query attention with one kv head whose key is the cached row and whose
// value is the row's first r elements.  This file holds what surrounds that attention:
//   * the head preparation: rotation of the queries' rotated part into q', and (for a layer that owns its cache) the RMS
//     norm of the latent and the rotation of the shared key part, written into the page;
//   * a product per head over strided rows, out[t][a][:] = W_a x[t][a][:], used for q' (W_a = W_uk_a^T) and for the value
//     expansion (W_a = W_uv_a): the plain kernel for any size and float32, and for bf16 a tensor-core kernel (mma.sync) over
//     tiles of 64 tokens x 64 columns.
// Rotation: of the rotated part's first `rot_dims` elements, (2i, 2i + 1) or (i, i + rot_dims/2) turn by pos * inv_freq[i].
// Norms, angles and sums are float32.
#define MB_LIB "attention_latent"
#define MB_LIB_ID 16
#include "common.cuh"
#include "launch.cuh"
#include "mma_helpers.cuh"

#define LF_THREADS 128

// row: [tokens][row_stride]: H heads of (dn + dr) query numbers, then (if write_kv) r latent numbers and dr key numbers.
// q_out: [tokens][H][r + dr]; only [r, r + dr) of every head is written here.  Page rows: [r + dr] = normed latent | rotated key part.
template <typename T>
__global__ void __launch_bounds__(LF_THREADS) latent_finish_kernel(
    const T* __restrict__ row, int row_stride, T* __restrict__ q_out, const float* __restrict__ c_weight, float eps,
    const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dims, int interleaved,
    const int* __restrict__ slot_mapping, T* __restrict__ k_cache, int H, int dn, int dr, int r, int page_size, int write_kv,
    const T* __restrict__ kv_row, int kv_stride) {
    PDL_ENTER();
    row = pdl_fresh(row); kv_row = pdl_fresh(kv_row);
    extern __shared__ float smem[];
    float* cs_tab = smem;                      // [half] cosines, [half] sines
    const int half = rot_dims >> 1;
    float* lat = smem + 2 * half;              // [r + dr]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* src = row + (size_t)t * row_stride;
    if (half > 0) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += LF_THREADS) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = cs;
            cs_tab[half + i] = sn;
        }
    }
    __syncthreads();
    const int D = r + dr;
    // the queries' rotated part
    for (int idx = threadIdx.x; idx < H * dr; idx += LF_THREADS) {
        const int a = idx / dr, i = idx - a * dr;
        const T* part = src + (size_t)a * (dn + dr) + dn;
        float v = to_f32(part[i]);
        if (i < rot_dims) {
            const bool low = interleaved ? (i & 1) == 0 : i < half;
            const int j = interleaved ? i >> 1 : low ? i : i - half;
            const int other = interleaved ? i ^ 1 : low ? i + half : i - half;
            const float b = to_f32(part[other]);
            v = low ? v * cs_tab[j] - b * cs_tab[half + j] : v * cs_tab[j] + b * cs_tab[half + j];
        }
        q_out[((size_t)t * H + a) * D + r + i] = from_f32<T>(v);
    }
    if (!write_kv) return;
    const int slot = slot_mapping[t];
    // the latent and the key part: behind the queries in the same row, or (queries that went through a latent of their own
    // come from a second product) in rows of their own
    const T* kv = kv_row != nullptr ? kv_row + (size_t)t * kv_stride : src + (size_t)H * (dn + dr);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += LF_THREADS) {
        const float v = to_f32(kv[i]);
        lat[i] = v;
        if (i < r) ss += v * v;
    }
    ss = block_sum(ss, scratch);               // (its barriers publish lat)
    if (slot < 0) return;
    const float factor = 1.0f / sqrtf(ss / (float)r + eps);
    T* dst = k_cache + (size_t)slot * D;       // one kv head: page * page_size + offset is the row
    for (int i = threadIdx.x; i < D; i += LF_THREADS) {
        float v;
        if (i < r) {
            v = lat[i] * factor * c_weight[i];
        } else {
            const int e = i - r;
            v = lat[i];
            if (e < rot_dims) {
                const bool low = interleaved ? (e & 1) == 0 : e < half;
                const int j = interleaved ? e >> 1 : low ? e : e - half;
                const int other = interleaved ? e ^ 1 : low ? e + half : e - half;
                const float b = lat[r + other];
                v = low ? v * cs_tab[j] - b * cs_tab[half + j] : v * cs_tab[j] + b * cs_tab[half + j];
            }
        }
        dst[i] = from_f32<T>(v);
    }
}

MB_API int mb_latent_finish(const void* row, int row_stride, int dtype, void* q_out, const float* c_weight, float eps, const int* positions,
                            const float* inv_freq, int rot_dims, int interleaved, const int* slot_mapping, void* k_cache, int tokens, int H,
                            int dn, int dr, int r, int page_size, int write_kv, const void* kv_row, int kv_stride, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (H <= 0 || dn < 0 || dr < 0 || r <= 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1)) return MB_ERR_BAD_SIZE;
    if (inv_freq == nullptr) rot_dims = 0;
    const size_t smem = (size_t)(rot_dims + r + dr) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(latent_finish_kernel<float>, tokens, LF_THREADS, smem, s, 0, (const float*)row, row_stride, (float*)q_out, c_weight,
                             eps, positions, inv_freq, rot_dims, interleaved, slot_mapping, (float*)k_cache, H, dn, dr, r, page_size, write_kv,
                             (const float*)kv_row, kv_stride);
    if (dtype == MB_BF16)
        return launch_kernel(latent_finish_kernel<bf16>, tokens, LF_THREADS, smem, s, 0, (const bf16*)row, row_stride, (bf16*)q_out, c_weight,
                             eps, positions, inv_freq, rot_dims, interleaved, slot_mapping, (bf16*)k_cache, H, dn, dr, r, page_size, write_kv,
                             (const bf16*)kv_row, kv_stride);
    return MB_ERR_BAD_DTYPE;
}

// ---- a product per head: out[t][a][n] = sum_k w[a][n][k] x[t][a][k] -------------------------------------------------------
// x: element (t, a, k) at x + t x_ld + a x_head + k;  w: [H][N][K];  out: element (t, a, n) at out + t o_ld + a o_head + n.
// Plain kernel: a block per (token, head, run of HP_COLS output columns); a warp per column, lanes along k in a fixed order,
// so a token's result does not depend on the batch.  (Few tokens bring few blocks otherwise: a single-token step of eight
// requests took 28 us for a product of half a megabyte of weights with one block per token and head.)
#define HP_THREADS 128
#define HP_COLS 16
template <typename T>
__global__ void __launch_bounds__(HP_THREADS) heads_product_kernel(const T* __restrict__ x, int x_ld, int x_head, const T* __restrict__ w,
                                                                   T* __restrict__ out, int o_ld, int o_head, int N, int K) {
    PDL_ENTER();
    x = pdl_fresh(x);
    extern __shared__ float xs[];              // [K]
    const int t = blockIdx.x, a = blockIdx.y;
    const T* xr = x + (size_t)t * x_ld + (size_t)a * x_head;
    for (int k = threadIdx.x; k < K; k += HP_THREADS) xs[k] = to_f32(xr[k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* wa = w + (size_t)a * N * K;
    T* dst = out + (size_t)t * o_ld + (size_t)a * o_head;
    const int n_end = min(N, (int)(blockIdx.z + 1) * HP_COLS);
    for (int n = blockIdx.z * HP_COLS + warp; n < n_end; n += HP_THREADS / 32) {
        const T* wr = wa + (size_t)n * K;
        float dot = 0.0f;
        for (int k = lane; k < K; k += 32) dot = fmaf(xs[k], to_f32(wr[k]), dot);
        dot = warp_sum(dot);
        if (lane == 0) dst[n] = from_f32<T>(dot);
    }
}

// bf16 on the tensor cores: a CTA takes 64 tokens x 64 columns of one head; K in steps of 32 (zero-filled past K) through a
// double buffer; rows of x and w must start on 16-byte boundaries (K, x_ld, x_head multiples of 8).
#define HT_M 64
#define HT_N 64
#define HT_K 32
#define HT_LD (HT_K + 8)
__global__ void __launch_bounds__(128) heads_product_tc_kernel(const bf16* __restrict__ x, int x_ld, int x_head, const bf16* __restrict__ w,
                                                               bf16* __restrict__ out, int o_ld, int o_head, int T, int N, int K) {
    PDL_ENTER();
    x = pdl_fresh(x);
    __shared__ __align__(16) bf16 sA[2][HT_M * HT_LD];
    __shared__ __align__(16) bf16 sB[2][HT_N * HT_LD];
    const int t0 = blockIdx.x * HT_M, n0 = blockIdx.y * HT_N, a = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* xa = x + (size_t)a * x_head;
    const bf16* wa = w + (size_t)a * N * K;
    auto load = [&](int buf, int k0) {
        for (int idx = threadIdx.x; idx < (HT_M + HT_N) * (HT_K / 8); idx += 128) {
            const int rr = idx / (HT_K / 8), c = idx % (HT_K / 8);
            const int k = k0 + c * 8;
            if (rr < HT_M) {
                bf16* d = sA[buf] + rr * HT_LD + c * 8;
                if (t0 + rr < T && k < K) cp_async16(d, xa + (size_t)(t0 + rr) * x_ld + k);
                else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
            } else {
                const int n = rr - HT_M;
                bf16* d = sB[buf] + n * HT_LD + c * 8;
                if (n0 + n < N && k < K) cp_async16(d, wa + (size_t)(n0 + n) * K + k);
                else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    float acc[HT_N / 8][4];
#pragma unroll
    for (int j = 0; j < HT_N / 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }
    const int nk = (K + HT_K - 1) / HT_K;
    load(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) load(buf ^ 1, (kt + 1) * HT_K);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sA[buf] + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HT_LD + (lane >> 4) * 8);
        const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(sB[buf] + ((lane & 7) + (lane >> 4) * 8) * HT_LD + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < HT_K / 16; ++kk) {
            uint32_t fa[4];
            ldsm_x4(a_addr + kk * 32, fa[0], fa[1], fa[2], fa[3]);
#pragma unroll
            for (int j = 0; j < HT_N / 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b_addr + (uint32_t)(j * 8 * HT_LD * 2 + kk * 32), b0, b1, b2, b3);
                mma_bf16_16816(acc[j], fa, b0, b1);
                mma_bf16_16816(acc[j + 1], fa, b2, b3);
            }
        }
        __syncthreads();                       // everyone is done with this buffer before the load after next fills it
    }
    cp_async_wait<0>();
    const int col = n0 + 2 * (lane & 3);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int t = t0 + warp * 16 + (lane >> 2) + 8 * rr;
        if (t >= T) continue;
        bf16* dst = out + (size_t)t * o_ld + (size_t)a * o_head;
#pragma unroll
        for (int j = 0; j < HT_N / 8; ++j) {
            const int c = col + j * 8;
            if (c + 1 < N) *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(acc[j][2 * rr], acc[j][2 * rr + 1]);
            else if (c < N) dst[c] = __float2bfloat16_rn(acc[j][2 * rr]);
        }
    }
}

static bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// fast: 1 asks for the tensor-core kernel where the layout allows (bf16, rows on 16-byte boundaries, even output offsets).
MB_API int mb_heads_product(const void* x, int x_ld, int x_head, const void* w, void* out, int o_ld, int o_head, int dtype, int tokens, int H,
                            int N, int K, int fast, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (H <= 0 || N <= 0 || K <= 0 || (size_t)K * 4 > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_BF16 && fast && K % 8 == 0 && x_ld % 8 == 0 && x_head % 8 == 0 && o_ld % 2 == 0 && o_head % 2 == 0 && aligned16(x) &&
        aligned16(w) && (((uintptr_t)out) & 3) == 0 && tokens >= 16)
        return launch_kernel(heads_product_tc_kernel, dim3((tokens + HT_M - 1) / HT_M, (N + HT_N - 1) / HT_N, H), 128, 0, s, 0, (const bf16*)x,
                             x_ld, x_head, (const bf16*)w, (bf16*)out, o_ld, o_head, tokens, N, K);
    dim3 grid(tokens, H, (N + HP_COLS - 1) / HP_COLS);
    if (dtype == MB_F32)
        return launch_kernel(heads_product_kernel<float>, grid, HP_THREADS, (size_t)K * 4, s, 0, (const float*)x, x_ld, x_head, (const float*)w,
                             (float*)out, o_ld, o_head, N, K);
    if (dtype == MB_BF16)
        return launch_kernel(heads_product_kernel<bf16>, grid, HP_THREADS, (size_t)K * 4, s, 0, (const bf16*)x, x_ld, x_head, (const bf16*)w,
                             (bf16*)out, o_ld, o_head, N, K);
    return MB_ERR_BAD_DTYPE;
}
