// Norms and activations that are not RMSNorm or SwiGLU: Dynamic Tanh, PolyNorm, a gated RMS norm over the whole row,
// the mixing of a row with the row before it (token shift), and a tanh cap on the logits.  Sums, norms and the
// transcendental functions are float32 whatever the activation dtype; every kernel takes its sizes as arguments.
#define MB_LIB "activations"
#define MB_LIB_ID 8
#include "common.cuh"
#include "launch.cuh"

// ---- Dynamic Tanh: out[t, i] = tanh(alpha * x[t, i]) * w[i] + b[i]; no statistic of the row enters ---------------------
template <typename TO>
__global__ void dyt_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                           const float* __restrict__ alpha, TO* __restrict__ out, size_t total, int n) {
    PDL_ENTER();
    x = pdl_fresh(x);
    const float a = alpha[0];
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const int i = (int)(idx % (size_t)n);
        out[idx] = from_f32<TO>(fmaf(tanhf(a * x[idx]), w[i], b != nullptr ? b[i] : 0.0f));
    }
}

static inline int blocks_for(size_t total, int threads) {
    const size_t want = (total + threads - 1) / threads;
    return (int)(want < (size_t)148 * 16 ? want : (size_t)148 * 16);
}

MB_API int mb_dyt(const float* x, const float* w, const float* b, const float* alpha, void* out, int out_dtype, int rows, int n,
                  cudaStream_t s) {
    const size_t total = (size_t)rows * n;
    if (total == 0) return 0;
    if (out_dtype == MB_F32) return launch_kernel(dyt_kernel<float>, blocks_for(total, 256), 256, 0, s, 0, x, w, b, alpha, (float*)out, total, n);
    if (out_dtype == MB_BF16) return launch_kernel(dyt_kernel<bf16>, blocks_for(total, 256), 256, 0, s, 0, x, w, b, alpha, (bf16*)out, total, n);
    return MB_ERR_BAD_DTYPE;
}

// ---- PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e, N(y) = y / sqrt(mean(y^2) + eps) over the row ---------------------
// One block of 1,024 threads per row; the three sums of squares (z^2, z^4, z^6) in one pass, the row read a second time
// (from L2) for the result.  VEC elements per load where the row allows (16 bytes).
template <typename TI, int VEC> struct RowLoad;
template <> struct RowLoad<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* v) { const float4 x = *reinterpret_cast<const float4*>(p); v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; }
};
template <> struct RowLoad<float, 1> { static __device__ __forceinline__ void load(const float* p, float* v) { v[0] = p[0]; } };
template <> struct RowLoad<bf16, 1> { static __device__ __forceinline__ void load(const bf16* p, float* v) { v[0] = __bfloat162float(p[0]); } };
template <> struct RowLoad<bf16, 4> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
};
template <typename TO, int VEC> __device__ __forceinline__ void row_store(TO* p, const float* v) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = from_f32<TO>(v[i]);
}
template <> __device__ __forceinline__ void row_store<float, 4>(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
template <> __device__ __forceinline__ void row_store<bf16, 4>(bf16* p, const float* v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = packed;
}

template <typename TI, typename TO, int VEC>
__global__ void __launch_bounds__(1024) polynorm_kernel(const TI* __restrict__ z, const float* __restrict__ coef, float eps,
                                                        TO* __restrict__ out, int n) {
    PDL_ENTER();
    z = pdl_fresh(z);
    __shared__ float scratch[32];
    const TI* row = z + (size_t)blockIdx.x * n;
    TO* dst = out + (size_t)blockIdx.x * n;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (int i = threadIdx.x * VEC; i < n; i += blockDim.x * VEC) {
        float v[VEC];
        RowLoad<TI, VEC>::load(row + i, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) { const float v2 = v[e] * v[e]; s1 += v2; s2 += v2 * v2; s3 += v2 * v2 * v2; }
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float r1 = coef[0] / sqrtf(s1 / (float)n + eps), r2 = coef[1] / sqrtf(s2 / (float)n + eps),
                r3 = coef[2] / sqrtf(s3 / (float)n + eps), e0 = coef[3];
    for (int i = threadIdx.x * VEC; i < n; i += blockDim.x * VEC) {
        float v[VEC];
        RowLoad<TI, VEC>::load(row + i, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) { const float v2 = v[e] * v[e]; v[e] = r1 * v[e] + r2 * v2 + r3 * (v2 * v[e]) + e0; }
        row_store<TO, VEC>(dst + i, v);
    }
}

template <typename TI, typename TO>
static int polynorm_launch(const void* z, const float* coef, float eps, void* out, int rows, int n, cudaStream_t s) {
    const bool vec = n % 4 == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0;
    const int threads = n >= 4096 ? 1024 : n >= 1024 ? 256 : 128;
    if (vec) return launch_kernel(polynorm_kernel<TI, TO, 4>, rows, threads, 0, s, 0, (const TI*)z, coef, eps, (TO*)out, n);
    return launch_kernel(polynorm_kernel<TI, TO, 1>, rows, threads, 0, s, 0, (const TI*)z, coef, eps, (TO*)out, n);
}

MB_API int mb_polynorm(const void* z, int z_dtype, const float* coef, float eps, void* out, int out_dtype, int rows, int n,
                       cudaStream_t s) {
    if (rows <= 0 || n <= 0) return 0;
    if (z_dtype == MB_F32 && out_dtype == MB_F32) return polynorm_launch<float, float>(z, coef, eps, out, rows, n, s);
    if (z_dtype == MB_F32 && out_dtype == MB_BF16) return polynorm_launch<float, bf16>(z, coef, eps, out, rows, n, s);
    if (z_dtype == MB_BF16 && out_dtype == MB_BF16) return polynorm_launch<bf16, bf16>(z, coef, eps, out, rows, n, s);
    return MB_ERR_BAD_DTYPE;
}

// ---- gated RMS norm over the whole row: out = o / sqrt(mean(o^2) + eps) * w * gate(g) ---------------------------------
// o is float32 (what a recurrence leaves); g is read with a stride (it may be a slice of a wider row); gate: 0 sigmoid,
// 1 silu, 2 none (g may then be null).
template <typename T>
__global__ void __launch_bounds__(1024) gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w,
                                                            const T* __restrict__ g, int g_stride, int gate, float eps,
                                                            T* __restrict__ out, int n) {
    PDL_ENTER();
    o = pdl_fresh(o);
    g = pdl_fresh(g);
    __shared__ float scratch[32];
    const float* row = o + (size_t)blockIdx.x * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = row[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = row[i] * scale * w[i];
        if (gate != 2) {
            const float z = to_f32(g[(size_t)blockIdx.x * g_stride + i]);
            const float sg = 1.0f / (1.0f + expf(-z));
            y *= gate == 0 ? sg : z * sg;
        }
        out[(size_t)blockIdx.x * n + i] = from_f32<T>(y);
    }
}

MB_API int mb_gated_rmsnorm(const float* o, const float* w, const void* g, int g_stride, int gate, float eps, void* out, int dtype,
                            int rows, int n, cudaStream_t s) {
    if (rows <= 0 || n <= 0) return 0;
    if (gate < 0 || gate > 2 || (gate != 2 && g == nullptr)) return MB_ERR_BAD_SIZE;
    const int threads = n >= 2048 ? 1024 : n >= 512 ? 256 : 128;         // a thread takes two or three elements of a wide row
    if (dtype == MB_F32) return launch_kernel(gated_rmsnorm_kernel<float>, rows, threads, 0, s, 0, o, w, (const float*)g, g_stride, gate, eps, (float*)out, n);
    if (dtype == MB_BF16) return launch_kernel(gated_rmsnorm_kernel<bf16>, rows, threads, 0, s, 0, o, w, (const bf16*)g, g_stride, gate, eps, (bf16*)out, n);
    return MB_ERR_BAD_DTYPE;
}

// ---- token shift: out[m, t, :] = h[t] + (h'[t] - h[t]) * mu[m], h' the row before in the same sequence ------------------
// The row before a step's first token of a request is what the request's state keeps (zeros at admission): `carry`
// points at it inside the state, one row of `state_stride` floats per slot.  Nothing is written to the state here (the
// first token's block of a request reads what its last token's block would write): the kernel that runs the recurrence
// stores the new last row.
template <typename T>
__global__ void shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ carry, long long state_stride,
                                 const int* __restrict__ req_index, const int* __restrict__ cu_tokens,
                                 const int* __restrict__ state_slots, const float* __restrict__ mu, int mixes,
                                 T* __restrict__ out, int tokens, int n) {
    PDL_ENTER();
    h = pdl_fresh(h);
    carry = pdl_fresh(carry);
    const int t = blockIdx.x;
    const int req = req_index[t];
    const bool first = cu_tokens[req] == t;
    const float* before = carry + (size_t)state_slots[req] * state_stride;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        const float now = to_f32(h[(size_t)t * n + i]);
        const float prev = first ? before[i] : to_f32(h[(size_t)(t - 1) * n + i]);
        const float d = prev - now;
        for (int m = 0; m < mixes; ++m)
            out[((size_t)m * tokens + t) * n + i] = from_f32<T>(fmaf(d, mu[(size_t)m * n + i], now));
    }
}

MB_API int mb_shift_mix(const void* h, int dtype, const float* carry, long long state_stride, const int* req_index,
                        const int* cu_tokens, const int* state_slots, const float* mu, int mixes, void* out, int tokens, int n,
                        cudaStream_t s) {
    if (tokens <= 0 || n <= 0 || mixes <= 0) return 0;
    const int threads = 128;
    // few tokens: a thread takes one column, so that every load of a token is in flight at once; many tokens: a block a token
    dim3 grid(tokens, tokens >= 512 ? 1 : (n + threads - 1) / threads);
    if (dtype == MB_F32)
        return launch_kernel(shift_mix_kernel<float>, grid, threads, 0, s, 0, (const float*)h, carry, state_stride, req_index, cu_tokens,
                             state_slots, mu, mixes, (float*)out, tokens, n);
    if (dtype == MB_BF16)
        return launch_kernel(shift_mix_kernel<bf16>, grid, threads, 0, s, 0, (const bf16*)h, carry, state_stride, req_index, cu_tokens,
                             state_slots, mu, mixes, (bf16*)out, tokens, n);
    return MB_ERR_BAD_DTYPE;
}

// ---- tanh (in place, any dtype) and the cap on logits: x <- cap * tanh(x / cap) -----------------------------------------
template <typename T>
__global__ void tanh_kernel(T* __restrict__ x, size_t total, float cap) {
    PDL_ENTER();
    x = pdl_fresh(x);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) x[idx] = from_f32<T>(cap * tanhf(to_f32(x[idx]) / cap));
}

MB_API int mb_tanh_cap(void* x, int dtype, size_t total, float cap, cudaStream_t s) {
    if (total == 0) return 0;
    if (!(cap > 0.0f)) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32) return launch_kernel(tanh_kernel<float>, blocks_for(total, 256), 256, 0, s, 0, (float*)x, total, cap);
    if (dtype == MB_BF16) return launch_kernel(tanh_kernel<bf16>, blocks_for(total, 256), 256, 0, s, 0, (bf16*)x, total, cap);
    return MB_ERR_BAD_DTYPE;
}

// ---- the square of relu, in place: x <- max(x, 0)^2 (the activation of a feed-forward without a gate) ----------------------
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, size_t total) {
    PDL_ENTER();
    x = pdl_fresh(x);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const float v = fmaxf(to_f32(x[idx]), 0.0f);
        x[idx] = from_f32<T>(v * v);
    }
}

MB_API int mb_relu2(void* x, int dtype, size_t total, cudaStream_t s) {
    if (total == 0) return 0;
    if (dtype == MB_F32) return launch_kernel(relu2_kernel<float>, blocks_for(total, 256), 256, 0, s, 0, (float*)x, total);
    if (dtype == MB_BF16) return launch_kernel(relu2_kernel<bf16>, blocks_for(total, 256), 256, 0, s, 0, (bf16*)x, total);
    return MB_ERR_BAD_DTYPE;
}

// ---- bias and activation in place: x[t, i] <- act(x[t, i] + b[i]); act 0: none, 1: gelu (erf), 2: gelu (tanh form) ---------
__device__ __forceinline__ float gelu_erf_f(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh_f(float v) { return 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v))); }

// (a row per blockIdx.x, its columns over blockIdx.y and the threads: no division per element)
template <typename T>
__global__ void bias_act_kernel(T* __restrict__ x, const float* __restrict__ b, int n, int act) {
    PDL_ENTER();
    x = pdl_fresh(x);
    T* row = x + (size_t)blockIdx.x * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        float v = to_f32(row[i]) + (b != nullptr ? b[i] : 0.0f);
        if (act == 1) v = gelu_erf_f(v);
        else if (act == 2) v = gelu_tanh_f(v);
        row[i] = from_f32<T>(v);
    }
}

static inline dim3 row_grid(int rows, int n) { return dim3(rows, (n + 1023) / 1024 < 64 ? (n + 1023) / 1024 : 64); }

MB_API int mb_bias_act(void* x, int dtype, const float* b, int rows, int n, int act, cudaStream_t s) {
    const size_t total = (size_t)rows * n;
    if (total == 0) return 0;
    if (act < 0 || act > 2) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32) return launch_kernel(bias_act_kernel<float>, row_grid(rows, n), 256, 0, s, 0, (float*)x, b, n, act);
    if (dtype == MB_BF16) return launch_kernel(bias_act_kernel<bf16>, row_grid(rows, n), 256, 0, s, 0, (bf16*)x, b, n, act);
    return MB_ERR_BAD_DTYPE;
}

// ---- a gated activation with capped inputs: out[t, c] = g sigmoid(alpha g) (u + shift) * row_scale ------------------------
// rows: [tokens][stride]: ff gate columns, then ff up columns; g = min(gate, limit), u = clamp(up, -limit, limit) where
// limit > 0 (else as they are).  scale_col >= 0: the row is multiplied by sigmoid(rows[t][scale_col]) (a number per token).
template <typename T>
__global__ void glu_capped_kernel(const T* __restrict__ rows, int stride, T* __restrict__ out, int tokens, int ff, float limit, float alpha,
                                  float shift, int scale_col) {
    PDL_ENTER();
    rows = pdl_fresh(rows);
    const size_t t = blockIdx.x;
    const T* row = rows + t * stride;
    const float row_scale = scale_col >= 0 ? 1.0f / (1.0f + expf(-to_f32(row[scale_col]))) : 1.0f;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ff; c += gridDim.y * blockDim.x) {
        float g = to_f32(row[c]), u = to_f32(row[ff + c]);
        if (limit > 0.0f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        out[t * ff + c] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + shift) * row_scale);
    }
}

MB_API int mb_glu_capped(const void* rows, int stride, int dtype, void* out, int tokens, int ff, float limit, float alpha, float shift,
                         int scale_col, cudaStream_t s) {
    const size_t total = (size_t)tokens * ff;
    if (total == 0) return 0;
    if (stride < 2 * ff || scale_col >= stride) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(glu_capped_kernel<float>, row_grid(tokens, ff), 256, 0, s, 0, (const float*)rows, stride, (float*)out, tokens, ff,
                             limit, alpha, shift, scale_col);
    if (dtype == MB_BF16)
        return launch_kernel(glu_capped_kernel<bf16>, row_grid(tokens, ff), 256, 0, s, 0, (const bf16*)rows, stride, (bf16*)out, tokens, ff,
                             limit, alpha, shift, scale_col);
    return MB_ERR_BAD_DTYPE;
}

// ---- a gate per head, in place: x[t, a, :] *= sigmoid(g[t, a]);  g: [tokens][g_stride] at column g_col -------------------
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ g, int g_stride, int g_col, size_t total, int heads, int dim) {
    PDL_ENTER();
    x = pdl_fresh(x); g = pdl_fresh(g);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    const size_t row = (size_t)heads * dim;
    for (; idx < total; idx += step) {
        const size_t t = idx / row;
        const int a = (int)((idx - t * row) / dim);
        const float gate = 1.0f / (1.0f + expf(-to_f32(g[t * g_stride + g_col + a])));
        x[idx] = from_f32<T>(to_f32(x[idx]) * gate);
    }
}

MB_API int mb_head_gate(void* x, int dtype, const void* g, int g_stride, int g_col, int tokens, int heads, int dim, cudaStream_t s) {
    const size_t total = (size_t)tokens * heads * dim;
    if (total == 0) return 0;
    if (dtype == MB_F32)
        return launch_kernel(head_gate_kernel<float>, blocks_for(total, 256), 256, 0, s, 0, (float*)x, (const float*)g, g_stride, g_col, total, heads, dim);
    if (dtype == MB_BF16)
        return launch_kernel(head_gate_kernel<bf16>, blocks_for(total, 256), 256, 0, s, 0, (bf16*)x, (const bf16*)g, g_stride, g_col, total, heads, dim);
    return MB_ERR_BAD_DTYPE;
}

// ---- the last row of every request of the step, kept for the next step's token shift: carry[slot] = h[last token] --------
template <typename T>
__global__ void keep_last_row_kernel(const T* __restrict__ h, float* __restrict__ carry, long long state_stride, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ state_slots, int n) {
    PDL_ENTER();
    h = pdl_fresh(h);
    const int req = blockIdx.x;
    const int first = cu_tokens[req], end = cu_tokens[req + 1];
    if (end <= first) return;
    float* dst = carry + (size_t)state_slots[req] * state_stride;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) dst[i] = to_f32(h[(size_t)(end - 1) * n + i]);
}

MB_API int mb_keep_last_row(const void* h, int dtype, float* carry, long long state_stride, const int* cu_tokens, const int* state_slots,
                            int requests, int n, cudaStream_t s) {
    if (requests <= 0 || n <= 0) return 0;
    dim3 grid(requests, (n + 255) / 256);
    if (dtype == MB_F32) return launch_kernel(keep_last_row_kernel<float>, grid, 256, 0, s, 0, (const float*)h, carry, state_stride, cu_tokens, state_slots, n);
    if (dtype == MB_BF16) return launch_kernel(keep_last_row_kernel<bf16>, grid, 256, 0, s, 0, (const bf16*)h, carry, state_stride, cu_tokens, state_slots, n);
    return MB_ERR_BAD_DTYPE;
}

// ---- a bias added to every row of the float32 residual: y[t, i] += b[i] -----------------------------------------------------
__global__ void add_row_bias_kernel(float* __restrict__ y, const float* __restrict__ b, int n) {
    PDL_ENTER();
    y = pdl_fresh(y);
    float* row = y + (size_t)blockIdx.x * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) row[i] += b[i];
}

MB_API int mb_add_row_bias(float* y, const float* b, int rows, int n, cudaStream_t s) {
    const size_t total = (size_t)rows * n;
    if (total == 0) return 0;
    return launch_kernel(add_row_bias_kernel, row_grid(rows, n), 256, 0, s, 0, y, b, n);
}

// ---- RMS norm of a column block of wider rows: out[t, :] = x[t, col : col + n] / rms * w, a block per row ------------------
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_cols_kernel(const T* __restrict__ x, int stride, int col, const float* __restrict__ w, float eps,
                                                           T* __restrict__ out, int n) {
    PDL_ENTER();
    x = pdl_fresh(x);
    __shared__ float scratch[32];
    const T* row = x + (size_t)blockIdx.x * stride + col;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(row[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float factor = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = from_f32<T>(to_f32(row[i]) * factor * w[i]);
}

MB_API int mb_rmsnorm_cols(const void* x, int stride, int col, int dtype, const float* w, float eps, void* out, int rows, int n, cudaStream_t s) {
    if (rows <= 0 || n <= 0) return 0;
    if (col < 0 || col + n > stride) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32) return launch_kernel(rmsnorm_cols_kernel<float>, rows, 256, 0, s, 0, (const float*)x, stride, col, w, eps, (float*)out, n);
    if (dtype == MB_BF16) return launch_kernel(rmsnorm_cols_kernel<bf16>, rows, 256, 0, s, 0, (const bf16*)x, stride, col, w, eps, (bf16*)out, n);
    return MB_ERR_BAD_DTYPE;
}
