// A selective state space layer with one decay per head and token (Mamba-2: Dao, Gu, "Transformers are SSMs: Generalized
// Models and Efficient Algorithms Through Structured State Space Duality"), around the in- and out-projections:
//   * a short causal convolution per channel over x | B | C with bias and silu; the last `taps - 1` inputs of a request are
//     part of its state (float32 [slot][taps - 1][channels], oldest first);
//   * per head h (group g = h / (heads / groups)):  dt = softplus(dt' + dt_bias_h),  a = exp(-exp(rate_h) dt),
//         S <- a S + dt B_g x_h^T   (S is N x P, float32, [slot][head][N][P]),   y = S^T C_g + skip_h x_h;
//   * y times silu(z), divided by its root mean square in `parts` equal parts of the row, times a weight.
// The step size, the decay, the state and the sums are float32 in both dtypes; x, B, C, z and dt' come as the projection
// left them.  A request's tokens are walked in order; requests, heads and slices of value channels side by side.
#define MB_LIB "ssm"
#define MB_LIB_ID 18
#include "common.cuh"
#include "launch.cuh"

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

// ---- convolution: a thread per (token, channel) ---------------------------------------------------------------------------
// in: [tokens][in_stride], the channels at column `in_col`; w: float32 [channels][taps] (the last column meets the current
// token); out: [tokens][channels] = silu(conv + bias).
template <typename T>
__global__ void ssm_conv_kernel(const T* __restrict__ in, int in_stride, int in_col, const float* __restrict__ w, const float* __restrict__ bias,
                                const float* __restrict__ carry, const int* __restrict__ req_index, const int* __restrict__ cu_tokens,
                                const int* __restrict__ slots, T* __restrict__ out, int tokens, int channels, int taps) {
    PDL_ENTER();
    in = pdl_fresh(in); carry = pdl_fresh(carry);
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= channels) return;
    const int req = req_index[t];
    const int first = cu_tokens[req];
    const float* before = carry + (size_t)slots[req] * (taps - 1) * channels;
    float sum = bias != nullptr ? bias[c] : 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                       // how many tokens before the current one
        const int at = t - back;
        float v;
        if (at >= first) v = to_f32(in[(size_t)at * in_stride + in_col + c]);
        else v = before[(size_t)(taps - 1 - (first - at)) * channels + c];      // first - at = 1: the newest kept input
        sum = fmaf(w[(size_t)c * taps + j], v, sum);
    }
    out[(size_t)t * channels + c] = from_f32<T>(silu_f(sum));
}

// The kept inputs after the step: a thread per (request, channel) reads what it needs of the old ones before it writes.
template <typename T>
__global__ void ssm_conv_carry_kernel(const T* __restrict__ in, int in_stride, int in_col, float* __restrict__ carry,
                                      const int* __restrict__ cu_tokens, const int* __restrict__ slots, int channels, int taps) {
    PDL_ENTER();
    in = pdl_fresh(in);
    const int c = blockIdx.x * blockDim.x + threadIdx.x, req = blockIdx.y;
    if (c >= channels) return;
    const int first = cu_tokens[req], count = cu_tokens[req + 1] - first;
    if (count <= 0) return;
    float* kept = carry + (size_t)slots[req] * (taps - 1) * channels;
    const int n = taps - 1;
    for (int j = 0; j < n; ++j) {
        const int at = count - n + j;                        // index among this step's tokens; negative: an older one
        const float v = at >= 0 ? to_f32(in[(size_t)(first + at) * in_stride + in_col + c]) : kept[(size_t)(j + count) * channels + c];
        kept[(size_t)j * channels + c] = v;                  // row j + count > j is read before row j is written
    }
}

MB_API int mb_ssm_conv(const void* in, int in_stride, int in_col, int dtype, const float* w, const float* bias, const float* carry,
                       const int* req_index, const int* cu_tokens, const int* slots, void* out, int tokens, int channels, int taps,
                       cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (channels <= 0 || taps <= 0 || taps > 64) return MB_ERR_BAD_SIZE;
    const int threads = 128;
    dim3 grid((channels + threads - 1) / threads, tokens);
    if (dtype == MB_F32)
        return launch_kernel(ssm_conv_kernel<float>, grid, threads, 0, s, 0, (const float*)in, in_stride, in_col, w, bias, carry, req_index,
                             cu_tokens, slots, (float*)out, tokens, channels, taps);
    if (dtype == MB_BF16)
        return launch_kernel(ssm_conv_kernel<bf16>, grid, threads, 0, s, 0, (const bf16*)in, in_stride, in_col, w, bias, carry, req_index,
                             cu_tokens, slots, (bf16*)out, tokens, channels, taps);
    return MB_ERR_BAD_DTYPE;
}

// After the convolution has read them: the kept inputs brought up to date (taps > 1).
MB_API int mb_ssm_conv_carry(const void* in, int in_stride, int in_col, int dtype, float* carry, const int* cu_tokens, const int* slots,
                             int requests, int channels, int taps, cudaStream_t s) {
    if (requests <= 0 || taps <= 1) return 0;
    if (channels <= 0 || taps > 64) return MB_ERR_BAD_SIZE;
    const int threads = 128;
    dim3 grid((channels + threads - 1) / threads, requests);
    if (dtype == MB_F32)
        return launch_kernel(ssm_conv_carry_kernel<float>, grid, threads, 0, s, 0, (const float*)in, in_stride, in_col, carry, cu_tokens, slots,
                             channels, taps);
    if (dtype == MB_BF16)
        return launch_kernel(ssm_conv_carry_kernel<bf16>, grid, threads, 0, s, 0, (const bf16*)in, in_stride, in_col, carry, cu_tokens, slots,
                             channels, taps);
    return MB_ERR_BAD_DTYPE;
}

// ---- the recurrence: a block per (request, head, slice of SS_COLS value channels) -----------------------------------------
// Four threads share a column of the state: thread (column, part) keeps the rows part, part + 4, ... in registers, ROWS of
// them.  Tokens are taken in runs of SS_RUN: their B, C, x and step sizes go to shared memory, then the run is walked
// without a barrier (the four partial sums of a column meet by shuffles).
#define SS_COLS 32
#define SS_THREADS (SS_COLS * 4)
#define SS_RUN 16

// mode 0: a request's tokens of the step in one walk, from its state slot and back into it.
// Long portions are cut into segments of `seg_len` tokens that are walked side by side (the recurrence is linear in the state):
// mode 1: every segment from a zero state, no outputs; its end state goes to seg_state[segment] and the product of its decays
//         to seg_decay[segment][head];
// (ssm_combine_kernel then turns the end states into the segments' start states, S <- decay_b S + end_b, segment after segment
//  from the slot's state, and leaves the last one in the slot;)
// mode 2: every segment again from its start state, for the outputs.
// blockIdx.x = request * segments + segment (one segment in mode 0).
template <typename T, int ROWS>
__global__ void __launch_bounds__(SS_THREADS) ssm_scan_kernel(
    const T* __restrict__ xbc, const T* __restrict__ dt_rows, int dt_stride, int dt_col, const float* __restrict__ dt_bias,
    const float* __restrict__ rate_log, const float* __restrict__ skip, float* __restrict__ state, const int* __restrict__ cu_tokens,
    const int* __restrict__ slots, float* __restrict__ y, int heads, int P, int N, int groups, int mode, int segments, int seg_len,
    float* __restrict__ seg_state, float* __restrict__ seg_decay) {
    PDL_ENTER();
    xbc = pdl_fresh(xbc); dt_rows = pdl_fresh(dt_rows);
    extern __shared__ float smem[];
    float* Bs = smem;                          // [SS_RUN][N]
    float* Cs = Bs + SS_RUN * N;               // [SS_RUN][N]
    float* xs = Cs + SS_RUN * N;               // [SS_RUN][SS_COLS]
    float* steps = xs + SS_RUN * SS_COLS;      // [SS_RUN] dt, [SS_RUN] decay
    const int req = blockIdx.x / segments, seg = blockIdx.x - req * segments;
    const int head = blockIdx.y, col0 = blockIdx.z * SS_COLS;
    int first = cu_tokens[req], count = cu_tokens[req + 1] - first;
    if (mode != 0) {
        first += seg * seg_len;
        count = max(0, min(seg_len, count - seg * seg_len));
    }
    if (count <= 0 && mode != 1) return;
    const int inner = heads * P, channels = inner + 2 * groups * N;
    const int g = head / (heads / groups);
    const int col = threadIdx.x >> 2, part = threadIdx.x & 3;
    const int p = col0 + col;
    const bool in_range = p < P;
    float* S = mode == 0 ? state + (((size_t)slots[req] * heads + head) * N) * P
                         : seg_state + (((size_t)blockIdx.x * heads + head) * N) * P;
    float s[ROWS];
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        const int n = part + 4 * j;
        s[j] = (mode != 1 && in_range && n < N) ? S[(size_t)n * P + p] : 0.0f;
    }
    const float rate = expf(rate_log[head]), bias = dt_bias[head], d_skip = skip[head];
    float log_decay = 0.0f;
    for (int base = 0; base < count; base += SS_RUN) {
        const int run = min(SS_RUN, count - base);
        __syncthreads();
        for (int i = threadIdx.x; i < run * N; i += SS_THREADS) {
            const int tt = i / N, n = i - tt * N;
            const T* row = xbc + (size_t)(first + base + tt) * channels;
            Bs[tt * N + n] = to_f32(row[inner + g * N + n]);
            Cs[tt * N + n] = to_f32(row[inner + groups * N + g * N + n]);
        }
        for (int i = threadIdx.x; i < run * SS_COLS; i += SS_THREADS) {
            const int tt = i / SS_COLS, cc = i - tt * SS_COLS;
            xs[i] = col0 + cc < P ? to_f32(xbc[(size_t)(first + base + tt) * channels + head * P + col0 + cc]) : 0.0f;
        }
        if (threadIdx.x < run) {
            const float dt = softplus_f(to_f32(dt_rows[(size_t)(first + base + threadIdx.x) * dt_stride + dt_col + head]) + bias);
            steps[threadIdx.x] = dt;
            steps[SS_RUN + threadIdx.x] = -rate * dt;
        }
        __syncthreads();
        for (int tt = 0; tt < run; ++tt) {
            const float dt = steps[tt], a = expf(steps[SS_RUN + tt]);
            log_decay += steps[SS_RUN + tt];
            const float x = xs[tt * SS_COLS + col];
            const float dx = dt * x;
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};                      // four chains instead of one of ROWS dependent sums
#pragma unroll
            for (int j = 0; j < ROWS; ++j) {
                const int n = part + 4 * j;
                if (n < N) {
                    s[j] = fmaf(a, s[j], dx * Bs[tt * N + n]);
                    sums[j & 3] = fmaf(s[j], Cs[tt * N + n], sums[j & 3]);
                }
            }
            float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            if (mode != 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (part == 0 && in_range) y[(size_t)(first + base + tt) * inner + head * P + p] = fmaf(d_skip, x, sum);
            }
        }
    }
    if (mode == 2) return;
    if (in_range) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int n = part + 4 * j;
            if (n < N) S[(size_t)n * P + p] = s[j];
        }
    }
    if (mode == 1 && threadIdx.x == 0 && blockIdx.z == 0) seg_decay[(size_t)blockIdx.x * heads + head] = expf(log_decay);
}

// The segments' end states turned into their start states, in place: a block per (request, head).
__global__ void __launch_bounds__(256) ssm_combine_kernel(float* __restrict__ state, const int* __restrict__ slots, float* __restrict__ seg_state,
                                                          const float* __restrict__ seg_decay, int heads, int elems, int segments) {
    PDL_ENTER();
    const int req = blockIdx.x, head = blockIdx.y;
    float* S = state + ((size_t)slots[req] * heads + head) * elems;
    for (int e = threadIdx.x; e < elems; e += blockDim.x) {
        float v = S[e];
        for (int b = 0; b < segments; ++b) {
            const size_t at = (size_t)req * segments + b;
            float* slot = seg_state + (at * heads + head) * elems + e;
            const float end = *slot;
            *slot = v;
            v = fmaf(seg_decay[at * heads + head], v, end);
        }
        S[e] = v;
    }
}

template <typename T>
static int ssm_scan_rows(int rows, dim3 grid, size_t smem, cudaStream_t s, const T* xbc, const T* dt_rows, int dt_stride, int dt_col,
                         const float* dt_bias, const float* rate_log, const float* skip, float* state, const int* cu_tokens, const int* slots,
                         float* y, int heads, int P, int N, int groups, int mode, int segments, int seg_len, float* seg_state, float* seg_decay) {
#define SS_CASE(R)                                                                                                                   \
    if (rows <= R)                                                                                                                   \
        return launch_kernel(ssm_scan_kernel<T, R>, grid, SS_THREADS, smem, s, 0, xbc, dt_rows, dt_stride, dt_col, dt_bias, rate_log, skip, \
                             state, cu_tokens, slots, y, heads, P, N, groups, mode, segments, seg_len, seg_state, seg_decay);
    SS_CASE(4) SS_CASE(8) SS_CASE(16) SS_CASE(32) SS_CASE(64)
#undef SS_CASE
    return MB_ERR_BAD_SIZE;
}

// xbc: [tokens][heads P + 2 groups N] after the convolution; dt_rows: the projection's rows, dt' of head h at column dt_col + h.
// mode 0 with segments = 1: one walk per request.  Modes 1 and 2 (see the kernel): `segments` segments of seg_len tokens a request,
// seg_state float32 [requests][segments][heads][N][P], seg_decay [requests][segments][heads]; mode 3: the combining step between them.
MB_API int mb_ssm_scan(const void* xbc, const void* dt_rows, int dt_stride, int dt_col, int dtype, const float* dt_bias, const float* rate_log,
                       const float* skip, float* state, const int* cu_tokens, const int* slots, float* y, int requests, int heads, int P, int N,
                       int groups, int mode, int segments, int seg_len, float* seg_state, float* seg_decay, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (heads <= 0 || P <= 0 || N <= 0 || N > 256 || groups <= 0 || heads % groups != 0 || mode < 0 || mode > 3) return MB_ERR_BAD_SIZE;
    if (mode == 0) segments = 1;
    if (segments <= 0 || (mode != 0 && (seg_len <= 0 || seg_state == nullptr || seg_decay == nullptr))) return MB_ERR_BAD_SIZE;
    if (mode == 3)
        return launch_kernel(ssm_combine_kernel, dim3(requests, heads), 256, 0, s, 0, state, slots, seg_state, (const float*)seg_decay, heads,
                             N * P, segments);
    dim3 grid(requests * segments, heads, (P + SS_COLS - 1) / SS_COLS);
    const size_t smem = (size_t)(2 * SS_RUN * N + SS_RUN * SS_COLS + 2 * SS_RUN) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    const int rows = (N + 3) / 4;
    if (dtype == MB_F32)
        return ssm_scan_rows<float>(rows, grid, smem, s, (const float*)xbc, (const float*)dt_rows, dt_stride, dt_col, dt_bias, rate_log, skip,
                                    state, cu_tokens, slots, y, heads, P, N, groups, mode, segments, seg_len, seg_state, seg_decay);
    if (dtype == MB_BF16)
        return ssm_scan_rows<bf16>(rows, grid, smem, s, (const bf16*)xbc, (const bf16*)dt_rows, dt_stride, dt_col, dt_bias, rate_log, skip,
                                   state, cu_tokens, slots, y, heads, P, N, groups, mode, segments, seg_len, seg_state, seg_decay);
    return MB_ERR_BAD_DTYPE;
}

// ---- gate, then norm in equal parts of the row: a block per (token, part) -------------------------------------------------
// out = (y silu(z)) / rms_part(y silu(z)) * weight;  z: [tokens][z_stride] at column z_col.
template <typename T>
__global__ void __launch_bounds__(256) ssm_gate_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int z_stride, int z_col,
                                                            const float* __restrict__ weight, float eps, T* __restrict__ out, int n, int parts) {
    PDL_ENTER();
    y = pdl_fresh(y); z = pdl_fresh(z);
    __shared__ float scratch[32];
    const int t = blockIdx.x, part = blockIdx.y;
    const int width = n / parts, c0 = part * width;
    const float* yr = y + (size_t)t * n + c0;
    const T* zr = z + (size_t)t * z_stride + z_col + c0;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_f32(zr[i]));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float factor = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_f32(zr[i]));
        out[(size_t)t * n + c0 + i] = from_f32<T>(v * factor * weight[c0 + i]);
    }
}

MB_API int mb_ssm_gate_norm(const float* y, const void* z, int z_stride, int z_col, int dtype, const float* weight, float eps, void* out,
                            int tokens, int n, int parts, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (n <= 0 || parts <= 0 || n % parts != 0) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, parts);
    if (dtype == MB_F32)
        return launch_kernel(ssm_gate_norm_kernel<float>, grid, 256, 0, s, 0, y, (const float*)z, z_stride, z_col, weight, eps, (float*)out, n, parts);
    if (dtype == MB_BF16)
        return launch_kernel(ssm_gate_norm_kernel<bf16>, grid, 256, 0, s, 0, y, (const bf16*)z, z_stride, z_col, weight, eps, (bf16*)out, n, parts);
    return MB_ERR_BAD_DTYPE;
}
