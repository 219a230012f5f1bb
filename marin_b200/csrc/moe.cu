// A routed feed-forward (mixture of experts): a router scores every expert for every token, the `top` best are chosen,
// and the token goes through those experts only.  Expert: down( silu(gate x) * (up x) ), no biases; or, `act_mode` 1, an
// expert without a gate, down( relu(up x)^2 ), whose first matrix is [experts][ff][h].  Instead of a router a table may
// name every token id's experts (mb_moe_table_route): the choice then depends on the token alone, with equal weights.
// The gated form is g sigmoid(alpha g) (u + shift) with g = gate x and u = up x, both capped where `act_limit` > 0
// (g <- min(g, limit), u <- clamp(u, -limit, limit)); alpha 1, shift 0 and no limit is silu(gate x) * (up x).
//   * router: z = W_r h in float32, score = sigmoid(z) or the softmax of z over the experts; the chosen experts' scores are
//     the weights, renormalised to sum 1 over the chosen ones if asked;
//   * the weight multiplies the expert's input (x = w h, the activation sees it) or its output (x = h, result times w).
// Kernels: the router with its top-k (a warp per token), the grouping of (token, choice) pairs by expert (offsets and an
// order), and the plain expert products for any size in both dtypes (a pair per block).  A pair's result never depends on
// which other pairs the step holds or on the order they were grouped in; a token's pairs are added in choice order.
// Weights: gate|up as [experts][2 ff][h], down as [experts][h][ff].  The gate and up rows of an expert lie either one after
// the other (gate rows first) or, `interleaved`, in alternating blocks of 16 rows (16 gate rows, the 16 up rows of the same
// columns, ...): the layout the dense product's fused SwiGLU epilogue reads, so that an expert's matrix can go to it as it is.
#define MB_LIB "moe"
#define MB_LIB_ID 14
#include "common.cuh"
#include "launch.cuh"

#define MR_THREADS 256

// Row of gate column c (which = 0) or up column c (which = 1) in an expert's gate|up matrix.
__host__ __device__ __forceinline__ int gate_up_row(int c, int which, int ff, int interleaved) {
    return interleaved ? (c / 16) * 32 + which * 16 + c % 16 : which * ff + c;
}

// ---- router and top-k: a token per block -------------------------------------------------------------------------------
// expert_out int32 [tokens][top], weight_out float32 [tokens][top], choices in order of decreasing score (the lower expert
// among equals).  score_mode 0: sigmoid, 1: softmax over all experts.  A warp takes every eighth expert; its lanes walk the
// row in a fixed order, so a token's logits do not depend on the batch.
template <typename T>
__global__ void __launch_bounds__(MR_THREADS) moe_route_kernel(const T* __restrict__ h_rows, const float* __restrict__ router,
                                                               const float* __restrict__ router_bias, int* __restrict__ expert_out, float* __restrict__ weight_out,
                                                               int tokens, int h, int E, int top, int score_mode, int renorm) {
    PDL_ENTER();
    h_rows = pdl_fresh(h_rows);
    extern __shared__ float smem[];
    float* xrow = smem;                        // [h] (first: 16-byte aligned)
    float* z = smem + h;                       // [E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const T* x = h_rows + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += MR_THREADS) xrow[i] = to_f32(x[i]);
    __syncthreads();
    for (int e = warp; e < E; e += MR_THREADS / 32) {
        const float* w = router + (size_t)e * h;
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
        int i = lane;
        if ((h & 3) == 0 && (((uintptr_t)w) & 15) == 0) {         // 16-byte loads, four of them in flight
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* x4 = reinterpret_cast<const float4*>(xrow);
            const int n4 = h >> 2;
            int j = lane;
            for (; j + 96 < n4; j += 128) {
                const float4 a0 = w4[j], a1 = w4[j + 32], a2 = w4[j + 64], a3 = w4[j + 96];
                const float4 b0 = x4[j], b1 = x4[j + 32], b2 = x4[j + 64], b3 = x4[j + 96];
                d0 = fmaf(b0.x, a0.x, fmaf(b0.y, a0.y, fmaf(b0.z, a0.z, fmaf(b0.w, a0.w, d0))));
                d1 = fmaf(b1.x, a1.x, fmaf(b1.y, a1.y, fmaf(b1.z, a1.z, fmaf(b1.w, a1.w, d1))));
                d2 = fmaf(b2.x, a2.x, fmaf(b2.y, a2.y, fmaf(b2.z, a2.z, fmaf(b2.w, a2.w, d2))));
                d3 = fmaf(b3.x, a3.x, fmaf(b3.y, a3.y, fmaf(b3.z, a3.z, fmaf(b3.w, a3.w, d3))));
            }
            for (; j < n4; j += 32) {
                const float4 a0 = w4[j], b0 = x4[j];
                d0 = fmaf(b0.x, a0.x, fmaf(b0.y, a0.y, fmaf(b0.z, a0.z, fmaf(b0.w, a0.w, d0))));
            }
            i = h;
        }
        for (; i + 96 < h; i += 128) {
            d0 = fmaf(xrow[i], w[i], d0); d1 = fmaf(xrow[i + 32], w[i + 32], d1);
            d2 = fmaf(xrow[i + 64], w[i + 64], d2); d3 = fmaf(xrow[i + 96], w[i + 96], d3);
        }
        for (; i < h; i += 32) d0 = fmaf(xrow[i], w[i], d0);
        const float dot = warp_sum((d0 + d1) + (d2 + d3));
        if (lane == 0) z[e] = router_bias != nullptr ? dot + router_bias[e] : dot;
    }
    __syncthreads();
    if (warp != 0) return;
    float denom = 1.0f, zmax = 0.0f;
    if (score_mode == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        zmax = warp_max(mx);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - zmax);
        denom = warp_sum(sum);
    }
    float chosen_sum = 0.0f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = c;                                   // logits that are not numbers order nothing: stay inside the table
        const float score = score_mode == 1 ? expf(best - zmax) / denom : 1.0f / (1.0f + expf(-best));
        chosen_sum += score;
        if (lane == 0) {
            expert_out[(size_t)t * top + c] = at;
            weight_out[(size_t)t * top + c] = score;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int c = 0; c < top; ++c) weight_out[(size_t)t * top + c] /= chosen_sum;
}

MB_API int mb_moe_route(const void* h_rows, int dtype, const float* router, const float* router_bias, int* expert_out, float* weight_out, int tokens, int h,
                        int E, int top, int score_mode, int renorm, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || h <= 0 || score_mode < 0 || score_mode > 1) return MB_ERR_BAD_SIZE;
    const size_t smem = (size_t)(E + h) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(moe_route_kernel<float>, tokens, MR_THREADS, smem, s, 0, (const float*)h_rows, router, router_bias, expert_out,
                             weight_out, tokens, h, E, top, score_mode, renorm);
    if (dtype == MB_BF16)
        return launch_kernel(moe_route_kernel<bf16>, tokens, MR_THREADS, smem, s, 0, (const bf16*)h_rows, router, router_bias, expert_out,
                             weight_out, tokens, h, E, top, score_mode, renorm);
    return MB_ERR_BAD_DTYPE;
}

// ---- experts named by a table over the token ids: expert_out[t][c] = table[ids[t]][c], every weight 1 / top ------------------
__global__ void moe_table_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, int* __restrict__ expert_out,
                                       float* __restrict__ weight_out, int tokens, int top, int vocab, int E) {
    PDL_ENTER();
    ids = pdl_fresh(ids);
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= tokens * top) return;
    const int t = p / top, c = p - t * top;
    int id = ids[t];
    id = id < 0 ? 0 : id >= vocab ? vocab - 1 : id;
    int e = table[(size_t)id * top + c];
    e = e < 0 ? 0 : e >= E ? E - 1 : e;                         // a table from a damaged file stays inside the experts
    expert_out[p] = e;
    weight_out[p] = 1.0f / (float)top;
}

MB_API int mb_moe_table_route(const int* ids, const int* table, int* expert_out, float* weight_out, int tokens, int top, int vocab, int E,
                              cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (top <= 0 || vocab <= 0 || E <= 0) return MB_ERR_BAD_SIZE;
    return launch_kernel(moe_table_route_kernel, (tokens * top + 127) / 128, 128, 0, s, 0, ids, table, expert_out, weight_out, tokens, top, vocab, E);
}

// ---- pairs grouped by expert: offsets[E + 1] and order[pairs] (the pairs of expert e are order[offsets[e] .. offsets[e+1])) ----
// One block.  Within an expert the pairs come in no fixed order: no result depends on it.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ expert_of, int pairs, int E, int* __restrict__ offsets,
                                                         int* __restrict__ order) {
    PDL_ENTER();
    expert_of = pdl_fresh(expert_of);
    extern __shared__ int counts[];            // [E] counts, then [E] cursors
    int* cursor = counts + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[expert_of[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { offsets[e] = run; cursor[e] = run; run += counts[e]; }
        offsets[E] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) order[atomicAdd(&cursor[expert_of[p]], 1)] = p;
}

MB_API int mb_moe_group(const int* expert_of, int pairs, int E, int* offsets, int* order, cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (E <= 0 || (size_t)E * 8 > 48 * 1024) return MB_ERR_BAD_SIZE;
    return launch_kernel(moe_group_kernel, 1, 1024, (size_t)E * 8, s, 0, expert_of, pairs, E, offsets, order);
}

// ---- plain expert products ---------------------------------------------------------------------------------------------
#define ME_THREADS 256

// act[p][c] = silu(gate_c . x) * (up_c . x) for pair p = token * top + choice, x = h[token] (times the pair's weight where the
// weight goes on the input), rounded to the activation dtype as the tensor-core path's operand would be.
template <typename T>
__global__ void __launch_bounds__(ME_THREADS) moe_gate_up_kernel(const T* __restrict__ h_rows, const T* __restrict__ w_gate_up,
                                                                 const int* __restrict__ expert_of, const float* __restrict__ weight_of,
                                                                 T* __restrict__ act, int h, int ff, int top, int weight_on_input,
                                                                 int interleaved, int act_mode, float act_limit, float act_alpha,
                                                                 float act_shift) {
    PDL_ENTER();
    h_rows = pdl_fresh(h_rows); expert_of = pdl_fresh(expert_of); weight_of = pdl_fresh(weight_of);
    extern __shared__ float x[];               // [h]
    const int p = blockIdx.x;
    const int token = p / top;
    const int e = expert_of[p];
    const float wgt = weight_on_input ? weight_of[p] : 1.0f;
    for (int i = threadIdx.x; i < h; i += ME_THREADS) x[i] = to_f32(from_f32<T>(to_f32(h_rows[(size_t)token * h + i]) * wgt));
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (act_mode == 1) {                                       // no gate: relu(up x)^2
        const T* only = w_gate_up + (size_t)e * ff * h;
        for (int c = warp; c < ff; c += ME_THREADS / 32) {
            const T* u = only + (size_t)c * h;
            float du = 0.0f;
            for (int i = lane; i < h; i += 32) du = fmaf(x[i], to_f32(u[i]), du);
            du = fmaxf(warp_sum(du), 0.0f);
            if (lane == 0) act[(size_t)p * ff + c] = from_f32<T>(du * du);
        }
        return;
    }
    const T* base = w_gate_up + (size_t)e * 2 * ff * h;
    for (int c = warp; c < ff; c += ME_THREADS / 32) {
        const T* g = base + (size_t)gate_up_row(c, 0, ff, interleaved) * h;
        const T* u = base + (size_t)gate_up_row(c, 1, ff, interleaved) * h;
        float dg = 0.0f, du = 0.0f;
        for (int i = lane; i < h; i += 32) { dg = fmaf(x[i], to_f32(g[i]), dg); du = fmaf(x[i], to_f32(u[i]), du); }
        dg = warp_sum(dg);
        du = warp_sum(du);
        if (act_limit > 0.0f) { dg = fminf(dg, act_limit); du = fminf(fmaxf(du, -act_limit), act_limit); }
        if (lane == 0) act[(size_t)p * ff + c] = from_f32<T>(dg / (1.0f + expf(-act_alpha * dg)) * (du + act_shift));
    }
}

// y[token][c] += sum over the token's choices, in choice order, of (down_c . act[pair]) (times the pair's weight where the
// weight goes on the output).  A token per block.
template <typename T>
__global__ void __launch_bounds__(ME_THREADS) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                              const int* __restrict__ expert_of, const float* __restrict__ weight_of,
                                                              float* __restrict__ y, int h, int ff, int top, int weight_on_input) {
    PDL_ENTER();
    act = pdl_fresh(act); expert_of = pdl_fresh(expert_of); weight_of = pdl_fresh(weight_of); y = pdl_fresh(y);
    extern __shared__ float a[];               // [ff]
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = 0; c < top; ++c) {
        const int p = token * top + c;
        const int e = expert_of[p];
        const float wgt = weight_on_input ? 1.0f : weight_of[p];
        __syncthreads();
        for (int i = threadIdx.x; i < ff; i += ME_THREADS) a[i] = to_f32(act[(size_t)p * ff + i]);
        __syncthreads();
        const T* base = w_down + (size_t)e * h * ff;
        for (int col = warp; col < h; col += ME_THREADS / 32) {
            const T* w = base + (size_t)col * ff;
            float dot = 0.0f;
            for (int i = lane; i < ff; i += 32) dot = fmaf(a[i], to_f32(w[i]), dot);
            dot = warp_sum(dot);
            if (lane == 0) y[(size_t)token * h + col] += dot * wgt;
        }
    }
}

// which = 0: act <- the activations of every pair; which = 1: y += the chosen experts' outputs, from act.
MB_API int mb_moe_experts_plain(const void* h_rows, int dtype, const void* w_gate_up, const void* w_down, const int* expert_of,
                                const float* weight_of, void* act, float* y, int tokens, int h, int ff, int top, int weight_on_input,
                                int interleaved, int which, int act_mode, float act_limit, float act_alpha, float act_shift, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (h <= 0 || ff <= 0 || top <= 0 || (size_t)h * 4 > 48 * 1024 || (size_t)ff * 4 > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32) {
        if (which == 0)
            return launch_kernel(moe_gate_up_kernel<float>, tokens * top, ME_THREADS, (size_t)h * 4, s, 0, (const float*)h_rows,
                                 (const float*)w_gate_up, expert_of, weight_of, (float*)act, h, ff, top, weight_on_input, interleaved, act_mode, act_limit, act_alpha, act_shift);
        return launch_kernel(moe_down_kernel<float>, tokens, ME_THREADS, (size_t)ff * 4, s, 0, (const float*)act, (const float*)w_down,
                             expert_of, weight_of, y, h, ff, top, weight_on_input);
    }
    if (dtype == MB_BF16) {
        if (which == 0)
            return launch_kernel(moe_gate_up_kernel<bf16>, tokens * top, ME_THREADS, (size_t)h * 4, s, 0, (const bf16*)h_rows,
                                 (const bf16*)w_gate_up, expert_of, weight_of, (bf16*)act, h, ff, top, weight_on_input, interleaved, act_mode, act_limit, act_alpha, act_shift);
        return launch_kernel(moe_down_kernel<bf16>, tokens, ME_THREADS, (size_t)ff * 4, s, 0, (const bf16*)act, (const bf16*)w_down,
                             expert_of, weight_of, y, h, ff, top, weight_on_input);
    }
    return MB_ERR_BAD_DTYPE;
}

// ---- bf16 experts on the tensor cores (mma.sync): pairs sorted by expert, one grouped product per projection --------------
// 1. gather: xs[i] = bf16(w h[token]) of the i-th pair in expert order (w = 1 where the weight goes on the output), with the
//    pair's token and weight beside it and, for every pair, where it went (inv).
// 2. gate|up: act[i][c] = silu(gate_c . xs[i]) * (up_c . xs[i]); a CTA takes 64 pairs of one expert x 64 columns, both
//    projections of those columns side by side (two accumulators), K in steps of 64 through a 3-stage cp.async ring.
// 3. down: out[i][:] = down . act[i]; with one choice per token it adds straight into y[token] (no two pairs share a row),
//    otherwise it leaves float32 rows that a last kernel adds into y in choice order.
// A pair's row is computed from that row's operands alone, whichever tile it lands in.
#include "mma_helpers.cuh"

#define GN 64
#define GK 64
#define GLD (GK + 8)
// stages of the cp.async ring: the down product has one weight tile per stage and few CTAs when few experts are chosen, so it
// keeps more stages in flight
#define G_STAGES_OF(MODE) ((MODE) == 0 ? 4 : 6)
#define G_NB_OF(MODE) ((MODE) == 0 ? 2 : 1)

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h_rows, const int* __restrict__ order, const float* __restrict__ weight_of,
                                  T* __restrict__ xs, int* __restrict__ token_sorted, float* __restrict__ weight_sorted,
                                  int* __restrict__ inv, int h, int top, int weight_on_input) {
    PDL_ENTER();
    h_rows = pdl_fresh(h_rows); order = pdl_fresh(order); weight_of = pdl_fresh(weight_of);
    const int i = blockIdx.x;
    const int p = order[i];
    const int token = p / top;
    const float w = weight_of[p];
    if (threadIdx.x == 0) { token_sorted[i] = token; weight_sorted[i] = w; inv[p] = i; }
    const float f = weight_on_input ? w : 1.0f;
    for (int c = threadIdx.x; c < h; c += blockDim.x) xs[(size_t)i * h + c] = from_f32<T>(to_f32(h_rows[(size_t)token * h + c]) * f);
}

// MODE 0: W [E][2 N][K] (gate rows, then up rows), result silu(gate) * up as bf16 [rows][N].
// MODE 1: W [E][N][K], result float32: row r goes to dst_rows[r] (null: r), times row_scale[r] (null: 1), added if `accumulate`.
// MODE 2: W [E][N][K] (experts without a gate), result relu(.)^2 as bf16 [rows][N].
// GMT: pairs per tile, 16, 32 or 64.  The four warps take 16 rows each where the tile has 64, two row groups x two column
// groups where it has 32, four column groups of 16 where it has 16: with few pairs per expert (single-token steps) a tile of
// 64 rows would spend the tensor pipe on rows that hold nothing (measured: 45 % of its cycles on 2 live rows of 64).
template <int MODE, int GMT>
__global__ void __launch_bounds__(128) moe_grouped_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W,
                                                          const int* __restrict__ offsets, int E, int N, int K, bf16* __restrict__ act_out,
                                                          float* __restrict__ f_out, const int* __restrict__ dst_rows,
                                                          const float* __restrict__ row_scale, int accumulate, int interleaved,
                                                          float act_limit, float act_alpha, float act_shift) {
    PDL_ENTER();
    A = pdl_fresh(A); offsets = pdl_fresh(offsets); dst_rows = pdl_fresh(dst_rows); row_scale = pdl_fresh(row_scale); f_out = pdl_fresh(f_out);
    constexpr int NB = G_NB_OF(MODE);
    constexpr int G_STAGES = G_STAGES_OF(MODE);
    constexpr int WR = GMT / 16, WC = 4 / WR, NT = (GN / 8) / WC;       // row groups, column groups, 8-column tiles per warp
    extern __shared__ __align__(16) uint8_t g_smem[];
    bf16* sA = reinterpret_cast<bf16*>(g_smem);                              // [G_STAGES][GMT][GLD]
    bf16* sB = sA + G_STAGES * GMT * GLD;                                    // [G_STAGES][NB][GN][GLD]
    // which expert's which tile this CTA is: tiles are numbered expert after expert
    int tile = blockIdx.x, e = 0, row0 = -1, row_end = 0;
    for (e = 0; e < E; ++e) {
        const int b = offsets[e], n = offsets[e + 1] - b;
        const int tiles = (n + GMT - 1) / GMT;
        if (tile < tiles) { row0 = b + tile * GMT; row_end = b + n; break; }
        tile -= tiles;
    }
    if (row0 < 0) return;
    const int col0 = blockIdx.y * GN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* We = W + (size_t)e * NB * N * K;
    const int a_rows = min(GMT, row_end - row0), b_rows = min(GN, N - col0);
    const int warp_r = warp % WR, warp_c = warp / WR;
    // rows of a tile past the expert's pairs, or past the last column, are zero in every stage and are never copied into
    for (int idx = threadIdx.x; idx < G_STAGES * GMT * (GK / 8); idx += 128) {
        const int r = (idx / (GK / 8)) % GMT;
        if (r >= a_rows) *reinterpret_cast<uint4*>(sA + (idx / (GK / 8)) * GLD + (idx % (GK / 8)) * 8) = make_uint4(0, 0, 0, 0);
    }
    if (b_rows < GN)
        for (int idx = threadIdx.x; idx < G_STAGES * NB * GN * (GK / 8); idx += 128) {
            const int r = (idx / (GK / 8)) % GN;
            if (r >= b_rows) *reinterpret_cast<uint4*>(sB + (idx / (GK / 8)) * GLD + (idx % (GK / 8)) * 8) = make_uint4(0, 0, 0, 0);
        }
    auto load = [&](int stage, int kt) {
        const int k0 = kt * GK;
        bf16* a = sA + stage * GMT * GLD;
        for (int idx = threadIdx.x; idx < a_rows * (GK / 8); idx += 128) {
            const int r = idx / (GK / 8), c = idx % (GK / 8);
            cp_async16(a + r * GLD + c * 8, A + (size_t)(row0 + r) * K + k0 + c * 8);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            bf16* b = sB + (stage * NB + nb) * GN * GLD;
            for (int idx = threadIdx.x; idx < b_rows * (GK / 8); idx += 128) {
                const int r = idx / (GK / 8), c = idx % (GK / 8);
                const int wrow = MODE == 0 ? gate_up_row(col0 + r, nb, N, interleaved) : col0 + r;
                cp_async16(b + r * GLD + c * 8, We + (size_t)wrow * K + k0 + c * 8);
            }
        }
    };
    float acc[NB][NT][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int j = 0; j < NT; ++j) { acc[nb][j][0] = acc[nb][j][1] = acc[nb][j][2] = acc[nb][j][3] = 0.0f; }
    const int nk = K / GK;
#pragma unroll
    for (int s = 0; s < G_STAGES - 1; ++s) {
        if (s < nk) load(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<G_STAGES - 2>();
        __syncthreads();                                       // stage kt is there, and everyone is done with stage kt - 1
        if (kt + G_STAGES - 1 < nk) load((kt + G_STAGES - 1) % G_STAGES, kt + G_STAGES - 1);
        cp_async_commit();
        const int stage = kt % G_STAGES;
        const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sA + stage * GMT * GLD + (warp_r * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * GLD + (lane >> 4) * 8);
#pragma unroll
        for (int kk = 0; kk < GK / 16; ++kk) {
            uint32_t a[4];
            ldsm_x4(a_addr + kk * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(sB + (stage * NB + nb) * GN * GLD + (warp_c * NT * 8 + (lane & 7) + (lane >> 4) * 8) * GLD + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(b_addr + (uint32_t)(j * 8 * GLD * 2 + kk * 32), b0, b1, b2, b3);
                    mma_bf16_16816(acc[nb][j], a, b0, b1);
                    mma_bf16_16816(acc[nb][j + 1], a, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    const int col = col0 + warp_c * NT * 8 + 2 * (lane & 3);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = row0 + warp_r * 16 + (lane >> 2) + 8 * rr;
        if (row >= row_end) continue;
        if (MODE == 0) {
            bf16* dst = act_out + (size_t)row * N;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int c = col + j * 8;
                if (c < N) {                                   // N is even: a pair of columns is inside or outside together
                    float g0 = acc[0][j][2 * rr], g1 = acc[0][j][2 * rr + 1];
                    float u0 = acc[NB - 1][j][2 * rr], u1 = acc[NB - 1][j][2 * rr + 1];
                    if (act_limit > 0.0f) {                    // capped inputs: g <- min(g, limit), u <- clamp(u, -limit, limit)
                        g0 = fminf(g0, act_limit); g1 = fminf(g1, act_limit);
                        u0 = fminf(fmaxf(u0, -act_limit), act_limit); u1 = fminf(fmaxf(u1, -act_limit), act_limit);
                    }
                    *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(g0 / (1.0f + __expf(-act_alpha * g0)) * (u0 + act_shift),
                                                                      g1 / (1.0f + __expf(-act_alpha * g1)) * (u1 + act_shift));
                }
            }
        } else if (MODE == 2) {
            bf16* dst = act_out + (size_t)row * N;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int c = col + j * 8;
                if (c < N) {
                    const float u0 = fmaxf(acc[0][j][2 * rr], 0.0f), u1 = fmaxf(acc[0][j][2 * rr + 1], 0.0f);
                    *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(u0 * u0, u1 * u1);
                }
            }
        } else {
            const size_t to = dst_rows != nullptr ? (size_t)dst_rows[row] : (size_t)row;
            const float f = row_scale != nullptr ? row_scale[row] : 1.0f;
            float* dst = f_out + to * N;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int c = col + j * 8;
                if (c < N) {
                    float2 v = make_float2(acc[0][j][2 * rr] * f, acc[0][j][2 * rr + 1] * f);
                    if (accumulate) { const float2 old = *reinterpret_cast<const float2*>(dst + c); v.x += old.x; v.y += old.y; }
                    *reinterpret_cast<float2*>(dst + c) = v;
                }
            }
        }
    }
}

// y[t][c] += sum over the token's choices, in choice order, of rows[inv[t top + choice]][c] (times the choice's weight, if given)
__global__ void moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ inv, const float* __restrict__ weight_of,
                                   float* __restrict__ y, int h, int top) {
    PDL_ENTER();
    rows = pdl_fresh(rows); inv = pdl_fresh(inv); y = pdl_fresh(y); weight_of = pdl_fresh(weight_of);
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < h; c += blockDim.x) {
        float a = y[(size_t)t * h + c];
        for (int k = 0; k < top; ++k) {
            const float v = rows[(size_t)inv[t * top + k] * h + c];
            a += weight_of != nullptr ? v * weight_of[t * top + k] : v;
        }
        y[(size_t)t * h + c] = a;
    }
}

#define G_SMEM(MODE, GMT) (G_STAGES_OF(MODE) * ((GMT) + G_NB_OF(MODE) * GN) * GLD * 2)

// Whether the tensor-core path takes these sizes: both inner sizes in whole steps of 64, rows 16-byte aligned.
MB_API int mb_moe_fast_supported(int h, int ff) { return h % GK == 0 && ff % GK == 0 && h % 8 == 0 && ff % 8 == 0; }

static int grouped_tiles(int pairs, int E, int gm) { return pairs / gm + E < pairs ? pairs / gm + E : pairs; }   // at most one partial tile per expert

// Pairs per tile: as few rows as the experts' shares need (the shares are not known on the host: their average decides).
static int grouped_rows(int pairs, int E) { return pairs <= 8 * E ? 16 : pairs <= 24 * E ? 32 : 64; }

template <int MODE, int GMT>
static int grouped_launch(const bf16* A, const bf16* W, const int* offsets, int E, int N, int K, bf16* act, float* out, const int* dst_rows,
                          const float* row_scale, int accumulate, int interleaved, int pairs, cudaStream_t s, float act_limit = 0.0f,
                          float act_alpha = 1.0f, float act_shift = 0.0f) {
    cudaFuncSetAttribute(moe_grouped_kernel<MODE, GMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM(MODE, GMT));
    return launch_kernel(moe_grouped_kernel<MODE, GMT>, dim3(grouped_tiles(pairs, E, GMT), (N + GN - 1) / GN), 128, G_SMEM(MODE, GMT), s, 0, A, W,
                         offsets, E, N, K, act, out, dst_rows, row_scale, accumulate, interleaved, act_limit, act_alpha, act_shift);
}

template <int MODE>
static int grouped_by_rows(const bf16* A, const bf16* W, const int* offsets, int E, int N, int K, bf16* act, float* out, const int* dst_rows,
                           const float* row_scale, int accumulate, int interleaved, int pairs, cudaStream_t s, float act_limit = 0.0f,
                           float act_alpha = 1.0f, float act_shift = 0.0f) {
    switch (grouped_rows(pairs, E)) {
        case 16: return grouped_launch<MODE, 16>(A, W, offsets, E, N, K, act, out, dst_rows, row_scale, accumulate, interleaved, pairs, s, act_limit, act_alpha, act_shift);
        case 32: return grouped_launch<MODE, 32>(A, W, offsets, E, N, K, act, out, dst_rows, row_scale, accumulate, interleaved, pairs, s, act_limit, act_alpha, act_shift);
    }
    return grouped_launch<MODE, 64>(A, W, offsets, E, N, K, act, out, dst_rows, row_scale, accumulate, interleaved, pairs, s, act_limit, act_alpha, act_shift);
}

// The pairs' inputs in expert order: xs bf16 [pairs][h], with each pair's token and weight beside it and where every pair went.
MB_API int mb_moe_gather(const void* h_rows, const int* order, const float* weight_of, void* xs, int* token_sorted, float* weight_sorted,
                         int* inv, int pairs, int h, int top, int weight_on_input, cudaStream_t s) {
    if (pairs <= 0) return 0;
    return launch_kernel(moe_gather_kernel<bf16>, pairs, 128, 0, s, 0, (const bf16*)h_rows, order, weight_of, (bf16*)xs, token_sorted,
                         weight_sorted, inv, h, top, weight_on_input);
}

// act bf16 [pairs][ff] = silu(gate xs) * (up xs), expert by expert; act_mode 1: relu(up xs)^2 with w_gate_up = [E][ff][h].
MB_API int mb_moe_grouped_gate_up(const void* xs, const void* w_gate_up, const int* offsets, void* act, int pairs, int h, int ff, int E,
                                  int interleaved, int act_mode, float act_limit, float act_alpha, float act_shift, cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (!mb_moe_fast_supported(h, ff) || E <= 0) return MB_ERR_BAD_SIZE;
    if (act_mode == 1)
        return grouped_by_rows<2>((const bf16*)xs, (const bf16*)w_gate_up, offsets, E, ff, h, (bf16*)act, nullptr, nullptr, nullptr, 0, 0, pairs, s);
    return grouped_by_rows<0>((const bf16*)xs, (const bf16*)w_gate_up, offsets, E, ff, h, (bf16*)act, nullptr, nullptr, nullptr, 0, interleaved,
                              pairs, s, act_limit, act_alpha, act_shift);
}

// out float32 = down act, expert by expert: row i goes to row dst_rows[i] of out (null: row i), times row_scale[i] (null: 1),
// added to what is there if `accumulate` (only where no two rows share a destination).
MB_API int mb_moe_grouped_down(const void* act, const void* w_down, const int* offsets, float* out, const int* dst_rows,
                               const float* row_scale, int accumulate, int pairs, int h, int ff, int E, cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (!mb_moe_fast_supported(h, ff) || E <= 0) return MB_ERR_BAD_SIZE;
    return grouped_by_rows<1>((const bf16*)act, (const bf16*)w_down, offsets, E, h, ff, nullptr, out, dst_rows, row_scale, accumulate, 0, pairs, s);
}

MB_API int mb_moe_combine(const float* rows, const int* inv, const float* weight_of, float* y, int tokens, int h, int top, cudaStream_t s) {
    if (tokens <= 0) return 0;
    return launch_kernel(moe_combine_kernel, tokens, 256, 0, s, 0, rows, inv, weight_of, y, h, top);
}
