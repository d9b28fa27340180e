// Routing of a mixture of experts, and the routing weights multiplied into the experts' columns
// of a stacked activation.
//
// Per token: logits z = W_r x in 32-bit (x may be in the compute dtype), scores s = sigmoid(z).
// The experts form `groups` equal runs of neighbours; a group's score is the sum of its
// `group_score` largest scores, and only experts of the `keep` best groups may be chosen. The
// `top` allowed experts with the largest scores are chosen (ties: the lower index) and weighted
// with s / (sum of the chosen s + 1e-20); all others get weight 0.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 512;
constexpr int ROUTE_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_experts_kernel(const T* __restrict__ x, int ld, const float* __restrict__ router,
                     float* __restrict__ weights, int hidden, int experts, int top, int groups,
                     int keep, int group_score) {
    __shared__ float score[MAX_EXPERTS];
    __shared__ float group_value[MAX_EXPERTS];
    __shared__ unsigned char allowed[MAX_EXPERTS];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* row = x + (size_t)t * ld;
    for (int e = threadIdx.x; e < experts; e += ROUTE_THREADS) allowed[e] = 0;
    // a warp per expert in turn; the lanes' partial sums are added in a fixed order
    for (int e = warp; e < experts; e += ROUTE_THREADS / 32) {
        const float* w = router + (size_t)e * hidden;
        float sum = 0.f;
        for (int c = lane; c < hidden; c += 32) sum = fmaf(to_float<T>(row[c]), w[c], sum);
        sum = warp_sum(sum);
        if (lane == 0) score[e] = 1.f / (1.f + expf(-sum));
    }
    __syncthreads();
    const int per = experts / groups;
    // a group's score: the sum of its largest `group_score` scores (one thread per group)
    for (int g = threadIdx.x; g < groups; g += ROUTE_THREADS) {
        float total = 0.f;
        unsigned long long taken_lo = 0ull;       // groups of up to 64 experts keep a mask;
        for (int pick = 0; pick < min(group_score, per); ++pick) {
            int best = -1;
            float best_value = -1.f;
            for (int i = 0; i < per; ++i) {
                const bool taken = per <= 64 ? ((taken_lo >> i) & 1ull) != 0ull
                                             : allowed[g * per + i] == 2;
                if (!taken && score[g * per + i] > best_value) { best_value = score[g * per + i]; best = i; }
            }
            if (best < 0) break;
            total += best_value;
            if (per <= 64) taken_lo |= 1ull << best; else allowed[g * per + best] = 2;
        }
        group_value[g] = total;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the `keep` best groups (ties: the lower index), then the `top` best allowed experts
        for (int e = 0; e < experts; ++e) allowed[e] = 0;
        for (int pick = 0; pick < keep; ++pick) {
            int best = -1;
            float best_value = -1.f;
            for (int g = 0; g < groups; ++g)
                if (group_value[g] > best_value) { best_value = group_value[g]; best = g; }
            if (best < 0) break;
            group_value[best] = -2.f;
            for (int i = 0; i < per; ++i) allowed[best * per + i] = 1;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += ROUTE_THREADS)
        weights[(size_t)t * experts + e] = 0.f;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        int chosen[64];
        int count = 0;
        for (int pick = 0; pick < top && pick < 64; ++pick) {
            int best = -1;
            float best_value = -1.f;
            for (int e = 0; e < experts; ++e)
                if (allowed[e] == 1 && score[e] > best_value) { best_value = score[e]; best = e; }
            if (best < 0) break;
            allowed[best] = 3;
            chosen[count++] = best;
            total += best_value;
        }
        const float inverse = 1.f / (total + 1e-20f);
        for (int i = 0; i < count; ++i)
            weights[(size_t)t * experts + chosen[i]] = score[chosen[i]] * inverse;
    }
}

// The second routing kernel: scores over all `outputs` of the router (sigmoid, or softmax over all
// of them), an optional correction per output that is added where the `top` best are chosen
// (ties: the lower index) and nowhere else, weights = the chosen outputs' scores, divided by their
// sum only with `normalize`. The first `experts` outputs are experts with tensors: their weights
// go to weights[t, experts]. The outputs behind them hand the token on as it is: the sum of their
// chosen weights goes to others[0][t]. With `shared_gate` the router has one more row behind its
// outputs, and others[1][t] = sigmoid of that row's product with the token.
// The logits are what a step of few tokens waits for: a warp a row of the router, sixteen warps a
// token, four values a lane and load (where the addresses allow) with four sums of their own, so
// that a row's loads are on their way together; the sums are added in a fixed order.
constexpr int GENERAL_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(GENERAL_THREADS)
route_general_kernel(const T* __restrict__ x, int ld, const float* __restrict__ router,
                     const float* __restrict__ correction, float* __restrict__ weights,
                     float* __restrict__ others, int tokens, int hidden, int experts, int outputs,
                     int top, int softmax, int normalize, int shared_gate, int wide) {
    __shared__ float score[MAX_EXPERTS + 1];
    __shared__ float choice[MAX_EXPERTS];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* row = x + (size_t)t * ld;
    const int rows = outputs + (shared_gate ? 1 : 0);
    for (int e = warp; e < rows; e += GENERAL_THREADS / 32) {
        const float* w = router + (size_t)e * hidden;
        float sum = 0.f;
        if (wide) {
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int c = lane * 4; c < hidden; c += 128) {
                const float4 weight = *reinterpret_cast<const float4*>(w + c);
                float value[4];
                if (sizeof(T) == 2) {
                    const uint2 packed = *reinterpret_cast<const uint2*>(row + c);
                    const T* four = reinterpret_cast<const T*>(&packed);
#pragma unroll
                    for (int k = 0; k < 4; ++k) value[k] = to_float<T>(four[k]);
                } else {
                    const float4 four = *reinterpret_cast<const float4*>(row + c);
                    value[0] = four.x; value[1] = four.y; value[2] = four.z; value[3] = four.w;
                }
                part[0] = fmaf(value[0], weight.x, part[0]);
                part[1] = fmaf(value[1], weight.y, part[1]);
                part[2] = fmaf(value[2], weight.z, part[2]);
                part[3] = fmaf(value[3], weight.w, part[3]);
            }
            sum = (part[0] + part[1]) + (part[2] + part[3]);
        } else {
            for (int c = lane; c < hidden; c += 32) sum = fmaf(to_float<T>(row[c]), w[c], sum);
        }
        sum = warp_sum(sum);
        if (lane == 0) score[e] = sum;
    }
    for (int e = threadIdx.x; e < experts; e += GENERAL_THREADS)
        weights[(size_t)t * experts + e] = 0.f;
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (softmax) {
        float most = -INFINITY, total = 0.f;
        for (int e = 0; e < outputs; ++e) most = fmaxf(most, score[e]);
        for (int e = 0; e < outputs; ++e) { score[e] = expf(score[e] - most); total += score[e]; }
        for (int e = 0; e < outputs; ++e) score[e] /= total;
    } else {
        for (int e = 0; e < outputs; ++e) score[e] = 1.f / (1.f + expf(-score[e]));
    }
    for (int e = 0; e < outputs; ++e)
        choice[e] = correction != nullptr ? score[e] + correction[e] : score[e];
    int chosen[64];
    int count = 0;
    float total = 0.f;
    for (int pick = 0; pick < top; ++pick) {
        int best = -1;
        float best_value = -INFINITY;
        for (int e = 0; e < outputs; ++e)
            if (choice[e] > best_value) { best_value = choice[e]; best = e; }
        if (best < 0) break;
        choice[best] = -INFINITY;
        chosen[count++] = best;
        total += score[best];
    }
    const float factor = normalize ? 1.f / (total + 1e-20f) : 1.f;
    float handed_on = 0.f;
    // (in ascending order of the outputs, so that the sum does not depend on the ranking)
    for (int e = experts; e < outputs; ++e)
        for (int i = 0; i < count; ++i)
            if (chosen[i] == e) handed_on += score[e] * factor;
    for (int i = 0; i < count; ++i)
        if (chosen[i] < experts) weights[(size_t)t * experts + chosen[i]] = score[chosen[i]] * factor;
    others[t] = handed_on;
    others[(size_t)tokens + t] = shared_gate ? 1.f / (1.f + expf(-score[outputs])) : 1.f;
}

// out[t, c] += factors[t] * x[t, c], taken in 32-bit
template <typename T>
__global__ void add_scaled_rows_kernel(T* __restrict__ out, const T* __restrict__ x, int ld,
                                       const float* __restrict__ factors, int hidden, long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / hidden;
    const int c = (int)(i - t * hidden);
    out[i] = from_float<T>(fmaf(factors[t], to_float<T>(x[t * ld + c]), to_float<T>(out[i])));
}

// x[t, e * width + f] *= weights[t, e] for e < experts; the `tail_width` columns behind them (a
// shared expert's) *= tail[t] (tail null: columns beyond experts * width stay).
template <typename T>
__global__ void scale_expert_columns_kernel(T* __restrict__ x, int ld, const float* __restrict__ weights,
                                            int experts, int width, long long total,
                                            const float* __restrict__ tail, int tail_width) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int across = experts * width + tail_width;
    const long long t = i / across;
    const int c = (int)(i - t * across);
    const float w = c < experts * width ? weights[t * experts + c / width] : tail[t];
    T* at = x + t * ld + c;
    *at = from_float<T>(to_float<T>(*at) * w);
}

// ------------------------------------------------------------------ tokens sorted by expert
// For the grouped products: every (token, chosen expert) pair gets a row in a buffer in which
// each expert's rows lie together and start on a multiple of 128 rows. One block.
//   pair_row[t, e]  the pair's row (-1: e was not chosen for t)
//   groups[tile]            {first row, first column} of the tile's expert in the stacked matrix
//                           of the first product: {expert * width, 0}; {-1, -1}: no rows
//   groups[tiles + tile]    the same for the second product: {0, expert * width}
// The order of an expert's rows is whatever the atomics make of it: a row's result does not
// depend on where it lies.
constexpr int SORT_THREADS = 1024;

__global__ void __launch_bounds__(SORT_THREADS)
sort_by_expert_kernel(const float* __restrict__ weights, int* __restrict__ pair_row,
                      int2* __restrict__ groups, int tokens, int experts, int width, int tiles) {
    __shared__ int count[MAX_EXPERTS];
    __shared__ int start[MAX_EXPERTS];
    griddep_launch();
    griddep_wait();
    for (int e = threadIdx.x; e < experts; e += SORT_THREADS) count[e] = 0;
    __syncthreads();
    const long long pairs = (long long)tokens * experts;
    for (long long i = threadIdx.x; i < pairs; i += SORT_THREADS)
        pair_row[i] = weights[i] > 0.f ? atomicAdd(&count[i % experts], 1) : -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = tile * 128;
            const int its = (count[e] + 127) / 128;
            for (int i = 0; i < its && tile < tiles; ++i, ++tile) {
                groups[tile] = make_int2(e * width, 0);
                groups[tiles + tile] = make_int2(0, e * width);
            }
        }
        for (; tile < tiles; ++tile) groups[tile] = groups[tiles + tile] = make_int2(-1, -1);
    }
    __syncthreads();
    for (long long i = threadIdx.x; i < pairs; i += SORT_THREADS)
        if (pair_row[i] >= 0) pair_row[i] += start[i % experts];
}

// sorted[pair_row[t, e], :] = x[t, :] for every chosen pair. One block per token; 16 bytes a
// copy where the rows allow it.
template <typename T>
__global__ void gather_by_expert_kernel(const T* __restrict__ x, int ld, const int* __restrict__ pair_row,
                                        T* __restrict__ sorted, int hidden, int experts) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    constexpr int PER = 16 / sizeof(T);
    const bool wide = hidden % PER == 0 && ld % PER == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(sorted) & 15) == 0;
    for (int e = 0; e < experts; ++e) {
        const int row = pair_row[(size_t)t * experts + e];
        if (row < 0) continue;
        const T* from = x + (size_t)t * ld;
        T* to = sorted + (size_t)row * hidden;
        if (wide) {
            for (int c = threadIdx.x * PER; c < hidden; c += blockDim.x * PER)
                *reinterpret_cast<uint4*>(to + c) = *reinterpret_cast<const uint4*>(from + c);
        } else {
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) to[c] = from[c];
        }
    }
}

// out[t, :] = sum over chosen e of weights[t, e] * y[pair_row[t, e], :] (+ shared[t, :]), in
// 32-bit, experts in ascending order. The token's pairs are looked up once, by one thread.
constexpr int MAX_TOP = 64;

template <typename T>
__global__ void combine_experts_kernel(const T* __restrict__ y, const int* __restrict__ pair_row,
                                       const float* __restrict__ weights, const T* __restrict__ shared_out,
                                       T* __restrict__ out, int hidden, int experts) {
    __shared__ int rows[MAX_TOP];
    __shared__ float factors[MAX_TOP];
    __shared__ int chosen;
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        int count = 0;
        for (int e = 0; e < experts && count < MAX_TOP; ++e) {
            const int row = pair_row[(size_t)t * experts + e];
            if (row >= 0) {
                rows[count] = row;
                factors[count++] = weights[(size_t)t * experts + e];
            }
        }
        chosen = count;
    }
    __syncthreads();
    const int count = chosen;
    constexpr int PER = 8 / sizeof(T);            // 4 bfloat16 or 2 floats a load
    const bool wide = hidden % PER == 0 && (reinterpret_cast<uintptr_t>(y) & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(shared_out) & 7) == 0;
    if (wide) {
        for (int c = threadIdx.x * PER; c < hidden; c += blockDim.x * PER) {
            float sum[PER];
            __align__(8) T piece[PER];
#pragma unroll
            for (int i = 0; i < PER; ++i) sum[i] = 0.f;
            if (shared_out != nullptr) {
                *reinterpret_cast<uint2*>(piece) =
                    *reinterpret_cast<const uint2*>(shared_out + (size_t)t * hidden + c);
#pragma unroll
                for (int i = 0; i < PER; ++i) sum[i] = to_float<T>(piece[i]);
            }
            for (int k = 0; k < count; ++k) {
                *reinterpret_cast<uint2*>(piece) =
                    *reinterpret_cast<const uint2*>(y + (size_t)rows[k] * hidden + c);
#pragma unroll
                for (int i = 0; i < PER; ++i) sum[i] = fmaf(factors[k], to_float<T>(piece[i]), sum[i]);
            }
#pragma unroll
            for (int i = 0; i < PER; ++i) piece[i] = from_float<T>(sum[i]);
            *reinterpret_cast<uint2*>(out + (size_t)t * hidden + c) = *reinterpret_cast<uint2*>(piece);
        }
        return;
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float sum = shared_out != nullptr ? to_float<T>(shared_out[(size_t)t * hidden + c]) : 0.f;
        for (int k = 0; k < count; ++k)
            sum = fmaf(factors[k], to_float<T>(y[(size_t)rows[k] * hidden + c]), sum);
        out[(size_t)t * hidden + c] = from_float<T>(sum);
    }
}

}  // namespace

MLXONE_API int mlxone_sort_by_expert(const float* weights, int* pair_row, int* groups, int tokens,
                                     int experts, int width, int tiles, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && experts > 0 && experts <= MAX_EXPERTS && tiles > 0,
                   "sort_by_expert: bad sizes");
    launch_kernel(sort_by_expert_kernel, dim3(1), dim3(SORT_THREADS), 0, stream, true, weights,
                  pair_row, reinterpret_cast<int2*>(groups), tokens, experts, width, tiles);
    MLXONE_LAUNCH_CHECK("sort_by_expert");
    return 0;
}

MLXONE_API int mlxone_gather_by_expert(const void* x, int ld, const int* pair_row, void* sorted,
                                       int tokens, int hidden, int experts, int dtype,
                                       cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && experts > 0, "gather_by_expert: bad sizes");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(gather_by_expert_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                      true, (const __nv_bfloat16*)x, ld, pair_row, (__nv_bfloat16*)sorted, hidden,
                      experts);
    else
        launch_kernel(gather_by_expert_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      (const float*)x, ld, pair_row, (float*)sorted, hidden, experts);
    MLXONE_LAUNCH_CHECK("gather_by_expert");
    return 0;
}

MLXONE_API int mlxone_combine_experts(const void* y, const int* pair_row, const float* weights,
                                      const void* shared_out, void* out, int tokens, int hidden,
                                      int experts, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && experts > 0, "combine_experts: bad sizes");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(combine_experts_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                      true, (const __nv_bfloat16*)y, pair_row, weights,
                      (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out, hidden, experts);
    else
        launch_kernel(combine_experts_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      (const float*)y, pair_row, weights, (const float*)shared_out, (float*)out,
                      hidden, experts);
    MLXONE_LAUNCH_CHECK("combine_experts");
    return 0;
}

MLXONE_API int mlxone_route_experts(const void* x, int ld, const float* router, float* weights,
                                    int tokens, int hidden, int experts, int top, int groups,
                                    int keep, int group_score, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && experts > 0 && experts <= MAX_EXPERTS,
                   "route_experts: 1 to %d experts", MAX_EXPERTS);
    MLXONE_REQUIRE(groups > 0 && experts % groups == 0 && keep > 0 && keep <= groups,
                   "route_experts: %d experts do not form %d groups of which %d are kept", experts,
                   groups, keep);
    MLXONE_REQUIRE(top > 0 && top <= 64 && top <= keep * (experts / groups) && group_score > 0,
                   "route_experts: top %d of %d allowed experts", top, keep * (experts / groups));
    if (dtype == MLXONE_BF16)
        launch_kernel(route_experts_kernel<__nv_bfloat16>, dim3(tokens), dim3(ROUTE_THREADS), 0,
                      stream, true, (const __nv_bfloat16*)x, ld, router, weights, hidden, experts, top,
                      groups, keep, group_score);
    else
        launch_kernel(route_experts_kernel<float>, dim3(tokens), dim3(ROUTE_THREADS), 0, stream, true,
                      (const float*)x, ld, router, weights, hidden, experts, top, groups, keep,
                      group_score);
    MLXONE_LAUNCH_CHECK("route_experts");
    return 0;
}

static int scale_expert_columns(void* x, int ld, const float* weights, int tokens, int experts,
                                int width, const float* tail, int tail_width, int dtype,
                                cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (tail == nullptr) tail_width = 0;
    MLXONE_REQUIRE(tokens > 0 && experts > 0 && width > 0 && tail_width >= 0 &&
                       ld >= experts * width + tail_width, "scale_expert_columns: bad sizes");
    const long long total = (long long)tokens * (experts * width + tail_width);
    const int blocks = ceil_div_host(total, 256);
    if (dtype == MLXONE_BF16)
        launch_kernel(scale_expert_columns_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                      true, (__nv_bfloat16*)x, ld, weights, experts, width, total, tail, tail_width);
    else
        launch_kernel(scale_expert_columns_kernel<float>, dim3(blocks), dim3(256), 0, stream, true,
                      (float*)x, ld, weights, experts, width, total, tail, tail_width);
    MLXONE_LAUNCH_CHECK("scale_expert_columns");
    return 0;
}

MLXONE_API int mlxone_scale_expert_columns(void* x, int ld, const float* weights, int tokens,
                                           int experts, int width, int dtype, cudaStream_t stream) {
    return scale_expert_columns(x, ld, weights, tokens, experts, width, nullptr, 0, dtype, stream);
}

// ... and the `tail_width` columns behind the experts' multiplied by tail[t]
MLXONE_API int mlxone_scale_expert_columns_tail(void* x, int ld, const float* weights, int tokens,
                                                int experts, int width, const float* tail,
                                                int tail_width, int dtype, cudaStream_t stream) {
    return scale_expert_columns(x, ld, weights, tokens, experts, width, tail, tail_width, dtype,
                                stream);
}

MLXONE_API int mlxone_route_general(const void* x, int ld, const float* router,
                                    const float* correction, float* weights, float* others,
                                    int tokens, int hidden, int experts, int identity, int top,
                                    int softmax, int normalize, int shared_gate, int dtype,
                                    cudaStream_t stream) {
    if (tokens == 0) return 0;
    const int outputs = experts + identity;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && experts > 0 && identity >= 0 && outputs <= MAX_EXPERTS,
                   "route_general: 1 to %d outputs of the router", MAX_EXPERTS);
    MLXONE_REQUIRE(top > 0 && top <= 64 && top <= outputs, "route_general: top %d of %d outputs", top,
                   outputs);
    // four values a load where rows start on 16 bytes (the router's) and on 4 values (the tokens')
    const size_t value = dtype == MLXONE_BF16 ? 2 : 4;
    const int wide = hidden % 4 == 0 && ld % 4 == 0 && (uintptr_t)x % (4 * value) == 0 &&
                     (uintptr_t)router % 16 == 0;
    if (dtype == MLXONE_BF16)
        launch_kernel(route_general_kernel<__nv_bfloat16>, dim3(tokens), dim3(GENERAL_THREADS), 0,
                      stream, true, (const __nv_bfloat16*)x, ld, router, correction, weights, others,
                      tokens, hidden, experts, outputs, top, softmax, normalize, shared_gate, wide);
    else
        launch_kernel(route_general_kernel<float>, dim3(tokens), dim3(GENERAL_THREADS), 0, stream,
                      true, (const float*)x, ld, router, correction, weights, others, tokens, hidden,
                      experts, outputs, top, softmax, normalize, shared_gate, wide);
    MLXONE_LAUNCH_CHECK("route_general");
    return 0;
}

MLXONE_API int mlxone_add_scaled_rows(void* out, const void* x, int ld, const float* factors,
                                      int tokens, int hidden, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    const long long total = (long long)tokens * hidden;
    if (dtype == MLXONE_BF16)
        launch_kernel(add_scaled_rows_kernel<__nv_bfloat16>, dim3(ceil_div_host(total, 256)),
                      dim3(256), 0, stream, true, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, ld,
                      factors, hidden, total);
    else
        launch_kernel(add_scaled_rows_kernel<float>, dim3(ceil_div_host(total, 256)), dim3(256), 0,
                      stream, true, (float*)out, (const float*)x, ld, factors, hidden, total);
    MLXONE_LAUNCH_CHECK("add_scaled_rows");
    return 0;
}
