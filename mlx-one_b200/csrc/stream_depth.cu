// The 32-bit stream of models that keep every layer's result: an embedding with a second table
// indexed by pairs of tokens, a causal convolution over time on what a sublayer reads, and the
// weighted sum of the streams kept so far.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ embedding with a pair table
// out[t, :] = table[ids[t], :] * scale + pairs[row(t), :], where row(t) = (previous * mul_prev +
// ids[t] * mul_cur) mod buckets and `previous` is the token before t in its request: ids[t - 1]
// within the step, else what the request's slot holds (token + 1; 0 = the sequence starts here,
// and the row is `buckets`). The block of a request's first token of the step is the only one
// that reads the slot; it then stores the request's last token of the step there.
template <typename T>
__global__ void embedding_pairs_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                       float scale, const T* __restrict__ pairs, int buckets,
                                       long long mul_prev, long long mul_cur,
                                       const int* __restrict__ token_request,
                                       const int* __restrict__ request_start,
                                       int* __restrict__ state, const int* __restrict__ slots,
                                       float* __restrict__ out, int hidden, int vocab,
                                       int* __restrict__ error_flag) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        id = 0;
    }
    const T* pair_row = nullptr;
    if (pairs != nullptr) {
        const int r = token_request[t];
        const int first = request_start[r];
        long long previous;
        if (t > first) {
            previous = ids[t - 1];
            if (previous < 0 || previous >= vocab) previous = 0;
        } else {
            int* slot = state + slots[r];
            previous = (long long)*slot - 1;
            __syncthreads();                       // every thread has read the slot
            if (threadIdx.x == 0) {
                int last = ids[request_start[r + 1] - 1];
                if (last < 0 || last >= vocab) last = 0;
                *slot = last + 1;
            }
        }
        const long long row = previous < 0 ? buckets : (previous * mul_prev + id * mul_cur) % buckets;
        pair_row = pairs + (size_t)row * hidden;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = to_float<T>(row[c]) * scale;
        if (pair_row != nullptr) v += to_float<T>(pair_row[c]);
        dst[c] = v;
    }
}

// ------------------------------------------------------------------ weighted sum of kept streams
// out[i] = sum_j weights[j] * kept[j * stride + i], j < count, added in that order; without
// weights a copy of kept[0]. `out` may be one of the streams beyond `count`.
template <int VEC>
__global__ void stream_average_kernel(const float* __restrict__ kept, long long stride,
                                      const float* __restrict__ weights, int count,
                                      float* __restrict__ out, long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= total) return;
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    if (weights == nullptr) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = kept[i + e];
    } else {
        for (int j = 0; j < count; ++j) {
            const float w = weights[j];
            const float* src = kept + j * stride + i;
            if (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
                acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
            } else {
                acc[0] = fmaf(w, src[0], acc[0]);
            }
        }
    }
    if (VEC == 4) {
        *reinterpret_cast<float4*>(out + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
        out[i] = acc[0];
    }
}

// ------------------------------------------------------------------ convolution over time
// out[t, c] = x[t, c] + sum_j w[c, j] * x[t - taps + 1 + j, c] over the tokens of t's request,
// with the taps - 1 rows before the step's first token taken from the request's slot
// (state[slot, k, c]: the row taps - 1 - k tokens before the step's first; zero before the
// sequence's start, because a fresh slot is zero). A thread owns one channel of a run of
// CONV_TOKENS tokens and carries the last taps - 1 inputs in registers. The thread of a
// request's first token of the step is the only one that reads the slot's channel; it then
// stores the last taps - 1 inputs of the step there.
constexpr int CONV_TOKENS = 16;
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(128)
stream_conv_kernel(const float* __restrict__ x, const float* __restrict__ kernel, int taps,
                   const int* __restrict__ token_request, const int* __restrict__ request_start,
                   float* __restrict__ state, long long slot_stride, const int* __restrict__ slots,
                   T* __restrict__ out, int tokens, int hidden, int write) {
    griddep_launch();
    griddep_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    const int t0 = blockIdx.y * CONV_TOKENS;
    const int t1 = min(t0 + CONV_TOKENS, tokens);
    const int before = taps - 1;
    float w[MAX_TAPS], window[MAX_TAPS];            // window[k]: the input before - k tokens back
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) w[j] = j < taps ? kernel[(size_t)c * taps + j] : 0.f;
    // The tokens that read a slot (the first taps - 1 of a request in this step) all belong to
    // the thread of the request's first token, also where they lie in the next run: no other
    // thread reads the slot's channel, which that thread overwrites. A thread therefore goes on
    // beyond its run only through early tokens of requests that start inside the run.
    int request = -1, last = -2;
    for (int t = t0; t < tokens; ++t) {
        const int r = token_request[t];
        const int first = request_start[r];
        const bool early = t - first < before;
        if (t < t1) {
            if (early && first < t0) continue;                   // the run before this one has it
        } else if (!(early && first >= t0 && first < t1)) {
            break;                       // (a request that starts in the next run is that run's)
        }
        if (r != request || t != last + 1) {
            request = r;
            float* slot = state != nullptr ? state + slots[r] * slot_stride + c : nullptr;
            // the inputs before token t: rows of this step, or of the slot
#pragma unroll
            for (int k = 0; k < MAX_TAPS; ++k) {
                if (k >= before) continue;
                const int source = t - before + k;
                window[k] = source >= first ? x[(size_t)source * hidden + c]
                                            : slot[(size_t)(before - (first - source)) * hidden];
            }
            if (t == first && write && slot != nullptr) {
                // what the next step finds: the last `before` inputs after this step's n tokens
                const int n = request_start[r + 1] - first;
#pragma unroll
                for (int k = 0; k < MAX_TAPS; ++k) {
                    if (k >= before) continue;
                    const int e = n - before + k;              // relative to the step's first token
                    // (e < 0: a row of the old slot, which `window` holds: row k + n)
                    float v = 0.f;
                    if (e >= 0) {
                        v = x[(size_t)(first + e) * hidden + c];
                    } else {
#pragma unroll
                        for (int q = 0; q < MAX_TAPS; ++q)
                            if (q == k + n) v = window[q];
                    }
                    slot[(size_t)k * hidden] = v;
                }
            }
        }
        last = t;
        const float now = x[(size_t)t * hidden + c];
        float acc = now;
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k)
            if (k < before) acc = fmaf(w[k], window[k], acc);
        acc = fmaf(w[before], now, acc);
        out[(size_t)t * hidden + c] = from_float<T>(acc);
#pragma unroll
        for (int k = 0; k < MAX_TAPS - 1; ++k)
            if (k < before - 1) window[k] = window[k + 1];
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k)
            if (k == before - 1) window[k] = now;
    }
}

template <typename T>
__global__ void stream_cast_kernel(const float* __restrict__ x, T* __restrict__ out, long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(x[i]);
}

}  // namespace

MLXONE_API int mlxone_embedding_pairs(const int* ids, const void* table, float scale,
                                      const void* pairs, int buckets, long long mul_prev,
                                      long long mul_cur, const int* token_request,
                                      const int* request_start, int* state, const int* slots,
                                      float* out, int tokens, int hidden, int vocab, int dtype,
                                      int* error_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding_pairs: bad sizes");
    MLXONE_REQUIRE(pairs == nullptr || (buckets > 0 && mul_prev >= 0 && mul_cur >= 0 &&
                                        state != nullptr && slots != nullptr),
                   "embedding_pairs: a pair table needs buckets, factors and the requests' slots");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(embedding_pairs_kernel<T>, dim3(tokens), dim3(threads), 0, stream, true, ids,
                      (const T*)table, scale, (const T*)pairs, buckets, mul_prev, mul_cur,
                      token_request, request_start, state, slots, out, hidden, vocab, error_flag);
    } else {
        using T = float;
        launch_kernel(embedding_pairs_kernel<T>, dim3(tokens), dim3(threads), 0, stream, true, ids,
                      (const T*)table, scale, (const T*)pairs, buckets, mul_prev, mul_cur,
                      token_request, request_start, state, slots, out, hidden, vocab, error_flag);
    }
    MLXONE_LAUNCH_CHECK("embedding_pairs");
    return 0;
}

MLXONE_API int mlxone_stream_average(const float* kept, long long stride, const float* weights,
                                     int count, float* out, long long total, cudaStream_t stream) {
    if (total == 0) return 0;
    MLXONE_REQUIRE(total > 0 && count >= 1 && stride >= total, "stream_average: bad sizes");
    const bool wide = total % 4 == 0 && stride % 4 == 0 &&
                      (reinterpret_cast<uintptr_t>(kept) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (wide)
        launch_kernel(stream_average_kernel<4>, dim3(ceil_div_host(total / 4, 256)), dim3(256), 0,
                      stream, true, kept, stride, weights, count, out, total);
    else
        launch_kernel(stream_average_kernel<1>, dim3(ceil_div_host(total, 256)), dim3(256), 0,
                      stream, true, kept, stride, weights, count, out, total);
    MLXONE_LAUNCH_CHECK("stream_average");
    return 0;
}

// `state` points at the sublayer's rows of slot 0 ([taps - 1, hidden]); slots lie `slot_stride`
// values apart. A null `kernel` only rounds the stream to the output type.
MLXONE_API int mlxone_stream_conv(const float* x, const float* kernel, int taps,
                                  const int* token_request, const int* request_start, float* state,
                                  long long slot_stride, const int* slots, void* out, int tokens,
                                  int hidden, int write, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0, "stream_conv: bad sizes");
    if (kernel == nullptr) {
        const long long total = (long long)tokens * hidden;
        if (dtype == MLXONE_BF16)
            launch_kernel(stream_cast_kernel<__nv_bfloat16>, dim3(ceil_div_host(total, 256)),
                          dim3(256), 0, stream, true, x, (__nv_bfloat16*)out, total);
        else
            launch_kernel(stream_cast_kernel<float>, dim3(ceil_div_host(total, 256)), dim3(256), 0,
                          stream, true, x, (float*)out, total);
        MLXONE_LAUNCH_CHECK("stream_cast");
        return 0;
    }
    MLXONE_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "stream_conv: 1 to %d taps, got %d", MAX_TAPS, taps);
    MLXONE_REQUIRE(taps == 1 || (state != nullptr && slots != nullptr),
                   "stream_conv: more than one tap needs the requests' slots");
    const dim3 grid(ceil_div_host(hidden, 128), ceil_div_host(tokens, CONV_TOKENS));
    MLXONE_REQUIRE(grid.y <= 65535, "stream_conv: too many tokens (%d)", tokens);
    if (dtype == MLXONE_BF16)
        launch_kernel(stream_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, x, kernel,
                      taps, token_request, request_start, state, slot_stride, slots,
                      (__nv_bfloat16*)out, tokens, hidden, write);
    else
        launch_kernel(stream_conv_kernel<float>, grid, dim3(128), 0, stream, true, x, kernel, taps,
                      token_request, request_start, state, slot_stride, slots, (float*)out, tokens,
                      hidden, write);
    MLXONE_LAUNCH_CHECK("stream_conv");
    return 0;
}
