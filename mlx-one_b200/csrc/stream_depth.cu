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
// sequence's start, because a fresh slot is zero). A thread owns VEC neighbouring channels of
// one token. A token with taps - 1 tokens of its request before it in the step reads rows of
// the step only. The first taps - 1 tokens of a request in the step belong to the thread of the
// first one: it is the only one that reads the slot's channels, and after the last read it
// stores the last taps - 1 inputs of the step there.
constexpr int MAX_TAPS = 16;

template <int VEC>
__device__ __forceinline__ void load_values(float (&v)[VEC], const float* p) {
    if constexpr (VEC == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = p[i];
    }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_values(T* p, const float (&v)[VEC]) {
    if constexpr (VEC == 4 && sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else if constexpr (VEC == 4 && sizeof(T) == 2) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = packed;
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) p[i] = from_float<T>(v[i]);
    }
}

// TAPS > 0: the number of taps is known when compiling, and a thread of four channels reads
// its TAPS x 4 weights (which lie side by side) 16 bytes at a time into registers.
template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(256)
stream_conv_kernel(const float* __restrict__ x, const float* __restrict__ kernel, int taps,
                   const int* __restrict__ token_request, const int* __restrict__ request_start,
                   float* state, long long slot_stride, const int* __restrict__ slots,
                   T* __restrict__ out, int tokens, int hidden, int write) {
    griddep_launch();
    griddep_wait();
    const int per_row = hidden / VEC;
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (long long)tokens * per_row) return;
    const int t = (int)(index / per_row);
    const int c = (int)(index - (long long)t * per_row) * VEC;
    const int r = token_request[t];
    const int first = request_start[r];
    const int before = taps - 1;
    const int place = t - first;
    if (place > 0 && place < before) return;        // the thread of the request's first token has it
    const float* w = kernel + (size_t)c * taps;     // channel c + v, tap j: w[v * taps + j]
    float now[VEC], acc[VEC], in[VEC];
    if constexpr (TAPS > 0 && VEC == 4) {
        if (place >= before) {
            float held[VEC * TAPS];
#pragma unroll
            for (int i = 0; i < TAPS; ++i) {
                const float4 four = reinterpret_cast<const float4*>(w)[i];
                held[4 * i] = four.x, held[4 * i + 1] = four.y;
                held[4 * i + 2] = four.z, held[4 * i + 3] = four.w;
            }
            load_values<VEC>(now, x + (size_t)t * hidden + c);
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = now[v];
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                load_values<VEC>(in, x + (size_t)(t - (TAPS - 1) + k) * hidden + c);
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] = fmaf(held[v * TAPS + k], in[v], acc[v]);
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(held[v * TAPS + TAPS - 1], now[v], acc[v]);
            store_values<T, VEC>(out + (size_t)t * hidden + c, acc);
            return;
        }
    }
    if (place >= before) {
        load_values<VEC>(now, x + (size_t)t * hidden + c);
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = now[v];
        for (int k = 0; k < before; ++k) {
            load_values<VEC>(in, x + (size_t)(t - before + k) * hidden + c);
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w[v * taps + k], in[v], acc[v]);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w[v * taps + before], now[v], acc[v]);
        store_values<T, VEC>(out + (size_t)t * hidden + c, acc);
        return;
    }
    // the request's first token of the step (and taps > 1): its first taps - 1 tokens, and the slot
    const int n = request_start[r + 1] - first;
    float* slot = state + slots[r] * slot_stride + c;
    const int early = min(n, before);
    for (int e = 0; e < early; ++e) {
        load_values<VEC>(now, x + (size_t)(first + e) * hidden + c);
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = now[v];
        for (int k = 0; k < before; ++k) {
            const int back = e - before + k;         // relative to the step's first token
            load_values<VEC>(in, back >= 0 ? x + (size_t)(first + back) * hidden + c
                                           : slot + (size_t)(before + back) * hidden);
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w[v * taps + k], in[v], acc[v]);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w[v * taps + before], now[v], acc[v]);
        store_values<T, VEC>(out + (size_t)(first + e) * hidden + c, acc);
    }
    if (write) {
        // what the next step finds: the last `before` inputs after this step's n tokens. Row k
        // takes a row of the step or, of a short step, the old row k + n, which lies behind
        // it and is still the old one while the rows are written in rising order.
        for (int k = 0; k < before; ++k) {
            const int e = n - before + k;
            load_values<VEC>(in, e >= 0 ? x + (size_t)(first + e) * hidden + c
                                        : slot + (size_t)(k + n) * hidden);
            store_values<float, VEC>(slot + (size_t)k * hidden, in);
        }
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
    const bool wide = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                      (state == nullptr || ((reinterpret_cast<uintptr_t>(state) & 15) == 0 &&
                                            slot_stride % 4 == 0));
    const long long threads = (long long)tokens * (wide ? hidden / 4 : hidden);
    const dim3 grid((unsigned)ceil_div_host(threads, 256));
#define MLXONE_STREAM_CONV(T, VEC, TAPS)                                                          \
    launch_kernel(stream_conv_kernel<T, VEC, TAPS>, grid, dim3(256), 0, stream, true, x, kernel,  \
                  taps, token_request, request_start, state, slot_stride, slots, (T*)out, tokens, \
                  hidden, write)
#define MLXONE_STREAM_CONV_WIDE(T)                                                                \
    switch ((reinterpret_cast<uintptr_t>(kernel) & 15) == 0 ? taps : 0) {                         \
        case 2: MLXONE_STREAM_CONV(T, 4, 2); break;                                               \
        case 3: MLXONE_STREAM_CONV(T, 4, 3); break;                                               \
        case 4: MLXONE_STREAM_CONV(T, 4, 4); break;                                               \
        case 5: MLXONE_STREAM_CONV(T, 4, 5); break;                                               \
        default: MLXONE_STREAM_CONV(T, 4, 0);                                                     \
    }
    if (dtype == MLXONE_BF16) {
        if (wide) MLXONE_STREAM_CONV_WIDE(__nv_bfloat16)
        else MLXONE_STREAM_CONV(__nv_bfloat16, 1, 0);
    } else {
        if (wide) MLXONE_STREAM_CONV_WIDE(float)
        else MLXONE_STREAM_CONV(float, 1, 0);
    }
#undef MLXONE_STREAM_CONV_WIDE
#undef MLXONE_STREAM_CONV
    MLXONE_LAUNCH_CHECK("stream_conv");
    return 0;
}
