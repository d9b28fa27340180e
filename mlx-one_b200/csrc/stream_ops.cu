// Operations on the 32-bit residual stream and on activations that have no product in them:
// vectors added before a pass of a loop, activations of a dense feed-forward, and the mean of
// several mixers' outputs, each divided by its root mean square.
#include "common.cuh"

// ------------------------------------------------------------------ add vectors
// residual[t, :] += delta_scale * delta[t, :] (if delta) + table[ids[t], :] (if table) +
// vector[:] (if vector).
template <typename T>
__global__ void add_vectors_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const int* __restrict__ ids, const T* __restrict__ table,
                                   const float* __restrict__ vector, int hidden, int vocab,
                                   float delta_scale) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const T* row = nullptr;
    if (table != nullptr) {
        int id = ids[t];
        id = min(max(id, 0), vocab - 1);          // (the embedding kernel has reported a bad id)
        row = table + (size_t)id * hidden;
    }
    float* dst = residual + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = dst[c];
        if (delta != nullptr) v = fmaf(delta_scale, to_float<T>(delta[(size_t)t * hidden + c]), v);
        if (row != nullptr) v += to_float<T>(row[c]);
        if (vector != nullptr) v += vector[c];
        dst[c] = v;
    }
}

MLXONE_API int mlxone_add_vectors(float* residual, const void* delta, const int* ids,
                                  const void* table, const float* vector, int tokens, int hidden,
                                  int vocab, int dtype, float delta_scale, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0, "add_vectors: bad sizes");
    MLXONE_REQUIRE(table == nullptr || (ids != nullptr && vocab > 0), "add_vectors: a table needs ids");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(add_vectors_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, (const __nv_bfloat16*)delta, ids, (const __nv_bfloat16*)table, vector,
                      hidden, vocab, delta_scale);
    else
        launch_kernel(add_vectors_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, (const float*)delta, ids, (const float*)table, vector, hidden, vocab,
                      delta_scale);
    MLXONE_LAUNCH_CHECK("add_vectors");
    return 0;
}

// ------------------------------------------------------------------ stream beside embeddings
// out[t, :hidden] = T(residual[t, :] + delta_scale * delta[t, :]), out[t, hidden:] =
// table[ids[t], :]: the input of a product that mixes the stream with the tokens' embeddings.
template <typename T>
__global__ void concat_stream_kernel(const float* __restrict__ residual, const T* __restrict__ delta,
                                     const int* __restrict__ ids, const T* __restrict__ table,
                                     T* __restrict__ out, int hidden, int vocab, float delta_scale) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = min(max(id, 0), vocab - 1);          // (the embedding kernel has reported a bad id)
    const T* row = table + (size_t)id * hidden;
    const float* src = residual + (size_t)t * hidden;
    T* dst = out + (size_t)t * 2 * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = src[c];
        if (delta != nullptr) v = fmaf(delta_scale, to_float<T>(delta[(size_t)t * hidden + c]), v);
        dst[c] = from_float<T>(v);
        dst[hidden + c] = row[c];
    }
}

MLXONE_API int mlxone_concat_stream(const float* residual, const void* delta, const int* ids,
                                    const void* table, void* out, int tokens, int hidden, int vocab,
                                    int dtype, float delta_scale, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "concat_stream: bad sizes");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(concat_stream_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                      true, residual, (const __nv_bfloat16*)delta, ids, (const __nv_bfloat16*)table,
                      (__nv_bfloat16*)out, hidden, vocab, delta_scale);
    else
        launch_kernel(concat_stream_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, (const float*)delta, ids, (const float*)table, (float*)out, hidden,
                      vocab, delta_scale);
    MLXONE_LAUNCH_CHECK("concat_stream");
    return 0;
}

// ------------------------------------------------------------------ soft cap
// x = cap * tanh(x / cap), in place, 32-bit.
__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap, float inverse) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] * inverse);
}

MLXONE_API int mlxone_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total == 0) return 0;
    MLXONE_REQUIRE(total > 0 && cap > 0.f, "softcap: bad arguments");
    launch_kernel(softcap_kernel, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream, true, x,
                  total, cap, 1.f / cap);
    MLXONE_LAUNCH_CHECK("softcap");
    return 0;
}

// ------------------------------------------------------------------ a factor on 32-bit values
__global__ void scale_values_kernel(float* __restrict__ x, long long total, float factor) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] *= factor;
}

MLXONE_API int mlxone_scale_values(float* x, long long total, float factor, cudaStream_t stream) {
    if (total == 0) return 0;
    MLXONE_REQUIRE(total > 0, "scale_values: bad arguments");
    launch_kernel(scale_values_kernel, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream, true, x,
                  total, factor);
    MLXONE_LAUNCH_CHECK("scale_values");
    return 0;
}

// ------------------------------------------------------------------ gate with any activation
// out[t, f] = act(gate_up[t, f]) * gate_up[t, width + f], in 32-bit.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width,
                                        long long total, int kind) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / width;
    const int f = (int)(i - t * width);
    const float gate = to_float<T>(gate_up[t * 2 * width + f]);
    const float up = to_float<T>(gate_up[t * 2 * width + width + f]);
    out[i] = from_float<T>(mlxone_activate(gate, kind) * up);
}

MLXONE_API int mlxone_gated_activation(const void* gate_up, void* out, int rows, int width, int kind,
                                       int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && width > 0 && kind >= 0 && kind <= 3, "gated_activation: bad arguments");
    const long long total = (long long)rows * width;
    const int blocks = ceil_div_host(total, 256);
    if (dtype == MLXONE_BF16)
        launch_kernel(gated_activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true,
                      (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total, kind);
    else
        launch_kernel(gated_activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, true,
                      (const float*)gate_up, (float*)out, width, total, kind);
    MLXONE_LAUNCH_CHECK("gated_activation");
    return 0;
}

// ------------------------------------------------------------------ activations
// (mlxone_activate in common.cuh: relu2, gelu_tanh, silu, relu, xielu with its two numbers)
__device__ __forceinline__ float activate(float z, int kind, float a, float b) {
    return mlxone_activate(z, kind, a, b);
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, long long total,
                                  int kind, float a, float b) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(activate(to_float<T>(x[i]), kind, a, b));
}

// bfloat16, eight values a thread
__global__ void activation_wide_kernel(const __nv_bfloat16* __restrict__ x,
                                       __nv_bfloat16* __restrict__ out, long long groups, int kind,
                                       float a, float b) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 packed;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        q[k] = __floats2bfloat162_rn(activate(__low2float(in[k]), kind, a, b),
                                     activate(__high2float(in[k]), kind, a, b));
    *reinterpret_cast<uint4*>(out + i * 8) = packed;
}

// `a` and `b`: the two numbers of an activation that has some (xielu), else ignored.
MLXONE_API int mlxone_activation_shaped(const void* x, void* out, long long total, int kind,
                                        float a, float b, int dtype, cudaStream_t stream) {
    if (total == 0) return 0;
    MLXONE_REQUIRE(total > 0 && kind >= 0 && kind <= 4, "activation: bad arguments");
    if (dtype == MLXONE_BF16 && total % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0)
        launch_kernel(activation_wide_kernel, dim3(ceil_div_host(total / 8, 256)), dim3(256), 0,
                      stream, true, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, total / 8, kind,
                      a, b);
    else if (dtype == MLXONE_BF16)
        launch_kernel(activation_kernel<__nv_bfloat16>, dim3(ceil_div_host(total, 256)), dim3(256), 0,
                      stream, true, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, total, kind, a, b);
    else
        launch_kernel(activation_kernel<float>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const float*)x, (float*)out, total, kind, a, b);
    MLXONE_LAUNCH_CHECK("activation");
    return 0;
}

MLXONE_API int mlxone_activation(const void* x, void* out, long long total, int kind, int dtype,
                                 cudaStream_t stream) {
    MLXONE_REQUIRE(kind >= 0 && kind <= 3, "activation: bad arguments");
    return mlxone_activation_shaped(x, out, total, kind, 0.f, 0.f, dtype, stream);
}

// ------------------------------------------------------------------ mean of normed branches
// residual[t, :] += (1 / n) * sum_b x_b[t, :] * rsqrt(mean(x_b[t, :]^2) + eps) * weight_b[:],
// for n <= 4 branches, all in 32-bit. One block per token; the sums of squares are added in an
// order that the row length fixes.
constexpr int MAX_BRANCHES = 4;

template <typename T>
struct Branches {
    const T* x[MAX_BRANCHES];
    const float* weight[MAX_BRANCHES];
};

template <typename T>
__global__ void normed_mean_add_kernel(float* __restrict__ residual, Branches<T> branches, int count,
                                       int hidden, float eps) {
    __shared__ float scratch[33];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    float inv[MAX_BRANCHES];
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b) {
        inv[b] = 0.f;
        if (b >= count) continue;
        const T* row = branches.x[b] + (size_t)t * hidden;
        float sum = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = to_float<T>(row[c]);
            sum = fmaf(v, v, sum);
        }
        sum = block_sum(sum, scratch);
        inv[b] = rsqrtf(sum / (float)hidden + eps);
    }
    const float share = 1.f / (float)count;
    float* dst = residual + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float total = 0.f;
#pragma unroll
        for (int b = 0; b < MAX_BRANCHES; ++b)
            if (b < count)
                total += to_float<T>(branches.x[b][(size_t)t * hidden + c]) * inv[b] *
                         branches.weight[b][c];
        dst[c] += total * share;
    }
}

// Rows of a multiple of 8 values, 16-byte aligned, up to 8192: a thread keeps its 8 (or 16)
// values of every branch in registers between the sums of squares and the output, so every row
// is read once, 16 bytes a load, and the branches' sums share one reduction over the block.
template <typename T>
__device__ __forceinline__ void load8(const T* src, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* src, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* src, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(p[i]); v[2 * i + 1] = __high2float(p[i]); }
}

template <typename T, int COUNT, int ITER>
__global__ void __launch_bounds__(512)
normed_mean_add_rows_kernel(float* __restrict__ residual, Branches<T> branches, int hidden,
                            float eps) {
    __shared__ float partial[COUNT][16];
    __shared__ float inverse[COUNT];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float x[COUNT][ITER][8];
    float sum[COUNT];
#pragma unroll
    for (int b = 0; b < COUNT; ++b) {
        sum[b] = 0.f;
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 8;
            if (c < hidden) {
                load8<T>(branches.x[b] + (size_t)t * hidden + c, x[b][i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) sum[b] = fmaf(x[b][i][e], x[b][i][e], sum[b]);
            }
        }
        sum[b] = warp_sum(sum[b]);
        if (lane == 0) partial[b][warp] = sum[b];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int b = 0; b < COUNT; ++b) {
            float v = lane < warps ? partial[b][lane] : 0.f;
            v = warp_sum(v);
            if (lane == 0) inverse[b] = rsqrtf(v / (float)hidden + eps);
        }
    }
    __syncthreads();
    const float share = 1.f / (float)COUNT;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = (threadIdx.x + i * blockDim.x) * 8;
        if (c >= hidden) continue;
        float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < COUNT; ++b) {
            float w[8];
            load8<float>(branches.weight[b] + c, w);
            const float inv = inverse[b];
#pragma unroll
            for (int e = 0; e < 8; ++e) total[e] += x[b][i][e] * inv * w[e];
        }
        float4* dst = reinterpret_cast<float4*>(residual + (size_t)t * hidden + c);
        float4 lo = dst[0], hi = dst[1];
        lo.x += total[0] * share; lo.y += total[1] * share; lo.z += total[2] * share; lo.w += total[3] * share;
        hi.x += total[4] * share; hi.y += total[5] * share; hi.z += total[6] * share; hi.w += total[7] * share;
        dst[0] = lo;
        dst[1] = hi;
    }
}

template <typename T>
bool launch_normed_rows(float* residual, const Branches<T>& b, int count, int tokens, int hidden,
                        float eps, cudaStream_t stream) {
    bool aligned = hidden % 8 == 0 && hidden <= 8192 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0;
    for (int i = 0; i < count; ++i)
        aligned = aligned && (reinterpret_cast<uintptr_t>(b.x[i]) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(b.weight[i]) & 15) == 0;
    if (!aligned || count < 1 || count > 2) return false;
    const int groups = hidden / 8;
    const int iter = groups > 512 ? 2 : 1;
    const int threads = ((groups + iter - 1) / iter + 31) / 32 * 32;
#define ROWS_KERNEL(COUNT, ITER)                                                              \
    launch_kernel(normed_mean_add_rows_kernel<T, COUNT, ITER>, dim3(tokens), dim3(threads), 0, \
                  stream, true, residual, b, hidden, eps)
    if (count == 1 && iter == 1) ROWS_KERNEL(1, 1);
    else if (count == 1) ROWS_KERNEL(1, 2);
    else if (iter == 1) ROWS_KERNEL(2, 1);
    else ROWS_KERNEL(2, 2);
#undef ROWS_KERNEL
    return true;
}

MLXONE_API int mlxone_normed_mean_add(float* residual, const void* const* x,
                                      const float* const* weight, int count, int tokens, int hidden,
                                      float eps, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(count >= 1 && count <= MAX_BRANCHES, "normed_mean_add: 1 to %d branches, got %d",
                   MAX_BRANCHES, count);
    MLXONE_REQUIRE(tokens > 0 && hidden > 0, "normed_mean_add: bad sizes");
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == MLXONE_BF16) {
        Branches<__nv_bfloat16> b = {};
        for (int i = 0; i < count; ++i) { b.x[i] = (const __nv_bfloat16*)x[i]; b.weight[i] = weight[i]; }
        if (!launch_normed_rows<__nv_bfloat16>(residual, b, count, tokens, hidden, eps, stream))
        launch_kernel(normed_mean_add_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                      true, residual, b, count, hidden, eps);
    } else {
        Branches<float> b = {};
        for (int i = 0; i < count; ++i) { b.x[i] = (const float*)x[i]; b.weight[i] = weight[i]; }
        if (!launch_normed_rows<float>(residual, b, count, tokens, hidden, eps, stream))
        launch_kernel(normed_mean_add_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, b, count, hidden, eps);
    }
    MLXONE_LAUNCH_CHECK("normed_mean_add");
    return 0;
}
