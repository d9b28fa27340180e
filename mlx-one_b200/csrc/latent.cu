// Attention over one latent row per token, and attention with two score maps per head: the
// steps around the attention kernels.
//
// latent_prepare: from the fused input product of a latent-attention mixer to the queries'
// rotated parts and the token's row [latent | rotated shared key part] in its request's pages.
// sigmoid_gate: values * sigmoid(gate). differential_combine: o = a1 - mix * a2 per head, divided
// by its root mean square, times a factor.
#include "common.cuh"

namespace {

// One block per token. `projected` holds, per token, heads * (head_dim + rot_dim) query values
// (head by head, the rotated part last), then latent + rot_dim values of the down product, then
// whatever else the mixer projected. queries [tokens, heads, latent + rot_dim]: only the last
// rot_dim values of every head are written here (the first `latent` are another product's
// output). The page row [latent + rot_dim] gets the latent divided by its root mean square
// times `norm_weight`, and the rotated shared key part. Rotation: the first `rotary_dim` values
// of a rotated part; pair i is (2i, 2i + 1) if `neighbours`, else (i, i + rotary_dim / 2).
// Dynamic shared memory: rotary_dim floats (cosines and sines).
template <typename T>
__global__ void __launch_bounds__(512)
latent_prepare_kernel(const T* __restrict__ projected, int ld, T* __restrict__ queries,
                      const float* __restrict__ norm_weight, float eps,
                      const float* __restrict__ inv_freq, int rotary_dim, int neighbours,
                      const int* __restrict__ positions, const int* __restrict__ token_request,
                      T* __restrict__ pages, const int* __restrict__ block_table, int table_width,
                      int page_size, int heads, int head_dim, int rot_dim, int latent, int write,
                      int* __restrict__ error_flag) {
    extern __shared__ float shared[];
    __shared__ float scratch[33];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int position = positions[t];
    const int half = rotary_dim / 2;
    float* cosines = shared;
    float* sines = shared + half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float sine, cosine;
        sincosf((float)position * inv_freq[j], &sine, &cosine);
        sines[j] = sine;
        cosines[j] = cosine;
    }
    __syncthreads();
    const int per_head = head_dim + rot_dim;
    const int row = latent + rot_dim;
    const T* source = projected + (size_t)t * ld;
    // value e of a rotated part that starts at `part`
    auto rotated = [&](const T* part, int e) -> float {
        const float v = to_float<T>(part[e]);
        if (e >= rotary_dim) return v;
        int pair, other;
        bool first;
        if (neighbours) {
            pair = e >> 1; first = (e & 1) == 0; other = e ^ 1;
        } else {
            first = e < half; pair = first ? e : e - half; other = first ? e + half : e - half;
        }
        const float w = to_float<T>(part[other]);
        // (u, v) -> (u cos - v sin, v cos + u sin)
        return first ? v * cosines[pair] - w * sines[pair] : v * cosines[pair] + w * sines[pair];
    };
#pragma unroll 4
    for (int i = threadIdx.x; i < heads * rot_dim; i += blockDim.x) {
        const int head = i / rot_dim, e = i % rot_dim;
        queries[((size_t)t * heads + head) * row + latent + e] =
            from_float<T>(rotated(source + (size_t)head * per_head + head_dim, e));
    }
    if (!write) return;
    const int r = token_request[t];
    const int block = position / page_size;
    const int page = block < table_width ? block_table[(size_t)r * table_width + block] : -1;
    if (page < 0) {
        if (threadIdx.x == 0) atomicExch(error_flag, 2);
        return;
    }
    T* dst = pages + ((size_t)page * page_size + position % page_size) * row;
    const T* down = source + (size_t)heads * per_head;
    float squares = 0.f;
    for (int e = threadIdx.x; e < latent; e += blockDim.x) {
        const float v = to_float<T>(down[e]);
        squares = fmaf(v, v, squares);
    }
    squares = block_sum(squares, scratch);
    const float inv = rsqrtf(squares / (float)latent + eps);
    for (int e = threadIdx.x; e < latent; e += blockDim.x)
        dst[e] = from_float<T>(to_float<T>(down[e]) * inv * norm_weight[e]);
    for (int e = threadIdx.x; e < rot_dim; e += blockDim.x)
        dst[latent + e] = from_float<T>(rotated(down + latent, e));
}

// out[t, c] = values[t, c] * sigmoid(gate[t * ld_gate + c])
template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ values, const T* __restrict__ gate,
                                    int ld_gate, T* __restrict__ out, int width, long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / width;
    const int c = (int)(i % width);
    const float g = to_float<T>(gate[t * ld_gate + c]);
    out[i] = from_float<T>(to_float<T>(values[i]) / (1.f + expf(-g)));
}

// The same for bfloat16 rows whose width and strides are multiples of 8: 16 bytes per thread.
__global__ void sigmoid_gate_wide_kernel(const __nv_bfloat16* __restrict__ values,
                                         const __nv_bfloat16* __restrict__ gate, int ld_gate,
                                         __nv_bfloat16* __restrict__ out, int width,
                                         long long groups) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = width >> 3;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) << 3;
    const uint4 v = *reinterpret_cast<const uint4*>(values + t * width + c);
    const uint4 g = *reinterpret_cast<const uint4*>(gate + t * ld_gate + c);
    const __nv_bfloat162* vs = reinterpret_cast<const __nv_bfloat162*>(&v);
    const __nv_bfloat162* gs = reinterpret_cast<const __nv_bfloat162*>(&g);
    uint4 result;
    __nv_bfloat162* rs = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(vs[j]), b = __bfloat1622float2(gs[j]);
        rs[j] = __floats2bfloat162_rn(a.x / (1.f + expf(-b.x)), a.y / (1.f + expf(-b.y)));
    }
    *reinterpret_cast<uint4*>(out + t * width + c) = result;
}

// maps [tokens, 2 * heads, row_dim]: head h of map m is row m * heads + h, its first value_dim
// values count. out [tokens, heads * value_dim]: o = a1 - mix * a2, o * rsqrt(mean(o^2) + eps) *
// factor. One warp per (token, head).
constexpr int COMBINE_WARPS = 4;
constexpr int COMBINE_MAX = 512 / 32;

template <typename T>
__global__ void __launch_bounds__(COMBINE_WARPS * 32)
differential_combine_kernel(const T* __restrict__ maps, T* __restrict__ out, long long items,
                            int heads, int row_dim, int value_dim, float mix, float eps,
                            float factor) {
    griddep_launch();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * COMBINE_WARPS + warp;
    if (item >= items) return;
    const long long t = item / heads;
    const int head = (int)(item % heads);
    const T* first = maps + ((size_t)t * 2 * heads + head) * row_dim;
    const T* second = first + (size_t)heads * row_dim;
    float o[COMBINE_MAX];
    float squares = 0.f;
#pragma unroll
    for (int i = 0; i < COMBINE_MAX; ++i) {
        const int e = lane + 32 * i;
        o[i] = 0.f;
        if (e < value_dim) {
            o[i] = to_float<T>(first[e]) - mix * to_float<T>(second[e]);
            squares = fmaf(o[i], o[i], squares);
        }
    }
    squares = warp_sum(squares);
    const float inv = rsqrtf(squares / (float)value_dim + eps) * factor;
    T* dst = out + ((size_t)t * heads + head) * value_dim;
#pragma unroll
    for (int i = 0; i < COMBINE_MAX; ++i) {
        const int e = lane + 32 * i;
        if (e < value_dim) dst[e] = from_float<T>(o[i] * inv);
    }
}

// The heads' outputs times a sigmoid gate: values [tokens, heads, row_dim], of which the first
// value_dim of a row count, -> out [tokens, heads * value_dim]; the gate has one number per value
// (rows [heads * value_dim]) or, with `per_head`, one per head (rows [heads]); its rows may be a
// slice of wider rows.
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ values, const T* __restrict__ gate, int ld_gate,
                                  T* __restrict__ out, int heads, int row_dim, int value_dim,
                                  int per_head, long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int width = heads * value_dim;
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const int head = c / value_dim, e = c - head * value_dim;
    const float g = to_float<T>(gate[t * ld_gate + (per_head ? head : c)]);
    const float v = to_float<T>(values[(t * heads + head) * row_dim + e]);
    // (16-bit storage: the hardware's exponential and reciprocal, far inside its rounding)
    out[i] = from_float<T>(sizeof(T) == 2 ? v * __frcp_rn(1.f + __expf(-g)) : v / (1.f + expf(-g)));
}

}  // namespace

MLXONE_API int mlxone_latent_prepare(const void* projected, int ld, void* queries,
                                     const float* norm_weight, float eps, const float* inv_freq,
                                     int rotary_dim, int neighbours, const int* positions,
                                     const int* token_request, void* pages, const int* block_table,
                                     int table_width, int page_size, int tokens, int heads,
                                     int head_dim, int rot_dim, int latent, int write, int dtype,
                                     int* error_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && heads > 0 && head_dim >= 0 && rot_dim >= 0 && latent > 0,
                   "latent_prepare: bad sizes");
    MLXONE_REQUIRE(ld >= heads * (head_dim + rot_dim) + latent + rot_dim,
                   "latent_prepare: rows of %d values are too short", ld);
    if (inv_freq == nullptr) rotary_dim = 0;
    MLXONE_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot_dim,
                   "latent_prepare: %d rotated dimensions in a part of %d", rotary_dim, rot_dim);
    const size_t shared = (size_t)rotary_dim * sizeof(float);
    // (the block's size follows the model's sizes alone, so a token's sums never change order)
    const int most = heads * rot_dim > latent ? heads * rot_dim : latent;
    const int threads = most >= 2048 ? 512 : most >= 512 ? 256 : 128;
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(latent_prepare_kernel<T>, dim3(tokens), dim3(threads), shared, stream, true,
                      (const T*)projected, ld, (T*)queries, norm_weight, eps, inv_freq, rotary_dim,
                      neighbours, positions, token_request, (T*)pages, block_table, table_width,
                      page_size, heads, head_dim, rot_dim, latent, write, error_flag);
    } else {
        using T = float;
        launch_kernel(latent_prepare_kernel<T>, dim3(tokens), dim3(threads), shared, stream, true,
                      (const T*)projected, ld, (T*)queries, norm_weight, eps, inv_freq, rotary_dim,
                      neighbours, positions, token_request, (T*)pages, block_table, table_width,
                      page_size, heads, head_dim, rot_dim, latent, write, error_flag);
    }
    MLXONE_LAUNCH_CHECK("latent_prepare");
    return 0;
}

MLXONE_API int mlxone_sigmoid_gate(const void* values, const void* gate, int ld_gate, void* out,
                                   int rows, int width, int dtype, cudaStream_t stream) {
    if (rows == 0 || width == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && width > 0 && ld_gate >= width, "sigmoid_gate: bad sizes");
    const long long total = (long long)rows * width;
    const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (dtype == MLXONE_BF16 && width % 8 == 0 && ld_gate % 8 == 0 && aligned(values) &&
        aligned(gate) && aligned(out)) {
        using T = __nv_bfloat16;
        launch_kernel(sigmoid_gate_wide_kernel, dim3(ceil_div_host(total / 8, 256)), dim3(256), 0,
                      stream, true, (const T*)values, (const T*)gate, ld_gate, (T*)out, width,
                      total / 8);
    } else if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(sigmoid_gate_kernel<T>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const T*)values, (const T*)gate, ld_gate, (T*)out, width, total);
    } else {
        using T = float;
        launch_kernel(sigmoid_gate_kernel<T>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const T*)values, (const T*)gate, ld_gate, (T*)out, width, total);
    }
    MLXONE_LAUNCH_CHECK("sigmoid_gate");
    return 0;
}

MLXONE_API int mlxone_differential_combine(const void* maps, void* out, int tokens, int heads,
                                           int row_dim, int value_dim, float mix, float eps,
                                           float factor, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && heads > 0 && value_dim > 0 && value_dim <= row_dim &&
                       value_dim <= COMBINE_MAX * 32,
                   "differential_combine: values of %d in rows of %d", value_dim, row_dim);
    const long long items = (long long)tokens * heads;
    const dim3 grid(ceil_div_host(items, COMBINE_WARPS));
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(differential_combine_kernel<T>, grid, dim3(COMBINE_WARPS * 32), 0, stream,
                      true, (const T*)maps, (T*)out, items, heads, row_dim, value_dim, mix, eps,
                      factor);
    } else {
        using T = float;
        launch_kernel(differential_combine_kernel<T>, grid, dim3(COMBINE_WARPS * 32), 0, stream,
                      true, (const T*)maps, (T*)out, items, heads, row_dim, value_dim, mix, eps,
                      factor);
    }
    MLXONE_LAUNCH_CHECK("differential_combine");
    return 0;
}

MLXONE_API int mlxone_gate_heads(const void* values, const void* gate, int ld_gate, void* out,
                                 int tokens, int heads, int row_dim, int value_dim, int per_head,
                                 int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(heads > 0 && value_dim > 0 && value_dim <= row_dim,
                   "gate_heads: values of %d in rows of %d", value_dim, row_dim);
    const long long total = (long long)tokens * heads * value_dim;
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(gate_heads_kernel<T>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const T*)values, (const T*)gate, ld_gate, (T*)out, heads, row_dim,
                      value_dim, per_head, total);
    } else {
        using T = float;
        launch_kernel(gate_heads_kernel<T>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const T*)values, (const T*)gate, ld_gate, (T*)out, heads, row_dim,
                      value_dim, per_head, total);
    }
    MLXONE_LAUNCH_CHECK("gate_heads");
    return 0;
}
