// A selective state space (Mamba-2 form) and the short convolutions over time that feed it.
//
// channel_conv: y_t[c] = act(sum_j w[c, j] u_(t - taps + 1 + j)[c] + bias[c]) over each request's
// tokens, the taps - 1 rows before a step's first token from the request's state slot
// ([taps - 1, channels], row k = the input at position history - (taps - 1) + k, zero before the
// sequence's start), where the step's last rows are left afterwards. The inputs may be a slice of
// wider rows. Products and sums are 32-bit, inputs, state and outputs the compute dtype.
//
// state_space_scan: per token and head, with dt = softplus(raw + dt_bias) and
// a = exp(-exp(A_log) dt), S = a S + (dt B) x^T and y = S^T C + D x, S [N, P] 32-bit in the
// request's slot ([heads][N][P]); x [heads, P], B and C [groups, N] come from the convolution's
// output (compute dtype) and are used in 32-bit. A column of S depends on no other column: a
// block holds 32 columns of one head of one request, its four warps every fourth row of them in
// registers (a lane = a column, so the state moves 128 bytes at a time), and walks the request's
// tokens of the step in order, eight at a time, with B, C, the step sizes, the decays and the
// block's slice of x staged in shared memory (the next eight tokens' raw values are fetched into
// registers meanwhile). The four warps' shares of an
// output meet in shared memory in a fixed order, so a token's result does not depend on how the
// tokens were cut into steps.
//
// Long portions are cut into segments that run side by side (the recurrence is linear in S):
// every segment but the last first runs from a zero state and leaves what its tokens add and the
// product of its decays; a short pass chains the segments; then every segment runs from its
// incoming state and writes its outputs.
//
// gated_group_norm: y * silu(z), divided by its root mean square in `groups` equal parts, times a
// weight, all in 32-bit, stored in the compute dtype; a warp per (token, part).
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
// silu of a value that is stored in T next: for 16-bit storage the hardware's exponential and
// reciprocal (a few units in the last place of 32 bits, far inside the storage's rounding) in
// place of the exact ones, which are most of a streaming kernel's instructions
template <typename T>
__device__ __forceinline__ float silu_for(float z) {
    if (sizeof(T) == 2) return z * __frcp_rn(1.f + __expf(-z));
    return silu(z);
}
__device__ __forceinline__ float softplus(float z) { return z > 30.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ convolution over time

constexpr int CONV_THREADS = 256;

// portions: one thread per (token, channel); the state is read only
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
channel_conv_kernel(const T* __restrict__ rows, int ld, const float* __restrict__ kernel,
                    const float* __restrict__ bias, const T* __restrict__ state,
                    const int* __restrict__ slots, const int* __restrict__ token_request,
                    const int* __restrict__ request_start, const int* __restrict__ history,
                    T* __restrict__ out, int tokens, int channels, int taps, int activation) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (i >= (long long)tokens * channels) return;
    const int t = (int)(i / channels), c = (int)(i - (long long)t * channels);
    const int r = token_request[t];
    const int first = request_start[r];
    const int before = history[r];
    const float* w = kernel + (size_t)c * taps;
    float sum = bias != nullptr ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;            // how many tokens before t
        const int source = t - back;
        float u = 0.f;
        if (source >= first) {
            u = to_float<T>(rows[(size_t)source * ld + c]);
        } else if (state != nullptr) {
            // position before - (first - source): row taps - 1 - (first - source) of the slot
            const int row = taps - 1 - (first - source);
            if (row >= 0 && before - (first - source) >= 0)
                u = to_float<T>(state[((size_t)slots[r] * (taps - 1) + row) * channels + c]);
        }
        sum = fmaf(w[j], u, sum);
    }
    if (activation == 1) sum = silu_for<T>(sum);
    out[(size_t)t * channels + c] = from_float<T>(sum);
}

// The same, 16 bytes of channels a thread (8 bfloat16 or 4 float), for channel counts, row
// strides and addresses that allow it and up to 8 taps (WIDE_TAPS: 4 or 8, the code for the
// taps that are there). A block of 256 threads takes WIDE_GROUPS runs of channels and WIDE_TOKENS
// tokens: its weights come once, coalesced, through shared memory into registers; a thread takes
// every fourth token of the block's, and every tap of a token is one 16-byte load, all taps asked
// for before the first is used. (Eight tokens a thread, unrolled, ran no faster than one: the
// code no longer fitted the instruction cache, and every warp runs it once.)
constexpr int WIDE_GROUPS = 64;
constexpr int WIDE_THREADS = 4 * WIDE_GROUPS;
constexpr int WIDE_TOKENS = 16;

template <typename T, int WIDE_TAPS>
__global__ void __launch_bounds__(WIDE_THREADS)
channel_conv_wide_kernel(const T* __restrict__ rows, int ld, const float* __restrict__ kernel,
                         const float* __restrict__ bias, const T* __restrict__ state,
                         const int* __restrict__ slots, const int* __restrict__ token_request,
                         const int* __restrict__ request_start, const int* __restrict__ history,
                         T* __restrict__ out, int tokens, int channels, int taps, int activation) {
    constexpr int V = 16 / sizeof(T);
    // the block's weights come in one run of the stored [channels, taps] and are kept tap by tap
    __shared__ __align__(16) float staged[WIDE_TAPS][WIDE_GROUPS * V];
    griddep_launch();
    const int block_first = blockIdx.x * WIDE_GROUPS * V;
    const int block_channels = min(WIDE_GROUPS * V, channels - block_first);
    for (int i = threadIdx.x; i < block_channels * taps; i += WIDE_THREADS)
        staged[i % taps][i / taps] = kernel[(size_t)block_first * taps + i];
    __syncthreads();
    const int group = blockIdx.x * WIDE_GROUPS + (threadIdx.x % WIDE_GROUPS);
    if (group >= channels / V) return;
    const int c = group * V;
    float w[V][WIDE_TAPS], b[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        b[v] = bias != nullptr ? bias[c + v] : 0.f;
#pragma unroll
        for (int j = 0; j < WIDE_TAPS; ++j)
            w[v][j] = j < taps ? staged[j][(threadIdx.x % WIDE_GROUPS) * V + v] : 0.f;
    }
    griddep_wait();
#pragma unroll 1
    for (int k = threadIdx.x / WIDE_GROUPS; k < WIDE_TOKENS; k += WIDE_THREADS / WIDE_GROUPS) {
        const int t = blockIdx.y * WIDE_TOKENS + k;
        if (t >= tokens) break;
        const int r = token_request[t];
        const int first = request_start[r];
        const int before = history[r];
        float sum[V];
#pragma unroll
        for (int v = 0; v < V; ++v) sum[v] = b[v];
        // all taps' rows are asked for before any is used (a tap without a row reads the step's
        // first row and counts for nothing)
        uint4 tap[WIDE_TAPS];
        bool have[WIDE_TAPS];
#pragma unroll
        for (int j = 0; j < WIDE_TAPS; ++j) {
            have[j] = false;
            if (j >= taps) continue;
            const int source = t - (taps - 1 - j);
            const T* from = rows + c;
            if (source >= first) {
                from = rows + (size_t)source * ld + c;
                have[j] = true;
            } else if (state != nullptr) {
                const int row = taps - 1 - (first - source);
                if (row >= 0 && before - (first - source) >= 0) {
                    from = state + ((size_t)slots[r] * (taps - 1) + row) * channels + c;
                    have[j] = true;
                }
            }
            tap[j] = *reinterpret_cast<const uint4*>(from);
        }
#pragma unroll
        for (int j = 0; j < WIDE_TAPS; ++j) {
            if (j >= taps || !have[j]) continue;
            const T* u = reinterpret_cast<const T*>(&tap[j]);
#pragma unroll
            for (int v = 0; v < V; ++v) sum[v] = fmaf(w[v][j], to_float<T>(u[v]), sum[v]);
        }
        uint4 packed;
        T* y = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] = from_float<T>(activation == 1 ? silu_for<T>(sum[v]) : sum[v]);
        *reinterpret_cast<uint4*>(out + (size_t)t * channels + c) = packed;
    }
}

// after a step with portions: the slot's rows become the last taps - 1 inputs (one thread per
// (request, channel) moves its column of the slot, lowest row first)
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
channel_conv_state_kernel(const T* __restrict__ rows, int ld, T* __restrict__ state,
                          const int* __restrict__ slots, const int* __restrict__ request_start,
                          int requests, int channels, int taps) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (i >= (long long)requests * channels) return;
    const int r = (int)(i / channels), c = (int)(i - (long long)r * channels);
    const int first = request_start[r], count = request_start[r + 1] - first;
    if (count <= 0) return;
    T* slot = state + (size_t)slots[r] * (taps - 1) * channels + c;
    for (int k = 0; k < taps - 1; ++k) {
        const int source = count - (taps - 1) + k;        // index among the step's tokens
        slot[(size_t)k * channels] = source >= 0 ? rows[(size_t)(first + source) * ld + c]
                                                  : slot[(size_t)(k + count) * channels];
    }
}

// a step of single tokens: one thread per (request, channel) reads its column of the slot,
// writes the output and shifts the column
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
channel_conv_single_kernel(const T* __restrict__ rows, int ld, const float* __restrict__ kernel,
                           const float* __restrict__ bias, T* __restrict__ state,
                           const int* __restrict__ slots, const int* __restrict__ history,
                           T* __restrict__ out, int requests, int channels, int taps,
                           int activation, int write) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (i >= (long long)requests * channels) return;
    const int r = (int)(i / channels), c = (int)(i - (long long)r * channels);
    const float* w = kernel + (size_t)c * taps;
    const T mine = rows[(size_t)r * ld + c];
    float sum = bias != nullptr ? bias[c] : 0.f;
    sum = fmaf(w[taps - 1], to_float<T>(mine), sum);
    if (taps > 1) {
        T* slot = state + (size_t)slots[r] * (taps - 1) * channels + c;
        const int before = history[r];
        for (int k = 0; k < taps - 1; ++k) {
            const T kept = slot[(size_t)k * channels];
            if (before - (taps - 1) + k >= 0) sum = fmaf(w[k], to_float<T>(kept), sum);
            if (write && k > 0) slot[(size_t)(k - 1) * channels] = kept;
        }
        if (write) slot[(size_t)(taps - 2) * channels] = mine;
    }
    if (activation == 1) sum = silu_for<T>(sum);
    out[(size_t)r * channels + c] = from_float<T>(sum);
}

// ------------------------------------------------------------------ the recurrence

constexpr int COLS = 32;          // columns of S per block
constexpr int LANES = 4;          // warps that share a column's rows
constexpr int THREADS = COLS * LANES;
constexpr int TOK = 8;            // tokens staged at a time

struct ScanArgs {
    const void* mixed;            // [tokens, channels]: x | B | C
    const void* steps;            // [tokens, ld_steps]: raw dt per head
    int ld_steps;
    const float* a_log;           // [heads]
    const float* dt_bias;         // [heads]
    const float* skip;            // [heads]
    float* state;                 // [slots][heads][N][P]
    const int* slots;
    const int* request_start;
    float* y;                     // [tokens, heads * P]
    int heads, value_dim, state_dim, groups;
    int write;
    // segments (0: a request's tokens are one run from its state slot)
    int segment;
    float* carried;               // [requests][segments][heads][N][P]
    float* decayed;               // [requests][segments][heads]: product of the segment's decays
    int max_segments;
};

// MODE 0: from the slot through all tokens, outputs, the state written back.
// MODE 1: a segment from a zero state: what it adds goes to `carried`, the product of its decays
//         to `decayed` (no outputs; the last segment of a request does not run).
// MODE 2: a segment from its incoming state in `carried` (segment 0: the slot's state, which the
//         chaining pass has copied there); outputs; the last segment writes the slot.
template <typename T, int NR, int MODE>
__global__ void __launch_bounds__(THREADS, NR <= 32 ? 4 : 2)
state_space_scan_kernel(ScanArgs a) {
    constexpr int NPAD = LANES * NR;                 // rows covered (>= state_dim)
    __shared__ float sb[TOK][NPAD];
    __shared__ float sc[TOK][NPAD];
    __shared__ float sx[TOK][COLS];
    __shared__ float sdecay[TOK], sdt[TOK];
    __shared__ float partial[TOK][LANES][COLS];
    griddep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y;
    const int request = MODE == 0 ? blockIdx.z : blockIdx.z / a.max_segments;
    const int seg = MODE == 0 ? 0 : blockIdx.z % a.max_segments;
    const int P = a.value_dim, N = a.state_dim;
    const int column = blockIdx.x * COLS + lane;
    const bool live = column < P;
    const int group = head / (a.heads / a.groups);
    const int inner = a.heads * P;
    const int channels = inner + 2 * a.groups * N;
    const float rate = expf(a.a_log[head]);
    const float bias = a.dt_bias[head], through = a.skip[head];
    griddep_wait();
    int first = a.request_start[request], last = a.request_start[request + 1];
    int segments = 1;
    if (MODE != 0) {
        segments = (last - first + a.segment - 1) / a.segment;
        if (seg >= segments || (MODE == 1 && seg == segments - 1)) return;
        first += seg * a.segment;
        last = min(first + a.segment, last);
    }
    if (first >= last) return;
    const size_t matrix = (size_t)N * P;
    float* slot = a.state + ((size_t)a.slots[request] * a.heads + head) * matrix;
    float* mine = MODE == 0 ? nullptr
                            : a.carried + (((size_t)request * a.max_segments + seg) * a.heads + head) * matrix;
    float s[NR];
    {
        const float* from = MODE == 0 ? slot : mine;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = warp + LANES * i;
            s[i] = (MODE != 1 && live && n < N) ? from[(size_t)n * P + column] : 0.f;
        }
    }
    float product = 1.f;
    const T* mixed = reinterpret_cast<const T*>(a.mixed);
    const T* steps = reinterpret_cast<const T*>(a.steps);
    // MODE 1 (no outputs, few registers): the raw values of the next eight tokens wait in
    // registers while the present eight are worked on: this thread's share of B and C (PER values
    // each), of the block's slice of x (two values) and, for the first threads, a token's step
    // size. The other modes stage a group of tokens when they come to it: with the outputs' sums
    // in flight too, the registers that fetching ahead takes cost more warps than the wait.
    constexpr int PER = TOK * NPAD / THREADS;
    T rb[PER], rc[PER], rx[TOK * COLS / THREADS], rdt;
    auto fetch = [&](int base) {
        const int count = min(TOK, last - base);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * THREADS;
            const int t = i / NPAD, n = i - t * NPAD;
            const bool have = t < count && n < N;
            const T* row = mixed + (size_t)(base + (have ? t : 0)) * channels + inner + (size_t)group * N;
            rb[k] = have ? row[n] : from_float<T>(0.f);
            rc[k] = have ? row[(size_t)a.groups * N + n] : from_float<T>(0.f);
        }
#pragma unroll
        for (int k = 0; k < TOK * COLS / THREADS; ++k) {
            const int i = threadIdx.x + k * THREADS;
            const int t = i / COLS, c = i - t * COLS;
            const int col = blockIdx.x * COLS + c;
            const bool have = t < count && col < P;
            rx[k] = have ? mixed[(size_t)(base + t) * channels + (size_t)head * P + col] : from_float<T>(0.f);
        }
        rdt = threadIdx.x < count ? steps[(size_t)(base + threadIdx.x) * a.ld_steps + head]
                                  : from_float<T>(0.f);
    };
    if (MODE == 1) fetch(first);
    for (int base = first; base < last; base += TOK) {
        const int count = min(TOK, last - base);
        __syncthreads();           // everyone is done with the tokens staged before
        if (MODE != 1) fetch(base);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * THREADS;
            const int t = i / NPAD, n = i - t * NPAD;
            sb[t][n] = to_float<T>(rb[k]);
            sc[t][n] = to_float<T>(rc[k]);
        }
#pragma unroll
        for (int k = 0; k < TOK * COLS / THREADS; ++k) {
            const int i = threadIdx.x + k * THREADS;
            sx[i / COLS][i % COLS] = to_float<T>(rx[k]);
        }
        if (threadIdx.x < TOK) {
            const float dt = softplus(to_float<T>(rdt) + bias);
            sdecay[threadIdx.x] = expf(-rate * dt);
            sdt[threadIdx.x] = dt;
        }
        __syncthreads();
        if (MODE == 1 && base + TOK < last) fetch(base + TOK);
        for (int t = 0; t < count; ++t) {
            const float decay = sdecay[t], x = sx[t][lane];
            const float enters = sdt[t] * x;              // dt x: what B is multiplied with
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int n = warp + LANES * i;
                s[i] = fmaf(decay, s[i], sb[t][n] * enters);
                if (MODE != 1) sum = fmaf(s[i], sc[t][n], sum);
            }
            if (MODE != 1) partial[t][warp][lane] = sum;
            if (MODE == 1) product *= decay;
        }
        if (MODE != 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < count * COLS; i += THREADS) {
                const int t = i / COLS, c = i - t * COLS;
                const int col = blockIdx.x * COLS + c;
                if (col < P) {
                    const float sum = ((partial[t][0][c] + partial[t][1][c]) + partial[t][2][c]) +
                                      partial[t][3][c];
                    a.y[(size_t)(base + t) * inner + (size_t)head * P + col] = fmaf(through, sx[t][c], sum);
                }
            }
        }
    }
    if (MODE == 1) {
        if (blockIdx.x == 0 && threadIdx.x == 0)
            a.decayed[((size_t)request * a.max_segments + seg) * a.heads + head] = product;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = warp + LANES * i;
            if (live && n < N) mine[(size_t)n * P + column] = s[i];
        }
    } else if (a.write && (MODE == 0 || seg == segments - 1)) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = warp + LANES * i;
            if (live && n < N) slot[(size_t)n * P + column] = s[i];
        }
    }
}

// The chaining pass, one thread per element of S of a (request, head): carried[seg] holds what
// segment seg adds from a zero state; afterwards it holds the state that segment seg starts from:
// in(0) = the slot's state, in(s + 1) = decayed(s) in(s) + added(s).
__global__ void __launch_bounds__(256)
state_space_chain_kernel(ScanArgs a, int requests) {
    griddep_launch();
    griddep_wait();
    const size_t matrix = (size_t)a.state_dim * a.value_dim;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    const int head = blockIdx.y, request = blockIdx.z;
    if (i >= (long long)matrix) return;
    const int count = a.request_start[request + 1] - a.request_start[request];
    const int segments = (count + a.segment - 1) / a.segment;
    if (segments < 1) return;
    float incoming = a.state[((size_t)a.slots[request] * a.heads + head) * matrix + i];
    for (int seg = 0; seg < segments; ++seg) {
        const size_t at = (((size_t)request * a.max_segments + seg) * a.heads + head) * matrix + i;
        const float added = seg < segments - 1 ? a.carried[at] : 0.f;
        a.carried[at] = incoming;
        if (seg < segments - 1)
            incoming = fmaf(a.decayed[((size_t)request * a.max_segments + seg) * a.heads + head],
                            incoming, added);
    }
}

template <typename T, int NR>
int launch_scan(const ScanArgs& a, int requests, int max_portion, cudaStream_t stream) {
    const int tiles = ceil_div_host(a.value_dim, COLS);
    if (a.segment == 0) {
        cudaError_t e = launch_kernel(state_space_scan_kernel<T, NR, 0>, dim3(tiles, a.heads, requests),
                                      dim3(THREADS), 0, stream, true, a);
        MLXONE_REQUIRE(e == cudaSuccess, "state_space_scan: launch failed: %s", cudaGetErrorString(e));
        return 0;
    }
    const dim3 grid(tiles, a.heads, requests * a.max_segments);
    state_space_scan_kernel<T, NR, 1><<<grid, THREADS, 0, stream>>>(a);
    MLXONE_LAUNCH_CHECK("state_space_scan (build)");
    const size_t matrix = (size_t)a.state_dim * a.value_dim;
    state_space_chain_kernel<<<dim3(ceil_div_host(matrix, 256), a.heads, requests), 256, 0, stream>>>(a, requests);
    MLXONE_LAUNCH_CHECK("state_space_scan (chain)");
    state_space_scan_kernel<T, NR, 2><<<grid, THREADS, 0, stream>>>(a);
    MLXONE_LAUNCH_CHECK("state_space_scan (scan)");
    return 0;
}

template <typename T>
int dispatch_scan(const ScanArgs& a, int requests, int max_portion, cudaStream_t stream) {
    const int per_warp = (a.state_dim + LANES - 1) / LANES;
    if (per_warp <= 4) return launch_scan<T, 4>(a, requests, max_portion, stream);
    if (per_warp <= 8) return launch_scan<T, 8>(a, requests, max_portion, stream);
    if (per_warp <= 16) return launch_scan<T, 16>(a, requests, max_portion, stream);
    if (per_warp <= 32) return launch_scan<T, 32>(a, requests, max_portion, stream);
    return launch_scan<T, 64>(a, requests, max_portion, stream);
}

// ------------------------------------------------------------------ gate and grouped norm

constexpr int NORM_THREADS = 256;

// a block per (token, part), for steps of few tokens
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
gated_group_norm_block_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld,
                              const float* __restrict__ weight, T* __restrict__ out, int inner,
                              int groups, float eps) {
    __shared__ float scratch[33];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const int size = inner / groups;
    const float* row = y + (size_t)t * inner + (size_t)part * size;
    const T* z = gate + (size_t)t * ld + (size_t)part * size;
    float squares = 0.f;
    for (int c = threadIdx.x; c < size; c += NORM_THREADS) {
        const float v = row[c] * silu_for<T>(to_float<T>(z[c]));
        squares = fmaf(v, v, squares);
    }
    const float inverse = rsqrtf(block_sum(squares, scratch) / (float)size + eps);
    for (int c = threadIdx.x; c < size; c += NORM_THREADS) {
        const float v = row[c] * silu_for<T>(to_float<T>(z[c]));
        out[(size_t)t * inner + (size_t)part * size + c] =
            from_float<T>(v * inverse * weight[(size_t)part * size + c]);
    }
}

// a warp per (token, part): up to KEPT values a lane stay in registers between the sum of squares
// and the output (parts of up to 32 * KEPT values; longer parts are read twice)
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld,
                        const float* __restrict__ weight, T* __restrict__ out, int inner,
                        int groups, float eps, long long items) {
    constexpr int KEPT = 16;
    griddep_launch();
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (NORM_THREADS / 32) + (threadIdx.x >> 5);
    if (item >= items) return;
    const long long t = item / groups;
    const int part = (int)(item - t * groups);
    const int size = inner / groups;
    const float* row = y + (size_t)t * inner + (size_t)part * size;
    const T* z = gate + (size_t)t * ld + (size_t)part * size;
    float kept[KEPT];
    float squares = 0.f;
#pragma unroll
    for (int k = 0; k < KEPT; ++k) {
        const int c = lane + 32 * k;
        kept[k] = c < size ? row[c] * silu_for<T>(to_float<T>(z[c])) : 0.f;
        squares = fmaf(kept[k], kept[k], squares);
    }
    for (int c = lane + 32 * KEPT; c < size; c += 32) {
        const float v = row[c] * silu_for<T>(to_float<T>(z[c]));
        squares = fmaf(v, v, squares);
    }
    const float inverse = rsqrtf(warp_sum(squares) / (float)size + eps);
    T* to = out + (size_t)t * inner + (size_t)part * size;
    const float* w = weight + (size_t)part * size;
#pragma unroll
    for (int k = 0; k < KEPT; ++k) {
        const int c = lane + 32 * k;
        if (c < size) to[c] = from_float<T>(kept[k] * inverse * w[c]);
    }
    for (int c = lane + 32 * KEPT; c < size; c += 32)
        to[c] = from_float<T>(row[c] * silu_for<T>(to_float<T>(z[c])) * inverse * w[c]);
}

}  // namespace

// Segments of this many tokens when a request brings at least twice as many in a step.
constexpr int SEGMENT = 64;

MLXONE_API long long mlxone_state_space_scratch(int tokens, int requests, int max_portion,
                                                int heads, int value_dim, int state_dim) {
    if (max_portion < 2 * SEGMENT) return 1;
    const long long segments = (max_portion + SEGMENT - 1) / SEGMENT;
    return (long long)requests * segments * heads * ((long long)value_dim * state_dim + 1);
}

MLXONE_API int mlxone_channel_conv(const void* rows, int ld, const float* kernel, const float* bias,
                                   void* state, const int* slots, const int* token_request,
                                   const int* request_start, const int* history, void* out,
                                   int tokens, int requests, int channels, int taps, int activation,
                                   int single, int write, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(taps >= 1 && channels >= 1, "channel_conv: bad sizes");
    MLXONE_REQUIRE(taps == 1 || state != nullptr, "channel_conv: taps > 1 need a state");
    MLXONE_REQUIRE(activation == 0 || activation == 1, "channel_conv: unknown activation");
#define CONV_LAUNCH(T)                                                                             \
    do {                                                                                           \
        cudaError_t e;                                                                             \
        if (single) {                                                                              \
            e = launch_kernel(channel_conv_single_kernel<T>,                                       \
                              dim3(ceil_div_host((long long)requests * channels, CONV_THREADS)),   \
                              dim3(CONV_THREADS), 0, stream, true, (const T*)rows, ld, kernel,     \
                              bias, (T*)state, slots, history, (T*)out, requests, channels, taps,  \
                              activation, write);                                                  \
            MLXONE_REQUIRE(e == cudaSuccess, "channel_conv: launch failed: %s",                    \
                           cudaGetErrorString(e));                                                 \
        } else {                                                                                   \
            constexpr int V = 16 / sizeof(T);                                                      \
            const bool wide = channels % V == 0 && ld % V == 0 && (uintptr_t)rows % 16 == 0 &&     \
                              (uintptr_t)out % 16 == 0 && (uintptr_t)state % 16 == 0 &&            \
                              taps <= 8 && tokens <= 65535 * WIDE_TOKENS;                          \
            if (wide)                                                                              \
                e = launch_kernel(taps <= 4 ? channel_conv_wide_kernel<T, 4>                       \
                                            : channel_conv_wide_kernel<T, 8>,                      \
                                  dim3(ceil_div_host(channels / V, WIDE_GROUPS),                   \
                                       ceil_div_host(tokens, WIDE_TOKENS)),                        \
                                  dim3(WIDE_THREADS), 0, stream, true, (const T*)rows, ld, kernel, \
                                  bias, (const T*)state, slots, token_request, request_start,      \
                                  history, (T*)out, tokens, channels, taps, activation);           \
            else                                                                                   \
                e = launch_kernel(channel_conv_kernel<T>,                                          \
                              dim3(ceil_div_host((long long)tokens * channels, CONV_THREADS)),     \
                              dim3(CONV_THREADS), 0, stream, true, (const T*)rows, ld, kernel,     \
                              bias, (const T*)state, slots, token_request, request_start, history, \
                              (T*)out, tokens, channels, taps, activation);                        \
            MLXONE_REQUIRE(e == cudaSuccess, "channel_conv: launch failed: %s",                    \
                           cudaGetErrorString(e));                                                 \
            if (write && taps > 1) {                                                               \
                channel_conv_state_kernel<T>                                                       \
                    <<<ceil_div_host((long long)requests * channels, CONV_THREADS), CONV_THREADS,  \
                       0, stream>>>((const T*)rows, ld, (T*)state, slots, request_start, requests, \
                                    channels, taps);                                               \
                MLXONE_LAUNCH_CHECK("channel_conv (state)");                                       \
            }                                                                                      \
        }                                                                                          \
    } while (0)
    if (dtype == MLXONE_BF16) CONV_LAUNCH(__nv_bfloat16); else CONV_LAUNCH(float);
#undef CONV_LAUNCH
    return 0;
}

MLXONE_API int mlxone_state_space_scan(const void* mixed, const void* steps, int ld_steps,
                                       const float* a_log, const float* dt_bias, const float* skip,
                                       float* state, const int* slots, const int* request_start,
                                       float* scratch, float* y, int tokens, int requests,
                                       int max_portion, int heads, int value_dim, int state_dim,
                                       int groups, int write, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0,
                   "state_space_scan: %d heads cannot share %d groups", heads, groups);
    MLXONE_REQUIRE(state_dim >= 1 && state_dim <= 256, "state_space_scan: state size %d is not in 1..256",
                   state_dim);
    ScanArgs a{};
    a.mixed = mixed; a.steps = steps; a.ld_steps = ld_steps; a.a_log = a_log; a.dt_bias = dt_bias;
    a.skip = skip; a.state = state; a.slots = slots; a.request_start = request_start; a.y = y;
    a.heads = heads; a.value_dim = value_dim; a.state_dim = state_dim; a.groups = groups;
    a.write = write;
    if (max_portion >= 2 * SEGMENT) {
        a.segment = SEGMENT;
        a.max_segments = (max_portion + SEGMENT - 1) / SEGMENT;
        a.carried = scratch;
        a.decayed = scratch + (size_t)requests * a.max_segments * heads * value_dim * state_dim;
    }
    return dtype == MLXONE_BF16 ? dispatch_scan<__nv_bfloat16>(a, requests, max_portion, stream)
                                : dispatch_scan<float>(a, requests, max_portion, stream);
}

MLXONE_API int mlxone_gated_group_norm(const float* y, const void* gate, int ld, const float* weight,
                                       void* out, int tokens, int inner, int groups, float eps,
                                       int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(groups >= 1 && inner % groups == 0, "gated_group_norm: %d values in %d parts",
                   inner, groups);
    cudaError_t e;
    const long long items = (long long)tokens * groups;
    const dim3 grid(ceil_div_host(items, NORM_THREADS / 32));
    // few tokens: a block per part (the step is bound by latency, and 256 threads a part have the
    // shorter chain); many: a warp per part (no barriers, values kept in registers)
    if (items < 1024 && groups <= 65535) {
        if (dtype == MLXONE_BF16)
            e = launch_kernel(gated_group_norm_block_kernel<__nv_bfloat16>, dim3(tokens, groups),
                              dim3(NORM_THREADS), 0, stream, true, y, (const __nv_bfloat16*)gate, ld,
                              weight, (__nv_bfloat16*)out, inner, groups, eps);
        else
            e = launch_kernel(gated_group_norm_block_kernel<float>, dim3(tokens, groups),
                              dim3(NORM_THREADS), 0, stream, true, y, (const float*)gate, ld, weight,
                              (float*)out, inner, groups, eps);
    } else if (dtype == MLXONE_BF16)
        e = launch_kernel(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(NORM_THREADS), 0, stream,
                          true, y, (const __nv_bfloat16*)gate, ld, weight, (__nv_bfloat16*)out, inner,
                          groups, eps, items);
    else
        e = launch_kernel(gated_group_norm_kernel<float>, grid, dim3(NORM_THREADS), 0, stream, true, y,
                          (const float*)gate, ld, weight, (float*)out, inner, groups, eps, items);
    MLXONE_REQUIRE(e == cudaSuccess, "gated_group_norm: launch failed: %s", cudaGetErrorString(e));
    return 0;
}
