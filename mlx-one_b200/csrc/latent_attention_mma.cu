// Attention over one latent row per token on tensor cores (bfloat16).
//
// A token keeps one row [latent | rotated key part] of R values in single-plane pages; the row
// is the key of every head and its first `latent` values are every head's value. A query row is
// a (token, head) pair; the rows of a request's portion are consecutive, token by token. So the
// heads of a token (and neighbouring tokens) share every key they read, and one block runs
// 16 * MT query rows against tiles of 64 keys that are copied asynchronously into shared memory
// (two buffers) while the tile before is in use.
//
// A block has 8 warps. For a tile, warp w computes the scores of keys 8w..8w+7 for all rows of
// the block (bfloat16 products, 32-bit sums) and leaves them, scaled and masked, in shared
// memory; after a barrier every warp reads the whole 16 MT x 64 scores, keeps the rows' running
// maximum and sum (32-bit; all warps hold the same numbers), rounds the weights to bfloat16 and
// multiplies them with its own columns of the latents: warp w owns the 8-column groups w, w + 8,
// ... of the output (up to 8 groups, so latents up to 512). The output's accumulators are 32-bit.
//
// Steps of single tokens cut every request's keys into `splits` runs of tiles that run side by
// side; each leaves (unnormalised output, maximum, sum) per row in scratch memory and a second
// kernel merges them.
//
// Sizes: R a multiple of 8 up to 576 (padded with zeros to a multiple of 16 in shared memory),
// latent a multiple of 8 up to 512. Anything else runs the general kernel.
#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int KEYS = 64;           // keys per tile
constexpr int WARPS = 8;
constexpr int GROUPS = 8;          // 8-column groups of the output per warp, at most
constexpr int SCORE_STRIDE = 72;   // floats per row of the scores in shared memory
constexpr int MAX_ROW = 576;
constexpr int MAX_LATENT = WARPS * GROUPS * 8;

__device__ __forceinline__ uint32_t shared_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void copy16(void* dst, const void* src, bool live) {
    const int bytes = live ? 16 : 0;          // 0 bytes read: the 16 bytes are filled with zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(shared_address(dst)),
                 "l"(src), "r"(bytes));
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copy_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(shared_address(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(shared_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(shared_address(p)));
}

// d += a (16x16, row) * b (16x8, col), bfloat16 in, float accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Copies keys first..first+63 of a request into a tile [64][stride]; rows beyond `last` or
// without a page are zero. A warp copies every eighth row, its lanes the row's 16-byte pieces.
__device__ __forceinline__ void load_keys(bf16* tile, int stride, const bf16* pages,
                                          const int* table, int table_width, int page_size,
                                          int row_size, int first, int last, int* error_flag) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = row_size >> 3;
    for (int row = warp; row < KEYS; row += WARPS) {
        const int key = first + row;
        bool live = key <= last;
        const bf16* source = pages;
        if (live) {
            const int block = key / page_size;
            const int page = block < table_width ? table[block] : -1;
            live = page >= 0;
            if (live) source = pages + ((size_t)page * page_size + (key - block * page_size)) * row_size;
            else if (lane == 0) atomicExch(error_flag, 3);
        }
        bf16* target = tile + row * stride;
        for (int chunk = lane; chunk < chunks; chunk += 32)
            copy16(target + chunk * 8, source + (live ? chunk * 8 : 0), live);
    }
}


constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Grid: (blocks of 16 MT rows over the longest portion, requests, splits). Dynamic shared
// memory: queries [16 MT][stride], keys 2 x [64][stride] (bfloat16, stride = R rounded up to 16,
// plus 8), scores [16 MT][72] floats. Scores are kept times log2(e), so weights are powers of 2.
// splits == 1: out [tokens, heads, R] gets its first `latent` values per row. Else partial
// [splits, total_rows, latent] and stats [splits, total_rows, 2] (maximum, sum) are written.
template <int MT>
__global__ void __launch_bounds__(WARPS * 32, 1)
latent_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages,
                        const int* __restrict__ block_table, int table_width, int page_size,
                        const int* __restrict__ positions, const int* __restrict__ request_start,
                        bf16* __restrict__ out, float* __restrict__ partial,
                        float* __restrict__ stats, int total_rows, int heads, int row_size,
                        int latent, float scale, int splits, int row_limit,
                        int* __restrict__ error_flag) {
    constexpr int ROWS = 16 * MT;
    extern __shared__ __align__(16) unsigned char raw[];
    const int request = blockIdx.y, split = blockIdx.z;
    const int start = request_start[request];
    const int rows = (request_start[request + 1] - start) * heads;
    const int row0 = blockIdx.x * ROWS;
    if (row0 >= rows || (row_limit > 0 && rows >= row_limit)) return;   // (the long kernel's)
    const int padded = (row_size + 15) & ~15;
    const int stride = padded + 8;
    bf16* q_tile = reinterpret_cast<bf16*>(raw);
    bf16* k_tiles[2] = {q_tile + ROWS * stride, q_tile + (ROWS + KEYS) * stride};
    float* scores = reinterpret_cast<float*>(q_tile + (ROWS + 2 * KEYS) * stride);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int history = positions[start];
    const int live_rows = min(ROWS, rows - row0);
    const int last_key = history + (row0 + live_rows - 1) / heads;
    const int tiles = last_key / KEYS + 1;
    const int per_split = (tiles + splits - 1) / splits;
    const int tile_first = split * per_split;
    const int tile_end = min(tiles, tile_first + per_split);
    const int* table = block_table + (size_t)request * table_width;
    const size_t first_row = (size_t)start * heads + row0;        // among all rows of the step

    // columns between R and its multiple of 16 are zero in every tile (nothing copies there)
    if (padded != row_size) {
        const int extra = padded - row_size;
        for (int i = threadIdx.x; i < (ROWS + 2 * KEYS) * extra; i += WARPS * 32)
            q_tile[(i / extra) * stride + row_size + i % extra] = __float2bfloat16_rn(0.f);
    }
    // Rows of earlier steps are in the pages whatever runs ahead of this kernel in the stream:
    // a first tile that holds only such rows is asked for before waiting for that kernel.
    const bool settled = tile_first * KEYS + KEYS <= history;
    if (tile_first < tile_end && settled)
        load_keys(k_tiles[0], stride, pages, table, table_width, page_size, row_size,
                  tile_first * KEYS, last_key, error_flag);
    griddep_wait();
    if (tile_first < tile_end && !settled)
        load_keys(k_tiles[0], stride, pages, table, table_width, page_size, row_size,
                  tile_first * KEYS, last_key, error_flag);
    {
        const int chunks = row_size >> 3;
        for (int piece = threadIdx.x; piece < ROWS * chunks; piece += WARPS * 32) {
            const int row = piece / chunks, chunk = piece - row * chunks;
            const bool live = row < live_rows;
            copy16(q_tile + row * stride + chunk * 8,
                   q + (live ? (first_row + row) * row_size + chunk * 8 : 0), live);
        }
    }
    copy_commit();

    // the positions of this thread's rows (g and g + 8 of every 16)
    int position[MT][2];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        position[m][0] = history + (row0 + m * 16 + g) / heads;
        position[m][1] = history + (row0 + m * 16 + g + 8) / heads;
    }
    float o[MT][GROUPS][4];
    float peak[MT][2], total[MT][2];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        peak[m][0] = peak[m][1] = -INFINITY;
        total[m][0] = total[m][1] = 0.f;
#pragma unroll
        for (int j = 0; j < GROUPS; ++j) o[m][j][0] = o[m][j][1] = o[m][j][2] = o[m][j][3] = 0.f;
    }
    const float factor = scale * LOG2E;

    for (int tile = tile_first; tile < tile_end; ++tile) {
        const bf16* keys = k_tiles[(tile - tile_first) & 1];
        copy_wait<0>();
        __syncthreads();
        if (tile + 1 < tile_end)
            load_keys(k_tiles[(tile + 1 - tile_first) & 1], stride, pages, table, table_width,
                      page_size, row_size, (tile + 1) * KEYS, last_key, error_flag);
        copy_commit();

        // ---- scores of this warp's 8 keys for all rows
        float s[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) s[m][0] = s[m][1] = s[m][2] = s[m][3] = 0.f;
        const bf16* key_rows = keys + (warp * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8;
        const bf16* query_rows = q_tile + (lane & 15) * stride + (lane >> 4) * 8;
        // (the next step's operands are asked for before this step's products are issued)
        {
            uint32_t b[2], a[MT][4];
            ldmatrix_x2(b, key_rows);
#pragma unroll
            for (int m = 0; m < MT; ++m) ldmatrix_x4(a[m], query_rows + m * 16 * stride);
#pragma unroll 4
            for (int k0 = 0; k0 < padded; k0 += 16) {
                uint32_t nb[2] = {b[0], b[1]}, na[MT][4];
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int i = 0; i < 4; ++i) na[m][i] = a[m][i];
                if (k0 + 16 < padded) {
                    ldmatrix_x2(nb, key_rows + k0 + 16);
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        ldmatrix_x4(na[m], query_rows + m * 16 * stride + k0 + 16);
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) mma_16816(s[m], a[m], b[0], b[1]);
                b[0] = nb[0], b[1] = nb[1];
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[m][i] = na[m][i];
            }
        }
        const int key0 = tile * KEYS + warp * 8 + 2 * t;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int limit = position[m][half];
                float2 v;
                v.x = key0 <= limit ? s[m][2 * half] * factor : -INFINITY;
                v.y = key0 + 1 <= limit ? s[m][2 * half + 1] * factor : -INFINITY;
                *reinterpret_cast<float2*>(scores + (m * 16 + g + 8 * half) * SCORE_STRIDE +
                                           warp * 8 + 2 * t) = v;
            }
        }
        __syncthreads();

        // ---- every warp: the rows' maximum and sum over the 64 keys, weights in bfloat16
        uint32_t p[MT][4][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float* row = scores + (m * 16 + g + 8 * half) * SCORE_STRIDE + 2 * t;
                float2 x[4][2];
                float highest = -INFINITY;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    x[kk][0] = *reinterpret_cast<const float2*>(row + 16 * kk);
                    x[kk][1] = *reinterpret_cast<const float2*>(row + 16 * kk + 8);
                    highest = fmaxf(highest, fmaxf(fmaxf(x[kk][0].x, x[kk][0].y),
                                                   fmaxf(x[kk][1].x, x[kk][1].y)));
                }
                highest = fmaxf(quad_max(highest), peak[m][half]);
                const float base = highest == -INFINITY ? 0.f : highest;
                const float shrink = exp2f(peak[m][half] - base);
                peak[m][half] = highest;
                float sum = 0.f;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                    for (int side = 0; side < 2; ++side) {
                        const float a = exp2f(x[kk][side].x - base), b = exp2f(x[kk][side].y - base);
                        sum += a + b;
                        p[m][kk][half + 2 * side] = pack_bf16(a, b);
                    }
                }
                total[m][half] = total[m][half] * shrink + quad_sum(sum);
#pragma unroll
                for (int j = 0; j < GROUPS; ++j) {
                    o[m][j][2 * half] *= shrink;
                    o[m][j][2 * half + 1] *= shrink;
                }
            }
        }

        // ---- this warp's columns of the output
        {
            uint32_t b[4] = {0u, 0u, 0u, 0u};
            if (warp * 8 < latent) ldmatrix_x4_trans(b, keys + lane * stride + warp * 8);
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const int column = (warp + WARPS * j) * 8;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t nb[4] = {b[0], b[1], b[2], b[3]};
                    const int next_column = half == 0 ? column : column + WARPS * 8;
                    if ((half == 0 || j + 1 < GROUPS) && next_column < latent)
                        ldmatrix_x4_trans(nb, keys + (32 * (1 - half) + lane) * stride + next_column);
                    if (column < latent) {
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            mma_16816(o[m][j], p[m][2 * half], b[0], b[1]);
                            mma_16816(o[m][j], p[m][2 * half + 1], b[2], b[3]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) b[i] = nb[i];
                }
            }
        }
    }
    copy_wait<0>();

    // ---- results
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = m * 16 + g + 8 * half;
            if (row >= live_rows) continue;
            const size_t global_row = first_row + row;
            if (splits == 1) {
                const float inverse = total[m][half] > 0.f ? 1.f / total[m][half] : 0.f;
#pragma unroll
                for (int j = 0; j < GROUPS; ++j) {
                    const int column = (warp + WARPS * j) * 8 + 2 * t;
                    if (column < latent)
                        *reinterpret_cast<uint32_t*>(out + global_row * row_size + column) =
                            pack_bf16(o[m][j][2 * half] * inverse, o[m][j][2 * half + 1] * inverse);
                }
            } else {
                const size_t at = (size_t)split * total_rows + global_row;
#pragma unroll
                for (int j = 0; j < GROUPS; ++j) {
                    const int column = (warp + WARPS * j) * 8 + 2 * t;
                    if (column < latent)
                        *reinterpret_cast<float2*>(partial + at * latent + column) =
                            make_float2(o[m][j][2 * half], o[m][j][2 * half + 1]);
                }
                if (warp == 0 && t == 0) {
                    stats[2 * at] = peak[m][half];
                    stats[2 * at + 1] = total[m][half];
                }
            }
        }
    }
}

// ---- portions of many rows
// A warp owns 16 query rows for the whole pass over the keys, as flash attention does: their
// scores of a tile of 64 keys stay in registers (8 accumulators of 16 x 8), the rows' maximum
// and sum are kept by the four lanes that hold a row, the weights go from the scores'
// accumulators straight into the operand of the second product, and the warp accumulates its
// rows' output columns in registers. No scores pass through shared memory and the block meets
// only once per tile, where the key buffers change hands.
//
// An output of 16 x 256 fills 128 registers, so wider latents are split between C = 2 warps
// that own the same 16 rows and one half of the columns each; both compute the rows' scores.
// A block has 8 warps: 128 / C rows. Shared memory: queries [128 / C][stride], keys
// 2 x [64][stride]. Requests with fewer than LONG_ROWS rows in the step are left to the kernel
// above (they would keep one warp busy and seven idle).
constexpr int LONG_TILES = 32;     // 8-column groups of the output per warp
constexpr int LONG_ROWS = 64;      // a request's rows from which this kernel takes it
constexpr size_t MAX_SHARED = 227 * 1024;   // what a block may ask for

template <int C>
__global__ void __launch_bounds__(WARPS * 32, 1)
latent_attention_long_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages,
                             const int* __restrict__ block_table, int table_width, int page_size,
                             const int* __restrict__ positions,
                             const int* __restrict__ request_start, bf16* __restrict__ out,
                             int heads, int row_size, int latent, float scale,
                             int* __restrict__ error_flag) {
    constexpr int ROWS = 16 * (WARPS / C);
    extern __shared__ __align__(16) unsigned char raw[];
    const int request = blockIdx.y;
    const int start = request_start[request];
    const int rows = (request_start[request + 1] - start) * heads;
    // (the blocks with the most keys first)
    const int row0 = (gridDim.x - 1 - blockIdx.x) * ROWS;
    if (row0 >= rows || rows < LONG_ROWS) return;
    const int padded = (row_size + 15) & ~15;
    const int stride = padded + 8;
    bf16* q_tile = reinterpret_cast<bf16*>(raw);
    bf16* k_tiles[2] = {q_tile + ROWS * stride, q_tile + (ROWS + KEYS) * stride};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = warp / C, side = warp % C;          // rows 16 group .., columns 256 side ..
    const int history = positions[start];
    const int live_rows = min(ROWS, rows - row0);
    const int last_key = history + (row0 + live_rows - 1) / heads;
    const int tiles = last_key / KEYS + 1;
    const int* table = block_table + (size_t)request * table_width;
    const size_t first_row = (size_t)start * heads + row0;

    if (padded != row_size) {
        const int extra = padded - row_size;
        for (int i = threadIdx.x; i < (ROWS + 2 * KEYS) * extra; i += WARPS * 32)
            q_tile[(i / extra) * stride + row_size + i % extra] = __float2bfloat16_rn(0.f);
    }
    {
        const int chunks = row_size >> 3;
        for (int piece = threadIdx.x; piece < ROWS * chunks; piece += WARPS * 32) {
            const int row = piece / chunks, chunk = piece - row * chunks;
            const bool live = row < live_rows;
            copy16(q_tile + row * stride + chunk * 8,
                   q + (live ? (first_row + row) * row_size + chunk * 8 : 0), live);
        }
    }
    load_keys(k_tiles[0], stride, pages, table, table_width, page_size, row_size, 0, last_key,
              error_flag);
    copy_commit();

    int position[2];
    position[0] = history + (row0 + group * 16 + g) / heads;
    position[1] = history + (row0 + group * 16 + g + 8) / heads;
    // (a warp whose rows all lie beyond the portion still meets the others at the barriers)
    const int warp_last = history + min(row0 + group * 16 + 15, rows - 1) / heads;
    const bool idle = group * 16 >= live_rows;
    float o[LONG_TILES][4];
#pragma unroll
    for (int j = 0; j < LONG_TILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float peak[2] = {-INFINITY, -INFINITY}, total[2] = {0.f, 0.f};
    const float factor = scale * LOG2E;
    const bf16* query_rows = q_tile + (group * 16 + (lane & 15)) * stride + (lane >> 4) * 8;

    for (int tile = 0; tile < tiles; ++tile) {
        const bf16* keys = k_tiles[tile & 1];
        copy_wait<0>();
        __syncthreads();
        if (tile + 1 < tiles)
            load_keys(k_tiles[(tile + 1) & 1], stride, pages, table, table_width, page_size,
                      row_size, (tile + 1) * KEYS, last_key, error_flag);
        copy_commit();
        if (idle || tile * KEYS > warp_last) continue;        // no key of the tile is visible

        // ---- scores of the warp's 16 rows against the tile's 64 keys
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        const bf16* key_rows = keys + ((lane & 7) + ((lane >> 4) << 3)) * stride +
                               ((lane >> 3) & 1) * 8;
        // (the next operands are asked for before the products on the present ones are issued)
        {
            uint32_t a[4], b[4];
            ldmatrix_x4(a, query_rows);
            ldmatrix_x4(b, key_rows);
#pragma unroll 2
            for (int k0 = 0; k0 < padded; k0 += 16) {
                uint32_t na[4] = {a[0], a[1], a[2], a[3]};
#pragma unroll
                for (int pair = 0; pair < 4; ++pair) {
                    uint32_t nb[4] = {b[0], b[1], b[2], b[3]};
                    if (pair < 3) {
                        ldmatrix_x4(nb, key_rows + (pair + 1) * 16 * stride + k0);
                    } else if (k0 + 16 < padded) {
                        ldmatrix_x4(na, query_rows + k0 + 16);
                        ldmatrix_x4(nb, key_rows + k0 + 16);
                    }
                    mma_16816(s[2 * pair], a, b[0], b[1]);
                    mma_16816(s[2 * pair + 1], a, b[2], b[3]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) b[i] = nb[i];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = na[i];
            }
        }
        // ---- the rows' maximum and sum; weights in bfloat16 as the next product's operand
        uint32_t p[4][4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int limit = position[half] - tile * KEYS - 2 * t;     // key j * 8 + x <= limit
            float highest = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][2 * half] = j * 8 <= limit ? s[j][2 * half] * factor : -INFINITY;
                s[j][2 * half + 1] = j * 8 + 1 <= limit ? s[j][2 * half + 1] * factor : -INFINITY;
                highest = fmaxf(highest, fmaxf(s[j][2 * half], s[j][2 * half + 1]));
            }
            highest = fmaxf(quad_max(highest), peak[half]);
            const float base = highest == -INFINITY ? 0.f : highest;
            const float shrink = exp2f(peak[half] - base);
            peak[half] = highest;
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float a = exp2f(s[j][2 * half] - base), b = exp2f(s[j][2 * half + 1] - base);
                sum += a + b;
                p[j >> 1][half + 2 * (j & 1)] = pack_bf16(a, b);
            }
            total[half] = total[half] * shrink + quad_sum(sum);
            // (a tile that raises no row's maximum leaves the warp's output as it is)
            if (__any_sync(0xffffffffu, shrink != 1.f)) {
#pragma unroll
                for (int j = 0; j < LONG_TILES; ++j) {
                    o[j][2 * half] *= shrink;
                    o[j][2 * half + 1] *= shrink;
                }
            }
        }
        // ---- the warp's columns of the output
        // Groups of four 8-column blocks: their four key fragments are asked for one group
        // ahead, and products that follow one another go to different accumulators.
        {
            constexpr int PER = 4, COUNT = 2 * (LONG_TILES / PER);
            uint32_t b[PER][4];
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                b[u][0] = b[u][1] = b[u][2] = b[u][3] = 0u;
                const int column = (side * LONG_TILES + u) * 8;
                if (column < latent) ldmatrix_x4_trans(b[u], keys + lane * stride + column);
            }
#pragma unroll
            for (int turn = 0; turn < COUNT; ++turn) {
                const int half = turn / (LONG_TILES / PER), first = (turn % (LONG_TILES / PER)) * PER;
                uint32_t nb[PER][4];
#pragma unroll
                for (int u = 0; u < PER; ++u) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) nb[u][i] = b[u][i];
                    if (turn + 1 < COUNT) {
                        const int next_half = (turn + 1) / (LONG_TILES / PER);
                        const int next_first = ((turn + 1) % (LONG_TILES / PER)) * PER;
                        const int column = (side * LONG_TILES + next_first + u) * 8;
                        if (column < latent)
                            ldmatrix_x4_trans(nb[u], keys + (32 * next_half + lane) * stride + column);
                    }
                }
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
                    for (int u = 0; u < PER; ++u) {
                        if ((side * LONG_TILES + first + u) * 8 < latent)
                            mma_16816(o[first + u], p[2 * half + sub], b[u][2 * sub], b[u][2 * sub + 1]);
                    }
                }
#pragma unroll
                for (int u = 0; u < PER; ++u)
#pragma unroll
                    for (int i = 0; i < 4; ++i) b[u][i] = nb[u][i];
            }
        }
    }
    copy_wait<0>();

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = group * 16 + g + 8 * half;
        if (row >= live_rows) continue;
        const size_t global_row = first_row + row;
        const float inverse = total[half] > 0.f ? 1.f / total[half] : 0.f;
#pragma unroll
        for (int j = 0; j < LONG_TILES; ++j) {
            const int column = (side * LONG_TILES + j) * 8 + 2 * t;
            if (column < latent)
                *reinterpret_cast<uint32_t*>(out + global_row * row_size + column) =
                    pack_bf16(o[j][2 * half] * inverse, o[j][2 * half + 1] * inverse);
        }
    }
}

template <int C>
size_t long_shared_bytes(int row_size) {
    const int stride = ((row_size + 15) & ~15) + 8;
    return (size_t)(16 * (WARPS / C) + 2 * KEYS) * stride * sizeof(bf16);
}

template <int C>
int launch_latent_long(const bf16* q, const bf16* pages, const int* block_table, int table_width,
                       int page_size, const int* positions, const int* request_start, bf16* out,
                       int requests, int max_rows, int heads, int row_size, int latent, float scale,
                       int* error_flag, cudaStream_t stream) {
    constexpr int ROWS = 16 * (WARPS / C);
    static bool prepared = false;
    if (!prepared) {
        cudaError_t err = cudaFuncSetAttribute(latent_attention_long_kernel<C>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)MAX_SHARED);
        MLXONE_REQUIRE(err == cudaSuccess, "latent attention: %s", cudaGetErrorString(err));
        prepared = true;
    }
    const dim3 grid((max_rows + ROWS - 1) / ROWS, requests);
    latent_attention_long_kernel<C><<<grid, WARPS * 32, long_shared_bytes<C>(row_size), stream>>>(
        q, pages, block_table, table_width, page_size, positions, request_start, out, heads,
        row_size, latent, scale, error_flag);
    MLXONE_LAUNCH_CHECK("latent_attention_long");
    return 0;
}

// One block per row: out = sum_s 2^(max_s - max) partial_s / sum_s 2^(max_s - max) sum_s. The
// splits' factors are worked out once (a lane per split) and left in shared memory.
constexpr int MAX_SPLITS = 32;

__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ partial, const float* __restrict__ stats,
                    bf16* __restrict__ out, int total_rows, int row_size, int latent, int splits) {
    __shared__ float factors[MAX_SPLITS];
    const int row = blockIdx.x;
    griddep_wait();
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        float peak = -INFINITY, sum = 0.f;
        if (s < splits) {
            const float2 both = *reinterpret_cast<const float2*>(stats + 2 * ((size_t)s * total_rows + row));
            peak = both.x, sum = both.y;
        }
        float highest = peak;
#pragma unroll
        for (int step = 16; step > 0; step >>= 1)
            highest = fmaxf(highest, __shfl_xor_sync(0xffffffffu, highest, step));
        const float weight = peak == -INFINITY ? 0.f : exp2f(peak - highest);
        float all = weight * sum;
#pragma unroll
        for (int step = 16; step > 0; step >>= 1) all += __shfl_xor_sync(0xffffffffu, all, step);
        factors[s] = all > 0.f ? weight / all : 0.f;
    }
    __syncthreads();
    for (int column = threadIdx.x; column < latent; column += blockDim.x) {
        float value = 0.f;
#pragma unroll 4
        for (int s = 0; s < splits; ++s)
            value = fmaf(factors[s], partial[((size_t)s * total_rows + row) * latent + column], value);
        out[(size_t)row * row_size + column] = __float2bfloat16_rn(value);
    }
}

template <int MT>
int launch_latent(const bf16* q, const bf16* pages, const int* block_table, int table_width,
                  int page_size, const int* positions, const int* request_start, bf16* out,
                  float* partial, float* stats, int total_rows, int requests, int max_rows,
                  int heads, int row_size, int latent, float scale, int splits, int row_limit,
                  int* error_flag, cudaStream_t stream) {
    constexpr int ROWS = 16 * MT;
    const int stride = ((row_size + 15) & ~15) + 8;
    const size_t shared = (size_t)(ROWS + 2 * KEYS) * stride * sizeof(bf16) +
                          (size_t)ROWS * SCORE_STRIDE * sizeof(float);
    static bool prepared = false;
    if (!prepared) {
        cudaError_t err = cudaFuncSetAttribute(latent_attention_kernel<MT>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)((size_t)(ROWS + 2 * KEYS) * (MAX_ROW + 8) * sizeof(bf16) +
                                                     (size_t)ROWS * SCORE_STRIDE * sizeof(float)));
        MLXONE_REQUIRE(err == cudaSuccess, "latent attention: %s", cudaGetErrorString(err));
        prepared = true;
    }
    const dim3 grid((max_rows + ROWS - 1) / ROWS, requests, splits);
    cudaError_t launched = launch_kernel(
        latent_attention_kernel<MT>, grid, dim3(WARPS * 32), shared, stream, true, q, pages,
        block_table, table_width, page_size, positions, request_start, out, partial, stats,
        total_rows, heads, row_size, latent, scale, splits, row_limit, error_flag);
    MLXONE_REQUIRE(launched == cudaSuccess, "latent attention: %s", cudaGetErrorString(launched));
    MLXONE_LAUNCH_CHECK("latent_attention_mma");
    return 0;
}

}  // namespace

// 1 if the tensor-core kernel takes rows of `row_size` values with `latent` of them the value.
MLXONE_API int mlxone_latent_attention_mma_fits(int row_size, int latent) {
    return row_size % 8 == 0 && row_size <= MAX_ROW && latent % 8 == 0 && latent <= MAX_LATENT &&
           latent <= row_size && latent > 0;
}

// q, out [tokens, heads, row_size] bfloat16; pages [pages, page_size, row_size]; max_portion: the
// most tokens a request brings. scratch (splits > 1 only; every request brings one token):
// splits * tokens * heads * (latent + 2) floats.
MLXONE_API int mlxone_latent_attention_mma(const void* q, const void* pages, const int* block_table,
                                           int table_width, int page_size, const int* positions,
                                           const int* request_start, void* out, float* scratch,
                                           int tokens, int requests, int max_portion, int heads,
                                           int row_size, int latent, float scale, int splits,
                                           int* error_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(mlxone_latent_attention_mma_fits(row_size, latent),
                   "latent attention: rows of %d with %d latent values do not fit", row_size, latent);
    MLXONE_REQUIRE(requests > 0 && heads > 0 && max_portion > 0 && page_size > 0 && table_width > 0,
                   "latent attention: bad sizes");
    MLXONE_REQUIRE(splits >= 1 && splits <= MAX_SPLITS &&
                       (splits == 1 || (max_portion == 1 && scratch != nullptr)),
                   "latent attention: keys are split only in steps of single tokens");
    const int total_rows = tokens * heads;
    float* partial = scratch;
    float* stats = scratch ? scratch + (size_t)splits * total_rows * latent : nullptr;
    const long long max_rows = (long long)max_portion * heads;
    int status = 0;
    int row_limit = 0;
    if (splits == 1 && max_rows >= LONG_ROWS) {
        // requests that bring many rows: the kernel whose warps own rows; the others (single
        // tokens beside a prompt's portion) stay with the kernel whose warps share the keys
        const bool halves = latent > 8 * LONG_TILES || long_shared_bytes<1>(row_size) > MAX_SHARED;
        status = halves
            ? launch_latent_long<2>((const bf16*)q, (const bf16*)pages, block_table, table_width,
                                    page_size, positions, request_start, (bf16*)out, requests,
                                    (int)max_rows, heads, row_size, latent, scale, error_flag, stream)
            : launch_latent_long<1>((const bf16*)q, (const bf16*)pages, block_table, table_width,
                                    page_size, positions, request_start, (bf16*)out, requests,
                                    (int)max_rows, heads, row_size, latent, scale, error_flag, stream);
        if (status || requests == 1) return status;
        row_limit = LONG_ROWS;
    }
    const int short_rows = row_limit > 0 ? row_limit - 1 : (int)max_rows;
    if (short_rows > 16)
        status = launch_latent<2>((const bf16*)q, (const bf16*)pages, block_table, table_width,
                                  page_size, positions, request_start, (bf16*)out, partial, stats,
                                  total_rows, requests, short_rows, heads, row_size, latent,
                                  scale, splits, row_limit, error_flag, stream);
    else
        status = launch_latent<1>((const bf16*)q, (const bf16*)pages, block_table, table_width,
                                  page_size, positions, request_start, (bf16*)out, partial, stats,
                                  total_rows, requests, short_rows, heads, row_size, latent,
                                  scale, splits, row_limit, error_flag, stream);
    if (status) return status;
    if (splits > 1) {
        cudaError_t launched = launch_kernel(latent_merge_kernel, dim3(total_rows), dim3(128), 0,
                                             stream, true, (const float*)partial,
                                             (const float*)stats, (bf16*)out, total_rows, row_size,
                                             latent, splits);
        MLXONE_REQUIRE(launched == cudaSuccess, "latent merge: %s", cudaGetErrorString(launched));
        MLXONE_LAUNCH_CHECK("latent_merge");
    }
    return 0;
}
