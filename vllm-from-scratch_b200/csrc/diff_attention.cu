// Differential attention over a paged cache: every head has two softmax maps (queries and keys of their
// own, `d` numbers each, laid out [map 1, map 2] head by head) over the same values, and its output is
//
//     o = a1 - lambda * a2,   o <- o * rsqrt(mean(o^2) + eps) * out_scale        (over the head's dv values)
//
// with a_m = softmax_j(cap(q_m . k_m,j * scale)) v_j, cap(s) = softcap * tanh(s / softcap) (softcap <= 0: none),
// over the keys j <= i that lie within the window (i - j < window) or among the first `keep_first` positions of
// the sequence.  Scores, softmax weights, the weighted sums, the difference and its norm are float32.
//
//   bias_rope_cache           from the packed projection [T, (H + G) * maps * d + G * dv]: the bias added, the first
//                             `rotary_dim` numbers of every map of every query and key head rotated by the
//                             position (pairs (i, i + rotary_dim / 2), angle = position * inv_freq[i] in float32),
//                             queries to q_out, keys and values into their pages
//   diff_paged_attention      float32 arithmetic, any sizes: a block is 16 consecutive queries of one request
//                             and one query head with both its maps; keys in tiles of 32 through the block table
//
// Pages: keys [pages, G, page_size, maps * d] (a position's keys of both maps side by side), values [pages, G,
// page_size, dv].
#include "common.cuh"

namespace b200 {

// W numbers of a row that are loaded and stored as one (16 bytes at most).
template <typename T, int W>
struct alignas(sizeof(T) * W) RowPiece { T v[W]; };

// A block is one token and `items_per_block` items of its row, a thread an item in turn.  An item is a piece of W
// numbers: of a value head, of the numbers of a map that are not rotated, or, where the map is rotated, the pieces
// of the first and of the second numbers of W pairs (i, i + half) together, so that a map has (d - half) / W items
// and every number is read once.  The token's cosines and sines are formed once a block, in shared memory.  W
// divides the map size, half the rotated numbers and the value size, and every row starts on a multiple of W.
template <typename T, int W>
__global__ void bias_rope_cache_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       const float* __restrict__ inv_freq, T* __restrict__ q_out,
                                       T* __restrict__ k_pages, T* __restrict__ v_pages, int q_units, int k_units,
                                       int v_heads, int maps, int d, int dv, int rotary_dim, int page_size,
                                       int items_per_block) {
    extern __shared__ float turn[];                 // [rotary_dim / 2] cosines, then as many sines
    using Piece = RowPiece<T, W>;
    overlap_trigger();
    overlap_wait();
    const int token = blockIdx.x;
    const int half = rotary_dim >> 1;
    const float position = (float)positions[token];
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(position * inv_freq[j], &turn[half + j], &turn[j]);
    __syncthreads();
    const int qk_width = (q_units + k_units) * d, width = qk_width + v_heads * dv;
    const int per_map = (d - half) / W, map_items = (q_units + k_units) * per_map;
    const int items = map_items + v_heads * dv / W;
    const int first = blockIdx.y * items_per_block, last = min(items, first + items_per_block);
    const T* row = qkv + (size_t)token * width;
    const int slot = k_pages != nullptr ? slots[token] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot - page * page_size : 0;
    const int k_heads = k_units / maps;
    for (int item = first + threadIdx.x; item < last; item += blockDim.x) {
        int column, j = 0, unit = 0;
        if (item >= map_items) {
            column = qk_width + (item - map_items) * W;
        } else {
            unit = item / per_map;
            j = (item - unit * per_map) * W;
            if (j >= half) j += half;                   // behind the pairs: the numbers that are not rotated
            column = unit * d + j;
        }
        if (column >= q_units * d && slot < 0) continue;
        T* dst;
        if (column >= qk_width) {
            const int head = (column - qk_width) / dv;
            dst = v_pages + (((size_t)page * v_heads + head) * page_size + offset) * dv + (column - qk_width - head * dv);
        } else if (unit < q_units) {
            dst = q_out + (size_t)token * q_units * d + column;
        } else {
            const int ku = unit - q_units;
            dst = k_pages + ((((size_t)page * k_heads + ku / maps) * page_size + offset) * maps + ku % maps) * d + j;
        }
        const Piece in = *reinterpret_cast<const Piece*>(row + column);
        float x[W];
#pragma unroll
        for (int w = 0; w < W; ++w) x[w] = to_float(in.v[w]) + (bias ? bias[column + w] : 0.0f);
        Piece made;
        if (column < qk_width && j < half) {
            const Piece second = *reinterpret_cast<const Piece*>(row + column + half);
            Piece turned;
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const float y = to_float(second.v[w]) + (bias ? bias[column + half + w] : 0.0f);
                float o1, o2;
                rotate_pair(x[w], y, turn[j + w], turn[half + j + w], o1, o2);
                made.v[w] = from_float<T>(o1);
                turned.v[w] = from_float<T>(o2);
            }
            *reinterpret_cast<Piece*>(dst + half) = turned;
        } else {
#pragma unroll
            for (int w = 0; w < W; ++w) made.v[w] = from_float<T>(x[w]);
        }
        *reinterpret_cast<Piece*>(dst) = made;
    }
}

template <typename T, int W>
void launch_bias_rope_cache(const void* qkv, const float* bias, const int* positions, const int* slots,
                            const float* inv_freq, void* q_out, void* k_pages, void* v_pages, int num_tokens,
                            int q_units, int k_units, int v_heads, int maps, int d, int dv, int rotary_dim,
                            int page_size, cudaStream_t stream) {
    // Many tokens: a block takes all of a token's row, so that its cosines and sines are formed once; few tokens:
    // an item to a thread, so that the launch has blocks enough.
    const int threads = 256;
    const int pieces = ((q_units + k_units) * (d - rotary_dim / 2) + v_heads * dv) / W;
    const int pieces_per_block = num_tokens >= 256 ? pieces : threads;
    dim3 grid(num_tokens, (pieces + pieces_per_block - 1) / pieces_per_block);
    const size_t smem = sizeof(float) * (size_t)rotary_dim;
    launch_overlapped_if(num_tokens <= kOverlapMostRows, bias_rope_cache_kernel<T, W>, grid, threads, smem, stream,
                         (const T*)qkv, bias, positions, slots, inv_freq, (T*)q_out, (T*)k_pages, (T*)v_pages, q_units,
                         k_units, v_heads, maps, d, dv, rotary_dim, page_size, pieces_per_block);
}

template <typename T>
void dispatch_bias_rope_cache(int pieces_of, const void* qkv, const float* bias, const int* positions, const int* slots,
                              const float* inv_freq, void* q_out, void* k_pages, void* v_pages, int num_tokens,
                              int q_units, int k_units, int v_heads, int maps, int d, int dv, int rotary_dim,
                              int page_size, cudaStream_t stream) {
#define B200_CASE(W)                                                                                                  \
    if (pieces_of == W)                                                                                               \
        return launch_bias_rope_cache<T, W>(qkv, bias, positions, slots, inv_freq, q_out, k_pages, v_pages, num_tokens, \
                                            q_units, k_units, v_heads, maps, d, dv, rotary_dim, page_size, stream);
    if constexpr (sizeof(T) == 2) { B200_CASE(8) }
    B200_CASE(4) B200_CASE(2)
#undef B200_CASE
    launch_bias_rope_cache<T, 1>(qkv, bias, positions, slots, inv_freq, q_out, k_pages, v_pages, num_tokens, q_units,
                                 k_units, v_heads, maps, d, dv, rotary_dim, page_size, stream);
}

constexpr int kQueryTile = 16;
constexpr int kKeyTile = 32;
constexpr int kWarps = 4;
constexpr int kRowsPerWarp = kQueryTile / kWarps;

struct DiffArgs {
    const int* query_start;
    const int* seq_lens;
    const int* block_table;
    int num_requests, max_pages, nq, nkv, d, dv, page_size, window, keep_first;
    float scale, softcap, lambda, eps, out_scale;
};

__device__ __forceinline__ bool key_visible(int q_pos, int kp, int window, int keep_first) {
    return kp <= q_pos && (window <= 0 || q_pos - kp < window || kp < keep_first);
}

template <typename T, int DPL>  // DPL: value elements per lane, dv <= 32 * DPL
__global__ void __launch_bounds__(kWarps * 32) diff_paged_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ out,
    const DiffArgs p) {
    overlap_trigger();
    overlap_wait();
    extern __shared__ float smem[];
    const int d = p.d, dv = p.dv, d2 = 2 * p.d, nq = p.nq, nkv = p.nkv;
    float* q_s = smem;                                   // [16][2 d]
    float* k_s = q_s + kQueryTile * d2;                  // [32][2 d + 1]
    float* v_s = k_s + kKeyTile * (d2 + 1);              // [32][dv]

    const int block = blockIdx.x;
    int lo = 0, hi = p.num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.query_start[mid] / kQueryTile + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = p.query_start[request];
    const int q_len = p.query_start[request + 1] - q_begin;
    const int local_tile = block - (q_begin / kQueryTile + request);
    const int tile_first = local_tile * kQueryTile;
    if (tile_first >= q_len) return;
    const int rows_here = min(kQueryTile, q_len - tile_first);
    const int seq_len = p.seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const int* table = p.block_table + (size_t)request * p.max_pages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_size = p.page_size, window = p.window, keep_first = p.keep_first;

    for (int idx = tid; idx < kQueryTile * d2; idx += blockDim.x) {
        const int row = idx / d2, j = idx - row * d2;
        float v = 0.0f;
        if (row < rows_here) v = to_float(q[((size_t)(q_begin + tile_first + row) * nq + head) * d2 + j]);
        q_s[idx] = v;
    }

    float acc[kRowsPerWarp][2][DPL];
    float row_max[kRowsPerWarp][2], row_sum[kRowsPerWarp][2];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            row_max[r][m] = -INFINITY;
            row_sum[r][m] = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[r][m][i] = 0.0f;
        }

    const int first_pos = past + tile_first;
    const int last_pos = first_pos + rows_here - 1;
    const int key_end = last_pos + 1;
    // Two runs of key tiles: the first positions that stay visible, then the window of the tile's queries.
    int window_begin = 0;
    if (window > 0) window_begin = (max(0, first_pos - window + 1) / kKeyTile) * kKeyTile;
    const int kept_end = (window > 0 && keep_first > 0) ? min(min(keep_first, key_end), window_begin) : 0;

    for (int run = 0; run < 2; ++run) {
        const int run_begin = run == 0 ? 0 : window_begin;
        const int run_end = run == 0 ? kept_end : key_end;
        for (int k0 = run_begin; k0 < run_end; k0 += kKeyTile) {
            __syncthreads();
            for (int idx = tid; idx < kKeyTile * d2; idx += blockDim.x) {
                const int key = idx / d2, j = idx - key * d2;
                const int kp = k0 + key;
                float kv = 0.0f;
                if (kp < run_end) {
                    const int page = table[kp / page_size];
                    if (page >= 0) kv = to_float(k_pages[(((size_t)page * nkv + kv_head) * page_size + kp % page_size) * d2 + j]);
                }
                k_s[key * (d2 + 1) + j] = kv;
            }
            for (int idx = tid; idx < kKeyTile * dv; idx += blockDim.x) {
                const int key = idx / dv, j = idx - key * dv;
                const int kp = k0 + key;
                float vv = 0.0f;
                if (kp < run_end) {
                    const int page = table[kp / page_size];
                    if (page >= 0) vv = to_float(v_pages[(((size_t)page * nkv + kv_head) * page_size + kp % page_size) * dv + j]);
                }
                v_s[key * dv + j] = vv;
            }
            __syncthreads();

#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const int row = warp * kRowsPerWarp + r;
                if (row >= rows_here) continue;                  // uniform within the warp
                const int q_pos = first_pos + row;
                const int kp = k0 + lane;
                const bool visible = kp < run_end && key_visible(q_pos, kp, window, keep_first);
                const float* q_row = q_s + row * d2;
                const float* k_row = k_s + lane * (d2 + 1);
                float pm[2];
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    float score = 0.0f;
                    for (int j = 0; j < d; ++j) score = fmaf(q_row[m * d + j], k_row[m * d + j], score);
                    score *= p.scale;
                    if (p.softcap > 0.0f) score = p.softcap * tanhf(score / p.softcap);
                    if (!visible) score = -INFINITY;
                    const float new_max = fmaxf(row_max[r][m], warp_max(score));
                    pm[m] = 0.0f;
                    if (new_max == -INFINITY) continue;
                    const float correction = expf(row_max[r][m] - new_max);
                    pm[m] = visible ? expf(score - new_max) : 0.0f;
                    row_sum[r][m] = row_sum[r][m] * correction + warp_sum(pm[m]);
                    row_max[r][m] = new_max;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) acc[r][m][i] *= correction;
                }
                for (int key = 0; key < kKeyTile; ++key) {
                    const float p0 = __shfl_sync(0xffffffffu, pm[0], key);
                    const float p1 = __shfl_sync(0xffffffffu, pm[1], key);
                    const float* v_row = v_s + key * dv;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const int j = lane + 32 * i;
                        if (j < dv) {
                            const float vv = v_row[j];
                            acc[r][0][i] = fmaf(p0, vv, acc[r][0][i]);
                            acc[r][1][i] = fmaf(p1, vv, acc[r][1][i]);
                        }
                    }
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int row = warp * kRowsPerWarp + r;
        if (row >= rows_here) continue;
        const float inv0 = row_sum[r][0] > 0.0f ? 1.0f / row_sum[r][0] : 0.0f;
        const float inv1 = row_sum[r][1] > 0.0f ? 1.0f / row_sum[r][1] : 0.0f;
        float o[DPL], squares = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            o[i] = 0.0f;
            if (lane + 32 * i < dv) o[i] = fmaf(-p.lambda, acc[r][1][i] * inv1, acc[r][0][i] * inv0);
            squares = fmaf(o[i], o[i], squares);
        }
        const float factor = rsqrtf(warp_sum(squares) / (float)dv + p.eps) * p.out_scale;
        T* dst = out + ((size_t)(q_begin + tile_first + row) * nq + head) * dv;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int j = lane + 32 * i;
            if (j < dv) dst[j] = from_float<T>(o[i] * factor);
        }
    }
}

template <typename T, int DPL>
int launch_diff(const void* q, const void* k_pages, const void* v_pages, void* out, const DiffArgs& p, int num_tokens,
                cudaStream_t stream) {
    auto kernel = diff_paged_attention_kernel<T, DPL>;
    const size_t smem = sizeof(float) * ((size_t)kQueryTile * 2 * p.d + (size_t)kKeyTile * (2 * p.d + 1) + (size_t)kKeyTile * p.dv);
    if (smem > 200 * 1024) return fail("diff_paged_attention", "heads too large for one block's shared memory");
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("diff_paged_attention", cudaGetErrorString(status));
    }
    dim3 grid(num_tokens / kQueryTile + p.num_requests, p.nq);
    launch_overlapped_if(num_tokens <= kOverlapMostRows, kernel, grid, kWarps * 32, smem, stream,
                         (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, p);
    return check_launch("diff_paged_attention");
}

template <typename T>
int dispatch_diff(const void* q, const void* k_pages, const void* v_pages, void* out, const DiffArgs& p, int num_tokens,
                  cudaStream_t stream) {
#define B200_CASE(DPL) \
    if (p.dv <= 32 * DPL) return launch_diff<T, DPL>(q, k_pages, v_pages, out, p, num_tokens, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(4) B200_CASE(8) B200_CASE(16)
#undef B200_CASE
    return fail("diff_paged_attention", "value heads above 512 are not built");
}

}  // namespace b200

// qkv rows: [q_units * d | k_units * d | v_heads * dv] with q_units = query heads * maps and k_units = v_heads * maps;
// bias float32 of the same width or null.  inv_freq float32 [rotary_dim / 2] (rotary_dim 0: no rotation).
// k_pages / v_pages may be null (nothing is stored).  dtype: 0 = float32, 1 = bfloat16.
B200_EXPORT int b200_bias_rope_cache(const void* qkv, const float* bias, const int* positions, const int* slots,
                                     const float* inv_freq, void* q_out, void* k_pages, void* v_pages, int num_tokens,
                                     int q_units, int v_heads, int maps, int d, int dv, int rotary_dim, int page_size,
                                     int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    if (maps <= 0 || q_units <= 0 || v_heads <= 0 || d <= 0 || dv <= 0) return fail("bias_rope_cache", "sizes must be positive");
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > d) return fail("bias_rope_cache", "rotary_dim must be even and at most d");
    if (rotary_dim > 0 && inv_freq == nullptr) return fail("bias_rope_cache", "frequencies are missing");
    if ((k_pages == nullptr) != (v_pages == nullptr)) return fail("bias_rope_cache", "key and value pages must be given together");
    if (k_pages && page_size <= 0) return fail("bias_rope_cache", "page_size must be positive");
    const int k_units = v_heads * maps;
    if (((size_t)q_units + k_units) * d + (size_t)v_heads * dv > 2147483647u) return fail("bias_rope_cache", "a row is too wide");
    if (dtype != 0 && dtype != 1) return fail("bias_rope_cache", "dtype must be 0 (float32) or 1 (bfloat16)");
    // The widest pieces (16 bytes at most) that the sizes and the addresses allow.
    const int size = dtype == 0 ? 4 : 2;
    const uintptr_t all = (uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages;
    int pieces_of = 16 / size;
    while (pieces_of > 1 && (d % pieces_of || dv % pieces_of || (rotary_dim / 2) % pieces_of ||
                             (all % (uintptr_t)(pieces_of * size)) != 0))
        pieces_of >>= 1;
    if (dtype == 0)
        dispatch_bias_rope_cache<float>(pieces_of, qkv, bias, positions, slots, inv_freq, q_out, k_pages, v_pages,
                                        num_tokens, q_units, k_units, v_heads, maps, d, dv, rotary_dim, page_size, stream);
    else
        dispatch_bias_rope_cache<__nv_bfloat16>(pieces_of, qkv, bias, positions, slots, inv_freq, q_out, k_pages, v_pages,
                                                num_tokens, q_units, k_units, v_heads, maps, d, dv, rotary_dim, page_size,
                                                stream);
    return check_launch("bias_rope_cache");
}

// q [T, nq * 2 d], out [T, nq * dv]; window <= 0: every earlier key is visible; softcap <= 0: none.
B200_EXPORT int b200_diff_paged_attention(const void* q, const void* k_pages, const void* v_pages, void* out,
                                          const int* query_start, const int* seq_lens, const int* block_table,
                                          int num_requests, int num_tokens, int max_pages, int nq, int nkv, int d, int dv,
                                          int page_size, float scale, float softcap, int window, int keep_first,
                                          float lambda, float eps, float out_scale, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens == 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv) return fail("diff_paged_attention", "query heads must be a multiple of key/value heads");
    if (nq > 65535) return fail("diff_paged_attention", "more than 65535 query heads");
    if (d <= 0 || dv <= 0 || page_size <= 0 || max_pages <= 0) return fail("diff_paged_attention", "sizes must be positive");
    DiffArgs p{query_start, seq_lens, block_table, num_requests, max_pages, nq, nkv, d, dv, page_size,
               window > 0 ? window : 0, window > 0 && keep_first > 0 ? keep_first : 0, scale, softcap, lambda, eps, out_scale};
    if (dtype == 0) return dispatch_diff<float>(q, k_pages, v_pages, out, p, num_tokens, stream);
    if (dtype == 1) return dispatch_diff<__nv_bfloat16>(q, k_pages, v_pages, out, p, num_tokens, stream);
    return fail("diff_paged_attention", "dtype must be 0 (float32) or 1 (bfloat16)");
}
