// Differential attention on the bfloat16 tensor cores: one kernel for portions of prompts (any mix of query
// lengths) and one for decode batches (one new token a request, a request's keys split over several blocks
// and merged).  Meaning of the arguments, masking and page layout: diff_attention.cu.
//
// A head's two maps share its tile of values.  A block has eight warps, four per map: the warps of map m read
// the map's half of the queries and of every key row, keep softmax statistics and an output of their own, and
// meet only at the end, where the warps of map 2 hand their normalised output over through shared memory and
// the warps of map 1 form o = a1 - lambda a2, its norm and the factor.  Scores are m16n8k16 bfloat16 products
// accumulating in float32; cap, mask, maximum, exponentials and sums are float32; the float32 weights enter the
// second product as three bfloat16 pieces whose sum is the weight to the last bit (split_bf16x3), so the
// weighted sum of the values is the one with float32 weights.
//
// The keys a block visits are a list: the first positions that stay visible whatever the window (those that lie
// before the window of the block's first query), then the window's keys up to the block's last query.  Tiles of
// 64 entries of that list go through two stages of shared memory (three in a decode block) by 16-byte asynchronous
// copies; where each entry's row lies in the pages is looked up through the block table once an entry, a turn
// ahead of the tile's copies.  Rows are padded by 16 bytes, which spreads the eight rows of an ldmatrix over all
// banks for every row length that is a multiple of 32 bytes.
#pragma once

#include "attention_bf16_kernels.cuh"

namespace b200 {

constexpr int kDiffThreads = 256;
constexpr int kDiffPad = 8;                     // bfloat16 elements behind every row of a tile
constexpr int kDiffDecodeStages = 3;            // tiles of shared memory of a decode block

struct DiffMmaArgs {
    const int* query_start;
    const int* seq_lens;
    const int* block_table;
    int num_requests, max_pages, nq, nkv, page_size, window, keep_first, token_offset;
    float scale, softcap, lambda, eps, out_scale;
};

// The list of keys of a block: entries [0, kept) are the positions 0 .. kept - 1, the entries behind them
// the positions first .. end - 1.
struct KeyList {
    int kept, first, end;
    __device__ __forceinline__ int count() const { return kept + end - first; }
    __device__ __forceinline__ int position(int entry) const { return entry < kept ? entry : first + entry - kept; }
};

__device__ __forceinline__ KeyList key_list(int first_query, int last_query, int window, int keep_first) {
    KeyList list;
    list.end = last_query + 1;
    list.first = window > 0 ? max(0, first_query - window + 1) : 0;
    list.kept = min(keep_first, list.first);
    return list;
}

// Where the rows of the entries e0 .. e0 + 63 of the list lie in the pages of key/value head `kv_head`, counted in
// rows: rows[i] for entry e0 + i, -1 for entries past the list and for pages that were given back.  One thread
// an entry looks its page up, so that the copies that follow divide nothing and wait for no table.
__device__ __forceinline__ void list_tile_rows(long long* rows, const int* __restrict__ table, const KeyList& list,
                                               int e0, int e_end, int kv_head, int nkv, int page_size) {
    if (threadIdx.x < kKeys) {
        const int entry = e0 + threadIdx.x;
        long long at = -1;
        if (entry < e_end) {
            const int kp = list.position(entry);
            const int index = kp / page_size;
            const int page = table[index];
            if (page >= 0) at = ((long long)page * nkv + kv_head) * page_size + (kp - index * page_size);
        }
        rows[threadIdx.x] = at;
    }
}

// A tile of 64 entries whose rows `rows` names: key rows [64][2 D + pad] and value rows [64][DV + pad]; zeros
// where there is no row.
template <int D, int DV>
__device__ __forceinline__ void load_list_tile(bf16* k_s, bf16* v_s, const bf16* __restrict__ k_pages,
                                               const bf16* __restrict__ v_pages, const long long* rows) {
    constexpr int kKeyChunks = 2 * D / 8, kValueChunks = DV / 8, kChunks = kKeyChunks + kValueChunks;
    for (int idx = threadIdx.x; idx < kKeys * kChunks; idx += kDiffThreads) {
        const int row = idx / kChunks, c = idx - row * kChunks;
        const long long at = rows[row];
        bf16* dst;
        const bf16* src;
        if (c < kKeyChunks) {
            dst = k_s + row * (2 * D + kDiffPad) + c * 8;
            src = k_pages + at * (2 * D) + c * 8;
        } else {
            dst = v_s + row * (DV + kDiffPad) + (c - kKeyChunks) * 8;
            src = v_pages + at * DV + (c - kKeyChunks) * 8;
        }
        if (at >= 0) cp_async16(dst, src);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
}

// 2^x by the special-function unit alone (two units in the last place; results below 2^-126 are zero, which a
// softmax weight may be).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_reciprocal(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// What turns a raw product q . k into the capped score in units of log2 e: with a cap, `in` = scale * 2 log2 e /
// cap and `out` = cap * log2 e; without, `in` = scale * log2 e and `out` = 0.
struct ScoreScale {
    float in, out;
};
__device__ __forceinline__ ScoreScale score_scale(float scale, float cap) {
    ScoreScale made;
    made.in = cap > 0.0f ? scale * (2.0f * kLog2e) / cap : scale * kLog2e;
    made.out = cap > 0.0f ? cap * kLog2e : 0.0f;
    return made;
}
// cap * tanh(s / cap) in units of log2 e, from one exponential and one reciprocal: tanh(y) = 1 - 2 / (e^(2 y) + 1).
// Its absolute error is a few units in the last place of 1, times cap.
__device__ __forceinline__ float capped_log2(float raw, const ScoreScale& by) {
    if (by.out <= 0.0f) return raw * by.in;
    const float e = fast_exp2(raw * by.in);
    return fmaf(-2.0f * by.out, fast_reciprocal(e + 1.0f), by.out);
}

// o += P V for 16 entries of a tile: the weights as three bfloat16 pieces (smallest first), `v_row` this lane's
// row and column half of the value tile for ldmatrix.  The products of one piece over all columns of the head
// stand together, so that two products into the same accumulator have the others between them.
template <int DV>
__device__ __forceinline__ void weighted_values(float (&o)[DV / 8][4], const unsigned (&pa)[4], const unsigned (&pm)[4],
                                                const unsigned (&pl)[4], const bf16* v_row) {
    constexpr int kBlocks = DV / 16, kAtOnce = kBlocks % 4 == 0 ? 4 : kBlocks % 2 == 0 ? 2 : 1;
#pragma unroll
    for (int j0 = 0; j0 < kBlocks; j0 += kAtOnce) {
        unsigned b[kAtOnce][4];
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i) ldmatrix_x4_trans(b[i], v_row + (j0 + i) * 16);
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i) {
            mma_bf16(o[2 * (j0 + i)], pl, b[i][0], b[i][1]);
            mma_bf16(o[2 * (j0 + i) + 1], pl, b[i][2], b[i][3]);
        }
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i) {
            mma_bf16(o[2 * (j0 + i)], pm, b[i][0], b[i][1]);
            mma_bf16(o[2 * (j0 + i) + 1], pm, b[i][2], b[i][3]);
        }
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i) {
            mma_bf16(o[2 * (j0 + i)], pa, b[i][0], b[i][1]);
            mma_bf16(o[2 * (j0 + i) + 1], pa, b[i][2], b[i][3]);
        }
    }
}

// The same sum for a decode block, transposed: o^T += V^T P^T for 16 entries of a tile.  The 16 x 16 blocks of the
// value tile are the first operand (16 columns of the head by 16 entries), the weights of eight query heads the
// second (their score fragments are that operand's fragments as they stand), so that a product's eight columns
// are eight query heads and none of its rows is padding.  `o[h][j]` holds columns 16 j .. 16 j + 15 of the output
// of the heads 8 h .. 8 h + 7: elements 0 and 1 the column 16 j + lane / 4 for the heads 8 h + 2 (lane % 4) and the
// next, elements 2 and 3 the column eight further on.
template <int DV, int kHalves>
__device__ __forceinline__ void weighted_values_transposed(float (&o)[kHalves][DV / 16][4], const unsigned (&pa)[4],
                                                           const unsigned (&pm)[4], const unsigned (&pl)[4],
                                                           const bf16* v_row) {
    constexpr int kBlocks = DV / 16, kAtOnce = kBlocks % 4 == 0 ? 4 : kBlocks % 2 == 0 ? 2 : 1;
#pragma unroll
    for (int j0 = 0; j0 < kBlocks; j0 += kAtOnce) {
        unsigned a[kAtOnce][4];
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i) {
            unsigned b[4];
            ldmatrix_x4_trans(b, v_row + (j0 + i) * 16);
            a[i][0] = b[0]; a[i][1] = b[2]; a[i][2] = b[1]; a[i][3] = b[3];
        }
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i)
#pragma unroll
            for (int h = 0; h < kHalves; ++h) mma_bf16(o[h][j0 + i], a[i], pl[h], pl[2 + h]);
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i)
#pragma unroll
            for (int h = 0; h < kHalves; ++h) mma_bf16(o[h][j0 + i], a[i], pm[h], pm[2 + h]);
#pragma unroll
        for (int i = 0; i < kAtOnce; ++i)
#pragma unroll
            for (int h = 0; h < kHalves; ++h) mma_bf16(o[h][j0 + i], a[i], pa[h], pa[2 + h]);
    }
}

// A warp's 16 rows against a tile of 64 entries: scores of its map, softmax update, the product with the values.
// `s` comes in as the raw products and is used up.
template <int DV>
__device__ __forceinline__ void softmax_and_values(float (&s)[8][4], float (&o)[DV / 8][4], float& m_a, float& m_b,
                                                   float& l_a, float& l_b, const bf16* v_s, int lane) {
    float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        max_a = fmaxf(max_a, fmaxf(s[nt][0], s[nt][1]));
        max_b = fmaxf(max_b, fmaxf(s[nt][2], s[nt][3]));
    }
    max_a = quad_max(max_a);
    max_b = quad_max(max_b);
    const float new_a = fmaxf(m_a, max_a), new_b = fmaxf(m_b, max_b);
    const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
    const float alpha_a = fast_exp2(m_a - ref_a), alpha_b = fast_exp2(m_b - ref_b);
    m_a = new_a;
    m_b = new_b;
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = fast_exp2(s[nt][0] - ref_a);
        s[nt][1] = fast_exp2(s[nt][1] - ref_a);
        s[nt][2] = fast_exp2(s[nt][2] - ref_b);
        s[nt][3] = fast_exp2(s[nt][3] - ref_b);
        sum_a += s[nt][0] + s[nt][1];
        sum_b += s[nt][2] + s[nt][3];
    }
    l_a = l_a * alpha_a + sum_a;
    l_b = l_b * alpha_b + sum_b;
    // once the maxima have settled a tile changes none of them: the factors are all 1 and the output stays
    if (__any_sync(0xffffffffu, alpha_a != 1.0f || alpha_b != 1.0f)) {
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            o[nt][0] *= alpha_a; o[nt][1] *= alpha_a; o[nt][2] *= alpha_b; o[nt][3] *= alpha_b;
        }
    }
    const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        unsigned pa[4], pm[4], pl[4];
        split_bf16x3(s[2 * kk][0], s[2 * kk][1], pa[0], pm[0], pl[0]);
        split_bf16x3(s[2 * kk][2], s[2 * kk][3], pa[1], pm[1], pl[1]);
        split_bf16x3(s[2 * kk + 1][0], s[2 * kk + 1][1], pa[2], pm[2], pl[2]);
        split_bf16x3(s[2 * kk + 1][2], s[2 * kk + 1][3], pa[3], pm[3], pl[3]);
        weighted_values<DV>(o, pa, pm, pl, v_s + (kk * 16 + (mi & 1) * 8 + ri) * (DV + kDiffPad) + (mi >> 1) * 8);
    }
}

// Raw products of a warp's 16 query rows (fragments `qa` of its map) with the 64 key rows of a tile.
template <int D>
__device__ __forceinline__ void score_products(float (&s)[8][4], const unsigned (&qa)[D / 16][4], const bf16* k_map,
                                               int lane) {
    const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const int key = np * 16 + (mi >> 1) * 8 + ri;
            unsigned b[4];
            ldmatrix_x4(b, k_map + key * (2 * D + kDiffPad) + (ks * 2 + (mi & 1)) * 8);
            mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
            mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
        }
    }
}

// The end of a block: the warps of map 2 hand a2 over, those of map 1 write (a1 - lambda a2) normalised.
// `o` is the warp's output divided by its row sums already.  exchange: float32 [rows][DV + 8].
template <int DV>
__device__ __forceinline__ void difference_norm_store(const float (&o)[DV / 8][4], int map, int row_a, int row_b,
                                                      float* exchange, bf16* out_a, bf16* out_b, float lambda,
                                                      float eps, float out_scale, int lane) {
    constexpr int kStride = DV + 8;
    if (map == 1) {
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<float2*>(exchange + row_a * kStride + col) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(exchange + row_b * kStride + col) = make_float2(o[nt][2], o[nt][3]);
        }
    }
    __syncthreads();
    if (map == 0) {
        float d[DV / 8][4];
        float squares_a = 0.0f, squares_b = 0.0f;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            const float2 xa = *reinterpret_cast<const float2*>(exchange + row_a * kStride + col);
            const float2 xb = *reinterpret_cast<const float2*>(exchange + row_b * kStride + col);
            d[nt][0] = fmaf(-lambda, xa.x, o[nt][0]);
            d[nt][1] = fmaf(-lambda, xa.y, o[nt][1]);
            d[nt][2] = fmaf(-lambda, xb.x, o[nt][2]);
            d[nt][3] = fmaf(-lambda, xb.y, o[nt][3]);
            squares_a += d[nt][0] * d[nt][0] + d[nt][1] * d[nt][1];
            squares_b += d[nt][2] * d[nt][2] + d[nt][3] * d[nt][3];
        }
        const float factor_a = rsqrtf(quad_sum(squares_a) / (float)DV + eps) * out_scale;
        const float factor_b = rsqrtf(quad_sum(squares_b) / (float)DV + eps) * out_scale;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            if (out_a) *reinterpret_cast<unsigned*>(out_a + col) = pack_bf16(d[nt][0] * factor_a, d[nt][1] * factor_a);
            if (out_b) *reinterpret_cast<unsigned*>(out_b + col) = pack_bf16(d[nt][2] * factor_b, d[nt][3] * factor_b);
        }
    }
}

template <int D, int DV>
__host__ __device__ constexpr int diff_stage_elements() { return kKeys * (2 * D + kDiffPad) + kKeys * (DV + kDiffPad); }

// ------------------------------------------------------------------ portions of prompts
// grid (query tiles, query heads).  A tile is 64 consecutive query tokens of one request, 16 to a warp of each
// map; request r owns the tiles [(start[r] - offset) / 64 + r, (start[r + 1] - offset) / 64 + r + 1).
template <int D, int DV>
__global__ void __launch_bounds__(kDiffThreads, DV <= 128 ? 2 : 1) diff_prefill_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    bf16* __restrict__ out, const DiffMmaArgs p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);
    constexpr int kRows = 64;
    constexpr int kStage = diff_stage_elements<D, DV>();
    // Late tiles of a long request have the most keys to visit: hand them out first.
    const int block = gridDim.x - 1 - blockIdx.x;
    int lo = 0, hi = p.num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((p.query_start[mid] - p.token_offset) / kRows + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = p.query_start[request];
    const int q_len = p.query_start[request + 1] - q_begin;
    const int tile_first = (block - ((q_begin - p.token_offset) / kRows + request)) * kRows;
    if (tile_first >= q_len) return;
    const int rows_here = min(kRows, q_len - tile_first);
    const int seq_len = p.seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y, nq = p.nq;
    const int kv_head = head / (nq / p.nkv);
    const int* table = p.block_table + (size_t)request * p.max_pages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int map = warp >> 2, group = warp & 3;
    const int window = p.window, keep_first = p.keep_first;

    const int row_a = group * 16 + (lane >> 2), row_b = row_a + 8;
    const bf16* q_tile = q + ((size_t)(q_begin + tile_first) * nq + head) * (2 * D) + map * D;
    unsigned qa[D / 16][4];
    load_q_fragments<D>(qa, row_a < rows_here ? q_tile + (size_t)row_a * nq * 2 * D : nullptr,
                        row_b < rows_here ? q_tile + (size_t)row_b * nq * 2 * D : nullptr, lane);

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;

    const int first_pos = past + tile_first;
    const int pos_a = first_pos + row_a, pos_b = first_pos + row_b;
    const int warp_first_pos = first_pos + group * 16;
    const int warp_last_pos = first_pos + min(group * 16 + 15, rows_here - 1);
    const KeyList list = key_list(first_pos, first_pos + rows_here - 1, window, keep_first);
    const int entries = list.count();
    const int tiles = (entries + kKeys - 1) / kKeys;
    const ScoreScale by = score_scale(p.scale, p.softcap);

    auto k_stage = [&](int s) { return stage_base + (size_t)s * kStage; };
    auto v_stage = [&](int s) { return stage_base + (size_t)s * kStage + kKeys * (2 * D + kDiffPad); };

    // rows_of(i): where the rows of tile i lie, made a turn before the tile's copies start
    long long* row_slots = reinterpret_cast<long long*>(stage_base + 2 * (size_t)kStage);
    auto rows_of = [&](int tile) { return row_slots + (tile & 1) * kKeys; };
    list_tile_rows(rows_of(0), table, list, 0, entries, kv_head, p.nkv, p.page_size);
    list_tile_rows(rows_of(1), table, list, kKeys, entries, kv_head, p.nkv, p.page_size);
    __syncthreads();
    load_list_tile<D, DV>(k_stage(0), v_stage(0), k_pages, v_pages, rows_of(0));
    cp_async_commit();
    for (int t = 0; t < tiles; ++t) {
        const int e0 = t * kKeys;
        if (t + 1 < tiles) {
            load_list_tile<D, DV>(k_stage((t + 1) & 1), v_stage((t + 1) & 1), k_pages, v_pages, rows_of(t + 1));
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // (the copies of tile t were started a turn ago from the slot that the rows of tile t + 2 now take)
        if (t + 2 < tiles)
            list_tile_rows(rows_of(t + 2), table, list, e0 + 2 * kKeys, entries, kv_head, p.nkv, p.page_size);
        // A tile wholly behind the kept positions is a run of consecutive positions from k0 on; a warp whose rows
        // all lie before it (causal) or whose windows all lie behind it has nothing to add.
        const bool plain_run = e0 >= list.kept;
        const int k0 = list.position(e0);
        bool active = group * 16 < rows_here;
        if (plain_run) {
            if (k0 > warp_last_pos) active = false;
            if (window > 0 && k0 + kKeys - 1 <= warp_first_pos - window && k0 >= keep_first) active = false;
        }
        if (active) {
            float s[8][4];
            score_products<D>(s, qa, k_stage(t & 1) + map * D, lane);
            const bool all_visible = plain_run && e0 + kKeys <= entries && k0 + kKeys - 1 <= warp_first_pos &&
                                     (window <= 0 || k0 > warp_last_pos - window);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = capped_log2(s[nt][e], by);
                    if (!all_visible) {
                        const int entry = e0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int kp = list.position(entry);
                        const int q_pos = e < 2 ? pos_a : pos_b;
                        const bool visible = entry < entries && kp <= q_pos &&
                                             (window <= 0 || q_pos - kp < window || kp < keep_first);
                        if (!visible) v = -INFINITY;
                    }
                    s[nt][e] = v;
                }
            softmax_and_values<DV>(s, o, m_a, m_b, l_a, l_b, v_stage(t & 1), lane);
        }
        __syncthreads();
    }

    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
        o[nt][0] *= inv_a; o[nt][1] *= inv_a; o[nt][2] *= inv_b; o[nt][3] *= inv_b;
    }
    bf16* out_tile = out + ((size_t)(q_begin + tile_first) * nq + head) * DV;
    difference_norm_store<DV>(o, map, row_a, row_b, reinterpret_cast<float*>(smem_raw),
                              row_a < rows_here ? out_tile + (size_t)row_a * nq * DV : nullptr,
                              row_b < rows_here ? out_tile + (size_t)row_b * nq * DV : nullptr, p.lambda, p.eps,
                              p.out_scale, lane);
}

template <int D, int DV>
int launch_diff_prefill_mma(const void* q, const void* k_pages, const void* v_pages, void* out, const DiffMmaArgs& p,
                            int num_tokens, cudaStream_t stream) {
    auto kernel = diff_prefill_mma_kernel<D, DV>;
    const int stages = 2 * diff_stage_elements<D, DV>() * (int)sizeof(bf16) + 2 * kKeys * (int)sizeof(long long);
    const int exchange = 64 * (DV + 8) * (int)sizeof(float);
    const int smem = stages > exchange ? stages : exchange;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (status != cudaSuccess) return fail("diff_prefill_attention", cudaGetErrorString(status));
    dim3 grid((num_tokens - p.token_offset) / 64 + p.num_requests, p.nq);
    kernel<<<grid, kDiffThreads, smem, stream>>>((const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, p);
    return check_launch("diff_prefill_attention");
}

// ------------------------------------------------------------------ decode batches
// grid (splits, key/value heads, requests): every request brings one token, so token == request.  The rows of
// a 16-row fragment are the query heads that share the key/value head (at most 16).  Of the eight warps four
// belong to each map, and each takes 16 of a tile's 64 entries; the warps of a map merge through shared memory,
// and with one split the block also forms the difference and its norm.  With several splits the merged
// (maximum, sum, output) of each map go to scratch: partial_o [(head * 2 + map) * splits + split][DV],
// partial_ml the same rows of [2].  The product with the values is the transposed one (weighted_values_transposed),
// over the first eight heads of the fragment (kHalves 1: up to eight query heads to a key/value head; the scores
// of the other eight rows are not even capped) or over both halves (kHalves 2).
template <int D, int DV, int kHalves>
__global__ void __launch_bounds__(kDiffThreads) diff_decode_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    bf16* __restrict__ out, float* __restrict__ partial_o, float* __restrict__ partial_ml, const DiffMmaArgs p,
    int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);
    constexpr int kStage = diff_stage_elements<D, DV>();
    overlap_trigger();
    overlap_wait();
    const int split = blockIdx.x, kv_head = blockIdx.y, request = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int map = warp >> 2, part = warp & 3;
    const int nq = p.nq, group = nq / p.nkv;
    const int seq_len = p.seq_lens[request];
    const KeyList list = key_list(seq_len - 1, seq_len - 1, p.window, p.keep_first);
    const int entries = list.count();
    int chunk = (entries + splits - 1) / splits;
    chunk = ((chunk + kKeys - 1) / kKeys) * kKeys;
    const int my_begin = split * chunk;
    const int my_end = min(entries, my_begin + chunk);
    const int tiles = my_end > my_begin ? (my_end - my_begin + kKeys - 1) / kKeys : 0;
    const int* table = p.block_table + (size_t)request * p.max_pages;
    const ScoreScale by = score_scale(p.scale, p.softcap);

    const int row_a = lane >> 2, row_b = row_a + 8;
    const bf16* q_base = q + ((size_t)request * nq + (size_t)kv_head * group) * (2 * D) + map * D;
    unsigned qa[D / 16][4];
    load_q_fragments<D>(qa, row_a < group ? q_base + (size_t)row_a * 2 * D : nullptr,
                        row_b < group ? q_base + (size_t)row_b * 2 * D : nullptr, lane);

    float o[kHalves][DV / 16][4];
#pragma unroll
    for (int h = 0; h < kHalves; ++h)
#pragma unroll
        for (int i = 0; i < DV / 16; ++i) o[h][i][0] = o[h][i][1] = o[h][i][2] = o[h][i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    // the heads of this lane's columns of the transposed output sit in the lanes 4 * head as rows of the scores
    const int column_lane = (lane & 3) * 8;

    auto k_stage = [&](int s) { return stage_base + (size_t)s * kStage; };
    auto v_stage = [&](int s) { return stage_base + (size_t)s * kStage + kKeys * (2 * D + kDiffPad); };

    // Two tiles are on their way while one is used (a group of copies is committed every turn, an empty one too,
    // so that the count behind the wait is the same every turn).
    // Where the rows of tile i lie is looked up a turn before the tile's copies start (slot i % stages).
    long long* row_slots = reinterpret_cast<long long*>(stage_base + kDiffDecodeStages * (size_t)kStage);
    auto rows_of = [&](int tile) { return row_slots + (tile % kDiffDecodeStages) * kKeys; };
#pragma unroll
    for (int s = 0; s < kDiffDecodeStages; ++s)
        list_tile_rows(rows_of(s), table, list, my_begin + s * kKeys, my_end, kv_head, p.nkv, p.page_size);
    __syncthreads();
#pragma unroll
    for (int s = 0; s < kDiffDecodeStages - 1; ++s) {
        if (s < tiles) load_list_tile<D, DV>(k_stage(s), v_stage(s), k_pages, v_pages, rows_of(s));
        cp_async_commit();
    }
    const int mi = lane >> 3, ri = lane & 7;
    for (int t = 0; t < tiles; ++t) {
        const int e0 = my_begin + t * kKeys;
        const int ahead = t + kDiffDecodeStages - 1;
        if (ahead < tiles)
            load_list_tile<D, DV>(k_stage(ahead % kDiffDecodeStages), v_stage(ahead % kDiffDecodeStages), k_pages, v_pages,
                                  rows_of(ahead));
        cp_async_commit();
        cp_async_wait<kDiffDecodeStages - 1>();
        __syncthreads();
        // the slot of tile t is free (its copies were started two turns ago): the rows of tile t + stages
        if (t + kDiffDecodeStages < tiles)
            list_tile_rows(rows_of(t + kDiffDecodeStages), table, list, e0 + kDiffDecodeStages * kKeys, my_end, kv_head,
                           p.nkv, p.page_size);
        const bf16* k_map = k_stage(t % kDiffDecodeStages) + map * D;
        const bf16* v_s = v_stage(t % kDiffDecodeStages);

        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int key = part * 16 + (mi >> 1) * 8 + ri;
            unsigned b[4];
            ldmatrix_x4(b, k_map + key * (2 * D + kDiffPad) + (ks * 2 + (mi & 1)) * 8);
            mma_bf16(s[0], qa[ks], b[0], b[1]);
            mma_bf16(s[1], qa[ks], b[2], b[3]);
        }
        float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2 * kHalves; ++e) {
                const int entry = e0 + part * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
                float v = capped_log2(s[nt][e], by);
                if (entry >= my_end) v = -INFINITY;       // every entry of the list is visible to the one query
                s[nt][e] = v;
                if (e < 2) max_a = fmaxf(max_a, v); else max_b = fmaxf(max_b, v);
            }
        max_a = quad_max(max_a);
        const float new_a = fmaxf(m_a, max_a);
        const float ref_a = new_a == -INFINITY ? 0.0f : new_a;
        const float alpha_a = fast_exp2(m_a - ref_a);
        m_a = new_a;
        float sum_a = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[nt][0] = fast_exp2(s[nt][0] - ref_a);
            s[nt][1] = fast_exp2(s[nt][1] - ref_a);
            sum_a += s[nt][0] + s[nt][1];
        }
        l_a = l_a * alpha_a + sum_a;
        float alpha_b = 1.0f;
        if constexpr (kHalves == 2) {
            max_b = quad_max(max_b);
            const float new_b = fmaxf(m_b, max_b);
            const float ref_b = new_b == -INFINITY ? 0.0f : new_b;
            alpha_b = fast_exp2(m_b - ref_b);
            m_b = new_b;
            float sum_b = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                s[nt][2] = fast_exp2(s[nt][2] - ref_b);
                s[nt][3] = fast_exp2(s[nt][3] - ref_b);
                sum_b += s[nt][2] + s[nt][3];
            }
            l_b = l_b * alpha_b + sum_b;
        } else {
            s[0][2] = s[0][3] = s[1][2] = s[1][3] = 0.0f;
        }
        unsigned pa[4], pm[4], pl[4];
        split_bf16x3(s[0][0], s[0][1], pa[0], pm[0], pl[0]);
        split_bf16x3(s[1][0], s[1][1], pa[2], pm[2], pl[2]);
        if constexpr (kHalves == 2) {
            split_bf16x3(s[0][2], s[0][3], pa[1], pm[1], pl[1]);
            split_bf16x3(s[1][2], s[1][3], pa[3], pm[3], pl[3]);
        } else {
            pa[1] = pm[1] = pl[1] = pa[3] = pm[3] = pl[3] = 0u;
        }
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
            const float alpha = h == 0 ? alpha_a : alpha_b;
            const float even = __shfl_sync(0xffffffffu, alpha, column_lane);
            const float odd = __shfl_sync(0xffffffffu, alpha, column_lane + 4);
#pragma unroll
            for (int j = 0; j < DV / 16; ++j) {
                o[h][j][0] *= even; o[h][j][1] *= odd; o[h][j][2] *= even; o[h][j][3] *= odd;
            }
        }
        weighted_values_transposed<DV, kHalves>(o, pa, pm, pl,
                                                v_s + (part * 16 + (mi & 1) * 8 + ri) * (DV + kDiffPad) + (mi >> 1) * 8);
        __syncthreads();
    }

    // the four warps of each map meet in shared memory
    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    float* red_o = reinterpret_cast<float*>(smem_raw);            // [8 warps][16][DV]
    float* red_ml = red_o + 8 * 16 * DV;                          // [8 warps][16][2]
    float* merged = red_ml + 8 * 16 * 2;                          // [2 maps][16][DV], normalised
#pragma unroll
    for (int h = 0; h < kHalves; ++h)
#pragma unroll
        for (int j = 0; j < DV / 16; ++j) {
            float* at = red_o + ((size_t)warp * 16 + h * 8 + (lane & 3) * 2) * DV + j * 16 + (lane >> 2);
            at[0] = o[h][j][0];
            at[DV] = o[h][j][1];
            at[8] = o[h][j][2];
            at[DV + 8] = o[h][j][3];
        }
    if ((lane & 3) == 0) {
        red_ml[(warp * 16 + row_a) * 2] = m_a; red_ml[(warp * 16 + row_a) * 2 + 1] = l_a;
        if constexpr (kHalves == 2) {
            red_ml[(warp * 16 + row_b) * 2] = m_b; red_ml[(warp * 16 + row_b) * 2 + 1] = l_b;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < 2 * group * DV; idx += kDiffThreads) {
        const int mp = idx / (group * DV), rest = idx - mp * group * DV;
        const int g = rest / DV, j = rest - g * DV;
        float m_star = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m_star = fmaxf(m_star, red_ml[((mp * 4 + w) * 16 + g) * 2]);
        float acc = 0.0f, l_sum = 0.0f;
        if (m_star != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float weight = exp2f(red_ml[((mp * 4 + w) * 16 + g) * 2] - m_star);
                acc += weight * red_o[((size_t)(mp * 4 + w) * 16 + g) * DV + j];
                l_sum += weight * red_ml[((mp * 4 + w) * 16 + g) * 2 + 1];
            }
        }
        if (splits == 1) {
            merged[(mp * 16 + g) * DV + j] = l_sum > 0.0f ? acc / l_sum : 0.0f;
        } else {
            const size_t row = (((size_t)request * nq + (size_t)kv_head * group + g) * 2 + mp) * splits + split;
            partial_o[row * DV + j] = acc;
            if (j == 0) {
                partial_ml[row * 2] = m_star;
                partial_ml[row * 2 + 1] = l_sum;
            }
        }
    }
    if (splits > 1) return;
    __syncthreads();
    for (int g = warp; g < group; g += kDiffThreads / 32) {
        const float* a1 = merged + g * DV;
        const float* a2 = merged + (16 + g) * DV;
        float squares = 0.0f;
        for (int j = lane; j < DV; j += 32) {
            const float d = fmaf(-p.lambda, a2[j], a1[j]);
            squares = fmaf(d, d, squares);
        }
        const float factor = rsqrtf(warp_sum(squares) / (float)DV + p.eps) * p.out_scale;
        bf16* dst = out + ((size_t)request * nq + (size_t)kv_head * group + g) * DV;
        for (int j = lane; j < DV; j += 32) dst[j] = __float2bfloat16_rn(fmaf(-p.lambda, a2[j], a1[j]) * factor);
    }
}

// One block per (token, query head): the splits of each map merged, then the difference and its norm.
template <int DV>
__global__ void __launch_bounds__(128) diff_merge_splits_kernel(
    const float* __restrict__ partial_o, const float* __restrict__ partial_ml, bf16* __restrict__ out, int splits,
    float lambda, float eps, float out_scale) {
    __shared__ float scratch[33];
    overlap_trigger();
    overlap_wait();
    const size_t head = blockIdx.x;
    constexpr int kHeld = (DV + 127) / 128;
    float m_star[2] = {-INFINITY, -INFINITY}, l_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        const float* ml = partial_ml + (head * 2 + mp) * splits * 2;
        for (int s = 0; s < splits; ++s) m_star[mp] = fmaxf(m_star[mp], ml[s * 2]);
        if (m_star[mp] != -INFINITY)
            for (int s = 0; s < splits; ++s) l_sum[mp] += exp2f(ml[s * 2] - m_star[mp]) * ml[s * 2 + 1];
    }
    float d[kHeld], squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
        const int j = threadIdx.x + i * 128;
        d[i] = 0.0f;
        if (j < DV) {
            float a[2];
#pragma unroll
            for (int mp = 0; mp < 2; ++mp) {
                const float* ml = partial_ml + (head * 2 + mp) * splits * 2;
                const float* po = partial_o + (head * 2 + mp) * splits * DV;
                float acc = 0.0f;
                if (m_star[mp] != -INFINITY)
                    for (int s = 0; s < splits; ++s) acc += exp2f(ml[s * 2] - m_star[mp]) * po[(size_t)s * DV + j];
                a[mp] = l_sum[mp] > 0.0f ? acc / l_sum[mp] : 0.0f;
            }
            d[i] = fmaf(-lambda, a[1], a[0]);
        }
        squares = fmaf(d[i], d[i], squares);
    }
    const float factor = rsqrtf(block_sum(squares, scratch) / (float)DV + eps) * out_scale;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
        const int j = threadIdx.x + i * 128;
        if (j < DV) out[head * DV + j] = __float2bfloat16_rn(d[i] * factor);
    }
}

template <int D, int DV>
constexpr int diff_decode_smem() {
    constexpr int stages = kDiffDecodeStages * diff_stage_elements<D, DV>() * (int)sizeof(bf16) +
                           kDiffDecodeStages * kKeys * (int)sizeof(long long);
    constexpr int merge = (8 * 16 * DV + 8 * 16 * 2 + 2 * 16 * DV) * (int)sizeof(float);
    return stages > merge ? stages : merge;
}

template <int D, int DV>
int launch_diff_decode_mma(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial_o,
                           float* partial_ml, const DiffMmaArgs& p, int splits, cudaStream_t stream) {
    // up to eight query heads to a key/value head fill one half of a fragment's rows
    auto kernel = p.nq / p.nkv > 8 ? diff_decode_mma_kernel<D, DV, 2> : diff_decode_mma_kernel<D, DV, 1>;
    constexpr int smem = diff_decode_smem<D, DV>();
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (status != cudaSuccess) return fail("diff_decode_attention", cudaGetErrorString(status));
    dim3 grid(splits, p.nkv, p.num_requests);
    launch_overlapped(kernel, grid, kDiffThreads, smem, stream, (const bf16*)q, (const bf16*)k_pages,
                      (const bf16*)v_pages, (bf16*)out, partial_o, partial_ml, p, splits);
    if (int rc = check_launch("diff_decode_attention")) return rc;
    if (splits > 1) {
        launch_overlapped(diff_merge_splits_kernel<DV>, p.num_requests * p.nq, 128, 0, stream,
                          (const float*)partial_o, (const float*)partial_ml, (bf16*)out, splits, p.lambda, p.eps,
                          p.out_scale);
        return check_launch("diff_merge_splits");
    }
    return 0;
}

}  // namespace b200
