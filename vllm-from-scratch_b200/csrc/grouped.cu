// Products in groups, and what a routed feed-forward needs around them.
//
//   route_experts      router logits in float32, sigmoid scores (or a softmax over all of them), a correction added for the choice
//                      only, the best groups of neighbouring experts, the `top` best experts of
//                      those groups; weights are the plain scores of the chosen, or those divided by their sum
//   expert_lists       from the chosen experts of every token: how many rows each expert has, where
//                      its rows begin, and each (token, choice) pair's row
//   grouped_gemm       C_g = A_g W_g^T for every group g, W_g [N, K] row-major.  The rows of a group
//                      are either the same rows for every group at a column offset of its own (heads:
//                      A and C hold the groups side by side in every row) or a list per group (experts:
//                      rows gathered from the tokens, written one after another).  bfloat16: mma.sync
//                      m16n8k16 with float32 accumulation; float32: fused multiply-adds in the order
//                      of k.  GATED: W_g holds 2 N rows, gate rows first, and C = act(gate) * up.
//                      Two forms in bfloat16: tiles of 32 x 64 staged through shared memory, and, for the
//                      few rows of a decode step, many small blocks that stream the matrices (see
//                      grouped_few_rows_bf16_kernel)
//   gather_rows        the tokens' rows list by list, for a library product that wants them side by side
//   combine_experts    y_t = sum over a token's choices of weight * its row, in float32, in the
//                      order of the choices
//   capped_swish_mul   out = g * sigmoid(slope g) * (u + offset), g = min(gate, limit), u = clamp(up)
//   gelu_gate_rows     out = gelu_tanh(g) * table[id, column ...]
//
// A row's result never depends on which other rows share its tile: every output element is one
// chain of products over k in a fixed order.
#include "common.cuh"

namespace b200 {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float sigmoid_fn(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ float4 load_four(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load_four(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
}

__device__ __forceinline__ void store_four(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store_four(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// ------------------------------------------------------------------------------- routing
// (value, index) pairs in the order "larger value first, then smaller index": true if a comes before b.
__device__ __forceinline__ bool ahead(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

template <typename T>
__global__ void route_experts_kernel(const T* __restrict__ x, const float* __restrict__ router,
                                     const float* __restrict__ correction, int* __restrict__ ids,
                                     float* __restrict__ weights, int K, int E, int top, int group_count,
                                     int group_keep, int group_top, int softmax_scores, int renormalise) {
    overlap_trigger();
    overlap_wait();
    extern __shared__ float route_smem[];
    float* score = route_smem;              // [E] sigmoid of the logit, or the softmax over all logits
    float* choice = score + E;              // [E] score + correction, -inf outside the kept groups
    float* marks = choice + E;              // [group_count]
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* row = x + (size_t)token * K;
    // Four consecutive elements a lane and step where the rows allow it (every lane's partial sums and the
    // order in which they are added depend on K alone, so a token's logits do not depend on the batch).
    const bool vector_ok = (K % 4 == 0) && (((uintptr_t)router | (uintptr_t)x) & 15) == 0 && ((K * sizeof(T)) % 8 == 0);
    for (int e = warp; e < E; e += warps) {
        const float* w = router + (size_t)e * K;
        float sum = 0.0f;
        if (vector_ok) {
            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 8
            for (int k = lane * 4; k < K; k += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + k);
                const float4 xv = load_four(row + k);
                part[0] = fmaf(wv.x, xv.x, part[0]); part[1] = fmaf(wv.y, xv.y, part[1]);
                part[2] = fmaf(wv.z, xv.z, part[2]); part[3] = fmaf(wv.w, xv.w, part[3]);
            }
            sum = (part[0] + part[1]) + (part[2] + part[3]);
        } else {
            for (int k = lane; k < K; k += 32) sum = fmaf(w[k], to_float(row[k]), sum);
        }
        sum = warp_sum(sum);
        if (lane == 0) score[e] = softmax_scores ? sum : sigmoid_fn(sum);
    }
    __syncthreads();
    if (softmax_scores) {
        // one warp: the largest logit, the sum of the exponentials (every lane's share and the order of the
        // lanes depend on E alone), then every score
        if (warp == 0) {
            float top_logit = -INFINITY;
            for (int e = lane; e < E; e += 32) top_logit = fmaxf(top_logit, score[e]);
            top_logit = warp_max(top_logit);
            float total = 0.0f;
            for (int e = lane; e < E; e += 32) total += expf(score[e] - top_logit);
            total = warp_sum(total);
            for (int e = lane; e < E; e += 32) score[e] = expf(score[e] - top_logit) / total;
        }
        __syncthreads();
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) choice[e] = correction ? score[e] + correction[e] : score[e];
    __syncthreads();
    if (group_count > 1 && group_keep < group_count) {
        const int per = E / group_count;
        for (int g = threadIdx.x; g < group_count; g += blockDim.x) {
            // the sum of the group's `group_top` largest choice scores
            float sum = 0.0f, pv = INFINITY;
            int pi = -1;
            for (int j = 0; j < group_top && j < per; ++j) {
                float bv = -INFINITY;
                int bi = -1;
                for (int i = 0; i < per; ++i) {
                    const float v = choice[g * per + i];
                    if (!(pi < 0 || ahead(pv, pi, v, i))) continue;       // taken already
                    if (bi < 0 || ahead(v, i, bv, bi)) { bv = v; bi = i; }
                }
                sum += bv;
                pv = bv;
                pi = bi;
            }
            marks[g] = sum;
        }
        __syncthreads();
        // A group is kept if fewer than `group_keep` groups come before it.
        for (int g = threadIdx.x; g < group_count; g += blockDim.x) {
            int before = 0;
            for (int o = 0; o < group_count; ++o)
                if (o != g && ahead(marks[o], o, marks[g], g)) ++before;
            if (before >= group_keep)
                for (int i = 0; i < per; ++i) choice[g * per + i] = -INFINITY;
        }
        __syncthreads();
    }
    if (warp != 0) return;
    float pv = INFINITY, chosen_sum = 0.0f;
    int pi = -1;
    for (int j = 0; j < top; ++j) {
        float bv = -INFINITY;
        int bi = -1;
        for (int e = lane; e < E; e += 32) {
            const float v = choice[e];
            if (!(pi < 0 || ahead(pv, pi, v, e))) continue;
            if (bi < 0 || ahead(v, e, bv, bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, offset);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, offset);
            if (oi >= 0 && (bi < 0 || ahead(ov, oi, bv, bi))) { bv = ov; bi = oi; }
        }
        if (bi < 0) bi = 0;         // fewer candidates than choices: cannot happen with top <= E
        if (lane == 0) {
            ids[(size_t)token * top + j] = bi;
            weights[(size_t)token * top + j] = score[bi];
        }
        chosen_sum += score[bi];            // every lane holds the same choice: one sum in the order of the choices
        pv = bv;
        pi = bi;
    }
    if (renormalise && lane == 0)
        for (int j = 0; j < top; ++j)
            weights[(size_t)token * top + j] = score[ids[(size_t)token * top + j]] / (chosen_sum + 1e-20f);
}

// One block.  offsets [E + 1]; sorted_pair [pairs]: the pairs (token * top + choice) expert by expert;
// position [pairs]: the row of each pair.
__global__ void expert_lists_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ offsets,
                                    int* __restrict__ sorted_pair, int* __restrict__ position) {
    overlap_trigger();
    overlap_wait();
    extern __shared__ int list_smem[];
    int* counts = list_smem;                // [E], then the running cursor of each expert
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int running = 0;
        for (int e = 0; e < E; ++e) {
            const int count = counts[e];
            offsets[e] = running;
            counts[e] = running;
            running += count;
        }
        offsets[E] = running;
    }
    __syncthreads();
    // Pairs whose expert has no list (a number outside [0, E)) leave rows past the last list unused: they
    // name the first pair, so that whoever gathers rows by this list reads a row that exists.
    for (int p = offsets[E] + threadIdx.x; p < pairs; p += blockDim.x) sorted_pair[p] = 0;
    // Pairs of one expert keep no particular order among themselves; a row's result does not depend
    // on where in its expert's list it stands.
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e < 0 || e >= E) { position[p] = -1; continue; }
        const int row = atomicAdd(&counts[e], 1);
        sorted_pair[row] = p;
        position[p] = row;
    }
}

template <typename T>
__global__ void combine_experts_kernel(const T* __restrict__ rows, const int* __restrict__ position,
                                       const float* __restrict__ weights, T* __restrict__ out, int width, int top,
                                       const int* __restrict__ ids, const T* __restrict__ x, int experts,
                                       const T* __restrict__ extra) {
    overlap_trigger();
    overlap_wait();
    const int token = blockIdx.x;
    // A pair without a row: an identity expert where its number lies behind the experts that have matrices
    // (its output is the token's own input row), else nothing.
    if (width % 4 == 0 && (((uintptr_t)rows | (uintptr_t)out | (uintptr_t)x | (uintptr_t)extra) & 15) == 0) {
        // four columns a thread and step: the same sums in the same order, fewer and wider loads
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < top; ++j) {
                const int row = position[(size_t)token * top + j];
                if (row < 0 && !(x != nullptr && ids[(size_t)token * top + j] >= experts)) continue;
                const float w = weights ? weights[(size_t)token * top + j] : 1.0f;
                const float4 v = row < 0 ? load_four(x + (size_t)token * width + i) : load_four(rows + (size_t)row * width + i);
                sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y);
                sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
            }
            if (extra != nullptr) {
                const float4 v = load_four(extra + (size_t)token * width + i);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            store_four(out + (size_t)token * width + i, sum);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float sum = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int row = position[(size_t)token * top + j];
            const float w = weights ? weights[(size_t)token * top + j] : 1.0f;
            if (row >= 0) sum = fmaf(w, to_float(rows[(size_t)row * width + i]), sum);
            else if (x != nullptr && ids[(size_t)token * top + j] >= experts)
                sum = fmaf(w, to_float(x[(size_t)token * width + i]), sum);
        }
        if (extra != nullptr) sum += to_float(extra[(size_t)token * width + i]);
        out[(size_t)token * width + i] = from_float<T>(sum);
    }
}

// out[r] = x[index[r] / divisor]: the tokens' rows in the order of the experts' lists, for a product that
// wants every list's rows side by side.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ index, int divisor,
                                   T* __restrict__ out, int width) {
    const size_t row = blockIdx.x;
    const T* src = x + (size_t)(index[row] / divisor) * width;
    T* dst = out + row * width;
    const int per = 16 / (int)sizeof(T);
    if (width % per == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        for (int i = threadIdx.x; i < width / per; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

// ----------------------------------------------------------------------- grouped products
struct GroupedArgs {
    const void* a;          // rows of A
    const void* w;          // [groups][N (2 N when gated)][K]
    void* c;
    const int* offsets;     // [groups + 1] first row of each group's list, or null: every group has `rows` rows
    const int* row_index;   // [rows of all lists] -> index, divided by `index_divisor` = row of A; null: the list's row
    int index_divisor;
    int rows;               // rows of a group without lists
    int groups;
    int N, K;
    long long lda, ldc;     // elements between rows of A and of C
    long long a_group, c_group;     // elements between groups within a row
    float act_limit, act_slope, act_offset;     // gated epilogue, see gated_value
    int act_kind;           // 0: silu(gate) * up; 1: capped: g sigmoid(slope g) (u + offset)
    // A factor per row on the products, ahead of the rounding and of the activation (an expert that is given
    // weight * x instead of x): indexed like row_index's entries where there is an index, else by the list's row.
    const float* row_scale;
};

__device__ __forceinline__ float row_scale_of(const GroupedArgs& p, int list_row) {
    if (p.row_scale == nullptr) return 1.0f;
    return p.row_scale[p.row_index ? p.row_index[list_row] : list_row];
}

__device__ __forceinline__ float gated_value(float gate, float up, const GroupedArgs& p) {
    if (p.act_kind == 0) return gate * sigmoid_fn(gate) * up;
    const float g = fminf(gate, p.act_limit);
    const float u = fminf(fmaxf(up, -p.act_limit), p.act_limit);
    return g * sigmoid_fn(p.act_slope * g) * (u + p.act_offset);
}

constexpr int kBM = 32, kBN = 64, kThreadsG = 128;

// Which group and which tile of its rows a block has: group g owns blocks [first(g), first(g + 1)) with
// first(g) = offsets[g] / kBM + g, which leaves every group ceil(rows / kBM) blocks at least.
template <int BM = kBM>
__device__ __forceinline__ bool find_tile(const GroupedArgs& p, int block, int& group, int& row0, int& rows_here,
                                          int& list_base) {
    if (p.offsets == nullptr) {
        const int tiles = (p.rows + BM - 1) / BM;
        group = block / tiles;
        row0 = (block - group * tiles) * BM;
        list_base = 0;
        rows_here = min(BM, p.rows - row0);
        return group < p.groups && rows_here > 0;
    }
    int lo = 0, hi = p.groups - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.offsets[mid] / BM + mid <= block) lo = mid; else hi = mid - 1;
    }
    group = lo;
    list_base = p.offsets[group];
    const int count = p.offsets[group + 1] - list_base;
    row0 = (block - (list_base / BM + group)) * BM;
    rows_here = min(BM, count - row0);
    return rows_here > 0;
}

__device__ __forceinline__ long long a_row_of(const GroupedArgs& p, int list_row) {
    return p.row_index ? (long long)(p.row_index[list_row] / p.index_divisor) : (long long)list_row;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Eight consecutive bfloat16 of a row of K elements beginning at k; zeros past the end.
__device__ __forceinline__ uint4 load8(const bf16* row, int k, int K, bool vector_ok) {
    if (row == nullptr || k >= K) return make_uint4(0, 0, 0, 0);
    if (vector_ok && k + 8 <= K) return *reinterpret_cast<const uint4*>(row + k);
    union { uint4 v; bf16 e[8]; } u;
#pragma unroll
    for (int i = 0; i < 8; ++i) u.e[i] = k + i < K ? row[k + i] : __float2bfloat16_rn(0.0f);
    return u.v;
}

template <bool GATED>
__global__ void __launch_bounds__(kThreadsG) grouped_gemm_bf16_kernel(const GroupedArgs p) {
    overlap_trigger();
    overlap_wait();
    constexpr int BK = 64, LD = BK + 8;
    constexpr int NB = GATED ? 2 : 1;
    __shared__ __align__(16) bf16 a_s[kBM][LD];
    __shared__ __align__(16) bf16 b_s[NB][kBN][LD];
    int group, row0, rows_here, list_base;
    if (!find_tile(p, blockIdx.x, group, row0, rows_here, list_base)) return;
    const int n0 = blockIdx.y * kBN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    const int K = p.K, N = p.N;
    const bf16* a = (const bf16*)p.a + (long long)group * p.a_group;
    const bf16* w = (const bf16*)p.w + (long long)group * (long long)(NB * N) * K;
    const bool vector_ok = (K % 8 == 0) && (p.lda % 8 == 0) && (p.a_group % 8 == 0)
                           && (((uintptr_t)p.a | (uintptr_t)p.w) & 15) == 0;

    // This thread's share of a tile: two pieces of eight of a row of A, and of two rows of each B.
    const int a_r = tid >> 2, a_k = (tid & 3) * 16;
    const bf16* a_src = a_r < rows_here ? a + a_row_of(p, list_base + row0 + a_r) * p.lda : nullptr;
    const bf16* b_src[NB][2];
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int n = n0 + (tid >> 2) + 32 * i;
            b_src[h][i] = n < N ? w + ((long long)h * N + n) * K : nullptr;
        }
    float acc[NB][4][4];
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int t = 0; t < 4; ++t) acc[h][t][0] = acc[h][t][1] = acc[h][t][2] = acc[h][t][3] = 0.0f;

    uint4 a_next[2], b_next[NB][2][2];
    auto fetch = [&](int k) {
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
            a_next[piece] = load8(a_src, k + a_k + 8 * piece, K, vector_ok);
#pragma unroll
            for (int h = 0; h < NB; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i) b_next[h][i][piece] = load8(b_src[h][i], k + a_k + 8 * piece, K, vector_ok);
        }
    };
    fetch(0);

    const int g = lane >> 2, t4 = lane & 3;
    for (int k0 = 0; k0 < K; k0 += BK) {
        __syncthreads();
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
            *reinterpret_cast<uint4*>(&a_s[a_r][a_k + 8 * piece]) = a_next[piece];
#pragma unroll
            for (int h = 0; h < NB; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    *reinterpret_cast<uint4*>(&b_s[h][(tid >> 2) + 32 * i][a_k + 8 * piece]) = b_next[h][i][piece];
        }
        __syncthreads();
        if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            unsigned af[4];
            af[0] = *reinterpret_cast<const unsigned*>(&a_s[wm * 16 + g][kk + 2 * t4]);
            af[1] = *reinterpret_cast<const unsigned*>(&a_s[wm * 16 + g + 8][kk + 2 * t4]);
            af[2] = *reinterpret_cast<const unsigned*>(&a_s[wm * 16 + g][kk + 2 * t4 + 8]);
            af[3] = *reinterpret_cast<const unsigned*>(&a_s[wm * 16 + g + 8][kk + 2 * t4 + 8]);
#pragma unroll
            for (int h = 0; h < NB; ++h)
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int n = wn * 32 + t * 8 + g;
                    const unsigned b0 = *reinterpret_cast<const unsigned*>(&b_s[h][n][kk + 2 * t4]);
                    const unsigned b1 = *reinterpret_cast<const unsigned*>(&b_s[h][n][kk + 2 * t4 + 8]);
                    mma_bf16(acc[h][t], af, b0, b1);
                }
        }
    }

    bf16* c = (bf16*)p.c + (long long)group * p.c_group;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = wm * 16 + g + 8 * half;
        if (r >= rows_here) continue;
        bf16* dst = c + (long long)(list_base + row0 + r) * p.ldc;
        const float factor = row_scale_of(p, list_base + row0 + r);
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = n0 + wn * 32 + t * 8 + 2 * t4 + e;
                if (n >= N) continue;
                float v = acc[0][t][2 * half + e] * factor;
                if (GATED) {
                    // both products are rounded as a projection's output is, then the activation in float32
                    const float gate = __bfloat162float(__float2bfloat16_rn(v));
                    const float up = __bfloat162float(__float2bfloat16_rn(acc[NB - 1][t][2 * half + e] * factor));
                    v = gated_value(gate, up, p);
                }
                dst[n] = __float2bfloat16_rn(v);
            }
    }
}

// Few rows over all lists (a decode step): the time is the stream of the matrices, so a block takes 16 rows
// of a list against only 16 columns (gated: 16 gate and 16 up rows of the matrix) over all of K, its four
// warps a quarter of the k-steps each, and every lane asks for its fragments of four k-steps (up to 24 loads
// of 16 bytes) before it multiplies: many small blocks with much in flight.  Fragments come straight from
// global memory: a lane's 16 bytes of a row are the operands of two m16n8k16 products, with the sixteen k of
// a product taken in the order in which the lanes hold them, the same for both operands.  The warps' sums
// meet in shared memory and are added in the order of the warps.  K a multiple of 32, rows 16-byte aligned.
constexpr int kFM = 16, kFN = 16;

// 16 bytes that are read once.  `volatile` keeps the loads of a lane in the order written, ahead of the
// products (which are `volatile` too): the compiler would otherwise hold back some of them to save registers.
__device__ __forceinline__ uint4 load_stream16(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
constexpr int kFewRowsMost = 128; // rows (of all lists; of a group without lists) up to which it is used

template <bool GATED>
__global__ void __launch_bounds__(kThreadsG, 3) grouped_few_rows_bf16_kernel(const GroupedArgs p) {
    overlap_trigger();
    overlap_wait();
    constexpr int NB = GATED ? 2 : 1, NT = kFN / 8, U = 4;
    __shared__ float red[4][NB][kFM][kFN + 1];
    int group, row0, rows_here, list_base;
    if (!find_tile<kFM>(p, blockIdx.x, group, row0, rows_here, list_base)) return;
    const int n0 = blockIdx.y * kFN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int K = p.K, N = p.N;
    const bf16* a = (const bf16*)p.a + (long long)group * p.a_group;
    const bf16* w = (const bf16*)p.w + (long long)group * (long long)(NB * N) * K;
    // A row that does not exist is read from one that does (the tile's first, the matrix's first): every
    // lane then issues the same loads, all of them before the first product.  What such a row gives lands
    // in a row or a column of the result that is not stored (a row of the result depends on its own row of
    // A alone, a column on its own row of W).
    const bool has_lo = g < rows_here, has_hi = g + 8 < rows_here;
    const bf16* a_lo = a + a_row_of(p, list_base + row0 + (has_lo ? g : 0)) * p.lda;
    const bf16* a_hi = a + a_row_of(p, list_base + row0 + (has_hi ? g + 8 : 0)) * p.lda;
    const bf16* b_row[NB][NT];
    bool has_b[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) has_b[nt] = n0 + nt * 8 + g < N;
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            b_row[h][nt] = w + ((long long)h * N + (has_b[nt] ? n0 + nt * 8 + g : 0)) * K;
    float acc[NB][NT][4];
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[h][nt][0] = acc[h][nt][1] = acc[h][nt][2] = acc[h][nt][3] = 0.0f;

    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int steps = K / 32;
    for (int s0 = warp; s0 < steps; s0 += 4 * U) {
        uint4 av[U][2], bv[U][NB][NT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + 4 * u;
            const int k = s * 32 + t4 * 8;
            if (s < steps) {            // the same for all lanes of the warp
#pragma unroll
                for (int h = 0; h < NB; ++h)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) bv[u][h][nt] = load_stream16(b_row[h][nt] + k);
                av[u][0] = load_stream16(a_lo + k);
                av[u][1] = load_stream16(a_hi + k);
            } else {
#pragma unroll
                for (int h = 0; h < NB; ++h)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) bv[u][h][nt] = zero;
                av[u][0] = av[u][1] = zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned first[4] = {av[u][0].x, av[u][1].x, av[u][0].y, av[u][1].y};
            const unsigned second[4] = {av[u][0].z, av[u][1].z, av[u][0].w, av[u][1].w};
#pragma unroll
            for (int h = 0; h < NB; ++h)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_bf16(acc[h][nt], first, bv[u][h][nt].x, bv[u][h][nt].y);
                    mma_bf16(acc[h][nt], second, bv[u][h][nt].z, bv[u][h][nt].w);
                }
        }
    }
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][h][g][nt * 8 + 2 * t4] = acc[h][nt][0];
            red[warp][h][g][nt * 8 + 2 * t4 + 1] = acc[h][nt][1];
            red[warp][h][g + 8][nt * 8 + 2 * t4] = acc[h][nt][2];
            red[warp][h][g + 8][nt * 8 + 2 * t4 + 1] = acc[h][nt][3];
        }
    __syncthreads();
    bf16* c = (bf16*)p.c + (long long)group * p.c_group;
    for (int idx = tid; idx < kFM * kFN; idx += kThreadsG) {
        const int r = idx / kFN, col = idx - r * kFN;
        if (r >= rows_here || n0 + col >= N) continue;
        float v[NB];
#pragma unroll
        for (int h = 0; h < NB; ++h) v[h] = ((red[0][h][r][col] + red[1][h][r][col]) + red[2][h][r][col]) + red[3][h][r][col];
        if (p.row_scale != nullptr) {
            const float factor = row_scale_of(p, list_base + row0 + r);
#pragma unroll
            for (int h = 0; h < NB; ++h) v[h] *= factor;
        }
        float value = v[0];
        if (GATED)
            value = gated_value(__bfloat162float(__float2bfloat16_rn(v[0])), __bfloat162float(__float2bfloat16_rn(v[NB - 1])), p);
        c[(long long)(list_base + row0 + r) * p.ldc + n0 + col] = __float2bfloat16_rn(value);
    }
}

template <bool GATED>
__global__ void __launch_bounds__(kThreadsG) grouped_gemm_f32_kernel(const GroupedArgs p) {
    overlap_trigger();
    overlap_wait();
    constexpr int BK = 16;
    constexpr int NB = GATED ? 2 : 1;
    __shared__ float a_s[kBM][BK + 1];
    __shared__ float b_s[NB][kBN][BK + 1];
    int group, row0, rows_here, list_base;
    if (!find_tile(p, blockIdx.x, group, row0, rows_here, list_base)) return;
    const int n0 = blockIdx.y * kBN;
    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;         // rows ty * 4 + i, columns tx + 16 * j
    const int K = p.K, N = p.N;
    const float* a = (const float*)p.a + (long long)group * p.a_group;
    const float* w = (const float*)p.w + (long long)group * (long long)(NB * N) * K;
    float acc[NB][4][4];
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        __syncthreads();
        for (int idx = tid; idx < kBM * BK; idx += kThreadsG) {
            const int r = idx / BK, k = idx - r * BK;
            float v = 0.0f;
            if (r < rows_here && k0 + k < K) v = a[a_row_of(p, list_base + row0 + r) * p.lda + k0 + k];
            a_s[r][k] = v;
        }
#pragma unroll
        for (int h = 0; h < NB; ++h)
            for (int idx = tid; idx < kBN * BK; idx += kThreadsG) {
                const int n = idx / BK, k = idx - n * BK;
                float v = 0.0f;
                if (n0 + n < N && k0 + k < K) v = w[((long long)h * N + n0 + n) * K + k0 + k];
                b_s[h][n][k] = v;
            }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = a_s[ty * 4 + i][k];
#pragma unroll
            for (int h = 0; h < NB; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float bv = b_s[h][tx + 16 * j][k];
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[h][i][j] = fmaf(av[i], bv, acc[h][i][j]);
                }
        }
    }
    float* c = (float*)p.c + (long long)group * p.c_group;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows_here) continue;
        float* dst = c + (long long)(list_base + row0 + r) * p.ldc;
        const float factor = row_scale_of(p, list_base + row0 + r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            dst[n] = GATED ? gated_value(acc[0][i][j] * factor, acc[NB - 1][i][j] * factor, p) : acc[0][i][j] * factor;
        }
    }
}

// ------------------------------------------------------------------------ elementwise
template <typename T>
__global__ void capped_swish_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, float limit,
                                        float slope, float offset, const float* __restrict__ row_scale,
                                        const int* __restrict__ row_index) {
    overlap_trigger();
    overlap_wait();
    const size_t token = blockIdx.x;
    const float f = row_scale ? row_scale[row_index ? row_index[token] : (int)token] : 1.0f;
    const T* row = gate_up + token * 2 * (size_t)inter;
    if (inter % 4 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < inter; i += gridDim.y * blockDim.x * 4) {
            const float4 gv = load_four(row + i), uv = load_four(row + inter + i);
            float4 r;
            float g, u;
            g = fminf(gv.x * f, limit); u = fminf(fmaxf(uv.x * f, -limit), limit); r.x = g * sigmoid_fn(slope * g) * (u + offset);
            g = fminf(gv.y * f, limit); u = fminf(fmaxf(uv.y * f, -limit), limit); r.y = g * sigmoid_fn(slope * g) * (u + offset);
            g = fminf(gv.z * f, limit); u = fminf(fmaxf(uv.z * f, -limit), limit); r.z = g * sigmoid_fn(slope * g) * (u + offset);
            g = fminf(gv.w * f, limit); u = fminf(fmaxf(uv.w * f, -limit), limit); r.w = g * sigmoid_fn(slope * g) * (u + offset);
            store_four(out + token * inter + i, r);
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
        const float g = fminf(to_float(row[i]) * f, limit);
        const float u = fminf(fmaxf(to_float(row[inter + i]) * f, -limit), limit);
        out[token * inter + i] = from_float<T>(g * sigmoid_fn(slope * g) * (u + offset));
    }
}

__device__ __forceinline__ float gelu_tanh_fn(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out = gelu_tanh(gate) * up for rows [gate | up]
template <typename T>
__global__ void gelu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
    overlap_trigger();
    overlap_wait();
    const size_t token = blockIdx.x;
    const T* row = gate_up + token * 2 * (size_t)inter;
    if (inter % 4 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < inter; i += gridDim.y * blockDim.x * 4) {
            const float4 gv = load_four(row + i), uv = load_four(row + inter + i);
            store_four(out + token * inter + i, make_float4(gelu_tanh_fn(gv.x) * uv.x, gelu_tanh_fn(gv.y) * uv.y,
                                                            gelu_tanh_fn(gv.z) * uv.z, gelu_tanh_fn(gv.w) * uv.w));
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x)
        out[token * inter + i] = from_float<T>(gelu_tanh_fn(to_float(row[i])) * to_float(row[inter + i]));
}

template <typename T>
__global__ void gelu_gate_rows_kernel(const T* __restrict__ gate, const T* __restrict__ table,
                                      const int* __restrict__ ids, T* __restrict__ out, int dim, int table_stride,
                                      int column, int vocab) {
    overlap_trigger();
    overlap_wait();
    const size_t token = blockIdx.x;
    const int id = ids[token];
    const bool known = id >= 0 && id < vocab;       // the embedding reports an id outside the table
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float e = known ? to_float(table[(size_t)id * table_stride + column + i]) : 0.0f;
        out[token * dim + i] = from_float<T>(gelu_tanh_fn(to_float(gate[token * dim + i])) * e);
    }
}

}  // namespace b200

// x [tokens, K] (dtype 0 float32, 1 bfloat16), router float32 [E, K], correction float32 [E] or null.
// ids int32 [tokens, top], weights float32 [tokens, top].  Groups: `group_count` equal groups of
// neighbouring experts, of which the `group_keep` with the largest sums of their `group_top` largest
// choice scores stay eligible (group_count <= 1 or group_keep >= group_count: all do).
B200_EXPORT int b200_route_experts(const void* x, const float* router, const float* correction, int* ids,
                                   float* weights, int tokens, int K, int E, int top, int group_count,
                                   int group_keep, int group_top, int softmax_scores, int renormalise, int dtype,
                                   cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if (E <= 0 || top <= 0 || top > E || K <= 0) return fail("route_experts", "sizes out of range");
    if (group_count < 1) group_count = 1;
    if (E % group_count) return fail("route_experts", "experts do not divide into equal groups");
    if (group_keep < 1 || group_top < 1) return fail("route_experts", "group_keep and group_top must be positive");
    if (top > (long long)min(group_keep, group_count) * (E / group_count))
        return fail("route_experts", "the kept groups hold fewer experts than are to be chosen");
    const size_t smem = sizeof(float) * (2 * (size_t)E + group_count);
    if (smem > 48 * 1024) return fail("route_experts", "too many experts for one block's shared memory");
    // a warp an expert where few tokens leave the SMs room for it
    const int threads = (tokens <= 4 * kOverlapMostRows && E > 4) ? 256 : 128;
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, route_experts_kernel<float>, tokens, threads, smem, stream,
            (const float*)x, router, correction, ids, weights, K, E, top, group_count, group_keep, group_top,
            softmax_scores, renormalise);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, route_experts_kernel<__nv_bfloat16>, tokens, threads, smem, stream,
            (const __nv_bfloat16*)x, router, correction, ids, weights, K, E, top, group_count, group_keep, group_top,
            softmax_scores, renormalise);
    else
        return fail("route_experts", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("route_experts");
}

B200_EXPORT int b200_expert_lists(const int* ids, int pairs, int E, int* offsets, int* sorted_pair, int* position,
                                  cudaStream_t stream) {
    using namespace b200;
    if (E <= 0 || pairs < 0) return fail("expert_lists", "sizes out of range");
    if ((size_t)E * sizeof(int) > 48 * 1024) return fail("expert_lists", "too many experts for one block's shared memory");
    launch_overlapped_if(pairs <= 8 * kOverlapMostRows, expert_lists_kernel, 1, pairs > 256 ? 1024 : 256,
                         (size_t)E * sizeof(int), stream, ids, pairs, E, offsets, sorted_pair, position);
    return check_launch("expert_lists");
}

B200_EXPORT int b200_gather_rows(const void* x, const int* index, int divisor, void* out, int rows, int width,
                                 int dtype, cudaStream_t stream) {
    using namespace b200;
    if (rows == 0) return 0;
    if (divisor <= 0 || width <= 0) return fail("gather_rows", "sizes out of range");
    if (dtype == 0)
        gather_rows_kernel<float><<<rows, 128, 0, stream>>>((const float*)x, index, divisor, (float*)out, width);
    else if (dtype == 1)
        gather_rows_kernel<__nv_bfloat16><<<rows, 128, 0, stream>>>((const __nv_bfloat16*)x, index, divisor,
                                                                  (__nv_bfloat16*)out, width);
    else
        return fail("gather_rows", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("gather_rows");
}

// ids, x, experts: pairs whose expert number is `experts` or more are identity experts, whose output is the
// token's row of x (both null: there are none).  extra [tokens, width] or null: rows added to every token's sum.
// weights null: every weight is 1 (experts whose weight went into their input).
B200_EXPORT int b200_combine_experts(const void* rows, const int* position, const float* weights, void* out,
                                     int tokens, int width, int top, const int* ids, const void* x, int experts,
                                     const void* extra, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if ((ids == nullptr) != (x == nullptr)) return fail("combine_experts", "identity experts need the choices and the inputs");
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, combine_experts_kernel<float>, tokens, threads, 0, stream,
            (const float*)rows, position, weights, (float*)out, width, top, ids, (const float*)x, experts, (const float*)extra);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, combine_experts_kernel<__nv_bfloat16>, tokens, threads, 0, stream,
            (const __nv_bfloat16*)rows, position, weights, (__nv_bfloat16*)out, width, top, ids, (const __nv_bfloat16*)x, experts,
            (const __nv_bfloat16*)extra);
    else
        return fail("combine_experts", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("combine_experts");
}

// See GroupedArgs.  `list_rows`: with offsets, the number of rows over all lists (it bounds the grid).
// gated: 0 plain; 1 silu(gate) * up; 2 the capped form with (limit, slope, offset).
// row_scale: float32 factors on the rows of the product (see GroupedArgs), or null.
B200_EXPORT int b200_grouped_gemm_scaled(const void* a, const void* w, void* c, const int* offsets, const int* row_index,
                                         int index_divisor, int rows, int list_rows, int groups, int N, int K,
                                         long long lda, long long ldc, long long a_group, long long c_group, int gated,
                                         float limit, float slope, float offset, const float* row_scale, int dtype,
                                         cudaStream_t stream) {
    using namespace b200;
    if (groups <= 0 || N <= 0 || K <= 0) return fail("grouped_gemm", "sizes out of range");
    if (row_index != nullptr && (offsets == nullptr || index_divisor <= 0))
        return fail("grouped_gemm", "a row index goes with lists and a positive divisor");
    long long tiles;
    if (offsets == nullptr) {
        if (rows <= 0) return 0;
        tiles = (long long)groups * ((rows + kBM - 1) / kBM);
    } else {
        if (list_rows <= 0) return 0;
        tiles = list_rows / kBM + groups;
    }
    const int n_tiles = (N + kBN - 1) / kBN;
    if (tiles > 2147483647LL || n_tiles > 65535) return fail("grouped_gemm", "grid out of range");
    GroupedArgs p;
    p.a = a; p.w = w; p.c = c; p.offsets = offsets; p.row_index = row_index; p.index_divisor = index_divisor;
    p.rows = rows; p.groups = groups; p.N = N; p.K = K; p.lda = lda; p.ldc = ldc; p.a_group = a_group;
    p.c_group = c_group; p.act_limit = limit; p.act_slope = slope; p.act_offset = offset;
    p.act_kind = gated == 2 ? 1 : 0;
    p.row_scale = row_scale;
    const dim3 grid((unsigned)tiles, n_tiles);
    const int most_rows = offsets ? list_rows : rows;       // of all lists; of every group without lists
    const bool overlap = most_rows <= kOverlapMostRows;
    // Few rows: the stream of the matrices sets the time, and the kernel of many small blocks serves.
    if (dtype == 1 && most_rows <= kFewRowsMost && K % 32 == 0 && lda % 8 == 0 && a_group % 8 == 0
        && (((uintptr_t)a | (uintptr_t)w) & 15) == 0) {
        const long long few_tiles = offsets ? (long long)list_rows / kFM + groups : (long long)groups * ((rows + kFM - 1) / kFM);
        const dim3 few_grid((unsigned)few_tiles, (N + kFN - 1) / kFN);
        if (few_grid.y > 65535) return fail("grouped_gemm", "grid out of range");
        if (gated) launch_overlapped_if(overlap, grouped_few_rows_bf16_kernel<true>, few_grid, kThreadsG, 0, stream, p);
        else launch_overlapped_if(overlap, grouped_few_rows_bf16_kernel<false>, few_grid, kThreadsG, 0, stream, p);
        return check_launch("grouped_gemm");
    }
    if (dtype == 0) {
        if (gated) launch_overlapped_if(overlap, grouped_gemm_f32_kernel<true>, grid, kThreadsG, 0, stream, p);
        else launch_overlapped_if(overlap, grouped_gemm_f32_kernel<false>, grid, kThreadsG, 0, stream, p);
    } else if (dtype == 1) {
        if (gated) launch_overlapped_if(overlap, grouped_gemm_bf16_kernel<true>, grid, kThreadsG, 0, stream, p);
        else launch_overlapped_if(overlap, grouped_gemm_bf16_kernel<false>, grid, kThreadsG, 0, stream, p);
    } else {
        return fail("grouped_gemm", "dtype must be 0 (float32) or 1 (bfloat16)");
    }
    return check_launch("grouped_gemm");
}

B200_EXPORT int b200_grouped_gemm(const void* a, const void* w, void* c, const int* offsets, const int* row_index,
                                  int index_divisor, int rows, int list_rows, int groups, int N, int K,
                                  long long lda, long long ldc, long long a_group, long long c_group, int gated,
                                  float limit, float slope, float offset, int dtype, cudaStream_t stream) {
    return b200_grouped_gemm_scaled(a, w, c, offsets, row_index, index_divisor, rows, list_rows, groups, N, K, lda, ldc,
                                    a_group, c_group, gated, limit, slope, offset, nullptr, dtype, stream);
}

// row_scale (float32, or null) with row_index (int32, or null: the row itself): row r of gate_up is multiplied by
// row_scale[row_index[r]] ahead of the caps.
B200_EXPORT int b200_capped_swish_mul_scaled(const void* gate_up, void* out, int tokens, int inter, float limit,
                                             float slope, float offset, const float* row_scale, const int* row_index,
                                             int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0 || inter == 0) return 0;
    const dim3 grid(tokens, tokens >= 512 ? 1 : min(8, (inter + 1023) / 1024));
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, capped_swish_mul_kernel<float>, grid, 256, 0, stream,
            (const float*)gate_up, (float*)out, inter, limit, slope, offset, row_scale, row_index);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, capped_swish_mul_kernel<__nv_bfloat16>, grid, 256, 0, stream,
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, limit, slope, offset, row_scale, row_index);
    else
        return fail("capped_swish_mul", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("capped_swish_mul");
}

B200_EXPORT int b200_capped_swish_mul(const void* gate_up, void* out, int tokens, int inter, float limit,
                                      float slope, float offset, int dtype, cudaStream_t stream) {
    return b200_capped_swish_mul_scaled(gate_up, out, tokens, inter, limit, slope, offset, nullptr, nullptr, dtype, stream);
}

B200_EXPORT int b200_gelu_mul(const void* gate_up, void* out, int tokens, int inter, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0 || inter == 0) return 0;
    const dim3 grid(tokens, tokens >= 512 ? 1 : min(8, (inter + 1023) / 1024));
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, gelu_mul_kernel<float>, grid, 256, 0, stream,
            (const float*)gate_up, (float*)out, inter);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, gelu_mul_kernel<__nv_bfloat16>, grid, 256, 0, stream,
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
    else
        return fail("gelu_mul", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("gelu_mul");
}

B200_EXPORT int b200_gelu_gate_rows(const void* gate, const void* table, const int* ids, void* out, int tokens,
                                    int dim, int table_stride, int column, int vocab, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0 || dim == 0) return 0;
    if (column < 0 || column + dim > table_stride) return fail("gelu_gate_rows", "columns outside the table");
    const int threads = dim >= 256 ? 256 : (dim + 31) / 32 * 32;
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, gelu_gate_rows_kernel<float>, tokens, threads, 0, stream,
            (const float*)gate, (const float*)table, ids, (float*)out, dim, table_stride, column, vocab);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, gelu_gate_rows_kernel<__nv_bfloat16>, tokens, threads, 0, stream,
            (const __nv_bfloat16*)gate, (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, dim, table_stride,
            column, vocab);
    else
        return fail("gelu_gate_rows", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("gelu_gate_rows");
}
