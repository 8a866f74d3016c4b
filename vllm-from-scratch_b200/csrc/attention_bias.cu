// Paged causal attention whose positions enter as a bias on the scores instead of a rotation, with
// keys and values of sizes of their own, in float32 arithmetic throughout (scores, softmax weights
// and the weighted sum of the values), for float32 and bfloat16 projections and pages.
//
//   head_norm_scale_cache   per-head RMSNorm of queries and keys (one weight vector for all heads),
//                           queries multiplied by a temperature that grows with the position,
//                           1 + coef * ln(floor((p + 1) / every) + 1); keys and values into their pages
//   biased_paged_attention  score(i, j) = q_i . k_j * scale - slope_h * (i - j), softmax over j <= i
//                           (and j > i - window where there is one)
//
// The attention kernel has the launch shape and the masking of the generic kernel in
// attention_generic.cu: a block is 16 consecutive queries of one request and one query head, found
// from the block index alone; keys come through the block table in tiles of 32.
//
// For bfloat16 pages with keys and values of one size of 64, 128 or 256 the two tensor-core kernels of
// attention_bf16_kernels.cuh serve instead, in their form with float32 weights: the decode kernel
// (keys split over blocks, merged) for requests that bring one token, the 64-row kernel for portions.
#include "attention_bf16_kernels.cuh"

namespace b200 {

template <typename T>
__global__ void head_norm_scale_cache_kernel(
    const T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, T* __restrict__ q_out,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv, int d, int dv, int page_size, float eps,
    float temp_coef, int temp_every, int row_stride, int norm_q, int norm_k) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const int token = blockIdx.x;
    const int warps = blockDim.x >> 5;
    const int head_slot = blockIdx.y * warps + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (head_slot >= nq + 2 * nkv) return;
    const bool is_q = head_slot < nq;
    const bool is_k = !is_q && head_slot < nq + nkv;
    if (!is_q && k_pages == nullptr) return;
    const size_t row = (size_t)token * (size_t)row_stride;
    int slot = 0;
    if (!is_q) {
        slot = slots[token];
        if (slot < 0) return;
    }
    const int page = slot / page_size, offset = slot - page * page_size;
    if (!is_q && !is_k) {
        if (dv == 0) return;                // keys only: they serve as the values too
        const int kv_head = head_slot - nq - nkv;
        const T* src = qkv + row + (size_t)(nq + nkv) * d + (size_t)kv_head * dv;
        T* dst = v_pages + (((size_t)page * nkv + kv_head) * page_size + offset) * dv;
        for (int j = lane; j < dv; j += 32) dst[j] = src[j];
        return;
    }
    const T* src = qkv + row + (size_t)head_slot * d;
    const float* weight = is_q ? q_weight : k_weight;
    float factor = 1.0f;
    if (is_q ? norm_q : norm_k) {           // with or without a weight vector
        float sum_sq = 0.0f;
        for (int j = lane; j < d; j += 32) {
            const float v = to_float(src[j]);
            sum_sq = fmaf(v, v, sum_sq);
        }
        factor = rsqrtf(warp_sum(sum_sq) / (float)d + eps);
    }
    float temperature = 1.0f;
    if (is_q && temp_every > 0)
        temperature = 1.0f + temp_coef * logf((float)((positions[token] + 1) / temp_every) + 1.0f);
    T* dst = is_q ? q_out + ((size_t)token * nq + head_slot) * d
                  : k_pages + (((size_t)page * nkv + (head_slot - nq)) * page_size + offset) * d;
    for (int j = lane; j < d; j += 32) {
        float v = to_float(src[j]) * factor;
        if (weight) v *= weight[j];
        dst[j] = from_float<T>(v * temperature);
    }
}

constexpr int kQueryTile = 16;
constexpr int kKeyTile = 32;
constexpr int kWarps = 4;
constexpr int kRowsPerWarp = kQueryTile / kWarps;

template <typename T, int DPL>  // DPL: value elements per lane, dv <= 32 * DPL
__global__ void __launch_bounds__(kWarps * 32) biased_paged_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    T* __restrict__ out, const int* __restrict__ query_start, const int* __restrict__ seq_lens,
    const int* __restrict__ block_table, const float* __restrict__ slopes, const float* __restrict__ sinks,
    int num_requests, int max_pages, int nq, int nkv, int d, int dv, int page_size, float scale, int window,
    const T* __restrict__ gate, int gate_stride, float gate_factor, int out_stride) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    extern __shared__ float smem[];
    float* q_s = smem;                                   // [16][d]
    float* k_s = q_s + kQueryTile * d;                   // [32][d + 1]
    float* v_s = k_s + kKeyTile * (d + 1);               // [32][dv]

    const int block = blockIdx.x;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (query_start[mid] / kQueryTile + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int local_tile = block - (q_begin / kQueryTile + request);
    const int tile_first = local_tile * kQueryTile;
    if (tile_first >= q_len) return;
    const int rows_here = min(kQueryTile, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const float slope = slopes ? slopes[head] : 0.0f;
    const int* table = block_table + (size_t)request * max_pages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int idx = tid; idx < kQueryTile * d; idx += blockDim.x) {
        const int row = idx / d, j = idx - row * d;
        float v = 0.0f;
        if (row < rows_here) v = to_float(q[((size_t)(q_begin + tile_first + row) * nq + head) * d + j]);
        q_s[idx] = v;
    }

    float acc[kRowsPerWarp][DPL];
    float row_max[kRowsPerWarp], row_sum[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        row_max[r] = -INFINITY;
        row_sum[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }

    const int first_pos = past + tile_first;
    const int last_pos = first_pos + rows_here - 1;
    int key_begin = 0;
    if (window > 0) key_begin = max(0, first_pos - window + 1);
    key_begin = (key_begin / kKeyTile) * kKeyTile;
    const int key_end = last_pos + 1;

    for (int k0 = key_begin; k0 < key_end; k0 += kKeyTile) {
        __syncthreads();
        for (int idx = tid; idx < kKeyTile * d; idx += blockDim.x) {
            const int key = idx / d, j = idx - key * d;
            const int kp = k0 + key;
            float kv = 0.0f;
            if (kp < key_end) {
                const int page = table[kp / page_size];
                if (page >= 0) kv = to_float(k_pages[(((size_t)page * nkv + kv_head) * page_size + kp % page_size) * d + j]);
            }
            k_s[key * (d + 1) + j] = kv;
        }
        for (int idx = tid; idx < kKeyTile * dv; idx += blockDim.x) {
            const int key = idx / dv, j = idx - key * dv;
            const int kp = k0 + key;
            float vv = 0.0f;
            if (kp < key_end) {
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
            const float* q_row = q_s + row * d;
            const float* k_row = k_s + lane * (d + 1);
            float score = 0.0f;
            for (int j = 0; j < d; ++j) score = fmaf(q_row[j], k_row[j], score);
            score = score * scale - slope * (float)(q_pos - kp);
            bool visible = kp <= q_pos;
            if (window > 0) visible = visible && (kp > q_pos - window);
            if (!visible) score = -INFINITY;
            const float new_max = fmaxf(row_max[r], warp_max(score));
            if (new_max == -INFINITY) continue;
            const float correction = expf(row_max[r] - new_max);
            const float p = visible ? expf(score - new_max) : 0.0f;
            row_sum[r] = row_sum[r] * correction + warp_sum(p);
            row_max[r] = new_max;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[r][i] *= correction;
            for (int key = 0; key < kKeyTile; ++key) {
                const float pk = __shfl_sync(0xffffffffu, p, key);
                const float* v_row = v_s + key * dv;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int j = lane + 32 * i;
                    if (j < dv) acc[r][i] = fmaf(pk, v_row[j], acc[r][i]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int row = warp * kRowsPerWarp + r;
        if (row >= rows_here) continue;
        float inv = row_sum[r] > 0.0f ? 1.0f / row_sum[r] : 0.0f;
        if (sinks != nullptr && row_max[r] != -INFINITY) {
            // one more term exp(sink) in the denominator, with no key and no value
            const float sink = sinks[head], top = fmaxf(row_max[r], sink);
            const float keep = expf(row_max[r] - top);
            inv = keep / (row_sum[r] * keep + expf(sink - top));
        }
        const size_t token = (size_t)(q_begin + tile_first + row);
        // a gate per token and head on the head's output, and rows that may be wider than the heads side by side
        if (gate != nullptr) inv *= gate_factor / (1.0f + expf(-to_float(gate[token * gate_stride + head])));
        T* dst = out + token * (out_stride ? (size_t)out_stride : (size_t)nq * dv) + (size_t)head * dv;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int j = lane + 32 * i;
            if (j < dv) dst[j] = from_float<T>(acc[r][i] * inv);
        }
    }
}

template <typename T, int DPL>
int launch_biased(const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
                  const int* seq_lens, const int* block_table, const float* slopes, const float* sinks,
                  int num_requests, int num_tokens, int max_pages, int nq, int nkv, int d, int dv, int page_size,
                  float scale, int window, const void* gate, int gate_stride, float gate_factor, int out_stride,
                  cudaStream_t stream) {
    auto kernel = biased_paged_attention_kernel<T, DPL>;
    const size_t smem = sizeof(float) * ((size_t)kQueryTile * d + (size_t)kKeyTile * (d + 1) + (size_t)kKeyTile * dv);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("biased_paged_attention", cudaGetErrorString(status));
    }
    dim3 grid(num_tokens / kQueryTile + num_requests, nq);
    launch_overlapped_if(num_tokens <= kOverlapMostRows, kernel, grid, kWarps * 32, smem, stream,
        (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, query_start, seq_lens, block_table, slopes, sinks,
        num_requests, max_pages, nq, nkv, d, dv, page_size, scale, window, (const T*)gate, gate_stride, gate_factor,
        out_stride);
    return check_launch("biased_paged_attention");
}

template <typename T>
int dispatch_biased(const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
                    const int* seq_lens, const int* block_table, const float* slopes, const float* sinks,
                    int num_requests, int num_tokens, int max_pages, int nq, int nkv, int d, int dv, int page_size,
                    float scale, int window, const void* gate, int gate_stride, float gate_factor, int out_stride,
                    cudaStream_t stream) {
#define B200_CASE(DPL)                                                                                       \
    if (dv <= 32 * DPL)                                                                                      \
        return launch_biased<T, DPL>(q, k_pages, v_pages, out, query_start, seq_lens, block_table, slopes,   \
                                     sinks, num_requests, num_tokens, max_pages, nq, nkv, d, dv, page_size,  \
                                     scale, window, gate, gate_stride, gate_factor, out_stride, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(4) B200_CASE(8) B200_CASE(16)
#undef B200_CASE
    return fail("biased_paged_attention", "value heads above 512 are not built");
}

}  // namespace b200

// qkv rows: [nq * d | nkv * d | nkv * dv], `row_stride` elements apart (0: packed).  norm_q / norm_k: whether
// queries / keys are divided by their root mean square per head; q_weight / k_weight may be null (no weight
// vector behind that norm).  temp_every <= 0 means no temperature, k_pages / v_pages may be null (nothing is
// stored), dv = 0 stores keys only (nq = 0 with it: rows of keys alone, normalised into their pages).
// dtype: 0 = float32, 1 = bfloat16.
B200_EXPORT int b200_head_norm_scale_cache(
    const void* qkv, const int* positions, const int* slots, const float* q_weight, const float* k_weight,
    void* q_out, void* k_pages, void* v_pages, int num_tokens, int nq, int nkv, int d, int dv, int page_size,
    float eps, float temp_coef, int temp_every, int row_stride, int norm_q, int norm_k, int dtype,
    cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    if (dv > 0 && (k_pages == nullptr) != (v_pages == nullptr))
        return fail("head_norm_scale_cache", "key and value pages must be given together");
    if (row_stride <= 0) row_stride = (nq + nkv) * d + nkv * dv;
    if (row_stride < (nq + nkv) * d + nkv * dv) return fail("head_norm_scale_cache", "row stride below the row's width");
    if (k_pages && page_size <= 0) return fail("head_norm_scale_cache", "page_size must be positive");
    const int warps = 4;
    dim3 grid(num_tokens, (nq + 2 * nkv + warps - 1) / warps);
    if (grid.y > 65535) return fail("head_norm_scale_cache", "too many heads");
    if (dtype == 0)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, head_norm_scale_cache_kernel<float>, grid, warps * 32, 0, stream,
            (const float*)qkv, positions, slots, q_weight, k_weight, (float*)q_out, (float*)k_pages, (float*)v_pages,
            nq, nkv, d, dv, page_size, eps, temp_coef, temp_every, row_stride, norm_q, norm_k);
    else if (dtype == 1)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, head_norm_scale_cache_kernel<__nv_bfloat16>, grid, warps * 32, 0, stream,
            (const __nv_bfloat16*)qkv, positions, slots, q_weight, k_weight, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, nq, nkv, d, dv, page_size, eps, temp_coef, temp_every,
            row_stride, norm_q, norm_k);
    else
        return fail("head_norm_scale_cache", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("head_norm_scale_cache");
}

// slopes: float32 [nq] or null (no bias).  sinks: float32 [nq] or null; a head's sink is one more term
// exp(sink) in its softmax denominator, unscaled, without a key or a value.  window <= 0: every earlier
// key is visible.  gate (run dtype, rows of gate_stride elements, a number per query head) or null: head h's
// output is multiplied by gate_factor * sigmoid(gate[token, h]).  out_stride: elements between the rows of
// out (0: nq * dv).
B200_EXPORT int b200_biased_paged_attention(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start, const int* seq_lens,
    const int* block_table, const float* slopes, const float* sinks, int num_requests, int num_tokens,
    int max_pages, int nq, int nkv, int d, int dv, int page_size, float scale, int window, const void* gate,
    int gate_stride, float gate_factor, int out_stride, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens == 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv) return fail("biased_paged_attention", "query heads must be a multiple of key/value heads");
    if (nq > 65535) return fail("biased_paged_attention", "more than 65535 query heads");
    if (d <= 0 || dv <= 0 || page_size <= 0 || max_pages <= 0) return fail("biased_paged_attention", "sizes must be positive");
    if (dtype == 0)
        return dispatch_biased<float>(q, k_pages, v_pages, out, query_start, seq_lens, block_table, slopes, sinks,
                                      num_requests, num_tokens, max_pages, nq, nkv, d, dv, page_size, scale, window,
                                      gate, gate_stride, gate_factor, out_stride, stream);
    if (dtype == 1)
        return dispatch_biased<__nv_bfloat16>(q, k_pages, v_pages, out, query_start, seq_lens, block_table, slopes,
                                              sinks, num_requests, num_tokens, max_pages, nq, nkv, d, dv, page_size,
                                              scale, window, gate, gate_stride, gate_factor, out_stride, stream);
    return fail("biased_paged_attention", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// ------------------------------------------------------------- bfloat16 on the tensor cores
// 1 if the tensor-core kernels with float32 weights take the shape.
B200_EXPORT int b200_biased_attention_bf16_supports(int nq, int nkv, int d, int dv) {
    return d == dv && (d == 64 || d == 128 || d == 256) && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && nq <= 65535
               ? 1 : 0;
}

B200_EXPORT int b200_biased_sm_count() { return b200::sm_count(); }

// cache_nkv: the heads the pages hold; nkv may be a multiple of it, the query heads then form more groups
// than there are cached heads and several groups read the same rows (many query heads on one cached head
// run as groups of at most 16).
// One query token per request (row r of q is request r).  With splits > 1, partial_o holds
// [requests * nq * splits * d] floats and partial_ml [requests * nq * splits * 2] floats of scratch.
B200_EXPORT int b200_biased_decode_attention_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, float* partial_o, float* partial_ml,
    const int* seq_lens, const int* block_table, const float* slopes, const float* sinks, int num_requests,
    int max_pages, int nq, int nkv, int d, int page_size, float scale, int window, int splits, int cache_nkv,
    const void* gate, int gate_stride, float gate_factor, int out_stride, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0) return 0;
    if (cache_nkv <= 0 || nkv % cache_nkv) return fail("biased_decode_attention", "the cached heads must divide the key/value heads");
    if (!b200_biased_attention_bf16_supports(nq, nkv, d, d)) return fail("biased_decode_attention", "shape not built");
    if (splits < 1 || nkv > 65535 || num_requests > 65535) return fail("biased_decode_attention", "grid out of range");
    if (splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("biased_decode_attention", "scratch for the splits is missing");
    OutForm form;
    form.gate = (const bf16*)gate; form.gate_stride = gate_stride; form.factor = gate_factor; form.out_stride = out_stride;
#define B200_CASE(D)                                                                                         \
    if (d == D)                                                                                              \
        return launch_decode<D, true>(q, k_pages, v_pages, out, partial_o, partial_ml, seq_lens, block_table, \
                                      num_requests, max_pages, nq, nkv, page_size, scale, window, splits,    \
                                      stream, slopes, sinks, cache_nkv, form);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("biased_decode_attention", "head_dim not built");
}

// Portions of prompts: q and out hold num_tokens rows and query_start rows of them; the num_requests
// requests given here begin at row token_offset.
B200_EXPORT int b200_biased_prefill_attention_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start, const int* seq_lens,
    const int* block_table, const float* slopes, const float* sinks, int num_requests, int num_tokens, int max_pages,
    int nq, int nkv, int d, int page_size, float scale, int window, int token_offset, int cache_nkv,
    const void* gate, int gate_stride, float gate_factor, int out_stride, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens - token_offset <= 0) return 0;
    if (cache_nkv <= 0 || nkv % cache_nkv) return fail("biased_prefill_attention", "the cached heads must divide the key/value heads");
    if (token_offset < 0) return fail("biased_prefill_attention", "negative token offset");
    if (!b200_biased_attention_bf16_supports(nq, nkv, d, d)) return fail("biased_prefill_attention", "shape not built");
    if (out_stride % 2) return fail("biased_prefill_attention", "rows of the output must be an even number of elements apart");
    OutForm form;
    form.gate = (const bf16*)gate; form.gate_stride = gate_stride; form.factor = gate_factor; form.out_stride = out_stride;
#define B200_CASE(D)                                                                                           \
    if (d == D)                                                                                                \
        return launch_prefill<D, true>(q, k_pages, v_pages, out, query_start, seq_lens, block_table,           \
                                       num_requests, num_tokens, max_pages, nq, nkv, page_size, scale, window, \
                                       token_offset, stream, slopes, sinks, cache_nkv, form);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("biased_prefill_attention", "head_dim not built");
}
