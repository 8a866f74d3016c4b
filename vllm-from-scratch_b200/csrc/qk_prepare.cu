// Between the projection of queries, keys and values and the attention over the pages, for mixers whose
// projections have biases, whose queries and keys are normalised per head or over the whole projection, and
// whose rotation turns neighbours or halves; and two small steps behind the attention.
//
//   qk_prepare_cache   row [q: nq * d | k: nkv * d | v: nkv * dv] (+ bias) -> RMSNorm of q and of k (none; per head
//                      with one weight vector of d numbers for all heads; or over all heads at once with weight
//                      vectors of nq * d and nkv * d numbers) -> rotation of the first `rotary_dim` numbers of every
//                      head of q and k by the angles position * inv_freq[i] (pairs (2i, 2i + 1) or (i, i + rotary_dim
//                      / 2)) -> q to q_out, k and v into their pages.  A row without keys (nkv = 0) is a layer that
//                      reads another layer's pages.
//   head_gate          out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * factor
//   scaled_sum         out = a * sa + b * sb
//
// Bias, statistics, weights, angles and the rotation are float32 in both run modes.  A token's head slots are
// divided over blocks of a few warps, a warp a slot (every block of a token forms the sums over the whole
// projection for itself where the norm is one over all heads: the row comes from L2 after the first).
#include "common.cuh"

namespace b200 {

constexpr int kNormNone = 0, kNormHead = 1, kNormWhole = 2;

struct PrepareArgs {
    const void* qkv;            // [T, row_stride]
    const float* bias;          // [nq * d + nkv * d + nkv * dv] or null
    const int* positions;       // [T]
    const int* slots;           // [T]; negative: nothing stored for the token
    const float* q_weight;      // per head: [d]; whole: [nq * d]; null: no weight behind the norm
    const float* k_weight;
    const float* inv_freq;      // [rotary_dim / 2] or null
    void* q_out;                // [T, nq * d]
    void* k_pages;              // [pages, nkv, page_size, d] or null
    void* v_pages;              // [pages, nkv, page_size, dv] or null
    int nq, nkv, d, dv, page_size, row_stride;
    int norm_kind, rotary_dim, interleaved;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(256) qk_prepare_cache_kernel(const PrepareArgs p) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    __shared__ float whole_s[2];
    extern __shared__ float turn_s[];           // [rotary_dim / 2] cosines, then as many sines
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int nq = p.nq, nkv = p.nkv, d = p.d, dv = p.dv;
    const T* row = (const T*)p.qkv + (size_t)token * p.row_stride;
    const int slot = p.slots[token];
    const bool store = p.k_pages != nullptr && nkv > 0 && slot >= 0;
    const int half = p.rotary_dim / 2;
    if (p.inv_freq != nullptr && half > 0) {
        const float position = (float)p.positions[token];
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(position * p.inv_freq[i], &turn_s[half + i], &turn_s[i]);
    }
    if (p.norm_kind == kNormWhole) {
        // two sums over the block, one after the other: all of q, then all of k
        for (int which = 0; which < 2; ++which) {
            const int first = which == 0 ? 0 : nq * d, count = which == 0 ? nq * d : nkv * d;
            float sum = 0.0f;
            for (int i = threadIdx.x; i < count; i += blockDim.x) {
                float v = to_float(row[first + i]);
                if (p.bias) v += p.bias[first + i];
                sum = fmaf(v, v, sum);
            }
            sum = block_sum(sum, scratch);
            if (threadIdx.x == 0) whole_s[which] = count > 0 ? rsqrtf(sum / (float)count + p.eps) : 0.0f;
        }
    }
    __syncthreads();
    const int page = store ? slot / p.page_size : 0, offset = store ? slot - page * p.page_size : 0;
    // A block's warps take the head slots blockIdx.y * warps .. (queries, then keys, then values), a slot each.
    for (int head_slot = blockIdx.y * warps + warp; head_slot < nq + 2 * nkv; head_slot += gridDim.y * warps) {
        const bool is_q = head_slot < nq, is_k = !is_q && head_slot < nq + nkv;
        if (!is_q && !store) continue;
        if (!is_q && !is_k) {
            const int kv_head = head_slot - nq - nkv;
            const int first = (nq + nkv) * d + kv_head * dv;
            T* dst = (T*)p.v_pages + (((size_t)page * nkv + kv_head) * p.page_size + offset) * dv;
            for (int j = lane; j < dv; j += 32) {
                float v = to_float(row[first + j]);
                if (p.bias) v += p.bias[first + j];
                dst[j] = from_float<T>(v);
            }
            continue;
        }
        const int first = head_slot * d;                    // q heads, then k heads, side by side
        const int head = is_q ? head_slot : head_slot - nq;
        const float* weight = is_q ? p.q_weight : p.k_weight;
        if (weight != nullptr && p.norm_kind == kNormWhole) weight += (size_t)head * d;
        float factor = 1.0f;
        if (p.norm_kind == kNormWhole) {
            factor = whole_s[is_q ? 0 : 1];
        } else if (p.norm_kind == kNormHead) {
            float sum = 0.0f;
            for (int j = lane; j < d; j += 32) {
                float v = to_float(row[first + j]);
                if (p.bias) v += p.bias[first + j];
                sum = fmaf(v, v, sum);
            }
            factor = rsqrtf(warp_sum(sum) / (float)d + p.eps);
        }
        T* dst = is_q ? (T*)p.q_out + ((size_t)token * nq + head) * d
                      : (T*)p.k_pages + (((size_t)page * nkv + head) * p.page_size + offset) * d;
        auto element = [&](int j) {
            float v = to_float(row[first + j]);
            if (p.bias) v += p.bias[first + j];
            v *= factor;
            if (weight != nullptr) v *= weight[j];
            return v;
        };
        // Pairs of numbers: the rotated ones first, then what lies behind rotary_dim two at a time.
        const int rotated = p.inv_freq != nullptr ? half : 0;
        const int pairs = rotated + (d - 2 * rotated + 1) / 2;
        for (int pair = lane; pair < pairs; pair += 32) {
            if (pair < rotated) {
                const int j1 = p.interleaved ? 2 * pair : pair, j2 = p.interleaved ? 2 * pair + 1 : pair + half;
                float o1, o2;
                rotate_pair(element(j1), element(j2), turn_s[pair], turn_s[half + pair], o1, o2);
                dst[j1] = from_float<T>(o1);
                dst[j2] = from_float<T>(o2);
            } else {
                const int j1 = 2 * rotated + 2 * (pair - rotated);
                dst[j1] = from_float<T>(element(j1));
                if (j1 + 1 < d) dst[j1 + 1] = from_float<T>(element(j1 + 1));
            }
        }
    }
}

__device__ __forceinline__ float4 four(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 four(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void put_four(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void put_four(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// The same for sizes that are multiples of four and rows that begin at 16 bytes (8 in bfloat16), with the pairs of
// a rotation neighbours (or none): a lane holds four consecutive numbers of a head (up to four such pieces for
// heads of up to 512), so a head is read once, both numbers of a pair lie in one lane, and every access is 8 or 16
// bytes wide.  The same arithmetic in the same order per number as in the kernel above but for the sums of
// squares, which are added four numbers a lane.
template <typename T>
__global__ void __launch_bounds__(256) qk_prepare_cache_vec_kernel(const PrepareArgs p) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    __shared__ float whole_s[2];
    extern __shared__ float turn_s[];           // [rotary_dim / 2] cosines, then as many sines
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int nq = p.nq, nkv = p.nkv, d = p.d, dv = p.dv;
    const T* row = (const T*)p.qkv + (size_t)token * p.row_stride;
    const int slot = p.slots[token];
    const bool store = p.k_pages != nullptr && nkv > 0 && slot >= 0;
    const int half = p.rotary_dim / 2;
    if (p.inv_freq != nullptr && half > 0) {
        const float position = (float)p.positions[token];
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(position * p.inv_freq[i], &turn_s[half + i], &turn_s[i]);
    }
    if (p.norm_kind == kNormWhole) {
        for (int which = 0; which < 2; ++which) {
            const int first = which == 0 ? 0 : nq * d, count = which == 0 ? nq * d : nkv * d;
            float sum = 0.0f;
            for (int i = threadIdx.x * 4; i < count; i += blockDim.x * 4) {
                float4 v = four(row + first + i);
                if (p.bias) { const float4 b = four(p.bias + first + i); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
                sum += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            }
            sum = block_sum(sum, scratch);
            if (threadIdx.x == 0) whole_s[which] = count > 0 ? rsqrtf(sum / (float)count + p.eps) : 0.0f;
        }
    }
    __syncthreads();
    const int page = store ? slot / p.page_size : 0, offset = store ? slot - page * p.page_size : 0;
    const int rotated = p.inv_freq != nullptr ? p.rotary_dim : 0;       // numbers of a head that are turned
    for (int head_slot = blockIdx.y * warps + warp; head_slot < nq + 2 * nkv; head_slot += gridDim.y * warps) {
        const bool is_q = head_slot < nq, is_k = !is_q && head_slot < nq + nkv;
        if (!is_q && !store) continue;
        if (!is_q && !is_k) {
            const int kv_head = head_slot - nq - nkv;
            const int first = (nq + nkv) * d + kv_head * dv;
            T* dst = (T*)p.v_pages + (((size_t)page * nkv + kv_head) * p.page_size + offset) * dv;
            for (int j = lane * 4; j < dv; j += 128) {
                float4 v = four(row + first + j);
                if (p.bias) { const float4 b = four(p.bias + first + j); v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
                put_four(dst + j, v);
            }
            continue;
        }
        const int first = head_slot * d;
        const int head = is_q ? head_slot : head_slot - nq;
        const float* weight = is_q ? p.q_weight : p.k_weight;
        if (weight != nullptr && p.norm_kind == kNormWhole) weight += (size_t)head * d;
        float4 v[4];
        float sum = 0.0f;
#pragma unroll
        for (int step = 0; step < 4; ++step) {
            const int j = (step * 32 + lane) * 4;
            if (j < d) {
                v[step] = four(row + first + j);
                if (p.bias) {
                    const float4 b = four(p.bias + first + j);
                    v[step].x += b.x; v[step].y += b.y; v[step].z += b.z; v[step].w += b.w;
                }
                sum += (v[step].x * v[step].x + v[step].y * v[step].y) + (v[step].z * v[step].z + v[step].w * v[step].w);
            }
        }
        float factor = 1.0f;
        if (p.norm_kind == kNormWhole) factor = whole_s[is_q ? 0 : 1];
        else if (p.norm_kind == kNormHead) factor = rsqrtf(warp_sum(sum) / (float)d + p.eps);
        T* dst = is_q ? (T*)p.q_out + ((size_t)token * nq + head) * d
                      : (T*)p.k_pages + (((size_t)page * nkv + head) * p.page_size + offset) * d;
#pragma unroll
        for (int step = 0; step < 4; ++step) {
            const int j = (step * 32 + lane) * 4;
            if (j >= d) continue;
            float4 r = make_float4(v[step].x * factor, v[step].y * factor, v[step].z * factor, v[step].w * factor);
            if (weight != nullptr) { const float4 w = four(weight + j); r.x *= w.x; r.y *= w.y; r.z *= w.z; r.w *= w.w; }
            if (j < rotated) {
                const int pair = j >> 1;
                rotate_pair(r.x, r.y, turn_s[pair], turn_s[half + pair], r.x, r.y);
            }
            if (j + 2 < rotated) {
                const int pair = (j >> 1) + 1;
                rotate_pair(r.z, r.w, turn_s[pair], turn_s[half + pair], r.z, r.w);
            }
            put_four(dst + j, r);
        }
    }
}

// out[t, h, :] = x[t, h, :] * sigmoid(gate[t * gate_stride + h]) * factor; one block per token.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, const T* __restrict__ gate, int gate_stride,
                                 T* __restrict__ out, int heads, int dv, float factor) {
    overlap_trigger();
    overlap_wait();
    const size_t token = blockIdx.x;
    const int width = heads * dv;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float z = to_float(gate[token * gate_stride + i / dv]);
        const float g = 1.0f / (1.0f + expf(-z));
        out[token * width + i] = from_float<T>(to_float(x[token * width + i]) * g * factor);
    }
}

template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* __restrict__ b, float sb,
                                  T* __restrict__ out, size_t count) {
    overlap_trigger();
    overlap_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<T>(fmaf(to_float(a[i]), sa, to_float(b[i]) * sb));
}

}  // namespace b200

// norm_kind: 0 none, 1 per head (weights of d numbers or null), 2 over all heads of q and of k at once (weights of
// nq * d and nkv * d numbers or null).  interleaved: 1 turns the neighbours (2i, 2i + 1), 0 the halves (i, i +
// rotary_dim / 2).  inv_freq null or rotary_dim 0: no rotation.  k_pages null or nkv 0: nothing is stored.
// row_stride <= 0: rows are packed.  dtype: 0 = float32, 1 = bfloat16.
B200_EXPORT int b200_qk_prepare_cache(
    const void* qkv, const float* bias, const int* positions, const int* slots, const float* q_weight,
    const float* k_weight, const float* inv_freq, void* q_out, void* k_pages, void* v_pages, int num_tokens, int nq,
    int nkv, int d, int dv, int page_size, int row_stride, int norm_kind, int rotary_dim, int interleaved, float eps,
    int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    const int width = (nq + nkv) * d + nkv * dv;
    if (nq <= 0 || nkv < 0 || d <= 0 || dv < 0) return fail("qk_prepare_cache", "sizes must be positive");
    if (row_stride <= 0) row_stride = width;
    if (row_stride < width) return fail("qk_prepare_cache", "row stride below the row's width");
    if (norm_kind < 0 || norm_kind > 2) return fail("qk_prepare_cache", "norm kind must be 0, 1 or 2");
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > d) return fail("qk_prepare_cache", "rotary_dim must be even and at most the head size");
    if (nkv > 0 && (k_pages == nullptr) != (v_pages == nullptr))
        return fail("qk_prepare_cache", "key and value pages must be given together");
    if (k_pages && page_size <= 0) return fail("qk_prepare_cache", "page_size must be positive");
    if (inv_freq == nullptr) rotary_dim = 0;
    PrepareArgs p = {qkv, bias, positions, slots, q_weight, k_weight, rotary_dim > 0 ? inv_freq : nullptr, q_out, k_pages,
                     v_pages, nq, nkv, d, dv, page_size, row_stride, norm_kind, rotary_dim, interleaved, eps};
    // A token's head slots go to as many blocks of eight warps as it takes to give the GPU two blocks an SM.
    const int heads = nq + 2 * nkv;
    const int warps = heads >= 8 ? 8 : heads >= 4 ? 4 : 2;
    const int sms = sm_count() > 0 ? sm_count() : 1;
    const int chunks = max(1, min((heads + warps - 1) / warps, (2 * sms + num_tokens - 1) / num_tokens));
    const dim3 grid(num_tokens, chunks);
    const size_t smem = sizeof(float) * (size_t)rotary_dim;
    const size_t element = dtype == 0 ? 4 : 2;
    const uintptr_t addresses = (uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)q_weight | (uintptr_t)k_weight |
                                (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages;
    const bool vec = d % 4 == 0 && dv % 4 == 0 && d <= 512 && row_stride % 4 == 0 && (addresses & 15) == 0 &&
                     (rotary_dim == 0 || interleaved) && (dtype == 0 || dtype == 1) && element > 0;
    if (vec && dtype == 0)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, qk_prepare_cache_vec_kernel<float>, grid, warps * 32, smem, stream, p);
    else if (vec)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, qk_prepare_cache_vec_kernel<__nv_bfloat16>, grid, warps * 32, smem, stream, p);
    else if (dtype == 0)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, qk_prepare_cache_kernel<float>, grid, warps * 32, smem, stream, p);
    else if (dtype == 1)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, qk_prepare_cache_kernel<__nv_bfloat16>, grid, warps * 32, smem, stream, p);
    else
        return fail("qk_prepare_cache", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("qk_prepare_cache");
}

B200_EXPORT int b200_head_gate(const void* x, const void* gate, int gate_stride, void* out, int tokens, int heads,
                               int dv, float factor, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if (heads <= 0 || dv <= 0 || gate_stride < heads) return fail("head_gate", "sizes must be positive and a gate row hold every head");
    const int width = heads * dv;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, head_gate_kernel<float>, tokens, threads, 0, stream,
            (const float*)x, (const float*)gate, gate_stride, (float*)out, heads, dv, factor);
    else if (dtype == 1)
        launch_overlapped_if(tokens <= kOverlapMostRows, head_gate_kernel<__nv_bfloat16>, tokens, threads, 0, stream,
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, heads, dv, factor);
    else
        return fail("head_gate", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("head_gate");
}

B200_EXPORT int b200_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, long long count, int dtype,
                                cudaStream_t stream) {
    using namespace b200;
    if (count <= 0) return 0;
    const int threads = 256;
    const long long blocks = (count + threads - 1) / threads;
    const int grid = (int)(blocks < 65535LL * 8 ? blocks : 65535LL * 8);
    if (dtype == 0)
        launch_overlapped_if(count <= 65536, scaled_sum_kernel<float>, grid, threads, 0, stream,
            (const float*)a, sa, (const float*)b, sb, (float*)out, (size_t)count);
    else if (dtype == 1)
        launch_overlapped_if(count <= 65536, scaled_sum_kernel<__nv_bfloat16>, grid, threads, 0, stream,
            (const __nv_bfloat16*)a, sa, (const __nv_bfloat16*)b, sb, (__nv_bfloat16*)out, (size_t)count);
    else
        return fail("scaled_sum", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("scaled_sum");
}
