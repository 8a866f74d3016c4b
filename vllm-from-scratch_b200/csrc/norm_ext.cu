// RMSNorm forms with a second operand, and the embedding with a bigram table.
//
//   add_normed_rmsnorm   residual += rms(x) * x_weight;  out = rms(residual) * weight
//                        (a norm behind a sublayer, the sum, and the norm in front of the next
//                        sublayer as one kernel; either half may be left out, and without
//                        `weight` the output is the sum itself in the output's type: what a
//                        sublayer reads where no norm stands in front of it)
//   paired_norm_mean     out = (rms(a) * wa + rms(b) * wb) / 2      (two mixers side by side)
//   gated_group_norm     out = rms_g(y * silu(z)) * w               (gate first, groups of channels)
//                        out = rms_g(y) * w * sigmoid(z)            (gate behind the norm)
//                        out = rms_g(y) * w * silu(z)               (gate behind the norm, silu)
//   bigram_embedding     residual = embed[id] * scale + bigram[(prev * a + id * b) mod buckets]
//
// rms(v) = v * rsqrt(mean(v^2) + eps); every statistic, sum and gate in float32.  One block per
// row (per row and group for the gated form).
#include "common.cuh"

namespace b200 {

template <typename T>
__global__ void add_normed_rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ x_weight, float x_eps,
                                          float* __restrict__ residual, const float* __restrict__ weight,
                                          T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    const int out_row = blockIdx.x;
    const int row = rows ? rows[out_row] : out_row;
    const size_t base = (size_t)row * hidden;
    const bool store = rows == nullptr;
    float sum_x = 0.0f;
    if (x != nullptr)
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_float(x[base + i]);
            sum_x = fmaf(v, v, sum_x);
        }
    const float inv_x = x != nullptr ? rsqrtf(block_sum(sum_x, scratch) / (float)hidden + x_eps) : 0.0f;
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = x != nullptr ? residual[base + i] + to_float(x[base + i]) * inv_x * x_weight[i] : residual[base + i];
        if (store && x != nullptr) residual[base + i] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    if (out == nullptr) return;
    // weight == nullptr: the rows of the sum themselves, rounded to the output's type.
    const float inv = weight != nullptr ? rsqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps) : 1.0f;
    const size_t out_base = (size_t)out_row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        // The thread that stored an element reads it back; gathered rows form the sum again.
        const float v = (store || x == nullptr) ? residual[base + i]
                                                : residual[base + i] + to_float(x[base + i]) * inv_x * x_weight[i];
        out[out_base + i] = from_float<T>(weight != nullptr ? v * inv * weight[i] : v);
    }
}

template <typename T>
__global__ void paired_norm_mean_kernel(const T* __restrict__ a, const float* __restrict__ wa,
                                        const T* __restrict__ b, const float* __restrict__ wb,
                                        T* __restrict__ out, int hidden, float eps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float sum_a = 0.0f, sum_b = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float va = to_float(a[base + i]), vb = to_float(b[base + i]);
        sum_a = fmaf(va, va, sum_a);
        sum_b = fmaf(vb, vb, sum_b);
    }
    const float inv_a = rsqrtf(block_sum(sum_a, scratch) / (float)hidden + eps);
    const float inv_b = rsqrtf(block_sum(sum_b, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float va = to_float(a[base + i]) * inv_a * wa[i], vb = to_float(b[base + i]) * inv_b * wb[i];
        out[base + i] = from_float<T>(0.5f * (va + vb));
    }
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// Four consecutive elements at a time (16 bytes of float32, 8 of bfloat16); a row of up to 16 elements per
// thread stays in registers between the passes, so every operand is read once.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float dot4(float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
constexpr int kRowSteps = 4;

template <typename T>
__global__ void add_normed_rmsnorm_vec_kernel(const T* __restrict__ x, const float* __restrict__ x_weight, float x_eps,
                                              float* __restrict__ residual, const float* __restrict__ weight,
                                              T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    const int out_row = blockIdx.x;
    const int row = rows ? rows[out_row] : out_row;
    const size_t base = (size_t)row * hidden;
    float4 xv[kRowSteps], rv[kRowSteps];
    float sum_x = 0.0f;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            xv[step] = x != nullptr ? load4(x + base + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            rv[step] = load4(residual + base + i);
            sum_x += dot4(xv[step]);
        }
    }
    const float inv_x = x != nullptr ? rsqrtf(block_sum(sum_x, scratch) / (float)hidden + x_eps) : 0.0f;
    float sum_sq = 0.0f;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            float4 v = rv[step];
            if (x != nullptr) {
                const float4 w = load4(x_weight + i);
                v.x += xv[step].x * inv_x * w.x; v.y += xv[step].y * inv_x * w.y;
                v.z += xv[step].z * inv_x * w.z; v.w += xv[step].w * inv_x * w.w;
                if (rows == nullptr) store4(residual + base + i, v);
            }
            sum_sq += dot4(v);
            rv[step] = v;
        }
    }
    if (out == nullptr) return;
    // weight == nullptr: the rows of the sum themselves, rounded to the output's type.
    const float inv = weight != nullptr ? rsqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps) : 1.0f;
    const size_t out_base = (size_t)out_row * hidden;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            const float4 v = rv[step];
            const float4 w = weight != nullptr ? load4(weight + i) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            store4(out + out_base + i, weight != nullptr
                ? make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w) : v);
        }
    }
}

// Two sums over the block at once; every thread gets both.  `scratch` holds 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) { scratch[warp] = a; scratch[33 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
        float ta = lane < warps ? scratch[lane] : 0.0f, tb = lane < warps ? scratch[33 + lane] : 0.0f;
        ta = warp_sum(ta);
        tb = warp_sum(tb);
        if (lane == 0) { scratch[32] = ta; scratch[65] = tb; }
    }
    __syncthreads();
    return make_float2(scratch[32], scratch[65]);
}

template <typename T>
__global__ void paired_norm_mean_vec_kernel(const T* __restrict__ a, const float* __restrict__ wa,
                                            const T* __restrict__ b, const float* __restrict__ wb,
                                            T* __restrict__ out, int hidden, float eps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[66];
    const size_t base = (size_t)blockIdx.x * hidden;
    float4 av[kRowSteps], bv[kRowSteps];
    float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            av[step] = load4(a + base + i);
            bv[step] = load4(b + base + i);
            sum_a += dot4(av[step]);
            sum_b += dot4(bv[step]);
        }
    }
    const float2 sums = block_sum2(sum_a, sum_b, scratch);
    const float inv_a = rsqrtf(sums.x / (float)hidden + eps);
    const float inv_b = rsqrtf(sums.y / (float)hidden + eps);
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            const float4 u = load4(wa + i), w = load4(wb + i), p = av[step], q = bv[step];
            store4(out + base + i, make_float4(0.5f * (p.x * inv_a * u.x + q.x * inv_b * w.x),
                                               0.5f * (p.y * inv_a * u.y + q.y * inv_b * w.y),
                                               0.5f * (p.z * inv_a * u.z + q.z * inv_b * w.z),
                                               0.5f * (p.w * inv_a * u.w + q.w * inv_b * w.w)));
        }
    }
}

template <typename T, bool GATE_FIRST>
__global__ void gated_group_norm_vec_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride,
                                            const float* __restrict__ weight, T* __restrict__ out, int width,
                                            int group_width, float eps, int silu_behind, int out_stride) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    const size_t token = blockIdx.x;
    const int first = blockIdx.y * group_width;
    const float* y_row = y + token * width + first;
    const T* g_row = gate + token * gate_stride + first;
    float4 v[kRowSteps], g[kRowSteps];
    float sum_sq = 0.0f;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < group_width) {
            v[step] = load4(y_row + i);
            const float4 z = load4(g_row + i);
            if (GATE_FIRST) {
                v[step].x *= z.x * sigmoid_f(z.x); v[step].y *= z.y * sigmoid_f(z.y);
                v[step].z *= z.z * sigmoid_f(z.z); v[step].w *= z.w * sigmoid_f(z.w);
            } else {
                g[step] = make_float4(sigmoid_f(z.x), sigmoid_f(z.y), sigmoid_f(z.z), sigmoid_f(z.w));
                if (silu_behind) { g[step].x *= z.x; g[step].y *= z.y; g[step].z *= z.z; g[step].w *= z.w; }
            }
            sum_sq += dot4(v[step]);
        }
    }
    const float inv = rsqrtf(block_sum(sum_sq, scratch) / (float)group_width + eps);
    T* o_row = out + token * out_stride + first;
#pragma unroll
    for (int step = 0; step < kRowSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < group_width) {
            const float4 w = load4(weight + first + i), p = v[step];
            float4 r = make_float4(p.x * inv * w.x, p.y * inv * w.y, p.z * inv * w.z, p.w * inv * w.w);
            if (!GATE_FIRST) { r.x *= g[step].x; r.y *= g[step].y; r.z *= g[step].z; r.w *= g[step].w; }
            store4(o_row + i, r);
        }
    }
}

// Narrow groups (a head's values): a warp a token and group, eight of them a block; a lane holds up to two pieces
// of four numbers.  FORM: 1 = silu of the gate ahead of the norm, 0 = sigmoid of the gate behind it, 2 = silu behind.
template <typename T, int FORM>
__global__ void gated_group_norm_warp_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride,
                                             const float* __restrict__ weight, T* __restrict__ out, int width,
                                             int group_width, float eps, int out_stride, int tokens, int groups) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)tokens * groups) return;
    const size_t token = (size_t)(unit / groups);
    const int first = (int)(unit - (long long)token * groups) * group_width, lane = threadIdx.x & 31;
    const float* y_row = y + token * width + first;
    const T* g_row = gate + token * gate_stride + first;
    float4 v[2], g[2];
    float sum_sq = 0.0f;
#pragma unroll
    for (int step = 0; step < 2; ++step) {
        const int i = (step * 32 + lane) * 4;
        if (i < group_width) {
            v[step] = load4(y_row + i);
            const float4 z = load4(g_row + i);
            if (FORM == 1) {
                v[step].x *= z.x * sigmoid_f(z.x); v[step].y *= z.y * sigmoid_f(z.y);
                v[step].z *= z.z * sigmoid_f(z.z); v[step].w *= z.w * sigmoid_f(z.w);
            } else {
                g[step] = make_float4(sigmoid_f(z.x), sigmoid_f(z.y), sigmoid_f(z.z), sigmoid_f(z.w));
                if (FORM == 2) { g[step].x *= z.x; g[step].y *= z.y; g[step].z *= z.z; g[step].w *= z.w; }
            }
            sum_sq += dot4(v[step]);
        }
    }
    const float inv = rsqrtf(warp_sum(sum_sq) / (float)group_width + eps);
    T* o_row = out + token * out_stride + first;
#pragma unroll
    for (int step = 0; step < 2; ++step) {
        const int i = (step * 32 + lane) * 4;
        if (i < group_width) {
            const float4 w = load4(weight + first + i), p = v[step];
            float4 r = make_float4(p.x * inv * w.x, p.y * inv * w.y, p.z * inv * w.z, p.w * inv * w.w);
            if (FORM != 1) { r.x *= g[step].x; r.y *= g[step].y; r.z *= g[step].z; r.w *= g[step].w; }
            store4(o_row + i, r);
        }
    }
}

// Threads for a row of `width` elements taken four at a time, at most kRowSteps times a thread; 0 if
// the row is too long for that.
inline int vec_threads(int width) {
    int threads = 32;
    while (threads < 1024 && threads * 4 * kRowSteps < width) threads *= 2;
    while (threads < 256 && threads * 4 < width) threads *= 2;        // short rows: one step a thread
    return threads * 4 * kRowSteps >= width ? threads : 0;
}

// GATE_FIRST: v = y * silu(z), out = rms_g(v) * w.  Otherwise out = rms_g(y) * w * sigmoid(z), or, with
// silu_behind, out = rms_g(y) * w * silu(z).
template <typename T, bool GATE_FIRST>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride,
                                        const float* __restrict__ weight, T* __restrict__ out, int width,
                                        int group_width, float eps, int silu_behind, int out_stride) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ float scratch[33];
    const size_t token = blockIdx.x;
    const int first = blockIdx.y * group_width;
    const float* y_row = y + token * width + first;
    const T* g_row = gate + token * gate_stride + first;
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
        float v = y_row[i];
        if (GATE_FIRST) {
            const float z = to_float(g_row[i]);
            v *= z * sigmoid_f(z);
        }
        sum_sq = fmaf(v, v, sum_sq);
    }
    const float inv = rsqrtf(block_sum(sum_sq, scratch) / (float)group_width + eps);
    T* o_row = out + token * out_stride + first;
    for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
        const float z = to_float(g_row[i]);
        float v = y_row[i];
        if (GATE_FIRST) v = v * (z * sigmoid_f(z)) * inv * weight[first + i];
        else v = v * inv * weight[first + i] * (silu_behind ? z * sigmoid_f(z) : sigmoid_f(z));
        o_row[i] = from_float<T>(v);
    }
}

// One block per token.  The token ahead of a portion's first token is the request's state
// (`previous[slot]`), which the block of that first token reads and then replaces by the
// portion's last token: no other block touches the word.
template <typename T>
__global__ void bigram_embedding_kernel(const T* __restrict__ table, const T* __restrict__ bigram,
                                        const int* __restrict__ ids, const int* __restrict__ positions,
                                        const int* __restrict__ token_request, const int* __restrict__ query_start,
                                        const int* __restrict__ slots, int* __restrict__ previous,
                                        float* __restrict__ residual, int hidden, int vocab, int buckets,
                                        int mul_prev, int mul_cur, float scale, int* __restrict__ error_flag) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    __shared__ int before_s;
    const int token = blockIdx.x;
    const int id = ids[token];
    if (threadIdx.x == 0) {
        const int request = token_request[token];
        const int first = query_start[request];
        int before = -1;
        if (token > first) {
            before = ids[token - 1];
        } else {
            const int slot = slots[request];
            if (positions[token] > 0) before = previous[slot];
            previous[slot] = ids[query_start[request + 1] - 1];
        }
        before_s = before;
    }
    __syncthreads();
    const int before = before_s;
    float* dst = residual + (size_t)token * hidden;
    if (id < 0 || id >= vocab || before >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, token + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    long long row = buckets;                                  // the first token of a sequence: the last row
    if (before >= 0) row = ((long long)before * mul_prev + (long long)id * mul_cur) % buckets;
    const T* src = table + (size_t)id * hidden;
    const T* add = bigram + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = fmaf(to_float(src[i]), scale, to_float(add[i]));
}

inline int row_threads(int width) {
    int threads = 64;
    while (threads < 1024 && threads * 4 < width) threads *= 2;
    return threads;
}

}  // namespace b200

// dtype: 0 = float32, 1 = bfloat16 (x and out; residual and weights are float32).  `weight` and
// `out` may both be null: only the sum is formed.  With `rows` the residual is left as it was.
B200_EXPORT int b200_add_normed_rmsnorm(const void* x, const float* x_weight, float x_eps, float* residual,
                                        const float* weight, void* out, const int* rows, int num_rows, int hidden,
                                        float eps, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_rows == 0) return 0;
    if (num_rows < 0 || hidden <= 0) return fail("add_normed_rmsnorm", "negative row count or width");
    if (weight != nullptr && out == nullptr) return fail("add_normed_rmsnorm", "a norm weight without an output");
    if (x == nullptr && out == nullptr) return 0;
    if (x != nullptr && x_weight == nullptr) return fail("add_normed_rmsnorm", "an addend without its norm weight");
    const uintptr_t addresses = (uintptr_t)x | (uintptr_t)x_weight | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out;
    if (hidden % 4 == 0 && (addresses & 15) == 0 && vec_threads(hidden) > 0 && (dtype == 0 || dtype == 1)) {
        const int threads = vec_threads(hidden);
        if (dtype == 0)
            launch_overlapped_if(num_rows <= kOverlapMostRows, add_normed_rmsnorm_vec_kernel<float>, num_rows, threads, 0, stream,
                (const float*)x, x_weight, x_eps, residual, weight, (float*)out, rows, hidden, eps);
        else
            launch_overlapped_if(num_rows <= kOverlapMostRows, add_normed_rmsnorm_vec_kernel<__nv_bfloat16>, num_rows, threads, 0, stream,
                (const __nv_bfloat16*)x, x_weight, x_eps, residual, weight, (__nv_bfloat16*)out, rows, hidden, eps);
        return check_launch("add_normed_rmsnorm");
    }
    const int threads = row_threads(hidden);
    if (dtype == 0)
        launch_overlapped_if(num_rows <= kOverlapMostRows, add_normed_rmsnorm_kernel<float>, num_rows, threads, 0, stream,
            (const float*)x, x_weight, x_eps, residual, weight, (float*)out, rows, hidden, eps);
    else if (dtype == 1)
        launch_overlapped_if(num_rows <= kOverlapMostRows, add_normed_rmsnorm_kernel<__nv_bfloat16>, num_rows, threads, 0, stream,
            (const __nv_bfloat16*)x, x_weight, x_eps, residual, weight, (__nv_bfloat16*)out, rows, hidden, eps);
    else
        return fail("add_normed_rmsnorm", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("add_normed_rmsnorm");
}

B200_EXPORT int b200_paired_norm_mean(const void* a, const float* wa, const void* b, const float* wb, void* out,
                                      int num_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_rows == 0) return 0;
    if (num_rows < 0 || hidden <= 0) return fail("paired_norm_mean", "negative row count or width");
    const uintptr_t addresses = (uintptr_t)a | (uintptr_t)wa | (uintptr_t)b | (uintptr_t)wb | (uintptr_t)out;
    if (hidden % 4 == 0 && (addresses & 15) == 0 && vec_threads(hidden) > 0 && (dtype == 0 || dtype == 1)) {
        const int threads = vec_threads(hidden);
        if (dtype == 0)
            launch_overlapped_if(num_rows <= kOverlapMostRows, paired_norm_mean_vec_kernel<float>, num_rows, threads, 0, stream,
                (const float*)a, wa, (const float*)b, wb, (float*)out, hidden, eps);
        else
            launch_overlapped_if(num_rows <= kOverlapMostRows, paired_norm_mean_vec_kernel<__nv_bfloat16>, num_rows, threads, 0, stream,
                (const __nv_bfloat16*)a, wa, (const __nv_bfloat16*)b, wb, (__nv_bfloat16*)out, hidden, eps);
        return check_launch("paired_norm_mean");
    }
    const int threads = row_threads(hidden);
    if (dtype == 0)
        launch_overlapped_if(num_rows <= kOverlapMostRows, paired_norm_mean_kernel<float>, num_rows, threads, 0, stream,
            (const float*)a, wa, (const float*)b, wb, (float*)out, hidden, eps);
    else if (dtype == 1)
        launch_overlapped_if(num_rows <= kOverlapMostRows, paired_norm_mean_kernel<__nv_bfloat16>, num_rows, threads, 0, stream,
            (const __nv_bfloat16*)a, wa, (const __nv_bfloat16*)b, wb, (__nv_bfloat16*)out, hidden, eps);
    else
        return fail("paired_norm_mean", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("paired_norm_mean");
}

// y: float32 [tokens, width]; gate: rows of `gate_stride` elements of which the first `width` are the
// gate; out: rows `out_stride` elements apart (0: `width`), of which the first `width` are written; groups
// equal parts of the width, each normalised by its own root mean square.  gate_first: 1 = silu of
// the gate ahead of the norm, 0 = sigmoid of the gate behind it, 2 = silu of the gate behind it.
B200_EXPORT int b200_gated_group_norm_rows(const float* y, const void* gate, int gate_stride, const float* weight,
                                           void* out, int out_stride, int tokens, int width, int groups, int gate_first,
                                           float eps, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if (out_stride <= 0) out_stride = width;
    if (out_stride < width) return fail("gated_group_norm", "rows of the output closer than they are wide");
    if (tokens < 0 || width <= 0 || groups <= 0 || width % groups) return fail("gated_group_norm", "width must divide into the groups");
    if (groups > 65535) return fail("gated_group_norm", "more than 65535 groups");
    const int group_width = width / groups;
    if (gate_first < 0 || gate_first > 2) return fail("gated_group_norm", "gate form must be 0, 1 or 2");
    const bool first = gate_first == 1;
    dim3 grid(tokens, groups);
    const uintptr_t addresses = (uintptr_t)y | (uintptr_t)gate | (uintptr_t)weight | (uintptr_t)out;
    if (group_width % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 && (addresses & 15) == 0 && vec_threads(group_width) > 0 &&
        (dtype == 0 || dtype == 1)) {
        if (group_width <= 256 && groups > 1) {
            const long long units = (long long)tokens * groups;
            const unsigned blocks = (unsigned)((units + 7) / 8);
#define B200_WARP(T, FORM)                                                                                       \
            launch_overlapped_if(tokens <= kOverlapMostRows, gated_group_norm_warp_kernel<T, FORM>, blocks, 256, 0, stream, y, \
                                 (const T*)gate, gate_stride, weight, (T*)out, width, group_width, eps, out_stride, tokens, groups)
            if (dtype == 0) { if (gate_first == 1) B200_WARP(float, 1); else if (gate_first == 2) B200_WARP(float, 2); else B200_WARP(float, 0); }
            else { if (gate_first == 1) B200_WARP(__nv_bfloat16, 1); else if (gate_first == 2) B200_WARP(__nv_bfloat16, 2); else B200_WARP(__nv_bfloat16, 0); }
#undef B200_WARP
            return check_launch("gated_group_norm");
        }
        const int threads = vec_threads(group_width);
#define B200_VEC(T, FIRST)                                                                                      \
        launch_overlapped_if(tokens <= kOverlapMostRows, gated_group_norm_vec_kernel<T, FIRST>, grid, threads, 0, stream, y, (const T*)gate, gate_stride, weight, \
                                                                            (T*)out, width, group_width, eps, gate_first == 2 ? 1 : 0, out_stride)
        if (dtype == 0 && first) B200_VEC(float, true);
        else if (dtype == 0) B200_VEC(float, false);
        else if (first) B200_VEC(__nv_bfloat16, true);
        else B200_VEC(__nv_bfloat16, false);
#undef B200_VEC
        return check_launch("gated_group_norm");
    }
    const int threads = row_threads(group_width);
#define B200_CASE(T, FIRST)                                                                             \
    launch_overlapped_if(tokens <= kOverlapMostRows, gated_group_norm_kernel<T, FIRST>, grid, threads, 0, stream, y, (const T*)gate, gate_stride, weight, \
                                                                    (T*)out, width, group_width, eps, gate_first == 2 ? 1 : 0, out_stride)
    if (dtype == 0 && first) B200_CASE(float, true);
    else if (dtype == 0) B200_CASE(float, false);
    else if (dtype == 1 && first) B200_CASE(__nv_bfloat16, true);
    else if (dtype == 1) B200_CASE(__nv_bfloat16, false);
    else return fail("gated_group_norm", "dtype must be 0 (float32) or 1 (bfloat16)");
#undef B200_CASE
    return check_launch("gated_group_norm");
}

// The same with the output's rows side by side.
B200_EXPORT int b200_gated_group_norm(const float* y, const void* gate, int gate_stride, const float* weight,
                                      void* out, int tokens, int width, int groups, int gate_first, float eps,
                                      int dtype, cudaStream_t stream) {
    return b200_gated_group_norm_rows(y, gate, gate_stride, weight, out, width, tokens, width, groups, gate_first, eps,
                                      dtype, stream);
}

B200_EXPORT int b200_bigram_embedding(const void* table, const void* bigram, const int* ids, const int* positions,
                                      const int* token_request, const int* query_start, const int* slots,
                                      int* previous, float* residual, int num_tokens, int hidden, int vocab,
                                      int buckets, int mul_prev, int mul_cur, float scale, int* error_flag, int dtype,
                                      cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    if (buckets <= 0) return fail("bigram_embedding", "buckets must be positive");
    const int threads = row_threads(hidden);
    if (dtype == 0)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, bigram_embedding_kernel<float>, num_tokens, threads, 0, stream,
            (const float*)table, (const float*)bigram, ids, positions, token_request, query_start, slots, previous,
            residual, hidden, vocab, buckets, mul_prev, mul_cur, scale, error_flag);
    else if (dtype == 1)
        launch_overlapped_if(num_tokens <= kOverlapMostRows, bigram_embedding_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream,
            (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, ids, positions, token_request, query_start,
            slots, previous, residual, hidden, vocab, buckets, mul_prev, mul_cur, scale, error_flag);
    else
        return fail("bigram_embedding", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("bigram_embedding");
}
