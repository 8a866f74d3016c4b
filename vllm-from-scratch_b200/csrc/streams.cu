// A residual that is kept as several streams (hyper-connections): X [tokens, S, H] in float32.
//
//   stream_mix_norm   one kernel for what lies between two sublayers:
//                       1. the update by the sublayer behind:  X'_t = sum_s mix[s, t] X_s + out[t] y
//                          (all streams at once from the old ones; or, at the start of a step, every
//                          stream set to the embedding's row),
//                       2. the read by the sublayer ahead:     u = sum_t in[t] X'_t   (no `in`: the plain sum),
//                       3. its RMSNorm:                        normed = u * rsqrt(mean(u^2) + eps) * w.
//                     Every step is optional; with a list of rows only those rows are read and normalised,
//                     written one after another, and X stays as it was (the model's last norm on the rows
//                     whose logits are wanted).
//
// All arithmetic is float32 in an order that the sizes alone fix: an element of X' is one chain of
// multiply-adds over s followed by the term of y, u one chain over t, the sum of squares a block sum.
#include "common.cuh"

namespace b200 {

constexpr int kMaxStreams = 16;

__device__ __forceinline__ float4 four_of(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 four_of(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
}
__device__ __forceinline__ void put_four(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void put_four(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&lo);
    raw.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// V: columns a thread takes at a time (4 where H and the pointers allow it, else 1).
template <typename T, int S, int V>
__global__ void stream_mix_norm_kernel(const T* __restrict__ y, const float* __restrict__ fresh,
                                       const float* __restrict__ mix, const float* __restrict__ out_w,
                                       float* __restrict__ streams, const float* __restrict__ in_w,
                                       const float* __restrict__ norm_w, float eps, T* __restrict__ normed,
                                       const int* __restrict__ rows, int H) {
    overlap_trigger();
    extern __shared__ float u_s[];                      // [H] the row that the sublayer ahead reads
    __shared__ float c_mix[kMaxStreams * kMaxStreams], c_out[kMaxStreams], c_in[kMaxStreams], scratch[33];
    // the small tables are weights: no kernel of the step writes them
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) c_mix[i] = mix ? mix[i] : 0.0f;
    if (threadIdx.x < S) {
        c_out[threadIdx.x] = out_w ? out_w[threadIdx.x] : 0.0f;
        c_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.0f;
    }
    overlap_wait();
    __syncthreads();
    const size_t token = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    const bool store = rows == nullptr && (y != nullptr || fresh != nullptr);
    float* x_row = streams + token * S * H;
    float squares = 0.0f;
    for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
        float x[S][V], made[S][V];
        if (fresh) {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if constexpr (V == 4) { const float4 v = four_of(fresh + token * H + j); x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w; }
                else x[s][0] = fresh[token * H + j];
            }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if constexpr (V == 4) { const float4 v = four_of(x_row + (size_t)s * H + j); x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w; }
                else x[s][0] = x_row[(size_t)s * H + j];
            }
        }
        if (y != nullptr && !fresh) {
            float yv[V];
            if constexpr (V == 4) { const float4 v = four_of(y + token * H + j); yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w; }
            else yv[0] = to_float(y[token * H + j]);
#pragma unroll
            for (int t = 0; t < S; ++t)
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    float sum = 0.0f;
#pragma unroll
                    for (int s = 0; s < S; ++s) sum = fmaf(c_mix[s * S + t], x[s][i], sum);
                    made[t][i] = fmaf(c_out[t], yv[i], sum);
                }
        } else {
#pragma unroll
            for (int t = 0; t < S; ++t)
#pragma unroll
                for (int i = 0; i < V; ++i) made[t][i] = x[t][i];
        }
        if (store) {
#pragma unroll
            for (int t = 0; t < S; ++t) {
                if constexpr (V == 4) put_four(x_row + (size_t)t * H + j, make_float4(made[t][0], made[t][1], made[t][2], made[t][3]));
                else x_row[(size_t)t * H + j] = made[t][0];
            }
        }
        if (normed != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i) {
                float u = 0.0f;
#pragma unroll
                for (int t = 0; t < S; ++t) u = fmaf(c_in[t], made[t][i], u);
                u_s[j + i] = u;
                squares = fmaf(u, u, squares);
            }
        }
    }
    if (normed == nullptr) return;
    const float root = rsqrtf(block_sum(squares, scratch) / (float)H + eps);
    T* dst = normed + (size_t)blockIdx.x * H;
    for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
        if constexpr (V == 4) {
            const float4 w = norm_w ? four_of(norm_w + j) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            put_four(dst + j, make_float4(u_s[j] * root * w.x, u_s[j + 1] * root * w.y, u_s[j + 2] * root * w.z,
                                          u_s[j + 3] * root * w.w));
        } else {
            dst[j] = from_float<T>(u_s[j] * root * (norm_w ? norm_w[j] : 1.0f));
        }
    }
}

template <typename T, int S, int V>
int launch_streams(const void* y, const float* fresh, const float* mix, const float* out_w, float* streams,
                   const float* in_w, const float* norm_w, float eps, void* normed, const int* rows, int out_rows,
                   int H, cudaStream_t stream) {
    auto kernel = stream_mix_norm_kernel<T, S, V>;
    const size_t smem = sizeof(float) * (size_t)H;
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("stream_mix_norm", cudaGetErrorString(status));
    }
    int threads = ((H / V + 31) / 32) * 32;
    threads = threads < 64 ? 64 : threads > 512 ? 512 : threads;
    launch_overlapped_if(out_rows <= kOverlapMostRows, kernel, out_rows, threads, smem, stream, (const T*)y, fresh, mix,
                         out_w, streams, in_w, norm_w, eps, (T*)normed, rows, H);
    return check_launch("stream_mix_norm");
}

template <typename T, int S>
int launch_streams_v(const void* y, const float* fresh, const float* mix, const float* out_w, float* streams,
                     const float* in_w, const float* norm_w, float eps, void* normed, const int* rows, int out_rows,
                     int H, cudaStream_t stream) {
    const uintptr_t all = (uintptr_t)y | (uintptr_t)fresh | (uintptr_t)streams | (uintptr_t)norm_w | (uintptr_t)normed;
    if constexpr (S <= 8)               // four columns of more streams than that would not stay in registers
        if (H % 4 == 0 && (all & 15) == 0)
            return launch_streams<T, S, 4>(y, fresh, mix, out_w, streams, in_w, norm_w, eps, normed, rows, out_rows, H, stream);
    return launch_streams<T, S, 1>(y, fresh, mix, out_w, streams, in_w, norm_w, eps, normed, rows, out_rows, H, stream);
}

template <typename T>
int dispatch_streams(int S, const void* y, const float* fresh, const float* mix, const float* out_w, float* streams,
                     const float* in_w, const float* norm_w, float eps, void* normed, const int* rows, int out_rows,
                     int H, cudaStream_t stream) {
#define B200_CASE(N)                                                                                                \
    if (S == N)                                                                                                     \
        return launch_streams_v<T, N>(y, fresh, mix, out_w, streams, in_w, norm_w, eps, normed, rows, out_rows, H, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(3) B200_CASE(4) B200_CASE(5) B200_CASE(6) B200_CASE(7) B200_CASE(8)
    B200_CASE(9) B200_CASE(10) B200_CASE(11) B200_CASE(12) B200_CASE(13) B200_CASE(14) B200_CASE(15) B200_CASE(16)
#undef B200_CASE
    return fail("stream_mix_norm", "more than 16 streams are not built");
}

}  // namespace b200

// streams: float32 [tokens, S, H], updated in place unless `rows` is given.
// y [tokens, H] (dtype) with mix float32 [S, S] (indexed [from, to]) and out_w float32 [S]: the update; or
// fresh float32 [tokens, H]: every stream is set to it; or neither: the streams are read as they are.
// normed [out_rows, H] (dtype) or null (update only); in_w float32 [S] or null (the plain sum); norm_w
// float32 [H] or null (no weight).  rows int32 [out_rows] or null (every token, out_rows = tokens).
// dtype: 0 = float32, 1 = bfloat16.
B200_EXPORT int b200_stream_mix_norm(const void* y, const float* fresh, const float* mix, const float* out_w,
                                     float* streams, const float* in_w, const float* norm_w, float eps, void* normed,
                                     const int* rows, int out_rows, int S, int H, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (out_rows == 0) return 0;
    if (S <= 0 || H <= 0) return fail("stream_mix_norm", "sizes must be positive");
    if (y != nullptr && fresh == nullptr && (mix == nullptr || out_w == nullptr))
        return fail("stream_mix_norm", "rows on their way into the streams need mix and out");
    if (dtype == 0)
        return dispatch_streams<float>(S, y, fresh, mix, out_w, streams, in_w, norm_w, eps, normed, rows, out_rows, H, stream);
    if (dtype == 1)
        return dispatch_streams<__nv_bfloat16>(S, y, fresh, mix, out_w, streams, in_w, norm_w, eps, normed, rows,
                                               out_rows, H, stream);
    return fail("stream_mix_norm", "dtype must be 0 (float32) or 1 (bfloat16)");
}
