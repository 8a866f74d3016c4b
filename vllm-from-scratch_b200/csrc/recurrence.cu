// Recurrences with a matrix of state per head, and the short causal convolution in front of one.
//
// Both mixers built on this file keep, per request and head, a float32 matrix S [N, dv] and step
//     S <- a_t S + k_t (s_t v_t)^T          y_t = S^T q_t + c v_t
// token by token:
//   decayed linear attention   a_t = decay_h (a constant of the head), k, q, v = silu of the projection,
//                              s_t = 1, c = 0, N = key size;
//   selective scan (SSD)       a_t = exp(-exp(A_log_h) dt_t), dt_t = softplus(dt + bias_h), k_t = B_t,
//                              q_t = C_t (shared by the heads of a group), v_t = x_t, s_t = dt_t, c = D_h.
// (Gated linear attention, whose decay is a vector over the rows of S, has a kernel of its own further down.)
// A block owns 32, 16 or 8 columns of one head's S for the tokens that one request brings in this
// step (fewer columns, and so more blocks, where a launch would otherwise leave SMs idle): its 256
// threads hold the rows of those columns in registers, 8, 16 or 32 parts of the rows, the per-token
// vectors k and q and the block's slice of v reach the warps through shared memory in tiles of 16
// tokens, every warp leaves its part of y per token in shared memory, and the parts are added in a
// fixed order.  The state is read from the request's slot before the first token and written back
// after the last, so a prompt may arrive in any portions; a slot is zeroed by the cache at admission.
// Everything but the loads of bfloat16 projections is float32.
//
// A long portion would be one long chain of dependent steps in few blocks.  It is therefore cut into
// segments of seg_len tokens that run side by side (mode 1): a request's first segment starts from its
// state, the others from zero, and each leaves the state it ends with and the product of its decays.
// One small kernel then walks over a request's segments, turns what each left into the state it
// should have started from (C_s = D_{s-1} C_{s-1} + S_{s-1}) and stores the last one in the slot; and
// the segments run once more (mode 2) to add what that state contributes, y_t += (a_first .. a_t) C^T q_t,
// in which nothing depends on the token ahead.
#include "common.cuh"

namespace b200 {

constexpr int kScanTile = 16;       // tokens staged at a time
constexpr int kScanThreads = 256;   // eight warps; a warp is COLS columns times 32 / COLS parts of the rows

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
// The activation of a projection or of the convolution in the mode whose projections are bfloat16:
// the hardware's exponential and division (a few units in the last place of float32, far inside what
// the rounding of the operand to bfloat16 leaves); the 32-bit mode takes the precise forms.
template <typename T> __device__ __forceinline__ float silu_of(float z) { return silu_f(z); }
template <> __device__ __forceinline__ float silu_of<__nv_bfloat16>(float z) { return __fdividef(z, 1.0f + __expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

struct ScanParams {
    // common
    const int* query_start;     // [R + 1]
    const int* slots;           // [R]
    float* state;               // [slots + 1, H, N, dv]
    float* y;                   // [T, H * dv]
    int heads, n, dv;
    // linear attention: packed projection rows [q | k | v] of `stride` elements
    const void* proj;
    int stride, off_q, off_k, off_v;
    const float* decay;         // [H]
    // selective scan: xbc float32 [T, xbc_width] = [x | B | C], dt from the projection
    const float* xbc;
    int xbc_width, off_b, off_c, group_heads;   // heads per group
    int off_dt;                 // column of dt in `proj`
    const float* dt_bias;       // [H]
    const float* a_log;         // [H]
    const float* skip;          // [H]
    // A long portion in segments (mode 1 and 2, see below): tokens per segment, segments a request at
    // most, the segments' states [R * segs, H, N, dv] and decays [R * segs, H].
    int mode, seg_len, segs;
    int tokens;                 // of the whole step (a step of few tokens is launched overlapped)
    float* seg_state;
    float* seg_decay;
};

// NPT: rows of S per thread; COLS: columns per block.  The state's rows are padded to NPT * 256 / COLS
// (zeros in k and q there).
template <typename T, int NPT, int COLS, bool SSD>
__global__ void __launch_bounds__(kScanThreads) recurrence_kernel(ScanParams p) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    extern __shared__ __align__(16) float scan_smem[];
    constexpr int kScanColumns = COLS, kScanParts = kScanThreads / COLS;
    constexpr int kRows = NPT * kScanParts;
    float* k_s = scan_smem;                                         // [tile][kRows]
    float* q_s = k_s + kScanTile * kRows;                           // [tile][kRows]
    float* v_s = q_s + kScanTile * kRows;                           // [tile][32]
    float* part_s = v_s + kScanTile * kScanColumns;                 // [tile][parts][32]
    float* a_s = part_s + kScanTile * kScanParts * kScanColumns;    // [tile]
    float* s_s = a_s + kScanTile;                                   // [tile]
    const int segs = p.mode == 0 ? 1 : p.segs;
    const int request = blockIdx.x / segs, segment = blockIdx.x - request * segs, head = blockIdx.y;
    const bool correct = p.mode == 2;
    const int tid = threadIdx.x, lane = tid % COLS, part = tid / COLS;      // lane: the thread's column
    const int column0 = blockIdx.z * kScanColumns, column = column0 + lane;
    const bool live = column < p.dv;
    int begin = p.query_start[request], end = p.query_start[request + 1];
    if (p.mode != 0) {
        begin += segment * p.seg_len;
        end = min(end, begin + p.seg_len);
        if (correct && segment == 0) return;        // the first segment started from the true state
    }
    if (begin >= end) return;
    const int n = p.n;
    const int row0 = part * NPT;
    float* state = p.state + (((size_t)p.slots[request] * p.heads + head) * n) * p.dv + column;
    float* left = p.mode == 0 ? state      // where the state goes at the end (mode 2: where it comes from)
                              : p.seg_state + (((size_t)blockIdx.x * p.heads + head) * n) * p.dv + column;
    const float* from = correct ? left : state;
    const bool starts_empty = p.mode == 1 && segment > 0;
    float S[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i)
        S[i] = (live && row0 + i < n && !starts_empty) ? from[(size_t)(row0 + i) * p.dv] : 0.0f;
    float decays = 1.0f;            // product of the decays of the tokens so far
    const T* proj = (const T*)p.proj;
    const float decay = SSD ? 0.0f : p.decay[head];
    const float skip = SSD ? p.skip[head] : 0.0f;
    const float a_neg = SSD ? -expf(p.a_log[head]) : 0.0f;
    const float dt_bias = SSD ? p.dt_bias[head] : 0.0f;
    const int group = SSD ? head / p.group_heads : 0;
    const size_t y_stride = (size_t)p.heads * p.dv;

    // A tile's inputs are fetched into registers while the tile ahead of it is computed, and reach
    // shared memory (through silu where the mixer has one) when that tile is done.
    constexpr int kThreadsHere = kScanThreads;
    constexpr int kPerKQ = kScanTile * kRows / kThreadsHere;            // elements of k (and of q) per thread
    constexpr int kPerV = (kScanTile * kScanColumns + kThreadsHere - 1) / kThreadsHere;   // of v (not every thread has one)
    float k_r[kPerKQ], q_r[kPerKQ], v_r[kPerV], a_r = 0.0f, s_r = 0.0f;
    auto fetch = [&](int t0) {
        const int count = min(kScanTile, end - t0);
#pragma unroll
        for (int j = 0; j < kPerKQ; ++j) {
            const int idx = tid + j * kThreadsHere;
            const int t = idx / kRows, i = idx - t * kRows;
            float kv = 0.0f, qv = 0.0f;         // rows past n and tokens past the end: zeros
            if (t < count && i < n) {
                const size_t token = (size_t)(t0 + t);
                if (SSD) {          // the second pass of a portion in segments needs q alone
                    const float* row = p.xbc + token * p.xbc_width;
                    if (!correct) kv = row[p.off_b + group * n + i];
                    qv = row[p.off_c + group * n + i];
                } else {
                    const T* row = proj + token * p.stride;
                    if (!correct) kv = to_float(row[p.off_k + head * n + i]);
                    qv = to_float(row[p.off_q + head * n + i]);
                }
            }
            k_r[j] = kv;
            q_r[j] = qv;
        }
#pragma unroll
        for (int j = 0; j < kPerV; ++j) {
            const int idx = tid + j * kThreadsHere;
            const int t = idx / kScanColumns, c = idx - t * kScanColumns;
            float v = 0.0f;
            if (t < count && column0 + c < p.dv && !correct) {      // t >= kScanTile for threads without an element
                const size_t token = (size_t)(t0 + t);
                if (SSD) v = p.xbc[token * p.xbc_width + head * p.dv + column0 + c];
                else v = to_float(proj[token * p.stride + p.off_v + head * p.dv + column0 + c]);
            }
            v_r[j] = v;
        }
        if (SSD && tid < count) a_r = to_float(proj[(size_t)(t0 + tid) * p.stride + p.off_dt + head]);
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < kPerKQ; ++j) {
            const int idx = tid + j * kThreadsHere;
            k_s[idx] = SSD ? k_r[j] : silu_of<T>(k_r[j]);
            q_s[idx] = SSD ? q_r[j] : silu_of<T>(q_r[j]);
        }
#pragma unroll
        for (int j = 0; j < kPerV; ++j)
            if (tid + j * kThreadsHere < kScanTile * kScanColumns) v_s[tid + j * kThreadsHere] = SSD ? v_r[j] : silu_of<T>(v_r[j]);
        if (tid < kScanTile) {
            if (SSD) {
                const float dt = softplus_f(a_r + dt_bias);
                a_s[tid] = expf(a_neg * dt);
                s_s[tid] = dt;
            } else {
                a_s[tid] = decay;
                s_s[tid] = 1.0f;
            }
        }
        (void)s_r;
    };

    fetch(begin);
    for (int t0 = begin; t0 < end; t0 += kScanTile) {
        const int count = min(kScanTile, end - t0);
        __syncthreads();            // the tile ahead has been added up and stored
        stage();
        __syncthreads();
        if (t0 + kScanTile < end) fetch(t0 + kScanTile);
        for (int t = 0; t < count; ++t) {
            const float a = a_s[t], sv = s_s[t] * v_s[t * kScanColumns + lane];
            const float* k_row = k_s + t * kRows + row0;
            const float* q_row = q_s + t * kRows + row0;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            decays *= a;
            if (correct) {
#pragma unroll
                for (int i = 0; i < NPT; i += 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(q_row + i);
                    acc[0] = fmaf(S[i], q4.x, acc[0]);
                    acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                    acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                    acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
                }
                part_s[(t * kScanParts + part) * kScanColumns + lane] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * decays;
                continue;
            }
#pragma unroll
            for (int i = 0; i < NPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(k_row + i);
                const float4 q4 = *reinterpret_cast<const float4*>(q_row + i);
                S[i] = fmaf(a, S[i], k4.x * sv);
                S[i + 1] = fmaf(a, S[i + 1], k4.y * sv);
                S[i + 2] = fmaf(a, S[i + 2], k4.z * sv);
                S[i + 3] = fmaf(a, S[i + 3], k4.w * sv);
                acc[0] = fmaf(S[i], q4.x, acc[0]);
                acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
            }
            part_s[(t * kScanParts + part) * kScanColumns + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int idx = tid; idx < count * kScanColumns; idx += blockDim.x) {
            const int t = idx / kScanColumns, c = idx - t * kScanColumns;
            if (column0 + c >= p.dv) continue;
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kScanParts; ++w) total += part_s[(t * kScanParts + w) * kScanColumns + c];
            float* y = p.y + (size_t)(t0 + t) * y_stride + head * p.dv + column0 + c;
            if (correct) *y += total;
            else *y = fmaf(skip, v_s[idx], total);
        }
    }
    if (correct) return;
    if (live) {
#pragma unroll
        for (int i = 0; i < NPT; ++i)
            if (row0 + i < n) left[(size_t)(row0 + i) * p.dv] = S[i];
    }
    if (p.mode == 1 && tid == 0 && blockIdx.z == 0) p.seg_decay[(size_t)blockIdx.x * p.heads + head] = decays;
}

// After the segments have run side by side: per request, segment after segment, what a segment left
// (the state it ends with when started from zero; the first one's from the true state) becomes the
// state it should have started from, and the last state goes to the request's slot.  One thread an
// element of a head's state.
__global__ void carry_states_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay,
                                    float* __restrict__ state, const int* __restrict__ query_start,
                                    const int* __restrict__ slots, int heads, int elements, int seg_len, int segs) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const int request = blockIdx.x, head = blockIdx.y;
    const int length = query_start[request + 1] - query_start[request];
    if (length <= 0) return;
    const int used = (length + seg_len - 1) / seg_len;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < elements; e += gridDim.z * blockDim.x) {
        float carried = 0.0f;
        for (int s = 0; s < used; ++s) {
            const size_t at = ((size_t)request * segs + s) * heads + head;
            float* cell = seg_state + at * elements + e;
            const float ended = *cell;
            if (s > 0) {
                *cell = carried;                                    // what the second pass starts from
                carried = fmaf(seg_decay[at], carried, ended);
            } else {
                carried = ended;
            }
        }
        state[((size_t)slots[request] * heads + head) * elements + e] = carried;
    }
}

template <typename T, int NPT, int COLS, bool SSD>
int launch_recurrence_rows(const ScanParams& p, int requests, cudaStream_t stream) {
    auto kernel = recurrence_kernel<T, NPT, COLS, SSD>;
    constexpr int kRows = NPT * kScanThreads / COLS;
    const size_t smem = sizeof(float) * ((size_t)2 * kScanTile * kRows + kScanTile * COLS +
                                         (size_t)kScanTile * kScanThreads + 2 * kScanTile);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("recurrence", cudaGetErrorString(status));
    }
    dim3 grid(requests * (p.mode == 0 ? 1 : p.segs), p.heads, (p.dv + COLS - 1) / COLS);
    launch_overlapped_if(p.tokens <= kOverlapMostRows, kernel, grid, kScanThreads, smem, stream, p);
    if (int status = check_launch("recurrence")) return status;
    if (p.mode != 1) return 0;
    const int elements = p.n * p.dv;
    launch_overlapped_if(false, carry_states_kernel, dim3(requests, p.heads, min((elements + 255) / 256, 64)), 256, 0, stream,
        p.seg_state, p.seg_decay, p.state, p.query_start, p.slots, p.heads, elements, p.seg_len, p.segs);
    if (int status = check_launch("carry_states")) return status;
    ScanParams again = p;
    again.mode = 2;
    launch_overlapped_if(false, kernel, grid, kScanThreads, smem, stream, again);
    return check_launch("recurrence (second pass)");
}

template <typename T, bool SSD>
int launch_recurrence(const ScanParams& p, int requests, cudaStream_t stream) {
    if (p.heads > 65535) return fail("recurrence", "more than 65535 heads");
    if ((p.dv + 7) / 8 > 65535) return fail("recurrence", "value heads too wide");
    if (p.n > 256) return fail("recurrence", "a state of more than 256 rows per head is not built");
    // Fewer columns a block while the launch would leave SMs without a block, as long as a thread
    // keeps four rows at least (64 rows of state for 16 columns, 128 for 8).
    const long long sms = sm_count() > 0 ? sm_count() : 1;
    int cols = 32;
    const long long rows_of_blocks = (long long)requests * (p.mode == 0 ? 1 : p.segs);
    while (cols > 8 && rows_of_blocks * p.heads * ((p.dv + cols - 1) / cols) < sms && p.n > 32 * (32 / cols)) cols /= 2;
#define B200_ROWS(NPT, COLS) return launch_recurrence_rows<T, NPT, COLS, SSD>(p, requests, stream)
    if (cols == 32) {
        if (p.n <= 32) B200_ROWS(4, 32);
        if (p.n <= 64) B200_ROWS(8, 32);
        if (p.n <= 128) B200_ROWS(16, 32);
        B200_ROWS(32, 32);
    }
    if (cols == 16) {
        if (p.n <= 64) B200_ROWS(4, 16);
        if (p.n <= 128) B200_ROWS(8, 16);
        B200_ROWS(16, 16);
    }
    if (p.n <= 128) B200_ROWS(4, 8);
    B200_ROWS(8, 8);
#undef B200_ROWS
}

// segs <= 1: every request's tokens in one chain.  Otherwise seg_state holds [requests * segs, heads, n, dv]
// floats and seg_decay [requests * segs, heads], and segs * seg_len covers the longest portion.
inline int set_segments(ScanParams& p, int seg_len, int segs, float* seg_state, float* seg_decay) {
    p.mode = 0; p.seg_len = 0; p.segs = 1; p.seg_state = nullptr; p.seg_decay = nullptr;
    if (segs <= 1) return 0;
    if (seg_len <= 0 || seg_state == nullptr || seg_decay == nullptr)
        return fail("recurrence", "segments need a length and scratch for their states and decays");
    p.mode = 1; p.seg_len = seg_len; p.segs = segs; p.seg_state = seg_state; p.seg_decay = seg_decay;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Gated linear attention: the state of a head decays per key channel,
//     S <- diag(a_t) S + k_t v_t^T          y_t = S^T (q_t * n^(-1/2))
// with a_t = sigmoid(z_t)^(1 / tau) = exp(-softplus(-z_t) / tau), z_t = gate[t] + gate_bias (one number per head
// and key channel, formed in float32 from the projection's output).  q, k and v are taken as projected (no
// activation).  The launch shape, the staging in tiles of 16 tokens and the order of the sums are those of
// recurrence_kernel; the decays of a tile lie in shared memory beside its keys, a row of numbers per token.
struct GatedScanParams {
    const int* query_start;     // [R + 1]
    const int* slots;           // [R]
    float* state;               // [slots + 1, H, N, dv]
    float* y;                   // [T, H * dv]
    int heads, n, dv;
    const void* proj;           // rows [.. q .. k .. v ..] of `stride` elements
    int stride, off_q, off_k, off_v;
    const void* gate;           // rows of `gate_stride` elements, the decays' logits at column off_gate
    int gate_stride, off_gate;
    const float* gate_bias;     // [H * N] or null
    float inv_tau, q_scale;
    int tokens;
    // A long portion in segments, as in ScanParams; a segment's decays are a row of N numbers per head:
    // seg_state [R * segs, H, N, dv], seg_decay [R * segs, H, N].
    int mode, seg_len, segs;
    float* seg_state;
    float* seg_decay;
};

template <typename T, int NPT, int COLS>
__global__ void __launch_bounds__(kScanThreads) gated_linear_kernel(GatedScanParams p) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    extern __shared__ __align__(16) float scan_smem[];
    constexpr int kScanColumns = COLS, kScanParts = kScanThreads / COLS;
    constexpr int kRows = NPT * kScanParts;
    float* k_s = scan_smem;                                         // [tile][kRows]
    float* q_s = k_s + kScanTile * kRows;                           // [tile][kRows]
    float* a_s = q_s + kScanTile * kRows;                           // [tile][kRows]
    float* v_s = a_s + kScanTile * kRows;                           // [tile][COLS]
    float* part_s = v_s + kScanTile * kScanColumns;                 // [tile][parts][COLS]
    const int segs = p.mode == 0 ? 1 : p.segs;
    const int request = blockIdx.x / segs, segment = blockIdx.x - request * segs, head = blockIdx.y;
    const bool correct = p.mode == 2;
    const int tid = threadIdx.x, lane = tid % COLS, part = tid / COLS;
    const int column0 = blockIdx.z * kScanColumns, column = column0 + lane;
    const bool live = column < p.dv;
    int begin = p.query_start[request], end = p.query_start[request + 1];
    if (p.mode != 0) {
        begin += segment * p.seg_len;
        end = min(end, begin + p.seg_len);
        if (correct && segment == 0) return;        // the first segment started from the true state
    }
    if (begin >= end) return;
    const int n = p.n;
    const int row0 = part * NPT;
    float* state = p.state + (((size_t)p.slots[request] * p.heads + head) * n) * p.dv + column;
    float* left = p.mode == 0 ? state      // where the state goes at the end (mode 2: where it comes from)
                              : p.seg_state + (((size_t)blockIdx.x * p.heads + head) * n) * p.dv + column;
    const float* from = correct ? left : state;
    const bool starts_empty = p.mode == 1 && segment > 0;
    float S[NPT], decays[NPT];          // decays: the product of a row's decays over the tokens so far
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        S[i] = (live && row0 + i < n && !starts_empty) ? from[(size_t)(row0 + i) * p.dv] : 0.0f;
        decays[i] = 1.0f;
    }
    const T* proj = (const T*)p.proj;
    const T* gate = (const T*)p.gate;
    const size_t y_stride = (size_t)p.heads * p.dv;

    constexpr int kPerKQ = kScanTile * kRows / kScanThreads;
    constexpr int kPerV = (kScanTile * kScanColumns + kScanThreads - 1) / kScanThreads;
    float k_r[kPerKQ], q_r[kPerKQ], z_r[kPerKQ], v_r[kPerV];
    auto fetch = [&](int t0) {
        const int count = min(kScanTile, end - t0);
#pragma unroll
        for (int j = 0; j < kPerKQ; ++j) {
            const int idx = tid + j * kScanThreads;
            const int t = idx / kRows, i = idx - t * kRows;
            float kv = 0.0f, qv = 0.0f, zv = 0.0f;      // rows past n and tokens past the end: zeros (their S stays 0)
            if (t < count && i < n) {
                const size_t token = (size_t)(t0 + t);
                const T* row = proj + token * p.stride;
                if (!correct) kv = to_float(row[p.off_k + head * n + i]);       // the second pass needs q and the decays alone
                qv = to_float(row[p.off_q + head * n + i]);
                zv = to_float(gate[token * p.gate_stride + p.off_gate + head * n + i]);
                if (p.gate_bias) zv += p.gate_bias[head * n + i];
            }
            k_r[j] = kv;
            q_r[j] = qv;
            z_r[j] = zv;
        }
#pragma unroll
        for (int j = 0; j < kPerV; ++j) {
            const int idx = tid + j * kScanThreads;
            const int t = idx / kScanColumns, c = idx - t * kScanColumns;
            float v = 0.0f;
            if (t < count && column0 + c < p.dv && !correct)
                v = to_float(proj[(size_t)(t0 + t) * p.stride + p.off_v + head * p.dv + column0 + c]);
            v_r[j] = v;
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < kPerKQ; ++j) {
            const int idx = tid + j * kScanThreads;
            k_s[idx] = k_r[j];
            q_s[idx] = q_r[j] * p.q_scale;
            a_s[idx] = expf(-softplus_f(-z_r[j]) * p.inv_tau);      // sigmoid(z) ^ (1 / tau), in float32
        }
#pragma unroll
        for (int j = 0; j < kPerV; ++j)
            if (tid + j * kScanThreads < kScanTile * kScanColumns) v_s[tid + j * kScanThreads] = v_r[j];
    };

    fetch(begin);
    for (int t0 = begin; t0 < end; t0 += kScanTile) {
        const int count = min(kScanTile, end - t0);
        __syncthreads();            // the tile ahead has been added up and stored
        stage();
        __syncthreads();
        if (t0 + kScanTile < end) fetch(t0 + kScanTile);
        for (int t = 0; t < count; ++t) {
            const float v = v_s[t * kScanColumns + lane];
            const float* k_row = k_s + t * kRows + row0;
            const float* q_row = q_s + t * kRows + row0;
            const float* a_row = a_s + t * kRows + row0;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (p.mode != 0) {
#pragma unroll
                for (int i = 0; i < NPT; i += 4) {
                    const float4 a4 = *reinterpret_cast<const float4*>(a_row + i);
                    decays[i] *= a4.x; decays[i + 1] *= a4.y; decays[i + 2] *= a4.z; decays[i + 3] *= a4.w;
                }
            }
            if (correct) {
                // what the state this segment should have started from adds: (a_first .. a_t) * C, row by row
#pragma unroll
                for (int i = 0; i < NPT; i += 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(q_row + i);
                    acc[0] = fmaf(S[i] * decays[i], q4.x, acc[0]);
                    acc[1] = fmaf(S[i + 1] * decays[i + 1], q4.y, acc[1]);
                    acc[2] = fmaf(S[i + 2] * decays[i + 2], q4.z, acc[2]);
                    acc[3] = fmaf(S[i + 3] * decays[i + 3], q4.w, acc[3]);
                }
                part_s[(t * kScanParts + part) * kScanColumns + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                continue;
            }
#pragma unroll
            for (int i = 0; i < NPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(k_row + i);
                const float4 q4 = *reinterpret_cast<const float4*>(q_row + i);
                const float4 a4 = *reinterpret_cast<const float4*>(a_row + i);
                S[i] = fmaf(a4.x, S[i], k4.x * v);
                S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * v);
                S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * v);
                S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * v);
                acc[0] = fmaf(S[i], q4.x, acc[0]);
                acc[1] = fmaf(S[i + 1], q4.y, acc[1]);
                acc[2] = fmaf(S[i + 2], q4.z, acc[2]);
                acc[3] = fmaf(S[i + 3], q4.w, acc[3]);
            }
            part_s[(t * kScanParts + part) * kScanColumns + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int idx = tid; idx < count * kScanColumns; idx += blockDim.x) {
            const int t = idx / kScanColumns, c = idx - t * kScanColumns;
            if (column0 + c >= p.dv) continue;
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kScanParts; ++w) total += part_s[(t * kScanParts + w) * kScanColumns + c];
            float* y = p.y + (size_t)(t0 + t) * y_stride + head * p.dv + column0 + c;
            if (correct) *y += total;
            else *y = total;
        }
    }
    if (correct) return;
    if (live) {
#pragma unroll
        for (int i = 0; i < NPT; ++i)
            if (row0 + i < n) left[(size_t)(row0 + i) * p.dv] = S[i];
    }
    if (p.mode == 1 && lane == 0 && blockIdx.z == 0) {
#pragma unroll
        for (int i = 0; i < NPT; ++i)
            if (row0 + i < n) p.seg_decay[((size_t)blockIdx.x * p.heads + head) * n + row0 + i] = decays[i];
    }
}

// As carry_states_kernel, with a decay per row of a head's state: seg_decay [R * segs, H, N].
__global__ void carry_states_rows_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay,
                                         float* __restrict__ state, const int* __restrict__ query_start,
                                         const int* __restrict__ slots, int heads, int n, int dv, int seg_len, int segs) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const int request = blockIdx.x, head = blockIdx.y;
    const int length = query_start[request + 1] - query_start[request];
    if (length <= 0) return;
    const int used = (length + seg_len - 1) / seg_len;
    const int elements = n * dv;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < elements; e += gridDim.z * blockDim.x) {
        const int row = e / dv;
        float carried = 0.0f;
        for (int s = 0; s < used; ++s) {
            const size_t at = ((size_t)request * segs + s) * heads + head;
            float* cell = seg_state + at * elements + e;
            const float ended = *cell;
            if (s > 0) {
                *cell = carried;                                    // what the second pass starts from
                carried = fmaf(seg_decay[at * n + row], carried, ended);
            } else {
                carried = ended;
            }
        }
        state[((size_t)slots[request] * heads + head) * elements + e] = carried;
    }
}

template <typename T, int NPT, int COLS>
int launch_gated_rows(const GatedScanParams& p, int requests, cudaStream_t stream) {
    auto kernel = gated_linear_kernel<T, NPT, COLS>;
    constexpr int kRows = NPT * kScanThreads / COLS;
    const size_t smem = sizeof(float) * ((size_t)3 * kScanTile * kRows + kScanTile * COLS + (size_t)kScanTile * kScanThreads);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("gated_linear_attention", cudaGetErrorString(status));
    }
    dim3 grid(requests * (p.mode == 0 ? 1 : p.segs), p.heads, (p.dv + COLS - 1) / COLS);
    launch_overlapped_if(p.tokens <= kOverlapMostRows, kernel, grid, kScanThreads, smem, stream, p);
    if (int status = check_launch("gated_linear_attention")) return status;
    if (p.mode != 1) return 0;
    const int elements = p.n * p.dv;
    launch_overlapped_if(false, carry_states_rows_kernel, dim3(requests, p.heads, min((elements + 255) / 256, 64)), 256, 0,
        stream, p.seg_state, p.seg_decay, p.state, p.query_start, p.slots, p.heads, p.n, p.dv, p.seg_len, p.segs);
    if (int status = check_launch("carry_states")) return status;
    GatedScanParams again = p;
    again.mode = 2;
    launch_overlapped_if(false, kernel, grid, kScanThreads, smem, stream, again);
    return check_launch("gated_linear_attention (second pass)");
}

template <typename T>
int launch_gated(const GatedScanParams& p, int requests, cudaStream_t stream) {
    if (p.heads > 65535) return fail("gated_linear_attention", "more than 65535 heads");
    if ((p.dv + 7) / 8 > 65535) return fail("gated_linear_attention", "value heads too wide");
    if (p.n > 256) return fail("gated_linear_attention", "a state of more than 256 rows per head is not built");
    const long long sms = sm_count() > 0 ? sm_count() : 1;
    int cols = 32;
    const long long rows_of_blocks = (long long)requests * (p.mode == 0 ? 1 : p.segs);
    while (cols > 8 && rows_of_blocks * p.heads * ((p.dv + cols - 1) / cols) < sms && p.n > 32 * (32 / cols)) cols /= 2;
#define B200_ROWS(NPT, COLS) return launch_gated_rows<T, NPT, COLS>(p, requests, stream)
    if (cols == 32) {
        if (p.n <= 32) B200_ROWS(4, 32);
        if (p.n <= 64) B200_ROWS(8, 32);
        if (p.n <= 128) B200_ROWS(16, 32);
        B200_ROWS(32, 32);
    }
    if (cols == 16) {
        if (p.n <= 64) B200_ROWS(4, 16);
        if (p.n <= 128) B200_ROWS(8, 16);
        B200_ROWS(16, 16);
    }
    if (p.n <= 128) B200_ROWS(4, 8);
    B200_ROWS(8, 8);
#undef B200_ROWS
}

// out[t, c] = silu(bias[c] + sum_i w[i, c] * in[t - (taps - 1 - i), c]) within one request (the taps'
// weights are handed over tap by tap, [taps, channels], so that a warp reads them side by side); inputs
// before the step's portion come from the request's state (its last taps - 1 inputs, oldest first,
// zeros before the sequence's start).
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int stride, int offset, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ state,
                                        const int* __restrict__ token_request, const int* __restrict__ query_start,
                                        const int* __restrict__ slots, float* __restrict__ out, int channels, int taps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const int token = blockIdx.x;
    const int request = token_request[token];
    const int place = token - query_start[request];        // index within this step's portion
    const float* kept = state + (size_t)slots[request] * (taps - 1) * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = bias[c];
        for (int i = 0; i < taps; ++i) {
            const int back = taps - 1 - i;
            float v;
            if (place - back >= 0) v = to_float(in[(size_t)(token - back) * stride + offset + c]);
            else v = kept[(size_t)(taps - 1 + place - back) * channels + c];
            acc = fmaf(w[(size_t)i * channels + c], v, acc);
        }
        out[(size_t)token * channels + c] = silu_of<T>(acc);
    }
}

// The same for four consecutive channels a thread (8- or 16-byte loads, one 16-byte store).
template <typename T>
__global__ void causal_conv_silu_vec_kernel(const T* __restrict__ in, int stride, int offset, const float* __restrict__ w,
                                            const float* __restrict__ bias, const float* __restrict__ state,
                                            const int* __restrict__ token_request, const int* __restrict__ query_start,
                                            const int* __restrict__ slots, float* __restrict__ out, int channels, int taps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    const int token = blockIdx.x;
    const int request = token_request[token];
    const int place = token - query_start[request];
    const float* kept = state + (size_t)slots[request] * (taps - 1) * channels;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < channels; c += gridDim.y * blockDim.x * 4) {
        float4 acc = *reinterpret_cast<const float4*>(bias + c);
        for (int i = 0; i < taps; ++i) {
            const int back = taps - 1 - i;
            float4 v;
            if (place - back >= 0) {
                const T* src = in + (size_t)(token - back) * stride + offset + c;
                if (sizeof(T) == 4) {
                    v = *reinterpret_cast<const float4*>(src);
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(src);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            } else {
                v = *reinterpret_cast<const float4*>(kept + (size_t)(taps - 1 + place - back) * channels + c);
            }
            const float4 w4 = *reinterpret_cast<const float4*>(w + (size_t)i * channels + c);
            acc.x = fmaf(w4.x, v.x, acc.x);
            acc.y = fmaf(w4.y, v.y, acc.y);
            acc.z = fmaf(w4.z, v.z, acc.z);
            acc.w = fmaf(w4.w, v.w, acc.w);
        }
        *reinterpret_cast<float4*>(out + (size_t)token * channels + c) =
            make_float4(silu_of<T>(acc.x), silu_of<T>(acc.y), silu_of<T>(acc.z), silu_of<T>(acc.w));
    }
}

// After the convolution: the request's last taps - 1 inputs, oldest first.  One thread per request
// and channel reads what it keeps of the old state before it writes.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ in, int stride, int offset, float* __restrict__ state,
                                  const int* __restrict__ query_start, const int* __restrict__ slots, int channels,
                                  int taps) {
    overlap_trigger();      // the kernel behind may be scheduled while this one runs ...
    overlap_wait();         // ... and this one touches nothing before the kernel ahead is done
    constexpr int kMost = 15;
    const int request = blockIdx.x;
    const int begin = query_start[request], length = query_start[request + 1] - begin;
    if (length <= 0) return;
    float* kept = state + (size_t)slots[request] * (taps - 1) * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float fresh[kMost];
#pragma unroll
        for (int i = 0; i < kMost; ++i) {
            if (i < taps - 1) {
                const int place = length - (taps - 1) + i;
                fresh[i] = place >= 0 ? to_float(in[(size_t)(begin + place) * stride + offset + c])
                                      : kept[(size_t)(i + length) * channels + c];
            }
        }
#pragma unroll
        for (int i = 0; i < kMost; ++i)
            if (i < taps - 1) kept[(size_t)i * channels + c] = fresh[i];
    }
}

}  // namespace b200

B200_EXPORT int b200_recurrence_sm_count() { return b200::sm_count(); }

// Decayed linear attention over the packed projection `proj` [T, stride] = [.. q .. k .. v ..] (columns
// off_q, off_k, off_v; q and k are heads x n, v heads x dv; silu is applied on load).  y: float32
// [T, heads * dv].  state: float32 [slots + 1, heads, n, dv].  dtype of proj: 0 float32, 1 bfloat16.
B200_EXPORT int b200_decayed_linear_attention(const void* proj, int stride, int off_q, int off_k, int off_v,
                                              const float* decay, const int* query_start, const int* slots,
                                              float* state, float* y, int tokens, int requests, int heads, int n,
                                              int dv, int seg_len, int segs, float* seg_state, float* seg_decay,
                                              int dtype, cudaStream_t stream) {
    using namespace b200;
    if (requests == 0) return 0;
    ScanParams p = {};
    p.query_start = query_start; p.slots = slots; p.state = state; p.y = y;
    p.heads = heads; p.n = n; p.dv = dv; p.tokens = tokens;
    p.proj = proj; p.stride = stride; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.decay = decay;
    if (int status = set_segments(p, seg_len, segs, seg_state, seg_decay)) return status;
    if (dtype == 0) return launch_recurrence<float, false>(p, requests, stream);
    if (dtype == 1) return launch_recurrence<__nv_bfloat16, false>(p, requests, stream);
    return fail("decayed_linear_attention", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// Selective scan.  xbc: float32 [T, xbc_width] = [x: heads * dv | B: groups * n | C: groups * n]
// (after the convolution and silu); dt: column off_dt + head of `proj` [T, stride]; y float32
// [T, heads * dv]; state float32 [slots + 1, heads, n, dv].
B200_EXPORT int b200_selective_scan(const float* xbc, int xbc_width, const void* proj, int stride, int off_dt,
                                    const float* dt_bias, const float* a_log, const float* skip,
                                    const int* query_start, const int* slots, float* state, float* y,
                                    int tokens, int requests, int heads, int groups, int n, int dv, int seg_len, int segs,
                                    float* seg_state, float* seg_decay, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (requests == 0) return 0;
    if (groups <= 0 || heads % groups) return fail("selective_scan", "heads must be a multiple of groups");
    ScanParams p = {};
    p.query_start = query_start; p.slots = slots; p.state = state; p.y = y;
    p.heads = heads; p.n = n; p.dv = dv; p.tokens = tokens;
    p.proj = proj; p.stride = stride; p.off_dt = off_dt;
    p.xbc = xbc; p.xbc_width = xbc_width; p.off_b = heads * dv; p.off_c = heads * dv + groups * n;
    p.group_heads = heads / groups;
    p.dt_bias = dt_bias; p.a_log = a_log; p.skip = skip;
    if (int status = set_segments(p, seg_len, segs, seg_state, seg_decay)) return status;
    if (dtype == 0) return launch_recurrence<float, true>(p, requests, stream);
    if (dtype == 1) return launch_recurrence<__nv_bfloat16, true>(p, requests, stream);
    return fail("selective_scan", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// Gated linear attention over the packed projection `proj` [T, stride] = [.. q .. k .. v ..] (columns off_q, off_k,
// off_v; q and k are heads x n, v heads x dv; no activation, q times q_scale).  The decays' logits are the
// columns off_gate .. off_gate + heads * n of `gate` [T, gate_stride] (same dtype as proj), plus gate_bias
// (float32 [heads * n] or null); decay = sigmoid(logit) ^ inv_tau.  y: float32 [T, heads * dv].  state: float32
// [slots + 1, heads, n, dv].  segs > 1: long portions run in segments of seg_len tokens side by side; seg_state holds
// [requests * segs, heads, n, dv] floats and seg_decay [requests * segs, heads, n].
B200_EXPORT int b200_gated_linear_attention(const void* proj, int stride, int off_q, int off_k, int off_v,
                                            const void* gate, int gate_stride, int off_gate, const float* gate_bias,
                                            float inv_tau, float q_scale, const int* query_start, const int* slots,
                                            float* state, float* y, int tokens, int requests, int heads, int n, int dv,
                                            int seg_len, int segs, float* seg_state, float* seg_decay, int dtype,
                                            cudaStream_t stream) {
    using namespace b200;
    if (requests == 0) return 0;
    GatedScanParams p = {};
    p.query_start = query_start; p.slots = slots; p.state = state; p.y = y;
    p.heads = heads; p.n = n; p.dv = dv; p.tokens = tokens;
    p.proj = proj; p.stride = stride; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v;
    p.gate = gate; p.gate_stride = gate_stride; p.off_gate = off_gate; p.gate_bias = gate_bias;
    p.inv_tau = inv_tau; p.q_scale = q_scale;
    p.mode = 0; p.seg_len = 0; p.segs = 1; p.seg_state = nullptr; p.seg_decay = nullptr;
    if (segs > 1) {
        if (seg_len <= 0 || seg_state == nullptr || seg_decay == nullptr)
            return fail("gated_linear_attention", "segments need a length and scratch for their states and decays");
        p.mode = 1; p.seg_len = seg_len; p.segs = segs; p.seg_state = seg_state; p.seg_decay = seg_decay;
    }
    if (dtype == 0) return launch_gated<float>(p, requests, stream);
    if (dtype == 1) return launch_gated<__nv_bfloat16>(p, requests, stream);
    return fail("gated_linear_attention", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// The convolution reads the state, the second kernel replaces it: call them in this order.
// in: [T, stride] with the channels at column `offset`; w float32 [taps, channels] (last row: the
// current token); state float32 [slots + 1, taps - 1, channels]; out float32 [T, channels].
B200_EXPORT int b200_causal_conv_silu(const void* in, int stride, int offset, const float* w, const float* bias,
                                      float* state, const int* token_request, const int* query_start,
                                      const int* slots, float* out, int tokens, int requests, int channels, int taps,
                                      int dtype, cudaStream_t stream) {
    using namespace b200;
    if (tokens == 0) return 0;
    if (taps < 1 || taps > 16) return fail("causal_conv_silu", "1 to 16 taps are built");
    if (dtype != 0 && dtype != 1) return fail("causal_conv_silu", "dtype must be 0 (float32) or 1 (bfloat16)");
    const int threads = 128;
    const int tiles = min((channels + threads - 1) / threads, 65535);
    const uintptr_t addresses = (uintptr_t)in | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)state | (uintptr_t)out;
    if (channels % 4 == 0 && stride % 4 == 0 && offset % 4 == 0 && (addresses & 15) == 0) {
        // A block first finds its token's request, slot and place (three loads in a row): few blocks a
        // token, each with many channels, so that this is paid once for much work.
        const int most = (channels / 4 + 2 * threads - 1) / (2 * threads);
        const int sms = sm_count() > 0 ? sm_count() : 1;
        const int wide = max(1, min(most, (2 * sms + tokens - 1) / tokens));
        if (dtype == 0)
            launch_overlapped_if(tokens <= kOverlapMostRows, causal_conv_silu_vec_kernel<float>, dim3(tokens, wide), 2 * threads, 0, stream,
                (const float*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
        else
            launch_overlapped_if(tokens <= kOverlapMostRows, causal_conv_silu_vec_kernel<__nv_bfloat16>, dim3(tokens, wide), 2 * threads, 0, stream,
                (const __nv_bfloat16*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
    } else if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, causal_conv_silu_kernel<float>, dim3(tokens, tiles), threads, 0, stream,
            (const float*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
    else
        launch_overlapped_if(tokens <= kOverlapMostRows, causal_conv_silu_kernel<__nv_bfloat16>, dim3(tokens, tiles), threads, 0, stream,
            (const __nv_bfloat16*)in, stride, offset, w, bias, state, token_request, query_start, slots, out, channels, taps);
    if (int status = check_launch("causal_conv_silu")) return status;
    if (taps == 1) return 0;
    if (dtype == 0)
        launch_overlapped_if(tokens <= kOverlapMostRows, conv_state_kernel<float>, dim3(requests, tiles), threads, 0, stream,
            (const float*)in, stride, offset, state, query_start, slots, channels, taps);
    else
        launch_overlapped_if(tokens <= kOverlapMostRows, conv_state_kernel<__nv_bfloat16>, dim3(requests, tiles), threads, 0, stream,
            (const __nv_bfloat16*)in, stride, offset, state, query_start, slots, channels, taps);
    return check_launch("conv_state");
}
