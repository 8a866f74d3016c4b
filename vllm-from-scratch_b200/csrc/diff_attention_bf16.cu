// Exported launcher of the bfloat16 tensor-core kernels for differential attention (diff_attention_mma.cuh),
// compiled for one pair of sizes: B200_DIFF_D numbers to a map of a query or key head, B200_DIFF_DV to a value
// head (both multiples of 16).  A model compiles the pair that its layers have and no other; sizes outside the
// ones this file takes run on the float32 kernel of diff_attention.cu.
#include "diff_attention_mma.cuh"

#ifndef B200_DIFF_D
#define B200_DIFF_D 64
#endif
#ifndef B200_DIFF_DV
#define B200_DIFF_DV 128
#endif

static_assert(B200_DIFF_D % 16 == 0 && B200_DIFF_DV % 16 == 0, "sizes must be multiples of 16");
static_assert(B200_DIFF_DV <= 256, "value heads above 256 would not fit the registers of a thread");
static_assert(2 * b200::diff_stage_elements<B200_DIFF_D, B200_DIFF_DV>() * 2 + 2 * 64 * 8 <= 220 * 1024 &&
              b200::diff_decode_smem<B200_DIFF_D, B200_DIFF_DV>() <= 220 * 1024, "tiles exceed shared memory");

B200_EXPORT int b200_diff_attention_bf16_sizes(int* d, int* dv) {
    *d = B200_DIFF_D;
    *dv = B200_DIFF_DV;
    return 0;
}

// The batch's first `num_decode` requests bring one token each (token r belongs to request r) and go to the
// decode kernel, their keys in `splits` parts (scratch: partial_o [num_decode * nq * 2 * splits * dv] floats,
// partial_ml [num_decode * nq * 2 * splits * 2], needed from two splits on); the others are portions of prompts.
// More than 16 query heads to a key/value head: num_decode must be 0.  Other arguments: diff_attention.cu.
B200_EXPORT int b200_diff_attention_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                         const int* query_start, const int* seq_lens, const int* block_table,
                                         int num_requests, int num_tokens, int max_pages, int nq, int nkv,
                                         int page_size, float scale, float softcap, int window, int keep_first,
                                         float lambda, float eps, float out_scale, int num_decode, int splits,
                                         float* partial_o, float* partial_ml, cudaStream_t stream) {
    using namespace b200;
    constexpr int D = B200_DIFF_D, DV = B200_DIFF_DV;
    if (num_requests == 0 || num_tokens == 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv) return fail("diff_attention_bf16", "query heads must be a multiple of key/value heads");
    if (nq > 65535 || nkv > 65535 || num_requests > 65535) return fail("diff_attention_bf16", "grid out of range");
    if (page_size <= 0 || max_pages <= 0) return fail("diff_attention_bf16", "sizes must be positive");
    if (num_decode < 0 || num_decode > num_requests) return fail("diff_attention_bf16", "num_decode out of range");
    if (num_decode > 0 && nq / nkv > 16) return fail("diff_attention_bf16", "more than 16 query heads to a key/value head");
    if (splits < 1) return fail("diff_attention_bf16", "splits must be positive");
    if (num_decode > 0 && splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("diff_attention_bf16", "scratch for the splits is missing");
    DiffMmaArgs p{query_start, seq_lens, block_table, num_requests, max_pages, nq, nkv, page_size,
                  window > 0 ? window : 0, window > 0 && keep_first > 0 ? keep_first : 0, 0,
                  scale, softcap, lambda, eps, out_scale};
    if (num_decode > 0) {
        DiffMmaArgs decode = p;
        decode.num_requests = num_decode;
        if (int rc = launch_diff_decode_mma<D, DV>(q, k_pages, v_pages, out, partial_o, partial_ml, decode, splits, stream))
            return rc;
    }
    if (num_decode < num_requests) {
        DiffMmaArgs rest = p;
        rest.query_start = query_start + num_decode;
        rest.seq_lens = seq_lens + num_decode;
        rest.block_table = block_table + (size_t)num_decode * max_pages;
        rest.num_requests = num_requests - num_decode;
        rest.token_offset = num_decode;
        return launch_diff_prefill_mma<D, DV>(q, k_pages, v_pages, out, rest, num_tokens, stream);
    }
    return 0;
}
