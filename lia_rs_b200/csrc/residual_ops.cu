// Operations on the 32-bit residual stream that belong to no layer:
//  * the embedding gather with a learned position vector added, optionally leaving a second copy of the result
//    (a model that feeds the embedding output in again later keeps it);
//  * the input of a re-injection x <- W [x; x0] + b: the two streams side by side in the product's element type,
//    and x set to b in every row so that the product can add into it.
#include "common.cuh"

namespace {
template <typename TW>
__global__ void embedding_positions_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                           const TW* __restrict__ table, const TW* __restrict__ position_table,
                                           float* __restrict__ out, float* __restrict__ copy, int n_tokens, int hidden,
                                           int vocab, int max_positions, float scale, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int token = tokens[t], pos = positions[t];
    const bool ok = token >= 0 && token < vocab && pos >= 0 && pos < max_positions;
    if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    const TW* row = table + (size_t)(ok ? token : 0) * hidden;
    const TW* prow = position_table + (size_t)(ok ? pos : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float value = ok ? to_float(row[i]) * scale + to_float(prow[i]) : 0.f;
        out[(size_t)t * hidden + i] = value;
        if (copy) copy[(size_t)t * hidden + i] = value;
    }
}

template <typename TO, typename TB>
__global__ void reinject_input_kernel(float* __restrict__ x, const float* __restrict__ x0, const TB* __restrict__ bias,
                                      TO* __restrict__ side_by_side, int n_tokens, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    float* xr = x + (size_t)t * hidden;
    const float* x0r = x0 + (size_t)t * hidden;
    TO* dst = side_by_side + (size_t)t * 2 * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        dst[i] = from_float<TO>(xr[i]);
        dst[hidden + i] = from_float<TO>(x0r[i]);
        xr[i] = bias ? to_float(bias[i]) : 0.f;
    }
}
}  // namespace

// out[t, :] = table[token_t, :] * scale + position_table[position_t, :], 32-bit; `copy` (optional) receives the same.
// A token id outside [0, vocab) or a position outside [0, max_positions) writes zeros and raises error flag 1.
LIA_EXPORT int lia_embedding_positions(const int* tokens, const int* positions, const void* table,
                                       const void* position_table, int table_dtype, float* out, float* copy,
                                       int n_tokens, int hidden, int vocab, int max_positions, float scale,
                                       int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (hidden <= 0 || vocab <= 0 || max_positions <= 0) return LIA_ERR_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LIA_BF16)
        return lia_launch(embedding_positions_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                          positions, (const __nv_bfloat16*)table, (const __nv_bfloat16*)position_table, out, copy,
                          n_tokens, hidden, vocab, max_positions, scale, error_flag);
    if (table_dtype == LIA_F32)
        return lia_launch(embedding_positions_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, positions,
                          (const float*)table, (const float*)position_table, out, copy, n_tokens, hidden, vocab,
                          max_positions, scale, error_flag);
    return LIA_ERR_DTYPE;
}

// side_by_side[t] = [x[t], x0[t]] in out_dtype ([n_tokens, 2 hidden]); then x[t] = bias (zeros without one).
LIA_EXPORT int lia_reinject_input(float* x, const float* x0, const void* bias, int bias_dtype, void* side_by_side,
                                  int out_dtype, int n_tokens, int hidden, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (hidden <= 0) return LIA_ERR_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
#define LIA_REINJECT(TO, TB)                                                                                           \
    return lia_launch(reinject_input_kernel<TO, TB>, dim3(n_tokens), dim3(threads), 0, stream, x, x0, (const TB*)bias, \
                      (TO*)side_by_side, n_tokens, hidden)
    if (out_dtype == LIA_BF16 && bias_dtype == LIA_BF16) LIA_REINJECT(__nv_bfloat16, __nv_bfloat16);
    if (out_dtype == LIA_BF16 && bias_dtype == LIA_F32) LIA_REINJECT(__nv_bfloat16, float);
    if (out_dtype == LIA_F32 && bias_dtype == LIA_BF16) LIA_REINJECT(float, __nv_bfloat16);
    if (out_dtype == LIA_F32 && bias_dtype == LIA_F32) LIA_REINJECT(float, float);
#undef LIA_REINJECT
    return LIA_ERR_DTYPE;
}
