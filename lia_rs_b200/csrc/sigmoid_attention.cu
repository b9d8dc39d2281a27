// Attention without a softmax over the paged cache: the weight of a visible key is
//     w = sigmoid(scale * (q . k) + head_bias[h]),
// weights are not normalised over the keys, out = sum_j w_j v_j, and the head's output may be multiplied by
// sigmoid(gate[t, h]) (a per-token, per-head output gate whose logit the caller computed).
//
// A token at position p of request slot s sees the keys j <= p that are also
//   * within the last `window` positions (window > 0), and
//   * in p's own block of `chunk` positions, blocks counted from position 0 of the sequence (chunk > 0):
//     floor(j / chunk) == floor(p / chunk).
// Keys have head size d, values dv (they may differ).  Scores, weights and the sums over keys are 32-bit.
//
// This file holds the kernel for every size and element type: one warp owns one (token, query head), walks the
// visible keys 32 at a time, each lane scoring one key, and accumulates the output with each lane owning value
// elements lane, lane + 32, ...  The order of the work depends on p, the window and the chunk alone, so a token's
// result does not depend on the batch it is in.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
sigmoid_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                 const int* __restrict__ positions, const int* __restrict__ slots,
                                 const int* __restrict__ block_table, int table_stride, const int* __restrict__ rows,
                                 T* __restrict__ out, int n_tokens, int nq, int nkv, int d, int dv, int page_size,
                                 int window, int chunk, float scale, const float* __restrict__ head_bias,
                                 const float* __restrict__ gate, int gate_stride, int num_pages,
                                 int* __restrict__ error_flag) {
    __shared__ float q_shared[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * nq) return;
    const int t = rows ? rows[item / nq] : (int)(item / nq);
    const int h = (int)(item % nq);
    if (t < 0) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int kvh = h / (nq / nkv);
    const T* qrow = q + ((size_t)t * nq + h) * d;
    for (int i = lane; i < d; i += 32) q_shared[warp][i] = to_float(qrow[i]);
    __syncwarp();
    const int* table = block_table + (size_t)slot * table_stride;
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) first = max(first, (pos / chunk) * chunk);
    const float bias = head_bias ? head_bias[h] : 0.f;
    const int pieces = (dv + 31) / 32;
    float acc[MAX_D / 32];
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] = 0.f;

    for (int base = first; base <= pos; base += 32) {
        const int j = base + lane;
        bool valid = j <= pos;
        int row = 0;
        if (valid) {
            row = cache_row_of(table, j, page_size, -1, num_pages, error_flag);
            valid = row >= 0;                       // a key without a page counts for nothing (and the flag is up)
            row = valid ? row : 0;
        }
        float weight = 0.f;
        if (valid) {
            const T* krow = k_pages + ((size_t)row * nkv + kvh) * d;
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot = fmaf(q_shared[warp][i], to_float(krow[i]), dot);
            weight = sigmoidf_(dot * scale + bias);
        }
        const int count = min(32, pos - base + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float wj = __shfl_sync(0xffffffffu, weight, jj);
            const int rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vrow = v_pages + ((size_t)rj * nkv + kvh) * dv;
#pragma unroll
            for (int c = 0; c < MAX_D / 32; ++c) {
                const int i = c * 32 + lane;
                if (c < pieces && i < dv) acc[c] = fmaf(wj, to_float(vrow[i]), acc[c]);
            }
        }
    }
    const float g = gate ? sigmoidf_(gate[(size_t)t * gate_stride + h]) : 1.0f;
    T* orow = out + ((size_t)t * nq + h) * dv;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = c * 32 + lane;
        if (c < pieces && i < dv) orow[i] = from_float<T>(acc[c] * g);
    }
}
}  // namespace

// q [tokens, nq, d], out [tokens, nq, dv]; k_pages [num_pages, page_size, nkv, d], v_pages [.., nkv, dv]; all of
// `dtype`.  head_bias [nq] 32-bit or null; gate: 32-bit logits, token t's head h at gate[t * gate_stride + h], or null.
// `rows` (optional) lists the n_tokens batch indices to compute; without it tokens 0..n_tokens-1.
LIA_EXPORT int lia_sigmoid_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                             const int* positions, const int* slots, const int* block_table,
                                             int table_stride, const int* rows, void* out, int n_tokens, int nq, int nkv,
                                             int d, int dv, int page_size, int window, int chunk, float scale,
                                             const float* head_bias, const float* gate, int gate_stride, int num_pages,
                                             int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || page_size <= 0)
        return LIA_ERR_SIZE;
    const long long items = (long long)n_tokens * nq;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return LIA_ERR_SIZE;
#define LIA_SIGMOID(T)                                                                                                  \
    sigmoid_attention_generic_kernel<T><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(                                  \
        (const T*)q, (const T*)k_pages, (const T*)v_pages, positions, slots, block_table, table_stride, rows, (T*)out, \
        n_tokens, nq, nkv, d, dv, page_size, window, chunk, scale, head_bias, gate, gate_stride, num_pages, error_flag)
    if (dtype == LIA_F32) LIA_SIGMOID(float);
    else if (dtype == LIA_BF16) LIA_SIGMOID(__nv_bfloat16);
    else return LIA_ERR_DTYPE;
#undef LIA_SIGMOID
    return lia_check_launch();
}
