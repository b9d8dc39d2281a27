// Rotary encoding over adjacent pairs (element 2i with element 2i+1) of the first `rotary_dim` elements of every
// q and k head, fused with the append of k and v to the paged cache.  The pair (u, v) of a token at position p
// becomes (u c - v s, v c + u s) with c = magnitude * cos(p f_i), s = magnitude * sin(p f_i); the elements beyond
// rotary_dim pass unchanged.  The frequencies f_i come ready from the host (any scaling rule is folded in there),
// the angle, its sine and cosine are 32-bit.
//   rows      [n_tokens, row_stride] 32-bit: nq heads of d (queries), nkv heads of d (keys), nkv heads of dv (values),
//             then whatever else the product that made the rows put there
//   q_out     [n_tokens, nq d]
//   k_pages   [num_pages, page_size, nkv, d],  v_pages [num_pages, page_size, nkv, dv]
// Keys and values may have different head sizes.  A token whose slot is negative is a row of nobody and is skipped.
#include "common.cuh"

namespace {
template <typename T>
__global__ void rotary_pairs_kernel(const float* __restrict__ rows, int row_stride, const int* __restrict__ positions,
                                    const int* __restrict__ slots, const int* __restrict__ block_table, int table_stride,
                                    T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens,
                                    int nq, int nkv, int d, int dv, int rotary_dim, const float* __restrict__ freq,
                                    float magnitude, int page_size, int num_pages, int write_kv,
                                    int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const float* row = rows + (size_t)t * row_stride;
    const int half = rotary_dim / 2;
    size_t cache_row = 0;
    bool cache_ok = false;
    if (write_kv) {
        const int page = block_table[(size_t)slot * table_stride + pos / page_size];
        cache_ok = page >= 0 && page < num_pages;
        if (!cache_ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
        cache_row = (size_t)(cache_ok ? page : 0) * page_size + pos % page_size;
    }
    extern __shared__ float rotation[];                  // [half] cosines, then [half] sines, both times the magnitude
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * freq[i], &s, &c);
        rotation[i] = c * magnitude;
        rotation[half + i] = s * magnitude;
    }
    __syncthreads();
    const int rotated_heads = nq + nkv;
    for (int w = threadIdx.x; w < rotated_heads * d; w += blockDim.x) {
        const int head = w / d, e = w % d;
        const float* x = row + head * d;
        float value = x[e];
        if (e < rotary_dim) {
            const float c = rotation[e >> 1], s = rotation[half + (e >> 1)];
            value = (e & 1) ? x[e] * c + x[e - 1] * s : x[e] * c - x[e + 1] * s;
        }
        if (head < nq) q_out[((size_t)t * nq + head) * d + e] = from_float<T>(value);
        else if (cache_ok) k_pages[(cache_row * nkv + (head - nq)) * d + e] = from_float<T>(value);
    }
    if (cache_ok) {
        const float* v = row + (size_t)(nq + nkv) * d;
        for (int w = threadIdx.x; w < nkv * dv; w += blockDim.x) v_pages[cache_row * nkv * dv + w] = from_float<T>(v[w]);
    }
}
}  // namespace

LIA_EXPORT int lia_rotary_pairs_kv_write(const float* rows, int row_stride, const int* positions, const int* slots,
                                         const int* block_table, int table_stride, void* q_out, void* k_pages,
                                         void* v_pages, int dtype, int n_tokens, int nq, int nkv, int d, int dv,
                                         int rotary_dim, const float* freq, float magnitude, int page_size,
                                         int num_pages, int write_kv, int* error_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) ||
        (rotary_dim > 0 && !freq) || row_stride < (nq + nkv) * d + nkv * dv)
        return LIA_ERR_SIZE;
    const size_t shared = (size_t)rotary_dim * sizeof(float);
    if (shared > 48 * 1024) return LIA_ERR_SIZE;
#define LIA_PAIRS(T)                                                                                                  \
    return lia_launch(rotary_pairs_kernel<T>, dim3(n_tokens), dim3(256), shared, stream, rows, row_stride, positions, \
                      slots, block_table, table_stride, (T*)q_out, (T*)k_pages, (T*)v_pages, n_tokens, nq, nkv, d,   \
                      dv, rotary_dim, freq, magnitude, page_size, num_pages, write_kv, error_flag)
    if (dtype == LIA_BF16) LIA_PAIRS(__nv_bfloat16);
    if (dtype == LIA_F32) LIA_PAIRS(float);
#undef LIA_PAIRS
    return LIA_ERR_DTYPE;
}
