// What a layer with a norm on both sides of each sublayer needs on the 32-bit residual stream:
//  * residual[r] += rms(y[r] + bias) * w        (the sublayer's output y, normed, joins the stream), and in the same
//    pass, optionally, next[r] = rms(residual[r]) * w2 in the compute element type (the input of the sublayer that
//    follows), so that the stream is read once between two sublayers;
//  * out[r, :] = act(in[r, :]) for 32-bit rows with any row stride: the activation between the two products of a dense
//    feed-forward (tanh form of GELU), SiLU, or a plain change of element type of some columns.
// Sums of squares, means and reciprocal roots are 32-bit; the order of a row's additions depends on the width alone.
#include "common.cuh"

namespace {
template <typename TO>
__global__ void norm_residual_kernel(const float* __restrict__ y, const float* __restrict__ bias,
                                     const float* __restrict__ weight, float* __restrict__ residual,
                                     const float* __restrict__ next_weight, TO* __restrict__ next, int rows, int hidden,
                                     float eps, float next_eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const float* yr = y + (size_t)r * hidden;
    float* xr = residual + (size_t)r * hidden;
    float sum = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = yr[i] + (bias ? bias[i] : 0.f);
        sum = fmaf(v, v, sum);
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
    float sum2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = yr[i] + (bias ? bias[i] : 0.f);
        const float x = xr[i] + v * inv * weight[i];
        xr[i] = x;
        sum2 = fmaf(x, x, sum2);
    }
    if (!next) return;
    sum2 = block_sum(sum2, scratch);
    const float inv2 = 1.0f / sqrtf(sum2 / (float)hidden + next_eps);
    TO* nr = next + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)          // (each thread reads back what it wrote itself)
        nr[i] = from_float<TO>(xr[i] * inv2 * next_weight[i]);
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TO, int ACT>
__global__ void activation_rows_kernel(const float* __restrict__ in, long long ld_in, TO* __restrict__ out,
                                       long long ld_out, int rows, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * width;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / width;
        const int i = (int)(e - r * width);
        const float z = in[r * ld_in + i];
        float a = z;
        if (ACT == 1) a = gelu_tanh(z);
        if (ACT == 2) a = z / (1.0f + expf(-z));
        out[r * ld_out + i] = from_float<TO>(a);
    }
}
}  // namespace

// residual [rows, hidden] += rms(y [rows, hidden] + bias [hidden] or nothing) * weight [hidden]; with `next`
// (next_dtype) also next = rms(residual) * next_weight.  Everything but `next` is 32-bit.
LIA_EXPORT int lia_norm_residual(const float* y, const float* bias, const float* weight, float* residual,
                                 const float* next_weight, void* next, int next_dtype, int rows, int hidden, float eps,
                                 float next_eps, cudaStream_t stream) {
    if (rows <= 0) return LIA_OK;
    if (hidden <= 0 || (next && !next_weight)) return LIA_ERR_SIZE;
    const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
    if (!next || next_dtype == LIA_F32)
        return lia_launch(norm_residual_kernel<float>, dim3(rows), dim3(threads), 0, stream, y, bias, weight, residual,
                          next_weight, (float*)next, rows, hidden, eps, next_eps);
    if (next_dtype == LIA_BF16)
        return lia_launch(norm_residual_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, y, bias, weight,
                          residual, next_weight, (__nv_bfloat16*)next, rows, hidden, eps, next_eps);
    return LIA_ERR_DTYPE;
}

// out[r, i] = act(in[r, i]), i < width; act: 0 identity, 1 GELU (tanh form), 2 SiLU.  Row strides in elements.
LIA_EXPORT int lia_activation_rows(const float* in, long long ld_in, void* out, int out_dtype, long long ld_out,
                                   int rows, int width, int act, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return LIA_OK;
    if (ld_in < width || ld_out < width || act < 0 || act > 2) return LIA_ERR_SIZE;
    const long long total = (long long)rows * width;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
#define LIA_ACT(TO, ACT)                                                                                     \
    return lia_launch(activation_rows_kernel<TO, ACT>, dim3(blocks), dim3(256), 0, stream, in, ld_in, (TO*)out, \
                      ld_out, rows, width)
    if (out_dtype == LIA_F32) {
        if (act == 0) LIA_ACT(float, 0);
        if (act == 1) LIA_ACT(float, 1);
        LIA_ACT(float, 2);
    }
    if (out_dtype == LIA_BF16) {
        if (act == 0) LIA_ACT(__nv_bfloat16, 0);
        if (act == 1) LIA_ACT(__nv_bfloat16, 1);
        LIA_ACT(__nv_bfloat16, 2);
    }
#undef LIA_ACT
    return LIA_ERR_DTYPE;
}
