// RMSNorm of the residual stream followed by a short causal convolution over time on each channel, for up to two
// readers of the normed rows at once:
//     h_t   = x_t * rsqrt(mean(x_t^2) + eps) * w                                  (32-bit)
//     out_r = h_t + sum_j c_r[:, j] * h_(t - taps + 1 + j),   r = 0, 1            (zeros before the sequence's start)
// with c_r [width, taps] the reader's taps (the last tap multiplies the token itself).  The taps - 1 normed rows
// before a request's next token are its state: state [slots, taps - 1, width] 32-bit, entry j holding the row of
// position (next position) - (taps - 1) + j.  A step brings each request's tokens as one run of consecutive batch
// rows; a token takes an earlier row from the batch where its request's run holds it and from the state otherwise.
//
// short_conv_kernel: a CTA takes TOK consecutive batch rows: the rows' inverse root mean squares (and those of the
// taps - 1 rows before them) by one warp per row, then a thread per channel.  With `single` (every run of the step
// is one token) the same thread also moves the state on; otherwise it leaves the normed rows of each run's last
// taps - 1 tokens in `tail` and short_conv_state_kernel, launched behind it, writes the state (a run's first tokens
// read the state that its last tokens replace).
#include "common.cuh"

namespace {
constexpr int TOK = 8;
constexpr int MAX_TAPS = 8;
constexpr int THREADS = 256;

template <typename TW, typename TC, typename TO>
__global__ void __launch_bounds__(THREADS)
short_conv_kernel(const float* __restrict__ x, const TW* __restrict__ norm_weight, const TC* __restrict__ taps0,
                  const TC* __restrict__ taps1, const int* __restrict__ positions, const int* __restrict__ slots,
                  float* __restrict__ state, float* __restrict__ tail, TO* __restrict__ out0, TO* __restrict__ out1,
                  int n_tokens, int width, int taps, float eps, int single) {
    __shared__ float inv_rms[TOK + MAX_TAPS];
    __shared__ int s_slot[TOK], s_pos[TOK], s_before[TOK], s_tail[TOK];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * TOK;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int reach = taps - 1;
    // what each token of the tile is: its slot and position, how many rows before it in the batch are its request's
    // (up to taps - 1), and whether it is among the last taps - 1 tokens of its run
    if (threadIdx.x < TOK) {
        const int t = t0 + threadIdx.x;
        int slot = -1, pos = 0, before = 0, is_tail = 0;
        if (t < n_tokens) {
            slot = slots[t];
            pos = positions[t];
            if (slot >= 0) {
                while (before < reach && t - before - 1 >= 0 && slots[t - before - 1] == slot) ++before;
                for (int k = 1; k <= reach && !is_tail; ++k) is_tail = (t + k >= n_tokens) || (slots[t + k] != slot);
                if (reach == 0) is_tail = 0;
            } else {
                pos = 0;
            }
        }
        s_slot[threadIdx.x] = slot;
        s_pos[threadIdx.x] = pos;
        s_before[threadIdx.x] = before;
        s_tail[threadIdx.x] = is_tail;
    }
    // inverse root mean square of rows t0 - reach .. t0 + TOK - 1; the order of the additions depends on the width alone
    for (int r = warp; r < TOK + reach; r += THREADS / 32) {
        const int row = t0 - reach + r;
        float sum = 0.f;
        if (row >= 0 && row < n_tokens) {
            const float* src = x + (size_t)row * width;
            for (int i = lane; i < width; i += 32) sum = fmaf(src[i], src[i], sum);
        }
        sum = warp_sum(sum);
        if (lane == 0) inv_rms[r] = 1.0f / sqrtf(sum / (float)width + eps);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += THREADS) {
        const float w = to_float(norm_weight[c]);
        float c0[MAX_TAPS], c1[MAX_TAPS];
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            // by distance back in time: entry k multiplies the row of position pos - k (tap taps - 1 - k)
            c0[j] = (j < taps && taps0) ? to_float(taps0[(size_t)c * taps + (taps - 1 - j)]) : 0.f;
            c1[j] = (j < taps && taps1) ? to_float(taps1[(size_t)c * taps + (taps - 1 - j)]) : 0.f;
        }
        for (int i = 0; i < TOK; ++i) {
            const int t = t0 + i;
            if (t >= n_tokens) break;
            const int slot = s_slot[i], pos = s_pos[i], before = s_before[i];
            // past[k]: the normed row of position pos - k (k = 0: the token itself), zero before the sequence's start
            float past[MAX_TAPS];
#pragma unroll
            for (int k = 0; k < MAX_TAPS; ++k) {
                float value = 0.f;
                if (k < taps && pos - k >= 0) {
                    if (k <= before) value = x[(size_t)(t - k) * width + c] * inv_rms[i - k + reach] * w;
                    else if (slot >= 0) value = state[((size_t)slot * reach + (before - k + reach)) * width + c];
                }
                past[k] = value;
            }
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int k = MAX_TAPS - 1; k >= 0; --k) {              // oldest row first
                sum0 = fmaf(c0[k], past[k], sum0);
                sum1 = fmaf(c1[k], past[k], sum1);
            }
            if (out0) out0[(size_t)t * width + c] = from_float<TO>(past[0] + sum0);
            if (out1) out1[(size_t)t * width + c] = from_float<TO>(past[0] + sum1);
            if (slot < 0 || reach == 0) continue;
            if (single) {
                // the run is this token alone: entry j of the new state is the row of position pos - (reach - 1 - j)
#pragma unroll
                for (int k = 0; k < MAX_TAPS - 1; ++k)
                    if (k < reach) state[((size_t)slot * reach + (reach - 1 - k)) * width + c] = past[k];
            } else if (s_tail[i]) {
                tail[(size_t)t * width + c] = past[0];
            }
        }
    }
}

// The state after a step that brought runs of several tokens: a CTA per batch row; the last row of each run writes
// its request's state from the normed rows of the run's last tokens (`tail`) and, where the run is shorter than
// taps - 1, from the entries of the old state that stay (they move down; a thread reads an entry before any thread
// of its channel, which is itself, writes over it).
__global__ void short_conv_state_kernel(const float* __restrict__ tail, const int* __restrict__ positions,
                                        const int* __restrict__ slots, float* __restrict__ state, int n_tokens,
                                        int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    if (t + 1 < n_tokens && slots[t + 1] == slot) return;          // not the run's last token
    const int reach = taps - 1, pos = positions[t];
    int before = 0;
    while (before < reach && t - before - 1 >= 0 && slots[t - before - 1] == slot) ++before;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        for (int j = 0; j < reach; ++j) {
            const int k = reach - 1 - j;                             // entry j is the row of position pos - k
            float value = 0.f;
            if (pos - k >= 0) {
                if (k <= before) value = tail[(size_t)(t - k) * width + c];
                else value = state[((size_t)slot * reach + (before - k + reach)) * width + c];   // an entry above j
            }
            state[((size_t)slot * reach + j) * width + c] = value;
        }
    }
}

template <typename TW, typename TC, typename TO>
int launch_short_conv(const float* x, const void* norm_weight, const void* taps0, const void* taps1, const int* positions,
                      const int* slots, float* state, float* tail, void* out0, void* out1, int n_tokens, int width,
                      int taps, float eps, int single, cudaStream_t stream) {
    const int code = lia_launch(short_conv_kernel<TW, TC, TO>, dim3((n_tokens + TOK - 1) / TOK), dim3(THREADS), 0, stream,
                                x, (const TW*)norm_weight, (const TC*)taps0, (const TC*)taps1, positions, slots, state,
                                tail, (TO*)out0, (TO*)out1, n_tokens, width, taps, eps, single);
    if (code != LIA_OK || single || taps <= 1) return code;
    return lia_launch(short_conv_state_kernel, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0, stream,
                      (const float*)tail, positions, slots, state, n_tokens, width, taps);
}
}  // namespace

// x [n_tokens, width] 32-bit; norm_weight [width]; taps0, taps1 [width, taps] (either may be null: that reader is
// absent); state [slots, taps - 1, width] 32-bit; tail [n_tokens, width] 32-bit scratch (unused with `single`);
// out0, out1 [n_tokens, width] of out_dtype (null with its taps).  weight_dtype: of the norm weight and of the taps.
// single: 1 when every request of the step brings one token (the state is then moved on by the same kernel).
LIA_EXPORT int lia_short_conv(const float* x, const void* norm_weight, const void* taps0, const void* taps1,
                              int weight_dtype, const int* positions, const int* slots, float* state, float* tail,
                              void* out0, void* out1, int out_dtype, int n_tokens, int width, int taps, float eps,
                              int single, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (width <= 0 || taps < 1 || taps > MAX_TAPS || (taps > 1 && !state) || (!single && taps > 1 && !tail))
        return LIA_ERR_SIZE;
#define LIA_CONV(TW, TO) \
    return launch_short_conv<TW, TW, TO>(x, norm_weight, taps0, taps1, positions, slots, state, tail, out0, out1, n_tokens, width, taps, eps, single, stream)
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_BF16) LIA_CONV(__nv_bfloat16, __nv_bfloat16);
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_F32) LIA_CONV(__nv_bfloat16, float);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_F32) LIA_CONV(float, float);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_BF16) LIA_CONV(float, __nv_bfloat16);
#undef LIA_CONV
    return LIA_ERR_DTYPE;
}
