// A recurrent mixer with input-dependent decay (selective scan), as three kernels over a step's rows.  A step brings
// runs of consecutive tokens (prompt portions) and single tokens of several requests; what a request carries from step
// to step lives in its slot of two state tensors, both 32-bit: the last taps - 1 inputs of the short convolution and
// the recurrence's state [channels, states].
//
//  * `causal_conv`: y_t[c] = act(bias[c] + sum_j taps[c, j] x_(t - n + 1 + j)[c]) (act: SiLU or none), inputs before the
//    run taken from the slot's state, zeros before the sequence's start.  It reads the state and does not change it.
//  * `conv_state_update`: the slot's state becomes the last taps - 1 inputs up to the end of the run.  A kernel of its
//    own, after the convolution: a run's first tokens read what its last tokens overwrite.
//  * `selective_scan`: dt = softplus(dt_raw + dt_bias);  S[c, n] <- exp(dt[c] A[c, n]) S[c, n] + dt[c] x[c] B[n];
//    y[c] = (sum_n S[c, n] C[n] + D[c] x[c]) * silu(z[c]), token by token along each run, the state read from and left
//    in the slot.  Decay, step size, exponentials and the state are 32-bit.  A channel is owned by 1 to 32 lanes, each
//    keeping up to 8 states in registers (up to 256 states).
//
// A row whose slot is negative belongs to nobody and is skipped.
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 8;

// how many of the rows just before row t continue the same run (at most `most`)
__device__ __forceinline__ int run_before(const int* __restrict__ positions, const int* __restrict__ slots, int t,
                                          int slot, int pos, int most) {
    int m = 0;
    while (m < most && t - m - 1 >= 0 && slots[t - m - 1] == slot && positions[t - m - 1] == pos - m - 1) ++m;
    return m;
}

// input of channel c at distance k (>= 1) before row t, whose run has m rows before t
__device__ __forceinline__ float input_before(const float* __restrict__ x, long long ld, const float* __restrict__ state,
                                              int channels, int taps, int t, int pos, int m, int k, int c) {
    if (pos - k < 0) return 0.f;
    if (k <= m) return x[(size_t)(t - k) * ld + c];
    return state[(size_t)(taps - 1 - (k - m)) * channels + c];     // the state's last row is the input just before the run
}

template <typename TO>
__global__ void causal_conv_kernel(const float* __restrict__ x, long long ld, const float* __restrict__ taps_weight,
                                   const float* __restrict__ bias, const float* __restrict__ state,
                                   long long state_stride, const int* __restrict__ positions, const int* __restrict__ slots,
                                   float* __restrict__ out, TO* __restrict__ out_copy, int n_tokens, int channels,
                                   int taps, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int m = run_before(positions, slots, t, slot, pos, taps - 1);
    const float* own = state + (size_t)slot * state_stride;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps - 1; ++j)
            y = fmaf(taps_weight[(size_t)c * taps + j], input_before(x, ld, own, channels, taps, t, pos, m, taps - 1 - j, c), y);
        y = fmaf(taps_weight[(size_t)c * taps + taps - 1], x[(size_t)t * ld + c], y);
        if (act == 1) y = y / (1.0f + expf(-y));
        out[(size_t)t * channels + c] = y;
        if (out_copy) out_copy[(size_t)t * channels + c] = from_float<TO>(y);
    }
}

__global__ void conv_state_update_kernel(const float* __restrict__ x, long long ld, float* __restrict__ state,
                                         long long state_stride, const int* __restrict__ positions, const int* __restrict__ slots, int n_tokens,
                                         int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    if (t + 1 < n_tokens && slots[t + 1] == slot && positions[t + 1] == pos + 1) return;      // not the run's last row
    const int m = run_before(positions, slots, t, slot, pos, taps - 1);
    float* own = state + (size_t)slot * state_stride;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float kept[MAX_TAPS];
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i) {
            if (i < taps - 1) {
                const int k = taps - 2 - i;                     // row i of the new state lies k inputs before this row's
                kept[i] = k == 0 ? x[(size_t)t * ld + c] : input_before(x, ld, own, channels, taps, t, pos, m, k, c);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < taps - 1) own[(size_t)i * channels + c] = kept[i];
    }
}

constexpr int SCAN_THREADS = 128;
constexpr int STATES_PER_LANE = 8;

__device__ __forceinline__ float softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename TO, int LPC>            // LPC lanes own one channel
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const float* __restrict__ x, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                      const float* __restrict__ A, const float* __restrict__ bc, long long ld_bc, int b_offset,
                      int c_offset, const float* __restrict__ D, const float* __restrict__ z, long long ld_z,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ segments, int n_segments,
                      const int* __restrict__ single_rows, int n_single, const int* __restrict__ slots,
                      TO* __restrict__ out, int channels, int states) {
    pdl_launch_dependents();
    pdl_wait();
    int first, count;
    if ((int)blockIdx.x < n_segments) {
        first = segments[3 * blockIdx.x];
        count = segments[3 * blockIdx.x + 2];
    } else {
        first = single_rows[blockIdx.x - n_segments];
        count = 1;
    }
    if (first < 0 || count <= 0) return;
    const int slot = slots[first];
    if (slot < 0) return;
    const int sub = threadIdx.x % LPC;
    const int c = blockIdx.y * (SCAN_THREADS / LPC) + threadIdx.x / LPC;
    const bool live = c < channels;
    const int cc = live ? c : 0;
    float S[STATES_PER_LANE], a[STATES_PER_LANE];
    float* own = state + (size_t)slot * state_stride + (size_t)cc * states;
#pragma unroll
    for (int i = 0; i < STATES_PER_LANE; ++i) {
        const int n = sub + i * LPC;
        S[i] = (live && n < states) ? own[n] : 0.f;
        a[i] = (live && n < states) ? A[(size_t)cc * states + n] : 0.f;
    }
    const float bias = dt_bias[cc], skip = D[cc];
    for (int r = 0; r < count; ++r) {
        const size_t t = (size_t)first + r;
        const float xv = x[t * channels + cc];
        const float dt = softplus(dt_raw[t * channels + cc] + bias);
        const float* b = bc + t * ld_bc + b_offset;
        const float* cvec = bc + t * ld_bc + c_offset;
        const float dx = dt * xv;
        float y = 0.f;
#pragma unroll
        for (int i = 0; i < STATES_PER_LANE; ++i) {
            const int n = sub + i * LPC;
            if (n < states) {
                S[i] = fmaf(expf(dt * a[i]), S[i], dx * b[n]);
                y = fmaf(S[i], cvec[n], y);
            }
        }
#pragma unroll
        for (int o = LPC / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (live && sub == 0) {
            const float g = z[t * ld_z + cc];
            out[t * channels + cc] = from_float<TO>((y + skip * xv) * (g / (1.0f + expf(-g))));
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < STATES_PER_LANE; ++i) {
            const int n = sub + i * LPC;
            if (n < states) own[n] = S[i];
        }
    }
}
}  // namespace

// x [n, ld] 32-bit (the first `channels` columns), taps_weight [channels, taps], bias [channels] or null,
// state (slot s at state + s state_stride: [taps - 1, channels]), all 32-bit.  out [n, channels] 32-bit; out_copy (optional) the same in `copy_dtype`.
LIA_EXPORT int lia_causal_conv(const float* x, long long ld, const float* taps_weight, const float* bias,
                               const float* state, long long state_stride, const int* positions, const int* slots,
                               float* out, void* out_copy,
                               int copy_dtype, int n_tokens, int channels, int taps, int act, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (channels <= 0 || taps < 1 || taps > MAX_TAPS || ld < channels || (taps > 1 && !state) || act < 0 || act > 1)
        return LIA_ERR_SIZE;
    const int threads = channels >= 1024 ? 256 : 128;
    if (!out_copy || copy_dtype == LIA_F32)
        return lia_launch(causal_conv_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, x, ld, taps_weight, bias,
                          state, state_stride, positions, slots, out, (float*)out_copy, n_tokens, channels, taps, act);
    if (copy_dtype == LIA_BF16)
        return lia_launch(causal_conv_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, x, ld, taps_weight,
                          bias, state, state_stride, positions, slots, out, (__nv_bfloat16*)out_copy, n_tokens, channels,
                          taps, act);
    return LIA_ERR_DTYPE;
}

LIA_EXPORT int lia_conv_state_update(const float* x, long long ld, float* state, long long state_stride,
                                     const int* positions, const int* slots, int n_tokens, int channels, int taps, cudaStream_t stream) {
    if (n_tokens <= 0 || taps <= 1) return LIA_OK;
    if (channels <= 0 || taps > MAX_TAPS || ld < channels || !state) return LIA_ERR_SIZE;
    const int threads = channels >= 1024 ? 256 : 128;
    return lia_launch(conv_state_update_kernel, dim3(n_tokens), dim3(threads), 0, stream, x, ld, state, state_stride,
                      positions, slots, n_tokens, channels, taps);
}

// x, dt_raw [n, channels]; dt_bias, D [channels]; A [channels, states] (negative: the decay's rate); bc [n, ld_bc] with B
// at column b_offset and C at c_offset (`states` each); z [n, ld_z]; state (slot s at state + s state_stride: [channels, states]): all 32-bit.
// segments [n_segments, 3] (first row, first position, count) and single_rows [n_single] name the step's runs.
// out [n, channels] of `out_dtype`.
LIA_EXPORT int lia_selective_scan(const float* x, const float* dt_raw, const float* dt_bias, const float* A,
                                  const float* bc, long long ld_bc, int b_offset, int c_offset, const float* D,
                                  const float* z, long long ld_z, float* state, long long state_stride,
                                  const int* segments, int n_segments,
                                  const int* single_rows, int n_single, const int* slots, void* out, int out_dtype,
                                  int channels, int states, cudaStream_t stream) {
    const int runs = n_segments + n_single;
    if (runs <= 0) return LIA_OK;
    if (channels <= 0 || states <= 0 || states > 32 * STATES_PER_LANE || n_segments < 0 || n_single < 0 ||
        ld_bc < b_offset + states || ld_bc < c_offset + states || ld_z < channels)
        return LIA_ERR_SIZE;
    int lpc = 1;
    while (lpc * STATES_PER_LANE < states) lpc *= 2;
    const dim3 grid(runs, (channels + SCAN_THREADS / lpc - 1) / (SCAN_THREADS / lpc));
    if (grid.y > 65535) return LIA_ERR_SIZE;
#define LIA_SCAN(TO, LPC)                                                                                              \
    return lia_launch(selective_scan_kernel<TO, LPC>, grid, dim3(SCAN_THREADS), 0, stream, x, dt_raw, dt_bias, A, bc,  \
                      ld_bc, b_offset, c_offset, D, z, ld_z, state, state_stride, segments, n_segments, single_rows, n_single, slots, \
                      (TO*)out, channels, states)
#define LIA_SCAN_LANES(TO)                \
    switch (lpc) {                        \
        case 1: LIA_SCAN(TO, 1);          \
        case 2: LIA_SCAN(TO, 2);          \
        case 4: LIA_SCAN(TO, 4);          \
        case 8: LIA_SCAN(TO, 8);          \
        case 16: LIA_SCAN(TO, 16);        \
        default: LIA_SCAN(TO, 32);        \
    }
    if (out_dtype == LIA_F32) LIA_SCAN_LANES(float)
    if (out_dtype == LIA_BF16) LIA_SCAN_LANES(__nv_bfloat16)
#undef LIA_SCAN_LANES
#undef LIA_SCAN
    return LIA_ERR_DTYPE;
}
