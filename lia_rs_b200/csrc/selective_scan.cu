// A recurrent mixer with input-dependent decay (selective scan), as three kernels over a step's rows.  A step brings
// runs of consecutive tokens (prompt portions) and single tokens of several requests; what a request carries from step
// to step lives in its slot of two state tensors, both 32-bit: the last taps - 1 inputs of the short convolution and
// the recurrence's state [channels, states].
//
//  * `causal_conv`: y_t[c] = act(bias[c] + sum_j taps[c, j] x_(t - n + 1 + j)[c]) (act: SiLU or none), inputs before the
//    run taken from the slot's state, zeros before the sequence's start.  It reads the state and does not change it,
//    except in a step of single tokens only, where it can leave the new state itself.
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
__device__ __forceinline__ float input_before(const float* __restrict__ x, long long ld, const float* state,
                                              int channels, int taps, int t, int pos, int m, int k, int c) {
    if (pos - k < 0) return 0.f;
    if (k <= m) return x[(size_t)(t - k) * ld + c];
    return state[(size_t)(taps - 1 - (k - m)) * channels + c];     // the state's last row is the input just before the run
}

template <typename TO>
__global__ void causal_conv_kernel(const float* __restrict__ x, long long ld, const float* __restrict__ taps_weight,
                                   const float* __restrict__ bias, const float* state,
                                   long long state_stride, const int* __restrict__ positions, const int* __restrict__ slots,
                                   float* __restrict__ out, TO* __restrict__ out_copy, int n_tokens, int channels,
                                   int taps, int act, float* state_out) {           // (state_out, if given, IS state)
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int pos = positions[t];
    const int m = run_before(positions, slots, t, slot, pos, taps - 1);
    const float* own = state + (size_t)slot * state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float y = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps - 1; ++j)
            y = fmaf(taps_weight[(size_t)c * taps + j], input_before(x, ld, own, channels, taps, t, pos, m, taps - 1 - j, c), y);
        y = fmaf(taps_weight[(size_t)c * taps + taps - 1], x[(size_t)t * ld + c], y);
        if (act == 1) y = y / (1.0f + expf(-y));
        out[(size_t)t * channels + c] = y;
        if (out_copy) out_copy[(size_t)t * channels + c] = from_float<TO>(y);
        if (state_out) {
            // A step of single tokens: nobody else reads this slot's state, so the thread that read a channel's inputs
            // moves them up by one and appends its own, and no second kernel runs.
            float* mine = state_out + (size_t)slot * state_stride;
            float kept[MAX_TAPS];
#pragma unroll
            for (int i = 0; i < MAX_TAPS - 1; ++i)
                if (i < taps - 1) kept[i] = i + 1 < taps - 1 ? mine[(size_t)(i + 1) * channels + c] : x[(size_t)t * ld + c];
#pragma unroll
            for (int i = 0; i < MAX_TAPS - 1; ++i)
                if (i < taps - 1) mine[(size_t)i * channels + c] = kept[i];
        }
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
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
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

constexpr int SCAN_THREADS = 64;
constexpr int STATES_PER_LANE = 8;

__device__ __forceinline__ float softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

constexpr int CHUNK = 64;             // tokens of a long run that one CTA walks when the run is cut

struct ScanArgs {
    const float* x; const float* dt_raw; const float* dt_bias; const float* A; const float* bc; long long ld_bc;
    int b_offset, c_offset;
    const float* D; const float* z; long long ld_z;
    float* state; long long state_stride;
    const int* segments; int n_segments; const int* single_rows; int n_single; const int* slots;
    void* out; int channels, states;
    float* chunk_state;               // [chunks][channels][states]: a chunk's end state from zero, later its start state
    float* chunk_dt;                  // [chunks][channels]: the sum of a chunk's step sizes
};

// Walks rows first .. first + count - 1 of one run for this thread's channel and states.  Tokens in groups of AHEAD:
// everything a group reads is asked for before its first token is computed, so that only the recurrence itself (an
// exponential and a multiply-add per state) lies between one token and the next.  Returns the sum of the step sizes.
template <typename TO, int LPC, bool OUTPUT>
__device__ __forceinline__ float walk(const ScanArgs& p, int first, int count, int cc, int sub, bool live,
                                      float (&S)[STATES_PER_LANE], const float (&a)[STATES_PER_LANE]) {
    const int channels = p.channels, states = p.states;
    const float bias = p.dt_bias[cc], skip = p.D[cc];
    TO* out = reinterpret_cast<TO*>(p.out);
    float dt_sum = 0.f;
    constexpr int AHEAD = 4;
    for (int r0 = 0; r0 < count; r0 += AHEAD) {
        float xv[AHEAD], dtv[AHEAD], gv[AHEAD], bv[AHEAD][STATES_PER_LANE], cv[AHEAD][STATES_PER_LANE];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const bool there = r0 + u < count;
            const size_t t = (size_t)first + (there ? r0 + u : r0);
            xv[u] = p.x[t * channels + cc];
            dtv[u] = p.dt_raw[t * channels + cc];
            if (OUTPUT) gv[u] = p.z[t * p.ld_z + cc];
            const float* b = p.bc + t * p.ld_bc + p.b_offset;
            const float* cvec = p.bc + t * p.ld_bc + p.c_offset;
#pragma unroll
            for (int i = 0; i < STATES_PER_LANE; ++i) {
                const int n = sub + i * LPC;
                bv[u][i] = n < states ? b[n] : 0.f;
                if (OUTPUT) cv[u][i] = n < states ? cvec[n] : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            if (r0 + u >= count) break;
            const size_t t = (size_t)first + r0 + u;
            const float dt = softplus(dtv[u] + bias);
            const float dx = dt * xv[u];
            dt_sum += dt;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < STATES_PER_LANE; ++i) {
                if (sub + i * LPC < states) {
                    S[i] = fmaf(expf(dt * a[i]), S[i], dx * bv[u][i]);
                    if (OUTPUT) y = fmaf(S[i], cv[u][i], y);
                }
            }
            if (OUTPUT) {
#pragma unroll
                for (int o = LPC / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (live && sub == 0) out[t * channels + cc] = from_float<TO>((y + skip * xv[u]) * (gv[u] / (1.0f + expf(-gv[u]))));
            }
        }
    }
    return dt_sum;
}

// The chunk of the cut runs that CTA `id` serves: (first row, rows, first row of its run), or rows 0 if there is none.
__device__ __forceinline__ void chunk_of(const ScanArgs& p, int id, int& first, int& count, int& run_first) {
    count = 0;
    for (int s = 0; s < p.n_segments; ++s) {
        const int seg_first = p.segments[3 * s], seg_count = p.segments[3 * s + 2];
        const int chunks = (seg_count + CHUNK - 1) / CHUNK;
        if (id < chunks) {
            first = seg_first + id * CHUNK;
            count = min(CHUNK, seg_count - id * CHUNK);
            run_first = seg_first;
            return;
        }
        id -= chunks;
    }
}

// MODE 0: whole runs (grid x: the portions, then the single tokens), state read from and left in the slot.
// MODE 1: chunks of the portions from a zero state; leaves each chunk's end state and the sum of its step sizes.
// MODE 2: chunks of the portions from the start states that `scan_carry_kernel` left; writes the outputs.
template <typename TO, int LPC, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(ScanArgs p) {
    pdl_launch_dependents();
    pdl_wait();
    int first = 0, count = 0, run_first = 0;
    if (MODE == 0) {
        if ((int)blockIdx.x < p.n_segments) {
            first = p.segments[3 * blockIdx.x];
            count = p.segments[3 * blockIdx.x + 2];
        } else {
            first = p.single_rows[blockIdx.x - p.n_segments];
            count = 1;
        }
        run_first = first;
    } else {
        chunk_of(p, blockIdx.x, first, count, run_first);
    }
    if (first < 0 || count <= 0) return;
    const int slot = p.slots[run_first];
    if (slot < 0) return;
    const int sub = threadIdx.x % LPC;
    const int c = blockIdx.y * (SCAN_THREADS / LPC) + threadIdx.x / LPC;
    const bool live = c < p.channels;
    const int cc = live ? c : 0;
    float S[STATES_PER_LANE], a[STATES_PER_LANE];
    float* own = MODE == 0 ? p.state + (size_t)slot * p.state_stride + (size_t)cc * p.states
                           : p.chunk_state + ((size_t)blockIdx.x * p.channels + cc) * p.states;
#pragma unroll
    for (int i = 0; i < STATES_PER_LANE; ++i) {
        const int n = sub + i * LPC;
        S[i] = (MODE != 1 && live && n < p.states) ? own[n] : 0.f;
        a[i] = (live && n < p.states) ? p.A[(size_t)cc * p.states + n] : 0.f;
    }
    const float dt_sum = walk<TO, LPC, MODE != 1>(p, first, count, cc, sub, live, S, a);
    if (live && MODE != 2) {
#pragma unroll
        for (int i = 0; i < STATES_PER_LANE; ++i) {
            const int n = sub + i * LPC;
            if (n < p.states) own[n] = S[i];
        }
        if (MODE == 1 && sub == 0) p.chunk_dt[(size_t)blockIdx.x * p.channels + cc] = dt_sum;
    }
}

// Between the two chunked passes: along each portion, the state at the start of every chunk (in place of the chunk's
// end state from zero), S <- exp(A sum(dt)) S + end, beginning with the slot's state; the last one is the slot's new state.
template <int LPC>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_carry_kernel(ScanArgs p) {
    pdl_launch_dependents();
    pdl_wait();
    int base = 0;
    for (int s = 0; s < (int)blockIdx.x; ++s) base += (p.segments[3 * s + 2] + CHUNK - 1) / CHUNK;
    const int run_first = p.segments[3 * blockIdx.x];
    const int chunks = (p.segments[3 * blockIdx.x + 2] + CHUNK - 1) / CHUNK;
    const int slot = p.slots[run_first];
    if (slot < 0) return;
    const int sub = threadIdx.x % LPC;
    const int c = blockIdx.y * (SCAN_THREADS / LPC) + threadIdx.x / LPC;
    if (c >= p.channels) return;
    float* own = p.state + (size_t)slot * p.state_stride + (size_t)c * p.states;
    float S[STATES_PER_LANE], a[STATES_PER_LANE];
#pragma unroll
    for (int i = 0; i < STATES_PER_LANE; ++i) {
        const int n = sub + i * LPC;
        S[i] = n < p.states ? own[n] : 0.f;
        a[i] = n < p.states ? p.A[(size_t)c * p.states + n] : 0.f;
    }
    for (int k = 0; k < chunks; ++k) {
        float* at = p.chunk_state + ((size_t)(base + k) * p.channels + c) * p.states;
        const float dt_sum = p.chunk_dt[(size_t)(base + k) * p.channels + c];
#pragma unroll
        for (int i = 0; i < STATES_PER_LANE; ++i) {
            const int n = sub + i * LPC;
            if (n < p.states) {
                const float end = at[n];
                at[n] = S[i];
                S[i] = fmaf(expf(a[i] * dt_sum), S[i], end);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < STATES_PER_LANE; ++i) {
        const int n = sub + i * LPC;
        if (n < p.states) own[n] = S[i];
    }
}
}  // namespace

// x [n, ld] 32-bit (the first `channels` columns), taps_weight [channels, taps], bias [channels] or null,
// state (slot s at state + s state_stride: [taps - 1, channels]), all 32-bit.  out [n, channels] 32-bit; out_copy (optional) the same in `copy_dtype`.
LIA_EXPORT int lia_causal_conv(const float* x, long long ld, const float* taps_weight, const float* bias,
                               const float* state, long long state_stride, const int* positions, const int* slots,
                               float* out, void* out_copy,
                               int copy_dtype, int n_tokens, int channels, int taps, int act, int update_single,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (channels <= 0 || taps < 1 || taps > MAX_TAPS || ld < channels || (taps > 1 && !state) || act < 0 || act > 1)
        return LIA_ERR_SIZE;
    const int threads = 128;
    // few tokens: a token's channels over several CTAs, so that the step's rows fill the device
    const dim3 grid(n_tokens, n_tokens >= 512 ? 1 : min(16, (channels + threads - 1) / threads));
    // `update_single`: every run of the step is a single token; the kernel then leaves the new state itself
    float* state_out = (update_single && taps > 1) ? const_cast<float*>(state) : nullptr;
    if (!out_copy || copy_dtype == LIA_F32)
        return lia_launch(causal_conv_kernel<float>, grid, dim3(threads), 0, stream, x, ld, taps_weight, bias,
                          state, state_stride, positions, slots, out, (float*)out_copy, n_tokens, channels, taps, act,
                          state_out);
    if (copy_dtype == LIA_BF16)
        return lia_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, ld, taps_weight,
                          bias, state, state_stride, positions, slots, out, (__nv_bfloat16*)out_copy, n_tokens, channels,
                          taps, act, state_out);
    return LIA_ERR_DTYPE;
}

LIA_EXPORT int lia_conv_state_update(const float* x, long long ld, float* state, long long state_stride,
                                     const int* positions, const int* slots, int n_tokens, int channels, int taps, cudaStream_t stream) {
    if (n_tokens <= 0 || taps <= 1) return LIA_OK;
    if (channels <= 0 || taps > MAX_TAPS || ld < channels || !state) return LIA_ERR_SIZE;
    const int threads = 128;
    const dim3 grid(n_tokens, n_tokens >= 512 ? 1 : min(16, (channels + threads - 1) / threads));
    return lia_launch(conv_state_update_kernel, grid, dim3(threads), 0, stream, x, ld, state, state_stride,
                      positions, slots, n_tokens, channels, taps);
}

// x, dt_raw [n, channels]; dt_bias, D [channels]; A [channels, states] (negative: the decay's rate); bc [n, ld_bc] with B
// at column b_offset and C at c_offset (`states` each); z [n, ld_z]; state (slot s at state + s state_stride:
// [channels, states]): all 32-bit.  segments [n_segments, 3] (first row, first position, count) and single_rows
// [n_single] name the step's runs.  out [n, channels] of `out_dtype`.
// `chunk_scratch` (32-bit, `chunk_floats` words; may be null): with it, and portions in the step, the portions are cut
// into chunks of 64 tokens that run side by side (a pass from zero states, a carry along each portion, a pass from the
// true start states); it must hold lia_selective_scan_chunk_floats(n_tokens, n_segments, channels, states) words.
// Without it every run is walked by one CTA per block of channels.
LIA_EXPORT long long lia_selective_scan_chunk_floats(int n_tokens, int n_segments, int channels, int states) {
    const long long chunks = (long long)n_tokens / CHUNK + n_segments;
    return chunks * channels * (states + 1);
}

namespace {
template <typename TO, int LPC>
int launch_scan(ScanArgs p, int n_tokens, bool chunked, cudaStream_t stream) {
    const int per_block = SCAN_THREADS / LPC;
    const unsigned blocks_y = (p.channels + per_block - 1) / per_block;
    if (blocks_y > 65535) return LIA_ERR_SIZE;
    if (!chunked) {
        const dim3 grid(p.n_segments + p.n_single, blocks_y);
        return lia_launch(selective_scan_kernel<TO, LPC, 0>, grid, dim3(SCAN_THREADS), 0, stream, p);
    }
    int rc = LIA_OK;
    if (p.n_single > 0) {                                   // the single tokens: whole runs, as ever
        ScanArgs q = p;
        q.n_segments = 0;
        rc = lia_launch(selective_scan_kernel<TO, LPC, 0>, dim3(p.n_single, blocks_y), dim3(SCAN_THREADS), 0, stream, q);
        if (rc != LIA_OK) return rc;
    }
    const dim3 chunks(n_tokens / CHUNK + p.n_segments, blocks_y);        // as many as the portions can have at most
    rc = lia_launch(selective_scan_kernel<TO, LPC, 1>, chunks, dim3(SCAN_THREADS), 0, stream, p);
    if (rc != LIA_OK) return rc;
    rc = lia_launch(scan_carry_kernel<LPC>, dim3(p.n_segments, blocks_y), dim3(SCAN_THREADS), 0, stream, p);
    if (rc != LIA_OK) return rc;
    return lia_launch(selective_scan_kernel<TO, LPC, 2>, chunks, dim3(SCAN_THREADS), 0, stream, p);
}
}  // namespace

LIA_EXPORT int lia_selective_scan(const float* x, const float* dt_raw, const float* dt_bias, const float* A,
                                  const float* bc, long long ld_bc, int b_offset, int c_offset, const float* D,
                                  const float* z, long long ld_z, float* state, long long state_stride,
                                  const int* segments, int n_segments,
                                  const int* single_rows, int n_single, const int* slots, void* out, int out_dtype,
                                  int channels, int states, int n_tokens, float* chunk_scratch, long long chunk_floats,
                                  cudaStream_t stream) {
    const int runs = n_segments + n_single;
    if (runs <= 0) return LIA_OK;
    if (channels <= 0 || states <= 0 || states > 32 * STATES_PER_LANE || n_segments < 0 || n_single < 0 ||
        ld_bc < b_offset + states || ld_bc < c_offset + states || ld_z < channels || n_tokens < n_single + 2 * n_segments)
        return LIA_ERR_SIZE;
    const bool chunked = chunk_scratch && n_segments > 0;
    if (chunked && chunk_floats < lia_selective_scan_chunk_floats(n_tokens, n_segments, channels, states)) return LIA_ERR_SIZE;
    ScanArgs p;
    p.x = x; p.dt_raw = dt_raw; p.dt_bias = dt_bias; p.A = A; p.bc = bc; p.ld_bc = ld_bc; p.b_offset = b_offset;
    p.c_offset = c_offset; p.D = D; p.z = z; p.ld_z = ld_z; p.state = state; p.state_stride = state_stride;
    p.segments = segments; p.n_segments = n_segments; p.single_rows = single_rows; p.n_single = n_single; p.slots = slots;
    p.out = out; p.channels = channels; p.states = states;
    p.chunk_state = chunk_scratch;
    p.chunk_dt = chunk_scratch ? chunk_scratch + ((long long)n_tokens / CHUNK + n_segments) * channels * states : nullptr;
    int lpc = 1;
    while (lpc * STATES_PER_LANE < states) lpc *= 2;
#define LIA_SCAN_LANES(TO)                                                     \
    switch (lpc) {                                                             \
        case 1: return launch_scan<TO, 1>(p, n_tokens, chunked, stream);       \
        case 2: return launch_scan<TO, 2>(p, n_tokens, chunked, stream);       \
        case 4: return launch_scan<TO, 4>(p, n_tokens, chunked, stream);       \
        case 8: return launch_scan<TO, 8>(p, n_tokens, chunked, stream);       \
        case 16: return launch_scan<TO, 16>(p, n_tokens, chunked, stream);     \
        default: return launch_scan<TO, 32>(p, n_tokens, chunked, stream);     \
    }
    if (out_dtype == LIA_F32) LIA_SCAN_LANES(float)
    if (out_dtype == LIA_BF16) LIA_SCAN_LANES(__nv_bfloat16)
#undef LIA_SCAN_LANES
    return LIA_ERR_DTYPE;
}
