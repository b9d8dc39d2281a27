// RMSNorm of the residual stream followed by a short causal convolution over time on each channel, for up to two
// readers of the normed rows at once:
//     h_t   = x_t * rsqrt(mean(x_t^2) + eps) * w                                  (32-bit)
//     out_r = h_t + sum_j c_r[:, j] * h_(t - taps + 1 + j),   r = 0, 1            (zeros before the sequence's start)
// with c_r [width, taps] the reader's taps (the last tap multiplies the token itself).  The taps - 1 normed rows
// before a request's next token are its state: state [slots, taps - 1, width] 32-bit, entry j holding the row of
// position (next position) - (taps - 1) + j.  A step brings each request's tokens as one run of consecutive batch
// rows; a token takes an earlier row from the batch where its request's run holds it and from the state otherwise.
//
// short_conv_kernel: a CTA takes TOK consecutive batch rows (8 for long steps, 1 for short ones) and one slice of the
// channels (grid y: as many slices as give the device two CTAs an SM): the rows' inverse root mean squares (and those
// of the taps - 1 rows before them) by the whole CTA, then a thread per channel.  With `single` (every run of the
// step is one token) the same thread also moves the state on; otherwise it leaves the normed rows of each run's last
// taps - 1 tokens in `tail` and short_conv_state_kernel, launched behind it, writes the state (a run's first tokens
// read the state that its last tokens replace).
#include "common.cuh"
#include <algorithm>

namespace {
constexpr int MAX_TAPS = 8;
constexpr int THREADS = 256;

// V channels a thread (4 where the width allows 16-byte loads, else 1); CAP: the most taps this instantiation holds.
template <int V> struct Lanes { float v[V]; };
template <int V> __device__ __forceinline__ Lanes<V> load_f32(const float* p) {
    Lanes<V> out;
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        out.v[0] = q.x; out.v[1] = q.y; out.v[2] = q.z; out.v[3] = q.w;
    } else {
        out.v[0] = *p;
    }
    return out;
}
template <int V> __device__ __forceinline__ void store_f32(float* p, const Lanes<V>& a) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
    else *p = a.v[0];
}
template <int V, typename T> __device__ __forceinline__ void store_out(T* p, const Lanes<V>& a) {
    if constexpr (V == 4) {
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
        } else {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(a.v[0], a.v[1]), hi = __floats2bfloat162_rn(a.v[2], a.v[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&lo);
            packed.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(p) = packed;
        }
    } else {
        *p = from_float<T>(a.v[0]);
    }
}

template <typename TW, typename TC, typename TO, int TOK, int V, int CAP>
__global__ void __launch_bounds__(THREADS)
short_conv_kernel(const float* __restrict__ x, const TW* __restrict__ norm_weight, const TC* __restrict__ taps0,
                  const TC* __restrict__ taps1, const int* __restrict__ positions, const int* __restrict__ slots,
                  float* __restrict__ state, float* __restrict__ tail, TO* __restrict__ out0, TO* __restrict__ out1,
                  int n_tokens, int width, int taps, float eps, int single) {
    __shared__ float inv_rms[TOK + MAX_TAPS];
    static_assert(TOK + MAX_TAPS <= THREADS, "a thread per row finishes the sums");
    __shared__ int s_slot[TOK], s_pos[TOK], s_before[TOK], s_tail[TOK];
    __shared__ float partial[TOK + MAX_TAPS][THREADS / 32];
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
    // inverse root mean square of rows t0 - reach .. t0 + TOK - 1 (of the tile's own rows alone where every run is one
    // token): every thread adds its elements of a row, the warps' sums meet in a fixed order, so the order of the
    // additions depends on the width alone
    // (the loads of all rows are asked for together: a row after the other would be a trip to memory each)
    constexpr int NEEDED = TOK + CAP - 1;
    {
        float sums[NEEDED];
        const float* rows[NEEDED];
#pragma unroll
        for (int r = 0; r < NEEDED; ++r) {
            const int row = t0 - reach + r;
            sums[r] = 0.f;
            rows[r] = (r >= (single ? reach : 0) && r < TOK + reach && row >= 0 && row < n_tokens) ? x + (size_t)row * width : nullptr;
        }
        for (int i = threadIdx.x * V; i < width; i += THREADS * V) {
#pragma unroll
            for (int r = 0; r < NEEDED; ++r) {
                if (rows[r]) {
                    const Lanes<V> a = load_f32<V>(rows[r] + i);
#pragma unroll
                    for (int e = 0; e < V; ++e) sums[r] = fmaf(a.v[e], a.v[e], sums[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < NEEDED; ++r) {
            const float sum = warp_sum(sums[r]);
            if (lane == 0) partial[r][warp] = sum;
        }
    }
    __syncthreads();
    if (threadIdx.x < TOK + reach) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) sum += partial[threadIdx.x][w];
        inv_rms[threadIdx.x] = 1.0f / sqrtf(sum / (float)width + eps);
    }
    __syncthreads();
    for (int c = (blockIdx.y * THREADS + threadIdx.x) * V; c < width; c += THREADS * gridDim.y * V) {
        Lanes<V> w;
#pragma unroll
        for (int e = 0; e < V; ++e) w.v[e] = to_float(norm_weight[c + e]);
        // the taps by distance back in time: entry k multiplies the row of position pos - k (tap taps - 1 - k)
        Lanes<V> c0[CAP], c1[CAP];
#pragma unroll
        for (int k = 0; k < CAP; ++k)
#pragma unroll
            for (int e = 0; e < V; ++e) {
                c0[k].v[e] = (k < taps && taps0) ? to_float(taps0[(size_t)(c + e) * taps + (taps - 1 - k)]) : 0.f;
                c1[k].v[e] = (k < taps && taps1) ? to_float(taps1[(size_t)(c + e) * taps + (taps - 1 - k)]) : 0.f;
            }
        // past[k]: the normed row of position pos - k (k = 0: the token itself), zero before the sequence's start
        Lanes<V> past[CAP];
        for (int i = 0; i < TOK; ++i) {
            const int t = t0 + i;
            if (t >= n_tokens) break;
            const int slot = s_slot[i], pos = s_pos[i], before = s_before[i];
            if (i >= 1 && before >= 1) {
                // the row ahead is the same request's: what it had at distance k - 1 is at distance k now
#pragma unroll
                for (int k = CAP - 1; k >= 1; --k) past[k] = past[k - 1];
            } else {
#pragma unroll
                for (int k = 1; k < CAP; ++k) {
                    Lanes<V> value;
#pragma unroll
                    for (int e = 0; e < V; ++e) value.v[e] = 0.f;
                    if (k < taps && pos - k >= 0) {
                        if (k <= before) {
                            value = load_f32<V>(x + (size_t)(t - k) * width + c);
#pragma unroll
                            for (int e = 0; e < V; ++e) value.v[e] = value.v[e] * inv_rms[i - k + reach] * w.v[e];
                        } else if (slot >= 0) {
                            value = load_f32<V>(state + ((size_t)slot * reach + (before - k + reach)) * width + c);
                        }
                    }
                    past[k] = value;
                }
            }
            past[0] = load_f32<V>(x + (size_t)t * width + c);
#pragma unroll
            for (int e = 0; e < V; ++e) past[0].v[e] = past[0].v[e] * inv_rms[i + reach] * w.v[e];
            Lanes<V> y0, y1;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int k = CAP - 1; k >= 0; --k) {               // oldest row first
                    sum0 = fmaf(c0[k].v[e], past[k].v[e], sum0);
                    sum1 = fmaf(c1[k].v[e], past[k].v[e], sum1);
                }
                y0.v[e] = past[0].v[e] + sum0;
                y1.v[e] = past[0].v[e] + sum1;
            }
            if (out0) store_out<V, TO>(out0 + (size_t)t * width + c, y0);
            if (out1) store_out<V, TO>(out1 + (size_t)t * width + c, y1);
            if (slot < 0 || reach == 0) continue;
            if (single) {
                // the run is this token alone: entry j of the new state is the row of position pos - (reach - 1 - j)
#pragma unroll
                for (int k = 0; k < CAP - 1; ++k)
                    if (k < reach) store_f32<V>(state + ((size_t)slot * reach + (reach - 1 - k)) * width + c, past[k]);
            } else if (s_tail[i]) {
                store_f32<V>(tail + (size_t)t * width + c, past[0]);
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

template <typename TW, typename TC, typename TO, int TOK, int V, int CAP>
int launch_tile(dim3 grid, cudaStream_t stream, const float* x, const void* norm_weight, const void* taps0, const void* taps1,
                const int* positions, const int* slots, float* state, float* tail, void* out0, void* out1, int n_tokens,
                int width, int taps, float eps, int single) {
    return lia_launch(short_conv_kernel<TW, TC, TO, TOK, V, CAP>, grid, dim3(THREADS), 0, stream, x, (const TW*)norm_weight,
                      (const TC*)taps0, (const TC*)taps1, positions, slots, state, tail, (TO*)out0, (TO*)out1, n_tokens, width,
                      taps, eps, single);
}

template <typename TW, typename TC, typename TO>
int launch_short_conv(const float* x, const void* norm_weight, const void* taps0, const void* taps1, const int* positions,
                      const int* slots, float* state, float* tail, void* out0, void* out1, int n_tokens, int width,
                      int taps, float eps, int single, int sms, cudaStream_t stream) {
    // long steps: 8 rows a CTA (the rows before a tile are normed once for 8 tokens, and a token takes its earlier rows
    // from the token ahead); short ones: a row a CTA.  Four channels a thread where every row allows 16-byte accesses.
    // The channels are cut into slices until the device has two CTAs an SM.
    const bool eight = n_tokens >= 1024;
    const uintptr_t together = (uintptr_t)x | (uintptr_t)state | (uintptr_t)tail | (uintptr_t)out0 | (uintptr_t)out1 | (uintptr_t)norm_weight;
    const bool four = width % 4 == 0 && (together & 15u) == 0;
    const int tiles = (n_tokens + (eight ? 8 : 1) - 1) / (eight ? 8 : 1);
    const int per_cta = THREADS * (four ? 4 : 1);
    const int most = (width + per_cta - 1) / per_cta;
    const int slices = std::max(1, std::min(most, (2 * std::max(sms, 1) + tiles - 1) / tiles));
    const dim3 grid(tiles, slices);
    int code;
#define LIA_TILE(TOK, V, CAP) \
    code = launch_tile<TW, TC, TO, TOK, V, CAP>(grid, stream, x, norm_weight, taps0, taps1, positions, slots, state, tail, out0, out1, n_tokens, width, taps, eps, single)
    if (taps <= 4) {
        if (eight && four) LIA_TILE(8, 4, 4);
        else if (eight) LIA_TILE(8, 1, 4);
        else if (four) LIA_TILE(1, 4, 4);
        else LIA_TILE(1, 1, 4);
    } else {
        if (eight) LIA_TILE(8, 1, MAX_TAPS);
        else LIA_TILE(1, 1, MAX_TAPS);
    }
#undef LIA_TILE
    if (code != LIA_OK || single || taps <= 1) return code;
    return lia_launch(short_conv_state_kernel, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0, stream,
                      (const float*)tail, positions, slots, state, n_tokens, width, taps);
}
}  // namespace

// x [n_tokens, width] 32-bit; norm_weight [width]; taps0, taps1 [width, taps] (either may be null: that reader is
// absent); state [slots, taps - 1, width] 32-bit; tail [n_tokens, width] 32-bit scratch (unused with `single`);
// out0, out1 [n_tokens, width] of out_dtype (null with its taps).  weight_dtype: of the norm weight and of the taps.
// single: 1 when every request of the step brings one token (the state is then moved on by the same kernel).
// sms: the device's SM count (how finely the channels are cut).
LIA_EXPORT int lia_short_conv(const float* x, const void* norm_weight, const void* taps0, const void* taps1,
                              int weight_dtype, const int* positions, const int* slots, float* state, float* tail,
                              void* out0, void* out1, int out_dtype, int n_tokens, int width, int taps, float eps,
                              int single, int sms, cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (width <= 0 || taps < 1 || taps > MAX_TAPS || (taps > 1 && !state) || (!single && taps > 1 && !tail))
        return LIA_ERR_SIZE;
#define LIA_CONV(TW, TO) \
    return launch_short_conv<TW, TW, TO>(x, norm_weight, taps0, taps1, positions, slots, state, tail, out0, out1, n_tokens, width, taps, eps, single, sms, stream)
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_BF16) LIA_CONV(__nv_bfloat16, __nv_bfloat16);
    if (weight_dtype == LIA_BF16 && out_dtype == LIA_F32) LIA_CONV(__nv_bfloat16, float);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_F32) LIA_CONV(float, float);
    if (weight_dtype == LIA_F32 && out_dtype == LIA_BF16) LIA_CONV(float, __nv_bfloat16);
#undef LIA_CONV
    return LIA_ERR_DTYPE;
}
